"""Typed configuration of the Lunadra decoder, read from its own ``config.json`` keys.

    {"architecture": "Lunadra", "vocab": V, "width": W, "residual_mult": r, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"}},
                           "right": {"heads", "kv_heads", "dim", "vdim", "conv"}, "left_scale", "right_scale"},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "mlstm", "mixer": {"heads", "dim", "vdim", "gate_cap"},
                 "mlp": {"kind": "moe", "router": {"experts", "identity", "top"}, "expert": {"ff", "limit"},
                         "shared": {"ff", "limit"}}}, ...]}

Every size and constant is read from there; nothing is the same for two layers unless the file says so.  A layer type
``mlstm_<anything>`` is an ``mlstm`` layer (and ``parallel_<anything>`` a ``parallel`` one).  The ranks of the gated delta mixer's low-rank projections are not in the
file: the checkpoint's tensors decide them (``rank`` is what random weights get).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, require_float, require_int
from .registry import register_preset_folder
from .vabelorn import _obj, _sub

# The file gives no longest sequence; position tables are made for what the engine is asked to hold, up to this.
MAX_POSITIONS = 1 << 17


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class GatedDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    rank: int = 16


@dataclass(frozen=True)
class SideBySide:
    left: WindowAttention
    right: GatedDelta
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class Mlstm:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseFf:
    ff: int


@dataclass(frozen=True)
class ExpertFf:
    ff: int
    limit: float


@dataclass(frozen=True)
class RoutedFf:
    experts: int
    identity: int
    top: int
    expert: ExpertFf
    shared: Optional[ExpertFf]


@dataclass(frozen=True)
class LunadraLayer:
    type: str                       # "parallel" | "mlstm" (also for "mlstm_<n>": the file's own name is kept in ``name``)
    mixer: Any                      # SideBySide | Mlstm
    mlp: Any                        # None | DenseFf | RoutedFf
    name: str = ""


def _expert(d: Any, where: str) -> ExpertFf:
    d = _obj(d, where)
    whole, num = _sub(d, where)
    return ExpertFf(ff=whole("ff"), limit=num("limit"))


def _mlp(d: Any, where: str):
    if d is None:
        return None
    d = _obj(d, where)
    kind = d.get("kind", "dense")
    if kind == "dense":
        whole, _ = _sub(d, where)
        return DenseFf(ff=whole("ff"))
    if kind == "moe":
        r = _obj(d.get("router"), where + ".router")
        whole, _ = _sub(r, where + ".router")
        experts, identity = whole("experts", minimum=0), whole("identity", minimum=0, default=0)
        top = whole("top")
        if top > experts + identity:
            raise ConfigError(f"config.json: {where}.router: 'top' ({top}) exceeds the {experts + identity} experts")
        shared = d.get("shared")
        return RoutedFf(experts=experts, identity=identity, top=top, expert=_expert(d.get("expert"), where + ".expert"),
                        shared=_expert(shared, where + ".shared") if shared else None)
    raise ConfigError(f"config.json: {where}: 'kind' must be 'dense' or 'moe', got {kind!r}")


def _mlp_dict(m) -> Any:
    if m is None:
        return None
    if isinstance(m, DenseFf):
        return {"kind": "dense", "ff": m.ff}
    d: Dict[str, Any] = {"kind": "moe", "router": {"experts": m.experts, "identity": m.identity, "top": m.top},
                         "expert": {"ff": m.expert.ff, "limit": m.expert.limit}}
    if m.shared is not None:
        d["shared"] = {"ff": m.shared.ff, "limit": m.shared.limit}
    return d


@dataclass(frozen=True)
class LunadraConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[LunadraLayer, ...]
    norm_eps: float
    residual_mult: float = 1.0
    pairs: Optional[PairTable] = None
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default="Lunadra")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LunadraConfig":
        vocab = require_int(d, "vocab")
        width = require_int(d, "width")
        _, nnum = _sub(_obj(d.get("norm"), "'norm'"), "'norm'")
        eps = nnum("eps")
        pairs = None
        big = (d.get("embedding") or {}).get("bigram") if isinstance(d.get("embedding"), dict) else None
        if big:
            whole, _ = _sub(_obj(big, "embedding.bigram"), "embedding.bigram")
            pairs = PairTable(buckets=whole("buckets"), mul_prev=whole("mul_prev", minimum=0), mul_cur=whole("mul_cur", minimum=0))
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            entry = _obj(entry, where)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), where + ".mixer")
            if isinstance(kind, str) and (kind == "parallel" or kind.startswith("parallel_")):
                lw = where + ".mixer.left"
                left = _obj(m.get("left"), lw)
                whole, num = _sub(left, lw)
                heads, kv = whole("heads"), whole("kv_heads", default=left.get("heads"))
                if heads % kv:
                    raise ConfigError(f"config.json: {lw}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
                dim = whole("dim")
                rot = left.get("rot") or {"base": 10000.0, "dims": 0}
                rwhole, rnum = _sub(_obj(rot, lw + ".rot"), lw + ".rot")
                dims = rwhole("dims", minimum=0)
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: {lw}.rot: 'dims' must be even and at most the head size {dim}, got {dims}")
                mask = left.get("mask")
                window = None
                if mask:
                    mwhole, _ = _sub(_obj(mask, lw + ".mask"), lw + ".mask")
                    window = mwhole("size")
                att = WindowAttention(heads=heads, kv_heads=kv, dim=dim, vdim=whole("vdim", default=dim), scale=num("scale"),
                                      window=window, rot_base=rnum("base"), rot_dims=dims)
                rw = where + ".mixer.right"
                right = _obj(m.get("right"), rw)
                whole, _ = _sub(right, rw)
                heads, kv = whole("heads"), whole("kv_heads", default=right.get("heads"))
                if heads % kv:
                    raise ConfigError(f"config.json: {rw}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
                dim = whole("dim")
                gd = GatedDelta(heads=heads, kv_heads=kv, dim=dim, vdim=whole("vdim", default=dim), conv=whole("conv"),
                                rank=whole("rank", default=16))
                _, mnum = _sub(m, where + ".mixer")
                mixer = SideBySide(left=att, right=gd, left_scale=mnum("left_scale", positive=False, default=1.0),
                                   right_scale=mnum("right_scale", positive=False, default=1.0))
                layer_type = "parallel"
            elif isinstance(kind, str) and (kind == "mlstm" or kind.startswith("mlstm_")):
                whole, num = _sub(m, where + ".mixer")
                dim = whole("dim")
                mixer = Mlstm(heads=whole("heads"), dim=dim, vdim=whole("vdim", default=dim), gate_cap=num("gate_cap"))
                layer_type = "mlstm"
            else:
                raise ConfigError(f"config.json: {where}: 'type' must be 'parallel' or 'mlstm', got {kind!r}")
            layers.append(LunadraLayer(type=layer_type, mixer=mixer, mlp=_mlp(entry.get("mlp"), where + ".mlp"), name=str(kind)))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: 'eos_token_id' {e} is outside the vocabulary (0..{vocab - 1})")
        bos = d.get("bos_token_id")
        return cls(vocab=vocab, width=width, layers=tuple(layers), norm_eps=eps,
                   residual_mult=require_float(d, "residual_mult", default=1.0), pairs=pairs, eos_token_id=eos_ids,
                   bos_token_id=None if bos is None else int(bos), architecture=str(d.get("architecture") or "Lunadra"))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "parallel":
                a, b = m.left, m.right
                left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                                        "rot": {"base": a.rot_base, "dims": a.rot_dims}}
                if a.window:
                    left["mask"] = {"size": a.window}
                mixer = {"left": left, "left_scale": m.left_scale, "right_scale": m.right_scale,
                         "right": {"heads": b.heads, "kv_heads": b.kv_heads, "dim": b.dim, "vdim": b.vdim, "conv": b.conv,
                                   "rank": b.rank}}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            layers.append({"type": layer.name or layer.type, "mixer": mixer, "mlp": _mlp_dict(layer.mlp)})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.pairs is not None:
            d["embedding"] = {"bigram": {"buckets": self.pairs.buckets, "mul_prev": self.pairs.mul_prev, "mul_cur": self.pairs.mul_cur}}
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return self.eos_token_id

    @property
    def bos_token(self) -> int:
        return self.bos_token_id if self.bos_token_id is not None else 0


register_preset_folder(os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets"))
