"""Typed configuration of the Vabelorn decoder, read from its own ``config.json`` keys.

The file names the model in ``architecture`` (a string) and describes every layer by itself:

    {"architecture": "Vabelorn", "vocab": V, "width": W, "logit_scale": s, "norm": {"eps": e},
     "token_side": {"dim": ds},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                                                 "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                 "mlp": {"kind": "dense", "ff": F}},
                {"type": "wkv", "mixer": {"heads", "dim"}, "mlp": null}, ...]}

Every size and constant is read from there; nothing is the same for two layers unless the file says so.  The
rank of a ``wkv`` layer's decay projection is not in the file: the checkpoint's tensor decides it
(``decay_rank`` is the rank that random weights get).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, require_float, require_int
from .registry import register_preset_folder

# The file gives no longest sequence; position tables are made for what the engine is asked to hold, up to this.
MAX_POSITIONS = 1 << 17


@dataclass(frozen=True)
class RotaryScaling:
    """YaRN: pairs that turn fewer than ``slow`` times over ``original`` positions are slowed by ``factor``,
    pairs that turn more than ``fast`` times are left alone, a linear ramp over the pair index in between."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotary:
    base: float
    dims: int
    scaling: Optional[RotaryScaling] = None


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotary


@dataclass(frozen=True)
class WkvMixer:
    heads: int
    dim: int
    decay_rank: int = 16


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class VabelornLayer:
    type: str                       # "attention" | "wkv"
    mixer: Any                      # AttentionMixer | WkvMixer
    mlp: Optional[DenseMlp]


def _obj(d: Any, where: str) -> Dict[str, Any]:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object, got {d!r}")
    return d


def _sub(d: Dict[str, Any], where: str):
    """``require_*`` on a nested object with the path in the message."""
    def num(key, **kw):
        try:
            return require_float(d, key, **kw)
        except ConfigError as e:
            raise ConfigError(str(e).replace("config.json:", f"config.json: {where}:")) from None

    def whole(key, **kw):
        try:
            return require_int(d, key, **kw)
        except ConfigError as e:
            raise ConfigError(str(e).replace("config.json:", f"config.json: {where}:")) from None
    return whole, num


def _rotary(d: Any, where: str, head: int) -> Rotary:
    d = _obj(d, where)
    whole, num = _sub(d, where)
    dims = whole("dims", minimum=0)
    if dims % 2 or dims > head:
        raise ConfigError(f"config.json: {where}: 'dims' must be even and at most the head size {head}, got {dims}")
    sc = d.get("scaling")
    scaling = None
    if sc:
        swhole, snum = _sub(_obj(sc, where + ".scaling"), where + ".scaling")
        scaling = RotaryScaling(factor=snum("factor"), original=snum("original"), fast=snum("fast"), slow=snum("slow"))
    return Rotary(base=num("base"), dims=dims, scaling=scaling)


@dataclass(frozen=True)
class VabelornConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[VabelornLayer, ...]
    norm_eps: float
    logit_scale: float = 1.0
    token_side_dim: int = 0
    eos_token_id: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default="Vabelorn")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VabelornConfig":
        vocab = require_int(d, "vocab")
        width = require_int(d, "width")
        _, nnum = _sub(_obj(d.get("norm"), "'norm'"), "'norm'")
        eps = nnum("eps")
        side = d.get("token_side")
        side_dim = 0
        if side:
            swhole, _ = _sub(_obj(side, "'token_side'"), "'token_side'")
            side_dim = swhole("dim")
        raw = d.get("layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            entry = _obj(entry, where)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), where + ".mixer")
            whole, num = _sub(m, where + ".mixer")
            if kind == "attention":
                heads, kv = whole("heads"), whole("kv_heads", default=m.get("heads"))
                if heads % kv:
                    raise ConfigError(f"config.json: {where}.mixer: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv})")
                dim = whole("dim")
                vdim = whole("vdim", default=dim)
                if vdim % 2:
                    raise ConfigError(f"config.json: {where}.mixer: 'vdim' ({vdim}) must be even (values are rotated in pairs)")
                mixer = AttentionMixer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=num("scale"),
                                       rot=_rotary(m.get("rot"), where + ".mixer.rot", dim))
            elif kind == "wkv":
                mixer = WkvMixer(heads=whole("heads"), dim=whole("dim"), decay_rank=whole("decay_rank", default=16))
            else:
                raise ConfigError(f"config.json: {where}: 'type' must be 'attention' or 'wkv', got {kind!r}")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp = _obj(mlp, where + ".mlp")
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp: 'kind' = {mlp.get('kind')!r} is not built (only 'dense')")
                fwhole, _ = _sub(mlp, where + ".mlp")
                mlp = DenseMlp(ff=fwhole("ff"))
            layers.append(VabelornLayer(type=kind, mixer=mixer, mlp=mlp))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else (eos,)))
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: 'eos_token_id' {e} is outside the vocabulary (0..{vocab - 1})")
        bos = d.get("bos_token_id")
        return cls(vocab=vocab, width=width, layers=tuple(layers), norm_eps=eps,
                   logit_scale=require_float(d, "logit_scale", default=1.0), token_side_dim=side_dim,
                   eos_token_id=eos_ids, bos_token_id=None if bos is None else int(bos),
                   architecture=str(d.get("architecture") or "Vabelorn"))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                rot: Dict[str, Any] = {"base": m.rot.base, "dims": m.rot.dims}
                if m.rot.scaling is not None:
                    s = m.rot.scaling
                    rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "rot": rot}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "decay_rank": m.decay_rank}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.mlp is None else {"kind": "dense", "ff": layer.mlp.ff}})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.token_side_dim:
            d["token_side"] = {"dim": self.token_side_dim}
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
