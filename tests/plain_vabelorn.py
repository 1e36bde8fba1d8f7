"""The Vabelorn decoder written out plainly and slowly in PyTorch, one function per mechanism, for the tests.

It shares no code with the package: it reads a configuration as a plain dict (the keys of ``config.json``) and
weights as a dict of tensors by checkpoint name, and computes everything in the dtype it is given (float64 by
default), one whole sequence at a time, with no cache.  ``decode_token_by_token`` runs the same mathematics as a
recurrence over explicit per-sequence state, so that prefill and decoding can be compared inside the oracle too.

Notation: ``x`` is the residual stream ``[T, width]``; ``rms(x) = x / sqrt(mean(x^2) + eps)``.

    layer:      x += norm1(mixer(x)) ; x += norm2(ff(x)) if the layer has a feed-forward ; x += side(x, token)
    side:       e = side_embed[token, i*ds:(i+1)*ds] ; y = P (gelu_tanh(G x) * e) ; rms(y) * w
    wkv:        shifted mixes, r k v g projections, data-dependent decay exp(-exp(.)), per-head matrix state
                S <- diag(w) S + k v^T read as (S + diag(u) k v^T)^T r, unit norm per head, weight, gate, W_o
    attention:  grouped heads, q/k RMS norm with weight, interleaved rotary on the first ``dims`` features with
                YaRN-scaled frequencies, values divided by their RMS and rotated by their own position over all
                features, softmax with a sink (one added to the denominator), output rotated back by the
                query's position, W_o
    output:     logits = E norm(x) * logit_scale with the embedding table E
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ``STORE``: None, or a 16-bit dtype in which the results of matrix products and what a cache keeps are rounded (and
# brought back), at about the places where an engine that runs in that dtype rounds.  It shows how far rounding alone
# moves the logits of a model: the measure against which a 16-bit run can be judged.  ``with stored(torch.bfloat16): ..``
STORE = None


class stored:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global STORE
        self.before, STORE = STORE, self.dtype

    def __exit__(self, *exc):
        global STORE
        STORE = self.before


def st(x: torch.Tensor) -> torch.Tensor:
    return x if STORE is None else x.to(STORE).to(x.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---- rotary angles -----------------------------------------------------------------------------------------
def key_frequencies(rot: dict, dtype=torch.float64) -> (torch.Tensor, float):
    """Frequencies of the ``dims/2`` rotated pairs of queries and keys, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f.to(dtype), 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(t: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f.to(dtype), 0.1 * math.log(factor) + 1.0


def value_frequencies(rot: dict, vdim: int, dtype=torch.float64) -> torch.Tensor:
    m = torch.arange(vdim // 2, dtype=torch.float64)
    return (float(rot["base"]) ** (-2.0 * m / vdim)).to(dtype)


def rotate_interleaved(x: torch.Tensor, angles: torch.Tensor, mult: float = 1.0) -> torch.Tensor:
    """``x [..., T, 2n]`` with pairs (2i, 2i+1); ``angles [T, n]``."""
    c, s = torch.cos(angles) * mult, torch.sin(angles) * mult
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


# ---- mixers ------------------------------------------------------------------------------------------------
def attention_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                    positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    rot = m["rot"]
    dims = int(rot["dims"])
    pos = torch.arange(T, dtype=h.dtype) if positions is None else positions.to(h.dtype)
    q = st(h @ W[p + "q"].T).view(T, H, d)
    k = st(h @ W[p + "k"].T).view(T, G, d)
    v = st(h @ W[p + "v"].T).view(T, G, dv)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    f, mult = key_frequencies(rot, h.dtype)
    ang = pos[:, None] * f[None, :]
    q = torch.cat([rotate_interleaved(q[..., :dims].transpose(0, 1), ang, mult).transpose(0, 1), q[..., dims:]], dim=-1)
    k = torch.cat([rotate_interleaved(k[..., :dims].transpose(0, 1), ang, mult).transpose(0, 1), k[..., dims:]], dim=-1)
    v = rms(v, eps)
    vang = pos[:, None] * value_frequencies(rot, dv, h.dtype)[None, :]
    v = st(rotate_interleaved(v.transpose(0, 1), vang).transpose(0, 1))        # [T, G, dv]
    q, k = st(q), st(k)
    out = torch.empty(T, H, dv, dtype=h.dtype)
    causal = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~causal, float("-inf"))
        e = torch.exp(s)                                                      # masked scores give 0
        pr = e / (1.0 + e.sum(dim=-1, keepdim=True))
        out[:, head] = pr @ v[:, g]
    out = rotate_interleaved(out.transpose(0, 1), -vang).transpose(0, 1)
    return st(st(out.reshape(T, H * dv)) @ W[p + "o"].T)


def wkv_decay(mix_w: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return torch.exp(-torch.exp(st(torch.tanh(st(mix_w @ W[p + "w1"].T))) @ W[p + "w2"].T + W[p + "w0"]))


def wkv_mixer(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
              state: Optional[dict] = None) -> torch.Tensor:
    """``state`` (optional) carries ``prev`` [width] and ``S`` [heads, dim, dim] in and out."""
    T, width = h.shape
    H, d = int(m["heads"]), int(m["dim"])
    prev0 = torch.zeros(width, dtype=h.dtype) if state is None else state["prev"]
    S = torch.zeros(H, d, d, dtype=h.dtype) if state is None else state["S"].clone()
    hp = torch.cat([prev0[None], h[:-1]], dim=0)
    mix = {s: st(h + (hp - h) * W[p + "mu." + s]) for s in "rkvgw"}
    r = st(mix["r"] @ W[p + "r"].T).view(T, H, d)
    k = st(mix["k"] @ W[p + "k"].T).view(T, H, d)
    v = st(mix["v"] @ W[p + "v"].T).view(T, H, d)
    gate = silu(st(mix["g"] @ W[p + "g"].T))
    w = wkv_decay(mix["w"], W, p).view(T, H, d)
    u = W[p + "u"].to(h.dtype)
    o = torch.empty(T, H, d, dtype=h.dtype)
    for t in range(T):
        kv = k[t, :, :, None] * v[t, :, None, :]                              # [H, d(key), d(value)]
        o[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t, :, :, None] * S + kv
    if state is not None:
        state["prev"], state["S"] = h[-1].clone(), S
    o = st(rms(o, eps).reshape(T, H * d) * W[p + "norm"] * gate)
    return st(o @ W[p + "o"].T)


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return st(st(silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T)


def side_input(x: torch.Tensor, tokens: torch.Tensor, W: Dict[str, torch.Tensor], layer: int, ds: int, eps: float) -> torch.Tensor:
    p = f"l{layer}.side."
    e = W["side.embed"][tokens][:, layer * ds:(layer + 1) * ds]
    y = st(st(gelu_tanh(st(x @ W[p + "gate"].T)) * e) @ W[p + "proj"].T)
    return rms(y, eps) * W[p + "norm"]


# ---- the model ---------------------------------------------------------------------------------------------
def as_dtype(weights: Dict[str, torch.Tensor], dtype) -> Dict[str, torch.Tensor]:
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None,
            state: Optional[list] = None, start: int = 0) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence.  With ``state`` (a list with one dict per layer, made by
    ``new_state``) the tokens continue the sequence that the state holds, at position ``start``."""
    W = as_dtype(weights, dtype)
    eps = float(cfg["norm"]["eps"])
    ds = int(cfg["token_side"]["dim"]) if cfg.get("token_side") else 0
    tok = torch.tensor(tokens, dtype=torch.long)
    x = W["embed"][tok]
    T = len(tokens)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}.mix."
        if layer["type"] == "attention":
            if state is None:
                mixed = attention_mixer(st(x), W, p, layer["mixer"], eps)
            else:
                # the plain way to continue: keep the mixer's inputs of all earlier tokens and run over all of them
                kept = state[i]
                kept["h"] = st(x) if kept.get("h") is None else torch.cat([kept["h"], st(x)], dim=0)
                mixed = attention_mixer(kept["h"], W, p, layer["mixer"], eps)[-T:]
        elif layer["type"] == "wkv":
            mixed = wkv_mixer(st(x), W, p, layer["mixer"], eps, None if state is None else state[i])
        else:
            raise ValueError(layer["type"])
        x = x + rms(mixed, eps) * W[f"l{i}.norm1"]
        if layer.get("mlp"):
            x = x + rms(dense_ff(st(x), W, f"l{i}.mlp."), eps) * W[f"l{i}.norm2"]
        if ds:
            x = x + side_input(st(x), tok, W, i, ds, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return st(rms(x, eps) * W["final.norm"]) @ W["embed"].T * float(cfg.get("logit_scale", 1.0))


def new_state(cfg: dict, dtype=torch.float64) -> list:
    out = []
    for layer in cfg["layers"]:
        if layer["type"] == "wkv":
            H, d = int(layer["mixer"]["heads"]), int(layer["mixer"]["dim"])
            out.append({"prev": torch.zeros(int(cfg["width"]), dtype=dtype), "S": torch.zeros(H, d, d, dtype=dtype)})
        else:
            out.append({"h": None})
    return out


def decode_token_by_token(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64) -> torch.Tensor:
    state = new_state(cfg, dtype)
    rows = [forward(cfg, weights, [t], dtype, state=state, start=i) for i, t in enumerate(tokens)]
    return torch.cat(rows, dim=0)


# ---- random models for the tests -----------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    width, vocab = int(cfg["width"]), int(cfg["vocab"])
    ds = int(cfg["token_side"]["dim"]) if cfg.get("token_side") else 0
    n = len(cfg["layers"])
    shapes = {"embed": (vocab, width), "final.norm": (width,)}
    if ds:
        shapes["side.embed"] = (vocab, n * ds)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes[p + "norm1"] = (width,)
        if layer["type"] == "attention":
            H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            shapes.update({p + "mix.q": (H * d, width), p + "mix.k": (G * d, width), p + "mix.v": (G * dv, width),
                           p + "mix.q.norm": (d,), p + "mix.k.norm": (d,), p + "mix.o": (width, H * dv)})
        else:
            H, d = int(m["heads"]), int(m["dim"])
            lora = int(m.get("decay_rank", 8))
            for s in "rkvgw":
                shapes[p + "mix.mu." + s] = (width,)
            for s in "rkvg":
                shapes[p + "mix." + s] = (H * d, width)
            shapes.update({p + "mix.w1": (lora, width), p + "mix.w2": (H * d, lora), p + "mix.w0": (H * d,),
                           p + "mix.u": (H, d), p + "mix.norm": (H * d,), p + "mix.o": (width, H * d)})
        if layer.get("mlp"):
            ff = int(layer["mlp"]["ff"])
            shapes.update({p + "norm2": (width,), p + "mlp.gate": (ff, width), p + "mlp.up": (ff, width),
                           p + "mlp.down": (width, ff)})
        if ds:
            shapes.update({p + "side.gate": (ds, width), p + "side.proj": (width, ds), p + "side.norm": (width,)})
    return shapes


def random_weights(cfg: dict, seed: int, sharpen: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights rounded to bfloat16 (as a checkpoint stores them), returned as float32.  Matrices N(0, 1/sqrt(in)),
    norm weights around one, mixing coefficients in (0, 1), decay offsets spread so that some channels forget
    fast and some slowly; ``sharpen`` multiplies the query norm weights so that attention is peaked."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith((".q.norm", ".k.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
            if name.endswith(".q.norm"):
                t = t * sharpen
        elif last in ("norm1", "norm2") or name.endswith((".side.norm", "final.norm", ".mix.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif last == "w0":
            t = -3.0 + 3.5 * torch.rand(shape, generator=g)
        elif last == "u":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
