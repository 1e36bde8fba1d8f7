"""The Lunadra decoder written out plainly and slowly in PyTorch, one function per mechanism, for the tests.

It shares no code with the package: it reads a configuration as a plain dict (the keys of ``config.json``) and
weights as a dict of tensors by checkpoint name, and computes everything in the dtype it is given (float64 by
default), one whole sequence at a time, with no cache.  ``Walker`` runs the same mathematics token by token over
explicit per-sequence state, so that whole prompts and decoding can be compared inside the oracle too.

Notation: ``x`` is the residual stream ``[T, width]``; ``unit(x) = x / sqrt(mean(x^2) + eps)``.

    embedding:  x_t = E[tok_t] + B[(tok_{t-1} * a + tok_t * b) mod n], and B[n] for t = 0
    layer:      h = unit(x) * w ;  x += r * (mixer(h) + ff(h))       one norm feeds both sublayers
    mlstm:      per head a matrix S, a vector n and a running maximum m (all start at 0):
                  m' = max(f + m, i) ; S' = e^(f + m - m') S + e^(i - m') k v^T ; n' likewise with k
                  o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
                with capped gates i = c tanh(. / c), f = logsigmoid(c tanh(. / c)); unit(o) per head, weight,
                sigmoid gate, W_o
    parallel:   a * window_attention(h) + b * delta(h)
      attention:  grouped heads, split-half rotary on the first ``dims`` features, a sliding window, softmax
      delta:      short causal convolutions and silu on q, k, v; q, k of length one; per head a matrix S:
                  S <- diag(g) S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q
                  with g = exp(-exp(A) softplus(. + dt)) per key channel; unit(o), weight, low-rank sigmoid gate, W_o
    ff dense:   D (relu(G h) * (U h))
    ff moe:     s = softmax(R h) ; the ``top`` largest of s + c are chosen and weighted with s itself ; the last
                ``identity`` router outputs stand for experts that return h ; a shared expert is added
      expert:     g = min(G h, L) ; u = clamp(U h, -L, L) ; D (g sigmoid(1.702 g) (u + 1))
    output:     logits = H (unit(x) * w)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

# ``STORE``: None, or a 16-bit dtype in which the results of matrix products are rounded (and brought back), at about
# the places where an engine that runs in that dtype rounds: the measure against which a 16-bit run is judged.
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


def lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return st(x @ w.T)


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


# ---- embedding ------------------------------------------------------------------------------------------------
def bigram_rows(tokens: List[int], cfg: dict, before: Optional[int] = None) -> List[int]:
    """Row of the pair table for every token; ``before``: the token that precedes the first one (None: none does)."""
    b = cfg["embedding"]["bigram"]
    n, a, c = int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])
    rows = []
    for t in tokens:
        rows.append(n if before is None else (before * a + t * c) % n)
        before = t
    return rows


def embed(tokens: List[int], cfg: dict, w: Dict[str, torch.Tensor], before: Optional[int] = None) -> torch.Tensor:
    x = w["embed"][tokens]
    if cfg.get("embedding", {}).get("bigram"):
        x = x + w["bigram"][bigram_rows(tokens, cfg, before)]
    return x


# ---- feed-forwards ----------------------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return lin(st(torch.relu(lin(h, w[p + ".gate"])) * lin(h, w[p + ".up"])), w[p + ".down"])


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = lin(h, w[p + ".gate"]).clamp(max=limit)
    u = lin(h, w[p + ".up"]).clamp(-limit, limit)
    return lin(st(g * torch.sigmoid(1.702 * g) * (u + 1.0)), w[p + ".down"])


def router(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, top: int):
    """(chosen indices ``[T, top]``, their weights) among all router outputs."""
    s = torch.softmax(h @ w[p + ".router"].T, dim=-1)
    chosen = torch.topk(s + w[p + ".correction"], top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def moe_ff(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    r = mlp["router"]
    real, top = int(r["experts"]), int(r["top"])
    chosen, weight = router(h, w, p, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            y = expert(h[t:t + 1], w, f"{p}.e{e}", float(mlp["expert"]["limit"]))[0] if e < real else h[t]
            out[t] += weight[t, j] * y
    if mlp.get("shared"):
        out = out + expert(h, w, p + ".shared", float(mlp["shared"]["limit"]))
    return out


def feed_forward(h: torch.Tensor, mlp: Optional[dict], w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    if mlp is None:
        return torch.zeros_like(h)
    return dense_ff(h, w, p) if mlp.get("kind", "dense") == "dense" else moe_ff(h, mlp, w, p)


# ---- mlstm ----------------------------------------------------------------------------------------------------
def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm_new_state(m: dict, dtype) -> dict:
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    return {"S": torch.zeros(H, d, dv, dtype=dtype), "n": torch.zeros(H, d, dtype=dtype), "m": torch.zeros(H, dtype=dtype)}


def mlstm(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float, state: dict) -> torch.Tensor:
    """All tokens of ``h`` one after the other from ``state``, which is updated in place."""
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cap = float(m["gate_cap"])
    T = h.shape[0]
    q = lin(h, w[p + ".q"]).view(T, H, d) * d ** -0.5
    k = lin(h, w[p + ".k"]).view(T, H, d)
    v = lin(h, w[p + ".v"]).view(T, H, dv)
    gi = capped(h @ w[p + ".i"].T + w[p + ".i.b"], cap)
    gf = F.logsigmoid(capped(h @ w[p + ".f"].T + w[p + ".f.b"], cap))
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            m_old = state["m"][a]
            m_new = torch.maximum(gf[t, a] + m_old, gi[t, a])
            keep, take = torch.exp(gf[t, a] + m_old - m_new), torch.exp(gi[t, a] - m_new)
            state["S"][a] = keep * state["S"][a] + take * torch.outer(k[t, a], v[t, a])
            state["n"][a] = keep * state["n"][a] + take * k[t, a]
            state["m"][a] = m_new
            den = torch.maximum((state["n"][a] @ q[t, a]).abs(), torch.exp(-m_new)) + 1e-6
            o[t, a] = state["S"][a].T @ q[t, a] / den
    y = unit(o, eps).reshape(T, H * dv) * w[p + ".norm"] * torch.sigmoid(lin(h, w[p + ".g"]))
    return lin(st(y), w[p + ".o"])


# ---- window attention -------------------------------------------------------------------------------------------
def rotate(x: torch.Tensor, pos: torch.Tensor, rot: dict) -> torch.Tensor:
    """``x [T, heads, dim]``: feature i of the first ``dims`` turns together with feature i + dims/2."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    half = dims // 2
    f = float(rot["base"]) ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    ang = pos.to(torch.float64)[:, None] * f
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def window_attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, past: Optional[dict] = None) -> torch.Tensor:
    """``past``: keys and values of the tokens before ``h`` (already turned), extended in place if given."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    t0 = 0 if past is None or past.get("k") is None else past["k"].shape[0]
    pos = torch.arange(t0, t0 + T)
    q = rotate(lin(h, w[p + ".q"]).view(T, H, d), pos, m["rot"])
    k = st(rotate(lin(h, w[p + ".k"]).view(T, G, d), pos, m["rot"]))
    v = lin(h, w[p + ".v"]).view(T, G, dv)
    if past is not None:
        if past.get("k") is not None:
            k, v = torch.cat([past["k"], k]), torch.cat([past["v"], v])
        past["k"], past["v"] = k, v
    size = m.get("mask", {}).get("size") if m.get("mask") else None
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        score = (st(q[:, a]) @ k[:, g].T) * float(m["scale"])
        i = pos[:, None]
        j = torch.arange(k.shape[0])[None, :]
        seen = (j <= i) if not size else (j <= i) & (i - j < int(size))
        score = score.masked_fill(~seen, float("-inf"))
        o[:, a] = torch.softmax(score, dim=-1) @ v[:, g]
    return lin(st(o.reshape(T, H * dv)), w[p + ".o"])


# ---- gated delta rule ---------------------------------------------------------------------------------------------
def delta_new_state(m: dict, dtype) -> dict:
    H, G, d, dv, taps = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"])
    return {"S": torch.zeros(H, d, dv, dtype=dtype),
            "q": torch.zeros(taps - 1, G * d, dtype=dtype), "k": torch.zeros(taps - 1, G * d, dtype=dtype),
            "v": torch.zeros(taps - 1, H * dv, dtype=dtype)}


def short_conv(x: torch.Tensor, taps_w: torch.Tensor, tail: torch.Tensor) -> (torch.Tensor, torch.Tensor):
    """``y_t = sum_j w[:, j] x_(t - taps + 1 + j)`` with ``tail`` standing for the inputs before ``x``; then silu.
    Returns the result and the new tail."""
    taps = taps_w.shape[1]
    full = torch.cat([tail, x])
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j:j + x.shape[0]] * taps_w[:, j]
    new_tail = full[full.shape[0] - (taps - 1):] if taps > 1 else tail
    return st(y * torch.sigmoid(y)), new_tail


def delta(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float, state: dict) -> torch.Tensor:
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q, state["q"] = short_conv(lin(h, w[p + ".q"]), w[p + ".q.conv"], state["q"])
    k, state["k"] = short_conv(lin(h, w[p + ".k"]), w[p + ".k.conv"], state["k"])
    v, state["v"] = short_conv(lin(h, w[p + ".v"]), w[p + ".v.conv"], state["v"])
    q, k, v = q.view(T, G, d), k.view(T, G, d), v.view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + ".b"].T)
    step = F.softplus(lin(h, w[p + ".a1"]) @ w[p + ".a2"].T + w[p + ".dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(w[p + ".A_log"])[None, :, None] * step)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            c = a // (H // G)
            S = g[t, a][:, None] * state["S"][a]
            u = beta[t, a] * (v[t, a] - S.T @ k[t, c])
            S = S + torch.outer(k[t, c], u)
            state["S"][a] = S
            o[t, a] = S.T @ q[t, c]
    gate = torch.sigmoid(lin(lin(h, w[p + ".g1"]), w[p + ".g2"])).view(T, H, dv)
    y = unit(o, eps) * w[p + ".norm"] * gate
    return lin(st(y.reshape(T, H * dv)), w[p + ".o"])


# ---- the model ------------------------------------------------------------------------------------------------------
class Walker:
    """One sequence's state; ``feed(tokens)`` runs them after what was fed before and returns logits ``[T, vocab]``
    (and the stream after every layer in ``self.streams`` if ``keep_streams``)."""

    def __init__(self, cfg: dict, w: Dict[str, torch.Tensor], dtype=torch.float64, keep_streams: bool = False) -> None:
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
        self.before = None
        self.keep_streams = keep_streams
        self.streams: List[torch.Tensor] = []
        self.state = []
        for layer in cfg["layers"]:
            m = layer["mixer"]
            if layer["type"] == "parallel":
                self.state.append({"left": {"k": None, "v": None}, "right": delta_new_state(m["right"], dtype)})
            else:
                self.state.append(mlstm_new_state(m, dtype))

    def feed(self, tokens: List[int]) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        eps, r = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
        x = embed(tokens, cfg, w, self.before)
        self.before = tokens[-1]
        self.streams = []
        for i, layer in enumerate(cfg["layers"]):
            p, m = f"l{i}", layer["mixer"]
            h = st(unit(x, eps) * w[p + ".norm1"])
            if layer["type"] == "parallel":
                mixed = (float(m["left_scale"]) * window_attention(h, m["left"], w, p + ".mix.left", self.state[i]["left"])
                         + float(m["right_scale"]) * delta(h, m["right"], w, p + ".mix.right", eps, self.state[i]["right"]))
            else:
                mixed = mlstm(h, m, w, p + ".mix", eps, self.state[i])
            x = x + r * (mixed + feed_forward(h, layer.get("mlp"), w, p + ".mlp"))
            if self.keep_streams:
                self.streams.append(x.clone())
        return lin(st(unit(x, eps) * w["final.norm"]), w["head"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64) -> torch.Tensor:
    """Logits of a whole sequence in one go."""
    return Walker(cfg, w, dtype).feed(tokens)


def decode_token_by_token(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64) -> torch.Tensor:
    walker = Walker(cfg, w, dtype)
    return torch.cat([walker.feed([t]) for t in tokens])


def random_weights(cfg: dict, seed: int, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Weights of a model of this design by checkpoint name (float32; the integer table has none here)."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])

    def mat(*shape, s=std):
        return torch.randn(*shape, generator=g) * s

    def near_one(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g)

    def expert_of(p, ff):
        w[p + ".gate"], w[p + ".up"], w[p + ".down"] = mat(ff, W, s=0.15), mat(ff, W, s=0.15), mat(W, ff)

    w: Dict[str, torch.Tensor] = {"embed": mat(int(cfg["vocab"]), W, s=1.0), "final.norm": near_one(W), "head": mat(int(cfg["vocab"]), W)}
    if cfg.get("embedding", {}).get("bigram"):
        w["bigram"] = mat(int(cfg["embedding"]["bigram"]["buckets"]) + 1, W, s=0.5)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        w[p + ".norm1"] = near_one(W)
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            q = p + ".mix.left"
            w[q + ".q"], w[q + ".k"] = mat(a["heads"] * a["dim"], W, s=0.3), mat(a["kv_heads"] * a["dim"], W, s=0.3)
            w[q + ".v"], w[q + ".o"] = mat(a["kv_heads"] * a["vdim"], W), mat(W, a["heads"] * a["vdim"])
            q = p + ".mix.right"
            for name, rows in (("q", b["kv_heads"] * b["dim"]), ("k", b["kv_heads"] * b["dim"]), ("v", b["heads"] * b["vdim"])):
                w[f"{q}.{name}"] = mat(rows, W, s=0.2)
                w[f"{q}.{name}.conv"] = mat(rows, b["conv"], s=0.5)
            rank = 6
            w[q + ".b"], w[q + ".A_log"] = mat(b["heads"], W, s=0.2), mat(b["heads"], s=0.5)
            w[q + ".a1"], w[q + ".a2"], w[q + ".dt_bias"] = mat(rank, W, s=0.2), mat(b["heads"] * b["dim"], rank, s=0.5), mat(b["heads"] * b["dim"], s=0.5) - 2.0
            w[q + ".g1"], w[q + ".g2"] = mat(rank, W, s=0.2), mat(b["heads"] * b["vdim"], rank, s=0.5)
            w[q + ".norm"], w[q + ".o"] = near_one(b["vdim"]), mat(W, b["heads"] * b["vdim"])
        else:
            q = p + ".mix"
            w[q + ".q"], w[q + ".k"] = mat(m["heads"] * m["dim"], W, s=0.2), mat(m["heads"] * m["dim"], W, s=0.2)
            w[q + ".v"], w[q + ".g"] = mat(m["heads"] * m["vdim"], W), mat(m["heads"] * m["vdim"], W)
            w[q + ".o"], w[q + ".norm"] = mat(W, m["heads"] * m["vdim"]), near_one(m["heads"] * m["vdim"])
            w[q + ".i"], w[q + ".i.b"] = mat(m["heads"], W, s=0.3), mat(m["heads"], s=1.0)
            w[q + ".f"], w[q + ".f.b"] = mat(m["heads"], W, s=0.3), mat(m["heads"], s=1.0) + 2.0
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        q = p + ".mlp"
        if mlp.get("kind", "dense") == "dense":
            expert_of(q, mlp["ff"])
        else:
            r = mlp["router"]
            for e in range(r["experts"]):
                expert_of(f"{q}.e{e}", mlp["expert"]["ff"])
            n = r["experts"] + r.get("identity", 0)
            w[q + ".router"], w[q + ".correction"] = mat(n, W, s=0.3), mat(n, s=0.05)
            if mlp.get("shared"):
                expert_of(q + ".shared", mlp["shared"]["ff"])
    return w
