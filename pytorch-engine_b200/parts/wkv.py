"""A linear-recurrence mixer with a matrix state per head: RWKV-style "wkv" time mixing with a
data-dependent decay (the kernels and their formulas: csrc/wkv.cu).

For a token with input ``h`` and the previous token's input ``h'`` (zeros before a sequence's first token):

    m_s  = h + (h' - h) * mu_s                       s in r, k, v, g, w
    r, k, v = W_r m_r, W_k m_k, W_v m_v              heads x head_dim each
    w    = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))       the decay, per head and key channel
    o    = (S + diag(u) k v^T)^T r ;  S <- diag(w) S + k v^T
    out  = W_o (o / rms_per_head(o) * gnorm * silu(W_g m_g))

What a sequence keeps between steps is of fixed size: ``h'`` and every head's ``S``, both float32 (a "state" entry
of the cache: zero when a slot is taken).  The recurrence, the decay and the per-head norm are float32 in every
run dtype; the matrix products run in the run dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .registry import register
from .spec import CacheRequest, WeightDecl

MIXES = ("r", "k", "v", "g", "w")
# tokens per chunk when a prompt is cut into chunks that run side by side; steps whose longest sequence has no more
# tokens than two chunks walk each sequence in one go
CHUNK_TOKENS = 64


@register("mixer", "wkv")
class WkvMixer:
    """params: ``hidden``, ``n_heads``, ``head_dim``, ``eps`` (of the per-head norm), ``decay_rank`` (rank of the
    decay's projection in a random model; a checkpoint's own tensors decide it).  weights: ``mu_r .. mu_w
    [hidden]``, ``r_proj, k_proj, v_proj, g_proj [heads*head_dim, hidden]``, ``w1 [rank, hidden]``, ``w2
    [heads*head_dim, rank]``, ``w0 [heads*head_dim]``, ``u [heads, head_dim]``, ``gnorm [heads*head_dim]``,
    ``o_proj [hidden, heads*head_dim]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, d = (int(params[k]) for k in ("hidden", "n_heads", "head_dim"))
        rank = int(params.get("decay_rank", 16))
        decls = {f"mu_{s}": WeightDecl((h,), "unit") for s in MIXES}
        for s in "rkvg":
            decls[f"{s}_proj"] = WeightDecl((nh * d, h))
        decls["w1"] = WeightDecl((rank, h), any_dims=(0,))
        decls["w2"] = WeightDecl((nh * d, rank), any_dims=(1,))
        decls["w0"] = WeightDecl((nh * d,))
        decls["u"] = WeightDecl((nh, d))
        decls["gnorm"] = WeightDecl((nh * d,), "norm")
        decls["o_proj"] = WeightDecl((h, nh * d))
        return decls

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        h, nh, d = (int(params[k]) for k in ("hidden", "n_heads", "head_dim"))
        return CacheRequest(kind="state", state_shapes=(("prev", (h,), "float32"), ("S", (nh, d, d), "float32")))

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.n_heads = int(params["n_heads"])
        self.head_dim = int(params["head_dim"])
        if self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is beyond what the recurrence kernel takes (<= 256)")
        self.eps = float(params.get("eps", 1e-5))
        self.inner = self.n_heads * self.head_dim
        f32 = torch.float32
        self.mu = torch.stack([weights[f"mu_{s}"].to(device=runtime.device, dtype=f32) for s in MIXES]).contiguous()
        # r, k, v, g stacked: one grouped launch for a handful of rows, one batched product otherwise
        self.proj = torch.stack([weights[f"{s}_proj"].to(device=runtime.device, dtype=runtime.dtype) for s in "rkvg"]).contiguous()
        self.w1 = runtime.adopt(weights["w1"])
        self.w2 = runtime.adopt(weights["w2"])
        if self.w1.shape[0] != self.w2.shape[1]:
            raise ValueError(f"the decay's two projections do not fit: w1 {tuple(self.w1.shape)}, w2 {tuple(self.w2.shape)}")
        self.rank = int(self.w1.shape[0])
        self.w0 = runtime.adopt(weights["w0"], f32)
        self.u = runtime.adopt(weights["u"], f32).reshape(-1)
        self.gnorm = runtime.adopt(weights["gnorm"], f32)
        self.o_proj = runtime.adopt(weights["o_proj"])

    def project(self, mixes: torch.Tensor, n: int, ctx):
        """r, k, v, g (views with one row stride) from the first four mixes: each mix times its own matrix."""
        rt = self.runtime
        stacked = self.proj.view(4 * self.inner, self.hidden)
        xs = mixes[:4]
        if (rt.gemm_backend is None and rt.own_small_gemm and n <= rt.small_gemm_rows
                and ops.gemm_smallm_grouped_supported(xs, stacked, self.inner)):
            out = ctx.buffer("wkv.rkvg", (n, 4 * self.inner), rt.dtype)
            ops.gemm_smallm_grouped(xs, stacked, out, self.inner)
            return [out[:, i * self.inner:(i + 1) * self.inner] for i in range(4)]
        if rt.gemm_backend is None:
            out = ctx.buffer("wkv.rkvg", (4, n, self.inner), rt.dtype)
            rt.batched_linear(xs, self.proj, out)
            return [out[i] for i in range(4)]
        outs = [ctx.buffer(f"wkv.{s}", (n, self.inner), rt.dtype) for s in "rkvg"]
        for i in range(4):
            rt.linear(mixes[i], self.proj[i], out=outs[i])
        return outs

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("a wkv mixer folds every token into its state; it cannot run without writing it")
        rt = self.runtime
        n = x.shape[0]
        prev, state = view.state("prev"), view.state("S")
        mixes = ctx.buffer("wkv.mixes", (len(MIXES), n, self.hidden), rt.dtype)
        ops.token_shift_mix(x, self.mu, prev, ctx.token_seq, ctx.seq_slot, ctx.seq_qstart, mixes, rt.status)
        rkvg = self.project(mixes, n, ctx)
        low = ctx.buffer("wkv.low", (n, self.rank), rt.dtype)
        rt.linear(mixes[4], self.w1, out=low)
        ops.tanh_(low)
        wlin = ctx.buffer("wkv.wlin", (n, self.inner), torch.float32)
        y = rt.linear(low, self.w2, out=wlin, out_dtype=torch.float32)
        if y.data_ptr() != wlin.data_ptr():
            wlin.copy_(y)
        out = ctx.buffer("wkv.out", (n, self.inner), rt.dtype)
        chunk, max_chunks, scratch = 0, 1, None
        if ctx.max_q > 2 * CHUNK_TOKENS:
            chunk = CHUNK_TOKENS
            max_chunks = -(-ctx.max_q // chunk)
            scratch = ctx.buffer("wkv.scratch", (ops.wkv_scratch_floats(ctx.n_seqs, self.n_heads, self.head_dim, max_chunks),),
                                 torch.float32)
        ops.wkv_recurrence(*rkvg, wlin, self.w0, self.u, self.gnorm, self.eps, out, state, prev, x, ctx.seq_slot,
                           ctx.seq_qstart, ctx.n_seqs, ctx.max_q, self.n_heads, self.head_dim, chunk, max_chunks, scratch,
                           rt.status)
        delta = ctx.buffer("wkv.delta", (n, self.hidden), rt.dtype)
        rt.linear(out, self.o_proj, out=delta)
        return delta
