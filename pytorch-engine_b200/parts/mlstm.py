"""A matrix-memory recurrence with exponential gates (the mLSTM cell of xLSTM; the kernel and its formulas:
csrc/mlstm.cu).

For a token with input ``h``, per head with key size ``d`` and value size ``dv``:

    q = W_q h / sqrt(d) ;  k = W_k h ;  v = W_v h
    i = cap tanh((w_i . h + b_i) / cap) ;  f = logsigmoid(cap tanh((w_f . h + b_f) / cap))
    m' = max(f + m, i) ;  S' = e^(f + m - m') S + e^(i - m') k v^T ;  n' = e^(f + m - m') n + e^(i - m') k
    o  = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
    out = W_o (o / rms_per_head(o) * norm * sigmoid(W_g h))

What a sequence keeps between steps is of fixed size: every head's ``S [d, dv]``, ``n [d]`` and ``m``, float32 (a
"state" entry of the cache, zero when a slot is taken: the running maximum starts at 0).  Gates, state and the
per-head norm are float32 in every run dtype; the gate pre-activations come from a product that writes float32.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .linear import fuse_rows
from .registry import register
from .spec import CacheRequest, WeightDecl


# tokens per chunk when a prompt is cut into chunks that run side by side; steps whose longest sequence has no more
# tokens than two chunks walk each sequence in one go
CHUNK_TOKENS = 64


@register("mixer", "mlstm")
class MlstmMixer:
    """params: ``hidden``, ``n_heads``, ``head_dim``, ``v_head_dim``, ``gate_cap``, ``eps`` (of the per-head norm).
    weights: ``q_proj, k_proj [heads*head_dim, hidden]``, ``v_proj, g_proj [heads*v_head_dim, hidden]``, ``i_proj,
    f_proj [heads, hidden]``, ``i_bias, f_bias [heads]``, ``norm [heads*v_head_dim]``, ``o_proj [hidden,
    heads*v_head_dim]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, nh, d, dv = (int(params[k]) for k in ("hidden", "n_heads", "head_dim", "v_head_dim"))
        return {"q_proj": WeightDecl((nh * d, h)), "k_proj": WeightDecl((nh * d, h)), "v_proj": WeightDecl((nh * dv, h)),
                "g_proj": WeightDecl((nh * dv, h)), "i_proj": WeightDecl((nh, h)), "f_proj": WeightDecl((nh, h)),
                "i_bias": WeightDecl((nh,)), "f_bias": WeightDecl((nh,)), "norm": WeightDecl((nh * dv,), "norm"),
                "o_proj": WeightDecl((h, nh * dv))}

    @classmethod
    def cache_request(cls, params) -> Optional[CacheRequest]:
        nh, d, dv = (int(params[k]) for k in ("n_heads", "head_dim", "v_head_dim"))
        return CacheRequest(kind="state", state_shapes=(("S", (nh, d, dv), "float32"), ("n", (nh, d), "float32"),
                                                        ("m", (nh,), "float32")))

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.n_heads = int(params["n_heads"])
        self.head_dim = int(params["head_dim"])
        self.v_dim = int(params["v_head_dim"])
        self.cap = float(params["gate_cap"])
        self.eps = float(params.get("eps", 1e-5))
        in_registers = self.head_dim <= 32 or (self.head_dim <= 64 and self.v_dim <= 512) or (self.head_dim <= 128 and self.v_dim <= 256)
        if self.v_dim > 1024 or (not in_registers and (self.head_dim * self.v_dim + 3 * self.head_dim) * 4 > 200 * 1024):
            raise ValueError(f"a head of {self.head_dim} x {self.v_dim} is beyond what the recurrence kernel keeps on chip")
        f32 = torch.float32
        self.qkvg = fuse_rows(runtime, [weights["q_proj"], weights["k_proj"], weights["v_proj"], weights["g_proj"]])
        self.gates = fuse_rows(runtime, [weights["i_proj"], weights["f_proj"]])
        self.gate_bias = torch.cat([weights["i_bias"].to(device=runtime.device, dtype=f32),
                                    weights["f_bias"].to(device=runtime.device, dtype=f32)]).contiguous()
        self.norm = runtime.adopt(weights["norm"], f32)
        self.o_proj = runtime.adopt(weights["o_proj"])

    def forward(self, x: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        if not writes_cache:
            raise ValueError("an mlstm mixer folds every token into its state; it cannot run without writing it")
        rt = self.runtime
        n = x.shape[0]
        qk, vv = self.n_heads * self.head_dim, self.n_heads * self.v_dim
        qkvg = ctx.buffer("mlstm.qkvg", (n, 2 * qk + 2 * vv), rt.dtype)
        rt.linear(x, self.qkvg, out=qkvg)
        gates = ctx.buffer("mlstm.gates", (n, 2 * self.n_heads), torch.float32)
        y = rt.linear(x, self.gates, out=gates, out_dtype=torch.float32)
        if y.data_ptr() != gates.data_ptr():
            gates.copy_(y)
        out = ctx.buffer("mlstm.out", (n, vv), rt.dtype)
        chunk, max_chunks, scratch = 0, 1, None
        if ctx.max_q > 2 * CHUNK_TOKENS:
            chunk = CHUNK_TOKENS
            max_chunks = -(-ctx.max_q // chunk)
            scratch = ctx.buffer("mlstm.scratch", (ops.mlstm_scratch_floats(ctx.n_seqs, self.n_heads, self.head_dim, self.v_dim,
                                                                          max_chunks),), torch.float32)
        ops.mlstm_recurrence(qkvg[:, :qk], qkvg[:, qk:2 * qk], qkvg[:, 2 * qk:2 * qk + vv], qkvg[:, 2 * qk + vv:], gates,
                             self.gate_bias, self.norm, self.cap, self.eps, self.head_dim ** -0.5, out, view.state("S"),
                             view.state("n"), view.state("m"), ctx.seq_slot, ctx.seq_qstart, ctx.n_seqs, ctx.max_q, self.n_heads,
                             self.head_dim, self.v_dim, rt.status, chunk, max_chunks, scratch)
        delta = ctx.buffer("mlstm.delta", (n, self.hidden), rt.dtype)
        rt.linear(out, self.o_proj, out=delta)
        return delta
