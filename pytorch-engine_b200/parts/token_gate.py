"""A per-layer token input: a narrow second embedding of the token itself, gated by the residual stream.

    e = table[token, col0 : col0 + dim] ;  y = P (gelu_tanh(G x) * e)

``table`` is one tensor ``[vocab, n_layers * dim]`` of which every layer reads its own columns; ``G [dim, hidden]``
and ``P [hidden, dim]`` belong to the layer.  The part is a feed-forward by interface (``forward(x, ctx) -> delta``);
the block arrangement norms and adds what it returns.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .registry import register
from .spec import WeightDecl


@register("feed_forward", "token_gate")
class TokenGatedInput:
    """params: ``hidden``, ``dim``, ``vocab``, ``table_width``, ``col0``.  weights: ``table [vocab, table_width]``,
    ``gate [dim, hidden]``, ``proj [hidden, dim]``."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    @classmethod
    def weight_decls(cls, params) -> Dict[str, WeightDecl]:
        h, d = int(params["hidden"]), int(params["dim"])
        return {"table": WeightDecl((int(params["vocab"]), int(params["table_width"])), "embedding"),
                "gate": WeightDecl((d, h)), "proj": WeightDecl((h, d))}

    def __init__(self, params, weights, runtime) -> None:
        self.runtime = runtime
        self.hidden = int(params["hidden"])
        self.dim = int(params["dim"])
        self.col0 = int(params["col0"])
        if self.col0 < 0 or self.col0 + self.dim > int(params["table_width"]):
            raise ValueError("the layer's columns lie outside the token table")
        self.table = runtime.adopt(weights["table"])
        self.gate = runtime.adopt(weights["gate"])
        self.proj = runtime.adopt(weights["proj"])

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        rt = self.runtime
        n = x.shape[0]
        gx = ctx.buffer("side.gx", (n, self.dim), rt.dtype)
        rt.linear(x, self.gate, out=gx)
        gated = ctx.buffer("side.gated", (n, self.dim), rt.dtype)
        ops.token_gate(gx, self.table, self.col0, ctx.tokens, gated, rt.status)
        delta = ctx.buffer("side.delta", (n, self.hidden), rt.dtype)
        rt.linear(gated, self.proj, out=delta)
        return delta
