"""Block arrangements: how two norms, a mixer and a feed-forward are wired around the residual
stream.  The stream is float32; a part's output ("delta") is added to it inside the next norm's
kernel, so a block hands its last delta on instead of adding it itself."""
from __future__ import annotations

from typing import Optional

import torch

from .registry import register


@register("arrangement", "pre_norm")
class PreNormBlock:
    """``h = x + mixer(norm1(x))``; ``out = h + ffn(norm2(h))`` (pygguf_engine/model.py:1025-1042)."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.mixer_norm = parts["mixer_norm"]
        self.mixer = parts["mixer"]
        self.ffn_norm = parts["ffn_norm"]
        self.ffn = parts["ffn"]
        self.name = spec.name

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx, view, writes_cache: bool = True):
        """``stream``: float32 residual ``[N, hidden]``, updated in place; ``pending``: the previous
        block's delta that is not added yet (or None).  Returns this block's own pending delta."""
        rt = self.runtime
        normed = ctx.buffer("block.normed", tuple(stream.shape), rt.dtype)
        self.mixer_norm.add_forward(stream, pending, normed)
        if writes_cache:
            mixed = self.mixer.forward(normed, ctx, view)
        else:
            mixed = self.mixer.forward(normed, ctx, view, writes_cache=False)
        self.ffn_norm.add_forward(stream, mixed, normed)
        return self.ffn.forward(normed, ctx)


@register("arrangement", "post_norm")
class PostNormBlock:
    """Norm on what a sublayer returns, not on what it reads: ``x += norm1(mixer(x))``; ``x += norm2(ffn(x))`` if the
    block has a feed-forward; ``x += side_norm(side(x))`` if it has a token side input.  Parts by name:
    ``mixer_norm, mixer`` and optionally ``ffn_norm, ffn`` and ``side_norm, side``.  The sublayers read the stream
    itself: in a float32 run directly, otherwise through a copy in the run dtype that every add leaves behind."""

    graph_safe = True  # launches only; nothing in forward() waits for the device

    def __init__(self, spec, parts, runtime) -> None:
        self.runtime = runtime
        self.name = spec.name
        self.steps = [(parts["mixer"], parts["mixer_norm"], True)]
        if "ffn" in parts:
            self.steps.append((parts["ffn"], parts["ffn_norm"], False))
        if "side" in parts:
            self.steps.append((parts["side"], parts["side_norm"], False))

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx, view, writes_cache: bool = True):
        rt = self.runtime
        if pending is not None:       # a block before this one left its last delta to be added
            stream.add_(pending)
            ctx.stream_copy = None
        same = rt.dtype == torch.float32
        x = stream
        if not same:
            x = getattr(ctx, "stream_copy", None)
            if x is None:
                x = ctx.buffer("block.x", tuple(stream.shape), rt.dtype)
                x.copy_(stream)
        cast = None if same else ctx.buffer("block.x", tuple(stream.shape), rt.dtype)
        for part, norm, is_mixer in self.steps:
            if is_mixer:
                delta = part.forward(x, ctx, view) if writes_cache else part.forward(x, ctx, view, writes_cache=False)
            else:
                delta = part.forward(x, ctx)
            norm.add_after(stream, delta, cast)
            x = stream if same else cast
        ctx.stream_copy = None if same else cast
        return None
