"""The Vabelorn decoder as a plan of parts.

A stack of post-norm blocks, each with its own mixer, chosen layer by layer in ``config.json``:

* ``attention``: grouped-query attention with q/k RMS norm, interleaved rotary encoding of the first ``rot.dims``
  features with YaRN-scaled frequencies, values divided by their root mean square and rotated by their own position
  (each head's output is turned back by the query's position), and a sink in the softmax
  (``parts/attention.py`` with ``sink``, ``v_norm``, ``value_position``, ``v_head_dim``);
* ``wkv``: a linear recurrence with a matrix state per head and a data-dependent decay (``parts/wkv.py``);

an optional SwiGLU feed-forward, and a per-layer token input (``parts/token_gate.py``).  Every sublayer's output
goes through an RMS norm before it is added (``post_norm`` in ``parts/block.py``).  The head is the embedding
table, its logits times ``logit_scale``.

Tensor names: ``embed``, ``side.embed``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q,k,v,o}``, ``l<i>.mix.{q,k}.norm`` (attention); ``l<i>.mix.mu.{r,k,v,g,w}``, ``l<i>.mix.{r,k,v,g,o}``,
``l<i>.mix.{w1,w2,w0,u,norm}`` (wkv); ``l<i>.mlp.{gate,up,down}``; ``l<i>.side.{gate,proj,norm}``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vabelorn import VabelornConfig
from ..parts.spec import BlockSpec, ModelPlan, PartSpec, RunStep


def vabelorn_plan(cfg: VabelornConfig) -> ModelPlan:
    h, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"dim": h, "eps": eps}, {"weight": name})
    positions = {}

    def position(spec: PartSpec) -> str:
        """One position encoding per distinct set of constants, shared by the layers that use it."""
        key = repr(sorted((k, repr(v)) for k, v in spec.params.items()))
        for name, have in positions.items():
            if repr(sorted((k, repr(v)) for k, v in have.params.items())) == key:
                return name
        name = f"rot{len(positions)}"
        positions[name] = spec
        return name

    blocks = []
    n_layers = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        m = layer.mixer
        if layer.type == "attention":
            scaling = None
            if m.rot.scaling is not None:
                s = m.rot.scaling
                scaling = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            qk_pos = None
            if m.rot.dims > 0:
                qk_pos = position(PartSpec("rope", {"rotary_dim": m.rot.dims, "theta": m.rot.base, "style": "interleaved",
                                                    "scaling": scaling, "max_positions": cfg.max_positions}))
            v_pos = position(PartSpec("rope", {"rotary_dim": m.vdim, "theta": m.rot.base, "style": "interleaved",
                                               "scaling": None, "max_positions": cfg.max_positions}))
            mixer = PartSpec(
                "attention",
                {"hidden": h, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                 "qk_norm": True, "eps": eps, "scale": m.scale, "window": None, "position": qk_pos, "sink": True,
                 "v_norm": "unit", "value_position": v_pos},
                {"q_proj": f"{p}.mix.q", "k_proj": f"{p}.mix.k", "v_proj": f"{p}.mix.v", "o_proj": f"{p}.mix.o",
                 "q_norm": f"{p}.mix.q.norm", "k_norm": f"{p}.mix.k.norm"})
        else:
            names = {f"mu_{s}": f"{p}.mix.mu.{s}" for s in "rkvgw"}
            names.update({f"{s}_proj": f"{p}.mix.{s}" for s in "rkvgo"})
            names.update({"w1": f"{p}.mix.w1", "w2": f"{p}.mix.w2", "w0": f"{p}.mix.w0", "u": f"{p}.mix.u",
                          "gnorm": f"{p}.mix.norm"})
            mixer = PartSpec("wkv", {"hidden": h, "n_heads": m.heads, "head_dim": m.dim, "eps": eps,
                                     "decay_rank": m.decay_rank}, names)
        parts = {"mixer_norm": ("norm", norm(f"{p}.norm1")), "mixer": ("mixer", mixer)}
        if layer.mlp is not None:
            parts["ffn_norm"] = ("norm", norm(f"{p}.norm2"))
            parts["ffn"] = ("feed_forward", PartSpec(
                "swiglu", {"hidden": h, "intermediate": layer.mlp.ff},
                {"gate_proj": f"{p}.mlp.gate", "up_proj": f"{p}.mlp.up", "down_proj": f"{p}.mlp.down"}))
        if cfg.token_side_dim:
            ds = cfg.token_side_dim
            parts["side_norm"] = ("norm", norm(f"{p}.side.norm"))
            parts["side"] = ("feed_forward", PartSpec(
                "token_gate", {"hidden": h, "dim": ds, "vocab": cfg.vocab, "table_width": n_layers * ds, "col0": i * ds},
                {"table": "side.embed", "gate": f"{p}.side.gate", "proj": f"{p}.side.proj"}))
        blocks.append(BlockSpec("post_norm", parts, name=f"layer {i}"))
    return ModelPlan(
        hidden_size=h,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": h}, {"weight": "embed"}),
        blocks=tuple(blocks),
        order=tuple(RunStep(block=i) for i in range(n_layers)),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": h, "scale": cfg.logit_scale}, {"weight": "embed"}),
        positions=positions,
    )


register_architecture("Vabelorn", VabelornConfig, vabelorn_plan, replace=True)
