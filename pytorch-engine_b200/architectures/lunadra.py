"""The Lunadra decoder as a plan of parts.

The embedding adds a hashed embedding of the pair (previous token, token) to the token's own
(``token_pair_embedding``).  Every block is a ``parallel`` arrangement (``parts/block.py``): one RMS norm feeds the
mixer and the feed-forward, and ``residual_mult`` times their sum is added to the stream.  Layer by layer ``config.json``
chooses

* ``mlstm`` (also written ``mlstm_<n>``): a matrix-memory recurrence with exponential gates (``parts/mlstm.py``);
* ``parallel``: two mixers side by side on the same input, weighted ``left_scale`` and ``right_scale``: grouped-query
  softmax attention with a sliding window and split-half rotary encoding of the first ``rot.dims`` features
  (``parts/attention.py``), and the gated delta rule behind short convolutions (``parts/delta_rule.py``);

and a feed-forward: none, a dense one with ``relu(gate) * up``, or routed experts with a clamped swish activation,
identity experts and a shared expert (``parts/moe.py``).  Final RMS norm, then an output head of its own.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``; ``l<i>.mix.{q,k,v,g,o,norm,i,f}``
and ``l<i>.mix.{i,f}.b`` (mlstm); ``l<i>.mix.left.{q,k,v,o}``, ``l<i>.mix.right.{q,k,v,b,o,norm,A_log,a1,a2,dt_bias,g1,g2}``
and ``l<i>.mix.right.{q,k,v}.conv`` (parallel); ``l<i>.mlp.{gate,up,down}`` (dense); ``l<i>.mlp.{router,correction}``,
``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down}`` (routed).
"""
from __future__ import annotations

from ..config.lunadra import DenseFf, LunadraConfig
from ..config.registry import register_architecture
from ..parts.spec import BlockSpec, ModelPlan, PartSpec, RunStep

# the factor inside the experts' swish, g * sigmoid(SWISH_ALPHA * g)
SWISH_ALPHA = 1.702


def lunadra_plan(cfg: LunadraConfig) -> ModelPlan:
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
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        m = layer.mixer
        parts = {"norm": ("norm", norm(f"{p}.norm1"))}
        params = {"mult": cfg.residual_mult}
        if layer.type == "parallel":
            a, b = m.left, m.right
            pos = None
            if a.rot_dims > 0:
                pos = position(PartSpec("rope", {"rotary_dim": a.rot_dims, "theta": a.rot_base, "style": "neox", "scaling": None,
                                                 "max_positions": cfg.max_positions, "exact": True}))
            q = f"{p}.mix.left"
            parts["left"] = ("mixer", PartSpec(
                "attention",
                {"hidden": h, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
                 "qk_norm": False, "eps": eps, "scale": a.scale, "window": a.window, "position": pos},
                {"q_proj": f"{q}.q", "k_proj": f"{q}.k", "v_proj": f"{q}.v", "o_proj": f"{q}.o"}))
            q = f"{p}.mix.right"
            parts["right"] = ("mixer", PartSpec(
                "gated_delta",
                {"hidden": h, "n_heads": b.heads, "n_kv_heads": b.kv_heads, "head_dim": b.dim, "v_head_dim": b.vdim,
                 "conv": b.conv, "eps": eps, "rank": b.rank},
                {"q_proj": f"{q}.q", "k_proj": f"{q}.k", "v_proj": f"{q}.v", "q_conv": f"{q}.q.conv", "k_conv": f"{q}.k.conv",
                 "v_conv": f"{q}.v.conv", "b_proj": f"{q}.b", "A_log": f"{q}.A_log", "a1": f"{q}.a1", "a2": f"{q}.a2",
                 "dt_bias": f"{q}.dt_bias", "g1": f"{q}.g1", "g2": f"{q}.g2", "norm": f"{q}.norm", "o_proj": f"{q}.o"}))
            params["mixer_weights"] = {"left": m.left_scale, "right": m.right_scale}
        else:
            q = f"{p}.mix"
            parts["mixer"] = ("mixer", PartSpec(
                "mlstm",
                {"hidden": h, "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "gate_cap": m.gate_cap, "eps": eps},
                {"q_proj": f"{q}.q", "k_proj": f"{q}.k", "v_proj": f"{q}.v", "g_proj": f"{q}.g", "i_proj": f"{q}.i",
                 "f_proj": f"{q}.f", "i_bias": f"{q}.i.b", "f_bias": f"{q}.f.b", "norm": f"{q}.norm", "o_proj": f"{q}.o"}))
        mlp = layer.mlp
        q = f"{p}.mlp"
        if isinstance(mlp, DenseFf):
            parts["ffn"] = ("feed_forward", PartSpec(
                "swiglu", {"hidden": h, "intermediate": mlp.ff, "activation": "relu"},
                {"gate_proj": f"{q}.gate", "up_proj": f"{q}.up", "down_proj": f"{q}.down"}))
        elif mlp is not None:
            names = {"router": f"{q}.router", "correction": f"{q}.correction"}
            for e in range(mlp.experts):
                names.update({f"e{e}.{s}": f"{q}.e{e}.{s}" for s in ("gate", "up", "down")})
            shared = None
            if mlp.shared is not None:
                shared = {"intermediate": mlp.shared.ff, "activation": "clamped_swish", "limit": mlp.shared.limit,
                          "alpha": SWISH_ALPHA}
                names.update({f"shared.{s}": f"{q}.shared.{s}" for s in ("gate", "up", "down")})
            parts["ffn"] = ("feed_forward", PartSpec(
                "routed_experts",
                {"hidden": h, "n_experts": mlp.experts, "n_identity": mlp.identity, "top": mlp.top, "intermediate": mlp.expert.ff,
                 "activation": "clamped_swish", "limit": mlp.expert.limit, "alpha": SWISH_ALPHA, "shared": shared}, names))
        blocks.append(BlockSpec("parallel", parts, name=f"layer {i}", params=params))
    if cfg.pairs is not None:
        embedding = PartSpec("token_pair_embedding",
                             {"vocab": cfg.vocab, "hidden": h, "buckets": cfg.pairs.buckets, "mul_prev": cfg.pairs.mul_prev,
                              "mul_cur": cfg.pairs.mul_cur}, {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("token_embedding", {"vocab": cfg.vocab, "hidden": h}, {"weight": "embed"})
    return ModelPlan(
        hidden_size=h,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=embedding,
        blocks=tuple(blocks),
        order=tuple(RunStep(block=i) for i in range(len(cfg.layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": h}, {"weight": "head"}),
        positions=positions,
    )


register_architecture("Lunadra", LunadraConfig, lunadra_plan, replace=True)
