"""What needs no GPU of the Lunadra architecture: its configuration file, its plan and tensor names, the cache entries
its parts ask for, and the plain implementation's own consistency (a sequence at once against the same sequence token
by token and in portions)."""
import copy
from importlib import import_module

import pytest
import torch

import plain_lunadra as plain

CFG = {"architecture": "Lunadra", "vocab": 83, "width": 40, "residual_mult": 0.75, "norm": {"eps": 1e-5},
       "embedding": {"bigram": {"buckets": 53, "mul_prev": 4, "mul_cur": 7}},
       "layers": [
           {"type": "parallel",
            "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 9},
                               "rot": {"base": 1000.0, "dims": 8}},
                      "right": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3},
                      "left_scale": 0.5, "right_scale": 1.5},
            "mlp": {"kind": "moe", "router": {"experts": 5, "identity": 2, "top": 3}, "expert": {"ff": 16, "limit": 1.0},
                    "shared": {"ff": 24, "limit": 2.0}}},
           {"type": "mlstm_2", "mixer": {"heads": 2, "dim": 8, "vdim": 16, "gate_cap": 9.0}, "mlp": {"kind": "dense", "ff": 32}},
           {"type": "mlstm", "mixer": {"heads": 1, "dim": 16, "vdim": 8, "gate_cap": 12.0}, "mlp": None}]}


def test_config_reads_every_layer_by_itself_and_writes_it_back(pe):
    cfg = pe.LunadraConfig.from_dict(CFG)
    left, right = cfg.layers[0].mixer.left, cfg.layers[0].mixer.right
    assert (left.window, left.rot_dims, left.vdim, right.conv, right.kv_heads) == (9, 8, 20, 3, 2)
    assert cfg.layers[0].mlp.identity == 2 and cfg.layers[0].mlp.shared.limit == 2.0
    assert cfg.layers[1].type == "mlstm" and cfg.layers[1].name == "mlstm_2" and cfg.layers[2].mlp is None
    assert cfg.pairs.buckets == 53 and cfg.residual_mult == 0.75
    assert pe.LunadraConfig.from_dict(cfg.to_dict()) == cfg
    assert pe.config.architecture_of(CFG).name == "Lunadra"
    for path, value, word in [(("layers", 0, "type"), "conv", "type"), (("layers", 0, "mixer", "left", "kv_heads"), 3, "multiple"),
                              (("layers", 0, "mixer", "left", "rot", "dims"), 14, "dims"), (("layers", 0, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 0, "mlp", "router", "top"), 8, "top"), (("norm",), None, "norm"),
                              (("layers", 1, "mixer", "gate_cap"), 0, "gate_cap"), (("layers", 0, "mixer", "right", "conv"), 0, "conv")]:
        bad = copy.deepcopy(CFG)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(pe.ConfigError, match=word):
            pe.LunadraConfig.from_dict(bad)
    # a model without a pair table and without windows is one too
    plainer = copy.deepcopy(CFG)
    del plainer["embedding"], plainer["layers"][0]["mixer"]["left"]["mask"]
    cfg2 = pe.LunadraConfig.from_dict(plainer)
    assert cfg2.pairs is None and cfg2.layers[0].mixer.left.window is None
    assert pe.config.architecture("Lunadra").plan(cfg2).embedding.kind == "token_embedding"


def test_plan_names_the_tensors_of_the_plain_implementation(pe):
    loader = import_module("pytorch-engine_b200.weights.loader")
    cfg = pe.LunadraConfig.from_dict(CFG)
    plan = pe.config.architecture("Lunadra").plan(cfg)
    want = loader.expected_tensors(plan)
    have = plain.random_weights(CFG, 0)
    assert set(want) == set(have)
    for name, decl in want.items():
        assert decl.fits(have[name].shape), name
    assert [b.arrangement for b in plan.blocks] == ["parallel"] * 3
    assert plan.blocks[0].mixer_names() == ("left", "right") and plan.blocks[1].mixer_names() == ("mixer",)
    assert plan.blocks[0].params["mixer_weights"] == {"left": 0.5, "right": 1.5} and plan.blocks[2].params["mult"] == 0.75
    assert "ffn" not in plan.blocks[2].parts and plan.blocks[0].part("ffn").kind == "routed_experts"
    assert plan.blocks[1].part("ffn").params["activation"] == "relu"
    assert plan.embedding.kind == "token_pair_embedding" and len(plan.positions) == 1


def test_cache_entries_of_the_parts(pe):
    """Windowed keys and values for the attention, fixed-size float32 state for the recurrences (with the convolutions'
    last inputs), one kept token for the pair embedding; a slot that is taken again starts from zeros."""
    parts = pe.parts
    reqs = {}
    cfg = pe.LunadraConfig.from_dict(CFG)
    plan = pe.config.architecture("Lunadra").plan(cfg)
    for i, b in enumerate(plan.blocks):
        for name in b.mixer_names():
            spec = b.part(name)
            reqs[(i, name)] = parts.lookup("mixer", spec.kind).cache_request(spec.params)
    reqs[(-1, "embedding")] = parts.lookup("embedding", plan.embedding.kind).cache_request(plan.embedding.params)
    assert reqs[(0, "left")].window == 9 and reqs[(0, "left")].value_dim == 20
    assert dict((n, s) for n, s, _ in reqs[(0, "right")].state_shapes) == {"S": (4, 8, 12), "conv": (2, 2 * 2 * 8 + 4 * 12)}
    assert dict((n, s) for n, s, _ in reqs[(1, "mixer")].state_shapes) == {"S": (2, 8, 16), "n": (2, 8), "m": (2,)}
    cache = pe.cache.PagedCache(reqs, max_tokens=256, max_slots=3, max_seq_len=128, dtype=torch.float32, device="cpu")
    s = cache.alloc_slot()
    cache.view((1, "mixer")).state("S")[s].fill_(3.0)
    cache.view((-1, "embedding")).state("last_token")[s].fill_(7)
    cache.reserve(s, 100)
    cache.commit(s, 100)
    cache.free_slot(s)
    assert cache.alloc_slot() == s
    assert float(cache.view((1, "mixer")).state("S")[s].abs().max()) == 0.0
    assert int(cache.view((-1, "embedding")).state("last_token")[s]) == 0
    cache.check()


def test_plain_implementation_whole_token_by_token_and_in_portions():
    w = plain.random_weights(CFG, 5)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, CFG["vocab"], (40,), generator=g).tolist()
    whole = plain.forward(CFG, w, toks)
    one = plain.decode_token_by_token(CFG, w, toks)
    assert (whole - one).abs().max() < 1e-9
    walker = plain.Walker(CFG, w)
    parts = torch.cat([walker.feed(toks[:7]), walker.feed(toks[7:9]), walker.feed(toks[9:])])
    assert (whole - parts).abs().max() < 1e-9
    # the window matters (a wider one gives other logits from the first position beyond it on) ...
    wider = copy.deepcopy(CFG)
    wider["layers"][0]["mixer"]["left"]["mask"]["size"] = 10
    other = plain.forward(wider, w, toks)
    assert (whole[:9] - other[:9]).abs().max() < 1e-12 and (whole[9] - other[9]).abs().max() > 1e-6
    # ... and so does the pair table: another previous token, other logits for this token only through that row
    rows = plain.bigram_rows([3, 4, 4], CFG)
    assert rows[0] == 53 and rows[1] == (3 * 4 + 4 * 7) % 53 and rows[2] == (4 * 4 + 4 * 7) % 53


def test_router_of_the_plain_implementation():
    w = {"p.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5]], dtype=torch.float64),
         "p.correction": torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64)}
    h = torch.tensor([[2.0, 0.0]], dtype=torch.float64)
    chosen, weight = plain.router(h, w, "p", 2)
    s = torch.softmax(torch.tensor([2.0, 0.0, 1.0], dtype=torch.float64), 0)
    assert chosen.tolist() == [[2, 0]] and torch.allclose(weight, s[[2, 0]][None])
