"""What needs no GPU of the Vabelorn architecture: its configuration file, its plan and tensor names, the loader's
handling of a dimension that the checkpoint decides, a cache whose values have a size of their own, and the plain
implementation's own consistency (a sequence at once against the same sequence token by token)."""
import copy

import pytest
import torch

import plain_vabelorn as plain

CFG = {"architecture": "Vabelorn", "vocab": 97, "width": 40, "logit_scale": 1.5, "norm": {"eps": 1e-5},
       "token_side": {"dim": 6},
       "layers": [
           {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3,
                                           "rot": {"base": 1000.0, "dims": 8,
                                                   "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}},
            "mlp": {"kind": "dense", "ff": 64}},
           {"type": "wkv", "mixer": {"heads": 2, "dim": 16, "decay_rank": 4}, "mlp": None}]}


def test_config_reads_every_layer_by_itself_and_writes_it_back(pe):
    cfg = pe.VabelornConfig.from_dict(CFG)
    assert cfg.layers[0].mixer.vdim == 20 and cfg.layers[0].mixer.rot.scaling.factor == 4.0
    assert cfg.layers[1].type == "wkv" and cfg.layers[1].mlp is None and cfg.token_side_dim == 6
    assert pe.VabelornConfig.from_dict(cfg.to_dict()) == cfg
    assert pe.config.architecture_of(CFG).name == "Vabelorn"          # named by the string key 'architecture'
    for path, value, word in [(("layers", 0, "type"), "conv", "type"), (("layers", 0, "mixer", "kv_heads"), 3, "multiple"),
                              (("layers", 0, "mixer", "rot", "dims"), 14, "dims"), (("layers", 0, "mlp", "kind"), "moe", "kind"),
                              (("norm",), None, "norm"), (("layers", 1, "mixer", "dim"), 0, "dim")]:
        bad = copy.deepcopy(CFG)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(pe.ConfigError, match=word):
            pe.VabelornConfig.from_dict(bad)


def test_plan_names_the_tensors_of_the_plain_implementation(pe):
    from importlib import import_module
    loader = import_module("pytorch-engine_b200.weights.loader")
    cfg = pe.VabelornConfig.from_dict(CFG)
    plan = pe.config.architecture("Vabelorn").plan(cfg)
    want = loader.expected_tensors(plan)
    shapes = plain.tensor_shapes(CFG)
    assert set(want) == set(shapes)
    for name, decl in want.items():
        assert decl.fits(shapes[name]), name
    assert [b.arrangement for b in plan.blocks] == ["post_norm", "post_norm"]
    assert "ffn" in plan.blocks[0].parts and "ffn" not in plan.blocks[1].parts and "side" in plan.blocks[1].parts
    # equal constants share one position encoding; the values' rotation is one of its own
    assert len(plan.positions) == 2


def test_loader_takes_the_rank_from_the_checkpoint(pe, tmp_path):
    from safetensors.torch import load_file, save_file

    cfg = pe.VabelornConfig.from_dict(CFG)
    folder = pe.write_random_model(str(tmp_path / "m"), cfg, seed=3)
    plan = pe.config.architecture("Vabelorn").plan(cfg)
    w = pe.load_weights(folder, plan)
    assert tuple(w["l1.mix.w1"].shape) == (4, 40)
    tensors = load_file(folder + "/model.safetensors")
    tensors["l1.mix.w1"] = torch.zeros(7, 40, dtype=torch.bfloat16)           # another rank: accepted
    tensors["l1.mix.w2"] = torch.zeros(32, 7, dtype=torch.bfloat16)
    save_file(tensors, folder + "/model.safetensors")
    assert tuple(pe.load_weights(folder, plan)["l1.mix.w2"].shape) == (32, 7)
    tensors["l1.mix.w1"] = torch.zeros(7, 41, dtype=torch.bfloat16)           # another width: refused
    save_file(tensors, folder + "/model.safetensors")
    with pytest.raises(pe.WeightError) as e:
        pe.load_weights(folder, plan)
    assert [n for n, _, _ in e.value.wrong_shape] == ["l1.mix.w1"]


def test_cache_with_values_of_their_own_size_and_state(pe):
    from importlib import import_module
    spec = import_module("pytorch-engine_b200.parts.spec")
    reqs = {0: spec.CacheRequest(kind="kv", kv_heads=2, head_dim=12, v_head_dim=20),
            1: spec.CacheRequest(kind="state", state_shapes=(("prev", (40,), "float32"), ("S", (2, 16, 16), "float32"))),
            2: spec.CacheRequest(kind="kv", kv_heads=2, head_dim=12)}
    cache = pe.cache.PagedCache(reqs, max_tokens=256, max_slots=3, max_seq_len=128, dtype=torch.float32, device="cpu")
    v0, v2 = cache.view(0), cache.view(2)
    assert v0.k_pages.shape == (4, 2, 64, 12) and v0.v_pages.shape == (4, 2, 64, 20)
    assert v2.k_pages.shape == v2.v_pages.shape == (4, 2, 64, 12)
    assert v0.group is not v2.group
    s = cache.alloc_slot()
    cache.view(1).state("S")[s].fill_(3.0)
    cache.reserve(s, 70)
    cache.commit(s, 70)
    cache.free_slot(s)
    s2 = cache.alloc_slot()
    assert s2 == s and float(cache.view(1).state("S")[s2].abs().max()) == 0.0      # the state starts at zero again
    cache.check()


def test_plain_implementation_at_once_and_token_by_token():
    w = plain.random_weights(CFG, 1, sharpen=3.0)
    toks = torch.randint(0, CFG["vocab"], (40,), generator=torch.Generator().manual_seed(0)).tolist()
    a = plain.forward(CFG, w, toks)
    b = plain.decode_token_by_token(CFG, w, toks)
    assert (a - b).abs().max() < 1e-9
    # the sink: attention weights sum to less than one; without scaling the frequencies are the plain powers
    f, mult = plain.key_frequencies({"base": 100.0, "dims": 4})
    assert mult == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    f2, mult2 = plain.key_frequencies(CFG["layers"][0]["mixer"]["rot"])
    assert mult2 > 1.0 and float(f2[0]) == 1.0 and float(f2[-1]) < 1000.0 ** (-6 / 8)
