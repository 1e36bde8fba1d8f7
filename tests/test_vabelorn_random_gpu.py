"""Vabelorn configurations drawn at random (sizes that are no multiple of anything, every layer order, groups of every
size, rotation of two features or of the whole head, with and without scaled frequencies, with and without
feed-forwards and token inputs, recurrence heads on every register tile of the kernel) against the plain
implementation: a prompt in two portions, tokens one by one, and a batch of two unequal requests."""
import random

import pytest
import torch

import plain_vabelorn as plain
from test_vabelorn_gpu import DEV, Models, _entry, _tokens

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([24, 50, 64, 100, 136])
    layers = []
    for _ in range(rng.randint(1, 4)):
        mlp = {"kind": "dense", "ff": rng.choice([30, 64, 100])} if rng.random() < 0.6 else None
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([6, 10, 16, 24, 40, 64, 72])
            rot = {"base": rng.choice([50.0, 1000.0, 1e5]), "dims": rng.randrange(2, dim + 1, 2)}
            if rng.random() < 0.5:
                rot["scaling"] = {"factor": rng.choice([1.5, 4.0, 16.0]), "original": rng.choice([16, 64, 300]),
                                  "fast": rng.choice([4.0, 32.0]), "slow": rng.choice([0.5, 1.0, 2.0])}
            layers.append({"type": "attention",
                           "mixer": {"heads": kv * rng.choice([1, 2, 5]), "kv_heads": kv, "dim": dim,
                                     "vdim": rng.choice([dim, dim, 4, 14, 32]), "scale": rng.choice([0.1, 0.3, dim ** -0.5]), "rot": rot},
                           "mlp": mlp})
        else:
            layers.append({"type": "wkv", "mixer": {"heads": rng.choice([1, 2, 3]), "dim": rng.choice([8, 20, 32, 48, 64, 100, 128, 160]),
                                                    "decay_rank": rng.choice([3, 8, 16])}, "mlp": mlp})
    cfg = {"architecture": "Vabelorn", "vocab": rng.choice([37, 128, 301]), "width": width,
           "logit_scale": rng.choice([0.25, 1.0, 3.0]), "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["token_side"] = {"dim": rng.choice([2, 5, 8, 16])}
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(8)))
def test_a_configuration_drawn_at_random(pe, seed, dtype):
    import test_vabelorn_gpu as base

    key = f"random{seed}"
    base.CONFIGS[key] = draw_config(seed)
    base.SEEDS[key] = 100 + seed
    try:
        models = Models(pe)
        eng = models.engine(key, dtype, max_context_len=512, max_cache_tokens=64 * 24)
        vocab = base.CONFIGS[key]["vocab"]
        a, b = _tokens(vocab, 210, seed), _tokens(vocab, 37, seed + 50)
        s = eng.alloc_slot()
        rows = [eng.step([_entry(pe, s, a[:139], range(139))]).clone(), eng.step([_entry(pe, s, a[139:200], range(61))]).clone()]
        for t in a[200:]:
            rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
        eng.free_slot(s)
        models.check(key, dtype, a, torch.cat(rows), range(210), f"seed {seed}: portions and single tokens")
        s1, s2 = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([_entry(pe, s1, b[:30], [29]), _entry(pe, s2, a[:150], [149])]).clone()
        got_b, got_a = [out[0:1]], [out[1:2]]
        for i in range(30, 37):
            out = eng.step([_entry(pe, s1, [b[i]], [0]), _entry(pe, s2, [a[120 + i]], [0])]).clone()
            got_b.append(out[0:1])
            got_a.append(out[1:2])
        eng.free_slot(s1)
        eng.free_slot(s2)
        models.check(key, dtype, b, torch.cat(got_b), range(29, 37), f"seed {seed}: the short request of a batch")
        models.check(key, dtype, a[:157], torch.cat(got_a), range(149, 157), f"seed {seed}: the long request of a batch")
        assert eng.runtime.status.tolist()[0] == 0
        eng.cache.check()
    finally:
        del base.CONFIGS[key], base.SEEDS[key]
