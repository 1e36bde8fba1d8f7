"""The Lunadra architecture on the engine against the plain implementation in ``plain_lunadra.py``: mechanisms at kernel
level with inputs made so that a fault shows, every mechanism alone as a one-layer model, then whole models: prompts,
token-by-token decoding, prompts in portions, unequal batches, slots and pages used again, long decoding, generation
through the entry point."""
import copy

import pytest
import torch

import plain_lunadra as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 3e-5, "bfloat16": 2e-2}


def _left(heads, kv, dim, vdim, scale, window, dims, base=10000.0):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": dims}}
    if window:
        d["mask"] = {"size": window}
    return d


def _moe(experts, identity, top, ff, limit, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


# The tests' own models.  A has sizes that are no multiple of 8 or 32 anywhere, groups of 3 and 2, a window that is no
# multiple of a page and one of exactly a page, partial and whole rotation, convolutions of 3 and 2 taps, one chosen
# expert without identity or shared experts and three chosen with both, a layer without feed-forward, a single head.
# B has the sizes that the tensor-core attention kernels take, no pair table, a multiplier of one, one tap.
CONFIGS = {
    "A": {"architecture": "Lunadra", "vocab": 131, "width": 72, "residual_mult": 0.6, "norm": {"eps": 2e-6},
          "embedding": {"bigram": {"buckets": 97, "mul_prev": 5, "mul_cur": 3}},
          "layers": [
              {"type": "parallel",
               "mixer": {"left": _left(6, 2, 16, 24, 0.3, 37, 8, 1000.0),
                         "right": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 20, "conv": 3},
                         "left_scale": 0.7, "right_scale": 1.1},
               "mlp": _moe(5, 0, 1, 40, 1.5)},
              {"type": "mlstm", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "gate_cap": 8.0}, "mlp": {"kind": "dense", "ff": 56}},
              {"type": "mlstm_2", "mixer": {"heads": 1, "dim": 40, "vdim": 12, "gate_cap": 10.0}, "mlp": None},
              {"type": "parallel",
               "mixer": {"left": _left(2, 2, 32, 32, 0.2, 64, 32, 300.0),
                         "right": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 40, "conv": 2},
                         "left_scale": 1.2, "right_scale": 0.5},
               "mlp": _moe(4, 3, 3, 24, 0.8, shared=(48, 1.2))}]},
    "B": {"architecture": "Lunadra", "vocab": 256, "width": 128, "residual_mult": 1.0, "norm": {"eps": 1e-6},
          "layers": [
              {"type": "mlstm", "mixer": {"heads": 2, "dim": 64, "vdim": 128, "gate_cap": 15.0}, "mlp": _moe(8, 2, 2, 64, 3.0, shared=(64, 3.0))},
              {"type": "parallel",
               "mixer": {"left": _left(4, 2, 64, 64, 0.125, 100, 64),
                         "right": {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 64, "conv": 1},
                         "left_scale": 1.0, "right_scale": 1.0},
               "mlp": {"kind": "dense", "ff": 256}}]},
}
SEEDS = {"A": 21, "B": 22}


def _tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _bf16_values(w):
    """Weights as a checkpoint holds them: rounded to bfloat16, so that a bfloat16 engine and the oracle start equal."""
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


class Models:
    def __init__(self, pe):
        self.pe = pe
        self.configs = dict(CONFIGS)
        self.weights = {}
        self.engines = {}
        self.refs = {}

    def add(self, key, cfg, seed):
        self.configs[key] = cfg
        SEEDS[key] = seed

    def w(self, key):
        if key not in self.weights:
            self.weights[key] = _bf16_values(plain.random_weights(self.configs[key], SEEDS[key]))
        return self.weights[key]

    def engine(self, key, dtype, **kw):
        ident = (key, dtype, tuple(sorted(kw.items())))
        if ident not in self.engines:
            cfg = self.pe.LunadraConfig.from_dict(self.configs[key])
            args = dict(dtype=dtype, max_context_len=1024, max_cache_tokens=64 * 40, max_batch=8)
            args.update(kw)
            self.engines[ident] = self.pe.Engine(None, config=cfg, weights={k: v.to(DEV) for k, v in self.w(key).items()}, **args)
        return self.engines[ident]

    def ref(self, key, toks):
        ident = (key, tuple(toks))
        if ident not in self.refs:
            self.refs[ident] = plain.forward(self.configs[key], self.w(key), toks).float()
        return self.refs[ident]

    def noise(self, key, toks):
        """How far rounding to bfloat16 alone moves each position's logits (root mean square over the vocabulary)."""
        ident = (key, tuple(toks), "noise")
        if ident not in self.refs:
            with plain.stored(torch.bfloat16):
                rounded = plain.forward(self.configs[key], self.w(key), toks)
            self.refs[ident] = (rounded - self.ref(key, toks).double()).pow(2).mean(dim=1).sqrt()
        return self.refs[ident]

    def check(self, key, dtype, toks, got, positions, what):
        """float32: every logit within 3e-5 of the largest.  bfloat16: the error is held against what rounding alone does
        in the plain implementation: on average no more than twice that, and at no more than one position in fifty (or
        one) above three times the larger of that position's own figure and the average."""
        positions = list(positions)
        ref = self.ref(key, toks)[positions]
        got = got.float().cpu()
        assert got.shape == ref.shape, what
        if dtype == "float32":
            err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
            assert err < TOL[dtype], f"{what}: error {err:.3e} (limit {TOL[dtype]:.0e})"
            return
        noise = self.noise(key, toks)
        err = (got.double() - ref.double()).pow(2).mean(dim=1).sqrt()
        floor = float(noise.mean())
        assert float(err.mean()) <= 2.0 * max(float(noise[positions].mean()), floor), \
            f"{what}: mean error {float(err.mean()):.3e}, rounding alone {float(noise[positions].mean()):.3e}"
        over = int((err > 3.0 * torch.clamp(noise[positions], min=floor)).sum())
        assert over <= max(1, len(positions) // 50), f"{what}: {over} of {len(positions)} positions beyond three times rounding"


@pytest.fixture(scope="module")
def models(pe):
    return Models(pe)


def _entry(pe, slot, toks, want):
    return pe.StepEntry(slot, toks, tuple(want))


def _batch(q_lens, slots):
    """(token_seq, seq_slot, seq_qstart) of a step, int32 on the device."""
    seq = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    qstart = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    return seq, torch.tensor(slots, dtype=torch.int32, device=DEV), qstart


# ---- mechanisms at kernel level -----------------------------------------------------------------------------------
def test_pair_embedding_first_tokens_kept_token_and_slots(pe):
    """Position 0 takes the table's last row whatever the slot kept before; a step's first token pairs with the kept
    token, later ones with their neighbour; products beyond 32 bits are taken in 64."""
    ops = pe.kernels.ops
    vocab, width, buckets, a, b = 70000, 24, 1009, 40009, 30011
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": a, "mul_cur": b}}}
    g = torch.Generator().manual_seed(0)
    w = {"embed": torch.randn(vocab, width, generator=g), "bigram": torch.randn(buckets + 1, width, generator=g)}
    last = torch.full((5,), 12345, dtype=torch.int32, device=DEV)         # stale values from earlier sequences
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    seqs = {3: [69999, 69998, 5, 69999, 0, 7], 1: [4, 69997, 69999]}
    for cuts in ([(3, 0, 4), (1, 0, 1)], [(3, 4, 5), (1, 1, 3)], [(3, 5, 6)]):
        toks = [t for s, lo, hi in cuts for t in seqs[s][lo:hi]]
        seq, slot, qstart = _batch([hi - lo for _, lo, hi in cuts], [s for s, _, _ in cuts])
        pos = torch.tensor([p for _, lo, hi in cuts for p in range(lo, hi)], dtype=torch.int32, device=DEV)
        out = torch.empty(len(toks), width, device=DEV)
        ops.embed_pair_gather(w["embed"].to(DEV), w["bigram"].to(DEV), torch.tensor(toks, dtype=torch.int32, device=DEV), seq, pos,
                              slot, qstart, last, out, buckets, a, b, status)
        want = torch.cat([plain.embed(seqs[s][lo:hi], cfg, w, seqs[s][lo - 1] if lo else None) for s, lo, hi in cuts])
        assert torch.equal(out.cpu(), want) and status.tolist()[0] == 0
    assert last.tolist()[3] == 7 and last.tolist()[1] == 69999 and last.tolist()[0] == 12345


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_convolution_continues_from_the_kept_inputs(pe, taps):
    """Whole sequences against the same sequences cut into steps of 1, 2 and many tokens, on slots whose kept inputs
    start at zero; two sequences of unequal length side by side."""
    ops = pe.kernels.ops
    C, lens = 20, [9, 14]
    g = torch.Generator().manual_seed(taps)
    xs = [torch.randn(n, C + 3, generator=g) for n in lens]             # the channels are columns 3.. of wider rows
    w = torch.randn(C, taps, generator=g)
    want = [plain.short_conv(x[:, 3:].double(), w.double(), torch.zeros(taps - 1, C, dtype=torch.float64))[0] for x in xs]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for cuts in ([9, 14], [1, 2, 1, 5, 20]):
        tail = torch.zeros(4, max(taps - 1, 1), C, device=DEV)
        got = [[], []]
        at = [0, 0]
        for step in cuts:
            live = [b for b in range(2) if at[b] < lens[b]]
            q = [min(step, lens[b] - at[b]) for b in live]
            seq, slot, qstart = _batch(q, [3 - b for b in live])
            x = torch.cat([xs[b][at[b]:at[b] + n] for b, n in zip(live, q)]).to(DEV)
            out = torch.empty(sum(q), C, device=DEV)
            ops.short_conv_silu(x, 3, w.to(DEV), tail, seq, slot, qstart, out, len(live), status)
            for b, n, lo in zip(live, q, qstart.tolist()):
                got[b].append(out[lo:lo + n].cpu())
                at[b] += n
        for b in range(2):
            assert (torch.cat(got[b]).double() - want[b]).abs().max() < 1e-5, (taps, cuts, b)
    assert status.tolist()[0] == 0


def test_router_choice_by_corrected_score_weight_by_the_score_itself(pe):
    """The correction moves the choice and not the weight; weights are not renormalised; among equal scores the
    lower index wins; ``top`` equal to the number of outputs chooses all."""
    ops = pe.kernels.ops
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5], [0.0, 0.0, 0.0, 0.0, 0.0], [-3.0, 4.0, 4.0, 1.0, 0.0]], device=DEV)
    c = torch.tensor([0.0, 0.0, 0.9, 0.0, 0.0], device=DEV)
    s = torch.softmax(z.double().cpu(), -1)
    for top in (1, 2, 5):
        chosen = torch.empty(3, top, dtype=torch.int32, device=DEV)
        weight = torch.empty(3, top, device=DEV)
        ops.moe_route(z, c, top, chosen, weight)
        if top < 5:         # row 1: all scores equal, the correction lifts entry 2, then the lowest index follows
            assert chosen.cpu().tolist() == ([[2, 0], [2, 0], [2, 1]] if top == 2 else [[2], [2], [2]]), top
        else:
            assert sorted(chosen[0].tolist()) == [0, 1, 2, 3, 4]
        assert (weight.cpu().double() - torch.gather(s, 1, chosen.cpu().long())).abs().max() < 1e-6
    assert int(torch.topk(s[0] + c.double().cpu(), 1).indices) == 2 and float(s[0, 2]) < float(s[0, 0])   # the case the test is for


class Pages:
    """A hand-made paged cache for kernel tests: sequence b's logical page i is physical page ``table[b][i]``."""

    def __init__(self, lens, kvh, d, dv, seed=0):
        g = torch.Generator().manual_seed(seed)
        n_pages = sum(-(-n // 64) for n in lens) + 3
        order = torch.randperm(n_pages, generator=g).tolist()
        self.table = torch.full((len(lens), max(-(-n // 64) for n in lens) + 1), -1, dtype=torch.int32)
        for b, n in enumerate(lens):
            for i in range(-(-n // 64)):
                self.table[b, i] = order.pop()
        self.k = torch.zeros(n_pages, kvh, 64, d)
        self.v = torch.zeros(n_pages, kvh, 64, dv)
        self.n_pages = n_pages

    def put(self, b, pos, k, v):
        page = int(self.table[b, pos // 64])
        self.k[page, :, pos % 64] = k
        self.v[page, :, pos % 64] = v


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window", [37, 64, 130])
def test_keys_just_inside_and_just_outside_the_window(pe, decode, window):
    """One key matches the query far better than all others.  If it lies at the window's oldest position the output
    is its value; one position further back it must not be seen at all, and the output is the average of the keys that
    are (all of score zero).  The query sits so that the edge falls before, on and behind page borders."""
    ops = pe.kernels.ops
    nh, nkv, d, dv = 6, 2, 16, 24
    g = torch.Generator().manual_seed(window)
    for n in (window, window + 1, 128, 129, 300):
        if n < window:
            continue
        i = n - 1                                   # the query's position
        for back, inside in ((window - 1, True), (window, False)):
            target = i - back
            if target < 0:
                continue
            pages = Pages([n], nkv, d, dv, seed=n + back)
            vals = torch.randn(n, nkv, dv, generator=g)
            for pos in range(n):
                k = torch.zeros(nkv, d)
                k[:, 0] = 1.0 if pos == target else 0.0
                pages.put(0, pos, k, vals[pos])
            q = torch.zeros(1, nh * d)
            q.view(1, nh, d)[:, :, 0] = 40.0
            qstart = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
            past = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
            slots = torch.zeros(1, dtype=torch.int32, device=DEV)
            out = torch.full((1, nh * dv), float("nan"), device=DEV)
            status = torch.zeros(4, dtype=torch.int32, device=DEV)
            max_splits = -(-n // 64) if decode else 0
            scratch = torch.zeros(ops.attention_generic_scratch_floats(1, nh, dv, max_splits), device=DEV) if decode else None
            ops.attention_generic_ex(decode, q.to(DEV), out, 1, 1, nh, nkv, d, dv, 1.0, window, False, None, None, 0, False, qstart,
                                     past, slots, pages.table.to(DEV), pages.n_pages, pages.k.to(DEV), pages.v.to(DEV), scratch, 64,
                                     max_splits, status)
            assert status.tolist()[0] == 0
            lo = max(0, i - window + 1)
            want = vals[target] if inside else vals[lo:i + 1].mean(0)
            want = want.repeat_interleave(nh // nkv, dim=0).view(1, nh * dv)
            assert (out.cpu() - want).abs().max() < 1e-3, (decode, window, n, inside)


# ---- every mechanism alone, as a model of one layer ---------------------------------------------------------------
ALONE = {
    "mlstm": {"type": "mlstm", "mixer": {"heads": 3, "dim": 24, "vdim": 40, "gate_cap": 6.0}, "mlp": None},
    "mlstm one head": {"type": "mlstm_7", "mixer": {"heads": 1, "dim": 8, "vdim": 72, "gate_cap": 20.0}, "mlp": None},
    "attention": {"type": "parallel", "mlp": None,
                  "mixer": {"left": _left(4, 1, 24, 16, 0.5, 50, 12, 500.0), "left_scale": 1.0, "right_scale": 0.0,
                            "right": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2}}},
    "delta": {"type": "parallel", "mlp": None,
              "mixer": {"left": _left(1, 1, 8, 8, 0.5, 8, 0), "left_scale": 0.0, "right_scale": 1.0,
                        "right": {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 12, "conv": 4}}},
    # key sizes beyond 64 (a state column in 128 registers) and beyond 128 (the state in shared memory)
    "mlstm wide": {"type": "mlstm", "mixer": {"heads": 2, "dim": 96, "vdim": 136, "gate_cap": 9.0}, "mlp": None},
    "mlstm widest": {"type": "mlstm", "mixer": {"heads": 1, "dim": 144, "vdim": 40, "gate_cap": 9.0}, "mlp": None},
    "delta wide": {"type": "parallel", "mlp": None,
                   "mixer": {"left": _left(1, 1, 8, 8, 0.5, 8, 0), "left_scale": 0.0, "right_scale": 1.0,
                             "right": {"heads": 2, "kv_heads": 1, "dim": 80, "vdim": 96, "conv": 2}}},
    "delta widest": {"type": "parallel", "mlp": None,
                     "mixer": {"left": _left(1, 1, 8, 8, 0.5, 8, 0), "left_scale": 0.0, "right_scale": 1.0,
                               "right": {"heads": 2, "kv_heads": 2, "dim": 136, "vdim": 24, "conv": 3}}},
    "dense": {"type": "mlstm", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "gate_cap": 5.0}, "mlp": {"kind": "dense", "ff": 100}},
    "experts": {"type": "mlstm", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "gate_cap": 5.0}, "mlp": _moe(7, 2, 2, 36, 1.0, shared=(20, 0.5))},
    "identity experts only": {"type": "mlstm", "mixer": {"heads": 1, "dim": 8, "vdim": 8, "gate_cap": 5.0}, "mlp": _moe(0, 3, 2, 8, 1.0)},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_alone_whole_and_token_by_token(pe, models, name, dtype):
    key = "alone " + name
    cfg = {"architecture": "Lunadra", "vocab": 90, "width": 48, "residual_mult": 0.9, "norm": {"eps": 1e-5},
           "embedding": {"bigram": {"buckets": 61, "mul_prev": 2, "mul_cur": 9}}, "layers": [copy.deepcopy(ALONE[name])]}
    models.add(key, cfg, 40 + sorted(ALONE).index(name))
    eng = models.engine(key, dtype, max_cache_tokens=64 * 12)
    toks = _tokens(90, 150, 9)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(150))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(150), f"{name} whole")
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:3], [2])]).clone()]
    for t in toks[3:150]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(2, 150), f"{name} token by token")


# ---- whole models -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_whole_prompt_and_its_first_tokens(pe, models, key, dtype):
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 300, 1)
    ref = models.ref(key, toks)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(300))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(300), f"{key} whole prompt")
    s = eng.alloc_slot()                               # a prompt of one token, on the slot that was just freed
    one = eng.step([_entry(pe, s, toks[:1], [0])]).clone()
    eng.free_slot(s)
    err = rel_err(one.cpu(), ref[:1])
    assert err < TOL[dtype], f"{key} one token on a used slot: {err:.3e}"
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_long_token_by_token_decoding_equals_the_prompt(pe, models, key, dtype):
    """A short prompt, then 240 tokens one by one (past every window, over three page borders, through CUDA graphs),
    against the plain implementation of the whole sequence."""
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 255, 2)
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:15], [14])]).clone()]
    for t in toks[15:]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(14, 255), f"{key} decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
@pytest.mark.parametrize("portion", [2, 3, 64, 65, 131])
def test_a_prompt_fed_in_portions(pe, models, key, dtype, portion):
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 280, 3)
    s = eng.alloc_slot()
    rows = []
    for lo in range(0, len(toks), portion):
        part = toks[lo:lo + portion]
        rows.append(eng.step([_entry(pe, s, part, range(len(part)))]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(len(toks)), f"{key} portions of {portion}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_unequal_batches_on_slots_used_again(pe, models, key, dtype):
    """Two batches in a row on the same slots and pages: unequal prompts in one step (among them one token), then one
    token each until the shorter ones have ended; each request against itself alone in the plain implementation."""
    eng = models.engine(key, dtype)
    vocab = CONFIGS[key]["vocab"]
    seen = []
    for batch in range(2):
        plan = [(1, 9), (200, 4), (65, 12), (33, 1), (130, 7)]
        seqs = [_tokens(vocab, p + dec, 100 * batch + i) for i, (p, dec) in enumerate(plan)]
        slots = [eng.alloc_slot() for _ in plan]
        seen.append(sorted(slots))
        got = {}
        out = eng.step([_entry(pe, s, q[:p], [p - 1]) for s, q, (p, dec) in zip(slots, seqs, plan)])
        for i, (p, dec) in enumerate(plan):
            got[i, p - 1] = out[i].clone()
        for step in range(max(dec for _, dec in plan)):
            live = [i for i, (p, dec) in enumerate(plan) if step < dec]
            out = eng.step([_entry(pe, slots[i], [seqs[i][plan[i][0] + step]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i, plan[i][0] + step] = out[r].clone()
                if step == plan[i][1] - 1:
                    eng.free_slot(slots[i])
        assert not eng.cache.live_slots
        for i, (p, dec) in enumerate(plan):
            rows = torch.stack([got[i, j] for j in range(p - 1, p + dec)])
            models.check(key, dtype, seqs[i], rows, range(p - 1, p + dec), f"{key} batch {batch} request {i}")
        eng.cache.check()
    assert seen[0] == seen[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("count", [12, 40])
def test_a_decode_batch_of_many(pe, models, dtype, count):
    """More sequences than the weight-streaming products take, inside the captured decode step: twelve (the experts'
    row-group kernel) and forty (80 pairs: in bfloat16 the library's product over row groups, recorded in the graph)."""
    key = "B"
    eng = models.engine(key, dtype, max_batch=count, max_cache_tokens=64 * (count + 2))
    vocab = CONFIGS[key]["vocab"]
    seqs = [_tokens(vocab, 3 + i % 13 + 6, 300 + i) for i in range(count)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = {i: [] for i in range(count)}
    out = eng.step([_entry(pe, s, q[:len(q) - 6], [len(q) - 7]) for s, q in zip(slots, seqs)]).clone()
    for i in range(count):
        got[i].append(out[i:i + 1])
    for step in range(6):
        out = eng.step([_entry(pe, s, [q[len(q) - 6 + step]], [0]) for s, q in zip(slots, seqs)]).clone()
        for i in range(count):
            got[i].append(out[i:i + 1])
    for s in slots:
        eng.free_slot(s)
    for i in (0, 5, count - 1):
        n = len(seqs[i])
        models.check(key, dtype, seqs[i], torch.cat(got[i]), range(n - 7, n), f"{key} request {i} of {count}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(pe, models, dtype):
    """``Engine.generate`` with unequal prompts: every generated token must be the plain implementation's best token
    for the sequence so far, or within rounding of it."""
    key = "A"
    eng = models.engine(key, dtype)
    prompts = [_tokens(CONFIGS[key]["vocab"], n, 50 + n) for n in (1, 17, 64, 140)]
    results = eng.generate(prompts, pe.SamplingParams.greedy_params(max_tokens=12))
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12
        ref = models.ref(key, p + r.token_ids)
        scale = float(ref.abs().max())
        for j, tok in enumerate(r.token_ids):
            row = ref[len(p) - 1 + j]
            margin = 2 * TOL[dtype] * scale
            if dtype == "bfloat16":      # a logit moves by several times its position's root-mean-square rounding error
                noise = models.noise(key, p + r.token_ids)
                margin = 8.0 * max(float(noise[len(p) - 1 + j]), float(noise.mean()))
            assert float(row.max() - row[tok]) <= margin, (dtype, len(p), j)
    assert not eng.cache.live_slots


def test_a_model_folder_written_at_random_loads_and_runs(pe, tmp_path):
    """config.json and safetensors through the loader (the low ranks are read off the tensors), against the plain
    implementation on the same file."""
    from safetensors.torch import load_file

    cfg = pe.LunadraConfig.from_dict(CONFIGS["A"])
    folder = pe.write_random_model(str(tmp_path / "m"), cfg, seed=4)
    assert pe.load_config(folder) == cfg
    eng = pe.Engine(folder, dtype="float32", max_context_len=256, max_cache_tokens=512, max_batch=2)
    toks = _tokens(cfg.vocab, 90, 8)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(90))])
    ref = plain.forward(CONFIGS["A"], {k: v.float() for k, v in load_file(folder + "/model.safetensors").items()}, toks)
    assert rel_err(got.cpu(), ref.float()) < TOL["float32"]
