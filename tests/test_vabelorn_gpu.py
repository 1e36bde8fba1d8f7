"""The Vabelorn architecture on the engine against the plain implementation in ``plain_vabelorn.py``: every mechanism
alone at kernel level (with inputs made so that a fault shows), then whole models: prompts, token-by-token decoding,
prompts in portions, unequal batches, slots and pages used again, long decoding, generation through the entry point."""
import math

import pytest
import torch

import plain_vabelorn as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 3e-5, "bfloat16": 2e-2}

YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
# The tests' own models.  P mixes both mixers with and without feed-forwards, value size below and above the key size,
# partial and whole rotation, one group of 2 and one of 1; Q has sizes that are no multiple of 8 anywhere, a group of 5, a
# single kv head, no token side input and no logit scale; R has the sizes that tensor-core kernels take.
CONFIGS = {
    "P": {"architecture": "Vabelorn", "vocab": 300, "width": 96, "logit_scale": 0.7, "norm": {"eps": 2e-6},
          "token_side": {"dim": 8},
          "layers": [
              {"type": "wkv", "mixer": {"heads": 3, "dim": 32, "decay_rank": 8}, "mlp": {"kind": "dense", "ff": 160}},
              {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 48, "vdim": 32, "scale": 0.2,
                                              "rot": {"base": 10000.0, "dims": 16, "scaling": YARN}}, "mlp": None},
              {"type": "attention", "mixer": {"heads": 6, "kv_heads": 6, "dim": 32, "vdim": 64, "scale": 0.25,
                                              "rot": {"base": 500.0, "dims": 32}}, "mlp": {"kind": "dense", "ff": 128}},
              {"type": "wkv", "mixer": {"heads": 2, "dim": 64, "decay_rank": 8}, "mlp": None}]},
    "Q": {"architecture": "Vabelorn", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
          "layers": [
              {"type": "attention", "mixer": {"heads": 5, "kv_heads": 1, "dim": 24, "vdim": 40, "scale": 0.3,
                                              "rot": {"base": 3000.0, "dims": 10, "scaling": {"factor": 2.0, "original": 32,
                                                                                             "fast": 4.0, "slow": 1.0}}},
               "mlp": {"kind": "dense", "ff": 100}},
              {"type": "wkv", "mixer": {"heads": 3, "dim": 24, "decay_rank": 5}, "mlp": {"kind": "dense", "ff": 52}}]},
    "R": {"architecture": "Vabelorn", "vocab": 512, "width": 256, "logit_scale": 2.0, "norm": {"eps": 1e-6},
          "token_side": {"dim": 16},
          "layers": [
              {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09,
                                              "rot": {"base": 100000.0, "dims": 64, "scaling": YARN}},
               "mlp": {"kind": "dense", "ff": 512}},
              {"type": "wkv", "mixer": {"heads": 4, "dim": 64, "decay_rank": 16}, "mlp": None},
              {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125,
                                              "rot": {"base": 10000.0, "dims": 64}}, "mlp": None}]},
}
SEEDS = {"P": 11, "Q": 12, "R": 13}
SHARPEN = {"float32": 3.0, "bfloat16": 1.5}


def _tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Models:
    def __init__(self, pe):
        self.pe = pe
        self.weights = {}
        self.engines = {}
        self.refs = {}

    def w(self, key, dtype):
        if (key, dtype) not in self.weights:
            self.weights[key, dtype] = plain.random_weights(CONFIGS[key], SEEDS[key], sharpen=SHARPEN[dtype])
        return self.weights[key, dtype]

    def engine(self, key, dtype, **kw):
        ident = (key, dtype, tuple(sorted(kw.items())))
        if ident not in self.engines:
            cfg = self.pe.VabelornConfig.from_dict(CONFIGS[key])
            args = dict(dtype=dtype, max_context_len=1024, max_cache_tokens=64 * 40, max_batch=8)
            args.update(kw)
            self.engines[ident] = self.pe.Engine(None, config=cfg, weights={k: v.to(DEV) for k, v in self.w(key, dtype).items()}, **args)
        return self.engines[ident]

    def ref(self, key, dtype, toks):
        ident = (key, dtype, tuple(toks))
        if ident not in self.refs:
            self.refs[ident] = plain.forward(CONFIGS[key], self.w(key, dtype), toks).float()
        return self.refs[ident]

    def noise(self, key, dtype, toks):
        """How far rounding to bfloat16 alone moves each position's logits (root mean square over the vocabulary):
        the plain implementation with its products and cached values rounded, against itself without."""
        ident = (key, dtype, tuple(toks), "noise")
        if ident not in self.refs:
            with plain.stored(torch.bfloat16):
                rounded = plain.forward(CONFIGS[key], self.w(key, dtype), toks)
            self.refs[ident] = (rounded - self.ref(key, dtype, toks).double()).pow(2).mean(dim=1).sqrt()
        return self.refs[ident]

    def check(self, key, dtype, toks, got, positions, what):
        """``got``: the engine's logits at ``positions`` of the sequence ``toks``.  float32: every logit within 3e-5 of
        the largest.  bfloat16: these models amplify a rounding here and there (a norm on a sublayer's output scales
        whatever it gets to unit size), so the error is held against what rounding alone does in the plain
        implementation: on average no more than twice that, and at no more than one position in fifty (or one) above
        three times the larger of that position's own figure and the average."""
        positions = list(positions)
        ref = self.ref(key, dtype, toks)[positions]
        got = got.float().cpu()
        assert got.shape == ref.shape, what
        if dtype == "float32":
            err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
            assert err < TOL[dtype], f"{what}: error {err:.3e} (limit {TOL[dtype]:.0e})"
            return
        noise = self.noise(key, dtype, toks)
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


def _close(got, ref, dtype, what):
    """For a sequence's first tokens, where little has been rounded yet."""
    err = float((got.double().cpu() - ref.double()).abs().max() / ref.double().abs().max())
    assert err < TOL[dtype], f"{what}: error {err:.3e} (limit {TOL[dtype]:.0e})"


# ---- mechanisms alone -----------------------------------------------------------------------------------------
def test_rotary_tables_interleaved_with_scaled_frequencies(pe):
    rt = pe.parts.Runtime(DEV, torch.float32)
    rot = {"base": 7000.0, "dims": 24, "scaling": {"factor": 4.0, "original": 128, "fast": 8.0, "slow": 2.0}}
    part = pe.parts.lookup("position", "rope")({"rotary_dim": 24, "theta": 7000.0, "max_positions": 700, "style": "interleaved",
                                                "scaling": rot["scaling"]}, {}, rt)
    f, mult = plain.key_frequencies(rot)
    assert mult != 1.0 and not torch.allclose(f, plain.key_frequencies({"base": 7000.0, "dims": 24})[0])
    ang = torch.arange(700, dtype=torch.float64)[:, None] * f[None]
    cos, sin, dims = part.tables()
    assert dims == 24 and part.interleaved
    assert (cos.cpu().double() - torch.cos(ang) * mult).abs().max() < 2e-4     # float32 angles at position 700
    assert (sin.cpu().double() - torch.sin(ang) * mult).abs().max() < 2e-4
    assert (cos[:50].cpu().double() - (torch.cos(ang) * mult)[:50]).abs().max() < 5e-6


class Pages:
    """A hand-made paged cache for kernel tests: sequence b's logical page i is physical page ``table[b][i]``."""

    def __init__(self, lens, kvh, d, dv, dtype, seed=0, shuffle=True):
        g = torch.Generator().manual_seed(seed)
        n_pages = sum(-(-n // 64) for n in lens) + 3
        order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
        self.table = torch.full((len(lens), max(-(-n // 64) for n in lens) + 1), -1, dtype=torch.int32)
        for b, n in enumerate(lens):
            for i in range(-(-n // 64)):
                self.table[b, i] = order.pop()
        self.k = torch.zeros(n_pages, kvh, 64, d, dtype=dtype)
        self.v = torch.zeros(n_pages, kvh, 64, dv, dtype=dtype)
        self.n_pages = n_pages

    def put(self, b, pos, k, v):
        page = int(self.table[b, pos // 64])
        self.k[page, :, pos % 64] = k
        self.v[page, :, pos % 64] = v

    def cuda(self):
        self.table, self.k, self.v = self.table.to(DEV), self.k.to(DEV), self.v.to(DEV)
        return self


def _attend(pe, decode, q, lens, q_lens, pages, nh, nkv, d, dv, scale, sink, out_tables=None, dtype=torch.float32):
    ops = pe.kernels.ops
    B = len(lens)
    qstart = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past = torch.tensor([n - ql for n, ql in zip(lens, q_lens)], dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    out = torch.full((sum(q_lens), nh * dv), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    max_splits = -(-max(lens) // 64) if decode else 0
    scratch = torch.full((ops.attention_generic_scratch_floats(B, nh, dv, max_splits),), float("nan"), device=DEV) if decode else None
    cos, sin, rot, inter = out_tables if out_tables else (None, None, 0, False)
    ops.attention_generic_ex(decode, q.to(DEV, dtype), out, B, max(q_lens), nh, nkv, d, dv, scale, 0, sink, cos, sin, rot, inter,
                             qstart, past, slots, pages.table, pages.n_pages, pages.k, pages.v, scratch, 64, max_splits, status)
    assert status.tolist()[0] == 0
    return out.float().cpu()


@pytest.mark.parametrize("decode", [False, True])
def test_a_far_key_among_hundreds_and_keys_at_page_borders(pe, decode):
    """One key matches the query, all others are orthogonal noise: the output must be that key's value, wherever
    the key lies (first position, either side of a page border, far back, the query's own position)."""
    nh, nkv, d, dv = 4, 2, 24, 40
    n = 453
    g = torch.Generator().manual_seed(5)
    for target in (0, 63, 64, 127, 128, 300, n - 2, n - 1):
        pages = Pages([n], nkv, d, dv, torch.float32, seed=target)
        q = torch.zeros(1, nh, d)
        q[:, :, 0] = 30.0
        vals = torch.randn(n, nkv, dv, generator=g)
        for pos in range(n):
            k = torch.randn(nkv, d, generator=g) * 0.1
            k[:, 0] = 1.0 if pos == target else 0.0
            pages.put(0, pos, k, vals[pos])
        got = _attend(pe, decode, q.view(1, nh * d), [n], [1], pages.cuda(), nh, nkv, d, dv, 1.0, True)
        want = vals[target].repeat_interleave(nh // nkv, dim=0).view(1, nh * dv)
        assert (got - want).abs().max() < 1e-3, (decode, target)


@pytest.mark.parametrize("decode", [False, True])
def test_the_sink_takes_the_weight_when_no_key_matches(pe, decode):
    """Scores far below zero: with the one in the denominator the output is nearly zero; a softmax without it
    would return an average of the values.  Scores at zero: n keys and the sink share the weight, 1/(n+1) each."""
    nh, nkv, d, dv = 2, 1, 16, 16
    n = 70
    pages = Pages([n], nkv, d, dv, torch.float32)
    for pos in range(n):
        pages.put(0, pos, torch.full((nkv, d), 1.0), torch.ones(nkv, dv))
    pages.cuda()
    q = torch.full((1, nh * d), -2.0)                # every score is -32
    got = _attend(pe, decode, q, [n], [1], pages, nh, nkv, d, dv, 1.0, True)
    assert got.abs().max() < 1e-10
    assert (_attend(pe, decode, q, [n], [1], pages, nh, nkv, d, dv, 1.0, False) - 1.0).abs().max() < 1e-5
    got = _attend(pe, decode, torch.zeros(1, nh * d), [n], [1], pages, nh, nkv, d, dv, 1.0, True)
    assert (got - n / (n + 1.0)).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_values_of_their_own_size_against_the_formula(pe, dtype):
    """Unequal sequences, prompts continued from a past, groups of 3, value size unlike the key size, output turned
    back by the query's position."""
    nh, nkv, d, dv = 6, 2, 40, 24
    lens, q_lens = [200, 65, 1, 130], [70, 65, 1, 2]
    g = torch.Generator().manual_seed(9)
    pages = Pages(lens, nkv, d, dv, dtype, seed=1)
    ks = [torch.randn(n, nkv, d, generator=g).to(dtype) for n in lens]
    vs = [torch.randn(n, nkv, dv, generator=g).to(dtype) for n in lens]
    for b, n in enumerate(lens):
        for pos in range(n):
            pages.put(b, pos, ks[b][pos], vs[b][pos])
    pages.cuda()
    q = torch.randn(sum(q_lens), nh, d, generator=g).to(dtype)
    rt = pe.parts.Runtime(DEV, torch.float32)
    vpos = pe.parts.lookup("position", "rope")({"rotary_dim": dv, "theta": 300.0, "max_positions": 256, "style": "interleaved"}, {}, rt)
    cos, sin, rot = vpos.tables()
    scale = 0.3
    for decode in (False, True):
        if decode:
            sel = [sum(q_lens[:b + 1]) - 1 for b in range(len(lens))]
            got = _attend(pe, True, q[sel].view(len(lens), -1), lens, [1] * len(lens), pages, nh, nkv, d, dv, scale, True,
                          (cos, sin, rot, True), dtype)
        else:
            got = _attend(pe, False, q.view(sum(q_lens), -1), lens, q_lens, pages, nh, nkv, d, dv, scale, True, (cos, sin, rot, True), dtype)
        row = 0
        f = plain.value_frequencies({"base": 300.0}, dv)
        for b, (n, ql) in enumerate(zip(lens, q_lens)):
            for i in (range(ql - 1, ql) if decode else range(ql)):
                p = n - ql + i
                qq = q[sum(q_lens[:b]) + i].double()
                for h in range(nh):
                    s = (ks[b][:p + 1, h // 3].double() @ qq[h]) * scale
                    e = torch.exp(s)
                    o = (e / (1 + e.sum())) @ vs[b][:p + 1, h // 3].double()
                    o = plain.rotate_interleaved(o[None], -(p * f)[None])[0]
                    tol = 2e-5 if dtype == torch.float32 else 2e-2
                    assert (got[row, h * dv:(h + 1) * dv].double() - o).abs().max() < tol, (decode, b, i, h)
                row += 1


@pytest.mark.parametrize("d,nh,nkv", [(64, 8, 2), (128, 4, 2), (128, 6, 1), (128, 6, 2), (128, 5, 1), (64, 16, 1), (64, 3, 3)])
def test_tensor_core_attention_with_sink_and_turned_outputs(pe, d, nh, nkv):
    """The mma.sync kernels (prompt and single token) and the tcgen05 prompt kernel with a sink and outputs turned back,
    against the float32-arithmetic kernel on the same bfloat16 cache; one key far back stands out for every query."""
    ops = pe.kernels.ops
    dtype = torch.bfloat16
    lens, q_lens = [700, 130, 64, 1], [250, 130, 3, 1]
    g = torch.Generator().manual_seed(d + nh)
    pages = Pages(lens, nkv, d, d, dtype, seed=4)
    q = torch.randn(sum(q_lens), nh, d, generator=g)
    for b, n in enumerate(lens):
        for pos in range(n):
            k = torch.randn(nkv, d, generator=g)
            if b == 0 and pos == 65:
                k = k + 3.0 * q[200, ::nh // nkv]            # the far key that the first sequence's row 200 looks for
            pages.put(b, pos, k.to(dtype), torch.randn(nkv, d, generator=g).to(dtype))
    pages.cuda()
    rt = pe.parts.Runtime(DEV, torch.float32)
    vpos = pe.parts.lookup("position", "rope")({"rotary_dim": d, "theta": 5000.0, "max_positions": 1024, "style": "interleaved"}, {}, rt)
    cos, sin, _ = vpos.tables()
    scale = 1.0 / math.sqrt(d)
    B = len(lens)
    qstart = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past = torch.tensor([n - ql for n, ql in zip(lens, q_lens)], dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    where = (qstart, past, slots, pages.table, pages.n_pages, pages.k, pages.v)
    qd = q.view(sum(q_lens), nh * d).to(DEV, dtype)
    want = _attend(pe, False, q.view(sum(q_lens), -1), lens, q_lens, pages, nh, nkv, d, d, scale, True, (cos, sin, d, True), dtype)
    plain_softmax = _attend(pe, False, q.view(sum(q_lens), -1), lens, q_lens, pages, nh, nkv, d, d, scale, False, None, dtype)
    assert (want - plain_softmax).abs().max() > 0.05          # sink and rotation do change the result
    got = torch.full_like(qd, float("nan"))
    ops.attention_mma(False, qd, got, B, max(q_lens), nh, nkv, d, scale, 0, *where, None, 0, 0, status, sink=True, out_cos=cos, out_sin=sin)
    assert status.tolist()[0] == 0 and (got.float().cpu() - want).abs().max() < 2e-2
    if ops.attention_umma_supported(dtype, d, nh, nkv):
        got = torch.full_like(qd, float("nan"))
        ops.attention_umma_prefill(qd, got, B, max(q_lens), nh, nkv, d, scale, 0, *where, status, sink=True, out_cos=cos, out_sin=sin)
        assert status.tolist()[0] == 0 and (got.float().cpu() - want).abs().max() < 2e-2
    # single tokens: every sequence's last row
    sel = [sum(q_lens[:b + 1]) - 1 for b in range(B)]
    one = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    past1 = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    split_keys, max_splits, floor = ops.attention_mma_decode_ranges(torch.device(DEV), d, B, nkv, 1024, 512)
    scratch = torch.full((ops.attention_generic_scratch_floats(B, nh, d, max_splits),), float("nan"), device=DEV)
    got = torch.full((B, nh * d), float("nan"), dtype=dtype, device=DEV)
    ops.attention_mma(True, qd[sel].contiguous(), got, B, 1, nh, nkv, d, scale, 0, one, past1, slots, pages.table, pages.n_pages,
                      pages.k, pages.v, scratch, split_keys, max_splits, status, min_range_keys=floor, sink=True, out_cos=cos, out_sin=sin)
    assert status.tolist()[0] == 0 and (got.float().cpu() - want[sel]).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,dv,dims,pasts,q_lens", [
    (3, 1, 20, 12, 8, [0, 61, 130], [5, 7, 1]),
    (4, 2, 64, 64, 16, [0, 10, 63], [200, 66, 90]),      # many tokens of sizes that the 16-byte-access form takes
    (5, 1, 48, 48, 48, [3, 0, 0], [260, 1, 2]),          # six lanes a head: no power of two
])
def test_norm_rotation_and_append_of_q_k_v(pe, dtype, nh, nkv, d, dv, dims, pasts, q_lens):
    """q/k norm with weights, interleaved rotation of part of the head, values divided by their root mean square and
    rotated over all their features, rows landing in the right page and row of the cache."""
    ops = pe.kernels.ops
    rot = {"base": 900.0, "dims": dims, "scaling": {"factor": 3.0, "original": 50, "fast": 6.0, "slow": 1.5}}
    rt = pe.parts.Runtime(DEV, torch.float32)
    mk = pe.parts.lookup("position", "rope")
    kp = mk({"rotary_dim": dims, "theta": 900.0, "max_positions": 400, "style": "interleaved", "scaling": rot["scaling"]}, {}, rt)
    vp = mk({"rotary_dim": dv, "theta": 900.0, "max_positions": 400, "style": "interleaved"}, {}, rt)
    g = torch.Generator().manual_seed(3)
    lens = [p + q for p, q in zip(pasts, q_lens)]
    pages = Pages(lens, nkv, d, dv, dtype, seed=2).cuda()
    n = sum(q_lens)
    qkv = torch.randn(n, (nh + nkv) * d + nkv * dv, generator=g).to(dtype)
    qw, kw = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    dev = qkv.to(DEV).clone()
    token_seq = torch.tensor(sum(([b] * q for b, q in enumerate(q_lens)), []), dtype=torch.int32, device=DEV)
    pos_list = sum(([p + i for i in range(q)] for p, q in zip(pasts, q_lens)), [])
    token_pos = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    qstart = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    eps = 1e-5
    ops.qkv_rotate_append(dev, n, nh, nkv, d, dv, qw.to(DEV), kw.to(DEV), eps, *kp.tables()[:2], dims, True, True, *vp.tables()[:2], dv, True,
                          token_seq, token_pos, torch.arange(3, dtype=torch.int32, device=DEV), qstart, pages.table, pages.n_pages,
                          pages.k, pages.v, True, status)
    assert status.tolist()[0] == 0
    x = qkv.double()
    pos = torch.tensor(pos_list, dtype=torch.float64)
    f, mult = plain.key_frequencies(rot)
    ang = pos[:, None] * f[None]
    tol = 1e-4 if dtype == torch.float32 else 3e-2     # float32: the angle itself, a position of some hundreds times a float32 frequency
    q = plain.rms(x[:, :nh * d].view(n, nh, d), eps) * qw.double()
    q = torch.cat([plain.rotate_interleaved(q[..., :dims].transpose(0, 1), ang, mult).transpose(0, 1), q[..., dims:]], -1)
    assert (dev[:, :nh * d].double().cpu().view(n, nh, d) - q).abs().max() < tol
    k = plain.rms(x[:, nh * d:(nh + nkv) * d].view(n, nkv, d), eps) * kw.double()
    k = torch.cat([plain.rotate_interleaved(k[..., :dims].transpose(0, 1), ang, mult).transpose(0, 1), k[..., dims:]], -1)
    v = plain.rms(x[:, (nh + nkv) * d:].view(n, nkv, dv), eps)
    v = plain.rotate_interleaved(v.transpose(0, 1), pos[:, None] * plain.value_frequencies(rot, dv)[None]).transpose(0, 1)
    for t in range(n):
        page = int(pages.table[int(token_seq[t]), pos_list[t] // 64])
        assert (pages.k[page, :, pos_list[t] % 64].double().cpu() - k[t]).abs().max() < tol
        assert (pages.v[page, :, pos_list[t] % 64].double().cpu() - v[t]).abs().max() < tol


def _wkv_inputs(n, H, d, g, dtype):
    hd = H * d
    r, k, v, gl = (torch.randn(n, hd, generator=g).to(dtype) for _ in range(4))
    k = k * 0.5
    wlin = torch.randn(n, hd, generator=g) * 1.5 - 1.0
    w0 = torch.randn(hd, generator=g) * 0.5
    u = torch.randn(hd, generator=g) * 0.5
    gn = 1 + 0.2 * torch.randn(hd, generator=g)
    return r, k, v, gl, wlin, w0, u, gn


def _wkv_plain(r, k, v, gl, wlin, w0, u, gn, H, d, eps, S):
    n = r.shape[0]
    r, k, v, gl = (t.double().view(n, H, d) for t in (r, k, v, gl))
    w = torch.exp(-torch.exp(wlin.double() + w0.double())).view(n, H, d)
    uu = u.double().view(H, d)
    out = torch.empty(n, H, d, dtype=torch.float64)
    for t in range(n):
        kv = k[t, :, :, None] * v[t, :, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + uu[:, :, None] * kv)
        S = w[t, :, :, None] * S + kv
    out = plain.rms(out, eps) * gn.double().view(H, d) * plain.silu(gl)
    return out.reshape(n, H * d), S


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d", [(3, 24), (2, 64), (1, 128), (2, 33), (1, 160), (2, 6)])
def test_recurrence_whole_chunked_and_token_by_token(pe, dtype, H, d):
    """Three sequences of unequal lengths, one of them continuing from a state: in one go, cut into chunks of 16 and of
    64, and one token at a time; every way against the plain recurrence, and the states they leave against each other."""
    ops = pe.kernels.ops
    g = torch.Generator().manual_seed(H * 100 + d)
    q_lens = [150, 1, 67]
    n, hd, width, eps = sum(q_lens), H * d, 40, 3e-6
    r, k, v, gl, wlin, w0, u, gn = _wkv_inputs(n, H, d, g, dtype)
    x = torch.randn(n, width, generator=g).to(dtype)
    S0 = torch.zeros(5, H, d, d)
    S0[3] = torch.randn(H, d, d, generator=g)                         # slot 3 (sequence 1) continues
    slots = [4, 3, 1]
    want, S_want = [], {}
    at = 0
    for b, ql in enumerate(q_lens):
        sl = slice(at, at + ql)
        o, S = _wkv_plain(r[sl], k[sl], v[sl], gl[sl], wlin[sl], w0, u, gn, H, d, eps, S0[slots[b]].double())
        want.append(o)
        S_want[slots[b]] = S
        at += ql
    want = torch.cat(want)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    dv = lambda t: t.to(DEV)
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    qstart = torch.tensor([0, 150, 151, 218], dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    states = []
    for chunk in (0, 16, 64):
        state, prev = dv(S0.clone()), torch.zeros(5, width, device=DEV)
        out = torch.full((n, hd), float("nan"), dtype=dtype, device=DEV)
        max_chunks = -(-max(q_lens) // chunk) if chunk else 1
        scratch = torch.full((ops.wkv_scratch_floats(3, H, d, max_chunks),), float("nan"), device=DEV) if chunk else None
        ops.wkv_recurrence(dv(r), dv(k), dv(v), dv(gl), dv(wlin), dv(w0), dv(u), dv(gn), eps, out, state, prev, dv(x), seq_slot, qstart,
                           3, max(q_lens), H, d, chunk, max_chunks, scratch, status)
        assert status.tolist()[0] == 0
        assert (out.double().cpu() - want).abs().max() < tol * max(1.0, float(want.abs().max())), chunk
        for s, S in S_want.items():
            assert (state[s].double().cpu() - S).abs().max() < 1e-4 * max(1.0, float(S.abs().max())), (chunk, s)
        assert torch.equal(state[0].cpu(), S0[0]) and torch.equal(state[2].cpu(), S0[2])   # slots not in the step are untouched
        for b, sl in enumerate(slots):
            assert torch.equal(prev[sl].cpu(), x[int(qstart[b + 1]) - 1].float())
        states.append(state.cpu())
    # one token at a time for the longest sequence, through the same entry point
    state, prev = dv(S0.clone()), torch.zeros(5, width, device=DEV)
    one = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    outs = []
    for t in range(150):
        sl = slice(t, t + 1)
        out = torch.empty((1, hd), dtype=dtype, device=DEV)
        ops.wkv_recurrence(dv(r[sl]), dv(k[sl]), dv(v[sl]), dv(gl[sl]), dv(wlin[sl]), dv(w0), dv(u), dv(gn), eps, out, state, prev,
                           dv(x[sl]), seq_slot[:1], one, 1, 1, H, d, 0, 1, None, status)
        outs.append(out.cpu())
    assert (torch.cat(outs).double() - want[:150]).abs().max() < tol * max(1.0, float(want.abs().max()))
    assert (state[4].cpu() - states[0][4]).abs().max() < 1e-5 * max(1.0, float(states[0][4].abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_takes_the_previous_token_or_the_state(pe, dtype):
    ops = pe.kernels.ops
    g = torch.Generator().manual_seed(1)
    width, q_lens, slots = 50, [3, 1, 4], [2, 0, 5]
    n = sum(q_lens)
    x = torch.randn(n, width, generator=g).to(dtype)
    mu = torch.rand(5, width, generator=g)
    prev = torch.randn(6, width, generator=g)
    out = torch.empty(5, n, width, dtype=dtype, device=DEV)
    token_seq = torch.tensor([0, 0, 0, 1, 2, 2, 2, 2], dtype=torch.int32, device=DEV)
    ops.token_shift_mix(x.to(DEV), mu.to(DEV), prev.to(DEV), token_seq, torch.tensor(slots, dtype=torch.int32, device=DEV),
                        torch.tensor([0, 3, 4, 8], dtype=torch.int32, device=DEV), out, torch.zeros(4, dtype=torch.int32, device=DEV))
    xp = torch.cat([prev[2][None], x[0:2].float(), prev[0][None], prev[5][None], x[4:7].float()])
    want = x.float()[None] + (xp - x.float())[None] * mu[:, None]
    assert (out.float().cpu() - want).abs().max() < (1e-6 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_then_add_and_token_gate(pe, dtype):
    ops = pe.kernels.ops
    g = torch.Generator().manual_seed(2)
    n, dim = 7, 90
    stream = torch.randn(n, dim, generator=g)
    delta = (torch.randn(n, dim, generator=g) * 3).to(dtype)
    w = 1 + 0.3 * torch.randn(dim, generator=g)
    s, cast = stream.to(DEV).clone(), torch.empty(n, dim, dtype=dtype, device=DEV)
    ops.rmsnorm_add(s, delta.to(DEV), w.to(DEV), 1e-5, cast)
    want = stream.double() + plain.rms(delta.double(), 1e-5) * w.double()
    assert (s.double().cpu() - want).abs().max() < 1e-5
    assert torch.equal(cast.cpu(), s.cpu().to(dtype))
    table = torch.randn(30, 24, generator=g).to(dtype)
    gx = torch.randn(n, 6, generator=g).to(dtype)
    toks = torch.tensor([3, 29, 0, 7, 7, 12, 1], dtype=torch.int32)
    out = torch.empty(n, 6, dtype=dtype, device=DEV)
    ops.token_gate(gx.to(DEV), table.to(DEV), 12, toks.to(DEV), out, torch.zeros(4, dtype=torch.int32, device=DEV))
    want = plain.gelu_tanh(gx.double()) * table.double()[toks.long()][:, 12:18]
    assert (out.double().cpu() - want).abs().max() < (1e-6 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("m", [1, 5, 8, 13])
def test_grouped_product_of_several_inputs(pe, m):
    """Four projections, each of an input of its own, in one launch of the weight-streaming kernel."""
    ops = pe.kernels.ops
    g = torch.Generator().manual_seed(m)
    G, R, K = 4, 48, 72
    xs = torch.randn(G, m, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(G * R, K, generator=g) / 8).to(torch.bfloat16)
    assert ops.gemm_smallm_grouped_supported(xs.to(DEV), w.to(DEV), R)
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, G * R), float("nan"), dtype=dtype, device=DEV)
        ops.gemm_smallm_grouped(xs.to(DEV), w.to(DEV), out, R)
        want = torch.cat([xs[i].double() @ w[i * R:(i + 1) * R].double().T for i in range(G)], dim=1)
        assert (out.double().cpu() - want).abs().max() < (2e-2 if dtype == torch.bfloat16 else 1e-4)


# ---- whole models -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["P", "Q", "R"])
def test_whole_prompt_and_its_first_tokens(pe, models, key, dtype):
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 300, 1)
    ref = models.ref(key, dtype, toks)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(300))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(300), f"{key} whole prompt")
    _close(got[:3], ref[:3], dtype, f"{key} first tokens")
    s = eng.alloc_slot()                               # a prompt of one token, on the slot that was just freed
    one = eng.step([_entry(pe, s, toks[:1], [0])]).clone()
    eng.free_slot(s)
    _close(one, ref[:1], dtype, f"{key} one token")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["P", "Q", "R"])
def test_token_by_token_decoding_equals_the_prompt(pe, models, key, dtype):
    """A short prompt, then 200 tokens one by one (over three page borders, through CUDA graphs), against the plain
    implementation of the whole sequence."""
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 215, 2)
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:15], [14])]).clone()]
    for t in toks[15:]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(14, 215), f"{key} decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["P", "Q"])
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
@pytest.mark.parametrize("key", ["P", "Q", "R"])
def test_unequal_batches_on_slots_used_again(pe, models, key, dtype):
    """Two batches in a row on the same slots and pages: unequal prompts in one step (among them one token and more than
    two chunks of the recurrence), then one token each until the shorter ones have ended; each request against itself
    alone in the plain implementation."""
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
@pytest.mark.parametrize("key", ["P", "R"])
def test_a_decode_batch_of_twelve(pe, models, key, dtype):
    """More sequences than the weight-streaming products take: the library products (one batched call for the
    recurrence's four projections) inside the captured decode step."""
    eng = models.engine(key, dtype, max_batch=12)
    vocab = CONFIGS[key]["vocab"]
    seqs = [_tokens(vocab, 3 + i + 6, 300 + i) for i in range(12)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = {i: [] for i in range(12)}
    out = eng.step([_entry(pe, s, q[:3 + i], [2 + i]) for i, (s, q) in enumerate(zip(slots, seqs))]).clone()
    for i in range(12):
        got[i].append(out[i:i + 1])
    for step in range(6):
        out = eng.step([_entry(pe, s, [q[3 + i + step]], [0]) for i, (s, q) in enumerate(zip(slots, seqs))]).clone()
        for i in range(12):
            got[i].append(out[i:i + 1])
    for s in slots:
        eng.free_slot(s)
    for i in (0, 5, 11):
        models.check(key, dtype, seqs[i], torch.cat(got[i]), range(2 + i, 9 + i), f"{key} request {i} of twelve")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(pe, models, dtype):
    """``Engine.generate`` with unequal prompts: every generated token must be the plain implementation's best token
    for the sequence so far, or within rounding of it."""
    key = "P"
    eng = models.engine(key, dtype)
    prompts = [_tokens(CONFIGS[key]["vocab"], n, 50 + n) for n in (1, 17, 64, 140)]
    results = eng.generate(prompts, pe.SamplingParams.greedy_params(max_tokens=12))
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12
        ref = models.ref(key, dtype, p + r.token_ids)
        scale = float(ref.abs().max())
        for j, tok in enumerate(r.token_ids):
            row = ref[len(p) - 1 + j]
            margin = 2 * TOL[dtype] * scale
            if dtype == "bfloat16":      # a logit moves by several times its position's root-mean-square rounding error
                noise = models.noise(key, dtype, p + r.token_ids)
                margin = 8.0 * max(float(noise[len(p) - 1 + j]), float(noise.mean()))
            assert float(row.max() - row[tok]) <= margin, (dtype, len(p), j)
    assert not eng.cache.live_slots


def test_a_model_folder_written_at_random_loads_and_runs(pe, tmp_path):
    """config.json and safetensors through the loader (the decay's rank is read off the tensors), against the plain
    implementation on the same file."""
    from safetensors.torch import load_file

    cfg = pe.VabelornConfig.from_dict(CONFIGS["Q"])
    folder = pe.write_random_model(str(tmp_path / "m"), cfg, seed=4)
    assert pe.load_config(folder) == cfg
    eng = pe.Engine(folder, dtype="float32", max_context_len=256, max_cache_tokens=512, max_batch=2)
    toks = _tokens(cfg.vocab, 90, 8)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(90))])
    ref = plain.forward(CONFIGS["Q"], {k: v.float() for k, v in load_file(folder + "/model.safetensors").items()}, toks)
    assert rel_err(got.cpu(), ref.float()) < TOL["float32"]
