"""The Zuzelorn design on the GPU: each mechanism's kernel alone against the plain
restatement, then whole models through the engine under every way of cutting the
work, and greedy generation through the library's own entry point."""
import numpy as np
import pytest
import torch

import plain_zuzelorn as pz
from helpers import rel_err, run_trace, trace_batches, trace_tail, trace_whole
from zuzelorn_models import CONFIGS, model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def ops():
    from janas_b200.csrc import ops as o
    return o


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed * 7919 + sum(shape) + len(shape))
    return torch.randn(*shape, generator=g) * scale


def bf(x):
    return x.to(torch.bfloat16).float()


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,dm", [(1, 50), (7, 256), (130, 1000)])
def test_dynamic_tanh(odt, n, dm):
    x, w, b = rnd(n, dm, scale=2.0), 1 + rnd(dm, scale=0.2, seed=1), rnd(dm, scale=0.3, seed=2)
    alpha = torch.tensor(0.7)
    want = pz.dynamic_tanh(x, w, b, alpha)
    got = ops().dyt(x.to(DEV), w.to(DEV), b.to(DEV), alpha.to(DEV), odt).float().cpu()
    assert (got - want).abs().max() <= (1e-6 if odt == torch.float32 else 1e-2)
    # with partial sums added first (in place), and with a choice of rows
    delta = rnd(3, n, dm, seed=3)
    xd = x.to(DEV).clone()
    got = ops().dyt(xd, w.to(DEV), b.to(DEV), alpha.to(DEV), torch.float32, delta=delta.to(DEV)).cpu()
    xs = x + delta[0] + delta[1] + delta[2]
    assert torch.allclose(xd.cpu(), xs, atol=1e-6)
    assert (got - pz.dynamic_tanh(xs, w, b, alpha)).abs().max() <= 2e-6
    rows = torch.tensor([n - 1, 0], dtype=torch.int32)
    got = ops().dyt(x.to(DEV), w.to(DEV), b.to(DEV), alpha.to(DEV), torch.float32, rows=rows.to(DEV)).cpu()
    assert (got - pz.dynamic_tanh(x[rows.long()], w, b, alpha)).abs().max() <= 1e-6


@pytest.mark.parametrize("n,dm,wide", [(1, 50, 0), (9, 192, 64), (200, 256, 0)])
def test_gate_and_residual(n, dm, wide):
    y, g = rnd(2, n, dm, seed=1), rnd(3, n, dm + wide, seed=2)
    yb, gb = rnd(dm, seed=3), rnd(dm, seed=4)
    x = rnd(n, dm, seed=5)
    post = (1 + rnd(dm, scale=0.2, seed=6), rnd(dm, scale=0.2, seed=7), torch.tensor([0.5]))
    nxt = (1 + rnd(dm, scale=0.2, seed=8), rnd(dm, scale=0.2, seed=9), torch.tensor([0.9]))
    gate = torch.sigmoid(g.sum(0)[:, :dm] + gb)
    want_mul = (y.sum(0) + yb) * gate
    got = ops().gate_mul(y.to(DEV), yb.to(DEV), g.to(DEV), gb.to(DEV)).cpu()
    assert (got - want_mul).abs().max() <= 2e-6
    want_x = x + pz.dynamic_tanh(want_mul, *post)
    xd = x.to(DEV).clone()
    h = ops().gated_dyt_residual(xd, y.to(DEV), yb.to(DEV), g.to(DEV), gb.to(DEV),
                                 tuple(t.to(DEV) for t in post), tuple(t.to(DEV) for t in nxt)).cpu()
    assert (xd.cpu() - want_x).abs().max() <= 3e-6
    assert (h - pz.dynamic_tanh(want_x, *nxt)).abs().max() <= 3e-6
    # without a next norm and without a bias on the result
    xd = x.to(DEV).clone()
    assert ops().gated_dyt_residual(xd, y.to(DEV), None, g.to(DEV), gb.to(DEV),
                                    tuple(t.to(DEV) for t in post)) is None
    assert (xd.cpu() - (x + pz.dynamic_tanh(y.sum(0) * gate, *post))).abs().max() <= 3e-6


@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,ff,S", [(1, 70, 1), (5, 1000, 2), (40, 5000, 1)])
def test_polynorm(odt, n, ff, S):
    z = rnd(S, n, ff, scale=1.5, seed=1)
    coef = torch.tensor([0.6, -0.3, 0.2, 0.05])
    want = pz.polynorm(z.sum(0), coef, 1e-5)
    got = ops().polynorm(z.to(DEV), coef.to(DEV), 1e-5, odt).float().cpu()
    tol = 2e-5 if odt == torch.float32 else 2e-2
    assert (got - want).abs().max() <= tol * want.abs().max()
    # a row's result does not depend on the rows beside it
    alone = ops().polynorm(z[:, -1:].contiguous().to(DEV), coef.to(DEV), 1e-5, odt).float().cpu()
    assert torch.equal(alone[0], got[-1])


def test_embed_with_positions():
    table, pos = bf(rnd(90, 100, seed=1)), bf(rnd(40, 100, seed=2))
    toks = torch.tensor([3, 89, 0, 3], dtype=torch.int32)
    rp = torch.tensor([0, 39, 7, 8], dtype=torch.int32)
    want = pz.embed(table, pos, [3], 0)
    for tdt in (torch.float32, torch.bfloat16):
        got = ops().embed_pos(table.to(tdt).to(DEV), pos.to(tdt).to(DEV), toks.to(DEV), rp.to(DEV)).cpu()
        assert torch.equal(got, table[toks.long()] + pos[rp.long()])
        assert torch.equal(got[0], want[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,extra", [(4, 2, 16, 32, 0), (3, 3, 10, 6, 0), (2, 1, 64, 64, 128)])
def test_biased_append(dtype, nh, nkv, hd, vd, extra):
    """q out, K and V into shuffled pages at the rows' positions, from partial sums and a bias;
    `extra` more columns follow q, k and v in the product (another matrix's rows)."""
    lens, rows = [70, 130], [(60, 10), (0, 130)]
    n = sum(c for _, c in rows)
    width = nh * hd + nkv * (hd + vd)
    prod = rnd(2, n, width + extra, seed=5)
    bias = rnd(width, seed=6)
    P = Paged(lens, nkv, hd, vd, dtype, 9)
    kc, vc = (torch.zeros(P.n_pages, nkv, PAGE, d, dtype=dtype, device=DEV) for d in (hd, vd))
    row_pos = torch.tensor([p for (p0, cnt) in rows for p in range(p0, p0 + cnt)], dtype=torch.int32)
    row_seq = torch.tensor([i for i, (p0, cnt) in enumerate(rows) for _ in range(cnt)], dtype=torch.int32)
    q = ops().qkv_bias_append(prod.to(DEV), bias.to(DEV), row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV),
                              kc, vc, nh, hd, dtype).float().cpu()
    full = (prod.sum(0)[:, :width] + bias)
    want = full.to(dtype).float()
    assert torch.equal(q.reshape(n, -1), want[:, :nh * hd])
    kc, vc = kc.float().cpu(), vc.float().cpu()
    for r in range(n):
        pg, at = int(P.table[row_seq[r], row_pos[r] // PAGE]), int(row_pos[r]) % PAGE
        assert torch.equal(kc[pg, :, at].reshape(-1), want[r, nh * hd:nh * hd + nkv * hd])
        assert torch.equal(vc[pg, :, at].reshape(-1), want[r, nh * hd + nkv * hd:])
    # a product that holds q alone
    q = ops().qkv_bias_append(prod[:, :, :nh * hd].contiguous().to(DEV), bias[:nh * hd].contiguous().to(DEV),
                              row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV), None, None, nh, hd, dtype)
    assert torch.equal(q.float().cpu().reshape(n, -1), want[:, :nh * hd])


# ------------------------------------------------------------------ attention
class Paged:
    """Keys and values of several sequences in pages that lie in no order."""

    def __init__(self, lens, nkv, hd, vd, dtype, seed):
        self.lens, self.nkv, self.hd, self.vd, self.dtype = lens, nkv, hd, vd, dtype
        need = [(n + PAGE - 1) // PAGE for n in lens]
        self.n_pages = sum(need) + 3
        perm = torch.randperm(self.n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        width = (max(need) + 7) // 8 * 8
        self.table = torch.full((len(lens), width), -1, dtype=torch.int32)
        for i, n in enumerate(need):
            for j in range(n):
                self.table[i, j] = perm.pop()
        self.k = [rnd(n, nkv, hd, seed=seed + 10 + i) for i, n in enumerate(lens)]
        self.v = [rnd(n, nkv, vd, seed=seed + 50 + i) for i, n in enumerate(lens)]
        if dtype == torch.bfloat16:
            self.k, self.v = [bf(t) for t in self.k], [bf(t) for t in self.v]

    def caches(self):
        kc = torch.zeros(self.n_pages, self.nkv, PAGE, self.hd)
        vc = torch.zeros(self.n_pages, self.nkv, PAGE, self.vd)
        for i, n in enumerate(self.lens):
            for t in range(n):
                pg = int(self.table[i, t // PAGE])
                kc[pg, :, t % PAGE] = self.k[i][t]
                vc[pg, :, t % PAGE] = self.v[i][t]
        return kc.to(self.dtype).to(DEV), vc.to(self.dtype).to(DEV)


def run_attention(dtype, hd, vd, nh, nkv, lens, rows, window=0, standout=(), mode="plain", seed=0,
                  sink_value=None, temp_sign=1.0):
    """rows: per sequence, (first position, count) of the rows that ask.  standout: (sequence,
    key position, query position): that key is made to dominate that query's scores in every head."""
    P = Paged(lens, nkv, hd, vd, dtype, seed)
    scale = 0.7 / hd ** 0.5
    temp = temp_sign * (1.0 + rnd(nh, seed=seed + 1).abs() * 0.5)
    sink = rnd(nh, seed=seed + 2) + 0.5 if sink_value is None else torch.full((nh,), float(sink_value))
    qs = []
    for i, (p0, cnt) in enumerate(rows):
        q = rnd(cnt, nh, hd, seed=seed + 100 + i)
        qs.append(bf(q) if dtype == torch.bfloat16 else q)
    for (si, kp, qp) in standout:
        p0, cnt = rows[si]
        G = nh // nkv
        for g in range(nkv):
            # the key takes the direction of the group's first query head; all heads of the group
            # get that direction too, so that the score is large for each
            d = qs[si][qp - p0, g * G].clone()
            d = d / d.norm()
            for a in range(g * G, (g + 1) * G):
                qs[si][qp - p0, a] = (d * 6.0 * temp_sign)
            P.k[si][kp, g] = d * (8.0 / scale / 6.0)
            P.v[si][kp, g] = 5.0
        if dtype == torch.bfloat16:
            qs[si], P.k[si], P.v[si] = bf(qs[si]), bf(P.k[si]), bf(P.v[si])
    want = [pz.sink_attention(qs[i], P.k[i][:p0 + cnt], P.v[i][:p0 + cnt], scale, temp, sink, pos0=p0,
                              window=window) for i, (p0, cnt) in enumerate(rows)]
    kc, vc = P.caches()
    q_all = torch.cat(qs).to(dtype).to(DEV)
    row_pos = torch.tensor([p for (p0, cnt) in rows for p in range(p0, p0 + cnt)], dtype=torch.int32)
    row_seq = torch.tensor([i for i, (p0, cnt) in enumerate(rows) for _ in range(cnt)], dtype=torch.int32)
    chunk = ops().attention_chunk()
    max_chunks = int(row_pos.max()) // chunk + 1
    if window:
        max_chunks = min(max_chunks, (window - 1) // chunk + 2)
    kw = dict(head_scale=temp.to(DEV), sink=sink.to(DEV))
    if mode == "plain":
        kw["force_simt"] = True
    elif mode == "blocks":
        per = ops().attention_block_positions(nh, nkv)
        r0, row0 = [], 0
        for (p0, cnt) in rows:
            r0.append(row0)
            row0 += cnt
        kw["blocks"] = ops().attention_blocks(r0, [p for p, _ in rows], [c for _, c in rows], per,
                                              torch.device(DEV))
    elif mode == "decode":
        kw["decode"] = True
    got = ops().attention(q_all, kc, vc, row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV), window, scale,
                          max_chunks, **kw).float().cpu()
    assert ops().attn_tc_error() == 0
    return got, torch.cat(want)


def close(got, want, dtype):
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = (got - want).abs().max() / want.abs().max()
    assert err <= tol, f"{err:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,vd,nh,nkv", [(16, 32, 4, 2), (24, 40, 6, 2), (8, 8, 3, 3), (64, 64, 4, 1),
                                          (128, 128, 2, 2), (64, 128, 8, 2), (48, 16, 10, 2)])
def test_sink_attention_plain_kernel(dtype, hd, vd, nh, nkv):
    lens = [1, 200, 67, 330]
    got, want = run_attention(dtype, hd, vd, nh, nkv, lens, [(0, 1), (0, 200), (60, 7), (329, 1)], seed=3)
    close(got, want, dtype)


@pytest.mark.parametrize("hd,nh,nkv", [(64, 4, 1), (64, 10, 5), (128, 2, 2), (128, 8, 2), (128, 40, 2)])
def test_sink_attention_tensor_core_kernels(hd, nh, nkv):
    dt = torch.bfloat16
    lens = [1, 300, 131, 520]
    got, want = run_attention(dt, hd, hd, nh, nkv, lens, [(0, 1), (0, 300), (100, 31), (0, 520)],
                              mode="blocks", seed=4)
    close(got, want, dt)
    got, want = run_attention(dt, hd, hd, nh, nkv, lens, [(0, 1), (299, 1), (130, 1), (519, 1)],
                              mode="decode", seed=5)
    close(got, want, dt)
    # a head's factor below zero: decode rows take it, prompts go to the plain kernel
    for mode, rows in (("decode", [(0, 1), (299, 1), (130, 1), (519, 1)]),
                       ("blocks", [(0, 1), (0, 300), (100, 31), (0, 520)])):
        got, want = run_attention(dt, hd, hd, nh, nkv, lens, rows, mode=mode, seed=6, temp_sign=-1.0)
        close(got, want, dt)


MODES = [(torch.float32, "plain", 16, 32), (torch.bfloat16, "plain", 24, 40), (torch.bfloat16, "blocks", 64, 64),
         (torch.bfloat16, "decode", 64, 64), (torch.bfloat16, "blocks", 128, 128),
         (torch.bfloat16, "decode", 128, 128)]


@pytest.mark.parametrize("dtype,mode,hd,vd", MODES)
def test_a_sink_that_outweighs_every_key(dtype, mode, hd, vd):
    # exp(sink) is far larger than every exp(score): the output all but vanishes; leaving
    # the sink out would give values of the order of 1
    rows = [(0, 1), (299, 1)] if mode == "decode" else [(0, 1), (0, 300)]
    got, want = run_attention(dtype, hd, vd, 4, 2, [1, 300], rows, mode=mode, sink_value=14.0, seed=7)
    assert want.abs().max() < 1e-2 and got.abs().max() < 1e-2 
    got, want = run_attention(dtype, hd, vd, 4, 2, [1, 300], rows, mode=mode, sink_value=-30.0, seed=7)
    close(got, want, dtype)


@pytest.mark.parametrize("dtype,mode,hd,vd", MODES)
def test_one_key_that_stands_out(dtype, mode, hd, vd):
    """A key far back, at a page's and a chunk's border, and the first one: made to dominate
    one query's scores, with a value that shows."""
    n = 900
    for kp, qp in [(3, 899), (0, 700), (63, 899), (64, 640), (127, 128), (128, 899), (767, 768), (512, 513)]:
        rows = [(qp, 1)] if mode == "decode" else [(max(0, qp - 40), min(41, qp + 1))]
        got, want = run_attention(dtype, hd, vd, 4, 2, [n], rows, mode=mode, standout=[(0, kp, qp)], seed=kp)
        assert want[-1].abs().max() > 3.0           # the key does dominate its query
        close(got, want, dtype)


@pytest.mark.parametrize("dtype,mode,hd,vd", MODES)
@pytest.mark.parametrize("window", [37, 128, 200])
def test_keys_at_a_windows_edge(dtype, mode, hd, vd, window):
    n = 600
    for qp in (window - 1, window, 300, 599):
        inside, outside = qp + 1 - window, qp - window
        rows = [(qp, 1)] if mode == "decode" else [(max(0, qp - 20), min(21, qp + 1))]
        got, want = run_attention(dtype, hd, vd, 4, 2, [n], rows, window=window, mode=mode,
                                  standout=[(0, inside, qp)], seed=qp)
        assert want[-1].abs().max() > 3.0
        close(got, want, dtype)
        if outside >= 0:
            got, want = run_attention(dtype, hd, vd, 4, 2, [n], rows, window=window, mode=mode,
                                      standout=[(0, outside, qp)], seed=qp)
            assert want[-1].abs().max() < 3.0       # just outside: it must not show
            close(got, want, dtype)


# ------------------------------------------------------------------ whole models
LENGTHS = {"ZA": [1, 2, 9, 70, 131, 260], "ZB": [1, 3, 64, 65, 200, 410], "ZC": [2, 17, 128, 129, 300, 640],
           "ZD": [1, 5, 33, 64, 190], "ZE": [1, 6, 63, 127, 270]}
FP32_TOL = 2e-5
BF16_TOL = 4e-2
_ENGINES = {}


def requests(name):
    rng = np.random.default_rng(300 + len(name) + ord(name[1]))
    return [rng.integers(0, CONFIGS[name]["vocab"], size=n).tolist() for n in LENGTHS[name]]


def engine(name, dtype, max_tokens=2048):
    from janas_b200.engine import Engine
    key = (name, dtype, max_tokens)
    if key not in _ENGINES:
        _ENGINES[key] = Engine.open(model(name)[0], dtype=dtype, max_tokens=max_tokens)
    return _ENGINES[key]


_PLAIN = {}


def plain_logits(name, toks, rounding=None):
    key = (name, tuple(toks), rounding)
    if key not in _PLAIN:
        _, c, w = model(name)
        _PLAIN[key] = pz.forward(c, w, list(toks), rounding).numpy()
    return _PLAIN[key]


def check(name, dtype, got, reqs, ids):
    for rid, toks in zip(ids, reqs):
        have = np.stack([got[rid][p] for p in range(len(toks))])
        if dtype == "float32":
            e = rel_err(have, plain_logits(name, toks))
            assert e <= FP32_TOL, f"{name} {rid} len {len(toks)}: {e:.3e}"
        else:
            e = rel_err(have, plain_logits(name, toks, "bfloat16"))
            assert e <= BF16_TOL, f"{name} {rid} len {len(toks)}: {e:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(name, dtype):
    reqs = requests(name)
    got = run_trace(engine(name, dtype), trace_whole(reqs))
    check(name, dtype, got, reqs, [f"r{i}" for i in range(len(reqs))])


def test_layer_by_layer():
    from janas_b200.engine.engine import StepEntry
    name = "ZA"
    toks = requests(name)[3]
    _, c, w = model(name)
    trace = []
    pz.forward(c, w, toks, None, trace)
    e = engine(name, "float32")
    s = e.new_sequence()
    got = e.step_trace([StepEntry(s, toks, [])])
    e.free_sequence(s)
    assert len(got) == len(trace)
    for i, (g, t) in enumerate(zip(got, trace)):
        err = np.abs(np.asarray(g).reshape(t.shape) - t.numpy()).max() / t.abs().max().item()
        assert err <= 1e-5, f"layer {i}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    reqs = requests(name)
    # long tails: decoding runs over page and chunk borders
    got = run_trace(engine(name, dtype), trace_tail(reqs, tail=140))
    check(name, dtype, got, reqs, [f"r{i}" for i in range(len(reqs))])


def trace_portions(reqs, sizes):
    """Each request alone, cut into portions whose sizes cycle through ``sizes``."""
    steps, k = [], 0
    for i, toks in enumerate(reqs):
        at, j = 0, i
        while at < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"step": k, "entries": [{"id": f"r{i}", "tokens": toks[at:at + n],
                                                  "want": list(range(n))}],
                          "end": [f"r{i}"] if at + n == len(toks) else []})
            at, j, k = at + n, j + 1, k + 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["ZA", "ZB", "ZC"])
def test_portions(name, dtype):
    reqs = requests(name)
    for sizes in ([2], [64, 3, 61, 2, 130], [7, 1, 128]):
        sel = reqs if sizes != [2] else reqs[:4]
        got = run_trace(engine(name, dtype), trace_portions(sel, sizes))
        check(name, dtype, got, sel, [f"r{i}" for i in range(len(sel))])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_batches_of_unequal_requests(name, dtype):
    reqs = requests(name)
    # two batches one after the other in a cache that holds little more than one of
    # them: slots and pages are used again; the shorter requests end earlier
    b0 = [(reqs[5 % len(reqs)], len(reqs[5 % len(reqs)]) - 20), (reqs[0], 1), (reqs[3], len(reqs[3]) - 33),
          (reqs[2], 2)]
    b1 = [(reqs[4], len(reqs[4]) - 9), (reqs[1], 1), (reqs[3], 40)]
    for b in (b0, b1):
        for i, (t, p) in enumerate(b):
            b[i] = (t, max(1, min(p, len(t))))
    need = max(sum((len(t) + 63) // 64 * 64 for t, _ in b) for b in (b0, b1))
    e = engine(name, dtype, max_tokens=need)
    got = run_trace(e, trace_batches([b0, b1, b0]))
    for b, batch in enumerate([b0, b1, b0]):
        check(name, dtype, got, [t for t, _ in batch], [f"b{b}r{i}" for i in range(len(batch))])
    e.cache.check()
    # in 32-bit a request's logits are the same bits whatever runs beside it
    if dtype == "float32":
        alone = run_trace(e, trace_tail([b0[0][0]], tail=20))
        for p in range(len(b0[0][0])):
            assert np.array_equal(alone["r0"][p], got["b0r0"][p])


def test_fused_and_step_by_step_agree():
    """The kernel that ends a sublayer in one pass against the same steps one by one
    (a model whose gates are absent takes the steps one by one)."""
    from janas_b200.config import config_from_dict
    from janas_b200.engine import Engine
    import dataclasses
    name = "ZA"
    folder, c, w = model(name)
    spec = config_from_dict(c).to_model_spec()
    layers = tuple(dataclasses.replace(l, block_params={**l.block_params, "fuse": False}) for l in spec.layers)
    slow = Engine.from_spec(dataclasses.replace(spec, layers=layers),
                            tensors={k: v.to(DEV) for k, v in w.items()}, dtype="float32", max_tokens=512)
    toks = requests(name)[4]
    got = run_trace(slow, trace_whole([toks]))
    have = np.stack([got["r0"][p] for p in range(len(toks))])
    assert rel_err(have, plain_logits(name, toks)) <= FP32_TOL
    fast = run_trace(engine(name, "float32"), trace_whole([toks]))
    assert rel_err(np.stack([fast["r0"][p] for p in range(len(toks))]), have) <= 1e-6


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["ZA", "ZC"])
def test_greedy_generation_through_the_entry_point(name):
    import janas_b200
    folder, c, w = model(name)
    llm = janas_b200.open(folder, janas_b200.LLMParams(n_ctx=c["max_positions"], dtype="float32", max_batch=4,
                                                       max_tokens=1024))
    prompts = [requests(name)[2], requests(name)[1], requests(name)[3][:50]]
    outs, _ = llm.generate_batch(prompts, [12, 5, 9])
    for p, o, n in zip(prompts, outs, [12, 5, 9]):
        seq = list(p)
        for _ in range(n):
            lg = pz.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            nxt = int(lg.argmax())
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            assert o[len(seq) - len(p)] == nxt
            seq.append(nxt)
    llm.close()
