"""The Dunavik design on the GPU: each mechanism's kernel alone against the plain
restatement, then whole models through the engine under every way of cutting the
work, and greedy generation through the library's own entry point."""
import math

import numpy as np
import pytest
import torch

import plain_dunavik as pd
from dunavik_models import CONFIGS, model
from helpers import rel_err, run_trace, trace_batches, trace_tail, trace_whole

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


def close(got, want, dtype, what="", bf16_tol=2e-2):
    tol = 2e-5 if dtype == torch.float32 else bf16_tol
    err = (got - want).abs().max() / want.abs().max()
    assert err <= tol, f"{what} {err:.3e}"


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,dm", [(1, 50), (7, 256), (130, 1000), (3, 4100)])
def test_layer_norm(odt, n, dm):
    x = rnd(n, dm, scale=2.0) + 3.0                    # a mean that matters
    w, b = 1 + rnd(dm, scale=0.2, seed=1), rnd(dm, scale=0.3, seed=2)
    want = pd.layer_norm(x, w, b, 1e-5)
    got = ops().layernorm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-5, odt).float().cpu()
    assert (got - want).abs().max() <= (2e-6 * want.abs().max() if odt == torch.float32 else 3e-2)
    # two stacks of partial sums join the stream first, times a factor, in place
    a, c = rnd(3, n, dm, seed=3), rnd(2, n, dm, seed=4)
    xd = x.to(DEV).clone()
    got = ops().layernorm(xd, w.to(DEV), b.to(DEV), 1e-5, torch.float32, a=a.to(DEV), b=c.to(DEV), mult=0.6).cpu()
    xs = x + 0.6 * (a.sum(0) + c.sum(0))
    assert torch.allclose(xd.cpu(), xs, atol=2e-6, rtol=1e-6)
    assert (got - pd.layer_norm(xs, w, b, 1e-5)).abs().max() <= 1e-5
    # one stack alone, and the add without a norm
    xd = x.to(DEV).clone()
    assert ops().layernorm(xd, None, None, 0.0, torch.float32, a=a.to(DEV), mult=1.0) is None
    assert torch.allclose(xd.cpu(), x + a.sum(0), atol=2e-6, rtol=1e-6)
    # a choice of rows; no bias
    rows = torch.tensor([n - 1, 0], dtype=torch.int32)
    got = ops().layernorm(x.to(DEV), w.to(DEV), None, 1e-5, torch.float32, rows=rows.to(DEV)).cpu()
    assert (got - pd.layer_norm(x[rows.long()], w, torch.zeros(dm), 1e-5)).abs().max() <= 1e-5


def test_layer_norm_is_not_an_rms_norm():
    x = rnd(4, 96) + 5.0
    w, b = torch.ones(96), torch.zeros(96)
    got = ops().layernorm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-6, torch.float32).cpu()
    assert got.mean(dim=1).abs().max() < 1e-5 and (got.var(dim=1, unbiased=False) - 1).abs().max() < 1e-4


@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,ff,S,extra", [(1, 70, 1, 0), (5, 1000, 2, 24), (40, 5000, 1, 0)])
def test_relu_squared(odt, n, ff, S, extra):
    z = rnd(S, n, ff + extra, seed=2)
    want = torch.relu(z.sum(0)[:, :ff]) ** 2
    got = ops().activation(z.to(DEV), "relu2", odt, ff).float().cpu()
    assert (got - want).abs().max() <= (1e-6 if odt == torch.float32 else 2e-2 * want.abs().max())
    assert (got[z.sum(0)[:, :ff] < 0] == 0).all()


@pytest.mark.parametrize("H,n,k,m", [(4, 1, 16, 40), (3, 8, 64, 384), (2, 70, 96, 64), (5, 200, 384, 128),
                                     (2, 300, 64, 200), (8, 1030, 128, 96)])
def test_one_product_per_head_in_one_launch(H, n, k, m):
    """Heads whose rows of activations and of weights are no multiple of any tile."""
    a, w = bf(rnd(H, n, k, seed=1)), bf(rnd(H * m, k, seed=2) / k ** 0.5)
    got = ops().linear_heads(a.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV)).sum(1).cpu()
    assert ops().gemm_tc_error() == 0
    want = torch.einsum("hnk,hmk->hnm", a, w.reshape(H, m, k))
    assert (got - want).abs().max() <= 1e-4 * max(1.0, float(want.abs().max()))


class Paged:
    """Rows of several sequences in pages that lie in no order."""

    def __init__(self, lens, seed):
        need = [(n + PAGE - 1) // PAGE for n in lens]
        self.lens = lens
        self.n_pages = sum(need) + 3
        perm = torch.randperm(self.n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        width = (max(need) + 7) // 8 * 8
        self.table = torch.full((len(lens), width), -1, dtype=torch.int32)
        for i, n in enumerate(need):
            for j in range(n):
                self.table[i, j] = perm.pop()

    def fill(self, per_seq, heads, dim, dtype):
        """per_seq[i]: [len, heads, dim] -> a cache tensor [pages, heads, PAGE, dim]"""
        c = torch.zeros(self.n_pages, heads, PAGE, dim)
        for i, n in enumerate(self.lens):
            for t in range(n):
                c[int(self.table[i, t // PAGE]), :, t % PAGE] = per_seq[i][t]
        return c.to(dtype).to(DEV)

    def read(self, cache, seq, pos):
        return cache[int(self.table[seq, pos // PAGE]), :, pos % PAGE]


def row_arrays(rows):
    row_pos = torch.tensor([p for (p0, cnt) in rows for p in range(p0, p0 + cnt)], dtype=torch.int32)
    row_seq = torch.tensor([i for i, (p0, cnt) in enumerate(rows) for _ in range(cnt)], dtype=torch.int32)
    return row_pos, row_seq


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,every", [(4, 2, 16, 32, 16), (3, 3, 10, 6, 1), (2, 1, 64, 64, 100)])
def test_query_temperature_and_append(dtype, nh, nkv, hd, vd, every):
    """q times its position's factor, K and V (no factor) into shuffled pages."""
    lens, rows = [70, 330], [(60, 10), (0, 330)]
    n = sum(c for _, c in rows)
    width = nh * hd + nkv * (hd + vd)
    prod = rnd(2, n, width, seed=5)
    P = Paged(lens, 9)
    kc, vc = (torch.zeros(P.n_pages, nkv, PAGE, d, dtype=dtype, device=DEV) for d in (hd, vd))
    row_pos, row_seq = row_arrays(rows)
    q = ops().qkv_bias_append(prod.to(DEV), None, row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV), kc, vc,
                              nh, hd, dtype, q_temp_coef=0.3, q_temp_every=every).float().cpu()
    full = prod.sum(0)
    t = pd.query_temperature(row_pos, 0.3, every)
    assert t.max() > 1.2 and t.min() >= 1.0
    want_q = (full[:, :nh * hd] * t[:, None]).to(dtype).float()
    assert (q.reshape(n, -1) - want_q).abs().max() <= (1e-6 if dtype == torch.float32 else 1e-2) * want_q.abs().max()
    want = full.to(dtype).float()
    kc, vc = kc.float().cpu(), vc.float().cpu()
    for r in range(0, n, 7):
        assert torch.equal(P.read(kc, int(row_seq[r]), int(row_pos[r])).reshape(-1), want[r, nh * hd:nh * hd + nkv * hd])
        assert torch.equal(P.read(vc, int(row_seq[r]), int(row_pos[r])).reshape(-1), want[r, nh * hd + nkv * hd:])


def run_window_attention(dtype, hd, vd, nh, nkv, lens, rows, window=0, cap=0.0, standout=(), seed=0,
                         decode=False, mode="plain"):
    """rows: per sequence, (first position, count) of the rows that ask.  standout: (sequence, key
    position, query position): that key is made to dominate that query's scores in the LAST head's
    group (the head whose slope is smallest)."""
    P = Paged(lens, seed)
    scale = 0.7 / hd ** 0.5
    ks = [rnd(n, nkv, hd, seed=seed + 10 + i) for i, n in enumerate(lens)]
    vs = [rnd(n, nkv, vd, seed=seed + 50 + i) for i, n in enumerate(lens)]
    qs = [rnd(cnt, nh, hd, seed=seed + 100 + i) for i, (p0, cnt) in enumerate(rows)]
    for (si, kp, qp) in standout:
        p0, cnt = rows[si]
        d = qs[si][qp - p0, nh - 1].clone()
        d = d / d.norm()
        G = nh // nkv
        for a in range(nh - G, nh):
            qs[si][qp - p0, a] = d * 6.0
        ks[si][kp, nkv - 1] = d * (40.0 / scale / 6.0)       # a raw score of 40 before the cap
        vs[si][kp, nkv - 1] = 5.0
    if dtype == torch.bfloat16:
        qs, ks, vs = [bf(t) for t in qs], [bf(t) for t in ks], [bf(t) for t in vs]
    want = [pd.attention_core(qs[i], ks[i][:p0 + cnt], vs[i][:p0 + cnt], scale, p0, window, cap, 8.0)
            for i, (p0, cnt) in enumerate(rows)]
    kc, vc = P.fill(ks, nkv, hd, dtype), P.fill(vs, nkv, vd, dtype)
    row_pos, row_seq = row_arrays(rows)
    chunk = ops().attention_chunk()
    max_chunks = int(row_pos.max()) // chunk + 1
    if window:
        max_chunks = min(max_chunks, (window - 1) // chunk + 2)
    slopes = torch.tensor([2.0 ** (-8.0 * (a + 1) / nh) for a in range(nh)], dtype=torch.float32)
    kw = {}
    if mode == "plain":
        kw["force_simt"] = True
    elif not decode:
        # the tensor-core kernel for prompts: runs of consecutive positions
        per = ops().attention_block_positions(nh, nkv)
        r0, at = [], 0
        for (p0, cnt) in rows:
            r0.append(at)
            at += cnt
        kw["blocks"] = ops().attention_blocks(r0, [p for p, _ in rows], [c for _, c in rows], per,
                                              torch.device(DEV))
    got = ops().attention(torch.cat(qs).to(dtype).to(DEV), kc, vc, row_pos.to(DEV), row_seq.to(DEV),
                          P.table.to(DEV), window, scale, max_chunks, decode=decode, softcap=cap,
                          slopes=slopes.to(DEV), **kw).float().cpu()
    assert ops().attn_tc_error() == 0
    return got, torch.cat(want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,vd,nh,nkv,window,cap", [(16, 32, 4, 2, 37, 20.0), (24, 40, 6, 2, 0, 0.0),
                                                     (8, 8, 3, 3, 200, 5.0), (64, 64, 4, 1, 130, 50.0),
                                                     (128, 128, 2, 2, 64, 0.0)])
def test_capped_sloped_window_attention(dtype, hd, vd, nh, nkv, window, cap):
    lens = [1, 200, 67, 330]
    got, want = run_window_attention(dtype, hd, vd, nh, nkv, lens, [(0, 1), (0, 200), (60, 7), (329, 1)],
                                     window, cap, seed=3)
    close(got, want, dtype)
    got, want = run_window_attention(dtype, hd, vd, nh, nkv, lens, [(0, 1), (199, 1), (66, 1), (329, 1)],
                                     window, cap, seed=4, decode=True)
    close(got, want, dtype)


@pytest.mark.parametrize("hd,nh,nkv,window,cap", [(64, 4, 1, 130, 50.0), (64, 10, 5, 0, 20.0), (128, 2, 2, 64, 8.0),
                                                   (128, 8, 2, 1000, 0.0), (128, 40, 2, 37, 25.0)])
def test_capped_sloped_window_attention_on_the_tensor_cores(hd, nh, nkv, window, cap):
    dt = torch.bfloat16
    lens = [1, 300, 131, 520]
    got, want = run_window_attention(dt, hd, hd, nh, nkv, lens, [(0, 1), (0, 300), (100, 31), (0, 520)],
                                     window, cap, seed=4, mode="tc")
    close(got, want, dt, "prompt rows")
    got, want = run_window_attention(dt, hd, hd, nh, nkv, lens, [(0, 1), (299, 1), (130, 1), (519, 1)],
                                     window, cap, seed=5, decode=True, mode="tc")
    close(got, want, dt, "decode rows")


def test_the_cap_and_the_slopes_matter():
    """Scores far above the cap: without it one key takes all the weight; and a head with a steep
    slope looks at its nearest keys only."""
    P = Paged([90], 1)
    q = torch.zeros(1, 2, 16)
    q[0, :, 0] = 1.0
    k = torch.zeros(90, 1, 16)
    k[:, 0, 0] = torch.linspace(100.0, 400.0, 90)          # raw scores far above the cap of 5
    v = torch.arange(90, dtype=torch.float32).reshape(90, 1, 1).repeat(1, 1, 16)
    slopes = torch.tensor([2.0 ** -4, 2.0 ** -8])
    want = pd.attention_core(q, k, v, 1.0, 89, 0, 5.0, 8.0)
    got = ops().attention(q.to(DEV), P.fill([k], 1, 16, torch.float32), P.fill([v], 1, 16, torch.float32),
                          torch.tensor([89], dtype=torch.int32, device=DEV),
                          torch.tensor([0], dtype=torch.int32, device=DEV), P.table.to(DEV), 0, 1.0, 1,
                          softcap=5.0, slopes=slopes.to(DEV)).cpu()
    close(got, want, torch.float32)
    # capped, the scores are all 5 and the weights follow the slopes alone: the steep head looks
    # at its last sixteen keys or so, the flat one at nearly all ninety
    assert 70.0 < float(got[0, 0, 0]) < 80.0 and 44.0 < float(got[0, 1, 0]) < 52.0


KERNELS = [(torch.float32, "plain", 32, 48), (torch.bfloat16, "plain", 32, 48), (torch.bfloat16, "tc", 64, 64),
           (torch.bfloat16, "tc", 128, 128)]


@pytest.mark.parametrize("dtype,mode,hd,vd", KERNELS)
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_that_stands_out(dtype, mode, hd, vd, decode):
    """A key far back, at a page's and a chunk's border, and the first one: made to dominate one
    query's scores in the head with the smallest slope, with a value that shows."""
    n = 900
    for kp, qp in [(3, 899), (0, 700), (63, 899), (64, 640), (127, 128), (128, 899), (767, 768), (512, 513)]:
        rows = [(qp, 1)] if decode else [(max(0, qp - 40), min(41, qp + 1))]
        got, want = run_window_attention(dtype, hd, vd, 4, 2, [n], rows, 0, 50.0, standout=[(0, kp, qp)], seed=kp,
                                         decode=decode, mode=mode)
        assert want[-1, 3].mean() > 3.0           # the key does dominate its query there
        close(got, want, dtype, f"key {kp} query {qp}")


@pytest.mark.parametrize("dtype,mode,hd,vd", KERNELS)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window", [1, 37, 64, 128, 200])
def test_keys_at_a_windows_edge(dtype, mode, hd, vd, decode, window):
    n = 600
    for qp in (window - 1, window, 300, 599):
        inside, outside = qp + 1 - window, qp - window
        rows = [(qp, 1)] if decode else [(max(0, qp - 20), min(21, qp + 1))]
        got, want = run_window_attention(dtype, hd, vd, 4, 2, [n], rows, window, 50.0, standout=[(0, inside, qp)],
                                         seed=qp, decode=decode, mode=mode)
        assert want[-1, 3].mean() > 3.0
        close(got, want, dtype, f"window {window} query {qp} inside")
        if outside >= 0:
            got, want = run_window_attention(dtype, hd, vd, 4, 2, [n], rows, window, 50.0,
                                             standout=[(0, outside, qp)], seed=qp, decode=decode, mode=mode)
            assert want[-1, 3].mean() < 2.0       # just outside: it must not show
            close(got, want, dtype, f"window {window} query {qp} outside")


# ------------------------------------------------------------ latent attention
def rope_tables(base, dims, n_pos):
    inv = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32)
    return ops().rope_table(inv.to(DEV), n_pos)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,dims,Dv,C,Cq", [(4, 16, 8, 8, 24, 40, 24), (3, 10, 6, 4, 6, 22, 14),
                                                (2, 64, 32, 32, 64, 96, 48), (1, 24, 16, 16, 40, 64, 32)])
def test_latent_attention_steps(dtype, H, D, R, dims, Dv, C, Cq):
    """The mixer's kernels in a row, from the products' sums to the gated heads, against the
    plain form that builds every head's keys and values: prompt rows of two sequences, then one
    more token of each from the cache."""
    eps, base, scale = 1e-5, 1000.0, 0.6 / (D + R) ** 0.5
    lens = [150, 70]
    P = Paged([n + 1 for n in lens], 5)
    cos, sin = rope_tables(base, dims, 256)
    wq, wc = 1 + rnd(Cq, scale=0.2, seed=1), 1 + rnd(C, scale=0.2, seed=2)
    w_uq, w_uk, w_uv = rnd(H * (D + R), Cq, seed=3) / Cq ** 0.5, rnd(H * D, C, seed=4) / C ** 0.5, rnd(H * Dv, C, seed=5) / C ** 0.5
    if dtype == torch.bfloat16:
        w_uq, w_uk, w_uv = bf(w_uq), bf(w_uk), bf(w_uv)
    G = H * Dv
    sums = [rnd(2, n + 1, Cq + C + R + G, seed=20 + i) for i, n in enumerate(lens)]      # [dq | dkv | gate]
    cache = torch.zeros(P.n_pages, 1, PAGE, C + R, dtype=dtype, device=DEV)
    w_ukT = ops().transpose_heads(w_uk.to(dtype).to(DEV), H)
    assert torch.equal(w_ukT.float().cpu().reshape(H, C, D), w_uk.to(dtype).float().reshape(H, D, C).transpose(1, 2))

    def rd(x):
        return bf(x) if dtype == torch.bfloat16 else x

    def plain(i, p0, cnt):
        z = sums[i].sum(0)
        pos = torch.arange(lens[i] + 1)
        cq = rd(pd.rms(z[:, :Cq], wq, eps))
        c = rd(pd.rms(z[:, Cq:Cq + C], wc, eps))
        kr = rd(pd.rotate_pairs(z[:, Cq + C:Cq + C + R], pos, base, dims))
        q = (cq @ w_uq.T).reshape(-1, H, D + R)
        q_plain, q_rot = rd(q[:, :, :D]), rd(pd.rotate_pairs(q[:, :, D:], pos, base, dims))
        out = pd.latent_core(q_plain[p0:p0 + cnt], q_rot[p0:p0 + cnt], c[:p0 + cnt], kr[:p0 + cnt], w_uk, w_uv,
                             scale, p0)
        gate = torch.sigmoid(z[p0:p0 + cnt, Cq + C + R:])
        return out.reshape(cnt, G) * gate, c, kr

    def run(rows, decode):
        row_pos, row_seq = row_arrays(rows)
        Pm = torch.cat([sums[i][:, p0:p0 + cnt] for i, (p0, cnt) in enumerate(rows)], dim=1).contiguous().to(DEV)
        n = Pm.shape[1]
        cq = ops().latent_down(Pm, Cq, wq.to(DEV), C, wc.to(DEV), R, cos, sin, row_pos.to(DEV), row_seq.to(DEV),
                               P.table.to(DEV), cache, eps)
        Q = ops().linear(cq, w_uq.to(dtype).to(DEV), force_simt=True)
        q_lat = ops().latent_queries(Q, w_ukT, H, D, R, C, cos, sin, row_pos.to(DEV), dtype)
        chunk = ops().attention_chunk()
        o = ops().attention(q_lat, cache, None, row_pos.to(DEV), row_seq.to(DEV), P.table.to(DEV), 0, scale,
                            int(row_pos.max()) // chunk + 1, decode=decode, value_dim=C, head_major=True)
        assert o.shape == (H, n, C)
        A = torch.stack([ops().linear(o[h], w_uv.to(dtype).to(DEV)[h * Dv:(h + 1) * Dv], force_simt=True)
                         for h in range(H)]).contiguous()
        return ops().heads_gate(A, Pm, Cq + C + R, dtype).float().cpu()

    got = run([(0, lens[0]), (0, lens[1])], False)
    want = torch.cat([plain(i, 0, lens[i])[0] for i in range(2)])
    close(got, want, dtype, "prompt", 4e-2)
    # the cache holds the normed latent and the rotated key part of every position
    _, c, kr = plain(1, 0, lens[1])
    row = P.read(cache.float().cpu(), 1, lens[1] - 1).reshape(-1)
    assert (row - torch.cat([c[lens[1] - 1], kr[lens[1] - 1]])).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * row.abs().max()
    got = run([(lens[0], 1), (lens[1], 1)], True)
    want = torch.cat([plain(i, lens[i], 1)[0] for i in range(2)])
    close(got, want, dtype, "one more token", 4e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_latent_that_stands_out(dtype):
    """One cached row far back, at page and chunk borders, dominates a query's scores: the
    weighted sum is that row's latent part (values are read from the keys' rows)."""
    C, R, H, n = 40, 8, 3, 900
    scale = 0.1
    for kp, qp in [(3, 899), (0, 700), (63, 899), (64, 640), (127, 128), (128, 899), (767, 768)]:
        rows_k = rnd(n, 1, C + R, seed=kp)
        q = rnd(1, H, C + R, seed=kp + 1)
        d = q[0, 0] / q[0, 0].norm()
        q[0, :] = d * 6.0
        rows_k[kp, 0] = d * (14.0 / scale / 6.0)
        if dtype == torch.bfloat16:
            rows_k, q = bf(rows_k), bf(q)
        want = pd.attention_core(q, rows_k, rows_k[:, :, :C], scale, qp)
        P = Paged([n], kp)
        got = ops().attention(q.to(dtype).to(DEV), P.fill([rows_k], 1, C + R, dtype), None,
                              torch.tensor([qp], dtype=torch.int32, device=DEV),
                              torch.tensor([0], dtype=torch.int32, device=DEV), P.table.to(DEV), 0, scale,
                              qp // ops().attention_chunk() + 1, decode=True, value_dim=C).float().cpu()
        assert (want[0, 0] - rows_k[kp, 0, :C]).abs().max() < 0.05 * rows_k[kp, 0].abs().max()
        close(got, want, dtype, f"key {kp} query {qp}")


# ------------------------------------------------------------------ whole models
LENGTHS = {"DA": [1, 2, 9, 70, 131, 260], "DB": [1, 3, 64, 65, 200, 410], "DC": [2, 17, 128, 129, 300, 520],
           "DD": [1, 5, 33, 64, 190, 330]}
FP32_TOL = 3e-5
BF16_TOL = 5e-2
_ENGINES = {}


def requests(name):
    rng = np.random.default_rng(500 + len(name) + ord(name[1]))
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
        _PLAIN[key] = pd.forward(c, w, list(toks), rounding).numpy()
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


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_layer_by_layer(name):
    from janas_b200.engine.engine import StepEntry
    toks = requests(name)[3]
    _, c, w = model(name)
    trace = []
    pd.forward(c, w, toks, None, trace)
    e = engine(name, "float32")
    s = e.new_sequence()
    got = e.step_trace([StepEntry(s, toks, [])])
    e.free_sequence(s)
    assert len(got) == len(trace) == len(pd.run_order(c))
    for i, (g, t) in enumerate(zip(got, trace)):
        err = np.abs(np.asarray(g).reshape(t.shape) - t.numpy()).max() / t.abs().max().item()
        assert err <= 1e-5, f"layer run {i}: {err:.3e}"


def test_every_part_shows():
    """The plain model without the embedding's second and third additions, without the cap, the
    slopes, the temperature or the gate is far from the engine's logits: the comparison tells."""
    name = "DA"
    toks = requests(name)[4]
    _, c, w = model(name)
    have = np.stack([run_trace(engine(name, "float32"), trace_whole([toks]))["r0"][p] for p in range(len(toks))])
    import copy
    for change in (lambda d: d["loop"].update(times=1), lambda d: d.update(residual_mult=1.0),
                   lambda d: d["layers"][1]["mixer"].pop("softcap"), lambda d: d["layers"][1]["mixer"].pop("q_temp"),
                   lambda d: d["layers"][1]["mixer"]["mask"].update(size=30),
                   lambda d: d["layers"][0]["mixer"]["rot"].update(base=20000.0)):
        d = copy.deepcopy(c)
        change(d)
        assert rel_err(have, pd.forward(d, w, toks).numpy()) > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    reqs = requests(name)
    # long tails: decoding runs over page, chunk and window borders
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
@pytest.mark.parametrize("name", ["DA", "DB", "DC"])
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
    b0 = [(reqs[5], len(reqs[5]) - 20), (reqs[0], 1), (reqs[3], len(reqs[3]) - 33), (reqs[2], 2)]
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


def test_prompts_per_head_and_on_the_latents_agree():
    """bfloat16 prompts of a latent mixer whose sizes the tensor-core kernel takes form keys and
    values per head; with that turned off they run on the latents like every other step.  Both
    agree with the plain model, and decoding goes on from the same cache."""
    from janas_b200.config import config_from_dict
    from janas_b200.engine import Engine
    import dataclasses
    name = "DC"
    folder, c, w = model(name)
    spec = config_from_dict(c).to_model_spec()
    assert spec.layers[1].mixer.kind == "latent_attention"
    layers = list(spec.layers)
    m = layers[1].mixer
    layers[1] = dataclasses.replace(layers[1], mixer=dataclasses.replace(m, params={**m.params, "per_head_prompts": False}))
    slow = Engine.from_spec(dataclasses.replace(spec, layers=tuple(layers)),
                            tensors={k: (v.to(torch.bfloat16) if v.dim() == 2 else v).to(DEV) for k, v in w.items()},
                            dtype="bfloat16",
                            max_tokens=2048)
    reqs = [requests(name)[4], requests(name)[2], requests(name)[5]]
    batch = [[(reqs[0], len(reqs[0]) - 30), (reqs[1], len(reqs[1])), (reqs[2], len(reqs[2]) - 70)]]
    ids = [f"b0r{i}" for i in range(3)]
    a = run_trace(slow, trace_batches(batch))
    b = run_trace(engine(name, "bfloat16"), trace_batches(batch))
    check(name, "bfloat16", a, reqs, ids)
    check(name, "bfloat16", b, reqs, ids)
    differ = max(float(np.abs(a[i][p] - b[i][p]).max()) for i, t in zip(ids, reqs) for p in range(len(t)))
    assert differ > 0.0        # two ways of rounding: the same bits would mean one path ran twice
    slow.close()


def test_the_latent_cache_has_no_values_of_its_own():
    e = engine("DA", "bfloat16")
    groups = e.cache._op("describe")["groups"]
    lat = [g for g in groups if g.get("values_in_keys")]
    assert len(lat) == 2 and sorted(g["head_dim"] for g in lat) == [24 + 4, 40 + 8]
    assert all(g["num_kv_heads"] == 1 for g in lat)
    win = [g for g in groups if not g.get("values_in_keys")]
    assert len(win) == 1 and win[0]["window"] == 37 and len(win[0]["entries"]) == 4      # two layers, two passes


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("name", ["DA", "DD"])
def test_greedy_generation_through_the_entry_point(name):
    import janas_b200
    folder, c, w = model(name)
    llm = janas_b200.open(folder, janas_b200.LLMParams(n_ctx=512, dtype="float32", max_batch=4, max_tokens=1024))
    prompts = [requests(name)[2], requests(name)[1], requests(name)[3][:50]]
    outs, _ = llm.generate_batch(prompts, [12, 5, 9])
    for p, o, n in zip(prompts, outs, [12, 5, 9]):
        seq = list(p)
        for _ in range(n):
            lg = pd.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            nxt = int(lg.argmax())
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            assert o[len(seq) - len(p)] == nxt
            seq.append(nxt)
    llm.close()


def test_long_decoding_with_captured_steps():
    """bfloat16 decode steps are captured and replayed: 300 tokens after a short prompt, a window
    that slides over them, against the plain model on the whole sequence."""
    name = "DC"
    rng = np.random.default_rng(77)
    toks = rng.integers(0, CONFIGS[name]["vocab"], size=340).tolist()
    got = run_trace(engine(name, "bfloat16"), trace_tail([toks], tail=300))
    check(name, "bfloat16", got, [toks], ["r0"])
