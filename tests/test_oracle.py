"""Pins of the CPU oracle (no GPU): an independent numpy restatement, invariants of the
path, hand-computable cases, and the committed golden vectors."""
import os

import numpy as np
import pytest

from tests import np_restatement as NP

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "c0_seed0.npz")


def logits(rng, rows, E, stride=None, quant=None):
    stride = stride or E
    p = rng.standard_normal((rows, stride)).astype(np.float32)
    if quant:
        p = (np.round(p * quant) / quant).astype(np.float32)
    return np.ascontiguousarray(p)


@pytest.mark.parametrize("rows,E,K,quant", [(512, 8, 2, None), (300, 128, 8, None), (100, 512, 10, None),
                                             (200, 128, 8, 8), (64, 16, 16, 2), (5, 3, 1, None)])
def test_route_matches_numpy(oracle, rows, E, K, quant):
    rng = np.random.default_rng(rows + E + K)
    proj = logits(rng, rows, E, E + 7, quant)
    idx, wt, count = oracle.route(proj, E, K)
    nidx, nwt, ncount = NP.route(proj, E, K)
    assert np.array_equal(idx, nidx)          # ties to the lower expert index
    assert np.array_equal(count, ncount)
    assert np.allclose(wt, nwt, rtol=1e-5, atol=0)
    assert np.allclose(wt.sum(1), 1.0, atol=1e-6)
    assert count.sum() == rows * K
    for r in range(min(rows, 16)):
        assert len(set(idx[r])) == K          # an expert is chosen at most once per token


def test_route_tie_rule_and_order(oracle):
    proj = np.zeros((3, 8), np.float32)
    proj[1] = [1, 3, 3, 2, 3, 0, 2, 1]
    proj[2] = [-1, -1, -1, 5, -1, -1, -1, -1]
    idx, wt, count = oracle.route(proj, 8, 4)
    assert idx[0].tolist() == [0, 1, 2, 3]            # all equal: lowest indices, ascending
    assert idx[1].tolist() == [1, 2, 4, 3]            # descending logit; equal logits by index
    assert idx[2].tolist() == [3, 0, 1, 2]
    assert np.allclose(wt[0], 0.25)
    e = np.exp(np.array([0, 0, 0, -1.0]))
    assert np.allclose(wt[1], e / e.sum(), rtol=1e-6)


def test_route_refuses_when_candidates_run_out(oracle):
    proj = np.full((2, 8), -np.inf, np.float32)
    proj[:, 0] = 1.0
    with pytest.raises(ValueError):
        oracle.route(proj, 8, 2)
    proj = np.full((2, 8), np.nan, np.float32)
    with pytest.raises(ValueError):
        oracle.route(proj, 8, 1)


def test_hand_case_two_experts(oracle):
    """E=2, K=1, d=8, I=64 reduced by hand: y = w_down . (silu(w_g . x) * (w_u . x))."""
    T, d, I = 4, 8, 64
    x = np.zeros((T, d), np.float16); x[:, 0] = [1, 2, -1, 0.5]
    proj = np.array([[1, 0], [0, 1], [2, 1], [0, 0]], np.float32)
    proj = np.ascontiguousarray(np.pad(proj, ((0, 0), (0, 2))))
    wgu = np.zeros((2, 2 * I, d), np.float16); wdown = np.zeros((2, d, I), np.float16)
    wgu[0, 0, 0], wgu[0, I, 0], wdown[0, 3, 0] = 1.0, 2.0, 0.5     # expert 0: gate x0, up 2*x0, out col 3
    wgu[1, 1, 0], wgu[1, I + 1, 0], wdown[1, 5, 1] = -1.0, 1.0, 4.0
    res = oracle.layer(proj, x.view(np.uint16), wgu.view(np.uint16), wdown.view(np.uint16), 1)
    assert res.idx.ravel().tolist() == [0, 1, 0, 0]
    assert res.count.tolist() == [3, 1] and res.off.tolist() == [0, 128]
    assert res.slot.ravel().tolist() == [0, 128, 1, 2]
    silu = lambda v: v / (1 + np.exp(-v))
    want = np.zeros((T, d))
    for t, e in enumerate([0, 1, 0, 0]):
        x0 = float(x[t, 0])
        if e == 0:
            want[t, 3] = 0.5 * silu(x0) * 2 * x0
        else:
            want[t, 5] = 4.0 * silu(-x0) * x0
    assert np.allclose(res.h[:, 0], want, rtol=2e-3, atol=1e-6)


@pytest.mark.parametrize("E,tile", [(8, 128), (128, 128), (512, 128), (5, 16)])
def test_scan_matches_numpy(oracle, E, tile):
    rng = np.random.default_rng(E)
    count = rng.integers(0, 3 * tile, E).astype(np.uint32)
    count[rng.integers(0, E)] = 0
    off, tiles = oracle.scan(count, tile)
    noff, ntiles = NP.scan(count, tile)
    assert np.array_equal(off, noff) and np.array_equal(tiles, ntiles)
    assert np.all(off % tile == 0)


@pytest.mark.parametrize("rows,E,K,d", [(512, 8, 2, 64), (300, 128, 8, 32), (17, 512, 10, 8)])
def test_scatter_is_stable_bijection(oracle, rows, E, K, d):
    rng = np.random.default_rng(rows)
    idx, _, count = oracle.route(logits(rng, rows, E), E, K)
    M = oracle.moe_rows(rows, K, E)
    off, tiles = oracle.scan(count, 128, M // 128)
    x16 = rng.integers(0, 65535, (rows, d)).astype(np.uint16)
    xp, slot, fill = oracle.scatter(idx, off, x16, M)
    assert np.array_equal(slot, NP.scatter_slots(idx, off))
    assert np.array_equal(fill, count)
    flat = slot.ravel()
    assert len(np.unique(flat)) == rows * K                 # injective
    assert np.array_equal(xp[flat], np.repeat(x16, K, 0))   # permute then gather = identity
    used = np.zeros(M, bool); used[flat] = True
    assert not xp[~used].any()                              # padding rows stay zero
    # inside an expert, positions ascend with the token index
    for e in np.unique(idx)[:8]:
        r, j = np.where(idx == e)
        assert np.all(np.diff(slot[r, j]) == 1) and slot[r[0], j[0]] == off[e]
    assert np.array_equal(tiles[slot // 128], idx)          # each row sits in a tile of its expert


def test_slot_scale(oracle):
    amax = np.zeros(4, np.uint32)
    amax[0] = np.float32(9.2).view(np.uint32)
    amax[1] = np.float32(np.inf).view(np.uint32)
    amax[3] = np.float32(0.75).view(np.uint32)
    assert oracle.slot_scale(amax, 0) == 2048.0        # 9.2 * 2048 lies in [16384, 32768)
    assert oracle.slot_scale(amax, 1) == 1.0           # inf: no scale (shader/cast_f16.comp:23-25)
    assert oracle.slot_scale(amax, 2) == 1.0           # zero
    assert oracle.slot_scale(amax, 3) == 32768.0
    assert oracle.slot_scale(amax, oracle.NO_SLOT) == 1.0


def test_mm_matches_float64(oracle):
    rng = np.random.default_rng(0)
    m, n, k, E = 256, 192, 96, 3
    A = (rng.standard_normal((m, k))).astype(np.float16)
    B = (rng.standard_normal((E, n, k)) * 0.1).astype(np.float16)
    tiles = np.array([2, 0xffffffff], np.uint32)
    C = oracle.mm(A.view(np.uint16), B.view(np.uint16), tiles, n, k, out=np.full((m, n), 5.0, np.float32))
    want = A[:128].astype(np.float64) @ B[2].astype(np.float64).T
    assert np.allclose(C[:128], want, rtol=1e-5, atol=1e-5)
    assert np.all(C[128:] == 5.0)                       # skipped tile untouched
    amax = np.zeros(4, np.uint32); amax[1] = np.float32(3.0).view(np.uint32)
    C2 = oracle.mm(A.view(np.uint16), B.view(np.uint16), tiles, n, k, amax=amax, sa=1)
    assert np.array_equal(C2[:128], C[:128] / 8192.0)   # 3.0 -> 2^(141-128); power of two: exact


def test_combine_matches_numpy(oracle):
    rng = np.random.default_rng(1)
    rows, K, d, M, hc = 40, 4, 24, 640, 3
    wt = rng.random((rows, K)).astype(np.float32)
    slot = rng.integers(0, M, (rows, K)).astype(np.uint32)
    y = rng.standard_normal((M, d)).astype(np.float32)
    proj = rng.standard_normal((rows, 10)).astype(np.float32)
    sh = rng.standard_normal((rows, d)).astype(np.float32)
    inj = rng.standard_normal((rows, 7)).astype(np.float32)
    h0 = rng.standard_normal((rows, hc, d)).astype(np.float32)
    got = oracle.combine(wt, slot, y, proj, sh, inj, h0.copy(), sg_off=9, inj_off=2, hc=hc)
    sig = lambda v: 1 / (1 + np.exp(-v.astype(np.float64)))
    acc = np.einsum("rk,rkd->rd", wt.astype(np.float64), y[slot].astype(np.float64)) + sig(proj[:, 9])[:, None] * sh
    want = h0 + acc[:, None, :] * 2 * sig(inj[:, 2:2 + hc] / hc)[:, :, None]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
    # plain residual: hc = 1, no injection -> h += acc exactly (2*sigmoid(0) = 1)
    h1 = oracle.combine(wt, slot, y, None, None, None, np.zeros((rows, 1, d), np.float32), sg_off=0)
    assert np.allclose(h1[:, 0], np.einsum("rk,rkd->rd", wt.astype(np.float64), y[slot].astype(np.float64)), rtol=1e-5, atol=1e-6)


def test_layer_matches_numpy_restatement(oracle, synth):
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c0"], T=160, E=8, S=128)
    inp = synth.layer_inputs(cfg, 3)
    res = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
    idx, wt, out = NP.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
    assert np.array_equal(res.idx, idx)
    assert np.allclose(res.wt, wt, rtol=1e-5)
    assert np.allclose(res.h[:, 0], out, rtol=2e-3, atol=2e-5)
    # skipping the power-of-two requantisation moves the result far less than the tolerance
    _, _, out1 = NP.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown, requantise=False)
    assert np.abs(out1 - out).max() < 1e-4


def test_row_mask_only_skips_products(oracle, synth):
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c0"], T=96)
    inp = synth.layer_inputs(cfg, 2)
    full = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    mask = np.zeros(cfg.T, np.uint8); mask[::3] = 1
    part = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, row_mask=mask)
    assert np.array_equal(part.slot, full.slot)
    assert np.allclose(part.h[::3], full.h[::3], rtol=1e-3, atol=1e-6)  # scale slot may differ by a power of two


def test_residual_rmsnorm(oracle):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((33, 72)).astype(np.float16)
    delta = rng.standard_normal((33, 72)).astype(np.float32)
    y = oracle.residual_rmsnorm(x.view(np.uint16), delta).view(np.float16).astype(np.float64)
    v = x.astype(np.float64) + delta
    want = v / np.sqrt((v * v).mean(1, keepdims=True) + 1e-6)
    assert np.allclose(y, want, rtol=2e-3, atol=1e-3)


def test_bf16_to_f16(oracle):
    rng = np.random.default_rng(6)
    f = (rng.standard_normal(4096) * 10.0 ** rng.integers(-9, 6, 4096)).astype(np.float32)
    bf = (f.view(np.uint32) >> 16).astype(np.uint16)                      # truncated bf16 bit patterns
    bf[:6] = [0x0000, 0x8000, 0x7f80, 0xff80, 0x477f, 0x0001]            # +-0, +-inf, 65280, a bf16 denormal
    words = np.ascontiguousarray(bf.view(np.uint32))
    got = oracle.bf16_to_f16(words).view(np.uint16)
    want = (bf.astype(np.uint32) << 16).view(np.float32)
    with np.errstate(over="ignore"):
        want16 = want.astype(np.float16).view(np.uint16)                  # numpy rounds to nearest even, overflow -> inf
    assert np.array_equal(got, want16)


def kd_inputs(seed, rows=24, vocab=3000):
    """A byte-level vocabulary (random strings of 1..16 bytes over a small alphabet so that prefixes
    collide, plus a few entries of length 0) and continuations spelled from its tokens."""
    rng = np.random.default_rng(seed)
    tb = np.zeros((vocab, 16), np.uint8)
    length = rng.integers(1, 17, vocab)
    length[rng.choice(vocab, 20, replace=False)] = 0
    for t in range(vocab):
        tb[t, :length[t]] = rng.integers(97, 101, length[t])
    toks = np.concatenate([tb.view(np.uint32).reshape(vocab, 4), length[:, None].astype(np.uint32)], axis=1)
    cont = np.zeros((rows, 5), np.uint32)
    for r in range(rows):
        s = np.concatenate([tb[t, :length[t]] for t in rng.integers(0, vocab, 6)])[:16]
        c = np.zeros(16, np.uint8)
        c[:len(s)] = s
        cont[r, :4] = c.view(np.uint32)
        cont[r, 4] = [0, 1, 5, 16, 40][r % 5] if r < 10 else rng.integers(0, 17)
    logits = (rng.standard_normal((rows, vocab)) * 3).astype(np.float32)
    return logits, np.ascontiguousarray(toks), cont


def test_kd_bytes_matches_numpy(oracle):
    logits, toks, cont = kd_inputs(21)
    got = oracle.kd_bytes(logits, toks, cont)
    byte, prob = NP.kd_bytes(logits, toks, cont)
    nd = np.minimum(cont[:, 4], 16)
    for r in range(logits.shape[0]):
        assert not got[r, nd[r]:].any()                                     # depths past the continuation stay zero
    assert np.array_equal(got & 0xffff, byte)
    p = (got >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
    assert np.all(np.abs(p - prob) <= 1e-3 * prob + 1e-7)                  # fp16 entries
    live = np.arange(16)[None, :] < nd[:, None]
    assert np.all(p[live].sum(-1) <= 1.0 + 2e-3) and np.all(p[live][:, 0] >= 0)


def test_golden_vectors(oracle, synth):
    """The committed vectors were produced by tests/golden/make_golden.py from this oracle after
    it agreed with the numpy restatement; they catch any later drift of either."""
    g = np.load(GOLDEN)
    cfg = synth.CONFIGS["c0"]
    inp = synth.layer_inputs(cfg, 0)
    assert int(g["x16_sum"]) == int(inp.x16.astype(np.uint64).sum())   # the generator itself is pinned
    assert int(g["wgu_sum"]) == int(inp.wgu.astype(np.uint64).sum())
    assert np.array_equal(g["proj_head"], inp.proj[:4, :8])
    res = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    for name in ("idx", "count", "off", "tiles", "slot", "amax"):
        assert np.array_equal(g[name], getattr(res, name)), name
    assert np.allclose(g["wt"], res.wt, rtol=1e-6, atol=0)
    assert np.allclose(g["h_rows"], res.h[::8, 0], rtol=1e-5, atol=1e-7)
    assert np.array_equal(g["xp_rows"], res.xp[:4])


def test_mixer_restatement_against_numpy(oracle):
    """mda_qwen_res_rec's restatement (norm, cast, dense product, silu, cast, dense product, read-out) against the
    same arithmetic written from the definition in numpy (float64 products of the fp16 operands)."""
    rng = np.random.default_rng(0)
    rows, d, nh, rank, pad = 64, 256, 4, 64, 128
    h = rng.standard_normal((rows, nh, d)).astype(np.float32)
    wn = (rng.standard_normal(nh * d) * 0.1).astype(np.float32)
    wd = np.zeros((pad, nh * d), np.float16)
    wd[:rank + nh] = (rng.standard_normal((rank + nh, nh * d)) * 0.03).astype(np.float16)
    wu = (rng.standard_normal((nh * d, rank)) * 0.05).astype(np.float16)
    x, t, hn = oracle.res_rec(h, wn, wd.view(np.uint16), wu.view(np.uint16), nh, rank, pad)
    hn2 = h / np.sqrt((h * h).mean(-1, keepdims=True) + 1e-6) * (1 + wn.reshape(nh, d))
    assert np.abs(hn2.reshape(rows, -1) - hn).max() < 1e-5
    t2 = hn2.reshape(rows, -1).astype(np.float64) @ wd.astype(np.float64).T
    assert np.abs(t2 - t).max() < 2e-3 * np.abs(t).max()          # the fp16 cast of hn
    assert np.all(t[:, rank + nh:] == 0)                          # padded weight rows
    u2 = t2[:, :rank] / nh
    u2 = u2 / (1 + np.exp(-u2))
    up2 = u2 @ wu.astype(np.float64).T
    x2 = (1 / (1 + np.exp(-up2.reshape(rows, nh, d))) * hn2).mean(1)
    assert np.abs(x2 - x).max() < 1e-3


def test_hc_ops_against_numpy(oracle):
    rng = np.random.default_rng(1)
    rows, d, nh = 9, 24, 4
    a = rng.standard_normal((rows, d)).astype(np.float32)
    b = rng.standard_normal((rows, 16)).astype(np.float32)
    h0 = rng.standard_normal((rows, nh, d)).astype(np.float32)
    got = oracle.hc(a, b, h0.copy().reshape(rows, nh * d), rows, d, nh, 1, 16, 5).reshape(rows, nh, d)
    g = 2.0 / (1.0 + np.exp(-b[:, 5:5 + nh] / nh))
    assert np.allclose(got, h0 + a[:, None, :] * g[:, :, None], atol=1e-6)
    a2, b2 = rng.standard_normal((rows, nh * d)).astype(np.float32), rng.standard_normal((rows, nh * d)).astype(np.float32)
    assert np.allclose(oracle.hc(a2, b2, h0.copy().reshape(rows, nh * d), rows, d, nh, 2), h0.reshape(rows, -1) + a2 + b2, atol=1e-6)
