"""Parity of each CUDA kernel with the CPU oracle, through the C ABI.

Integer outputs (expert indices, counts, offsets, tile schedule, permutation) must be
bit-exact; router weights within 1e-5 relative; products within 2e-2 relative / 1e-3
absolute (the bars stated for this path)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL_WT = 1e-5
RTOL_OUT, ATOL_OUT = 2e-2, 1e-3


def close_out(got, ref):
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    return bool(np.all(err <= ATOL_OUT + RTOL_OUT * np.abs(ref)))


def rand_logits(rng, rows, E, stride, quant=None):
    p = rng.standard_normal((rows, stride)).astype(np.float32)
    if quant:
        p = np.round(p * quant) / quant  # many exact ties
    return np.ascontiguousarray(p.astype(np.float32))


@pytest.mark.parametrize("rows,E,K,stride,quant", [
    (512, 8, 2, 136, None), (4096, 128, 8, 256, None), (1000, 512, 10, 640, None),
    (7, 128, 8, 128, None), (1, 3, 3, 3, None), (129, 130, 16, 131, None),
    (300, 128, 8, 256, 8), (64, 16, 4, 16, 1), (257, 512, 16, 517, 4),
])
def test_route(ctx, oracle, rows, E, K, stride, quant):
    rng = np.random.default_rng(rows * 1000 + E)
    proj = rand_logits(rng, rows, E, stride, quant)
    if quant == 1:
        proj[:8] = 0.25  # all-equal rows: selection must be experts 0..K-1 in order
    ridx, rwt, rcount = oracle.route(proj, E, K)
    d_proj = ctx.upload(proj)
    d_idx, d_wt = ctx.alloc(rows * K * 4).fill(0xdeadbeef), ctx.alloc(rows * K * 4).fill(0x7fc00000)
    d_count = ctx.zeros(E * 4)
    ctx.route(d_proj, d_idx, d_wt, d_count, rows, E, K, stride)
    ctx.flush()
    idx = d_idx.read(np.uint32, (rows, K))
    wt = d_wt.read(np.float32, (rows, K))
    count = d_count.read(np.uint32, (E,))
    assert np.array_equal(idx, ridx)
    assert np.array_equal(count, rcount)
    assert np.all(np.abs(wt - rwt) <= RTOL_WT * np.abs(rwt))
    if quant == 1:
        assert np.array_equal(idx[:8], np.tile(np.arange(K, dtype=np.uint32), (8, 1)))


def test_route_refuses_too_few_candidates(ctx, mc):
    proj = np.full((4, 8), -np.inf, np.float32)
    proj[:, :2] = 1.0
    d_proj = ctx.upload(proj)
    d_idx, d_wt, d_count = ctx.alloc(64), ctx.alloc(64), ctx.zeros(32)
    ctx.route(d_proj, d_idx, d_wt, d_count, 4, 8, 3, 8)
    with pytest.raises(mc.MoeCudaError) as e:
        ctx.flush()
    assert e.value.code == mc.MOE_ERR_ROUTE
    # sticky: later calls are no-ops and the status stays
    ctx.route(d_proj, d_idx, d_wt, d_count, 4, 8, 2, 8)
    assert ctx.status() == mc.MOE_ERR_ROUTE


def test_route_nan_never_selected(ctx, oracle):
    rng = np.random.default_rng(5)
    proj = rand_logits(rng, 64, 32, 32)
    proj[:, ::3] = np.nan
    ridx, rwt, rcount = oracle.route(proj, 32, 4)
    d = ctx.upload(proj)
    d_idx, d_wt, d_count = ctx.alloc(64 * 4 * 4), ctx.alloc(64 * 4 * 4), ctx.zeros(32 * 4)
    ctx.route(d, d_idx, d_wt, d_count, 64, 32, 4, 32)
    ctx.flush()
    assert np.array_equal(d_idx.read(np.uint32, (64, 4)), ridx)
    assert np.array_equal(d_count.read(np.uint32, (32,)), rcount)


@pytest.mark.parametrize("E,tile,counts", [
    (8, 128, [110, 158, 0, 1, 127, 128, 129, 500]),
    (128, 128, None), (512, 128, None), (3, 16, [0, 0, 5]), (1, 128, [4096]),
])
def test_scan(ctx, oracle, E, tile, counts):
    rng = np.random.default_rng(E)
    count = np.array(counts, np.uint32) if counts else rng.integers(0, 400, E).astype(np.uint32)
    ntiles = int(((count.astype(np.int64) + tile - 1) // tile).sum()) + 5
    roff, rtiles = oracle.scan(count, tile, ntiles)
    d_count = ctx.upload(count)
    d_off = ctx.alloc(E * 4).fill(0xdeadbeef)
    d_tiles = ctx.alloc(ntiles * 4).fill(0xffffffff)
    ctx.scan(d_count, d_off, d_tiles, E, tile)
    ctx.flush()
    assert np.array_equal(d_off.read(np.uint32, (E,)), roff)
    assert np.array_equal(d_tiles.read(np.uint32, (ntiles,)), rtiles)


@pytest.mark.parametrize("rows,E,K,d", [(512, 8, 2, 256), (4096, 128, 8, 2048), (129, 512, 10, 64), (1, 4, 4, 8),
                                         (777, 128, 8, 520)])
def test_scatter(ctx, oracle, mc, rows, E, K, d):
    rng = np.random.default_rng(rows + E)
    proj = rand_logits(rng, rows, E, E)
    if rows > 100:
        proj[:, 1] += 4.0  # one crowded expert, some empty ones
        proj[:, 2] -= 50.0
    idx, _, count = oracle.route(proj, E, K)
    M = oracle.moe_rows(rows, K, E)
    off, _ = oracle.scan(count, 128, M // 128)
    x16 = rng.integers(0, 0x7bff, (rows, d)).astype(np.uint16)
    rxp, rslot, rfill = oracle.scatter(idx, off, x16, M)
    d_idx, d_off, d_x = ctx.upload(idx), ctx.upload(off), ctx.upload(x16)
    d_fill = ctx.zeros(E * 4)
    d_xp = ctx.zeros(M * d * 2)
    d_slot = ctx.alloc(rows * K * 4).fill(0xdeadbeef)
    ctx.scatter(d_idx, d_off, d_fill, d_x, d_xp, d_slot, rows, K, d // 8)
    ctx.flush()
    assert np.array_equal(d_slot.read(np.uint32, (rows, K)), rslot)
    assert np.array_equal(d_fill.read(np.uint32, (E,)), rfill)
    assert np.array_equal(d_xp.read(np.uint16, (M, d)), rxp)
    # calling again (same context scratch) gives the same permutation
    d_fill.fill(0)
    ctx.scatter(d_idx, d_off, d_fill, d_x, d_xp, d_slot, rows, K, d // 8)
    ctx.flush()
    assert np.array_equal(d_slot.read(np.uint32, (rows, K)), rslot)


def test_scatter_leaves_words_after_fill_alone(ctx, oracle):
    """moe_cuda_scatter has no expert count (src/pc.h:381-385) and scans the reference's 512 experts; like the
    shader's atomics it must only touch fill[e] of experts that occur in idx.  fill is E words long
    (src/qwen.c:171); the words behind it are canaries here."""
    rows, E, K, d = 300, 8, 2, 64
    rng = np.random.default_rng(5)
    idx, _, count = oracle.route(rand_logits(rng, rows, E, E), E, K)
    M = oracle.moe_rows(rows, K, E)
    off, _ = oracle.scan(count, 128, M // 128)
    x16 = rng.integers(0, 0x7bff, (rows, d)).astype(np.uint16)
    fill0 = np.full(E + 504, 0xabcd1234, np.uint32)
    fill0[:E] = 0
    d_fill = ctx.upload(fill0)
    d_xp, d_slot = ctx.zeros(M * d * 2), ctx.alloc(rows * K * 4)
    ctx.scatter(ctx.upload(idx), ctx.upload(off), d_fill, ctx.upload(x16), d_xp, d_slot, rows, K, d // 8)
    ctx.flush()
    fill = d_fill.read(np.uint32, (E + 504,))
    assert np.array_equal(fill[:E], count)
    assert np.all(fill[E:] == 0xabcd1234)


def _f16(rng, shape, std):
    return (rng.standard_normal(shape).astype(np.float32) * std).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("m,n,k,E,sa", [
    (128, 128, 64, 1, False), (128, 256, 64, 1, False), (256, 384, 128, 3, False), (512, 1024, 256, 4, True),
    (384, 640, 96, 2, False), (1280, 256, 2048, 8, False), (256, 2048, 768, 5, True), (128, 128, 8, 1, False),
])
def test_mm(ctx, oracle, mc, m, n, k, E, sa):
    """moe_cuda_mm against the oracle's product: same tile schedule, skipped tiles untouched,
    slot scale applied.  Covers one K block, ragged K (96, 8), the 128-column tail, many experts."""
    rng = np.random.default_rng(m + n + k)
    A = _f16(rng, (m, k), 1.0)
    B = _f16(rng, (E, n, k), 0.05)
    tiles = rng.integers(0, E, m // 128).astype(np.uint32)
    if m // 128 >= 3:
        tiles[1] = 0xffffffff  # a skipped tile in the middle
    amax = np.zeros(4, np.uint32)
    slot = mc.NO_SLOT
    if sa:
        amax[2] = np.float32(37.5).view(np.uint32)
        slot = 2
    ref = oracle.mm(A, B, tiles, n, k, amax=amax, sa=slot, out=np.full((m, n), 1e30, np.float32))
    d_A, d_B, d_tiles, d_amax = ctx.upload(A), ctx.upload(B), ctx.upload(tiles), ctx.upload(amax)
    d_C = ctx.upload(np.full((m, n), 1e30, np.float32))  # poisoned, as src/test_matmul_f16.c:84-89 does
    ctx.mm(d_A, d_B, d_C, d_amax, d_tiles, m, n, k, sa=slot, experts_in_B=E)
    ctx.flush()
    got = d_C.read(np.float32, (m, n))
    assert close_out(got, ref), f"max err {np.abs(got - ref).max()}"
    # the reference's own criterion for its fp16 products: max_err / max_ref < 1e-2 (src/test_matmul_f16.c:28-39)
    live = ref != 1e30
    assert np.abs(got - ref)[live].max() / np.abs(ref[live]).max() < 1e-2
    assert np.array_equal(got[~live], ref[~live])  # skipped tiles keep the poison


@pytest.mark.parametrize("rows,E,K,d,shared,hc", [(512, 8, 2, 256, False, 1), (300, 128, 8, 2048, True, 1),
                                                   (64, 16, 4, 520, True, 4), (1, 4, 4, 8, False, 1)])
def test_combine(ctx, oracle, rows, E, K, d, shared, hc):
    rng = np.random.default_rng(rows + d)
    M = oracle.moe_rows(rows, K, E)
    wt = rng.random((rows, K)).astype(np.float32)
    slot = rng.integers(0, M, (rows, K)).astype(np.uint32)
    y = rng.standard_normal((M, d)).astype(np.float32)
    proj = rng.standard_normal((rows, E + 128)).astype(np.float32)
    sh = rng.standard_normal((rows, d)).astype(np.float32) if shared else None
    inj = rng.standard_normal((rows, 12)).astype(np.float32) if hc > 1 else None
    h0 = rng.standard_normal((rows, hc, d)).astype(np.float32)
    ref = oracle.combine(wt, slot, y, proj, sh, inj, h0.copy(), sg_off=E, inj_off=3 if hc > 1 else 0, hc=hc)
    d_h = ctx.upload(h0)
    ctx.combine(ctx.upload(wt), ctx.upload(slot), ctx.upload(y), ctx.upload(proj), ctx.upload(sh) if shared else None,
                ctx.upload(inj) if inj is not None else None, d_h, rows, d, K, E + 128, E,
                inj_stride=12 if hc > 1 else 0, inj_off=3 if hc > 1 else 0, hc=hc)
    ctx.flush()
    got = d_h.read(np.float32, (rows, hc, d))
    if not shared and hc == 1:
        assert np.array_equal(got, ref)  # same operations in the same order: bit-exact
    else:
        assert np.allclose(got, ref, rtol=1e-5, atol=1e-6)  # expf differs in the last place


def test_glue(ctx, oracle, mc):
    rng = np.random.default_rng(3)
    rows, n = 384, 192
    a = (rng.standard_normal((rows, 2 * n)) * 3).astype(np.float32)
    ref_hp = oracle.swiglu(a, n, 2 * n, 0, n)
    d_a, d_hp = ctx.upload(a), ctx.alloc(rows * n * 4)
    ctx.swiglu(d_a, d_hp, rows, n, 2 * n, 0, n)
    ctx.flush()
    hp = d_hp.read(np.float32, (rows, n))
    assert np.allclose(hp, ref_hp, rtol=2e-6, atol=1e-7)
    amax = np.zeros(4, np.uint32)
    oracle.absmax(hp, amax, 1)
    d_amax = ctx.zeros(16)
    ctx.absmax(d_hp, d_amax, rows * n, 1)
    ctx.flush()
    assert np.array_equal(d_amax.read(np.uint32, (4,)), amax)
    ref16 = oracle.cast_f16(hp, amax, 1)
    d_16 = ctx.alloc(rows * n * 2)
    ctx.cast_f16(d_hp, d_16, d_amax, rows * n, 1)
    ctx.flush()
    assert np.array_equal(d_16.read(np.uint16, (rows, n)), ref16)
    assert 16384 <= np.abs(ref16.view(np.float16).astype(np.float32)).max() < 32768  # shader/cast_f16.comp scale


def test_bf16_to_f16_in_place(ctx, oracle):
    """The weight-upload conversion (shader/qwen_bf16.comp): bit-exact, odd word counts, specials."""
    rng = np.random.default_rng(8)
    for n_words in (1, 3, 4, 1000003):
        bf = rng.integers(0, 1 << 16, 2 * n_words).astype(np.uint16)
        bf[(bf & 0x7f80) == 0x7f80] &= 0xff80                            # keep infinities, drop NaN payloads
        words = np.ascontiguousarray(bf.view(np.uint32))
        d = ctx.upload(words)
        ctx.bf16_to_f16(d, n_words)
        ctx.flush()
        assert np.array_equal(d.read(np.uint32, (n_words,)), oracle.bf16_to_f16(words))


def test_kd_bytes(ctx, oracle):
    """The distillation sink (shader/kd_bytes.comp): bytes as the oracle's wherever the masses are not
    within rounding of one another, probabilities to fp16 accuracy; the shader itself sums in
    arrival order, so bit-exactness is not defined for it."""
    from tests.test_oracle import kd_inputs
    for seed, rows, vocab in ((31, 24, 3000), (32, 5, 70001)):
        logits, toks, cont = kd_inputs(seed, rows, vocab)
        d_out = ctx.alloc(rows * 16 * 8 * 4)
        d_out.fill(0xdeadbeef)
        ctx.kd_bytes(ctx.upload(logits), ctx.upload(toks), ctx.upload(cont), d_out, rows, vocab)
        ctx.flush()
        got = d_out.read(np.uint32, (rows, 16, 8))
        ref = oracle.kd_bytes(logits, toks, cont)
        pg = (got >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        pr = (ref >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        assert np.all(np.abs(pg - pr) <= 1.5e-3 * pr + 1e-7)
        differ = (got & 0xffff) != (ref & 0xffff)
        # a different byte is only acceptable between two candidates of (nearly) the same mass
        nxt = np.concatenate([pr[..., 1:], pr[..., -1:]], -1)
        prv = np.concatenate([pr[..., :1], pr[..., :-1]], -1)
        near = (np.abs(pr - nxt) <= 1.5e-3 * pr + 1e-7) | (np.abs(pr - prv) <= 1.5e-3 * pr + 1e-7)
        assert not (differ & ~near).any() and not differ[..., 0].any()
        assert differ.mean() < 0.01


def test_fill_and_copy(ctx):
    b = ctx.alloc(4 * 1003)
    b.fill(0x12345678)
    ctx.flush()
    assert np.all(b.read(np.uint32, (1003,)) == 0x12345678)
    b.fill(0xffffffff)
    assert np.all(b.read(np.uint32, (1003,)) == 0xffffffff)


def test_bad_shapes_set_sticky_status(mc):
    with mc.Ctx(0) as c:
        c.check()
        b = c.alloc(1024)
        c.route(b, b, b, b, 4, 513, 2, 513)  # experts > 512
        assert c.status() == mc.MOE_ERR_ARG
        assert "experts" in c.last_error()
    with mc.Ctx(0) as c:
        b = c.alloc(1 << 16)
        c.mm(b, b, b, None, b, 100, 128, 64)  # m not a multiple of 128
        assert c.status() == mc.MOE_ERR_ARG


def test_bounded_wait_runs_out_and_reports(mc):
    """A cross-GPU flag wait whose peer never signals: the kernel gives up after the context's
    limit, returns, and the host reads MOE_ERR_TIMEOUT with the site of the wait.  Nothing
    faults or hangs; the context stays refused afterwards (sticky)."""
    import time
    with mc.Ctx(0) as c:
        c.check()
        mc.lib().moe_cuda_set_wait_ns(c.p, 20_000_000)   # 20 ms
        t0 = time.perf_counter()
        mc.lib().moe_cuda_wait_selftest(c.p)
        with pytest.raises(mc.MoeCudaError) as e:
            c.flush()
        assert time.perf_counter() - t0 < 1.5
        assert e.value.code == mc.MOE_ERR_TIMEOUT
        assert "site 20" in c.last_error()
        assert mc.lib().moe_cuda_alloc(c.p, 64) is None  # later calls are no-ops
    with mc.Ctx(0) as c:                                 # the device is still usable
        c.check()
        b = c.zeros(64)
        c.flush()
        assert np.all(b.read(np.uint32, (16,)) == 0)


def test_alloc_refusal_is_sticky(mc):
    with mc.Ctx(0) as c:
        c.check()
        mc.lib().moe_cuda_fail_alloc_after(c.p, 1)
        with pytest.raises(mc.MoeCudaError) as e:
            c.alloc(64)
        assert e.value.code == mc.MOE_ERR_NOMEM
        assert mc.lib().moe_cuda_alloc(c.p, 64) is None  # later calls are no-ops
