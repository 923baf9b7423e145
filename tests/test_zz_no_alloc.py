"""moe_cuda_scatter_noalloc: the scatter for hosts that must not allocate device memory while
the layer runs (their whole budget went to weights and fixed buffers at start-up, or they cannot
take the device-wide stall an allocation causes).  It keeps its per-block expert table in a
fixed array inside the library instead of growable scratch, so its results must equal
moe_cuda_scatter's bit for bit -- also on a second call, which finds the table full of the
first call's values.  Collected last so that a run stopping at the first failure has already
run every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(oracle, rng, rows, E, K, d):
    proj = np.ascontiguousarray(rng.standard_normal((rows, E)).astype(np.float32))
    proj[:, 1] += 3.0
    idx, _, count = oracle.route(proj, E, K)
    M = oracle.moe_rows(rows, K, E)
    off, _ = oracle.scan(count, 128, M // 128)
    x16 = rng.integers(0, 0x7bff, (rows, d)).astype(np.uint16)
    return idx, off, x16, M


def test_noalloc_scatter_equals_scatter_twice(ctx, oracle):
    rng = np.random.default_rng(11)
    for rows, E, K, d in [(4096, 128, 8, 256), (333, 64, 4, 72)]:  # two calls in a row share the table
        idx, off, x16, M = _case(oracle, rng, rows, E, K, d)
        d_idx, d_off, d_x = ctx.upload(idx), ctx.upload(off), ctx.upload(x16)
        out = {}
        for name in ("plain", "noalloc"):
            d_fill, d_xp = ctx.zeros(E * 4), ctx.zeros(M * d * 2)
            d_slot = ctx.alloc(rows * K * 4).fill(0xdeadbeef)
            if name == "plain":
                ctx.scatter(d_idx, d_off, d_fill, d_x, d_xp, d_slot, rows, K, d // 8)
            else:
                ctx.scatter_noalloc(d_idx, d_off, d_fill, d_x, d_xp, d_slot, rows, K, d // 8, E)
            ctx.flush()
            out[name] = (d_slot.read(np.uint32, (rows, K)), d_fill.read(np.uint32, (E,)), d_xp.read(np.uint16, (M, d)))
        for a, b in zip(out["plain"], out["noalloc"]):
            assert np.array_equal(a, b)
        _, rslot, _ = oracle.scatter(idx, off, x16, M)
        assert np.array_equal(out["noalloc"][0], rslot)


def test_noalloc_scatter_leaves_device_memory_as_it_found_it(ctx, oracle):
    """What the name promises: once the first call on the device has looked up the table's
    address, a call changes nothing in the amount of device memory in use (cudaMemGetInfo, read
    through torch)."""
    import torch
    rng = np.random.default_rng(12)
    rows, E, K, d = 2048, 128, 8, 128
    idx, off, x16, M = _case(oracle, rng, rows, E, K, d)
    d_idx, d_off, d_x = ctx.upload(idx), ctx.upload(off), ctx.upload(x16)
    d_fill, d_xp, d_slot = ctx.zeros(E * 4), ctx.zeros(M * d * 2), ctx.alloc(rows * K * 4)
    ctx.scatter_noalloc(d_idx, d_off, d_fill, d_x, d_xp, d_slot, rows, K, d // 8, E)   # first call: address look-up
    ctx.flush()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        d_fill.fill(0)
        ctx.scatter_noalloc(d_idx, d_off, d_fill, d_x, d_xp, d_slot, rows, K, d // 8, E)
    ctx.flush()
    free1, _ = torch.cuda.mem_get_info(0)
    assert free1 == free0, f"device memory in use changed by {free0 - free1} bytes across moe_cuda_scatter_noalloc"


def test_noalloc_scatter_refuses_oversize(mc):
    with mc.Ctx(0) as c:
        c.check()
        b = c.alloc(64)
        c.scatter_noalloc(b, b, b, b, b, b, 1 << 20, 16, 8, 512)  # 262144 blocks x 512 experts > 2 Mi words
        assert c.status() == mc.MOE_ERR_ARG
        assert "fixed table" in c.last_error()
