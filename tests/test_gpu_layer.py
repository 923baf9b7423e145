"""Whole-layer parity: libmoe_cuda's fused and unfused layer against the CPU oracle on the
seeded synthetic shapes."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL_OUT, ATOL_OUT = 2e-2, 1e-3


def run_layer(ctx, mc, cfg, inp, flags=0, h0=None):
    d = {}
    d["proj"], d["x16"] = ctx.upload(inp.proj), ctx.upload(inp.x16)
    d["wgu"], d["wdown"] = ctx.upload(inp.wgu), ctx.upload(inp.wdown)
    if cfg.S:
        d["wsgu"], d["wsdown"] = ctx.upload(inp.wsgu), ctx.upload(inp.wsdown)
    T, K, E = inp.x16.shape[0], cfg.K, cfg.E
    M = mc.moe_rows(T, K, E)
    d["h"] = ctx.upload(h0) if h0 is not None else ctx.zeros(T * cfg.d * 4)
    out = {n: ctx.alloc(T * K * 4) for n in ("idx", "slot", "wt")}
    out["count"], out["off"] = ctx.alloc(E * 4), ctx.alloc(E * 4)
    out["tiles"] = ctx.alloc(M // 128 * 4)
    ctx.layer(rows=T, d=cfg.d, experts=E, topk=K, inter=cfg.I, shared=cfg.S, pstride=cfg.pstride, hc=1,
              flags=flags, **d, **out)
    ctx.flush()
    res = {
        "idx": out["idx"].read(np.uint32, (T, K)), "slot": out["slot"].read(np.uint32, (T, K)),
        "wt": out["wt"].read(np.float32, (T, K)), "count": out["count"].read(np.uint32, (E,)),
        "off": out["off"].read(np.uint32, (E,)), "tiles": out["tiles"].read(np.uint32, (M // 128,)),
        "h": d["h"].read(np.float32, (T, 1, cfg.d)),
    }
    return res


def check(res, ref):
    assert np.array_equal(res["idx"], ref.idx)
    assert np.array_equal(res["count"], ref.count)
    assert np.array_equal(res["off"], ref.off)
    assert np.array_equal(res["tiles"], ref.tiles)
    assert np.array_equal(res["slot"], ref.slot)
    assert np.all(np.abs(res["wt"] - ref.wt) <= 1e-5 * np.abs(ref.wt))
    err = np.abs(res["h"] - ref.h)
    bad = err > ATOL_OUT + RTOL_OUT * np.abs(ref.h)
    assert not bad.any(), f"{bad.sum()} outputs outside tolerance, max err {err.max():.3e}, max ref {np.abs(ref.h).max():.3e}"
    return float(err.max())


@pytest.mark.parametrize("flags", [0, 2, 1, 8, 10, 16, 24, 32, 34, 48])  # default (chunked pairs, row gather), fp32 ye, unfused, no pairs, materialised xp, tiled, tiled + xp
def test_c0_tiny(ctx, mc, synth, oracle, flags):
    cfg = synth.CONFIGS["c0"]
    inp = synth.layer_inputs(cfg, 0)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    check(run_layer(ctx, mc, cfg, inp, flags), ref)


def test_c0_accumulates_into_h(ctx, mc, synth, oracle):
    cfg = synth.CONFIGS["c0"]
    inp = synth.layer_inputs(cfg, 1)
    h0 = np.random.default_rng(0).standard_normal((cfg.T, 1, cfg.d)).astype(np.float32)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, h=h0.copy())
    check(run_layer(ctx, mc, cfg, inp, 0, h0), ref)


@pytest.mark.parametrize("name,flags", [("c1", 0), ("c1", 1), ("c1", 8), ("c1", 16), ("c1", 32), ("c1", 48), ("c3", 0), ("c3", 32), ("c3b", 0), ("c3b", 32)])
def test_30b_shape(ctx, mc, synth, oracle, name, flags):
    cfg = synth.CONFIGS[name]
    inp = synth.layer_inputs(cfg, 0)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    check(run_layer(ctx, mc, cfg, inp, flags), ref)


@pytest.mark.parametrize("T", [1, 7, 16, 64, 129, 256])
def test_decode_sweep(ctx, mc, synth, oracle, T):
    """Small-T batches with the 30B-A3B weights shape (shrunk expert count keeps the CPU side quick)."""
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c1"], T=T, E=32, name=f"c3-decode-T{T}")
    inp = synth.layer_inputs(cfg, 0)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    check(run_layer(ctx, mc, cfg, inp, 0), ref)


def test_refused_row_is_skipped_by_the_queued_kernels(ctx, mc, synth, oracle):
    """A row of NaN logits cannot be routed.  The layer call fails with MOE_ERR_ROUTE, and the
    kernels already queued behind the router act on "no expert, weight 0" for that row -- not on
    what the previous call left in idx/wt -- so every other row still gets its exact result."""
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c0"], T=256, name="c0-T256")
    inp = synth.layer_inputs(cfg, 2)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    T, K, E = cfg.T, cfg.K, cfg.E
    proj = inp.proj.copy()
    bad = 37
    proj[bad, :E] = np.nan
    d = dict(x16=ctx.upload(inp.x16), wgu=ctx.upload(inp.wgu), wdown=ctx.upload(inp.wdown))
    d_h = ctx.zeros(T * cfg.d * 4)
    d_idx = ctx.alloc(T * K * 4).fill(3)          # stale values a previous call could have left
    d_slot = ctx.alloc(T * K * 4).fill(5)
    d_wt = ctx.alloc(T * K * 4).fill(0x3f800000)
    ctx.layer(rows=T, d=cfg.d, experts=E, topk=K, inter=cfg.I, shared=0, pstride=cfg.pstride, hc=1, proj=ctx.upload(proj),
              h=d_h, idx=d_idx, slot=d_slot, wt=d_wt, **d)
    with pytest.raises(mc.MoeCudaError) as e:
        ctx.flush()
    assert e.value.code == mc.MOE_ERR_ROUTE
    out = {}
    with mc.Ctx(0) as reader:   # the failed context refuses every call; a second one reads its buffers
        for name, buf, dt, shape in (("idx", d_idx, np.uint32, (T, K)), ("slot", d_slot, np.uint32, (T, K)),
                                     ("wt", d_wt, np.float32, (T, K)), ("h", d_h, np.float32, (T, cfg.d))):
            a = np.empty(shape, dt)
            mc.lib().moe_cuda_read(reader.p, a.ctypes.data, buf.ptr, a.nbytes)
            reader.check()
            out[name] = a
    assert np.all(out["idx"][bad] == 0xffffffff) and np.all(out["slot"][bad] == 0xffffffff) and np.all(out["wt"][bad] == 0)
    assert np.all(out["h"][bad] == 0)
    # the other rows: same experts; their outputs are within tolerance of a reference computed without the bad row's pairs
    keep = np.arange(T) != bad
    assert np.array_equal(out["idx"][keep], ref.idx[keep])
    err = np.abs(out["h"][keep] - ref.h[keep, 0])
    assert np.all(err <= ATOL_OUT + RTOL_OUT * np.abs(ref.h[keep, 0]))


def test_shared_expert_small(ctx, mc, synth, oracle):
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c2"], T=300, E=64, name="c2-small")
    inp = synth.layer_inputs(cfg, 0)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
    check(run_layer(ctx, mc, cfg, inp, 0), ref)
    check(run_layer(ctx, mc, cfg, inp, 1), ref)


def test_upstream_projection_on_gpu_then_layer(ctx, mc, synth, oracle):
    """The product just upstream of the path (src/qwen.c:845: router logits, shared-gate logit and the
    padding columns in one fp16 product with fp32 output) runs on the same grouped kernel with a
    single "expert"; the layer then routes on those GPU logits and the oracle re-routes on the
    same downloaded values, so both sides see bit-identical router inputs."""
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c1"], T=640, E=128, name="c1-T640")
    inp = synth.layer_inputs(cfg, 4)
    wr, wsg = synth.router_weights(cfg, 4)
    T, d, pcols = cfg.T, cfg.d, cfg.pstride                      # E + 128 columns, a multiple of 128
    wd = np.zeros((1, pcols, d), np.float16)                     # packed like mda_qwen_put_moe (src/qwen.c:441-452)
    wd[0, :cfg.E] = wr.astype(np.float16)
    wd[0, cfg.E] = wsg.astype(np.float16)
    wd16 = wd.view(np.uint16)
    tiles0 = np.zeros(T // 128, np.uint32)
    ref_proj = oracle.mm(inp.x16, wd16, tiles0, pcols, d)
    d_x, d_proj = ctx.upload(inp.x16), ctx.alloc(T * pcols * 4)
    ctx.mm(d_x, ctx.upload(wd16), d_proj, None, ctx.upload(tiles0), T, pcols, d, experts_in_B=1)
    ctx.flush()
    proj = d_proj.read(np.float32, (T, pcols))
    assert np.allclose(proj, ref_proj, rtol=1e-3, atol=1e-4)
    assert np.abs(proj - inp.proj).max() < 0.05                  # fp16 router weights move the logits only slightly
    ref = oracle.layer(proj, inp.x16, inp.wgu, inp.wdown, cfg.K)  # the oracle routes on the GPU's logits
    d_h = ctx.zeros(T * d * 4)
    d_idx, d_slot = ctx.alloc(T * cfg.K * 4), ctx.alloc(T * cfg.K * 4)
    ctx.layer(rows=T, d=d, experts=cfg.E, topk=cfg.K, inter=cfg.I, shared=0, pstride=pcols, hc=1, proj=d_proj, x16=d_x,
              wgu=ctx.upload(inp.wgu), wdown=ctx.upload(inp.wdown), h=d_h, idx=d_idx, slot=d_slot)
    ctx.flush()
    assert np.array_equal(d_idx.read(np.uint32, (T, cfg.K)), ref.idx)
    assert np.array_equal(d_slot.read(np.uint32, (T, cfg.K)), ref.slot)
    h = d_h.read(np.float32, (T, 1, d))
    assert np.all(np.abs(h - ref.h) <= ATOL_OUT + RTOL_OUT * np.abs(ref.h))
