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


# 0 fused (row gather), 2 fp32 expert outputs, 1 reference sequence, 16 materialised xp, 4 / 12 chunked products
@pytest.mark.parametrize("flags", [0, 2, 1, 16, 4, 12])
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


@pytest.mark.parametrize("name,flags", [("c1", 0), ("c1", 1), ("c1", 16), ("c1", 4), ("c3", 0), ("c3", 16), ("c3b", 0)])
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


def test_shared_expert_small(ctx, mc, synth, oracle):
    import dataclasses
    cfg = dataclasses.replace(synth.CONFIGS["c2"], T=300, E=64, name="c2-small")
    inp = synth.layer_inputs(cfg, 0)
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
    check(run_layer(ctx, mc, cfg, inp, 0), ref)
    check(run_layer(ctx, mc, cfg, inp, 1), ref)
