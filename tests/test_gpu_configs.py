"""The named benchmark configurations at full size: the 80B-A3B shape with its shared expert, and
the stacked configuration (layer -> residual -> RMSNorm -> next layer) with per-layer weights."""
import dataclasses

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL_OUT, ATOL_OUT = 2e-2, 1e-3


def test_c1_token_order_and_residual_properties(ctx, mc, synth):
    """Full-size 30B-A3B shape, no oracle involved: a token's output does not depend on where the token
    sits in the batch (bit-exact under a permutation of the tokens), and the layer adds its result to
    whatever the residual stream h held (one rounded fp32 addition per element)."""
    cfg = synth.CONFIGS["c1"]
    inp = synth.layer_inputs(cfg, 3)
    T, K, E, d = cfg.T, cfg.K, cfg.E, cfg.d
    wgu, wdown = ctx.upload(inp.wgu), ctx.upload(inp.wdown)

    def run(proj, x16, h0=None):
        h = ctx.upload(h0) if h0 is not None else ctx.zeros(T * d * 4)
        ctx.layer(rows=T, d=d, experts=E, topk=K, inter=cfg.I, shared=0, pstride=cfg.pstride, hc=1,
                  proj=ctx.upload(proj), x16=ctx.upload(x16), wgu=wgu, wdown=wdown, h=h)
        ctx.flush()
        return h.read(np.float32, (T, d))

    base = run(inp.proj, inp.x16)
    assert np.isfinite(base).all() and np.abs(base).max() > 0
    perm = np.random.default_rng(11).permutation(T)
    moved = run(np.ascontiguousarray(inp.proj[perm]), np.ascontiguousarray(inp.x16[perm]))
    assert np.array_equal(moved, base[perm])
    h0 = np.random.default_rng(12).standard_normal((T, d)).astype(np.float32)
    assert np.array_equal(run(inp.proj, inp.x16, h0), h0 + base)


def test_c2_80b_shape_full_size(ctx, mc, synth, oracle):
    """T=16384, d=2048, E=512, top-10, I=512, shared S=512 against the full CPU oracle, plus the
    size-independent properties of the path."""
    cfg = synth.CONFIGS["c2"]
    inp = synth.layer_inputs(cfg, 0)
    T, K, E, d = cfg.T, cfg.K, cfg.E, cfg.d
    M = mc.moe_rows(T, K, E)
    bufs = dict(proj=ctx.upload(inp.proj), x16=ctx.upload(inp.x16), wgu=ctx.upload(inp.wgu), wdown=ctx.upload(inp.wdown),
                wsgu=ctx.upload(inp.wsgu), wsdown=ctx.upload(inp.wsdown), h=ctx.zeros(T * d * 4))
    out = {n: ctx.alloc(T * K * 4) for n in ("idx", "slot", "wt")}
    out["count"], out["off"], out["tiles"] = ctx.alloc(E * 4), ctx.alloc(E * 4), ctx.alloc(M // 128 * 4)
    ctx.layer(rows=T, d=d, experts=E, topk=K, inter=cfg.I, shared=cfg.S, pstride=cfg.pstride, hc=1, **bufs, **out)
    ctx.flush()
    idx, slot = out["idx"].read(np.uint32, (T, K)), out["slot"].read(np.uint32, (T, K))
    wt, count = out["wt"].read(np.float32, (T, K)), out["count"].read(np.uint32, (E,))
    off, tiles = out["off"].read(np.uint32, (E,)), out["tiles"].read(np.uint32, (M // 128,))
    h = bufs["h"].read(np.float32, (T, d))
    # properties that hold at any size
    assert count.sum() == T * K and np.allclose(wt.sum(1), 1.0, atol=1e-5)
    assert len(np.unique(slot)) == T * K                      # the permutation is injective
    assert np.array_equal(tiles[slot // 128], idx)            # every row sits in a tile of its expert
    assert np.all(off % 128 == 0) and np.isfinite(h).all()
    ref = oracle.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, K, inp.wsgu, inp.wsdown)
    assert np.array_equal(idx, ref.idx) and np.array_equal(count, ref.count)
    assert np.array_equal(off, ref.off) and np.array_equal(tiles, ref.tiles) and np.array_equal(slot, ref.slot)
    assert np.all(np.abs(wt - ref.wt) <= 1e-5 * np.abs(ref.wt))
    err = np.abs(h - ref.h[:, 0])
    assert np.all(err <= ATOL_OUT + RTOL_OUT * np.abs(ref.h[:, 0])), err.max()


def _stack(ctx, mc, synth, oracle, cfg, layers, seed0=0):
    """x <- fp16(RMSNorm(x + moe(x))) per layer, eps 1e-6.  Every layer is checked with the same
    inputs on both sides: the oracle re-routes on the activations the GPU produced."""
    T, K, E, d, I = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I
    x16 = synth.activations(cfg, seed0)
    d_x, d_y = ctx.upload(x16), ctx.alloc(T * d * 2)
    worst = 0.0
    for layer in range(layers):
        wr, wsg = synth.router_weights(cfg, seed0 + layer)
        wgu, wdown = synth.expert_weights(cfg, seed0 + layer)
        proj = synth.projection(cfg, x16, wr, wsg, synth.zipf_bias(cfg, seed0 + layer))
        d_wgu, d_wdown, d_proj = ctx.upload(wgu), ctx.upload(wdown), ctx.upload(proj)
        ctx.layer(rows=T, d=d, experts=E, topk=K, inter=I, shared=0, pstride=cfg.pstride, hc=1, proj=d_proj, x16=d_x,
                  wgu=d_wgu, wdown=d_wdown, y16=d_y, eps=1e-6)
        ctx.flush()
        y_gpu = d_y.read(np.uint16, (T, d))
        ref = oracle.layer(proj, x16, wgu, wdown, K)
        y_ref = oracle.residual_rmsnorm(x16, np.ascontiguousarray(ref.h[:, 0]))
        a, b = y_gpu.view(np.float16).astype(np.float32), y_ref.view(np.float16).astype(np.float32)
        err = np.abs(a - b)
        assert np.all(err <= 2e-3 + RTOL_OUT * np.abs(b)), (layer, err.max())   # fp16 output: one ulp at |y|~4 is 2e-3
        assert abs(float(np.sqrt((a * a).mean(1)).mean()) - 1.0) < 1e-2          # rows leave the norm with unit RMS
        worst = max(worst, float(err.max()))
        x16 = y_gpu                                   # next layer runs on what the GPU produced
        d_x, d_y = d_y, d_x
        for b_ in (d_wgu, d_wdown, d_proj):
            b_.free()
    return worst


def test_c4_stack_three_layers_full_shape(ctx, mc, synth, oracle):
    _stack(ctx, mc, synth, oracle, synth.CONFIGS["c1"], layers=3)


def test_c4_stack_48_layers_small_shape(ctx, mc, synth, oracle):
    cfg = dataclasses.replace(synth.CONFIGS["c1"], T=384, d=512, E=16, K=4, I=256, name="c4-small")
    _stack(ctx, mc, synth, oracle, cfg, layers=48)
