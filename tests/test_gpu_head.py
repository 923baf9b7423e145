"""The steps either side of the MoE layers: the hyper-connection residual mixer (mda_qwen_res_rec,
src/qwen.c:641-663) and the teacher's head (mda_qwen_head, src/qwen.c:1080-1099) with the
distillation sink behind it -- each kernel against the CPU oracle, then the C host mirror
(r-mda_b200/host/moe_head.c) end to end through ctypes."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _f16(rng, shape, std):
    return (rng.standard_normal(shape).astype(np.float32) * std).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("rows,groups,gsize,op", [(37, 4, 256, 0), (5, 1, 2048, 0), (64, 4, 200, 1), (1, 3, 7, 0)])
def test_norm(ctx, oracle, rows, groups, gsize, op):
    rng = np.random.default_rng(rows + gsize)
    x = rng.standard_normal((rows, groups * gsize)).astype(np.float32) * 3.0
    w = (rng.standard_normal(16 + groups * gsize) * 0.2).astype(np.float32)
    ref = oracle.norm(x, w, groups, gsize, op=op, w_off=16, eps=1e-6, scale=0.37)
    d_y = ctx.alloc(x.nbytes).fill(0x7fc00000)
    ctx.norm(ctx.upload(x), ctx.upload(w), d_y, rows, groups, gsize, op=op, w_off=16, eps=1e-6, scale=0.37)
    ctx.flush()
    got = d_y.read(np.float32, x.shape)
    assert np.all(np.abs(got - ref) <= 2e-6 * np.abs(ref) + 1e-7)   # the sum of squares is reduced in another order


@pytest.mark.parametrize("op", [0, 1, 2])
def test_hc(ctx, oracle, op):
    rng = np.random.default_rng(op)
    rows, d, hc, stride, off = 50, 192, 4, 24, 17
    if op == 0:
        a, b = rng.standard_normal((rows, hc * d)).astype(np.float32), rng.standard_normal((rows, hc * d)).astype(np.float32)
        h0 = np.full((rows, d), np.nan, np.float32)
    elif op == 1:
        a, b = rng.standard_normal((rows, d)).astype(np.float32), rng.standard_normal((rows, stride)).astype(np.float32)
        h0 = rng.standard_normal((rows, hc * d)).astype(np.float32)
    else:
        a, b = rng.standard_normal((rows, hc * d)).astype(np.float32), rng.standard_normal((rows, hc * d)).astype(np.float32)
        h0 = rng.standard_normal((rows, hc * d)).astype(np.float32)
    ref = oracle.hc(a, b, h0.copy(), rows, d, hc, op, stride, off)
    d_h = ctx.upload(h0)
    ctx.hc(ctx.upload(a), ctx.upload(b), d_h, rows, d, hc, op, stride, off)
    ctx.flush()
    got = d_h.read(np.float32, h0.shape)
    assert np.all(np.abs(got - ref) <= 1e-6 * np.abs(ref) + 1e-6)


def test_elem_op1(ctx, oracle):
    rng = np.random.default_rng(3)
    rows, n, stride = 33, 320, 384
    a = rng.standard_normal((rows, stride)).astype(np.float32) * 4.0
    ref = oracle.silu_scaled(a, n, stride, 0, 0.25)
    d_y = ctx.alloc(rows * n * 4)
    ctx.swiglu(ctx.upload(a), d_y, rows, n, stride, 0, 0, op=1, scale=0.25)
    ctx.flush()
    got = d_y.read(np.float32, (rows, n))
    assert np.all(np.abs(got - ref) <= 1e-6 * np.abs(ref) + 1e-7)


@pytest.mark.parametrize("rows,n,k,slot", [(200, 384, 1024, True), (64, 128, 320, False), (256, 1280, 256, True), (1, 128, 8, False)])
def test_dense(ctx, oracle, rows, n, k, slot):
    """mda_qwen_mm: any row count (rows beyond A read as zero, rows beyond C are not written)."""
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, k)).astype(np.float32) * 2.0
    amax = np.zeros(256, np.uint32)
    a16 = oracle.cast(x, amax, 3) if slot else x.astype(np.float16).view(np.uint16)
    w16 = _f16(rng, (n, k), 0.05)
    ref = oracle.dense(a16, w16, amax, 3 if slot else 0xFFFFFFFF)
    canary = np.full((rows + 130, n), 7.0, np.float32)
    d_c = ctx.upload(canary)
    ctx.dense(ctx.upload(a16), ctx.upload(w16), d_c, ctx.upload(amax), rows, n, k, sa=3 if slot else 0xFFFFFFFF)
    ctx.flush()
    got = d_c.read(np.float32, canary.shape)
    assert np.all(got[rows:] == 7.0)
    assert np.all(np.abs(got[:rows] - ref) <= 1e-3 + 2e-2 * np.abs(ref))
    assert np.all(np.abs(got[:rows] - ref) <= 1e-5 * np.abs(ref) + 1e-5 * np.abs(ref).max())   # same products, fp32 sums in another order


class Mix(C.Structure):
    _fields_ = ([("c", C.c_void_p)] + [(n, C.c_uint32) for n in ("d", "hc", "hc_rank", "hc_pad", "rows", "vocab")]
                + [(n, C.c_void_p) for n in ("hn", "a16", "t", "u", "up", "x", "logits", "amax")] + [("n_slots", C.c_uint32)])


class MixW(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("norm", "down", "up")]


class KdSink(C.Structure):
    _fields_ = [("toks", C.c_void_p), ("cont", C.c_void_p), ("outp", C.c_void_p), ("chunks", C.c_uint32)]


SINK = C.CFUNCTYPE(C.c_bool, C.c_void_p, C.POINTER(Mix), C.c_uint32, C.c_uint32)   # moe_head_sink_t


@pytest.fixture(scope="module")
def headlib(pkg):
    pkg.build.build_host()
    L = C.CDLL(pkg.build.HOST_LIB)
    L.moe_mix_open.restype = C.c_bool
    L.moe_mix_open.argtypes = [C.POINTER(Mix), C.c_void_p] + [C.c_uint32] * 6
    L.moe_mix_close.argtypes = [C.POINTER(Mix)]
    L.moe_mix_slots_begin.argtypes = [C.POINTER(Mix)]
    L.moe_mix_res_rec.argtypes = [C.POINTER(Mix), C.c_void_p, C.c_uint32, C.POINTER(MixW)]
    L.moe_head.restype = C.c_bool
    L.moe_head.argtypes = [C.POINTER(Mix), C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(MixW), C.c_void_p, SINK, C.c_void_p]
    L.moe_kd_sink.restype = C.c_bool
    L.moe_kd_sink.argtypes = [C.c_void_p, C.POINTER(Mix), C.c_uint32, C.c_uint32]
    return L


def _mixer_weights(rng, d, hc, rank, pad):
    wn = (rng.standard_normal(hc * d) * 0.1).astype(np.float32)
    wd = np.zeros((pad, hc * d), np.float16)                     # rows beyond rank + hc stay zero (mda_qwen_pad_to)
    wd[:rank + hc] = (rng.standard_normal((rank + hc, hc * d)) * 0.03).astype(np.float16)
    wu = (rng.standard_normal((hc * d, rank)) * 0.05).astype(np.float16)
    return wn, wd.view(np.uint16), wu.view(np.uint16)


def test_mixer_then_layer_injection(ctx, mc, oracle, headlib):
    """mda_qwen_res_rec through the C mirror: the layer input x and the injection scalars t against the oracle."""
    rng = np.random.default_rng(21)
    rows, d, hc, rank, pad = 192, 256, 4, 64, 128
    h = rng.standard_normal((rows, hc, d)).astype(np.float32)
    wn, wd, wu = _mixer_weights(rng, d, hc, rank, pad)
    x_ref, t_ref, _ = oracle.res_rec(h, wn, wd, wu, hc, rank, pad)
    q = Mix()
    assert headlib.moe_mix_open(C.byref(q), ctx.p, d, hc, rank, pad, rows, 0)
    w = MixW(ctx.upload(wn).ptr, ctx.upload(wd).ptr, ctx.upload(wu).ptr)
    headlib.moe_mix_slots_begin(C.byref(q))
    headlib.moe_mix_res_rec(C.byref(q), ctx.upload(h).ptr, rows, C.byref(w))
    ctx.flush()
    x, t = np.empty((rows, d), np.float32), np.empty((rows, pad), np.float32)
    mc.lib().moe_cuda_read(ctx.p, x.ctypes.data, q.x, x.nbytes)
    mc.lib().moe_cuda_read(ctx.p, t.ctypes.data, q.t, t.nbytes)
    ctx.check()
    # The GPU's norm reduces in another order, so a few of its fp32 values round to the neighbouring fp16
    # value in the cast (one fp16 step at |hn| ~ 4 is 4e-3, times a weight of ~0.1): fp16-level tolerances.
    et, ex = np.abs(t - t_ref), np.abs(x - x_ref)
    assert np.all(et <= 2e-3 + 2e-3 * np.abs(t_ref)), et.max()
    assert np.all(ex <= 1e-3 + 2e-3 * np.abs(x_ref)), ex.max()
    assert np.median(et) < 1e-5 and np.median(ex) < 1e-5                 # and nearly all values agree far better
    headlib.moe_mix_close(C.byref(q))


def test_head_in_chunks_with_the_distillation_sink(ctx, mc, oracle, headlib):
    """mda_qwen_head: mixer, cast, vocabulary product in chunks of head_rows, and after every chunk the sink
    (mda_teach_sink's kd_bytes launch).  Logits against the oracle's; the byte distributions against the
    oracle's kd_bytes on the GPU's own logits."""
    from tests.test_oracle import kd_inputs
    rng = np.random.default_rng(22)
    rows, head_rows, d, hc, rank, pad, vocab = 384, 128, 256, 4, 64, 128, 3072
    _, toks, cont = kd_inputs(41, rows, vocab)
    h = rng.standard_normal((rows, hc, d)).astype(np.float32)
    wn, wd, wu = _mixer_weights(rng, d, hc, rank, pad)
    lm = _f16(rng, (vocab, d), 0.2)
    x_ref, _, _ = oracle.res_rec(h, wn, wd, wu, hc, rank, pad)
    q = Mix()
    assert headlib.moe_mix_open(C.byref(q), ctx.p, d, hc, rank, pad, head_rows, vocab)
    w = MixW(ctx.upload(wn).ptr, ctx.upload(wd).ptr, ctx.upload(wu).ptr)
    d_out = ctx.alloc(rows * 16 * 8 * 4).fill(0xdeadbeef)
    sink = KdSink(ctx.upload(toks).ptr, ctx.upload(cont).ptr, d_out.ptr, 0)
    logits_seen = []

    @SINK
    def tap(cx, qq, row0, n):   # the sink the caller passes: keeps the chunk's logits, then runs the library's sink
        lg = np.empty((n, vocab), np.float32)
        mc.lib().moe_cuda_read(ctx.p, lg.ctypes.data, qq.contents.logits, lg.nbytes)
        logits_seen.append((row0, lg))
        return bool(headlib.moe_kd_sink(cx, qq, row0, n))

    ok = headlib.moe_head(C.byref(q), ctx.upload(h).ptr, rows, head_rows, C.byref(w), ctx.upload(lm).ptr, tap, C.byref(sink))
    ctx.check()
    assert ok and sink.chunks == rows // head_rows and [r for r, _ in logits_seen] == [0, 128, 256]
    logits = np.concatenate([lg for _, lg in logits_seen])
    for row0 in range(0, rows, head_rows):   # every chunk has its own scale slots, like the reference (slots_begin per chunk)
        amax = np.zeros(256, np.uint32)
        x16 = oracle.cast(np.ascontiguousarray(x_ref[row0:row0 + head_rows]), amax, 0)
        ref = oracle.dense(x16, lm, amax, 0)
        got = logits[row0:row0 + head_rows]
        assert np.all(np.abs(got - ref) <= 1e-3 + 2e-2 * np.abs(ref))
    outp = d_out.read(np.uint32, (rows, 16, 8))
    ref_out = oracle.kd_bytes(np.ascontiguousarray(logits), toks, cont)
    pg = (outp >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
    pr = (ref_out >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
    assert np.all(np.abs(pg - pr) <= 1.5e-3 * pr + 1e-7)
    assert ((outp & 0xffff) != (ref_out & 0xffff)).mean() < 0.01
    headlib.moe_mix_close(C.byref(q))
