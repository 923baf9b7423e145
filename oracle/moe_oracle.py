"""ctypes front end of the CPU oracle (libmoe_ref.so).

TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the benchmark's CPU
baseline legs import this module; nothing in the product path does.

PARITY UNPINNED: the reference (GLSL over Vulkan) holds no golden vectors for
the MoE path and cannot run here; see oracle/moe_ref.h.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmoe_ref.so")

NO_SLOT = 0xFFFFFFFF
TILE = 128  # MDA_QWEN_TILE, src/qwen.h:14


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the library is missing or stale."""
    src = [os.path.join(_HERE, f) for f in ("moe_ref.c", "moe_ref.h", "Makefile")]
    stale = (not os.path.exists(_SO)) or any(
        os.path.getmtime(s) > os.path.getmtime(_SO) for s in src
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libmoe_ref.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.moe_ref_threads.restype = C.c_int
        _lib.moe_ref_route.restype = C.c_int
        _lib.moe_ref_layer.restype = C.c_int
        _lib.moe_ref_slot_scale.restype = C.c_float
        _lib.moe_ref_h2f.restype = C.c_float
        _lib.moe_ref_h2f.argtypes = [C.c_uint16]
        _lib.moe_ref_f2h.restype = C.c_uint16
        _lib.moe_ref_f2h.argtypes = [C.c_float]
    return _lib


def threads() -> int:
    return int(lib().moe_ref_threads())


def use_all_cores() -> int:
    """Give the oracle every core this process may run on, whatever OMP_NUM_THREADS says
    (torch.distributed.run sets it to 1 for its children).  Returns the thread count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().moe_ref_set_threads(C.c_int(n))
    return threads()


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _chk(a, dtype, name):
    assert a.dtype == dtype and a.flags["C_CONTIGUOUS"], f"{name}: want contiguous {dtype}, got {a.dtype}"
    return a


def moe_rows(rows: int, topk: int, experts: int, tile: int = TILE) -> int:
    """src/qwen.c:68-70 mda_qwen_moe_rows."""
    n = rows * topk + experts * (tile - 1)
    return (n + tile - 1) // tile * tile


def route(proj, experts, topk):
    """shader/moe_route.comp.  proj [rows, stride] fp32 -> idx u32, wt f32, count u32."""
    _chk(proj, np.float32, "proj")
    rows, stride = proj.shape
    idx = np.empty((rows, topk), np.uint32)
    wt = np.empty((rows, topk), np.float32)
    count = np.zeros(experts, np.uint32)
    rc = lib().moe_ref_route(_p(proj), C.c_uint32(rows), C.c_uint32(experts), C.c_uint32(topk),
                             C.c_uint32(stride), _p(idx), _p(wt), _p(count))
    if rc != 0:
        raise ValueError(f"moe_ref_route refused: {rc}")
    return idx, wt, count


def scan(count, tile=TILE, ntiles=None):
    """shader/moe_scan.comp.  Returns off u32[E], tiles u32[ntiles] (pre-filled with ~0)."""
    _chk(count, np.uint32, "count")
    E = count.shape[0]
    padded = int(((count.astype(np.int64) + tile - 1) // tile).sum())
    if ntiles is None:
        ntiles = padded
    assert ntiles >= padded
    off = np.zeros(E, np.uint32)
    tiles = np.full(ntiles, 0xFFFFFFFF, np.uint32)
    lib().moe_ref_scan(_p(count), C.c_uint32(E), C.c_uint32(tile), _p(off), _p(tiles))
    return off, tiles


def scatter(idx, off, x16, mrows):
    """shader/moe_scatter.comp, sequential.  x16 uint16 view of fp16 [rows, d]."""
    _chk(idx, np.uint32, "idx"); _chk(off, np.uint32, "off"); _chk(x16, np.uint16, "x16")
    rows, topk = idx.shape
    d = x16.shape[1]
    assert d % 8 == 0
    fill = np.zeros(off.shape[0], np.uint32)
    xp = np.zeros((mrows, d), np.uint16)  # src/qwen.c:798 zero fill
    slot = np.empty((rows, topk), np.uint32)
    lib().moe_ref_scatter(_p(idx), _p(off), _p(fill), _p(x16), _p(xp), _p(slot),
                          C.c_uint32(rows), C.c_uint32(topk), C.c_uint32(d // 8))
    return xp, slot, fill


def mm(A, B, tiles, n, k, amax=None, sa=NO_SLOT, sb=NO_SLOT, row_mask=None, out=None):
    """shader/matmul_f16_moe.comp.  A u16 [m,k], B u16 [E,n,k] -> C f32 [m,n]."""
    _chk(A, np.uint16, "A"); _chk(B, np.uint16, "B"); _chk(tiles, np.uint32, "tiles")
    m = A.shape[0]
    assert m % 128 == 0 and tiles.shape[0] >= m // 128
    Cm = np.zeros((m, n), np.float32) if out is None else out
    if amax is None:
        amax = np.zeros(4, np.uint32)
    lib().moe_ref_mm(_p(A), _p(B), _p(Cm), _p(amax), _p(tiles), C.c_uint32(m), C.c_uint32(n),
                     C.c_uint32(k), C.c_uint32(sa), C.c_uint32(sb), _p(row_mask))
    return Cm


def swiglu(a, n, astride, ao, bo):
    _chk(a, np.float32, "a")
    rows = a.size // astride
    y = np.empty((rows, n), np.float32)
    lib().moe_ref_swiglu(_p(a), _p(y), C.c_uint32(rows), C.c_uint32(n), C.c_uint32(astride),
                         C.c_uint32(ao), C.c_uint32(bo))
    return y


def silu_scaled(a, n, astride, ao, scale):
    """shader/qwen_elem.comp op 1: y = silu(a[:, ao:ao+n] * scale)."""
    _chk(a, np.float32, "a")
    rows = a.size // astride
    y = np.empty((rows, n), np.float32)
    lib().moe_ref_silu_scaled(_p(a), _p(y), C.c_uint32(rows), C.c_uint32(n), C.c_uint32(astride), C.c_uint32(ao),
                              C.c_float(scale))
    return y


def norm(x, w, groups, gsize, op=0, w_off=0, eps=1e-6, scale=1.0):
    """shader/qwen_norm.comp ops 0 / 1 on x [rows, groups*gsize] with mda_qwen_norm_pc's strides."""
    _chk(x, np.float32, "x")
    rows = x.size // (groups * gsize)
    y = np.empty_like(x)
    lib().moe_ref_norm(_p(x), _p(w), _p(y), C.c_uint32(rows), C.c_uint32(groups), C.c_uint32(gsize), C.c_uint32(w_off),
                       C.c_uint32(op), C.c_float(eps), C.c_float(scale))
    return y


def hc(a, b, h, rows, d, n_hc, op, inj_stride=0, inj_off=0):
    """shader/qwen_hc.comp; h is written (op 0) or accumulated into (ops 1, 2) in place."""
    _chk(a, np.float32, "a"); _chk(b, np.float32, "b"); _chk(h, np.float32, "h")
    lib().moe_ref_hc(_p(a), _p(b), _p(h), C.c_uint32(rows), C.c_uint32(d), C.c_uint32(n_hc), C.c_uint32(op),
                     C.c_uint32(inj_stride), C.c_uint32(inj_off))
    return h


def dense(A16, W16, amax=None, sa=NO_SLOT):
    """mda_qwen_mm (src/qwen.c:541-570): C[rows, n] = A16[rows, k] * W16[n, k]^T / scale(sa), fp32 accumulate --
    the grouped product's arithmetic over a dense tile schedule."""
    rows, k = A16.shape
    n = W16.shape[0]
    m = (rows + 127) // 128 * 128
    Ap = np.zeros((m, k), np.uint16)
    Ap[:rows] = A16
    out = mm(Ap, np.ascontiguousarray(W16.reshape(1, n, k)), np.zeros(m // 128, np.uint32), n, k, amax=amax, sa=sa)
    return out[:rows]


def cast(x, amax, slot):
    """mda_qwen_cast (src/qwen.c:517-539): absmax into the slot, then the fp16 cast with the slot's power-of-two scale."""
    absmax(x, amax, slot)
    return cast_f16(x, amax, slot)


def res_rec(h, wnorm, wdown16, wup16, n_hc, hc_rank, hc_pad, eps=1e-6):
    """mda_qwen_res_rec (src/qwen.c:641-663): the hyper-connection mixer.  h fp32 [rows, n_hc, d]; wnorm fp32
    [n_hc * d] (norm weight rows of the streams); wdown16 fp16 [hc_pad, n_hc*d]; wup16 fp16 [n_hc*d, hc_rank].
    Returns x [rows, d] (the layer's input), t [rows, hc_pad] (columns hc_rank.. are the injection scalars), hn."""
    rows, _, d = h.shape
    d4 = n_hc * d
    amax = np.zeros(256, np.uint32)
    hn = norm(np.ascontiguousarray(h.reshape(rows, d4)), wnorm, n_hc, d, op=0, eps=eps)      # :645-647
    hn16 = cast(hn, amax, 0)                                                                 # :648
    t = dense(hn16, wdown16, amax, 0)                                                        # :649
    u = silu_scaled(np.ascontiguousarray(t), hc_rank, hc_pad, 0, 1.0 / n_hc)                 # :650-659
    u16 = cast(u, amax, 1)                                                                   # :660
    up = dense(u16, wup16, amax, 1)                                                          # :661
    x = np.empty((rows, d), np.float32)
    hc(np.ascontiguousarray(up), hn, x, rows, d, n_hc, 0)                                    # :662
    return x, t, hn


def absmax(x, amax, slot):
    _chk(x, np.float32, "x"); _chk(amax, np.uint32, "amax")
    lib().moe_ref_absmax(_p(x), C.c_uint64(x.size), _p(amax), C.c_uint32(slot))
    return amax


def cast_f16(src, amax, slot):
    _chk(src, np.float32, "src")
    dst = np.empty(src.shape, np.uint16)
    lib().moe_ref_cast_f16(_p(src), _p(dst), C.c_uint64(src.size), _p(amax), C.c_uint32(slot))
    return dst


def slot_scale(amax, slot):
    return float(lib().moe_ref_slot_scale(_p(amax), C.c_uint32(slot)))


def combine(wt, slot, y, proj, sh, inj, h, sg_off, inj_off=0, hc=1):
    """shader/moe_combine.comp; h [rows, hc, d] is accumulated into in place."""
    _chk(wt, np.float32, "wt"); _chk(slot, np.uint32, "slot"); _chk(y, np.float32, "y")
    _chk(h, np.float32, "h")
    rows, topk = wt.shape
    d = y.shape[1]
    pstride = proj.shape[1] if proj is not None else 0
    inj_stride = inj.shape[1] if inj is not None else 0
    lib().moe_ref_combine(_p(wt), _p(slot), _p(y), _p(proj), _p(sh), _p(inj), _p(h),
                          C.c_uint32(rows), C.c_uint32(d), C.c_uint32(topk), C.c_uint32(pstride),
                          C.c_uint32(sg_off), C.c_uint32(inj_stride), C.c_uint32(inj_off),
                          C.c_uint32(hc))
    return h


def residual_rmsnorm(x16, delta, eps=1e-6):
    _chk(x16, np.uint16, "x16"); _chk(delta, np.float32, "delta")
    rows, d = x16.shape
    y = np.empty((rows, d), np.uint16)
    lib().moe_ref_residual_rmsnorm(_p(x16), _p(delta), _p(y), C.c_uint32(rows), C.c_uint32(d),
                                   C.c_float(eps))
    return y


def bf16_to_f16(w):
    """shader/qwen_bf16.comp on a copy: uint32 words of two bf16 -> two fp16."""
    _chk(w, np.uint32, "w")
    out = w.copy()
    lib().moe_ref_bf16_to_f16(_p(out), C.c_uint64(out.size))
    return out


def kd_bytes(logits, toks, cont):
    """shader/kd_bytes.comp.  logits f32 [rows, vocab], toks u32 [vocab, 5], cont u32 [rows, 5] -> u32 [rows, 16, 8]."""
    _chk(logits, np.float32, "logits"); _chk(toks, np.uint32, "toks"); _chk(cont, np.uint32, "cont")
    rows, vocab = logits.shape
    assert toks.shape == (vocab, 5) and cont.shape == (rows, 5)
    out = np.empty((rows, 16, 8), np.uint32)
    lib().moe_ref_kd_bytes(_p(logits), _p(toks), _p(cont), _p(out), C.c_uint32(rows), C.c_uint32(vocab))
    return out


class _Layer(C.Structure):
    _fields_ = [
        ("rows", C.c_uint32), ("d", C.c_uint32), ("experts", C.c_uint32), ("topk", C.c_uint32),
        ("inter", C.c_uint32), ("shared", C.c_uint32), ("pstride", C.c_uint32), ("hc", C.c_uint32),
        ("tile", C.c_uint32),
        ("proj", C.c_void_p), ("x16", C.c_void_p), ("wgu", C.c_void_p), ("wdown", C.c_void_p),
        ("wsgu", C.c_void_p), ("wsdown", C.c_void_p), ("inj", C.c_void_p), ("h", C.c_void_p),
        ("idx", C.c_void_p), ("slot", C.c_void_p), ("count", C.c_void_p), ("off", C.c_void_p),
        ("tiles", C.c_void_p), ("wt", C.c_void_p),
        ("mrows", C.c_uint32),
        ("xp", C.c_void_p), ("ye", C.c_void_p), ("hp16", C.c_void_p), ("amax", C.c_void_p),
        ("row_mask", C.c_void_p),
    ]


@dataclass
class LayerResult:
    idx: np.ndarray
    wt: np.ndarray
    count: np.ndarray
    off: np.ndarray
    tiles: np.ndarray
    slot: np.ndarray
    xp: np.ndarray
    ye: np.ndarray
    hp16: np.ndarray
    amax: np.ndarray
    h: np.ndarray
    mrows: int
    extra: dict = field(default_factory=dict)


def layer(proj, x16, wgu, wdown, topk, wsgu=None, wsdown=None, h=None, row_mask=None, hc=1,
          inj=None) -> LayerResult:
    """One MoE layer in the order of src/qwen.c:788-907.

    proj f32 [rows, pstride] (logits in columns < E; shared gate logit at column E),
    x16 u16 [rows, d], wgu u16 [E, 2I, d], wdown u16 [E, d, I].  h (f32 [rows, hc, d]) is the
    residual the layer accumulates into; zeros when omitted.
    """
    _chk(proj, np.float32, "proj"); _chk(x16, np.uint16, "x16")
    _chk(wgu, np.uint16, "wgu"); _chk(wdown, np.uint16, "wdown")
    rows, d = x16.shape
    E, twoI, _ = wgu.shape
    I = twoI // 2
    S = 0 if wsgu is None else wsgu.shape[0] // 2
    M = moe_rows(rows, topk, E)
    if h is None:
        h = np.zeros((rows, hc, d), np.float32)
    res = LayerResult(
        idx=np.empty((rows, topk), np.uint32), wt=np.empty((rows, topk), np.float32),
        count=np.zeros(E, np.uint32), off=np.zeros(E, np.uint32),
        tiles=np.empty(M // TILE, np.uint32), slot=np.empty((rows, topk), np.uint32),
        xp=np.empty((M, d), np.uint16), ye=np.empty((M, d), np.float32),
        hp16=np.empty((M, I), np.uint16), amax=np.zeros(4, np.uint32), h=h, mrows=M)
    L = _Layer(rows=rows, d=d, experts=E, topk=topk, inter=I, shared=S, pstride=proj.shape[1],
               hc=hc, tile=TILE, proj=_p(proj), x16=_p(x16), wgu=_p(wgu), wdown=_p(wdown),
               wsgu=_p(wsgu), wsdown=_p(wsdown), inj=_p(inj), h=_p(h), idx=_p(res.idx),
               slot=_p(res.slot), count=_p(res.count), off=_p(res.off), tiles=_p(res.tiles),
               wt=_p(res.wt), mrows=M, xp=_p(res.xp), ye=_p(res.ye), hp16=_p(res.hp16),
               amax=_p(res.amax), row_mask=_p(row_mask))
    rc = lib().moe_ref_layer(C.byref(L))
    if rc != 0:
        raise ValueError(f"moe_ref_layer refused: {rc}")
    return res
