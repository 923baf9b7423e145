"""ctypes binding of libmoe_cuda's C ABI (include/moe_cuda.h), for tests and the
benchmark driver.  There is no fallback: if the library is missing, or no
sm_100 device is usable, calls raise."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

NO_SLOT = 0xFFFFFFFF
TILE = 128
MOE_OK, MOE_ERR_CUDA, MOE_ERR_ARG, MOE_ERR_NOMEM, MOE_ERR_ROUTE, MOE_ERR_TIMEOUT, MOE_ERR_COMM, MOE_ERR_UNSUPPORTED = range(8)
LAYER_UNFUSED, LAYER_YE_F32, LAYER_CHUNKED, LAYER_NO_PAIR, LAYER_MATERIALIZE_XP, LAYER_TILED = 1, 2, 4, 8, 16, 32
PROF_STAGES = ("route", "scan", "scatter", "gate_up", "down", "shared", "combine")


class PcRoute(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("experts", C.c_uint32), ("topk", C.c_uint32), ("stride", C.c_uint32)]


class PcScan(C.Structure):
    _fields_ = [("experts", C.c_uint32), ("tile", C.c_uint32)]


class PcScatter(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("topk", C.c_uint32), ("d8", C.c_uint32)]


class PcMm(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32), ("sa", C.c_uint32), ("sb", C.c_uint32)]


class PcCombine(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("rows", "d", "topk", "pstride", "sg_off", "inj_stride", "inj_off", "hc")]


class PcElem(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("rows", "n", "astride", "ao", "bo", "op")] + [("scale", C.c_float)]


class PcSlot(C.Structure):  # mda_pc_absmax_t and mda_pc_cast_t share this layout
    _fields_ = [("n", C.c_uint32), ("slot", C.c_uint32)]


class PcBf16(C.Structure):
    _fields_ = [("n", C.c_uint32)]


class PcNorm(C.Structure):
    _fields_ = ([(n, C.c_uint32) for n in ("rows", "groups", "gsize", "in_stride", "in_off", "in_gstride", "out_stride",
                                             "out_off", "out_gstride", "w_off", "wstride", "op", "rot", "seqlen", "z_stride",
                                             "z_off", "z_gstride")]
                + [(n, C.c_float) for n in ("eps", "scale", "theta")])


class PcHc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("rows", "d", "hc", "op", "inj_stride", "inj_off")]


class PcDense(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("rows", "n", "k", "sa")]


class PcKd(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("vocab", C.c_uint32)]


class Layer(C.Structure):
    _fields_ = (
        [(n, C.c_uint32) for n in ("rows", "d", "experts", "topk", "inter", "shared", "pstride", "hc",
                                   "inj_stride", "inj_off")]
        + [(n, C.c_void_p) for n in ("proj", "x16", "wgu", "wdown", "wsgu", "wsdown", "inj", "h",
                                     "idx", "slot", "count", "off", "tiles", "wt", "y16")]
        + [("eps", C.c_float), ("flags", C.c_uint32)]
    )


class EpCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("experts", "topk", "d", "inter", "max_rows", "micro_batches", "transfer")]


_lib = None


def lib_path() -> str:
    return _build.LIB


def lib() -> C.CDLL:
    """Load the CUDA library; build it first if its sources are newer."""
    global _lib
    if _lib is None:
        if not os.path.exists(_build.LIB):
            _build.build_cuda()
        if not os.path.exists(_build.LIB):
            raise RuntimeError("libmoe_cuda.so is missing and could not be built; there is no CPU fallback")
        L = C.CDLL(_build.LIB)
        vp, u32, sz = C.c_void_p, C.c_uint32, C.c_size_t
        L.moe_cuda_create.restype = vp
        L.moe_cuda_create.argtypes = [C.c_int, vp]
        L.moe_cuda_destroy.argtypes = [vp]
        L.moe_cuda_status.restype = C.c_int
        L.moe_cuda_status.argtypes = [vp]
        L.moe_cuda_last_error.restype = C.c_char_p
        L.moe_cuda_last_error.argtypes = [vp]
        L.moe_cuda_stream.restype = vp
        L.moe_cuda_stream.argtypes = [vp]
        L.moe_cuda_fail_alloc_after.argtypes = [vp, C.c_int]
        L.moe_cuda_set_wait_ns.argtypes = [vp, C.c_uint64]
        L.moe_cuda_wait_selftest.argtypes = [vp]
        L.moe_cuda_alloc.restype = vp
        L.moe_cuda_alloc.argtypes = [vp, sz]
        L.moe_cuda_alloc_pinned.restype = vp
        L.moe_cuda_alloc_pinned.argtypes = [vp, sz]
        L.moe_cuda_free.argtypes = [vp, vp]
        L.moe_cuda_free_pinned.argtypes = [vp, vp]
        L.moe_cuda_fill.argtypes = [vp, vp, sz, u32]
        L.moe_cuda_copy.argtypes = [vp, vp, vp, sz]
        L.moe_cuda_write.argtypes = [vp, vp, vp, sz]
        L.moe_cuda_read.argtypes = [vp, vp, vp, sz]
        L.moe_cuda_read_async.argtypes = [vp, vp, vp, sz]
        L.moe_cuda_flush.argtypes = [vp]
        L.moe_cuda_route.argtypes = [vp, vp, vp, vp, vp, PcRoute]
        L.moe_cuda_scan.argtypes = [vp, vp, vp, vp, PcScan]
        L.moe_cuda_scatter.argtypes = [vp, vp, vp, vp, vp, vp, vp, PcScatter]
        L.moe_cuda_mm.argtypes = [vp, vp, vp, vp, vp, vp, PcMm, u32]
        L.moe_cuda_scatter_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, PcScatter, u32]
        L.moe_cuda_combine.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, PcCombine]
        L.moe_cuda_swiglu.argtypes = [vp, vp, vp, PcElem]
        L.moe_cuda_absmax.argtypes = [vp, vp, vp, PcSlot]
        L.moe_cuda_cast_f16.argtypes = [vp, vp, vp, vp, PcSlot]
        L.moe_cuda_bf16_to_f16.argtypes = [vp, vp, PcBf16]
        L.moe_cuda_kd_bytes.argtypes = [vp, vp, vp, vp, vp, PcKd]
        L.moe_cuda_norm.argtypes = [vp, vp, vp, vp, vp, PcNorm]
        L.moe_cuda_hc.argtypes = [vp, vp, vp, vp, PcHc]
        L.moe_cuda_dense.argtypes = [vp, vp, vp, vp, vp, PcDense]
        L.moe_cuda_moe_rows.restype = u32
        L.moe_cuda_moe_rows.argtypes = [u32, u32, u32]
        L.moe_cuda_layer.argtypes = [vp, C.POINTER(Layer)]
        L.moe_cuda_ep_unique_id.restype = C.c_int
        L.moe_cuda_ep_unique_id.argtypes = [vp]
        L.moe_cuda_ep_rows.restype = u32
        L.moe_cuda_ep_rows.argtypes = [u32, u32, u32, u32]
        L.moe_cuda_ep_init.argtypes = [vp, vp, C.c_int, C.c_int, C.POINTER(EpCfg)]
        L.moe_cuda_ep_layer.argtypes = [vp, C.POINTER(Layer)]
        L.moe_cuda_prof.argtypes = [vp, C.c_int]
        L.moe_cuda_prof_read.argtypes = [vp, C.POINTER(C.c_float)]
        L.moe_cuda_launches.restype = C.c_uint64
        L.moe_cuda_launches.argtypes = [vp]
        _lib = L
    return _lib


class MoeCudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"moe_cuda status {code}: {msg}")
        self.code = code


class DevBuf:
    """A device allocation owned by a context (mda_vkc_buf_t in the reference)."""

    def __init__(self, ctx: "Ctx", nbytes: int):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        self.ptr = lib().moe_cuda_alloc(ctx.p, self.nbytes)
        ctx.check()

    def write(self, a: np.ndarray) -> "DevBuf":
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        lib().moe_cuda_write(self.ctx.p, self.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes)
        self.ctx.flush()
        return self

    def read(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        lib().moe_cuda_read(self.ctx.p, out.ctypes.data_as(C.c_void_p), self.ptr, out.nbytes)
        self.ctx.check()
        return out

    def fill(self, word: int) -> "DevBuf":
        lib().moe_cuda_fill(self.ctx.p, self.ptr, self.nbytes, word)
        return self

    def free(self):
        if self.ptr:
            lib().moe_cuda_free(self.ctx.p, self.ptr)
            self.ptr = None


def _ptr(b):
    if b is None:
        return None
    if isinstance(b, DevBuf):
        return b.ptr
    return b


class Ctx:
    """One device + one in-order stream + a sticky status (mda_vkc_t in the reference)."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.p = lib().moe_cuda_create(device, stream)
        if not self.p:
            raise MemoryError("moe_cuda_create returned NULL")
        self.bufs: list[DevBuf] = []

    def status(self) -> int:
        return lib().moe_cuda_status(self.p)

    def last_error(self) -> str:
        return lib().moe_cuda_last_error(self.p).decode()

    def check(self):
        s = self.status()
        if s != MOE_OK:
            raise MoeCudaError(s, self.last_error())

    def flush(self):
        lib().moe_cuda_flush(self.p)
        self.check()

    def stream(self) -> int:
        return lib().moe_cuda_stream(self.p)

    def launches(self) -> int:
        return int(lib().moe_cuda_launches(self.p))

    def alloc(self, nbytes: int) -> DevBuf:
        b = DevBuf(self, max(int(nbytes), 16))
        self.bufs.append(b)
        return b

    def upload(self, a: np.ndarray) -> DevBuf:
        return self.alloc(a.nbytes).write(a)

    def zeros(self, nbytes: int) -> DevBuf:
        return self.alloc(nbytes).fill(0)

    def close(self):
        if self.p:
            for b in self.bufs:
                b.free()
            self.bufs = []
            lib().moe_cuda_destroy(self.p)
            self.p = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- the kernels, argument order = the shaders' binding order ----
    def route(self, proj, idx, wt, count, rows, experts, topk, stride):
        lib().moe_cuda_route(self.p, _ptr(proj), _ptr(idx), _ptr(wt), _ptr(count), PcRoute(rows, experts, topk, stride))

    def scan(self, count, off, tiles, experts, tile=TILE):
        lib().moe_cuda_scan(self.p, _ptr(count), _ptr(off), _ptr(tiles), PcScan(experts, tile))

    def scatter(self, idx, off, fill, x16, xp, slot, rows, topk, d8):
        lib().moe_cuda_scatter(self.p, _ptr(idx), _ptr(off), _ptr(fill), _ptr(x16), _ptr(xp), _ptr(slot),
                               PcScatter(rows, topk, d8))

    def scatter_noalloc(self, idx, off, fill, x16, xp, slot, rows, topk, d8, experts):
        lib().moe_cuda_scatter_noalloc(self.p, _ptr(idx), _ptr(off), _ptr(fill), _ptr(x16), _ptr(xp), _ptr(slot),
                                       PcScatter(rows, topk, d8), experts)

    def mm(self, A, B, Cout, amax, tiles, m, n, k, sa=NO_SLOT, sb=NO_SLOT, experts_in_B=1):
        lib().moe_cuda_mm(self.p, _ptr(A), _ptr(B), _ptr(Cout), _ptr(amax), _ptr(tiles), PcMm(m, n, k, sa, sb),
                          experts_in_B)

    def combine(self, wt, slot, y, proj, sh, inj, h, rows, d, topk, pstride, sg_off, inj_stride=0, inj_off=0, hc=1):
        lib().moe_cuda_combine(self.p, _ptr(wt), _ptr(slot), _ptr(y), _ptr(proj), _ptr(sh), _ptr(inj), _ptr(h),
                               PcCombine(rows, d, topk, pstride, sg_off, inj_stride, inj_off, hc))

    def swiglu(self, a, y, rows, n, astride, ao, bo, op=0, scale=1.0):
        lib().moe_cuda_swiglu(self.p, _ptr(a), _ptr(y), PcElem(rows, n, astride, ao, bo, op, scale))

    def norm(self, x, w, y, rows, groups, gsize, op=0, w_off=0, eps=1e-6, scale=1.0):
        """mda_qwen_norm_pc's strides (src/qwen.c:582-604): contiguous groups, one weight row per group."""
        pc = PcNorm(rows, groups, gsize, groups * gsize, 0, gsize, groups * gsize, 0, gsize, w_off, gsize, op, 0, 1, 0, 0, 0,
                    eps, scale, 1.0)
        lib().moe_cuda_norm(self.p, _ptr(x), _ptr(w), _ptr(y), None, pc)

    def hc(self, a, b, h, rows, d, hc, op, inj_stride=0, inj_off=0):
        lib().moe_cuda_hc(self.p, _ptr(a), _ptr(b), _ptr(h), PcHc(rows, d, hc, op, inj_stride, inj_off))

    def dense(self, A16, W, Cout, amax, rows, n, k, sa=NO_SLOT):
        lib().moe_cuda_dense(self.p, _ptr(A16), _ptr(W), _ptr(Cout), _ptr(amax), PcDense(rows, n, k, sa))

    def absmax(self, x, amax, n, slot):
        lib().moe_cuda_absmax(self.p, _ptr(x), _ptr(amax), PcSlot(n, slot))

    def cast_f16(self, src, dst, amax, n, slot):
        lib().moe_cuda_cast_f16(self.p, _ptr(src), _ptr(dst), _ptr(amax), PcSlot(n, slot))

    def bf16_to_f16(self, w, n_words):
        lib().moe_cuda_bf16_to_f16(self.p, _ptr(w), PcBf16(n_words))

    def kd_bytes(self, logits, toks, cont, outp, rows, vocab):
        lib().moe_cuda_kd_bytes(self.p, _ptr(logits), _ptr(toks), _ptr(cont), _ptr(outp), PcKd(rows, vocab))

    def layer(self, **kw):
        L = Layer()
        for k, v in kw.items():   # DevBuf, raw device address (int) or None for pointers; numbers otherwise
            setattr(L, k, _ptr(v) if isinstance(v, DevBuf) or v is None else v)
        lib().moe_cuda_layer(self.p, C.byref(L))

    def ep_init(self, unique_id: bytes, rank: int, world: int, experts, topk, d, inter, max_rows, micro_batches=0,
                transfer=0):
        assert len(unique_id) == 128
        buf = C.create_string_buffer(unique_id, 128)
        cfg = EpCfg(experts, topk, d, inter, max_rows, micro_batches, transfer)
        lib().moe_cuda_ep_init(self.p, buf, rank, world, C.byref(cfg))
        self.check()

    def ep_layer(self, **kw):
        L = Layer()
        for k, v in kw.items():
            setattr(L, k, _ptr(v) if isinstance(v, DevBuf) or v is None else v)
        lib().moe_cuda_ep_layer(self.p, C.byref(L))

    def prof(self, on: bool):
        lib().moe_cuda_prof(self.p, 1 if on else 0)

    def prof_read(self) -> dict:
        ms = (C.c_float * len(PROF_STAGES))()
        lib().moe_cuda_prof_read(self.p, ms)
        return {n: float(ms[i]) for i, n in enumerate(PROF_STAGES)}


def ep_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    rc = lib().moe_cuda_ep_unique_id(buf)
    if rc != MOE_OK:
        raise MoeCudaError(rc, "could not create an NCCL unique id")
    return buf.raw


def moe_rows(rows: int, topk: int, experts: int) -> int:
    return int(lib().moe_cuda_moe_rows(rows, topk, experts))
