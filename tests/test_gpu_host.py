"""The C host-side mirror of the reference's call sites (r-mda_b200/host/moe_host.c: mda_qwen_route_rec /
mda_qwen_moe_rec with the dispatch target swapped) driven through ctypes: the
step-by-step sequence and the fused entry point against the CPU oracle."""
import ctypes as C
import dataclasses

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class HostCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("d", "experts", "topk", "inter", "shared", "hc", "hc_pad", "hc_rank")]


class HostScratch(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("p", "a16", "t", "idx", "wt", "slot", "count", "off", "fill", "tiles", "xp",
                                          "g", "hp", "hp16", "ye", "hs", "sh", "gs", "hs16", "tiles0")] + [("moe_rows", C.c_uint32)]


class Host(C.Structure):
    _fields_ = [("c", C.c_void_p), ("cfg", HostCfg), ("sc", HostScratch), ("wgu", C.c_void_p), ("wdown", C.c_void_p),
                ("wsgu", C.c_void_p), ("wsdown", C.c_void_p), ("amax", C.c_void_p), ("n_slots", C.c_uint32),
                ("chunk", C.c_uint32)]


@pytest.fixture(scope="module")
def hostlib(pkg):
    pkg.build.build_host()
    L = C.CDLL(pkg.build.HOST_LIB)
    L.moe_host_open.restype = C.c_bool
    L.moe_host_open.argtypes = [C.POINTER(Host), C.c_void_p, HostCfg, C.c_uint32]
    L.moe_host_close.argtypes = [C.POINTER(Host)]
    L.moe_host_slots_begin.argtypes = [C.POINTER(Host)]
    L.moe_host_moe_rec.argtypes = [C.POINTER(Host), C.c_void_p, C.c_uint32]
    L.moe_host_moe_rec_fused.argtypes = [C.POINTER(Host), C.c_void_p, C.c_uint32, C.c_uint32]
    L.moe_host_moe_cols.restype = C.c_uint32
    L.moe_host_moe_cols.argtypes = [HostCfg]
    L.moe_host_moe_rows.restype = C.c_uint32
    L.moe_host_moe_rows.argtypes = [HostCfg, C.c_uint32]
    return L


@pytest.mark.parametrize("shared,hc", [(0, 1), (128, 1), (0, 4)])
def test_host_sequence_matches_oracle(ctx, mc, synth, oracle, hostlib, shared, hc):
    cfg = dataclasses.replace(synth.CONFIGS["c0"], T=320, E=16, K=4, d=256, I=256, S=shared)
    inp = synth.layer_inputs(cfg, 9)
    hcfg = HostCfg(cfg.d, cfg.E, cfg.K, cfg.I, cfg.S, hc, 8, 2)
    assert hostlib.moe_host_moe_rows(hcfg, cfg.T) == oracle.moe_rows(cfg.T, cfg.K, cfg.E)
    pcols = hostlib.moe_host_moe_cols(hcfg)
    assert pcols == cfg.E + 128 + 2 * cfg.S
    proj = np.zeros((cfg.T, pcols), np.float32)
    proj[:, :cfg.E + 128] = inp.proj
    rng = np.random.default_rng(0)
    inj = rng.standard_normal((cfg.T, 8)).astype(np.float32)
    h0 = rng.standard_normal((cfg.T, hc, cfg.d)).astype(np.float32)
    ref = oracle.layer(proj, inp.x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown, h=h0.copy(), hc=hc,
                       inj=np.ascontiguousarray(inj[:, 2:2 + hc]))
    for fused in (False, True):
        q = Host()
        assert hostlib.moe_host_open(C.byref(q), ctx.p, hcfg, cfg.T)
        L = mc.lib()
        L.moe_cuda_write(ctx.p, q.sc.p, proj.ctypes.data, proj.nbytes)
        L.moe_cuda_write(ctx.p, q.sc.a16, inp.x16.ctypes.data, inp.x16.nbytes)
        L.moe_cuda_write(ctx.p, q.sc.t, inj.ctypes.data, inj.nbytes)
        q.wgu, q.wdown = ctx.upload(inp.wgu).ptr, ctx.upload(inp.wdown).ptr
        if cfg.S:
            q.wsgu, q.wsdown = ctx.upload(inp.wsgu).ptr, ctx.upload(inp.wsdown).ptr
        d_h = ctx.upload(h0)
        hostlib.moe_host_slots_begin(C.byref(q))
        if fused:
            hostlib.moe_host_moe_rec_fused(C.byref(q), d_h.ptr, cfg.T, 0)
        else:
            hostlib.moe_host_moe_rec(C.byref(q), d_h.ptr, cfg.T)
        ctx.flush()
        h = d_h.read(np.float32, (cfg.T, hc, cfg.d))
        slot = np.empty((cfg.T, cfg.K), np.uint32)
        L.moe_cuda_read(ctx.p, slot.ctypes.data, q.sc.slot, slot.nbytes)
        assert np.array_equal(slot, ref.slot)
        err = np.abs(h - ref.h)
        assert np.all(err <= 1e-3 + 2e-2 * np.abs(ref.h)), (fused, err.max())
        hostlib.moe_host_close(C.byref(q))
