"""Throughput of the three pieces beside the MoE layer, one JSON line each:

    python bench_micro.py bf16     in-place bf16 -> fp16 conversion of a 1 GiB bank (moe_cuda_bf16_to_f16)
    python bench_micro.py upload   one 30B-A3B layer's MoE weights: page-locked banks -> device + conversion
    python bench_micro.py kd       distillation sink on 1024 rows x 151 936 tokens (moe_cuda_kd_bytes)

Timed with the host clock between stream synchronisations over several calls, after warm-up; the
buffers (>= 0.6 GB) are larger than L2.  Needs a B200; there is no CPU fallback."""
from __future__ import annotations

import ctypes as C
import json
import sys
import time

import numpy as np

import __graft_entry__ as entry


def timed(ctx, fn, warm, reps):
    for _ in range(warm):
        fn()
    ctx.flush()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    ctx.flush()
    return (time.perf_counter() - t0) / reps


def bench_bf16(mc, ctx, hbm):
    n_words = 256 << 20                      # 1 GiB bank, 512 Mi values
    d = ctx.alloc(n_words * 4)
    d.fill(0x3f803f80)
    dt = timed(ctx, lambda: ctx.bf16_to_f16(d, n_words), 3, 10)
    gbs = 2 * n_words * 4 / dt / 1e9          # every byte read once and written once
    return {"kernel": "moe_bf16_to_f16_kernel", "bytes": 2 * n_words * 4, "ms": dt * 1e3, "GB/s": gbs, "frac_hbm": gbs / hbm}


def bench_upload(pkg, mc, ctx, hbm):
    class Stage(C.Structure):
        _fields_ = [("host", C.c_void_p), ("size", C.c_uint64), ("used", C.c_uint64)]

    class Bank(C.Structure):
        _fields_ = [("dense", Stage), ("gu", Stage), ("down", Stage), ("moe", C.c_uint64), ("sdown", C.c_uint64),
                    ("pinned", C.c_bool), ("fail", C.c_bool), ("c", C.c_void_p)]

    class BankCfg(C.Structure):
        _fields_ = [(n, C.c_uint32) for n in ("d", "experts", "inter", "shared")]

    pkg.build.build_host()
    L = C.CDLL(pkg.build.HOST_LIB)
    L.moe_bank_open.restype = C.c_bool
    L.moe_bank_open.argtypes = [C.POINTER(Bank), C.c_void_p, BankCfg]
    L.moe_bank_upload.argtypes = [C.POINTER(Bank), C.c_void_p, C.c_void_p, C.c_void_p, C.c_bool]
    L.moe_bank_close.argtypes = [C.POINTER(Bank)]
    bank = Bank()
    if not L.moe_bank_open(C.byref(bank), ctx.p, BankCfg(2048, 128, 768, 0)):
        raise SystemExit("page-locked banks could not be allocated")
    stages = (bank.dense, bank.gu, bank.down)
    for st in stages:                         # any finite bf16 pattern: the copy and the conversion do not look at it
        C.memset(st.host, 0x3c, st.size)
        st.used = st.size
    total = sum(st.size for st in stages)
    dev = [ctx.alloc(st.size) for st in stages]
    dt = timed(ctx, lambda: L.moe_bank_upload(C.byref(bank), dev[0].ptr, dev[1].ptr, dev[2].ptr, True), 1, 4)
    ctx.check()
    L.moe_bank_close(C.byref(bank))
    return {"path": "moe_bank_upload (3 host-to-device copies + conversion)", "bytes": total, "ms": dt * 1e3,
            "GB/s": total / dt / 1e9, "bound": "host-to-device link"}


def bench_kd(mc, ctx, hbm):
    rows, vocab = 1024, 151936
    rng = np.random.default_rng(0)
    tb = rng.integers(97, 123, (vocab, 16)).astype(np.uint8)      # lower-case strings of 1..8 bytes
    length = rng.integers(1, 9, vocab)
    for k in range(16):
        tb[length <= k, k] = 0
    toks = np.ascontiguousarray(np.concatenate([tb.view(np.uint32).reshape(vocab, 4), length[:, None].astype(np.uint32)], 1))
    cont = np.zeros((rows, 5), np.uint32)
    cont[:, :4] = rng.integers(97, 123, (rows, 16)).astype(np.uint8).view(np.uint32).reshape(rows, 4)
    cont[:, 4] = 8
    d_l = ctx.alloc(rows * vocab * 4)
    d_l.fill(0x3f000000)                      # every logit 0.5: the arithmetic does not depend on the values
    d_t, d_c, d_o = ctx.upload(toks), ctx.upload(cont), ctx.alloc(rows * 128 * 4)
    dt = timed(ctx, lambda: ctx.kd_bytes(d_l, d_t, d_c, d_o, rows, vocab), 2, 5)
    gbs = rows * vocab * 4 / dt / 1e9         # algorithmic bytes: each logit once
    return {"kernel": "moe_kd_bytes_kernel", "rows": rows, "vocab": vocab, "bytes": rows * vocab * 4, "ms": dt * 1e3,
            "GB/s": gbs, "frac_hbm": gbs / hbm}


def main():
    which = sys.argv[1] if len(sys.argv) > 1 else ""
    if which not in ("bf16", "upload", "kd"):
        raise SystemExit(__doc__)
    pkg = entry.load_package()
    mc = pkg.moe_cuda
    from bench import peaks
    hbm = peaks()["hbm_gbs"]
    with mc.Ctx(0) as ctx:
        out = {"bf16": lambda: bench_bf16(mc, ctx, hbm), "upload": lambda: bench_upload(pkg, mc, ctx, hbm),
               "kd": lambda: bench_kd(mc, ctx, hbm)}[which]()
        ctx.check()
    out["hbm_peak_GB/s"] = hbm
    print(json.dumps(out))


if __name__ == "__main__":
    main()
