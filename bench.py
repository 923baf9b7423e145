#!/usr/bin/env python
"""Benchmark of the MoE forward path (route -> scan -> scatter -> grouped SwiGLU products ->
combine) through libmoe_cuda's C ABI.

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference

A step is one pass of one MoE layer of the "30B-A3B" shape (T=4096 tokens per GPU, d=2048, E=128,
top-8, I=768; seeded synthetic fp16 weights and activations).  Rank 0 prints one JSON line.  Every
line of this library's arm carries a "parity" object: the result of a step is compared with the CPU
oracle on the same inputs (routing and permutation bit-exact, outputs within 2e-2 relative / 1e-3
absolute), and the run exits non-zero if that does not hold.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "MoE layer tokens/s (route->scatter->grouped GEMM->combine)"
STACK_METRIC = "teacher-forward MoE stack tokens/s (48 x [projection -> route -> grouped GEMM -> combine -> residual + RMSNorm])"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
RTOL_OUT, ATOL_OUT, RTOL_WT = 2e-2, 1e-3, 1e-5

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, the
# weight-stationary gate_up grouped product (moe_mm_ws_kernel<SWIGLU_F16, pair>), at the 30B-A3B shape:
# one Nsight Compute capture of a full-size launch (no scaling involved).
NCU_TRAFFIC_BYTES = {"c1": 955979264 + 47768064}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            m = json.load(f)
        return {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]),
                "bf16_tflops_sustained": float(m.get("bf16_tflops_sustained", m["bf16_tflops"])), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms during the timed region (query only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.f,
                                      stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        self.f.seek(0)
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
                pw.append(float(c[3]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons)}


def pinned_array(mc, ctx, shape, dtype):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = mc.lib().moe_cuda_alloc_pinned(ctx.p, n)
    ctx.check()
    buf = (ctypes.c_uint8 * n).from_address(p)
    return np.frombuffer(buf, dtype=dtype).reshape(shape), p


def workload_config(cfg, n_gpus):
    return {"workload": f"{cfg.name}: T={cfg.T} tokens per GPU, d={cfg.d}, E={cfg.E}, top-{cfg.K}, I={cfg.I}"
                        + (f", shared S={cfg.S}" if cfg.S else "") + (f", {cfg.layers} layers" if cfg.layers > 1 else ""),
            "global_tokens": cfg.T * n_gpus,
            "parallelism": "single GPU" if n_gpus == 1 else f"expert-parallel ep{n_gpus}: E/{n_gpus} experts per GPU",
            "l2": "inputs larger than L2: 1.2 GB of expert weights are streamed from HBM every step"}


# ---- the checker: the CPU oracle on the same inputs --------------------------------------------
def parity_mask(T: int, rows: int = 512):
    """Rows whose outputs are compared: all of them up to 4096 tokens, else `rows` evenly spaced ones
    (routing, counts, offsets and the permutation are always compared for every row)."""
    if T <= 4096:
        return None
    m = np.zeros(T, np.uint8)
    m[np.linspace(0, T - 1, rows).astype(np.int64)] = 1
    return m


def oracle_layer(inp, cfg, mask=None, tokens=None):
    from oracle import moe_oracle as O
    proj, x16 = inp.proj, inp.x16
    if tokens is not None and tokens < proj.shape[0]:
        proj, x16 = np.ascontiguousarray(proj[:tokens]), np.ascontiguousarray(x16[:tokens])
    return O.layer(proj, x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown, row_mask=mask)


def parity_report(ref, got: dict, mask=None, slot_want=None) -> dict:
    """got: idx, wt, count, off, slot, h of one step of this library on the oracle's inputs.
    slot_want overrides the expected permutation (expert parallel: rows inside the owner's buffer)."""
    exact = {"idx": bool(np.array_equal(got["idx"], ref.idx))}
    if "count" in got:
        exact["count"] = bool(np.array_equal(got["count"], ref.count))
    if "off" in got:
        exact["off"] = bool(np.array_equal(got["off"], ref.off))
    exact["slot"] = bool(np.array_equal(got["slot"], ref.slot if slot_want is None else slot_want))
    wt_ok = bool(np.all(np.abs(got["wt"] - ref.wt) <= RTOL_WT * np.abs(ref.wt)))
    rows = np.arange(ref.h.shape[0]) if mask is None else np.nonzero(mask)[0]
    rh = ref.h.reshape(ref.h.shape[0], -1)[rows]
    gh = got["h"].reshape(got["h"].shape[0], -1)[rows]
    err = np.abs(gh - rh)
    out_ok = bool(np.all(err <= ATOL_OUT + RTOL_OUT * np.abs(rh)))
    return {"checked": True, "against": "CPU oracle, same inputs", "bit_exact": all(exact.values()), "bit_exact_fields": exact,
            "router_weights_within_1e-5": wt_ok, "outputs_within_2e-2_rel_1e-3_abs": out_ok, "max_err": float(err.max()),
            "max_abs_ref": float(np.abs(rh).max()), "rows_checked": int(len(rows)), "ok": all(exact.values()) and wt_ok and out_ok}


def cpu_baseline(cfg, inp, sample_tokens: int, reps: int = 1):
    """Times the CPU oracle on the first `sample_tokens` tokens of the workload (all experts' weights
    resident) on every core the process may use.  Returns the record and the oracle's result."""
    from oracle import moe_oracle as O
    O.use_all_cores()
    T = min(sample_tokens, cfg.T)
    best, res = None, None
    for _ in range(reps):
        t0 = time.perf_counter()
        res = oracle_layer(inp, cfg, tokens=T)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    rec = {"value": T / best, "unit": "tokens/s", "cores": O.threads(), "kind": "port",
           "sample": f"first {T} of {cfg.T} tokens of the workload, whole layer on the CPU oracle, best of {reps}",
           "seconds": best}
    return rec, (res if T == cfg.T else None)


def run_reference(args):
    """The reference arm: the reference's own implementation of the path is GLSL over Vulkan and
    cannot run on this box, so its scalar C restatement (the oracle) is timed on the host cores.
    With N > 1 the GPU arm's batch is N x T tokens over the same E experts; rank 0 alone times a
    bounded sample of that batch with all host threads, the other ranks leave at once."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import dataclasses
    pkg = entry.load_package()
    synth = pkg.synth
    cfg = synth.CONFIGS[args.config]
    from oracle import moe_oracle as O
    cores = O.use_all_cores()
    n = max(args.gpus, 1)
    T_all = cfg.T * n
    T = min(args.ref_tokens, T_all, 16384)
    gcfg = dataclasses.replace(cfg, T=T)   # synthetic rows are a function of (seed, row), so this is a prefix of the N x T batch
    inp = synth.layer_inputs(gcfg, 0)
    for _ in range(args.warmup):
        oracle_layer(inp, gcfg)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle_layer(inp, gcfg)
    dt = (time.perf_counter() - t0) / args.steps
    v = T / (dt * cfg.layers)   # a stack of `layers` equal layers: one is timed, the rest scaled
    sample = (f"each step = first {T} of the {T_all} tokens of the workload through one whole layer"
              + (f"; the workload's {cfg.layers} layers are equal in cost, so tokens/s = that / {cfg.layers}" if cfg.layers > 1 else ""))
    metric = METRIC if cfg.layers == 1 else STACK_METRIC
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(cfg, args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference shaders need Vulkan: unavailable on this box; timed its scalar C restatement",
    }), flush=True)


def run_ours(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # Libraries (NCCL's version banner, for one) write to stdout; keep stdout for the one JSON line.
    sys.stdout.flush()
    args.real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    mc, synth = pkg.moe_cuda, pkg.synth
    stream = torch.cuda.Stream(device=local)
    ctx = mc.Ctx(local, stream.cuda_stream)
    ctx.check()
    if args.config == "kd":
        if world > 1:
            raise SystemExit("--config kd is a one-GPU leg")
        return run_kd(args, ctx, mc, stream, local)
    cfg = synth.CONFIGS[args.config]
    if world > 1:
        from bench_ep import run_ep  # noqa: F401  (expert-parallel driver)
        return run_ep(args, ctx, mc, synth, cfg, stream, rank, world, local)
    if cfg.layers > 1 and args.stream_layers:
        return run_stream(args, ctx, mc, synth, cfg, stream, local)
    if cfg.layers > 1:
        return run_stack(args, ctx, mc, synth, cfg, stream, local)
    return run_layer(args, ctx, mc, synth, cfg, stream, local)


def emit(args, out, ok=True):
    """Print the result line on the process's original stdout; a failed parity check ends the run with an error."""
    sys.stdout.flush()
    os.dup2(args.real_stdout, 1)
    print(json.dumps(out), flush=True)
    if not ok:
        print("bench.py: the timed layer's result does not match the CPU oracle", file=sys.stderr, flush=True)
        os._exit(1)


def timed_steps(torch, stream, fn, steps):
    """K steps between two CUDA events on the launching stream, a device synchronisation on both sides."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(steps):
            fn()
        ev1.record(stream)
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / steps


def sustained_run(torch, stream, fn, ms_per_step, local, flops_per_step, pk, tokens_per_step, seconds=2.5):
    """The same step back to back for a few seconds: what a caller that runs 48 layers x many chunks
    sees once the part has settled at its power limit.  Clocks are only read, never set."""
    n = max(20, int(seconds * 1e3 / max(ms_per_step, 1e-3)))
    fn()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    ms = timed_steps(torch, stream, fn, n)
    clk = sampler.stop()
    tf = flops_per_step / (ms * 1e-3) / 1e12
    return {"tokens_per_s": tokens_per_step / (ms * 1e-3), "ms_per_step": ms, "steps": n, "seconds": n * ms * 1e-3,
            "sm_mhz_median": clk["sm_mhz"], "power_w_max": clk.get("power_w_max"), "reasons": clk["reasons"],
            "TFLOP/s_all_kernels": tf, "frac_of_sustained_peak": tf / pk["bf16_tflops_sustained"],
            "sustained_peak_TFLOP/s": pk["bf16_tflops_sustained"]}


def issue_efficiency(count, chunked: bool):
    """Real rows / rows the tensor cores are asked to multiply: the token-major kernel pads every expert to
    128-row tiles (shader/moe_scan.comp:19), the chunked kernel rounds each chunk of <= 256 rows to 16."""
    c = count.astype(np.int64)
    real = int(c.sum())
    if chunked:
        nch = (c + 255) // 256
        per = np.where(nch > 0, ((c + np.maximum(nch, 1) - 1) // np.maximum(nch, 1) + 15) // 16 * 16, 0)
        issued = 0
        for cnt, n, p in zip(c, nch, per):
            for j in range(int(n)):
                v = max(0, min(int(p), int(cnt) - j * int(p)))
                issued += (v + 15) // 16 * 16
    else:
        issued = int(((c + 127) // 128 * 128).sum())
    return {"real_rows": real, "issued_rows": issued, "real_over_issued": real / issued if issued else None}


def run_layer(args, ctx, mc, synth, cfg, stream, local):
    """One GPU, one MoE layer per step (configs c0 .. c3b)."""
    import torch

    T, K, E, d, I = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I
    inp = synth.layer_inputs(cfg, 0)
    d_wgu, d_wdown = ctx.upload(inp.wgu), ctx.upload(inp.wdown)
    d_wsgu = ctx.upload(inp.wsgu) if cfg.S else None
    d_wsdown = ctx.upload(inp.wsdown) if cfg.S else None
    d_proj, d_x = ctx.upload(inp.proj), ctx.upload(inp.x16)
    d_h = ctx.zeros(T * d * 4)
    lay = dict(rows=T, d=d, experts=E, topk=K, inter=I, shared=cfg.S, pstride=cfg.pstride, hc=1,
               proj=d_proj, x16=d_x, wgu=d_wgu, wdown=d_wdown, wsgu=d_wsgu, wsdown=d_wsdown, h=d_h, flags=args.flags)

    def step():
        ctx.layer(**lay)

    # ---- device-resident throughput ----
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    ctx.flush()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    l0 = ctx.launches()
    ms = timed_steps(torch, stream, step, args.steps)
    ctx.check()
    launches = ctx.launches() - l0

    # ---- one more step of the same workload, checked against the CPU oracle ----
    outs = {n: ctx.alloc(T * K * 4) for n in ("idx", "slot", "wt")}
    outs["count"], outs["off"] = ctx.alloc(E * 4), ctx.alloc(E * 4)
    d_h.fill(0)
    ctx.layer(**dict(lay, **outs))
    ctx.flush()
    got = {"idx": outs["idx"].read(np.uint32, (T, K)), "slot": outs["slot"].read(np.uint32, (T, K)),
           "wt": outs["wt"].read(np.float32, (T, K)), "count": outs["count"].read(np.uint32, (E,)),
           "off": outs["off"].read(np.uint32, (E,)), "h": d_h.read(np.float32, (T, d))}

    # ---- per-stage device times (CUDA events between the stages, same workload) ----
    ctx.prof(True)
    stage_ms = {n: 0.0 for n in mc.PROF_STAGES}
    for _ in range(args.steps):
        step()
        for n, v in ctx.prof_read().items():
            stage_ms[n] += v / args.steps
    ctx.prof(False)

    # ---- end to end through the C ABI with host buffers ----
    # Every step copies its own inputs host->device from pinned memory and its result device->host.
    # Three contexts (three in-order streams) take steps in turn, so one step's copies overlap the
    # others' kernels; a step's host buffers are reused only after its flush.
    L = mc.lib()
    extra = [mc.Ctx(local, torch.cuda.Stream(device=local).cuda_stream) for _ in range(2)]
    lanes = []
    for cx in [ctx] + extra:
        hp, _ = pinned_array(mc, cx, inp.proj.shape, np.float32)
        hx, _ = pinned_array(mc, cx, inp.x16.shape, np.uint16)
        ho, _ = pinned_array(mc, cx, (T, d), np.float32)
        hp[:], hx[:] = inp.proj, inp.x16
        dp, dx, dh = (d_proj, d_x, d_h) if cx is ctx else (cx.upload(inp.proj), cx.upload(inp.x16), cx.zeros(T * d * 4))
        lanes.append(dict(ctx=cx, hp=hp, hx=hx, ho=ho, lay=dict(lay, proj=dp, x16=dx, h=dh), dp=dp, dx=dx, dh=dh))
    h_proj, h_x, h_out = lanes[0]["hp"], lanes[0]["hx"], lanes[0]["ho"]

    def e2e_issue(ln):
        cx = ln["ctx"]
        L.moe_cuda_write(cx.p, ln["dp"].ptr, ln["hp"].ctypes.data, ln["hp"].nbytes)
        L.moe_cuda_write(cx.p, ln["dx"].ptr, ln["hx"].ctypes.data, ln["hx"].nbytes)
        L.moe_cuda_fill(cx.p, ln["dh"].ptr, T * d * 4, 0)
        cx.layer(**ln["lay"])
        L.moe_cuda_read_async(cx.p, ln["ho"].ctypes.data, ln["dh"].ptr, ln["ho"].nbytes)

    def e2e_run(n):
        for i in range(n):
            ln = lanes[i % len(lanes)]
            if i >= len(lanes):
                ln["ctx"].flush()      # that lane's previous result is on the host; its buffers are free again
            e2e_issue(ln)
        for ln in lanes:
            ln["ctx"].flush()

    e2e_run(warm + 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_run(args.steps)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps   # wall clock between synchronisations: three streams
    for ln in lanes:
        ln["ctx"].check()
        assert np.array_equal(lanes[0]["ho"], ln["ho"]), "the end-to-end lanes disagree"
    e2e_matches = bool(np.array_equal(lanes[0]["ho"], got["h"]))   # same inputs, deterministic kernels
    clocks = sampler.stop()

    pk = peaks()
    sustained = None if args.no_sustained else sustained_run(torch, stream, step, ms, local, cfg.flops(), pk, T)

    # ---- the CPU legs: the timed baseline and the parity check of the step above ----
    cpu, ref = (None, None) if args.no_cpu else cpu_baseline(cfg, inp, args.ref_tokens)
    mask = parity_mask(T)
    if args.no_parity:
        parity = {"checked": False}
    else:
        if ref is None or mask is not None:
            from oracle import moe_oracle as O
            O.use_all_cores()
            ref = oracle_layer(inp, cfg, mask=mask)
        parity = parity_report(ref, got, mask)
        parity["e2e_result_equals_checked_result"] = e2e_matches

    gemm1_flops = T * K * 4 * d * I          # gate_up product, unpadded
    gemm2_flops = T * K * 2 * d * I
    tf1 = gemm1_flops / (stage_ms["gate_up"] * 1e-3) / 1e12
    tf2 = gemm2_flops / (stage_ms["down"] * 1e-3) / 1e12
    scatter_bytes = T * d * 2 + T * K * d * 2 + T * K * 8   # each token row in once, out once per routed pair
    combine_bytes = T * K * d * 2 + T * K * 8 + 2 * T * d * 4   # expert outputs are kept fp16 in the fused layer
    route_bytes = T * E * 4 + T * K * 8 + E * 4
    gbs = lambda b, m: b / (m * 1e-3) / 1e9 if m > 0 else None
    gu_bytes = E * 2 * I * d * 2 + T * K * d * 2 + T * K * I * 2
    chunked = not (args.flags & (mc.LAYER_TILED | mc.LAYER_UNFUSED)) and d % 128 == 0
    eff = issue_efficiency(got["count"], chunked)
    stages = {
        "route": {"ms": stage_ms["route"], "GB/s": gbs(route_bytes, stage_ms["route"])},
        "scan": {"ms": stage_ms["scan"]},
        "scatter": ({"ms": stage_ms["scatter"], "GB/s": gbs(scatter_bytes, stage_ms["scatter"]),
                     "frac_hbm": gbs(scatter_bytes, stage_ms["scatter"]) / pk["hbm_gbs"]}
                    if chunked or (args.flags & mc.LAYER_MATERIALIZE_XP) else
                    {"ms": stage_ms["scatter"], "note": "ranks and slot tables only; the gate_up product gathers the rows"}),
        "front_end_ms": stage_ms["route"] + stage_ms["scan"] + stage_ms["scatter"],
        "gate_up": {"ms": stage_ms["gate_up"], "TFLOP/s": tf1, "frac_tensor": tf1 / pk["bf16_tflops"],
                    "weight_GB/s": gbs(E * 2 * I * d * 2, stage_ms["gate_up"]), "real_over_issued_flops": eff["real_over_issued"]},
        "down": {"ms": stage_ms["down"], "TFLOP/s": tf2, "frac_tensor": tf2 / pk["bf16_tflops"],
                 "weight_GB/s": gbs(E * I * d * 2, stage_ms["down"]), "real_over_issued_flops": eff["real_over_issued"]},
        "combine": {"ms": stage_ms["combine"], "GB/s": gbs(combine_bytes, stage_ms["combine"]),
                    "frac_hbm": gbs(combine_bytes, stage_ms["combine"]) / pk["hbm_gbs"]},
    }
    if cfg.S:
        stages["shared"] = {"ms": stage_ms["shared"]}
    kernel = ("moe_mm_ws_kernel<SWIGLU_F16, pair> (gate_up grouped product, weight-stationary, SwiGLU fused)" if chunked else
              "moe_mm_kernel<SWIGLU_F16, GATHER> (gate_up grouped product, row gather + SwiGLU fused)")
    out = {
        "metric": METRIC, "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(cfg, 1),
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(h_proj.nbytes + h_x.nbytes),
                "d2h_bytes_per_step": int(h_out.nbytes), "ms_per_step": e2e_ms,
                "how": "three contexts take steps in turn so copies overlap kernels; wall clock between device synchronisations"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "parity": parity,
        "roofline": {"bound": "tensor", "kernel": kernel,
                     "achieved": tf1, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf1 / pk["bf16_tflops"],
                     "traffic": NCU_TRAFFIC_BYTES.get(args.config) if chunked else None, "peak_source": pk["source"] + " (burst)",
                     "flops_per_launch": gemm1_flops, "ms_per_launch": stage_ms["gate_up"],
                     # the same launch against the other roof: weights once, each routed row in once, fp16 result out once
                     "hbm_view": {"algorithmic_bytes": gu_bytes, "achieved": gbs(gu_bytes, stage_ms["gate_up"]), "peak": pk["hbm_gbs"],
                                  "unit": "GB/s", "frac": gbs(gu_bytes, stage_ms["gate_up"]) / pk["hbm_gbs"],
                                  "flop_per_byte": gemm1_flops / gu_bytes, "ridge_flop_per_byte": pk["bf16_tflops"] * 1e3 / pk["hbm_gbs"]}},
        "stages": stages,
    }
    if sustained is not None:
        out["sustained"] = sustained
    if cpu is not None:
        out["cpu_baseline"] = cpu
    for cx in extra:
        cx.close()
    ctx.close()
    emit(args, out, ok=parity.get("ok", True))


def run_kd(args, ctx, mc, stream, local):
    """The distillation sink next to the layer (moe_cuda_kd_bytes = shader/kd_bytes.comp) on 1024 rows of
    logits over a 151 936-token byte-level vocabulary of lower-case strings; HBM bound by its algorithmic
    bytes (every logit once).  A few rows are compared with the CPU oracle."""
    import torch

    rows, vocab = 1024, 151936
    pk = peaks()
    rng = np.random.default_rng(0)
    tb = rng.integers(97, 123, (vocab, 16)).astype(np.uint8)      # strings of 1..8 bytes
    length = rng.integers(1, 9, vocab)
    for k in range(16):
        tb[length <= k, k] = 0
    toks = np.ascontiguousarray(np.concatenate([tb.view(np.uint32).reshape(vocab, 4), length[:, None].astype(np.uint32)], 1))
    cont = np.zeros((rows, 5), np.uint32)
    cont[:, :4] = rng.integers(97, 123, (rows, 16)).astype(np.uint8).view(np.uint32).reshape(rows, 4)
    cont[:, 4] = 8
    dev = torch.device("cuda", local)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    logits = torch.randn((rows, vocab), device=dev, generator=gen, dtype=torch.float32) * 3.0
    d_t, d_c, d_o = ctx.upload(toks), ctx.upload(cont), ctx.alloc(rows * 128 * 4)
    fn = lambda: ctx.kd_bytes(logits.data_ptr(), d_t, d_c, d_o, rows, vocab)
    torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        fn()
    ctx.flush()
    sampler = ClockSampler(local)
    sampler.start()
    ms = timed_steps(torch, stream, fn, args.steps)
    clocks = sampler.stop()
    ctx.check()
    parity = {"checked": False}
    if not args.no_parity:
        from oracle import moe_oracle as O
        O.use_all_cores()
        nchk = 8
        got = d_o.read(np.uint32, (rows, 16, 8))[:nchk]
        ref = O.kd_bytes(np.ascontiguousarray(logits[:nchk].cpu().numpy()), toks, cont[:nchk])
        pg = (got >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        pr = (ref >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        close = np.abs(pg - pr) <= 1.5e-3 * pr + 1e-7
        parity = {"checked": True, "against": "CPU oracle, first %d rows" % nchk, "probabilities_within_1.5e-3_rel": bool(close.all()),
                  "true_byte_entries_equal": bool(np.array_equal(got[..., 0] & 0xffff, ref[..., 0] & 0xffff)),
                  "byte_entries_differing": float(((got & 0xffff) != (ref & 0xffff)).mean())}
        parity["ok"] = parity["probabilities_within_1.5e-3_rel"] and parity["true_byte_entries_equal"] and parity["byte_entries_differing"] < 0.01
    nbytes = rows * vocab * 4
    gbs = nbytes / (ms * 1e-3) / 1e9
    out = {"metric": "distillation sink rows/s (kd_bytes over a byte-level vocabulary)", "value": rows / (ms * 1e-3), "unit": "rows/s",
           "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": "kd: 1024 rows x 151936 logits, 16 depths x 8 entries out", "l2": "622 MB of logits per step, larger than L2"},
           "gpu_launches": 2 * args.steps, "clocks": clocks, "parity": parity,
           "roofline": {"bound": "hbm", "kernel": "moe_kd_bytes_kernel (+ moe_kd_sort_kernel once per call)", "achieved": gbs,
                        "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "traffic": None,
                        "peak_source": pk["source"], "bytes_per_launch": nbytes, "ms_per_launch": ms}}
    ctx.close()
    emit(args, out, ok=parity.get("ok", True))


def stack_weights(torch, cfg, dev, e_lo=0, e_hi=None):
    """Per-layer seeded weights generated on the device (58 GB of fp16 for the whole stack on one GPU):
    wgu / wdown of experts e_lo..e_hi-1 and the upstream projection's weight rows [E router rows, the
    shared-gate row, zeros up to E+128] (the packing of mda_qwen_put_moe, src/qwen.c:441-452)."""
    E, d, I, NL, pcols = cfg.E, cfg.d, cfg.I, cfg.layers, cfg.pstride
    e_hi = E if e_hi is None else e_hi
    gen = torch.Generator(device=dev)
    layers = []
    for l in range(NL):
        ws = []
        for e in range(e_lo, e_hi):   # seeded per (layer, expert) so that any rank can make any expert slice
            gen.manual_seed(100000 * (l + 1) + e)
            ws.append((torch.randn(3 * I * d, device=dev, generator=gen, dtype=torch.float32) * 0.02).half())
        w = torch.stack(ws)
        wgu, wdown = w[:, :2 * I * d].contiguous(), w[:, 2 * I * d:].contiguous()
        del w, ws
        gen.manual_seed(7000 + l)
        wd = torch.zeros(pcols * d, device=dev, dtype=torch.float16)
        wd[:(E + 1) * d] = (torch.randn((E + 1) * d, device=dev, generator=gen, dtype=torch.float32) * 0.02).half()
        layers.append((wgu, wdown, wd))
    torch.cuda.synchronize()
    return layers


def stack_parity(torch, cfg, x16, weights, gpu_layer_outputs, layers_checked, mask_rows=256):
    """The first `layers_checked` layers of the stack against the oracle: the oracle takes the GPU's own
    router logits of each layer (so both sides route on bit-identical inputs) and the GPU's fp16
    activations entering that layer; routing is compared on every row, the layer's fp16 output
    RMSNorm(x + moe(x)) on `mask_rows` evenly spaced rows within 2e-2 relative / 2e-3 absolute (the output
    is fp16 with unit RMS: one ulp at |y| ~ 4 is already 2e-3)."""
    from oracle import moe_oracle as O
    O.use_all_cores()
    T, K, E, d, I = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I
    mask = np.zeros(T, np.uint8)
    mask[np.linspace(0, T - 1, mask_rows).astype(np.int64)] = 1
    rows = np.nonzero(mask)[0]
    ok, worst, exact = True, 0.0, True
    for l in range(layers_checked):
        wgu, wdown, _ = weights[l]
        g = gpu_layer_outputs[l]
        ref = O.layer(g["proj"], g["x_in"], wgu.view(torch.int16).cpu().numpy().view(np.uint16).reshape(E, 2 * I, d),
                      wdown.view(torch.int16).cpu().numpy().view(np.uint16).reshape(E, d, I), K, row_mask=mask)
        exact = exact and bool(np.array_equal(g["idx"], ref.idx))
        want = O.residual_rmsnorm(np.ascontiguousarray(g["x_in"][rows]), np.ascontiguousarray(ref.h[rows, 0]), 1e-6)
        a = g["x_out"][rows].view(np.float16).astype(np.float32)
        b = want.view(np.float16).astype(np.float32)
        err = np.abs(a - b)
        worst = max(worst, float(err.max()))
        ok = ok and bool(np.all(err <= 2e-3 + RTOL_OUT * np.abs(b)))
    return {"checked": True, "against": "CPU oracle per layer, on the GPU's logits and input activations of that layer",
            "layers_checked": layers_checked, "rows_checked": int(len(rows)), "bit_exact": exact,
            "outputs_within_2e-2_rel_2e-3_abs": ok, "max_err": worst, "ok": ok and exact}


def run_stack(args, ctx, mc, synth, cfg, stream, local):
    """Config 4 on one GPU: the teacher-forward stack -- `layers` MoE layers of the 30B-A3B shape back to
    back on T=4096 tokens, each with its own seeded weights resident in HBM, each followed by a residual
    add and RMSNorm (eps 1e-6, fused into the combine).  Because the activations change from layer to
    layer, the upstream projection (router logits, src/qwen.c:845) runs on the GPU too, on the grouped
    kernel with one "expert"; it is timed as part of the step.  One step = one pass of the whole stack."""
    import torch

    T, K, E, d, I, NL = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I, cfg.layers
    dev = torch.device("cuda", local)
    pcols = cfg.pstride
    layers = stack_weights(torch, cfg, dev)
    x16 = synth.activations(cfg, 0)
    d_x0 = ctx.upload(x16)
    d_xa, d_xb = ctx.alloc(T * d * 2), ctx.alloc(T * d * 2)
    d_proj = ctx.alloc(T * pcols * 4)
    d_tiles0 = ctx.zeros(T // 128 * 4)
    d_idx = ctx.alloc(T * K * 4)
    h_x, _ = pinned_array(mc, ctx, x16.shape, np.uint16)
    h_y, _ = pinned_array(mc, ctx, x16.shape, np.uint16)
    h_x[:] = x16
    L = mc.lib()

    def stack(host: bool, n_layers=NL, keep=None):
        if host:
            L.moe_cuda_write(ctx.p, d_x0.ptr, h_x.ctypes.data, h_x.nbytes)
        src, dst = d_x0, d_xa
        for l, (wgu, wdown, wd) in enumerate(layers[:n_layers]):
            ctx.mm(src, wd.data_ptr(), d_proj, None, d_tiles0, T, pcols, d, experts_in_B=1)
            ctx.layer(rows=T, d=d, experts=E, topk=K, inter=I, shared=0, pstride=pcols, hc=1, proj=d_proj, x16=src,
                      wgu=wgu.data_ptr(), wdown=wdown.data_ptr(), y16=dst, eps=1e-6, flags=args.flags, idx=d_idx)
            if keep is not None:   # the parity pass: keep what the oracle needs of this layer
                ctx.flush()
                keep.append({"proj": d_proj.read(np.float32, (T, pcols)), "x_in": src.read(np.uint16, (T, d)),
                             "x_out": dst.read(np.uint16, (T, d)), "idx": d_idx.read(np.uint32, (T, K))})
            src, dst = dst, (d_xb if dst is d_xa else d_xa)
        if host:
            L.moe_cuda_read(ctx.p, h_y.ctypes.data, src.ptr, h_y.nbytes)
        return src

    warm = max(args.warmup, 3)
    for _ in range(warm):
        stack(False)
    ctx.flush()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    l0 = ctx.launches()
    ms = timed_steps(torch, stream, lambda: stack(False), args.steps)
    ctx.check()
    launches = ctx.launches() - l0
    e2e_ms = timed_steps(torch, stream, lambda: stack(True), args.steps)
    clocks = sampler.stop()
    last = stack(False)
    ctx.flush()
    y = last.read(np.uint16, (T, d)).view(np.float16).astype(np.float32)
    if args.no_parity:
        parity = {"checked": False}
    else:
        kept = []
        stack(False, n_layers=args.stack_check_layers, keep=kept)
        parity = stack_parity(torch, cfg, x16, layers, kept, args.stack_check_layers)
    pk = peaks()
    flops = NL * (cfg.flops() + 2 * T * pcols * d)
    tf = flops / (ms * 1e-3) / 1e12
    out = {
        "metric": STACK_METRIC,
        "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": dict(workload_config(cfg, 1), layers=NL, weights_resident_GB=round(NL * (E * 3 * d * I * 2) / 1e9, 1)),
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(h_x.nbytes),
                "d2h_bytes_per_step": int(h_y.nbytes), "ms_per_step": e2e_ms},
        "gpu_launches": int(launches), "clocks": clocks, "parity": parity,
        "per_layer_ms": ms / NL, "layer_tokens_per_s": T * NL / (ms * 1e-3),
        "roofline": {"bound": "tensor", "kernel": "whole stack (all kernels)", "achieved": tf,
                     "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops_sustained"],
                     "traffic": None, "peak_source": pk["source"] + " (sustained: a step runs for tens of milliseconds)"},
        "output_rms": float(np.sqrt((y * y).mean())),
    }
    ctx.close()
    emit(args, out, ok=parity.get("ok", True))


def run_stream(args, ctx, mc, synth, cfg, stream, local):
    """The teacher's weight streaming (mda_qwen_prefetch / mda_qwen_upload, src/qwen.c:381-394,1101-1134) for
    `--stream-layers` layers of the stack: the layers' bf16 expert tensors sit in page-locked host memory, the
    device holds two banks, and layer l+1 is uploaded and converted to fp16 in place on a copy stream while layer l
    computes.  Reports the streamed time per layer beside the upload alone and the compute alone, and checks that
    the streamed pass gives bit for bit the output of the same layers run from resident weights."""
    import torch

    T, K, E, d, I = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I
    NL = args.stream_layers
    dev = torch.device("cuda", local)
    pcols = cfg.pstride
    import dataclasses
    layers = stack_weights(torch, dataclasses.replace(cfg, layers=NL), dev)
    L = mc.lib()
    host = []
    for wgu, wdown, wd in layers:   # what the shards hold: bf16
        hg = torch.empty(wgu.numel(), dtype=torch.int16).pin_memory()
        hd = torch.empty(wdown.numel(), dtype=torch.int16).pin_memory()
        hg.copy_(wgu.reshape(-1).float().bfloat16().view(torch.int16))
        hd.copy_(wdown.reshape(-1).float().bfloat16().view(torch.int16))
        host.append((hg, hd))
    # resident fp16 copies of exactly those bf16 values, for the comparison pass
    resident = [(hg.to(dev).view(torch.bfloat16).half(), hd.to(dev).view(torch.bfloat16).half()) for hg, hd in host]
    x16 = synth.activations(cfg, 0)
    d_x0 = ctx.upload(x16)
    d_xa, d_xb = ctx.alloc(T * d * 2), ctx.alloc(T * d * 2)
    d_proj = ctx.alloc(T * pcols * 4)
    d_tiles0 = ctx.zeros(T // 128 * 4)
    banks = [(ctx.alloc(E * 2 * I * d * 2), ctx.alloc(E * d * I * 2)) for _ in range(2)]
    up = mc.Ctx(local)
    s_main = torch.cuda.ExternalStream(ctx.stream(), device=local)
    s_up = torch.cuda.ExternalStream(up.stream(), device=local)
    ev_up = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    bank_used = [False, False]

    def upload(l):
        b = l % 2
        hg, hd = host[l]
        if bank_used[b]:
            s_up.wait_event(ev_done[b])                       # the layer that last used this bank is finished
        L.moe_cuda_write(up.p, banks[b][0].ptr, hg.data_ptr(), hg.numel() * 2)
        L.moe_cuda_bf16_to_f16(up.p, banks[b][0].ptr, mc.PcBf16(hg.numel() // 2))
        L.moe_cuda_write(up.p, banks[b][1].ptr, hd.data_ptr(), hd.numel() * 2)
        L.moe_cuda_bf16_to_f16(up.p, banks[b][1].ptr, mc.PcBf16(hd.numel() // 2))
        ev_up[b].record(s_up)

    def layer(l, src, dst, wgu_ptr, wdown_ptr):
        ctx.mm(src, layers[l][2].data_ptr(), d_proj, None, d_tiles0, T, pcols, d, experts_in_B=1)
        ctx.layer(rows=T, d=d, experts=E, topk=K, inter=I, shared=0, pstride=pcols, hc=1, proj=d_proj, x16=src,
                  wgu=wgu_ptr, wdown=wdown_ptr, y16=dst, eps=1e-6, flags=args.flags)

    def streamed():
        src, dst = d_x0, d_xa
        upload(0)
        for l in range(NL):
            if l + 1 < NL:
                upload(l + 1)                                 # runs under layer l
            s_main.wait_event(ev_up[l % 2])
            layer(l, src, dst, banks[l % 2][0].ptr, banks[l % 2][1].ptr)
            ev_done[l % 2].record(s_main)
            bank_used[l % 2] = True
            src, dst = dst, (d_xb if dst is d_xa else d_xa)
        return src

    def from_resident():
        src, dst = d_x0, d_xa
        for l in range(NL):
            layer(l, src, dst, resident[l][0].data_ptr(), resident[l][1].data_ptr())
            src, dst = dst, (d_xb if dst is d_xa else d_xa)
        return src

    def wall(fn, reps):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            out = fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / reps, out

    ms_stream, last = wall(streamed, args.steps)
    y_stream = last.read(np.uint16, (T, d))
    ms_res, last = wall(from_resident, args.steps)
    y_res = last.read(np.uint16, (T, d))

    def uploads_only():
        for l in range(NL):
            upload(l)
        return None
    bank_used[0] = bank_used[1] = False                      # nothing computes now: the uploads run back to back
    ms_up, _ = wall(uploads_only, args.steps)
    same = bool(np.array_equal(y_stream, y_res))
    bytes_layer = (E * 3 * d * I) * 2
    out = {
        "metric": "teacher-forward MoE layers with weights streamed from page-locked host memory (ms per layer)",
        "value": ms_stream / NL, "unit": "ms/layer", "n_gpus": 1, "steps": args.steps, "warmup": 1, "ms_per_step": ms_stream,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": dict(workload_config(cfg, 1), layers=NL, streamed_bytes_per_layer=bytes_layer),
        "upload_only_ms_per_layer": ms_up / NL, "compute_only_ms_per_layer": ms_res / NL,
        "upload_GB/s": bytes_layer / (ms_up / NL * 1e-3) / 1e9,
        "hidden_ms_per_layer": (ms_up + ms_res - ms_stream) / NL,
        "parity": {"checked": True, "against": "the same layers from resident weights (whose path is checked against the oracle by --config c4)",
                   "bit_exact": same, "ok": same},
    }
    up.close()
    ctx.close()
    emit(args, out, ok=same)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c1", choices=["c0", "c1", "c2", "c3", "c3b", "c4", "kd"])
    ap.add_argument("--ref-tokens", type=int, default=1 << 30, help="tokens per CPU sample/step (default: the whole workload, at most 16384)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline leg")
    ap.add_argument("--no-parity", action="store_true", help="skip the comparison of a step's result with the CPU oracle")
    ap.add_argument("--no-sustained", action="store_true", help="skip the seconds-long run behind the timed steps")
    ap.add_argument("--stack-check-layers", type=int, default=2, help="config c4: leading layers compared with the oracle")
    ap.add_argument("--stream-layers", type=int, default=0, help="config c4 on one GPU: stream this many layers' weights from host memory instead of keeping the stack resident")
    ap.add_argument("--flags", type=int, default=0, help="MOE_LAYER_* flags passed to moe_cuda_layer")
    ap.add_argument("--micro-batches", type=int, default=0, help="expert parallel: token slices per layer (0 = automatic)")
    ap.add_argument("--ep-transfer", type=int, default=0, help="expert parallel: 0 automatic, 1 one row per pair, 2 one row per owning GPU")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
