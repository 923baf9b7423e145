#!/usr/bin/env python
"""Benchmark of the MoE forward path (route -> scan -> scatter -> grouped SwiGLU products ->
combine) through libmoe_cuda's C ABI.

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference

A step is one pass of one MoE layer of the "30B-A3B" shape (T=4096 tokens per GPU, d=2048, E=128,
top-8, I=768; seeded synthetic fp16 weights and activations).  Rank 0 prints one JSON line.
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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel, the
# gate_up grouped product with row gather, at the 30B-A3B shape, from the Nsight Compute capture
# summarised in profiles/moe_mm_kernel_30B-A3B.md (full-size launch, no scaling involved).
NCU_TRAFFIC_BYTES = {"c1": 883223040 + 58677504}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            m = json.load(f)
        return {"hbm_gbs": float(m["hbm_gbs"]), "bf16_tflops": float(m["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms during the timed region."""
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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def pinned_array(mc, ctx, shape, dtype):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = mc.lib().moe_cuda_alloc_pinned(ctx.p, n)
    ctx.check()
    buf = (ctypes.c_uint8 * n).from_address(p)
    return np.frombuffer(buf, dtype=dtype).reshape(shape), p


def cpu_baseline(cfg, inp, sample_tokens: int, reps: int = 1):
    """Times the CPU oracle on the first `sample_tokens` tokens of the workload (all experts'
    weights resident), on all host threads OpenMP gives it."""
    from oracle import moe_oracle as O
    T = min(sample_tokens, cfg.T)
    proj, x16 = np.ascontiguousarray(inp.proj[:T]), np.ascontiguousarray(inp.x16[:T])
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        O.layer(proj, x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": T / best, "unit": "tokens/s", "cores": O.threads(), "kind": "port",
            "sample": f"first {T} of {cfg.T} tokens of the workload, whole layer on the CPU oracle, best of {reps}",
            "seconds": best}


def run_reference(args):
    """The reference arm: the reference's own implementation of the path is GLSL over Vulkan and
    cannot run on this box, so its scalar C restatement (the oracle) is timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pkg = entry.load_package()
    synth = pkg.synth
    cfg = synth.CONFIGS[args.config]
    inp = synth.layer_inputs(cfg, 0)
    from oracle import moe_oracle as O
    T = min(args.ref_tokens, cfg.T)
    proj, x16 = np.ascontiguousarray(inp.proj[:T]), np.ascontiguousarray(inp.x16[:T])
    for _ in range(args.warmup):
        O.layer(proj, x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.layer(proj, x16, inp.wgu, inp.wdown, cfg.K, inp.wsgu, inp.wsdown)
    dt = (time.perf_counter() - t0) / args.steps
    v = T / dt
    sample = f"each step = first {T} of {cfg.T} tokens of the workload through the whole layer"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(cfg, args.gpus),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": O.threads(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference shaders need Vulkan: unavailable on this box; timed its scalar C restatement",
    }))


def workload_config(cfg, n_gpus):
    return {"workload": f"{cfg.name}: T={cfg.T} tokens per GPU, d={cfg.d}, E={cfg.E}, top-{cfg.K}, I={cfg.I}"
                        + (f", shared S={cfg.S}" if cfg.S else ""),
            "global_tokens": cfg.T * n_gpus,
            "parallelism": "single GPU" if n_gpus == 1 else f"expert-parallel ep{n_gpus}: E/{n_gpus} experts per GPU",
            "l2": "inputs larger than L2: 1.2 GB of expert weights are streamed from HBM every step"}


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
    cfg = synth.CONFIGS[args.config]
    stream = torch.cuda.Stream(device=local)
    ctx = mc.Ctx(local, stream.cuda_stream)
    ctx.check()
    T, K, E, d, I = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I

    if world > 1:
        from bench_ep import run_ep  # noqa: F401  (expert-parallel driver)
        return run_ep(args, ctx, mc, synth, cfg, stream, rank, world, local)

    if cfg.layers > 1:
        return run_stack(args, ctx, mc, synth, cfg, stream, local)

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
    for _ in range(max(args.warmup, 3)):
        step()
    ctx.flush()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ctx.launches()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
    torch.cuda.synchronize()
    ctx.check()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = ctx.launches() - l0

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

    e2e_run(max(args.warmup, 3) + 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_run(args.steps)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps   # wall clock between synchronisations: two streams
    for ln in lanes:
        ln["ctx"].check()
        assert np.array_equal(lanes[0]["ho"], ln["ho"]), "the end-to-end lanes disagree"
    clocks = sampler.stop()

    pk = peaks()
    gemm1_flops = T * K * 4 * d * I          # gate_up product, unpadded
    gemm2_flops = T * K * 2 * d * I
    tf1 = gemm1_flops / (stage_ms["gate_up"] * 1e-3) / 1e12
    tf2 = gemm2_flops / (stage_ms["down"] * 1e-3) / 1e12
    scatter_bytes = 2 * T * K * d * 2 + T * K * 8
    combine_bytes = T * K * d * 2 + T * K * 8 + 2 * T * d * 4   # expert outputs are kept fp16 in the fused layer
    route_bytes = T * E * 4 + T * K * 8 + E * 4
    gbs = lambda b, m: b / (m * 1e-3) / 1e9 if m > 0 else None
    stages = {
        "route": {"ms": stage_ms["route"], "GB/s": gbs(route_bytes, stage_ms["route"])},
        "scan": {"ms": stage_ms["scan"]},
        "scatter": ({"ms": stage_ms["scatter"], "GB/s": gbs(scatter_bytes, stage_ms["scatter"]),
                     "frac_hbm": gbs(scatter_bytes, stage_ms["scatter"]) / pk["hbm_gbs"]}
                    if args.flags & mc.LAYER_MATERIALIZE_XP else
                    {"ms": stage_ms["scatter"], "note": "ranks and slot tables only; the gate_up product gathers the rows"}),
        "gate_up": {"ms": stage_ms["gate_up"], "TFLOP/s": tf1, "frac_tensor": tf1 / pk["bf16_tflops"],
                    "weight_GB/s": gbs(E * 2 * I * d * 2, stage_ms["gate_up"])},
        "down": {"ms": stage_ms["down"], "TFLOP/s": tf2, "frac_tensor": tf2 / pk["bf16_tflops"],
                 "weight_GB/s": gbs(E * I * d * 2, stage_ms["down"])},
        "combine": {"ms": stage_ms["combine"], "GB/s": gbs(combine_bytes, stage_ms["combine"]),
                    "frac_hbm": gbs(combine_bytes, stage_ms["combine"]) / pk["hbm_gbs"]},
    }
    if cfg.S:
        stages["shared"] = {"ms": stage_ms["shared"]}
    out = {
        "metric": METRIC, "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(cfg, 1),
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(h_proj.nbytes + h_x.nbytes),
                "d2h_bytes_per_step": int(h_out.nbytes), "ms_per_step": e2e_ms,
                "how": "three contexts take steps in turn so copies overlap kernels; wall clock between device synchronisations"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "moe_mm_kernel<SWIGLU_F16, GATHER> (gate_up grouped product, row gather + SwiGLU fused)",
                     "achieved": tf1, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf1 / pk["bf16_tflops"],
                     "traffic": NCU_TRAFFIC_BYTES.get(args.config) if args.flags == 0 else None, "peak_source": pk["source"] + " (burst)",
                     "flops_per_launch": gemm1_flops, "ms_per_launch": stage_ms["gate_up"]},
        "stages": stages,
    }
    if not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(cfg, inp, args.ref_tokens)
    for cx in extra:
        cx.close()
    ctx.close()
    emit(args, out)


def emit(args, out):
    """Print the result line on the process's original stdout."""
    sys.stdout.flush()
    os.dup2(args.real_stdout, 1)
    print(json.dumps(out), flush=True)


def run_stack(args, ctx, mc, synth, cfg, stream, local):
    """Config 4: the teacher-forward stack -- `layers` MoE layers of the 30B-A3B shape back to back
    on T=4096 tokens, each with its own seeded weights resident in HBM, each followed by a residual
    add and RMSNorm (eps 1e-6, fused into the combine).  Because the activations change from layer
    to layer, the upstream projection (router logits, src/qwen.c:845) runs on the GPU too, on the
    grouped kernel with one "expert"; it is timed as part of the step.  One step = one pass of the
    whole stack."""
    import torch

    T, K, E, d, I, NL = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I, cfg.layers
    dev = torch.device("cuda", local)
    pcols = cfg.pstride
    gen = torch.Generator(device=dev)
    layers = []
    for l in range(NL):   # seeded per layer; generated on the device (58 GB of fp16 in all)
        gen.manual_seed(1000 + l)
        wgu = (torch.randn(E * 2 * I * d, device=dev, generator=gen, dtype=torch.float32) * 0.02).half()
        wdown = (torch.randn(E * d * I, device=dev, generator=gen, dtype=torch.float32) * 0.02).half()
        wd = torch.zeros(pcols * d, device=dev, dtype=torch.float16)
        wd[:(E + 1) * d] = (torch.randn((E + 1) * d, device=dev, generator=gen, dtype=torch.float32) * 0.02).half()
        layers.append((wgu, wdown, wd))
    torch.cuda.synchronize()
    x16 = synth.activations(cfg, 0)
    d_x0 = ctx.upload(x16)
    d_xa, d_xb = ctx.alloc(T * d * 2), ctx.alloc(T * d * 2)
    d_proj = ctx.alloc(T * pcols * 4)
    d_tiles0 = ctx.zeros(T // 128 * 4)
    h_x, _ = pinned_array(mc, ctx, x16.shape, np.uint16)
    h_y, _ = pinned_array(mc, ctx, x16.shape, np.uint16)
    h_x[:] = x16
    L = mc.lib()

    def stack(host: bool):
        if host:
            L.moe_cuda_write(ctx.p, d_x0.ptr, h_x.ctypes.data, h_x.nbytes)
        src, dst = d_x0, d_xa
        for wgu, wdown, wd in layers:
            ctx.mm(src, wd.data_ptr(), d_proj, None, d_tiles0, T, pcols, d, experts_in_B=1)
            ctx.layer(rows=T, d=d, experts=E, topk=K, inter=I, shared=0, pstride=pcols, hc=1, proj=d_proj, x16=src,
                      wgu=wgu.data_ptr(), wdown=wdown.data_ptr(), y16=dst, eps=1e-6, flags=args.flags)
            src, dst = dst, (d_xb if dst is d_xa else d_xa)
        if host:
            L.moe_cuda_read(ctx.p, h_y.ctypes.data, src.ptr, h_y.nbytes)
        return src

    for _ in range(max(args.warmup, 3)):
        stack(False)
    ctx.flush()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ctx.launches()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            last = stack(False)
        ev1.record(stream)
    torch.cuda.synchronize()
    ctx.check()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = ctx.launches() - l0
    with torch.cuda.stream(stream):
        ev0.record(stream)
        for _ in range(args.steps):
            stack(True)
        ev1.record(stream)
    torch.cuda.synchronize()
    e2e_ms = ev0.elapsed_time(ev1) / args.steps
    clocks = sampler.stop()
    y = last.read(np.uint16, (T, d)).view(np.float16).astype(np.float32)
    pk = peaks()
    flops = NL * (cfg.flops() + 2 * T * pcols * d)
    out = {
        "metric": "teacher-forward MoE stack tokens/s (48 x [projection -> route -> grouped GEMM -> combine -> residual + RMSNorm])",
        "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": dict(workload_config(cfg, 1), layers=NL, weights_resident_GB=round(NL * (E * 3 * d * I * 2) / 1e9, 1)),
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(h_x.nbytes),
                "d2h_bytes_per_step": int(h_y.nbytes), "ms_per_step": e2e_ms},
        "gpu_launches": int(launches), "clocks": clocks,
        "per_layer_ms": ms / NL, "layer_tokens_per_s": T * NL / (ms * 1e-3),
        "roofline": {"bound": "tensor", "kernel": "whole stack (all kernels)", "achieved": flops / (ms * 1e-3) / 1e12,
                     "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"],
                     "traffic": None, "peak_source": pk["source"] + " (burst)"},
        "output_rms": float(np.sqrt((y * y).mean())),
    }
    ctx.close()
    emit(args, out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c1", choices=["c0", "c1", "c2", "c3", "c3b", "c4"])
    ap.add_argument("--ref-tokens", type=int, default=1 << 30, help="tokens per CPU sample/step (default: the whole workload)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
