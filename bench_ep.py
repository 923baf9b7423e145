"""Expert-parallel leg of bench.py (N > 1 GPUs of one box, one rank per GPU).

Weak scaling: every rank brings T=4096 tokens of its own (global batch 4096*N) and owns E/N experts;
rows cross NVLink once per (token, owning GPU) up to 4 GPUs and once per (token, expert) pair beyond."""
from __future__ import annotations

import dataclasses
import json
import time

import numpy as np


def run_ep(args, ctx, mc, synth, cfg, stream, rank, world, local):
    import torch
    import torch.distributed as dist

    from bench import METRIC, ClockSampler, emit, peaks, pinned_array, workload_config

    T, K, E, d, I = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I
    if cfg.S:
        raise SystemExit("the expert-parallel path has no shared expert; use --config c1 / c3 / c3b")
    el = E // world
    gcfg = dataclasses.replace(cfg, T=T * world)
    x16 = synth.activations(gcfg, 0, rank * T, (rank + 1) * T)
    wr, wsg = synth.router_weights(cfg, 0)
    proj = synth.projection(cfg, x16, wr, wsg, synth.zipf_bias(cfg, 0))
    wgu, wdown = synth.expert_weights(cfg, 0, rank * el, (rank + 1) * el)

    uid = [mc.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    ctx.ep_init(uid[0], rank, world, E, K, d, I, T, args.micro_batches, args.ep_transfer)
    per_gpu = args.ep_transfer == 2 or (args.ep_transfer == 0 and world <= 4)
    d_wgu, d_wdown = ctx.upload(wgu), ctx.upload(wdown)
    d_proj, d_x = ctx.upload(proj), ctx.upload(x16)
    d_h = ctx.zeros(T * d * 4)
    d_idx = ctx.alloc(T * K * 4)
    lay = dict(rows=T, d=d, experts=E, topk=K, inter=I, shared=0, pstride=cfg.pstride, hc=1,
               proj=d_proj, x16=d_x, wgu=d_wgu, wdown=d_wdown, h=d_h, idx=d_idx)

    def step():
        ctx.ep_layer(**lay)

    def timed(fn, steps):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(steps):
                fn()
            ev1.record(stream)
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1) / steps], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)   # the slowest rank sets the time
        return float(ms.item())

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    ctx.flush()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    l0 = ctx.launches()
    ms = timed(step, args.steps)
    launches = ctx.launches() - l0
    ctx.check()

    ctx.prof(True)
    stage_ms = {n: 0.0 for n in mc.PROF_STAGES}
    for _ in range(args.steps):
        step()
        for n, v in ctx.prof_read().items():
            stage_ms[n] += v / args.steps
    ctx.prof(False)

    h_proj, _ = pinned_array(mc, ctx, proj.shape, np.float32)
    h_x, _ = pinned_array(mc, ctx, x16.shape, np.uint16)
    h_out, _ = pinned_array(mc, ctx, (T, d), np.float32)
    h_proj[:], h_x[:] = proj, x16
    L = mc.lib()

    def e2e_step():
        L.moe_cuda_write(ctx.p, d_proj.ptr, h_proj.ctypes.data, h_proj.nbytes)
        L.moe_cuda_write(ctx.p, d_x.ptr, h_x.ctypes.data, h_x.nbytes)
        L.moe_cuda_fill(ctx.p, d_h.ptr, T * d * 4, 0)
        step()
        L.moe_cuda_read(ctx.p, h_out.ctypes.data, d_h.ptr, h_out.nbytes)

    for _ in range(warm):
        e2e_step()
    e2e_ms = timed(e2e_step, args.steps)
    ctx.check()
    clocks = sampler.stop()

    idx = d_idx.read(np.uint32, (T, K))
    owner = idx // el
    remote_pairs = int((owner != rank).sum())
    dests = np.zeros((T, world), bool)
    dests[np.arange(T)[:, None], owner] = True          # a row goes once to every GPU owning one of its experts
    dests[:, rank] = False
    rp = torch.tensor([remote_pairs, int(dests.sum())], device="cuda", dtype=torch.float64)
    dist.all_reduce(rp, op=dist.ReduceOp.MAX)
    remote_pairs, remote_rows = int(rp[0].item()), int(rp[1].item())
    ctx.flush()

    if rank == 0:
        pk = peaks()
        nv_peak = 770.0  # GB/s per direction per GPU, measured peer copy on this pool
        gemm1_flops = T * K * 4 * d * I   # per rank: on average every rank receives T*K rows
        tf1 = gemm1_flops / (stage_ms["gate_up"] * 1e-3) / 1e12
        tf2 = (gemm1_flops / 2) / (stage_ms["down"] * 1e-3) / 1e12
        if per_gpu:
            disp_bytes = remote_rows * d * 2 + remote_pairs * 12  # rows once per GPU + 4- and 8-byte records per pair
            ret_bytes = remote_rows * d * 2                       # one fp16 partial row per (token, owning GPU)
        else:
            disp_bytes = ret_bytes = remote_pairs * d * 2         # one row per (token, expert) pair each way
        gbs = lambda b, m: b / (m * 1e-3) / 1e9 if m > 0 else None
        out = {
            "metric": METRIC, "value": T * world / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(cfg, world),
            "e2e": {"value": T * world / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h_proj.nbytes + h_x.nbytes) * world,
                    "d2h_bytes_per_step": int(h_out.nbytes) * world, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "moe_mm_kernel<SWIGLU_F16> (gate_up grouped product), rank 0",
                         "achieved": tf1, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf1 / pk["bf16_tflops"],
                         "traffic": None, "peak_source": pk["source"] + " (burst)",
                         "flops_per_launch": gemm1_flops, "ms_per_launch": stage_ms["gate_up"]},
            "nvlink": {"dispatch_bytes_per_gpu": disp_bytes, "return_bytes_per_gpu": ret_bytes,
                       "dispatch_GB/s": gbs(disp_bytes, stage_ms["scatter"]), "return_GB/s": gbs(ret_bytes, stage_ms["combine"]),
                       "peak_GB/s": nv_peak,
                       "dispatch_frac": gbs(disp_bytes, stage_ms["scatter"]) / nv_peak,
                       "return_frac": gbs(ret_bytes, stage_ms["combine"]) / nv_peak,
                       "transfer": "per GPU" if per_gpu else "per pair",
                       "note": "per GPU: scatter stage = row send (once per destination GPU) + record scatter + barrier, combine stage = peer loads of one partial row per owning GPU (the owner-side partial sums sit in the down stage); per pair: scatter stage = peer-store scatter + barrier, combine stage = peer-load gather"},
            "stages_rank0_ms": {"route": stage_ms["route"], "counts all-gather + plan": stage_ms["scan"],
                                "scatter + dispatch + barrier": stage_ms["scatter"], "gate_up": stage_ms["gate_up"],
                                "down": stage_ms["down"], "barrier": stage_ms["shared"],
                                "combine + return": stage_ms["combine"]},
            "stages_note": {"gate_up_TFLOP/s": tf1, "down_TFLOP/s": tf2},
        }
        emit(args, out)
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()
