"""Expert-parallel leg of bench.py (N > 1 GPUs of one box, one rank per GPU).

Weak scaling: every rank brings T=4096 tokens of its own (global batch 4096*N) and owns E/N experts;
rows cross NVLink once per (token, owning GPU) up to 4 GPUs and once per (token, expert) pair beyond.
Config c4 runs the 48-layer stack the same way (per-layer weights sharded E/N per rank, residual +
RMSNorm fused into the expert-parallel combine).  Rank 0 checks one step of every rank against the CPU
oracle's single-device layer on the global batch before it prints the line."""
from __future__ import annotations

import dataclasses
import time

import numpy as np


def peer_copy_peak(torch, dist, local, world, mbytes=256, reps=5):
    """GB/s per direction and GPU of plain peer copies while every rank copies to its right-hand
    neighbour at once (cudaMemcpyPeer under torch's copy_), CUDA events, best of `reps`.  It is the
    denominator of the NVLink fractions: measured in this run, not assumed."""
    n = mbytes << 20
    peer = (local + 1) % world
    src = torch.empty(n, dtype=torch.uint8, device=f"cuda:{local}")
    dst = torch.empty(n, dtype=torch.uint8, device=f"cuda:{peer}")
    dst.copy_(src)
    torch.cuda.synchronize(local)
    torch.cuda.synchronize(peer)
    best = None
    for _ in range(reps):
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize(local)
        torch.cuda.synchronize(peer)
        ms = e0.elapsed_time(e1)
        best = ms if best is None else min(best, ms)
    del src, dst
    t = torch.tensor([n / (best * 1e-3) / 1e9], device=f"cuda:{local}")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)   # the slowest pair
    return float(t.item())


def gather_rows(torch, dist, a: np.ndarray, local):
    """All ranks' copies of a per-rank array, stacked along axis 0, on every rank."""
    t = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1)).to(f"cuda:{local}")
    out = torch.empty(t.numel() * dist.get_world_size(), dtype=torch.uint8, device=f"cuda:{local}")
    dist.all_gather_into_tensor(out, t)
    return out.cpu().numpy().view(a.dtype).reshape((-1,) + a.shape[1:])


def ep_parity(torch, dist, local, rank, world, cfg, synth, O, got, eff_mb, rows_per_rank=256):
    """One step of every rank against the oracle's single-device layer on the global batch.  Rank 0
    regenerates the global inputs and all experts' weights (every tensor is a function of its seed and
    row), routes / scans / scatters every token and runs the products for `rows_per_rank` evenly spaced
    tokens of each rank.  Expert indices, router weights and the permutation (rows inside the owning
    rank's buffer of the token's slice) are compared for every token of every rank."""
    from bench import ATOL_OUT, RTOL_OUT, RTOL_WT
    pkg_ep = __import__("__graft_entry__").load_package().ep_plan
    T, K, E, d = cfg.T, cfg.K, cfg.E, cfg.d
    sel = np.linspace(0, T - 1, rows_per_rank).astype(np.int64)
    idx_all = gather_rows(torch, dist, got["idx"], local).reshape(world, T, K)
    slot_all = gather_rows(torch, dist, got["slot"], local).reshape(world, T, K)
    wt_all = gather_rows(torch, dist, got["wt"], local).reshape(world, T, K)
    h_all = gather_rows(torch, dist, np.ascontiguousarray(got["h"][sel]), local).reshape(world, rows_per_rank, d)
    rep = None
    if rank == 0:
        O.use_all_cores()
        gcfg = dataclasses.replace(cfg, T=T * world)
        inp = synth.layer_inputs(gcfg, 0)
        mask = np.zeros(T * world, np.uint8)
        for r in range(world):
            mask[r * T + sel] = 1
        ref = O.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, K, inp.wsgu, inp.wsdown, row_mask=mask)
        ridx = ref.idx.reshape(world, T, K)
        exact_idx = bool(np.array_equal(idx_all, ridx))
        wt_ok = bool(np.all(np.abs(wt_all - ref.wt.reshape(world, T, K)) <= RTOL_WT * np.abs(ref.wt.reshape(world, T, K))))
        exact_slot = True
        for r in range(world):
            want = np.empty((T, K), np.int64)
            for a, b in pkg_ep.slices(T, eff_mb):
                cnt_m = np.stack([np.bincount(ridx[q, a:b].ravel(), minlength=E) for q in range(world)]).astype(np.uint32)
                dst_off = pkg_ep.plan(cnt_m, r)[0]
                mine = ridx[r, a:b]
                want[a:b] = dst_off[mine].astype(np.int64) + pkg_ep.local_ranks(mine)
            exact_slot = exact_slot and bool(np.array_equal(slot_all[r], want))
        rh = np.stack([ref.h[r * T + sel, 0] for r in range(world)])
        err = np.abs(h_all - rh)
        out_ok = bool(np.all(err <= ATOL_OUT + RTOL_OUT * np.abs(rh)))
        rep = {"checked": True, "against": "CPU oracle, single-device layer on the global batch", "bit_exact": exact_idx and exact_slot,
               "bit_exact_fields": {"idx": exact_idx, "slot": exact_slot}, "router_weights_within_1e-5": wt_ok,
               "outputs_within_2e-2_rel_1e-3_abs": out_ok, "max_err": float(err.max()), "max_abs_ref": float(np.abs(rh).max()),
               "rows_checked": int(world * rows_per_rank), "tokens_routed_and_placed": int(world * T), "ranks": world,
               "ok": exact_idx and exact_slot and wt_ok and out_ok}
    dist.barrier()
    return rep


class HostPipe:
    """End-to-end steps with host buffers for one rank: uploads and downloads run on two copy streams
    (two plain contexts of the library) around the expert-parallel context's stream, over three sets of
    device buffers, so that step i+1's inputs go up and step i-1's result comes down while step i
    computes.  Only copies wait on copies; the layer's cross-GPU waits stay on the layer's stream."""

    DEPTH = 3   # sets of device and host buffers: a step's download may still run while the next two steps compute

    def __init__(self, torch, mc, ctx, local, make_step, in_arrays, out_bytes):
        self.torch, self.mc, self.ctx, self.L = torch, mc, ctx, mc.lib()
        self.s_main = torch.cuda.ExternalStream(ctx.stream(), device=local)
        self.up, self.down = mc.Ctx(local), mc.Ctx(local)
        self.s_up = torch.cuda.ExternalStream(self.up.stream(), device=local)
        self.s_down = torch.cuda.ExternalStream(self.down.stream(), device=local)
        import bench
        self.sets = []
        for _ in range(self.DEPTH):
            host_in, dev_in = [], []
            for a in in_arrays:
                h, _ = bench.pinned_array(mc, ctx, a.shape, a.dtype)
                h[:] = a
                host_in.append(h)
                dev_in.append(ctx.alloc(a.nbytes))
            host_out, _ = bench.pinned_array(mc, ctx, (out_bytes,), np.uint8)
            dev_out = ctx.alloc(out_bytes)
            ev = {n: torch.cuda.Event() for n in ("up", "layer", "down")}
            self.sets.append(dict(host_in=host_in, dev_in=dev_in, host_out=host_out, dev_out=dev_out, ev=ev, used=False))
        self.step_fns = [make_step(s["dev_in"], s["dev_out"]) for s in self.sets]
        self.h2d = sum(a.nbytes for a in in_arrays)
        self.d2h = out_bytes

    def issue(self, i):
        s = self.sets[i % self.DEPTH]
        L, ev = self.L, s["ev"]
        if s["used"]:
            self.s_up.wait_event(ev["layer"])       # the layer that last read these inputs is done
        for h, dbuf in zip(s["host_in"], s["dev_in"]):
            L.moe_cuda_write(self.up.p, dbuf.ptr, h.ctypes.data, h.nbytes)
        ev["up"].record(self.s_up)
        self.s_main.wait_event(ev["up"])
        if s["used"]:
            self.s_main.wait_event(ev["down"])      # the previous result of this set is on the host
        self.step_fns[i % self.DEPTH]()
        ev["layer"].record(self.s_main)
        self.s_down.wait_event(ev["layer"])
        L.moe_cuda_read_async(self.down.p, s["host_out"].ctypes.data, s["dev_out"].ptr, self.d2h)
        ev["down"].record(self.s_down)
        s["used"] = True

    def run(self, n):
        for i in range(n):
            self.issue(i)
        self.up.flush()
        self.ctx.flush()
        self.down.flush()

    def close(self):
        self.up.close()
        self.down.close()


def run_ep(args, ctx, mc, synth, cfg, stream, rank, world, local):
    import torch
    import torch.distributed as dist

    import bench
    from bench import METRIC, ClockSampler, emit, peaks, workload_config
    from oracle import moe_oracle as O

    T, K, E, d, I, S, NL = cfg.T, cfg.K, cfg.E, cfg.d, cfg.I, cfg.S, cfg.layers
    el = E // world
    dev = torch.device("cuda", local)
    pcols = cfg.pstride
    gcfg = dataclasses.replace(cfg, T=T * world)
    x16 = synth.activations(gcfg, 0, rank * T, (rank + 1) * T)
    stack = NL > 1

    uid = [mc.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    ctx.ep_init(uid[0], rank, world, E, K, d, I, T, args.micro_batches, args.ep_transfer)
    per_gpu = args.ep_transfer == 2 or (args.ep_transfer == 0 and world <= 4)
    eff_mb = args.micro_batches if args.micro_batches else (2 if (world >= 4 and not per_gpu) else 1)
    d_idx, d_slot, d_wt = ctx.alloc(T * K * 4), ctx.alloc(T * K * 4), ctx.alloc(T * K * 4)

    if not stack:
        wr, wsg = synth.router_weights(cfg, 0)
        proj = synth.projection(cfg, x16, wr, wsg, synth.zipf_bias(cfg, 0))
        wgu, wdown = synth.expert_weights(cfg, 0, rank * el, (rank + 1) * el)
        wsgu, wsdown = synth.shared_weights(cfg, 0)
        d_wgu, d_wdown = ctx.upload(wgu), ctx.upload(wdown)
        d_wsgu = ctx.upload(wsgu) if S else None
        d_wsdown = ctx.upload(wsdown) if S else None
        d_proj, d_x = ctx.upload(proj), ctx.upload(x16)
        d_h = ctx.zeros(T * d * 4)
        in_arrays, out_bytes = [proj, x16], T * d * 4

        def make_step(dev_in, dev_out, outs=None):
            lay = dict(rows=T, d=d, experts=E, topk=K, inter=I, shared=S, pstride=pcols, hc=1, proj=dev_in[0], x16=dev_in[1],
                       wgu=d_wgu, wdown=d_wdown, wsgu=d_wsgu, wsdown=d_wsdown, h=dev_out, idx=d_idx)
            lay.update(outs or {})
            return lambda: ctx.ep_layer(**lay)

        step = make_step([d_proj, d_x], d_h)

        def make_host_step(dev_in, dev_out):
            inner = make_step(dev_in, dev_out)

            def f():
                mc.lib().moe_cuda_fill(ctx.p, dev_out.ptr, T * d * 4, 0)
                inner()
            return f
        flops_step = cfg.flops()
    else:
        # config 4: per-layer weights of this rank's experts, router rows replicated; x <- RMSNorm(x + moe(x))
        layers = bench.stack_weights(torch, cfg, dev, rank * el, (rank + 1) * el)
        d_x = ctx.upload(x16)
        d_xa, d_xb = ctx.alloc(T * d * 2), ctx.alloc(T * d * 2)
        d_proj = ctx.alloc(T * pcols * 4)
        d_tiles0 = ctx.zeros((T + 127) // 128 * 4)
        in_arrays, out_bytes = [x16], T * d * 2
        last = {}

        def make_step(dev_in, dev_out, outs=None, n_layers=NL, keep=None):
            def f():
                src, dst = dev_in[0], d_xa
                for l, (wgu_l, wdown_l, wd) in enumerate(layers[:n_layers]):
                    ctx.mm(src, wd.data_ptr(), d_proj, None, d_tiles0, T, pcols, d, experts_in_B=1)   # router logits, src/qwen.c:845
                    final = l == n_layers - 1 and dev_out is not None
                    out_l = dev_out if final else dst
                    lay = dict(rows=T, d=d, experts=E, topk=K, inter=I, shared=0, pstride=pcols, hc=1, proj=d_proj, x16=src,
                               wgu=wgu_l.data_ptr(), wdown=wdown_l.data_ptr(), y16=out_l, eps=1e-6, idx=d_idx)
                    lay.update(outs or {})
                    ctx.ep_layer(**lay)
                    if keep is not None:
                        ctx.flush()
                        keep.append({"proj": d_proj.read(np.float32, (T, pcols)), "x_in": src.read(np.uint16, (T, d)),
                                     "x_out": out_l.read(np.uint16, (T, d)), "idx": outs["idx"].read(np.uint32, (T, K))})
                    src, dst = out_l, (d_xb if dst is d_xa else d_xa)
                last["buf"] = src
            return f

        d_y = ctx.alloc(T * d * 2)
        step = make_step([d_x], d_y)
        make_host_step = make_step
        flops_step = NL * (cfg.flops() + 2 * T * pcols * d)

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
    clocks = sampler.stop()

    # ---- one more step, checked against the CPU oracle on the global batch ----
    outs = dict(idx=d_idx, slot=d_slot, wt=d_wt)
    if args.no_parity:
        parity = {"checked": False}
    elif not stack:
        d_h.fill(0)
        make_step([d_proj, d_x], d_h, outs)()
        ctx.flush()
        got = {"idx": d_idx.read(np.uint32, (T, K)), "slot": d_slot.read(np.uint32, (T, K)), "wt": d_wt.read(np.float32, (T, K)),
               "h": d_h.read(np.float32, (T, d))}
        parity = ep_parity(torch, dist, local, rank, world, cfg, synth, O, got, eff_mb)
    else:
        kept = []
        nl = args.stack_check_layers
        make_step([d_x], d_y, outs, n_layers=nl, keep=kept)()
        sel = np.linspace(0, T - 1, 256).astype(np.int64)
        parity = None
        ok_all, exact_all, worst = True, True, 0.0
        wcfg = dataclasses.replace(cfg, layers=nl)
        full_w = bench.stack_weights(torch, wcfg, dev) if rank == 0 else None
        for l in range(nl):
            g = kept[l]
            proj_g = gather_rows(torch, dist, g["proj"], local)
            xin_g = gather_rows(torch, dist, g["x_in"], local)
            idx_g = gather_rows(torch, dist, g["idx"], local)
            xout_g = gather_rows(torch, dist, np.ascontiguousarray(g["x_out"][sel]), local).reshape(world, 256, d)
            if rank == 0:
                O.use_all_cores()
                mask = np.zeros(T * world, np.uint8)
                rows = np.concatenate([r * T + sel for r in range(world)])
                mask[rows] = 1
                wgu_l, wdown_l, _ = full_w[l]
                ref = O.layer(proj_g, xin_g, wgu_l.view(torch.int16).cpu().numpy().view(np.uint16).reshape(E, 2 * I, d),
                              wdown_l.view(torch.int16).cpu().numpy().view(np.uint16).reshape(E, d, I), K, row_mask=mask)
                exact_all = exact_all and bool(np.array_equal(idx_g, ref.idx))
                want = O.residual_rmsnorm(np.ascontiguousarray(xin_g[rows]), np.ascontiguousarray(ref.h[rows, 0]), 1e-6)
                a = xout_g.reshape(-1, d).view(np.float16).astype(np.float32)
                b = want.view(np.float16).astype(np.float32)
                err = np.abs(a - b)
                worst = max(worst, float(err.max()))
                ok_all = ok_all and bool(np.all(err <= 2e-3 + bench.RTOL_OUT * np.abs(b)))
        del full_w
        if rank == 0:
            parity = {"checked": True, "against": "CPU oracle per layer on the global batch, on the GPUs' logits and input activations of that layer",
                      "layers_checked": nl, "rows_checked": int(world * 256), "tokens_routed": int(world * T), "bit_exact": exact_all,
                      "outputs_within_2e-2_rel_2e-3_abs": ok_all, "max_err": worst, "ranks": world, "ok": ok_all and exact_all}
        dist.barrier()

    # ---- per-stage device times: every token slice timed on its own stream, the slices added up ----
    stage_ms = {n: 0.0 for n in mc.PROF_STAGES}
    if not stack:
        ctx.prof(True)
        for _ in range(args.steps):
            step()
            for n, v in ctx.prof_read().items():
                stage_ms[n] += v / args.steps
        ctx.prof(False)

    # ---- end to end with host buffers: uploads and downloads on copy streams around the layer ----
    pipe = HostPipe(torch, mc, ctx, local, make_host_step, in_arrays, out_bytes)
    pipe.run(warm + 1)
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    pipe.run(args.steps)
    torch.cuda.synchronize()
    e2e_local = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([e2e_local], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    ctx.check()
    e2e_same = None
    if not stack and not args.no_parity:
        a = np.frombuffer(pipe.sets[0]["host_out"], dtype=np.float32).reshape(T, d)
        e2e_same = bool(np.array_equal(a, got["h"]))
    pipe.close()

    # ---- the same step for a few seconds (sustained clocks) ----
    sustained = None
    if not args.no_sustained:
        n = max(20, int(2.5e3 / max(ms, 1e-3)))
        step()
        s2 = ClockSampler(local)
        s2.start()
        time.sleep(0.3)
        sms = timed(step, n)
        c2 = s2.stop()
        pk0 = peaks()
        tf = flops_step / (sms * 1e-3) / 1e12   # per rank: on average every rank multiplies T*K rows
        sustained = {"tokens_per_s": T * world / (sms * 1e-3), "ms_per_step": sms, "steps": n, "seconds": n * sms * 1e-3,
                     "sm_mhz_median": c2["sm_mhz"], "power_w_max": c2.get("power_w_max"), "reasons": c2["reasons"],
                     "TFLOP/s_all_kernels_per_gpu": tf, "frac_of_sustained_peak": tf / pk0["bf16_tflops_sustained"],
                     "sustained_peak_TFLOP/s": pk0["bf16_tflops_sustained"]}

    nv_peak = peer_copy_peak(torch, dist, local, world)

    idx = d_idx.read(np.uint32, (T, K))   # every step leaves its expert indices here
    owner = idx // el
    remote_pairs = int((owner != rank).sum())
    dests = np.zeros((T, world), bool)
    dests[np.arange(T)[:, None], np.minimum(owner, world - 1)] = True   # a row goes once to every GPU owning one of its experts
    dests[:, rank] = False
    rp = torch.tensor([remote_pairs, int(dests.sum())], device="cuda", dtype=torch.float64)
    dist.all_reduce(rp, op=dist.ReduceOp.MAX)
    remote_pairs, remote_rows = int(rp[0].item()), int(rp[1].item())
    ctx.flush()

    if rank == 0:
        pk = peaks()
        gbs = lambda b, m: b / (m * 1e-3) / 1e9 if m > 0 else None
        out = {
            "metric": METRIC if not stack else bench.STACK_METRIC,
            "value": T * world / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(cfg, world),
            "e2e": {"value": T * world / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(pipe.h2d) * world, "d2h_bytes_per_step": int(pipe.d2h) * world, "ms_per_step": e2e_ms,
                    "how": "per rank: two copy streams around the layer's stream, three sets of device buffers, pinned host memory; wall clock between device synchronisations, slowest rank",
                    "result_equals_checked_result": e2e_same},
            "gpu_launches": int(launches), "clocks": clocks, "parity": parity,
            "micro_batches": eff_mb, "transfer": "per GPU" if per_gpu else "per pair",
        }
        if stack:
            tf = flops_step / (ms * 1e-3) / 1e12
            out["per_layer_ms"] = ms / NL
            out["layer_tokens_per_s"] = T * world * NL / (ms * 1e-3)
            out["roofline"] = {"bound": "tensor", "kernel": "whole stack, all kernels of rank 0's GPU", "achieved": tf,
                               "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": tf / pk["bf16_tflops_sustained"],
                               "traffic": None, "peak_source": pk["source"] + " (sustained: a step runs for tens of milliseconds)"}
        else:
            gemm1_flops = T * K * 4 * d * I   # per rank: on average every rank receives T*K rows
            tf1 = gemm1_flops / (stage_ms["gate_up"] * 1e-3) / 1e12
            tf2 = (gemm1_flops / 2) / (stage_ms["down"] * 1e-3) / 1e12
            if per_gpu:
                disp_bytes = remote_rows * d * 2 + remote_pairs * 12  # rows once per GPU + 4- and 8-byte records per pair
                ret_bytes = remote_rows * d * 2                       # one fp16 partial row per (token, owning GPU)
            else:
                disp_bytes = ret_bytes = remote_pairs * d * 2         # one row per (token, expert) pair each way
            gu_kernel = ("moe_mm_kernel<SWIGLU_F16, GATHER> (gate_up grouped product over the received rows, 128-row tiles), rank 0" if per_gpu
                         else "moe_mm_ws_kernel<SWIGLU_F16, pair> (gate_up grouped product over chunks of the received rows), rank 0")
            out["roofline"] = {"bound": "tensor", "kernel": gu_kernel,
                               "achieved": tf1, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": tf1 / pk["bf16_tflops"],
                               "traffic": None, "peak_source": pk["source"] + " (burst)",
                               "flops_per_launch": gemm1_flops / eff_mb, "launches_per_step": eff_mb, "ms_per_step_all_launches": stage_ms["gate_up"]}
            out["nvlink"] = {"dispatch_bytes_per_gpu": disp_bytes, "return_bytes_per_gpu": ret_bytes,
                             "dispatch_GB/s": gbs(disp_bytes, stage_ms["scatter"]), "return_GB/s": gbs(ret_bytes, stage_ms["combine"]),
                             "peak_GB/s": nv_peak, "peak_source": "measured in this run: every rank copies 256 MB to its neighbour at once (peer copy, CUDA events, slowest pair, best of 5)",
                             "dispatch_frac": gbs(disp_bytes, stage_ms["scatter"]) / nv_peak,
                             "return_frac": gbs(ret_bytes, stage_ms["combine"]) / nv_peak,
                             "note": "stage times hold the local copies, the record scatter and the wait for the slowest rank as well; with several token slices a slice's transfer shares the GPU with another slice's products"}
            out["stages_rank0_ms"] = {"route": stage_ms["route"], "counts exchange + plan": stage_ms["scan"],
                                      "dispatch + barrier" + (" + shared expert" if S else ""): stage_ms["scatter"], "gate_up": stage_ms["gate_up"],
                                      "down" + (" + partial sums" if per_gpu else ""): stage_ms["down"], "barrier": stage_ms["shared"],
                                      "combine + return": stage_ms["combine"]}
            out["stages_cover"] = f"sum over the {eff_mb} token slice(s), each timed on its own stream"
            out["stages_note"] = {"gate_up_TFLOP/s": tf1, "down_TFLOP/s": tf2}
        if sustained is not None:
            out["sustained"] = sustained
        emit(args, out, ok=(parity or {}).get("ok", True))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()
