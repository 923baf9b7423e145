"""Run under torch.distributed.run with one rank per GPU: the expert-parallel layer
(moe_cuda_ep_layer) against the CPU oracle's single-device layer on the whole batch.
Prints "EP_CHECK_OK <world>" on rank 0 when every rank agrees."""
import dataclasses
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    mc, synth, epp = pkg.moe_cuda, pkg.synth, pkg.ep_plan
    ok = True
    cache = {}
    # transfer 1: one row per (token, expert) pair each way; 2: one row per (token, owning GPU)
    # (tokens per rank, E, K, d, I, shared S, Zipf beta, token slices, transfer)
    for T_local, E, K, d, I, S, beta, nmb, transfer in [
            (300, 32, 4, 512, 256, 0, 0.0, 1, 1), (300, 32, 4, 512, 256, 0, 0.0, 2, 1),
            (300, 32, 4, 512, 256, 0, 0.0, 1, 2), (300, 32, 4, 512, 256, 0, 0.0, 2, 2),
            (300, 32, 4, 512, 256, 0, 0.0, 4, 1), (300, 32, 4, 512, 256, 128, 0.0, 3, 1), (300, 32, 4, 512, 256, 128, 0.0, 1, 2),
            (1024, 128, 8, 2048, 768, 0, 1.0, 0, 1), (1024, 128, 8, 2048, 768, 0, 1.0, 2, 2), (1024, 128, 8, 2048, 768, 0, 1.0, 0, 0),
            (1024, 128, 8, 2048, 768, 256, 0.0, 4, 1)]:
        key = (T_local, E, K, d, I, S, beta)
        if key not in cache:
            cfg = dataclasses.replace(synth.CONFIGS["c1"], T=T_local * world, E=E, K=K, d=d, I=I, S=S, zipf_beta=beta)
            inp = synth.layer_inputs(cfg, 7)
            cache = {key: (cfg, inp, O.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, K, inp.wsgu, inp.wsdown))}
        cfg, inp, full = cache[key]
        el = E // world
        lo, hi = rank * T_local, (rank + 1) * T_local
        uid = [mc.ep_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        per_gpu = transfer == 2 or (transfer == 0 and world <= 4)
        eff_mb = nmb if nmb else (2 if (world >= 4 and not per_gpu) else 1)   # the library's automatic choice
        # expected rows: inside the owner's buffer of the token's micro-batch, rows of an expert are ordered
        # (source rank, token) -- the single-device order restricted to that micro-batch
        want = np.empty((T_local, K), np.int64)
        for m, (a, b) in enumerate(epp.slices(T_local, eff_mb)):
            cnt_m = np.stack([np.bincount(full.idx[r * T_local + a:r * T_local + b].ravel(), minlength=E)
                              for r in range(world)]).astype(np.uint32)
            dst_off = epp.plan(cnt_m, rank)[0]
            mine = full.idx[lo + a:lo + b]
            want[a:b] = dst_off[mine].astype(np.int64) + epp.local_ranks(mine)
        with mc.Ctx(local) as ctx:
            ctx.ep_init(uid[0], rank, world, E, K, d, I, T_local, nmb, transfer)
            d_proj, d_x = ctx.upload(np.ascontiguousarray(inp.proj[lo:hi])), ctx.upload(np.ascontiguousarray(inp.x16[lo:hi]))
            d_wgu = ctx.upload(np.ascontiguousarray(inp.wgu[rank * el:(rank + 1) * el]))
            d_wdown = ctx.upload(np.ascontiguousarray(inp.wdown[rank * el:(rank + 1) * el]))
            d_wsgu = ctx.upload(inp.wsgu) if S else None
            d_wsdown = ctx.upload(inp.wsdown) if S else None
            d_idx, d_slot, d_wt = ctx.alloc(T_local * K * 4), ctx.alloc(T_local * K * 4), ctx.alloc(T_local * K * 4)
            for rep in range(2):    # the second pass reuses the peer buffers
                d_h = ctx.zeros(T_local * d * 4)
                ctx.ep_layer(rows=T_local, d=d, experts=E, topk=K, inter=I, shared=S, pstride=cfg.pstride, hc=1,
                             proj=d_proj, x16=d_x, wgu=d_wgu, wdown=d_wdown, wsgu=d_wsgu, wsdown=d_wsdown, h=d_h, idx=d_idx,
                             slot=d_slot, wt=d_wt)
                ctx.flush()
                idx = d_idx.read(np.uint32, (T_local, K))
                slot = d_slot.read(np.uint32, (T_local, K))
                h = d_h.read(np.float32, (T_local, d))
                err = np.abs(h - full.h[lo:hi, 0])
                good = (np.array_equal(idx, full.idx[lo:hi]) and np.array_equal(slot, want)
                        and bool(np.all(err <= 1e-3 + 2e-2 * np.abs(full.h[lo:hi, 0]))))
                if not good:
                    print(f"rank {rank}: mismatch T{T_local} E{E} S{S} mb{nmb} transfer{transfer} rep{rep}: idx {np.array_equal(idx, full.idx[lo:hi])} "
                          f"slot {np.array_equal(slot, want)} max err {err.max():.3e}", flush=True)
                ok = ok and good
            dist.barrier()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print(f"EP_CHECK_OK {world}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
