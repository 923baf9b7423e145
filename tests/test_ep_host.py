"""Expert-parallel host logic on CPU: two gloo ranks run the layout arithmetic of the EP path
(counts exchange, rows sent once per destination rank, owner-side tile schedule and source-row table,
partial sums per owning rank on the way back) with the CPU oracle
standing in for the kernels, and must reproduce the single-process layer."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T_local, fail_rank, per_gpu, q):
    sys.path.insert(0, ROOT)
    import dataclasses
    import __graft_entry__ as entry
    from oracle import moe_oracle as O
    pkg = entry.load_package()
    synth, epp = pkg.synth, pkg.ep_plan
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        cfg = dataclasses.replace(synth.CONFIGS["c0"], T=T_local * world, E=8, K=2, d=64, I=128)
        inp = synth.layer_inputs(cfg, 5)
        full = O.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)   # what one GPU would compute
        el = cfg.E // world
        lo, hi = rank * T_local, (rank + 1) * T_local
        proj, x16 = np.ascontiguousarray(inp.proj[lo:hi]), np.ascontiguousarray(inp.x16[lo:hi])
        wgu, wdown = inp.wgu[rank * el:(rank + 1) * el], inp.wdown[rank * el:(rank + 1) * el]
        idx, wt, count = O.route(proj, cfg.E, cfg.K)
        assert np.array_equal(idx, full.idx[lo:hi]) and np.array_equal(wt, full.wt[lo:hi])
        if rank == fail_rank:
            raise RuntimeError("injected: this rank leaves before the counts exchange")
        # all-gather of the counts
        gathered = [torch.zeros(cfg.E, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(count.astype(np.int64)))
        cnt_all = np.stack([g.numpy() for g in gathered]).astype(np.uint32)
        dst_off, off_local, tiles = epp.plan(cnt_all, rank)
        dest_row = dst_off[idx].astype(np.int64) + epp.local_ranks(idx)
        owner = idx // el
        # the permutation is the single-GPU one restricted to each expert
        want_row = (full.slot[lo:hi].astype(np.int64) - full.off[idx].astype(np.int64)
                    + np.array([epp.plan(cnt_all, o)[1] for o in range(world)]).reshape(-1)[idx])
        assert np.array_equal(dest_row, want_row)
        mcap = epp.ep_rows(world, T_local, cfg.E, cfg.K)
        if per_gpu:
            # dispatch: a row travels once per destination rank into that rank's receive buffer (slot =
            # source rank, token); every (token, expert) pair travels as a 4-byte record into the owner's
            # source-row table.  Every rank learns all of it and keeps what is addressed to it.
            dests = epp.dest_ranks(idx, el, world)
            assert dests.sum() <= owner.size and np.array_equal(dests.any(1), np.ones(T_local, bool))
            objs = [None] * world
            dist.all_gather_object(objs, (rank, dests, x16, owner.ravel(), dest_row.ravel(),
                                          np.repeat(np.arange(T_local), cfg.K)))
            xr = np.full((world * T_local, cfg.d), 0x7e00, np.uint16)      # fp16 NaN: a row that never arrived would show
            have = np.zeros(world * T_local, bool)
            src_row = np.full(mcap, -1, np.int64)
            for s, dst, rows_x, ow, drow, tok in objs:
                sel = dst[:, rank]
                xr[s * T_local + np.nonzero(sel)[0]] = rows_x[sel]
                have[s * T_local + np.nonzero(sel)[0]] = True
                selp = ow == rank
                assert (src_row[drow[selp]] == -1).all()      # no two pairs land on the same row
                src_row[drow[selp]] = s * T_local + tok[selp]
            live = src_row >= 0
            assert have[src_row[live]].all()                  # every row a record points at was sent
            xp = np.zeros((mcap, cfg.d), np.uint16)           # what the owner's product gathers
            xp[live] = xr[src_row[live]]
        else:
            # per pair, "peer stores": every rank learns all (owner, row, data) triples and keeps its own
            objs = [None] * world
            dist.all_gather_object(objs, (owner.ravel(), dest_row.ravel(), np.repeat(x16, cfg.K, 0)))
            xp = np.zeros((mcap, cfg.d), np.uint16)
            for ow, rows, data in objs:
                sel = ow == rank
                assert not xp[rows[sel]].any()          # no two pairs land on the same row
                xp[rows[sel]] = data[sel]
        tl = np.full(mcap // 128, 0xffffffff, np.uint32)
        tl[:len(tiles)] = tiles
        g = O.mm(xp, wgu, tl, 2 * cfg.I, cfg.d)
        hp16 = O.cast_f16(O.swiglu(g, cfg.I, 2 * cfg.I, 0, cfg.I), np.zeros(4, np.uint32), O.NO_SLOT)
        ye = O.mm(hp16, wdown, tl, cfg.d, cfg.I)
        if per_gpu:
            # return: the owner adds wt * (expert output row) over the pairs of a token it holds, in j order,
            # and leaves one fp16 partial row per (source rank, token); the home rank adds the partial rows
            # of the owning ranks in ascending rank order
            recs = [None] * world
            dist.all_gather_object(recs, (rank, owner.ravel(), dest_row.ravel(), np.repeat(np.arange(T_local), cfg.K), wt.ravel()))
            part = np.zeros((world, T_local, cfg.d), np.float32)
            for s, ow, drow, tok, w in recs:
                for i in np.nonzero(ow == rank)[0]:       # ascending pair index = (token, j) order
                    part[s, tok[i]] = part[s, tok[i]] + np.float32(w[i]) * ye[drow[i]]
            parts = [None] * world
            dist.all_gather_object(parts, part.astype(np.float16))
            h = np.zeros((T_local, cfg.d), np.float32)
            for g in range(world):
                sel = dests[:, g]
                h[sel] += parts[g][rank][sel].astype(np.float32)
        else:
            # per pair, "peer loads": gather each pair's row back from its owner, accumulate in j order
            yes = [None] * world
            dist.all_gather_object(yes, ye)
            h = np.zeros((T_local, cfg.d), np.float32)
            for j in range(cfg.K):
                rows = np.stack([yes[o][r] for o, r in zip(owner[:, j], dest_row[:, j])])
                h += wt[:, j:j + 1] * rows
        err = np.abs(h - full.h[lo:hi, 0])
        assert np.all(err <= 1e-3 + 2e-2 * np.abs(full.h[lo:hi, 0])), err.max()
        q.put((rank, "ok", float(err.max())))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "fail", repr(e)))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, T_local, fail_rank=-1, per_gpu=True):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, world, port, T_local, fail_rank, per_gpu, q)) for r in range(world)]
    for p in ps:
        p.start()
    out = [q.get(timeout=120) for _ in range(world)]
    for p in ps:
        p.join(30)
    return sorted(out)


@pytest.mark.parametrize("per_gpu", [True, False], ids=["per_gpu", "per_pair"])
def test_two_ranks_reproduce_single_gpu_layer(per_gpu):
    out = _run(2, 96, per_gpu=per_gpu)
    assert [o[1] for o in out] == ["ok", "ok"], out


@pytest.mark.parametrize("per_gpu", [True, False], ids=["per_gpu", "per_pair"])
def test_four_ranks_ragged_tokens(per_gpu):
    out = _run(4, 37, per_gpu=per_gpu)
    assert [o[1] for o in out] == ["ok"] * 4, out


def test_rank_that_leaves_is_noticed_by_the_others():
    """Host-side failure injection: one rank raises before the collective; the other must come
    back with an error from its bounded collective instead of hanging."""
    out = _run(2, 32, fail_rank=1)
    assert out[1][1] == "fail" and "injected" in out[1][2]
    assert out[0][1] == "fail"      # timed out / connection closed, reported as an error


def test_plan_matches_hand_case():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    epp = entry.load_package().ep_plan
    cnt = np.array([[3, 0, 130, 1], [2, 0, 0, 127]], np.uint32)   # 2 ranks x 4 experts, 2 experts per rank
    d0, off0, t0 = epp.plan(cnt, 0)
    d1, off1, t1 = epp.plan(cnt, 1)
    assert d0.tolist() == [0, 128, 0, 256] and d1.tolist() == [3, 128, 130, 257]
    assert off0.tolist() == [0, 128] and t0.tolist() == [0]            # expert 1 is empty: no tile
    assert off1.tolist() == [0, 256] and t1.tolist() == [0, 0, 1]
    assert epp.ep_rows(2, 64, 4, 2) == (2 * 64 * 2 + 2 * 127 + 127) // 128 * 128


def test_token_slices_cover_the_rows_once():
    """The slices moe_cuda_ep_layer cuts a rank's tokens into: disjoint, in order, 8-row aligned starts,
    together exactly the rows -- for every slice count the library accepts, ragged and tiny row counts too."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    epp = entry.load_package().ep_plan
    for rows in (0, 1, 7, 8, 9, 37, 300, 1024, 4096, 4101):
        for nmb in (1, 2, 3, 4):
            sl = epp.slices(rows, nmb)
            assert len(sl) == nmb and sl[0][0] == 0 and sl[-1][1] == rows
            for (a, b), (c, d) in zip(sl, sl[1:]):
                assert b == c and a <= b and c <= d
            assert all(a % 8 == 0 or a == rows for a, _ in sl)
    assert epp.slices(4096, 2) == [(0, 2048), (2048, 4096)]
    assert epp.slices(300, 4) == [(0, 80), (80, 160), (160, 240), (240, 300)]
    assert epp.slices(9, 4) == [(0, 8), (8, 9), (9, 9), (9, 9)]       # later slices may be empty


def test_sliced_plan_places_every_pair_once():
    """With the tokens of every rank cut into slices, each slice has its own counts, plan and buffers: the rows of a
    slice form, inside every owner's buffer of that slice, the single-device order restricted to the slice."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    epp = entry.load_package().ep_plan
    rng = np.random.default_rng(4)
    world, T, E, K, nmb = 4, 100, 16, 4, 3
    el = E // world
    idx = np.stack([np.stack([rng.permutation(E)[:K] for _ in range(T)]) for _ in range(world)]).astype(np.uint32)
    for a, b in epp.slices(T, nmb):
        cnt = np.stack([np.bincount(idx[r, a:b].ravel(), minlength=E) for r in range(world)]).astype(np.uint32)
        seen = {o: set() for o in range(world)}
        for r in range(world):
            dst_off = epp.plan(cnt, r)[0]
            rows = dst_off[idx[r, a:b]].astype(np.int64) + epp.local_ranks(idx[r, a:b])
            for o, row in zip((idx[r, a:b] // el).ravel(), rows.ravel()):
                assert row not in seen[int(o)]
                seen[int(o)].add(int(row))
        for o in range(world):
            off_local, tiles = epp.plan(cnt, o)[1:]
            tot = cnt[:, o * el:(o + 1) * el].sum(0)
            want = set()
            for e in range(el):
                want |= set(range(int(off_local[e]), int(off_local[e]) + int(tot[e])))
            assert seen[o] == want                       # exactly the non-padding rows of the owner's tiles
            assert len(tiles) == int(((tot + 127) // 128).sum())
