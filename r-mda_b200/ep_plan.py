"""Host-side model of the expert-parallel layout (the arithmetic of `moe_ep_plan_kernel` and of
the peer addressing in the scatter and combine kernels), in numpy.  Used by the CPU rank harness
in the tests and by the benchmark to size buffers; the GPU path does not call it."""
from __future__ import annotations

import numpy as np

TILE = 128


def ep_rows(world: int, max_rows: int, experts: int, topk: int) -> int:
    """Rows of each rank's expert-contiguous buffers (`moe_cuda_ep_rows`): worst case."""
    el = experts // world
    n = world * max_rows * min(topk, el) + el * (TILE - 1)
    return (n + TILE - 1) // TILE * TILE


def slices(rows: int, nmb: int):
    """Row ranges of the token slices `moe_cuda_ep_layer` cuts `rows` tokens into: equal parts rounded
    up to the router's 8-row blocks, the last slice takes the rest (possibly nothing)."""
    part = rows if nmb == 1 else ((rows + nmb - 1) // nmb + 7) // 8 * 8
    out = []
    for m in range(nmb):
        lo = min(m * part, rows)
        hi = rows if m == nmb - 1 else min((m + 1) * part, rows)
        out.append((lo, hi))
    return out


def plan(cnt_all: np.ndarray, rank: int):
    """cnt_all [G, E]: pairs of each source rank per global expert.  Returns
    dst_off [E] (first row of `rank`'s rows of expert e inside the owner's buffer),
    off_local [E/G] (first row of each of `rank`'s own experts) and its tile schedule."""
    G, E = cnt_all.shape
    el = E // G
    tot = cnt_all.sum(0).astype(np.int64)
    padded = (tot + TILE - 1) // TILE * TILE
    off_in_owner = np.zeros(E, np.int64)
    for o in range(G):
        seg = padded[o * el:(o + 1) * el]
        off_in_owner[o * el:(o + 1) * el] = np.concatenate([[0], np.cumsum(seg)[:-1]])
    before = cnt_all[:rank].sum(0).astype(np.int64)
    dst_off = off_in_owner + before
    mine = slice(rank * el, (rank + 1) * el)
    tiles = np.repeat(np.arange(el), padded[mine] // TILE).astype(np.uint32)
    return dst_off.astype(np.uint32), off_in_owner[mine].astype(np.uint32), tiles


def local_ranks(idx: np.ndarray) -> np.ndarray:
    """For each (token, j) pair of one rank: how many earlier pairs of that rank chose the same expert."""
    flat = idx.ravel().astype(np.int64)
    order = np.argsort(flat, kind="stable")
    sorted_e = flat[order]
    first = np.searchsorted(sorted_e, sorted_e, side="left")
    rank = np.empty(len(flat), np.int64)
    rank[order] = np.arange(len(flat)) - first
    return rank.reshape(idx.shape)


def dest_ranks(idx: np.ndarray, el: int, world: int) -> np.ndarray:
    """bool [T, world]: the GPUs a token row is sent to -- once each, however many of the token's
    experts live there (the addressing of `moe_ep_send_kernel`)."""
    mask = np.zeros((idx.shape[0], world), bool)
    mask[np.arange(idx.shape[0])[:, None], idx // el] = True
    return mask
