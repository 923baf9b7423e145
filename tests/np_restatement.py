"""An independent numpy restatement of the MoE path's arithmetic, written from the
algorithm's definition rather than from the C oracle, used to pin the oracle (the
reference holds no golden vectors for this path).

It deliberately uses different formulations: stable sorts instead of selection loops,
softmax over all experts then renormalisation (the wording of the benchmark configs)
instead of the shader's softmax over the selected logits, float64 accumulation."""
import numpy as np


def route(proj, E, K):
    logits = proj[:, :E].astype(np.float64)
    order = np.argsort(-logits, axis=1, kind="stable")[:, :K]  # ties -> lower expert index
    p = np.exp(logits - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)                               # softmax over all experts
    sel = np.take_along_axis(p, order, 1)
    wt = sel / sel.sum(1, keepdims=True)                       # renormalised top-k
    count = np.bincount(order.ravel(), minlength=E)
    return order.astype(np.uint32), wt, count.astype(np.uint32)


def scan(count, tile):
    padded = (count.astype(np.int64) + tile - 1) // tile * tile
    off = np.concatenate([[0], np.cumsum(padded)[:-1]])
    tiles = np.repeat(np.arange(len(count)), padded // tile)
    return off.astype(np.uint32), tiles.astype(np.uint32)


def scatter_slots(idx, off):
    flat = idx.ravel().astype(np.int64)
    order = np.argsort(flat, kind="stable")           # pairs grouped by expert, token order kept
    sorted_e = flat[order]
    first = np.searchsorted(sorted_e, sorted_e, side="left")
    rank = np.arange(len(flat)) - first
    slot = np.empty(len(flat), np.int64)
    slot[order] = off[sorted_e].astype(np.int64) + rank
    return slot.reshape(idx.shape).astype(np.uint32)


def h2f(u16):
    return u16.view(np.float16).astype(np.float64)


def silu(v):
    return v / (1.0 + np.exp(-v))


def layer(proj, x16, wgu, wdown, K, wsgu=None, wsdown=None, requantise=True):
    """Float64 MoE layer with fp16 rounding of the intermediate, per token (no permutation)."""
    T, d = x16.shape
    E, twoI, _ = wgu.shape
    I = twoI // 2
    idx, wt, _ = route(proj, E, K)
    x = h2f(x16)
    out = np.zeros((T, d))
    # global power-of-two scale of the intermediate (shader/cast_f16.comp): needs the max first
    hs = {}
    for e in range(E):
        rows = np.where((idx == e).any(1))[0]
        if len(rows) == 0:
            continue
        g = x[rows] @ h2f(wgu[e]).T
        hs[e] = (rows, silu(g[:, :I]) * g[:, I:])
    amax = max((np.abs(h).max() for _, h in hs.values()), default=0.0)
    scale = 1.0
    if requantise and amax > 0:
        eb = int(np.floor(np.log2(np.float32(amax)))) + 127
        scale = 2.0 ** (141 - eb)
    for e, (rows, h) in hs.items():
        h16 = (h * scale).astype(np.float32).astype(np.float16).astype(np.float64) / scale
        y = h16 @ h2f(wdown[e]).T
        j = np.argmax(idx[rows] == e, axis=1)
        out[rows] += wt[rows, j][:, None] * y
    if wsgu is not None:
        S = wsgu.shape[0] // 2
        g = x @ h2f(wsgu).T
        h = silu(g[:, :S]) * g[:, S:]
        sh = h.astype(np.float32).astype(np.float16).astype(np.float64) @ h2f(wsdown).T
        sg = 1.0 / (1.0 + np.exp(-proj[:, E].astype(np.float64)))
        out += sg[:, None] * sh
    return idx, wt, out


def kd_bytes(logits, toks, cont):
    """Per-byte teacher distributions along the true continuation, from the definition: at depth l,
    among the tokens longer than l bytes that agree with the continuation on its first l bytes,
    the probability that byte l is the true one, and the seven most probable other bytes.
    Returns (byte u32 [rows, 16, 8], probability f64 [rows, 16, 8]); depths >= cont[:, 4] are zero."""
    V = toks.shape[0]
    tb = np.ascontiguousarray(toks[:, :4]).view(np.uint8).reshape(V, 16)      # little-endian bytes
    length = toks[:, 4].astype(np.int64)
    rows = logits.shape[0]
    byte = np.zeros((rows, 16, 8), np.uint32)
    prob = np.zeros((rows, 16, 8), np.float64)
    for r in range(rows):
        c = np.ascontiguousarray(cont[r, :4]).view(np.uint8)
        nd = min(int(cont[r, 4]), 16)
        lg = logits[r].astype(np.float64)
        e = np.where(length > 0, np.exp(lg - lg.max()), 0.0)
        agree = np.concatenate([np.ones((V, 1), bool), np.cumprod(tb == c, axis=1).astype(bool)], axis=1)  # [V, 17]
        for l in range(nd):
            alive = agree[:, l] & (length > l)
            total = max(e[alive].sum(), 1e-30)
            byte[r, l, 0], prob[r, l, 0] = c[l], e[alive & agree[:, l + 1]].sum() / total
            other = alive & ~agree[:, l + 1]
            mass = np.bincount(tb[other, l], weights=e[other], minlength=256)
            top = np.argsort(-mass, kind="stable")[:7]                          # ties -> lower byte
            byte[r, l, 1:], prob[r, l, 1:] = top, mass[top] / total
    return byte, prob
