"""Seeded synthetic MoE-layer inputs for the named benchmark shapes.

Every tensor is a pure function of (seed, tensor id, block index) through
numpy's counter-based Philox generator, so any expert slice can be regenerated
on any rank without generating the rest.  fp16 tensors are returned as uint16
bit patterns (what the C ABI takes).

The shapes stand in for the public "30B-A3B" / "80B-A3B" model families and for
the distillation batch of 8 sequences x 2 copies x 256 tokens; no checkpoint or
dataset is involved.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, replace

import numpy as np

MOE_PAD = 128  # MDA_QWEN_MOE_PAD, src/qwen.h:22: proj row = [E logits | pad 128 | ...]

T_WGU, T_WDOWN, T_X, T_ROUTER, T_SGATE, T_WSGU, T_WSDOWN, T_ZIPF = range(8)


@dataclass(frozen=True)
class MoEConfig:
    name: str
    T: int
    d: int
    E: int
    K: int
    I: int
    S: int = 0            # shared expert intermediate size (0 = none)
    zipf_beta: float = 0.0  # router bias = beta * log(Zipf(1.2) weight); 0 = near-uniform
    layers: int = 1

    @property
    def pstride(self) -> int:
        return self.E + MOE_PAD

    @property
    def mrows(self) -> int:
        """round128(T*K + E*127), src/qwen.c:68-70."""
        n = self.T * self.K + self.E * 127
        return (n + 127) // 128 * 128

    def flops(self) -> int:
        """Unpadded grouped-product flops: T*K*6*d*I (+ T*6*d*S for the shared expert)."""
        return self.T * self.K * 6 * self.d * self.I + self.T * 6 * self.d * self.S

    def with_tokens(self, T: int) -> "MoEConfig":
        return replace(self, T=T, name=f"{self.name}-T{T}")


CONFIGS = {
    "c0": MoEConfig("c0-tiny", T=512, d=256, E=8, K=2, I=512),
    "c1": MoEConfig("c1-30B-A3B", T=4096, d=2048, E=128, K=8, I=768),
    "c2": MoEConfig("c2-80B-A3B", T=16384, d=2048, E=512, K=10, I=512, S=512),
    "c3": MoEConfig("c3-skewed", T=4096, d=2048, E=128, K=8, I=768, zipf_beta=1.0),
    "c3b": MoEConfig("c3-skewed-60pct", T=4096, d=2048, E=128, K=8, I=768, zipf_beta=0.55),
    "c4": MoEConfig("c4-stack48", T=4096, d=2048, E=128, K=8, I=768, layers=48),
}


def _rng(seed: int, tensor: int, block: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[(seed << 8) | tensor, block]))


def _normal_f16(seed, tensor, block, shape, std) -> np.ndarray:
    v = _rng(seed, tensor, block).standard_normal(shape, dtype=np.float32)
    v *= np.float32(std)
    return v.astype(np.float16).view(np.uint16)  # astype rounds to nearest even


def expert_weights(cfg: MoEConfig, seed: int, e_lo: int = 0, e_hi: int | None = None, threads: int = 8):
    """fp16 ~N(0, 0.02): wgu [n, 2I, d] (gate rows then up rows, as HF gate_up_proj;
    src/qwen.c:102,848-856) and wdown [n, d, I] for experts e_lo..e_hi-1."""
    e_hi = cfg.E if e_hi is None else e_hi
    n = e_hi - e_lo
    wgu = np.empty((n, 2 * cfg.I, cfg.d), np.uint16)
    wdown = np.empty((n, cfg.d, cfg.I), np.uint16)

    def one(i):
        wgu[i] = _normal_f16(seed, T_WGU, e_lo + i, (2 * cfg.I, cfg.d), 0.02)
        wdown[i] = _normal_f16(seed, T_WDOWN, e_lo + i, (cfg.d, cfg.I), 0.02)

    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(one, range(n)))
    return wgu, wdown


def shared_weights(cfg: MoEConfig, seed: int):
    if cfg.S == 0:
        return None, None
    wsgu = _normal_f16(seed, T_WSGU, 0, (2 * cfg.S, cfg.d), 0.02)
    wsdown = _normal_f16(seed, T_WSDOWN, 0, (cfg.d, cfg.S), 0.02)
    return wsgu, wsdown


def activations(cfg: MoEConfig, seed: int, row_lo: int = 0, row_hi: int | None = None) -> np.ndarray:
    """fp16 ~N(0,1) [rows, d]; generated in blocks of 256 rows so row ranges are reproducible."""
    row_hi = cfg.T if row_hi is None else row_hi
    B = 256
    out = np.empty((row_hi - row_lo, cfg.d), np.uint16)
    for b in range(row_lo // B, (row_hi + B - 1) // B):
        blk = _normal_f16(seed, T_X, b, (B, cfg.d), 1.0)
        lo, hi = max(row_lo, b * B), min(row_hi, (b + 1) * B)
        out[lo - row_lo:hi - row_lo] = blk[lo - b * B:hi - b * B]
    return out


def router_weights(cfg: MoEConfig, seed: int):
    """Router gate fp32 ~N(0, 0.02) [E, d] and the shared-expert gate vector [d]."""
    wr = _rng(seed, T_ROUTER, 0).standard_normal((cfg.E, cfg.d), dtype=np.float32) * np.float32(0.02)
    wsg = _rng(seed, T_SGATE, 0).standard_normal(cfg.d, dtype=np.float32) * np.float32(0.02)
    return wr, wsg


def zipf_bias(cfg: MoEConfig, seed: int) -> np.ndarray:
    """beta * log(w_e), w_e proportional to rank_e^-1.2 under a seeded permutation of ranks."""
    if cfg.zipf_beta == 0.0:
        return np.zeros(cfg.E, np.float32)
    ranks = _rng(seed, T_ZIPF, 0).permutation(cfg.E) + 1
    w = ranks.astype(np.float64) ** -1.2
    w /= w.sum()
    return (cfg.zipf_beta * np.log(w)).astype(np.float32)


def projection(cfg: MoEConfig, x16: np.ndarray, wr: np.ndarray, wsg: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """The upstream projection's output row: fp32 [rows, E + 128] with router logits in
    columns < E and the shared expert's gate logit in column E (src/qwen.c:55-57,845,891).
    Computed once on the host and handed to both the oracle and the GPU, so the
    top-k inputs are bit-identical on both sides."""
    x = x16.view(np.float16).astype(np.float32)
    proj = np.zeros((x.shape[0], cfg.pstride), np.float32)
    proj[:, :cfg.E] = x @ wr.T + bias[None, :]
    proj[:, cfg.E] = x @ wsg
    return proj


@dataclass
class LayerInputs:
    cfg: MoEConfig
    seed: int
    x16: np.ndarray
    proj: np.ndarray
    wgu: np.ndarray
    wdown: np.ndarray
    wsgu: np.ndarray | None
    wsdown: np.ndarray | None


def layer_inputs(cfg: MoEConfig, seed: int = 0, weights: bool = True) -> LayerInputs:
    x16 = activations(cfg, seed)
    wr, wsg = router_weights(cfg, seed)
    proj = projection(cfg, x16, wr, wsg, zipf_bias(cfg, seed))
    wgu = wdown = wsgu = wsdown = None
    if weights:
        wgu, wdown = expert_weights(cfg, seed)
        wsgu, wsdown = shared_weights(cfg, seed)
    return LayerInputs(cfg, seed, x16, proj, wgu, wdown, wsgu, wsdown)
