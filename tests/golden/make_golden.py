"""Writes tests/golden/c0_seed0.npz: outputs of the CPU oracle on the tiny configuration
(T=512, d=256, E=8, top-2, I=512, seed 0), kept as a regression pin.

The reference holds no golden vectors for the MoE path and cannot run here (GLSL over Vulkan),
so these vectors come from the oracle itself; before writing them this script checks the oracle
against the independent numpy restatement in tests/np_restatement.py.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402
from tests import np_restatement as NP  # noqa: E402


def main():
    synth = entry.load_package().synth
    cfg = synth.CONFIGS["c0"]
    inp = synth.layer_inputs(cfg, 0)
    res = O.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    idx, wt, out = NP.layer(inp.proj, inp.x16, inp.wgu, inp.wdown, cfg.K)
    assert np.array_equal(res.idx, idx)
    assert np.allclose(res.wt, wt, rtol=1e-5)
    assert np.array_equal(res.slot, NP.scatter_slots(res.idx, res.off))
    assert np.allclose(res.h[:, 0], out, rtol=2e-3, atol=2e-5)
    np.savez_compressed(
        os.path.join(ROOT, "tests", "golden", "c0_seed0.npz"),
        x16_sum=np.uint64(inp.x16.astype(np.uint64).sum()), wgu_sum=np.uint64(inp.wgu.astype(np.uint64).sum()),
        proj_head=inp.proj[:4, :8], idx=res.idx, wt=res.wt, count=res.count, off=res.off, tiles=res.tiles,
        slot=res.slot, amax=res.amax, h_rows=res.h[::8, 0], xp_rows=res.xp[:4])
    print("wrote c0_seed0.npz")


if __name__ == "__main__":
    main()
