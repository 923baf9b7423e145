"""Arithmetic that bench.py reports beside the measured times (no GPU needed)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_issue_efficiency_tiled_pads_to_128_rows():
    count = np.array([1, 128, 129, 0, 300], np.uint32)
    eff = bench.issue_efficiency(count, chunked=False)
    assert eff["real_rows"] == 558
    assert eff["issued_rows"] == 128 + 128 + 256 + 0 + 384
    assert abs(eff["real_over_issued"] - 558 / 896) < 1e-12


def test_issue_efficiency_chunked_rounds_chunks_to_16():
    # moe_chunk_kernel: chunks of at most 256 rows of near-equal size, MMA width rounded up to 16
    count = np.array([1, 256, 257, 0, 302, 600], np.uint32)
    eff = bench.issue_efficiency(count, chunked=True)
    # 1 -> 16; 256 -> 256; 257 -> two chunks 144 wide: 144 rows, then 113 -> 128; 302 -> two chunks 160 wide: 160 rows,
    # then 142 -> 144; 600 -> three chunks 208 wide: 208, 208, then 184 -> 192
    assert eff["issued_rows"] == 16 + 256 + (144 + 128) + 0 + (160 + 144) + (208 + 208 + 192)
    assert eff["real_rows"] == int(count.sum())


def test_30b_routing_counts_waste_little_with_chunks():
    rng = np.random.default_rng(0)
    count = rng.integers(213, 303, 128).astype(np.uint32)
    tiled = bench.issue_efficiency(count, chunked=False)["real_over_issued"]
    chunked = bench.issue_efficiency(count, chunked=True)["real_over_issued"]
    assert chunked > 0.95 > tiled
