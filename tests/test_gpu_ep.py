"""Expert-parallel layer on 2+ GPUs against the single-device oracle (child processes, one per GPU)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ep_layer_matches_single_device_oracle():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(ROOT, "tests", "ep_check.py")],
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and f"EP_CHECK_OK {world}" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
