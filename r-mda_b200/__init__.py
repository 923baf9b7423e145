"""libmoe_cuda: the distillation teacher's MoE forward path as CUDA for sm_100a.

The product is the C-ABI shared library built from csrc/ (include/moe_cuda.h)
plus the C host-side mirror in host/.  The Python modules here are the test and
benchmark front end: `moe_cuda` (ctypes binding), `synth` (seeded inputs of the
named shapes) and `build` (nvcc / gcc recipes).

The directory name has a hyphen, so import it through `__graft_entry__.load_package()`,
which registers it as the module `r_mda_b200`.
"""
from . import build, ep_plan, moe_cuda, synth  # noqa: F401
