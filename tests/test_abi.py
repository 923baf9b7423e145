"""The C-ABI library loads without a GPU, exports every symbol its header declares, and refuses
to work (instead of falling back to the CPU) when no sm_100 device is usable."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "moe_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(mc):
    lib = mc.lib()
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/moe_cuda.h but not exported"


def test_push_constant_layouts(mc):
    # sizes of src/pc.h:369-404 and of the glue structs
    assert ctypes.sizeof(mc.PcRoute) == 16 and ctypes.sizeof(mc.PcScan) == 8 and ctypes.sizeof(mc.PcScatter) == 12
    assert ctypes.sizeof(mc.PcMm) == 20 and ctypes.sizeof(mc.PcCombine) == 32
    assert ctypes.sizeof(mc.PcElem) == 28 and ctypes.sizeof(mc.PcSlot) == 8


def test_header_shares_the_reference_structs(tmp_path):
    """tests/abi_pc_check.c includes the reference's unmodified src/pc.h before include/moe_cuda.h and
    _Static_asserts sizes and offsets of src/pc.h:369-404; it must compile as C17 without a warning."""
    import subprocess
    import pytest
    ref_src = os.environ.get("MOE_REFERENCE_SRC", "/root/reference/src")
    if not os.path.exists(os.path.join(ref_src, "pc.h")):
        pytest.skip("the reference tree is not mounted on this machine")
    obj = tmp_path / "abi_pc_check.o"
    r = subprocess.run(["gcc", "-std=gnu17", "-Wall", "-Wextra", "-Werror", "-c", "-I", ref_src, "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "tests", "abi_pc_check.c"), "-o", str(obj)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_no_cpu_fallback_without_device(mc):
    import torch
    if torch.cuda.is_available():
        return  # covered by the GPU tests
    c = mc.Ctx(0)
    assert c.status() == mc.MOE_ERR_CUDA
    assert "no usable CUDA device" in c.last_error()
    assert mc.lib().moe_cuda_alloc(c.p, 64) is None   # every later call is a no-op
    c.close()


def test_moe_rows_formula(mc, oracle):
    for rows, k, e in [(512, 2, 8), (4096, 8, 128), (16384, 10, 512), (1, 1, 1)]:
        assert mc.moe_rows(rows, k, e) == oracle.moe_rows(rows, k, e)
    assert mc.lib().moe_cuda_ep_rows(8, 4096, 128, 8) == (8 * 4096 * 8 + 16 * 127 + 127) // 128 * 128


def test_host_mirror_builds(pkg):
    assert os.path.exists(pkg.build.build_host())


def test_product_path_does_not_touch_the_oracle():
    """Nothing under the package or bench's own arm may import or link the oracle."""
    pkg_dir = os.path.join(ROOT, "r-mda_b200")
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".c", ".h", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "moe_ref" not in text and "moe_oracle" not in text, os.path.join(dirpath, f)


def test_layer_flags_match_the_header(mc):
    """The Python front end's MOE_LAYER_* values are the header's."""
    text = open(os.path.join(ROOT, "include", "moe_cuda.h")).read()
    header = {m.group(1): int(m.group(2)) for m in re.finditer(r"#define\s+MOE_LAYER_([A-Z0-9_]+)\s+(\d+)u", text)}
    assert set(header) == {"UNFUSED", "YE_F32", "CHUNKED", "NO_PAIR", "MATERIALIZE_XP", "TILED"}
    for name, value in header.items():
        assert getattr(mc, "LAYER_" + name) == value
    assert len(set(header.values())) == len(header) and all(v & (v - 1) == 0 for v in header.values())
