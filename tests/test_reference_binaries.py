"""MotifCL's OWN test executables, compiled unmodified from the MotifCL tree and linked against
the CUDA runtime adapter (motifcl_b200/adapter) instead of MotifCL's Vulkan runtime.  They are
built where the MotifCL tree is mounted (motifcl_b200/adapter/Makefile) and travel prebuilt; where
they are absent the tests skip.  Exit code 77 is MotifCL's "skip" convention."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "motifcl_b200", "adapter", "_build")
BINARIES = ["test_vulkan_counter_fused", "test_vulkan_memory_native", "test_matmul_transpose_b_autograd"]


def _run(name):
    path = os.path.join(BUILD, name)
    if not os.path.isfile(path):
        pytest.skip(f"{name} was not built on this machine (needs the MotifCL tree)")
    return subprocess.run([path], capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("name", BINARIES)
def test_reference_binary_skips_without_a_device(name):
    import motifcl_b200 as mb
    if mb.lib().mcl_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    r = _run(name)
    out = (r.stdout + r.stderr).lower()
    assert r.returncode == 77 and ("skip" in out or "no cuda device" in out)


@pytest.mark.gpu
@pytest.mark.parametrize("name", BINARIES)
def test_reference_binary_passes_on_the_cuda_backend(name):
    """tests/test_vulkan_counter_fused.cpp: same-seed layers start identical; forward and grad_x
    within 2e-5 of decode_weight + matmul_transpose_b / a host loop; the autograd-driven update
    equals a direct apply_update_backward exactly (state, scale, v); state and scale change.
    tests/test_vulkan_memory_native.cpp: teacher recovery (loss halves, ternary accuracy >= 0.8) and
    a 4-block reversible + counter stack whose loss falls.
    tests/test_matmul_transpose_b_autograd.cpp: NT matmul gradients vs the NN path (<= 1e-4) and
    gradient accumulation on a shared tensor."""
    r = _run(name)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout and "FAIL" not in r.stdout
