"""MotifCL's OWN test executables, compiled unmodified from the MotifCL tree and linked against
the CUDA runtime adapter (motifcl_b200/adapter) instead of MotifCL's Vulkan runtime.  They are
built where the MotifCL tree is mounted (motifcl_b200/adapter/Makefile) and travel prebuilt; where
they are absent the tests skip.  Exit code 77 is MotifCL's "skip" convention."""
import os
import re
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


CL_BINARIES = ["cl/test_counter_state", "cl/test_memory_truth_gate", "cl/test_buffer", "cl/test_tensor",
               "cl/test_backend_lifetime"]
CL_ENV = {"MOTIFCL_KERNEL_DIR": os.path.join(ROOT, "motifcl_b200", "adapter", "cl_sources")}


@pytest.mark.parametrize("name", CL_BINARIES)
def test_reference_opencl_binary_skips_without_a_device(name):
    import motifcl_b200 as mb
    if mb.lib().mcl_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    r = _run_env(name, CL_ENV)
    assert r.returncode == 77 and "no opencl platforms" in (r.stdout + r.stderr).lower()


@pytest.mark.gpu
@pytest.mark.parametrize("name", CL_BINARIES)
def test_reference_opencl_binary_passes_through_the_opencl_seam(name):
    """MotifCL's OpenCL-only counter tests, unmodified, with motifcl_b200/adapter/cuda_opencl_shim.cpp in the place of
    libOpenCL.  tests/test_counter_state.cpp: 800 steps of forward + mse_loss + backward on a 16 x 16 layer recover a
    ternary teacher (final mse <= 5e-3, ternary accuracy >= 0.9; the input has no requires_grad).
    tests/test_memory_truth_gate.cpp: the memory-native update allocates less than a quarter of a dense weight while
    the dense apply_update_seed path allocates at least half; grad_x from the packed state equals decode + matmul
    within 1e-4.  tests/test_buffer.cpp, test_tensor.cpp, test_backend_lifetime.cpp: upload / download round trip,
    Tensor::ones (fill_f32), a tensor that outlives its backend.  All exit 0 on success and print the reason otherwise."""
    r = _run_env(name, CL_ENV)
    assert r.returncode == 0, r.stdout + r.stderr


def _run_env(name, env, timeout=600):
    path = os.path.join(BUILD, name)
    if not os.path.isfile(path):
        pytest.skip(f"{name} was not built on this machine (needs the MotifCL tree)")
    e = dict(os.environ)
    e.update({k: str(v) for k, v in env.items()})
    return subprocess.run([path], capture_output=True, text=True, timeout=timeout, env=e)


@pytest.mark.gpu
def test_reference_block_stack_bench_runs_on_the_cuda_backend():
    """tests/bench_ternary15m.cpp, MotifCL's own harness for its tok/s figure: the 6-block ternary15m
    stack (36 counter layers, rmsnorm, attention, swiglu, 32k-vocab head, cross-entropy), forward +
    backward + counter updates + sgd.  It exits non-zero on a failed op or a non-finite loss; the loss
    of the last step must be below the first one's."""
    r = _run_env("bench_ternary15m", {"BENCH_BATCHED": 1, "BENCH_B": 4, "BENCH_STEPS": 10})
    assert r.returncode == 0, r.stdout + r.stderr
    losses = [float(line.rsplit("loss", 1)[1]) for line in r.stdout.splitlines() if " loss " in line]
    assert len(losses) == 2 and losses[1] < losses[0], r.stdout
    assert "tok/s=" in r.stdout


@pytest.mark.gpu
def test_reference_trainer_learns_synthetic_records(tmp_path):
    """tools/train_ternary15m.cpp unchanged, on seeded synthetic records with a learnable next-token rule
    (90 % of transitions follow next = (31*cur + 7) mod 512): embedding, rope, causal attention, adam and the
    counter updates all have to work for the logged loss to fall well below ln(32000) = 10.37."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "motifcl_b200", "adapter"))
    import make_synthetic_records as msr
    data = tmp_path / "data"
    msr.write_dataset(str(data), seq=64, train_records=512, val_records=32, seed=7)
    r = _run_env("train_ternary15m", {"DATA_DIR": data, "OUT_DIR": tmp_path / "out", "STEPS": 120, "BATCH": 8, "SEQ": 64,
                                      "LOG_EVERY": 20, "EVAL_EVERY": 1000, "CKPT_EVERY": 60, "RESUME": 0})
    assert r.returncode == 0, r.stdout + r.stderr
    losses = [float(m.group(1)) for m in re.finditer(r"^step \d+ loss ([0-9.]+)", r.stdout, flags=re.M)]
    assert len(losses) >= 5, r.stdout
    assert losses[-1] < 8.0 and losses[-1] < losses[0] - 1.5, r.stdout
    # the checkpoint the trainer wrote with MotifCL's own save_tensor pins this package's reader of those files:
    # every counter linear of every block loads, with the shapes of the ternary15m stack and a valid 6-bit state
    import numpy as np
    from motifcl_b200 import checkpoint, codec
    out = str(tmp_path / "out")
    dims = {"wq": (288, 288), "wk": (288, 288), "wv": (288, 288), "wo": (288, 288), "wup": (1536, 288), "wdown": (288, 768)}
    seen = 0
    for layer in range(6):
        for name in checkpoint.LINEAR_NAMES:
            st, sc, v = checkpoint.load_counter_linear(out, checkpoint.block_prefix(layer, name))
            O, I = dims[name]
            assert st.shape == (O * I // 4 * 3,) and sc.shape == (O,) and v.shape == (O,), (layer, name, st.shape, sc.shape)
            codes = codec.unpack_codes(st.reshape(O, -1), I)
            assert codes.max() < 63 and np.isfinite(sc).all() and (sc > 0).all() and (v >= 0).all()
            t, c = codec.decode(codes, 11)
            assert set(np.unique(t)) <= {-1, 0, 1} and np.abs(c).max() <= 10
            seen += 1
    assert seen == 36
    emb = checkpoint.load_tensor(os.path.join(out, "emb.mt"))
    assert emb.dtype == np.float32 and emb.shape == (32000, 288)
