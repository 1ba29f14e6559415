"""The C++ host mirror of `nn::rl` (noetic_tensor_b200/host/noetic_rl.hpp): it must compile with
g++ alone (CPU test), and its own test program — the reference's rl tests restated in C++ over
the C ABI — must pass on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.path.join(ROOT, "tests", "cpp", "test_rl_host.cpp")
PROGRAM = os.path.join(ROOT, "tests", "cpp", "_build", "test_rl_host")


def _program():
    from noetic_tensor_b200 import _build

    return _build.build_host_program(SOURCE, PROGRAM)


def test_host_mirror_compiles_and_refuses_to_run_without_a_gpu():
    import torch

    exe = _program()
    assert os.access(exe, os.X_OK)
    if not torch.cuda.is_available():
        r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
        assert r.returncode == 2 and "no CUDA device" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_host_mirror_passes_the_reference_style_tests():
    r = subprocess.run([_program()], capture_output=True, text=True, timeout=300)
    print(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "all passed" in r.stdout
