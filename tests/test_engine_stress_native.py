"""Host-side logic of the C++ copy engine under stress, without a GPU.

``tests/native/engine_stress.cpp`` compiles the engine's real source against a stand-in
CUDA runtime (``tests/native/fake_cuda/cuda_runtime.h``: streams are threads with random
delays and bounded queues, events follow CUDA's capture rules) and a stand-in kernel that
adds known constants.  Every scenario (tiny to oversized staging buffer, inline or
threaded write-backs, loads from the helper thread or from the caller, out-of-order
steps, host gradients) must end with exactly the expected values in host memory.  The
same program is also run under ThreadSanitizer when the toolchain has it."""

import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "native", "engine_stress.cpp")
INC = os.path.join(HERE, "native", "fake_cuda")


def build(tmp_path, name, extra):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / name)
    cmd = [gxx, "-std=c++17", "-O1", "-g", "-pthread", "-I", INC, SRC, "-o", exe] + extra
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    return exe, proc


@pytest.mark.timeout(600)
def test_engine_survives_random_schedules(tmp_path):
    exe, proc = build(tmp_path, "engine_stress", [])
    assert proc.returncode == 0, proc.stderr[-2000:]
    run = subprocess.run([exe, "4"], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and "all scenarios ok" in run.stdout, (run.stdout[-2000:], run.stderr[-2000:])


@pytest.mark.timeout(900)
def test_engine_threads_are_race_free_under_tsan(tmp_path):
    exe, proc = build(tmp_path, "engine_stress_tsan", ["-fsanitize=thread"])
    if proc.returncode != 0:
        pytest.skip("toolchain cannot link ThreadSanitizer")
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66")
    run = subprocess.run([exe, "2"], capture_output=True, text=True, timeout=600, env=env)
    if "FATAL: ThreadSanitizer" in run.stderr:  # e.g. unsupported address-space layout of the host
        pytest.skip("ThreadSanitizer cannot run on this host")
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-4000:]
    assert run.returncode == 0 and "all scenarios ok" in run.stdout, (run.stdout[-2000:], run.stderr[-2000:])
