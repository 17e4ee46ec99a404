"""Failure paths of the library's host code, without a GPU: runtime.cu, memory.cu and caching.cu are compiled with
g++ against the stand-in CUDA runtime of tests/fake_cuda and driven by tests/native/host_failures.cpp, one
process per mode (late and clean-up failures of context creation, errors a failing call would leave as the
thread's last CUDA error, a host heap that stays exhausted, the allocator's release-and-retry). After homura's
tools/check_rocm_host_failures.py."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "native" / "host_failures.cpp"
EXE = ROOT / "build" / "host_failures"
DEPENDS = [SRC, ROOT / "tests" / "fake_cuda" / "cuda_runtime.h", ROOT / "include" / "homura_cuda.h",
           ROOT / "include" / "homura_cuda_alloc.h"] + [ROOT / "homura_b200" / "csrc" / f for f in
                                                        ("runtime.cu", "memory.cu", "caching.cu", "common.cuh")]
MODES = ["late-failure", "probe-failure", "probe-then-destroy-failure", "destroy-failure-without-memory",
         "destroy-failure", "destroy-failure-without-memory-explicit", "probe-failure-without-memory", "persistent-oom",
         "exception-without-memory", "probe-malloc-failure-then-retry", "earlier-error-before-the-probe", "malloc-failure",
         "memset-failure", "allocator-release-and-retry", "allocator-synchronize-failure"]


@pytest.fixture(scope="module")
def harness():
    EXE.parent.mkdir(parents=True, exist_ok=True)
    if not EXE.exists() or EXE.stat().st_mtime < max(p.stat().st_mtime for p in DEPENDS):
        subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-Wno-subobject-linkage", "-DHMC_FAKE_CUDA",
                        "-I", str(ROOT / "tests" / "fake_cuda"), "-x", "c++", str(SRC), "-o", str(EXE)], check=True)
    return EXE


def test_the_list_of_modes_is_the_harness_s(harness):
    out = subprocess.run([str(harness), "--list"], capture_output=True, text=True, check=True)
    assert out.stdout.split() == MODES


@pytest.mark.parametrize("mode", MODES)
def test_host_failure_mode(harness, mode):
    out = subprocess.run([str(harness), mode], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, f"{mode}:\n{out.stderr}"
