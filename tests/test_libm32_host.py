"""The device's single-precision exp, log, log1p, expm1, tanh and pow (homura_b200/csrc/libm32.cuh) restate the
host C library's algorithms; the same header compiles for the host, where tests/native/libm32_check.cpp compares
each function with the library's own. Here: every 509th float argument (8.4 M per function, all exponents and
both signs) and 4 M pairs for powf; run the program with a stride of 1 for all 2^32 arguments (about 40 s on 8
cores)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "native" / "libm32_check.cpp"
EXE = ROOT / "build" / "libm32_check"


def _host_has_fma() -> bool:
    try:
        return " fma " in Path("/proc/cpuinfo").read_text()
    except OSError:
        return False


@pytest.fixture(scope="module")
def checker():
    EXE.parent.mkdir(parents=True, exist_ok=True)
    header = ROOT / "homura_b200" / "csrc" / "libm32.cuh"
    if not EXE.exists() or EXE.stat().st_mtime < max(SRC.stat().st_mtime, header.stat().st_mtime):
        cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fopenmp", str(SRC), "-o", str(EXE)]
        if _host_has_fma():
            cmd.insert(1, "-mfma")
        subprocess.run(cmd, check=True)
    return EXE


def test_restated_functions_return_the_c_librarys_bits(checker):
    if not _host_has_fma():
        pytest.skip("the C library picks its non-FMA expf / logf / powf on this host; the restatement follows the FMA build")
    env = dict(os.environ, OMP_NUM_THREADS=str(min(8, os.cpu_count() or 1)))
    out = subprocess.run([str(checker), "509", str(1 << 22)], capture_output=True, text=True, env=env)
    lines = [l.split() for l in out.stdout.splitlines() if l and not l.startswith(" ")]
    assert {l[0] for l in lines} == {"expf", "logf", "expm1f", "tanhf", "log1pf", "powf2", "powf"}, out.stdout
    for name, compared, bad, *_ in lines:
        assert int(compared) > 4_000_000 and int(bad) == 0, out.stdout
    assert out.returncode == 0
