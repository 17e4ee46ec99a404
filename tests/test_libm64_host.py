"""The device's double-precision exp, expm1, tanh and log1p (homura_b200/csrc/libm64.cuh) restate the host C
library's algorithms; the same header compiles for the host, where tests/native/libm64_check.cpp compares each
function with the library's own. Here: 8 M seeded arguments per function (random bit patterns, the whole finite range,
small arguments) and the special values; run the program without arguments for 2^28 per function (a minute on 8
cores)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "native" / "libm64_check.cpp"
EXE = ROOT / "build" / "libm64_check"


def _host_has_fma() -> bool:
    try:
        return " fma " in Path("/proc/cpuinfo").read_text()
    except OSError:
        return False


@pytest.fixture(scope="module")
def checker():
    EXE.parent.mkdir(parents=True, exist_ok=True)
    header = ROOT / "homura_b200" / "csrc" / "libm64.cuh"
    if not EXE.exists() or EXE.stat().st_mtime < max(SRC.stat().st_mtime, header.stat().st_mtime):
        cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-fopenmp", str(SRC), "-o", str(EXE)]
        if _host_has_fma():
            cmd.insert(1, "-mfma")
        subprocess.run(cmd, check=True)
    return EXE


def test_restated_functions_return_the_c_librarys_bits(checker):
    if not _host_has_fma():
        pytest.skip("the C library picks its non-FMA exp / expm1 / tanh / log1p on this host; the restatement follows the FMA build")
    env = dict(os.environ, OMP_NUM_THREADS=str(min(8, os.cpu_count() or 1)))
    out = subprocess.run([str(checker), str(1 << 23)], capture_output=True, text=True, env=env)
    lines = [l.split() for l in out.stdout.splitlines() if l]
    assert {l[0] for l in lines} == {"exp", "expm1", "tanh", "log1p"}, out.stdout
    for name, compared, bad, *_ in lines:
        assert int(compared) > 8_000_000 and int(bad) == 0, out.stdout
    assert out.returncode == 0
