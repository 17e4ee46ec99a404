"""Builds the CUDA library (and nothing else): every ``csrc/*.cu`` is compiled for sm_100a with nvcc and
linked into ``homura_b200/libhomura_cuda.so``, which exports only the ``hmc_*`` symbols.

This is what homura's ``build.rs`` does for its ROCm layer (hipcc per file, hidden visibility, no
contraction of a*b+c), restated for nvcc. Flags that matter for results:

* ``-fmad=false``: a product followed by a sum is two roundings, as on the CPU; fused multiply-adds
  appear only where the code calls ``fma`` explicitly (homura's ``-ffp-contract=off``).
* no ``-use_fast_math``; division, square root and denormals stay IEEE (nvcc's defaults).

Run as ``python -m homura_b200.build`` or call :func:`build`. Objects are cached under ``build/obj`` and
rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = ROOT / "build" / "obj"
LIB = PKG / "libhomura_cuda.so"
SHARD_LIB = PKG / "libhomura_cuda_shard.so"

ARCH = os.environ.get("HOMURA_CUDA_ARCH", "sm_100a")
NVCC_FLAGS = [
    "-gencode", f"arch=compute_{ARCH[3:]},code={ARCH}",
    "-O3", "-std=c++17", "-lineinfo", "-fmad=false",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Werror",
    "-Werror", "all-warnings",
    "--expt-relaxed-constexpr",
    "-Xcudafe", "--diag_suppress=unsigned_compare_with_zero",
]

# Sources that need NCCL go into their own library so that the single-GPU library has no such
# dependency.
SHARD_SOURCES = {"shard.cu"}


def nvcc() -> str:
    cuda = os.environ.get("CUDA_PATH") or os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    exe = Path(cuda) / "bin" / "nvcc"
    if exe.exists():
        return str(exe)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: set CUDA_PATH")
    return found


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(src: Path, header_time: float, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, header_time):
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        (OBJ / (src.stem + ".ptxas.txt")).write_text(proc.stderr)
    return obj


def _link(objs: list[Path], lib: Path, extra: list[str]) -> None:
    newest = max(o.stat().st_mtime for o in objs)
    if lib.exists() and lib.stat().st_mtime > newest:
        return
    cmd = [nvcc(), "-shared", "-o", str(lib), *map(str, objs), "-cudart", "shared", *extra]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed for {lib.name}:\n{proc.stdout}\n{proc.stderr}")


def build(verbose: bool = False, jobs: int | None = None) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = _newest_header()
    jobs = jobs or max(1, (os.cpu_count() or 2))
    with concurrent.futures.ThreadPoolExecutor(jobs) as pool:
        objs = list(pool.map(lambda s: _compile(s, header_time, verbose), sources))
    core = [o for o, s in zip(objs, sources) if s.name not in SHARD_SOURCES]
    shard = [o for o, s in zip(objs, sources) if s.name in SHARD_SOURCES]
    _link(core, LIB, [])
    if shard:
        _link(shard, SHARD_LIB, [f"-L{PKG}", "-l:libhomura_cuda.so", "-lnccl", "-Xlinker", "-rpath=$ORIGIN"])
    return LIB


if __name__ == "__main__":
    build(verbose="-v" in sys.argv)
    print(LIB)
