"""Builds the CPU checker: ``oracle/oracle.cpp`` -> ``oracle/_build/liboracle.so`` (g++ -O2, no fast-math,
no contraction of a*b+c, so the arithmetic is that of homura's Rust CPU backend on x86-64), and, where
homura's sources are present (the directory named by the environment variable ``HOMURA_SRC``),
``oracle/_ref/libref_casts.so``: homura's own C++
restatement of its casts (``csrc/elem.hpp``) compiled for the host from where it lies, used to cross-check
the oracle's conversions. TEST INFRASTRUCTURE: nothing that ships may load these libraries.
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "liboracle.so"
REF_LIB = HERE / "_ref" / "libref_casts.so"
# A checkout of homura, if there is one: HOMURA_SRC names it (the default is a `reference` directory in the home directory).
REFERENCE = Path(os.environ.get("HOMURA_SRC") or Path.home() / "reference")
CXXFLAGS = ["-O2", "-std=c++17", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-Wall", "-Wno-sign-compare",
            "-Wno-type-limits"]


def _stale(lib: Path, sources: list[Path]) -> bool:
    return not lib.exists() or lib.stat().st_mtime < max(s.stat().st_mtime for s in sources)


def build() -> Path:
    src = HERE / "oracle.cpp"
    header = HERE.parent / "include" / "homura_cuda.h"
    if _stale(LIB, [src, header]):
        LIB.parent.mkdir(exist_ok=True)
        subprocess.run(["g++", *CXXFLAGS, str(src), "-o", str(LIB), "-lm"], check=True)
    return LIB


def build_ref() -> Path | None:
    """The reference's cast header for the host, only where the reference is present."""
    elem = REFERENCE / "csrc" / "elem.hpp"
    shim = HERE / "ref_casts.cpp"
    if not elem.exists() or not shim.exists():
        return REF_LIB if REF_LIB.exists() else None
    if _stale(REF_LIB, [shim, elem]):
        REF_LIB.parent.mkdir(exist_ok=True)
        subprocess.run(["g++", *CXXFLAGS, "-I", str(HERE / "ref_shim"), "-I", str(REFERENCE / "csrc"), str(shim), "-o",
                        str(REF_LIB)], check=True)
    return REF_LIB


if __name__ == "__main__":
    print(build())
    print(build_ref())
