"""The C-ABI library loads without a GPU, exports every symbol the headers declare, reports the struct
layout the binding assumes (the check homura's Rust side makes against hmr_abi_check,
src/backend/rocm/tests.rs:10-59), and the committed binding is what the generator produces."""
import ctypes
import re
import subprocess
import sys
from pathlib import Path

import homura_b200
from homura_b200 import ffi

ROOT = Path(__file__).resolve().parent.parent


def declared(header: Path):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(hmc_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    lib = homura_b200.load()
    for header in ["homura_cuda.h", "homura_cuda_alloc.h"]:
        names = declared(ROOT / "include" / header)
        assert len(names) >= 10
        for name in names:
            assert hasattr(lib, name), f"{name} is declared in {header} but not exported"
            assert name in ffi.FUNCTIONS, f"{name} has no binding"
    # the sharding header is served by two libraries: the NCCL entry points live in their own
    shard = homura_b200.load_shard()
    for name in declared(ROOT / "include" / "homura_cuda_shard.h"):
        home = shard if name.startswith("hmc_comm_") else lib
        assert hasattr(home, name), f"{name} is declared in homura_cuda_shard.h but not exported"
        assert name in ffi.FUNCTIONS, f"{name} has no binding"


def test_binding_is_up_to_date():
    r = subprocess.run([sys.executable, "-m", "homura_b200.gen_cuda_ffi", "--check"], cwd=ROOT, capture_output=True)
    assert r.returncode == 0, r.stderr.decode()


def test_abi_check_matches_the_binding():
    lib = homura_b200.load()
    info = ffi.hmc_abi_info()
    lib.hmc_abi_check(ctypes.byref(info))
    assert info.abi_info_size == ctypes.sizeof(ffi.hmc_abi_info)
    assert info.properties_size == ctypes.sizeof(ffi.hmc_device_properties)
    assert info.properties_align == ctypes.alignment(ffi.hmc_device_properties)
    P = ffi.hmc_device_properties
    assert list(info.properties_offsets) == [P.name.offset, P.arch.offset, P.multiprocessor_count.offset,
                                             P.warp_size.offset, P.total_memory.offset]
    assert list(info.status_values) == [0, 1, 2, 3, 4]
    assert (info.name_len, info.arch_len) == (ffi.HMC_NAME_LEN, ffi.HMC_ARCH_LEN)
    D = ffi.hmc_tensor_desc
    assert info.desc_size == ctypes.sizeof(D) and info.desc_align == ctypes.alignment(D)
    assert list(info.desc_offsets) == [D.data.offset, D.offset.offset, D.dtype.offset, D.ndim.offset, D.sizes.offset,
                                       D.strides.offset]
    assert list(info.dtype_values) == list(range(10))
    assert info.max_dims == 25
    assert info.adamw_scalars_size == ctypes.sizeof(ffi.hmc_adamw_scalars)


def test_errors_are_per_thread_messages():
    lib = homura_b200.load()
    assert lib.hmc_test_fail(b"first failure") == ffi.HMC_INVALID
    assert lib.hmc_last_error() == b"first failure"
    assert lib.hmc_built_archs() == b"sm_100a"
    import threading
    seen = []
    def other():
        seen.append(lib.hmc_last_error())
        lib.hmc_test_fail(b"second")
        seen.append(lib.hmc_last_error())
    t = threading.Thread(target=other)
    t.start(); t.join()
    assert seen == [b"", b"second"]
    assert lib.hmc_last_error() == b"first failure"


def test_null_and_invalid_arguments_are_refused_without_a_gpu():
    lib = homura_b200.load()
    assert lib.hmc_device_count(None) == ffi.HMC_INVALID
    d = ffi.hmc_tensor_desc()
    assert lib.hmc_unary(None, 0, ctypes.byref(d), ctypes.byref(d)) == ffi.HMC_INVALID
    assert lib.hmc_last_error() == b"null context"
    n = ctypes.c_int64()
    d.ndim = 26
    assert lib.hmc_reduce_workspace(ctypes.byref(d), ctypes.byref(d), 0, ctypes.byref(n)) == ffi.HMC_INVALID
    assert b"26 dimensions" in lib.hmc_last_error()
    d.ndim, d.dtype = 1, 77
    assert lib.hmc_reduce_workspace(ctypes.byref(d), ctypes.byref(d), 0, ctypes.byref(n)) == ffi.HMC_INVALID


def test_reduce_plans_depend_on_sizes_and_strides_only():
    """Plans are computed on the host, so every plan can be reached and inspected without a GPU."""
    lib = homura_b200.load()
    def plan(kept, red, dtype=ffi.HMC_F32):
        k, r = ffi.hmc_tensor_desc(), ffi.hmc_tensor_desc()
        for d, dims in ((k, kept), (r, red)):
            d.dtype, d.ndim = dtype, len(dims)
            for i, (n, s) in enumerate(dims):
                d.sizes[i], d.strides[i] = n, s
        kind, splits, chunk = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        assert lib.hmc_test_reduce_plan(ctypes.byref(k), ctypes.byref(r), ctypes.byref(kind), ctypes.byref(splits),
                                        ctypes.byref(chunk)) == 0
        ws = ctypes.c_int64()
        assert lib.hmc_reduce_workspace(ctypes.byref(k), ctypes.byref(r), 0, ctypes.byref(ws)) == 0
        return kind.value, splits.value, chunk.value, ws.value
    # rows of [16384, 4096]: enough rows to give every warp one, no split, no workspace
    assert plan([(16384, 4096)], [(4096, 1)]) == (1032, 1, 4096, 0)
    # rows of [1000, 4096]: a block per row
    assert plan([(1000, 4096)], [(4096, 1)]) == (1256, 1, 4096, 0)
    # columns of [16384, 4096]: adjacent outputs, the reduced range cut into chunks with partials
    kind, splits, chunk, ws = plan([(4096, 1)], [(16384, 4096)])
    assert kind == 1 and splits > 1 and splits * chunk >= 16384 and ws == splits * 4096 * 16
    # full reduction of 2^26 elements
    kind, splits, chunk, ws = plan([], [(1 << 26, 1)])
    assert kind == 1256 and splits > 256 and chunk % 1024 == 0 and ws == splits * 16
    # short rows: a warp, or a single lane
    assert plan([(1000, 100)], [(100, 1)])[0] == 1032
    assert plan([(100000, 3)], [(3, 1)])[0] == 1001
