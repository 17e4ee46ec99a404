"""The debugging aids, each in a fresh process because they are switched on by the environment:
HOMURA_CUDA_DEBUG=1 (poisoned allocations between guard bands, checked on the host) and HMC_TIMING_LOG (device
time of every entry that queues work)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def run(code: str, **env):
    e = dict(os.environ, **env)
    out = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], cwd=ROOT / "tests", env=e, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    return out.stdout


def test_poison_and_guard_bands():
    out = run("""
        import sys
        sys.path.insert(0, "..")
        import numpy as np
        from homura_b200 import ffi
        from homura_b200.host import BOOL, F32, BF16, I32, BackendError, CudaBackend, TensorData
        be = CudaBackend(0)
        assert be.debug
        # memory nothing wrote: NaN, -1, true
        assert np.isnan(be.download(be.empty((1000,), F32))).all()
        assert (be.download(be.empty((7,), I32)) == -1).all()
        assert (be.download(be.empty((5,), BOOL)) != 0).all()
        # ordinary work on odd shapes leaves every guard band intact
        x = be.upload(np.arange(33 * 1001, dtype=np.float32).reshape(33, 1001), F32)
        y, r, c = be.empty((33, 1001), F32), be.empty((33,), F32), be.empty((1001,), F32)
        be.unary(ffi.HMC_UNARY_SQRT, y, x)
        be.copy(y, x.narrow(1, 0, 1).expand(33, 1001))
        be.reduce(ffi.HMC_REDUCE_SUM, r, x, [False, True])
        be.reduce(ffi.HMC_REDUCE_SUM, c, x, [True, False])
        be.softmax(y, x, 1, False)
        t = be.empty((1001, 33), BF16)
        be.copy(t, x.t())
        be.synchronize()
        be.check_guards()
        # a destination described four elements longer than its storage is refused before anything is queued ...
        from homura_b200 import host
        small = be.empty((12,), F32)
        lying = TensorData(small.storage, F32, (16,), (1,))
        try:
            be.fill(lying, 1.0)
            print("not refused")
        except BackendError as e:
            assert "reaches element 15 of a storage of 12" in str(e), str(e)
        # ... and, with that check switched off (a kernel that went beyond its description), the write lands in the
        # guard band
        host.CHECK_REACH = False
        be.fill(lying, 1.0)
        be.synchronize()
        try:
            be.check_guards()
            print("missed")
        except BackendError as e:
            assert "past its end" in str(e), str(e)
            print("caught")
        be._guarded.clear()
        be.close()
    """, HOMURA_CUDA_DEBUG="1")
    assert "caught" in out and "not refused" not in out


def test_timing_log(tmp_path):
    log = tmp_path / "timing.log"
    run("""
        import sys
        sys.path.insert(0, "..")
        import numpy as np
        from homura_b200 import ffi
        from homura_b200.host import F32, CudaBackend
        be = CudaBackend(0)
        x = be.upload(np.ones(1 << 20, dtype=np.float32), F32)
        y, s = be.empty((1 << 20,), F32), be.empty((), F32)
        for _ in range(3):
            be.unary(ffi.HMC_UNARY_EXP, y, x)
            be.reduce(ffi.HMC_REDUCE_SUM, s, y, [True])
        be.synchronize()
        be.close()
    """, HMC_TIMING_LOG=str(log), HMC_NVTX="1")
    lines = [l.split("\t") for l in log.read_text().splitlines()]
    names = [l[0] for l in lines]
    assert names.count("hmc_unary") == 3 and names.count("hmc_reduce") == 3, names
    assert "hmc_copy_from_host" in names
    assert all(float(l[1]) >= 0.0 for l in lines if l[0] in ("hmc_unary", "hmc_reduce"))
