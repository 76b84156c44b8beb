"""The bounds-checked build of the kernel library (``python -m gruboros_b200.build --checks`` -> ``-DGRB_CHECKS``).

compute-sanitizer is not available on the test machines, so the library can check itself instead: in that build every
epilogue, reduce-scatter and gather compares the tile index, rank and element offset it is about to use with the
extents the caller passed; a violation records a status code in the launch's error word and the access is SKIPPED
(nothing traps or faults).  Two things are tested, each in a child process that loads the checked library through
``GRB_LIB``: the ordinary small-shape kernel and sharding tests pass under it with the error word untouched, and
extents that are deliberately too small are reported while the memory behind them stays untouched.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
CHECKED = ROOT / "gruboros_b200" / "lib" / "libgrb_checks.so"


def _env():
    if not CHECKED.exists():
        from gruboros_b200 import build
        build.build(checks=True)
    env = dict(os.environ)
    env["GRB_LIB"] = str(CHECKED)
    return env


def test_kernel_and_sharding_tests_pass_under_the_checked_build():
    res = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "tests/test_kernels_gpu.py", "tests/test_fsdp_gpu.py",
                          "tests/test_dp_gpu.py", "-k", "not bounded_wait"], cwd=str(ROOT), env=_env(), capture_output=True,
                         text=True, timeout=1200)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]


VIOLATIONS = r"""
import torch
from gruboros_b200.ops import kernels as K, _lib as L
assert "checks" in str(L.LIB_PATH)
dev = "cuda"
M, N, Kd, world = 256, 256, 192, 2
dy = torch.randn(Kd, M, device=dev).bfloat16()
x = torch.randn(Kd, N, device=dev).bfloat16()
# reduce-scatter into two "peer" buffers that really hold M*N/2 elements each, declared as holding only a quarter
n = M * N
bufs = [torch.zeros(n, device=dev) for _ in range(world)]
ptrs = [b.data_ptr() for b in bufs]
K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_SCATTER, dy, x, M, N, Kd, ldo=N, scatter=(ptrs, n // world, 0, False, n // 4))
try:
    L.check_device_status()
    raise SystemExit("an out-of-range reduce-scatter offset was not reported")
except RuntimeError as e:
    assert "status 32" in str(e), e
# elements at or beyond the declared extent were never touched; those inside it were written
assert float(bufs[0][n // 4:].abs().max()) == 0.0 and float(bufs[1].abs().max()) == 0.0
assert float(bufs[0][:n // 4].abs().max()) > 0.0
# the same call with the true extent is clean and complete
K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_SCATTER, dy, x, M, N, Kd, ldo=N, scatter=(ptrs, n // world, 0, False, n))
L.check_device_status()
assert float(bufs[1][n // 2:].abs().max()) > 0.0
# chunk gather into a destination declared too small: reported, and nothing is written past the declared capacity
shift = 6
shards = [torch.arange(512, device=dev, dtype=torch.float32).bfloat16() for _ in range(world)]
dst = torch.full((1024,), -1.0, device=dev, dtype=torch.bfloat16)
K.gather_chunks([s.data_ptr() for s in shards], shift, 0, 1024, dst.data_ptr(), 512, 256)
try:
    L.check_device_status()
    raise SystemExit("a gather past the workspace was not reported")
except RuntimeError as e:
    assert "status 33" in str(e), e
assert float(dst[256:].max()) == -1.0 and float(dst[:256].min()) >= 0.0
print("violations reported, memory intact")
"""


def test_violations_are_reported_and_the_access_is_skipped():
    res = subprocess.run([sys.executable, "-c", VIOLATIONS], cwd=str(ROOT), env=_env(), capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "memory intact" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
