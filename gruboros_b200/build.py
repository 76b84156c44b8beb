"""Builds the sm_100a kernels in ``gruboros_b200/csrc`` into ``gruboros_b200/lib/libgrb.so``.

The kernels use inline PTX that only exists on sm_100a, so there is exactly
one target.  Plain ``nvcc`` is used (no torch headers are needed: the library
exposes a C interface that ``gruboros_b200.ops`` drives through ctypes), which
keeps a full rebuild to a few seconds and lets the library cross-compile on a
machine without a GPU.

    python -m gruboros_b200.build [--force] [--verbose] [--checks]

``--checks`` builds a second library, ``lib/libgrb_checks.so``, with ``-DGRB_CHECKS``: every epilogue, scatter and
gather checks the tile index, rank and element offset it is about to use against the extents the caller passed, and
on a violation records a status code in the launch's error word and skips the access (nothing traps).  Select it
with ``GRB_LIB=<path>``; ``tests/test_checks_gpu.py`` runs the small-shape kernel tests against it.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libgrb.so"
OBJDIR = LIBDIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.iterdir()):
        if p.suffix in (".cu", ".cuh", ".h", ".cpp"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, verbose: bool, extra=(), objdir: Path = None) -> Path:
    obj = (objdir or OBJDIR) / (src.stem + ".o")
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}")
    return obj


LIB_CHECKS = LIBDIR / "libgrb_checks.so"


def build(force: bool = False, verbose: bool = False, checks: bool = False) -> Path:
    """Compile every source under ``csrc`` for sm_100a and link ``libgrb.so`` (``checks``: ``libgrb_checks.so`` with
    ``-DGRB_CHECKS``).  Returns its path."""
    LIBDIR.mkdir(exist_ok=True)
    lib = LIB_CHECKS if checks else LIB
    objdir = LIBDIR / ("obj_checks" if checks else "obj")
    objdir.mkdir(exist_ok=True)
    extra = ("-DGRB_CHECKS",) if checks else ()
    stamp = LIBDIR / (lib.stem + ".sha256")
    digest = _digest()
    if not force and lib.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return lib
    nvcc = _nvcc()
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(nvcc, s, verbose, extra, objdir), srcs))
    link = [nvcc, "-shared", "-o", str(lib), *map(str, objs)]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    stamp.write_text(digest)
    return lib


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--checks", action="store_true", help="build lib/libgrb_checks.so with -DGRB_CHECKS")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.checks))


if __name__ == "__main__":
    main()
