"""ctypes binding of ``libgrb.so`` (the sm_100a kernels under ``gruboros_b200/csrc``).

The library has a plain C interface taking raw device pointers and a CUDA
stream, so calls cost a few microseconds of host time and need no torch
headers at build time.  ``lib()`` raises if the library is missing: on a GPU
machine the CUDA path must never silently fall back to eager PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB = None
LIB_PATH = Path(os.environ.get("GRB_LIB") or Path(__file__).resolve().parent.parent / "lib" / "libgrb.so")

MAJOR_K, MAJOR_MN = 0, 1
EPI_STORE_BF16, EPI_STORE_F32, EPI_BIAS_GELU, EPI_RESID_F32, EPI_GELU_BWD, EPI_RED_F32, EPI_CE, EPI_RED_SCATTER = range(8)


class EpiArgs(C.Structure):
    _fields_ = [
        ("out0", C.c_void_p),
        ("out1", C.c_void_p),
        ("aux", C.c_void_p),
        ("bias", C.c_void_p),
        ("ldo", C.c_int64),
        ("alpha", C.c_float),
        ("rowss", C.c_void_p),
        ("rowss_parts", C.c_int),
        ("rowss_inv_d", C.c_float),
        ("rowss_eps", C.c_float),
        ("rstd_out", C.c_void_p),
        ("out2", C.c_void_p),
        ("normw", C.c_void_p),
        ("ssq_out", C.c_void_p),
        ("colsum", C.c_void_p),
        ("world", C.c_int),
        ("chunk_aligned", C.c_int),
        ("flat_off", C.c_int64),
        ("shard", C.c_int64),
        ("peers", C.c_void_p * 8),
        ("compact", C.c_int),
        ("n_copy", C.c_int),
        ("copy_src", C.c_void_p * 8),
        ("copy_dst", C.c_void_p * 8),
        ("copy_bytes", C.c_int64 * 8),
        ("gather_lo", C.c_int64),
        ("gather_hi", C.c_int64),
        ("gather_dst", C.c_void_p),
        ("peer_limit", C.c_int64),
        ("gather_cap", C.c_int64),
        ("chk_err", C.c_void_p),
    ]


_P, _I, _L, _F = C.c_void_p, C.c_int, C.c_int64, C.c_float

_SIGS = {
    "grb_gemm": [_I, _I, _I, _P, _L, _P, _L, _I, _I, _I, _I, C.POINTER(EpiArgs), _P, _I, _P],
    "grb_gemm_pair": [_I, _I, _I, _P, _L, _P, _L, _I, _I, _I, _I, C.POINTER(EpiArgs), _P, _I, _P],
    "grb_gather_chunks": [C.POINTER(C.c_void_p), _I, _I, _L, _L, _P, _L, _L, _P, _P],
    "grb_copy_segments": [_I, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64), _P],
    "grb_scan_fwd": [_P, _P, _L, _P, _P, _L, _P, _I, _I, _I, _P, _P],
    "grb_scan_bwd": [_P, _P, _L, _P, _L, _P, _L, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _P, _P],
    "grb_embed_fwd": [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _P],
    "grb_rmsnorm_fwd": [_P, _P, _P, _P, _L, _I, _F, _P],
    "grb_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _P, _P],
    "grb_colsum_bf16": [_P, _L, _L, _I, _P, _P],
    "grb_sum_scale": [_P, _L, _F, _P, _I, _P],
    "grb_cast_f32_bf16": [_P, _P, _L, _P],
    "grb_sfadamw_interleaved_step": [_P, _P, _P, _P, _P, _I, _I, _I, _L, _F, _F, _F, _F, _F, _F, _F, _F, _I, _L, _P, _P],
    "grb_sfadamw_interleaved_range_step": [_P, _P, _P, _P, _P, _I, _I, _I, _L, _L, _F, _F, _F, _F, _F, _F, _F, _F, _I, _L, _P, _P],
    "grb_gather_interleaved": [_P, _P, _I, _I, _I, _L, _I, _I, _P],
    "grb_sample": [_P, _I, _I, _F, _I, _F, _P, C.c_uint64, _P, _P, _P, _I, _P, _P],
    "grb_decode_tc": [_I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "grb_decode_gemv": [_I, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    "grb_sfadamw_step": [_P, _P, _P, _P, _P, _L, _F, _F, _F, _F, _F, _F, _F, _F, _I, _P],
    "grb_merge": [_P, _P, _F, _P, _P, _F, _P, _P, _F, _P, _L, _P],
}


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    """Load (once) and return the kernel library; raises if it has not been built."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -m gruboros_b200.build` (needs nvcc) before using the CUDA path"
            )
        _LIB = C.CDLL(str(LIB_PATH))
        for name, sig in _SIGS.items():
            fn = getattr(_LIB, name, None)
            if fn is None:
                continue
            fn.argtypes = sig
            fn.restype = C.c_int
    return _LIB


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: kernel library returned error {rc}")


_ERR = {}


def err_flag(device=None) -> torch.Tensor:
    """Per-device int32 word that bounded device-side waits set when they give up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _ERR.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _ERR[dev] = t
    return t


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a timed-out wait."""
    flag = err_flag(device)
    code = int(flag.item())
    if code != 0:
        flag.zero_()
        raise RuntimeError(f"device-side wait timed out (status {code}); results of the last launches are invalid")
