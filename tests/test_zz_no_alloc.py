"""The allocation-free cross-entropy entry point (``csrc/ce_static.h``) against the regular two-kernel path.

Some hosts of the kernel library cannot allocate device memory when they call it: they run inside another
runtime's memory pool, or every byte of the GPU was handed out at start-up, or they sit in a loop that must not
risk the device-wide synchronisation an allocation can cause.  For them ``grb_ce_loss_static`` keeps the per-row
loss buffer that sits between the logits GEMM and the loss reduction in a fixed device array inside the library.
The test calls it through its exported C symbol, several times in a row with different sizes (the array keeps the
previous call's contents, which must not matter), and compares with ``gemm(EPI_CE)`` + ``sum_scale`` on buffers
that torch allocated.  This file sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gruboros_b200.ops import kernels as K
    from gruboros_b200.ops import _lib as L

DEV = "cuda"
MAX_ROWS = 131072      # GRB_CE_STATIC_MAX_ROWS


def _entry():
    fn = L.lib().grb_ce_loss_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                   C.c_int64, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
    return fn


def _case(M, V, D, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = torch.randn(M, D, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(V, D, device=DEV, generator=g) * 0.2).to(torch.bfloat16)
    labels = torch.randint(0, V, (M,), device=DEV, dtype=torch.uint8, generator=g)
    return x, w, labels


def _regular(x, w, labels, with_grad):
    M, D = x.shape
    V = w.shape[0]
    rows = torch.zeros(M, device=DEV)
    dlog = torch.zeros(M, V, device=DEV, dtype=torch.bfloat16) if with_grad else None
    loss = torch.zeros(1, device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, x, w, M, V, D, out0=dlog, out1=rows, aux=labels, ldo=V, alpha=1.0 / M)
    K.sum_scale(rows, 1.0 / M, loss)
    return loss, dlog


def _static(fn, x, w, labels, with_grad):
    M, D = x.shape
    V = w.shape[0]
    dlog = torch.zeros(M, V, device=DEV, dtype=torch.bfloat16) if with_grad else None
    loss = torch.full((1,), float("nan"), device=DEV)
    rc = fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), labels.data_ptr(), M, V, D, L.ptr(dlog), V,
            1.0 / M, 1.0 / M, loss.data_ptr(), L.err_flag(x.device).data_ptr(), L.stream())
    assert rc == 0, f"grb_ce_loss_static returned {rc}"
    return loss, dlog


def test_static_cross_entropy_matches_regular_path_on_consecutive_calls():
    fn = _entry()
    # big first, then smaller ones, so that later calls find stale losses of earlier rows in the shared array;
    # the last case has enough row tiles for the CTA-pair kernel
    for M, V, D, with_grad, seed in [(1000, 256, 264, True, 1), (300, 200, 128, True, 2), (77, 256, 64, False, 3),
                                     (12800, 256, 128, True, 4)]:
        x, w, labels = _case(M, V, D, seed)
        want_loss, want_d = _regular(x, w, labels, with_grad)
        got_loss, got_d = _static(fn, x, w, labels, with_grad)
        L.check_device_status()
        ref = torch.nn.functional.cross_entropy(x.float() @ w.float().t(), labels.long())
        torch.testing.assert_close(got_loss, want_loss, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(got_loss[0], ref, rtol=1e-4, atol=1e-3)
        if with_grad:
            torch.testing.assert_close(got_d.float(), want_d.float(), rtol=2e-2, atol=4e-3 / M)


def test_static_cross_entropy_rejects_more_rows_than_the_array_holds():
    fn = _entry()
    x, w, labels = _case(8, 256, 64, 5)
    loss = torch.zeros(1, device=DEV)
    rc = fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), labels.data_ptr(), MAX_ROWS + 1, 256, 64, None, 256,
            1.0, 1.0, loss.data_ptr(), L.err_flag(x.device).data_ptr(), L.stream())
    assert rc == -60
    rc = fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), labels.data_ptr(), 0, 256, 64, None, 256,
            1.0, 1.0, loss.data_ptr(), L.err_flag(x.device).data_ptr(), L.stream())
    assert rc == -60
