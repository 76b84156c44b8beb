"""Kernels whose reduction order is fixed must give bit-identical results when run twice on the same inputs, and
must not touch anything outside their outputs (guard zones filled with a NaN pattern around every output)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gruboros_b200.ops import kernels as K
    from gruboros_b200.ops import _lib as L

DEV = "cuda"
GUARD = 64


def guarded(shape, dtype):
    """A tensor of `shape` carved out of a NaN-filled buffer with guard elements on both sides."""
    n = 1
    for d in shape:
        n *= d
    n_al = (n + 63) // 64 * 64
    buf = torch.full((n_al + 2 * GUARD,), float("nan"), device=DEV, dtype=dtype)
    return buf, buf[GUARD:GUARD + n].view(*shape)


def guards_intact(buf, n):
    n_al = (n + 63) // 64 * 64
    return bool(torch.isnan(buf[:GUARD]).all()) and bool(torch.isnan(buf[GUARD + n:GUARD + n_al + GUARD]).all())


def rnd(*s):
    return torch.randn(*s, device=DEV).bfloat16()


def twice(run, outs):
    """run() writes the tensors in `outs` (list of (buffer, view)); returns nothing.  Checks equality of two runs."""
    run()
    torch.cuda.synchronize()
    first = [v.clone() for _, v in outs]
    for _, v in outs:
        v.fill_(float("nan"))
    run()
    torch.cuda.synchronize()
    for (buf, v), f in zip(outs, first):
        assert not torch.isnan(v.float()).any(), "an output element was not written"
        assert torch.equal(v, f), "two runs differ"
        assert guards_intact(buf, v.numel()), "a guard zone was overwritten"
    L.check_device_status()


@pytest.mark.parametrize("mode", ["1cta", "2cta"])
@pytest.mark.parametrize("M,N,Kd", [(300, 200, 136), (1000, 776, 520)])
def test_gemm_store_epilogues_are_deterministic(mode, M, N, Kd):
    old, K.GEMM_MODE = K.GEMM_MODE, mode
    try:
        a, b, bias = rnd(M, Kd), rnd(N, Kd), torch.randn(N, device=DEV)
        o16 = guarded((M, N), torch.bfloat16)
        twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, a, b, M, N, Kd, out0=o16[1]), [o16])
        o32 = guarded((M, N), torch.float32)
        twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_F32, a, b, M, N, Kd, out0=o32[1]), [o32])
        pre, act = guarded((M, N), torch.bfloat16), guarded((M, N), torch.bfloat16)
        twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_BIAS_GELU, a, b, M, N, Kd, out0=pre[1], out1=act[1], bias=bias), [pre, act])
        res = torch.randn(M, N, device=DEV)
        out = guarded((M, N), torch.float32)
        twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_RESID_F32, a, b, M, N, Kd, out0=out[1], aux=res), [out])
    finally:
        K.GEMM_MODE = old


@pytest.mark.parametrize("mode", ["1cta", "2cta"])
def test_folded_rmsnorm_is_deterministic(mode):
    """The partial sums of squares are stored per 128-column part and added in a fixed order (no atomics), so the
    producer's outputs and the consumer's row-scaled result are bitwise reproducible; guard zones stay intact."""
    old, K.GEMM_MODE = K.GEMM_MODE, mode
    try:
        M, D, Kp, N = 300, 520, 136, 200
        a, b, res, w = rnd(M, Kp), rnd(D, Kp), torch.randn(M, D, device=DEV), torch.randn(D, device=DEV)
        parts = (D + 127) // 128
        x, xw, ssq = guarded((M, D), torch.float32), guarded((M, D), torch.bfloat16), guarded((M, parts), torch.float32)
        twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_RESID_F32, a, b, M, D, Kp, out0=x[1], aux=res,
                             next_norm=(w, xw[1], ssq[1])), [x, xw, ssq])
        wc = rnd(N, D)
        o16, rstd = guarded((M, N), torch.bfloat16), guarded((M,), torch.float32)
        xw_in, ssq_in = xw[1].clone(), ssq[1].clone()
        twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, xw_in, wc, M, N, D, out0=o16[1],
                             rownorm=(ssq_in, D, 1e-6, rstd[1])), [o16, rstd])
    finally:
        K.GEMM_MODE = old


def test_cross_entropy_epilogue_is_deterministic():
    M, V, D = 513, 256, 128
    x, w = rnd(M, D), rnd(V, D) * 0.2
    labels = torch.randint(0, V, (M,), device=DEV, dtype=torch.uint8)
    loss, dlog = guarded((M,), torch.float32), guarded((M, V), torch.bfloat16)
    twice(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, x, w, M, V, D, out0=dlog[1], out1=loss[1], aux=labels, ldo=V, alpha=1.0 / M),
          [loss, dlog])


@pytest.mark.parametrize("B,T,Cc", [(2, 131, 192), (3, 64, 64)])
def test_scan_is_deterministic(B, T, Cc):
    ku, g = rnd(B, T, 2 * Cc), rnd(B, T, Cc)
    h0 = torch.rand(B, Cc, device=DEV) + 0.1
    h, hl = guarded((B, T, Cc), torch.bfloat16), guarded((B, Cc), torch.float32)
    twice(lambda: K.scan_fwd(ku[..., Cc:], ku[..., :Cc], h[1], h0=h0, h_last=hl[1]), [h, hl])
    dku, dh0 = guarded((B, T, 2 * Cc), torch.bfloat16), guarded((B, Cc), torch.float32)
    hh = h[1].clone()
    twice(lambda: K.scan_bwd(ku[..., Cc:], ku[..., :Cc], hh, g, dku[1][..., Cc:], dku[1][..., :Cc], h0=h0, dh0=dh0[1]), [dku, dh0])


def test_rmsnorm_forward_and_optimizer_are_deterministic():
    M, D = 129, 520
    x, w = torch.randn(M, D, device=DEV), torch.rand(D, device=DEV) + 0.5
    y, rstd = guarded((M, D), torch.bfloat16), guarded((M,), torch.float32)
    twice(lambda: K.rmsnorm_fwd(x, w, y[1], rstd[1], 1e-6), [y, rstd])
    n = 100_003 // 64 * 64
    y0, z0, v0, g0 = (torch.randn(n, device=DEV) for _ in range(4))
    v0.abs_()
    yb, zb, vb, gb = (guarded((n,), torch.float32) for _ in range(4))
    wb = guarded((n,), torch.bfloat16)

    def run():
        for (_, dst), src in zip((yb, zb, vb, gb), (y0, z0, v0, g0)):
            dst.copy_(src)
        K.sfadamw_step(yb[1], zb[1], vb[1], gb[1], wb[1], lr=1e-3, beta1=0.9, beta2=0.995, bias2=0.3, eps=1e-8, wd=1e-2, ckp1=0.2)

    twice(run, [yb, zb, vb, gb, wb])


def test_decode_gemv_is_deterministic():
    B, N, Kd = 3, 200, 1032
    x, w = torch.randn(B, Kd, device=DEV), rnd(N, Kd) * 0.03
    nw, bias = torch.rand(Kd, device=DEV) + 0.5, torch.randn(N, device=DEV)
    out = guarded((B, N), torch.float32)
    twice(lambda: K.decode_gemv(K.DEC_GELU, x, w, out[1], norm_w=nw, bias=bias, eps=1e-6), [out])
