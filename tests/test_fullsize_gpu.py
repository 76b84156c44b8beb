"""Full-size numerics of the tcgen05 GEMM epilogues: M = 16376 rows (8 x 2047, ragged: 63.97 row tiles of 256, more
than one wave of the persistent scheduler, split-K with real wave counts) and the 1B model's N / K, checked on
sampled rows and columns against an fp64 product of the same bf16 operands.  The small-shape tests cover every
branch; these cover tile wrap-around, the ragged last row tile and 64 k-blocks and more per tile."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gruboros_b200.ops import kernels as K
    from gruboros_b200.ops import _lib as L

DEV = "cuda"
M = 8 * 2047
D, DI, FH = 2048, 3072, 8192


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def sample_rows(n=64):
    g = torch.Generator().manual_seed(5)
    rows = torch.randint(0, M, (n,), generator=g)
    rows[:4] = torch.tensor([0, 255, M - 1, M - 120])        # first tile, tile edge, last (ragged) tile
    return rows.to(DEV)


def close(got, want, rtol, atol, what):
    got, want = got.double(), want.double()
    err = (got - want).abs()
    bad = err > atol + rtol * want.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} mismatches, max err {err.max().item():.4g}"


def test_store_bf16_gate_shape():
    a, b = rnd(M, D), rnd(2 * DI, D, scale=0.05)
    out = torch.full((M, 2 * DI), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, a, b, M, 2 * DI, D, out0=out)
    L.check_device_status()
    assert not torch.isnan(out.float()).any()
    r = sample_rows()
    close(out[r], a[r].double() @ b.double().t(), 1e-2, 2e-2, "gate shape, bf16 store")


def test_bias_gelu_ff1_shape():
    a, b = rnd(M, D), rnd(FH, D, scale=0.03)
    bias = torch.randn(FH, device=DEV)
    der = torch.full((M, FH), float("nan"), device=DEV, dtype=torch.bfloat16)
    act = torch.full_like(der, float("nan"))
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_BIAS_GELU, a, b, M, FH, D, out0=der, out1=act, bias=bias)
    L.check_device_status()
    assert not torch.isnan(act.float()).any() and not torch.isnan(der.float()).any()
    r = sample_rows()
    pre = (a[r].double() @ b.double().t() + bias.double()).requires_grad_(True)
    g = torch.nn.functional.gelu(pre)
    g.sum().backward()
    close(act[r], g.detach(), 1e-2, 2e-2, "FF1 shape, gelu")
    close(der[r], pre.grad, 1e-2, 1e-2, "FF1 shape, gelu'")


def test_residual_with_next_norm_ff2_shape_and_consumer():
    a, b = rnd(M, FH, scale=0.5), rnd(D, FH, scale=0.03)
    resid = torch.randn(M, D, device=DEV)
    bias, w = torch.randn(D, device=DEV), torch.randn(D, device=DEV)
    x = torch.full((M, D), float("nan"), device=DEV)
    xw = torch.full((M, D), float("nan"), device=DEV, dtype=torch.bfloat16)
    ssq = torch.full((M, D // 128), float("nan"), device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_RESID_F32, a, b, M, D, FH, out0=x, aux=resid, bias=bias, next_norm=(w, xw, ssq))
    L.check_device_status()
    assert not torch.isnan(x).any() and not torch.isnan(ssq).any() and not torch.isnan(xw.float()).any()
    r = sample_rows()
    xref = resid[r].double() + a[r].double() @ b.double().t() + bias.double()
    close(x[r], xref, 1e-4, 3e-2, "FF2 shape, residual")
    close(xw[r], x[r].double() * w.double(), 1e-2, 1e-2, "x * w")
    close(ssq.double().sum(1), x.double().pow(2).sum(1), 1e-4, 1e-2, "sums of squares, all rows")
    # consumer: gate GEMM on the unnormalised operand, rows scaled in the epilogue
    eps = torch.finfo(torch.float32).eps
    wg = rnd(2 * DI, D, scale=0.05)
    ku = torch.full((M, 2 * DI), float("nan"), device=DEV, dtype=torch.bfloat16)
    rstd = torch.full((M,), float("nan"), device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, xw, wg, M, 2 * DI, D, out0=ku, rownorm=(ssq, D, eps, rstd))
    L.check_device_status()
    rs = torch.rsqrt(x.double().pow(2).mean(1) + eps)
    close(rstd, rs, 1e-5, 1e-6, "rstd of every row")
    close(ku[r], (xw[r].double() @ wg.double().t()) * rs[r][:, None], 1e-2, 2e-2, "gate GEMM with folded norm")


def test_gelu_bwd_dgrad_shape_with_colsum():
    dy, w2 = rnd(M, D, scale=0.5), rnd(D, FH, scale=0.03)
    saved = rnd(M, FH)
    rowscale = torch.rand(M, device=DEV) + 0.5
    out = torch.full((M, FH), float("nan"), device=DEV, dtype=torch.bfloat16)
    csum = torch.zeros(FH, device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_GELU_BWD, dy, w2, M, FH, D, out0=out, aux=saved, rowscale=rowscale, colsum=csum)
    L.check_device_status()
    r = sample_rows()
    raw = (dy[r].double() @ w2.double()) * saved[r].double()
    close(out[r], raw * rowscale[r].double()[:, None], 1e-2, 2e-2, "FF2 dgrad shape, gelu' x row scale")
    cols = torch.arange(0, FH, 97, device=DEV)
    full = (dy.double() @ w2[:, cols].double()) * saved[:, cols].double()
    close(csum[cols], full.sum(0), 2e-3, 2e-3 * math.sqrt(M), "bias-gradient column sums")


@pytest.mark.parametrize("splitk", [1, 2, 4, -1])
def test_wgrad_red_gate_shape(splitk):
    dy, x = rnd(M, 2 * DI, scale=0.5), rnd(M, D)
    base = torch.randn(2 * DI, D, device=DEV)
    out = base.clone()
    K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_F32, dy, x, 2 * DI, D, M, out0=out, ldo=D, splitk=splitk)
    L.check_device_status()
    rows = torch.tensor([0, 1, 255, 256, 3071, 3072, 6143, 4000], device=DEV)
    want = base[rows].double() + dy[:, rows].double().t() @ x.double()
    close(out[rows], want, 1e-3, 2e-3 * math.sqrt(M), f"gate wgrad, split-K {splitk}")


@pytest.mark.parametrize("n_out,k_out", [(256, 2048), (2048, 8192)])
def test_wgrad_stream_k_other_shapes(n_out, k_out):
    """Stream-K where a pair's run covers a fraction of a tile (8 tiles over 74 pairs) and where it covers several."""
    dy, x = rnd(M, n_out, scale=0.5), rnd(M, k_out)
    out = torch.zeros(n_out, k_out, device=DEV)
    K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_F32, dy, x, n_out, k_out, M, out0=out, ldo=k_out, splitk=-1)
    L.check_device_status()
    rows = torch.tensor([0, 1, 127, 128, 255, n_out - 1], device=DEV)
    want = dy[:, rows].double().t() @ x.double()
    close(out[rows], want, 1e-3, 2e-3 * math.sqrt(M), "stream-K wgrad")


def test_cross_entropy_full_rows():
    x, w = rnd(M, D), rnd(256, D, scale=0.05)
    labels = torch.randint(0, 256, (M,), device=DEV, dtype=torch.uint8)
    loss_rows = torch.full((M,), float("nan"), device=DEV)
    dlog = torch.full((M, 256), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, x, w, M, 256, D, out0=dlog, out1=loss_rows, aux=labels, ldo=256, alpha=1.0)
    L.check_device_status()
    logits = (x.double() @ w.double().t()).requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(logits, labels.long(), reduction="none")
    ref.sum().backward()
    close(loss_rows, ref.detach(), 1e-4, 2e-3, "cross-entropy of every row")
    close(dlog, logits.grad, 2e-2, 4e-3, "d logits of every row")
