"""Numerics of every sm_100a kernel against a plain PyTorch fp32/fp64 restatement of the same op.

bf16 operands are generated on the bf16 grid, so the only differences are accumulation order
(fp32 in tensor memory vs. fp32/fp64 in PyTorch) and the rounding of bf16 outputs.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from gruboros_b200.ops import kernels as K
    from gruboros_b200.ops import reference as R
    from gruboros_b200.ops import _lib as L

DEV = "cuda"


@pytest.fixture(params=["1cta", "2cta"])
def gemm_mode(request):
    """Run a GEMM test with the single-CTA kernel and with the CTA-pair (cta_group::2) kernel."""
    old = K.GEMM_MODE
    K.GEMM_MODE = request.param
    yield request.param
    K.GEMM_MODE = old


def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV) * scale).to(dtype)


def assert_close(got, want, rtol, atol, what=""):
    got, want = got.double(), want.double()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = err > tol
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} mismatches, max err {err.max().item():.4g}, "
            f"first at {idx}: got {got[tuple(idx)].item():.6g} want {want[tuple(idx)].item():.6g}")


GEMM_SHAPES = [(128, 256, 64), (256, 512, 256), (384, 256, 1024), (300, 200, 136), (1000, 776, 520), (64, 8, 64)]


@pytest.mark.parametrize("M,N,Kd", GEMM_SHAPES)
def test_gemm_forward_layout(M, N, Kd, gemm_mode):
    a, b = rnd(M, Kd), rnd(N, Kd)
    out = torch.full((M, N), float("nan"), device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_F32, a, b, M, N, Kd, out0=out)
    L.check_device_status()
    assert_close(out, a.float() @ b.float().t(), 1e-4, 1e-3 * math.sqrt(Kd), "KK gemm")


@pytest.mark.parametrize("M,N,Kd", GEMM_SHAPES[:5])
def test_gemm_dgrad_layout(M, N, Kd, gemm_mode):
    # D[M,N] = A[M,K] @ Bt[K,N] with Bt read MN-major
    a, bt = rnd(M, Kd), rnd(Kd, N)
    out = torch.full((M, N), float("nan"), device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_STORE_F32, a, bt, M, N, Kd, out0=out)
    L.check_device_status()
    assert_close(out, a.float() @ bt.float(), 1e-4, 1e-3 * math.sqrt(Kd), "K-MN gemm")


@pytest.mark.parametrize("M,N,Kd", GEMM_SHAPES[:5])
@pytest.mark.parametrize("splitk", [1, 3, -1])
def test_gemm_wgrad_layout(M, N, Kd, splitk, gemm_mode):
    # D[M,N] = At[K,M]^T @ Bt[K,N], both MN-major, accumulated by red.add into a pre-filled buffer
    M = (M + 7) // 8 * 8   # the leading dimension of an MN-major operand must be a multiple of 8 elements
    at, bt = rnd(Kd, M), rnd(Kd, N)
    base = torch.randn(M, N, device=DEV)
    out = base.clone()
    K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_F32, at, bt, M, N, Kd, out0=out, splitk=splitk)
    L.check_device_status()
    assert_close(out, base + at.float().t() @ bt.float(), 1e-4, 1e-3 * math.sqrt(Kd), "MN-MN gemm")


def test_gemm_epilogues(gemm_mode):
    M, N, Kd = 300, 520, 264
    a, b = rnd(M, Kd, scale=0.5), rnd(N, Kd, scale=0.5)
    bias = torch.randn(N, device=DEV)
    ref = a.float() @ b.float().t()
    # bf16 store with alpha
    o = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, a, b, M, N, Kd, out0=o, alpha=0.5)
    assert_close(o, 0.5 * ref, 1e-2, 1e-2, "store bf16")
    # bias + gelu: derivative (saved for backward) and activation
    der = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    act = torch.zeros_like(der)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_BIAS_GELU, a, b, M, N, Kd, out0=der, out1=act, bias=bias)
    pre64 = (ref + bias).double().requires_grad_(True)
    torch.nn.functional.gelu(pre64).sum().backward()
    assert_close(der, pre64.grad, 1e-2, 1e-2, "gelu derivative")
    assert_close(act, torch.nn.functional.gelu(ref + bias), 1e-2, 2e-2, "gelu")
    # residual: out = resid + acc + bias, separate input and output buffers, and in place
    resid = torch.randn(M, N, device=DEV)
    o32 = torch.zeros(M, N, device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_RESID_F32, a, b, M, N, Kd, out0=o32, aux=resid, bias=bias)
    assert_close(o32, resid + ref + bias, 1e-4, 2e-2, "residual")
    inplace = resid.clone()
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_RESID_F32, a, b, M, N, Kd, out0=inplace, aux=inplace)
    assert_close(inplace, resid + ref, 1e-4, 2e-2, "residual in place")
    # gelu backward on a dgrad-layout GEMM: accumulator x saved derivative, optional row scale, bias-gradient column sums
    bt = rnd(Kd, N, scale=0.5)
    saved = rnd(M, N)
    ref2 = a.float() @ bt.float()
    og = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_GELU_BWD, a, bt, M, N, Kd, out0=og, aux=saved)
    assert_close(og, ref2 * saved.float(), 1e-2, 2e-2, "gelu bwd")
    rowscale = torch.rand(M, device=DEV) + 0.5
    csum = torch.ones(N, device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_GELU_BWD, a, bt, M, N, Kd, out0=og, aux=saved, rowscale=rowscale, colsum=csum)
    L.check_device_status()
    assert_close(og, ref2 * saved.float() * rowscale[:, None], 1e-2, 2e-2, "gelu bwd, row scale")
    assert_close(csum, 1 + (ref2.double() * saved.double()).sum(0), 1e-3, 1e-3 * math.sqrt(M), "gelu bwd column sums")


@pytest.mark.parametrize("M,D,N", [(300, 2048, 520), (1000, 3072, 264), (130, 128, 256), (77, 320, 64)])
def test_rmsnorm_folded_into_gemms(M, D, N, gemm_mode):
    """Producer (residual epilogue) leaves bf16 x * w and partial sums of x^2; consumers scale accumulator rows."""
    Kp = 136
    a, b = rnd(M, Kp, scale=0.5), rnd(D, Kp, scale=0.5)
    resid = torch.randn(M, D, device=DEV)
    bias = torch.randn(D, device=DEV)
    w = torch.randn(D, device=DEV)
    eps = torch.finfo(torch.float32).eps
    parts = (D + 127) // 128
    x = torch.full((M, D), float("nan"), device=DEV)
    xw = torch.full((M, D), float("nan"), device=DEV, dtype=torch.bfloat16)
    ssq = torch.full((M, parts), float("nan"), device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_RESID_F32, a, b, M, D, Kp, out0=x, aux=resid, bias=bias, next_norm=(w, xw, ssq))
    L.check_device_status()
    xref = resid.double() + a.double() @ b.double().t() + bias.double()
    assert_close(x, xref, 1e-4, 2e-2, "residual stream")
    assert_close(xw, x.double() * w.double(), 1e-2, 1e-2, "x * w")
    assert_close(ssq.double().sum(1), x.double().pow(2).sum(1), 1e-4, 1e-3, "sum of squares")
    # consumers: bf16 store, fp32 store, bias + GELU, cross-entropy - all equal rmsnorm(x, w) @ wc^T
    wc = rnd(N, D, scale=0.2)
    rs = torch.rsqrt(x.double().pow(2).mean(1) + eps)
    want = (xw.double() @ wc.double().t()) * rs[:, None]
    rstd = torch.full((M,), float("nan"), device=DEV)
    o16 = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, xw, wc, M, N, D, out0=o16, rownorm=(ssq, D, eps, rstd))
    assert_close(o16, want, 1e-2, 2e-2, "folded norm, bf16 store")
    assert_close(rstd, rs, 1e-5, 1e-6, "rstd out")
    o32 = torch.zeros(M, N, device=DEV)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_F32, xw, wc, M, N, D, out0=o32, rownorm=(ssq, D, eps, None))
    assert_close(o32, want, 1e-4, 2e-2, "folded norm, fp32 store")
    bn = torch.randn(N, device=DEV)
    der, act = torch.zeros_like(o16), torch.zeros_like(o16)
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_BIAS_GELU, xw, wc, M, N, D, out0=der, out1=act, bias=bn, rownorm=(ssq, D, eps, None))
    assert_close(act, torch.nn.functional.gelu(want + bn.double()), 1e-2, 2e-2, "folded norm, gelu")
    if N <= 256:
        labels = torch.randint(0, N, (M,), device=DEV, dtype=torch.uint8)
        loss_rows = torch.zeros(M, device=DEV)
        dlog = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, xw, wc, M, N, D, out0=dlog, out1=loss_rows, aux=labels, ldo=N, alpha=0.5,
               rownorm=(ssq, D, eps, rstd))
        logits = want.clone().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(logits, labels.long(), reduction="none")
        ref.sum().backward()
        assert_close(loss_rows, ref.detach(), 1e-4, 2e-3, "folded norm, ce loss")
        assert_close(dlog.float(), 0.5 * logits.grad * rs[:, None], 2e-2, 4e-3 * rs.max().item(), "folded norm, ce grad (x rstd)")
    L.check_device_status()
    # the consumer's x wrapped into the usual form: x * rstd * w
    assert_close((xw.double() * rs[:, None]), R.rmsnorm_ref(x.double(), w.double(), eps), 1e-2, 1e-2, "normalised operand")



@pytest.mark.parametrize("M,V,D", [(300, 256, 264), (513, 200, 128)])
def test_gemm_cross_entropy(M, V, D, gemm_mode):
    x, w = rnd(M, D), rnd(V, D, scale=0.2)
    labels = torch.randint(0, V, (M,), device=DEV, dtype=torch.uint8)
    loss_rows = torch.zeros(M, device=DEV)
    dlog = torch.zeros(M, V, device=DEV, dtype=torch.bfloat16)
    scale = 1.0 / M
    K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, x, w, M, V, D, out0=dlog, out1=loss_rows, aux=labels, alpha=scale)
    L.check_device_status()
    logits = (x.float() @ w.float().t()).requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(logits, labels.long(), reduction="none")
    ref.sum().backward()
    assert_close(loss_rows, ref.detach(), 1e-4, 1e-3, "ce loss")
    assert_close(dlog.float() / scale, logits.grad, 2e-2, 4e-3, "ce grad")


SCAN_SHAPES = [(2, 1, 64), (2, 5, 64), (3, 64, 128), (2, 65, 192), (2, 200, 72), (1, 2047, 64), (2, 300, 8)]


@pytest.mark.parametrize("B,T,Cc", SCAN_SHAPES)
@pytest.mark.parametrize("carry", [False, True])
def test_scan_forward_backward(B, T, Cc, carry):
    ld = 2 * Cc + 8          # row stride larger than the two halves, still a multiple of 8
    ku = rnd(B, T, ld)
    u, k = ku[..., :Cc], ku[..., Cc:2 * Cc]
    h0 = torch.rand(B, Cc, device=DEV) + 0.1 if carry else None
    h = torch.full((B, T, Cc), float("nan"), device=DEV, dtype=torch.bfloat16)
    h_last = torch.zeros(B, Cc, device=DEV)
    K.scan_fwd(k, u, h, h0=h0, h_last=h_last)
    L.check_device_status()
    kd, ud = k.double().requires_grad_(True), u.double().requires_grad_(True)
    h0d = h0.double().requires_grad_(True) if carry else None
    href, hl = R.scan_ref(kd, ud, h0d)
    assert_close(h, href.detach(), 1e-2, 1e-3, "scan fwd")
    assert_close(h_last, hl.detach(), 1e-4, 1e-5, "scan h_last")
    # backward, using the bf16 forward output as the saved activation like the training path does
    g = rnd(B, T, Cc)
    dh_last = torch.randn(B, Cc, device=DEV) if carry else None
    loss = (href * g.double()).sum()
    if carry:
        loss = loss + (hl * dh_last.double()).sum()
    loss.backward()
    dku = torch.full((B, T, ld), float("nan"), device=DEV, dtype=torch.bfloat16)
    du, dk = dku[..., :Cc], dku[..., Cc:2 * Cc]
    dh0 = torch.zeros(B, Cc, device=DEV)
    K.scan_bwd(k, u, h, g, dk, du, h0=h0, dh_last=dh_last, dh0=dh0)
    L.check_device_status()
    scale = max(1.0, kd.grad.abs().max().item())
    assert_close(dk, kd.grad, 3e-2, 1e-2 * scale, "scan dk")
    assert_close(du, ud.grad, 3e-2, 1e-2 * scale, "scan du")
    if carry:
        assert_close(dh0, h0d.grad, 1e-3, 1e-3 * scale, "scan dh0")
    # per-row scale on the outputs (the rstd of a norm folded into the GEMM that produced k, u)
    rowscale = torch.rand(B * T, device=DEV) + 0.5
    K.scan_bwd(k, u, h, g, dk, du, h0=h0, dh_last=dh_last, dh0=dh0, rowscale=rowscale)
    L.check_device_status()
    rsb = rowscale.view(B, T, 1).double()
    assert_close(dk, kd.grad * rsb, 3e-2, 1.5e-2 * scale, "scan dk, row scale")
    assert_close(du, ud.grad * rsb, 3e-2, 1.5e-2 * scale, "scan du, row scale")


def test_scan_outputs_whose_rows_are_not_16_byte_multiples():
    """h, dk, du with a row stride of 68 elements (136 bytes) cannot have tensor maps: the kernels then store from the
    lanes instead of through bulk tensor stores; same results."""
    B, T, Cc = 2, 70, 68
    ku = rnd(B, T, 144)
    u, k = ku[..., :Cc], ku[..., 72:72 + Cc]               # both 16-byte aligned, row stride 288 bytes
    h0 = torch.rand(B, Cc, device=DEV) + 0.1
    h = torch.full((B, T, Cc), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.scan_fwd(k, u, h, h0=h0)
    L.check_device_status()
    kd, ud = k.double().requires_grad_(True), u.double().requires_grad_(True)
    href, _ = R.scan_ref(kd, ud, h0.double())
    assert_close(h, href.detach(), 1e-2, 1e-3, "scan fwd, lane stores")
    # backward reads h and dL/dh through tensor maps (rows of 72 elements here); only dk, du are unaligned
    h72, g = rnd(B, T, 72)[..., :Cc], rnd(B, T, 72)[..., :Cc]
    h72.copy_(h)
    (href * g.double()).sum().backward()
    dk = torch.full((B, T, Cc), float("nan"), device=DEV, dtype=torch.bfloat16)
    du = torch.full((B, T, Cc), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.scan_bwd(k, u, h72, g, dk, du, h0=h0)
    L.check_device_status()
    scale = max(1.0, kd.grad.abs().max().item())
    assert_close(dk, kd.grad, 3e-2, 1e-2 * scale, "scan dk, lane stores")
    assert_close(du, ud.grad, 3e-2, 1e-2 * scale, "scan du, lane stores")


def test_scan_extreme_inputs_stay_finite():
    """Saturated gates and candidates (|k|, |u| up to 3e4): the exponentials overflow or flush to zero, the results
    must still be finite and equal the fp64 recurrence."""
    B, T, Cc = 2, 40, 64
    vals = torch.tensor([-3e4, -200.0, -60.0, -41.0, -5.0, 0.0, 5.0, 41.0, 60.0, 200.0, 3e4], device=DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    k = vals[torch.randint(0, len(vals), (B, T, Cc), device=DEV, generator=g)].bfloat16()
    u = vals[torch.randint(0, len(vals), (B, T, Cc), device=DEV, generator=g)].bfloat16().clamp(max=60.0)
    h0 = torch.rand(B, Cc, device=DEV) + 0.1
    h = torch.full((B, T, Cc), float("nan"), device=DEV, dtype=torch.bfloat16)
    hl = torch.zeros(B, Cc, device=DEV)
    K.scan_fwd(k, u, h, h0=h0, h_last=hl)
    href, hlr = R.scan_ref(k.double(), u.double(), h0.double())
    assert torch.isfinite(h.float()).all() and torch.isfinite(hl).all()
    assert_close(h, href, 1e-2, 1e-3, "scan fwd, saturated inputs")
    dk, du = torch.full_like(h, float("nan")), torch.full_like(h, float("nan"))
    K.scan_bwd(k, u, h, rnd(B, T, Cc), dk, du, h0=h0)
    L.check_device_status()
    assert torch.isfinite(dk.float()).all() and torch.isfinite(du.float()).all()


def test_scan_matches_reference_logspace():
    """Against the log-space formulation the reference model evaluates (cumsum + logcumsumexp), in fp64."""
    import torch.nn.functional as F
    B, T, Cc = 2, 257, 64
    ku = rnd(B, T, 2 * Cc)
    u, k = ku[..., :Cc], ku[..., Cc:]
    h0 = torch.rand(B, Cc, device=DEV) + 0.1
    kd, ud = k.double(), u.double()
    log_coeffs = -F.softplus(kd)
    log_g = torch.where(ud >= 0, (F.relu(ud) + 0.5).log(), -F.softplus(-ud))
    log_values = torch.cat((h0.double().log().unsqueeze(1), -F.softplus(-kd) + log_g), 1)
    log_coeffs = F.pad(log_coeffs, (0, 0, 1, 0))
    a_star = log_coeffs.cumsum(1)
    href = (a_star + (log_values - a_star).logcumsumexp(1)).exp()[:, 1:]
    h = torch.zeros(B, T, Cc, device=DEV, dtype=torch.bfloat16)
    K.scan_fwd(k, u, h, h0=h0)
    L.check_device_status()
    assert_close(h, href, 1e-2, 1e-3, "scan vs log-space")


@pytest.mark.parametrize("M,D", [(37, 128), (300, 2048), (129, 520), (1000, 2048), (700, 520), (650, 3072), (1200, 4096), (600, 2560)])
def test_rmsnorm(M, D):
    x = torch.randn(M, D, device=DEV) * 2
    w = torch.randn(D, device=DEV)
    eps = torch.finfo(torch.float32).eps
    y = torch.zeros(M, D, device=DEV, dtype=torch.bfloat16)
    rstd = torch.zeros(M, device=DEV)
    K.rmsnorm_fwd(x, w, y, rstd, eps)
    assert_close(y, R.rmsnorm_ref(x, w, eps), 1e-2, 1e-2, "rmsnorm fwd")
    dy = rnd(M, D)
    dres_in = torch.randn(M, D, device=DEV)
    xd, wd = x.double().requires_grad_(True), w.double().requires_grad_(True)
    (R.rmsnorm_ref(xd, wd, eps) * dy.double()).sum().backward()
    dres_out = torch.zeros(M, D, device=DEV)
    dres16 = torch.zeros(M, D, device=DEV, dtype=torch.bfloat16)
    dw = torch.zeros(D, device=DEV)
    dcol = torch.zeros(D, device=DEV)
    K.rmsnorm_bwd(dy, x, rstd, w, dres_in, dres_out, dres16, dw, dcol)
    want = dres_in.double() + xd.grad
    assert_close(dres_out, want, 1e-4, 1e-4, "rmsnorm dx")
    assert_close(dres16, want, 1e-2, 1e-2, "rmsnorm dx bf16")
    assert_close(dw, wd.grad, 1e-3, 1e-3 * math.sqrt(M), "rmsnorm dw")
    assert_close(dcol, want.sum(0), 1e-3, 1e-3 * math.sqrt(M), "residual column sum")
    # without an incoming residual gradient and without the optional outputs (the final norm of the model)
    out2 = torch.full((M, D), float("nan"), device=DEV)
    dw2 = torch.zeros(D, device=DEV)
    K.rmsnorm_bwd(dy, x, rstd, w, None, out2, None, dw2, None)
    L.check_device_status()
    assert_close(out2, xd.grad, 1e-4, 1e-4, "rmsnorm dx, no residual")
    assert_close(dw2, wd.grad, 1e-3, 1e-3 * math.sqrt(M), "rmsnorm dw, no residual")
    # `prescaled`: the incoming gradient is rstd * dy (the norm lives in its consumer GEMM's epilogue)
    dys = (dy.float() * rstd[:, None]).bfloat16()
    xd2, wd2 = x.double().requires_grad_(True), w.double().requires_grad_(True)
    (R.rmsnorm_ref(xd2, wd2, eps) * (dys.double() / rstd.double()[:, None])).sum().backward()
    out3 = torch.full((M, D), float("nan"), device=DEV)
    dw3, dcol3 = torch.zeros(D, device=DEV), torch.zeros(D, device=DEV)
    K.rmsnorm_bwd(dys, x, rstd, w, dres_in, out3, dres16, dw3, dcol3, prescaled=True)
    L.check_device_status()
    want3 = dres_in.double() + xd2.grad
    assert_close(out3, want3, 1e-4, 1e-4, "rmsnorm dx, prescaled")
    assert_close(dw3, wd2.grad, 1e-3, 1e-3 * math.sqrt(M), "rmsnorm dw, prescaled")
    assert_close(dcol3, want3.sum(0), 1e-3, 1e-3 * math.sqrt(M), "residual column sum, prescaled")


def test_embed_colsum_sum_cast():
    B, T, D, V = 3, 50, 128, 256
    tokens = torch.randint(0, V, (B, T + 1), device=DEV, dtype=torch.uint8)
    E = torch.randn(V, D, device=DEV)
    x = torch.zeros(B * T, D, device=DEV)
    labels = torch.zeros(B * T, device=DEV, dtype=torch.uint8)
    onehot = torch.zeros(B * T, V, device=DEV, dtype=torch.bfloat16)
    K.embed_fwd(tokens, T, E, x, labels, onehot)
    ids = tokens[:, :-1].reshape(-1).long()
    assert torch.equal(x, E[ids])
    assert torch.equal(labels, tokens[:, 1:].reshape(-1))
    assert torch.equal(onehot.float(), torch.nn.functional.one_hot(ids, V).float())
    # with the first RMSNorm's inputs
    nw = torch.randn(D, device=DEV)
    x2, xw = torch.zeros_like(x), torch.zeros(B * T, D, device=DEV, dtype=torch.bfloat16)
    ssq = torch.full((B * T, 3), float("nan"), device=DEV)
    K.embed_fwd(tokens, T, E, x2, None, None, next_norm=(nw, xw, ssq))
    assert torch.equal(x2, x)
    assert_close(xw, x.double() * nw.double(), 1e-2, 1e-2, "embedding x * w")
    assert_close(ssq.sum(1), x.double().pow(2).sum(1), 1e-5, 1e-4, "embedding sum of squares")
    assert torch.count_nonzero(ssq[:, 1:]) == 0
    a = rnd(1000, 520)
    out = torch.ones(520, device=DEV)
    K.colsum_bf16(a, out)
    assert_close(out, 1 + a.float().sum(0), 1e-4, 1e-3, "colsum")
    v = torch.randn(16376, device=DEV)
    acc = torch.zeros(1, device=DEV)
    K.sum_scale(v, 0.5, acc)
    K.sum_scale(v, 0.5, acc, accumulate=True)
    assert_close(acc, v.double().sum().reshape(1), 1e-4, 1e-3, "sum_scale")
    src = torch.randn(1003, device=DEV)
    dst = torch.zeros(1003, device=DEV, dtype=torch.bfloat16)
    K.cast_f32_bf16(src, dst)
    assert torch.equal(dst, src.bfloat16())


def test_sfadamw_and_merge():
    n = 100003
    n = (n // 4) * 4 + 3
    y, z, v, g = (torch.randn(n, device=DEV) for _ in range(4))
    v = v.abs()
    hp = dict(lr=1e-3, beta1=0.9, beta2=0.999, bias2=1 - 0.999 ** 3, eps=1e-8, wd=0.01, ckp1=1 / 3)
    yr, zr, vr = R.sfadamw_ref(y.double(), z.double(), v.double(), g.double(), **hp)
    w16 = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    K.sfadamw_step(y, z, v, g, w16, **hp)
    assert_close(y, yr, 1e-5, 1e-6, "sf y")
    assert_close(z, zr, 1e-5, 1e-6, "sf z")
    assert_close(v, vr, 1e-5, 1e-7, "sf v")
    assert torch.equal(w16, y.bfloat16())
    assert torch.count_nonzero(g) == 0
    # merge: blend, clone, skip
    d0, d1, d2 = (torch.randn(n, device=DEV) for _ in range(3))
    s0, s1, s2 = (torch.randn(n, device=DEV) for _ in range(3))
    e0, e1, e2 = d0.clone(), d1.clone(), d2.clone()
    K.merge([(d0, s0, 0.3), (d1, s1, 1.0), (d2, s2, 0.0)], w16, n)
    assert_close(d0, e0 + 0.3 * (s0 - e0), 1e-6, 1e-6, "merge blend")
    assert torch.equal(d1, s1)
    assert torch.equal(d2, e2)
    assert torch.equal(w16, d0.bfloat16())


def test_bounded_wait_reports_timeout():
    """A GEMM whose error word is checked after a clean run stays zero; the status plumbing raises when set."""
    flag = L.err_flag()
    flag.fill_(7)
    with pytest.raises(RuntimeError):
        L.check_device_status()
    assert int(flag.item()) == 0
