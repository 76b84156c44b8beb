"""Small, self-contained launches of each fused kernel for profiling under Nsight Compute.

    python -m gruboros_b200.tools.profile_cases CASE          # runs CASE three times (two warm-ups + one to capture)
    python -m gruboros_b200.tools.profile_cases --list

Inputs are larger than the 126 MB L2 but at most a few hundred MB, so a full-section capture of the third launch
finishes in seconds:   ncu --set full --clock-control none -k regex:<kernel> -s 2 -c 1 -o out python -m ... CASE
Multi-rank paths (reduce-scatter epilogue, gossip merge, side copy) are exercised on ONE GPU with every "peer"
pointer aimed at local memory - the instruction stream is the one that runs over NVLink.
"""
from __future__ import annotations

import sys

import torch

from ..ops import kernels as K

M, D, DI, F, V = 16376, 2048, 3072, 8192, 256


def rnd(*s):
    return torch.randn(*s, device="cuda").bfloat16()


def case_scan_fwd():
    ku = rnd(8, 2047, 2 * DI)
    h = torch.empty(8, 2047, DI, device="cuda", dtype=torch.bfloat16)
    h0 = torch.rand(8, DI, device="cuda") + 0.1
    hl = torch.empty(8, DI, device="cuda")
    return lambda: K.scan_fwd(ku[..., DI:], ku[..., :DI], h, h0=h0, h_last=hl)


def case_scan_bwd():
    ku, h, g = rnd(8, 2047, 2 * DI), rnd(8, 2047, DI).abs(), rnd(8, 2047, DI)
    dku = torch.empty_like(ku)
    h0 = torch.rand(8, DI, device="cuda") + 0.1
    return lambda: K.scan_bwd(ku[..., DI:], ku[..., :DI], h, g, dku[..., DI:], dku[..., :DI], h0=h0)


def case_rmsnorm_bwd():
    x, dres = torch.randn(M, D, device="cuda"), torch.randn(M, D, device="cuda")
    dy, w, rstd = rnd(M, D), torch.ones(D, device="cuda"), torch.rand(M, device="cuda") + 0.5
    out, o16 = torch.empty_like(x), torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    dw, dc = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    return lambda: K.rmsnorm_bwd(dy, x, rstd, w, dres, out, o16, dw, dc)


def case_sfadamw():
    n = 64 * 1024 * 1024
    y, z, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    w16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    return lambda: K.sfadamw_step(y, z, v, g, w16, lr=1e-3, beta1=0.9, beta2=0.995, bias2=0.5, eps=1e-8, wd=1e-4, ckp1=0.1)


def case_merge():
    n = 32 * 1024 * 1024
    d = [torch.randn(n, device="cuda") for _ in range(3)]
    s = [torch.randn(n, device="cuda") for _ in range(3)]
    w16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    return lambda: K.merge([(d[0], s[0], 0.3), (d[1], s[1], 0.3), (d[2], s[2], 0.3)], w16, n)


def case_gemm_ce():
    x, w = rnd(M, D), rnd(V, D) * 0.1
    labels = torch.randint(0, V, (M,), device="cuda", dtype=torch.uint8)
    loss, dlog = torch.empty(M, device="cuda"), torch.empty(M, V, device="cuda", dtype=torch.bfloat16)
    return lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, x, w, M, V, D, out0=dlog, out1=loss, aux=labels, ldo=V, alpha=1.0 / M)


def case_gemm_gate():
    """Gate projection as a 1B layer issues it: A = unnormalised bf16 x * w, rows scaled by rstd in the epilogue."""
    xw, w = rnd(M, D), rnd(2 * DI, D)
    ssq = torch.rand(M, D // 128, device="cuda") * 128 + 1.0
    rstd = torch.empty(M, device="cuda")
    ku = torch.empty(M, 2 * DI, device="cuda", dtype=torch.bfloat16)
    return lambda: K.linear_fwd(xw, w, ku, rownorm=(ssq, D, 1e-6, rstd))


def case_gemm_gate_plain():
    """The same product without the folded norm (plain bf16 store)."""
    xn, w = rnd(M, D), rnd(2 * DI, D)
    ku = torch.empty(M, 2 * DI, device="cuda", dtype=torch.bfloat16)
    return lambda: K.linear_fwd(xn, w, ku)


def case_gemm_resid():
    """Output projection: residual add, plus the next RMSNorm's inputs (bf16 x * w, partial sums of squares)."""
    h, w = rnd(M, DI), rnd(D, DI)
    x, out = torch.randn(M, D, device="cuda"), torch.empty(M, D, device="cuda")
    nw, xw, ssq = torch.ones(D, device="cuda"), torch.empty(M, D, device="cuda", dtype=torch.bfloat16), torch.empty(M, D // 128, device="cuda")
    return lambda: K.linear_fwd(h, w, out, epi=K.EPI_RESID_F32, aux=x, next_norm=(nw, xw, ssq))


def case_gemm_ff1():
    """FF1: folded norm, bias, GELU and its derivative."""
    xw, w, b = rnd(M, D), rnd(F, D) * 0.05, torch.zeros(F, device="cuda")
    ssq = torch.rand(M, D // 128, device="cuda") * 128 + 1.0
    der, act = (torch.empty(M, F, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    return lambda: K.linear_fwd(xw, w, der, epi=K.EPI_BIAS_GELU, out1=act, bias=b, rownorm=(ssq, D, 1e-6, None))


def case_gemm_ff2_dgrad():
    """FF2 dgrad: x saved GELU derivative x rstd, with the bias-gradient column sums."""
    dy, w, saved = rnd(M, D), rnd(D, F) * 0.05, rnd(M, F)
    out = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    rs, cs = torch.rand(M, device="cuda") + 0.5, torch.zeros(F, device="cuda")
    return lambda: K.linear_dgrad(dy, w, out, epi=K.EPI_GELU_BWD, aux=saved, rowscale=rs, colsum=cs)


def case_gemm_gate_wgrad():
    """Gate weight gradient dy^T x on one GPU: both operands MN-major, fp32 red.add into the gradient, split-K 3."""
    dy, x = rnd(M, 2 * DI), rnd(M, D)
    dw = torch.zeros(2 * DI, D, device="cuda")
    return lambda: K.linear_wgrad(dy, x, dw, splitk=3)


def case_gemm_wgrad_scatter():
    dy, x = rnd(M, 2 * DI), rnd(M, D)
    world, n = 4, 2 * DI * D
    shard = n // world
    bufs = [torch.zeros(n, device="cuda") for _ in range(world)]        # every rank's flat gradient buffer (local here)
    ptrs = [b.data_ptr() for b in bufs]
    return lambda: K.linear_wgrad(dy, x, None, splitk=1, scatter=(ptrs, shard, 0))


def case_gemm_sidecopy():
    xn, w = rnd(M, D), rnd(2 * DI, D)
    ku = torch.empty(M, 2 * DI, device="cuda", dtype=torch.bfloat16)
    src = torch.randn(100 * 1024 * 1024, device="cuda").bfloat16()       # 200 MB "remote shard"
    dst = torch.empty_like(src)
    seg = [(src.data_ptr(), dst.data_ptr(), src.numel() * 2)]
    return lambda: K.linear_fwd(xn, w, ku, sidecopy=seg)


def _decode_case(epi, N, Kd, norm, bias):
    # a different weight matrix per launch (the decode step never re-reads a matrix from L2)
    ws = [rnd(2 * N if epi == K.DEC_GATE else N, Kd) * 0.02 for _ in range(3)]
    x = torch.randn(1, Kd, device="cuda")
    out = torch.zeros(1, N, device="cuda")
    nw = torch.ones(Kd, device="cuda") if norm else None
    b = torch.zeros(N, device="cuda") if bias else None
    it = iter(range(10 ** 9))
    return lambda: K.decode_gemv(epi, x, ws[next(it) % 3], out, norm_w=nw, bias=b, eps=1e-6)


def case_decode_tc_ff1():
    ws = [rnd(F, D) * 0.02 for _ in range(3)]
    x, nw, out = torch.randn(1, D, device="cuda"), torch.ones(D, device="cuda"), torch.zeros(1, F, device="cuda")
    it = iter(range(10 ** 9))
    return lambda: K.decode_tc(K.IN_NORM, x, ws[next(it) % 3], out, vec=nw, eps=1e-6)


def case_decode_tc_ff2():
    ws = [rnd(D, F) * 0.02 for _ in range(3)]
    a, b1, out = torch.randn(1, F, device="cuda"), torch.zeros(F, device="cuda"), torch.zeros(1, D, device="cuda")
    it = iter(range(10 ** 9))
    return lambda: K.decode_tc(K.IN_GELU, a, ws[next(it) % 3], out, vec=b1)


def case_decode_ff1():
    return _decode_case(K.DEC_GELU, F, D, True, True)


def case_decode_ff2():
    return _decode_case(K.DEC_RESID, D, F, False, True)


def case_decode_gate():
    return _decode_case(K.DEC_GATE, DI, D, True, False)


CASES = {n[5:]: f for n, f in globals().items() if n.startswith("case_")}


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] == "--list":
        print("\n".join(CASES))
        return 0
    fn = CASES[argv[0]]()
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    from ..ops import _lib
    _lib.check_device_status()
    print(f"{argv[0]}: ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
