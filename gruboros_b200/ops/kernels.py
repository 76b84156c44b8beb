"""Python entry points of the sm_100a kernels.  Every function takes CUDA tensors,
launches on the current stream and returns nothing it did not allocate itself.

Shapes use M = B*T rows; bf16 operands, fp32 accumulation.  The plain-PyTorch
restatement of each op (used on CPU and as the numerical reference in tests)
lives in ``gruboros_b200.ops.reference``.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib as L
from ._lib import (EPI_BIAS_GELU, EPI_CE, EPI_GELU_BWD, EPI_RED_F32, EPI_RED_SCATTER, EPI_RESID_F32, EPI_STORE_BF16,
                   EPI_STORE_F32, MAJOR_K, MAJOR_MN, EpiArgs)

LAUNCHES = 0  # number of kernels of this library launched by this process
# Which tcgen05 GEMM kernel runs: "auto" picks the CTA-pair kernel (cta_group::2, 256x256 tiles per pair of SMs)
# when the problem has enough tiles to fill the machine and the single-CTA kernel (128x256 tiles) otherwise.
GEMM_MODE = os.environ.get("GRB_GEMM", "auto")


def _count(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


def gemm(major_a: int, major_b: int, epi: int, a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int, *,
         out0=None, out1=None, aux=None, bias=None, ldo: int | None = None, alpha: float = 1.0, splitk: int = 1,
         lda: int | None = None, ldb: int | None = None, max_ctas: int = 0, scatter=None, sidecopy=None,
         rownorm=None, next_norm=None, colsum=None, rowscale=None, gather=None) -> None:
    """D[M,N] = A * B^T on the tcgen05 tensor cores with a fused epilogue (see ``csrc/gemm_sm100.h``).

    ``a``/``b`` are bf16 matrices whose last dimension is contiguous: [M,K]/[N,K] when K-major,
    [K,M]/[K,N] when MN-major.  ``out0`` may be any device address (a raw int is accepted, e.g. a
    peer GPU's buffer for ``EPI_RED_F32``).

    RMSNorm folded into the GEMMs: ``next_norm=(w, xw16, ssq)`` (``EPI_RESID_F32``) makes the epilogue also write
    ``xw16 = bf16(x * w)`` and the per-row partial sums of squares ``ssq`` [M, ceil(N/128)] of its fp32 output x;
    ``rownorm=(ssq, dim, eps, rstd_out)`` makes a GEMM whose ``a`` is such an ``xw16`` scale accumulator row r by
    ``rsqrt(sum(ssq[r]) / dim + eps)`` - together ``rmsnorm(x, w) @ b^T`` without a separate normalisation pass;
    ``rstd_out`` (fp32 [M] or None) receives the row scales for the backward pass.
    ``rowscale`` (fp32 [M]) multiplies accumulator rows by a ready-made vector instead (backward of such a GEMM).
    ``colsum`` (``EPI_GELU_BWD``): fp32 [N] vector that receives the column sums of the unscaled result.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    e = EpiArgs()
    e.out0 = out0 if isinstance(out0, int) else L.ptr(out0)
    e.out1 = L.ptr(out1)
    e.aux = L.ptr(aux)
    e.bias = L.ptr(bias)
    e.ldo = int(ldo if ldo is not None else N)
    e.alpha = float(alpha)
    if rownorm is not None:
        ssq, dim, eps, rstd_out = rownorm
        assert ssq.dtype == torch.float32 and ssq.shape[0] >= M and ssq.is_contiguous()
        e.rowss, e.rowss_parts, e.rowss_inv_d, e.rowss_eps = ssq.data_ptr(), ssq.shape[1], 1.0 / dim, float(eps)
        e.rstd_out = L.ptr(rstd_out)
    if rowscale is not None:
        assert rownorm is None and rowscale.dtype == torch.float32 and rowscale.numel() >= M
        e.rowss, e.rowss_parts = rowscale.data_ptr(), 0
    if next_norm is not None:
        assert epi == EPI_RESID_F32
        w, xw16, ssq = next_norm
        assert ssq.shape[1] == -(-N // 128) and xw16.stride(0) == e.ldo and ssq.is_contiguous()
        e.normw, e.out2, e.ssq_out = w.data_ptr(), xw16.data_ptr(), ssq.data_ptr()
    if colsum is not None:
        assert epi == EPI_GELU_BWD
        e.colsum = colsum.data_ptr()
    if scatter is not None:
        # (peer base pointers of the flat gradient buffer, elements per owner, flat offset of this matrix[, compact]);
        # compact: every peer buffer holds only that rank's owned chunks, packed (fully sharded training)
        peers, shard, flat_off = scatter[:3]
        e.compact = int(len(scatter) > 3 and bool(scatter[3]))
        e.peer_limit = int(scatter[4]) if len(scatter) > 4 else 0      # elements per peer buffer (checked build)
        e.world = len(peers)
        e.shard, e.flat_off = int(shard), int(flat_off)
        # shard: ownership descriptor (> 0 contiguous shard size, < 0 round-robin chunks of 2^(-shard) elements)
        e.chunk_aligned = int(flat_off % 32 == 0 and e.ldo % 32 == 0 and (shard % 32 == 0 if shard > 0 else -shard >= 5))
        for i, p in enumerate(peers):
            e.peers[i] = p
    if sidecopy:
        # [(src_ptr, dst_ptr, nbytes)] copied by spare warps of the CTA-pair kernel while the GEMM runs
        e.n_copy = len(sidecopy)
        for i, (sp, dp, nb) in enumerate(sidecopy):
            e.copy_src[i], e.copy_dst[i], e.copy_bytes[i] = sp, dp, nb
    if gather is not None:
        # (packed bf16 shard pointer of every rank, chunk shift, lo, hi, destination pointer): all-gather elements
        # [lo, hi) of a chunk-dealt flat space into local memory with the CTA-pair kernel's copy warps
        assert scatter is None, "a GEMM carries either the gradient scatter or a weight gather"
        gp, gshift, glo, ghi, gdst = gather[:5]
        e.peer_limit, e.gather_cap = (int(gather[5]), int(gather[6])) if len(gather) > 6 else (0, 0)
        e.world, e.shard = len(gp), -int(gshift)
        for i, p in enumerate(gp):
            e.peers[i] = p
        e.gather_lo, e.gather_hi, e.gather_dst = int(glo), int(ghi), int(gdst)
    lda = int(lda if lda is not None else a.stride(0))
    ldb = int(ldb if ldb is not None else b.stride(0))
    pair_tiles = -(-M // 256) * -(-N // 256) * max(1, splitk)
    if splitk < 0:      # stream-K (accumulating epilogues): work is dealt in k-block runs, so count those
        pair_tiles = -(-M // 256) * -(-N // 256) * -(-K // 64) // 8
    use_pair = GEMM_MODE == "2cta" or (GEMM_MODE == "auto" and pair_tiles >= 48)
    if sidecopy and not use_pair:
        copy_segments(sidecopy)          # the single-CTA kernel has no copy warps
    if gather is not None and not use_pair:
        gather_chunks(*gather)
        e.gather_lo = e.gather_hi = 0
    fn = L.lib().grb_gemm_pair if use_pair else L.lib().grb_gemm
    rc = fn(major_a, major_b, epi, a.data_ptr(), lda, b.data_ptr(), ldb, M, N, K, splitk, C.byref(e),
            L.err_flag(a.device).data_ptr(), max_ctas, L.stream())
    L.check(rc, "grb_gemm_pair" if use_pair else "grb_gemm")
    _count()


def linear_fwd(x16, w16, out, *, epi=EPI_STORE_BF16, **kw):
    """out = x16 [M,K] @ w16[N,K]^T."""
    M, K = x16.shape
    N = w16.shape[0]
    gemm(MAJOR_K, MAJOR_K, epi, x16, w16, M, N, K, out0=out, **kw)


def linear_dgrad(dy16, w16, out, *, epi=EPI_STORE_BF16, **kw):
    """out [M,K] = dy16 [M,N] @ w16 [N,K]  (w16 read MN-major, no transposed copy)."""
    M, N = dy16.shape
    K = w16.shape[1]
    gemm(MAJOR_K, MAJOR_MN, epi, dy16, w16, M, K, N, out0=out, **kw)


def linear_wgrad(dy16, x16, dw, *, accumulate=True, splitk=1, alpha=1.0, M=None, scatter=None):
    """dw [N,K] (+)= dy16[M,N]^T @ x16[M,K]; both operands read MN-major.

    ``scatter=(peer_ptrs, shard, flat_off)`` turns the epilogue into the data-parallel reduce-scatter: every
    element is added into the flat gradient buffer of the rank that owns it (``dw`` is then ignored).
    ``splitk``: > 1 splits the reduction into that many equal parts per output tile; -1 deals equal runs of
    (tile, k-block) units to the SM pairs instead ("stream-K": full machine whatever the tile count)."""
    Mr = dy16.shape[0] if M is None else M
    N, K = dy16.shape[1], x16.shape[1]
    if scatter is not None:
        gemm(MAJOR_MN, MAJOR_MN, EPI_RED_SCATTER, dy16, x16, N, K, Mr, ldo=K, splitk=splitk, alpha=alpha, scatter=scatter)
        return
    epi = EPI_RED_F32 if (accumulate or splitk > 1 or splitk < 0) else EPI_STORE_F32
    gemm(MAJOR_MN, MAJOR_MN, epi, dy16, x16, N, K, Mr, out0=dw, ldo=K, splitk=splitk, alpha=alpha)


def scan_fwd(k, u, h, *, h0=None, h_last=None):
    """minGRU recurrence.  k, u: bf16 [B,T,C] views (row stride may exceed C); h: bf16 [B,T,C] output."""
    B, T, Cc = k.shape
    assert k.stride(2) == 1 and u.stride(1) == k.stride(1) and k.stride(0) == T * k.stride(1)
    rc = L.lib().grb_scan_fwd(k.data_ptr(), u.data_ptr(), k.stride(1), L.ptr(h0), h.data_ptr(), h.stride(1),
                              L.ptr(h_last), B, T, Cc, L.err_flag(k.device).data_ptr(), L.stream())
    L.check(rc, "grb_scan_fwd")
    _count()


def scan_bwd(k, u, h, g, dk, du, *, h0=None, dh_last=None, dh0=None, rowscale=None):
    """Backward of ``scan_fwd``: g = dL/dh (bf16 [B,T,C]); writes dk, du (bf16 views with a common row stride).
    ``rowscale`` (fp32 [B*T], optional) multiplies row (b, t) of dk and du - the rstd of an RMSNorm folded into the
    GEMM that produced k and u, so that its wgrad / dgrad can run on the unnormalised operand."""
    B, T, Cc = k.shape
    assert dk.stride(1) == du.stride(1)
    rc = L.lib().grb_scan_bwd(k.data_ptr(), u.data_ptr(), k.stride(1), h.data_ptr(), h.stride(1), g.data_ptr(),
                              g.stride(1), L.ptr(h0), L.ptr(dh_last), dk.data_ptr(), du.data_ptr(), dk.stride(1),
                              L.ptr(dh0), L.ptr(rowscale), B, T, Cc, L.err_flag(k.device).data_ptr(), L.stream())
    L.check(rc, "grb_scan_bwd")
    _count()


def embed_fwd(tokens, T, E, x, labels=None, onehot=None, next_norm=None):
    """x[b*T+t] = E[tokens[b,t]]; labels[b*T+t] = tokens[b,t+1]; optional bf16 one-hot rows for the embedding wgrad.
    ``next_norm=(w, xw16, ssq)``: also the inputs of a folded RMSNorm (see ``gemm``): xw16 = bf16(x * w), ssq [M, parts]."""
    B = tokens.shape[0]
    V, D = E.shape
    nw, xw, ssq = next_norm if next_norm is not None else (None, None, None)
    rc = L.lib().grb_embed_fwd(tokens.data_ptr(), tokens.stride(0), B, T, D, V, E.data_ptr(), x.data_ptr(),
                               L.ptr(labels), L.ptr(onehot), L.ptr(nw), L.ptr(xw), L.ptr(ssq),
                               ssq.shape[1] if ssq is not None else 0, L.stream())
    L.check(rc, "grb_embed_fwd")
    _count()


def rmsnorm_fwd(x, w, y16, rstd, eps):
    M, D = x.shape
    L.check(L.lib().grb_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y16.data_ptr(), L.ptr(rstd), M, D, eps, L.stream()),
            "grb_rmsnorm_fwd")
    _count()


DEC_STORE, DEC_GATE, DEC_RESID, DEC_GELU = 0, 1, 2, 3


def decode_gemv(epi: int, x, w16, out, *, norm_w=None, bias=None, eps: float = 0.0, has_prev: bool = True, sms: int = 0,
                overlap: bool = False):
    """Decode-step matrix-vector product with fused prologue / epilogue (see ``csrc/decode.h``).

    x fp32 [B, K] (B <= 8), w16 bf16 [N, K] ([2N, K] for DEC_GATE), out fp32 [B, N] (state, updated in place for
    DEC_GATE and DEC_RESID).  ``overlap`` lets the kernel start (and prefetch its weights) before the previous kernel on
    the stream has finished."""
    B, Kd = x.shape
    N = out.shape[1]
    assert w16.shape[1] == Kd and w16.shape[0] == (2 * N if epi == DEC_GATE else N)
    rc = L.lib().grb_decode_gemv(epi, x.data_ptr(), L.ptr(norm_w), w16.data_ptr(), L.ptr(bias), out.data_ptr(), B, N, Kd,
                                 eps, int(has_prev), sms, int(overlap), L.err_flag(x.device).data_ptr(), L.stream())
    L.check(rc, "grb_decode_gemv")
    _count()


def sample(logits, tok_out, *, temperature=1.0, top_k=0, top_p=0.0, u=None, seed=0, counter=None, history=None,
           probs_out=None):
    """Draw one token per row of fp32 ``logits`` [B, V <= 256] into the uint8 tensor ``tok_out`` (see ``csrc/sample.h``)."""
    B, V = logits.shape
    rc = L.lib().grb_sample(logits.data_ptr(), B, V, float(temperature), int(top_k), float(top_p), L.ptr(u), int(seed),
                            L.ptr(counter), tok_out.data_ptr(), L.ptr(history), history.shape[1] if history is not None else 0,
                            L.ptr(probs_out), L.stream())
    L.check(rc, "grb_sample")
    _count()


IN_NORM, IN_GATE, IN_GELU = 0, 1, 2


def decode_tc(mode: int, src, w16, out, *, vec=None, state=None, state_out=None, out_bias=None, zero=None, copy=None,
              eps: float = 0.0, sms: int = 0, overlap: bool = False):
    """Decode-step product on the tensor cores: out [B, N] += W [N, K] . in, ``in`` derived from ``src`` by ``mode``
    (see ``csrc/decode.h``).  ``zero``: tensor to clear; ``copy``: (dst, src) tensors to copy - housekeeping of a chain."""
    B = src.shape[0]
    N, Kd = w16.shape
    assert out.shape == (B, N) and src.shape[1] == (2 * Kd if mode == IN_GATE else Kd)
    cd, cs = copy if copy is not None else (None, None)
    rc = L.lib().grb_decode_tc(mode, src.data_ptr(), L.ptr(vec), L.ptr(state), L.ptr(state_out), w16.data_ptr(),
                               out.data_ptr(), L.ptr(out_bias), L.ptr(zero), zero.numel() if zero is not None else 0,
                               L.ptr(cd), L.ptr(cs), cd.numel() if cd is not None else 0, B, N, Kd, eps, sms,
                               int(overlap), L.err_flag(src.device).data_ptr(), L.stream())
    L.check(rc, "grb_decode_tc")
    _count()


def rmsnorm_bwd(dy16, x, rstd, w, dres_in, dres_out, dres16, dw, dcol=None, ring=True, prescaled=False):
    """RMSNorm backward fused with the residual-gradient accumulation (``csrc/elementwise.cu``).  ``prescaled``:
    ``dy16`` is the gradient w.r.t. the unnormalised x * w (the norm was folded into its consumer GEMM)."""
    M, D = x.shape
    L.check(L.lib().grb_rmsnorm_bwd(dy16.data_ptr(), x.data_ptr(), rstd.data_ptr(), w.data_ptr(), L.ptr(dres_in),
                                    dres_out.data_ptr(), L.ptr(dres16), dw.data_ptr(), L.ptr(dcol), M, D, int(prescaled),
                                    L.err_flag(x.device).data_ptr() if ring else None, L.stream()),
            "grb_rmsnorm_bwd")
    _count()


def colsum_bf16(a16, out):
    M, N = a16.shape
    L.check(L.lib().grb_colsum_bf16(a16.data_ptr(), a16.stride(0), M, N, out.data_ptr(), L.stream()), "grb_colsum_bf16")
    _count()


def sum_scale(v, scale, out, accumulate=False):
    L.check(L.lib().grb_sum_scale(v.data_ptr(), v.numel(), scale, out.data_ptr(), int(accumulate), L.stream()),
            "grb_sum_scale")
    _count()


def cast_f32_bf16(src, dst):
    L.check(L.lib().grb_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), L.stream()), "grb_cast_f32_bf16")
    _count()


def sfadamw_step(y, z, v, g, w16, *, lr, beta1, beta2, bias2, eps, wd, ckp1, gscale=1.0, zero_grad=True):
    L.check(L.lib().grb_sfadamw_step(y.data_ptr(), z.data_ptr(), v.data_ptr(), g.data_ptr(), L.ptr(w16), y.numel(),
                                     lr, beta1, beta2, bias2, eps, wd, ckp1, gscale, int(zero_grad), L.stream()),
            "grb_sfadamw_step")
    _count()


def merge(pairs, w16, n):
    """pairs: up to three (dst_tensor, src_ptr_or_tensor, alpha); dst = (1-alpha) dst + alpha src, fused bf16 recast."""
    args = []
    for i in range(3):
        if i < len(pairs):
            d, s, al = pairs[i]
            args += [d.data_ptr(), s if isinstance(s, int) else s.data_ptr(), float(al)]
        else:
            args += [None, None, 0.0]
    L.check(L.lib().grb_merge(*args, L.ptr(w16), n, L.stream()), "grb_merge")
    _count()


def gather_chunks(shard_ptrs, chunk_shift, lo, hi, dst_ptr, shard_numel=0, dst_numel=0):
    """Stand-alone all-gather of bf16 elements [lo, hi) of a flat space dealt round-robin in chunks of
    2^chunk_shift elements: element i comes from the packed shard of rank (i >> chunk_shift) % world.
    shard_numel / dst_numel (elements each shard / the destination holds) feed the checked build's bounds checks."""
    n = len(shard_ptrs)
    arr = (C.c_void_p * n)(*shard_ptrs)
    L.check(L.lib().grb_gather_chunks(arr, n, int(chunk_shift), int(lo), int(hi), int(dst_ptr), int(shard_numel),
                                      int(dst_numel), L.err_flag().data_ptr(), L.stream()), "grb_gather_chunks")
    _count()


def copy_segments(segments):
    """Copy [(src_ptr, dst_ptr, nbytes)] (up to 8 per launch; 16-byte aligned; src may be peer memory)."""
    for i in range(0, len(segments), 8):
        part = segments[i:i + 8]
        n = len(part)
        src = (C.c_void_p * n)(*[sgm[0] for sgm in part])
        dst = (C.c_void_p * n)(*[sgm[1] for sgm in part])
        nb = (C.c_int64 * n)(*[sgm[2] for sgm in part])
        L.check(L.lib().grb_copy_segments(n, src, dst, nb, L.stream()), "grb_copy_segments")
        _count()
