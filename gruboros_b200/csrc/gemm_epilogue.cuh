// Fused GEMM epilogues shared by the one-CTA and the CTA-pair tcgen05 kernels.
//
// tcgen05.ld hands each thread one accumulator ROW (TMEM lane) x 32 columns.  Writing that straight to global
// memory makes every warp store touch 32 different cache lines, 16 bytes each, and the L1-to-crossbar request
// rate - not the tensor pipe - ends up limiting the kernel.  So each warp first transposes its 32 x 32 chunk
// through a private shared-memory staging tile; afterwards a lane owns 4 consecutive columns of a row, 8 lanes
// cover a 128-byte row segment and every load / store / reduction instruction moves whole cache lines.
// The cross-entropy epilogue keeps the row-per-thread form (it needs whole rows and writes little).
#pragma once
#include "ptx.cuh"
#include "owner.cuh"
#include "gemm_sm100.h"

namespace grb {

constexpr int EPI_BN = 256;   // accumulator columns per tile

// Checked build (-DGRB_CHECKS): `cond` is what an access about to be made relies on.  When it does not hold, the
// code is recorded in the launch's error word and the caller skips the access - nothing traps, the kernel runs to
// its end and the host reads the word.  In the normal build this is the constant true.
__device__ __forceinline__ bool grb_ok(const EpiArgs& e, bool cond, int code) {
#ifdef GRB_CHECKS
  if (!cond) {
    if (e.chk_err) atomicExch(e.chk_err, code);
    return false;
  }
#endif
  return true;
}

// Exact (erf) GELU and its derivative.  erf comes from Abramowitz & Stegun 7.1.26 (|error| < 1.5e-7, far below
// the bf16 rounding of the outputs); its exponential exp(-x^2/2) is the same one the Gaussian density needs, so
// value and derivative cost one ex2, one reciprocal and a dozen FMAs - about a third of erff + expf.
__device__ __forceinline__ void gelu_parts(float x, float& cdf, float& pdf) {
  const float ax = fabsf(x) * 0.70710678118654752f;              // |x| / sqrt(2)
  float e, t;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-0.72134752044448170f * x * x));   // exp(-x^2 / 2)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.f)));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  const float erf_abs = fmaf(-p * t, e, 1.f);                     // erf(|x| / sqrt 2)
  cdf = 0.5f + copysignf(0.5f * erf_abs, x);
  pdf = 0.3989422804014327f * e;
}
// The same for two neighbouring elements with packed fp32 arithmetic (half the fp32-pipe instructions).  The
// polynomial carries the factor -1/2, so h = 0.5 erf(|x| / sqrt 2) falls out of one fma with the exponential.
__device__ __forceinline__ void gelu_parts2(float2 x, float2& cdf, float2& pdf) {
  const float2 ea = fmul2(fmul2(x, x), splat2(-0.72134752044448170f));
  float2 e, t;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(ea.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(ea.y));
  const float2 den = ffma2(make_float2(fabsf(x.x), fabsf(x.y)), splat2(0.3275911f * 0.70710678118654752f), splat2(1.f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.x) : "f"(den.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.y) : "f"(den.y));
  float2 p = ffma2(splat2(-0.5f * 1.061405429f), t, splat2(0.5f * 1.453152027f));
  p = ffma2(p, t, splat2(-0.5f * 1.421413741f));
  p = ffma2(p, t, splat2(0.5f * 0.284496736f));
  p = ffma2(p, t, splat2(-0.5f * 0.254829592f));
  const float2 h = ffma2(fmul2(p, t), e, splat2(0.5f));
  cdf = fadd2(make_float2(copysignf(h.x, x.x), copysignf(h.y, x.y)), splat2(0.5f));
  pdf = fmul2(e, splat2(0.3989422804014327f));
}
__device__ __forceinline__ float gelu_f(float x) {
  float cdf, pdf;
  gelu_parts(x, cdf, pdf);
  return x * cdf;
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  float cdf, pdf;
  gelu_parts(x, cdf, pdf);
  return fmaf(x, pdf, cdf);
}

// The A operand of a GEMM may be the UNNORMALISED bf16 x * w of an RMSNorm whose per-row sums of squares were left
// (in `rowss_parts` partial sums per row) by the GEMM that produced x.  Scaling a row of A commutes with the
// contraction, so the consumer multiplies its accumulator rows by rsqrt(mean(x^2) + eps) here instead of a separate
// normalisation pass over x (reference: nn.RMSNorm before every block, mingru/minLM.py:120,130,137).  The partial
// sums are added in a fixed order, so the result does not depend on scheduling.
__device__ __forceinline__ float row_scale(const EpiArgs& e, int row, int M) {
  if (e.rowss == nullptr || row >= M) return 1.f;
  if (e.rowss_parts <= 0) return __ldg(e.rowss + row);            // ready-made scale vector
  const float* p = e.rowss + static_cast<size_t>(row) * e.rowss_parts;
  float s = 0.f;
  for (int i = 0; i < e.rowss_parts; ++i) s += __ldg(p + i);
  return rsqrtf(fmaf(s, e.rowss_inv_d, e.rowss_eps));
}

constexpr int EPI_STAGE_LD = 32;                         // floats per staged row; 16-byte chunk j of row r sits at chunk j ^ (r & 7)
                                                         // (conflict-free for the row-per-lane writes and the 8-lanes-per-row reads)
constexpr int EPI_STAGE_FLOATS = 32 * EPI_STAGE_LD;      // per warp
constexpr int EPI_STAGE_BYTES = EPI_STAGE_FLOATS * 4;

// ------------------------------------------------------------- cross-entropy (row per thread)
template <int EPI>
__device__ __forceinline__ void epilogue_row(const EpiArgs& e, uint32_t taddr, int row, int n0, int M, int N,
                                             int c_begin, int c_end) {
  const bool row_ok = row < M;
  if constexpr (EPI == EPI_CE) {
    // 256-way softmax cross-entropy on the accumulator row, v = rowscale * acc.
    // loss_rows[row] = logsumexp(v) - v[label];  dlogits = (softmax - onehot) * alpha * rowscale
    float* loss_rows = reinterpret_cast<float*>(e.out1);
    __nv_bfloat16* dlog = reinterpret_cast<__nv_bfloat16*>(e.out0);
    const uint8_t* labels = reinterpret_cast<const uint8_t*>(e.aux);
    const int label = row_ok ? static_cast<int>(labels[row]) : 0;
    const float rs = row_scale(e, row, M);     // logits = rs * accumulator (final RMSNorm folded in)
    if (e.rstd_out && row_ok) e.rstd_out[row] = rs;
    const float dscale = e.alpha * rs;         // ... and d logits carry rs too: the gradient w.r.t. the unnormalised operand
    float mx = -INFINITY;
    uint32_t r[32];
    for (int c = 0; c < EPI_BN; c += 32) {
      if (n0 + c >= N) break;
      __syncwarp();
      tmem_ld32(taddr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + c + j < N) mx = fmaxf(mx, rs * __uint_as_float(r[j]));
    }
    float sum = 0.f, picked = 0.f;
    for (int c = 0; c < EPI_BN; c += 32) {
      if (n0 + c >= N) break;
      __syncwarp();
      tmem_ld32(taddr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float v = rs * __uint_as_float(r[j]);
        if (n0 + c + j < N) {
          sum += __expf(v - mx);
          if (n0 + c + j == label) picked = v;
        }
      }
    }
    const float lse = mx + __logf(sum);
    if (row_ok && loss_rows) loss_rows[row] = lse - picked;
    if (dlog) {
      for (int c = 0; c < EPI_BN; c += 32) {
        if (n0 + c >= N) break;
        __syncwarp();
        tmem_ld32(taddr + c, r);
        tmem_ld_wait();
        if (row_ok) {
          __nv_bfloat16* dst = dlog + static_cast<size_t>(row) * e.ldo + n0 + c;
          if (n0 + c + 32 <= N) {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float p0 = __expf(rs * __uint_as_float(r[j]) - lse) - ((n0 + c + j) == label ? 1.f : 0.f);
              float p1 = __expf(rs * __uint_as_float(r[j + 1]) - lse) - ((n0 + c + j + 1) == label ? 1.f : 0.f);
              pk[j >> 1] = pack_bf16(p0 * dscale, p1 * dscale);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(dst)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          } else {
            for (int j = 0; j < 32 && n0 + c + j < N; ++j) {
              float p = __expf(rs * __uint_as_float(r[j]) - lse) - ((n0 + c + j) == label ? 1.f : 0.f);
              dst[j] = __float2bfloat16(p * dscale);
            }
          }
        }
      }
    }
    return;
  }
}

// ------------------------------------------------------------- element-wise epilogues (staged, coalesced)
// One call handles 4 consecutive columns (col .. col+3) of one row.  `n_ok` = how many of them are inside N.
//   bv       : bias of the four columns (zeros when there is none)
//   pre      : when have_pre, the 16 bytes (RESID) / 8 bytes (GELU') of `aux` for these elements, loaded earlier by the
//              caller so that the load latency is not paid between two stores
//   rscale   : row scale of this row (1 without a folded RMSNorm)
//   nw, ssq  : RESID with a following RMSNorm: its weight for the four columns; ssq accumulates x^2 of the row
//   cs       : GELU': running column sums of the unscaled result (bias gradient)
template <int EPI>
__device__ __forceinline__ void epilogue_apply4(const EpiArgs& e, float4 v, float4 bv, int row, int col, int n_ok,
                                                bool vec_ok, bool have_pre, uint4 pre, float rscale, float4 nw,
                                                float& ssq, float (&cs)[4]) {
  const size_t off = static_cast<size_t>(row) * e.ldo + col;
  const float sc = e.alpha * (EPI == EPI_GELU_BWD ? 1.f : rscale);
  const float2 x01 = ffma2(make_float2(v.x, v.y), splat2(sc), make_float2(bv.x, bv.y));
  const float2 x23 = ffma2(make_float2(v.z, v.w), splat2(sc), make_float2(bv.z, bv.w));
  float x[4] = {x01.x, x01.y, x23.x, x23.y};
  const bool vec = vec_ok && n_ok == 4;
  if constexpr (EPI == EPI_STORE_BF16 || EPI == EPI_BIAS_GELU || EPI == EPI_GELU_BWD) {
    __nv_bfloat16* o0 = reinterpret_cast<__nv_bfloat16*>(e.out0) + off;
    if constexpr (EPI == EPI_GELU_BWD) {
      const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(e.aux) + off;
      if (vec) {
        const uint2 u = have_pre ? make_uint2(pre.x, pre.y) : *reinterpret_cast<const uint2*>(a);
        x[0] *= bf16_lo(u.x); x[1] *= bf16_hi(u.x);
        x[2] *= bf16_lo(u.y); x[3] *= bf16_hi(u.y);
      } else {
        for (int j = 0; j < n_ok; ++j) x[j] *= __bfloat162float(a[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < n_ok) cs[j] += x[j];
        x[j] *= rscale;
      }
    }
    if constexpr (EPI == EPI_BIAS_GELU) {
      // one evaluation of the Gaussian cdf / pdf serves the activation and its derivative
      float act[4], der[4];
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const float2 xx = make_float2(x[j], x[j + 1]);
        float2 cdf, pdf;
        gelu_parts2(xx, cdf, pdf);
        const float2 a2 = fmul2(xx, cdf), d2 = ffma2(xx, pdf, cdf);
        act[j] = a2.x; act[j + 1] = a2.y;
        der[j] = d2.x; der[j + 1] = d2.y;
      }
      __nv_bfloat16* o1 = reinterpret_cast<__nv_bfloat16*>(e.out1) + off;
      if (vec) {
        *reinterpret_cast<uint2*>(o0) = make_uint2(pack_bf16(der[0], der[1]), pack_bf16(der[2], der[3]));
        *reinterpret_cast<uint2*>(o1) = make_uint2(pack_bf16(act[0], act[1]), pack_bf16(act[2], act[3]));
      } else {
        for (int j = 0; j < n_ok; ++j) { o0[j] = __float2bfloat16(der[j]); o1[j] = __float2bfloat16(act[j]); }
      }
    } else {
      if (vec) *reinterpret_cast<uint2*>(o0) = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
      else for (int j = 0; j < n_ok; ++j) o0[j] = __float2bfloat16(x[j]);
    }
  } else if constexpr (EPI == EPI_STORE_F32 || EPI == EPI_RESID_F32) {
    float* o0 = reinterpret_cast<float*>(e.out0) + off;
    if constexpr (EPI == EPI_RESID_F32) {
      const float* rin = reinterpret_cast<const float*>(e.aux) + off;    // residual input (may alias out0)
      if (vec) {
        const uint4 y = have_pre ? pre : *reinterpret_cast<const uint4*>(rin);
        x[0] += __uint_as_float(y.x); x[1] += __uint_as_float(y.y); x[2] += __uint_as_float(y.z); x[3] += __uint_as_float(y.w);
      } else {
        for (int j = 0; j < n_ok; ++j) x[j] += rin[j];
      }
    }
    if (vec) *reinterpret_cast<float4*>(o0) = make_float4(x[0], x[1], x[2], x[3]);
    else for (int j = 0; j < n_ok; ++j) o0[j] = x[j];
    if constexpr (EPI == EPI_RESID_F32) {
      if (e.out2) {
        // operand of the GEMM behind the next RMSNorm (x * w, not yet divided by the row's rms) and the row's x^2
        __nv_bfloat16* o2 = reinterpret_cast<__nv_bfloat16*>(e.out2) + off;
        const float wv[4] = {nw.x, nw.y, nw.z, nw.w};
        if (vec) {
          *reinterpret_cast<uint2*>(o2) = make_uint2(pack_bf16(x[0] * wv[0], x[1] * wv[1]), pack_bf16(x[2] * wv[2], x[3] * wv[3]));
          ssq += x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
        } else {
          for (int j = 0; j < n_ok; ++j) { o2[j] = __float2bfloat16(x[j] * wv[j]); ssq += x[j] * x[j]; }
        }
      }
    }
  } else if constexpr (EPI == EPI_RED_F32) {
    float* o0 = reinterpret_cast<float*>(e.out0) + off;
    if (vec) asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o0), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]) : "memory");
    else for (int j = 0; j < n_ok; ++j) atomicAdd(o0 + j, x[j]);
  } else if constexpr (EPI == EPI_RED_SCATTER) {
    // reduce-scatter fused into wgrad: add straight into the gradient shard of the rank that owns the element
    const int64_t idx = e.flat_off + static_cast<int64_t>(row) * e.ldo + col;
    if (e.compact) {
      // owners hold only their own chunks, packed: address by the position inside the owner's shard
      int owner; long long local;
      if (vec && e.chunk_aligned) {
        grb_chunk_place(idx, static_cast<int>(-e.shard), static_cast<unsigned>(e.world), owner, local);
        if (!grb_ok(e, owner < e.world && (e.peer_limit == 0 || local + 4 <= e.peer_limit), GRB_CHK_PEER)) return;
        float* o0 = reinterpret_cast<float*>(e.peers[owner]) + local;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o0), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]) : "memory");
      } else {
        for (int j = 0; j < n_ok; ++j) {
          grb_chunk_place(idx + j, static_cast<int>(-e.shard), static_cast<unsigned>(e.world), owner, local);
          if (!grb_ok(e, owner < e.world && (e.peer_limit == 0 || local < e.peer_limit), GRB_CHK_PEER)) return;
          atomicAdd(reinterpret_cast<float*>(e.peers[owner]) + local, x[j]);
        }
      }
    } else if (vec && e.chunk_aligned) {
      const int owner = grb_owner(idx, e.shard, e.world);
      if (!grb_ok(e, owner >= 0 && owner < e.world && idx >= 0 && (e.peer_limit == 0 || idx + 4 <= e.peer_limit), GRB_CHK_PEER)) return;
      float* o0 = reinterpret_cast<float*>(e.peers[owner]) + idx;
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o0), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]) : "memory");
    } else {
      for (int j = 0; j < n_ok; ++j) {
        const int owner = grb_owner(idx + j, e.shard, e.world);
        if (!grb_ok(e, owner >= 0 && owner < e.world && (e.peer_limit == 0 || idx + j < e.peer_limit), GRB_CHK_PEER)) return;
        atomicAdd(reinterpret_cast<float*>(e.peers[owner]) + idx + j, x[j]);
      }
    }
  }
}

// Warp-cooperative epilogue of a 32-row x [c_begin, c_end) slab of the accumulator tile.
//   taddr : TMEM address of (first lane of this warp's quadrant, column 0 of the accumulator)
//   row0  : global row of the quadrant's first lane;  n0 : global column of accumulator column 0
//   stage : this warp's EPI_STAGE_FLOATS floats of shared memory
// [c_begin, c_end) is one 128-column half of the tile, which is also the unit of the sum-of-squares partials.
template <int EPI>
__device__ __forceinline__ void epilogue_warp(const EpiArgs& e, uint32_t taddr, int row0, int n0, int M, int N,
                                              int c_begin, int c_end, float* stage, int lane) {
  const bool vec_ok = (e.ldo & 3) == 0;
  const int c4 = lane & 7, r4 = lane >> 3;
  uint32_t r[32];
  // after the transposition this lane handles rows 4 * it + r4 (it = 0..7): fetch their row scales once per tile
  float rsv[8];
  {
    const float mine = row_scale(e, row0 + lane, M);
    if (e.rstd_out && n0 == 0 && c_begin == 0 && row0 + lane < M) e.rstd_out[row0 + lane] = mine;
#pragma unroll
    for (int it = 0; it < 8; ++it) rsv[it] = __shfl_sync(0xffffffffu, mine, 4 * it + r4);
  }
  constexpr bool SSQ = (EPI == EPI_RESID_F32);
  constexpr bool CSUM = (EPI == EPI_GELU_BWD);
  float ssq[SSQ ? 8 : 1];
#pragma unroll
  for (int it = 0; it < (SSQ ? 8 : 1); ++it) ssq[it] = 0.f;
#pragma unroll 1
  for (int c = c_begin; c < c_end; c += 32) {
    const int col0 = n0 + c;
    if (col0 >= N) break;                     // uniform across the warp
    const int col = col0 + 4 * c4;
    const int n_ok = min(4, N - col);
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n_ok > 0 && e.bias) {
      bv.x = e.bias[col];
      if (n_ok > 1) bv.y = e.bias[col + 1];
      if (n_ok > 2) bv.z = e.bias[col + 2];
      if (n_ok > 3) bv.w = e.bias[col + 3];
    }
    float4 nw = make_float4(0.f, 0.f, 0.f, 0.f);
    if constexpr (SSQ) {
      if (n_ok > 0 && e.out2) {
        nw.x = e.normw[col];
        if (n_ok > 1) nw.y = e.normw[col + 1];
        if (n_ok > 2) nw.z = e.normw[col + 2];
        if (n_ok > 3) nw.w = e.normw[col + 3];
      }
    }
    // All eight rows' reads of `aux` are issued before the first store: with aux possibly aliasing out0 the
    // compiler must otherwise keep every load behind the previous store and the latencies add up.
    constexpr bool PRE = (EPI == EPI_RESID_F32 || EPI == EPI_GELU_BWD);
    const bool have_pre = PRE && vec_ok && n_ok == 4;   // n_ok == 4 also implies the chunk is inside N
    uint4 pre[PRE ? 8 : 1];
#pragma unroll
    for (int it = 0; it < (PRE ? 8 : 1); ++it) pre[it] = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (PRE) {
      if (have_pre) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int row = row0 + 4 * it + r4;
          if (row < M) {
            const size_t off = static_cast<size_t>(row) * e.ldo + col;
            if constexpr (EPI == EPI_RESID_F32) {
              pre[it] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(e.aux) + off);
            } else {
              const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(e.aux) + off);
              pre[it].x = u.x; pre[it].y = u.y;
            }
          }
        }
      }
    }
    __syncwarp();                             // previous chunk fully read out of the staging tile
    tmem_ld32(taddr + c, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float4*>(stage + lane * EPI_STAGE_LD + 4 * (j ^ (lane & 7))) =
          make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                      __uint_as_float(r[4 * j + 3]));
    __syncwarp();
    float cs[4] = {0.f, 0.f, 0.f, 0.f};
    if (n_ok > 0) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rr = 4 * it + r4;
        const int row = row0 + rr;
        if (row < M) {
          const float4 v = *reinterpret_cast<const float4*>(stage + rr * EPI_STAGE_LD + 4 * (c4 ^ (rr & 7)));
          epilogue_apply4<EPI>(e, v, bv, row, col, n_ok, vec_ok, have_pre, pre[PRE ? it : 0], rsv[it], nw,
                               ssq[SSQ ? it : 0], cs);
        }
      }
    }
    if constexpr (CSUM) {
      if (e.colsum) {
        // column sums of this 32 x 32 chunk: the four lanes that share a column group (r4 = 0..3) combine, then
        // one lane per group adds into the bias-gradient vector
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          cs[j] += __shfl_xor_sync(0xffffffffu, cs[j], 8);
          cs[j] += __shfl_xor_sync(0xffffffffu, cs[j], 16);
        }
        if (r4 == 0 && n_ok > 0) {
          float* dst = e.colsum + col;
          if (n_ok == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(cs[0]), "f"(cs[1]), "f"(cs[2]), "f"(cs[3]) : "memory");
          else
            for (int j = 0; j < n_ok; ++j) atomicAdd(dst + j, cs[j]);
        }
      }
    }
  }
  if constexpr (SSQ) {
    if (e.ssq_out && n0 + c_begin < N) {
      // sum of squares of this warp's 32 rows over its column part: the eight lanes of a row combine, then lane
      // c4 == it stores the value of row 4 * it + r4 (every lane stores exactly one row)
      const int part = (n0 + c_begin) >> 7, parts = (N + 127) >> 7;
      float mine = 0.f;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        float t = ssq[it];
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 4);
        if (c4 == it) mine = t;
      }
      const int row = row0 + 4 * c4 + r4;
      if (row < M && grb_ok(e, part >= 0 && part < parts, GRB_CHK_PARTS)) e.ssq_out[static_cast<size_t>(row) * parts + part] = mine;
    }
  }
}

// bf16 store epilogue through TMA: no transposition pass at all.  Each thread packs its accumulator row chunk
// (32 columns -> 64 bytes) and writes it into a [32 rows][64 B] shared-memory tile in the 64-byte-swizzle pattern
// (conflict-free for row-per-thread 16-byte stores); one lane then issues a bulk tensor store of the tile, which
// also clips rows >= M and columns >= N.  Two tiles per warp alternate so a store overlaps the next chunk.
//   tiles : this warp's 4 KB of shared memory, 512-byte aligned
__device__ __forceinline__ void epilogue_tma_store_bf16(const EpiArgs& e, const void* tmC, uint32_t taddr, int row0,
                                                        int n0, int M, int N, int c_begin, int c_end, uint8_t* tiles, int lane) {
  uint32_t r[32];
  int buf = 0;
  const float rs = row_scale(e, row0 + lane, M);                // of this thread's accumulator row
  if (e.rstd_out && n0 == 0 && c_begin == 0 && row0 + lane < M) e.rstd_out[row0 + lane] = rs;
  const float sc = e.alpha * rs;
#pragma unroll 1
  for (int c = c_begin; c < c_end; c += 32) {
    const int col0 = n0 + c;
    if (col0 >= N) break;
    __syncwarp();
    tmem_ld32(taddr + c, r);
    tmem_ld_wait();
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the tile written two chunks ago was read
    __syncwarp();
    uint8_t* tile = tiles + buf * 2048;
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        v[t] = __uint_as_float(r[8 * j + t]) * sc;
        if (e.bias && col0 + 8 * j + t < N) v[t] += e.bias[col0 + 8 * j + t];
      }
      *reinterpret_cast<uint4*>(tile + lane * 64 + ((j ^ sw) << 4)) =
          make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    }
    fence_proxy_async_smem();
    __syncwarp();
    // a bulk tensor store must start at a non-negative coordinate whose x is a multiple of 16 bytes
    if (lane == 0 && grb_ok(e, col0 >= 0 && (col0 & 7) == 0 && row0 >= 0, GRB_CHK_TMA_STORE)) {
      uint64_t pol;
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
      asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(
                       reinterpret_cast<uint64_t>(tmC)),
                   "r"(smem_u32(tile)), "r"(col0), "r"(row0), "l"(pol)
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    buf ^= 1;
  }
}
__device__ __forceinline__ void epilogue_tma_store_drain(int lane) {
  if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  __syncwarp();
}

// Chunk gather (EpiArgs::gather_*): 16-byte units of 8 bf16; unit i of the range holds elements lo + 8 i .., which
// live in the packed shard of rank (chunk % world).
__device__ __forceinline__ uint4 gather_load(const EpiArgs& e, int64_t el, int shift) {
  int owner; long long local;
  grb_chunk_place(el, shift, static_cast<unsigned>(e.world), owner, local);
  if (!grb_ok(e, owner < e.world && (e.peer_limit == 0 || local + 8 <= e.peer_limit), GRB_CHK_GATHER)) return make_uint4(0u, 0u, 0u, 0u);
  return *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(e.peers[owner]) + local);
}
__device__ __forceinline__ void gather_chunks(const EpiArgs& e, int block, int nblocks, int tid, int nthreads) {
  if (e.gather_hi <= e.gather_lo) return;
  const int shift = static_cast<int>(-e.shard);
  const int64_t lo = e.gather_lo;
  int64_t units = (e.gather_hi - lo) >> 3;
  if (!grb_ok(e, e.gather_cap == 0 || (units << 3) <= e.gather_cap, GRB_CHK_GATHER)) units = e.gather_cap >> 3;   // never past the workspace
  uint4* dst = reinterpret_cast<uint4*>(e.gather_dst);
  const int64_t stride = static_cast<int64_t>(nblocks) * nthreads;
  int64_t i = static_cast<int64_t>(block) * nthreads + tid;
  // eight independent 16-byte peer loads in flight per thread: the copy warps are few (64 threads per CTA) and an
  // NVLink round trip is long, so the bytes in flight, not the issue rate, set the gather's bandwidth
  for (; i + 7 * stride < units; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gather_load(e, lo + ((i + j * stride) << 3), shift);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[i + j * stride] = v[j];
  }
  for (; i < units; i += stride) dst[i] = gather_load(e, lo + (i << 3), shift);
}

// Cooperative copy of the segments in `e` by `nthreads` threads of each of `nblocks` blocks (16-byte units,
// block-cyclic so that consecutive threads read consecutive addresses), then the chunk gather if one is attached.
__device__ __forceinline__ void side_copy(const EpiArgs& e, int block, int nblocks, int tid, int nthreads) {
  gather_chunks(e, block, nblocks, tid, nthreads);
  for (int sgm = 0; sgm < e.n_copy; ++sgm) {
    const uint4* src = reinterpret_cast<const uint4*>(e.copy_src[sgm]);
    uint4* dst = reinterpret_cast<uint4*>(e.copy_dst[sgm]);
    const int64_t units = e.copy_bytes[sgm] >> 4;
    const int64_t stride = static_cast<int64_t>(nblocks) * nthreads;
    int64_t i = static_cast<int64_t>(block) * nthreads + tid;
    for (; i + 3 * stride < units; i += 4 * stride) {       // four independent 16-byte loads in flight per thread
      const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
      dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
    }
    for (; i < units; i += stride) dst[i] = src[i];
  }
}

}  // namespace grb
