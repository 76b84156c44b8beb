// Fused GEMM epilogues shared by the one-CTA and the CTA-pair tcgen05 kernels.
// Each epilogue thread owns one accumulator row (one TMEM lane) of its CTA's 128-row tile and walks a range
// of the 256 accumulator columns in chunks of 32 (tcgen05.ld 32x32b.x32).
#pragma once
#include "ptx.cuh"
#include "gemm_sm100.h"

namespace grb {

constexpr int EPI_BN = 256;   // accumulator columns per tile

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}

// ------------------------------------------------------------- epilogues
// Each epilogue thread owns one accumulator row (TMEM lane) of the tile and
// walks its 256 columns in chunks of 32.
template <int EPI>
__device__ __forceinline__ void epilogue_row(const EpiArgs& e, uint32_t taddr, int row, int n0, int M, int N,
                                             int c_begin, int c_end) {
  const bool row_ok = row < M;
  if constexpr (EPI == EPI_CE) {
    // 256-way softmax cross-entropy on the accumulator row.
    // loss_rows[row] = logsumexp(v) - v[label];  dlogits = (softmax - onehot) * alpha
    float* loss_rows = reinterpret_cast<float*>(e.out1);
    __nv_bfloat16* dlog = reinterpret_cast<__nv_bfloat16*>(e.out0);
    const uint8_t* labels = reinterpret_cast<const uint8_t*>(e.aux);
    const int label = row_ok ? static_cast<int>(labels[row]) : 0;
    float mx = -INFINITY;
    uint32_t r[32];
    for (int c = 0; c < EPI_BN; c += 32) {
      if (n0 + c >= N) break;
      __syncwarp();
      tmem_ld32(taddr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + c + j < N) mx = fmaxf(mx, __uint_as_float(r[j]));
    }
    float sum = 0.f, picked = 0.f;
    for (int c = 0; c < EPI_BN; c += 32) {
      if (n0 + c >= N) break;
      __syncwarp();
      tmem_ld32(taddr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float v = __uint_as_float(r[j]);
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
              float p0 = __expf(__uint_as_float(r[j]) - lse) - ((n0 + c + j) == label ? 1.f : 0.f);
              float p1 = __expf(__uint_as_float(r[j + 1]) - lse) - ((n0 + c + j + 1) == label ? 1.f : 0.f);
              pk[j >> 1] = pack_bf16(p0 * e.alpha, p1 * e.alpha);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<uint4*>(dst)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          } else {
            for (int j = 0; j < 32 && n0 + c + j < N; ++j) {
              float p = __expf(__uint_as_float(r[j]) - lse) - ((n0 + c + j) == label ? 1.f : 0.f);
              dst[j] = __float2bfloat16(p * e.alpha);
            }
          }
        }
      }
    }
    return;
  } else {
    uint32_t r[32];
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 32) {
      const int col = n0 + c;
      if (col >= N) break;           // uniform across the warp
      __syncwarp();
      tmem_ld32(taddr + c, r);       // .sync.aligned: every lane takes part
      tmem_ld_wait();
      if (!row_ok) continue;
      const bool full = (col + 32 <= N);
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * e.alpha;
      if (e.bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (full || col + j < N) v[j] += e.bias[col + j];
      }
      const size_t off = static_cast<size_t>(row) * e.ldo + col;

      if constexpr (EPI == EPI_STORE_BF16 || EPI == EPI_BIAS_GELU || EPI == EPI_GELU_BWD) {
        __nv_bfloat16* o0 = reinterpret_cast<__nv_bfloat16*>(e.out0) + off;
        if constexpr (EPI == EPI_GELU_BWD) {
          // v <- v * gelu'(a), a = saved pre-activation (bf16)
          const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(e.aux) + off;
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 u = reinterpret_cast<const uint4*>(a)[q];
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                v[q * 8 + 2 * t] *= gelu_grad_f(bf16_lo(w[t]));
                v[q * 8 + 2 * t + 1] *= gelu_grad_f(bf16_hi(w[t]));
              }
            }
          } else {
            for (int j = 0; j < 32 && col + j < N; ++j) v[j] *= gelu_grad_f(__bfloat162float(a[j]));
          }
        }
        if (full) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            reinterpret_cast<uint4*>(o0)[q] =
                make_uint4(pack_bf16(v[8 * q], v[8 * q + 1]), pack_bf16(v[8 * q + 2], v[8 * q + 3]),
                           pack_bf16(v[8 * q + 4], v[8 * q + 5]), pack_bf16(v[8 * q + 6], v[8 * q + 7]));
        } else {
          for (int j = 0; j < 32 && col + j < N; ++j) o0[j] = __float2bfloat16(v[j]);
        }
        if constexpr (EPI == EPI_BIAS_GELU) {
          // out0 = pre-activation (kept for backward), out1 = gelu(pre-activation)
          __nv_bfloat16* o1 = reinterpret_cast<__nv_bfloat16*>(e.out1) + off;
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              reinterpret_cast<uint4*>(o1)[q] = make_uint4(
                  pack_bf16(gelu_f(v[8 * q]), gelu_f(v[8 * q + 1])), pack_bf16(gelu_f(v[8 * q + 2]), gelu_f(v[8 * q + 3])),
                  pack_bf16(gelu_f(v[8 * q + 4]), gelu_f(v[8 * q + 5])),
                  pack_bf16(gelu_f(v[8 * q + 6]), gelu_f(v[8 * q + 7])));
          } else {
            for (int j = 0; j < 32 && col + j < N; ++j) o1[j] = __float2bfloat16(gelu_f(v[j]));
          }
        }
      } else if constexpr (EPI == EPI_STORE_F32 || EPI == EPI_RESID_F32) {
        float* o0 = reinterpret_cast<float*>(e.out0) + off;
        const float* rin = reinterpret_cast<const float*>(e.aux) + off;   // residual input (may alias out0)
        if (full) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float4 x = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            if constexpr (EPI == EPI_RESID_F32) {
              const float4 y = reinterpret_cast<const float4*>(rin)[q];
              x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
            }
            reinterpret_cast<float4*>(o0)[q] = x;
          }
        } else {
          for (int j = 0; j < 32 && col + j < N; ++j) {
            if constexpr (EPI == EPI_RESID_F32) o0[j] = rin[j] + v[j]; else o0[j] = v[j];
          }
        }
      } else if constexpr (EPI == EPI_RED_SCATTER) {
        // reduce-scatter fused into wgrad: add this partial tile straight into the owner's gradient shard
        const int64_t idx = e.flat_off + static_cast<int64_t>(row) * e.ldo + col;
        if (full && e.chunk_aligned) {
          float* o0 = reinterpret_cast<float*>(e.peers[idx / e.shard]) + idx;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o0 + 4 * q), "f"(v[4 * q]),
                         "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3])
                         : "memory");
        } else {
          for (int j = 0; j < 32 && col + j < N; ++j)
            atomicAdd(reinterpret_cast<float*>(e.peers[(idx + j) / e.shard]) + idx + j, v[j]);
        }
      } else if constexpr (EPI == EPI_RED_F32) {
        // fire-and-forget fp32 reduction into out0 (local or a peer's memory)
        float* o0 = reinterpret_cast<float*>(e.out0) + off;
        if (full) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o0 + 4 * q), "f"(v[4 * q]),
                         "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3])
                         : "memory");
        } else {
          for (int j = 0; j < 32 && col + j < N; ++j) atomicAdd(o0 + j, v[j]);
        }
      }
    }
  }
}

}  // namespace grb
