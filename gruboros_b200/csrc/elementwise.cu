// Memory-bound kernels around the GEMMs: embedding gather (+ one-hot / label
// preparation), RMSNorm forward / backward, column sums for bias gradients,
// loss reduction and dtype casts.  All are plain streaming kernels sized for
// HBM bandwidth: 16-byte accesses, one warp per row, rows re-read from L1.
//
// Reference ops replaced: nn.Embedding (mingru/minLM.py:58,97), nn.RMSNorm
// (mingru/minLM.py:67-74,120,130,137) and the autograd of both.
#include "ptx.cuh"
#include "elementwise.h"
#include <algorithm>

namespace grb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------ embedding
// tokens: uint8 [B, stride]; row r = b*T + t reads tokens[b*stride + t] and (label) tokens[b*stride + t + 1].
// Writes x[r,:] = E[id,:] (fp32), labels[r] (if non-null), onehot[r, 0..V) bf16 (if non-null).
// With normw: also xw[r,:] = bf16(x * normw) and ssq[r, 0..parts) = (sum of x^2, 0, 0, ...) - the inputs of the first
// RMSNorm in the form the GEMMs with a folded norm consume (gemm_sm100.h: rowss).
__global__ void embed_fwd_kernel(const uint8_t* __restrict__ tokens, int64_t stride, int B, int T, int D, int V,
                                 const float* __restrict__ E, float* __restrict__ x, uint8_t* __restrict__ labels,
                                 __nv_bfloat16* __restrict__ onehot, const float* __restrict__ normw,
                                 __nv_bfloat16* __restrict__ xw, float* __restrict__ ssq, int parts) {
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t M = static_cast<int64_t>(B) * T;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps_per_block + warp; r < M;
       r += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const int b = static_cast<int>(r / T), t = static_cast<int>(r % T);
    const int id = tokens[b * stride + t];
    const float4* src = reinterpret_cast<const float4*>(E + static_cast<size_t>(id) * D);
    float4* dst = reinterpret_cast<float4*>(x + static_cast<size_t>(r) * D);
    if (normw) {
      uint2* xr = reinterpret_cast<uint2*>(xw + static_cast<size_t>(r) * D);
      float ss = 0.f;
      for (int i = lane; i < D / 4; i += 32) {
        const float4 v = src[i];
        const float4 g = reinterpret_cast<const float4*>(normw)[i];
        dst[i] = v;
        xr[i] = make_uint2(pack_bf16(v.x * g.x, v.y * g.y), pack_bf16(v.z * g.z, v.w * g.w));
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
      ss = warp_sum(ss);
      for (int i = lane; i < parts; i += 32) ssq[static_cast<size_t>(r) * parts + i] = i == 0 ? ss : 0.f;
    } else {
      for (int i = lane; i < D / 4; i += 32) dst[i] = src[i];
    }
    if (labels && lane == 0) labels[r] = tokens[b * stride + t + 1];
    if (onehot) {
      __nv_bfloat16* oh = onehot + static_cast<size_t>(r) * V;
      for (int i = lane; i < V; i += 32) oh[i] = __float2bfloat16(i == id ? 1.f : 0.f);
    }
  }
}

// -------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w  -> bf16; rstd saved for backward.
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int64_t M, int D,
                                   float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = D / 4;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps_per_block + warp; r < M;
       r += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * D);
    float ss = 0.f;
    for (int i = lane; i < nv; i += 32) {
      const float4 v = xr[i];
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd) rstd[r] = rs;
    uint2* yr = reinterpret_cast<uint2*>(y + static_cast<size_t>(r) * D);
    const float4* wr = reinterpret_cast<const float4*>(w);
    for (int i = lane; i < nv; i += 32) {
      const float4 v = xr[i];
      const float4 g = wr[i];
      yr[i] = make_uint2(pack_bf16(v.x * rs * g.x, v.y * rs * g.y), pack_bf16(v.z * rs * g.z, v.w * rs * g.w));
    }
  }
}

// Backward of y = xhat * w, xhat = x * rstd, fused with the residual-gradient accumulation:
//   dxhat = dy * w;  c = mean(dxhat * xhat);  dx = rstd * (dxhat - xhat * c)
//   dres_out = dres_in + dx         (fp32, + optional bf16 copy for the next GEMM)
//   dw      += sum_rows dy * xhat   (per-warp shared-memory partials, one atomic per column per CTA)
//   dcol    += sum_rows dres_out    (optional: gradient of a bias added to the residual stream)
// `prescaled`: the norm was folded into its consumer GEMM (A operand = x * w, accumulator rows scaled by rstd), whose
// backward produced dy' = rstd * dy (the gradient w.r.t. x * w).  In terms of dy' the same quantities are
//   dx = dy' * w - x * rstd^2 * mean(dy' * w * x),   dw += sum_rows dy' * x.
// Both forms are  dx = so * (dy * w) - x * (so * rstd^2 * dot / D),  dw += so * dy * x,  dot = sum(dy * w * x),
// with so = rstd (plain) or 1 (prescaled).
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                                   const float* __restrict__ rstd, const float* __restrict__ w,
                                   const float* __restrict__ dres_in, float* __restrict__ dres_out,
                                   __nv_bfloat16* __restrict__ dres16, float* __restrict__ dw,
                                   float* __restrict__ dcol, int64_t M, int D, int prescaled) {
  extern __shared__ float sacc[];   // [warps][D] dw partials, then [warps][D] dcol partials
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nv = D / 4;
  float* my_dw = sacc + static_cast<size_t>(warp) * D;
  float* my_dc = sacc + static_cast<size_t>(warps_per_block + warp) * D;
  for (int i = lane; i < D; i += 32) { my_dw[i] = 0.f; if (dcol) my_dc[i] = 0.f; }
  __syncwarp();
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps_per_block + warp; r < M;
       r += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(r) * D);
    const uint2* dyr = reinterpret_cast<const uint2*>(dy + static_cast<size_t>(r) * D);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const float rs = rstd[r];
    float dot = 0.f;
    for (int i = lane; i < nv; i += 32) {
      const float4 xv = xr[i];
      const float4 g = wr[i];
      const uint2 d = dyr[i];
      dot += bf16_lo(d.x) * g.x * xv.x + bf16_hi(d.x) * g.y * xv.y + bf16_lo(d.y) * g.z * xv.z + bf16_hi(d.y) * g.w * xv.w;
    }
    dot = warp_sum(dot);
    const float so = prescaled ? 1.f : rs;
    const float sx = so * rs * rs * dot / D;
    const float4* dri = dres_in ? reinterpret_cast<const float4*>(dres_in + static_cast<size_t>(r) * D) : nullptr;
    float4* dro = reinterpret_cast<float4*>(dres_out + static_cast<size_t>(r) * D);
    uint2* dr16 = dres16 ? reinterpret_cast<uint2*>(dres16 + static_cast<size_t>(r) * D) : nullptr;
    for (int i = lane; i < nv; i += 32) {
      const float4 xv = xr[i];
      const float4 g = wr[i];
      const uint2 d = dyr[i];
      const float d0 = bf16_lo(d.x), d1 = bf16_hi(d.x), d2 = bf16_lo(d.y), d3 = bf16_hi(d.y);
      const float h0 = xv.x * so, h1 = xv.y * so, h2 = xv.z * so, h3 = xv.w * so;
      float4 o;
      o.x = so * d0 * g.x - xv.x * sx;
      o.y = so * d1 * g.y - xv.y * sx;
      o.z = so * d2 * g.z - xv.z * sx;
      o.w = so * d3 * g.w - xv.w * sx;
      if (dri) { const float4 p = dri[i]; o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w; }
      dro[i] = o;
      if (dr16) dr16[i] = make_uint2(pack_bf16(o.x, o.y), pack_bf16(o.z, o.w));
      float4* a = reinterpret_cast<float4*>(my_dw) + i;
      float4 av = *a;
      av.x += d0 * h0; av.y += d1 * h1; av.z += d2 * h2; av.w += d3 * h3;
      *a = av;
      if (dcol) {
        float4* q = reinterpret_cast<float4*>(my_dc) + i;
        float4 qv = *q;
        qv.x += o.x; qv.y += o.y; qv.z += o.z; qv.w += o.w;
        *q = qv;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f, t = 0.f;
    for (int wv = 0; wv < warps_per_block; ++wv) {
      s += sacc[static_cast<size_t>(wv) * D + i];
      if (dcol) t += sacc[static_cast<size_t>(warps_per_block + wv) * D + i];
    }
    atomicAdd(dw + i, s);
    if (dcol) atomicAdd(dcol + i, t);
  }
}

// Faster variant for D <= 4096: a CTA of 256 threads walks groups of RB rows; thread t owns the float4 columns
// t, t+256, ... of every row, so the dw / dcol partial sums stay in registers for the whole kernel and only the
// per-row dot product needs a block reduction (one __syncthreads per group, double-buffered partials).
template <int NCH>
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                        const float* __restrict__ rstd, const float* __restrict__ w,
                        const float* __restrict__ dres_in, float* __restrict__ dres_out,
                        __nv_bfloat16* __restrict__ dres16, float* __restrict__ dw, float* __restrict__ dcol,
                        int64_t M, int D, int prescaled) {
  constexpr int RB = NCH == 1 ? 4 : 2;
  __shared__ float part[2][RB][8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nv = D / 4;
  float4 wv[NCH], adw[NCH], adc[NCH];
  bool act[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    act[j] = tid + 256 * j < nv;
    wv[j] = act[j] ? reinterpret_cast<const float4*>(w)[tid + 256 * j] : make_float4(0, 0, 0, 0);
    adw[j] = make_float4(0, 0, 0, 0);
    adc[j] = make_float4(0, 0, 0, 0);
  }
  int buf = 0;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * RB; r0 < M; r0 += static_cast<int64_t>(gridDim.x) * RB, buf ^= 1) {
    float4 xv[RB][NCH], pv[RB][NCH];      // x, incoming residual gradient (prefetched with the first loads)
    uint2 dv[RB][NCH];
    float dot[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int64_t row = r0 + r;
      dot[r] = 0.f;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        if (row < M && act[j]) {
          xv[r][j] = reinterpret_cast<const float4*>(x + static_cast<size_t>(row) * D)[tid + 256 * j];
          dv[r][j] = reinterpret_cast<const uint2*>(dy + static_cast<size_t>(row) * D)[tid + 256 * j];
          pv[r][j] = dres_in ? reinterpret_cast<const float4*>(dres_in + static_cast<size_t>(row) * D)[tid + 256 * j]
                             : make_float4(0, 0, 0, 0);
        } else {
          xv[r][j] = make_float4(0, 0, 0, 0);
          pv[r][j] = make_float4(0, 0, 0, 0);
          dv[r][j] = make_uint2(0, 0);
        }
        dot[r] += bf16_lo(dv[r][j].x) * wv[j].x * xv[r][j].x + bf16_hi(dv[r][j].x) * wv[j].y * xv[r][j].y +
                  bf16_lo(dv[r][j].y) * wv[j].z * xv[r][j].z + bf16_hi(dv[r][j].y) * wv[j].w * xv[r][j].w;
      }
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const float s = warp_sum(dot[r]);
      if (lane == 0) part[buf][r][warp] = s;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const int64_t row = r0 + r;
      if (row >= M) break;
      float tot = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) tot += part[buf][r][k];
      const float rs = rstd[row];
      const float so = prescaled ? 1.f : rs;
      const float sx = so * rs * rs * tot / D;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        if (!act[j]) continue;
        const size_t off = static_cast<size_t>(row) * D / 4 + tid + 256 * j;
        const float d0 = bf16_lo(dv[r][j].x), d1 = bf16_hi(dv[r][j].x), d2 = bf16_lo(dv[r][j].y), d3 = bf16_hi(dv[r][j].y);
        const float h0 = xv[r][j].x * so, h1 = xv[r][j].y * so, h2 = xv[r][j].z * so, h3 = xv[r][j].w * so;
        float4 o;
        o.x = so * d0 * wv[j].x - xv[r][j].x * sx;
        o.y = so * d1 * wv[j].y - xv[r][j].y * sx;
        o.z = so * d2 * wv[j].z - xv[r][j].z * sx;
        o.w = so * d3 * wv[j].w - xv[r][j].w * sx;
        o.x += pv[r][j].x; o.y += pv[r][j].y; o.z += pv[r][j].z; o.w += pv[r][j].w;
        reinterpret_cast<float4*>(dres_out)[off] = o;
        if (dres16) reinterpret_cast<uint2*>(dres16)[off] = make_uint2(pack_bf16(o.x, o.y), pack_bf16(o.z, o.w));
        adw[j].x += d0 * h0; adw[j].y += d1 * h1; adw[j].z += d2 * h2; adw[j].w += d3 * h3;
        adc[j].x += o.x; adc[j].y += o.y; adc[j].z += o.z; adc[j].w += o.w;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    if (!act[j]) continue;
    const int c0 = 4 * (tid + 256 * j);
    atomicAdd(dw + c0, adw[j].x); atomicAdd(dw + c0 + 1, adw[j].y); atomicAdd(dw + c0 + 2, adw[j].z); atomicAdd(dw + c0 + 3, adw[j].w);
    if (dcol) {
      atomicAdd(dcol + c0, adc[j].x); atomicAdd(dcol + c0 + 1, adc[j].y); atomicAdd(dcol + c0 + 2, adc[j].z); atomicAdd(dcol + c0 + 3, adc[j].w);
    }
  }
}

// Variant of the above whose inputs arrive through a ring of row slots in shared memory, filled by bulk copies
// (cp.async.bulk, one mbarrier per slot): the bytes in flight per SM are the ring (up to 8 rows: 8 x 20 KB for D = 2048)
// instead of what two CTAs can hold in registers, which is what a streaming kernel of 32 KB per row needs to keep
// HBM busy.  Two CTAs per SM walk rows blockIdx.x, blockIdx.x + gridDim.x, ...; per row there is one mbarrier
// wait and one __syncthreads (the block reduction of the row's dot product), after which every thread holds its
// part of the row in registers and the slot is refilled.  Same results as rmsnorm_bwd_rows_kernel.
constexpr int RING_MAX_SLOTS = 8;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int NCH>
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_ring_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                        const float* __restrict__ rstd, const float* __restrict__ w,
                        const float* __restrict__ dres_in, float* __restrict__ dres_out,
                        __nv_bfloat16* __restrict__ dres16, float* __restrict__ dw, float* __restrict__ dcol,
                        int64_t M, int D, int slots, int* err, int prescaled) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full[RING_MAX_SLOTS];
  __shared__ float part[2][8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nv = D / 4;
  const uint32_t xb = D * 4, yb = D * 2;
  const uint32_t slot_bytes = xb + (dres_in ? xb : 0) + yb;     // x | dres_in | dy, all multiples of 16 bytes
  const int64_t first = blockIdx.x, stride = gridDim.x;
  const int64_t nrows = first < M ? (M - first + stride - 1) / stride : 0;

  if (tid == 0) {
    for (int i = 0; i < RING_MAX_SLOTS; ++i) mbar_init(&full[i], 1);
    fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int64_t i) {                                  // thread 0: start the copies of this CTA's i-th row
    const int64_t row = first + i * stride;
    uint8_t* dst = ring + static_cast<size_t>(i % slots) * slot_bytes;
    uint64_t* bar = &full[i % slots];
    mbar_expect_tx(bar, slot_bytes);
    bulk_load(dst, x + row * D, xb, bar);
    if (dres_in) bulk_load(dst + xb, dres_in + row * D, xb, bar);
    bulk_load(dst + slot_bytes - yb, dy + row * D, yb, bar);
  };
  if (tid == 0)
    for (int64_t i = 0; i < nrows && i < slots; ++i) issue(i);

  float4 wv[NCH], adw[NCH], adc[NCH];
  bool act[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    act[j] = tid + 256 * j < nv;
    wv[j] = act[j] ? reinterpret_cast<const float4*>(w)[tid + 256 * j] : make_float4(0, 0, 0, 0);
    adw[j] = make_float4(0, 0, 0, 0);
    adc[j] = make_float4(0, 0, 0, 0);
  }
  float rs_next = nrows > 0 ? rstd[first] : 0.f;
  bool ok = true;
  int64_t done = 0;
  for (int64_t i = 0; i < nrows; ++i) {
    const int slot = static_cast<int>(i % slots);
    const int64_t row = first + i * stride;
    const float rs = rs_next;
    if (i + 1 < nrows) rs_next = rstd[row + stride];
    if (!mbar_wait(&full[slot], static_cast<uint32_t>((i / slots) & 1))) ok = false;
    if (!__syncthreads_and(ok)) { ok = false; break; }          // block-uniform
    done = i + 1;
    const uint8_t* src = ring + static_cast<size_t>(slot) * slot_bytes;
    float4 xv[NCH], pv[NCH];
    uint2 dv[NCH];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      if (act[j]) {
        xv[j] = reinterpret_cast<const float4*>(src)[tid + 256 * j];
        pv[j] = dres_in ? reinterpret_cast<const float4*>(src + xb)[tid + 256 * j] : make_float4(0, 0, 0, 0);
        dv[j] = reinterpret_cast<const uint2*>(src + slot_bytes - yb)[tid + 256 * j];
      } else {
        xv[j] = make_float4(0, 0, 0, 0);
        pv[j] = make_float4(0, 0, 0, 0);
        dv[j] = make_uint2(0, 0);
      }
      dot += bf16_lo(dv[j].x) * wv[j].x * xv[j].x + bf16_hi(dv[j].x) * wv[j].y * xv[j].y +
             bf16_lo(dv[j].y) * wv[j].z * xv[j].z + bf16_hi(dv[j].y) * wv[j].w * xv[j].w;
    }
    const float sdot = warp_sum(dot);
    if (lane == 0) part[i & 1][warp] = sdot;
    __syncthreads();                                            // partial sums visible; every thread has read the slot
    if (tid == 0 && i + slots < nrows) {
      fence_proxy_async_smem();                                 // those reads before the copy that overwrites the slot
      issue(i + slots);
    }
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += part[i & 1][k];
    const float so = prescaled ? 1.f : rs;
    const float sx = so * rs * rs * tot / D;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      if (!act[j]) continue;
      const size_t off = static_cast<size_t>(row) * D / 4 + tid + 256 * j;
      const float d0 = bf16_lo(dv[j].x), d1 = bf16_hi(dv[j].x), d2 = bf16_lo(dv[j].y), d3 = bf16_hi(dv[j].y);
      const float h0 = xv[j].x * so, h1 = xv[j].y * so, h2 = xv[j].z * so, h3 = xv[j].w * so;
      float4 o;
      o.x = so * d0 * wv[j].x - xv[j].x * sx + pv[j].x;
      o.y = so * d1 * wv[j].y - xv[j].y * sx + pv[j].y;
      o.z = so * d2 * wv[j].z - xv[j].z * sx + pv[j].z;
      o.w = so * d3 * wv[j].w - xv[j].w * sx + pv[j].w;
      reinterpret_cast<float4*>(dres_out)[off] = o;
      if (dres16) reinterpret_cast<uint2*>(dres16)[off] = make_uint2(pack_bf16(o.x, o.y), pack_bf16(o.z, o.w));
      adw[j].x += d0 * h0; adw[j].y += d1 * h1; adw[j].z += d2 * h2; adw[j].w += d3 * h3;
      adc[j].x += o.x; adc[j].y += o.y; adc[j].z += o.z; adc[j].w += o.w;
    }
  }
  if (!ok) {
    // a copy did not arrive in time: report; give the copies still outstanding one more bounded wait each so that
    // nothing lands in shared memory after the CTA has gone; the column sums of this CTA are dropped
    if (tid == 0) {
      atomicExch(err, 11);
      const int64_t issued = nrows < done + slots ? nrows : done + slots;
      for (int64_t i = done; i < issued; ++i) mbar_wait(&full[i % slots], static_cast<uint32_t>((i / slots) & 1));
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    if (!act[j]) continue;
    const int c0 = 4 * (tid + 256 * j);
    atomicAdd(dw + c0, adw[j].x); atomicAdd(dw + c0 + 1, adw[j].y); atomicAdd(dw + c0 + 2, adw[j].z); atomicAdd(dw + c0 + 3, adw[j].w);
    if (dcol) {
      atomicAdd(dcol + c0, adc[j].x); atomicAdd(dcol + c0 + 1, adc[j].y); atomicAdd(dcol + c0 + 2, adc[j].z); atomicAdd(dcol + c0 + 3, adc[j].w);
    }
  }
}

// --------------------------------------------------------------- colsum
// out[n] += sum_rows a[row, n] for bf16 a [M, ld].  Block = 256 columns x a strip of rows.
__global__ void colsum_bf16_kernel(const __nv_bfloat16* __restrict__ a, int64_t ld, int64_t M, int N,
                                   float* __restrict__ out) {
  __shared__ float red[8][256 + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 256 + lane * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < N) {
    for (int64_t r = static_cast<int64_t>(blockIdx.y) * 8 + warp; r < M; r += static_cast<int64_t>(gridDim.y) * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(a + static_cast<size_t>(r) * ld + col);
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = threadIdx.x;   // 256 threads
  float s = 0.f;
#pragma unroll
  for (int wv = 0; wv < 8; ++wv) s += red[wv][c];
  if (blockIdx.x * 256 + c < N) atomicAdd(out + blockIdx.x * 256 + c, s);
}

// ----------------------------------------------------------------- misc
// out[0] (+)= scale * sum(v[0..n))   single block
__global__ void sum_scale_kernel(const float* __restrict__ v, int64_t n, float scale, float* __restrict__ out,
                                 int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += v[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + t * scale;
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t n) {
  const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    const float4 a = *reinterpret_cast<const float4*>(in + i);
    const float4 b = *reinterpret_cast<const float4*>(in + i + 4);
    *reinterpret_cast<uint4*>(out + i) =
        make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
  } else {
    for (int64_t j = i; j < n; ++j) out[j] = __float2bfloat16(in[j]);
  }
}

static int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace grb

using namespace grb;
#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -5)

extern "C" int grb_embed_fwd(const uint8_t* tokens, int64_t stride, int B, int T, int D, int V, const float* E,
                             float* x, uint8_t* labels, void* onehot, const float* normw, void* xw, float* ssq, int parts,
                             void* stream) {
  if (D % 4) return -30;
  const int64_t M = static_cast<int64_t>(B) * T;
  if (M == 0) return 0;
  const int blocks = static_cast<int>(std::min<int64_t>((M + 7) / 8, num_sms() * 8));
  if (normw && (!xw || !ssq || parts < 1)) return -32;
  embed_fwd_kernel<<<blocks, 256, 0, ST(stream)>>>(tokens, stride, B, T, D, V, E, x, labels,
                                                  reinterpret_cast<__nv_bfloat16*>(onehot), normw,
                                                  reinterpret_cast<__nv_bfloat16*>(xw), ssq, parts);
  return LAUNCH_OK();
}

extern "C" int grb_rmsnorm_fwd(const float* x, const float* w, void* y, float* rstd, int64_t M, int D, float eps,
                               void* stream) {
  if (D % 4) return -30;
  if (M == 0) return 0;
  const int blocks = static_cast<int>(std::min<int64_t>((M + 7) / 8, num_sms() * 8));
  rmsnorm_fwd_kernel<<<blocks, 256, 0, ST(stream)>>>(x, w, reinterpret_cast<__nv_bfloat16*>(y), rstd, M, D, eps);
  return LAUNCH_OK();
}

template <int NCH>
static int launch_rmsnorm_ring(const __nv_bfloat16* dy, const float* x, const float* rstd, const float* w,
                               const float* dres_in, float* dres_out, __nv_bfloat16* d16, float* dw, float* dcol, int64_t M,
                               int D, int* err, int prescaled, cudaStream_t st) {
  const size_t slot = static_cast<size_t>(D) * (dres_in ? 10 : 6);
  // two CTAs per SM: while one waits at its per-row block barrier the other computes (with a single CTA the two
  // barriers per row serialise the rows and the ring is slower than the register version)
  constexpr int kCtasPerSm = 2;
  int slots = static_cast<int>((200 * 1024 / kCtasPerSm) / slot);
  if (slots > RING_MAX_SLOTS) slots = RING_MAX_SLOTS;
  if (slots < 2) return -31;
  const size_t smem = slot * slots;
  static size_t granted = 0;
  if (smem > 40 * 1024 && smem > granted) {
    if (cudaFuncSetAttribute(rmsnorm_bwd_ring_kernel<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return -4;
    granted = smem;
  }
  const int blocks = static_cast<int>(std::min<int64_t>(M, static_cast<int64_t>(num_sms()) * kCtasPerSm));
  rmsnorm_bwd_ring_kernel<NCH><<<blocks, 256, smem, st>>>(dy, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, slots, err,
                                                          prescaled);
  return LAUNCH_OK();
}

extern "C" int grb_rmsnorm_bwd(const void* dy, const float* x, const float* rstd, const float* w, const float* dres_in,
                               float* dres_out, void* dres16, float* dw, float* dcol, int64_t M, int D, int prescaled,
                               int* err, void* stream) {
  if (D % 4) return -30;
  if (M == 0) return 0;
  // shared-memory ring fed by bulk copies: needs 16-byte rows in every input and a ring that fits
  const bool aligned = D % 8 == 0 && !((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) |
                                        reinterpret_cast<uintptr_t>(dres_in)) & 15);
  if (err && aligned && D <= 3072 && M >= 4 * num_sms()) {      // (wider rows need more registers than two CTAs per SM leave)
    const __nv_bfloat16* dyp = reinterpret_cast<const __nv_bfloat16*>(dy);
    __nv_bfloat16* d16 = reinterpret_cast<__nv_bfloat16*>(dres16);
    switch ((D / 4 + 255) / 256) {
      case 1: return launch_rmsnorm_ring<1>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, err, prescaled, ST(stream));
      case 2: return launch_rmsnorm_ring<2>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, err, prescaled, ST(stream));
      default: return launch_rmsnorm_ring<3>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, err, prescaled, ST(stream));
    }
  }
  if (D <= 4096) {
    const int nch = (D / 4 + 255) / 256;
    const int blocks = static_cast<int>(std::min<int64_t>((M + 1) / 2, num_sms() * 4));
    const __nv_bfloat16* dyp = reinterpret_cast<const __nv_bfloat16*>(dy);
    __nv_bfloat16* d16 = reinterpret_cast<__nv_bfloat16*>(dres16);
    switch (nch) {
      case 1: rmsnorm_bwd_rows_kernel<1><<<blocks, 256, 0, ST(stream)>>>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, prescaled); break;
      case 2: rmsnorm_bwd_rows_kernel<2><<<blocks, 256, 0, ST(stream)>>>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, prescaled); break;
      case 3: rmsnorm_bwd_rows_kernel<3><<<blocks, 256, 0, ST(stream)>>>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, prescaled); break;
      default: rmsnorm_bwd_rows_kernel<4><<<blocks, 256, 0, ST(stream)>>>(dyp, x, rstd, w, dres_in, dres_out, d16, dw, dcol, M, D, prescaled); break;
    }
    return LAUNCH_OK();
  }
  int warps = 8;
  while (warps > 1 && static_cast<size_t>(2 * warps) * D * sizeof(float) > 160 * 1024) warps >>= 1;
  const size_t smem = static_cast<size_t>(2 * warps) * D * sizeof(float);
  if (smem > 200 * 1024) return -31;
  static size_t smem_set = 0;
  if (smem > smem_set) {
    if (cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return -4;
    smem_set = smem;
  }
  const int blocks = static_cast<int>(std::min<int64_t>((M + warps - 1) / warps, num_sms()));
  rmsnorm_bwd_kernel<<<blocks, warps * 32, smem, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(dy), x, rstd, w,
                                                               dres_in, dres_out,
                                                               reinterpret_cast<__nv_bfloat16*>(dres16), dw, dcol, M, D,
                                                               prescaled);
  return LAUNCH_OK();
}

extern "C" int grb_colsum_bf16(const void* a, int64_t ld, int64_t M, int N, float* out, void* stream) {
  if (N % 8 || ld % 8) return -30;
  if (M == 0) return 0;
  dim3 grid((N + 255) / 256, static_cast<unsigned>(std::min<int64_t>((M + 63) / 64, 64)));
  colsum_bf16_kernel<<<grid, 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(a), ld, M, N, out);
  return LAUNCH_OK();
}

extern "C" int grb_sum_scale(const float* v, int64_t n, float scale, float* out, int accumulate, void* stream) {
  sum_scale_kernel<<<1, 1024, 0, ST(stream)>>>(v, n, scale, out, accumulate);
  return LAUNCH_OK();
}

extern "C" int grb_cast_f32_bf16(const float* in, void* out, int64_t n, void* stream) {
  if (n == 0) return 0;
  const int64_t threads = (n + 7) / 8;
  cast_f32_bf16_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, ST(stream)>>>(
      in, reinterpret_cast<__nv_bfloat16*>(out), n);
  return LAUNCH_OK();
}
