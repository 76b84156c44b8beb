// minGRU recurrence, forward and backward, for sm_100a.
//
//   z_t = sigmoid(k_t),  g(u) = u + 0.5 (u >= 0) | sigmoid(u) (u < 0)
//   h_t = (1 - z_t) * h_{t-1} + z_t * g(u_t),     h_{-1} = h0 (or 0)
//
// This is the linear-space form of the log-space Heinsen scan the reference
// evaluates with softplus / cumsum / logcumsumexp (mingru/minGRU.py:16-28,
// 56-69); all terms are convex combinations of positive numbers, so fp32 in
// linear space is at least as accurate as the reference's fp32 log-space path.
//
// Layout: k, u, h are bf16 [B, T, C] with a row stride (k and u are usually the
// two column halves of one GEMM output).  One CTA owns 64 channels of one batch
// row and walks T in order, so no inter-CTA communication is needed.  Raw tiles
// arrive through a 4-stage TMA ring.  Inside a super-step the four warps each
// take a slice of consecutive time steps, scan it locally from a zero state
// (keeping per-step (prefix-product, local value) pairs in registers), exchange
// slice aggregates through shared memory, and finish with one FMA per element.  Results go to a per-warp staging tile
// and leave with one bulk tensor store per slice (which also clips the ragged ends of T and C); super-steps that lie
// wholly inside T run a variant of the slice loop without any bounds handling.
#include <type_traits>

#include "ptx.cuh"
#include "tmap.h"
#include "scan.h"

namespace grb {

constexpr int SC_CH = 64;
#ifndef GRB_SCAN_WARPS
#define GRB_SCAN_WARPS 4
#endif
#ifndef GRB_SCAN_FSTEPS
#define GRB_SCAN_FSTEPS 16
#endif
#ifndef GRB_SCAN_RSTEPS
#define GRB_SCAN_RSTEPS 8
#endif
constexpr int SC_NW = GRB_SCAN_WARPS;               // warps per CTA: each takes a slice of a super-step
constexpr int SC_THREADS = 32 * SC_NW;
#ifndef GRB_SCAN_STAGES
#define GRB_SCAN_STAGES 3
#endif
constexpr int SC_STAGES = GRB_SCAN_STAGES;

constexpr int F_STEPS = GRB_SCAN_FSTEPS;                       // steps per warp per super-step
constexpr int F_TS = SC_NW * F_STEPS;
constexpr int F_TILE = F_TS * SC_CH * 2;          // bytes of one tensor tile
constexpr int F_STAGE_BYTES = 2 * F_TILE;         // k, u
constexpr int F_OUT_WARP = F_STEPS * SC_CH * 2;   // staging tile of one warp: its slice of h

constexpr int R_STEPS = GRB_SCAN_RSTEPS;
constexpr int R_TS = SC_NW * R_STEPS;
constexpr int R_TILE = R_TS * SC_CH * 2;
constexpr int R_STAGE_BYTES = 4 * R_TILE;         // k, u, h_prev, g
constexpr int R_OUT_WARP = 2 * R_STEPS * SC_CH * 2;   // staging tiles of one warp: its slices of dk and du

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcpf(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Both bf16 halves of a word clamped from below at -40 with one instruction (bf16(-40) = 0xC220).  The clamp keeps
// (1 + e^-k)(1 + e^-u) finite (<= e^80 < FLT_MAX); large positive inputs need none: their exponentials flush to zero.
__device__ __forceinline__ uint32_t clamp_below_bf16x2(uint32_t w) {
  uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(w), "r"(0xC220C220u));
  return r;
}

// a = 1 - z, z = sigmoid(k), g = g(u), gp = g'(u) for inputs already clamped from below.  Two exponentials and one
// reciprocal serve both sigmoids.
__device__ __forceinline__ void gate_act(float k, float u, float& a, float& z, float& g, float& gp) {
  const float ea = ex2f(-1.4426950408889634f * k);    // e^{-k}
  const float eb = ex2f(-1.4426950408889634f * u);    // e^{-u}
  const float r = rcpf((1.f + ea) * (1.f + eb));
  z = r * (1.f + eb);
  const float s = r * (1.f + ea);                     // sigmoid(u)
  a = ea * z;
  const bool pos = u >= 0.f;
  g = pos ? u + 0.5f : s;
  gp = pos ? 1.f : s * (eb * s);
}
// Forward only needs g: u + 0.5 lies above sigmoid(u) exactly where u >= 0 (the sigmoid is concave there and its
// slope at 0 is 1/4; for u < 0 it is convex and stays above its tangent 0.5 + u/4 > 0.5 + u), so g = max of the two.
__device__ __forceinline__ void gate_act_fwd(float k, float u, float& a, float& b) {
  const float ea = ex2f(-1.4426950408889634f * k);
  const float eb = ex2f(-1.4426950408889634f * u);
  const float r = rcpf((1.f + ea) * (1.f + eb));
  const float z = r * (1.f + eb);
  const float s = r * (1.f + ea);
  a = ea * z;
  b = z * fmaxf(u + 0.5f, s);
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* desc, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_store_3d(const void* desc, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(desc)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// The staging tile a bulk store was issued from may be rewritten / released once the store has read it.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

struct ScanFwdArgs {
  int B, T, C;
  const float* h0;       // [B, C] or null
  __nv_bfloat16* h;      // [B, T, ldh]
  int64_t ldh;
  float* h_last;         // [B, C] or null
  int* err;
};

// TMA_OUT: h leaves through the staging tile and a bulk tensor store (needs a tensor map of h: 16-byte aligned base
// and row stride); otherwise every lane stores its own values.
template <bool TMA_OUT>
__global__ void __launch_bounds__(SC_THREADS)
scan_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmU,
                const __grid_constant__ CUtensorMap tmH, const ScanFwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* out_stage = smem + SC_STAGES * F_STAGE_BYTES;                      // [SC_NW][F_STEPS][64] bf16
  uint64_t* full = reinterpret_cast<uint64_t*>(out_stage + SC_NW * F_OUT_WARP);
  float2* agg = reinterpret_cast<float2*>(full + SC_STAGES);   // [2][SC_NW][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, c0 = blockIdx.x * SC_CH;
  const int ch = c0 + 2 * lane;
  const int nss = (p.T + F_TS - 1) / F_TS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SC_STAGES; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmU);
    if (TMA_OUT) tma_prefetch_desc(&tmH);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < SC_STAGES && s < nss; ++s) {
      mbar_expect_tx(&full[s], F_STAGE_BYTES);
      tma_load_3d(smem + s * F_STAGE_BYTES, &tmK, &full[s], c0, s * F_TS, b);
      tma_load_3d(smem + s * F_STAGE_BYTES + F_TILE, &tmU, &full[s], c0, s * F_TS, b);
    }
  }

  float c_0 = 0.f, c_1 = 0.f;   // carried hidden state of this lane's two channels
  if (p.h0) {
    if (ch < p.C) c_0 = p.h0[static_cast<size_t>(b) * p.C + ch];
    if (ch + 1 < p.C) c_1 = p.h0[static_cast<size_t>(b) * p.C + ch + 1];
  }
  uint32_t* my_stage = reinterpret_cast<uint32_t*>(out_stage + warp * F_OUT_WARP) + lane;

  for (int ss = 0; ss < nss; ++ss) {
    const int stage = ss % SC_STAGES;
    const uint32_t phase = (ss / SC_STAGES) & 1;
    const int par = ss & 1;
    bool ok = mbar_wait(&full[stage], phase);

    float S0[F_STEPS], S1[F_STEPS], P0[F_STEPS], P1[F_STEPS];
    const int tbase = ss * F_TS + warp * F_STEPS;
    {
      const uint32_t* sk = reinterpret_cast<const uint32_t*>(smem + stage * F_STAGE_BYTES) + (warp * F_STEPS) * (SC_CH / 2) + lane;
      const uint32_t* su = sk + F_TILE / 4;
      float s0 = 0.f, s1 = 0.f, q0 = 1.f, q1 = 1.f;
      // local scan of the slice from a zero state; `masked` adds the handling of time steps at or beyond T
      auto slice = [&](auto masked) {
#pragma unroll
        for (int i = 0; i < F_STEPS; ++i) {
          const uint32_t kk = clamp_below_bf16x2(sk[i * (SC_CH / 2)]), uu = clamp_below_bf16x2(su[i * (SC_CH / 2)]);
          float a0, b0, a1, b1;
          gate_act_fwd(bf16_lo(kk), bf16_lo(uu), a0, b0);
          gate_act_fwd(bf16_hi(kk), bf16_hi(uu), a1, b1);
          if (decltype(masked)::value && tbase + i >= p.T) { a0 = 1.f; a1 = 1.f; b0 = 0.f; b1 = 0.f; }
          s0 = fmaf(a0, s0, b0); s1 = fmaf(a1, s1, b1);
          q0 *= a0; q1 *= a1;
          S0[i] = s0; S1[i] = s1; P0[i] = q0; P1[i] = q1;
        }
      };
      if ((ss + 1) * F_TS <= p.T) slice(std::false_type{});
      else slice(std::true_type{});
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane] = make_float2(q0, s0);
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane + 1] = make_float2(q1, s1);
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    if (!all_ok) {
      if (threadIdx.x == 0) atomicExch(p.err, 11);
      break;
    }
    if (threadIdx.x == 0 && ss + SC_STAGES < nss) {
      const int nx = ss + SC_STAGES;
      mbar_expect_tx(&full[stage], F_STAGE_BYTES);
      tma_load_3d(smem + stage * F_STAGE_BYTES, &tmK, &full[stage], c0, nx * F_TS, b);
      tma_load_3d(smem + stage * F_STAGE_BYTES + F_TILE, &tmU, &full[stage], c0, nx * F_TS, b);
    }
    // state entering this warp's slice, and the state leaving the super-step
    float in0 = c_0, in1 = c_1;
#pragma unroll
    for (int w = 0; w < SC_NW; ++w) {
      const float2 x0 = agg[(par * SC_NW + w) * SC_CH + 2 * lane];
      const float2 x1 = agg[(par * SC_NW + w) * SC_CH + 2 * lane + 1];
      c_0 = fmaf(x0.x, c_0, x0.y);
      c_1 = fmaf(x1.x, c_1, x1.y);
      if (w + 1 == warp) { in0 = c_0; in1 = c_1; }
    }
    if constexpr (TMA_OUT) {
      if (tbase < p.T) {                        // uniform across the warp
        if (lane == 0) tma_store_wait_read();   // the store issued a super-step ago has read the tile
        __syncwarp();
#pragma unroll
        for (int i = 0; i < F_STEPS; ++i)
          my_stage[i * (SC_CH / 2)] = pack_bf16(fmaf(P0[i], in0, S0[i]), fmaf(P1[i], in1, S1[i]));
        fence_proxy_async_smem();
        __syncwarp();
        // rows at or beyond T and channels at or beyond C are clipped by the store
        if (lane == 0) tma_store_3d(&tmH, out_stage + warp * F_OUT_WARP, c0, tbase, b);
      }
    } else if (ch < p.C) {
      __nv_bfloat16* hp = p.h + (static_cast<size_t>(b) * p.T + tbase) * p.ldh + ch;
#pragma unroll
      for (int i = 0; i < F_STEPS; ++i) {
        if (tbase + i < p.T) {
          const float v0 = fmaf(P0[i], in0, S0[i]);
          const float v1 = fmaf(P1[i], in1, S1[i]);
          if (ch + 1 < p.C) *reinterpret_cast<uint32_t*>(hp + i * p.ldh) = pack_bf16(v0, v1);
          else hp[i * p.ldh] = __float2bfloat16(v0);
        }
      }
    }
  }
  if (TMA_OUT && lane == 0) tma_store_wait_read();   // before the shared memory is released
  if (warp == 0 && p.h_last) {
    if (ch < p.C) p.h_last[static_cast<size_t>(b) * p.C + ch] = c_0;
    if (ch + 1 < p.C) p.h_last[static_cast<size_t>(b) * p.C + ch + 1] = c_1;
  }
}

struct ScanBwdArgs {
  int B, T, C;
  const float* h0;        // [B, C] or null
  const float* dh_last;   // [B, C] or null: gradient flowing into the final hidden state
  __nv_bfloat16* dk;      // [B, T, ldd]
  __nv_bfloat16* du;      // [B, T, ldd]
  int64_t ldd;
  float* dh0;             // [B, C] or null
  const float* rowscale;  // [B * T] or null: factor applied to row (b, t) of dk and du
  int* err;
};

// Reverse scan.  With a_t = 1 - z_t and G_t = dL/dh_t (direct), define
//   mu_t = a_t * (G_t + mu_{t+1})      (gradient reaching h_{t-1} through step t)
//   lambda_t = G_t + mu_{t+1}          (total gradient of h_t)
//   dk_t = lambda_t * (g(u_t) - h_{t-1}) * z_t * a_t,   du_t = lambda_t * z_t * g'(u_t)
// TMA_OUT as in the forward kernel (tensor maps of dk and du).
template <bool TMA_OUT>
__global__ void __launch_bounds__(SC_THREADS)
scan_bwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmU,
                const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmG,
                const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDU, const ScanBwdArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* out_stage = smem + SC_STAGES * R_STAGE_BYTES;                      // [SC_NW][dk, du][R_STEPS][64] bf16
  uint64_t* full = reinterpret_cast<uint64_t*>(out_stage + SC_NW * R_OUT_WARP);
  float2* agg = reinterpret_cast<float2*>(full + SC_STAGES);   // [2][SC_NW][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, c0 = blockIdx.x * SC_CH;
  const int ch = c0 + 2 * lane;
  const int nss = (p.T + R_TS - 1) / R_TS;

  auto issue = [&](int j, int stage) {
    const int t0 = (nss - 1 - j) * R_TS;
    uint8_t* s = smem + stage * R_STAGE_BYTES;
    mbar_expect_tx(&full[stage], R_STAGE_BYTES);
    tma_load_3d(s, &tmK, &full[stage], c0, t0, b);
    tma_load_3d(s + R_TILE, &tmU, &full[stage], c0, t0, b);
    tma_load_3d(s + 2 * R_TILE, &tmH, &full[stage], c0, t0 - 1, b);   // h_{t-1}; row -1 reads zeros
    tma_load_3d(s + 3 * R_TILE, &tmG, &full[stage], c0, t0, b);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < SC_STAGES; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmU); tma_prefetch_desc(&tmH); tma_prefetch_desc(&tmG);
    if (TMA_OUT) { tma_prefetch_desc(&tmDK); tma_prefetch_desc(&tmDU); }
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int s = 0; s < SC_STAGES && s < nss; ++s) issue(s, s);

  float h00 = 0.f, h01 = 0.f;
  if (p.h0) {
    if (ch < p.C) h00 = p.h0[static_cast<size_t>(b) * p.C + ch];
    if (ch + 1 < p.C) h01 = p.h0[static_cast<size_t>(b) * p.C + ch + 1];
  }
  float m_0 = 0.f, m_1 = 0.f;   // mu carried from later time steps
  if (p.dh_last) {
    if (ch < p.C) m_0 = p.dh_last[static_cast<size_t>(b) * p.C + ch];
    if (ch + 1 < p.C) m_1 = p.dh_last[static_cast<size_t>(b) * p.C + ch + 1];
  }
  uint32_t* my_dk = reinterpret_cast<uint32_t*>(out_stage + warp * R_OUT_WARP) + lane;
  uint32_t* my_du = my_dk + R_OUT_WARP / 8;

  for (int j = 0; j < nss; ++j) {
    const int ss = nss - 1 - j;
    const int stage = j % SC_STAGES;
    const uint32_t phase = (j / SC_STAGES) & 1;
    const int par = j & 1;
    const int tbase = ss * R_TS + warp * R_STEPS;
    const bool inside = ss > 0 && (ss + 1) * R_TS <= p.T;     // no step of this super-step is 0 or >= T
    // row scales of this warp's steps, requested before the wait on the tiles so that their latency is hidden
    float rsc[R_STEPS];
#pragma unroll
    for (int i = 0; i < R_STEPS; ++i)
      rsc[i] = (p.rowscale && (inside || tbase + i < p.T)) ? __ldg(p.rowscale + static_cast<size_t>(b) * p.T + tbase + i) : 1.f;
    bool ok = mbar_wait(&full[stage], phase);

    // per step: lambda_loc = G + mu_loc(next), rn = prod of a over later steps of the slice, c1, c2
    float L0[R_STEPS], L1[R_STEPS], Q0[R_STEPS], Q1[R_STEPS], C10[R_STEPS], C11[R_STEPS], C20[R_STEPS], C21[R_STEPS];
    {
      const uint32_t* sk = reinterpret_cast<const uint32_t*>(smem + stage * R_STAGE_BYTES) + (warp * R_STEPS) * (SC_CH / 2) + lane;
      const uint32_t* su = sk + R_TILE / 4;
      const uint32_t* sh = sk + 2 * (R_TILE / 4);
      const uint32_t* sg = sk + 3 * (R_TILE / 4);
      float mu0 = 0.f, mu1 = 0.f, r0 = 1.f, r1 = 1.f;
      auto slice = [&](auto masked) {
        constexpr bool MASKED = decltype(masked)::value;
#pragma unroll
        for (int i = R_STEPS - 1; i >= 0; --i) {
          const uint32_t kk = clamp_below_bf16x2(sk[i * (SC_CH / 2)]), uu = clamp_below_bf16x2(su[i * (SC_CH / 2)]);
          const uint32_t hh = sh[i * (SC_CH / 2)], gg = sg[i * (SC_CH / 2)];
          float a0, z0, g0, d0, a1, z1, g1, d1;
          gate_act(bf16_lo(kk), bf16_lo(uu), a0, z0, g0, d0);
          gate_act(bf16_hi(kk), bf16_hi(uu), a1, z1, g1, d1);
          float hp0 = bf16_lo(hh), hp1 = bf16_hi(hh);
          float G0 = bf16_lo(gg), G1 = bf16_hi(gg);
          const int t = tbase + i;
          if (MASKED && t == 0) { hp0 = h00; hp1 = h01; }
          float c10 = (g0 - hp0) * z0 * a0, c11 = (g1 - hp1) * z1 * a1;
          float c20 = z0 * d0, c21 = z1 * d1;
          if (MASKED && t >= p.T) { a0 = 1.f; a1 = 1.f; G0 = 0.f; G1 = 0.f; c10 = c11 = c20 = c21 = 0.f; }
          L0[i] = G0 + mu0; L1[i] = G1 + mu1;
          Q0[i] = r0; Q1[i] = r1;
          C10[i] = c10; C11[i] = c11; C20[i] = c20; C21[i] = c21;
          mu0 = a0 * L0[i]; mu1 = a1 * L1[i];
          r0 *= a0; r1 *= a1;
        }
      };
      if (inside) slice(std::false_type{});
      else slice(std::true_type{});
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane] = make_float2(r0, mu0);
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane + 1] = make_float2(r1, mu1);
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    if (!all_ok) {
      if (threadIdx.x == 0) atomicExch(p.err, 12);
      break;
    }
    if (threadIdx.x == 0 && j + SC_STAGES < nss) issue(j + SC_STAGES, stage);

    float in0 = m_0, in1 = m_1;
#pragma unroll
    for (int w = SC_NW - 1; w >= 0; --w) {
      if (w == warp) { in0 = m_0; in1 = m_1; }
      const float2 x0 = agg[(par * SC_NW + w) * SC_CH + 2 * lane];
      const float2 x1 = agg[(par * SC_NW + w) * SC_CH + 2 * lane + 1];
      m_0 = fmaf(x0.x, m_0, x0.y);
      m_1 = fmaf(x1.x, m_1, x1.y);
    }
    if constexpr (TMA_OUT) {
      if (tbase < p.T) {                        // uniform across the warp
        if (lane == 0) tma_store_wait_read();   // the stores issued a super-step ago have read the tiles
        __syncwarp();
#pragma unroll
        for (int i = 0; i < R_STEPS; ++i) {
          const float l0 = fmaf(Q0[i], in0, L0[i]) * rsc[i];
          const float l1 = fmaf(Q1[i], in1, L1[i]) * rsc[i];
          my_dk[i * (SC_CH / 2)] = pack_bf16(l0 * C10[i], l1 * C11[i]);
          my_du[i * (SC_CH / 2)] = pack_bf16(l0 * C20[i], l1 * C21[i]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {                        // rows at or beyond T and channels at or beyond C are clipped
          tma_store_3d(&tmDK, out_stage + warp * R_OUT_WARP, c0, tbase, b);
          tma_store_3d(&tmDU, out_stage + warp * R_OUT_WARP + R_OUT_WARP / 2, c0, tbase, b);
        }
      }
    } else if (ch < p.C) {
      const size_t row0 = (static_cast<size_t>(b) * p.T + tbase) * p.ldd + ch;
#pragma unroll
      for (int i = 0; i < R_STEPS; ++i) {
        if (tbase + i < p.T) {
          const float l0 = fmaf(Q0[i], in0, L0[i]) * rsc[i];
          const float l1 = fmaf(Q1[i], in1, L1[i]) * rsc[i];
          const size_t o = row0 + static_cast<size_t>(i) * p.ldd;
          if (ch + 1 < p.C) {
            *reinterpret_cast<uint32_t*>(p.dk + o) = pack_bf16(l0 * C10[i], l1 * C11[i]);
            *reinterpret_cast<uint32_t*>(p.du + o) = pack_bf16(l0 * C20[i], l1 * C21[i]);
          } else {
            p.dk[o] = __float2bfloat16(l0 * C10[i]);
            p.du[o] = __float2bfloat16(l0 * C20[i]);
          }
        }
      }
    }
  }
  if (TMA_OUT && lane == 0) tma_store_wait_read();   // before the shared memory is released
  if (warp == 0 && p.dh0) {
    if (ch < p.C) p.dh0[static_cast<size_t>(b) * p.C + ch] = m_0;
    if (ch + 1 < p.C) p.dh0[static_cast<size_t>(b) * p.C + ch + 1] = m_1;
  }
}

constexpr int F_SMEM = SC_STAGES * F_STAGE_BYTES + SC_NW * F_OUT_WARP + 128 + SC_STAGES * 8 + 2 * SC_NW * SC_CH * 8;
constexpr int R_SMEM = SC_STAGES * R_STAGE_BYTES + SC_NW * R_OUT_WARP + 128 + SC_STAGES * 8 + 2 * SC_NW * SC_CH * 8;
// All (C / 64) x B CTAs of the 1B and 3B shapes are meant to be resident at once: three per SM.
static_assert(3 * (F_SMEM + 1024) <= 233472 && 3 * (R_SMEM + 1024) <= 233472, "three scan CTAs per SM must fit");

template <typename Kern>
static int allow_smem(Kern kern, int bytes, bool& done) {
  if (done) return 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -4;
  done = true;
  return 0;
}

}  // namespace grb

using namespace grb;

extern "C" int grb_scan_fwd(const void* k, const void* u, int64_t ldku, const float* h0, void* h, int64_t ldh,
                            float* h_last, int B, int T, int C, int* err, void* stream) {
  if (B <= 0 || T <= 0 || C <= 0) return 0;
  if (C % 2) return -20;
  CUtensorMap tmK, tmU, tmH;
  int rc = make_tmap_btc_bf16(&tmK, k, C, T, B, ldku, SC_CH, F_TS);
  if (rc) return rc;
  rc = make_tmap_btc_bf16(&tmU, u, C, T, B, ldku, SC_CH, F_TS);
  if (rc) return rc;
  // the output leaves through bulk tensor stores when its layout allows a tensor map (16-byte aligned base and rows)
  const bool tma_out = make_tmap_btc_bf16(&tmH, h, C, T, B, ldh, SC_CH, F_STEPS) == 0;
  if (!tma_out) tmH = tmK;
  static bool attr[2] = {false, false};
  rc = tma_out ? allow_smem(scan_fwd_kernel<true>, F_SMEM, attr[1]) : allow_smem(scan_fwd_kernel<false>, F_SMEM, attr[0]);
  if (rc) return rc;
  ScanFwdArgs a{B, T, C, h0, reinterpret_cast<__nv_bfloat16*>(h), ldh, h_last, err};
  dim3 grid((C + SC_CH - 1) / SC_CH, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tma_out) scan_fwd_kernel<true><<<grid, SC_THREADS, F_SMEM, st>>>(tmK, tmU, tmH, a);
  else scan_fwd_kernel<false><<<grid, SC_THREADS, F_SMEM, st>>>(tmK, tmU, tmH, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_scan_bwd(const void* k, const void* u, int64_t ldku, const void* h, int64_t ldh, const void* g,
                            int64_t ldg, const float* h0, const float* dh_last, void* dk, void* du, int64_t ldd,
                            float* dh0, const float* rowscale, int B, int T, int C, int* err, void* stream) {
  if (B <= 0 || T <= 0 || C <= 0) return 0;
  if (C % 2) return -20;
  CUtensorMap tmK, tmU, tmH, tmG, tmDK, tmDU;
  int rc = make_tmap_btc_bf16(&tmK, k, C, T, B, ldku, SC_CH, R_TS);
  if (rc) return rc;
  rc = make_tmap_btc_bf16(&tmU, u, C, T, B, ldku, SC_CH, R_TS);
  if (rc) return rc;
  rc = make_tmap_btc_bf16(&tmH, h, C, T, B, ldh, SC_CH, R_TS);
  if (rc) return rc;
  rc = make_tmap_btc_bf16(&tmG, g, C, T, B, ldg, SC_CH, R_TS);
  if (rc) return rc;
  const bool tma_out = make_tmap_btc_bf16(&tmDK, dk, C, T, B, ldd, SC_CH, R_STEPS) == 0 &&
                       make_tmap_btc_bf16(&tmDU, du, C, T, B, ldd, SC_CH, R_STEPS) == 0;
  if (!tma_out) tmDK = tmDU = tmK;
  static bool attr[2] = {false, false};
  rc = tma_out ? allow_smem(scan_bwd_kernel<true>, R_SMEM, attr[1]) : allow_smem(scan_bwd_kernel<false>, R_SMEM, attr[0]);
  if (rc) return rc;
  ScanBwdArgs a{B, T, C, h0, dh_last, reinterpret_cast<__nv_bfloat16*>(dk), reinterpret_cast<__nv_bfloat16*>(du), ldd, dh0, rowscale, err};
  dim3 grid((C + SC_CH - 1) / SC_CH, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tma_out) scan_bwd_kernel<true><<<grid, SC_THREADS, R_SMEM, st>>>(tmK, tmU, tmH, tmG, tmDK, tmDU, a);
  else scan_bwd_kernel<false><<<grid, SC_THREADS, R_SMEM, st>>>(tmK, tmU, tmH, tmG, tmDK, tmDU, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
