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
// arrive through a 3-stage TMA ring.  Inside a super-step the four warps each
// take a slice of consecutive time steps, scan it locally from a zero state
// (keeping per-step (prefix-product, local value) pairs in registers), exchange
// slice aggregates through shared memory, and finish with one FMA per element.
// Results go to a per-warp staging tile and leave with one bulk tensor store
// per slice (which also clips the ragged ends of T and C); super-steps that lie
// wholly inside T run a variant of the slice loop without any bounds handling.
// A thread owns two adjacent channels and does their fp32 arithmetic with
// packed instructions (ptx.cuh: ffma2 / fmul2 / fadd2).
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

// Forward, both channels of a word at once; k and u already clamped.  Returns a = 1 - z and b = z g(u), z = sigmoid(k).
// Two exponentials and one reciprocal per channel serve both sigmoids.
// u + 0.5 lies above sigmoid(u) exactly where u >= 0 (the sigmoid is concave there and its slope at 0 is 1/4; for
// u < 0 it is convex and stays above its tangent 0.5 + u/4 > 0.5 + u), so g = max of the two; and z sigmoid(u) is
// the shared reciprocal r = 1 / ((1 + e^-k)(1 + e^-u)) itself, so b = max(z (u + 0.5), r).
__device__ __forceinline__ void gate_act_fwd2(uint32_t kk, uint32_t uu, float2& a, float2& b) {
  const float2 c = splat2(-1.4426950408889634f);
  const float2 kf = make_float2(bf16_lo(kk), bf16_hi(kk)), uf = make_float2(bf16_lo(uu), bf16_hi(uu));
  const float2 ka = fmul2(kf, c), ua = fmul2(uf, c);
  const float2 ea = make_float2(ex2f(ka.x), ex2f(ka.y));   // e^{-k}
  const float2 eb = make_float2(ex2f(ua.x), ex2f(ua.y));   // e^{-u}
  const float2 p = fadd2(eb, splat2(1.f));                  // 1 + e^{-u}
  const float2 d = ffma2(ea, p, p);                         // (1 + e^{-k})(1 + e^{-u})
  const float2 r = make_float2(rcpf(d.x), rcpf(d.y));
  const float2 z = fmul2(r, p);
  a = fmul2(ea, z);
  const float2 t = fmul2(z, fadd2(uf, splat2(0.5f)));
  b = make_float2(fmaxf(t.x, r.x), fmaxf(t.y, r.y));
}

// Backward, both channels of a word at once: a = 1 - z, z, g(u) and g'(u).
__device__ __forceinline__ void gate_act_bwd2(uint32_t kk, uint32_t uu, float2& a, float2& z, float2& g, float2& gp) {
  const float2 c = splat2(-1.4426950408889634f);
  const float2 kf = make_float2(bf16_lo(kk), bf16_hi(kk)), uf = make_float2(bf16_lo(uu), bf16_hi(uu));
  const float2 ka = fmul2(kf, c), ua = fmul2(uf, c);
  const float2 ea = make_float2(ex2f(ka.x), ex2f(ka.y));
  const float2 eb = make_float2(ex2f(ua.x), ex2f(ua.y));
  const float2 p = fadd2(eb, splat2(1.f)), q = fadd2(ea, splat2(1.f));
  const float2 d = fmul2(p, q);
  const float2 r = make_float2(rcpf(d.x), rcpf(d.y));
  z = fmul2(r, p);
  const float2 s = fmul2(r, q);                            // sigmoid(u)
  a = fmul2(ea, z);
  const float2 lin = fadd2(uf, splat2(0.5f));
  const float2 ds = fmul2(fmul2(s, eb), s);                // sigmoid'(u)
  const bool p0 = uf.x >= 0.f, p1 = uf.y >= 0.f;
  g = make_float2(p0 ? lin.x : s.x, p1 ? lin.y : s.y);
  gp = make_float2(p0 ? 1.f : ds.x, p1 ? 1.f : ds.y);
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

    float2 S[F_STEPS], P[F_STEPS];
    const int tbase = ss * F_TS + warp * F_STEPS;
    {
      const uint32_t* sk = reinterpret_cast<const uint32_t*>(smem + stage * F_STAGE_BYTES) + (warp * F_STEPS) * (SC_CH / 2) + lane;
      const uint32_t* su = sk + F_TILE / 4;
      float2 sc = splat2(0.f), q = splat2(1.f);
      // local scan of the slice from a zero state; `masked` adds the handling of time steps at or beyond T
      auto slice = [&](auto masked) {
#pragma unroll
        for (int i = 0; i < F_STEPS; ++i) {
          const uint32_t kk = clamp_below_bf16x2(sk[i * (SC_CH / 2)]), uu = clamp_below_bf16x2(su[i * (SC_CH / 2)]);
          float2 a, bb;
          gate_act_fwd2(kk, uu, a, bb);
          if (decltype(masked)::value && tbase + i >= p.T) { a = splat2(1.f); bb = splat2(0.f); }
          sc = ffma2(a, sc, bb);
          q = fmul2(q, a);
          S[i] = sc; P[i] = q;
        }
      };
      if ((ss + 1) * F_TS <= p.T) slice(std::false_type{});
      else slice(std::true_type{});
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane] = make_float2(q.x, sc.x);
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane + 1] = make_float2(q.y, sc.y);
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
        {
          const float2 v = ffma2(P[i], make_float2(in0, in1), S[i]);
          my_stage[i * (SC_CH / 2)] = pack_bf16(v.x, v.y);
        }
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
          const float v0 = fmaf(P[i].x, in0, S[i].x);
          const float v1 = fmaf(P[i].y, in1, S[i].y);
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
    float2 L[R_STEPS], Q[R_STEPS], C1[R_STEPS], C2[R_STEPS];
    {
      const uint32_t* sk = reinterpret_cast<const uint32_t*>(smem + stage * R_STAGE_BYTES) + (warp * R_STEPS) * (SC_CH / 2) + lane;
      const uint32_t* su = sk + R_TILE / 4;
      const uint32_t* sh = sk + 2 * (R_TILE / 4);
      const uint32_t* sg = sk + 3 * (R_TILE / 4);
      float2 mu = splat2(0.f), rr = splat2(1.f);
      auto slice = [&](auto masked) {
        constexpr bool MASKED = decltype(masked)::value;
#pragma unroll
        for (int i = R_STEPS - 1; i >= 0; --i) {
          const uint32_t kk = clamp_below_bf16x2(sk[i * (SC_CH / 2)]), uu = clamp_below_bf16x2(su[i * (SC_CH / 2)]);
          const uint32_t hh = sh[i * (SC_CH / 2)], gg = sg[i * (SC_CH / 2)];
          float2 a, z, g, d;
          gate_act_bwd2(kk, uu, a, z, g, d);
          float2 hp = make_float2(bf16_lo(hh), bf16_hi(hh));
          float2 G = make_float2(bf16_lo(gg), bf16_hi(gg));
          const int t = tbase + i;
          if (MASKED && t == 0) hp = make_float2(h00, h01);
          float2 c1 = fmul2(ffma2(hp, splat2(-1.f), g), fmul2(z, a));
          float2 c2 = fmul2(z, d);
          if (MASKED && t >= p.T) { a = splat2(1.f); G = splat2(0.f); c1 = splat2(0.f); c2 = splat2(0.f); }
          L[i] = fadd2(G, mu);
          Q[i] = rr;
          C1[i] = c1; C2[i] = c2;
          mu = fmul2(a, L[i]);
          rr = fmul2(rr, a);
        }
      };
      if (inside) slice(std::false_type{});
      else slice(std::true_type{});
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane] = make_float2(rr.x, mu.x);
      agg[(par * SC_NW + warp) * SC_CH + 2 * lane + 1] = make_float2(rr.y, mu.y);
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
          const float2 l = fmul2(ffma2(Q[i], make_float2(in0, in1), L[i]), splat2(rsc[i]));
          const float2 vk = fmul2(l, C1[i]), vu = fmul2(l, C2[i]);
          my_dk[i * (SC_CH / 2)] = pack_bf16(vk.x, vk.y);
          my_du[i * (SC_CH / 2)] = pack_bf16(vu.x, vu.y);
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
          const float l0 = fmaf(Q[i].x, in0, L[i].x) * rsc[i];
          const float l1 = fmaf(Q[i].y, in1, L[i].y) * rsc[i];
          const size_t o = row0 + static_cast<size_t>(i) * p.ldd;
          if (ch + 1 < p.C) {
            *reinterpret_cast<uint32_t*>(p.dk + o) = pack_bf16(l0 * C1[i].x, l1 * C1[i].y);
            *reinterpret_cast<uint32_t*>(p.du + o) = pack_bf16(l0 * C2[i].x, l1 * C2[i].y);
          } else {
            p.dk[o] = __float2bfloat16(l0 * C1[i].x);
            p.du[o] = __float2bfloat16(l0 * C2[i].x);
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
