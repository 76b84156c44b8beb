// Decode-step matrix-vector products on the tcgen05 tensor cores.
//
// For up to 16 sequences a decode step reads every weight once, so the kernel is a weight-streaming pipeline and
// the arithmetic is a by-product:  acc[128 weight rows, 16 sequences] += W_tile[128, 64] * in[16, 64]^T per k-block,
// with W_tile brought in by TMA (128-byte swizzle, a ring of stages), `in` staged ONCE per CTA in shared memory in
// the same canonical layout, and the accumulator in tensor memory.  A CTA owns one 128-row tile of W and one slice
// of K (split-K fills the SMs for the narrow matrices); partial results are added to the output with fp32 atomics,
// so every output is either the residual stream itself (x += W in) or a pre-activation buffer that a later kernel
// of the chain zeroes again.  What would be the epilogue non-linearity of one product is therefore the input
// transform of the next:
//     gate  : in = RMSNorm(x) * w          ku    += Wg in      (1/rms, a scalar per sequence, scales the accumulator)
//     out   : in = lerp(h, g(ku_c), sigmoid(ku_g)) (also stored, in a second buffer, as the new state)   x += Wo in
//     ff1   : in = RMSNorm(x) * w          a_pre += W1 in
//     ff2   : in = gelu(a_pre + b1)        x     += W2 in + b2
//     head  : in = RMSNorm(x) * w          logits += Wl in
// The recurrence is the reference's single-step branch (mingru/minGRU.py:47-52); the reference itself runs these
// as nn.Linear calls and ATen element-wise kernels.
//
// Launch order inside a CTA: barriers + tensor-memory allocation, then the first ring of weight loads (weights do
// not depend on the previous kernel), then griddepcontrol.wait (a no-op unless launched with programmatic stream
// serialisation), then the input transform, then MMAs as stages land, then the atomic epilogue.
#include "decode.h"
#include "ptx.cuh"
#include "tmap.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace grb {
namespace dtc {

constexpr int BM = 128;                 // weight rows per CTA
constexpr int BN = 16;                  // sequences (MMA N); rows >= B of the staged input are zero
constexpr int BK = 64;                  // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int A_STAGE_BYTES = BM * BK * 2;      // 16 KB
constexpr int B_KB_BYTES = BN * BK * 2;         // 2 KB of staged input per k-block
constexpr int MAX_STAGES = 8;
constexpr int MAX_KB_PER_CTA = 16;              // bounds the staged input (32 KB)
constexpr int XF_WARPS = 8;                     // input-transform warps; the first four also run the epilogue
constexpr int XF_THREADS = 32 * XF_WARPS;
constexpr int NUM_THREADS = 64 + XF_THREADS;    // warp 0: TMA, warp 1: MMA, warps 2..: input transform (+ epilogue)
constexpr int TMEM_COLS = 32;

enum { IN_NORM = 0, IN_GATE = 1, IN_GELU = 2 };

struct Args {
  const float* src;        // IN_NORM: x [B, K];  IN_GATE: ku [B, 2K] (candidate | gate);  IN_GELU: a_pre [B, K]
  const float* vec;        // IN_NORM: norm weight [K];  IN_GELU: bias b1 [K];  IN_GATE: unused
  const float* state;      // IN_GATE: hidden state h_{t-1} [B, K]
  float* state_out;        // IN_GATE: h_t [B, K]; a different buffer, since other CTAs still read h_{t-1}
  float* out;              // [B, N] accumulated with atomics
  const float* out_bias;   // [N] added once (by the first k-slice), or null
  float* zero_buf;         // buffer that is dead by now and must be zero for a later kernel, or null
  int zero_n;
  float* copy_dst;         // housekeeping copy (the previous kernel's h_t into the state), or null
  const float* copy_src;
  int copy_n;
  int B, N, K;
  int kb_per, stages;
  float eps;
  int* err;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float gate_g(float u) { return u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u)); }
__device__ __forceinline__ float sigmoid_f(float k) { return 1.f / (1.f + expf(-k)); }
__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }

// Timing experiment (-DGRB_DEC_TRACE): the first CTA stamps %globaltimer at the phases of each role into `zero_buf`'s
// place (the host passes a scratch tensor there and no housekeeping).  Not compiled into the library.
#ifdef GRB_DEC_TRACE
#define DTC_STAMP(slot)                                                                       \
  do {                                                                                        \
    if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0) {                                    \
      unsigned long long t_;                                                                  \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
      reinterpret_cast<unsigned long long*>(a.copy_dst)[slot] = t_;                           \
    }                                                                                         \
  } while (0)
#else
#define DTC_STAMP(slot) do {} while (0)
#endif

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS) decode_tc_kernel(const __grid_constant__ CUtensorMap tmW, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int S = a.stages;
  uint8_t* sA = smem;                                         // S stages of W
  uint8_t* sB = smem + static_cast<size_t>(S) * A_STAGE_BYTES;  // kb_per k-blocks of staged input
  __shared__ uint64_t full[MAX_STAGES], empty[MAX_STAGES], bready, tdone;
  __shared__ uint32_t tmem_slot;
  __shared__ float red[BN][XF_WARPS];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y;
  if (warp == 0) DTC_STAMP(0);
  const int nkb_total = (a.K + BK - 1) / BK;
  const int kb0 = split * a.kb_per, kb1 = min(nkb_total, kb0 + a.kb_per);
  const int nkb = kb1 - kb0;                                  // >= 1 by construction of the grid

  if (threadIdx.x == 0) {
    for (int i = 0; i < MAX_STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(&bready, XF_THREADS);
    mbar_init(&tdone, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0) DTC_STAMP(1);

  bool ok = true;
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const int first = min(S, nkb);
    if (lane == 0)
      for (int i = 0; i < first; ++i) {                       // before the previous kernel has finished
        mbar_expect_tx(&full[i], A_STAGE_BYTES);
        tma_load_2d(sA + static_cast<size_t>(i) * A_STAGE_BYTES, &tmW, &full[i], (kb0 + i) * BK, tile * BM);
      }
    if (lane == 0)
      for (int i = first; i < nkb; ++i)                       // the rest of the slice: at least into L2 meanwhile
        asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(&tmW)),
                     "r"((kb0 + i) * BK), "r"(tile * BM)
                     : "memory");
    DTC_STAMP(2);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    DTC_STAMP(3);
    int issued = first;
    for (int i = first; i < nkb && ok; ++i) {
      const int st = i % S;
      if (!__all_sync(0xffffffffu, mbar_wait(&empty[st], ((i / S) - 1) & 1))) { ok = false; break; }
      if (lane == 0) {
        mbar_expect_tx(&full[st], A_STAGE_BYTES);
        tma_load_2d(sA + static_cast<size_t>(st) * A_STAGE_BYTES, &tmW, &full[st], (kb0 + i) * BK, tile * BM);
      }
      issued = i + 1;
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(a.err, 8);
    // nothing may still be landing in this CTA's shared memory when it exits: the consumer's last commit (tdone)
    // follows every load it used; loads it never reached (only after a failure) get one bounded wait each
    const bool finished = __all_sync(0xffffffffu, mbar_wait(&tdone, 0));
    if (!finished || *reinterpret_cast<volatile int*>(a.err) != 0)
      for (int i = max(0, issued - S); i < issued; ++i) mbar_wait(&full[i % S], (i / S) & 1);
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, 0);
    if (!__all_sync(0xffffffffu, mbar_wait(&bready, 0))) ok = false;
    tc_fence_after();
    DTC_STAMP(4);
    for (int i = 0; i < nkb && ok; ++i) {
      const int st = i % S;
      if (!__all_sync(0xffffffffu, mbar_wait(&full[st], (i / S) & 1))) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t sa = smem_u32(sA + static_cast<size_t>(st) * A_STAGE_BYTES);
        const uint32_t sb = smem_u32(sB + static_cast<size_t>(i) * B_KB_BYTES);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(tmem_base, umma_smem_desc(sa + k * 32, 16, 1024), umma_smem_desc(sb + k * 32, 16, 1024), idesc,
                    (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[st]);
        if (i == nkb - 1) umma_commit(&tdone);
      }
      __syncwarp();
      if (i == 0) DTC_STAMP(5);
    }
    DTC_STAMP(6);
    if (!ok) {
      if (lane == 0) {
        atomicExch(a.err, 9);
        mbar_arrive(&tdone);          // release the waiters; the epilogue checks the status word and skips its adds
      }
    }
  } else {
    // ------------------------------------------- input transform (all XF warps), then epilogue (first four)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = threadIdx.x - 64;                           // 0..XF_THREADS-1
    const int K = a.K;
    // a buffer the chain needs zeroed later
    if (a.zero_buf) {
      const int ncta = gridDim.x * gridDim.y, cta = blockIdx.y * gridDim.x + blockIdx.x;
      for (int i = cta * XF_THREADS + t; i < a.zero_n; i += ncta * XF_THREADS) a.zero_buf[i] = 0.f;
    }
#ifndef GRB_DEC_TRACE
    if (a.copy_dst) {
      const int ncta = gridDim.x * gridDim.y, cta = blockIdx.y * gridDim.x + blockIdx.x;
      for (int i = cta * XF_THREADS + t; i < a.copy_n; i += ncta * XF_THREADS) a.copy_dst[i] = a.copy_src[i];
    }
#endif
    // work items = (sequence row b, 16-byte chunk c of the CTA's k-slice), spread over the transform threads with the chunk
    // as the fast index (adjacent threads read adjacent addresses); rows b >= B are zero fill
    const int nchunks = nkb * 8;                              // <= 128
    for (int item = t; item < nchunks * BN; item += XF_THREADS) {
      const int b = item / nchunks, c = item - b * nchunks;
      const int kbl = c >> 3, j = c & 7;                      // k-block within the slice, chunk within its 128-byte row
      const int k = (kb0 + kbl) * BK + j * 8;
      uint4 pk = make_uint4(0u, 0u, 0u, 0u);
      if (b < a.B && k < K) {                                 // K % 8 == 0: a chunk is inside or outside as a whole
        float v[8];
        if constexpr (MODE == IN_GATE) {
          const float* kc = a.src + static_cast<size_t>(b) * 2 * K + k;
          const float* hp = a.state + static_cast<size_t>(b) * K + k;
          const float4 c0 = *reinterpret_cast<const float4*>(kc), c1 = *reinterpret_cast<const float4*>(kc + 4);
          const float4 g0 = *reinterpret_cast<const float4*>(kc + K), g1 = *reinterpret_cast<const float4*>(kc + K + 4);
          const float4 h0 = *reinterpret_cast<const float4*>(hp), h1 = *reinterpret_cast<const float4*>(hp + 4);
          const float cu[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float gk[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
          const float hh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = fmaf(sigmoid_f(gk[e]), gate_g(cu[e]) - hh[e], hh[e]);
          if (tile == 0) {                                    // exactly one CTA per k-slice stores the new state
            float* ho = a.state_out + static_cast<size_t>(b) * K + k;
            *reinterpret_cast<float4*>(ho) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(ho + 4) = make_float4(v[4], v[5], v[6], v[7]);
          }
        } else {
          const float* sp = a.src + static_cast<size_t>(b) * K + k;
          const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
          float4 v0 = make_float4(1.f, 1.f, 1.f, 1.f), v1 = v0;
          if (MODE == IN_GELU) v0 = v1 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (a.vec) {
            v0 = *reinterpret_cast<const float4*>(a.vec + k);
            v1 = *reinterpret_cast<const float4*>(a.vec + k + 4);
          }
          const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = MODE == IN_NORM ? sv[e] * vv[e] : gelu_erf(sv[e] + vv[e]);
        }
        pk = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
      }
      // canonical K-major 128-byte-swizzle layout: 8-row groups of 1 KB, row r at r*128, chunk j at (j ^ r)*16
      *reinterpret_cast<uint4*>(sB + static_cast<size_t>(kbl) * B_KB_BYTES + (b >> 3) * 1024 + (b & 7) * 128 +
                                ((j ^ (b & 7)) << 4)) = pk;
    }
    fence_proxy_async_smem();                                 // generic-proxy writes -> visible to the tensor core
    mbar_arrive(&bready);
    if (warp == 2) DTC_STAMP(7);

    // RMSNorm's 1/rms is one scalar per sequence: it multiplies the finished accumulator, so the sum of squares
    // over the whole of K is computed here, while the weights stream, instead of before the staging
    float rstd[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) rstd[b] = 1.f;
    if constexpr (MODE == IN_NORM) {
      for (int b = 0; b < a.B; ++b) {
        float s = 0.f;
        for (int k = t * 4; k < K; k += 4 * XF_THREADS) {
          const float4 v = *reinterpret_cast<const float4*>(a.src + static_cast<size_t>(b) * K + k);
          s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) red[b][warp - 2] = s;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(XF_THREADS) : "memory");
#pragma unroll
      for (int b = 0; b < 8; ++b)
        if (b < a.B) {
          float tot = 0.f;
#pragma unroll
          for (int w = 0; w < XF_WARPS; ++w) tot += red[b][w];
          rstd[b] = rsqrtf(tot / K + a.eps);
        }
    }

    // ---- epilogue (warps 2-5): lane i of quadrant q holds weight row tile*128 + q*32 + i, register b = sequence b
    const int q = warp & 3;
    if (warp < 6 && !__all_sync(0xffffffffu, mbar_wait(&tdone, 0))) { ok = false; if (lane == 0) atomicExch(a.err, 10); }
    tc_fence_after();
    if (warp == 2) DTC_STAMP(8);
    if (warp < 6 && ok && *reinterpret_cast<volatile int*>(a.err) == 0) {
      uint32_t r[16];
      tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16), r);
      tmem_ld_wait();
      const int row = tile * BM + q * 32 + lane;
      if (row < a.N) {
        const float bias = (a.out_bias && split == 0) ? a.out_bias[row] : 0.f;
#pragma unroll
        for (int b = 0; b < 8; ++b)
          if (b < a.B) atomicAdd(a.out + static_cast<size_t>(b) * a.N + row, fmaf(__uint_as_float(r[b]), rstd[b], bias));
      }
    }
  }

  if (warp == 2) DTC_STAMP(9);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (warp == 0) DTC_STAMP(10);
}

template <int MODE>
int launch(const CUtensorMap& tm, const Args& a, dim3 grid, size_t smem, bool pdl, cudaStream_t st) {
  static size_t granted = 0;                                  // one per MODE (this function template)
  if (smem > 40 * 1024 && smem > granted) {
    if (cudaFuncSetAttribute(decode_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return -4;
    granted = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t err = cudaLaunchKernelEx(&cfg, decode_tc_kernel<MODE>, tm, a);
  if (err == cudaSuccess) err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -(1000 + static_cast<int>(err));
}

}  // namespace dtc
}  // namespace grb

extern "C" int grb_decode_tc(int mode, const float* src, const float* vec, const float* state, float* state_out,
                             const void* W, float* out, const float* out_bias, float* zero_buf, int zero_n,
                             float* copy_dst, const float* copy_src, int copy_n, int B, int N, int K, float eps,
                             int num_sms, int overlap, int* err, void* stream) {
  using namespace grb;
  using namespace grb::dtc;
  if (B < 1 || B > 8 || N < 1 || K < 8 || K % 8 || !err || !src || !W || !out) return -40;
  if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(src)) & 15) return -41;
  if (vec && (reinterpret_cast<uintptr_t>(vec) & 15)) return -41;
  if (mode == IN_GATE && (!state || !state_out || state == state_out ||
                          ((reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(state_out)) & 15)))
    return -41;
  const int sms = num_sms > 0 ? num_sms : 148;
  const int tiles = (N + BM - 1) / BM;
  const int nkb = (K + BK - 1) / BK;
  int split = (sms + tiles - 1) / tiles;                      // about one CTA per SM
  if (split > nkb) split = nkb;
  if (split < 1) split = 1;
  int kb_per = (nkb + split - 1) / split;
  if (kb_per > MAX_KB_PER_CTA) kb_per = MAX_KB_PER_CTA;
  split = (nkb + kb_per - 1) / kb_per;
  // ring depth: as deep as leaves room for a second CTA on the SM (the next kernel of the chain, started early)
  const size_t b_bytes = static_cast<size_t>(kb_per) * B_KB_BYTES;
  int stages = kb_per < MAX_STAGES ? kb_per : MAX_STAGES;
  while (stages > 2 && 2 * (static_cast<size_t>(stages) * A_STAGE_BYTES + b_bytes + 1024 + 2048) > 227 * 1024) --stages;
  const size_t smem = static_cast<size_t>(stages) * A_STAGE_BYTES + b_bytes + 1024;
  CUtensorMap tm;
  const int rc = make_tmap_2d_bf16(&tm, W, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), BK, BM,
                                   true);
  if (rc) return rc;
  Args a{src, vec, state, state_out, out, out_bias, zero_buf, zero_n, copy_dst, copy_src, copy_n, B, N, K, kb_per, stages, eps, err};
  dim3 grid(tiles, split);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (mode) {
    case IN_NORM: return launch<IN_NORM>(tm, a, grid, smem, overlap != 0, st);
    case IN_GATE: return launch<IN_GATE>(tm, a, grid, smem, overlap != 0, st);
    case IN_GELU: return launch<IN_GELU>(tm, a, grid, smem, overlap != 0, st);
  }
  return -43;
}
