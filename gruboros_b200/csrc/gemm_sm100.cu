// bf16 GEMM for sm_100a built directly on tcgen05.mma / TMEM / TMA.
//
//   D[M,N] = A[M,K] * B[N,K]^T  (fp32 accumulate in tensor memory)
//
// One persistent CTA per SM walks a static tile schedule.  Six warps:
//   warp 0      TMA producer   (cp.async.bulk.tensor, 128B swizzle, 3-stage ring)
//   warp 1      MMA issuer     (tcgen05.mma 128x256x16, accumulators in TMEM)
//   warps 2..9  epilogue       (tcgen05.ld -> fused math -> global; two warps per TMEM lane
//                               quadrant, each owning 128 of the 256 accumulator columns)
// Two 256-column accumulators are allocated so that the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Either operand may be "K-major" (reduction dim contiguous in global memory)
// or "MN-major" (the M/N dim contiguous), so that the forward GEMM, dgrad and
// wgrad of a Linear all read the tensors where they already live:
//   forward  y  = x  W^T : A = x  [M,K]  K-major, B = W [N,K] K-major
//   dgrad    dx = dy W   : A = dy [M,N]  K-major, B = W [N,K] MN-major
//   wgrad    dW = dy^T x : A = dy [M,N] MN-major, B = x [M,K] MN-major
// Ragged edges rely on TMA zero-fill for loads and predicates for stores.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference
// (mingru/minGRU.py:45,71; mingru/minLM.py:17-23,75) and their autograd.
#include "ptx.cuh"
#include "gemm_sm100.h"
#include "tmap.h"
#include "gemm_epilogue.cuh"
#include <cstdio>

namespace grb {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;     // one 64(MN) x 64(red) MN-major box: 8 KB
constexpr int NUM_EPI_WARPS = 8;              // two warps per TMEM lane quadrant, each takes half the columns
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + NUM_EPI_WARPS * EPI_STAGE_BYTES;

struct GemmShape {
  int M, N, K;
  int splitk;       // >1 only with the accumulate epilogue
  int* err;         // device error word (0 = ok)
};

// ---------------------------------------------------------------- kernel
template <int MAJ_A, int MAJ_B, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmShape s,
            const EpiArgs e) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + STAGES;          // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;      // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  float* epi_stage = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);   // per-warp transposition tiles

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int ntm = (s.M + BM - 1) / BM;
  const int ntn = (s.N + BN - 1) / BN;
  const int nkb_total = (s.K + BK - 1) / BK;
  const int splitk = s.splitk > 0 ? s.splitk : 1;
  const int kb_per = (nkb_total + splitk - 1) / splitk;
  const int ntiles = ntm * ntn * splitk;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 32 * NUM_EPI_WARPS); }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (split, m, n): groups of GM m-tiles share their n sweep for L2 reuse
  constexpr int GM = 16;
  auto tile_coords = [&](int t, int& sp, int& tm, int& tn) {
    sp = t / (ntm * ntn);
    const int r = t - sp * (ntm * ntn);
    const int per_group = GM * ntn;
    const int g = r / per_group;
    const int first_m = g * GM;
    const int gsz = min(GM, ntm - first_m);
    const int in = r - g * per_group;
    tm = first_m + in % gsz;
    tn = in / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    int stage = 0; uint32_t phase = 0; bool ok = true;
    for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
      int sp, tm, tn; tile_coords(t, sp, tm, tn);
      const int kb0 = sp * kb_per, kb1 = min(nkb_total, kb0 + kb_per);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) { ok = false; break; }
        if (lane == 0) {
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          if constexpr (MAJ_A == MAJOR_K) {
            tma_load_2d(sa, &tmA, &full[stage], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * CHUNK_BYTES, &tmA, &full[stage], tm * BM + 64 * j, kb * BK);
          }
          if constexpr (MAJ_B == MAJOR_K) {
            tma_load_2d(sb, &tmB, &full[stage], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * CHUNK_BYTES, &tmB, &full[stage], tn * BN + 64 * j, kb * BK);
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && lane == 0) atomicExch(s.err, 1);
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, MAJ_A == MAJOR_MN, MAJ_B == MAJOR_MN);
    int stage = 0; uint32_t phase = 0; bool ok = true;
    int acc = 0; uint32_t accphase = 0;
    for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
      int sp, tm, tn; tile_coords(t, sp, tm, tn);
      const int kb0 = sp * kb_per, kb1 = min(nkb_total, kb0 + kb_per);
      if (!mbar_wait(&tempty[acc], accphase ^ 1)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[stage], phase)) { ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad, bd;
            if constexpr (MAJ_A == MAJOR_K) ad = umma_smem_desc(sa + k * UMMA_K * 2, 16, 1024);
            else ad = umma_smem_desc(sa + k * UMMA_K * 128, CHUNK_BYTES, 1024);
            if constexpr (MAJ_B == MAJOR_K) bd = umma_smem_desc(sb + k * UMMA_K * 2, 16, 1024);
            else bd = umma_smem_desc(sb + k * UMMA_K * 128, CHUNK_BYTES, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);               // frees the smem stage when the MMAs retire
          if (kb == kb1 - 1) umma_commit(&tfull[acc]);  // accumulator complete
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (kb1 <= kb0 && lane == 0) umma_commit(&tfull[acc]);  // empty split: nothing issued
      __syncwarp();
      acc ^= 1; if (acc == 0) accphase ^= 1;
    }
    if (!ok && lane == 0) atomicExch(s.err, 2);
  } else {
    // ---------------------------------------------------------- epilogue
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;       // which 128 accumulator columns this warp handles
    // the cross-entropy epilogue needs whole rows in one thread: the first four warps take all 256 columns
    const int c_begin = (EPI == EPI_CE) ? 0 : half * (BN / 2);
    const int c_end = (EPI == EPI_CE) ? (half == 0 ? BN : 0) : (half + 1) * (BN / 2);
    int acc = 0; uint32_t accphase = 0; bool ok = true;
    for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x) {
      int sp, tm, tn; tile_coords(t, sp, tm, tn);
      const int kb0 = sp * kb_per, kb1 = min(nkb_total, kb0 + kb_per);
      if (!mbar_wait(&tfull[acc], accphase)) { ok = false; break; }
      tc_fence_after();
      if (kb1 > kb0 && c_end > c_begin) {
        const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
        if constexpr (EPI == EPI_CE)
          epilogue_row<EPI>(e, taddr, tm * BM + q * 32 + lane, tn * BN, s.M, s.N, c_begin, c_end);
        else
          epilogue_warp<EPI>(e, taddr, tm * BM + q * 32, tn * BN, s.M, s.N, c_begin, c_end,
                             epi_stage + (warp - 2) * EPI_STAGE_FLOATS, lane);
      }
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
      acc ^= 1; if (acc == 0) accphase ^= 1;
    }
    if (!ok && lane == 0) atomicExch(s.err, 3);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host
static int g_num_sms = 0;

template <int MAJ_A, int MAJ_B, int EPI>
static int launch(const void* A, int64_t lda, const void* B, int64_t ldb, int M, int N, int K, int splitk,
                  const EpiArgs& e, int* err, int max_ctas, cudaStream_t st) {
  CUtensorMap tmA, tmB;
  int rc;
  // K-major:  global [rows, K]  -> inner = K, outer = rows, box 64 x tile-rows
  // MN-major: global [K, rows]  -> inner = rows, outer = K, box 64 x 64
  if (MAJ_A == MAJOR_K) rc = make_tmap_2d_bf16(&tmA, A, K, M, lda, 64, BM, true);
  else rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, 64, BK, true);
  if (rc) return rc;
  if (MAJ_B == MAJOR_K) rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, 64, BN, true);
  else rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, 64, BK, true);
  if (rc) return rc;
  auto kern = gemm_kernel<MAJ_A, MAJ_B, EPI>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    attr_done = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int ntiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (splitk > 0 ? splitk : 1);
  int grid = ntiles < g_num_sms ? ntiles : g_num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid <= 0) return 0;
  GemmShape s{M, N, K, splitk, err};
  EpiArgs ec = e;
  ec.chk_err = err;
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(tmA, tmB, s, ec);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace grb

using namespace grb;

extern "C" int grb_gemm(int major_a, int major_b, int epi, const void* A, int64_t lda, const void* B, int64_t ldb,
                        int M, int N, int K, int splitk, const EpiArgs* e, int* err, int max_ctas, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (epi != EPI_RED_F32 && epi != EPI_RED_SCATTER && splitk > 1) return -10;
  if (epi == EPI_CE && N > BN) return -11;
#define GRB_CASE(MA, MB, EP)                                                   \
  if (major_a == MA && major_b == MB && epi == EP)                             \
    return launch<MA, MB, EP>(A, lda, B, ldb, M, N, K, splitk, *e, err, max_ctas, st);
  GRB_CASE(MAJOR_K, MAJOR_K, EPI_STORE_BF16)
  GRB_CASE(MAJOR_K, MAJOR_K, EPI_STORE_F32)
  GRB_CASE(MAJOR_K, MAJOR_K, EPI_BIAS_GELU)
  GRB_CASE(MAJOR_K, MAJOR_K, EPI_RESID_F32)
  GRB_CASE(MAJOR_K, MAJOR_K, EPI_CE)
  GRB_CASE(MAJOR_K, MAJOR_MN, EPI_STORE_BF16)
  GRB_CASE(MAJOR_K, MAJOR_MN, EPI_STORE_F32)
  GRB_CASE(MAJOR_K, MAJOR_MN, EPI_GELU_BWD)
  GRB_CASE(MAJOR_MN, MAJOR_MN, EPI_STORE_F32)
  GRB_CASE(MAJOR_MN, MAJOR_MN, EPI_RED_F32)
  GRB_CASE(MAJOR_MN, MAJOR_MN, EPI_RED_SCATTER)
#undef GRB_CASE
  return -12;
}
