// CTA-pair variant of the tcgen05 GEMM: two CTAs of a 2-CTA cluster (two SMs) cooperate on one 256 x 256
// accumulator tile with tcgen05.mma.cta_group::2.
//
// Each CTA loads only ITS half of both operands per 64-deep k-block - 128 rows of A (its half of M) and
// 128 rows of B (its half of N), 32 KB instead of the 48 KB a lone CTA needs for half the tile - so the
// shared-memory fill traffic per FLOP drops by a third.  A ring stage holds TWO k-blocks (64 KB per CTA, three
// stages) and the MMA warp signals a stage's release with ONE commit that arrives on both CTAs' barriers
// (tcgen05.commit with a CTA mask): every commit costs the tensor pipe a few dozen clocks, and going from two
// commits per k-block to one per two k-blocks was worth 17 % on the model's shapes.  The MMA is issued by the
// even ("leader") CTA only; the hardware reads A and B from both CTAs' shared memory and writes each CTA's
// 128 accumulator rows into that CTA's own tensor memory.  The TMA loads are ordinary per-CTA loads whose
// completion bytes are counted on the leader's barrier; nothing is broadcast between the CTAs.
//
//   producer warp (both CTAs)   wait own empty[s] -> TMA A-half, B-half -> leader's full[s]
//   MMA warp      (leader)      wait full[s] -> 8 x tcgen05.mma.cta_group::2 -> one tcgen05.commit onto both CTAs'
//                               empty[s]; after the last k-block also onto both CTAs' tfull[acc]
//   copy warps    (both CTAs)  optional: stream peer-memory segments into local memory (FSDP all-gather of the
//                               next layer's weights) while the tensor cores work
//   epilogue warps (both CTAs)  wait own tfull[acc] -> tcgen05.ld own rows -> fused epilogue -> arrive on the
//                               leader's tempty[acc]
// Work is dealt either as whole tiles (optionally split along K into `splitk` equal parts), or - for the accumulating
// epilogues, splitk < 0 - as equal contiguous runs of (tile, k-block) units, one run per CTA pair ("stream-K"): every
// pair gets the same number of k-blocks whatever the tile count, a tile that a run only partly covers is added into
// the output like a split-K part, and there are at most (tiles + pairs) partial reductions instead of tiles x splitk.
// Every wait is bounded; both CTAs always reach the final cluster barrier before tensor memory is freed.
#include "ptx.cuh"
#include "gemm_sm100.h"
#include "tmap.h"
#include "gemm_epilogue.cuh"
#include <cstdio>

namespace grb {
namespace pair {

constexpr int BM = 128;            // rows of A per CTA  (tile M = 256 per pair)
constexpr int BNH = 128;           // rows of B per CTA  (tile N = 256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
#ifndef GRB_PAIR_STAGES
#define GRB_PAIR_STAGES 3
#endif
#ifndef GRB_PAIR_KSUB
#define GRB_PAIR_KSUB 2
#endif
#ifndef GRB_PAIR_GM
#define GRB_PAIR_GM 8
#endif
constexpr int STAGES = GRB_PAIR_STAGES;
constexpr int KSUB = GRB_PAIR_KSUB;           // 64-deep k-blocks per ring stage (one barrier round trip and one commit each)
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_STAGE_BYTES = BNH * BK * 2;   // 16 KB
constexpr int SUB_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int STAGE_BYTES = KSUB * SUB_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_COPY_WARPS = 2;               // side-copy warps (idle unless EpiArgs::n_copy > 0)
constexpr int NUM_THREADS = 64 + 32 * NUM_EPI_WARPS + 32 * NUM_COPY_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 1024 /*barriers*/ + NUM_EPI_WARPS * EPI_STAGE_BYTES;
#ifndef GRB_TMA_STORE
#define GRB_TMA_STORE 1
#endif

struct Shape {
  int M, N, K, splitk;
  int* err;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Per-CTA TMA load whose completion bytes are counted on a barrier that may live in the peer CTA.  The operand tiles
// are re-read by many CTAs, so they are tagged evict-last in L2 (the streaming output is tagged evict-first).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* desc, uint32_t bar_cluster_addr, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at shared::cluster address `bar_cluster_addr` (own or peer CTA) once every MMA issued so
// far by this thread has retired.
__device__ __forceinline__ void umma2_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
// ... on the same barrier of both CTAs of the pair, with one instruction (the arrival is multicast to the CTAs in the
// mask; no data moves).
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

// One unit of work of a CTA pair: k-blocks [kb0, kb1) of output tile (tm, tn).
struct Work {
  int tm, tn, kb0, kb1;
};

// Deals the work of a launch to the pairs (see the header comment); all three warp roles walk the same sequence.
struct WorkIter {
  int ntm, ntn, nkb, kb_per, ntiles;     // kb_per: k-blocks per split part (whole-tile mode)
  bool stream;
  long long pos, end;                    // stream-K: this pair's run of (tile * nkb + kb) units; else: tile part index / count
  int step;

  __device__ __forceinline__ void tile_coords(int r, int& tm, int& tn) const {
    constexpr int GM = GRB_PAIR_GM;      // row tiles per raster group: a wave of pairs shares ~GM A panels and ~pairs/GM B panels
    const int per_group = GM * ntn;
    const int g = r / per_group;
    const int first_m = g * GM;
    const int gsz = min(GM, ntm - first_m);
    const int in = r - g * per_group;
    tm = first_m + in % gsz;
    tn = in / gsz;
  }
  __device__ __forceinline__ bool next(Work& w) {
    if (pos >= end) return false;
    if (stream) {
      const int t = static_cast<int>(pos / nkb);
      w.kb0 = static_cast<int>(pos - static_cast<long long>(t) * nkb);
      w.kb1 = static_cast<int>(min(static_cast<long long>(nkb), w.kb0 + (end - pos)));
      tile_coords(t, w.tm, w.tn);
      pos += w.kb1 - w.kb0;
    } else {
      const int t = static_cast<int>(pos);
      const int sp = t / ntiles;
      tile_coords(t - sp * ntiles, w.tm, w.tn);
      w.kb0 = sp * kb_per;
      w.kb1 = min(nkb, w.kb0 + kb_per);
      pos += step;
    }
    return true;
  }
};

__device__ __forceinline__ WorkIter make_work(int M, int N, int K, int splitk, int pair_id, int npairs) {
  WorkIter it;
  it.ntm = (M + 2 * BM - 1) / (2 * BM);
  it.ntn = (N + BN - 1) / BN;
  it.nkb = (K + BK - 1) / BK;
  it.ntiles = it.ntm * it.ntn;
  it.stream = splitk < 0;
  if (it.stream) {
    const long long total = static_cast<long long>(it.ntiles) * it.nkb;
    long long run = (total + npairs - 1) / npairs;
    run = (run + KSUB - 1) / KSUB * KSUB;            // whole ring stages
    it.pos = min(total, run * pair_id);
    it.end = min(total, run * (pair_id + 1));
    it.kb_per = it.nkb; it.step = 0;
  } else {
    const int sk = splitk > 0 ? splitk : 1;
    it.kb_per = (it.nkb + sk - 1) / sk;
    it.pos = pair_id; it.end = static_cast<long long>(it.ntiles) * sk; it.step = npairs;
  }
  return it;
}

template <int MAJ_A, int MAJ_B, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const Shape s, const EpiArgs e) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  float* epi_stage = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 1024);  // per-warp staging tiles (1 KB aligned)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 2 * NUM_EPI_WARPS); }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();          // barriers of both CTAs are initialised, tensor memory is allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer (both CTAs)
    int stage = 0; uint32_t phase = 0; bool ok = true;
    const uint64_t pol = l2_policy_evict_last();
    WorkIter it = make_work(s.M, s.N, s.K, s.splitk, pair_id, npairs);
    Work w;
    while (ok && it.next(w)) {
      const int row_a = w.tm * 2 * BM + static_cast<int>(rank) * BM;
      const int row_b = w.tn * BN + static_cast<int>(rank) * BNH;
      for (int kb = w.kb0; kb < w.kb1; kb += KSUB) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) { ok = false; break; }
        if (lane == 0) {
          const int nsub = min(KSUB, w.kb1 - kb);
          if (leader) mbar_expect_tx(&full[stage], 2 * nsub * SUB_BYTES);   // both CTAs' bytes land on the leader's barrier
          const uint32_t fb = map_to_cta(smem_u32(&full[stage]), 0);
          for (int sub = 0; sub < nsub; ++sub) {
            uint8_t* sa = smem + stage * STAGE_BYTES + sub * SUB_BYTES;
            uint8_t* sb = sa + A_STAGE_BYTES;
            const int kk = (kb + sub) * BK;
            if constexpr (MAJ_A == MAJOR_K) {
              tma_load_2d_pair(sa, &tmA, fb, kk, row_a, pol);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * CHUNK_BYTES, &tmA, fb, row_a + 64 * j, kk, pol);
            }
            if constexpr (MAJ_B == MAJOR_K) {
              tma_load_2d_pair(sb, &tmB, fb, kk, row_b, pol);
            } else {
#pragma unroll
              for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * CHUNK_BYTES, &tmB, fb, row_b + 64 * j, kk, pol);
            }
          }
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && lane == 0) atomicExch(s.err, 4);
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN, MAJ_A == MAJOR_MN, MAJ_B == MAJOR_MN);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int acc = 0; uint32_t accphase = 0;
      WorkIter it = make_work(s.M, s.N, s.K, s.splitk, pair_id, npairs);
      Work w;
      while (ok && it.next(w)) {
        if (!mbar_wait(&tempty[acc], accphase ^ 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; kb += KSUB) {
          if (!mbar_wait(&full[stage], phase)) { ok = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const int nsub = min(KSUB, w.kb1 - kb);
            for (int sub = 0; sub < nsub; ++sub) {
              const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES + sub * SUB_BYTES);
              const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                uint64_t ad, bd;
                if constexpr (MAJ_A == MAJOR_K) ad = umma_smem_desc(sa + k * UMMA_K * 2, 16, 1024);
                else ad = umma_smem_desc(sa + k * UMMA_K * 128, CHUNK_BYTES, 1024);
                if constexpr (MAJ_B == MAJOR_K) bd = umma_smem_desc(sb + k * UMMA_K * 2, 16, 1024);
                else bd = umma_smem_desc(sb + k * UMMA_K * 128, CHUNK_BYTES, 1024);
                umma2_bf16(d_tmem, ad, bd, idesc, (kb + sub > w.kb0 || k > 0) ? 1u : 0u);
              }
            }
            umma2_commit_both(&empty[stage]);
            if (kb + KSUB >= w.kb1) umma2_commit_both(&tfull[acc]);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (w.kb1 <= w.kb0 && lane == 0) umma2_commit_both(&tfull[acc]);
        __syncwarp();
        acc ^= 1; if (acc == 0) accphase ^= 1;
      }
      if (!ok && lane == 0) atomicExch(s.err, 5);
    }
  } else if (warp >= 2 + NUM_EPI_WARPS) {
    // ---------------------------------------------------------- side copy (all-gather prefetch)
    if (e.n_copy > 0 || e.gather_hi > e.gather_lo)
      side_copy(e, blockIdx.x, gridDim.x, threadIdx.x - 32 * (2 + NUM_EPI_WARPS), 32 * NUM_COPY_WARPS);
  } else {
    // ---------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int c_begin = (EPI == EPI_CE) ? 0 : half * (BN / 2);
    const int c_end = (EPI == EPI_CE) ? (half == 0 ? BN : 0) : (half + 1) * (BN / 2);
    int acc = 0; uint32_t accphase = 0; bool ok = true;
    WorkIter it = make_work(s.M, s.N, s.K, s.splitk, pair_id, npairs);
    Work w;
    while (ok && it.next(w)) {
      const int tm = w.tm, tn = w.tn;
      if (!mbar_wait(&tfull[acc], accphase)) { ok = false; break; }
      tc_fence_after();
      const bool tile_ok = grb_ok(e, tm >= 0 && tm < it.ntm && tn >= 0 && tn < it.ntn && w.kb0 >= 0 && w.kb1 <= it.nkb, GRB_CHK_TILE);
      if (tile_ok && w.kb1 > w.kb0 && c_end > c_begin) {
        const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
        const int row0 = tm * 2 * BM + static_cast<int>(rank) * BM + q * 32;
        if constexpr (EPI == EPI_CE)
          epilogue_row<EPI>(e, taddr, row0 + lane, tn * BN, s.M, s.N, c_begin, c_end);
        else if constexpr (EPI == EPI_STORE_BF16 && GRB_TMA_STORE)
          epilogue_tma_store_bf16(e, &tmC, taddr, row0, tn * BN, s.M, s.N, c_begin, c_end,
                                  reinterpret_cast<uint8_t*>(epi_stage) + (warp - 2) * 4096, lane);
        else
          epilogue_warp<EPI>(e, taddr, row0, tn * BN, s.M, s.N, c_begin, c_end, epi_stage + (warp - 2) * EPI_STAGE_FLOATS, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&tempty[acc]), 0));
      acc ^= 1; if (acc == 0) accphase ^= 1;
    }
    if constexpr (EPI == EPI_STORE_BF16 && GRB_TMA_STORE) epilogue_tma_store_drain(lane);
    if (!ok && lane == 0) atomicExch(s.err, 6);
  }

  tc_fence_before();
  cluster_sync_all();          // nobody touches the peer's shared or tensor memory after this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <int MAJ_A, int MAJ_B, int EPI>
static int launch(const void* A, int64_t lda, const void* B, int64_t ldb, int M, int N, int K, int splitk,
                  const EpiArgs& e, int* err, int max_ctas, cudaStream_t st) {
  CUtensorMap tmA, tmB, tmC = {};
  int rc;
  if (MAJ_A == MAJOR_K) rc = make_tmap_2d_bf16(&tmA, A, K, M, lda, 64, BM, true);
  else rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, 64, BK, true);
  if (rc) return rc;
  if (MAJ_B == MAJOR_K) rc = make_tmap_2d_bf16(&tmB, B, K, N, ldb, 64, BNH, true);
  else rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, 64, BK, true);
  if (rc) return rc;
  if (EPI == EPI_STORE_BF16 && GRB_TMA_STORE) {
    // output tile map for the TMA-store epilogue: bf16 [M, N] row-major, box 32 columns x 32 rows, 64-byte swizzle
    rc = make_tmap_2d_bf16_sw(&tmC, e.out0, N, M, e.ldo, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  auto kern = gemm_pair_kernel<MAJ_A, MAJ_B, EPI>;
  static int max_pairs = -1;
  if (max_pairs < 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -4;
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2, 1, 1);
    q.blockDim = dim3(NUM_THREADS, 1, 1);
    q.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    q.attrs = at; q.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n <= 0) return -6;
    max_pairs = n;
  }
  const int out_tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  long long ntiles = static_cast<long long>(out_tiles) * (splitk > 0 ? splitk : 1);
  if (splitk < 0) {       // stream-K: as many pairs as there are runs of at least eight k-blocks
    const long long units = static_cast<long long>(out_tiles) * ((K + BK - 1) / BK);
    ntiles = units / 8 > 0 ? units / 8 : 1;
  }
  int pairs = ntiles < max_pairs ? static_cast<int>(ntiles) : max_pairs;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (pairs <= 0) return 0;
  Shape s{M, N, K, splitk, err};
  EpiArgs ec = e;
  ec.chk_err = err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, s, ec) == cudaSuccess ? 0 : -5;
}

}  // namespace pair
}  // namespace grb

using namespace grb;

extern "C" int grb_gemm_pair(int major_a, int major_b, int epi, const void* A, int64_t lda, const void* B, int64_t ldb,
                             int M, int N, int K, int splitk, const EpiArgs* e, int* err, int max_ctas, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (epi != EPI_RED_F32 && epi != EPI_RED_SCATTER && (splitk > 1 || splitk < 0)) return -10;
  if (epi == EPI_CE && N > pair::BN) return -11;
#define GRB_CASE(MA, MB, EP)                                                   \
  if (major_a == MA && major_b == MB && epi == EP)                             \
    return pair::launch<MA, MB, EP>(A, lda, B, ldb, M, N, K, splitk, *e, err, max_ctas, st);
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

namespace grb {
__global__ void __launch_bounds__(256) copy_segments_kernel(const EpiArgs e) { side_copy(e, blockIdx.x, gridDim.x, threadIdx.x, 256); }
}  // namespace grb

extern "C" int grb_gather_chunks(void* const* shard_ptrs, int world, int chunk_shift, int64_t lo, int64_t hi, void* dst,
                                 int64_t peer_limit, int64_t dst_cap, int* err, void* stream) {
  if (hi <= lo) return 0;
  if (world < 1 || world > 8 || chunk_shift < 5 || (lo & 7) || (hi & 7) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -2;
  EpiArgs e = {};
  e.world = world;
  e.shard = -chunk_shift;
  for (int r = 0; r < world; ++r) e.peers[r] = shard_ptrs[r];
  e.gather_lo = lo; e.gather_hi = hi; e.gather_dst = dst;
  e.peer_limit = peer_limit; e.gather_cap = dst_cap; e.chk_err = err;
  static int sms = 0;
  if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  grb::copy_segments_kernel<<<sms * 2, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(e);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_copy_segments(int n, const void* const* src, void* const* dst, const int64_t* bytes, void* stream) {
  if (n <= 0) return 0;
  if (n > 8) return -13;
  EpiArgs e = {};
  e.n_copy = n;
  for (int i = 0; i < n; ++i) {
    if ((reinterpret_cast<uintptr_t>(src[i]) | reinterpret_cast<uintptr_t>(dst[i]) | static_cast<uintptr_t>(bytes[i])) & 15) return -2;
    e.copy_src[i] = src[i]; e.copy_dst[i] = dst[i]; e.copy_bytes[i] = bytes[i];
  }
  static int sms = 0;
  if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  grb::copy_segments_kernel<<<sms * 2, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(e);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
