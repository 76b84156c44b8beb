// C interface of the tcgen05 GEMM (gemm_sm100.cu).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Which dimension of an operand is contiguous in global memory.
enum { MAJOR_K = 0, MAJOR_MN = 1 };

// Fused epilogues.  `acc` is the fp32 accumulator, v = acc * alpha * rowscale[row] (+ bias[col]), where rowscale is 1
// unless `rowss` is given (see EpiArgs: the RMSNorm of the A operand applied after the contraction).
enum {
  EPI_STORE_BF16 = 0,  // out0[bf16] = v
  EPI_STORE_F32 = 1,   // out0[f32]  = v
  EPI_BIAS_GELU = 2,   // out0[bf16] = gelu'(v) (what the backward pass multiplies by), out1[bf16] = gelu(v)
  EPI_RESID_F32 = 3,   // out0[f32] = x = aux[f32] + v   (residual stream; aux may alias out0); with `normw`:
                       // out2[bf16] = x * normw[col] and ssq_out[row, tile part] = sum over the part's columns of x^2
                       // (the inputs of the NEXT RMSNorm, which its consumer GEMM finishes through `rowss`)
  EPI_GELU_BWD = 4,    // out0[bf16] = acc * alpha * aux[bf16] * rowscale[row]   (aux = gelu' saved by EPI_BIAS_GELU);
                       // with `colsum`: colsum[col] += sum over rows of acc * alpha * aux (the bias gradient)
  EPI_RED_F32 = 5,     // red.add.f32 out0 += v      (wgrad accumulate; out0 may be peer memory)
  EPI_RED_SCATTER = 7, // red.add.f32 into the buffer of the rank that owns the element (data-parallel
                       // reduce-scatter fused into wgrad): element index i = flat_off + row*ldo + col of the flat
                       // gradient space belongs to rank i / shard, whose buffer base is peers[rank]
  EPI_CE = 6           // N<=256: out1[f32][row] = CE loss of row vs aux[u8] label,
                       //         out0[bf16] = (softmax - onehot) * alpha   (either may be null)
};

typedef struct EpiArgs {
  void* out0;
  void* out1;
  const void* aux;
  const float* bias;
  int64_t ldo;   // leading dimension (elements) of out0/out1/out2/aux
  float alpha;
  // RMSNorm folded into the GEMMs.  A producer (EPI_RESID_F32 with normw) leaves, per row, `rowss_parts` partial
  // sums of squares (one per 128 output columns); a consumer GEMM whose A operand is the unnormalised bf16 x * normw
  // scales its accumulator rows by rsqrt(sum(parts) * rowss_inv_d + rowss_eps), which equals normalising first.
  const float* rowss;  // [M, rowss_parts] or null; with rowss_parts == 0 an [M] vector of ready-made row scales
  int rowss_parts;
  float rowss_inv_d;
  float rowss_eps;
  float* rstd_out;     // [M] or null: the row scales, written once per row (by the tiles of output column 0) for backward
  void* out2;          // EPI_RESID_F32: bf16 [M, ldo] x * normw (null: not produced)
  const float* normw;  // [N] weight of the next RMSNorm
  float* ssq_out;      // [M, ceil(N / 128)] partial sums of squares of x
  float* colsum;       // EPI_GELU_BWD: [N] fp32, accumulated with atomics (null: not produced)
  // EPI_RED_SCATTER only
  int world;
  int chunk_aligned;   // flat_off, ldo and the shard / chunk size are multiples of 32: a 32-column chunk never straddles two owners
  int64_t flat_off;
  int64_t shard;       // ownership descriptor (owner.cuh): > 0 contiguous shards of that many elements, < 0 chunks of 2^(-shard)
  void* peers[8];
  int compact;         // EPI_RED_SCATTER: peers[r] holds only rank r's owned elements, packed (owner.cuh: grb_local_index)
                       // - fully sharded training, where no rank has a full-size gradient buffer
  // Side copy (CTA-pair kernel only): while the tensor cores work, two extra warps per CTA stream up to 8
  // segments src[i] -> dst[i] (bytes multiple of 16, 16-byte aligned; src may be a peer GPU's memory).  Used to
  // all-gather the NEXT layer's sharded weights over NVLink underneath the current gate GEMM.
  int n_copy;
  const void* copy_src[8];
  void* copy_dst[8];
  int64_t copy_bytes[8];
  // Chunk gather (same copy warps): rebuild bf16 elements [gather_lo, gather_hi) of a flat space whose chunks are dealt
  // round-robin over `world` ranks (shard < 0) from the ranks' packed shards peers[r] into gather_dst (element
  // gather_lo lands at gather_dst[0]).  This is the all-gather of the NEXT layer's sharded weights; it shares
  // `peers`, `world` and `shard` with the scatter epilogue, so a GEMM carries one or the other.
  int64_t gather_lo, gather_hi;   // multiples of 8 elements; gather_hi <= gather_lo: nothing to gather
  void* gather_dst;
  // Extents for the checked build (-DGRB_CHECKS, `python -m gruboros_b200.build --checks`): elements that every
  // peers[r] buffer holds and that gather_dst holds (0: unknown, not checked).  In that build an epilogue that is
  // about to touch an element outside these extents, outside [M, N] or through an out-of-range rank records a
  // status code in the error word and skips the access instead of making it.
  int64_t peer_limit;
  int64_t gather_cap;
  int* chk_err;        // filled in by the launcher (the launch's error word); callers leave it null
} EpiArgs;

// Status codes of the checked build (written to the error word like the time-out codes).
enum { GRB_CHK_TILE = 31, GRB_CHK_PEER = 32, GRB_CHK_GATHER = 33, GRB_CHK_TMA_STORE = 34, GRB_CHK_PARTS = 35 };

// Stand-alone version of the chunk gather, for the first layer of a pass.
// peer_limit / dst_cap: elements each shard / dst holds (0: unknown), used by the checked build; err: error word.
int grb_gather_chunks(void* const* shard_ptrs, int world, int chunk_shift, int64_t lo, int64_t hi, void* dst,
                      int64_t peer_limit, int64_t dst_cap, int* err, void* stream);

// Stand-alone version of the side copy (same segment format), for the first layer of a pass.
int grb_copy_segments(int n, const void* const* src, void* const* dst, const int64_t* bytes, void* stream);

// D[M,N] = A * B^T with the operand layouts named by major_a / major_b:
//   MAJOR_K : A is [M,K] (B is [N,K]) row-major with leading dimension lda (ldb)
//   MAJOR_MN: A is [K,M] (B is [K,N]) row-major with leading dimension lda (ldb)
// splitk > 1 is only valid with EPI_RED_F32.  `err` is a device int that a
// bounded wait sets non-zero if it gave up.  max_ctas > 0 caps the grid.
// Returns 0 or a negative host-side error code.
int grb_gemm(int major_a, int major_b, int epi, const void* A, int64_t lda, const void* B, int64_t ldb, int M, int N,
             int K, int splitk, const EpiArgs* e, int* err, int max_ctas, void* stream);

#ifdef __cplusplus
}
#endif
