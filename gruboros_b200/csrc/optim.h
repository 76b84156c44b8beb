// C interface of the fused optimizer and merge kernels (optim.cu).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// One Schedule-Free AdamW step over flat fp32 buffers of n elements (16-byte aligned):
//   g *= gscale; v = beta2 v + (1-beta2) g^2; gh = g / (sqrt(v / bias2) + eps) + wd y
//   y = lerp(y, z, ckp1) + lr (beta1 (1 - ckp1) - 1) gh;  z -= lr gh
// w16 (optional) receives bf16(y); zero_grad != 0 clears g in the same pass.
int grb_sfadamw_step(float* y, float* z, float* v, float* g, void* w16, int64_t n, float lr, float beta1, float beta2,
                     float bias2, float eps, float wd, float ckp1, float gscale, int zero_grad, void* stream);
// Sharded variant: this rank owns flat elements [begin, begin+count) (multiples of 4); y, g are full flat buffers,
// z, v hold the shard only; bf16(y) is stored into all `world` mirrors w16_peers[r] (peer pointers).
int grb_sfadamw_shard_step(float* y, float* z, float* v, float* g, void* const* w16_peers, int world, int64_t begin,
                           int64_t count, float lr, float beta1, float beta2, float bias2, float eps, float wd,
                           float ckp1, float gscale, int zero_grad, void* mc16, void* stream);
// mc16 (nullable, here and below): multicast address of all ranks' bf16 mirrors (parallel/nvls.py); when given, each
// new bf16 value is published with ONE multimem.st instead of one store per rank.
// dst_j = (1 - alpha_j) dst_j + alpha_j src_j for up to three buffer pairs (null dst or alpha 0 skips a pair);
// src_j may be a peer GPU's memory.  w16 (optional) receives bf16 of the merged first pair.
int grb_merge(float* dst0, const float* src0, float alpha0, float* dst1, const float* src1, float alpha1, float* dst2,
              const float* src2, float alpha2, void* w16, int64_t n, void* stream);
// Round-robin chunk ownership (owner.cuh, chunks of 2^chunk_shift elements): the sharded step over this rank's
// `count` owned elements (z, v compact; holder_shard > 0: the bf16 value goes only to the mirror of rank
// idx / holder_shard, which holds that range of the sharded weights, instead of to every rank), and the gather that rebuilds full buffers from the owners for checkpoints
// (compact = 1: sources are the owners' compact arrays; skip_own: leave this rank's own elements untouched).
int grb_sfadamw_interleaved_step(float* y, float* z, float* v, float* g, void* const* w16_peers, int world, int rank,
                                 int chunk_shift, int64_t count, float lr, float beta1, float beta2, float bias2, float eps,
                                 float wd, float ckp1, float gscale, int zero_grad, int64_t holder_shard, void* mc16,
                                 void* stream);
// ... and the same step restricted to the owned elements inside the flat range [lo, hi) (multiples of 4): the
// per-layer update that data parallelism folds into backward.
int grb_sfadamw_interleaved_range_step(float* y, float* z, float* v, float* g, void* const* w16_peers, int world, int rank,
                                       int chunk_shift, int64_t lo, int64_t hi, float lr, float beta1, float beta2,
                                       float bias2, float eps, float wd, float ckp1, float gscale, int zero_grad,
                                       int64_t holder_shard, void* mc16, void* stream);
int grb_gather_interleaved(float* dst, void* const* src_peers, int world, int rank, int chunk_shift, int64_t n, int compact,
                           int skip_own, void* stream);
#ifdef __cplusplus
}
#endif
