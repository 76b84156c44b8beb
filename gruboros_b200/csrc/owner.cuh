// Which rank owns element `idx` of the flat parameter space (data parallel: the owner reduces the gradient of the
// element, keeps its optimizer state and publishes its new value).
//   own > 0 : contiguous shards of `own` elements (rank r owns [r * own, (r + 1) * own)); the sharded-weights mode
//             needs this, because it all-gathers contiguous ranges.
//   own < 0 : chunks of 2^(-own) elements dealt round-robin.  A weight matrix is then spread over all ranks, so the
//             gradient tiles that every rank produces for the same layer at the same time fan out to all owners
//             instead of converging on the one rank whose shard holds that matrix (whose NVLink ingress would carry
//             (world - 1) x the matrix per GEMM).
#pragma once

__host__ __device__ __forceinline__ int grb_owner(long long idx, long long own, int world) {
  return own > 0 ? static_cast<int>(idx / own) : static_cast<int>((idx >> (-own)) % world);
}
// Position of an owned element inside its owner's compact state arrays (z, v).
__host__ __device__ __forceinline__ long long grb_local_index(long long idx, long long own, int world) {
  if (own > 0) return idx % own;
  const int sh = static_cast<int>(-own);
  return (((idx >> sh) / world) << sh) + (idx & ((1ll << sh) - 1));
}
// The same for chunk ownership (own < 0) with 32-bit arithmetic on the chunk index (flat spaces stay far below
// 2^31 chunks), for hot loops: owner and packed position of element idx.
__host__ __device__ __forceinline__ void grb_chunk_place(long long idx, int shift, unsigned world, int& owner, long long& local) {
  const unsigned c = static_cast<unsigned>(idx >> shift);
  const unsigned q = c / world;
  owner = static_cast<int>(c - q * world);
  local = (static_cast<long long>(q) << shift) + (idx & ((1ll << shift) - 1));
}
