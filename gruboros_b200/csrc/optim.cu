// Fused Schedule-Free AdamW step and the gossip merge kernel for sm_100a.
//
// The optimizer the reference uses is schedulefree.AdamWScheduleFree
// (train.py:19,635,808): about ten _foreach_ passes over every parameter per
// step.  Here one pass over flat fp32 buffers reads g, y, z, v and writes
// y, z, v plus the bf16 copy of y that the GEMMs consume, and clears g.
//
// The merge kernel is the data plane of the evolutionary gossip
// (gossip/evolutionary_node.py:250-313,591-725): the loser reads the winner's
// flat buffers (a peer pointer over NVLink, or a local pointer) and blends
// them into its own in the same pass that moves them.
#include "ptx.cuh"
#include "optim.h"

namespace grb {

struct SfArgs {
  float lr, beta1, beta2, bias2, eps, wd, ckp1, gscale;
};

__device__ __forceinline__ void sf_update(float g, float& y, float& z, float& v, const SfArgs& a) {
  g *= a.gscale;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v / a.bias2) + a.eps;
  const float gh = g / denom + a.wd * y;
  y = y + a.ckp1 * (z - y);
  y = y + a.lr * (a.beta1 * (1.f - a.ckp1) - 1.f) * gh;
  z = z - a.lr * gh;
}

__global__ void __launch_bounds__(256)
sfadamw_kernel(float* __restrict__ y, float* __restrict__ z, float* __restrict__ v, float* __restrict__ g,
               __nv_bfloat16* __restrict__ w16, int64_t n, SfArgs a, int zero_grad) {
  const int64_t nvec = n / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 yv = reinterpret_cast<float4*>(y)[i];
    float4 zv = reinterpret_cast<float4*>(z)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    sf_update(gv.x, yv.x, zv.x, vv.x, a);
    sf_update(gv.y, yv.y, zv.y, vv.y, a);
    sf_update(gv.z, yv.z, zv.z, vv.z, a);
    sf_update(gv.w, yv.w, zv.w, vv.w, a);
    reinterpret_cast<float4*>(y)[i] = yv;
    reinterpret_cast<float4*>(z)[i] = zv;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (w16) reinterpret_cast<uint2*>(w16)[i] = make_uint2(pack_bf16(yv.x, yv.y), pack_bf16(yv.z, yv.w));
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) {
      float gg = g[i], yy = y[i], zz = z[i], vv = v[i];
      sf_update(gg, yy, zz, vv, a);
      y[i] = yy; z[i] = zz; v[i] = vv;
      if (w16) w16[i] = __float2bfloat16(yy);
      if (zero_grad) g[i] = 0.f;
    }
  }
}

// Sharded step (data parallel, optimizer state partitioned by element range): this rank owns flat elements
// [begin, begin + count); y and g are the full flat buffers, z and v hold only the shard.  The updated bf16
// weights are stored into every rank's mirror (w16s.p[r], peer pointers) - the parameter all-gather fused
// into the update.
struct PeerTable16 {
  __nv_bfloat16* p[8];
  __nv_bfloat16* mc;   // multicast address of the mirrors (NVSwitch replicates one store into every rank's copy), or null
};

// Four bf16 values to every rank's mirror: one multimem store when the mirrors are bound to a multicast object,
// otherwise one ordinary store per rank through the peer pointers.  `at` is in units of four elements.
__device__ __forceinline__ void publish_bf16x4(const PeerTable16& t, int world, int64_t at, uint2 w) {
  if (t.mc) {
    const unsigned long long v = (static_cast<unsigned long long>(w.y) << 32) | w.x;
    asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(reinterpret_cast<uint2*>(t.mc) + at), "l"(v) : "memory");
  } else {
    for (int r = 0; r < world; ++r) reinterpret_cast<uint2*>(t.p[r])[at] = w;
  }
}

__global__ void __launch_bounds__(256)
sfadamw_shard_kernel(float* __restrict__ y, float* __restrict__ z, float* __restrict__ v, float* __restrict__ g,
                     PeerTable16 w16s, int world, int64_t begin, int64_t count, SfArgs a, int zero_grad) {
  const int64_t nvec = count / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  float4* y4 = reinterpret_cast<float4*>(y + begin);
  float4* g4 = reinterpret_cast<float4*>(g + begin);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 gv = g4[i];
    float4 yv = y4[i];
    float4 zv = reinterpret_cast<float4*>(z)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    sf_update(gv.x, yv.x, zv.x, vv.x, a);
    sf_update(gv.y, yv.y, zv.y, vv.y, a);
    sf_update(gv.z, yv.z, zv.z, vv.z, a);
    sf_update(gv.w, yv.w, zv.w, vv.w, a);
    y4[i] = yv;
    reinterpret_cast<float4*>(z)[i] = zv;
    reinterpret_cast<float4*>(v)[i] = vv;
    const uint2 w = make_uint2(pack_bf16(yv.x, yv.y), pack_bf16(yv.z, yv.w));
    publish_bf16x4(w16s, world, begin / 4 + i, w);
    if (zero_grad) g4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// The same update for round-robin chunk ownership (owner.cuh, own < 0): thread work item j is the j-th float4 of
// this rank's compact state (z, v); its element lives at chunk (j-th owned chunk) * world + rank of the flat space.
__global__ void __launch_bounds__(256)
sfadamw_interleaved_kernel(float* __restrict__ y, float* __restrict__ z, float* __restrict__ v, float* __restrict__ g,
                           PeerTable16 w16s, int world, int rank, int chunk_shift, int64_t nvec, SfArgs a, int zero_grad,
                           int64_t holder_shard) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int vshift = chunk_shift - 2;                              // float4 units per chunk = 2^vshift
  const int64_t vmask = (int64_t(1) << vshift) - 1;
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < nvec; j += stride) {
    const int64_t i = ((((j >> vshift) * world + rank) << vshift) + (j & vmask));   // float4 index in the flat space
    float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 yv = reinterpret_cast<float4*>(y)[i];
    float4 zv = reinterpret_cast<float4*>(z)[j];
    float4 vv = reinterpret_cast<float4*>(v)[j];
    sf_update(gv.x, yv.x, zv.x, vv.x, a);
    sf_update(gv.y, yv.y, zv.y, vv.y, a);
    sf_update(gv.z, yv.z, zv.z, vv.z, a);
    sf_update(gv.w, yv.w, zv.w, vv.w, a);
    reinterpret_cast<float4*>(y)[i] = yv;
    reinterpret_cast<float4*>(z)[j] = zv;
    reinterpret_cast<float4*>(v)[j] = vv;
    const uint2 w = make_uint2(pack_bf16(yv.x, yv.y), pack_bf16(yv.z, yv.w));
    if (holder_shard > 0) {            // weights sharded at rest: only the rank that holds this range gets the value
      reinterpret_cast<uint2*>(w16s.p[(4 * i) / holder_shard])[i] = w;
    } else {
      publish_bf16x4(w16s, world, i, w);
    }
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// The same update restricted to the flat range [lo4, hi4) (float4 units): the owned chunks first_chunk, first_chunk +
// world, ... (n_chunks of them) are walked and elements outside the range are skipped.  This is the per-layer
// update folded into backward under round-robin ownership: a chunk that straddles two layers is updated in two parts.
__global__ void __launch_bounds__(256)
sfadamw_interleaved_range_kernel(float* __restrict__ y, float* __restrict__ z, float* __restrict__ v, float* __restrict__ g,
                                 PeerTable16 w16s, int world, int chunk_shift, int64_t first_chunk, int64_t n_chunks,
                                 int64_t lo4, int64_t hi4, SfArgs a, int zero_grad, int64_t holder_shard) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int vshift = chunk_shift - 2;
  const int64_t vmask = (int64_t(1) << vshift) - 1;
  const int64_t items = n_chunks << vshift;
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < items; t += stride) {
    const int64_t chunk = first_chunk + (t >> vshift) * world;
    const int64_t i = (chunk << vshift) + (t & vmask);              // float4 index in the flat space
    if (i < lo4 || i >= hi4) continue;
    const int64_t j = ((chunk / world) << vshift) + (t & vmask);    // float4 index in this rank's compact state
    float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 yv = reinterpret_cast<float4*>(y)[i];
    float4 zv = reinterpret_cast<float4*>(z)[j];
    float4 vv = reinterpret_cast<float4*>(v)[j];
    sf_update(gv.x, yv.x, zv.x, vv.x, a);
    sf_update(gv.y, yv.y, zv.y, vv.y, a);
    sf_update(gv.z, yv.z, zv.z, vv.z, a);
    sf_update(gv.w, yv.w, zv.w, vv.w, a);
    reinterpret_cast<float4*>(y)[i] = yv;
    reinterpret_cast<float4*>(z)[j] = zv;
    reinterpret_cast<float4*>(v)[j] = vv;
    const uint2 w = make_uint2(pack_bf16(yv.x, yv.y), pack_bf16(yv.z, yv.w));
    if (holder_shard > 0) {
      reinterpret_cast<uint2*>(w16s.p[(4 * i) / holder_shard])[i] = w;
    } else {
      publish_bf16x4(w16s, world, i, w);
    }
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Checkpoint support for round-robin chunk ownership: dst[idx] = the owner's value of element idx, for every idx in
// [0, n).  compact = 0: the sources are full flat buffers (parameters), compact = 1: each source is its owner's
// compact array (optimizer state).  skip_own leaves this rank's own elements alone (they are already in place).
struct PeerTableF {
  const float* p[8];
};
__global__ void __launch_bounds__(256)
gather_interleaved_kernel(float* __restrict__ dst, PeerTableF src, int world, int rank, int chunk_shift, int64_t nvec,
                          int compact, int skip_own) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int vshift = chunk_shift - 2;
  const int64_t vmask = (int64_t(1) << vshift) - 1;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int64_t chunk = i >> vshift;
    const int owner = static_cast<int>(chunk % world);
    if (skip_own && owner == rank) continue;
    const int64_t from = compact ? (((chunk / world) << vshift) + (i & vmask)) : i;
    reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src.p[owner])[from];
  }
}

// dst_j = (1 - alpha_j) * dst_j + alpha_j * src_j for up to three fp32 buffer pairs of n elements
// (parameters y, Schedule-Free z, second moment v); alpha 1 is a clonal copy, alpha 0 skips the pair.
// src_j may live on a peer GPU.  w16 (optional) receives the bf16 copy of the merged first pair.
struct MergeArgs {
  float* dst[3];
  const float* src[3];
  float alpha[3];
};

__global__ void __launch_bounds__(256)
merge_kernel(MergeArgs m, __nv_bfloat16* __restrict__ w16, int64_t n) {
  const int64_t nvec = n / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      if (m.dst[j] == nullptr || m.alpha[j] == 0.f) continue;
      const float al = m.alpha[j];
      const float4 s = reinterpret_cast<const float4*>(m.src[j])[i];
      float4 d;
      if (al == 1.f) {
        d = s;
      } else {
        d = reinterpret_cast<float4*>(m.dst[j])[i];
        d.x += al * (s.x - d.x); d.y += al * (s.y - d.y); d.z += al * (s.z - d.z); d.w += al * (s.w - d.w);
      }
      reinterpret_cast<float4*>(m.dst[j])[i] = d;
      if (j == 0 && w16) reinterpret_cast<uint2*>(w16)[i] = make_uint2(pack_bf16(d.x, d.y), pack_bf16(d.z, d.w));
    }
  }
  if (blockIdx.x == 0) {
    for (int64_t i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) {
      for (int j = 0; j < 3; ++j) {
        if (m.dst[j] == nullptr || m.alpha[j] == 0.f) continue;
        const float d = m.alpha[j] == 1.f ? m.src[j][i] : m.dst[j][i] + m.alpha[j] * (m.src[j][i] - m.dst[j][i]);
        m.dst[j][i] = d;
        if (j == 0 && w16) w16[i] = __float2bfloat16(d);
      }
    }
  }
}

static int grid_for(int64_t nvec) {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  int64_t b = (nvec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  return static_cast<int>(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace grb

using namespace grb;

extern "C" int grb_sfadamw_step(float* y, float* z, float* v, float* g, void* w16, int64_t n, float lr, float beta1,
                                float beta2, float bias2, float eps, float wd, float ckp1, float gscale,
                                int zero_grad, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(g)) & 15)
    return -2;
  if (w16 && (reinterpret_cast<uintptr_t>(w16) & 7)) return -2;
  SfArgs a{lr, beta1, beta2, bias2, eps, wd, ckp1, gscale};
  sfadamw_kernel<<<grid_for(n / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      y, z, v, g, reinterpret_cast<__nv_bfloat16*>(w16), n, a, zero_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_merge(float* dst0, const float* src0, float alpha0, float* dst1, const float* src1, float alpha1,
                         float* dst2, const float* src2, float alpha2, void* w16, int64_t n, void* stream) {
  if (n <= 0) return 0;
  MergeArgs m;
  m.dst[0] = dst0; m.src[0] = src0; m.alpha[0] = alpha0;
  m.dst[1] = dst1; m.src[1] = src1; m.alpha[1] = alpha1;
  m.dst[2] = dst2; m.src[2] = src2; m.alpha[2] = alpha2;
  for (int j = 0; j < 3; ++j)
    if (m.dst[j] && ((reinterpret_cast<uintptr_t>(m.dst[j]) | reinterpret_cast<uintptr_t>(m.src[j])) & 15)) return -2;
  merge_kernel<<<grid_for(n / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      m, reinterpret_cast<__nv_bfloat16*>(w16), n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_sfadamw_shard_step(float* y, float* z, float* v, float* g, void* const* w16_peers, int world,
                                      int64_t begin, int64_t count, float lr, float beta1, float beta2, float bias2,
                                      float eps, float wd, float ckp1, float gscale, int zero_grad, void* mc16, void* stream) {
  if (count <= 0) return 0;
  if (world > 8 || (begin % 4) || (count % 4)) return -2;
  SfArgs a{lr, beta1, beta2, bias2, eps, wd, ckp1, gscale};
  PeerTable16 t;
  t.mc = reinterpret_cast<__nv_bfloat16*>(mc16);
  for (int r = 0; r < world; ++r) t.p[r] = reinterpret_cast<__nv_bfloat16*>(w16_peers[r]);
  sfadamw_shard_kernel<<<grid_for(count / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      y, z, v, g, t, world, begin, count, a, zero_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_sfadamw_interleaved_step(float* y, float* z, float* v, float* g, void* const* w16_peers, int world,
                                            int rank, int chunk_shift, int64_t count, float lr, float beta1, float beta2,
                                            float bias2, float eps, float wd, float ckp1, float gscale, int zero_grad,
                                            int64_t holder_shard, void* mc16, void* stream) {
  if (count <= 0) return 0;
  if (world > 8 || chunk_shift < 5 || (count & ((int64_t(1) << chunk_shift) - 1))) return -2;
  SfArgs a{lr, beta1, beta2, bias2, eps, wd, ckp1, gscale};
  PeerTable16 t;
  t.mc = reinterpret_cast<__nv_bfloat16*>(mc16);
  for (int r = 0; r < world; ++r) t.p[r] = reinterpret_cast<__nv_bfloat16*>(w16_peers[r]);
  sfadamw_interleaved_kernel<<<grid_for(count / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      y, z, v, g, t, world, rank, chunk_shift, count / 4, a, zero_grad, holder_shard);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_sfadamw_interleaved_range_step(float* y, float* z, float* v, float* g, void* const* w16_peers, int world,
                                                  int rank, int chunk_shift, int64_t lo, int64_t hi, float lr, float beta1,
                                                  float beta2, float bias2, float eps, float wd, float ckp1, float gscale,
                                                  int zero_grad, int64_t holder_shard, void* mc16, void* stream) {
  if (hi <= lo) return 0;
  if (world > 8 || world < 1 || rank < 0 || rank >= world || chunk_shift < 5 || (lo & 3) || (hi & 3) || lo < 0) return -2;
  // owned chunks that intersect [lo, hi): the first chunk index >= lo's chunk that is congruent to rank
  const int64_t c_lo = lo >> chunk_shift, c_hi = (hi - 1) >> chunk_shift;
  int64_t first = c_lo + ((rank - c_lo % world) % world + world) % world;
  if (first > c_hi) return 0;
  const int64_t n_chunks = (c_hi - first) / world + 1;
  SfArgs a{lr, beta1, beta2, bias2, eps, wd, ckp1, gscale};
  PeerTable16 t;
  t.mc = reinterpret_cast<__nv_bfloat16*>(mc16);
  for (int r = 0; r < world; ++r) t.p[r] = reinterpret_cast<__nv_bfloat16*>(w16_peers[r]);
  sfadamw_interleaved_range_kernel<<<grid_for((n_chunks << chunk_shift) / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      y, z, v, g, t, world, chunk_shift, first, n_chunks, lo / 4, hi / 4, a, zero_grad, holder_shard);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_gather_interleaved(float* dst, void* const* src_peers, int world, int rank, int chunk_shift, int64_t n,
                                      int compact, int skip_own, void* stream) {
  if (n <= 0) return 0;
  if (world > 8 || chunk_shift < 5 || (n & ((int64_t(1) << chunk_shift) - 1))) return -2;
  PeerTableF t;
  for (int r = 0; r < world; ++r) t.p[r] = reinterpret_cast<const float*>(src_peers[r]);
  gather_interleaved_kernel<<<grid_for(n / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      dst, t, world, rank, chunk_shift, n / 4, compact, skip_own);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
