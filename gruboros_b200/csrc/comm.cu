// Intra-node communication runtime over NVLink / NVSwitch peer memory.
//
// One process per GPU.  Each rank allocates its symmetric buffers here (plain
// cudaMalloc, so that a CUDA IPC handle names exactly the buffer), ships the
// 64-byte handles to its peers over a host side channel once, and maps the
// peers' buffers.  After that all data moves by loads / stores / reductions
// that kernels issue on peer pointers; the host only exchanges scalars.
//
// Replaces the reference's transport (gloo barriers, raw TCP sockets and a
// shared file system: gossip/network_utils.py, gossip/evolutionary_node.py:392-725).
//
// Cross-GPU ordering uses a per-rank flag array: rank r publishes step s by
// storing s into slot r of every peer's array (release, system scope); a
// rank waits until all slots of its own array reach s.  The wait is bounded
// by a wall-clock limit and reports expiry through an error word.
#include "ptx.cuh"
#include "comm.h"
#include "owner.cuh"

namespace grb {

struct PeerTable {
  void* p[GRB_MAX_RANKS];
};

__global__ void signal_kernel(PeerTable flags, int world, int rank, unsigned long long value) {
  const int peer = threadIdx.x;
  if (peer < world) {
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(flags.p[peer]) + rank;
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(value) : "memory");
  }
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void wait_kernel(const unsigned long long* flags, int world, unsigned long long value,
                            unsigned long long timeout_ns, int* err) {
  const int peer = threadIdx.x;
  if (peer < world) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned long long v = 0;
    bool ok = false;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + peer) : "memory");
      if (v >= value) { ok = true; break; }
      if (globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(200);
    }
    if (!ok) atomicExch(err, 21);
  }
}

// Small-gradient exchange.  Each block owns one range [off, off+cnt) of the flat gradient buffer.  Elements whose
// owner (idx / shard) is another rank are added into the owner's buffer and cleared locally.
__global__ void push_add_ranges_kernel(float* local, PeerTable grads, const long long* ranges, long long shard,
                                       int rank, int world) {
  const long long off = ranges[2 * blockIdx.x], cnt = ranges[2 * blockIdx.x + 1];
  for (long long i = threadIdx.x; i < cnt; i += blockDim.x) {
    const long long idx = off + i;
    const int owner = grb_owner(idx, shard, world);
    if (owner != rank) {
      const float v = local[idx];
      if (v != 0.f) atomicAdd(reinterpret_cast<float*>(grads.p[owner]) + idx, v);
      local[idx] = 0.f;
    }
  }
}

// Owner -> everyone copy of fp32 values (parameters the kernels read in fp32: norm weights, biases, embedding).
__global__ void bcast_ranges_kernel(const float* local, PeerTable datas, const long long* ranges, long long shard,
                                    int rank, int world) {
  const long long off = ranges[2 * blockIdx.x], cnt = ranges[2 * blockIdx.x + 1];
  for (long long i = threadIdx.x; i < cnt; i += blockDim.x) {
    const long long idx = off + i;
    if (grb_owner(idx, shard, world) == rank) {
      const float v = local[idx];
      for (int p = 0; p < world; ++p)
        if (p != rank) reinterpret_cast<float*>(datas.p[p])[idx] = v;
    }
  }
}

}  // namespace grb

using namespace grb;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int grb_comm_malloc(size_t bytes, void** ptr, void* handle64) {
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return -40;
  if (cudaMemset(*ptr, 0, bytes) != cudaSuccess) return -41;
  if (handle64) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) return -42;
    static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
    memcpy(handle64, &h, 64);
  }
  return 0;
}

extern "C" int grb_comm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -43; }

extern "C" int grb_comm_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -44;
}

extern "C" int grb_comm_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -45; }

extern "C" int grb_comm_signal(void* const* peer_flags, int world, int rank, unsigned long long value, void* stream) {
  if (world > GRB_MAX_RANKS) return -46;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = peer_flags[i];
  signal_kernel<<<1, 32, 0, ST(stream)>>>(t, world, rank, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_comm_wait(const void* local_flags, int world, unsigned long long value,
                             unsigned long long timeout_ns, int* err, void* stream) {
  if (world > GRB_MAX_RANKS) return -46;
  wait_kernel<<<1, 32, 0, ST(stream)>>>(reinterpret_cast<const unsigned long long*>(local_flags), world, value,
                                        timeout_ns, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_push_add_ranges(float* local, void* const* peer_grads, int world, int rank, const void* ranges,
                                   int nranges, long long shard, void* stream) {
  if (world > GRB_MAX_RANKS) return -46;
  if (nranges <= 0) return 0;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = peer_grads[i];
  push_add_ranges_kernel<<<nranges, 256, 0, ST(stream)>>>(local, t, reinterpret_cast<const long long*>(ranges), shard, rank, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int grb_bcast_ranges(const float* local, void* const* peer_datas, int world, int rank, const void* ranges,
                                int nranges, long long shard, void* stream) {
  if (world > GRB_MAX_RANKS) return -46;
  if (nranges <= 0) return 0;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = peer_datas[i];
  bcast_ranges_kernel<<<nranges, 256, 0, ST(stream)>>>(local, t, reinterpret_cast<const long long*>(ranges), shard, rank, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
