// C interface of the NVLink peer-memory runtime (comm.cu).
#pragma once
#include <stddef.h>
#include <stdint.h>
#define GRB_MAX_RANKS 8
#ifdef __cplusplus
extern "C" {
#endif
// Symmetric buffer: zero-filled cudaMalloc allocation plus its 64-byte CUDA IPC handle (handle64 may be null).
int grb_comm_malloc(size_t bytes, void** ptr, void* handle64);
int grb_comm_free(void* ptr);
// Map / unmap a peer's buffer from its IPC handle (enables peer access on first use).
int grb_comm_open(const void* handle64, void** ptr);
int grb_comm_close(void* ptr);
// Publish `value` in slot `rank` of every rank's flag array (peer_flags[p] = base of rank p's uint64[world] array).
int grb_comm_signal(void* const* peer_flags, int world, int rank, unsigned long long value, void* stream);
// Wait until every slot of the local flag array is >= value; after timeout_ns sets *err = 21 and returns.
int grb_comm_wait(const void* local_flags, int world, unsigned long long value, unsigned long long timeout_ns,
                  int* err, void* stream);
// ranges: device int64 [nranges][2] = (offset, count) into the flat fp32 buffers; shard = ownership descriptor
// (owner.cuh: > 0 elements per contiguous shard, < 0 round-robin chunks of 2^(-shard) elements).
// push_add: add locally accumulated gradients of non-owned elements into their owner's buffer and clear them.
int grb_push_add_ranges(float* local, void* const* peer_grads, int world, int rank, const void* ranges, int nranges,
                        long long shard, void* stream);
// bcast: the owner of each element copies its fp32 value to every peer.
int grb_bcast_ranges(const float* local, void* const* peer_datas, int world, int rank, const void* ranges, int nranges,
                     long long shard, void* stream);
#ifdef __cplusplus
}
#endif
