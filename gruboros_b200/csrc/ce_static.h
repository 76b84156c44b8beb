// Mean 256-way cross-entropy (logits GEMM + loss) for callers that must not allocate device memory.
// This entry point has no counterpart in the reference; it exists for hosts that embed the library.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

// Largest number of rows (tokens) one call may process.  The per-row losses of a call live in a fixed array of
// this many floats (512 KB) inside the library image; every GPU that loads the library holds it until exit.
#define GRB_CE_STATIC_MAX_ROWS 131072

// loss_out[0] = loss_scale_out * sum over rows of CE(x16[row,:] . w16^T, labels[row]);
// dlogits (optional, bf16 [M, ldd]) = (softmax - onehot) * grad_scale.
//
// Who this is for: code that drives the kernels from a context in which cudaMalloc is off limits - a plug-in
// that runs inside another runtime's memory pool and may only touch the buffers it is handed, a service whose
// device memory is fully budgeted at start-up, or a latency-critical loop where an allocation (which can
// synchronise the whole device) is not acceptable.  The regular path (grb_gemm with EPI_CE followed by
// grb_sum_scale) wants a caller-provided [M] fp32 buffer for the per-row losses between its two kernels; this
// variant keeps that buffer in a file-scope device array instead, so the caller passes only inputs and outputs.
//
//   x16    bf16 [M, K] row-major, leading dimension ldx (the normalised hidden states)
//   w16    bf16 [V, K] row-major, leading dimension ldw, V <= 256
//   labels uint8 [M]
//   err    device int that a bounded in-kernel wait sets non-zero when it gives up (same word as grb_gemm)
//
// Returns 0, or a negative code: -60 M > GRB_CE_STATIC_MAX_ROWS (or M < 1), -61 the address of the device
// array could not be obtained on the current device, other codes as grb_gemm.
//
// Rules of use:
//   * The call allocates nothing: no cudaMalloc / cudaFree, no library routine that allocates.
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress with that
//     device current) and remembers it.  Make that first call outside any stream capture.
//   * All calls on a device share the one array, which keeps whatever the previous call left there.  Nothing
//     in it has to start at zero: rows [0, M) are overwritten before they are read and rows beyond M are never
//     read.  Two calls that overlap on the GPU (different streams, no ordering between them) race on it; order
//     them on one stream or with an event.
int grb_ce_loss_static(const void* x16, int64_t ldx, const void* w16, int64_t ldw, const uint8_t* labels, int M, int V,
                       int K, void* dlogits, int64_t ldd, float grad_scale, float loss_scale_out, float* loss_out,
                       int* err, void* stream);

#ifdef __cplusplus
}
#endif
