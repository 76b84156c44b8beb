// C interface of the minGRU scan kernels (scan.cu).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// Forward: k, u bf16 [B,T,C] with row stride ldku (elements); h bf16 [B,T,C] with row stride ldh.
// h0 / h_last are fp32 [B,C] and may be null.  C must be even.  `err` is a device int that a
// bounded wait sets non-zero when it gives up.  Returns 0 or a negative host-side error code.
int grb_scan_fwd(const void* k, const void* u, int64_t ldku, const float* h0, void* h, int64_t ldh, float* h_last,
                 int B, int T, int C, int* err, void* stream);
// Backward: g = dL/dh bf16 [B,T,C] (row stride ldg), h = saved forward output.  Writes dk, du (bf16, row stride
// ldd) and optionally dh0 (fp32 [B,C]).  dh_last (fp32 [B,C], may be null) is the gradient of the final state.
// rowscale (fp32 [B*T], may be null) multiplies row (b, t) of dk and du.
int grb_scan_bwd(const void* k, const void* u, int64_t ldku, const void* h, int64_t ldh, const void* g, int64_t ldg,
                 const float* h0, const float* dh_last, void* dk, void* du, int64_t ldd, float* dh0,
                 const float* rowscale, int B, int T, int C, int* err, void* stream);
#ifdef __cplusplus
}
#endif
