// C interface of the streaming kernels (elementwise.cu).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// normw (nullable): also write xw = bf16(x * normw) and ssq [M, parts] = (sum of x^2, 0, ...) for a folded RMSNorm.
int grb_embed_fwd(const uint8_t* tokens, int64_t stride, int B, int T, int D, int V, const float* E, float* x,
                  uint8_t* labels, void* onehot, const float* normw, void* xw, float* ssq, int parts, void* stream);
int grb_rmsnorm_fwd(const float* x, const float* w, void* y, float* rstd, int64_t M, int D, float eps, void* stream);
// prescaled != 0: dy is the gradient w.r.t. the unnormalised x * w (norm folded into the consumer GEMM).
int grb_rmsnorm_bwd(const void* dy, const float* x, const float* rstd, const float* w, const float* dres_in,
                    float* dres_out, void* dres16, float* dw, float* dcol, int64_t M, int D, int prescaled, int* err,
                    void* stream);
int grb_colsum_bf16(const void* a, int64_t ld, int64_t M, int N, float* out, void* stream);
int grb_sum_scale(const float* v, int64_t n, float scale, float* out, int accumulate, void* stream);
int grb_cast_f32_bf16(const float* in, void* out, int64_t n, void* stream);
#ifdef __cplusplus
}
#endif
