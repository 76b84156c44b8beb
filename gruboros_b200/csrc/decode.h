// C interface of the decode (matrix-vector) kernels (decode.cu).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// out[b, n] = epilogue(sum_k W[n, k] * in[b, k]) for b < B <= 8, W bf16 row-major [N, K] (K % 8 == 0).
//   norm_w != null : in = RMSNorm(x) * norm_w (eps as given), else in = x; either way rounded to bf16
//   epi 0 : out = acc + bias
//   epi 1 : minGRU step; W is [2N, K] (candidate rows then gate rows); out (the hidden state) is updated in place:
//           out = has_prev ? lerp(out, g(acc_cand), sigmoid(acc_gate)) : g(acc_cand) * sigmoid(acc_gate)
//   epi 2 : out += acc + bias
//   epi 3 : out = gelu(acc + bias)            (erf form)
// bias may be null.  overlap != 0 launches with programmatic stream serialisation: the kernel may start while the
// previous kernel on the stream is still running, prefetches its weights into L2 and only then waits for it, so a
// chain of these calls streams weights without gaps.  err: device status word, set to 7 if a bounded wait for a
// weight copy gives up.  Returns 0, a negative code for unsupported arguments, or
// -(1000 + cudaError) if the launch failed.
int grb_decode_gemv(int epi, const float* x, const float* norm_w, const void* W, const float* bias, float* out, int B,
                    int N, int K, float eps, int has_prev, int num_sms, int overlap, int* err, void* stream);

// Tensor-core variant (decode_tc.cu): out[b, n] += sum_k W[n, k] * in[b, k] (+ out_bias[n], once) with fp32 atomics;
// split over K so that about one CTA per SM streams weights.  `in` is computed from `src` on the way in:
//   mode 0 : in = RMSNorm(src) * vec                       (src [B, K], vec = norm weight [K])
//   mode 1 : in = lerp(state, g(src_c), sigmoid(src_g))    (src [B, 2K] = candidate | gate pre-activations); the new
//            state is also written to state_out (must differ from state)
//   mode 2 : in = gelu(src + vec)                          (vec = bias [K] or null)
// Housekeeping for a chain of calls: zero_buf[0..zero_n) is cleared and copy_src[0..copy_n) is copied to copy_dst
// (either may be null); both must be dead / complete before this call in stream order.
int grb_decode_tc(int mode, const float* src, const float* vec, const float* state, float* state_out, const void* W,
                  float* out, const float* out_bias, float* zero_buf, int zero_n, float* copy_dst,
                  const float* copy_src, int copy_n, int B, int N, int K, float eps, int num_sms, int overlap, int* err,
                  void* stream);
#ifdef __cplusplus
}
#endif
