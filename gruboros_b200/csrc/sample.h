// C interface of the sampling kernel (sample.cu).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// One token per sequence from logits [B, V] (V <= 256).  temperature 0 = greedy; top_k <= 0 and top_p <= 0 switch
// the filters off.  u_in: optional [B] uniforms in [0, 1) (else generated from seed, *step_counter and the sequence
// index).  tok_out [B] bytes; history (optional) [B, hist_len] gets the token at column step_counter[0].
// step_counter (optional, two int64 in device memory): [0] is incremented after the draw, [1] is added to seed, so a
// captured graph can be replayed with a new seed.  probs_out (optional) [B, V]: the filtered distribution.
int grb_sample(const float* logits, int B, int V, float temperature, int top_k, float top_p, const float* u_in,
               uint64_t seed, int64_t* step_counter, uint8_t* tok_out, int64_t* history, int hist_len, float* probs_out,
               void* stream);
#ifdef __cplusplus
}
#endif
