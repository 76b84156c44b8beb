// Next-token sampling for byte-level vocabularies (V <= 256) in one kernel: temperature, top-k, top-p (nucleus),
// then an inverse-CDF draw; one block per sequence, one thread per vocabulary entry.  The sampled token goes straight
// into the decoder's input buffer and into a history row, and the step counter lives on the device, so the kernel
// can sit in front of the decode step inside one CUDA graph and a whole generation needs no host round trip.
// Filtering follows the reference's `sample` (generate.py:30-79): logits / T; top-k keeps every entry with fewer
// than k strictly larger ones (ties at the k-th value stay); top-p sorts descending and drops an entry when the
// probability mass in front of it already exceeds p (the first entry that crosses the threshold stays).
#include "sample.h"
#include <cuda_runtime.h>
#include <math_constants.h>

namespace grb {
namespace {

__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = sh[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) r = fmaxf(r, sh[w]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) r += sh[w];
  __syncthreads();
  return r;
}

// counter-based generator: one uniform in [0, 1) per (seed, step, sequence)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long step, unsigned int b) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (step * 1024ull + b + 1ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(256) sample_kernel(const float* __restrict__ logits, int V, float temperature, int top_k,
                                                     float top_p, const float* __restrict__ u_in, unsigned long long seed,
                                                     long long* step_counter, unsigned char* tok_out, long long* history,
                                                     int hist_len, float* probs_out) {
  __shared__ float l[256], p[256], red[8];
  __shared__ int winner;
  const int i = threadIdx.x, b = blockIdx.x;
  const bool in = i < V;
  const long long step = step_counter ? step_counter[0] : 0;
  if (step_counter) seed += static_cast<unsigned long long>(step_counter[1]);   // per-generation seed, set by the host
  float li = in ? logits[static_cast<size_t>(b) * V + i] : -CUDART_INF_F;
  int tok;
  if (temperature == 0.f) {
    // greedy: largest logit, lowest index among equals
    l[i] = li;
    __syncthreads();
    const float m = block_max(li, red);
    if (i == 0) winner = 256;
    __syncthreads();
    if (in && li == m) atomicMin(&winner, i);
    __syncthreads();
    tok = winner;
    if (probs_out && in) probs_out[static_cast<size_t>(b) * V + i] = i == tok ? 1.f : 0.f;
  } else {
    li = in ? li / temperature : li;
    l[i] = li;
    __syncthreads();
    bool keep = in;
    if (top_k > 0 && top_k < V) {
      int greater = 0;
      for (int j = 0; j < V; ++j) greater += l[j] > li ? 1 : 0;
      keep = keep && greater < top_k;
    }
    const float m = block_max(keep ? li : -CUDART_INF_F, red);
    float pi = keep ? __expf(li - m) : 0.f;
    const float tot = block_sum(pi, red);
    pi /= tot;
    p[i] = pi;
    __syncthreads();
    if (top_p > 0.f) {
      // probability mass sorted in front of entry i (descending value, lower index first among equals)
      float before = 0.f;
      for (int j = 0; j < V; ++j)
        if (l[j] > li || (l[j] == li && j < i)) before += p[j];
      if (before > top_p) pi = 0.f;
    }
    const float tot2 = block_sum(pi, red);
    pi /= tot2;
    __syncthreads();
    p[i] = pi;
    __syncthreads();
    if (probs_out && in) probs_out[static_cast<size_t>(b) * V + i] = pi;
    // inverse CDF in index order: the token is the first index whose running sum exceeds u
    const float u = u_in ? u_in[b] : uniform01(seed, static_cast<unsigned long long>(step), b);
    float run = 0.f;
    for (int j = 0; j <= i && j < V; ++j) run += p[j];
    if (i == 0) winner = 256;
    __syncthreads();
    if (in && pi > 0.f && run > u) atomicMin(&winner, i);
    __syncthreads();
    if (winner == 256) {                      // u beyond the rounded total: take the last entry with mass
      if (i == 0) winner = -1;
      __syncthreads();
      if (in && pi > 0.f) atomicMax(&winner, i);
      __syncthreads();
    }
    tok = winner;
  }
  if (i == 0) {
    tok_out[b] = static_cast<unsigned char>(tok);
    if (history && step < hist_len) history[static_cast<size_t>(b) * hist_len + step] = tok;
  }
}

__global__ void bump_kernel(long long* counter) { *counter += 1; }

}  // namespace
}  // namespace grb

extern "C" int grb_sample(const float* logits, int B, int V, float temperature, int top_k, float top_p, const float* u_in,
                          uint64_t seed, int64_t* step_counter, uint8_t* tok_out, int64_t* history, int hist_len,
                          float* probs_out, void* stream) {
  if (B < 1 || V < 1 || V > 256 || !logits || !tok_out || temperature < 0.f) return -50;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  grb::sample_kernel<<<B, 256, 0, st>>>(logits, V, temperature, top_k, top_p, u_in, seed,
                                        reinterpret_cast<long long*>(step_counter), tok_out,
                                        reinterpret_cast<long long*>(history), hist_len, probs_out);
  if (step_counter) grb::bump_kernel<<<1, 1, 0, st>>>(reinterpret_cast<long long*>(step_counter));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
