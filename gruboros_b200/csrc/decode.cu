// Token-by-token decoding: weight-streaming matrix-vector kernels with the layer's element-wise work fused in.
//
// One decode step of a minLM layer is four launches of one kernel template:
//   gate   h   <- lerp(h, g(Wh xn), sigmoid(Wz xn)),  xn = RMSNorm(x)      (prologue: norm, epilogue: minGRU step)
//   out    x   <- x + Wo h                                                  (epilogue: residual)
//   ff1    a   <- gelu(W1 RMSNorm(x) + b1)                                  (prologue: norm, epilogue: bias + GELU)
//   ff2    x   <- x + W2 a + b2                                             (epilogue: bias + residual)
// and the head is the same kernel with a norm prologue and a plain store.  With up to 8 sequences per step the
// work is reading every weight once, so the kernel is shaped for HBM: a warp owns whole weight rows and pulls them
// through its own ring of bulk copies in shared memory, the input vectors (times the norm weight) sit in shared
// memory as bf16 - the operand precision of the training GEMMs - and accumulation is fp32 on the CUDA cores.
// This is the bit-reproducible fallback chain; the default decode chain is the tensor-core one in decode_tc.cu.
// The recurrence is the reference's single-step branch (mingru/minGRU.py:47-52); there is no counterpart of these
// kernels in the reference, which calls nn.Linear.
#include "decode.h"
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace grb {
namespace {

enum { DEC_STORE = 0, DEC_GATE = 1, DEC_RESID = 2, DEC_GELU = 3 };

struct DecArgs {
  const float* x;               // [B, K] input, fp32
  const float* norm_w;          // [K] RMSNorm weight, or null for no prologue
  const __nv_bfloat16* W;       // [N, K]   (DEC_GATE: [2N, K], rows n = candidate, N + n = gate)
  const float* bias;            // [N] or null
  float* out;                   // [B, N]
  int B, N, K;
  float eps;
  int has_prev;                 // DEC_GATE: out holds h_{t-1}; otherwise the step starts from nothing (h = z g(u))
  int* err;                     // status word set when a bounded wait gives up
  int slots;                    // ring depth per warp
};

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float dot8(const uint4& w, const uint4& x) {
  return bf16_lo(w.x) * bf16_lo(x.x) + bf16_hi(w.x) * bf16_hi(x.x) + bf16_lo(w.y) * bf16_lo(x.y) +
         bf16_hi(w.y) * bf16_hi(x.y) + bf16_lo(w.z) * bf16_lo(x.z) + bf16_hi(w.z) * bf16_hi(x.z) +
         bf16_lo(w.w) * bf16_lo(x.w) + bf16_hi(w.w) * bf16_hi(x.w);
}

constexpr int DEC_WARPS = 8;
constexpr int DEC_MAX_SLOTS = 6;        // weight segments in flight per warp (the launch picks 1..6 to fit shared memory)
constexpr int DEC_SEG_BYTES = 4096;     // one segment: 256 16-byte chunks (of one row, or 128 + 128 of the two gate rows)

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// BT = sequences handled (B rounded up to 1, 2, 4 or 8); rows b >= B of the staged input are zero.
//
// A CTA is 8 warps; warp w of CTA c owns output rows c*8+w, c*8+w + 8*gridDim, ...  A row is cut into segments of
// 4 KB of weights.  Every warp runs its own ring of `slots` segments in shared memory, filled by bulk copies
// (cp.async.bulk, completion counted on one mbarrier per slot) that one lane issues: the bytes in flight are
// bounded by shared memory, not by registers, so a small matrix is in flight almost whole from the first cycle.
//   1. Fill the ring.  Weights do not depend on the previous kernel of the step, so this happens before waiting
//      for that kernel (griddepcontrol; without the programmatic-serialisation launch attribute both instructions
//      do nothing).
//   2. Stage in = x * norm_w as bf16 in shared memory and, on the way, each sequence's sum of squares (RMSNorm's
//      1/rms is a per-sequence scalar, so it multiplies the finished dot product instead of every element).
//   3. Per segment: wait for its barrier, multiply from shared memory, hand the slot to the segment `slots`
//      ahead; after a row's last segment reduce over the warp and let lane b finish sequence b.
// Every wait is bounded; on expiry the status word is set and the warp stops issuing (its outstanding copies, if
// any arrive later, target shared memory that stays allocated until the other warps are done; the CTA then waits
// once more, bounded, for them before it exits).
template <int EPI, int BT>
__global__ void __launch_bounds__(32 * DEC_WARPS) decode_gemv_kernel(const DecArgs a) {
  extern __shared__ __align__(128) uint8_t dsm[];
  constexpr int NR = EPI == DEC_GATE ? 2 : 1;                 // weight rows per output (candidate + gate)
  constexpr int SEGC = 256 / NR;                              // 16-byte chunks per weight row and segment
  constexpr int CH = SEGC / 32;                               // ... per lane
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K = a.K;
  const int S = a.slots;
  uint8_t* ring = dsm + (static_cast<size_t>(warp) * S) * DEC_SEG_BYTES;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(dsm + static_cast<size_t>(DEC_WARPS) * S * DEC_SEG_BYTES);
  __shared__ uint64_t bars[DEC_WARPS][DEC_MAX_SLOTS];
  __shared__ float red[BT][DEC_WARPS];

  const int nchunk = K >> 3;                                  // 16-byte chunks per row
  const int P = (nchunk + SEGC - 1) / SEGC;                   // segments per row
  const int first = blockIdx.x * DEC_WARPS + warp, stride = gridDim.x * DEC_WARPS;
  const int rows_w = first < a.N ? (a.N - first + stride - 1) / stride : 0;
  const int nseg = rows_w * P;
  const uint4* W4 = reinterpret_cast<const uint4*>(a.W);

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < DEC_MAX_SLOTS; ++i) mbar_init(&bars[warp][i], 1);
    fence_mbar_init();
  }
  __syncwarp();

  // lane 0: start the copy of segment `sgm` into its slot
  auto issue = [&](int sgm) {
    const int row = first + (sgm / P) * stride, p = sgm % P;
    const int c0 = p * SEGC;
    const int nc = min(SEGC, nchunk - c0);
    uint64_t* bar = &bars[warp][sgm % S];
    uint8_t* dst = ring + static_cast<size_t>(sgm % S) * DEC_SEG_BYTES;
    mbar_expect_tx(bar, static_cast<uint32_t>(NR * nc * 16));
#pragma unroll
    for (int r = 0; r < NR; ++r)
      bulk_g2s(dst + r * (DEC_SEG_BYTES / NR), W4 + (static_cast<size_t>(row) + static_cast<size_t>(r) * a.N) * nchunk + c0,
               static_cast<uint32_t>(nc * 16), bar);
  };

  // ---- 1. independent of the previous kernel
  if (lane == 0)
    for (int sgm = 0; sgm < min(S, nseg); ++sgm) issue(sgm);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- 2. stage the input
  {
    float ss[BT];
#pragma unroll
    for (int b = 0; b < BT; ++b) ss[b] = 0.f;
    for (int k = tid * 4; k < K; k += 128 * DEC_WARPS) {
      float4 nw = make_float4(1.f, 1.f, 1.f, 1.f);
      if (a.norm_w) nw = *reinterpret_cast<const float4*>(a.norm_w + k);
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < a.B) v = *reinterpret_cast<const float4*>(a.x + static_cast<size_t>(b) * K + k);
        ss[b] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        *reinterpret_cast<uint2*>(xs + static_cast<size_t>(b) * K + k) =
            make_uint2(pack_bf16(v.x * nw.x, v.y * nw.y), pack_bf16(v.z * nw.z, v.w * nw.w));
      }
    }
#pragma unroll
    for (int b = 0; b < BT; ++b) {
      const float t = warp_sum_f(ss[b]);
      if (lane == 0) red[b][warp] = t;
    }
  }
  __syncthreads();

  // ---- 3. segments
  float acc[NR][BT];
#pragma unroll
  for (int r = 0; r < NR; ++r)
#pragma unroll
    for (int b = 0; b < BT; ++b) acc[r][b] = 0.f;
  bool ok = true;
  int done = 0;                                               // segments whose copy has been waited for
  for (int sgm = 0; sgm < nseg; ++sgm) {
    const int slot = sgm % S;
    if (!__all_sync(0xffffffffu, mbar_wait(&bars[warp][slot], (sgm / S) & 1))) { ok = false; break; }   // warp-uniform
    done = sgm + 1;
    const int p = sgm % P;
    const int c0 = p * SEGC;
    const uint8_t* src = ring + static_cast<size_t>(slot) * DEC_SEG_BYTES;
#pragma unroll
    for (int u = 0; u < CH; ++u) {
      const int cl = u * 32 + lane;                           // chunk within the segment
      if (c0 + cl < nchunk) {
        uint4 w[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) w[r] = *reinterpret_cast<const uint4*>(src + r * (DEC_SEG_BYTES / NR) + cl * 16);
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + static_cast<size_t>(b) * K + 8 * (c0 + cl));
#pragma unroll
          for (int r = 0; r < NR; ++r) acc[r][b] += dot8(w[r], xv);
        }
      }
    }
    __syncwarp();                                             // every lane is done reading the slot
    if (lane == 0 && sgm + S < nseg) {
      fence_proxy_async_smem();                               // order those reads before the copy that overwrites them
      issue(sgm + S);
    }
    if (p != P - 1) continue;
    // last segment of a row: reduce and finish; lane b handles sequence b
    const int n = first + (sgm / P) * stride;
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int b = 0; b < BT; ++b) acc[r][b] = warp_sum_f(acc[r][b]);
#pragma unroll
    for (int b = 0; b < BT; ++b) {
      if (lane == b && b < a.B) {
        float rs = 1.f;
        if (a.norm_w) {
          float t = 0.f;
#pragma unroll
          for (int q = 0; q < DEC_WARPS; ++q) t += red[b][q];
          rs = rsqrtf(t / K + a.eps);
        }
        float* o = a.out + static_cast<size_t>(b) * a.N + n;
        float v = acc[0][b] * rs;
        if constexpr (EPI == DEC_GATE) {
          const float u = v, k = acc[NR - 1][b] * rs;
          const float cand = u >= 0.f ? u + 0.5f : 1.f / (1.f + expf(-u));
          const float z = 1.f / (1.f + expf(-k));
          *o = a.has_prev ? fmaf(z, cand - *o, *o) : cand * z;
        } else {
          if (a.bias) v += a.bias[n];
          if constexpr (EPI == DEC_RESID) *o += v;
          else if constexpr (EPI == DEC_GELU) *o = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
          else *o = v;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
      for (int b = 0; b < BT; ++b) acc[r][b] = 0.f;
  }
  if (!ok) {
    // a copy did not arrive in time: report, then give what is still outstanding one more bounded wait each so
    // that nothing lands in shared memory after the CTA is gone
    if (lane == 0) atomicExch(a.err, 7);
    const int issued = min(nseg, done + S);
    for (int sgm = done; sgm < issued; ++sgm)
      if (!mbar_wait(&bars[warp][sgm % S], (sgm / S) & 1)) break;
  }
}

template <int EPI, int BT>
size_t& smem_granted() {
  static size_t v = 0;
  return v;
}

template <int EPI>
int launch_bt(const DecArgs& a, int blocks, size_t smem, bool pdl, cudaStream_t st) {
  auto go = [&](auto kern, size_t& set) -> int {
    // static shared memory counts against the default 48 KB too, hence the margin; `set` is this kernel's own record
    // of the largest size already granted, so replays and captures after the first use make no attribute call
    if (smem > 32 * 1024 && smem > set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return -4;
      set = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(32 * DEC_WARPS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kern, a);
    if (err == cudaSuccess) err = cudaGetLastError();
    return err == cudaSuccess ? 0 : -(1000 + static_cast<int>(err));      // -(1000 + cudaError) for the caller to report
  };
  if (a.B <= 1) return go(decode_gemv_kernel<EPI, 1>, smem_granted<EPI, 1>());
  if (a.B <= 2) return go(decode_gemv_kernel<EPI, 2>, smem_granted<EPI, 2>());
  if (a.B <= 4) return go(decode_gemv_kernel<EPI, 4>, smem_granted<EPI, 4>());
  return go(decode_gemv_kernel<EPI, 8>, smem_granted<EPI, 8>());
}

}  // namespace
}  // namespace grb

extern "C" int grb_decode_gemv(int epi, const float* x, const float* norm_w, const void* W, const float* bias,
                               float* out, int B, int N, int K, float eps, int has_prev, int num_sms, int overlap,
                               int* err, void* stream) {
  using namespace grb;
  if (B < 1 || B > 8 || N < 1 || K < 8 || K % 8 || !err) return -40;
  if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15) return -41;
  if (norm_w && (reinterpret_cast<uintptr_t>(norm_w) & 15)) return -41;
  const int bt = B <= 1 ? 1 : B <= 2 ? 2 : B <= 4 ? 4 : 8;
  const size_t xs_bytes = static_cast<size_t>(bt) * K * 2;
  // Ring depth: the deepest that leaves room for a second CTA on the SM - the next kernel of the step, started
  // early, fills its ring while this one computes; if the staged input is too large for that, the deepest that fits.
  constexpr size_t kSmemSm = 227 * 1024, kPerCta = 2048;      // per-CTA reservation + static shared memory, rounded up
  const size_t ring1 = static_cast<size_t>(DEC_WARPS) * DEC_SEG_BYTES;
  int slots = 0;
  for (int sl = DEC_MAX_SLOTS; sl >= 2 && !slots; --sl)
    if (2 * (sl * ring1 + xs_bytes + kPerCta) <= kSmemSm) slots = sl;
  for (int sl = DEC_MAX_SLOTS; sl >= 1 && !slots; --sl)
    if (sl * ring1 + xs_bytes + kPerCta <= kSmemSm) slots = sl;
  if (!slots) return -42;
  const size_t smem = slots * ring1 + xs_bytes;
  DecArgs a{x, norm_w, reinterpret_cast<const __nv_bfloat16*>(W), bias, out, B, N, K, eps, has_prev, err, slots};
  // one CTA per SM at most: every CTA pays the input staging once, warps walk their rows through the ring, and
  // the other half of the SM stays free for the next kernel of the step
  const int sms = num_sms > 0 ? num_sms : 148;
  int blocks = (N + DEC_WARPS - 1) / DEC_WARPS;
  if (blocks > sms) blocks = sms;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (epi) {
    case DEC_STORE: return launch_bt<DEC_STORE>(a, blocks, smem, overlap != 0, st);
    case DEC_GATE: return launch_bt<DEC_GATE>(a, blocks, smem, overlap != 0, st);
    case DEC_RESID: return launch_bt<DEC_RESID>(a, blocks, smem, overlap != 0, st);
    case DEC_GELU: return launch_bt<DEC_GELU>(a, blocks, smem, overlap != 0, st);
  }
  return -43;
}
