// Allocation-free cross-entropy: the logits GEMM with the fused 256-way cross-entropy epilogue, then the
// reduction of the per-row losses, with the per-row buffer that sits between the two kernels held in a
// file-scope device array instead of caller- or library-allocated memory.  See ce_static.h for who needs this
// and the rules of use.
#include "ce_static.h"
#include "elementwise.h"
#include "gemm_sm100.h"
#include <cuda_runtime.h>
#include <mutex>

extern "C" int grb_gemm_pair(int major_a, int major_b, int epi, const void* A, int64_t lda, const void* B, int64_t ldb,
                             int M, int N, int K, int splitk, const EpiArgs* e, int* err, int max_ctas, void* stream);

namespace {

// Per-row losses of the call in flight.  In host code this name is only a handle for the runtime, not a device
// address: the address a kernel can use comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float g_row_loss[GRB_CE_STATIC_MAX_ROWS];

constexpr int kMaxDevices = 64;
float* g_row_loss_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of g_row_loss on the current device (looked up on the first call per device).
float* row_loss_on_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_row_loss_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_row_loss) != cudaSuccess || !p) return nullptr;
    g_row_loss_addr[dev] = static_cast<float*>(p);
  }
  return g_row_loss_addr[dev];
}

}  // namespace

extern "C" int grb_ce_loss_static(const void* x16, int64_t ldx, const void* w16, int64_t ldw, const uint8_t* labels,
                                  int M, int V, int K, void* dlogits, int64_t ldd, float grad_scale,
                                  float loss_scale_out, float* loss_out, int* err, void* stream) {
  if (M < 1 || M > GRB_CE_STATIC_MAX_ROWS) return -60;
  float* rows = row_loss_on_current_device();
  if (!rows) return -61;
  EpiArgs e = {};
  e.out0 = dlogits;
  e.out1 = rows;
  e.aux = labels;
  e.ldo = dlogits ? ldd : V;
  e.alpha = grad_scale;
  // same kernel choice as the regular path: CTA pairs once there are enough 256-row tiles to fill the machine
  const int pair_tiles = (M + 255) / 256;
  const int rc = pair_tiles >= 48
                     ? grb_gemm_pair(MAJOR_K, MAJOR_K, EPI_CE, x16, ldx, w16, ldw, M, V, K, 1, &e, err, 0, stream)
                     : grb_gemm(MAJOR_K, MAJOR_K, EPI_CE, x16, ldx, w16, ldw, M, V, K, 1, &e, err, 0, stream);
  if (rc) return rc;
  return grb_sum_scale(rows, M, loss_scale_out, loss_out, 0, stream);
}
