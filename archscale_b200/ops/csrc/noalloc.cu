// RMSNorm backward without any allocation: the per-CTA weight-gradient partials live in a
// file-scope device array.  See noalloc.h for who needs this and for the rules of use.
#include <stdio.h>

#include "api.h"
#include "noalloc.h"

// Scratch for the dw partial sums, [n_ctas, cols] fp32, n_ctas ≤ 296, cols ≤ 4096.
// In host code this name is only a handle for cudaGetSymbolAddress — never a device pointer.
static __device__ __align__(256) float g_noalloc_scratch[B200_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device
char g_err[256] = "";

int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}
}  // namespace

extern "C" const char* b200_noalloc_last_error(void) { return g_err; }

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* w,
                                        int w_dtype, const float* rstd, void* dx, float* dw, int rows, int cols,
                                        cudaStream_t stream) {
  if (rows < 0 || cols <= 0) return fail(-10, "b200_rmsnorm_bwd_noalloc: rows/cols must be positive");
  if (cols % 8) return fail(-11, "b200_rmsnorm_bwd_noalloc: cols must be a multiple of 8");
  if (cols > B200_NOALLOC_MAX_COLS) {
    snprintf(g_err, sizeof(g_err), "b200_rmsnorm_bwd_noalloc: cols=%d exceeds the built-in scratch (max %d columns)",
             cols, B200_NOALLOC_MAX_COLS);
    return -12;
  }
  if (b200_rmsnorm_bwd_partials(rows, cols) > B200_NOALLOC_MAX_CTAS)
    return fail(-13, "b200_rmsnorm_bwd_noalloc: grid larger than the built-in scratch");
  if (rows == 0) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(-14, "b200_rmsnorm_bwd_noalloc: cannot determine the current device");
  if (g_scratch_ptr[dev] == nullptr) {
    // once per device, with that device current (it is: we just read it)
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_err, sizeof(g_err), "b200_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return -15;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  const int rc = b200_rmsnorm_bwd(dy, dy_dtype, x, x_dtype, w, w_dtype, rstd, dx, w ? g_scratch_ptr[dev] : nullptr,
                                  w ? dw : nullptr, rows, cols, stream);
  if (rc != 0) return fail(rc, "b200_rmsnorm_bwd_noalloc: kernel launch failed");
  g_err[0] = 0;
  return 0;
}
