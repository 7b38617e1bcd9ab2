// Differential-attention combine:  y = RMSNorm(a1 − λ·a2)·w·c   over rows of W = 2·head_dim elements (W ∈ {128, 256}),
// λ a device scalar (it depends on learned vectors), c = 1 − λ_init.  One warp per row.
// Backward: da = rmsnorm_bwd(dy·w·c);  da1 = da;  da2 = −λ·da;  dλ = −Σ da·a2;  dw += dy·c·â  (â = normalised row).
#include "sm100.cuh"
#include "api.h"

namespace b200 {

__device__ __forceinline__ float da_wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <int EPL> __device__ __forceinline__ void da_ld(const __nv_bfloat16* p, float (&v)[EPL]) {
#pragma unroll
  for (int e = 0; e < EPL; e += 2) { const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p + e)); v[e] = f.x; v[e + 1] = f.y; }
}
template <int EPL> __device__ __forceinline__ void da_st(__nv_bfloat16* p, const float (&v)[EPL]) {
#pragma unroll
  for (int e = 0; e < EPL; e += 2) *reinterpret_cast<uint32_t*>(p + e) = pack_bf16x2(v[e], v[e + 1]);
}

template <int EPL>
__global__ void __launch_bounds__(256) diff_combine_fwd_kernel(const __nv_bfloat16* __restrict__ a1, const __nv_bfloat16* __restrict__ a2,
                                                               const float* __restrict__ lam, const float* __restrict__ w, float c,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, long long rows,
                                                               float eps) {
  constexpr int W = EPL * 32;
  const int lane = threadIdx.x & 31;
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float l = *lam;
  float x1[EPL], x2[EPL];
  da_ld<EPL>(a1 + row * W + lane * EPL, x1);
  da_ld<EPL>(a2 + row * W + lane * EPL, x2);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) { x1[e] -= l * x2[e]; ss += x1[e] * x1[e]; }
  const float rs = rsqrtf(da_wsum(ss) / W + eps);
  if (lane == 0) rstd[row] = rs;
#pragma unroll
  for (int e = 0; e < EPL; ++e) x1[e] = x1[e] * rs * w[lane * EPL + e] * c;
  da_st<EPL>(y + row * W + lane * EPL, x1);
}

template <int EPL>
__global__ void __launch_bounds__(256) diff_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ a1,
                                                               const __nv_bfloat16* __restrict__ a2, const float* __restrict__ lam,
                                                               const float* __restrict__ w, float c, const float* __restrict__ rstd,
                                                               __nv_bfloat16* __restrict__ da1, __nv_bfloat16* __restrict__ da2,
                                                               float* __restrict__ dlam, float* __restrict__ dw, long long rows) {
  constexpr int W = EPL * 32;
  __shared__ float s_dw[W];
  __shared__ float s_dl;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s_dw[i] = 0.f;
  if (threadIdx.x == 0) s_dl = 0.f;
  __syncthreads();
  const float l = *lam;
  float dwr[EPL], dl = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) dwr[e] = 0.f;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; row < rows; row += n_warps) {
    float x1[EPL], x2[EPL], g[EPL];
    da_ld<EPL>(a1 + row * W + lane * EPL, x1);
    da_ld<EPL>(a2 + row * W + lane * EPL, x2);
    da_ld<EPL>(dy + row * W + lane * EPL, g);
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float ah = (x1[e] - l * x2[e]) * rs;
      dwr[e] += g[e] * c * ah;
      g[e] = g[e] * w[lane * EPL + e] * c;
      dot += g[e] * ah;
      x1[e] = ah;
    }
    const float c1 = da_wsum(dot) / W;
    float o2[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float d = (g[e] - x1[e] * c1) * rs;
      dl -= d * x2[e];
      g[e] = d;
      o2[e] = -l * d;
    }
    da_st<EPL>(da1 + row * W + lane * EPL, g);
    da_st<EPL>(da2 + row * W + lane * EPL, o2);
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) atomicAdd(&s_dw[lane * EPL + e], dwr[e]);
  dl = da_wsum(dl);
  if (lane == 0) atomicAdd(&s_dl, dl);
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x) atomicAdd(&dw[i], s_dw[i]);
  if (threadIdx.x == 0) atomicAdd(dlam, s_dl);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_diff_combine_fwd(const void* a1, const void* a2, const float* lam, const float* w, float c, void* y, float* rstd,
                                     long long rows, int width, float eps, cudaStream_t st) {
  if (rows == 0) return 0;
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  typedef __nv_bfloat16 bf;
  if (width == 256) diff_combine_fwd_kernel<8><<<grid, 256, 0, st>>>((const bf*)a1, (const bf*)a2, lam, w, c, (bf*)y, rstd, rows, eps);
  else if (width == 128) diff_combine_fwd_kernel<4><<<grid, 256, 0, st>>>((const bf*)a1, (const bf*)a2, lam, w, c, (bf*)y, rstd, rows, eps);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
// dlam (1 float) and dw (width floats) must be zero on entry
extern "C" int b200_diff_combine_bwd(const void* dy, const void* a1, const void* a2, const float* lam, const float* w, float c,
                                     const float* rstd, void* da1, void* da2, float* dlam, float* dw, long long rows, int width,
                                     cudaStream_t st) {
  if (rows == 0) return 0;
  long long need = (rows + 7) / 8;
  const unsigned grid = static_cast<unsigned>(need < 148 * 8 ? need : 148 * 8);
  typedef __nv_bfloat16 bf;
  if (width == 256) diff_combine_bwd_kernel<8><<<grid, 256, 0, st>>>((const bf*)dy, (const bf*)a1, (const bf*)a2, lam, w, c, rstd, (bf*)da1, (bf*)da2, dlam, dw, rows);
  else if (width == 128) diff_combine_bwd_kernel<4><<<grid, 256, 0, st>>>((const bf*)dy, (const bf*)a1, (const bf*)a2, lam, w, c, rstd, (bf*)da1, (bf*)da2, dlam, dw, rows);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
