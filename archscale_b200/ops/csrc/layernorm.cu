// LayerNorm forward / backward (phi4-mini-flash family): y = (x − mean)·rstd·w + b, fp32 statistics.
// One warp per row.  The backward is persistent: each warp walks a strided set of rows, keeps its slice of
// dw / db in registers (a lane owns columns lane·8 + 256·i), and the eight warps of a CTA combine their
// slices in shared memory once at the end; per-CTA partials are summed by a second small kernel.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int LN_MAX_CHUNKS = 10;      // columns ≤ 10·256 = 2560 (register-resident dw / db slices)
constexpr int LN_BWD_CTAS = 296;

template <typename T> __device__ __forceinline__ void ln_ld8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void ln_ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void ln_ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void ln_st8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void ln_st8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void ln_st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]); u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float ln_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ bias, T* __restrict__ y,
                                                            float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                                            int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const T* xr = x + static_cast<size_t>(row) * cols;
  float s = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8]; ln_ld8(xr + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
  }
  const float mean = ln_warp_sum(s) / cols;
  float ss = 0.f;                                   // second pass over the (L1-resident) row: centred sum of squares
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8]; ln_ld8(xr + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) { const float d = v[i] - mean; ss += d * d; }
  }
  const float rstd = rsqrtf(ln_warp_sum(ss) / cols + eps);
  if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
  T* yr = y + static_cast<size_t>(row) * cols;
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8]; ln_ld8(xr + c, v);
    float g[8], bb[8];
    if (w) ln_ld8(w + c, g);
    if (bias) ln_ld8(bias + c, bb);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float o = (v[i] - mean) * rstd;
      if (w) o *= g[i];
      if (bias) o += bb[i];
      v[i] = o;
    }
    ln_st8(yr + c, v);
  }
}

template <typename T, int NCH>
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                            const float* __restrict__ w, const float* __restrict__ mean,
                                                            const float* __restrict__ rstd, T* __restrict__ dx,
                                                            float* __restrict__ part, int rows, int cols) {
  extern __shared__ float ln_s[];                   // [2][cols]: dw, db of the CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) ln_s[c] = 0.f;
  __syncthreads();
  float dwr[NCH][8], dbr[NCH][8];
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) { dwr[j][i] = 0.f; dbr[j][i] = 0.f; }
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const T* xr = x + static_cast<size_t>(row) * cols;
    const T* dyr = dy + static_cast<size_t>(row) * cols;
    const float mu = mean[row], rs = rstd[row];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = lane * 8 + j * 256;
      if (c < cols) {
        float xv[8], dv[8], wv[8];
        ln_ld8(xr + c, xv); ln_ld8(dyr + c, dv);
        if (w) ln_ld8(w + c, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float h = (xv[i] - mu) * rs;
          const float g = w ? dv[i] * wv[i] : dv[i];
          c1 += g * h; c2 += g;
          dwr[j][i] += dv[i] * h; dbr[j][i] += dv[i];
        }
      }
    }
    c1 = ln_warp_sum(c1) / cols;
    c2 = ln_warp_sum(c2) / cols;
    T* dxr = dx + static_cast<size_t>(row) * cols;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {               // second pass: the row is still in L1
      const int c = lane * 8 + j * 256;
      if (c < cols) {
        float xv[8], dv[8], wv[8], o[8];
        ln_ld8(xr + c, xv); ln_ld8(dyr + c, dv);
        if (w) ln_ld8(w + c, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float h = (xv[i] - mu) * rs;
          const float g = w ? dv[i] * wv[i] : dv[i];
          o[i] = (g - h * c1 - c2) * rs;
        }
        ln_st8(dxr + c, o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = lane * 8 + j * 256;
    if (c < cols) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { atomicAdd(&ln_s[c + i], dwr[j][i]); atomicAdd(&ln_s[cols + c + i], dbr[j][i]); }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * cols; c += blockDim.x) part[static_cast<size_t>(blockIdx.x) * 2 * cols + c] = ln_s[c];
}

__global__ void __launch_bounds__(1024) layernorm_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, float* __restrict__ db,
                                                                int n, int cols) {
  const float t = column_sum_block(part, n, 2 * cols);
  const int c = blockIdx.x * 32 + threadIdx.x;
  if (threadIdx.x < 32 && c < 2 * cols) { if (c < cols) dw[c] = t; else db[c - cols] = t; }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_layernorm_bwd_partials(int rows) {
  const int need = (rows + 7) / 8;
  return need < LN_BWD_CTAS ? need : LN_BWD_CTAS;
}

// x, y: [rows, cols] bf16 (dtype 1) or fp32 (0); w, bias: fp32 [cols] or null; mean, rstd: fp32 [rows]
extern "C" int b200_layernorm_fwd(const void* x, int dtype, const float* w, const float* bias, void* y, float* mean, float* rstd,
                                  int rows, int cols, float eps, cudaStream_t st) {
  if (rows == 0) return 0;
  if (cols % 8) return -1;
  const int grid = (rows + 7) / 8;
  if (dtype == 1) layernorm_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, w, bias, (__nv_bfloat16*)y, mean, rstd, rows, cols, eps);
  else layernorm_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x, w, bias, (float*)y, mean, rstd, rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// part: fp32 scratch [b200_layernorm_bwd_partials(rows), 2, cols]; dw, db: fp32 [cols]
extern "C" int b200_layernorm_bwd(const void* dy, const void* x, int dtype, const float* w, const float* mean, const float* rstd,
                                  void* dx, float* part, float* dw, float* db, int rows, int cols, cudaStream_t st) {
  if (rows == 0) return 0;
  if (cols % 8 || cols > LN_MAX_CHUNKS * 256) return -1;
  const int grid = b200_layernorm_bwd_partials(rows);
  const int nch = (cols + 255) / 256;
  const size_t smem = sizeof(float) * 2 * cols;
#define LN_L(T, N) layernorm_bwd_kernel<T, N><<<grid, 256, smem, st>>>((const T*)dy, (const T*)x, w, mean, rstd, (T*)dx, part, rows, cols)
#define LN_D(N) { if (dtype == 1) LN_L(__nv_bfloat16, N); else LN_L(float, N); }
  if (nch <= 4) LN_D(4) else if (nch <= 8) LN_D(8) else LN_D(10)
#undef LN_D
#undef LN_L
  layernorm_reduce_kernel<<<(2 * cols + 31) / 32, 1024, 0, st>>>(part, dw, db, grid, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
