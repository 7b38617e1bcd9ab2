// Gated RMSNorm with groups (Mamba-2, Gated DeltaNet, GMU with a norm):
//   norm_before_gate:   y = (x · rstd_g · w) · silu(z)          rstd_g over the group's columns of x
//   otherwise:          y = (x·silu(z)) · rstd_g · w            rstd_g over the group's columns of x·silu(z)
// Forward: one warp per (row, group).  Backward: a CTA works on one group (its 8 warps stride the rows), so the weight
// gradient of the group's columns is accumulated in shared memory and flushed with one atomic per column per CTA.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

template <typename T> __device__ __forceinline__ void gn_ld8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void gn_ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void gn_ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void gn_st8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void gn_st8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void gn_st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]); u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float gn_wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float gn_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gn_dsilu(float x) { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f + x * (1.f - s)); }

template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ z, const float* __restrict__ w,
                                                                T* __restrict__ y, float* __restrict__ rstd, long long rows, int cols,
                                                                int gsize, float eps, int nbg) {
  const int lane = threadIdx.x & 31;
  const int ngroups = cols / gsize;
  const long long unit = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;     // (row, group)
  if (unit >= rows * ngroups) return;
  const long long row = unit / ngroups;
  const int g0 = static_cast<int>(unit - row * ngroups) * gsize;
  const T* xr = x + row * cols + g0;
  const T* zr = z ? z + row * cols + g0 : nullptr;
  float ss = 0.f;
  for (int c = lane * 8; c < gsize; c += 256) {
    float xv[8]; gn_ld8(xr + c, xv);
    if (zr && !nbg) {
      float zv[8]; gn_ld8(zr + c, zv);
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] *= gn_silu(zv[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += xv[i] * xv[i];
  }
  const float rs = rsqrtf(gn_wsum(ss) / gsize + eps);
  if (lane == 0) rstd[unit] = rs;
  T* yr = y + row * cols + g0;
  for (int c = lane * 8; c < gsize; c += 256) {
    float xv[8], wv[8], zv[8];
    gn_ld8(xr + c, xv); gn_ld8(w + g0 + c, wv);
    if (zr) gn_ld8(zr + c, zv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = zr ? gn_silu(zv[i]) : 1.f;
      xv[i] = xv[i] * s * rs * wv[i];             // same product either way; only what rstd was measured on differs
    }
    gn_st8(yr + c, xv);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gated_rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ z,
                                                                const float* __restrict__ w, const float* __restrict__ rstd,
                                                                T* __restrict__ dx, T* __restrict__ dz, float* __restrict__ dw,
                                                                long long rows, int cols, int gsize, int nbg) {
  extern __shared__ float gn_dw[];                 // [gsize]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ngroups = cols / gsize;
  const int grp = blockIdx.x % ngroups;
  const int g0 = grp * gsize;
  const int ctas_per_group = gridDim.x / ngroups;  // host launches a multiple of ngroups
  const int cta_in_group = blockIdx.x / ngroups;
  for (int c = threadIdx.x; c < gsize; c += blockDim.x) gn_dw[c] = 0.f;
  __syncthreads();
  for (long long row = static_cast<long long>(cta_in_group) * 8 + warp; row < rows; row += static_cast<long long>(ctas_per_group) * 8) {
    const T* xr = x + row * cols + g0;
    const T* zr = z ? z + row * cols + g0 : nullptr;
    const T* dyr = dy + row * cols + g0;
    const float rs = rstd[row * ngroups + grp];
    float dot = 0.f;                               // Σ gw · xin  (xin = what was normalised)
    for (int c = lane * 8; c < gsize; c += 256) {
      float xv[8], dv[8], wv[8], zv[8];
      gn_ld8(xr + c, xv); gn_ld8(dyr + c, dv); gn_ld8(w + g0 + c, wv);
      if (zr) gn_ld8(zr + c, zv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float s = zr ? gn_silu(zv[i]) : 1.f;
        const float xin = nbg ? xv[i] : xv[i] * s;
        const float g = nbg ? dv[i] * s : dv[i];
        dot += g * wv[i] * xin;
      }
    }
    const float c1 = gn_wsum(dot) * rs * rs * rs / gsize;
    T* dxr = dx + row * cols + g0;
    T* dzr = dz ? dz + row * cols + g0 : nullptr;
    for (int c = lane * 8; c < gsize; c += 256) {
      float xv[8], dv[8], wv[8], zv[8], ox[8], oz[8];
      gn_ld8(xr + c, xv); gn_ld8(dyr + c, dv); gn_ld8(w + g0 + c, wv);
      if (zr) gn_ld8(zr + c, zv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float s = zr ? gn_silu(zv[i]) : 1.f;
        const float ds = zr ? gn_dsilu(zv[i]) : 0.f;
        const float xin = nbg ? xv[i] : xv[i] * s;
        const float g = nbg ? dv[i] * s : dv[i];
        const float dxin = g * wv[i] * rs - xin * c1;
        atomicAdd(&gn_dw[c + i], g * xin * rs);
        if (nbg) { ox[i] = dxin; oz[i] = dv[i] * (xv[i] * rs * wv[i]) * ds; }
        else { ox[i] = dxin * s; oz[i] = dxin * xv[i] * ds; }
      }
      gn_st8(dxr + c, ox);
      if (dzr) gn_st8(dzr + c, oz);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < gsize; c += blockDim.x) atomicAdd(&dw[g0 + c], gn_dw[c]);
}

}  // namespace b200

using namespace b200;

// x, z, y: [rows, cols] bf16 (1) / fp32 (0); w fp32 [cols]; rstd fp32 [rows · cols/gsize]; gsize % 8 == 0
extern "C" int b200_gated_rmsnorm_fwd(const void* x, const void* z, const float* w, void* y, float* rstd, int dtype, long long rows,
                                      int cols, int gsize, float eps, int norm_before_gate, cudaStream_t st) {
  if (rows == 0) return 0;
  if (gsize % 8 || cols % gsize) return -1;
  const long long units = rows * (cols / gsize);
  const unsigned grid = static_cast<unsigned>((units + 7) / 8);
  if (dtype == 1) gated_rmsnorm_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)z, w, (__nv_bfloat16*)y, rstd, rows, cols, gsize, eps, norm_before_gate);
  else gated_rmsnorm_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (const float*)z, w, (float*)y, rstd, rows, cols, gsize, eps, norm_before_gate);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dw fp32 [cols] must be zero on entry; dz may be null when z is null
extern "C" int b200_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z, const float* w, const float* rstd, void* dx, void* dz,
                                      float* dw, int dtype, long long rows, int cols, int gsize, int norm_before_gate, cudaStream_t st) {
  if (rows == 0) return 0;
  if (gsize % 8 || cols % gsize || gsize > 12288) return -1;
  const int ngroups = cols / gsize;
  int per = (148 * 4 + ngroups - 1) / ngroups;
  const long long need = (rows + 7) / 8;
  if (per > need) per = static_cast<int>(need);
  if (per < 1) per = 1;
  const unsigned grid = static_cast<unsigned>(per * ngroups);
  const size_t smem = sizeof(float) * gsize;
  if (dtype == 1) {
    auto k = gated_rmsnorm_bwd_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<grid, 256, smem, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)z, w, rstd, (__nv_bfloat16*)dx, (__nv_bfloat16*)dz, dw, rows, cols, gsize, norm_before_gate);
  } else {
    auto k = gated_rmsnorm_bwd_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<grid, 256, smem, st>>>((const float*)dy, (const float*)x, (const float*)z, w, rstd, (float*)dx, (float*)dz, dw, rows, cols, gsize, norm_before_gate);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
