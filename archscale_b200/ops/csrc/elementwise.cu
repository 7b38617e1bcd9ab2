// SwiGLU forward / backward on bf16 with fp32 math; 16-byte vector accesses.
// The packed variants read the gate and up halves of a [rows, 2I] GEMM output in place.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]); u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// g, u at g_ptr + row*g_stride + c ; y at row*I + c   (plain variant: rows = n/8 "rows" of 8 with strides 8)
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                                         __nv_bfloat16* __restrict__ y, int64_t rows, int I, int64_t in_stride) {
  const int vec_per_row = I / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row; const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float gv[8], uv[8], o[8];
    ld8(g + r * in_stride + c, gv); ld8(u + r * in_stride + c, uv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gv[e] * sigmoidf_(gv[e]) * uv[e];
    st8(y + r * I + c, o);
  }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                                         const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dg,
                                                         __nv_bfloat16* __restrict__ du, int64_t rows, int I, int64_t in_stride) {
  const int vec_per_row = I / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row; const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float gv[8], uv[8], dv[8], og[8], ou[8];
    ld8(g + r * in_stride + c, gv); ld8(u + r * in_stride + c, uv); ld8(dy + r * I + c, dv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float s = sigmoidf_(gv[e]);
      og[e] = dv[e] * uv[e] * s * (1.f + gv[e] * (1.f - s));
      ou[e] = dv[e] * gv[e] * s;
    }
    st8(dg + r * in_stride + c, og); st8(du + r * in_stride + c, ou);
  }
}

static inline int ew_grid(int64_t vecs) {
  int64_t b = (vecs + 255) / 256;
  const int64_t cap = 148 * 16;
  return static_cast<int>(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace b200

using namespace b200;
typedef __nv_bfloat16 bf16;

extern "C" int b200_swiglu_fwd(const void* g, const void* u, void* y, int64_t n, cudaStream_t s) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(n / 8), 256, 0, s>>>((const bf16*)g, (const bf16*)u, (bf16*)y, n / 8, 8, 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_swiglu_bwd(const void* g, const void* u, const void* dy, void* dg, void* du, int64_t n, cudaStream_t s) {
  if (n % 8) return -1;
  if (n == 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(n / 8), 256, 0, s>>>((const bf16*)g, (const bf16*)u, (const bf16*)dy, (bf16*)dg, (bf16*)du, n / 8, 8, 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_swiglu_packed_fwd(const void* x, void* y, int64_t rows, int I, cudaStream_t s) {
  if (I % 8) return -1;
  if (rows == 0) return 0;
  const bf16* xp = (const bf16*)x;
  swiglu_fwd_kernel<<<ew_grid(rows * (I / 8)), 256, 0, s>>>(xp, xp + I, (bf16*)y, rows, I, 2 * (int64_t)I);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_swiglu_packed_bwd(const void* x, const void* dy, void* dx, int64_t rows, int I, cudaStream_t s) {
  if (I % 8) return -1;
  if (rows == 0) return 0;
  const bf16* xp = (const bf16*)x; bf16* dxp = (bf16*)dx;
  swiglu_bwd_kernel<<<ew_grid(rows * (I / 8)), 256, 0, s>>>(xp, xp + I, (const bf16*)dy, dxp, dxp + I, rows, I, 2 * (int64_t)I);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
