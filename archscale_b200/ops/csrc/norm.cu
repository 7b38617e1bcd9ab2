// RMSNorm forward / backward.  One warp per row, 16-byte vector loads, fp32 statistics.
// Forward reads the row twice (the second pass hits L1) so any row length works without keeping the
// row in registers.  Backward is persistent: each CTA walks a strided set of rows, writes dx and
// accumulates dw in shared memory; per-CTA partials are reduced by a second tiny kernel.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]); u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const TX* __restrict__ x, const TW* __restrict__ w,
                                                          TO* __restrict__ out, float* __restrict__ rstd_out, int rows,
                                                          int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const TX* xr = x + static_cast<size_t>(row) * cols;
  float ss = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8]; Vec8<TX>::load(xr + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / cols + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
  TO* orow = out + static_cast<size_t>(row) * cols;
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8]; Vec8<TX>::load(xr + c, v);
    if (w) {
      float g[8]; Vec8<TW>::load(w + c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * g[i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd;
    }
    Vec8<TO>::store(orow + c, v);
  }
}

template <typename TDY, typename TX, typename TW>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const TDY* __restrict__ dy, const TX* __restrict__ x,
                                                          const TW* __restrict__ w, const float* __restrict__ rstd,
                                                          TX* __restrict__ dx, float* __restrict__ dw_partial, int rows,
                                                          int cols) {
  extern __shared__ float dw_s[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (w) { for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_s[c] = 0.f; __syncthreads(); }
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const TX* xr = x + static_cast<size_t>(row) * cols;
    const TDY* dyr = dy + static_cast<size_t>(row) * cols;
    const float rs = rstd[row];
    float dot = 0.f;
    for (int c = lane * 8; c < cols; c += 256) {
      float xv[8], dv[8]; Vec8<TX>::load(xr + c, xv); Vec8<TDY>::load(dyr + c, dv);
      if (w) {
        float g[8]; Vec8<TW>::load(w + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += dv[i] * g[i] * xv[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += dv[i] * xv[i];
      }
    }
    dot = warp_sum(dot);
    const float c1 = dot * rs * rs * rs / cols;   // mean(dy·w·x̂)·rstd, with x̂ = x·rstd
    TX* dxr = dx + static_cast<size_t>(row) * cols;
    for (int c = lane * 8; c < cols; c += 256) {
      float xv[8], dv[8], o[8]; Vec8<TX>::load(xr + c, xv); Vec8<TDY>::load(dyr + c, dv);
      if (w) {
        float g[8]; Vec8<TW>::load(w + c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[i] = dv[i] * g[i] * rs - xv[i] * c1;
          atomicAdd(&dw_s[c + i], dv[i] * xv[i] * rs);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = dv[i] * rs - xv[i] * c1;
      }
      Vec8<TX>::store(dxr + c, o);
    }
  }
  if (w) {
    __syncthreads();
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_partial[static_cast<size_t>(blockIdx.x) * cols + c] = dw_s[c];
  }
}

__global__ void __launch_bounds__(1024) reduce_partials_kernel(const float* __restrict__ part, float* __restrict__ out, int n, int cols) {
  const float t = column_sum_block(part, n, cols);
  const int c = blockIdx.x * 32 + threadIdx.x;
  if (threadIdx.x < 32 && c < cols) out[c] = t;
}


// ---------------------------------------------------------------------------------------------
// Fused residual-add + RMSNorm (pre-norm transformer block):
//   x = res + h_scale·h  (written back as the new residual stream, fp32 or bf16)   n = rmsnorm(x)·w  (bf16)
// With a bf16 stream the sum is rounded to bf16 before it is normalised, so that forward and backward see the same x.
// Backward in one pass: d_res = g_res + rmsnorm_bwd(g_n),  d_h = bf16(h_scale·d_res); the weight
// gradient is accumulated in registers (a lane owns columns lane·8 + 256·i), then per CTA in shared
// memory, then written as per-CTA partials.
template <typename TRES, typename TW, bool HAS_H, typename TOUT = float>
__global__ void __launch_bounds__(256) add_rmsnorm_fwd_kernel(const TRES* __restrict__ res, const __nv_bfloat16* __restrict__ h,
                                                              float h_scale, const TW* __restrict__ w, TOUT* __restrict__ res_out,
                                                              __nv_bfloat16* __restrict__ n_out, float* __restrict__ rstd_out,
                                                              int rows, int cols, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + warp;
  if (row >= rows) return;
  const size_t base = static_cast<size_t>(row) * cols;
  float ss = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8]; Vec8<TRES>::load(res + base + c, v);
    if (HAS_H) {
      float hv[8]; Vec8<__nv_bfloat16>::load(h + base + c, hv);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += h_scale * hv[i];
      Vec8<TOUT>::store(res_out + base + c, v);
      if (sizeof(TOUT) == 2) Vec8<TOUT>::load(res_out + base + c, v);      // the rounded values (L1 hit)
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / cols + eps);
  if (lane == 0) rstd_out[row] = rstd;
  for (int c = lane * 8; c < cols; c += 256) {
    float v[8];
    if (HAS_H) Vec8<TOUT>::load(res_out + base + c, v);   // just written by this lane (L1 hit)
    else Vec8<TRES>::load(res + base + c, v);
    float g[8]; Vec8<TW>::load(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * g[i];
    Vec8<__nv_bfloat16>::store(n_out + base + c, v);
  }
}

// cols ≤ NCH·256, a multiple of 8: a lane owns the 8-element vectors at columns lane·8 + i·256 (i < NCH) that lie inside the
// row; widths that are not a multiple of 256 (1984, 1536, …) leave the last chunk partly or wholly empty.
// FULL: cols == NCH·256, no bounds checks (they cost the common widths ≈ 40 % when left in).
// TG: type of the residual-stream gradient in and out (fp32, or bf16 for a bf16 stream).
template <typename TX, typename TW, int NCH, bool FULL, typename TG = float>
__global__ void __launch_bounds__(256) add_rmsnorm_bwd_kernel(const TG* __restrict__ g_res, const __nv_bfloat16* __restrict__ g_n,
                                                              const TX* __restrict__ x, const TW* __restrict__ w,
                                                              const float* __restrict__ rstd, TG* __restrict__ d_res,
                                                              __nv_bfloat16* __restrict__ d_h, float h_scale,
                                                              float* __restrict__ dw_partial, int rows, int cols) {
  extern __shared__ float dw_s[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_s[c] = 0.f;
  __syncthreads();
  float dwacc[NCH][8];
#pragma unroll
  for (int i = 0; i < NCH; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
  float wreg[NCH][8];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    if (FULL || lane * 8 + i * 256 < cols) Vec8<TW>::load(w + lane * 8 + i * 256, wreg[i]);
    else {
#pragma unroll
      for (int e = 0; e < 8; ++e) wreg[i][e] = 0.f;
    }
  }
  // Partial rows: a chunk that lies beyond the row loads from the row's last vector instead (always in bounds, no branch
  // around the loads, so the compiler still issues all of a row's loads together) and its gradient vector is zeroed.
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const size_t base = static_cast<size_t>(row) * cols;
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane * 8 + i * 256;
      const bool valid = FULL || c < cols;
      const int cl = FULL ? c : min(c, cols - 8);
      float xv[8], dv[8]; Vec8<TX>::load(x + base + cl, xv); Vec8<__nv_bfloat16>::load(g_n + base + cl, dv);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += valid ? dv[e] * wreg[i][e] * xv[e] : 0.f;
    }
    dot = warp_sum(dot);
    const float c1 = dot * rs * rs * rs / cols;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = lane * 8 + i * 256;
      const bool valid = FULL || c < cols;
      const int cl = FULL ? c : min(c, cols - 8);
      float xv[8], dv[8], o[8]; Vec8<TX>::load(x + base + cl, xv); Vec8<__nv_bfloat16>::load(g_n + base + cl, dv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[e] = dv[e] * wreg[i][e] * rs - xv[e] * c1;
        dwacc[i][e] += valid ? dv[e] * xv[e] * rs : 0.f;
      }
      if (g_res) {
        float gr[8]; Vec8<TG>::load(g_res + base + cl, gr);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += gr[e];
      }
      if (valid) {
        if (d_res) Vec8<TG>::store(d_res + base + c, o);
        if (d_h) {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] *= h_scale;
          Vec8<__nv_bfloat16>::store(d_h + base + c, o);
        }
      }
    }
  }
  // the eight warps add their sums in turn (a lane owns its columns within a warp): a fixed order, so that the weight
  // gradient repeats bit for bit from run to run, which shared-memory atomics would not give
  for (int turn = 0; turn < 8; ++turn) {
    if (warp == turn) {
#pragma unroll
      for (int i = 0; i < NCH; ++i)
        if (FULL || lane * 8 + i * 256 < cols) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dw_s[lane * 8 + i * 256 + e] += dwacc[i][e];
        }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_partial[static_cast<size_t>(blockIdx.x) * cols + c] = dw_s[c];
}

// The same backward with every row split over a PAIR of warps (cols == NCH·256, NCH even): a lane keeps NCH/2 chunks of the
// weight-gradient accumulator instead of NCH and reads the weight from shared memory, which brings the kernel under 128
// registers and two CTAs onto an SM (the one-warp-per-row form needs 255 registers at 2048 columns).  The two partial dot products of a row meet
// in shared memory behind a 64-thread named barrier; two buffers alternate so that one barrier per row suffices.
template <typename TX, typename TW, int NCH, typename TG>
__global__ void __launch_bounds__(256, 2) add_rmsnorm_bwd2_kernel(const TG* __restrict__ g_res, const __nv_bfloat16* __restrict__ g_n,
                                                                 const TX* __restrict__ x, const TW* __restrict__ w,
                                                                 const float* __restrict__ rstd, TG* __restrict__ d_res,
                                                                 __nv_bfloat16* __restrict__ d_h, float h_scale,
                                                                 float* __restrict__ dw_partial, int rows, int cols) {
  extern __shared__ float dw_s[];                                       // [cols] weight-gradient sums, then [cols] the weight in fp32
  __shared__ float dot_s[2][8];
  constexpr int NCL = NCH / 2;
  float* w_s = dw_s + cols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = warp >> 1, half = warp & 1;
  const int c0 = lane * 8 + half * NCL * 256;                           // first column of this lane
  for (int c = threadIdx.x * 8; c < cols; c += blockDim.x * 8) {
    float t[8]; Vec8<TW>::load(w + c, t);
#pragma unroll
    for (int e = 0; e < 8; ++e) { w_s[c + e] = t[e]; dw_s[c + e] = 0.f; }
  }
  __syncthreads();
  float dwacc[NCL][8];
#pragma unroll
  for (int i = 0; i < NCL; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
  int it = 0;
  for (int row = blockIdx.x * 4 + pair; row < rows; row += gridDim.x * 4, ++it) {
    const size_t base = static_cast<size_t>(row) * cols + c0;
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NCL; ++i) {
      float xv[8], dv[8], wv[8];
      Vec8<TX>::load(x + base + i * 256, xv);
      Vec8<__nv_bfloat16>::load(g_n + base + i * 256, dv);
      Vec8<float>::load(w_s + c0 + i * 256, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += dv[e] * wv[e] * xv[e];
    }
    dot = warp_sum(dot);
    if (lane == 0) dot_s[it & 1][warp] = dot;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    dot = dot_s[it & 1][pair * 2] + dot_s[it & 1][pair * 2 + 1];
    const float c1 = dot * rs * rs * rs / cols;
#pragma unroll
    for (int i = 0; i < NCL; ++i) {
      float xv[8], dv[8], wv[8], o[8];             // second read of the row: L1 / L2 hits
      Vec8<TX>::load(x + base + i * 256, xv);
      Vec8<__nv_bfloat16>::load(g_n + base + i * 256, dv);
      Vec8<float>::load(w_s + c0 + i * 256, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[e] = dv[e] * wv[e] * rs - xv[e] * c1;
        dwacc[i][e] += dv[e] * xv[e] * rs;
      }
      if (g_res) {
        float gr[8]; Vec8<TG>::load(g_res + base + i * 256, gr);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += gr[e];
      }
      if (d_res) Vec8<TG>::store(d_res + base + i * 256, o);
      if (d_h) {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= h_scale;
        Vec8<__nv_bfloat16>::store(d_h + base + i * 256, o);
      }
    }
  }
  for (int turn = 0; turn < 8; ++turn) {            // fixed order of the eight warps: repeatable sums (see above)
    if (warp == turn) {
#pragma unroll
      for (int i = 0; i < NCL; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) dw_s[c0 + i * 256 + e] += dwacc[i][e];
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_partial[static_cast<size_t>(blockIdx.x) * cols + c] = dw_s[c];
}

constexpr int kBwdCtas = 148 * 2;

}  // namespace b200

using namespace b200;

#include <cstdlib>
// ARCHSCALE_B200_NORM_BWD=warp keeps the one-warp-per-row backward for the widths the warp-pair kernel takes.
static bool use_pair_rows() {
  static const bool v = [] { const char* e = std::getenv("ARCHSCALE_B200_NORM_BWD"); return !(e && e[0] == 'w'); }();
  return v;
}

#define DISPATCH_3(xd, wd, od, CALL)                                                           \
  if (xd == 0 && wd == 0 && od == 0) { CALL(float, float, float) }                              \
  else if (xd == 0 && wd == 0 && od == 1) { CALL(float, float, __nv_bfloat16) }                 \
  else if (xd == 0 && wd == 1 && od == 1) { CALL(float, __nv_bfloat16, __nv_bfloat16) }         \
  else if (xd == 0 && wd == 1 && od == 0) { CALL(float, __nv_bfloat16, float) }                 \
  else if (xd == 1 && wd == 1 && od == 1) { CALL(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16) } \
  else if (xd == 1 && wd == 0 && od == 1) { CALL(__nv_bfloat16, float, __nv_bfloat16) }         \
  else if (xd == 1 && wd == 0 && od == 0) { CALL(__nv_bfloat16, float, float) }                 \
  else if (xd == 1 && wd == 1 && od == 0) { CALL(__nv_bfloat16, __nv_bfloat16, float) }         \
  else return -1;

extern "C" int b200_rmsnorm_fwd(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                                float* rstd, int rows, int cols, float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (cols % 8) return -1;
  const int grid = (rows + 7) / 8;
#define CALL(TX, TW, TO)                                                                                          \
  rmsnorm_fwd_kernel<TX, TW, TO><<<grid, 256, 0, stream>>>(static_cast<const TX*>(x), static_cast<const TW*>(w), \
                                                           static_cast<TO*>(out), rstd, rows, cols, eps);
  DISPATCH_3(x_dtype, w_dtype, out_dtype, CALL)
#undef CALL
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_rmsnorm_bwd_partials(int rows, int cols) {
  const int need = (rows + 7) / 8;
  return need < kBwdCtas ? need : kBwdCtas;
}

extern "C" int b200_add_rmsnorm_bwd(const void* g_res, const void* g_n, const void* x, int x_dtype, const void* w, int w_dtype,
                                    const float* rstd, void* d_res, void* d_h, float h_scale, float* dw_partial, float* dw,
                                    int rows, int cols, cudaStream_t stream, int g_dtype);

extern "C" int b200_rmsnorm_bwd(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* w, int w_dtype,
                                const float* rstd, void* dx, float* dw_partial, float* dw, int rows, int cols,
                                cudaStream_t stream) {
  if (rows == 0) return 0;
  if (cols % 8) return -1;
  // bf16 upstream gradient, a weight and one of the model widths: the kernel of the fused residual-add variant (weight
  // gradient accumulated in registers, one shared-memory add per column and CTA instead of one per element) does this job
  // with no residual gradient: dx is its bf16 output for bf16 x, its fp32 output for fp32 x
  if (dy_dtype == 1 && w && cols >= 512 && cols <= 4096)
    return b200_add_rmsnorm_bwd(nullptr, dy, x, x_dtype, w, w_dtype, rstd, x_dtype == 0 ? dx : nullptr,
                                x_dtype == 1 ? dx : nullptr, 1.f, dw_partial, dw, rows, cols, stream, 0);
  const int grid = b200_rmsnorm_bwd_partials(rows, cols);
  const size_t smem = w ? sizeof(float) * cols : 0;
#define CALL(TDY, TW, TX)                                                                                     \
  {                                                                                                           \
    auto kern = rmsnorm_bwd_kernel<TDY, TX, TW>;                                                              \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    kern<<<grid, 256, smem, stream>>>(static_cast<const TDY*>(dy), static_cast<const TX*>(x),                \
                                      static_cast<const TW*>(w), rstd, static_cast<TX*>(dx), dw_partial, rows, cols); \
  }
  DISPATCH_3(dy_dtype, w_dtype, x_dtype, CALL)
#undef CALL
  if (w) reduce_partials_kernel<<<(cols + 31) / 32, 1024, 0, stream>>>(dw_partial, dw, grid, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// out_dtype: type of the new residual stream res_out (0 fp32, 1 bf16; a bf16 stream needs bf16 res).
extern "C" int b200_add_rmsnorm_fwd(const void* res, int res_dtype, const void* h, float h_scale, const void* w, int w_dtype,
                                    void* res_out, void* n_out, float* rstd, int rows, int cols, float eps,
                                    cudaStream_t stream, int out_dtype) {
  if (rows == 0) return 0;
  if (cols % 8) return -1;
  const int grid = (rows + 7) / 8;
  typedef __nv_bfloat16 bf;
  if (out_dtype == 1) {
    if (res_dtype != 1) return -1;
#define LB(TW, HH)                                                                                                    \
  add_rmsnorm_fwd_kernel<bf, TW, HH, bf><<<grid, 256, 0, stream>>>(static_cast<const bf*>(res), static_cast<const bf*>(h), \
                                                                   h_scale, static_cast<const TW*>(w), static_cast<bf*>(res_out), \
                                                                   static_cast<bf*>(n_out), rstd, rows, cols, eps)
    if (h) { if (w_dtype == 0) LB(float, true); else LB(bf, true); }
    else { if (w_dtype == 0) LB(float, false); else LB(bf, false); }
#undef LB
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
#define L(TRES, TW, HH)                                                                                              \
  add_rmsnorm_fwd_kernel<TRES, TW, HH><<<grid, 256, 0, stream>>>(static_cast<const TRES*>(res), static_cast<const bf*>(h), \
                                                                 h_scale, static_cast<const TW*>(w), static_cast<float*>(res_out), \
                                                                 static_cast<bf*>(n_out), rstd, rows, cols, eps)
  if (h) {
    if (res_dtype == 0 && w_dtype == 0) L(float, float, true);
    else if (res_dtype == 0 && w_dtype == 1) L(float, bf, true);
    else if (res_dtype == 1 && w_dtype == 0) L(bf, float, true);
    else L(bf, bf, true);
  } else {
    if (res_dtype == 0 && w_dtype == 0) L(float, float, false);
    else if (res_dtype == 0 && w_dtype == 1) L(float, bf, false);
    else if (res_dtype == 1 && w_dtype == 0) L(bf, float, false);
    else L(bf, bf, false);
  }
#undef L
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// cols: a multiple of 8 up to 4096 (register-resident dw accumulators); returns -2 otherwise.
// g_dtype: type of g_res and d_res (0 fp32, 1 bf16; bf16 gradients need bf16 x).
extern "C" int b200_add_rmsnorm_bwd(const void* g_res, const void* g_n, const void* x, int x_dtype, const void* w, int w_dtype,
                                    const float* rstd, void* d_res, void* d_h, float h_scale, float* dw_partial, float* dw,
                                    int rows, int cols, cudaStream_t stream, int g_dtype) {
  if (rows == 0) return 0;
  if (g_dtype == 1 && x_dtype != 1) return -1;
  const int grid = b200_rmsnorm_bwd_partials(rows, cols);
  const size_t smem = sizeof(float) * cols;
  typedef __nv_bfloat16 bf;
#define L(TX, TW, NCH, TG)                                                                                             \
  do {                                                                                                                 \
    if (cols == NCH * 256)                                                                                             \
      add_rmsnorm_bwd_kernel<TX, TW, NCH, true, TG><<<grid, 256, smem, stream>>>(                                      \
          static_cast<const TG*>(g_res), static_cast<const bf*>(g_n), static_cast<const TX*>(x), static_cast<const TW*>(w), rstd, \
          static_cast<TG*>(d_res), static_cast<bf*>(d_h), h_scale, dw_partial, rows, cols);                            \
    else                                                                                                               \
      add_rmsnorm_bwd_kernel<TX, TW, NCH, false, TG><<<grid, 256, smem, stream>>>(                                     \
          static_cast<const TG*>(g_res), static_cast<const bf*>(g_n), static_cast<const TX*>(x), static_cast<const TW*>(w), rstd, \
          static_cast<TG*>(d_res), static_cast<bf*>(d_h), h_scale, dw_partial, rows, cols);                            \
  } while (0)
#define LN(NCH)                                                         \
  if (g_dtype == 1 && w_dtype == 0) L(bf, float, NCH, bf);              \
  else if (g_dtype == 1) L(bf, bf, NCH, bf);                            \
  else if (x_dtype == 0 && w_dtype == 0) L(float, float, NCH, float);   \
  else if (x_dtype == 0 && w_dtype == 1) L(float, bf, NCH, float);      \
  else if (x_dtype == 1 && w_dtype == 0) L(bf, float, NCH, float);      \
  else L(bf, bf, NCH, float);
  // the instantiation with the fewest 256-column chunks that covers the row (the kernel skips what lies beyond `cols`)
  if (cols % 8 || cols > 4096) return -2;
  if (use_pair_rows() && cols == 2048) {      // wider rows spill at 128 registers; 1024-wide rows measured no faster this way
#define L2(TX, TW, NCH, TG)                                                                                            \
  add_rmsnorm_bwd2_kernel<TX, TW, NCH, TG><<<grid, 256, 2 * smem, stream>>>(                                               \
      static_cast<const TG*>(g_res), static_cast<const bf*>(g_n), static_cast<const TX*>(x), static_cast<const TW*>(w), rstd, \
      static_cast<TG*>(d_res), static_cast<bf*>(d_h), h_scale, dw_partial, rows, cols)
#define LN2(NCH)                                                         \
  if (g_dtype == 1 && w_dtype == 0) L2(bf, float, NCH, bf);              \
  else if (g_dtype == 1) L2(bf, bf, NCH, bf);                            \
  else if (x_dtype == 0 && w_dtype == 0) L2(float, float, NCH, float);   \
  else if (x_dtype == 0 && w_dtype == 1) L2(float, bf, NCH, float);      \
  else if (x_dtype == 1 && w_dtype == 0) L2(bf, float, NCH, float);      \
  else L2(bf, bf, NCH, float);
    LN2(8)
#undef LN2
#undef L2
    reduce_partials_kernel<<<(cols + 31) / 32, 1024, 0, stream>>>(dw_partial, dw, grid, cols);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
  if (cols <= 1024) { LN(4) }
  else if (cols <= 2048) { LN(8) }
  else if (cols <= 2560) { LN(10) }
  else if (cols <= 3072) { LN(12) }
  else { LN(16) }
#undef LN
#undef L
  reduce_partials_kernel<<<(cols + 31) / 32, 1024, 0, stream>>>(dw_partial, dw, grid, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
