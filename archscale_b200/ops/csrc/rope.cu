// Fused per-head RMSNorm (QK-norm) + rotary embedding (NeoX halves) for q:[N,H,D] and k:[N,G,D], bf16.
// One warp per (token, head) row; D ∈ {64, 128} so a lane owns D/32 contiguous elements and its
// rotation partner (i ± D/2) lives in lane ^ 16.  Statistics and rotation in fp32.
// Backward undoes the rotation (conjugate), then applies the RMSNorm backward; the weight gradient
// is accumulated per warp in registers, per CTA in shared memory and written as per-CTA partials
// (deterministic two-stage reduction).
#include "sm100.cuh"
#include "api.h"

namespace b200 {

template <int EPL> __device__ __forceinline__ void ld_row(const __nv_bfloat16* p, float (&v)[EPL]);
template <> __device__ __forceinline__ void ld_row<4>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <> __device__ __forceinline__ void ld_row<2>(const __nv_bfloat16* p, float (&v)[2]) {
  const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p));
  v[0] = a.x; v[1] = a.y;
}
template <int EPL> __device__ __forceinline__ void st_row(__nv_bfloat16* p, const float (&v)[EPL]);
template <> __device__ __forceinline__ void st_row<4>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 u; u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = u;
}
template <> __device__ __forceinline__ void st_row<2>(__nv_bfloat16* p, const float (&v)[2]) {
  *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(v[0], v[1]);
}
template <typename TW> __device__ __forceinline__ float ldw(const TW* w, int i);
template <> __device__ __forceinline__ float ldw<float>(const float* w, int i) { return w[i]; }
template <> __device__ __forceinline__ float ldw<__nv_bfloat16>(const __nv_bfloat16* w, int i) { return __bfloat162float(w[i]); }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int EPL, typename TW>
__global__ void __launch_bounds__(256) qknorm_rope_fwd_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const TW* __restrict__ qw,
    const TW* __restrict__ kw, const __nv_bfloat16* __restrict__ cosb, const __nv_bfloat16* __restrict__ sinb,
    __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko, float* __restrict__ q_rstd,
    float* __restrict__ k_rstd, int64_t n_tokens, int T, int H, int G, float eps, int64_t q_ts, int64_t k_ts) {
  constexpr int D = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t q_rows = n_tokens * H, rows = q_rows + n_tokens * G;
  for (int64_t r = warp_global; r < rows; r += n_warps) {
    const bool is_q = r < q_rows;
    const int64_t rr = is_q ? r : r - q_rows;
    const int heads = is_q ? H : G;
    const int64_t tok = rr / heads;
    // inputs may be column slices of a wider (fused projection) matrix: token stride q_ts / k_ts elements
    const __nv_bfloat16* src = (is_q ? q + tok * q_ts : k + tok * k_ts) + (rr - tok * heads) * D + lane * EPL;
    __nv_bfloat16* dst = (is_q ? qo : ko) + rr * D + lane * EPL;
    const TW* w = is_q ? qw : kw;
    float x[EPL];
    ld_row<EPL>(src, x);
    if (w) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) ss += x[e] * x[e];
      ss = wsum(ss);
      const float rs = rsqrtf(ss / D + eps);
      if (lane == 0) (is_q ? q_rstd : k_rstd)[rr] = rs;
#pragma unroll
      for (int e = 0; e < EPL; ++e) x[e] = x[e] * rs * ldw<TW>(w, lane * EPL + e);
    }
    if (cosb) {
      const int t = static_cast<int>(tok % T);
      const int ci = (lane & 15) * EPL;
      float o[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
        const float c = __bfloat162float(cosb[static_cast<size_t>(t) * (D / 2) + ci + e]);
        const float s = __bfloat162float(sinb[static_cast<size_t>(t) * (D / 2) + ci + e]);
        o[e] = lane < 16 ? x[e] * c - other * s : other * s + x[e] * c;
      }
      st_row<EPL>(dst, o);
    } else {
      st_row<EPL>(dst, x);
    }
  }
}

template <int EPL, typename TW>
__global__ void __launch_bounds__(256) qknorm_rope_bwd_kernel(
    const __nv_bfloat16* __restrict__ dqo, const __nv_bfloat16* __restrict__ dko, const __nv_bfloat16* __restrict__ q,
    const __nv_bfloat16* __restrict__ k, const TW* __restrict__ qw, const TW* __restrict__ kw,
    const __nv_bfloat16* __restrict__ cosb, const __nv_bfloat16* __restrict__ sinb, const float* __restrict__ q_rstd,
    const float* __restrict__ k_rstd, __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk,
    float* __restrict__ dw_partial /* [grid, 2, D] */, int64_t n_tokens, int T, int H, int G, int64_t q_ts, int64_t k_ts) {
  constexpr int D = EPL * 32;
  __shared__ float dw_s[2][D];
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&dw_s[0][0])[i] = 0.f;
  __syncthreads();
  const int64_t warp_global = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t q_rows = n_tokens * H, rows = q_rows + n_tokens * G;
  float dwq[EPL], dwk[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) dwq[e] = dwk[e] = 0.f;
  for (int64_t r = warp_global; r < rows; r += n_warps) {
    const bool is_q = r < q_rows;
    const int64_t rr = is_q ? r : r - q_rows;
    const int heads = is_q ? H : G;
    const int64_t tok = rr / heads;
    const size_t off = rr * D + lane * EPL;
    float g[EPL];
    ld_row<EPL>((is_q ? dqo : dko) + off, g);
    if (cosb) {
      const int t = static_cast<int>(tok % T);
      const int ci = (lane & 15) * EPL;
      float o[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, g[e], 16);
        const float c = __bfloat162float(cosb[static_cast<size_t>(t) * (D / 2) + ci + e]);
        const float s = __bfloat162float(sinb[static_cast<size_t>(t) * (D / 2) + ci + e]);
        o[e] = lane < 16 ? g[e] * c + other * s : -other * s + g[e] * c;
      }
#pragma unroll
      for (int e = 0; e < EPL; ++e) g[e] = o[e];
    }
    const TW* w = is_q ? qw : kw;
    if (w) {
      float x[EPL];
      ld_row<EPL>((is_q ? q + tok * q_ts : k + tok * k_ts) + (rr - tok * heads) * D + lane * EPL, x);
      const float rs = (is_q ? q_rstd : k_rstd)[rr];
      float dot = 0.f;
      float gw[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        gw[e] = g[e] * ldw<TW>(w, lane * EPL + e);
        dot += gw[e] * x[e];
        if (is_q) dwq[e] += g[e] * x[e] * rs; else dwk[e] += g[e] * x[e] * rs;
      }
      dot = wsum(dot);
      const float c1 = dot * rs * rs * rs / D;
#pragma unroll
      for (int e = 0; e < EPL; ++e) g[e] = gw[e] * rs - x[e] * c1;
    }
    st_row<EPL>((is_q ? dq : dk) + off, g);
  }
  if (qw) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      atomicAdd(&dw_s[0][lane * EPL + e], dwq[e]);
      atomicAdd(&dw_s[1][lane * EPL + e], dwk[e]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x)
      dw_partial[static_cast<size_t>(blockIdx.x) * 2 * D + i] = (&dw_s[0][0])[i];
  }
}

__global__ void qk_dw_reduce_kernel(const float* __restrict__ part, float* __restrict__ dqw, float* __restrict__ dkw, int n, int D) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * D) return;
  float s = 0.f;
  for (int b = 0; b < n; ++b) s += part[static_cast<size_t>(b) * 2 * D + i];
  if (i < D) dqw[i] = s; else dkw[i - D] = s;
}

constexpr int kRopeGrid = 148 * 8;

}  // namespace b200

using namespace b200;
typedef __nv_bfloat16 bf16;

extern "C" int b200_qknorm_rope_grid() { return kRopeGrid; }

extern "C" int b200_qknorm_rope_fwd(const void* q, const void* k, const void* qw, const void* kw, int w_dtype,
                                    const void* cos, const void* sin, void* qo, void* ko, float* q_rstd, float* k_rstd,
                                    int64_t n_tokens, int T, int H, int G, int D, float eps, int64_t q_ts, int64_t k_ts, cudaStream_t st) {
  if (n_tokens == 0) return 0;
#define LAUNCH(EPL, TW)                                                                                               \
  qknorm_rope_fwd_kernel<EPL, TW><<<kRopeGrid, 256, 0, st>>>((const bf16*)q, (const bf16*)k, (const TW*)qw, (const TW*)kw, \
                                                             (const bf16*)cos, (const bf16*)sin, (bf16*)qo, (bf16*)ko,  \
                                                             q_rstd, k_rstd, n_tokens, T, H, G, eps, q_ts, k_ts)
  if (D == 128) { if (w_dtype == 1) LAUNCH(4, bf16); else LAUNCH(4, float); }
  else if (D == 64) { if (w_dtype == 1) LAUNCH(2, bf16); else LAUNCH(2, float); }
  else return -1;
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_qknorm_rope_bwd(const void* dqo, const void* dko, const void* q, const void* k, const void* qw,
                                     const void* kw, int w_dtype, const void* cos, const void* sin, const float* q_rstd,
                                     const float* k_rstd, void* dq, void* dk, float* dqw, float* dkw, float* dw_partial,
                                     int64_t n_tokens, int T, int H, int G, int D, int64_t q_ts, int64_t k_ts, cudaStream_t st) {
  if (n_tokens == 0) return 0;
#define LAUNCH(EPL, TW)                                                                                                \
  qknorm_rope_bwd_kernel<EPL, TW><<<kRopeGrid, 256, 0, st>>>((const bf16*)dqo, (const bf16*)dko, (const bf16*)q, (const bf16*)k, \
                                                             (const TW*)qw, (const TW*)kw, (const bf16*)cos, (const bf16*)sin,  \
                                                             q_rstd, k_rstd, (bf16*)dq, (bf16*)dk, dw_partial, n_tokens, T, H, G, q_ts, k_ts)
  if (D == 128) { if (w_dtype == 1) LAUNCH(4, bf16); else LAUNCH(4, float); }
  else if (D == 64) { if (w_dtype == 1) LAUNCH(2, bf16); else LAUNCH(2, float); }
  else return -1;
#undef LAUNCH
  if (qw) qk_dw_reduce_kernel<<<(2 * D + 127) / 128, 128, 0, st>>>(dw_partial, dqw, dkw, kRopeGrid, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
