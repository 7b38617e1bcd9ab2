// Depthwise causal conv1d (width ≤ 4) + optional SiLU on token-major activations x:[B, L, C] (bf16 or fp32).
//   y[b,t,c] = act( bias[c] + Σ_j w[c,j] · x[b, t-(W-1)+j, c] ),  taps that cross a document boundary
//   (seq_idx[b,t'] != seq_idx[b,t]) or the start of the sequence read 0.
// A thread owns 8 consecutive channels and walks TSTEP time steps with the window in registers, so every
// x element is loaded once (plus a W-1 halo) with 16-byte accesses.
// Backward recomputes the pre-activation, forms g = dy·act'(pre) and accumulates
//   dx[t'] += w[c,j]·g[t] (t' = t-(W-1)+j),  dw[c,j] += g[t]·x[t'],  db[c] += g[t]
// dx is produced gather-style (deterministic); dw/db use fp32 atomics on C·(W+1) addresses.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int CV_TSTEP = 16;

template <typename T> struct V8;
template <> struct V8<float> {
  static __device__ __forceinline__ void ld(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct V8<__nv_bfloat16> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]); u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f + x * (1.f - s)); }

// weights: [C, W] fp32 (converted by the caller), bias: [C] fp32 or null; xs / dys: row strides (elements) of x / dy,
// whose rows may be slices of a wider matrix; y, dx are dense [B, L, C].
template <typename T, int W>
__global__ void __launch_bounds__(128) conv1d_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                         const int* __restrict__ seq_idx, T* __restrict__ y, int B, int L, int C, int silu, int xs) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;       // channel vector index
  const int c0 = cv * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * CV_TSTEP, b = blockIdx.z;
  float wk[W][8], bs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    bs[e] = bias ? bias[c0 + e] : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) wk[j][e] = w[(c0 + e) * W + j];
  }
  const T* xb = x + static_cast<size_t>(b) * L * xs + c0;
  T* yb = y + static_cast<size_t>(b) * L * C + c0;
  const int* sb = seq_idx ? seq_idx + static_cast<size_t>(b) * L : nullptr;
  float win[W][8];           // win[j] = x[t-(W-1)+j]
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {
    const int tt = t0 - (W - 1) + j;
    if (tt >= 0) V8<T>::ld(xb + static_cast<size_t>(tt) * xs, win[j]);
    else {
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = 0.f;
    }
  }
  int sid_hist[W];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) { const int tt = t0 - (W - 1) + j; sid_hist[j] = (sb && tt >= 0) ? sb[tt] : -1; }
  for (int t = t0; t < min(t0 + CV_TSTEP, L); ++t) {
    V8<T>::ld(xb + static_cast<size_t>(t) * xs, win[W - 1]);
    const int sid = sb ? sb[t] : 0;
    sid_hist[W - 1] = sid;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bs[e];
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const bool ok = !sb || sid_hist[j] == sid;
      if (ok) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += wk[j][e] * win[j][e];
      }
    }
    if (silu) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = silu_f(acc[e]);
    }
    V8<T>::st(yb + static_cast<size_t>(t) * C, acc);
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      sid_hist[j] = sid_hist[j + 1];
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
    }
  }
}

// g[t] = dy[t]·act'(pre[t]);  dx[t'] = Σ_j w[j]·g[t'+(W-1)-j] (same-document taps only)
// A thread owns 8 channels and CV_TSTEP_BWD consecutive positions and walks the output steps once with two rolling
// windows (the last W inputs, the last W values of g): one load of x and dy, one activation derivative per step.  dx of a
// position is complete W−1 steps later, so the walk runs W−1 steps past the block's end (reading, not owning, those
// steps).  Weight / bias gradients belong to the block that owns the output step; they leave through atomics once per
// thread (W·8 + 8 of them per 128 positions).
constexpr int CV_TSTEP_BWD = 128;

template <typename T, int W>
__global__ void __launch_bounds__(128) conv1d_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ bias, const int* __restrict__ seq_idx,
                                                         T* __restrict__ dx, float* __restrict__ dw, float* __restrict__ db, int B, int L,
                                                         int C, int silu, int xs, int dys) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  const int c0 = cv * 8;
  if (c0 >= C) return;
  const int t0 = blockIdx.y * CV_TSTEP_BWD, b = blockIdx.z;
  float wk[W][8], bs[8], dwa[W][8], dba[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    bs[e] = bias ? bias[c0 + e] : 0.f; dba[e] = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) { wk[j][e] = w[(c0 + e) * W + j]; dwa[j][e] = 0.f; }
  }
  const size_t base = static_cast<size_t>(b) * L * C + c0;
  const int* sb = seq_idx ? seq_idx + static_cast<size_t>(b) * L : nullptr;
  const int t_end = min(t0 + CV_TSTEP_BWD, L);
  // windows: slot k holds step t − (W−1) + k, slot W−1 the current step
  float xw[W][8], gw[W][8];
  int sw[W];                                            // document ids of the window's steps (−1: before the sequence)
#pragma unroll
  for (int k = 0; k < W; ++k) {
    const int tt = t0 - W + k;                          // the window "before" step t0 (shifted in at the loop top)
    sw[k] = (tt >= 0) ? (sb ? sb[tt] : 0) : -1;
    if (tt >= 0) V8<T>::ld(x + (static_cast<size_t>(b) * L + tt) * xs + c0, xw[k]);
    else {
#pragma unroll
      for (int e = 0; e < 8; ++e) xw[k][e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) gw[k][e] = 0.f;
  }
  for (int t = t0; t < t_end + W - 1; ++t) {
    // shift the windows by one step
#pragma unroll
    for (int k = 0; k < W - 1; ++k) {
      sw[k] = sw[k + 1];
#pragma unroll
      for (int e = 0; e < 8; ++e) { xw[k][e] = xw[k + 1][e]; gw[k][e] = gw[k + 1][e]; }
    }
    if (t < L) {
      sw[W - 1] = sb ? sb[t] : 0;
      V8<T>::ld(x + (static_cast<size_t>(b) * L + t) * xs + c0, xw[W - 1]);
      float pre[8], g[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) pre[e] = bs[e];
#pragma unroll
      for (int k = 0; k < W; ++k) {
        if (sw[k] == sw[W - 1]) {
#pragma unroll
          for (int e = 0; e < 8; ++e) pre[e] += wk[k][e] * xw[k][e];
        }
      }
      V8<T>::ld(dy + (static_cast<size_t>(b) * L + t) * dys + c0, g);
      if (silu) {
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] *= dsilu_f(pre[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) gw[W - 1][e] = g[e];
      if (t < t_end) {                                  // this block owns output step t: its weight / bias gradients
#pragma unroll
        for (int k = 0; k < W; ++k) {
          if (sw[k] == sw[W - 1]) {
#pragma unroll
            for (int e = 0; e < 8; ++e) dwa[k][e] += g[e] * xw[k][e];
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) dba[e] += g[e];
      }
    } else {
      sw[W - 1] = -2;                                   // past the end: matches no document
#pragma unroll
      for (int e = 0; e < 8; ++e) gw[W - 1][e] = 0.f;
    }
    // position tp = t − (W−1) has now seen every output step that read it: slot k of the windows is step tp + k, tap W−1−k
    const int tp = t - (W - 1);
    if (tp >= t0 && tp < t_end) {
      float dxa[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) dxa[e] = 0.f;
#pragma unroll
      for (int k = 0; k < W; ++k) {
        if (sw[k] == sw[0]) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dxa[e] += wk[W - 1 - k][e] * gw[k][e];
        }
      }
      V8<T>::st(dx + base + static_cast<size_t>(tp) * C, dxa);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    if (db) atomicAdd(&db[c0 + e], dba[e]);
#pragma unroll
    for (int j = 0; j < W; ++j) atomicAdd(&dw[(c0 + e) * W + j], dwa[j][e]);
  }
}

}  // namespace b200

using namespace b200;

template <typename T>
static int conv_fwd_t(const void* x, const float* w, const float* bias, const int* seq_idx, void* y, int B, int L, int C, int W,
                      int silu, int xs, cudaStream_t st) {
  dim3 grid((C / 8 + 127) / 128, (L + CV_TSTEP - 1) / CV_TSTEP, B);
  switch (W) {
    case 2: conv1d_fwd_kernel<T, 2><<<grid, 128, 0, st>>>((const T*)x, w, bias, seq_idx, (T*)y, B, L, C, silu, xs); break;
    case 3: conv1d_fwd_kernel<T, 3><<<grid, 128, 0, st>>>((const T*)x, w, bias, seq_idx, (T*)y, B, L, C, silu, xs); break;
    case 4: conv1d_fwd_kernel<T, 4><<<grid, 128, 0, st>>>((const T*)x, w, bias, seq_idx, (T*)y, B, L, C, silu, xs); break;
    default: return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
template <typename T>
static int conv_bwd_t(const void* dy, const void* x, const float* w, const float* bias, const int* seq_idx, void* dx, float* dw,
                      float* db, int B, int L, int C, int W, int silu, int xs, int dys, cudaStream_t st) {
  dim3 grid((C / 8 + 127) / 128, (L + CV_TSTEP_BWD - 1) / CV_TSTEP_BWD, B);
  switch (W) {
    case 2: conv1d_bwd_kernel<T, 2><<<grid, 128, 0, st>>>((const T*)dy, (const T*)x, w, bias, seq_idx, (T*)dx, dw, db, B, L, C, silu, xs, dys); break;
    case 3: conv1d_bwd_kernel<T, 3><<<grid, 128, 0, st>>>((const T*)dy, (const T*)x, w, bias, seq_idx, (T*)dx, dw, db, B, L, C, silu, xs, dys); break;
    case 4: conv1d_bwd_kernel<T, 4><<<grid, 128, 0, st>>>((const T*)dy, (const T*)x, w, bias, seq_idx, (T*)dx, dw, db, B, L, C, silu, xs, dys); break;
    default: return -1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_conv1d_fwd(const void* x, int dtype, const float* w, const float* bias, const int* seq_idx, void* y, int B,
                               int L, int C, int W, int silu, int xs, cudaStream_t st) {
  if (C % 8 || xs % 8) return -1;
  if (B * L == 0) return 0;
  return dtype == 1 ? conv_fwd_t<__nv_bfloat16>(x, w, bias, seq_idx, y, B, L, C, W, silu, xs, st)
                    : conv_fwd_t<float>(x, w, bias, seq_idx, y, B, L, C, W, silu, xs, st);
}
// dw [C, W] and db [C] (fp32) must be zero on entry.
extern "C" int b200_conv1d_bwd(const void* dy, const void* x, int dtype, const float* w, const float* bias, const int* seq_idx,
                               void* dx, float* dw, float* db, int B, int L, int C, int W, int silu, int xs, int dys,
                               cudaStream_t st) {
  if (C % 8 || xs % 8 || dys % 8) return -1;
  if (B * L == 0) return 0;
  return dtype == 1 ? conv_bwd_t<__nv_bfloat16>(dy, x, w, bias, seq_idx, dx, dw, db, B, L, C, W, silu, xs, dys, st)
                    : conv_bwd_t<float>(dy, x, w, bias, seq_idx, dx, dw, db, B, L, C, W, silu, xs, dys, st);
}
