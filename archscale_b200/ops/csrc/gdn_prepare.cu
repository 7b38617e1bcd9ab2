// Row-wise part of the chunked gated delta rule ("prepare" stage), forward and backward: everything that is element-wise or a
// reduction over one token's head vector, fused with the layout change from token-major activations [B, T, H, D] to the
// chunk-major operands [B·H, Tp, D] (Tp = T rounded up to the 64-token chunk) that the chunk-parallel products and the
// recurrence kernel (gdn_chunk.cu) take.  In the reference this work sits inside fla's Triton kernels
// (`lit_gpt/gated_deltanet.py:315-326`: chunk_gated_delta_rule with use_qk_l2norm_in_kernel=True).
//
// With gc the inclusive cumulative log-decay inside the chunk and gl its value at the chunk's last token:
//     qn = scale · q / sqrt(q·q + eps)         kn = k / sqrt(k·k + eps)            vc = v
//     qg = qn · exp(gc)                        kd = kn · exp(gl − gc)
// all written as bf16.  Rows t >= T (padding of the last chunk) are written as zeros.  The backward takes the gradients of
// the five outputs and returns dq, dk, dv plus two per-row dot products from which the caller forms the gradient of gc:
//     a_row = <dqg, qg>,  s_row = <dkd, kd>;   d gc_row = a_row − s_row,   d gl += Σ_rows s_row.
// One warp per (token, head) row; a lane owns DK/32 (DV/32) consecutive elements.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "api.h"

namespace b200 {

template <int N>
__device__ __forceinline__ void ld_bf16(const __nv_bfloat16* p, float (&v)[N]) {
  if constexpr (N == 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  } else if constexpr (N == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 2; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  } else {
    static_assert(N == 16, "4, 8 or 16 elements per lane");
    ld_bf16<8>(p, *reinterpret_cast<float(*)[8]>(&v[0]));
    ld_bf16<8>(p + 8, *reinterpret_cast<float(*)[8]>(&v[8]));
  }
}
template <int N>
__device__ __forceinline__ void st_bf16(__nv_bfloat16* p, const float (&v)[N]) {
  if constexpr (N == 8) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  } else if constexpr (N == 4) {
    uint2 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 2; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
    static_assert(N == 16, "4, 8 or 16 elements per lane");
    st_bf16<8>(p, *reinterpret_cast<const float(*)[8]>(&v[0]));
    st_bf16<8>(p + 8, *reinterpret_cast<const float(*)[8]>(&v[8]));
  }
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int GP_CHUNK = 64;

template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_prepare_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                             const __nv_bfloat16* __restrict__ v, const float* __restrict__ gc,
                                                             __nv_bfloat16* __restrict__ qn, __nv_bfloat16* __restrict__ kn,
                                                             __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ kd,
                                                             __nv_bfloat16* __restrict__ qg, int B, int T, int Tp, int H, float scale,
                                                             float eps) {
  constexpr int EK = DK / 32, EV = DV / 32;
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;     // over [B·H, Tp]
  if (row >= static_cast<long long>(B) * H * Tp) return;
  const int t = static_cast<int>(row % Tp);
  const int bh = static_cast<int>(row / Tp), b = bh / H, h = bh % H;
  const size_t out_k = static_cast<size_t>(row) * DK + lane * EK, out_v = static_cast<size_t>(row) * DV + lane * EV;
  float qv[EK], kv[EK], vv[EV];
  if (t < T) {
    const size_t in_row = (static_cast<size_t>(b) * T + t) * H + h;
    ld_bf16<EK>(q + in_row * DK + lane * EK, qv);
    ld_bf16<EK>(k + in_row * DK + lane * EK, kv);
    ld_bf16<EV>(v + in_row * DV + lane * EV, vv);
  } else {
#pragma unroll
    for (int i = 0; i < EK; ++i) { qv[i] = 0.f; kv[i] = 0.f; }
#pragma unroll
    for (int i = 0; i < EV; ++i) vv[i] = 0.f;
  }
  float sq = 0.f, sk = 0.f;
#pragma unroll
  for (int i = 0; i < EK; ++i) { sq += qv[i] * qv[i]; sk += kv[i] * kv[i]; }
  sq = wsum(sq); sk = wsum(sk);
  const float rq = rsqrtf(sq + eps) * scale, rk = rsqrtf(sk + eps);
  const float g = gc[row], gl = gc[row - t % GP_CHUNK + GP_CHUNK - 1];
  const float ec = __expf(g), ed = __expf(gl - g);
  float o1[EK], o2[EK];
#pragma unroll
  for (int i = 0; i < EK; ++i) { o1[i] = qv[i] * rq; o2[i] = o1[i] * ec; }
  st_bf16<EK>(qn + out_k, o1);
  st_bf16<EK>(qg + out_k, o2);
#pragma unroll
  for (int i = 0; i < EK; ++i) { o1[i] = kv[i] * rk; o2[i] = o1[i] * ed; }
  st_bf16<EK>(kn + out_k, o1);
  st_bf16<EK>(kd + out_k, o2);
  st_bf16<EV>(vc + out_v, vv);
}

template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_prepare_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                             const float* __restrict__ gc, const __nv_bfloat16* __restrict__ dqn,
                                                             const __nv_bfloat16* __restrict__ dkn, const __nv_bfloat16* __restrict__ dvc,
                                                             const __nv_bfloat16* __restrict__ dkd, const __nv_bfloat16* __restrict__ dqg,
                                                             __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk,
                                                             __nv_bfloat16* __restrict__ dv, float* __restrict__ a_row,
                                                             float* __restrict__ s_row, int B, int T, int Tp, int H, float scale, float eps) {
  constexpr int EK = DK / 32, EV = DV / 32;
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= static_cast<long long>(B) * H * Tp) return;
  const int t = static_cast<int>(row % Tp);
  const int bh = static_cast<int>(row / Tp), b = bh / H, h = bh % H;
  if (t >= T) {                                         // padding rows: their operands were zeros, nothing flows back
    if (lane == 0) { a_row[row] = 0.f; s_row[row] = 0.f; }
    return;
  }
  const size_t in_row = (static_cast<size_t>(b) * T + t) * H + h;
  const size_t ck = static_cast<size_t>(row) * DK + lane * EK, cv = static_cast<size_t>(row) * DV + lane * EV;
  float qv[EK], kv[EK];
  ld_bf16<EK>(q + in_row * DK + lane * EK, qv);
  ld_bf16<EK>(k + in_row * DK + lane * EK, kv);
  float sq = 0.f, sk = 0.f;
#pragma unroll
  for (int i = 0; i < EK; ++i) { sq += qv[i] * qv[i]; sk += kv[i] * kv[i]; }
  sq = wsum(sq); sk = wsum(sk);
  const float rq = rsqrtf(sq + eps), rk = rsqrtf(sk + eps);
  const float g = gc[row], gl = gc[row - t % GP_CHUNK + GP_CHUNK - 1];
  const float ec = __expf(g), ed = __expf(gl - g);
  float g1[EK], g2[EK];
  // q side: qn = scale·q·rq, qg = qn·ec
  ld_bf16<EK>(dqn + ck, g1);
  ld_bf16<EK>(dqg + ck, g2);
  float dot_a = 0.f, dot_u = 0.f;
#pragma unroll
  for (int i = 0; i < EK; ++i) {
    const float qhat = qv[i] * rq;                      // unit direction (without the scale)
    dot_a += g2[i] * qhat;                              // <dqg, qn> / scale, completed below
    g1[i] = (g1[i] + g2[i] * ec) * scale;               // gradient w.r.t. the unit direction
    dot_u += g1[i] * qhat;
  }
  dot_a = wsum(dot_a); dot_u = wsum(dot_u);
#pragma unroll
  for (int i = 0; i < EK; ++i) g1[i] = rq * (g1[i] - dot_u * qv[i] * rq);
  st_bf16<EK>(dq + in_row * DK + lane * EK, g1);
  // k side: kn = k·rk, kd = kn·ed
  ld_bf16<EK>(dkn + ck, g1);
  ld_bf16<EK>(dkd + ck, g2);
  float dot_s = 0.f, dot_k = 0.f;
#pragma unroll
  for (int i = 0; i < EK; ++i) {
    const float khat = kv[i] * rk;
    dot_s += g2[i] * khat;
    g1[i] = g1[i] + g2[i] * ed;
    dot_k += g1[i] * khat;
  }
  dot_s = wsum(dot_s); dot_k = wsum(dot_k);
#pragma unroll
  for (int i = 0; i < EK; ++i) g1[i] = rk * (g1[i] - dot_k * kv[i] * rk);
  st_bf16<EK>(dk + in_row * DK + lane * EK, g1);
  float vv[EV];
  ld_bf16<EV>(dvc + cv, vv);
  st_bf16<EV>(dv + in_row * DV + lane * EV, vv);
  if (lane == 0) {
    a_row[row] = dot_a * scale * ec;                    // <dqg, qg>
    s_row[row] = dot_s * ed;                            // <dkd, kd>
  }
}

}  // namespace b200

#define GP_DISPATCH(DKV, DVV, CALL)                                       \
  if (DKV == 128 && DVV == 128) { CALL(128, 128) }                        \
  else if (DKV == 128 && DVV == 256) { CALL(128, 256) }                   \
  else if (DKV == 256 && DVV == 256) { CALL(256, 256) }                   \
  else if (DKV == 256 && DVV == 512) { CALL(256, 512) }                   \
  else return -1;

// q, k [B, T, H, Dk], v [B, T, H, Dv] bf16 contiguous; gc [B·H, Tp] fp32; outputs [B·H, Tp, D] bf16.  Tp % 64 == 0.
extern "C" int b200_gdn_prepare_fwd(const void* q, const void* k, const void* v, const float* gc, void* qn, void* kn, void* vc,
                                    void* kd, void* qg, int B, int T, int Tp, int H, int Dk, int Dv, float scale, float eps,
                                    cudaStream_t st) {
  using namespace b200;
  typedef __nv_bfloat16 bf;
  if (Tp % GP_CHUNK || Tp < T) return -1;
  const long long rows = static_cast<long long>(B) * H * Tp;
  if (rows == 0) return 0;
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
#define CALL(DK_, DV_)                                                                                                      \
  gdn_prepare_fwd_kernel<DK_, DV_><<<grid, 256, 0, st>>>((const bf*)q, (const bf*)k, (const bf*)v, gc, (bf*)qn, (bf*)kn, (bf*)vc, \
                                                         (bf*)kd, (bf*)qg, B, T, Tp, H, scale, eps);
  GP_DISPATCH(Dk, Dv, CALL)
#undef CALL
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_gdn_prepare_bwd(const void* q, const void* k, const float* gc, const void* dqn, const void* dkn, const void* dvc,
                                    const void* dkd, const void* dqg, void* dq, void* dk, void* dv, float* a_row, float* s_row,
                                    int B, int T, int Tp, int H, int Dk, int Dv, float scale, float eps, cudaStream_t st) {
  using namespace b200;
  typedef __nv_bfloat16 bf;
  if (Tp % GP_CHUNK || Tp < T) return -1;
  const long long rows = static_cast<long long>(B) * H * Tp;
  if (rows == 0) return 0;
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
#define CALL(DK_, DV_)                                                                                                       \
  gdn_prepare_bwd_kernel<DK_, DV_><<<grid, 256, 0, st>>>((const bf*)q, (const bf*)k, gc, (const bf*)dqn, (const bf*)dkn,      \
                                                         (const bf*)dvc, (const bf*)dkd, (const bf*)dqg, (bf*)dq, (bf*)dk,   \
                                                         (bf*)dv, a_row, s_row, B, T, Tp, H, scale, eps);
  GP_DISPATCH(Dk, Dv, CALL)
#undef CALL
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
