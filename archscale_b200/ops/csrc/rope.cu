// Fused per-head RMSNorm (QK-norm) + rotary embedding (NeoX halves) for q:[N,H,D] and k:[N,G,D], bf16.
// One warp per token (all its heads); D ∈ {64, 128} so a lane owns D/32 contiguous elements of a head row and its
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

// One warp per TOKEN: cos / sin and the norm gains are loaded once and serve all H + G heads of the token, there is no
// per-row index arithmetic, and the heads are walked four at a time so that four 256-byte rows are in flight per warp.
constexpr int ROPE_U = 4;

// Where the heads of a token sit.  Dense rows [tokens, heads, D] are q_hpg = H, k_gs = D; the output of a fused QKV projection
// laid out per key/value group as [group][q_per_kv query heads, key head, value head][D] is q_hpg = q_per_kv and
// q_gs = k_gs = (q_per_kv + 2)·D with the key / value base pointers advanced to their slot of group 0.
struct QKLayout {
  long long q_ts, k_ts;      // token strides (elements)
  long long q_gs, k_gs;      // stride between groups of query heads / between key (value) heads
  int q_hpg;                 // query heads per group
};

// Copies G head rows of one token between two head strides; kept out of line so that the row copy does not change how the
// compiler schedules the norm / rotation loops around it (inlined, both kernels ran about twice as long).
template <int EPL>
__device__ __noinline__ void copy_head_rows(const __nv_bfloat16* src, long long sstride, __nv_bfloat16* dst, long long dstride, int G) {
  for (int g0 = 0; g0 < G; g0 += ROPE_U) {
    float x[ROPE_U][EPL];
#pragma unroll
    for (int u = 0; u < ROPE_U; ++u)
      if (g0 + u < G) ld_row<EPL>(src + (g0 + u) * sstride, x[u]);
#pragma unroll
    for (int u = 0; u < ROPE_U; ++u)
      if (g0 + u < G) st_row<EPL>(dst + (g0 + u) * dstride, x[u]);
  }
}

// GROUPED: the per-group layout (else every head of a part is D elements after the previous one: dense rows or the blocked
// fused projection, for which the loops below reduce to the plain walk over heads).  WITH_V: also copy the value heads.
template <int EPL, typename TW, bool GROUPED, bool WITH_V>
__global__ void __launch_bounds__(256, 4) qknorm_rope_fwd_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const TW* __restrict__ qw,
    const TW* __restrict__ kw, const __nv_bfloat16* __restrict__ cosb, const __nv_bfloat16* __restrict__ sinb,
    __nv_bfloat16* __restrict__ qo, __nv_bfloat16* __restrict__ ko, float* __restrict__ q_rstd,
    float* __restrict__ k_rstd, int64_t n_tokens, int T, int H, int G, float eps, const QKLayout L,
    const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ vo) {
  constexpr int D = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int ci = (lane & 15) * EPL;
  float wq[EPL], wk[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    wq[e] = qw ? ldw<TW>(qw, lane * EPL + e) : 1.f;
    wk[e] = kw ? ldw<TW>(kw, lane * EPL + e) : 1.f;
  }
  for (int64_t tok = warp_global; tok < n_tokens; tok += n_warps) {
    float cs[EPL], sn[EPL];
    if (cosb) {
      const size_t co = static_cast<size_t>(tok % T) * (D / 2) + ci;
      ld_row<EPL>(cosb + co, cs);
      ld_row<EPL>(sinb + co, sn);
    }
#pragma unroll 1
    for (int part = 0; part < 2; ++part) {      // the token's query heads, then its key heads
      // inputs may be column slices of a wider (fused projection) matrix, dense or interleaved per group: see QKLayout.
      // Heads are walked group by group (one group of H heads for dense rows), so no head index is ever divided.
      const int per = part ? G : (GROUPED ? L.q_hpg : H), n_groups = (part || !GROUPED) ? 1 : H / L.q_hpg;
      const long long gstride = (part || !GROUPED) ? 0 : L.q_gs, hstride = (GROUPED && part) ? L.k_gs : D;
      const bool has_w = part ? kw != nullptr : qw != nullptr;
      for (int grp = 0; grp < n_groups; ++grp) {
        const __nv_bfloat16* src = (part ? k + tok * L.k_ts : q + tok * L.q_ts) + grp * gstride + lane * EPL;
        __nv_bfloat16* dst = (part ? ko + tok * G * D : qo + tok * H * D) + static_cast<long long>(grp) * per * D + lane * EPL;
        float* rstd = (part ? k_rstd + tok * G : q_rstd + tok * H) + grp * per;
        for (int h0 = 0; h0 < per; h0 += ROPE_U) {
          float x[ROPE_U][EPL];
#pragma unroll
          for (int u = 0; u < ROPE_U; ++u)
            if (h0 + u < per) ld_row<EPL>(src + (h0 + u) * hstride, x[u]);
#pragma unroll
          for (int u = 0; u < ROPE_U; ++u) {
            if (h0 + u >= per) continue;          // warp-uniform
            if (has_w) {
              float ss = 0.f;
#pragma unroll
              for (int e = 0; e < EPL; ++e) ss += x[u][e] * x[u][e];
              ss = wsum(ss);
              const float rs = rsqrtf(ss / D + eps);
              if (lane == 0) rstd[h0 + u] = rs;
#pragma unroll
              for (int e = 0; e < EPL; ++e) x[u][e] = x[u][e] * rs * (part ? wk[e] : wq[e]);
            }
            if (cosb) {
              float o[EPL];
#pragma unroll
              for (int e = 0; e < EPL; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, x[u][e], 16);
                o[e] = lane < 16 ? x[u][e] * cs[e] - other * sn[e] : other * sn[e] + x[u][e] * cs[e];
              }
              st_row<EPL>(dst + (h0 + u) * D, o);
            } else {
              st_row<EPL>(dst + (h0 + u) * D, x[u]);
            }
          }
        }
      }
    }
    if (WITH_V)                                     // the value heads, copied out of the fused projection into dense rows
      copy_head_rows<EPL>(v + tok * L.k_ts + lane * EPL, GROUPED ? L.k_gs : D, vo + tok * G * D + lane * EPL, D, G);
  }
}

template <int EPL, typename TW, bool GROUPED, bool WITH_V>
__global__ void __launch_bounds__(256, 2) qknorm_rope_bwd_kernel(
    const __nv_bfloat16* __restrict__ dqo, const __nv_bfloat16* __restrict__ dko, const __nv_bfloat16* __restrict__ q,
    const __nv_bfloat16* __restrict__ k, const TW* __restrict__ qw, const TW* __restrict__ kw,
    const __nv_bfloat16* __restrict__ cosb, const __nv_bfloat16* __restrict__ sinb, const float* __restrict__ q_rstd,
    const float* __restrict__ k_rstd, __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk,
    float* __restrict__ dw_partial /* [grid, 2, D] */, int64_t n_tokens, int T, int H, int G, const QKLayout L,
    const QKLayout LO /* layout of dq, dk (and dv_dst) */, const __nv_bfloat16* __restrict__ dvo, __nv_bfloat16* __restrict__ dv_dst) {
  constexpr int D = EPL * 32;
  __shared__ float dw_s[2][D];
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&dw_s[0][0])[i] = 0.f;
  __syncthreads();
  const int64_t warp_global = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int ci = (lane & 15) * EPL;
  float dwq[EPL], dwk[EPL], wq[EPL], wk[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    dwq[e] = dwk[e] = 0.f;
    wq[e] = qw ? ldw<TW>(qw, lane * EPL + e) : 1.f;
    wk[e] = kw ? ldw<TW>(kw, lane * EPL + e) : 1.f;
  }
  for (int64_t tok = warp_global; tok < n_tokens; tok += n_warps) {
    float cs[EPL], sn[EPL];
    if (cosb) {
      const size_t co = static_cast<size_t>(tok % T) * (D / 2) + ci;
      ld_row<EPL>(cosb + co, cs);
      ld_row<EPL>(sinb + co, sn);
    }
#pragma unroll 1
    for (int part = 0; part < 2; ++part) {
      const int per = part ? G : (GROUPED ? L.q_hpg : H), n_groups = (part || !GROUPED) ? 1 : H / L.q_hpg;      // LO: same grouping
      const long long gstride = (part || !GROUPED) ? 0 : L.q_gs, hstride = (GROUPED && part) ? L.k_gs : D;
      const long long o_gstride = (part || !GROUPED) ? 0 : LO.q_gs, o_hstride = (GROUPED && part) ? LO.k_gs : D;
      const bool has_w = part ? kw != nullptr : qw != nullptr;
      for (int grp = 0; grp < n_groups; ++grp) {
        const long long dense = static_cast<long long>(grp) * per * D + lane * EPL;
        const __nv_bfloat16* gsrc = (part ? dko + tok * G * D : dqo + tok * H * D) + dense;
        __nv_bfloat16* gdst = (part ? dk + tok * LO.k_ts : dq + tok * LO.q_ts) + grp * o_gstride + lane * EPL;
        const __nv_bfloat16* xsrc = (part ? k + tok * L.k_ts : q + tok * L.q_ts) + grp * gstride + lane * EPL;
        const float* rstd = (part ? k_rstd + tok * G : q_rstd + tok * H) + grp * per;
        for (int h0 = 0; h0 < per; h0 += ROPE_U) {
          float g[ROPE_U][EPL], x[ROPE_U][EPL], rs[ROPE_U];
#pragma unroll
          for (int u = 0; u < ROPE_U; ++u) {
            if (h0 + u >= per) continue;
            ld_row<EPL>(gsrc + (h0 + u) * D, g[u]);
            if (has_w) { ld_row<EPL>(xsrc + (h0 + u) * hstride, x[u]); rs[u] = rstd[h0 + u]; }
          }
#pragma unroll
          for (int u = 0; u < ROPE_U; ++u) {
            if (h0 + u >= per) continue;
            if (cosb) {
              float o[EPL];
#pragma unroll
              for (int e = 0; e < EPL; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, g[u][e], 16);
                o[e] = lane < 16 ? g[u][e] * cs[e] + other * sn[e] : -other * sn[e] + g[u][e] * cs[e];
              }
#pragma unroll
              for (int e = 0; e < EPL; ++e) g[u][e] = o[e];
            }
            if (has_w) {
              float dot = 0.f;
              float gw[EPL];
#pragma unroll
              for (int e = 0; e < EPL; ++e) {
                gw[e] = g[u][e] * (part ? wk[e] : wq[e]);
                dot += gw[e] * x[u][e];
                if (part) dwk[e] += g[u][e] * x[u][e] * rs[u]; else dwq[e] += g[u][e] * x[u][e] * rs[u];
              }
              dot = wsum(dot);
              const float c1 = dot * rs[u] * rs[u] * rs[u] / D;
#pragma unroll
              for (int e = 0; e < EPL; ++e) g[u][e] = gw[e] * rs[u] - x[u][e] * c1;
            }
            st_row<EPL>(gdst + (h0 + u) * o_hstride, g[u]);
          }
        }
      }
    }
    if (WITH_V)                                     // the value gradient takes its slot of the fused-projection gradient
      copy_head_rows<EPL>(dvo + static_cast<size_t>(tok) * G * D + lane * EPL, D, dv_dst + tok * LO.k_ts + lane * EPL,
                          GROUPED ? LO.k_gs : D, G);
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

// partials are [n, 2·D]: columns 0..D−1 belong to dqw, D..2D−1 to dkw
__global__ void __launch_bounds__(1024) qk_dw_reduce_kernel(const float* __restrict__ part, float* __restrict__ dqw, float* __restrict__ dkw, int n, int D) {
  const float t = column_sum_block(part, n, 2 * D);
  const int c = blockIdx.x * 32 + threadIdx.x;
  if (threadIdx.x < 32 && c < 2 * D) { if (c < D) dqw[c] = t; else dkw[c - D] = t; }
}

constexpr int kRopeGrid = 148 * 8;

}  // namespace b200

using namespace b200;
typedef __nv_bfloat16 bf16;

extern "C" int b200_qknorm_rope_grid() { return kRopeGrid; }

// q_hpg / gs: see QKLayout (q_hpg = H, gs = D for dense rows).  v / vo: optional value heads (k's layout) copied to dense rows.
extern "C" int b200_qknorm_rope_fwd_ex(const void* q, const void* k, const void* v, const void* qw, const void* kw, int w_dtype,
                                       const void* cos, const void* sin, void* qo, void* ko, void* vo, float* q_rstd, float* k_rstd,
                                       int64_t n_tokens, int T, int H, int G, int D, float eps, int64_t q_ts, int64_t k_ts,
                                       int q_hpg, int64_t q_gs, int64_t k_gs, cudaStream_t st) {
  if (n_tokens == 0) return 0;
  if (q_hpg <= 0 || H % q_hpg) return -1;
  const QKLayout L{q_ts, k_ts, q_gs, k_gs, q_hpg};
  const bool grouped = q_hpg != H, with_v = v != nullptr;
  if (!grouped && k_gs != D) return -1;
#define LAUNCH2(EPL, TW, GR, WV)                                                                                      \
  qknorm_rope_fwd_kernel<EPL, TW, GR, WV><<<kRopeGrid, 256, 0, st>>>((const bf16*)q, (const bf16*)k, (const TW*)qw, (const TW*)kw, \
                                                             (const bf16*)cos, (const bf16*)sin, (bf16*)qo, (bf16*)ko,  \
                                                             q_rstd, k_rstd, n_tokens, T, H, G, eps, L, (const bf16*)v, (bf16*)vo)
#define LAUNCH(EPL, TW)                                                        \
  do {                                                                         \
    if (grouped) { if (with_v) LAUNCH2(EPL, TW, true, true); else LAUNCH2(EPL, TW, true, false); } \
    else { if (with_v) LAUNCH2(EPL, TW, false, true); else LAUNCH2(EPL, TW, false, false); }       \
  } while (0)
  if (D == 128) { if (w_dtype == 1) LAUNCH(4, bf16); else LAUNCH(4, float); }
  else if (D == 64) { if (w_dtype == 1) LAUNCH(2, bf16); else LAUNCH(2, float); }
  else return -1;
#undef LAUNCH
#undef LAUNCH2
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_qknorm_rope_fwd(const void* q, const void* k, const void* qw, const void* kw, int w_dtype,
                                    const void* cos, const void* sin, void* qo, void* ko, float* q_rstd, float* k_rstd,
                                    int64_t n_tokens, int T, int H, int G, int D, float eps, int64_t q_ts, int64_t k_ts, cudaStream_t st) {
  return b200_qknorm_rope_fwd_ex(q, k, nullptr, qw, kw, w_dtype, cos, sin, qo, ko, nullptr, q_rstd, k_rstd, n_tokens, T, H, G, D, eps,
                                 q_ts, k_ts, H, 0, D, st);
}

// dq / dk are written with the layout (o_q_ts, o_k_ts, o_q_hpg, o_q_gs, o_k_gs); dvo (dense) is copied to dv_dst in k's output layout.
extern "C" int b200_qknorm_rope_bwd_ex(const void* dqo, const void* dko, const void* dvo, const void* q, const void* k, const void* qw,
                                       const void* kw, int w_dtype, const void* cos, const void* sin, const float* q_rstd,
                                       const float* k_rstd, void* dq, void* dk, void* dv_dst, float* dqw, float* dkw,
                                       float* dw_partial, int64_t n_tokens, int T, int H, int G, int D, int64_t q_ts, int64_t k_ts,
                                       int q_hpg, int64_t q_gs, int64_t k_gs, int64_t o_q_ts, int64_t o_k_ts, int o_q_hpg,
                                       int64_t o_q_gs, int64_t o_k_gs, cudaStream_t st) {
  if (n_tokens == 0) return 0;
  if (q_hpg <= 0 || o_q_hpg != q_hpg || H % q_hpg) return -1;       // input and output share one grouping
  const QKLayout L{q_ts, k_ts, q_gs, k_gs, q_hpg}, LO{o_q_ts, o_k_ts, o_q_gs, o_k_gs, o_q_hpg};
  const bool grouped = q_hpg != H, with_v = dvo != nullptr;
  if (!grouped && (k_gs != D || o_k_gs != D)) return -1;
#define LAUNCH2(EPL, TW, GR, WV)                                                                                       \
  qknorm_rope_bwd_kernel<EPL, TW, GR, WV><<<kRopeGrid, 256, 0, st>>>((const bf16*)dqo, (const bf16*)dko, (const bf16*)q, (const bf16*)k, \
                                                             (const TW*)qw, (const TW*)kw, (const bf16*)cos, (const bf16*)sin,  \
                                                             q_rstd, k_rstd, (bf16*)dq, (bf16*)dk, dw_partial, n_tokens, T, H, G, L, LO, \
                                                             (const bf16*)dvo, (bf16*)dv_dst)
#define LAUNCH(EPL, TW)                                                        \
  do {                                                                         \
    if (grouped) { if (with_v) LAUNCH2(EPL, TW, true, true); else LAUNCH2(EPL, TW, true, false); } \
    else { if (with_v) LAUNCH2(EPL, TW, false, true); else LAUNCH2(EPL, TW, false, false); }       \
  } while (0)
  if (D == 128) { if (w_dtype == 1) LAUNCH(4, bf16); else LAUNCH(4, float); }
  else if (D == 64) { if (w_dtype == 1) LAUNCH(2, bf16); else LAUNCH(2, float); }
  else return -1;
#undef LAUNCH
#undef LAUNCH2
  if (qw) qk_dw_reduce_kernel<<<(2 * D + 31) / 32, 1024, 0, st>>>(dw_partial, dqw, dkw, kRopeGrid, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_qknorm_rope_bwd(const void* dqo, const void* dko, const void* q, const void* k, const void* qw,
                                     const void* kw, int w_dtype, const void* cos, const void* sin, const float* q_rstd,
                                     const float* k_rstd, void* dq, void* dk, float* dqw, float* dkw, float* dw_partial,
                                     int64_t n_tokens, int T, int H, int G, int D, int64_t q_ts, int64_t k_ts, cudaStream_t st) {
  return b200_qknorm_rope_bwd_ex(dqo, dko, nullptr, q, k, qw, kw, w_dtype, cos, sin, q_rstd, k_rstd, dq, dk, nullptr, dqw, dkw,
                                 dw_partial, n_tokens, T, H, G, D, q_ts, k_ts, H, 0, D, static_cast<int64_t>(H) * D,
                                 static_cast<int64_t>(G) * D, H, 0, D, st);
}
