// Optimizer elementwise work on flat fp32 shards, one pass per stage instead of chains of foreach ops.
//
//   muon_momentum      m ← mu·m + g·s;  u ← (nesterov ? g·s + mu·m : m) as bf16        (s: optional device scalar, e.g. the
//                                                                                      gradient-clip coefficient)
//   adamw_fused        one pass of AdamW over a slice (moments, bias correction, decoupled decay, update), or — for the
//                      hyperball rule — moments + direction u = m̂/(√v̂ + eps) written out with Σx² and Σu² accumulated
//   seg_sq_norm        acc[k(i)] += x[i]²                                               segment = one matrix of the flat shard
//   seg_axpy_sq        x[i] ← x[i] − coef[k(i)]·u[i];  acc[k(i)] += x[i]²               (hyperball step + norm of the result)
//   seg_scale          x[i] ← x[i]·scale[k(i)]                                          (renormalisation)
//
// Segments are described by `bounds` (nseg + 1 ascending element offsets inside the buffer, multiples of 4) and `kidx`
// (slot of each segment in the coefficient / accumulator vectors).  A thread finds its segment by binary search over the
// handful of bounds; per-block partial sums go through shared memory so that global atomics stay in the thousands.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int OPT_THREADS = 256;
constexpr int OPT_VEC_PER_THREAD = 4;                       // float4 each → 4096 elements per block
constexpr int OPT_MAX_SEG_PER_BLOCK = 8;

__device__ __forceinline__ int seg_of(const long long* __restrict__ bounds, int nseg, long long i) {
  int lo = 0, hi = nseg;                                    // bounds[lo] ≤ i < bounds[hi]
  while (lo + 1 < hi) {
    const int mid = (lo + hi) >> 1;
    if (bounds[mid] <= i) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(OPT_THREADS) muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ m,
                                                                   __nv_bfloat16* __restrict__ u, long long n4, float mu,
                                                                   int nesterov, const float* __restrict__ gscale) {
  const float s = gscale ? *gscale : 1.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<const float4*>(m)[i];
    gv.x *= s; gv.y *= s; gv.z *= s; gv.w *= s;
    mv.x = mu * mv.x + gv.x; mv.y = mu * mv.y + gv.y; mv.z = mu * mv.z + gv.z; mv.w = mu * mv.w + gv.w;
    reinterpret_cast<float4*>(m)[i] = mv;
    float4 o = mv;
    if (nesterov) { o.x = gv.x + mu * mv.x; o.y = gv.y + mu * mv.y; o.z = gv.z + mu * mv.z; o.w = gv.w + mu * mv.w; }
    uint2 p;
    p.x = pack_bf16x2(o.x, o.y); p.y = pack_bf16x2(o.z, o.w);
    reinterpret_cast<uint2*>(u)[i] = p;
  }
}

// MODE 0: x ← x·(1 − lr·wd) − lr·m̂/(√v̂ + eps).  MODE 1: only the moments change; u_out ← m̂/(√v̂ + eps), acc[0] += Σx², acc[1] += Σu².
template <int MODE>
__global__ void __launch_bounds__(OPT_THREADS) adamw_fused_kernel(float* __restrict__ x, const float* __restrict__ g, float* __restrict__ m,
                                                                 float* __restrict__ v, float* __restrict__ u_out, long long n4, float lr,
                                                                 float b1, float b2, float eps, float wd, float inv_bc1, float inv_sqrt_bc2,
                                                                 const float* __restrict__ gscale, float* __restrict__ acc) {
  const float s = gscale ? *gscale : 1.f;
  const float decay = 1.f - lr * wd;
  float sx = 0.f, su = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 xv = reinterpret_cast<float4*>(x)[i];
    float ga[4] = {gv.x * s, gv.y * s, gv.z * s, gv.w * s};
    float ma[4] = {mv.x, mv.y, mv.z, mv.w}, va[4] = {vv.x, vv.y, vv.z, vv.w}, xa[4] = {xv.x, xv.y, xv.z, xv.w}, ua[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      ma[e] += (1.f - b1) * (ga[e] - ma[e]);                       // lerp, as torch._foreach_lerp_
      va[e] = b2 * va[e] + (1.f - b2) * ga[e] * ga[e];
      ua[e] = (ma[e] * inv_bc1) / (sqrtf(va[e]) * inv_sqrt_bc2 + eps);
      if (MODE == 0) xa[e] = xa[e] * decay - lr * ua[e];
      else { sx += xa[e] * xa[e]; su += ua[e] * ua[e]; }
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if (MODE == 0) reinterpret_cast<float4*>(x)[i] = make_float4(xa[0], xa[1], xa[2], xa[3]);
    else reinterpret_cast<float4*>(u_out)[i] = make_float4(ua[0], ua[1], ua[2], ua[3]);
  }
  if (MODE == 1) {
    __shared__ float s_acc[2][OPT_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { sx += __shfl_xor_sync(0xffffffffu, sx, o); su += __shfl_xor_sync(0xffffffffu, su, o); }
    if ((threadIdx.x & 31) == 0) { s_acc[0][threadIdx.x >> 5] = sx; s_acc[1][threadIdx.x >> 5] = su; }
    __syncthreads();
    if (threadIdx.x < 2) {
      float t = 0.f;
      for (int k = 0; k < OPT_THREADS / 32; ++k) t += s_acc[threadIdx.x][k];
      atomicAdd(&acc[threadIdx.x], t);
    }
  }
}

// MODE 0: acc += x²; MODE 1: x -= coef·u (u bf16), acc += x²; MODE 2: x *= coef
template <int MODE>
__global__ void __launch_bounds__(OPT_THREADS) seg_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ u, long long n4,
                                                         const long long* __restrict__ bounds, const int* __restrict__ kidx,
                                                         int nseg, const float* __restrict__ coef, float* __restrict__ acc) {
  __shared__ float s_part[OPT_MAX_SEG_PER_BLOCK];
  __shared__ int s_first;
  const long long base4 = static_cast<long long>(blockIdx.x) * OPT_THREADS * OPT_VEC_PER_THREAD;
  if (threadIdx.x == 0) s_first = seg_of(bounds, nseg, base4 * 4);
  if (threadIdx.x < OPT_MAX_SEG_PER_BLOCK) s_part[threadIdx.x] = 0.f;
  __syncthreads();
  const int first = s_first;
#pragma unroll
  for (int v = 0; v < OPT_VEC_PER_THREAD; ++v) {
    const long long i4 = base4 + v * OPT_THREADS + threadIdx.x;
    float sq = 0.f;
    int seg = first;
    if (i4 < n4) {
      seg = seg_of(bounds, nseg, i4 * 4);
      float4 xv = reinterpret_cast<float4*>(x)[i4];
      if (MODE == 1) {
        const float c = coef[kidx[seg]];
        const uint2 uv = reinterpret_cast<const uint2*>(u)[i4];
        const float2 a = unpack_bf16x2(uv.x), b = unpack_bf16x2(uv.y);
        xv.x -= c * a.x; xv.y -= c * a.y; xv.z -= c * b.x; xv.w -= c * b.y;
        reinterpret_cast<float4*>(x)[i4] = xv;
      } else if (MODE == 2) {
        const float c = coef[kidx[seg]];
        xv.x *= c; xv.y *= c; xv.z *= c; xv.w *= c;
        reinterpret_cast<float4*>(x)[i4] = xv;
      }
      if (MODE != 2) sq = xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
    }
    if (MODE != 2) {
      // lanes of a warp may straddle a segment boundary: reduce per distinct segment value
      const unsigned full = 0xffffffffu;
      const int seg0 = __shfl_sync(full, seg, 0);
      const bool uniform = __all_sync(full, seg == seg0);
      if (uniform) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(full, sq, o);
        if ((threadIdx.x & 31) == 0 && sq != 0.f) {
          const int slot = seg0 - first;
          if (slot < OPT_MAX_SEG_PER_BLOCK) atomicAdd(&s_part[slot], sq); else atomicAdd(&acc[kidx[seg0]], sq);
        }
      } else if (sq != 0.f) {
        const int slot = seg - first;
        if (slot < OPT_MAX_SEG_PER_BLOCK) atomicAdd(&s_part[slot], sq); else atomicAdd(&acc[kidx[seg]], sq);
      }
    }
  }
  if (MODE != 2) {
    __syncthreads();
    if (threadIdx.x < OPT_MAX_SEG_PER_BLOCK && first + static_cast<int>(threadIdx.x) < nseg && s_part[threadIdx.x] != 0.f)
      atomicAdd(&acc[kidx[first + threadIdx.x]], s_part[threadIdx.x]);
  }
}

}  // namespace b200

using namespace b200;

static inline unsigned opt_grid_stride(long long n4) {
  long long b = (n4 + OPT_THREADS - 1) / OPT_THREADS;
  return static_cast<unsigned>(b < 148 * 16 ? (b > 0 ? b : 1) : 148 * 16);
}

// g, m: fp32 [n]; u: bf16 [n]; n % 4 == 0; gscale: device scalar or null
extern "C" int b200_muon_momentum(const float* g, float* m, void* u, long long n, float mu, int nesterov, const float* gscale,
                                  cudaStream_t st) {
  if (n % 4) return -1;
  if (n == 0) return 0;
  muon_momentum_kernel<<<opt_grid_stride(n / 4), OPT_THREADS, 0, st>>>(g, m, static_cast<__nv_bfloat16*>(u), n / 4, mu, nesterov, gscale);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// mode 0 / 1 / 2 as described at the top; bounds: int64 [nseg + 1] on the device, bounds[0] = 0 … bounds[nseg] ≥ n
extern "C" int b200_seg_update(int mode, float* x, const void* u, long long n, const long long* bounds, const int* kidx, int nseg,
                               const float* coef, float* acc, cudaStream_t st) {
  if (n % 4 || nseg <= 0) return -1;
  if (n == 0) return 0;
  const long long n4 = n / 4;
  const unsigned grid = static_cast<unsigned>((n4 + OPT_THREADS * OPT_VEC_PER_THREAD - 1) / (OPT_THREADS * OPT_VEC_PER_THREAD));
  const __nv_bfloat16* up = static_cast<const __nv_bfloat16*>(u);
  if (mode == 0) seg_kernel<0><<<grid, OPT_THREADS, 0, st>>>(x, up, n4, bounds, kidx, nseg, coef, acc);
  else if (mode == 1) seg_kernel<1><<<grid, OPT_THREADS, 0, st>>>(x, up, n4, bounds, kidx, nseg, coef, acc);
  else if (mode == 2) seg_kernel<2><<<grid, OPT_THREADS, 0, st>>>(x, up, n4, bounds, kidx, nseg, coef, acc);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// One AdamW step over a contiguous fp32 slice (n % 4 == 0, 16-byte aligned pointers).  mode 0: update x in place;
// mode 1: leave x, write the direction to u_out (fp32) and add Σx², Σu² to acc[0], acc[1].  gscale: device scalar
// multiplied into the gradient (gradient-clip coefficient) or null.  bc1 = 1 − β1^t, bc2 = 1 − β2^t.
extern "C" int b200_adamw_fused(int mode, float* x, const float* g, float* m, float* v, float* u_out, long long n, float lr,
                                float beta1, float beta2, float eps, float wd, float bc1, float bc2, const float* gscale,
                                float* acc, cudaStream_t st) {
  if (n % 4 || (mode != 0 && mode != 1) || (mode == 1 && (!u_out || !acc))) return -1;
  if (n == 0) return 0;
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = 1.f / sqrtf(bc2);
  const unsigned grid = opt_grid_stride(n / 4);
  if (mode == 0)
    adamw_fused_kernel<0><<<grid, OPT_THREADS, 0, st>>>(x, g, m, v, nullptr, n / 4, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, gscale, nullptr);
  else
    adamw_fused_kernel<1><<<grid, OPT_THREADS, 0, st>>>(x, g, m, v, u_out, n / 4, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, gscale, acc);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
