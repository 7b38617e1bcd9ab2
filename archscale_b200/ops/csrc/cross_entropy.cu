// Cross-entropy forward + backward over a chunk of logits, in place.
// One CTA per row: pass 1 computes the running max / sum-exp (online softmax) and Σx with 16-byte
// loads, pass 2 re-reads the row (L2-resident) and overwrites it with d loss / d logits:
//   p·(1 + 2·z·lse) − (1−ε)·onehot(target) − ε/V          (0 for ignored rows)
// loss[row] = (1−ε)(lse − x_t) + ε(lse − mean x) + z·lse².
#include <cstring>
#include <type_traits>
#include "sm100.cuh"
#include "api.h"

namespace b200 {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T, int VEC>
__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ target,
                                                         float* __restrict__ loss, int vocab, int64_t row_stride,
                                                         int ignore_index, float eps_ls, float zs) {
  __shared__ float red_m[16], red_s[16], red_x[16];
  __shared__ float s_lse, s_sumx;
  const int row = blockIdx.x;
  T* x = logits + static_cast<size_t>(row) * row_stride;
  const int64_t tgt = target[row];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int nvec = vocab / VEC;
  typedef typename std::conditional<sizeof(T) == 2, uint4, float4>::type VT;  // 16 bytes
  if (tgt == ignore_index) {
    VT z; memset(&z, 0, sizeof(z));
    for (int i = tid; i < nvec; i += nthr) reinterpret_cast<VT*>(x)[i] = z;
    for (int i = nvec * VEC + tid; i < vocab; i += nthr) x[i] = from_f<T>(0.f);
    if (tid == 0) loss[row] = 0.f;
    return;
  }
  float m = -INFINITY, s = 0.f, sx = 0.f;
  for (int i = tid; i < nvec; i += nthr) {
    VT v = reinterpret_cast<const VT*>(x)[i];
    const T* e = reinterpret_cast<const T*>(&v);
    float f[VEC]; float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < VEC; ++j) { f[j] = to_f<T>(e[j]); lm = fmaxf(lm, f[j]); sx += f[j]; }
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc; m = nm;
  }
  for (int i = nvec * VEC + tid; i < vocab; i += nthr) {
    const float f = to_f<T>(x[i]); sx += f;
    const float nm = fmaxf(m, f); s = s * __expf(m - nm) + __expf(f - nm); m = nm;
  }
  // block reduce (max, sum) pairs
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm)); m = nm;
    sx += __shfl_xor_sync(0xffffffffu, sx, o);
  }
  const int warp = tid >> 5, lane = tid & 31, nw = nthr >> 5;
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; red_x[warp] = sx; }
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? red_m[lane] : -INFINITY; s = lane < nw ? red_s[lane] : 0.f; sx = lane < nw ? red_x[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm)); m = nm;
      sx += __shfl_xor_sync(0xffffffffu, sx, o);
    }
    if (lane == 0) { s_lse = m + __logf(s); s_sumx = sx; }
  }
  __syncthreads();
  const float lse = s_lse;
  const float xt = to_f<T>(x[tgt]);
  __syncthreads();  // everyone has read x[tgt] before it is overwritten
  const float pscale = 1.f + 2.f * zs * lse;
  const float sub = eps_ls / vocab;
  for (int i = tid; i < nvec; i += nthr) {
    VT v = reinterpret_cast<const VT*>(x)[i];
    T* e = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int idx = i * VEC + j;
      float g = __expf(to_f<T>(e[j]) - lse) * pscale - sub;
      if (idx == tgt) g -= (1.f - eps_ls);
      e[j] = from_f<T>(g);
    }
    reinterpret_cast<VT*>(x)[i] = v;
  }
  for (int i = nvec * VEC + tid; i < vocab; i += nthr) {
    float g = __expf(to_f<T>(x[i]) - lse) * pscale - sub;
    if (i == tgt) g -= (1.f - eps_ls);
    x[i] = from_f<T>(g);
  }
  if (tid == 0) loss[row] = (1.f - eps_ls) * (lse - xt) + eps_ls * (lse - s_sumx / vocab) + zs * lse * lse;
}

}  // namespace b200

extern "C" int b200_cross_entropy_fwd_bwd(void* logits, int dtype, const int64_t* target, float* loss, int rows, int vocab,
                                          int64_t row_stride, int ignore_index, float label_smoothing,
                                          float lse_square_scale, cudaStream_t stream) {
  using namespace b200;
  if (rows == 0) return 0;
  if (dtype == 1) {
    if ((row_stride % 8) || (reinterpret_cast<uintptr_t>(logits) % 16)) return -1;
    ce_fwd_bwd_kernel<__nv_bfloat16, 8><<<rows, 512, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), target, loss, vocab,
                                                                  row_stride, ignore_index, label_smoothing, lse_square_scale);
  } else {
    if ((row_stride % 4) || (reinterpret_cast<uintptr_t>(logits) % 16)) return -1;
    ce_fwd_bwd_kernel<float, 4><<<rows, 512, 0, stream>>>(static_cast<float*>(logits), target, loss, vocab, row_stride,
                                                           ignore_index, label_smoothing, lse_square_scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
