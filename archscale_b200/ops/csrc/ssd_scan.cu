// The sequential part of the chunked SSD (Mamba-2) scan: the state that enters each chunk,
//     S_in[0] = 0,   S_in[n+1] = keep[n] · S_in[n] + add[n]
// over the chunks n of one sequence, for every element of the (heads × head_dim × state) state.  Everything around it
// (the quadratic work inside a chunk, the chunk summaries `add`, the outputs from S_in) is batched matrix products; this
// recurrence is what the reference's `mamba_chunk_scan_combined` (`lit_gpt/mamba2.py:229-253,289-305`) runs in its
// state-passing kernel.  In PyTorch it is a loop of 2·chunks small element-wise launches plus as many again in autograd.
//
// Layouts: add, S_in, d_S_in, d_add  [B, nC, E] fp32 with E = H · PN (PN = head_dim · state, a multiple of 1024);
// keep [B, nC, H]; d_keep_part [B, nC, H, PN / 1024] (summed by the caller: fixed order, reproducible).
// One thread owns four consecutive state elements for the whole sequence; a CTA of 256 threads covers 1024 elements of one
// head, so the per-chunk sums of the backward pass (d keep = Σ G·S over the head's state) are block reductions.
#include <cuda_runtime.h>

#include "api.h"

namespace b200 {

__global__ void __launch_bounds__(256) ssd_state_fwd_kernel(const float4* __restrict__ add, const float* __restrict__ keep,
                                                           float4* __restrict__ s_in, int nC, int H, int PN) {
  const int b = blockIdx.y;
  const size_t e4 = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;          // float4 index inside [E]
  const int h = static_cast<int>(blockIdx.x / (PN / 1024));
  const size_t E4 = static_cast<size_t>(H) * PN / 4;
  const float4* a = add + static_cast<size_t>(b) * nC * E4 + e4;
  float4* o = s_in + static_cast<size_t>(b) * nC * E4 + e4;
  const float* kp = keep + static_cast<size_t>(b) * nC * H + h;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int U = 8;                                  // loads of U chunks are in flight before the dependent FMAs
  for (int n0 = 0; n0 < nC; n0 += U) {
    float4 av[U]; float kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (n0 + u < nC) { av[u] = a[static_cast<size_t>(n0 + u) * E4]; kv[u] = kp[static_cast<size_t>(n0 + u) * H]; }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (n0 + u < nC) {
        o[static_cast<size_t>(n0 + u) * E4] = s;
        s.x = fmaf(s.x, kv[u], av[u].x); s.y = fmaf(s.y, kv[u], av[u].y);
        s.z = fmaf(s.z, kv[u], av[u].z); s.w = fmaf(s.w, kv[u], av[u].w);
      }
  }
}

// G = gradient w.r.t. the state after chunk n (zero after the last chunk: the final state is not an output).
//   d_add[n] = G;   d_keep[n] += Σ G · S_in[n];   G ← d_S_in[n] + keep[n] · G
__global__ void __launch_bounds__(256) ssd_state_bwd_kernel(const float4* __restrict__ d_s_in, const float4* __restrict__ s_in,
                                                           const float* __restrict__ keep, float4* __restrict__ d_add,
                                                           float* __restrict__ d_keep_part, int nC, int H, int PN) {
  __shared__ float red[8];
  const int b = blockIdx.y;
  const int per_head = PN / 1024;
  const size_t e4 = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
  const int h = static_cast<int>(blockIdx.x / per_head), part = static_cast<int>(blockIdx.x % per_head);
  const size_t E4 = static_cast<size_t>(H) * PN / 4;
  const size_t base = static_cast<size_t>(b) * nC * E4 + e4;
  const float* kp = keep + static_cast<size_t>(b) * nC * H + h;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int U = 4;
  for (int n1 = nC; n1 > 0; n1 -= U) {
    float4 dv[U], sv[U]; float kv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int n = n1 - 1 - u;
      if (n >= 0) { dv[u] = d_s_in[base + static_cast<size_t>(n) * E4]; sv[u] = s_in[base + static_cast<size_t>(n) * E4]; kv[u] = kp[static_cast<size_t>(n) * H]; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int n = n1 - 1 - u;
      if (n < 0) break;
      d_add[base + static_cast<size_t>(n) * E4] = g;
      float dk = g.x * sv[u].x + g.y * sv[u].y + g.z * sv[u].z + g.w * sv[u].w;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dk += __shfl_xor_sync(0xffffffffu, dk, o);
      if (lane == 0) red[warp] = dk;
      __syncthreads();
      if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        d_keep_part[((static_cast<size_t>(b) * nC + n) * H + h) * per_head + part] = t;
      }
      __syncthreads();
      g.x = fmaf(g.x, kv[u], dv[u].x); g.y = fmaf(g.y, kv[u], dv[u].y);
      g.z = fmaf(g.z, kv[u], dv[u].z); g.w = fmaf(g.w, kv[u], dv[u].w);
    }
  }
}

}  // namespace b200

extern "C" int b200_ssd_state_fwd(const float* add, const float* keep, float* s_in, int B, int nC, int H, int PN, cudaStream_t st) {
  if (B <= 0 || nC <= 0) return 0;
  if (PN % 1024) return -1;
  using namespace b200;
  ssd_state_fwd_kernel<<<dim3(H * (PN / 1024), B), 256, 0, st>>>(reinterpret_cast<const float4*>(add), keep,
                                                                 reinterpret_cast<float4*>(s_in), nC, H, PN);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_ssd_state_bwd(const float* d_s_in, const float* s_in, const float* keep, float* d_add, float* d_keep_part,
                                  int B, int nC, int H, int PN, cudaStream_t st) {
  if (B <= 0 || nC <= 0) return 0;
  if (PN % 1024) return -1;
  using namespace b200;
  ssd_state_bwd_kernel<<<dim3(H * (PN / 1024), B), 256, 0, st>>>(reinterpret_cast<const float4*>(d_s_in),
                                                                 reinterpret_cast<const float4*>(s_in), keep,
                                                                 reinterpret_cast<float4*>(d_add), d_keep_part, nC, H, PN);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
