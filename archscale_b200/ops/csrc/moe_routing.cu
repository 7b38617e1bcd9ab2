// MoE routing without a host round trip.
//
//   topk_indices      per token: indices of the K largest of E router logits, ties to the lower index
//                     (the `stable_topk` rule of the reference, lit_gpt/moe.py:33-39); E ≤ 256, K ≤ 16
//   routing_layout    stable counting sort of the N·K (token, slot) pairs by expert into a layout where
//                     every expert's segment starts at a multiple of 256 rows (so GEMM tiles never
//                     straddle experts and the wgrad K-loop never reads a neighbour's rows):
//                       counts[E], offsets[E+1] (padded), slot_pair[capacity] (pair id or −1), pair_slot[N·K]
//                     three small kernels: per-chunk histograms → per-chunk bases → stable placement
//   gather_rows       xs[slot] = x[pair/K] (zeros in padding slots), optionally scaled per pair
//   combine_rows      out[t] = Σ_k w[t,k] · y[pair_slot[t·K+k]]      (deterministic, no atomics)
//   pair_dots         d w[t,k] = <y[slot], dout[t]>                   (gradient of the gate weights)
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int RT_CHUNK = 2048;   // pairs per CTA in the layout kernels
constexpr int RT_ALIGN = 256;    // expert segments start at multiples of this many rows (one tile of the two-CTA grouped GEMM)

template <int E_MAX>
__global__ void __launch_bounds__(128) topk_indices_kernel(const float* __restrict__ logits, int* __restrict__ idx, int N, int E, int K) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= N) return;
  float v[E_MAX];
  const float* row = logits + static_cast<size_t>(t) * E;
#pragma unroll
  for (int e = 0; e < E_MAX; ++e) v[e] = e < E ? row[e] : -INFINITY;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY; int bi = 0;
#pragma unroll
    for (int e = 0; e < E_MAX; ++e) if (v[e] > best) { best = v[e]; bi = e; }   // strict > keeps the lowest index on ties
    idx[static_cast<size_t>(t) * K + k] = bi;
#pragma unroll
    for (int e = 0; e < E_MAX; ++e) if (e == bi) v[e] = -INFINITY;
  }
}

// hist[chunk][e]
__global__ void __launch_bounds__(256) route_hist_kernel(const int* __restrict__ expert_of_pair, int n_pairs, int E,
                                                         int* __restrict__ hist) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * RT_CHUNK;
  for (int i = threadIdx.x; i < RT_CHUNK; i += blockDim.x) {
    const int pidx = base + i;
    if (pidx < n_pairs) atomicAdd(&sh[expert_of_pair[pidx]], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[static_cast<size_t>(blockIdx.x) * E + e] = sh[e];
}

// one CTA; thread e: counts[e], padded offsets, base[chunk][e] = offsets[e] + Σ_{c'<chunk} hist[c'][e]
__global__ void __launch_bounds__(256) route_scan_kernel(const int* __restrict__ hist, int n_chunks, int E, int* __restrict__ counts,
                                                         int* __restrict__ offsets, int* __restrict__ base) {
  __shared__ int s_cnt[256], s_off[257];
  const int e = threadIdx.x;
  int total = 0;
  if (e < E) for (int c = 0; c < n_chunks; ++c) total += hist[static_cast<size_t>(c) * E + e];
  s_cnt[e] = e < E ? total : 0;
  __syncthreads();
  if (e == 0) {
    int acc = 0;
    for (int i = 0; i < E; ++i) { s_off[i] = acc; acc += (s_cnt[i] + RT_ALIGN - 1) / RT_ALIGN * RT_ALIGN; }
    s_off[E] = acc;
  }
  __syncthreads();
  if (e < E) {
    counts[e] = s_cnt[e];
    offsets[e] = s_off[e];
    int run = s_off[e];
    for (int c = 0; c < n_chunks; ++c) { base[static_cast<size_t>(c) * E + e] = run; run += hist[static_cast<size_t>(c) * E + e]; }
  }
  if (e == 0) offsets[E] = s_off[E];
}

// stable placement inside each chunk: pairs are visited in rounds of 256 in pair-id order
__global__ void __launch_bounds__(256) route_place_kernel(const int* __restrict__ expert_of_pair, int n_pairs, int E,
                                                          const int* __restrict__ base, int* __restrict__ slot_pair,
                                                          int* __restrict__ pair_slot) {
  extern __shared__ int sh[];          // running[E] then warp_cnt[8][E]
  int* running = sh;
  int* warp_cnt = sh + E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) running[e] = base[static_cast<size_t>(blockIdx.x) * E + e];
  __syncthreads();
  const int chunk0 = blockIdx.x * RT_CHUNK;
  for (int round = 0; round < RT_CHUNK / 256; ++round) {
    const int pidx = chunk0 + round * 256 + threadIdx.x;
    const bool valid = pidx < n_pairs;
    const int e = valid ? expert_of_pair[pidx] : -1;
    for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) warp_cnt[i] = 0;
    __syncthreads();
    // rank inside the warp among lanes with the same expert
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1));
    if (valid && rank_in_warp == 0) warp_cnt[warp * E + e] = __popc(same);
    __syncthreads();
    if (valid) {
      int before = 0;
      for (int w = 0; w < warp; ++w) before += warp_cnt[w * E + e];
      const int slot = running[e] + before + rank_in_warp;
      slot_pair[slot] = pidx;
      pair_slot[pidx] = slot;
    }
    __syncthreads();
    for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
      int tot = 0;
      for (int w = 0; w < 8; ++w) tot += warp_cnt[w * E + ee];
      running[ee] += tot;
    }
    __syncthreads();
  }
}

// xs[slot, :] = scale · x[pair / K, :]   (bf16 rows of C elements, 16-byte vectors; zero for padding slots)
// A pair index outside [0, n_pairs) (a corrupted table) is reported in the status word and its row is written as zeros.
__global__ void __launch_bounds__(256) gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ slot_pair,
                                                          const float* __restrict__ pair_scale, __nv_bfloat16* __restrict__ xs,
                                                          int capacity, int C, int K, const int* __restrict__ offsets, int E,
                                                          int n_pairs, int* __restrict__ status) {
  const int vec_per_row = C / 8;
  const int used = offsets[E];
  // one (index -> row -> store) chain per thread and pass; four independent chains per thread were measured slower
  // (0.45 against 0.36 ms for 524,288 rows of 2 KB): the kernel runs at the rate at which 1 GB can be written
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < static_cast<size_t>(used) * vec_per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int slot = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i % vec_per_row) * 8;
    int pr = slot_pair[slot];
    if (pr >= n_pairs) {
      if (status) atomicCAS(status, 0, STATUS_INDEX_RANGE);
      pr = -1;
    }
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (pr >= 0) {
      v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(pr / K) * C + c);
      if (pair_scale) {
        const float s = pair_scale[pr];
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); w[e] = pack_bf16x2(f.x * s, f.y * s); }
        v = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    *reinterpret_cast<uint4*>(xs + static_cast<size_t>(slot) * C + c) = v;
  }
}

// out[t, :] = alpha · (Σ_k w[t,k] · y[pair_slot[t·K + k], :] + add[t, :])      (add may be null)
__global__ void __launch_bounds__(256) combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pair_slot,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int N, int C,
                                                           int K, const __nv_bfloat16* __restrict__ add, float alpha, int capacity,
                                                           int* __restrict__ status) {
  const int vec_per_row = C / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < static_cast<size_t>(N) * vec_per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i % vec_per_row) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (add) {
      const uint4 v = *reinterpret_cast<const uint4*>(add + static_cast<size_t>(t) * C + c);
      const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(ww[e]); acc[2 * e] = f.x; acc[2 * e + 1] = f.y; }
    }
    for (int k = 0; k < K; ++k) {
      const int slot = pair_slot[static_cast<size_t>(t) * K + k];
      if (slot < 0 || slot >= capacity) {            // a slot outside the row buffer: reported, contributes nothing
        if (status) atomicCAS(status, 0, STATUS_INDEX_RANGE);
        continue;
      }
      const float wk = w ? w[static_cast<size_t>(t) * K + k] : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(slot) * C + c);
      const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(ww[e]); acc[2 * e] += wk * f.x; acc[2 * e + 1] += wk * f.y; }
    }
    uint4 o;
    o.x = pack_bf16x2(alpha * acc[0], alpha * acc[1]); o.y = pack_bf16x2(alpha * acc[2], alpha * acc[3]);
    o.z = pack_bf16x2(alpha * acc[4], alpha * acc[5]); o.w = pack_bf16x2(alpha * acc[6], alpha * acc[7]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * C + c) = o;
  }
}

// dots[pair] = <y[pair_slot[pair], :], g[pair / K, :]>     one warp per pair
__global__ void __launch_bounds__(256) pair_dots_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ g,
                                                        const int* __restrict__ pair_slot, float* __restrict__ dots, int n_pairs,
                                                        int C, int K, int capacity, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const size_t pr = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
  if (pr >= static_cast<size_t>(n_pairs)) return;
  const int slot = pair_slot[pr];
  if (slot < 0 || slot >= capacity) {                // warp-uniform: every lane reads the same slot
    if (lane == 0) { if (status) atomicCAS(status, 0, STATUS_INDEX_RANGE); dots[pr] = 0.f; }
    return;
  }
  const __nv_bfloat16* a = y + static_cast<size_t>(slot) * C;
  const __nv_bfloat16* b = g + (pr / K) * C;
  float s = 0.f;
  for (int c = lane * 8; c < C; c += 256) {
    const uint4 va = *reinterpret_cast<const uint4*>(a + c), vb = *reinterpret_cast<const uint4*>(b + c);
    const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 fa = unpack_bf16x2(wa[e]), fb = unpack_bf16x2(wb[e]); s += fa.x * fb.x + fa.y * fb.y; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) dots[pr] = s;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_topk_indices(const float* logits, int* idx, int N, int E, int K, cudaStream_t st) {
  if (N == 0) return 0;
  if (E > 256 || K > E) return -1;
  const int grid = (N + 127) / 128;
  if (E <= 64) topk_indices_kernel<64><<<grid, 128, 0, st>>>(logits, idx, N, E, K);
  else if (E <= 128) topk_indices_kernel<128><<<grid, 128, 0, st>>>(logits, idx, N, E, K);
  else topk_indices_kernel<256><<<grid, 128, 0, st>>>(logits, idx, N, E, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_routing_chunks(int n_pairs) { return (n_pairs + RT_CHUNK - 1) / RT_CHUNK; }
extern "C" int b200_routing_capacity(int n_pairs, int E) { return (n_pairs + E * (RT_ALIGN - 1) + RT_ALIGN - 1) / RT_ALIGN * RT_ALIGN; }

// scratch: int32 [2 · n_chunks · E]
extern "C" int b200_routing_layout(const int* expert_of_pair, int n_pairs, int E, int* counts, int* offsets, int* slot_pair,
                                   int* pair_slot, int capacity, int* scratch, cudaStream_t st) {
  if (E > 256) return -1;
  const int n_chunks = b200_routing_chunks(n_pairs);
  int* hist = scratch;
  int* base = scratch + static_cast<size_t>(n_chunks) * E;
  if (cudaMemsetAsync(slot_pair, 0xff, sizeof(int) * capacity, st) != cudaSuccess) return -3;   // −1 = padding
  route_hist_kernel<<<n_chunks, 256, E * sizeof(int), st>>>(expert_of_pair, n_pairs, E, hist);
  route_scan_kernel<<<1, 256, 0, st>>>(hist, n_chunks, E, counts, offsets, base);
  route_place_kernel<<<n_chunks, 256, 9 * E * sizeof(int), st>>>(expert_of_pair, n_pairs, E, base, slot_pair, pair_slot);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_gather_rows(const void* x, const int* slot_pair, const float* pair_scale, void* xs, int capacity, int C,
                                int K, const int* offsets, int E, cudaStream_t st, int n_pairs, int* status) {
  if (C % 8) return -1;
  gather_rows_kernel<<<148 * 8, 256, 0, st>>>((const __nv_bfloat16*)x, slot_pair, pair_scale, (__nv_bfloat16*)xs, capacity, C, K,
                                              offsets, E, n_pairs, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_combine_rows(const void* y, const int* pair_slot, const float* w, void* out, int N, int C, int K,
                                 const void* add, float alpha, cudaStream_t st, int capacity, int* status) {
  if (C % 8) return -1;
  if (N == 0) return 0;
  combine_rows_kernel<<<148 * 8, 256, 0, st>>>((const __nv_bfloat16*)y, pair_slot, w, (__nv_bfloat16*)out, N, C, K,
                                             (const __nv_bfloat16*)add, alpha, capacity, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_pair_dots(const void* y, const void* g, const int* pair_slot, float* dots, int n_pairs, int C, int K,
                              cudaStream_t st, int capacity, int* status) {
  if (C % 8) return -1;
  if (n_pairs == 0) return 0;
  const size_t threads = static_cast<size_t>(n_pairs) * 32;
  pair_dots_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)g,
                                                                           pair_slot, dots, n_pairs, C, K, capacity, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
