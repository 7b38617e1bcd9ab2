// Peer-memory collectives over NVLink 5 / NVSwitch with plain loads and stores (no NCCL, no multicast).
// Every rank owns a "symmetric heap" (one cudaMalloc block, same size on all ranks, mapped into every
// peer with CUDA IPC); an object lives at the same offset in every heap, so a kernel reaches rank p's
// copy through `peers[p] + offset`.
//
//   symm_barrier            all ranks signal all peers and wait (bounded) — a device-side barrier
//   allgather_pull          local_full[p·S .. (p+1)·S) ← peer p's shard, for all p (16-byte loads)
//   reduce_scatter_pull     out[i] (+)= scale · Σ_p peer_p.full[r·S + i]   fp32, fixed rank order
//   gather_ranges / …       used by the distributed Muon step (flat U → owner, O → shards)
//
// Signals are 32-bit epoch counters in the heaps' signal areas: a rank writes `epoch` into slot
// [its rank] of every peer with a system-scope release store; waiting is an acquire load in a spin
// bounded by a clock limit, after which the kernel records STATUS_TIMEOUT_PEER and returns.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

struct Peers {
  void* base[8];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Returns false on timeout.  Epochs only grow; wrap-around safe comparison.
__device__ __forceinline__ bool wait_signal(const uint32_t* slot, uint32_t epoch, int* status, long long limit) {
  long long t0 = clock64();
  while (static_cast<int32_t>(ld_acquire_sys(slot) - epoch) < 0) {
    if (clock64() - t0 > limit) {
      if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// One CTA of `world` threads.  signal area layout: uint32 slots[channel][8].
__global__ void symm_barrier_kernel(Peers peers, size_t signal_off, int channel, int rank, int world, uint32_t epoch,
                                    int* status, long long limit) {
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();
  uint32_t* theirs = reinterpret_cast<uint32_t*>(static_cast<char*>(peers.base[p]) + signal_off) + channel * 8 + rank;
  st_release_sys(theirs, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(static_cast<char*>(peers.base[rank]) + signal_off) + channel * 8 + p;
  wait_signal(mine, epoch, status, limit);
}

// Post-only / wait-only halves (producer signals "my data for `channel` is ready"; consumers wait for all peers).
__global__ void symm_post_kernel(Peers peers, size_t signal_off, int channel, int rank, int world, uint32_t epoch) {
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<uint32_t*>(static_cast<char*>(peers.base[p]) + signal_off) + channel * 8 + rank, epoch);
}
__global__ void symm_wait_kernel(Peers peers, size_t signal_off, int channel, int rank, int world, uint32_t epoch,
                                 int* status, long long limit) {
  const int p = threadIdx.x;
  if (p >= world) return;
  wait_signal(reinterpret_cast<const uint32_t*>(static_cast<char*>(peers.base[rank]) + signal_off) + channel * 8 + p,
              epoch, status, limit);
}

// dst (local, contiguous [world · shard_bytes]) ← every peer's shard at heap offset src_off.
__global__ void __launch_bounds__(512) allgather_pull_kernel(Peers peers, size_t src_off, uint4* __restrict__ dst,
                                                            size_t shard_vec /* uint4 per shard */, int rank, int world) {
  // 8 independent 16-byte loads in flight per thread: NVLink latency is ~µs, so bandwidth = bytes in flight
  constexpr int U = 8;
  const size_t chunk = static_cast<size_t>(blockDim.x) * U;
  const size_t chunks_per_shard = (shard_vec + chunk - 1) / chunk;
  const size_t total_chunks = chunks_per_shard * world;
  for (size_t c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    // start with the next rank so that the ranks do not all read the same peer at once
    const int step = static_cast<int>(c / chunks_per_shard);
    const int p = (rank + step) % world;
    const size_t j0 = (c - static_cast<size_t>(step) * chunks_per_shard) * chunk + threadIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.base[p]) + src_off);
    uint4* d = dst + static_cast<size_t>(p) * shard_vec;
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) { const size_t j = j0 + static_cast<size_t>(u) * blockDim.x; if (j < shard_vec) v[u] = src[j]; }
#pragma unroll
    for (int u = 0; u < U; ++u) { const size_t j = j0 + static_cast<size_t>(u) * blockDim.x; if (j < shard_vec) d[j] = v[u]; }
  }
}

// out[i] = (accumulate ? out[i] : 0) + scale · Σ_p full_p[rank·S + i]; full_p at heap offset full_off, fp32.
__global__ void __launch_bounds__(256) reduce_scatter_pull_kernel(Peers peers, size_t full_off, float4* __restrict__ out,
                                                                 size_t shard_vec /* float4 per shard */, int rank,
                                                                 int world, float scale, int accumulate) {
  // The loads from all (≤ 8) peers for U vectors are issued before any of them is consumed: with a
  // round trip of several µs over NVLink, throughput is the number of bytes in flight.
  constexpr int U = 2;
  const float4* src[8];
#pragma unroll
  for (int p = 0; p < 8; ++p)
    src[p] = reinterpret_cast<const float4*>(static_cast<const char*>(peers.base[p < world ? p : 0]) + full_off) +
             static_cast<size_t>(rank) * shard_vec;
  const size_t chunk = static_cast<size_t>(blockDim.x) * U;
  for (size_t c0 = blockIdx.x * chunk; c0 < shard_vec; c0 += static_cast<size_t>(gridDim.x) * chunk) {
    float4 v[8][U];
#pragma unroll
    for (int p = 0; p < 8; ++p)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = c0 + threadIdx.x + static_cast<size_t>(u) * blockDim.x;
        v[p][u] = (p < world && i < shard_vec) ? src[p][i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = c0 + threadIdx.x + static_cast<size_t>(u) * blockDim.x;
      if (i >= shard_vec) continue;
      float4 a = v[0][u];
#pragma unroll
      for (int p = 1; p < 8; ++p) {   // fixed rank order → bitwise reproducible
        a.x += v[p][u].x; a.y += v[p][u].y; a.z += v[p][u].z; a.w += v[p][u].w;
      }
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
      if (accumulate) { const float4 o = out[i]; a.x += o.x; a.y += o.y; a.z += o.z; a.w += o.w; }
      out[i] = a;
    }
  }
}

// Same as reduce_scatter_pull for a 16-bit payload summed in fp32 (Muon: O returns to the shards; every
// element is non-zero on exactly one rank, so the sum is exact).
__global__ void __launch_bounds__(256) reduce_scatter_pull_bf16_kernel(Peers peers, size_t full_off, uint4* __restrict__ out,
                                                                      size_t shard_vec /* uint4 (8 bf16) per shard */,
                                                                      int rank, int world) {
  constexpr int U = 2;
  const uint4* src[8];
#pragma unroll
  for (int p = 0; p < 8; ++p)
    src[p] = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.base[p < world ? p : 0]) + full_off) +
             static_cast<size_t>(rank) * shard_vec;
  const size_t chunk = static_cast<size_t>(blockDim.x) * U;
  for (size_t c0 = blockIdx.x * chunk; c0 < shard_vec; c0 += static_cast<size_t>(gridDim.x) * chunk) {
    uint4 v[8][U];
#pragma unroll
    for (int p = 0; p < 8; ++p)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = c0 + threadIdx.x + static_cast<size_t>(u) * blockDim.x;
        v[p][u] = (p < world && i < shard_vec) ? src[p][i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t i = c0 + threadIdx.x + static_cast<size_t>(u) * blockDim.x;
      if (i >= shard_vec) continue;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const uint32_t w[4] = {v[p][u].x, v[p][u].y, v[p][u].z, v[p][u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); acc[2 * e] += f.x; acc[2 * e + 1] += f.y; }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      out[i] = o;
    }
  }
}

static inline int comm_grid(size_t vecs, int max_ctas) {
  size_t b = (vecs + 511) / 512;
  if (b < 1) b = 1;
  return static_cast<int>(b < static_cast<size_t>(max_ctas) ? b : max_ctas);
}

}  // namespace b200

using namespace b200;

// Peers may be seconds apart (lazy initialisation in the first steps), so waits on a peer use a far
// longer limit than waits inside one kernel; tests of the timeout path shorten it.
static long long g_peer_wait_limit = 120000000000LL;   // ≈ 60 s
extern "C" void b200_set_peer_wait_limit_cycles(long long cycles) { g_peer_wait_limit = cycles; }

static Peers make_peers(const void* const* bases, int world) {
  Peers p;
  for (int i = 0; i < 8; ++i) p.base[i] = i < world ? const_cast<void*>(bases[i]) : nullptr;
  return p;
}

extern "C" int b200_symm_barrier(const void* const* bases, size_t signal_off, int channel, int rank, int world,
                                 uint32_t epoch, int* status, cudaStream_t st) {
  if (world > 8) return -1;
  symm_barrier_kernel<<<1, 32, 0, st>>>(make_peers(bases, world), signal_off, channel, rank, world, epoch, status, g_peer_wait_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_symm_post(const void* const* bases, size_t signal_off, int channel, int rank, int world,
                              uint32_t epoch, cudaStream_t st) {
  if (world > 8) return -1;
  symm_post_kernel<<<1, 32, 0, st>>>(make_peers(bases, world), signal_off, channel, rank, world, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_symm_wait(const void* const* bases, size_t signal_off, int channel, int rank, int world,
                              uint32_t epoch, int* status, cudaStream_t st) {
  if (world > 8) return -1;
  symm_wait_kernel<<<1, 32, 0, st>>>(make_peers(bases, world), signal_off, channel, rank, world, epoch, status, g_peer_wait_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_allgather_pull(const void* const* bases, size_t src_off, void* dst, size_t shard_bytes, int rank,
                                   int world, int max_ctas, cudaStream_t st) {
  if (world > 8 || shard_bytes % 16 || src_off % 16) return -1;
  const size_t sv = shard_bytes / 16;
  allgather_pull_kernel<<<comm_grid(sv * world, max_ctas), 512, 0, st>>>(make_peers(bases, world), src_off,
                                                                         static_cast<uint4*>(dst), sv, rank, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_reduce_scatter_pull(const void* const* bases, size_t full_off, float* out, size_t shard_elems, int rank,
                                        int world, float scale, int accumulate, int max_ctas, cudaStream_t st) {
  if (world > 8 || shard_elems % 4 || full_off % 16) return -1;
  const size_t sv = shard_elems / 4;
  reduce_scatter_pull_kernel<<<comm_grid(sv, max_ctas), 256, 0, st>>>(make_peers(bases, world), full_off,
                                                                      reinterpret_cast<float4*>(out), sv, rank, world,
                                                                      scale, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_reduce_scatter_pull_bf16(const void* const* bases, size_t full_off, void* out, size_t shard_elems,
                                             int rank, int world, int max_ctas, cudaStream_t st) {
  if (world > 8 || shard_elems % 8 || full_off % 16) return -1;
  const size_t sv = shard_elems / 8;
  reduce_scatter_pull_bf16_kernel<<<comm_grid(sv, max_ctas), 256, 0, st>>>(make_peers(bases, world), full_off,
                                                                           static_cast<uint4*>(out), sv, rank, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
