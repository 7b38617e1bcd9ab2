// Peer-memory collectives over NVLink 5 / NVSwitch with plain loads and stores (no NCCL, no multicast).
// Every rank owns a "symmetric heap" (one cudaMalloc block, same size on all ranks, mapped into every
// peer with CUDA IPC); an object lives at the same offset in every heap, so a kernel reaches rank p's
// copy through `peers[p] + offset`.
//
//   symm_barrier            all ranks signal all peers and wait (bounded) — a device-side barrier
//   allgather_pull          local_full[p·S .. (p+1)·S) ← peer p's shard, for all p (16-byte loads)
//   reduce_scatter_pull     out[i] (+)= scale · Σ_p peer_p.full[r·S + i]   fp32, fixed rank order
//   pull_pieces             a host-built list of ranges copied from named peers (Muon: U → owners, O → shards)
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

// A list of copies from peers: piece i moves `len` 16-byte vectors from vector `src` of the object at heap offset `obj_off`
// in rank `rank`'s heap to vector `dst` of the local buffer.  The table is built once on the host (the owned matrices of
// the Muon step never change) with every piece cut to at most kPiece vectors, so one CTA takes one piece per round.
struct PullPiece {
  long long src, dst;
  int len, rank;
};
constexpr int kPullPieceVecs = 512 * 8;

__global__ void __launch_bounds__(512) pull_pieces_kernel(Peers peers, size_t obj_off, uint4* __restrict__ dst,
                                                         const PullPiece* __restrict__ table, int n_pieces) {
  constexpr int U = 8;
  for (int i = blockIdx.x; i < n_pieces; i += gridDim.x) {
    const PullPiece pc = table[i];
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(peers.base[pc.rank]) + obj_off) + pc.src;
    uint4* d = dst + pc.dst;
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) { const int j = threadIdx.x + u * 512; if (j < pc.len) v[u] = src[j]; }
#pragma unroll
    for (int u = 0; u < U; ++u) { const int j = threadIdx.x + u * 512; if (j < pc.len) d[j] = v[u]; }
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
// table: device array of n_pieces PullPiece records (see above); len ≤ 4096 vectors each.
extern "C" int b200_pull_pieces(const void* const* bases, size_t obj_off, void* dst, const void* table, int n_pieces,
                                int world, int max_ctas, cudaStream_t st) {
  if (world > 8 || obj_off % 16) return -1;
  if (n_pieces <= 0) return 0;
  const int grid = n_pieces < max_ctas ? n_pieces : max_ctas;
  pull_pieces_kernel<<<grid, 512, 0, st>>>(make_peers(bases, world), obj_off, static_cast<uint4*>(dst),
                                           static_cast<const PullPiece*>(table), n_pieces);
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

// ------------------------------------------------------------------------------------------------
// Expert-parallel dispatch / combine by peer pulls.  Every rank publishes in its heap:
//   send rows   [rows_cap, C] bf16, expert-sorted (segment of expert e starts at offsets[e], counts[e] rows)
//   counts[E], offsets[E+1]
// The owner of local expert e_l (global e = rank·E_l + e_l) lays its receive buffer out expert-major,
// sources in rank order inside an expert, expert segments starting at multiples of 256 rows, and records
// in `table[src][e_l]` where each source's rows start (sources read it to pull their results back).
namespace b200 {

struct EpArgs {
  const void* peer[8];
  size_t off_counts, off_offsets, off_table, off_send;   // heap offsets (same on every rank)
  char* recv_local;        // destination of the pulled rows (local memory, recv_cap rows)
  int rank, world, e_local, C, recv_cap;
};

// one CTA: build recv_offsets[e_local+1] (local device array) and table (in my heap); flag overflow
__global__ void ep_plan_kernel(EpArgs a, int* __restrict__ recv_offsets, int* status) {
  __shared__ int s_total[256];
  const int el = threadIdx.x;
  if (el < a.e_local) {
    int tot = 0;
    for (int s = 0; s < a.world; ++s)
      tot += reinterpret_cast<const int*>(static_cast<const char*>(a.peer[s]) + a.off_counts)[a.rank * a.e_local + el];
    s_total[el] = tot;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < a.e_local; ++e) { recv_offsets[e] = acc; acc += (s_total[e] + 255) / 256 * 256; }
    recv_offsets[a.e_local] = acc;
    if (acc > a.recv_cap && status) atomicCAS(status, 0, STATUS_EP_OVERFLOW);
  }
  __syncthreads();
  if (el < a.e_local) {
    int* table = reinterpret_cast<int*>(static_cast<char*>(const_cast<void*>(a.peer[a.rank])) + a.off_table);
    int run = recv_offsets[el];
    for (int s = 0; s < a.world; ++s) {
      table[s * a.e_local + el] = run;
      run += reinterpret_cast<const int*>(static_cast<const char*>(a.peer[s]) + a.off_counts)[a.rank * a.e_local + el];
    }
  }
}

// grid (e_local, world, chunks): copy the rows of (source s, local expert el) into my recv buffer;
// the last source also zero-fills the padding rows of the expert segment.
__global__ void __launch_bounds__(256) ep_pull_kernel(EpArgs a, const int* __restrict__ recv_offsets) {
  const int el = blockIdx.x, s = blockIdx.y;
  const int e = a.rank * a.e_local + el;
  const char* src_base = static_cast<const char*>(a.peer[s]);
  const int cnt = reinterpret_cast<const int*>(src_base + a.off_counts)[e];
  const int src_row = reinterpret_cast<const int*>(src_base + a.off_offsets)[e];
  const int* table = reinterpret_cast<const int*>(static_cast<const char*>(a.peer[a.rank]) + a.off_table);
  const int dst_row = table[s * a.e_local + el];
  const int vec_per_row = a.C / 8;
  const uint4* src = reinterpret_cast<const uint4*>(src_base + a.off_send) + static_cast<size_t>(src_row) * vec_per_row;
  // second guard (the host refuses to launch this kernel when the plan exceeds the capacity)
  if (recv_offsets[a.e_local] > a.recv_cap || dst_row + cnt > a.recv_cap) return;
  uint4* dst = reinterpret_cast<uint4*>(a.recv_local) + static_cast<size_t>(dst_row) * vec_per_row;
  const size_t total = static_cast<size_t>(cnt) * vec_per_row;
  constexpr int U = 8;
  for (size_t i0 = (blockIdx.z * static_cast<size_t>(blockDim.x)) * U + threadIdx.x; i0 < total;
       i0 += static_cast<size_t>(gridDim.z) * blockDim.x * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) { const size_t i = i0 + static_cast<size_t>(u) * blockDim.x; if (i < total) v[u] = src[i]; }
#pragma unroll
    for (int u = 0; u < U; ++u) { const size_t i = i0 + static_cast<size_t>(u) * blockDim.x; if (i < total) dst[i] = v[u]; }
  }
  if (s == a.world - 1) {
    const size_t pad_begin = static_cast<size_t>(dst_row + cnt) * vec_per_row;
    const size_t pad_end = static_cast<size_t>(recv_offsets[el + 1]) * vec_per_row;
    uint4* base = reinterpret_cast<uint4*>(a.recv_local);
    for (size_t i = pad_begin + blockIdx.z * static_cast<size_t>(blockDim.x) + threadIdx.x; i < pad_end;
         i += static_cast<size_t>(gridDim.z) * blockDim.x)
      base[i] = make_uint4(0u, 0u, 0u, 0u);
  }
}

// grid (E, chunks): pull my rows of global expert e back from its owner's result buffer into `dst`
// (local, same expert-sorted layout as my send buffer).
__global__ void __launch_bounds__(256) ep_return_kernel(EpArgs a, size_t off_result, uint4* __restrict__ dst) {
  const int e = blockIdx.x;
  const int owner = e / a.e_local, el = e - owner * a.e_local;
  const char* me = static_cast<const char*>(a.peer[a.rank]);
  const int cnt = reinterpret_cast<const int*>(me + a.off_counts)[e];
  const int my_row = reinterpret_cast<const int*>(me + a.off_offsets)[e];
  const char* ob = static_cast<const char*>(a.peer[owner]);
  const int their_row = reinterpret_cast<const int*>(ob + a.off_table)[a.rank * a.e_local + el];
  const int vec_per_row = a.C / 8;
  const uint4* src = reinterpret_cast<const uint4*>(ob + off_result) + static_cast<size_t>(their_row) * vec_per_row;
  uint4* d = dst + static_cast<size_t>(my_row) * vec_per_row;
  const size_t total = static_cast<size_t>(cnt) * vec_per_row;
  constexpr int U = 8;
  for (size_t i0 = (blockIdx.y * static_cast<size_t>(blockDim.x)) * U + threadIdx.x; i0 < total;
       i0 += static_cast<size_t>(gridDim.y) * blockDim.x * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) { const size_t i = i0 + static_cast<size_t>(u) * blockDim.x; if (i < total) v[u] = src[i]; }
#pragma unroll
    for (int u = 0; u < U; ++u) { const size_t i = i0 + static_cast<size_t>(u) * blockDim.x; if (i < total) d[i] = v[u]; }
  }
}

}  // namespace b200

static b200::EpArgs make_ep(const void* const* bases, size_t off_counts, size_t off_offsets, size_t off_table, size_t off_send,
                            void* recv_local, int rank, int world, int e_local, int C, int recv_cap) {
  b200::EpArgs a;
  for (int i = 0; i < 8; ++i) a.peer[i] = i < world ? bases[i] : nullptr;
  a.off_counts = off_counts; a.off_offsets = off_offsets; a.off_table = off_table; a.off_send = off_send;
  a.recv_local = static_cast<char*>(recv_local);
  a.rank = rank; a.world = world; a.e_local = e_local; a.C = C; a.recv_cap = recv_cap;
  return a;
}

// Step 1: layout of the rows this rank will receive (recv_offsets[e_local+1], 256-aligned) and the table
// its peers read to find their results.  The caller reads recv_offsets[e_local] to size its buffers.
extern "C" int b200_ep_plan(const void* const* bases, size_t off_counts, size_t off_table, int rank, int world, int e_local,
                            int recv_cap, int* recv_offsets, int* status, cudaStream_t st) {
  if (world > 8 || e_local > 256) return -1;
  b200::EpArgs a = make_ep(bases, off_counts, 0, off_table, 0, nullptr, rank, world, e_local, 8, recv_cap);
  b200::ep_plan_kernel<<<1, 256, 0, st>>>(a, recv_offsets, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Step 2: pull the rows into `recv_local` (recv_cap rows of C bf16).
extern "C" int b200_ep_pull(const void* const* bases, size_t off_counts, size_t off_offsets, size_t off_table, size_t off_send,
                            void* recv_local, int rank, int world, int e_local, int C, int recv_cap,
                            const int* recv_offsets, cudaStream_t st) {
  if (world > 8 || e_local > 256 || C % 8) return -1;
  b200::EpArgs a = make_ep(bases, off_counts, off_offsets, off_table, off_send, recv_local, rank, world, e_local, C, recv_cap);
  b200::ep_pull_kernel<<<dim3(e_local, world, 8), 256, 0, st>>>(a, recv_offsets);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_ep_return(const void* const* bases, size_t off_counts, size_t off_offsets, size_t off_table,
                              size_t off_result, void* dst, int rank, int world, int e_local, int C, cudaStream_t st) {
  if (world > 8 || C % 8) return -1;
  b200::EpArgs a = make_ep(bases, off_counts, off_offsets, off_table, 0, nullptr, rank, world, e_local, C, 0);
  b200::ep_return_kernel<<<dim3(e_local * world, 4), 256, 0, st>>>(a, off_result, static_cast<uint4*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
