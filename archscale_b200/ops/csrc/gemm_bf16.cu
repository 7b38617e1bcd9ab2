// bf16 GEMM on the 5th-generation tensor cores:  D = alpha · op(A) · op(B) (+ beta · C)
//
// Persistent, warp-specialised kernel, one CTA per SM, 192 threads:
//   warp 0      TMA producer  — fills a 4-stage shared-memory ring (A 128×64, B 256×64 per stage)
//   warp 1      MMA issuer    — one thread issues tcgen05.mma (M128 × N256 × K16) into one of two
//                               256-column fp32 accumulators in tensor memory
//   warps 2..5  epilogue      — tcgen05.ld the finished accumulator (32 lanes × 32 columns per
//                               instruction), scale / add C, store bf16 or accumulate into fp32
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
//
// Operand layouts (all via TMA tensor maps with 128-byte swizzle, no multicast):
//   A: K-major   (row-major [M,K])  or MN-major (row-major [K,M], i.e. Aᵀ is stored)
//   B: K-major   (row-major [N,K])  or MN-major (row-major [K,N])
// which covers forward (NT), dgrad (NN) and wgrad (TN) of a linear layer without any transpose copy.
//
// All waits are bounded (sm100.cuh); on expiry the kernel records a status code and exits cleanly.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;

// All-gather fused into the GEMM (FSDP forward): the first `n_copy` CTAs do not compute; they pull every
// rank's low-precision shard (symmetric heap, NVLink loads) into the local gathered buffer `dst`, chunk by
// chunk in address order, and publish a flag per chunk.  The producer warp of a computing CTA waits
// (bounded) for the chunks that hold the rows of B it is about to load, so math on the first rows of
// the weight overlaps the transfer of the rest of the unit's parameters.
struct AgParams {
  const void* peer[8];     // heap bases as mapped in this process
  size_t src_off;          // offset of the low-precision shard in every heap
  char* dst;               // local gathered buffer (world · shard_bytes)
  size_t shard_bytes;
  size_t b_off;            // byte offset of B inside dst
  uint32_t* flags;         // one per chunk of dst, value = epoch when the chunk is complete
  uint32_t epoch;
  int rank, world, n_copy;
  int gather_a;            // 1: the gathered buffer is the A operand ([M, K] rows in rank order) instead of B
  size_t a_off;            // byte offset of A inside dst (gather_a)
};
constexpr size_t AG_CHUNK = 256 * 1024;

// GEMM with the reduce-scatter of its output fused in (tensor-parallel row-parallel layer, FUSED_AG = 2):
// every rank computes the full [M, N] partial product into `part` (its symmetric heap), finishing the row blocks of
// the other ranks' slices first and its own last; each epilogue warp bumps a per-row-block counter (release, system
// scope) after its stores.  By the time a rank reaches the tiles of its own slice its peers have (at equal speed)
// finished theirs for those rows: the epilogue of an own tile waits (bounded) for the peers' counters, adds their
// partial rows with loads from peer memory to the accumulator it just read from TMEM and writes `out_local`
// [M / world, N] — the transfer of a tile overlaps the main loop of the next one.
struct RsParams {
  const void* peer[8];     // heap bases as mapped in this process
  size_t part_off;         // offset of the [M, N] bf16 partial-product buffer in every heap
  size_t cnt_off;          // offset of the per-row-block counters (uint32, one per 128 rows) in every heap
  uint32_t expect;         // counter value that marks a complete row block for this call (4 warps · N tiles · calls)
  int rank, world;
  __nv_bfloat16* out_local;
};

// Grouped (mixture-of-experts) GEMMs.  Activations are stored expert-sorted with every expert's segment
// starting at a multiple of 128 rows (offsets[E+1], device memory, written by the routing kernels):
//   GROUPED = 1  rows grouped:  out[r, :] = A[r, :] · op(B[e(r)])   — B holds E matrices back to back
//                (forward up/down projection with B [E·N, K] K-major; dgrad with B [E·K, N] N-major)
//   GROUPED = 2  wgrad: out[e] (M×N) (+)= A[rows of e, :M]ᵀ · B[rows of e, :N]   (TN, K-loop over the segment)
struct GroupParams {
  const int* offsets;   // [E+1], multiples of 128
  int E;
  int b_rows;           // rows of one expert's matrix inside B (N for K-major B, K for N-major B)
};

struct GemmParams {
  void* out;
  const void* cin;
  int M, N, K;
  int ldc;          // row stride of out / cin in elements
  float alpha, beta;
  int accumulate;   // fp32 output: out += result
  int* status;
  // Serial split-K (fp32 accumulating output only): the K loop of every output tile is cut into `split_k` pieces that
  // different CTAs compute; they add their partial tile to `out` one after the other, in split order, handing over
  // through one counter per (tile, epilogue warp) in `sem` (zero between launches).  Fills the last wave of long-K
  // weight-gradient GEMMs whose tile count is a poor multiple of the SM count; the summation order stays fixed.
  int split_k;
  uint32_t* sem;
};


// Copier CTA: one thread drives bulk-asynchronous copies (peer global → shared → local global) through a
// 3-deep ring of 64 KiB buffers, so ~192 KiB are in flight per CTA; NVLink round trips are several µs and
// bandwidth is what is in flight.  A chunk's flag is published once the stores of its pieces completed.
constexpr int AG_PIECE = 64 * 1024, AG_BUFS = 3, AG_PIECES_PER_CHUNK = AG_CHUNK / AG_PIECE;

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}

__device__ void ag_copier(const AgParams& ag, uint8_t* smem, int* status) {
  if (threadIdx.x != 0) return;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AG_BUFS * AG_PIECE);
  volatile int abort_local = 0;
  for (int b = 0; b < AG_BUFS; ++b) mbar_init(&bars[b], 1);
  mbar_fence_init();
  const size_t total = ag.shard_bytes * ag.world;
  const size_t n_chunks = (total + AG_CHUNK - 1) / AG_CHUNK;
  const size_t my_chunks = n_chunks > blockIdx.x ? (n_chunks - blockIdx.x + ag.n_copy - 1) / ag.n_copy : 0;
  const size_t n_pieces = my_chunks * AG_PIECES_PER_CHUNK;
  auto piece_range = [&](size_t i, size_t& beg, size_t& end, size_t& chunk) {
    chunk = blockIdx.x + (i / AG_PIECES_PER_CHUNK) * ag.n_copy;
    beg = chunk * AG_CHUNK + (i % AG_PIECES_PER_CHUNK) * AG_PIECE;
    end = beg + AG_PIECE;
    if (beg > total) beg = total;
    if (end > total) end = total;
  };
  auto issue_load = [&](size_t i) {
    size_t beg, end, chunk; piece_range(i, beg, end, chunk);
    const int buf = static_cast<int>(i % AG_BUFS);
    if (end <= beg) { mbar_arrive(&bars[buf]); return; }
    mbar_arrive_expect_tx(&bars[buf], static_cast<uint32_t>(end - beg));
    size_t pos = beg;
    while (pos < end) {   // a piece may straddle a shard boundary: one bulk copy per owner
      const int owner = static_cast<int>(pos / ag.shard_bytes);
      const size_t within = pos - static_cast<size_t>(owner) * ag.shard_bytes;
      size_t n = ag.shard_bytes - within;
      if (n > end - pos) n = end - pos;
      bulk_g2s(smem + buf * AG_PIECE + (pos - beg), static_cast<const char*>(ag.peer[owner]) + ag.src_off + within,
               static_cast<uint32_t>(n), &bars[buf]);
      pos += n;
    }
  };
  auto publish = [&](size_t chunk) {
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
    st_release_gpu(ag.flags + chunk, ag.epoch);
  };
  for (size_t i = 0; i < n_pieces && i < AG_BUFS; ++i) issue_load(i);
  for (size_t i = 0; i < n_pieces; ++i) {
    const int buf = static_cast<int>(i % AG_BUFS);
    if (!mbar_wait(&bars[buf], static_cast<uint32_t>((i / AG_BUFS) & 1), &abort_local, status, STATUS_TIMEOUT_PEER)) break;
    size_t beg, end, chunk; piece_range(i, beg, end, chunk);
    if (end > beg) bulk_s2g(ag.dst + beg, smem + buf * AG_PIECE, static_cast<uint32_t>(end - beg));
    tma_store_commit();
    if (i + AG_BUFS < n_pieces) {
      // buffer `buf` is refilled by piece i+3: its store must have finished reading shared memory
      tma_store_wait_read<0>();
      issue_load(i + AG_BUFS);
    }
    if (i % AG_PIECES_PER_CHUNK == AG_PIECES_PER_CHUNK - 1) {
      tma_store_wait<0>();       // all stores of this chunk have completed
      publish(chunk);
    }
  }
  tma_store_wait<0>();
}

// Wait until dst bytes [lo, hi) are complete.  Returns false on timeout.
__device__ __forceinline__ bool ag_wait(const AgParams& ag, size_t lo, size_t hi, volatile int* abort_flag, int* status) {
  for (size_t c = lo / AG_CHUNK; c * AG_CHUNK < hi; ++c) {
    long long t0 = clock64();
    while (ld_acquire_gpu(ag.flags + c) != ag.epoch) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles * 8) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER);
        return false;
      }
      __nanosleep(100);
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");   // chunk was written through the generic proxy, TMA reads it
  return true;
}

struct Tile {
  int m0;        // first row of the A / output tile (for GROUPED=2: first output row inside the expert's matrix)
  int n0;        // first output column
  int b_row;     // row offset added to B's row coordinate (expert base)
  int kb0, kb1;  // K-block range
  size_t out_off;  // element offset added to the output pointer (expert base for GROUPED=2)
  int split;       // split-K piece of this work item (0 without split-K)
  int tile_id;     // output tile index (semaphore slot)
};

template <int A_MN, int B_MN, int OUT_F32, int FUSED_AG = 0, int GROUPED = 0>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p, const AgParams ag, const GroupParams gp, const RsParams rs) {
  if (FUSED_AG == 1 && static_cast<int>(blockIdx.x) < ag.n_copy) {   // copier CTAs: lowest indices, scheduled first
    extern __shared__ uint8_t smem_copier[];
    ag_copier(ag, reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_copier) + 1023) & ~uintptr_t(1023)), p.status);
    return;
  }
  const int cta = FUSED_AG == 1 ? static_cast<int>(blockIdx.x) - ag.n_copy : static_cast<int>(blockIdx.x);
  const int n_cta = FUSED_AG == 1 ? static_cast<int>(gridDim.x) - ag.n_copy : static_cast<int>(gridDim.x);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;      // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ int s_off[258];
  if (GROUPED == 1 || GROUPED == 2) {
    for (int i = threadIdx.x; i <= gp.E; i += blockDim.x) s_off[i] = gp.offsets[i];
    __syncthreads();
  }
  const int num_n = (p.N + BN - 1) / BN;
  const int num_m = GROUPED == 1 ? s_off[GROUPED ? gp.E : 0] / BM : (p.M + BM - 1) / BM;
  const int SK = (GROUPED == 0 && FUSED_AG == 0 && OUT_F32 && p.split_k > 1) ? p.split_k : 1;
  const int num_tiles = ((GROUPED == 2 || GROUPED == 3) ? gp.E : 1) * num_m * num_n * SK;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  auto tile_coords = [&](int t, int& m_idx, int& n_idx) {
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(num_m - first_m, GROUP_M);
    const int r = t - g * per_group;
    m_idx = first_m + (r % gsz);
    n_idx = r / gsz;
    if (FUSED_AG == 2) {       // row blocks of the next rank's slice first, this rank's own slice last
      const int per = num_m / rs.world;
      m_idx = (m_idx + ((rs.rank + 1) % rs.world) * per) % num_m;
    }
  };
  auto get_tile = [&](int t, Tile& tl) {
    if (GROUPED == 3) {          // batched: gp.E matrices of identical shape, 3-D tensor maps
      const int per_b = num_m * num_n;
      const int bi = t / per_b, r = t - bi * per_b;
      tl.m0 = (r % num_m) * BM; tl.n0 = (r / num_m) * BN; tl.b_row = bi;
      tl.kb0 = 0; tl.kb1 = num_kb;
      tl.out_off = static_cast<size_t>(bi) * p.M * p.ldc;
    } else if (GROUPED == 2) {
      const int per_e = num_m * num_n;
      const int e = t / per_e, r = t - e * per_e;
      tl.m0 = (r % num_m) * BM; tl.n0 = (r / num_m) * BN; tl.b_row = 0;
      tl.kb0 = s_off[e] / BK; tl.kb1 = s_off[e + 1] / BK;
      tl.out_off = static_cast<size_t>(e) * p.M * p.ldc;
    } else {
      // split-K: all pieces 0 come first in the global order, so a piece only ever waits for work with a smaller index
      const int base_tiles = num_m * num_n;
      const int split = SK > 1 ? t / base_tiles : 0;
      const int tt = t - split * base_tiles;
      int mi, ni; tile_coords(tt, mi, ni);
      tl.m0 = mi * BM; tl.n0 = ni * BN; tl.kb0 = 0; tl.kb1 = num_kb; tl.out_off = 0; tl.b_row = 0;
      tl.split = split; tl.tile_id = tt;
      if (SK > 1) {
        const int per = (num_kb + SK - 1) / SK;
        tl.kb0 = split * per < num_kb ? split * per : num_kb;
        tl.kb1 = tl.kb0 + per < num_kb ? tl.kb0 + per : num_kb;
      }
      if (GROUPED == 1) {
        int lo = 0, hi = gp.E;          // expert whose segment holds row m0
        while (lo + 1 < hi) { const int mid = (lo + hi) >> 1; if (s_off[mid] <= tl.m0) lo = mid; else hi = mid; }
        tl.b_row = lo * gp.b_rows;
      }
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int t = cta; t < num_tiles; t += n_cta) {
        Tile tl; get_tile(t, tl);
        const int m0 = tl.m0, n0 = tl.n0;
        if (FUSED_AG == 1) {
          const size_t row_bytes = static_cast<size_t>(p.K) * 2;
          if (ag.gather_a) {
            const int m_hi = m0 + BM < p.M ? m0 + BM : p.M;
            if (!ag_wait(ag, ag.a_off + m0 * row_bytes, ag.a_off + m_hi * row_bytes, abort_flag, p.status)) goto done;
          } else {
            const int n_hi = n0 + BN < p.N ? n0 + BN : p.N;
            if (!ag_wait(ag, ag.b_off + n0 * row_bytes, ag.b_off + n_hi * row_bytes, abort_flag, p.status)) goto done;
          }
        }
        for (int kb = tl.kb0; kb < tl.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          if (GROUPED == 3) {
            if (A_MN) {
#pragma unroll
              for (int c = 0; c < BM / 64; ++c) tma_load_3d(sa + c * (64 * BK * 2), &tmap_a, &full_bar[stage], m0 + c * 64, kb * BK, tl.b_row);
            } else {
              tma_load_3d(sa, &tmap_a, &full_bar[stage], kb * BK, m0, tl.b_row);
            }
            if (B_MN) {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c) tma_load_3d(sb + c * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + c * 64, kb * BK, tl.b_row);
            } else {
              tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * BK, n0, tl.b_row);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (64 * BK * 2), &tmap_a, &full_bar[stage], m0 + c * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * BK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + c * 64, (GROUPED == 1 ? tl.b_row : 0) + kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * BK, (GROUPED == 1 ? tl.b_row : 0) + n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      // per-K16 advance of the descriptor start address (in 16-byte units)
      constexpr uint32_t a_kstep = A_MN ? (16 * 128) >> 4 : 32 >> 4;
      constexpr uint32_t b_kstep = B_MN ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = cta; t < num_tiles; t += n_cta, ++it) {
        const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        Tile tl; get_tile(t, tl);
        for (int kb = tl.kb0; kb < tl.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint64_t da = A_MN ? make_smem_desc(sa, 64 * BK * 2, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t db = B_MN ? make_smem_desc(sb, 64 * BK * 2, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_bf16(d_tmem, da + static_cast<uint64_t>(k * a_kstep), db + static_cast<uint64_t>(k * b_kstep), idesc,
                      (kb != tl.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (tl.kb0 == tl.kb1) mbar_arrive(&tmem_full[acc]);   // empty expert segment: nothing was issued
        else umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int it = 0;
    for (int t = cta; t < num_tiles; t += n_cta, ++it) {
      Tile tl; get_tile(t, tl);
      const bool empty_tile = tl.kb0 == tl.kb1;
      const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const int row = tl.m0 + q * 32 + lane;
      const int col0 = tl.n0;
      const int row_limit = GROUPED == 1 ? min(s_off[gp.E], p.M) : p.M;     // never past the rows the caller allocated
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      int acc_flag = p.accumulate;
      if (OUT_F32 && SK > 1) {
        // wait for the previous piece of this tile (this warp's 32 rows) to have been added
        if (tl.split > 0) {
          bool ok = true;
          if (lane == 0) {
            const uint32_t* sp = p.sem + tl.tile_id * 4 + q;
            const long long t0 = clock64();
            while (ld_acquire_gpu(sp) != static_cast<uint32_t>(tl.split)) {
              if (*abort_flag || clock64() - t0 > kWaitLimitCycles * 4) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM_EMPTY);
                ok = false;
                break;
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) goto done;
          acc_flag = 1;
        }
      }
      // FUSED_AG == 2: a tile of this rank's own slice is finished here — the peers computed their partial products of
      // these rows first, so the epilogue adds them (loads from peer memory) and writes the reduced rows directly.
      bool own_tile = false;
      if (FUSED_AG == 2) {
        const int per = num_m / rs.world;
        const int blk = tl.m0 / BM;
        own_tile = blk / per == rs.rank;
        if (own_tile) {
          bool ok = true;
          if (lane == 0) {
            for (int pq = 0; pq < rs.world && ok; ++pq) {
              if (pq == rs.rank) continue;
              const uint32_t* cq = reinterpret_cast<const uint32_t*>(static_cast<const char*>(rs.peer[pq]) + rs.cnt_off) + blk;
              const long long t0 = clock64();
              while (true) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(cq) : "memory");
                if (static_cast<int32_t>(v - rs.expect) >= 0) break;
                if (*abort_flag || clock64() - t0 > kWaitLimitCycles * 8) {
                  *abort_flag = 1;
                  if (p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_PEER);
                  ok = false;
                  break;
                }
                __nanosleep(200);
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) goto done;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (empty_tile) {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        const int col = col0 + c * 32;
        if (row < row_limit && col < p.N) {
          if (OUT_F32) {
            float* o = reinterpret_cast<float*>(p.out) + tl.out_off + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha,
                                       __uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha);
                if (acc_flag) {
                  const float4 old = *reinterpret_cast<const float4*>(o + j);
                  v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                }
                *reinterpret_cast<float4*>(o + j) = v;
              }
            }
          } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + tl.out_off + static_cast<size_t>(row) * p.ldc + col;
            if (FUSED_AG == 2 && own_tile)
              o = rs.out_local + static_cast<size_t>(row - rs.rank * (num_m / rs.world) * BM) * p.N + col;
            const __nv_bfloat16* ci = p.cin ? reinterpret_cast<const __nv_bfloat16*>(p.cin) + tl.out_off + static_cast<size_t>(row) * p.ldc + col : nullptr;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < p.N) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]) * p.alpha;
                if (FUSED_AG == 2 && own_tile) {
#pragma unroll
                  for (int pq = 0; pq < 8; ++pq) {
                    if (pq < rs.world && pq != rs.rank) {
                      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(static_cast<const char*>(rs.peer[pq]) + rs.part_off) +
                                                 static_cast<size_t>(row) * p.ldc + col + j;
                      const uint4 pv = *reinterpret_cast<const uint4*>(src);
                      const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                      for (int e = 0; e < 4; ++e) {
                        const float2 c2 = unpack_bf16x2(pw[e]);
                        f[2 * e] += c2.x; f[2 * e + 1] += c2.y;
                      }
                    }
                  }
                }
                if (ci) {
                  const uint4 cv = *reinterpret_cast<const uint4*>(ci + j);
                  const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 c2 = unpack_bf16x2(cw[e]);
                    f[2 * e] += p.beta * c2.x; f[2 * e + 1] += p.beta * c2.y;
                  }
                }
                uint4 ov;
                ov.x = pack_bf16x2(f[0], f[1]); ov.y = pack_bf16x2(f[2], f[3]);
                ov.z = pack_bf16x2(f[4], f[5]); ov.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(o + j) = ov;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (OUT_F32 && SK > 1) {
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu(p.sem + tl.tile_id * 4 + q, tl.split + 1 == SK ? 0u : static_cast<uint32_t>(tl.split + 1));
      }
      if (FUSED_AG == 2 && !own_tile) {
        // this warp's 32 rows × 256 columns of the tile are stored: publish them to the peers
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          uint32_t* cnt = reinterpret_cast<uint32_t*>(const_cast<char*>(static_cast<const char*>(rs.peer[rs.rank])) + rs.cnt_off);
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt + tl.m0 / BM) : "memory");
        }
      }
    }
  }

done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map: inner dimension `inner` (contiguous), `outer` rows of `row_stride_elems`.
int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 3-D bf16 tensor map: [inner (contiguous), rows, batch]; box covers one batch entry.
int make_tmap_3d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch,
                      uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[3] = {inner, rows, batch};
  cuuint64_t gstride[2] = {row_stride_elems * 2, batch_stride_elems * 2};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 3-D fp32 tensor map [inner (contiguous), rows, batch] with a box of 16 floats × box_rows × 1 and the 64-byte swizzle: the
// target of the attention backward's bulk reductions (cp.reduce.async.bulk.tensor, add) into its fp32 dQ accumulator.
int make_tmap_3d_f32_sw64(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch,
                          uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[3] = {inner, rows, batch};
  cuuint64_t gstride[2] = {row_stride_elems * 4, batch_stride_elems * 4};
  cuuint32_t box[3] = {16, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

uint32_t* g_splitk_sem = nullptr;      // shared with the two-CTA kernel (gemm2_bf16.cu)
int g_splitk_sem_len = 0;

// Pieces per output tile that best fill whole waves of `sms` CTAs (1 = no split); every piece keeps ≥ 64 K-blocks.
int choose_split_k(int tiles, int num_kb, int sms, int slots_per_tile) {
  auto eff = [&](int s) { const long long w = static_cast<long long>(tiles) * s; return static_cast<double>(w) / (((w + sms - 1) / sms) * sms); };
  int best = 1;
  double best_eff = eff(1);
  for (int s = 2; s <= 4; ++s) {
    if (num_kb / s < 64 || tiles * slots_per_tile > g_splitk_sem_len) break;
    if (eff(s) > best_eff * 1.08) { best = s; best_eff = eff(s); }
  }
  return best;
}

template <int A_MN, int B_MN, int OUT_F32>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms, cudaStream_t st) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  GemmParams pp = p;
  if (OUT_F32 && p.accumulate && g_splitk_sem != nullptr) {
    pp.split_k = choose_split_k(tiles, (p.K + BK - 1) / BK, sms, 4);
    pp.sem = g_splitk_sem;
  }
  const int work = tiles * (pp.split_k > 1 ? pp.split_k : 1);
  const int grid = work < sms ? work : sms;
  AgParams none{};
  GroupParams nog{};
  kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, pp, none, nog, RsParams{});
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

// Workspace of the serial split-K path: `n` zero-initialised uint32 counters on the current device (4 per output tile).
// Without it (the default) weight-gradient GEMMs never split.
extern "C" void b200_gemm_set_splitk_workspace(uint32_t* sem, int n) {
  b200::g_splitk_sem = sem;
  b200::g_splitk_sem_len = n;
}

extern "C" int b200_gemm_bf16(int mode, const void* A, const void* B, void* out, const void* cin, int M, int N, int K,
                              int lda, int ldb, int ldc, float alpha, float beta, int out_f32, int accumulate,
                              int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // The tensor-map encoder is a driver call and needs the primary context current in this thread
  // (autograd worker threads may not have touched the runtime yet).
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  // A
  if (mode == 2) rc = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);      // stored [K, M]
  else           rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);      // stored [M, K]
  if (rc) return rc;
  // B
  if (mode == 0) rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BN);      // stored [N, K]
  else           rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);      // stored [K, N]
  if (rc) return rc;
  GemmParams p{out, cin, M, N, K, ldc, alpha, beta, accumulate, status};
  if (mode == 0) return out_f32 ? launch_variant<0, 0, 1>(ta, tb, p, num_sms, stream) : launch_variant<0, 0, 0>(ta, tb, p, num_sms, stream);
  if (mode == 1) return out_f32 ? launch_variant<0, 1, 1>(ta, tb, p, num_sms, stream) : launch_variant<0, 1, 0>(ta, tb, p, num_sms, stream);
  if (mode == 2) return out_f32 ? launch_variant<1, 1, 1>(ta, tb, p, num_sms, stream) : launch_variant<1, 1, 0>(ta, tb, p, num_sms, stream);
  return -4;
}

// out[M,N] (bf16) = A[M,K] · Bᵀ where B[N,K] sits at byte offset b_off of the gathered buffer `dst` that this
// same launch fills from all ranks' shards (see AgParams).  `flags` needs one uint32 per 256 KiB of dst
// and must never hold `epoch` from an earlier launch (use a fresh epoch per call).
extern "C" int b200_ag_gemm_bf16(const void* A, void* out, int M, int N, int K, int lda, int ldc,
                                 const void* const* bases, size_t src_off, void* dst, size_t shard_bytes, size_t b_off,
                                 uint32_t* flags, uint32_t epoch, int rank, int world, int n_copy, int num_sms,
                                 int* status, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || world > 8 || (shard_bytes % 16) || (b_off % 16)) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, static_cast<const char*>(dst) + b_off, K, N, K, BK, BN);
  if (rc) return rc;
  GemmParams p{out, nullptr, M, N, K, ldc, 1.f, 0.f, 0, status};
  AgParams ag{};
  for (int i = 0; i < 8; ++i) ag.peer[i] = i < world ? bases[i] : nullptr;
  ag.src_off = src_off; ag.dst = static_cast<char*>(dst); ag.shard_bytes = shard_bytes; ag.b_off = b_off;
  ag.flags = flags; ag.epoch = epoch; ag.rank = rank; ag.world = world; ag.n_copy = n_copy;
  auto kern = gemm_bf16_kernel<0, 0, 0, 1>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int compute = num_sms - n_copy;
  if (compute > tiles) compute = tiles;
  if (compute < 1) return -6;
  GroupParams nog{};
  kern<<<compute + n_copy, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, ag, nog, RsParams{});
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Tensor-parallel column-parallel layer: out[M,N] (bf16) = A[M,K] · B[N,K]ᵀ where A is the concatenation, in rank order,
// of every rank's [M/world, K] activation chunk (at `src_off` of each symmetric heap).  The same launch pulls the chunks
// into the local buffer `dst` ([M, K], ordinary device memory) and multiplies row blocks as they arrive.
extern "C" int b200_ag_a_gemm_bf16(const void* const* bases, size_t src_off, void* dst, size_t shard_bytes, const void* B,
                                   void* out, int M, int N, int K, int ldb, int ldc, uint32_t* flags, uint32_t epoch, int rank,
                                   int world, int n_copy, int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || world > 8 || (shard_bytes % 16)) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, dst, K, M, K, BK, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc;
  GemmParams p{out, nullptr, M, N, K, ldc, 1.f, 0.f, 0, status};
  AgParams ag{};
  for (int i = 0; i < 8; ++i) ag.peer[i] = i < world ? bases[i] : nullptr;
  ag.src_off = src_off; ag.dst = static_cast<char*>(dst); ag.shard_bytes = shard_bytes; ag.b_off = 0;
  ag.flags = flags; ag.epoch = epoch; ag.rank = rank; ag.world = world; ag.n_copy = n_copy;
  ag.gather_a = 1; ag.a_off = 0;
  auto kern = gemm_bf16_kernel<0, 0, 0, 1>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int compute = num_sms - n_copy;
  if (compute > tiles) compute = tiles;
  if (compute < 1) return -6;
  GroupParams nog{};
  kern<<<compute + n_copy, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, ag, nog, RsParams{});
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Tensor-parallel row-parallel layer: out_local[M/world, N] (bf16) = this rank's rows of Σ_ranks A_r[M,K_r] · B_r[N,K_r]ᵀ.
// `part_off` / `cnt_off`: the [M, N] bf16 partial-product buffer and the per-128-row counters inside every symmetric heap;
// `expect` = counter value of a finished row block after this call (counters only grow: add 4 · ceil(N/256) per call).
// Every rank must launch the same call; the grid is at most one CTA per SM so all CTAs are resident while they wait.
extern "C" int b200_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, int lda, int ldb, const void* const* bases,
                                 size_t part_off, size_t cnt_off, uint32_t expect, void* out_local, int rank, int world,
                                 int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > 8 || M % (BM * world) || N % 8 || (part_off % 16) || (cnt_off % 4)) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BN);
  if (rc) return rc;
  void* part = const_cast<char*>(static_cast<const char*>(bases[rank])) + part_off;
  GemmParams p{part, nullptr, M, N, K, N, 1.f, 0.f, 0, status};
  RsParams rs{};
  for (int i = 0; i < 8; ++i) rs.peer[i] = i < world ? bases[i] : nullptr;
  rs.part_off = part_off; rs.cnt_off = cnt_off; rs.expect = expect; rs.rank = rank; rs.world = world;
  rs.out_local = static_cast<__nv_bfloat16*>(out_local);
  auto kern = gemm_bf16_kernel<0, 0, 0, 2>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  AgParams none{};
  GroupParams nog{};
  kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, nog, rs);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Grouped GEMMs over an expert-sorted, 128-row-aligned activation layout (see GroupParams).
//   kind 0: out[rows, N] = A[rows, K] · B[e]ᵀ   with B stored [E·N, K]           (forward projections)
//   kind 1: out[rows, N] = A[rows, K] · B[e]    with B stored [E·K, N]           (dgrad)
//   kind 2: out[e][M, N] (+)= A[rows_e, M]ᵀ · B[rows_e, N], fp32 or bf16 output  (wgrad)
// `capacity` = number of rows allocated in the sorted layout (upper bound of offsets[E]).
extern "C" int b200_grouped_gemm_bf16(int kind, const void* A, const void* B, void* out, const int* offsets, int E,
                                      int capacity, int M, int N, int K, int out_f32, int accumulate, int num_sms,
                                      int* status, cudaStream_t stream) {
  using namespace b200;
  if (E <= 0 || E > 256 || capacity <= 0) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  AgParams none{};
  GroupParams gp{offsets, E, 0};
  if (kind == 0 || kind == 1) {
    // A: [capacity, K] K-major
    rc = make_tmap_2d_bf16(&ta, A, K, capacity, K, BK, BM);
    if (rc) return rc;
    if (kind == 0) { rc = make_tmap_2d_bf16(&tb, B, K, static_cast<uint64_t>(E) * N, K, BK, BN); gp.b_rows = N; }
    else           { rc = make_tmap_2d_bf16(&tb, B, N, static_cast<uint64_t>(E) * K, N, 64, BK); gp.b_rows = K; }
    if (rc) return rc;
    GemmParams p{out, nullptr, capacity, N, K, N, 1.f, 0.f, 0, status};
    const int max_tiles = (capacity / BM) * ((N + BN - 1) / BN);
    const int grid = max_tiles < num_sms ? (max_tiles > 0 ? max_tiles : 1) : num_sms;
    if (kind == 0) {
      auto kern = gemm_bf16_kernel<0, 0, 0, 0, 1>;
      static bool cfg = false;
      if (!cfg) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2; cfg = true; }
      kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, gp, RsParams{});
    } else {
      auto kern = gemm_bf16_kernel<0, 1, 0, 0, 1>;
      static bool cfg = false;
      if (!cfg) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2; cfg = true; }
      kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, gp, RsParams{});
    }
  } else if (kind == 2) {
    // A: [capacity, M] (MN-major), B: [capacity, N] (MN-major); K = rows of the expert's segment
    rc = make_tmap_2d_bf16(&ta, A, M, capacity, M, 64, BK);
    if (rc) return rc;
    rc = make_tmap_2d_bf16(&tb, B, N, capacity, N, 64, BK);
    if (rc) return rc;
    GemmParams p{out, nullptr, M, N, capacity, N, 1.f, 0.f, accumulate, status};
    const int tiles = E * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < num_sms ? tiles : num_sms;
    if (out_f32) {
      auto kern = gemm_bf16_kernel<1, 1, 1, 0, 2>;
      static bool cfg = false;
      if (!cfg) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2; cfg = true; }
      kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, gp, RsParams{});
    } else {
      auto kern = gemm_bf16_kernel<1, 1, 0, 0, 2>;
      static bool cfg = false;
      if (!cfg) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2; cfg = true; }
      kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, gp, RsParams{});
    }
  } else {
    return -4;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Batched GEMM over `batch` contiguous matrices of identical shape (Newton–Schulz on stacked experts):
//   out[b] = alpha · op(A[b]) · op(B[b]) + beta · C[b], bf16 in / bf16 out, mode as in b200_gemm_bf16 (0: NT, 1: NN).
extern "C" int b200_gemm_bf16_batched(int mode, const void* A, const void* B, void* out, const void* cin, int batch, int M,
                                      int N, int K, float alpha, float beta, int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  if (mode != 0 && mode != 1) return -4;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_3d_bf16(&ta, A, K, M, batch, K, static_cast<uint64_t>(M) * K, BK, BM);
  if (rc) return rc;
  if (mode == 0) rc = make_tmap_3d_bf16(&tb, B, K, N, batch, K, static_cast<uint64_t>(N) * K, BK, BN);
  else           rc = make_tmap_3d_bf16(&tb, B, N, K, batch, N, static_cast<uint64_t>(K) * N, 64, BK);
  if (rc) return rc;
  GemmParams p{out, cin, M, N, K, N, alpha, beta, 0, status};
  AgParams none{};
  GroupParams gp{nullptr, batch, 0};
  const int tiles = batch * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  if (mode == 0) {
    auto kern = gemm_bf16_kernel<0, 0, 0, 0, 3>;
    static bool cfg = false;
    if (!cfg) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2; cfg = true; }
    kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, gp, RsParams{});
  } else {
    auto kern = gemm_bf16_kernel<0, 1, 0, 0, 3>;
    static bool cfg = false;
    if (!cfg) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) != cudaSuccess) return -2; cfg = true; }
    kern<<<grid, NUM_THREADS, GEMM_SMEM_BYTES, stream>>>(ta, tb, p, none, gp, RsParams{});
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
