// Attention backward on tcgen05, deterministic (no atomics).  Three kernels:
//
//   attn_bwd_delta   δ[b,h,r] = Σ_d dO·O                               (one warp per row/head)
//   attn_bwd_dq      CTA per (query tile, head, batch), loop over key tiles:
//                      S = Q·Kᵀ, dP = dO·Vᵀ  →  dS = P∘(dP − δ) (bf16, in TMEM)  →  dQ += dS·K, ·scale at the end
//   attn_bwd_dkdv    CTA per (key tile, kv head, batch), loop over the query heads of the group and
//                    their query tiles, in the transposed domain so that the lane index is the key row:
//                      Sᵀ = K·Qᵀ, dPᵀ = V·dOᵀ  →  Pᵀ, dSᵀ (bf16, in TMEM)  →  dV += Pᵀ·dO, dK += dSᵀ·Q
//                    GQA reduction over the group's query heads happens in the TMEM accumulators.
//
// P is recomputed from the saved log-sum-exp.  The bf16 P / dS values overwrite the fp32 S / dP columns
// in place (16 packed columns land inside the 32 columns a warp just read).  Inner tiles are processed as two
// halves of 64 columns with two (S, dP) buffers: 2 × 128 columns + the 128-column accumulators ≤ 512.
// Masking rule as in the forward: row r sees keys lo(r) ≤ k ≤ r.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int BT = 128;                 // tile edge (queries and keys)
constexpr int BWD_THREADS = 384;            // warp 0 TMA, warp 1 MMA (S), warps 2..9 softmax, warp 10 MMA (accumulations), warp 11 MMA (dP)
constexpr int ACC_WARP = 10;
constexpr int DP_WARP = 11;
constexpr float kLog2e_b = 1.4426950408889634f;

int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer);

struct AttnBwdParams {
  const float* lse;        // [B,H,T] natural log
  const float* delta;      // [B,H,T]
  const int* row_start;    // [B*T] or null
  const int* doc_end;      // [B*T] exclusive end of the document of each position, or null
  __nv_bfloat16* dq;       // [B,T,H,D]
  __nv_bfloat16* dk;       // [B,T,G,D]
  __nv_bfloat16* dv;
  int B, T, H, G;
  int window_left;
  float scale, scale_log2;
  int* status;
  long long* trace;        // optional [8][64] clock64 stamps of the first dK/dV CTA (development aid, null in normal use)
};
#define BWD_TRACE(ev, hx) do { if (p.trace && traced && (hx) < 64) p.trace[(ev) * 64 + (hx)] = clock64(); } while (0)

__device__ __forceinline__ int lo_of_row(const AttnBwdParams& p, int b, int r) {
  int lo = p.row_start ? p.row_start[static_cast<size_t>(b) * p.T + r] : 0;
  if (p.window_left >= 0) lo = max(lo, r - p.window_left);
  return lo;
}

// ------------------------------------------------------------------------------------------- δ
// delta[b, h, t] = <o[b, t, h, :], d_o[b, t, h, :]>.  A block takes 32 consecutive tokens of one sequence and all heads: a
// group of D/8 lanes reads one row with 16-byte loads, the sums go through shared memory, and the [B, H, T] result is written
// 128 bytes at a time along t (one 4-byte store per row at stride T, as a warp-per-row kernel does, ran at 2.3 TB/s).
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                             float* __restrict__ delta, int B, int T, int H) {
  extern __shared__ float sdelta[];                                      // [H][32]
  constexpr int LPR = D / 8;                                             // lanes per row: 16 (D 128) or 8 (D 64)
  constexpr int RPW = 32 / LPR;                                          // rows per warp and step
  const int tiles_t = (T + 31) / 32;
  const int b = blockIdx.x / tiles_t, t0 = (blockIdx.x % tiles_t) * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, li = lane % LPR;
  const int n_rows = 32 * H;                                             // local row r = tl · H + h
  for (int r0 = warp * RPW; r0 < n_rows; r0 += 8 * RPW * 2) {           // two rows in flight per lane group
    float s[2] = {0.f, 0.f};
    uint4 x[2], y[2];
    bool ok[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int r = r0 + sub + u * 8 * RPW;
      const int tl = r / H;
      ok[u] = r < n_rows && t0 + tl < T;
      x[u] = y[u] = make_uint4(0u, 0u, 0u, 0u);
      if (ok[u]) {
        const size_t off = ((static_cast<size_t>(b) * T + t0) * H + r) * D + li * 8;
        x[u] = *reinterpret_cast<const uint4*>(o + off);
        y[u] = *reinterpret_cast<const uint4*>(d_o + off);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t xa[4] = {x[u].x, x[u].y, x[u].z, x[u].w}, ya[4] = {y[u].x, y[u].y, y[u].z, y[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 p = unpack_bf16x2(xa[e]), q = unpack_bf16x2(ya[e]);
        s[u] += p.x * q.x + p.y * q.y;
      }
#pragma unroll
      for (int ofs = LPR / 2; ofs > 0; ofs >>= 1) s[u] += __shfl_xor_sync(0xffffffffu, s[u], ofs);
      const int r = r0 + sub + u * 8 * RPW;
      if (li == 0 && r < n_rows) sdelta[(r % H) * 32 + r / H] = s[u];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_rows; i += 256) {
    const int h = i >> 5, tl = i & 31;
    if (t0 + tl < T) delta[(static_cast<size_t>(b) * H + h) * T + t0 + tl] = sdelta[i];
  }
}

template <int D>
struct BwdSmem {
  static constexpr int TILE = BT * D * 2;                       // one [128 × D] bf16 tile
  static constexpr int FIXED = 2 * TILE;                        // the two tiles loaded once
  static constexpr int RING = 2 * 2 * TILE;                     // 2 stages × 2 tiles
  static constexpr int AUX = 2 * 3 * BT * 4;                    // per stage: lse·log2e, δ, lo (dkdv only)
  static constexpr int TOTAL = FIXED + RING + AUX + 1024 + 256;
};

__device__ __forceinline__ void named_bar_sync_256() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Both kernels below walk their inner tiles in halves of 64 columns so that two (S, dP) buffers, 64 fp32 columns
// each, fit in tensor memory beside the accumulators.  The MMA thread runs one half ahead: while the 8 softmax
// warps turn half h into P / dS, the tensor pipe computes S, dP of half h+1 and the accumulation of half h−1.
// The 8 softmax warps form two groups of four (one warp per TMEM lane quarter); group c converts the halves that live in
// buffer c, 32 fp32 columns at a time, packing the bf16 result into the first 16 of the 32 columns just read, so the
// TS-MMA reads k-step k (16 rows of the contraction) at column (k/2)·32 + (k%2)·8.
constexpr int HB = 64;
__device__ __forceinline__ uint32_t packed_col(int k) { return static_cast<uint32_t>((k >> 1) * 32 + (k & 1) * 8); }

// ------------------------------------------------------------------------------------------- dQ
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const AttnBwdParams p) {
  using SM = BwdSmem<D>;
  constexpr int DC = D / 64;
  constexpr int CHUNK_BYTES = 128 * 64 * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  uint8_t* sdo = smem + SM::TILE;
  uint8_t* ring = smem + SM::FIXED;                 // stage s: K then V
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + SM::RING + SM::AUX);
  uint64_t* fixed_full = bars;      // 1
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* kv_empty = bars + 3;    // [2]
  // The dQ accumulator takes 128 of the 512 tensor-memory columns, which leaves room for THREE (S, dP) half-tile buffers:
  // a buffer's cycle (products → softmax → accumulation → free) is latency-bound, so three in flight instead of two
  // raise the rate at which halves complete.  Half hx lives in buffer hx % 3; warp group hx % 2 converts it.
  uint64_t* sdp_full = bars + 5;    // [3]  S and dP of a half are in TMEM buffer b
  uint64_t* ds_full = bars + 8;     // [3]  (count 4) dS of buffer b written by a warp group
  uint64_t* acc_done = bars + 11;   // 1    all dQ MMAs finished
  uint64_t* buf_free = bars + 12;   // [3]  accumulation MMAs that read buffer b have completed
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + BT - 1) / BT;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int q0 = qt * BT;
  const int r_last = min(q0 + BT, p.T) - 1;
  const int j_begin = lo_of_row(p, b, q0) / BT;
  const int n_tiles = r_last / BT + 1 - j_begin;
  const int n_half = 2 * n_tiles;

  if (threadIdx.x == 0) {
    mbar_init(fixed_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int s = 0; s < 3; ++s) { mbar_init(&sdp_full[s], 2); mbar_init(&ds_full[s], 4); mbar_init(&buf_free[s], 1); }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t T_DQ = tmem_base + 384;            // buffers b = 0..2: S[b] = base + 128 b, dP[b] = base + 128 b + 64

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(fixed_full, 2 * SM::TILE);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        tma_load_2d(sq + c * CHUNK_BYTES, &tmap_q, fixed_full, h * D + c * 64, b * p.T + q0);
        tma_load_2d(sdo + c * CHUNK_BYTES, &tmap_do, fixed_full, h * D + c * 64, b * p.T + q0);
      }
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1; const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        uint8_t* sk = ring + st * 2 * SM::TILE;
        uint8_t* sv = sk + SM::TILE;
        const int k0 = (j_begin + t) * BT;
        mbar_arrive_expect_tx(&kv_full[st], 2 * SM::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          tma_load_2d(sk + c * CHUNK_BYTES, &tmap_k, &kv_full[st], g * D + c * 64, b * p.T + k0);
          tma_load_2d(sv + c * CHUNK_BYTES, &tmap_v, &kv_full[st], g * D + c * 64, b * p.T + k0);
        }
      }
    }
  } else if (warp == 1 || warp == DP_WARP) {
    if (lane == 0) {
      // S = Q·Kᵀ is issued by warp 1 and dP = dO·Vᵀ by warp DP_WARP: one thread issues a tcgen05.mma only every ~100 cycles, and
      // the softmax of a half cannot start before both products are in tensor memory.  sdp_full counts both commits.
      const bool is_dp = warp == DP_WARP;
      constexpr uint32_t idesc_s = make_idesc_bf16(BT, HB, 0, 0);
      if (!mbar_wait(fixed_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      const uint32_t sa = smem_u32(is_dp ? sdo : sq);
      // keys hf·64.. of the tile: rows 8192 bytes into each 64-column chunk
      auto issue_one = [&](int hx) -> bool {
        const int t = hx >> 1, hf = hx & 1, st = t & 1, buf = hx % 3;
        if (hf == 0 && !mbar_wait(&kv_full[st], (t >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t sb = smem_u32(ring + st * 2 * SM::TILE) + hf * 8192 + (is_dp ? SM::TILE : 0);
        const uint32_t td = tmem_base + buf * 128 + (is_dp ? 64 : 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * CHUNK_BYTES + (k % 4) * 32;
          umma_bf16(td, make_smem_desc(sa + off, 16, 1024), make_smem_desc(sb + off, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(&sdp_full[buf]);
        return true;
      };
      // buf_free[b] orders the reuse of buffer b: S, dP of half hx+2 may overwrite it once the accumulation MMAs of half hx
      // (which read dS from it) have completed.
      for (int hx = 0; hx < n_half; ++hx) {
        if (hx >= 3 && !mbar_wait(&buf_free[hx % 3], ((hx - 3) / 3) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        if (!issue_one(hx)) goto done;
      }
    }
  } else if (warp == ACC_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_dq = make_idesc_bf16(BT, D, 0, 1);        // dQ += dS·K, K is N-major
      for (int hx = 0; hx < n_half; ++hx) {
        const int t = hx >> 1, hf = hx & 1, st = t & 1, buf = hx % 3;
        if (!mbar_wait(&ds_full[buf], (hx / 3) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        tc_fence_after();
        const uint32_t sk = smem_u32(ring + st * 2 * SM::TILE);
        const uint32_t tdp = tmem_base + buf * 128 + 64;
#pragma unroll
        for (int k = 0; k < HB / 16; ++k)
          umma_bf16_ts(T_DQ, tdp + packed_col(k), make_smem_desc(sk + (hf * 4 + k) * 2048, CHUNK_BYTES, 1024), idesc_dq,
                       (hx | k) != 0);
        umma_commit(&buf_free[buf]);
        if (hf == 1) umma_commit(&kv_empty[st]);
      }
      umma_commit(acc_done);
    }
  } else {
    const int qtr = warp & 3, ch = (warp - 2) >> 2;
    const int r = q0 + qtr * 32 + lane;
    const bool row_valid = r < p.T;
    const int lo_r = row_valid ? lo_of_row(p, b, r) : 0;
    const int lo_last = lo_of_row(p, b, r_last);
    const size_t stat_idx = (static_cast<size_t>(b) * p.H + h) * p.T + (row_valid ? r : 0);
    const float lse2 = row_valid ? p.lse[stat_idx] * kLog2e_b : 0.f;
    const float dlt = row_valid ? p.delta[stat_idx] : 0.f;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    // Ping-pong: warp group `ch` owns the halves with hx & 1 == ch (in buffer hx % 3) and converts all 64 columns of such a half,
    // so the load → exp2 → store chains of two consecutive halves overlap instead of running back to back.
    for (int hx = ch; hx < n_half; hx += 2) {
      const int t = hx >> 1, hf = hx & 1, buf = hx % 3;
      const int kt0 = (j_begin + t) * BT;
      if (!mbar_wait(&sdp_full[buf], (hx / 3) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const bool full_tile = (kt0 + BT - 1 <= q0) && (kt0 >= lo_last);
      const float sl2 = p.scale_log2;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int k0 = kt0 + hf * HB + cc * 32;
        const uint32_t ts = tmem_base + buf * 128 + cc * 32 + lane_off, tdp = ts + 64;
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(ts, sr);
        tmem_ld_32x32(tdp, dr);
        tmem_ld_wait();
        uint32_t w[16];
        if (full_tile && row_valid) {                 // no key of this tile is masked for any row: 4 ops per element
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = exp2f(fmaf(__uint_as_float(sr[2 * e]), sl2, -lse2));
            const float p1 = exp2f(fmaf(__uint_as_float(sr[2 * e + 1]), sl2, -lse2));
            w[e] = pack_bf16x2(p0 * (__uint_as_float(dr[2 * e]) - dlt), p1 * (__uint_as_float(dr[2 * e + 1]) - dlt));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            float ds2[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int kk = k0 + 2 * e + u;
              float pr = exp2f(fmaf(__uint_as_float(sr[2 * e + u]), sl2, -lse2));
              if (kk > r || kk < lo_r || !row_valid) pr = 0.f;
              ds2[u] = pr * (__uint_as_float(dr[2 * e + u]) - dlt);
            }
            w[e] = pack_bf16x2(ds2[0], ds2[1]);
          }
        }
        tmem_st_32x16(tdp, w);                        // in place: the first 16 of the 32 columns just read
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[buf]);
    }
    if (!mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
    tc_fence_after();
    __nv_bfloat16* orow = p.dq + ((static_cast<size_t>(b) * p.T + r) * p.H + h) * D;
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
      const int col = ch * (D / 2) + c * 32;
      uint32_t rr[32];
      if (n_tiles > 0) { tmem_ld_32x32(T_DQ + col + lane_off, rr); tmem_ld_wait(); }
      else {
#pragma unroll
        for (int e = 0; e < 32; ++e) rr[e] = 0u;
      }
      if (row_valid) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 o;      // dS was formed without the softmax scale: apply it once here
          o.x = pack_bf16x2(__uint_as_float(rr[e]) * p.scale, __uint_as_float(rr[e + 1]) * p.scale);
          o.y = pack_bf16x2(__uint_as_float(rr[e + 2]) * p.scale, __uint_as_float(rr[e + 3]) * p.scale);
          o.z = pack_bf16x2(__uint_as_float(rr[e + 4]) * p.scale, __uint_as_float(rr[e + 5]) * p.scale);
          o.w = pack_bf16x2(__uint_as_float(rr[e + 6]) * p.scale, __uint_as_float(rr[e + 7]) * p.scale);
          *reinterpret_cast<uint4*>(orow + col + e) = o;
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

// ------------------------------------------------------------------------------------------- dK, dV
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                     const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                     const AttnBwdParams p) {
  using SM = BwdSmem<D>;
  constexpr int DC = D / 64;
  constexpr int CHUNK_BYTES = 128 * 64 * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sk = smem;
  uint8_t* sv = smem + SM::TILE;
  uint8_t* ring = smem + SM::FIXED;                 // stage s: Q then dO
  float* aux = reinterpret_cast<float*>(ring + SM::RING);   // stage s: [lse2 | delta | lo] × 128
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + SM::RING + SM::AUX);
  uint64_t* fixed_full = bars;      // 1
  uint64_t* qd_full = bars + 1;     // [2]
  uint64_t* qd_empty = bars + 3;    // [2]
  uint64_t* sdp_full = bars + 5;    // [2]
  uint64_t* ds_full = bars + 7;     // [2] (count 4)
  uint64_t* acc_done = bars + 9;    // 1
  uint64_t* buf_free = bars + 10;   // [2]
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int k0 = jt * BT;
  const int k_last = min(k0 + BT, p.T) - 1;
  const int group = p.H / p.G;
  // query rows that can see a key of this tile: k0 ≤ r ≤ r_hi
  int r_hi = p.T - 1;
  if (p.window_left >= 0) r_hi = min(r_hi, k_last + p.window_left);
  if (p.doc_end) r_hi = min(r_hi, p.doc_end[static_cast<size_t>(b) * p.T + k_last] - 1);
  const int i_begin = k0 / BT, i_end = r_hi / BT + 1;
  const int tiles_per_head = i_end - i_begin;
  const int n_iter = tiles_per_head * group;
  const int n_half = 2 * n_iter;
  const bool traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0;

  if (threadIdx.x == 0) {
    mbar_init(fixed_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qd_full[s], 1); mbar_init(&qd_empty[s], 1);
      mbar_init(&sdp_full[s], 2); mbar_init(&ds_full[s], 4); mbar_init(&buf_free[s], 1);
    }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t T_DV = tmem_base + 256, T_DK = tmem_base + 384;   // Sᵀ[b] = base + 128 b, dPᵀ[b] = base + 128 b + 64

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(fixed_full, 2 * SM::TILE);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        tma_load_2d(sk + c * CHUNK_BYTES, &tmap_k, fixed_full, g * D + c * 64, b * p.T + k0);
        tma_load_2d(sv + c * CHUNK_BYTES, &tmap_v, fixed_full, g * D + c * 64, b * p.T + k0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1; const uint32_t ph = (it >> 1) & 1;
        const int hq = g * group + it / tiles_per_head;
        const int q0 = (i_begin + it % tiles_per_head) * BT;
        if (!mbar_wait(&qd_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        uint8_t* sqs = ring + st * 2 * SM::TILE;
        uint8_t* sdos = sqs + SM::TILE;
        mbar_arrive_expect_tx(&qd_full[st], 2 * SM::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          tma_load_2d(sqs + c * CHUNK_BYTES, &tmap_q, &qd_full[st], hq * D + c * 64, b * p.T + q0);
          tma_load_2d(sdos + c * CHUNK_BYTES, &tmap_do, &qd_full[st], hq * D + c * 64, b * p.T + q0);
        }
      }
    }
  } else if (warp == 1 || warp == DP_WARP) {
    if (lane == 0) {
      // Sᵀ = K·Qᵀ by warp 1, dPᵀ = V·dOᵀ by warp DP_WARP (64 queries per half); see the dQ kernel
      const bool is_dp = warp == DP_WARP;
      constexpr uint32_t idesc_s = make_idesc_bf16(BT, HB, 0, 0);
      if (!mbar_wait(fixed_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      const uint32_t sa = smem_u32(is_dp ? sv : sk);
      auto issue_one = [&](int hx) -> bool {
        const int it = hx >> 1, hf = hx & 1, st = it & 1, buf = hx & 1;
        if (hf == 0 && !mbar_wait(&qd_full[st], (it >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t sb = smem_u32(ring + st * 2 * SM::TILE) + hf * 8192 + (is_dp ? SM::TILE : 0);
        const uint32_t td = tmem_base + buf * 128 + (is_dp ? 64 : 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * CHUNK_BYTES + (k % 4) * 32;
          umma_bf16(td, make_smem_desc(sa + off, 16, 1024), make_smem_desc(sb + off, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(&sdp_full[buf]);
        return true;
      };
      for (int hx = 0; hx < n_half; ++hx) {
        if (!is_dp) BWD_TRACE(3, hx);
        if (hx >= 2 && !mbar_wait(&buf_free[hx & 1], ((hx - 2) >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        if (!issue_one(hx)) goto done;
        if (!is_dp) BWD_TRACE(4, hx);
      }
    }
  } else if (warp == ACC_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_acc = make_idesc_bf16(BT, D, 0, 1);      // dV += Pᵀ·dO, dK += dSᵀ·Q (N-major B)
      for (int hx = 0; hx < n_half; ++hx) {
        const int it = hx >> 1, hf = hx & 1, st = it & 1, buf = hx & 1;
        BWD_TRACE(5, hx);
        if (!mbar_wait(&ds_full[buf], (hx >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        tc_fence_after();
        BWD_TRACE(6, hx);
        const uint32_t sqa = smem_u32(ring + st * 2 * SM::TILE), sdoa = sqa + SM::TILE;
        const uint32_t ts = tmem_base + buf * 128, tdp = ts + 64;
#pragma unroll
        for (int k = 0; k < HB / 16; ++k) {
          umma_bf16_ts(T_DV, ts + packed_col(k), make_smem_desc(sdoa + (hf * 4 + k) * 2048, CHUNK_BYTES, 1024), idesc_acc,
                       (hx | k) != 0);
          umma_bf16_ts(T_DK, tdp + packed_col(k), make_smem_desc(sqa + (hf * 4 + k) * 2048, CHUNK_BYTES, 1024), idesc_acc,
                       (hx | k) != 0);
        }
        umma_commit(&buf_free[buf]);
        if (hf == 1) umma_commit(&qd_empty[st]);
        BWD_TRACE(7, hx);
      }
      umma_commit(acc_done);
    }
  } else {
    const int qtr = warp & 3, ch = (warp - 2) >> 2;
    const int kk = k0 + qtr * 32 + lane;              // this thread's key row
    const bool key_valid = kk < p.T;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    bool ok = true;     // after a timed-out wait the thread keeps meeting its peers at the named barrier, idle
    const bool plain_causal = p.row_start == nullptr && p.window_left < 0 && k0 + BT <= p.T;
    // Ping-pong: warp group `ch` owns the halves with hx & 1 == ch, i.e. always the query columns ch·64 … ch·64+63 of a
    // tile (buffer ch), and converts all 64 of them; it fills and reads only its own 64 entries of the per-query
    // statistics, so the two groups never wait for each other.
    const int tid128 = qtr * 32 + lane;               // 0..127 inside the group
    for (int hx = ch; hx < n_half; hx += 2) {
      const int it = hx >> 1, hf = hx & 1, st = it & 1, buf = hx & 1;
      const int hq = g * group + it / tiles_per_head;
      const int q0 = (i_begin + it % tiles_per_head) * BT;
      float* a_lse = aux + st * 3 * BT;
      float* a_dlt = a_lse + BT;
      int* a_lo = reinterpret_cast<int*>(a_dlt + BT);
      if (qtr == 0) BWD_TRACE(0, hx);
      if (ok && tid128 < HB) {
        const int col = hf * HB + tid128;
        const int rq = q0 + col;
        const bool v = rq < p.T;
        const size_t si = (static_cast<size_t>(b) * p.H + hq) * p.T + (v ? rq : 0);
        a_lse[col] = v ? p.lse[si] * kLog2e_b : 0.f;
        a_dlt[col] = v ? p.delta[si] : 0.f;
        a_lo[col] = v ? lo_of_row(p, b, rq) : 0x7fffffff;    // invalid query rows see nothing
      }
      if (ch == 0) asm volatile("bar.sync 1, 128;" ::: "memory"); else asm volatile("bar.sync 2, 128;" ::: "memory");
      if (!ok) continue;
      if (!mbar_wait(&sdp_full[buf], (hx >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; continue; }
      tc_fence_after();
      if (qtr == 0) BWD_TRACE(1, hx);
      const float sl2 = p.scale_log2;
      // every (key, query) pair of the tile is visible: queries at or after the last key, no window / document bound
      const bool full_tile = plain_causal && q0 >= k0 + BT - 1 && q0 + BT <= p.T;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const uint32_t ts = tmem_base + buf * 128 + cc * 32 + lane_off, tdp = ts + 64;
        const int cbase = hf * HB + cc * 32;          // first query column (within the 128-query tile) of this chunk
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(ts, sr);
        tmem_ld_32x32(tdp, dr);
        tmem_ld_wait();
        uint32_t wp[16], wd[16];
        if (full_tile) {
          const float4* l4 = reinterpret_cast<const float4*>(a_lse + cbase);
          const float4* d4 = reinterpret_cast<const float4*>(a_dlt + cbase);
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4) {
            const float4 ls = l4[v4], dl = d4[v4];
            const float lsa[4] = {ls.x, ls.y, ls.z, ls.w}, dla[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int c = 4 * v4 + 2 * h2;
              const float p0 = exp2f(fmaf(__uint_as_float(sr[c]), sl2, -lsa[2 * h2]));
              const float p1 = exp2f(fmaf(__uint_as_float(sr[c + 1]), sl2, -lsa[2 * h2 + 1]));
              wp[c >> 1] = pack_bf16x2(p0, p1);
              wd[c >> 1] = pack_bf16x2(p0 * (__uint_as_float(dr[c]) - dla[2 * h2]), p1 * (__uint_as_float(dr[c + 1]) - dla[2 * h2 + 1]));
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            float pv[2], dv2[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int col = cbase + 2 * e + u;
              const int rq = q0 + col;
              float pr = exp2f(fmaf(__uint_as_float(sr[2 * e + u]), sl2, -a_lse[col]));
              if (!key_valid || kk > rq || kk < a_lo[col]) pr = 0.f;
              pv[u] = pr;
              dv2[u] = pr * (__uint_as_float(dr[2 * e + u]) - a_dlt[col]);
            }
            wp[e] = pack_bf16x2(pv[0], pv[1]);
            wd[e] = pack_bf16x2(dv2[0], dv2[1]);
          }
        }
        tmem_st_32x16(ts, wp);
        tmem_st_32x16(tdp, wd);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[buf]);
      if (qtr == 0) BWD_TRACE(2, hx);
    }
    if (!ok) goto done;
    if (!mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
    tc_fence_after();
    const size_t obase = ((static_cast<size_t>(b) * p.T + kk) * p.G + g) * D;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* orow = (which ? p.dk : p.dv) + obase;
      const uint32_t tsrc = which ? T_DK : T_DV;
      const float osc = which ? p.scale : 1.f;     // dSᵀ was formed without the softmax scale
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        const int col = ch * (D / 2) + c * 32;
        uint32_t rr[32];
        if (n_iter > 0) { tmem_ld_32x32(tsrc + col + lane_off, rr); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rr[e] = 0u;
        }
        if (key_valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(rr[e]) * osc, __uint_as_float(rr[e + 1]) * osc);
            o.y = pack_bf16x2(__uint_as_float(rr[e + 2]) * osc, __uint_as_float(rr[e + 3]) * osc);
            o.z = pack_bf16x2(__uint_as_float(rr[e + 4]) * osc, __uint_as_float(rr[e + 5]) * osc);
            o.w = pack_bf16x2(__uint_as_float(rr[e + 6]) * osc, __uint_as_float(rr[e + 7]) * osc);
            *reinterpret_cast<uint4*>(orow + col + e) = o;
          }
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

template <int D>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv,
                      const AttnBwdParams& p, cudaStream_t st) {
  auto kq = attn_bwd_dq_kernel<D>;
  auto kkv = attn_bwd_dkdv_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::TOTAL) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::TOTAL) != cudaSuccess) return -2;
    configured = true;
  }
  const int nt = (p.T + BT - 1) / BT;
  kkv<<<dim3(nt, p.G, p.B), BWD_THREADS, BwdSmem<D>::TOTAL, st>>>(tq, tdo, tk, tv, p);
  kq<<<dim3(nt, p.H, p.B), BWD_THREADS, BwdSmem<D>::TOTAL, st>>>(tq, tdo, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

// δ[b,h,r] = Σ_d dO·O alone (also used by the single-kernel backward in attention_bwd1.cu)
extern "C" int b200_attn_bwd_delta(const void* out, const void* d_out, float* delta, int B, int T, int H, int D, cudaStream_t stream) {
  using namespace b200;
  if (D != 64 && D != 128) return -1;
  const int grid = B * ((T + 31) / 32);
  const size_t dsm = static_cast<size_t>(H) * 32 * sizeof(float);
  if (dsm > 48 * 1024) return -1;
  if (D == 128) attn_bwd_delta_kernel<128><<<grid, 256, dsm, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, delta, B, T, H);
  else attn_bwd_delta_kernel<64><<<grid, 256, dsm, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, delta, B, T, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

long long* g_attn_bwd_trace = nullptr;   // also read by the single-kernel backward (attention_bwd1.cu)
extern "C" void b200_attn_bwd_set_trace(long long* buf) { g_attn_bwd_trace = buf; }

extern "C" int b200_attn_bwd(const void* d_out, const void* q, const void* k, const void* v, const void* out,
                             const float* lse, float* delta, const int* row_start, const int* doc_end, void* dq, void* dk,
                             void* dv, int B, int T, int H, int G, int D, int window_left, float scale, int* status,
                             cudaStream_t stream) {
  using namespace b200;
  if (B <= 0 || T <= 0) return 0;
  if ((D != 64 && D != 128) || H % G) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  const int grid = B * ((T + 31) / 32);
  const size_t dsm = static_cast<size_t>(H) * 32 * sizeof(float);
  if (dsm > 48 * 1024) return -1;
  if (D == 128) attn_bwd_delta_kernel<128><<<grid, 256, dsm, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, delta, B, T, H);
  else attn_bwd_delta_kernel<64><<<grid, 256, dsm, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, delta, B, T, H);
  CUtensorMap tq, tdo, tk, tv;
  const uint64_t hd = static_cast<uint64_t>(H) * D, gd = static_cast<uint64_t>(G) * D, bt = static_cast<uint64_t>(B) * T;
  int rc = make_tmap_2d_bf16(&tq, q, hd, bt, hd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tdo, d_out, hd, bt, hd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tk, k, gd, bt, gd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tv, v, gd, bt, gd, 64, 128);
  if (rc) return rc;
  AttnBwdParams p{lse, delta, row_start, doc_end, (__nv_bfloat16*)dq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv,
                  B, T, H, G, window_left, scale, scale * kLog2e_b, status, g_attn_bwd_trace};
  return D == 128 ? launch_bwd<128>(tq, tdo, tk, tv, p, stream) : launch_bwd<64>(tq, tdo, tk, tv, p, stream);
}
