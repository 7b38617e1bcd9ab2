// Attention backward in ONE kernel: five products per (key tile, query tile) pair instead of the seven of the two-kernel
// form (attention_bwd.cu computes S and dP twice, once per kernel), and one exponential per score instead of two.
//
// A CTA owns a key tile of 128 rows of one KV head and walks the query tiles (of all query heads of the group) that can
// see it, in the transposed domain (lane = key row):
//     Sᵀ = K·Qᵀ,  dPᵀ = V·dOᵀ                         (SS MMAs, N = 128 queries: full tensor rate)
//     Pᵀ = exp2(Sᵀ·c − lse),  dSᵀ = Pᵀ∘(dPᵀ − δ)      (8 conversion warps; Pᵀ → tensor memory in place of Sᵀ,
//                                                       dSᵀ → one swizzled bf16 tile in shared memory)
//     dV += Pᵀ·dO          (A from tensor memory)
//     dK += dSᵀ·Q          (A = the dSᵀ tile read K-major)
//     dQ_i = dS·K          (A = the SAME tile read MN-major: rows of 64 queries per key are what both views want)
// dK / dV accumulate in tensor memory over the whole loop (GQA reduction included).  dQ_i is a per-pair partial result: it
// is produced in the tensor-memory columns that held dPᵀ (free once dSᵀ is in shared memory), read out by four more warps
// (through a ring of three 8 KB shared-memory pieces) and added into an fp32 accumulator in global memory with bulk tensor
// reductions (cp.reduce.async.bulk.tensor, add: whole 64-byte row pieces per L2 operation; per-thread red.global of rows
// 8 KB apart was several times slower); a small kernel scales and converts it afterwards.  The sum order of dQ over key tiles therefore depends on scheduling: results are
// not bitwise reproducible (the two-kernel form in attention_bwd.cu is, and stays available).
//
// TMEM columns: Sᵀ/Pᵀ 0..127 | dPᵀ → dQ_i 128..255 | dV 256..256+D | dK 384..384+D.
// Shared memory: K, V (fixed) | Q two stages | dO one stage | dSᵀ tile | dQ ring | per-query lse·log2e, δ, lo for two stages.
// Warps: 0 TMA, 1 MMA (one thread issues every product: MMAs of one thread execute in issue order, so "dV += Pᵀ·dO"
// followed by the next Sᵀ into the same columns needs no barrier), 2..3 idle, 4..11 conversion (two groups of four: group
// c owns query columns 64c..64c+63), 12..15 dQ read-out.  Registers are rebalanced with setmaxnreg.
// Issue order in the steady state, after dSᵀ of tile i is in shared memory:
//     dQ_i, dK += …_i, dV += …_{i+1}, [dQ_i read out] dPᵀ_{i+1}, Sᵀ_{i+2}
// so that the read-out of dQ_i runs under dK/dV, the conversion of Pᵀ_{i+1} under dQ_i/dK and that of dSᵀ_{i+1} under
// Sᵀ_{i+2}.
// Masking rule as in the forward: query r sees keys lo(r) ≤ k ≤ r.
#include "sm100.cuh"
#include "api.h"

extern long long* g_attn_bwd_trace;     // attention_bwd.cu: set through b200_attn_bwd_set_trace

namespace b200 {

constexpr int B1T = 128;
constexpr int B1_THREADS = 512;
constexpr float kLog2e_b1 = 1.4426950408889634f;

int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_3d_f32_sw64(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch,
                          uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_rows);

struct AttnBwd1Params {
  const float* lse;        // [B,H,T] natural log
  const float* delta;      // [B,H,T]
  const int* row_start;    // [B*T] or null
  const int* doc_end;      // [B*T] or null
  float* dq_acc;           // [B,T,H,D] fp32, zero on entry
  __nv_bfloat16* dk;       // [B,T,G,D]
  __nv_bfloat16* dv;
  int B, T, H, G;
  int window_left;
  float scale, scale_log2;
  int* status;
  long long* trace;        // optional [12][64] clock64 stamps of the first CTA (development aid, null in normal use)
};
#define B1_TRACE(ev, it) do { if (p.trace && traced && (it) < 64) p.trace[(ev) * 64 + (it)] = clock64(); } while (0)

template <int D>
struct Bwd1Smem {
  static constexpr int TILE = B1T * D * 2;
  static constexpr int DS_BYTES = B1T * B1T * 2;
  static constexpr int DQ_PIECE = B1T * 16 * 4;          // 128 queries × 16 head-dim columns, fp32
  static constexpr int DQ_RING = 3 * DQ_PIECE;
  static constexpr int AUX = 2 * 3 * B1T * 4;
  static constexpr int TOTAL = 2 * TILE /*K,V*/ + 2 * TILE /*Q ring*/ + TILE /*dO*/ + DS_BYTES + DQ_RING + AUX + 1024 + 256;
};

// AND of a predicate over the 128 threads of named barrier 3 (the read-out warps): every one of them gets the same answer.
__device__ __forceinline__ bool readout_all(bool v) {
  uint32_t out;
  asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, 3, 128, q; selp.u32 %0, 1, 0, p; }"
               : "=r"(out) : "r"(static_cast<uint32_t>(v)) : "memory");
  return out != 0;
}

template <int D>
__global__ void __launch_bounds__(B1_THREADS, 1)
attn_bwd1_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                 const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                 const __grid_constant__ CUtensorMap tmap_dq, const AttnBwd1Params p) {
  using SM = Bwd1Smem<D>;
  constexpr int DC = D / 64;
  constexpr int CHUNK_BYTES = 128 * 64 * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sk = smem;
  uint8_t* sv = smem + SM::TILE;
  uint8_t* sqr = smem + 2 * SM::TILE;                 // Q stage s at sqr + s·TILE
  uint8_t* sdo = smem + 4 * SM::TILE;
  uint8_t* sds = smem + 5 * SM::TILE;                 // dSᵀ: two chunks [128 keys × 64 queries], 128-byte rows, swizzled
  uint8_t* sdq = sds + SM::DS_BYTES;                  // dQ ring: three pieces [128 queries × 16 floats], 64-byte rows, swizzled
  float* aux = reinterpret_cast<float*>(sdq + SM::DQ_RING);    // stage s: [lse2 | delta | lo] × 128
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(aux) + SM::AUX);
  uint64_t* kv_full = bars;          // 1
  uint64_t* q_full = bars + 1;       // [2]
  uint64_t* q_empty = bars + 3;      // [2]  dK of the tile has completed (Q stage free)
  uint64_t* do_full = bars + 5;      // 1
  uint64_t* do_empty = bars + 6;     // 1    dV of the tile has completed (dO buffer free)
  uint64_t* s_full = bars + 7;       // 1
  uint64_t* dp_full = bars + 8;      // 1
  uint64_t* p_ready = bars + 9;      // 1    (count 8) Pᵀ is in tensor memory
  uint64_t* ds_ready = bars + 10;    // 1    (count 8) dSᵀ is in shared memory and dPᵀ has been read
  uint64_t* dq_full = bars + 11;     // 1    dQ_i is in tensor memory
  uint64_t* dq_empty = bars + 12;    // 1    (count 4) dQ_i has been read out
  uint64_t* acc_done = bars + 13;    // 1
  uint64_t* ds_free = bars + 14;     // 1    dK and dQ of the tile have completed (dSᵀ tile free)
  uint64_t* aux_full = bars + 15;    // [2]  (count 2) statistics of the tile are in shared memory
  uint64_t* aux_empty = bars + 17;   // [2]  (count 8) the conversion warps are done with them
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp == 1 || warp == 4 || warp == 12);
  // key tile on the slow grid axis: CTAs start in order of decreasing work under a causal mask (tile 0 sees every query)
  const int jt = blockIdx.y, g = blockIdx.x % p.G, b = blockIdx.x / p.G;
  const int k0 = jt * B1T;
  const int k_last = min(k0 + B1T, p.T) - 1;
  const int group = p.H / p.G;
  int r_hi = p.T - 1;                                  // last query row that can see a key of this tile
  if (p.window_left >= 0) r_hi = min(r_hi, k_last + p.window_left);
  if (p.doc_end) r_hi = min(r_hi, p.doc_end[static_cast<size_t>(b) * p.T + k_last] - 1);
  const int i_begin = k0 / B1T, i_end = r_hi / B1T + 1;
  const int tiles_per_head = i_end - i_begin;
  const int n_iter = tiles_per_head * group;           // ≥ 1

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    mbar_init(do_full, 1); mbar_init(do_empty, 1); mbar_init(s_full, 1); mbar_init(dp_full, 1);
    mbar_init(p_ready, 8); mbar_init(ds_ready, 8); mbar_init(dq_full, 1); mbar_init(dq_empty, 4); mbar_init(acc_done, 1);
    mbar_init(ds_free, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&aux_full[s], 2); mbar_init(&aux_empty[s], 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t T_S = tmem_base, T_DP = tmem_base + 128, T_DV = tmem_base + 256, T_DK = tmem_base + 384;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA
      mbar_arrive_expect_tx(kv_full, 2 * SM::TILE);
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        tma_load_2d(sk + c * CHUNK_BYTES, &tmap_k, kv_full, g * D + c * 64, b * p.T + k0);
        tma_load_2d(sv + c * CHUNK_BYTES, &tmap_v, kv_full, g * D + c * 64, b * p.T + k0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1; const uint32_t ph = (it >> 1) & 1;
        const int hq = g * group + it / tiles_per_head;
        const int q0 = (i_begin + it % tiles_per_head) * B1T;
        if (!mbar_wait_relaxed(&q_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        mbar_arrive_expect_tx(&q_full[st], SM::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_2d(sqr + st * SM::TILE + c * CHUNK_BYTES, &tmap_q, &q_full[st], hq * D + c * 64, b * p.T + q0);
        if (!mbar_wait_relaxed(do_empty, (it & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        mbar_arrive_expect_tx(do_full, SM::TILE);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_2d(sdo + c * CHUNK_BYTES, &tmap_do, do_full, hq * D + c * 64, b * p.T + q0);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA (one thread, dependency order)
      constexpr uint32_t idesc_s = make_idesc_bf16(B1T, B1T, 0, 0);        // Sᵀ = K·Qᵀ, dPᵀ = V·dOᵀ (all K-major)
      constexpr uint32_t idesc_acc = make_idesc_bf16(B1T, D, 0, 1);       // dV, dK: B = dO / Q read N-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(B1T, D, 1, 1);        // dQ_i = dS·K: A = dSᵀ tile read MN-major, B = K N-major
      if (!mbar_wait(kv_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      const uint32_t ska = smem_u32(sk), sva = smem_u32(sv), sdoa = smem_u32(sdo), sdsa = smem_u32(sds);
      auto issue_s = [&](int it) -> bool {
        const int st = it & 1;
        if (!mbar_wait(&q_full[st], (it >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t sqa = smem_u32(sqr + st * SM::TILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * CHUNK_BYTES + (k % 4) * 32;
          umma_bf16(T_S, make_smem_desc(ska + off, 16, 1024), make_smem_desc(sqa + off, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(s_full);
        return true;
      };
      auto issue_dp = [&](int it) -> bool {   // dO of the tile is in shared memory (issue_dv waited for it, or the prologue)
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * CHUNK_BYTES + (k % 4) * 32;
          umma_bf16(T_DP, make_smem_desc(sva + off, 16, 1024), make_smem_desc(sdoa + off, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(dp_full);
        return true;
      };
      auto issue_dv = [&](int it) -> bool {   // dV += Pᵀ·dO
        if (!mbar_wait(p_ready, it & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < B1T / 16; ++k)     // packed Pᵀ: 16 queries = 8 columns; group c's 64 queries start at column 64c
          umma_bf16_ts(T_DV, T_S + (k >> 2) * 64 + (k & 3) * 8, make_smem_desc(sdoa + k * 2048, CHUNK_BYTES, 1024), idesc_acc,
                       (it | k) != 0);
        return true;
      };
      // prologue: Sᵀ_0, dPᵀ_0, dV_0, Sᵀ_1
      if (!issue_s(0)) goto done;
      if (!mbar_wait(do_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      issue_dp(0);
      if (!issue_dv(0)) goto done;
      umma_commit(do_empty);                   // dPᵀ_0 and dV_0 have read dO_0
      if (1 < n_iter && !issue_s(1)) goto done;
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1; const uint32_t ph = it & 1;
        const uint32_t sqa = smem_u32(sqr + st * SM::TILE);
        if (!mbar_wait(ds_ready, ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        B1_TRACE(0, it);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < B1T / 16; ++k)     // dQ_i = dS·K.  A: the dSᵀ tile MN-major (M = queries, K = keys): 16 keys = 2048 bytes
          umma_bf16(T_DP, make_smem_desc(sdsa + k * 2048, CHUNK_BYTES, 1024), make_smem_desc(ska + k * 2048, CHUNK_BYTES, 1024),
                    idesc_dq, k != 0);
        umma_commit(dq_full);
#pragma unroll
        for (int k = 0; k < B1T / 16; ++k)     // dK += dSᵀ·Q.  A: the tile K-major (K = queries): chunk k/4, 32 bytes per 16 queries
          umma_bf16(T_DK, make_smem_desc(sdsa + (k >> 2) * CHUNK_BYTES + (k & 3) * 32, 16, 1024),
                    make_smem_desc(sqa + k * 2048, CHUNK_BYTES, 1024), idesc_acc, (it | k) != 0);
        umma_commit(&q_empty[st]);
        umma_commit(ds_free);
        B1_TRACE(1, it);
        if (it + 1 < n_iter) {
          if (!mbar_wait(do_full, (it + 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
          if (!issue_dv(it + 1)) goto done;
          B1_TRACE(2, it);
          // dPᵀ of the next tile goes into the columns of dQ_i: wait for the read-out
          if (!mbar_wait(dq_empty, ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
          B1_TRACE(3, it);
          issue_dp(it + 1);
          umma_commit(do_empty);
          if (it + 2 < n_iter && !issue_s(it + 2)) goto done;
          B1_TRACE(4, it);
        }
      }
      umma_commit(acc_done);
    } else if (warp >= 2) {
      // ---------------------------------------------------------------- per-query statistics, one tile ahead of the conversion
      const int t64 = (warp - 2) * 32 + lane;
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const int hq = g * group + it / tiles_per_head;
        const int q0 = (i_begin + it % tiles_per_head) * B1T;
        float* a_lse = aux + st * 3 * B1T;
        float* a_dlt = a_lse + B1T;
        int* a_lo = reinterpret_cast<int*>(a_dlt + B1T);
        bool okw = mbar_wait_relaxed(&aux_empty[st], ((it >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY);
        if (!__all_sync(0xffffffffu, okw)) break;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int col = t64 + u * 64;
          const int rq = q0 + col;
          const bool v = rq < p.T;
          const size_t si = (static_cast<size_t>(b) * p.H + hq) * p.T + (v ? rq : 0);
          a_lse[col] = v ? p.lse[si] * kLog2e_b1 : 0.f;
          a_dlt[col] = v ? p.delta[si] : 0.f;
          a_lo[col] = v ? (p.row_start ? max(p.row_start[static_cast<size_t>(b) * p.T + rq], p.window_left >= 0 ? rq - p.window_left : 0)
                                       : (p.window_left >= 0 ? max(rq - p.window_left, 0) : 0))
                        : 0x7fffffff;                 // invalid query rows see nothing
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&aux_full[st]);
      }
    }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
    // ------------------------------------------------------------------ conversion: Pᵀ and dSᵀ
    const int qtr = warp & 3, ch = (warp - 4) >> 2;
    const int kk = k0 + qtr * 32 + lane;               // this thread's key row
    const bool key_valid = kk < p.T;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const int krow = qtr * 32 + lane;
    const bool plain_causal = p.row_start == nullptr && p.window_left < 0 && k0 + B1T <= p.T;
    const int tid128 = qtr * 32 + lane;
    const float sl2 = p.scale_log2;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int st = it & 1; const uint32_t ph = it & 1;
      const int hq = g * group + it / tiles_per_head;
      const int q0 = (i_begin + it % tiles_per_head) * B1T;
      const float* a_lse = aux + st * 3 * B1T;
      const float* a_dlt = a_lse + B1T;
      const int* a_lo = reinterpret_cast<const int*>(a_dlt + B1T);
      if (ok && !mbar_wait(&aux_full[st], (it >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) ok = false;
      const bool full_tile = plain_causal && q0 >= k0 + B1T - 1 && q0 + B1T <= p.T;
      const int cbase = ch * 64;
      uint32_t pk[32];                                  // Pᵀ of this thread's 64 queries, packed bf16 (kept for dSᵀ)
      // ---- Pᵀ
      if (ok && !mbar_wait(s_full, ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      B1_TRACE(5, it);
      if (ok) {
        tc_fence_after();
        uint32_t sr[64];
        tmem_ld_32x32(T_S + cbase + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
        tmem_ld_32x32(T_S + cbase + 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
        tmem_ld_wait();
        if (full_tile) {                                // every (key, query) pair of the tile is visible
          const float4* l4 = reinterpret_cast<const float4*>(a_lse + cbase);
#pragma unroll
          for (int v4 = 0; v4 < 16; ++v4) {
            const float4 ls = l4[v4];
            pk[2 * v4] = pack_bf16x2(exp2f(fmaf(__uint_as_float(sr[4 * v4]), sl2, -ls.x)),
                                     exp2f(fmaf(__uint_as_float(sr[4 * v4 + 1]), sl2, -ls.y)));
            pk[2 * v4 + 1] = pack_bf16x2(exp2f(fmaf(__uint_as_float(sr[4 * v4 + 2]), sl2, -ls.z)),
                                         exp2f(fmaf(__uint_as_float(sr[4 * v4 + 3]), sl2, -ls.w)));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float pv[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int col = cbase + 2 * e + u;
              const int rq = q0 + col;
              float pr = exp2f(fmaf(__uint_as_float(sr[2 * e + u]), sl2, -a_lse[col]));
              if (!key_valid || kk > rq || kk < a_lo[col]) pr = 0.f;
              pv[u] = pr;
            }
            pk[e] = pack_bf16x2(pv[0], pv[1]);
          }
        }
        tmem_st_32x16(T_S + cbase + lane_off, *reinterpret_cast<uint32_t(*)[16]>(&pk[0]));
        tmem_st_32x16(T_S + cbase + 16 + lane_off, *reinterpret_cast<uint32_t(*)[16]>(&pk[16]));
        tmem_st_wait();
        tc_fence_before();
      }
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(p_ready);
      B1_TRACE(6, it);
      // ---- dSᵀ → shared memory (the tile of the previous pair must have been consumed)
      if (ok && it > 0 && !mbar_wait(ds_free, (it - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) ok = false;
      if (ok && !mbar_wait(dp_full, ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      B1_TRACE(7, it);
      if (ok) {
        tc_fence_after();
        uint32_t dr[64];
        tmem_ld_32x32(T_DP + cbase + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&dr[0]));
        tmem_ld_32x32(T_DP + cbase + 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&dr[32]));
        tmem_ld_wait();
        tc_fence_before();
        uint8_t* row = sds + ch * CHUNK_BYTES + krow * 128;     // this key's 64 queries of chunk ch: 8 pieces of 16 bytes
        const float4* d4 = reinterpret_cast<const float4*>(a_dlt + cbase);
#pragma unroll
        for (int v8 = 0; v8 < 8; ++v8) {
          uint32_t w4[4];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int v4 = v8 * 2 + j;                  // queries cbase + 4·v4 .. + 3
            const float4 dl = d4[v4];
            const float2 pa = unpack_bf16x2(pk[2 * v4]), pb = unpack_bf16x2(pk[2 * v4 + 1]);
            w4[2 * j] = pack_bf16x2(pa.x * (__uint_as_float(dr[4 * v4]) - dl.x), pa.y * (__uint_as_float(dr[4 * v4 + 1]) - dl.y));
            w4[2 * j + 1] = pack_bf16x2(pb.x * (__uint_as_float(dr[4 * v4 + 2]) - dl.z), pb.y * (__uint_as_float(dr[4 * v4 + 3]) - dl.w));
          }
          *reinterpret_cast<uint4*>(row + ((v8 ^ (krow & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
        fence_proxy_async_smem();                       // generic-proxy stores → visible to the MMA's async-proxy reads
      }
      __syncwarp();
      if (ok && lane == 0) { mbar_arrive(ds_ready); mbar_arrive(&aux_empty[st]); }
      B1_TRACE(8, it);
    }
    // ---- epilogue: dV, dK (group ch stores head-dim columns [ch·D/2, (ch+1)·D/2))
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const size_t obase = ((static_cast<size_t>(b) * p.T + kk) * p.G + g) * D;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* orow = (which ? p.dk : p.dv) + obase;
        const uint32_t tsrc = which ? T_DK : T_DV;
        const float osc = which ? p.scale : 1.f;       // dSᵀ was formed without the softmax scale
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          const int col = ch * (D / 2) + c * 32;
          uint32_t rr[32];
          tmem_ld_32x32(tsrc + col + lane_off, rr);
          tmem_ld_wait();
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
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
    // ------------------------------------------------------------------ dQ read-out: thread = query row of the tile
    const int qtr = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const int r = qtr * 32 + lane;
    const uint32_t sw = (r >> 1) & 3;                  // 64-byte swizzle: 16-byte piece index ^= address bits 7..8
    uint32_t piece = 0;                                 // ring position, counted over the whole loop
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int hq = g * group + it / tiles_per_head;
      const int q0 = (i_begin + it % tiles_per_head) * B1T;
      if (ok && !mbar_wait_relaxed(dq_full, it & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
      ok = readout_all(ok);                             // the four warps go on together or not at all (they share a barrier below)
      if (!ok) break;
      B1_TRACE(9, it);
      tc_fence_after();
      uint32_t rr[D];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_32x32(T_DP + c * 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&rr[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);             // the columns are free for the next dPᵀ
      B1_TRACE(10, it);
#pragma unroll
      for (int c = 0; c < D / 16; ++c, ++piece) {
        // the piece written three steps ago has been read by its reduction: thread 0 checked before the last barrier
        uint8_t* row = sdq + (piece % 3) * SM::DQ_PIECE + r * 64;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(row + ((j ^ sw) << 4)) =
              make_uint4(rr[c * 16 + 4 * j], rr[c * 16 + 4 * j + 1], rr[c * 16 + 4 * j + 2], rr[c * 16 + 4 * j + 3]);
        fence_proxy_async_smem();
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (threadIdx.x == 12 * 32) {
          tma_reduce_add_3d(&tmap_dq, sdq + (piece % 3) * SM::DQ_PIECE, hq * D + c * 16, q0, b);
          tma_store_commit();
          tma_store_wait_read<1>();
        }
      }
      B1_TRACE(11, it);
    }
    if (threadIdx.x == 12 * 32) tma_store_wait<0>();
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

// dq (bf16) = scale · dq_acc (fp32); n % 8 == 0
__global__ void __launch_bounds__(256) attn_bwd1_finish_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n8,
                                                              float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(acc)[2 * i], c = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    uint4 o;
    o.x = pack_bf16x2(a.x * scale, a.y * scale); o.y = pack_bf16x2(a.z * scale, a.w * scale);
    o.z = pack_bf16x2(c.x * scale, c.y * scale); o.w = pack_bf16x2(c.z * scale, c.w * scale);
    reinterpret_cast<uint4*>(dq)[i] = o;
  }
}

template <int D>
static int launch_bwd1(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv,
                       const CUtensorMap& tdq, const AttnBwd1Params& p, cudaStream_t st) {
  auto kern = attn_bwd1_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd1Smem<D>::TOTAL) != cudaSuccess) return -2;
    configured = true;
  }
  const int nt = (p.T + B1T - 1) / B1T;
  kern<<<dim3(p.G * p.B, nt), B1_THREADS, Bwd1Smem<D>::TOTAL, st>>>(tq, tdo, tk, tv, tdq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

// Single-kernel backward.  dq_acc: fp32 scratch [B,T,H,D] (zeroed here); delta: fp32 scratch [B,H,T]; otherwise the
// contract of b200_attn_bwd.  dQ sums are not bitwise reproducible (see the top of this file).
extern "C" int b200_attn_bwd_delta(const void* out, const void* d_out, float* delta, int B, int T, int H, int D, cudaStream_t stream);

extern "C" int b200_attn_bwd1(const void* d_out, const void* q, const void* k, const void* v, const void* out, const float* lse,
                              float* delta, float* dq_acc, const int* row_start, const int* doc_end, void* dq, void* dk, void* dv,
                              int B, int T, int H, int G, int D, int window_left, float scale, int* status, cudaStream_t stream) {
  using namespace b200;
  if (B <= 0 || T <= 0) return 0;
  if ((D != 64 && D != 128) || H % G) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  int rc = b200_attn_bwd_delta(out, d_out, delta, B, T, H, D, stream);
  if (rc) return rc;
  const size_t n = static_cast<size_t>(B) * T * H * D;
  if (cudaMemsetAsync(dq_acc, 0, n * sizeof(float), stream) != cudaSuccess) return -6;
  CUtensorMap tq, tdo, tk, tv, tdq;
  const uint64_t hd = static_cast<uint64_t>(H) * D, gd = static_cast<uint64_t>(G) * D, bt = static_cast<uint64_t>(B) * T;
  rc = make_tmap_2d_bf16(&tq, q, hd, bt, hd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tdo, d_out, hd, bt, hd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tk, k, gd, bt, gd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tv, v, gd, bt, gd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_3d_f32_sw64(&tdq, dq_acc, hd, T, B, hd, static_cast<uint64_t>(T) * hd, 128);
  if (rc) return rc;
  AttnBwd1Params p{lse, delta, row_start, doc_end, dq_acc, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv,
                   B, T, H, G, window_left, scale, scale * kLog2e_b1, status, g_attn_bwd_trace};
  rc = D == 128 ? launch_bwd1<128>(tq, tdo, tk, tv, tdq, p, stream) : launch_bwd1<64>(tq, tdo, tk, tv, tdq, p, stream);
  if (rc) return rc;
  const long long n8 = static_cast<long long>(n / 8);
  long long blocks = (n8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  attn_bwd1_finish_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), n8, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
