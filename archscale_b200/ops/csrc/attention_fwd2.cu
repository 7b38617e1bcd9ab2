// Attention forward on SM pairs (tcgen05.mma.cta_group::2), head_dim 128: causal / sliding-window / packed-varlen, GQA.
//
// A cluster of two CTAs owns two adjacent query tiles of 128 rows (256 query rows per MMA): CTA r keeps its own Q tile,
// 64 of the 128 keys of every K tile and 64 of the 128 head-dim columns of every V tile in shared memory, and one thread
// of the even ("leader") CTA issues M256 × N128 × K16 MMAs that read both CTAs' shared memory.  One instruction therefore
// does the work of two one-CTA instructions — the one-CTA kernel (attention_fwd.cu) is bound by the rate at which
// tcgen05.mma instructions can be issued (≈85 cycles each, whatever their N) — and each CTA stages half the K/V bytes.
//
// Per CTA, 352 threads:
//   warp 0       TMA: Q once, then its K / V halves through a 4-stage ring; every load signals the leader's `full` barrier
//   warp 1       (leader) S_j = Q·K_jᵀ into one of two 128-column TMEM buffers of each CTA
//   warp 10      (leader) O += P_j·V_j, P_j (bf16) read from each CTA's TMEM as the A operand
//   warps 2..9   softmax of the CTA's own 128 rows by TWO warp groups: group w owns key columns 64w..64w+63 of every
//                tile, so two threads share a row.  One warp per scheduler cannot hide the latency of its own
//                load → max → exp2 → pack → store chain (measured: the tile time did not move when the MMA work per
//                instruction doubled); two warps per scheduler, each with half the chain, can.  The two halves of a row
//                exchange their maxima through shared memory (one named barrier per tile), use the same running max,
//                keep separate row sums (added at the end) and each rescale / store their own 64 columns of O.
//                Online softmax in base 2 with lazy rescaling of O; a quarter of the exponentials is evaluated on the
//                FMA pipe (Cody–Waite split + cubic) instead of MUFU.
// tcgen05.commit arrives on the barriers of both CTAs; the softmax warps of both CTAs arrive on the leader's barriers.
// No TMA load uses cluster multicast.  Every wait is bounded; both CTAs leave through a cluster barrier.
//
// Masking as in attention_fwd.cu: query row r sees keys lo(r) ≤ k ≤ r.  The pair walks the union of its two tiles' key
// ranges; the odd tile's extra diagonal tile is fully masked for the even tile (≈3 % more MMA work at T = 4096).
//
// TMEM columns (per CTA): S0 0..127 | S1 128..255 | P0 256..319 | P1 320..383 | O 384..511.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int A2_BM = 128, A2_BN = 128, A2_D = 128;
constexpr int A2_THREADS = 352;
constexpr int A2_PV_WARP = 10;
constexpr int A2_SOFTMAX_THREADS = 256;
constexpr int A2_STAGES = 4;
constexpr int A2_Q_BYTES = A2_BM * A2_D * 2;            // 32 KB: this CTA's query tile
constexpr int A2_KH_BYTES = (A2_BN / 2) * A2_D * 2;     // 16 KB: 64 keys × 128
constexpr int A2_VH_BYTES = A2_BN * (A2_D / 2) * 2;     // 16 KB: 128 keys × 64 head-dim columns
constexpr int A2_STAGE_BYTES = A2_KH_BYTES + A2_VH_BYTES;
constexpr int A2_SMEM = A2_Q_BYTES + A2_STAGES * A2_STAGE_BYTES + 1024 + 512 + 6 * A2_BM * 4;
constexpr float kLog2e2 = 1.4426950408889634f, kLn2_2 = 0.6931471805599453f;

struct AttnFwd2Params {
  __nv_bfloat16* out;      // [B, T, H, D]
  float* lse;              // [B, H, T]
  const int* row_start;    // [B*T] or null
  int B, T, H, G;
  int window_left;         // < 0: unlimited
  float scale_log2;
  int* status;
};

// 2^x on the FMA pipe: floor by a round-down add of 1.5·2^23, cubic for the fraction (max relative error 8.6e-5, below
// bf16 resolution), exponent added into the float's bit pattern.  x is clamped at −126, so a masked score (−inf) gives 2^−126.
__device__ __forceinline__ float exp2_fma(float x) {
  x = fmaxf(x, -126.f);
  float xr;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(xr) : "f"(x), "f"(12582912.f));
  const float f = x - (xr - 12582912.f);
  const float pl = fmaf(fmaf(fmaf(0.07706617563962936f, f, 0.22764593362808228f), f, 0.6951165795326233f), f, 1.f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(xr) << 23));
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(A2_THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnFwd2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  uint8_t* ring = smem + A2_Q_BYTES;                // stage s: K half at ring + s·STAGE, V half right after
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + A2_STAGES * A2_STAGE_BYTES);
  uint64_t* q_full = bars;                          // leader
  uint64_t* k_full = bars + 1;                      // [STAGES] leader
  uint64_t* v_full = k_full + A2_STAGES;            // [STAGES] leader
  uint64_t* k_empty = v_full + A2_STAGES;           // [STAGES] each CTA
  uint64_t* v_empty = k_empty + A2_STAGES;          // [STAGES] each CTA
  uint64_t* s_full = v_empty + A2_STAGES;           // [2] each CTA
  uint64_t* s_empty = s_full + 2;                   // [2] leader, 16 arrivals (8 warps × 2 CTAs)
  uint64_t* p_full = s_empty + 2;                   // [2] leader, 16 arrivals
  uint64_t* p_empty = p_full + 2;                   // [2] each CTA
  uint64_t* o_done = p_empty + 2;                   // each CTA
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  float* xmax = reinterpret_cast<float*>(tmem_ptr + 4);          // [2 tile parities][2 groups][128 rows]
  float* xsum = xmax + 2 * 2 * A2_BM;                            // [2 groups][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int n_qt = (p.T + A2_BM - 1) / A2_BM;
  const int n_pairs = (n_qt + 1) >> 1;
  const int pr = n_pairs - 1 - (static_cast<int>(blockIdx.x) >> 1);      // heavy (late) pairs first
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int q0p = pr * 2 * A2_BM;
  const int q0 = q0p + rank * A2_BM;
  const int r_last_pair = min(q0p + 2 * A2_BM, p.T) - 1;
  const int r_last = min(q0 + A2_BM, p.T) - 1;
  auto lo_of = [&](int r) {
    int lo = p.row_start ? p.row_start[static_cast<size_t>(b) * p.T + r] : 0;
    if (p.window_left >= 0) lo = max(lo, r - p.window_left);
    return lo;
  };
  const int j_begin = lo_of(q0p) / A2_BN;
  const int n_tiles = r_last_pair / A2_BN + 1 - j_begin;                 // ≥ 1, the same in both CTAs

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < A2_STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 16); mbar_init(&p_full[s], 16); mbar_init(&p_empty[s], 1);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) { tmem_alloc_2sm(tmem_ptr, 512); tmem_relinquish_2sm(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t T_S0 = tmem_base, T_P0 = tmem_base + 256, T_O = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      if (rank == 0) mbar_arrive_expect_tx(q_full, 2 * A2_Q_BYTES);
#pragma unroll
      for (int c = 0; c < 2; ++c) tma_load_2d_2sm(sq + c * 16384, &tmap_q, q_full, h * A2_D + c * 64, b * p.T + q0);
      int st = 0; uint32_t ph = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int k0 = (j_begin + t) * A2_BN;
        uint8_t* sk = ring + st * A2_STAGE_BYTES;
        uint8_t* sv = sk + A2_KH_BYTES;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        if (rank == 0) mbar_arrive_expect_tx(&k_full[st], 2 * A2_KH_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)        // this CTA's 64 keys, two 64-element chunks of the head dim
          tma_load_2d_2sm(sk + c * 8192, &tmap_k, &k_full[st], g * A2_D + c * 64, b * p.T + k0 + rank * 64);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        if (rank == 0) mbar_arrive_expect_tx(&v_full[st], 2 * A2_VH_BYTES);
        tma_load_2d_2sm(sv, &tmap_v, &v_full[st], g * A2_D + rank * 64, b * p.T + k0);   // all 128 keys, this CTA's 64 columns
        if (++st == A2_STAGES) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(2 * A2_BM, A2_BN, 0, 0);     // S = Q·Kᵀ, both K-major
      if (!mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      const uint32_t sqa = smem_u32(sq);
      int st = 0; uint32_t ph = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int buf = t & 1; const uint32_t bph = (t >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
        if (!mbar_wait(&s_empty[buf], bph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t sk = smem_u32(ring + st * A2_STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < A2_D / 16; ++k)
          umma_bf16_2sm(T_S0 + buf * 128, make_smem_desc(sqa + (k / 4) * 16384 + (k % 4) * 32, 16, 1024),
                        make_smem_desc(sk + (k / 4) * 8192 + (k % 4) * 32, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        umma_commit_2sm(&s_full[buf], 3);
        umma_commit_2sm(&k_empty[st], 3);
        if (++st == A2_STAGES) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == A2_PV_WARP) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_o = make_idesc_bf16(2 * A2_BM, A2_D, 0, 1);      // O += P·V, V is N-major (64 columns per CTA)
      int st = 0; uint32_t ph = 0;
      for (int t = 0; t < n_tiles; ++t) {
        const int buf = t & 1; const uint32_t bph = (t >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
        if (!mbar_wait(&p_full[buf], bph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        tc_fence_after();
        const uint32_t sv = smem_u32(ring + st * A2_STAGE_BYTES + A2_KH_BYTES);
#pragma unroll
        for (int k = 0; k < A2_BN / 16; ++k)      // A: 8 packed columns per 16 keys; B: 16 key rows = 2048 bytes further
          umma_bf16_ts_2sm(T_O, T_P0 + buf * 64 + k * 8, make_smem_desc(sv + k * 2048, A2_VH_BYTES, 1024), idesc_o,
                           (t | k) != 0 ? 1u : 0u);
        umma_commit_2sm(&v_empty[st], 3);
        umma_commit_2sm(&p_empty[buf], 3);
        umma_commit_2sm(o_done, 3);
        if (++st == A2_STAGES) { st = 0; ph ^= 1; }
      }
    }
  } else {
    const int qtr = warp & 3, wg = (warp - 2) >> 2;              // TMEM lane quarter of this warp; column half of its group
    const int row_in_tile = qtr * 32 + lane;
    const int r = q0 + row_in_tile;
    const bool row_valid = r < p.T;
    const int lo_r = row_valid ? lo_of(r) : 0;
    const int lo_last = lo_of(r_last);
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const float sl2 = p.scale_log2;
    float m_used = -1e30f, l_sum = 0.f;
    bool ok = true;      // after a timed-out wait the thread keeps meeting its partner group at the named barrier, idle
    for (int t = 0; t < n_tiles; ++t) {
      const int buf = t & 1; const uint32_t bph = (t >> 1) & 1;
      const int k0 = (j_begin + t) * A2_BN + wg * 64;            // first key column of this thread's half
      float s[64];
      float mloc = -INFINITY;
      if (ok && !mbar_wait(&s_full[buf], bph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tmem_ld_32x32(T_S0 + buf * 128 + wg * 64 + c * 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_leader(&s_empty[buf]);        // S buffer may be overwritten by S_{t+2}
        const int kt0 = (j_begin + t) * A2_BN;
        const bool full_tile = (kt0 + A2_BN - 1 <= q0) && (kt0 >= lo_last);
        if (!full_tile) {
#pragma unroll
          for (int e = 0; e < 64; ++e) {
            const int kk = k0 + e;
            if (kk > r || kk < lo_r) s[e] = -INFINITY;
          }
        }
        float mx8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) mx8[e] = s[e];
#pragma unroll
        for (int e = 8; e < 64; ++e) mx8[e & 7] = fmaxf(mx8[e & 7], s[e]);
        mloc = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
        xmax[(buf * 2 + wg) * A2_BM + row_in_tile] = mloc;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");              // both halves of every row have published their maximum
      if (!ok) continue;
      const float mx = fmaxf(mloc, xmax[(buf * 2 + (wg ^ 1)) * A2_BM + row_in_tile]) * sl2;
      // lazy rescale: only when the running max grew by more than 8 (factor 256); decided per warp, and the same way in
      // both groups (their warps with the same lane quarter see the same 32 rows)
      const bool need = (mx - m_used) > 8.f;
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = fmaxf(m_used, mx);
        const float alpha = exp2f(m_used - m_new);
        if (t > 0) {
          // O of all previous tiles must be complete before it is rescaled: wait for P·V of tile t−1
          if (!mbar_wait(o_done, (t - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; continue; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 2; ++c) {                          // this group's 64 columns of O
            uint32_t rr[32];
            tmem_ld_32x32(T_O + wg * 64 + c * 32 + lane_off, rr);
            tmem_ld_wait();
            uint32_t w0[16], w1[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              w0[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
              w1[e] = __float_as_uint(__uint_as_float(rr[16 + e]) * alpha);
            }
            tmem_st_32x16(T_O + wg * 64 + c * 32 + lane_off, w0);
            tmem_st_32x16(T_O + wg * 64 + c * 32 + 16 + lane_off, w1);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      if (!mbar_wait(&p_empty[buf], bph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) { ok = false; continue; }
      tc_fence_after();
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float x0 = fmaf(s[c * 32 + 2 * e], sl2, -m_used), x1 = fmaf(s[c * 32 + 2 * e + 1], sl2, -m_used);
          // every fourth pair on the FMA pipe, the rest on MUFU: the two pipes finish a tile at about the same time
          const float p0 = (e & 3) == 3 ? exp2_fma(x0) : exp2f(x0);
          const float p1 = (e & 3) == 3 ? exp2_fma(x1) : exp2f(x1);
          rs4[e & 3] += p0 + p1;
          w[e] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(T_P0 + buf * 64 + wg * 32 + c * 16 + lane_off, w);
      }
      tmem_st_wait();
      l_sum += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&p_full[buf]);
    }
    // epilogue: the row sum is the sum of the two halves; each group normalises and stores its 64 columns of O
    xsum[wg * A2_BM + row_in_tile] = l_sum;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!ok) goto done;
    l_sum += xsum[(wg ^ 1) * A2_BM + row_in_tile];
    if (!mbar_wait(o_done, (n_tiles - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
    tc_fence_after();
    const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
    __nv_bfloat16* orow = p.out + ((static_cast<size_t>(b) * p.T + r) * p.H + h) * A2_D + wg * 64;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t rr[32];
      tmem_ld_32x32(T_O + wg * 64 + c * 32 + lane_off, rr);
      tmem_ld_wait();
      if (row_valid) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(rr[e]) * inv_l, __uint_as_float(rr[e + 1]) * inv_l);
          o.y = pack_bf16x2(__uint_as_float(rr[e + 2]) * inv_l, __uint_as_float(rr[e + 3]) * inv_l);
          o.z = pack_bf16x2(__uint_as_float(rr[e + 4]) * inv_l, __uint_as_float(rr[e + 5]) * inv_l);
          o.w = pack_bf16x2(__uint_as_float(rr[e + 6]) * inv_l, __uint_as_float(rr[e + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + c * 32 + e) = o;
        }
      }
    }
    if (row_valid && wg == 0)
      p.lse[(static_cast<size_t>(b) * p.H + h) * p.T + r] = l_sum > 0.f ? (m_used + log2f(l_sum)) * kLn2_2 : -INFINITY;
  }

done:
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // neither CTA signals into the shared memory of one that has exited
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer);

}  // namespace b200

// Same contract as b200_attn_fwd, head_dim 128 only (returns -1 otherwise).
extern "C" int b200_attn_fwd_pair(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start,
                                  int B, int T, int H, int G, int D, int window_left, float scale, int* status,
                                  cudaStream_t stream) {
  using namespace b200;
  if (B <= 0 || T <= 0) return 0;
  if (D != A2_D || H % G) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap tq, tk, tv;
  const uint64_t hd = static_cast<uint64_t>(H) * D, gd = static_cast<uint64_t>(G) * D, bt = static_cast<uint64_t>(B) * T;
  int rc = make_tmap_2d_bf16(&tq, q, hd, bt, hd, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tk, k, gd, bt, gd, 64, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tv, v, gd, bt, gd, 64, 128);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM) != cudaSuccess) return -2;
    configured = true;
  }
  AttnFwd2Params p{static_cast<__nv_bfloat16*>(out), lse, row_start, B, T, H, G, window_left, scale * kLog2e2, status};
  const int n_qt = (T + A2_BM - 1) / A2_BM;
  dim3 grid(2 * ((n_qt + 1) / 2), H, B);
  attn_fwd_pair_kernel<<<grid, A2_THREADS, A2_SMEM, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
