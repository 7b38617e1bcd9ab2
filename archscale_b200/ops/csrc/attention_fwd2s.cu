// Causal / sliding-window / packed-varlen attention forward on tcgen05 (GQA, head_dim 64 or 128).
//
// One CTA per (query tile of 128 rows, head, batch) runs TWO independent online-softmax streams over the key tiles:
// stream 0 takes the even tiles, stream 1 the odd ones, each with its own score buffer, running max / sum and output
// accumulator in tensor memory; the two partial results are merged at the end (the split-KV identity).  Measured on the
// one-stream predecessor: tensor pipe 41 % busy, MUFU 38 %, issue slots 30 % — no unit saturated, the time went into the
// serial chain  S ready → load → max → exp2 → pack → store → P·V  of a single warp per scheduler.  Splitting the columns
// of a tile over two warp groups did not help either (both groups sit in the same phase at the same time and queue up
// for MUFU together).  Two streams are out of phase by construction: while one group is in its exp2 phase the other
// waits for its S, loads or reduces, and the tensor pipe always has the other stream's MMAs to run.
//
// 384 threads in three warp groups, registers re-balanced with setmaxnreg (56 / 224 / 224 per thread):
//   warps 0..3    warp 0 TMA (Q once, then K/V tiles of 128 keys; stage s of the 2-stage ring belongs to stream s);
//                 warp 1 / warp 2 the MMA thread of stream 0 / 1:  S = Q·Kᵀ into the stream's 128 score columns, then (once
//                 the softmax group has written P) O_w += P·V with P read from tensor memory as the A operand.  P overwrites
//                 S in place; the next S of the stream is issued by the same thread after that P·V, and MMAs of one thread
//                 execute in issue order, so the overwrite needs no extra barrier.
//   warps 4..7    softmax group of stream 0, warps 8..11 of stream 1: thread t owns query row t.  All 128 scores of the row
//                 are loaded with four tcgen05.ld in flight and one wait (a tensor-memory load returns after ≈500 cycles:
//                 a chunked two-pass variant with eight dependent loads per tile ran at half the speed).  Base-2 online
//                 softmax with lazy rescaling of O_w (only when the max grew by more than 2^8); a quarter of the
//                 exponentials runs on the FMA pipe (Cody–Waite split + cubic) instead of MUFU.
// Epilogue: the groups exchange (max, sum) per row through shared memory, each group merges and stores half of the
// head-dim columns, reading both accumulators from tensor memory.
//
// Masking is one rule for all modes: query row r sees keys k with lo(r) ≤ k ≤ r, where
// lo(r) = max(row_start[r], r − window_left); row_start comes from cu_seqlens for packed documents.
// KV tiles entirely outside [lo(first row), last row] are skipped.
//
// TMEM columns: S0/P0 0..127 | S1/P1 128..255 | O0 256..256+D | O1 384..384+D.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int A2_BM = 128, A2_BN = 128;
constexpr int A2_THREADS = 384;          // three warp groups: producers / MMA issuers, softmax stream 0, softmax stream 1
constexpr float kLog2e_2 = 1.4426950408889634f, kLn2_2 = 0.6931471805599453f;

struct AttnFwd2Params {
  __nv_bfloat16* out;      // [B, T, H, D]
  float* lse;              // [B, H, T]
  const int* row_start;    // [B*T] first visible key of each row (batch-local) or null
  int B, T, H, G;
  int window_left;         // < 0: unlimited
  float scale_log2;        // softmax scale · log2(e)
  int* status;
  long long* trace;        // optional [16][64] clock64 stamps of the first CTA (null in normal use)
};

// Timeline probe: row (stream·8 + event), column = tile index inside the stream; only CTA (0,0,0) and one thread per role.
#define A2_TRACE(w, ev, i) do { if (p.trace && traced && (i) < 64) p.trace[((w) * 8 + (ev)) * 64 + (i)] = clock64(); } while (0)

template <int D>
struct Attn2Smem {
  static constexpr int Q_BYTES = A2_BM * D * 2;
  static constexpr int KV_BYTES = A2_BN * D * 2;
  static constexpr int STAGES = 2;
  static constexpr int XCHG_BYTES = 4 * A2_BM * 4;         // (max, sum) × 2 streams × 128 rows
  static constexpr int TOTAL = Q_BYTES + STAGES * 2 * KV_BYTES + 1024 + 256 + XCHG_BYTES;
};

// 2^x on the FMA pipe: floor by a round-down add of 1.5·2^23, cubic for the fraction (max relative error 8.6e-5, below
// bf16 resolution), exponent added into the float's bit pattern.  x is clamped at −126, so a masked score (−inf) gives 2^−126.
__device__ __forceinline__ float exp2_fma2(float x) {
  x = fmaxf(x, -126.f);
  float xr;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(xr) : "f"(x), "f"(12582912.f));
  const float f = x - (xr - 12582912.f);
  const float pl = fmaf(fmaf(fmaf(0.07706617563962936f, f, 0.22764593362808228f), f, 0.6951165795326233f), f, 1.f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(xr) << 23));
}

template <int D>
__global__ void __launch_bounds__(A2_THREADS, 1)
attn_fwd_2s_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnFwd2Params p) {
  using SM = Attn2Smem<D>;
  constexpr int DC = D / 64;                       // 64-element chunks of the head dim (TMA boxes)
  constexpr int CHUNK_BYTES = 128 * 64 * 2;        // one box: 128 rows × 64 elements
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  uint8_t* skv = smem + SM::Q_BYTES;               // stage s (= stream s): K at skv + s·2·KV, V right after K
  uint64_t* bars = reinterpret_cast<uint64_t*>(skv + SM::STAGES * 2 * SM::KV_BYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* v_full = bars + 3;        // [2]
  uint64_t* k_empty = bars + 5;       // [2]  K stage free: S of its tile has completed
  uint64_t* v_empty = bars + 7;       // [2]  V stage free: P·V of its tile has completed
  uint64_t* s_full = bars + 9;        // [2]
  uint64_t* p_full = bars + 11;       // [2]  (count 4) P of the stream's current tile is in tensor memory
  uint64_t* o_done = bars + 13;       // [2]  P·V of the stream's current tile has completed
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  float* xchg = reinterpret_cast<float*>(bars + 16);      // [stream][max | sum][row]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: better tail behaviour under causal masking
  const int n_qt = (p.T + A2_BM - 1) / A2_BM;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int q0 = qt * A2_BM;
  const int r_last = min(q0 + A2_BM, p.T) - 1;
  auto lo_of = [&](int r) {
    int lo = p.row_start ? p.row_start[static_cast<size_t>(b) * p.T + r] : 0;
    if (p.window_left >= 0) lo = max(lo, r - p.window_left);
    return lo;
  };
  const int lo_first = lo_of(q0);
  const int j_begin = lo_first / A2_BN;
  const int j_end = r_last / A2_BN + 1;          // exclusive
  const int n_tiles = j_end - j_begin;            // ≥ 1; stream w takes tiles w, w+2, …
  const bool traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (warp < 3 || (warp & 3) == 0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4); mbar_init(&o_done[s], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DC; ++c) tma_load_2d(sq + c * CHUNK_BYTES, &tmap_q, q_full, h * D + c * 64, b * p.T + q0);
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1; const uint32_t ph = (t >> 1) & 1;
        // K and V of a stage are released separately: K of tile t+2 lands while tile t is still in its softmax
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        uint8_t* sk = skv + st * 2 * SM::KV_BYTES;
        uint8_t* sv = sk + SM::KV_BYTES;
        const int k0 = (j_begin + t) * A2_BN;
        mbar_arrive_expect_tx(&k_full[st], SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_2d(sk + c * CHUNK_BYTES, &tmap_k, &k_full[st], g * D + c * 64, b * p.T + k0);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        mbar_arrive_expect_tx(&v_full[st], SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_2d(sv + c * CHUNK_BYTES, &tmap_v, &v_full[st], g * D + c * 64, b * p.T + k0);
      }
    }
  } else if (warp == 1 || warp == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (lane == 0) {
      const int w = warp - 1;
      constexpr uint32_t idesc_s = make_idesc_bf16(A2_BM, A2_BN, 0, 0);       // S = Q·Kᵀ  (both K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(A2_BM, D, 0, 1);            // O += P·V  (V is N-major)
      const uint32_t T_S = tmem_base + w * 128, T_O = tmem_base + 256 + w * 128;
      const uint32_t sk = smem_u32(skv + w * 2 * SM::KV_BYTES), sv = sk + SM::KV_BYTES;
      const uint32_t sqa = smem_u32(sq);
      if (!mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      int i = 0;
      for (int t = w; t < n_tiles; t += 2, ++i) {
        const uint32_t ph = i & 1;
        A2_TRACE(w, 4, i);
        if (!mbar_wait(&k_full[w], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
        tc_fence_after();
        // the stream's previous P·V (which read P from these columns) was issued by this thread: it executes first
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * CHUNK_BYTES + (k % 4) * 32;
          umma_bf16(T_S, make_smem_desc(sqa + off, 16, 1024), make_smem_desc(sk + off, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[w]);
        umma_commit(&k_empty[w]);
        A2_TRACE(w, 5, i);
        if (!mbar_wait(&v_full[w], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
        if (!mbar_wait(&p_full[w], ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        tc_fence_after();
        A2_TRACE(w, 6, i);
#pragma unroll
        for (int k = 0; k < A2_BN / 16; ++k) {
          // A: P columns (two bf16 per 32-bit column → 8 columns per K=16); B: 16 key rows = 2048 bytes further
          umma_bf16_ts(T_O, T_S + k * 8, make_smem_desc(sv + k * 2048, CHUNK_BYTES, 1024), idesc_o, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[w]);
        umma_commit(&o_done[w]);
        A2_TRACE(w, 7, i);
      }
    }
  } else if (warp == 3) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");     // every warp of the group has to give its registers back
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int w = (warp - 4) >> 2;                    // stream of this softmax group
    const int qtr = warp & 3;                         // TMEM lane quarter this warp may access
    const int row_in_tile = qtr * 32 + lane;
    const int r = q0 + row_in_tile;
    const bool row_valid = r < p.T;
    const int lo_r = row_valid ? lo_of(r) : 0;
    const int lo_last = lo_of(r_last);
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const uint32_t T_S = tmem_base + w * 128 + lane_off, T_O = tmem_base + 256 + w * 128 + lane_off;
    const float sl2 = p.scale_log2;
    float m_used = -1e30f, l_sum = 0.f;
    // The two groups take turns in the exp2 phase (named barriers 2 and 3, one "token" passed back and forth): in step
    // they would queue up for MUFU together and then for the tensor pipe together; out of step one group's exponentials
    // run while the other stream's P·V and next S execute.  Order: stream 0 tile 0, stream 1 tile 0, stream 0 tile 1, …
    // Every thread runs every iteration and every barrier operation, also after a failed wait (ok == false).
    const int n0 = (n_tiles + 1) >> 1, n1 = n_tiles >> 1;
    bool ok = true;
    int i = 0;
    if (w == 1) asm volatile("bar.arrive 2, 256;" ::: "memory");       // stream 0 goes first
    for (int t = w; t < n_tiles; t += 2, ++i) {
      const uint32_t ph = i & 1;
      const int k0 = (j_begin + t) * A2_BN;
      float s[128];
      const bool full_tile = (k0 + A2_BN - 1 <= q0) && (k0 >= lo_last);
      A2_TRACE(w, 0, i);
      if (ok && !mbar_wait(&s_full[w], ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
      ok = __all_sync(0xffffffffu, ok);            // warp-uniform: the warp-wide vote and the barriers below need every lane
      if (ok) {
      tc_fence_after();
      A2_TRACE(w, 1, i);
      // this row's 128 raw scores: four loads in flight, one wait; the softmax scale is folded into the exponent below
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(T_S + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_ld_wait();
      if (!full_tile) {
#pragma unroll
        for (int e = 0; e < 128; ++e) {
          const int kk = k0 + e;
          if (kk > r || kk < lo_r) s[e] = -INFINITY;
        }
      }
      float mx8[8];                                  // eight independent chains instead of one of length 128
#pragma unroll
      for (int e = 0; e < 8; ++e) mx8[e] = s[e];
#pragma unroll
      for (int e = 8; e < 128; ++e) mx8[e & 7] = fmaxf(mx8[e & 7], s[e]);
      const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * sl2;
      A2_TRACE(w, 2, i);
      // lazy rescale: only when the running max grew by more than 8 (factor 256); decided per warp
      const bool need = (mx - m_used) > 8.f;
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = fmaxf(m_used, mx);
        const float alpha = exp2f(m_used - m_new);
        if (i > 0) {
          // O_w of all previous tiles must be complete before it is rescaled: wait for the stream's last P·V
          if (!mbar_wait(&o_done[w], (i - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
          ok = __all_sync(0xffffffffu, ok);
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[32];
            tmem_ld_32x32(T_O + c * 32, rr);
            tmem_ld_wait();
            uint32_t w0[16], w1[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              w0[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
              w1[e] = __float_as_uint(__uint_as_float(rr[16 + e]) * alpha);
            }
            tmem_st_32x16(T_O + c * 32, w0);
            tmem_st_32x16(T_O + c * 32 + 16, w1);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      }
      if (w == 0) asm volatile("bar.sync 2, 256;" ::: "memory"); else asm volatile("bar.sync 3, 256;" ::: "memory");
      // P = 2^(s·scale − m_used) as packed bf16 over the first 64 score columns (every score is in registers by now)
      if (ok) {
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t wv[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float x0 = fmaf(s[c * 32 + 2 * e], sl2, -m_used), x1 = fmaf(s[c * 32 + 2 * e + 1], sl2, -m_used);
            // every fourth pair on the FMA pipe, the rest on MUFU
            const float p0 = (e & 3) == 3 ? exp2_fma2(x0) : exp2f(x0);
            const float p1 = (e & 3) == 3 ? exp2_fma2(x1) : exp2f(x1);
            rs4[e & 3] += p0 + p1;
            wv[e] = pack_bf16x2(p0, p1);
          }
          tmem_st_32x16(T_S + c * 16, wv);
        }
        tmem_st_wait();
        l_sum += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      }
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&p_full[w]);
      A2_TRACE(w, 3, i);
      // pass the turn on if the other stream still has a tile after this one
      if (w == 0) { if (i < n1) asm volatile("bar.arrive 3, 256;" ::: "memory"); }
      else        { if (i + 1 < n0) asm volatile("bar.arrive 2, 256;" ::: "memory"); }
    }
    // ---- epilogue: merge the two streams.  n_w tiles went through stream w.
    xchg[(w * 2 + 0) * A2_BM + row_in_tile] = m_used;
    xchg[(w * 2 + 1) * A2_BM + row_in_tile] = l_sum;
    asm volatile("bar.sync 1, 256;" ::: "memory");      // every softmax thread arrives here, also after a failed wait
    if (!ok) goto done;
    {
      const float m0 = xchg[0 * A2_BM + row_in_tile], l0 = xchg[1 * A2_BM + row_in_tile];
      const float m1 = xchg[2 * A2_BM + row_in_tile], l1 = xchg[3 * A2_BM + row_in_tile];
      const float m = fmaxf(m0, m1);
      const float a0 = exp2f(m0 - m), a1 = n1 > 0 ? exp2f(m1 - m) : 0.f;
      const float l = l0 * a0 + l1 * a1;
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      if (n0 > 0 && !mbar_wait(&o_done[0], (n0 - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      if (n1 > 0 && !mbar_wait(&o_done[1], (n1 - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const float c0 = a0 * inv_l, c1 = a1 * inv_l;
      const uint32_t T_O0 = tmem_base + 256 + lane_off, T_O1 = tmem_base + 384 + lane_off;
      __nv_bfloat16* orow = p.out + ((static_cast<size_t>(b) * p.T + r) * p.H + h) * D;
      // group w stores head-dim columns [w·D/2, (w+1)·D/2)
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        const int col = w * (D / 2) + c * 32;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(T_O0 + col, r0);
        if (n1 > 0) tmem_ld_32x32(T_O1 + col, r1);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            float f[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              f[u] = __uint_as_float(r0[e + u]) * c0;
              if (n1 > 0) f[u] = fmaf(__uint_as_float(r1[e + u]), c1, f[u]);
            }
            uint4 o;
            o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
            o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(orow + col + e) = o;
          }
        }
      }
      if (row_valid && w == 0)
        p.lse[(static_cast<size_t>(b) * p.H + h) * p.T + r] = l > 0.f ? (m + log2f(l)) * kLn2_2 : -INFINITY;
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

int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer);

template <int D>
static int launch_attn_fwd_2s(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwd2Params& p,
                           cudaStream_t st) {
  auto kern = attn_fwd_2s_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Attn2Smem<D>::TOTAL) != cudaSuccess) return -2;
    configured = true;
  }
  dim3 grid((p.T + A2_BM - 1) / A2_BM, p.H, p.B);
  kern<<<grid, A2_THREADS, Attn2Smem<D>::TOTAL, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

// Timeline probe of the forward kernel (development aid): pass a device buffer of 16·64 int64 to record clock64 stamps of
// the first CTA of every following launch, or null to switch it off.
static long long* g_attn2_trace = nullptr;
extern "C" void b200_attn_fwd_2s_set_trace(long long* buf) { g_attn2_trace = buf; }

extern "C" int b200_attn_fwd_2s(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start,
                             int B, int T, int H, int G, int D, int window_left, float scale, int* status,
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
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d_bf16(&tq, q, static_cast<uint64_t>(H) * D, static_cast<uint64_t>(B) * T, static_cast<uint64_t>(H) * D, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tk, k, static_cast<uint64_t>(G) * D, static_cast<uint64_t>(B) * T, static_cast<uint64_t>(G) * D, 64, 128);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tv, v, static_cast<uint64_t>(G) * D, static_cast<uint64_t>(B) * T, static_cast<uint64_t>(G) * D, 64, 128);
  if (rc) return rc;
  AttnFwd2Params p{static_cast<__nv_bfloat16*>(out), lse, row_start, B, T, H, G, window_left, scale * kLog2e_2, status, g_attn2_trace};
  return D == 128 ? launch_attn_fwd_2s<128>(tq, tk, tv, p, stream) : launch_attn_fwd_2s<64>(tq, tk, tv, p, stream);
}
