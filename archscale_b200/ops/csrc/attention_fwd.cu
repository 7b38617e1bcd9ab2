// Causal / sliding-window / packed-varlen attention forward on tcgen05 (GQA, head_dim 64 or 128).
//
// One CTA per (query tile of 128 rows, head, batch); 224 threads:
//   warp 0      TMA: Q once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 1      MMA: S_j = Q·K_jᵀ into one of two 128-column TMEM buffers
//   warp 6      MMA: O += P_j·V_j with P_j (bf16) read from TMEM as the A operand and V_j from shared memory (N-major)
//   warps 2..5  softmax: thread t owns query row t — tcgen05.ld its 128 scores, online softmax in
//               base 2 with lazy rescaling of O (only when the running max grew by more than 2^8),
//               write P_j to TMEM (packed bf16), finally normalise O and store it with the LSE
// S_{j+1} is issued before the softmax of S_j finishes, so tensor cores and MUFU overlap.
//
// Masking is one rule for all modes: query row r sees keys k with lo(r) ≤ k ≤ r, where
// lo(r) = max(row_start[r], r − window_left); row_start comes from cu_seqlens for packed documents.
// KV tiles entirely outside [lo(first row), last row] are skipped.
//
// TMEM columns: S0 0..127 | S1 128..255 | P0 256..319 | P1 320..383 | O 384..511.
#include <stdlib.h>
#include <string.h>
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int ATT_BM = 128, ATT_BN = 128;
constexpr int ATT_THREADS = 224;          // warp 0 TMA, warp 1 MMA (S), warps 2..5 softmax, warp 6 MMA (P·V)
constexpr int ATT_PV_WARP = 6;
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

struct AttnFwdParams {
  __nv_bfloat16* out;      // [B, T, H, D]
  float* lse;              // [B, H, T]
  const int* row_start;    // [B*T] first visible key of each row (batch-local) or null
  int B, T, H, G;
  int window_left;         // < 0: unlimited
  float scale_log2;        // softmax scale · log2(e)
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int Q_BYTES = ATT_BM * D * 2;
  static constexpr int KV_BYTES = ATT_BN * D * 2;
  static constexpr int STAGES = 2;
  static constexpr int TOTAL = Q_BYTES + STAGES * 2 * KV_BYTES + 1024 + 256;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnFwdParams p) {
  using SM = AttnSmem<D>;
  constexpr int DC = D / 64;                       // 64-element chunks of the head dim (TMA boxes)
  constexpr int CHUNK_BYTES = 128 * 64 * 2;        // one box: 128 rows × 64 elements
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sq = smem;
  uint8_t* skv = smem + SM::Q_BYTES;               // stage s: K at skv + s·2·KV, V right after K
  uint64_t* bars = reinterpret_cast<uint64_t*>(skv + SM::STAGES * 2 * SM::KV_BYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* v_full = bars + 3;        // [2]
  uint64_t* k_empty = bars + 5;       // [2]  K stage free: S of its tile has completed
  uint64_t* s_full = bars + 7;        // [2]
  uint64_t* s_empty = bars + 9;       // [2]
  uint64_t* p_full = bars + 11;       // [2]
  uint64_t* p_empty = bars + 13;      // [2]
  uint64_t* o_done = bars + 15;       // 1
  uint64_t* v_empty = bars + 16;      // [2]  V stage free: P·V of its tile has completed
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: better tail behaviour under causal masking
  const int n_qt = (p.T + ATT_BM - 1) / ATT_BM;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int q0 = qt * ATT_BM;
  const int r_last = min(q0 + ATT_BM, p.T) - 1;
  auto lo_of = [&](int r) {
    int lo = p.row_start ? p.row_start[static_cast<size_t>(b) * p.T + r] : 0;
    if (p.window_left >= 0) lo = max(lo, r - p.window_left);
    return lo;
  };
  const int lo_first = lo_of(q0);
  const int j_begin = lo_first / ATT_BN;
  const int j_end = r_last / ATT_BN + 1;          // exclusive
  const int n_tiles = j_end - j_begin;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 4); mbar_init(&p_full[s], 4); mbar_init(&p_empty[s], 1);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t T_S0 = tmem_base, T_P0 = tmem_base + 256, T_O = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DC; ++c) tma_load_2d(sq + c * CHUNK_BYTES, &tmap_q, q_full, h * D + c * 64, b * p.T + q0);
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1; const uint32_t ph = (t >> 1) & 1;
        // K and V stages are released separately: the K of tile t+2 can land while tile t is still in its softmax, so the
        // next S = Q·Kᵀ never waits for a load (with one barrier for both, K waited for P·V and the softmax warps for S)
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        uint8_t* sk = skv + st * 2 * SM::KV_BYTES;
        uint8_t* sv = sk + SM::KV_BYTES;
        const int k0 = (j_begin + t) * ATT_BN;
        mbar_arrive_expect_tx(&k_full[st], SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_2d(sk + c * CHUNK_BYTES, &tmap_k, &k_full[st], g * D + c * 64, b * p.T + k0);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        mbar_arrive_expect_tx(&v_full[st], SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_2d(sv + c * CHUNK_BYTES, &tmap_v, &v_full[st], g * D + c * 64, b * p.T + k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);       // S = Q·Kᵀ  (both K-major)
      if (!mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
      auto issue_s = [&](int t) -> bool {
        const int st = t & 1; const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(skv + st * 2 * SM::KV_BYTES);
        const uint32_t sqa = smem_u32(sq);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * CHUNK_BYTES + (k % 4) * 32;
          umma_bf16(T_S0 + st * 128, make_smem_desc(sqa + off, 16, 1024), make_smem_desc(sk + off, 16, 1024), idesc_s,
                    k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      // One thread can issue a tcgen05.mma only every ~100 cycles: S and P·V are issued by two threads (this one and warp
      // ATT_PV_WARP) so that neither stream waits behind the other's issue slots.  s_empty / p_empty order the buffer reuse.
      for (int t = 0; t < n_tiles; ++t)
        if (!issue_s(t)) goto done;
    }
  } else if (warp == ATT_PV_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_o = make_idesc_bf16(ATT_BM, D, 0, 1);            // O += P·V  (V is N-major)
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1; const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
        if (!mbar_wait(&p_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        tc_fence_after();
        const uint32_t sv = smem_u32(skv + st * 2 * SM::KV_BYTES + SM::KV_BYTES);
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          // A: P columns (two bf16 per 32-bit column → 8 columns per K=16); B: 16 key rows = 2048 bytes further
          umma_bf16_ts(T_O, T_P0 + st * 64 + k * 8, make_smem_desc(sv + k * 2048, CHUNK_BYTES, 1024), idesc_o,
                       (t | k) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(&p_empty[st]);
        umma_commit(o_done);
      }
    }
  } else {
    const int qtr = warp & 3;
    const int row_in_tile = qtr * 32 + lane;
    const int r = q0 + row_in_tile;
    const bool row_valid = r < p.T;
    const int lo_r = row_valid ? lo_of(r) : 0;
    const int lo_last = lo_of(r_last);
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    float m_used = -1e30f, l_sum = 0.f;
    for (int t = 0; t < n_tiles; ++t) {
      const int st = t & 1; const uint32_t ph = (t >> 1) & 1;
      const int k0 = (j_begin + t) * ATT_BN;
      if (!mbar_wait(&s_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      // this row's 128 raw scores: four loads in flight, one wait; the softmax scale is folded into the exponent below
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld_32x32(T_S0 + st * 128 + c * 32 + lane_off, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[st]);     // S buffer may be overwritten by S_{t+2}
      const bool full_tile = (k0 + ATT_BN - 1 <= q0) && (k0 >= lo_last);
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
      const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) *
                       p.scale_log2;
      // lazy rescale: only when the running max grew by more than 8 (factor 256); decided per warp
      const bool need = (mx - m_used) > 8.f;
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = fmaxf(m_used, mx);
        const float alpha = exp2f(m_used - m_new);
        if (t > 0) {
          // O of all previous tiles must be complete before it is rescaled: wait for P·V of tile t−1
          if (!mbar_wait(o_done, (t - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[32];
            tmem_ld_32x32(T_O + c * 32 + lane_off, rr);
            tmem_ld_wait();
            uint32_t w0[16], w1[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              w0[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
              w1[e] = __float_as_uint(__uint_as_float(rr[16 + e]) * alpha);
            }
            tmem_st_32x16(T_O + c * 32 + lane_off, w0);
            tmem_st_32x16(T_O + c * 32 + 16 + lane_off, w1);
          }
          tmem_st_wait();
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      // P = 2^(s − m_used), packed to bf16 and written to TMEM; row sum in fp32
      if (!mbar_wait(&p_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
      tc_fence_after();
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      const float sl2 = p.scale_log2;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float p0 = exp2f(fmaf(s[c * 32 + 2 * e], sl2, -m_used)), p1 = exp2f(fmaf(s[c * 32 + 2 * e + 1], sl2, -m_used));
          rs4[e & 3] += p0 + p1;
          w[e] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(T_P0 + st * 64 + c * 16 + lane_off, w);
      }
      const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      tmem_st_wait();
      l_sum += rs;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[st]);
    }
    // epilogue: O / l, LSE
    if (n_tiles > 0) {
      if (!mbar_wait(o_done, (n_tiles - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
    }
    const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
    __nv_bfloat16* orow = p.out + ((static_cast<size_t>(b) * p.T + r) * p.H + h) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t rr[32];
      if (n_tiles > 0) { tmem_ld_32x32(T_O + c * 32 + lane_off, rr); tmem_ld_wait(); }
      else {
#pragma unroll
        for (int e = 0; e < 32; ++e) rr[e] = 0u;
      }
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
    if (row_valid) p.lse[(static_cast<size_t>(b) * p.H + h) * p.T + r] = l_sum > 0.f ? (m_used + log2f(l_sum)) * kLn2 : -INFINITY;
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
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwdParams& p,
                           cudaStream_t st) {
  auto kern = attn_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<D>::TOTAL) != cudaSuccess) return -2;
    configured = true;
  }
  dim3 grid((p.T + ATT_BM - 1) / ATT_BM, p.H, p.B);
  kern<<<grid, ATT_THREADS, AttnSmem<D>::TOTAL, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

extern "C" int b200_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start,
                             int B, int T, int H, int G, int D, int window_left, float scale, int* status,
                             cudaStream_t stream) {
  using namespace b200;
  if (B <= 0 || T <= 0) return 0;
  if ((D != 64 && D != 128) || H % G) return -1;
  static const bool two_stream = [] { const char* e = getenv("ARCHSCALE_B200_ATTN_FWD"); return e && !strcmp(e, "2stream"); }();
  if (two_stream) return b200_attn_fwd_2s(q, k, v, out, lse, row_start, B, T, H, G, D, window_left, scale, status, stream);
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
  AttnFwdParams p{static_cast<__nv_bfloat16*>(out), lse, row_start, B, T, H, G, window_left, scale * kLog2e, status};
  return D == 128 ? launch_attn_fwd<128>(tq, tk, tv, p, stream) : launch_attn_fwd<64>(tq, tk, tv, p, stream);
}
