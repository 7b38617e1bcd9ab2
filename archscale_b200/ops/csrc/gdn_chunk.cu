// Chunked gated delta rule: the sequential part, on tcgen05.
//
// In the chunk (WY) form of the gated delta rule everything is a batched matmul over independent chunks of 64 tokens
// except one recurrence over the chunks of a sequence.  With the state kept transposed, X = Sᵀ ∈ R^{Dv×Dk}, one
// step of that recurrence for chunk n reads
//
//     P  = X · Aᵀ                      A  ∈ R^{64×Dk}
//     V  = C + sgn_p · Pᵀ              C, V ∈ R^{64×Dv}
//     X ← a_n · X + sgn_v · Vᵀ · Bm  (+ Eᵀ · F)     Bm, F ∈ R^{64×Dk},  E ∈ R^{64×Dv}
//
// and emits V and the state X that the chunk saw.  The forward pass is this with A = W, C = U, Bm = K·decay,
// sgn_p = −1, sgn_v = +1 (V = the corrected values, X = S at the chunk start); the backward pass is the same
// kernel run over the chunks in reverse with A = K·decay, C = QKᵀ·dO, Bm = W, sgn_p = +1, sgn_v = −1 and the extra
// term E = dO, F = Q·decay (V = dV, X = the gradient of the state at the chunk end).
//
// The value columns of the state are independent, so a CTA owns 128 of them for one (batch, head): X lives in
// tensor memory as a 128-lane × Dk fp32 accumulator for the whole sequence, a bf16 copy of it sits beside it as
// the A operand of P = X·Aᵀ (tcgen05.mma with A from tensor memory), and the four epilogue warps (one TMEM lane
// quarter each, thread = value column) turn P into V, rescale X by the next chunk's decay and emit both.
// A / Bm / E / F tiles arrive by TMA into 128-byte-swizzled shared memory; C and V move with plain loads / stores
// (64 bytes per warp and token).  Every wait is bounded.
#include "sm100.cuh"
#include "api.h"

namespace b200 {

int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer);

constexpr int GC = 64;             // chunk length (tokens)
constexpr int GDV = 128;           // value columns per CTA = TMEM lanes
constexpr int GDN_THREADS = 192;   // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int GCH = GC * 64 * 2;   // one [64 tokens × 64 columns] bf16 shared-memory chunk

struct GdnParams {
  const __nv_bfloat16* c_add;   // [BH, Tp, DV]
  const float* decay;           // [BH, nC]   a_n = exp(sum of the chunk's log-decays)
  __nv_bfloat16* v_out;         // [BH, Tp, DV]
  __nv_bfloat16* x_all;         // [BH, nC, DV, DK]   state seen by each chunk
  float* x_final;               // [BH, DV, DK] state after the last processed chunk, or null
  int BH, Tp, DV, nC;
  float sgn_p, sgn_v;
  int reverse;
  int* status;
};

template <int DK, int EXTRA>
struct GdnSmem {
  static constexpr int KC = DK / 64;
  static constexpr int AB_STAGE = 2 * KC * GCH;               // A then Bm
  static constexpr int EF = EXTRA ? (2 + KC) * GCH : 0;       // E (2 chunks of 64 value columns) then F
  static constexpr int VB = GDV * 128;                        // sgn_v·Vᵀ as a K-major A operand: 128 rows × 64 tokens
  static constexpr int TOTAL = 2 * AB_STAGE + EF + VB + 1024 + 256;
};

template <int DK, int EXTRA>
__global__ void __launch_bounds__(GDN_THREADS, 1)
gdn_state_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_bm,
                 const __grid_constant__ CUtensorMap tmap_e, const __grid_constant__ CUtensorMap tmap_f, const GdnParams p) {
  using SM = GdnSmem<DK, EXTRA>;
  constexpr int KC = SM::KC;
  constexpr uint32_t NCOLS = DK == 256 ? 512 : 256;           // X (DK) + bf16 X (DK/2) + P (64), rounded to a power of two
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* sef = smem + 2 * SM::AB_STAGE;
  uint8_t* svb = sef + SM::EF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(svb + SM::VB);
  uint64_t* ab_full = bars;        // [2]
  uint64_t* ab_empty = bars + 2;   // [2]
  uint64_t* ef_full = bars + 4;
  uint64_t* ef_empty = bars + 5;
  uint64_t* bar_p = bars + 6;      // P of this step is in tensor memory
  uint64_t* bar_v = bars + 7;      // (count 4) sgn_v·Vᵀ is in shared memory, P has been read
  uint64_t* bar_x = bars + 8;      // the state update of this step has completed
  uint64_t* bar_xb = bars + 9;     // (count 4) bf16 X written, fp32 X rescaled for the next step
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dvb = blockIdx.x, bh = blockIdx.y;
  const int nC = p.nC;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&ab_full[s], 1); mbar_init(&ab_empty[s], 1); }
    mbar_init(ef_full, 1); mbar_init(ef_empty, 1);
    mbar_init(bar_p, 1); mbar_init(bar_v, 4); mbar_init(bar_x, 1); mbar_init(bar_xb, 4);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_ptr, NCOLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const uint32_t T_X = tmem_base, T_XB = tmem_base + DK, T_P = tmem_base + DK + DK / 2;

  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < nC; ++s) {
        const int n = p.reverse ? nC - 1 - s : s;
        const int st = s & 1; const uint32_t ph = (s >> 1) & 1;
        const int row = bh * p.Tp + n * GC;
        if (!mbar_wait(&ab_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
        uint8_t* sa = ring + st * SM::AB_STAGE;
        mbar_arrive_expect_tx(&ab_full[st], SM::AB_STAGE);
#pragma unroll
        for (int c = 0; c < KC; ++c) {
          tma_load_2d(sa + c * GCH, &tmap_a, &ab_full[st], c * 64, row);
          tma_load_2d(sa + (KC + c) * GCH, &tmap_bm, &ab_full[st], c * 64, row);
        }
        if (EXTRA) {
          if (!mbar_wait(ef_empty, (s & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
          mbar_arrive_expect_tx(ef_full, SM::EF);
#pragma unroll
          for (int c = 0; c < 2; ++c) tma_load_2d(sef + c * GCH, &tmap_e, ef_full, dvb * GDV + c * 64, row);
#pragma unroll
          for (int c = 0; c < KC; ++c) tma_load_2d(sef + (2 + c) * GCH, &tmap_f, ef_full, c * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_p = make_idesc_bf16(GDV, GC, 0, 0);    // P = X(bf16, TMEM) · Aᵀ, A K-major
      constexpr uint32_t idesc_x = make_idesc_bf16(GDV, DK, 0, 1);    // X += (sgn_v·Vᵀ) · Bm, Bm N-major
      constexpr uint32_t idesc_e = make_idesc_bf16(GDV, DK, 1, 1);    // X += Eᵀ · F, both MN-major
      const uint32_t svba = smem_u32(svb), sefa = smem_u32(sef);
      for (int s = 0; s < nC; ++s) {
        const int st = s & 1; const uint32_t ph = (s >> 1) & 1;
        if (!mbar_wait(&ab_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
        if (!mbar_wait(bar_xb, s & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t sa = smem_u32(ring + st * SM::AB_STAGE), sbm = sa + KC * GCH;
#pragma unroll
        for (int k = 0; k < DK / 16; ++k)
          umma_bf16_ts(T_P, T_XB + 8 * k, make_smem_desc(sa + (k / 4) * GCH + (k % 4) * 32, 16, 1024), idesc_p, k != 0);
        umma_commit(bar_p);
        if (EXTRA) {
          if (!mbar_wait(ef_full, s & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < GC / 16; ++k)
            umma_bf16(T_X, make_smem_desc(sefa + k * 2048, GCH, 1024), make_smem_desc(sefa + 2 * GCH + k * 2048, GCH, 1024),
                      idesc_e, 1u);
          umma_commit(ef_empty);
        }
        if (!mbar_wait(bar_v, s & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < GC / 16; ++k)
          umma_bf16(T_X, make_smem_desc(svba + k * 32, 16, 1024), make_smem_desc(sbm + k * 2048, GCH, 1024), idesc_x, 1u);
        umma_commit(bar_x);
        umma_commit(&ab_empty[st]);
      }
    }
  } else {
    const int q = warp & 3;                              // TMEM lane quarter of this warp
    const int row = q * 32 + lane;                       // value column inside the CTA's block
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const size_t dvcol = static_cast<size_t>(dvb) * GDV + row;
    const int n_first = p.reverse ? nC - 1 : 0;
    {   // zero state: fp32 X, bf16 X, and the state seen by the first chunk
      uint32_t z[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) z[e] = 0u;
#pragma unroll
      for (int c = 0; c < (DK + DK / 2) / 16; ++c) tmem_st_32x16(T_X + c * 16 + lane_off, z);
      uint4* xr = reinterpret_cast<uint4*>(p.x_all + ((static_cast<size_t>(bh) * nC + n_first) * p.DV + dvcol) * DK);
#pragma unroll
      for (int e = 0; e < DK / 8; ++e) xr[e] = make_uint4(0u, 0u, 0u, 0u);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_xb);
    }
    for (int s = 0; s < nC; ++s) {
      const int n = p.reverse ? nC - 1 - s : s;
      const size_t tok0 = static_cast<size_t>(bh) * p.Tp + static_cast<size_t>(n) * GC;
      const unsigned short* crow = reinterpret_cast<const unsigned short*>(p.c_add) + tok0 * p.DV + dvcol;
      unsigned short* vrow = reinterpret_cast<unsigned short*>(p.v_out) + tok0 * p.DV + dvcol;
      unsigned short cv[GC];
#pragma unroll
      for (int i = 0; i < GC; ++i) cv[i] = __ldg(crow + static_cast<size_t>(i) * p.DV);
      if (!mbar_wait(bar_p, s & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t pr[32];
        tmem_ld_32x32(T_P + hh * 32 + lane_off, pr);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int i = hh * 32 + 2 * e;
          const float v0 = __bfloat162float(__ushort_as_bfloat16(cv[i])) + p.sgn_p * __uint_as_float(pr[2 * e]);
          const float v1 = __bfloat162float(__ushort_as_bfloat16(cv[i + 1])) + p.sgn_p * __uint_as_float(pr[2 * e + 1]);
          const __nv_bfloat16 b0 = __float2bfloat16_rn(v0), b1 = __float2bfloat16_rn(v1);
          vrow[static_cast<size_t>(i) * p.DV] = __bfloat16_as_ushort(b0);
          vrow[static_cast<size_t>(i + 1) * p.DV] = __bfloat16_as_ushort(b1);
          w[e] = pack_bf16x2(p.sgn_v * __bfloat162float(b0), p.sgn_v * __bfloat162float(b1));
        }
        // row `row` of the K-major operand: 16-byte piece j (8 tokens) sits at slot j ^ (row % 8) of the 128-byte row
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = hh * 4 + jj;
          *reinterpret_cast<uint4*>(svb + row * 128 + ((j ^ (row & 7)) << 4)) =
              make_uint4(w[4 * jj], w[4 * jj + 1], w[4 * jj + 2], w[4 * jj + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_v);

      if (!mbar_wait(bar_x, s & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const bool last = s == nC - 1;
      const int nn = p.reverse ? n - 1 : n + 1;            // the chunk that sees the state just formed
      const float a_next = last ? 1.f : p.decay[static_cast<size_t>(bh) * nC + nn];
      uint4* xr = last ? nullptr
                       : reinterpret_cast<uint4*>(p.x_all + ((static_cast<size_t>(bh) * nC + nn) * p.DV + dvcol) * DK);
      float* xf = (last && p.x_final) ? p.x_final + (static_cast<size_t>(bh) * p.DV + dvcol) * DK : nullptr;
#pragma unroll 2
      for (int c = 0; c < DK / 32; ++c) {
        uint32_t xv[32];
        tmem_ld_32x32(T_X + c * 32 + lane_off, xv);
        tmem_ld_wait();
        if (!last) {
          uint32_t xb[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) xb[e] = pack_bf16x2(__uint_as_float(xv[2 * e]), __uint_as_float(xv[2 * e + 1]));
          tmem_st_32x16(T_XB + c * 16 + lane_off, xb);
#pragma unroll
          for (int e = 0; e < 4; ++e) xr[c * 4 + e] = make_uint4(xb[4 * e], xb[4 * e + 1], xb[4 * e + 2], xb[4 * e + 3]);
          uint32_t lo[16], hi[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            lo[e] = __float_as_uint(__uint_as_float(xv[e]) * a_next);
            hi[e] = __float_as_uint(__uint_as_float(xv[16 + e]) * a_next);
          }
          tmem_st_32x16(T_X + c * 32 + lane_off, lo);
          tmem_st_32x16(T_X + c * 32 + 16 + lane_off, hi);
        } else if (xf) {
#pragma unroll
          for (int e = 0; e < 8; ++e)
            reinterpret_cast<float4*>(xf + c * 32)[e] = make_float4(__uint_as_float(xv[4 * e]), __uint_as_float(xv[4 * e + 1]),
                                                                    __uint_as_float(xv[4 * e + 2]), __uint_as_float(xv[4 * e + 3]));
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_xb);
    }
  }

done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, NCOLS);
  }
}

template <int DK, int EXTRA>
static int launch_gdn(const CUtensorMap& ta, const CUtensorMap& tbm, const CUtensorMap& te, const CUtensorMap& tf,
                      const GdnParams& p, cudaStream_t st) {
  auto k = gdn_state_kernel<DK, EXTRA>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GdnSmem<DK, EXTRA>::TOTAL) != cudaSuccess) return -2;
    configured = true;
  }
  k<<<dim3(p.DV / GDV, p.BH), GDN_THREADS, GdnSmem<DK, EXTRA>::TOTAL, st>>>(ta, tbm, te, tf, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

// One pass of the chunk recurrence (see the top of this file).  a_op, bm_op, f_op: [BH, Tp, DK] bf16; c_add, e_op,
// v_out: [BH, Tp, DV] bf16; decay: [BH, Tp/64] fp32; x_all: [BH, Tp/64, DV, DK] bf16; x_final: [BH, DV, DK] fp32 or
// null.  e_op / f_op null → no extra term.  DK ∈ {128, 256}, DV a multiple of 128, Tp a multiple of 64.
extern "C" int b200_gdn_state(const void* a_op, const void* c_add, const void* bm_op, const void* e_op, const void* f_op,
                              const float* decay, void* v_out, void* x_all, float* x_final, int BH, int Tp, int DK, int DV,
                              float sgn_p, float sgn_v, int reverse, int* status, cudaStream_t stream) {
  using namespace b200;
  if (BH <= 0 || Tp <= 0) return 0;
  if ((DK != 128 && DK != 256) || DV % GDV || Tp % GC || ((e_op == nullptr) != (f_op == nullptr))) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  const uint64_t rows = static_cast<uint64_t>(BH) * Tp;
  CUtensorMap ta, tbm, te, tf;
  int rc = make_tmap_2d_bf16(&ta, a_op, DK, rows, DK, 64, GC);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tbm, bm_op, DK, rows, DK, 64, GC);
  if (rc) return rc;
  const bool extra = e_op != nullptr;
  rc = make_tmap_2d_bf16(&te, extra ? e_op : c_add, DV, rows, DV, 64, GC);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tf, extra ? f_op : a_op, DK, rows, DK, 64, GC);
  if (rc) return rc;
  GdnParams p{(const __nv_bfloat16*)c_add, decay, (__nv_bfloat16*)v_out, (__nv_bfloat16*)x_all, x_final,
              BH, Tp, DV, Tp / GC, sgn_p, sgn_v, reverse, status};
  if (DK == 256) return extra ? launch_gdn<256, 1>(ta, tbm, te, tf, p, stream) : launch_gdn<256, 0>(ta, tbm, te, tf, p, stream);
  return extra ? launch_gdn<128, 1>(ta, tbm, te, tf, p, stream) : launch_gdn<128, 0>(ta, tbm, te, tf, p, stream);
}
