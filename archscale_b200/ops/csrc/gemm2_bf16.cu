// bf16 GEMM with one 256×256 output tile per PAIR of SMs (tcgen05.mma.cta_group::2).
//
// A cluster of two CTAs (two SMs of one TPC) works on one tile: each CTA stages 128 rows of A and 128 of the 256 rows
// of B in its own shared memory (6-stage ring, 32 KB per stage and CTA) and one thread of the even ("leader") CTA
// issues M256 × N256 × K16 MMAs that read both CTAs' shared memory and write 128 accumulator rows × 256 fp32 columns
// into EACH CTA's tensor memory.  Against the one-CTA 128×256 tile this moves a third less operand data from L2
// per FLOP and halves the B traffic per SM, which is what bounds that kernel.
//
// Per CTA, 192 threads: warp 0 TMA producer (both CTAs; every load signals the leader's `full` barrier), warp 1
// allocates tensor memory (both CTAs) and issues the MMAs (leader only), warps 2..5 epilogue (each CTA stores its own
// 128 rows; two 256-column accumulators let the epilogue of tile i overlap the main loop of tile i+1).  tcgen05.commit
// arrives on the `empty` / `tmem_full` barriers of both CTAs; the epilogue warps of both CTAs arrive on the leader's
// `tmem_empty`.  No TMA load uses cluster multicast.  Every wait is bounded; the two CTAs leave together through a
// cluster barrier so that neither signals into shared memory of a CTA that has exited.
//
// Layouts as in gemm_bf16.cu: A K-major [M,K] or MN-major [K,M]; B K-major [N,K] or MN-major [K,N].
#include "sm100.cuh"
#include "api.h"

namespace b200 {

int make_tmap_2d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_inner, uint32_t box_outer);
int make_tmap_3d_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch,
                      uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_rows);

constexpr int T2_BM = 256, T2_BN = 256, T2_BK = 64, T2_STAGES = 6;
constexpr int T2_HALF = 128;                          // rows of A / rows of B held by one CTA
constexpr int T2_OP_BYTES = T2_HALF * T2_BK * 2;      // 16 KB
constexpr int T2_STAGE_BYTES = 2 * T2_OP_BYTES;       // A then B
constexpr int T2_SMEM_BYTES = T2_STAGES * T2_STAGE_BYTES + 1024 + 256;
constexpr int T2_GROUP_M = 8;
constexpr int T2_THREADS = 192;

// Grouped / batched problems (same conventions as the one-CTA kernel):
//   GROUPED 1  rows of A are grouped by expert (offsets[E+1], multiples of 256); expert e multiplies its rows with B_e
//   GROUPED 2  per-expert weight gradient: out[e] = A[seg_e]ᵀ · B[seg_e], the K range of expert e is its row segment
//   GROUPED 3  `E` independent problems of identical shape (3-D tensor maps, batch index = third coordinate)
struct Group2Params {
  const int* offsets;
  int E;
  int b_rows;           // rows of one expert's matrix inside B (GROUPED 1)
  const float* alpha_vec;   // GROUPED 3: optional per-problem factors multiplied into alpha / beta (device arrays of E floats)
  const float* beta_vec;
  int sym;              // GROUPED 3, square outputs known to be symmetric (X·Xᵀ, polynomials of a symmetric matrix): only the
                        // tiles on and above the diagonal are computed, an off-diagonal tile is also stored transposed
};

struct Gemm2Params {
  void* out;
  const void* cin;
  int M, N, K;
  int ldc;
  float alpha, beta;
  int accumulate;
  int* status;
  // serial split-K for accumulating fp32 output (see GemmParams in gemm_bf16.cu); 8 counters per tile (CTA rank × epilogue warp)
  int split_k;
  uint32_t* sem;
  // SwiGLU in the epilogue (NT products with bf16 output, plain or GROUPED 1).  B holds [gate rows | up rows] per (expert)
  // matrix, glu_half rows each.  A tile pairs 128 gate columns with the 128 up columns of the same index: the leader CTA
  // loads the gate rows as its half of the B operand and its peer the up rows, so that every epilogue thread finds
  // gate j in accumulator column j and up j in column 128 + j of its row.  out (may be null) receives the pre-activation
  // [M, 2·glu_half] as without the fusion, out2 [M, glu_half] (leading dimension ldc2) receives silu(gate)·up computed from
  // the bf16-rounded values, i.e. bit for bit what the separate SwiGLU kernel makes of `out`.
  int glu_half;
  void* out2;
  int ldc2;
};

extern uint32_t* g_splitk_sem;
extern int g_splitk_sem_len;
int choose_split_k(int tiles, int num_kb, int sms, int slots_per_tile);

struct Tile2 {
  int m0, n0;      // first row / column of the 256×256 tile (inside the expert's / batch entry's matrix)
  int b_row;       // GROUPED 1: first row of the expert's matrix in B; GROUPED 3: batch index
  int kb0, kb1;    // K-block range
  size_t out_off;  // element offset of the expert's / batch entry's output
  int split, tile_id;
};

template <int A_MN, int B_MN, int OUT_F32, int GROUPED = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Gemm2Params p,
                  const Group2Params gp) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T2_STAGES * T2_STAGE_BYTES);
  uint64_t* full_bar = bars;                          // [STAGES]  used in the leader CTA
  uint64_t* empty_bar = bars + T2_STAGES;             // [STAGES]  each CTA's producer waits on its own
  uint64_t* tmem_full = bars + 2 * T2_STAGES;         // [2]       each CTA's epilogue waits on its own
  uint64_t* tmem_empty = bars + 2 * T2_STAGES + 2;    // [2]       used in the leader CTA, 8 arrivals (4 warps × 2 CTAs)
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * T2_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int pair = static_cast<int>(blockIdx.x) >> 1, n_pair = static_cast<int>(gridDim.x) >> 1;
  __shared__ int s_off[258];
  if (GROUPED == 1 || GROUPED == 2) {
    for (int i = threadIdx.x; i <= gp.E; i += blockDim.x) s_off[i] = gp.offsets[i];
    __syncthreads();
  }
  const int glu = (!OUT_F32 && !A_MN && !B_MN && (GROUPED == 0 || GROUPED == 1)) ? p.glu_half : 0;
  const int num_n = glu ? (glu + T2_HALF - 1) / T2_HALF : (p.N + T2_BN - 1) / T2_BN;
  const int num_m = GROUPED == 1 ? s_off[gp.E] / T2_BM : (p.M + T2_BM - 1) / T2_BM;
  const int SK = (GROUPED == 0 && OUT_F32 && p.split_k > 1) ? p.split_k : 1;
  const bool sym = GROUPED == 3 && gp.sym != 0;
  const int per_problem = sym ? num_m * (num_m + 1) / 2 : num_m * num_n;
  const int num_tiles = ((GROUPED == 2 || GROUPED == 3) ? gp.E : 1) * per_problem * SK;
  const int num_kb = (p.K + T2_BK - 1) / T2_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 8); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) { tmem_alloc_2sm(tmem_ptr, 512); tmem_relinquish_2sm(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  auto get_tile = [&](int t, Tile2& tl) {
    tl.kb0 = 0; tl.kb1 = num_kb; tl.out_off = 0; tl.b_row = 0; tl.split = 0; tl.tile_id = t;
    if (SK > 1) {        // all pieces 0 come first in the global order: a piece only ever waits for work with a smaller index
      const int base_tiles = num_m * num_n;
      tl.split = t / base_tiles;
      t -= tl.split * base_tiles;
      tl.tile_id = t;
      const int per = (num_kb + SK - 1) / SK;
      tl.kb0 = tl.split * per < num_kb ? tl.split * per : num_kb;
      tl.kb1 = tl.kb0 + per < num_kb ? tl.kb0 + per : num_kb;
    }
    if (GROUPED == 2 || GROUPED == 3) {
      const int per = per_problem;
      const int e = t / per;
      int r = t - e * per;
      if (sym) {           // row mi of the upper triangle holds num_m − mi tiles
        int mi = 0;
        while (r >= num_m - mi) { r -= num_m - mi; ++mi; }
        tl.m0 = mi * T2_BM; tl.n0 = (mi + r) * T2_BN;
      } else {
        tl.m0 = (r % num_m) * T2_BM; tl.n0 = (r / num_m) * T2_BN;
      }
      tl.out_off = static_cast<size_t>(e) * p.M * p.ldc;
      if (GROUPED == 2) { tl.kb0 = s_off[e] / T2_BK; tl.kb1 = s_off[e + 1] / T2_BK; }
      else tl.b_row = e;
    } else {
      const int per_group = T2_GROUP_M * num_n;
      const int g = t / per_group;
      const int first_m = g * T2_GROUP_M;
      const int gsz = min(num_m - first_m, T2_GROUP_M);
      const int r = t - g * per_group;
      tl.m0 = (first_m + (r % gsz)) * T2_BM;
      tl.n0 = (r / gsz) * T2_BN;
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
      for (int t = pair; t < num_tiles; t += n_pair) {
        Tile2 tl; get_tile(t, tl);
        const int ma = tl.m0 + rank * T2_HALF, nb = glu ? tl.n0 / 2 + rank * glu : tl.n0 + rank * T2_HALF;
        for (int kb = tl.kb0; kb < tl.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
          uint8_t* sa = smem + stage * T2_STAGE_BYTES;
          uint8_t* sb = sa + T2_OP_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * T2_STAGE_BYTES);   // both CTAs' loads
          if (GROUPED == 3) {
            if (A_MN) {
#pragma unroll
              for (int c = 0; c < 2; ++c) tma_load_3d_2sm(sa + c * (64 * T2_BK * 2), &tmap_a, &full_bar[stage], ma + c * 64, kb * T2_BK, tl.b_row);
            } else {
              tma_load_3d_2sm(sa, &tmap_a, &full_bar[stage], kb * T2_BK, ma, tl.b_row);
            }
            if (B_MN) {
#pragma unroll
              for (int c = 0; c < 2; ++c) tma_load_3d_2sm(sb + c * (64 * T2_BK * 2), &tmap_b, &full_bar[stage], nb + c * 64, kb * T2_BK, tl.b_row);
            } else {
              tma_load_3d_2sm(sb, &tmap_b, &full_bar[stage], kb * T2_BK, nb, tl.b_row);
            }
            if (++stage == T2_STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          const int brow = GROUPED == 1 ? tl.b_row : 0;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_2sm(sa + c * (64 * T2_BK * 2), &tmap_a, &full_bar[stage], ma + c * 64, kb * T2_BK);
          } else {
            tma_load_2d_2sm(sa, &tmap_a, &full_bar[stage], kb * T2_BK, ma);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_2sm(sb + c * (64 * T2_BK * 2), &tmap_b, &full_bar[stage], nb + c * 64, brow + kb * T2_BK);
          } else {
            tma_load_2d_2sm(sb, &tmap_b, &full_bar[stage], kb * T2_BK, brow + nb);
          }
          if (++stage == T2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(T2_BM, T2_BN, A_MN, B_MN);
      constexpr uint32_t a_kstep = A_MN ? (16 * 128) >> 4 : 32 >> 4;
      constexpr uint32_t b_kstep = B_MN ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = pair; t < num_tiles; t += n_pair, ++it) {
        const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * T2_BN;
        Tile2 tl; get_tile(t, tl);
        for (int kb = tl.kb0; kb < tl.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * T2_STAGE_BYTES);
          const uint32_t sb = sa + T2_OP_BYTES;
          const uint64_t da = A_MN ? make_smem_desc(sa, 64 * T2_BK * 2, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t db = B_MN ? make_smem_desc(sb, 64 * T2_BK * 2, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < T2_BK / 16; ++k)
            umma_bf16_2sm(d_tmem, da + static_cast<uint64_t>(k * a_kstep), db + static_cast<uint64_t>(k * b_kstep), idesc,
                          (kb != tl.kb0 || k != 0) ? 1u : 0u);
          umma_commit_2sm(&empty_bar[stage], 3);          // frees the stage in both CTAs
          if (++stage == T2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (tl.kb0 == tl.kb1) { mbar_arrive(&tmem_full[acc]); mbar_arrive_peer(&tmem_full[acc]); }   // empty expert: nothing was issued
        else umma_commit_2sm(&tmem_full[acc], 3);         // both CTAs' epilogues may read their half
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    for (int t = pair; t < num_tiles; t += n_pair, ++it) {
      Tile2 tl; get_tile(t, tl);
      const int m0 = tl.m0, n0 = tl.n0;
      const bool empty_tile = tl.kb0 == tl.kb1;
      const int row_limit = GROUPED == 1 ? min(s_off[gp.E], p.M) : p.M;     // never past the rows the caller allocated
      const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const int row = m0 + rank * T2_HALF + q * 32 + lane;
      const float alpha = (GROUPED == 3 && gp.alpha_vec) ? p.alpha * gp.alpha_vec[tl.b_row] : p.alpha;
      const float beta = (GROUPED == 3 && gp.beta_vec) ? p.beta * gp.beta_vec[tl.b_row] : p.beta;
      int acc_flag = p.accumulate;
      uint32_t* sem = nullptr;
      if (OUT_F32 && SK > 1) {
        // wait until the previous piece of this tile has been added to this warp's 32 rows
        sem = p.sem + (tl.tile_id * 2 + rank) * 4 + q;
        if (tl.split > 0) {
          bool ok = true;
          if (lane == 0) {
            const long long t0 = clock64();
            while (ld_acquire_gpu(sem) != static_cast<uint32_t>(tl.split)) {
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
      const uint32_t taddr = tmem_base + acc * T2_BN + (static_cast<uint32_t>(q * 32) << 16);
      if (glu) {
#pragma unroll 1
        for (int c = 0; c < T2_HALF / 32; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c * 32, rg);
          tmem_ld_32x32(taddr + T2_HALF + c * 32, ru);
          tmem_ld_wait();
          const int col = n0 / 2 + c * 32;              // gate column; its up column is glu + col
          if (row < row_limit && col < glu && !empty_tile) {
            __nv_bfloat16* hg = p.out ? reinterpret_cast<__nv_bfloat16*>(p.out) + tl.out_off + static_cast<size_t>(row) * p.ldc + col : nullptr;
            __nv_bfloat16* oa = reinterpret_cast<__nv_bfloat16*>(p.out2) + static_cast<size_t>(row) * p.ldc2 + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < glu) {
                uint32_t gw[4], uw[4], aw[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  gw[e] = pack_bf16x2(__uint_as_float(rg[j + 2 * e]) * alpha, __uint_as_float(rg[j + 2 * e + 1]) * alpha);
                  uw[e] = pack_bf16x2(__uint_as_float(ru[j + 2 * e]) * alpha, __uint_as_float(ru[j + 2 * e + 1]) * alpha);
                  const float2 g2 = unpack_bf16x2(gw[e]), u2 = unpack_bf16x2(uw[e]);
                  aw[e] = pack_bf16x2(g2.x * (1.f / (1.f + __expf(-g2.x))) * u2.x, g2.y * (1.f / (1.f + __expf(-g2.y))) * u2.y);
                }
                if (hg) {
                  *reinterpret_cast<uint4*>(hg + j) = make_uint4(gw[0], gw[1], gw[2], gw[3]);
                  *reinterpret_cast<uint4*>(hg + glu + j) = make_uint4(uw[0], uw[1], uw[2], uw[3]);
                }
                *reinterpret_cast<uint4*>(oa + j) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
              }
            }
          } else if (row < row_limit && col < glu) {    // expert without rows: nothing was accumulated
            __nv_bfloat16* oa = reinterpret_cast<__nv_bfloat16*>(p.out2) + static_cast<size_t>(row) * p.ldc2 + col;
            for (int j = 0; j < 32 && col + j < glu; j += 8) *reinterpret_cast<uint4*>(oa + j) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < T2_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (empty_tile) {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        const int col = n0 + c * 32;
        if (row < row_limit && col < p.N) {
          if (OUT_F32) {
            float* o = reinterpret_cast<float*>(p.out) + tl.out_off + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha,
                                       __uint_as_float(r[j + 2]) * alpha, __uint_as_float(r[j + 3]) * alpha);
                if (acc_flag) {
                  const float4 old = *reinterpret_cast<const float4*>(o + j);
                  v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                }
                *reinterpret_cast<float4*>(o + j) = v;
              }
            }
          } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + tl.out_off + static_cast<size_t>(row) * p.ldc + col;
            const __nv_bfloat16* ci = p.cin ? reinterpret_cast<const __nv_bfloat16*>(p.cin) + tl.out_off + static_cast<size_t>(row) * p.ldc + col : nullptr;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < p.N) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]) * alpha;
                if (ci) {
                  const uint4 cv = *reinterpret_cast<const uint4*>(ci + j);
                  const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 c2 = unpack_bf16x2(cw[e]);
                    f[2 * e] += beta * c2.x; f[2 * e + 1] += beta * c2.y;
                  }
                }
                uint4 ov;
                ov.x = pack_bf16x2(f[0], f[1]); ov.y = pack_bf16x2(f[2], f[3]);
                ov.z = pack_bf16x2(f[4], f[5]); ov.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(o + j) = ov;
                if (GROUPED == 3 && sym && n0 != m0) {      // transposed copy: lanes hold consecutive rows → 64-byte segments
                  __nv_bfloat16* ot = reinterpret_cast<__nv_bfloat16*>(p.out) + tl.out_off + static_cast<size_t>(col + j) * p.ldc + row;
#pragma unroll
                  for (int e = 0; e < 8; ++e)
                    if (col + j + e < p.N) ot[static_cast<size_t>(e) * p.ldc] = __float2bfloat16_rn(f[e]);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tmem_empty[acc]);
      if (OUT_F32 && SK > 1) {
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu(sem, tl.split + 1 == SK ? 0u : static_cast<uint32_t>(tl.split + 1));
      }
    }
  }

done:
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

template <int A_MN, int B_MN, int OUT_F32>
static int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const Gemm2Params& p, int sms, cudaStream_t st) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((p.M + T2_BM - 1) / T2_BM) * ((p.N + T2_BN - 1) / T2_BN);
  const int pairs = sms / 2;
  Gemm2Params pp = p;
  pp.split_k = 1; pp.sem = nullptr;
  if (OUT_F32 && p.accumulate && g_splitk_sem != nullptr) {
    pp.split_k = choose_split_k(tiles, (p.K + T2_BK - 1) / T2_BK, pairs, 8);
    pp.sem = g_splitk_sem;
  }
  const int work = tiles * pp.split_k;
  const int grid = 2 * (work < pairs ? work : pairs);
  kern<<<grid, T2_THREADS, T2_SMEM_BYTES, st>>>(ta, tb, pp, Group2Params{});
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int A_MN, int B_MN, int OUT_F32, int GROUPED>
static int launch2_grouped(const CUtensorMap& ta, const CUtensorMap& tb, const Gemm2Params& p, const Group2Params& gp, int tiles,
                           int sms, cudaStream_t st) {
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, OUT_F32, GROUPED>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int pairs = sms / 2;
  const int grid = 2 * (tiles < pairs ? (tiles > 0 ? tiles : 1) : pairs);
  kern<<<grid, T2_THREADS, T2_SMEM_BYTES, st>>>(ta, tb, p, gp);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace b200

// Same contract as b200_gemm_bf16 (modes 0 NT, 1 NN, 2 TN; bf16 or fp32 output, optional α·AB + β·C or accumulate).
extern "C" int b200_gemm2_bf16(int mode, const void* A, const void* B, void* out, const void* cin, int M, int N, int K,
                               int lda, int ldb, int ldc, float alpha, float beta, int out_f32, int accumulate,
                               int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  if (mode == 2) rc = make_tmap_2d_bf16(&ta, A, M, K, lda, 64, T2_BK);        // stored [K, M]
  else           rc = make_tmap_2d_bf16(&ta, A, K, M, lda, T2_BK, T2_HALF);   // stored [M, K]
  if (rc) return rc;
  if (mode == 0) rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, T2_BK, T2_HALF);   // stored [N, K]
  else           rc = make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, T2_BK);        // stored [K, N]
  if (rc) return rc;
  Gemm2Params p{out, cin, M, N, K, ldc, alpha, beta, accumulate, status, 1, nullptr};
  if (mode == 0) return out_f32 ? launch2<0, 0, 1>(ta, tb, p, num_sms, stream) : launch2<0, 0, 0>(ta, tb, p, num_sms, stream);
  if (mode == 1) return out_f32 ? launch2<0, 1, 1>(ta, tb, p, num_sms, stream) : launch2<0, 1, 0>(ta, tb, p, num_sms, stream);
  if (mode == 2) return out_f32 ? launch2<1, 1, 1>(ta, tb, p, num_sms, stream) : launch2<1, 1, 0>(ta, tb, p, num_sms, stream);
  return -4;
}

// act [M, I] = silu(A·B_gateᵀ) ∘ (A·B_upᵀ) with B [2I, K] = [gate rows | up rows]; h (may be null) also receives the
// pre-activation [M, 2I].  A [M, K] with leading dimension lda; I a multiple of 8.
extern "C" int b200_gemm2_swiglu_bf16(const void* A, const void* B, void* h, void* act, int M, int I, int K, int lda, int ldb,
                                      int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if (I % 8) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, T2_BK, T2_HALF);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, B, K, 2 * static_cast<uint64_t>(I), ldb, T2_BK, T2_HALF);
  if (rc) return rc;
  Gemm2Params p{h, nullptr, M, 2 * I, K, 2 * I, 1.f, 0.f, 0, status, 1, nullptr, I, act, I};
  auto kern = gemm2_bf16_kernel<0, 0, 0>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((M + T2_BM - 1) / T2_BM) * ((I + T2_HALF - 1) / T2_HALF);
  const int pairs = num_sms / 2;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  kern<<<grid, T2_THREADS, T2_SMEM_BYTES, stream>>>(ta, tb, p, Group2Params{});
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// The same over expert segments (GROUPED 1): A rows grouped by expert (offsets[E+1], multiples of 256), B [E · 2I, K].
extern "C" int b200_grouped_gemm2_swiglu_bf16(const void* A, const void* B, void* h, void* act, const int* offsets, int E,
                                              int capacity, int I, int K, int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (E <= 0 || E > 256 || capacity <= 0 || capacity % T2_BM || I % 8) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, capacity, K, T2_BK, T2_HALF);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, B, K, static_cast<uint64_t>(E) * 2 * I, K, T2_BK, T2_HALF);
  if (rc) return rc;
  Group2Params gp{offsets, E, 2 * I, nullptr, nullptr, 0};
  Gemm2Params p{h, nullptr, capacity, 2 * I, K, 2 * I, 1.f, 0.f, 0, status, 1, nullptr, I, act, I};
  const int max_tiles = (capacity / T2_BM) * ((I + T2_HALF - 1) / T2_HALF);
  return launch2_grouped<0, 0, 0, 1>(ta, tb, p, gp, max_tiles, num_sms, stream);
}

// Grouped GEMM over expert segments, same contract as b200_grouped_gemm_bf16 except that `offsets` (and `capacity`) must
// be multiples of 256 rows and N a multiple of 256 for kinds 0 / 1.
extern "C" int b200_grouped_gemm2_bf16(int kind, const void* A, const void* B, void* out, const int* offsets, int E,
                                       int capacity, int M, int N, int K, int out_f32, int accumulate, int num_sms,
                                       int* status, cudaStream_t stream) {
  using namespace b200;
  if (E <= 0 || E > 256 || capacity <= 0 || capacity % T2_BM) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  Group2Params gp{offsets, E, 0, nullptr, nullptr, 0};
  if (kind == 0 || kind == 1) {
    if (N % T2_BN) return -1;
    rc = make_tmap_2d_bf16(&ta, A, K, capacity, K, T2_BK, T2_HALF);
    if (rc) return rc;
    if (kind == 0) { rc = make_tmap_2d_bf16(&tb, B, K, static_cast<uint64_t>(E) * N, K, T2_BK, T2_HALF); gp.b_rows = N; }
    else           { rc = make_tmap_2d_bf16(&tb, B, N, static_cast<uint64_t>(E) * K, N, 64, T2_BK); gp.b_rows = K; }
    if (rc) return rc;
    Gemm2Params p{out, nullptr, capacity, N, K, N, 1.f, 0.f, 0, status, 1, nullptr};
    const int max_tiles = (capacity / T2_BM) * (N / T2_BN);
    return kind == 0 ? launch2_grouped<0, 0, 0, 1>(ta, tb, p, gp, max_tiles, num_sms, stream)
                     : launch2_grouped<0, 1, 0, 1>(ta, tb, p, gp, max_tiles, num_sms, stream);
  }
  if (kind == 2) {
    rc = make_tmap_2d_bf16(&ta, A, M, capacity, M, 64, T2_BK);
    if (rc) return rc;
    rc = make_tmap_2d_bf16(&tb, B, N, capacity, N, 64, T2_BK);
    if (rc) return rc;
    Gemm2Params p{out, nullptr, M, N, capacity, N, 1.f, 0.f, accumulate, status, 1, nullptr};
    const int tiles = E * ((M + T2_BM - 1) / T2_BM) * ((N + T2_BN - 1) / T2_BN);
    return out_f32 ? launch2_grouped<1, 1, 1, 2>(ta, tb, p, gp, tiles, num_sms, stream)
                   : launch2_grouped<1, 1, 0, 2>(ta, tb, p, gp, tiles, num_sms, stream);
  }
  return -4;
}

// Batched GEMM, same contract as b200_gemm_bf16_batched; `symmetric`: the (square) results are symmetric matrices (and so is C),
// compute the upper triangle of tiles only and mirror it.  alpha_vec / beta_vec (device, `batch` floats, or null): per-problem
// factors multiplied into alpha / beta.
extern "C" int b200_gemm2_bf16_batched(int mode, const void* A, const void* B, void* out, const void* cin, int batch, int M,
                                       int N, int K, float alpha, float beta, const float* alpha_vec, const float* beta_vec,
                                       int symmetric, int num_sms, int* status, cudaStream_t stream) {
  using namespace b200;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  if (mode < 0 || mode > 2) return -4;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc;
  if (mode == 2) rc = make_tmap_3d_bf16(&ta, A, M, K, batch, M, static_cast<uint64_t>(K) * M, 64, T2_BK);        // stored [K, M]
  else           rc = make_tmap_3d_bf16(&ta, A, K, M, batch, K, static_cast<uint64_t>(M) * K, T2_BK, T2_HALF);   // stored [M, K]
  if (rc) return rc;
  if (mode == 0) rc = make_tmap_3d_bf16(&tb, B, K, N, batch, K, static_cast<uint64_t>(N) * K, T2_BK, T2_HALF);
  else           rc = make_tmap_3d_bf16(&tb, B, N, K, batch, N, static_cast<uint64_t>(K) * N, 64, T2_BK);
  if (rc) return rc;
  Gemm2Params p{out, cin, M, N, K, N, alpha, beta, 0, status, 1, nullptr};
  if (symmetric && M != N) return -1;
  Group2Params gp{nullptr, batch, 0, alpha_vec, beta_vec, symmetric};
  const int nm = (M + T2_BM - 1) / T2_BM;
  const int tiles = batch * (symmetric ? nm * (nm + 1) / 2 : nm * ((N + T2_BN - 1) / T2_BN));
  if (mode == 0) return launch2_grouped<0, 0, 0, 3>(ta, tb, p, gp, tiles, num_sms, stream);
  if (mode == 1) return launch2_grouped<0, 1, 0, 3>(ta, tb, p, gp, tiles, num_sms, stream);
  return launch2_grouped<1, 1, 0, 3>(ta, tb, p, gp, tiles, num_sms, stream);
}
