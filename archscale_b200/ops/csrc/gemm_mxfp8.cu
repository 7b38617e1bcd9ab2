// Block-scaled MXFP8 (OCP microscaling: e4m3 elements, one E8M0 scale per 32 elements along K) on the
// 5th-generation tensor cores:  out[M,N] = alpha · (A ⊙ sfA) · (B ⊙ sfB)ᵀ, both operands K-major.
//
//   quantisers   bf16 → e4m3 + E8M0, row-wise (blocks along the contiguous dimension) or column-wise (the
//                transposed operand is written, blocks along the original rows), so that forward, dgrad and
//                wgrad of a linear layer are all "NT" GEMMs over K-major fp8 operands.
//   GEMM         persistent warp-specialised kernel (TMA producer / MMA issuer / 4 epilogue warps) issuing
//                tcgen05.mma.kind::mxf8f6f4.block_scale, tile 128 × 192 × 128, 5-stage ring, two TMEM
//                accumulators (2 × 192 columns) so the epilogue of a tile overlaps the next main loop.
//
// Scale factors are stored in global memory in the order the tensor core wants them in TMEM, in 512-byte
// chunks that cover 128 rows × 4 K-blocks:  byte (m % 32)·16 + ((m / 32) % 4)·4 + (kb % 4) of chunk
// (m / 128, kb / 4).  A chunk is fetched with one bulk copy and moved to tensor memory with one
// tcgen05.cp.32x128b.warpx4: lane m % 32 of every lane quarter, column (m / 32) % 4, byte kb % 4.
// A 192-wide B tile starts at a multiple of 64 rows; when that is the middle of a chunk the MMA is given
// the scale address two columns further (rows 64.. of the first chunk), and two chunks are always loaded.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

constexpr int QBM = 128, QBN = 192, QBK = 128, QSTAGES = 5;
constexpr int QA_BYTES = QBM * QBK, QB_BYTES = QBN * QBK;
constexpr int QSFA_OFF = QA_BYTES + QB_BYTES, QSFB_OFF = QSFA_OFF + 512;
constexpr int QSTAGE_BYTES = 43008;                               // 42 KiB: keeps every stage 1024-byte aligned
constexpr int QSMEM_BYTES = QSTAGES * QSTAGE_BYTES + 1024 + 256;
constexpr int Q_TMEM_SFA = 384, Q_TMEM_SFB = 392;                 // columns after the two accumulators
constexpr int Q_GROUP_M = 16;

struct QGemmParams {
  void* out;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int M, N, K, ldc;
  float alpha;
  int accumulate;
  int* status;
};

__device__ __forceinline__ void q_bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Unswizzled K-major descriptor of a 32-row × 16-byte scale chunk: 8-row groups are 128 bytes apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t tsfa,
                                          uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// e4m3 × e4m3, E8M0 scales, fp32 accumulate, both operands K-major
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int M, int N) {
  return (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(M >> 4) << 24);
}

template <int OUT_F32>
__global__ void __launch_bounds__(192, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const QGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + QSTAGES * QSTAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + QSTAGES;
  uint64_t* tmem_full = bars + 2 * QSTAGES;
  uint64_t* tmem_empty = bars + 2 * QSTAGES + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * QSTAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, n_cta = gridDim.x;
  const int num_m = (p.M + QBM - 1) / QBM, num_n = (p.N + QBN - 1) / QBN;
  const int num_tiles = num_m * num_n;
  const int KC = p.K / QBK;                      // K chunks of 128 elements = 4 scale blocks
  const int n_chunks_n = (p.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < QSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
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

  auto tile_coords = [&](int t, int& m0, int& n0) {
    const int per_group = Q_GROUP_M * num_n;
    const int g = t / per_group, first_m = g * Q_GROUP_M;
    const int gsz = min(num_m - first_m, Q_GROUP_M);
    const int r = t - g * per_group;
    m0 = (first_m + (r % gsz)) * QBM;
    n0 = (r / gsz) * QBN;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int t = cta; t < num_tiles; t += n_cta) {
        int m0, n0; tile_coords(t, m0, n0);
        const int c0 = n0 >> 7;                                  // first 128-row scale chunk of the B tile
        const int nb = (c0 + 1 < n_chunks_n) ? 2 : 1;
        for (int kb = 0; kb < KC; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
          uint8_t* sa = smem + stage * QSTAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], QA_BYTES + QB_BYTES + 512 + 512 * nb);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * QBK, m0);
          tma_load_2d(sa + QA_BYTES, &tmap_b, &full_bar[stage], kb * QBK, n0);
          q_bulk_g2s(sa + QSFA_OFF, p.sfa + (static_cast<size_t>(m0 >> 7) * KC + kb) * 512, 512, &full_bar[stage]);
          q_bulk_g2s(sa + QSFB_OFF, p.sfb + (static_cast<size_t>(c0) * KC + kb) * 512, 512, &full_bar[stage]);
          if (nb == 2)
            q_bulk_g2s(sa + QSFB_OFF + 512, p.sfb + (static_cast<size_t>(c0 + 1) * KC + kb) * 512, 512, &full_bar[stage]);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc0 = make_idesc_mxf8(QBM, QBN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = cta; t < num_tiles; t += n_cta, ++it) {
        const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        tc_fence_after();
        int m0, n0; tile_coords(t, m0, n0);
        const uint32_t d_tmem = tmem_base + acc * QBN;
        const uint32_t tsfa = tmem_base + Q_TMEM_SFA;
        const uint32_t tsfb = tmem_base + Q_TMEM_SFB + ((n0 >> 5) & 3);   // 0 or 2: rows 64.. of the first chunk
        for (int kb = 0; kb < KC; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * QSTAGE_BYTES);
          tmem_cp_sf(tmem_base + Q_TMEM_SFA, make_sf_desc(sa + QSFA_OFF));
          tmem_cp_sf(tmem_base + Q_TMEM_SFB, make_sf_desc(sa + QSFB_OFF));
          tmem_cp_sf(tmem_base + Q_TMEM_SFB + 4, make_sf_desc(sa + QSFB_OFF + 512));
          const uint64_t da = make_smem_desc(sa, 16, 1024);
          const uint64_t db = make_smem_desc(sa + QA_BYTES, 16, 1024);
#pragma unroll
          for (uint32_t k = 0; k < QBK / 32; ++k) {
            // K-block k of the stage: operands advance 32 bytes, the scale of byte k of each column is used
            const uint32_t idesc = idesc0 | (k << 4) | (k << 29);
            umma_mxf8(d_tmem, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc,
                      tsfa | (k << 30), tsfb | (k << 30), (kb != 0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == QSTAGES) { stage = 0; phase ^= 1; }
        }
        if (KC == 0) mbar_arrive(&tmem_full[acc]);
        else umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    for (int t = cta; t < num_tiles; t += n_cta, ++it) {
      int m0, n0; tile_coords(t, m0, n0);
      const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * QBN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < QBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (KC == 0) {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        const int col = n0 + c * 32;
        if (row < p.M && col < p.N) {
          if (OUT_F32) {
            float* o = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha,
                                       __uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha);
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(o + j);
                  v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                }
                *reinterpret_cast<float4*>(o + j) = v;
              }
            }
          } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < p.N) {
                uint4 ov;
                ov.x = pack_bf16x2(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha);
                ov.y = pack_bf16x2(__uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha);
                ov.z = pack_bf16x2(__uint_as_float(r[j + 4]) * p.alpha, __uint_as_float(r[j + 5]) * p.alpha);
                ov.w = pack_bf16x2(__uint_as_float(r[j + 6]) * p.alpha, __uint_as_float(r[j + 7]) * p.alpha);
                *reinterpret_cast<uint4*>(o + j) = ov;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
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

// ------------------------------------------------------------------ quantisers
// Smallest power of two ≥ amax / 448 as a biased E8M0 exponent (clamped to [1, 253]).
__device__ __forceinline__ uint32_t e8m0_for_amax(float amax) {
  const uint32_t b = __float_as_uint(__fdiv_rn(amax, 448.f));   // exact: powers of two must not round up
  uint32_t ex = (b >> 23) & 0xffu;
  if (b & 0x7fffffu) ex += 1;
  return min(max(ex, 1u), 253u);
}
__device__ __forceinline__ size_t sf_offset(int row, int kb, int KC) {
  return (static_cast<size_t>(row >> 7) * KC + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}
__device__ __forceinline__ uint32_t cvt4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// One thread per 32-element block of a row.  x: [R, C] bf16 (row stride ld), q: [R, C] e4m3, C % 128 == 0.
__global__ void __launch_bounds__(256) mxfp8_quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int R, int C) {
  const int nblk = C >> 5;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(R) * nblk) return;
  const int r = static_cast<int>(idx / nblk), kb = static_cast<int>(idx % nblk);
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ld + kb * 32);
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 u = src[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(w[e]);
      v[i * 8 + 2 * e] = f.x; v[i * 8 + 2 * e + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  const uint32_t ex = e8m0_for_amax(amax);
  const float inv = __uint_as_float((254u - ex) << 23);
  uint4* dst = reinterpret_cast<uint4*>(q + static_cast<size_t>(r) * C + kb * 32);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 o;
    o.x = cvt4_e4m3(v[i * 16 + 0] * inv, v[i * 16 + 1] * inv, v[i * 16 + 2] * inv, v[i * 16 + 3] * inv);
    o.y = cvt4_e4m3(v[i * 16 + 4] * inv, v[i * 16 + 5] * inv, v[i * 16 + 6] * inv, v[i * 16 + 7] * inv);
    o.z = cvt4_e4m3(v[i * 16 + 8] * inv, v[i * 16 + 9] * inv, v[i * 16 + 10] * inv, v[i * 16 + 11] * inv);
    o.w = cvt4_e4m3(v[i * 16 + 12] * inv, v[i * 16 + 13] * inv, v[i * 16 + 14] * inv, v[i * 16 + 15] * inv);
    dst[i] = o;
  }
  sf[sf_offset(r, kb, nblk >> 2)] = static_cast<uint8_t>(ex);
}

// Column-wise: writes the transposed operand qT [C, R] with scale blocks along R; with ROWS it also writes the row-wise
// operand q [R, C] from the same shared-memory tile (one read of a tensor that is needed in both orientations).
// R % 128 == 0, C % 64 == 0 (ROWS: C % 128 == 0).
template <int ROWS>
__global__ void __launch_bounds__(256) mxfp8_quant_colwise_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                                 uint8_t* __restrict__ qT, uint8_t* __restrict__ sfT,
                                                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int R, int C) {
  __shared__ __align__(16) __nv_bfloat16 s[128][72];
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 64, tid = threadIdx.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = tid + 256 * i, row = idx >> 3, cv = idx & 7;
    const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0 + row) * ld + c0 + cv * 8);
    *reinterpret_cast<uint4*>(&s[row][cv * 8]) = u;
  }
  __syncthreads();
  {
    const int c = tid & 63, rb = tid >> 6;
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) { v[j] = __bfloat162float(s[rb * 32 + j][c]); amax = fmaxf(amax, fabsf(v[j])); }
    const uint32_t ex = e8m0_for_amax(amax);
    const float inv = __uint_as_float((254u - ex) << 23);
    uint4* dst = reinterpret_cast<uint4*>(qT + static_cast<size_t>(c0 + c) * R + r0 + rb * 32);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 o;
      o.x = cvt4_e4m3(v[i * 16 + 0] * inv, v[i * 16 + 1] * inv, v[i * 16 + 2] * inv, v[i * 16 + 3] * inv);
      o.y = cvt4_e4m3(v[i * 16 + 4] * inv, v[i * 16 + 5] * inv, v[i * 16 + 6] * inv, v[i * 16 + 7] * inv);
      o.z = cvt4_e4m3(v[i * 16 + 8] * inv, v[i * 16 + 9] * inv, v[i * 16 + 10] * inv, v[i * 16 + 11] * inv);
      o.w = cvt4_e4m3(v[i * 16 + 12] * inv, v[i * 16 + 13] * inv, v[i * 16 + 14] * inv, v[i * 16 + 15] * inv);
      dst[i] = o;
    }
    sfT[sf_offset(c0 + c, (r0 >> 5) + rb, R >> 7)] = static_cast<uint8_t>(ex);
  }
  if (ROWS) {
    const int row = tid >> 1, blk = tid & 1;                              // 128 rows × 2 blocks of 32 columns
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = *reinterpret_cast<const uint4*>(&s[row][blk * 32 + i * 8]);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(w[e]);
        v[i * 8 + 2 * e] = f.x; v[i * 8 + 2 * e + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    const uint32_t ex = e8m0_for_amax(amax);
    const float inv = __uint_as_float((254u - ex) << 23);
    uint4* dst = reinterpret_cast<uint4*>(q + static_cast<size_t>(r0 + row) * C + c0 + blk * 32);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 o;
      o.x = cvt4_e4m3(v[i * 16 + 0] * inv, v[i * 16 + 1] * inv, v[i * 16 + 2] * inv, v[i * 16 + 3] * inv);
      o.y = cvt4_e4m3(v[i * 16 + 4] * inv, v[i * 16 + 5] * inv, v[i * 16 + 6] * inv, v[i * 16 + 7] * inv);
      o.z = cvt4_e4m3(v[i * 16 + 8] * inv, v[i * 16 + 9] * inv, v[i * 16 + 10] * inv, v[i * 16 + 11] * inv);
      o.w = cvt4_e4m3(v[i * 16 + 12] * inv, v[i * 16 + 13] * inv, v[i * 16 + 14] * inv, v[i * 16 + 15] * inv);
      dst[i] = o;
    }
    sf[sf_offset(r0 + row, (c0 >> 5) + blk, C >> 7)] = static_cast<uint8_t>(ex);
  }
}

typedef CUresult (*EncodeTiledFnQ)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int make_tmap_2d_u8(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer) {
  static EncodeTiledFnQ fn = nullptr;
  if (!fn) {
    void* ptr_fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr_fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<EncodeTiledFnQ>(ptr_fn);
  }
  cuuint64_t gdim[2] = {inner, outer};
  cuuint64_t gstride[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}


// =====================================================================================================================
// NVFP4: e2m1 elements (two per byte, element 2i in the low nibble), one unsigned E4M3 scale per 16 elements along K and
// one fp32 scale per tensor:  x ≈ tensor_scale · block_scale · e2m1.   tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X
// consumes 64 elements (32 bytes) of K per instruction and the four block scales of that span from one 32-bit column of
// tensor memory per 32 rows, so the 512-byte scale chunk above (128 rows × 4 scales) is exactly one instruction's worth and
// the quantisers reuse sf_offset() with 16-element blocks and K/64 chunks per row chunk.
//   tile 128 × 192 × 256 elements (128 bytes of K per row and stage), 4-stage ring of 46 KB, two accumulators.
// The epilogue reads the two tensors' largest magnitudes from device memory and forms the product of the tensor scales
// itself (no host round trip, no launch in between).
constexpr int FBK = 256, FSTAGES = 4;                                   // elements of K per stage
constexpr int FA_BYTES = QBM * 128, FB_BYTES = QBN * 128;
constexpr int FSFA_OFF = FA_BYTES + FB_BYTES, FSFB_OFF = FSFA_OFF + 2048;
constexpr int FSTAGE_BYTES = FSFB_OFF + 4096;                           // 47104 = 46 KiB, a multiple of 1024
constexpr int FSMEM_BYTES = FSTAGES * FSTAGE_BYTES + 1024 + 256;
constexpr int F_TMEM_SFA = 384, F_TMEM_SFB = 400;                       // 16 + 32 columns after the two accumulators
static_assert(FSTAGE_BYTES % 1024 == 0, "stages must stay 1024-byte aligned");

// tensor scale from the tensor's largest magnitude: amax / (6 · 448), or 1 for an all-zero tensor
__device__ __forceinline__ float nvfp4_tensor_scale(float amax) {
  return amax > 0.f ? __fmul_rn(amax, static_cast<float>(1.0 / 2688.0)) : 1.f;
}
__device__ __forceinline__ void umma_nvf4(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t tsfa,
                                          uint32_t tsfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
// e2m1 × e2m1 (format code 1 in both operand fields), unsigned E4M3 scales (scale-format bit clear), fp32 accumulate
__host__ __device__ constexpr uint32_t make_idesc_nvf4(int M, int N) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

template <int OUT_F32>
__global__ void __launch_bounds__(192, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const QGemmParams p,
                  const float* __restrict__ amax_a, const float* __restrict__ amax_b) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FSTAGES * FSTAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + FSTAGES;
  uint64_t* tmem_full = bars + 2 * FSTAGES;
  uint64_t* tmem_empty = bars + 2 * FSTAGES + 2;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * FSTAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, n_cta = gridDim.x;
  const int num_m = (p.M + QBM - 1) / QBM, num_n = (p.N + QBN - 1) / QBN;
  const int num_tiles = num_m * num_n;
  const int KC = p.K / FBK;                      // stages along K: 256 elements = 4 instructions = 4 scale chunks
  const int n_chunks_n = (p.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < FSTAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
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

  auto tile_coords = [&](int t, int& m0, int& n0) {
    const int per_group = Q_GROUP_M * num_n;
    const int g = t / per_group, first_m = g * Q_GROUP_M;
    const int gsz = min(num_m - first_m, Q_GROUP_M);
    const int r = t - g * per_group;
    m0 = (first_m + (r % gsz)) * QBM;
    n0 = (r / gsz) * QBN;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (int t = cta; t < num_tiles; t += n_cta) {
        int m0, n0; tile_coords(t, m0, n0);
        const int c0 = n0 >> 7;                                  // first 128-row scale chunk of the B tile
        const int nb = (c0 + 1 < n_chunks_n) ? 2 : 1;
        for (int kb = 0; kb < KC; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) goto done;
          uint8_t* sa = smem + stage * FSTAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], FA_BYTES + FB_BYTES + 2048 + 2048 * nb);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * 128, m0);                      // coordinates in bytes
          tma_load_2d(sa + FA_BYTES, &tmap_b, &full_bar[stage], kb * 128, n0);
          // the four chunks of one row chunk and one stage are adjacent in memory
          q_bulk_g2s(sa + FSFA_OFF, p.sfa + (static_cast<size_t>(m0 >> 7) * KC + kb) * 2048, 2048, &full_bar[stage]);
          q_bulk_g2s(sa + FSFB_OFF, p.sfb + (static_cast<size_t>(c0) * KC + kb) * 2048, 2048, &full_bar[stage]);
          if (nb == 2)
            q_bulk_g2s(sa + FSFB_OFF + 2048, p.sfb + (static_cast<size_t>(c0 + 1) * KC + kb) * 2048, 2048, &full_bar[stage]);
          if (++stage == FSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_nvf4(QBM, QBN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = cta; t < num_tiles; t += n_cta, ++it) {
        const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) goto done;
        tc_fence_after();
        int m0, n0; tile_coords(t, m0, n0);
        const uint32_t d_tmem = tmem_base + acc * QBN;
        const uint32_t sfb_shift = (n0 >> 5) & 3;                         // 0 or 2: rows 64.. of the first row chunk
        for (int kb = 0; kb < KC; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, STATUS_TIMEOUT_FULL)) goto done;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * FSTAGE_BYTES);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k) {
            tmem_cp_sf(tmem_base + F_TMEM_SFA + 4 * k, make_sf_desc(sa + FSFA_OFF + 512 * k));
            tmem_cp_sf(tmem_base + F_TMEM_SFB + 8 * k, make_sf_desc(sa + FSFB_OFF + 512 * k));
            tmem_cp_sf(tmem_base + F_TMEM_SFB + 8 * k + 4, make_sf_desc(sa + FSFB_OFF + 2048 + 512 * k));
          }
          const uint64_t da = make_smem_desc(sa, 16, 1024);
          const uint64_t db = make_smem_desc(sa + FA_BYTES, 16, 1024);
#pragma unroll
          for (uint32_t k = 0; k < 4; ++k)                               // 64 elements = 32 bytes of K per instruction
            umma_nvf4(d_tmem, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc,
                      tmem_base + F_TMEM_SFA + 4 * k, tmem_base + F_TMEM_SFB + 8 * k + sfb_shift,
                      (kb != 0 || k != 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == FSTAGES) { stage = 0; phase ^= 1; }
        }
        if (KC == 0) mbar_arrive(&tmem_full[acc]);
        else umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    const float alpha = p.alpha * __fmul_rn(nvfp4_tensor_scale(*amax_a), nvfp4_tensor_scale(*amax_b));
    int it = 0;
    for (int t = cta; t < num_tiles; t += n_cta, ++it) {
      int m0, n0; tile_coords(t, m0, n0);
      const int acc = it & 1; const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) goto done;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * QBN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < QBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (KC == 0) {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        const int col = n0 + c * 32;
        if (row < p.M && col < p.N) {
          if (OUT_F32) {
            float* o = reinterpret_cast<float*>(p.out) + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha,
                                       __uint_as_float(r[j + 2]) * alpha, __uint_as_float(r[j + 3]) * alpha);
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(o + j);
                  v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                }
                *reinterpret_cast<float4*>(o + j) = v;
              }
            }
          } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < p.N) {
                uint4 ov;
                ov.x = pack_bf16x2(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha);
                ov.y = pack_bf16x2(__uint_as_float(r[j + 2]) * alpha, __uint_as_float(r[j + 3]) * alpha);
                ov.z = pack_bf16x2(__uint_as_float(r[j + 4]) * alpha, __uint_as_float(r[j + 5]) * alpha);
                ov.w = pack_bf16x2(__uint_as_float(r[j + 6]) * alpha, __uint_as_float(r[j + 7]) * alpha);
                *reinterpret_cast<uint4*>(o + j) = ov;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
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

// ---- NVFP4 quantisers.  amax[0] = max |x| over the tensor (nvfp4_amax_kernel); tensor scale = amax / (6 · 448), 1 if zero.
// block scale = E4M3(amax_block · (1 / (6 · tensor_scale))), round to nearest; element = e2m1(x / (block · tensor)), round to
// nearest even, saturating at 6.
__device__ __forceinline__ float nvfp4_block_scale(float amax, float tensor_scale, uint8_t* code) {
  // amax · (1 / (6 · tensor_scale)) with every step rounded to nearest: the same three operations as the PyTorch
  // restatement, so that both give the same scale even where the exact quotient is a tie between two E4M3 values
  const float want = fminf(__fmul_rn(amax, __frcp_rn(__fmul_rn(tensor_scale, 6.f))), 448.f);
  const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
  *code = static_cast<uint8_t>(b);
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  const float sb = __half2float(*reinterpret_cast<const __half*>(&h));
  return sb > 0.f ? __frcp_rn(sb * tensor_scale) : 0.f;                 // multiply by this, then round to e2m1
}

// Stochastic rounding of four values to e2m1 in one instruction (the converter rounds a magnitude up to the next grid value
// with probability (a − lower) / (upper − lower), drawing on the 32 random bits it is given).  The first operand of the vector
// lands in the most significant nibble, so the values are passed last-first to get element 0 into nibble 0.
__device__ __forceinline__ uint32_t e2m1x4_sr(float x0, float x1, float x2, float x3, uint32_t rbits) {
  uint16_t d;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(d) : "f"(x3), "f"(x2), "f"(x1), "f"(x0), "r"(rbits));
  return d;
}
// 32 random bits from a counter (the 32-bit finaliser of MurmurHash3 over index ^ seed): no state, any element order.
__device__ __forceinline__ uint32_t hashed_bits(uint32_t seed, unsigned long long index) {
  uint32_t x = static_cast<uint32_t>(index) * 0x9E3779B1u ^ static_cast<uint32_t>(index >> 32) ^ seed;
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}
// v ← (sign ⊙ v) · H16 / 4 with H16 the 16 × 16 Sylvester Hadamard matrix (four butterfly stages); orthogonal.
__device__ __forceinline__ void hadamard16(float (&v)[16], uint32_t sign_mask) {
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = (sign_mask >> j) & 1u ? -v[j] : v[j];
#pragma unroll
  for (int h = 1; h < 16; h <<= 1)
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (!(j & h)) { const float a = v[j], b = v[j | h]; v[j] = a + b; v[j | h] = a - b; }
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] *= 0.25f;
}

// Quantise 16 values held in registers: returns the two packed words and the scale code.  SR: stochastic rounding of the
// elements with random bits hashed from (seed, index of every fourth element).
template <bool SR>
__device__ __forceinline__ uint2 nvfp4_pack16(const float (&v)[16], float ts, uint8_t* code, uint32_t seed = 0,
                                              unsigned long long index = 0) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
  const float inv = nvfp4_block_scale(amax, ts, code);
  uint32_t lo = 0, hi = 0;
  if (SR) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {                    // one hash and one conversion per four elements
      lo |= e2m1x4_sr(v[4 * g] * inv, v[4 * g + 1] * inv, v[4 * g + 2] * inv, v[4 * g + 3] * inv, hashed_bits(seed, index + 4 * g)) << (16 * g);
      hi |= e2m1x4_sr(v[8 + 4 * g] * inv, v[9 + 4 * g] * inv, v[10 + 4 * g] * inv, v[11 + 4 * g] * inv,
                      hashed_bits(seed, index + 8 + 4 * g)) << (16 * g);
    }
  } else {
    // the converter instruction, two values at a time (round to nearest even, saturating); + 0 turns the −0 of a negative
    // value times a zero scale into +0, as the PyTorch restatement has it
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      lo |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(__fadd_rn(v[2 * e] * inv, 0.f), __fadd_rn(v[2 * e + 1] * inv, 0.f)),
                                                            __NV_E2M1, cudaRoundNearest)) << (8 * e);
      hi |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(__fadd_rn(v[8 + 2 * e] * inv, 0.f), __fadd_rn(v[9 + 2 * e] * inv, 0.f)),
                                                            __NV_E2M1, cudaRoundNearest)) << (8 * e);
    }
  }
  return make_uint2(lo, hi);
}
__device__ __forceinline__ void unpack16(const uint4& u0, const uint4& u1, float (&v)[16]) {
  const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
  for (int e = 0; e < 8; ++e) { const float2 f = unpack_bf16x2(w[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
}

// One thread per 16-element block of a row.  x: [R, C] bf16, q: [R, C/2] bytes, C % 256 == 0.  (A thread per 64 elements,
// with whole 32-byte sectors and aligned scale words out, was measured slower: 0.072 against 0.076 ms net became 0.083 for
// 32768 × 2048 — consecutive threads then read 128 bytes apart.)
template <bool SR>
__global__ void __launch_bounds__(256) nvfp4_quant_rowwise_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                 const float* __restrict__ amax_t, int R, int C, uint32_t seed) {
  const int nblk = C >> 4;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(R) * nblk) return;
  const int r = static_cast<int>(idx / nblk), kb = static_cast<int>(idx % nblk);
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ld + kb * 16);
  const uint4 u0 = src[0], u1 = src[1];
  float v[16];
  unpack16(u0, u1, v);
  uint8_t code;
  const uint2 w = nvfp4_pack16<SR>(v, nvfp4_tensor_scale(*amax_t), &code, seed, static_cast<unsigned long long>(r) * C + kb * 16);
  *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * (C >> 1) + kb * 8) = w;
  sf[sf_offset(r, kb, nblk >> 2)] = code;
}

// Column-wise: writes the transposed operand qT [C, R/2] with 16-element scale blocks along R; with ROWS it also writes
// the row-wise operand q [R, C/2] (blocks along C) from the same shared-memory tile, so that a tensor needed in both
// orientations (an activation for forward and weight gradient, an output gradient for both backward products) is read
// once.  Tile 128 rows × 64 columns.  R % 256 == 0, C % 64 == 0 (ROWS: C % 256 == 0).
// SR: stochastic rounding of both outputs.  RHT: every 16-element block of the TRANSPOSED operand is multiplied by
// diag(sign) · H16 / 4 before it is quantised (both operands of a weight-gradient product get the same transform, which
// cancels in the product and spreads outliers over the block); its tensor scale is then taken from 4 · amax, the bound of
// a transformed element.
template <int ROWS, bool SR, bool RHT>
__global__ void __launch_bounds__(256) nvfp4_quant_colwise_kernel(const __nv_bfloat16* __restrict__ x, int ld,
                                                                 uint8_t* __restrict__ qT, uint8_t* __restrict__ sfT,
                                                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                 const float* __restrict__ amax_t, int R, int C, uint32_t seed,
                                                                 uint32_t sign_mask) {
  __shared__ __align__(16) __nv_bfloat16 s[128][72];
  const int r0 = blockIdx.y * 128, c0 = blockIdx.x * 64, tid = threadIdx.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = tid + 256 * i, row = idx >> 3, cv = idx & 7;
    const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0 + row) * ld + c0 + cv * 8);
    *reinterpret_cast<uint4*>(&s[row][cv * 8]) = u;
  }
  __syncthreads();
  const float ts = nvfp4_tensor_scale(*amax_t);
  {
    const int c = tid & 63, rb = tid >> 6;                               // 32 rows = two blocks per thread
    uint32_t words[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __bfloat162float(s[rb * 32 + h * 16 + j][c]);
      if (RHT) hadamard16(v, sign_mask);
      uint8_t code;
      const uint2 w = nvfp4_pack16<SR>(v, RHT ? nvfp4_tensor_scale(4.f * *amax_t) : ts, &code, seed ^ 0x5bd1e995u,
                                       static_cast<unsigned long long>(c0 + c) * R + r0 + rb * 32 + h * 16);
      words[2 * h] = w.x; words[2 * h + 1] = w.y;
      sfT[sf_offset(c0 + c, (r0 >> 4) + rb * 2 + h, R >> 6)] = code;
    }
    *reinterpret_cast<uint4*>(qT + static_cast<size_t>(c0 + c) * (R >> 1) + ((r0 + rb * 32) >> 1)) =
        make_uint4(words[0], words[1], words[2], words[3]);
  }
  if (ROWS) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {                                        // 128 rows × 4 blocks of 16 columns
      const int item = tid + 256 * i, row = item >> 2, blk = item & 3;
      const uint4 u0 = *reinterpret_cast<const uint4*>(&s[row][blk * 16]);
      const uint4 u1 = *reinterpret_cast<const uint4*>(&s[row][blk * 16 + 8]);
      float v[16];
      unpack16(u0, u1, v);
      uint8_t code;
      const uint2 w = nvfp4_pack16<SR>(v, ts, &code, seed, static_cast<unsigned long long>(r0 + row) * C + c0 + blk * 16);
      *reinterpret_cast<uint2*>(q + static_cast<size_t>(r0 + row) * (C >> 1) + ((c0 + blk * 16) >> 1)) = w;
      sf[sf_offset(r0 + row, (c0 >> 4) + blk, C >> 6)] = code;
    }
  }
}

// amax[0] = max(amax[0], max |x|) over a [R, C] bf16 tensor with row stride ld (amax zeroed by the caller); C % 8 == 0.
// (Four loads in flight per thread, strided over the grid or consecutive within the block, were both measured slower
// than this plain grid-stride loop: 0.054 against 0.043 ms for 134 MB.)
__global__ void __launch_bounds__(256) nvfp4_amax_kernel(const __nv_bfloat16* __restrict__ x, int ld, float* __restrict__ amax,
                                                        int R, int C) {
  const int vec_per_row = C >> 3;
  const size_t total = static_cast<size_t>(R) * vec_per_row;
  float m = 0.f;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(x + (i / vec_per_row) * ld + (i % vec_per_row) * 8);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = unpack_bf16x2(w[e]); m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y))); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));   // m ≥ 0: bit order = value order
}

}  // namespace b200

using namespace b200;

// Bytes of the scale buffer of an operand with `rows` rows and K elements per row (zero-fill it once: rows
// beyond the operand inside the last 128-row chunk are never written by the quantisers).
extern "C" size_t b200_mxfp8_sf_bytes(int rows, int K) { return static_cast<size_t>((rows + 127) / 128) * (K / 128) * 512; }

// colwise 0: row-wise (q, sf); 1: column-wise, the transposed operand (into q, sf); 2: both from one read of x
// (row-wise into q, sf and the transposed operand into qT, sfT).
extern "C" int b200_mxfp8_quantize(const void* x, int ld, void* q, void* sf, int R, int C, int colwise, cudaStream_t st,
                                   void* qT, void* sfT) {
  if (R <= 0 || C <= 0) return 0;
  if (ld % 8) return -1;
  if (!colwise) {
    if (C % 128) return -1;
    const long long total = static_cast<long long>(R) * (C / 32);
    mxfp8_quant_rowwise_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
        (const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, R, C);
  } else if (colwise == 1) {
    if (R % 128 || C % 64) return -1;
    mxfp8_quant_colwise_kernel<0><<<dim3(C / 64, R / 128), 256, 0, st>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf,
                                                                         nullptr, nullptr, R, C);
  } else {
    if (R % 128 || C % 128 || !qT || !sfT) return -1;
    mxfp8_quant_colwise_kernel<1><<<dim3(C / 64, R / 128), 256, 0, st>>>((const __nv_bfloat16*)x, ld, (uint8_t*)qT, (uint8_t*)sfT,
                                                                         (uint8_t*)q, (uint8_t*)sf, R, C);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// out[M,N] = alpha · A[M,K] · B[N,K]ᵀ with e4m3 operands (row strides lda, ldb bytes) and chunked E8M0 scales.
extern "C" int b200_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* out, int M, int N, int K,
                               int lda, int ldb, int ldc, float alpha, int out_f32, int accumulate, int num_sms, int* status,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % QBK || lda % 16 || ldb % 16 || N % 8) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_u8(&ta, A, K, M, lda, QBK, QBM);
  if (rc) return rc;
  rc = make_tmap_2d_u8(&tb, B, K, N, ldb, QBK, QBN);
  if (rc) return rc;
  QGemmParams p{out, (const uint8_t*)sfa, (const uint8_t*)sfb, M, N, K, ldc, alpha, accumulate, status};
  const int tiles = ((M + QBM - 1) / QBM) * ((N + QBN - 1) / QBN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  static bool configured[2] = {false, false};
  if (out_f32) {
    if (!configured[1]) {
      if (cudaFuncSetAttribute(gemm_mxfp8_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, QSMEM_BYTES) != cudaSuccess) return -2;
      configured[1] = true;
    }
    gemm_mxfp8_kernel<1><<<grid, 192, QSMEM_BYTES, stream>>>(ta, tb, p);
  } else {
    if (!configured[0]) {
      if (cudaFuncSetAttribute(gemm_mxfp8_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, QSMEM_BYTES) != cudaSuccess) return -2;
      configured[0] = true;
    }
    gemm_mxfp8_kernel<0><<<grid, 192, QSMEM_BYTES, stream>>>(ta, tb, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---- NVFP4 entry points ---------------------------------------------------------------------------------------------
// Bytes of the scale buffer of an operand with `rows` rows and K elements per row (one byte per 16 elements, 128-row chunks).
extern "C" size_t b200_nvfp4_sf_bytes(int rows, int K) { return static_cast<size_t>((rows + 127) / 128) * (K / 64) * 512; }

extern "C" int b200_nvfp4_amax(const void* x, int ld, float* amax, int R, int C, cudaStream_t st) {
  if (R <= 0 || C <= 0) return 0;
  if (ld % 8 || C % 8) return -1;
  const size_t vecs = static_cast<size_t>(R) * (C / 8);
  const int grid = static_cast<int>(vecs / 256 + 1 < 148 * 8 ? vecs / 256 + 1 : 148 * 8);
  nvfp4_amax_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, amax, R, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// mode 0: row-wise (q, sf); 1: column-wise (qT, sfT); 2: both from one read of x.  amax: device pointer to max |x|.
// stochastic: stochastic rounding of the elements (seed selects the random numbers); rht: random Hadamard transform of the
// transposed operand with the signs of sign_mask (its tensor scale then belongs to 4 · amax).
extern "C" int b200_nvfp4_quantize(const void* x, int ld, void* q, void* sf, void* qT, void* sfT, const float* amax, int R, int C,
                                   int mode, cudaStream_t st, int stochastic, unsigned seed, int rht, unsigned sign_mask) {
  if (R <= 0 || C <= 0) return 0;
  if (ld % 8) return -1;
  if (mode == 0) {
    if (C % 256) return -1;
    const long long total = static_cast<long long>(R) * (C / 16);
    const unsigned grid = static_cast<unsigned>((total + 255) / 256);
    if (stochastic)
      nvfp4_quant_rowwise_kernel<true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, amax, R, C, seed);
    else
      nvfp4_quant_rowwise_kernel<false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, (uint8_t*)q, (uint8_t*)sf, amax, R, C, seed);
  } else {
    if (R % 256 || C % 64 || (mode == 2 && C % 256)) return -1;
    const dim3 grid(C / 64, R / 128);
#define QC(RW, SRV, RH)                                                                                                  \
  nvfp4_quant_colwise_kernel<RW, SRV, RH><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, (uint8_t*)qT, (uint8_t*)sfT, \
                                                                (uint8_t*)q, (uint8_t*)sf, amax, R, C, seed, sign_mask)
    const int key = (mode == 2 ? 4 : 0) | (stochastic ? 2 : 0) | (rht ? 1 : 0);
    switch (key) {
      case 0: QC(0, false, false); break;
      case 1: QC(0, false, true); break;
      case 2: QC(0, true, false); break;
      case 3: QC(0, true, true); break;
      case 4: QC(1, false, false); break;
      case 5: QC(1, false, true); break;
      case 6: QC(1, true, false); break;
      default: QC(1, true, true); break;
    }
#undef QC
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// out[M,N] = alpha · scale(amax_a) · scale(amax_b) · A[M,K] · B[N,K]ᵀ with packed e2m1 operands (K elements = K/2 bytes per
// row; row strides lda, ldb in bytes), chunked E4M3 block scales and the two tensors' largest magnitudes in device memory.
extern "C" int b200_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, const float* amax_a,
                               const float* amax_b, void* out, int M, int N, int K, int lda, int ldb, int ldc, float alpha,
                               int out_f32, int accumulate, int num_sms, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % FBK || lda % 16 || ldb % 16 || N % 8) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -5;
    ctx_bound = true;
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_u8(&ta, A, K / 2, M, lda, 128, QBM);
  if (rc) return rc;
  rc = make_tmap_2d_u8(&tb, B, K / 2, N, ldb, 128, QBN);
  if (rc) return rc;
  QGemmParams p{out, (const uint8_t*)sfa, (const uint8_t*)sfb, M, N, K, ldc, alpha, accumulate, status};
  const int tiles = ((M + QBM - 1) / QBM) * ((N + QBN - 1) / QBN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  static bool configured[2] = {false, false};
  if (out_f32) {
    if (!configured[1]) {
      if (cudaFuncSetAttribute(gemm_nvfp4_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FSMEM_BYTES) != cudaSuccess) return -2;
      configured[1] = true;
    }
    gemm_nvfp4_kernel<1><<<grid, 192, FSMEM_BYTES, stream>>>(ta, tb, p, amax_a, amax_b);
  } else {
    if (!configured[0]) {
      if (cudaFuncSetAttribute(gemm_nvfp4_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, FSMEM_BYTES) != cudaSuccess) return -2;
      configured[0] = true;
    }
    gemm_nvfp4_kernel<0><<<grid, 192, FSMEM_BYTES, stream>>>(ta, tb, p, amax_a, amax_b);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
