// Intra-chunk part of the SSD (Mamba-2) scan, forward and backward, without materialising the per-head 64×64 weight tensors:
//     Y[i, p] = Σ_{j ≤ i, same document} CB[i, j] · exp(cs_i − cs_j) · dt_j · X[j, p]
// per (batch, chunk, head), with CB = C·Bᵀ of the chunk (shared by the heads of a group), cs the inclusive cumulative log-decay
// inside the chunk.  In the reference this is the chunk-scan part of `mamba_chunk_scan_combined` (`lit_gpt/mamba2.py:289-305`);
// as PyTorch ops it is a chain of broadcast / mask / exp / multiply passes over [B, chunks, H, 64, 64] fp32 tensors (268 MB each
// at B8 L4096 H32) plus operand permutes around a batched matmul.
//
// The work is small (2·64·64·P FLOP per problem, ≈ 9 GFLOP per pass at that size), so these are plain fp32 CUDA-core kernels
// with the 64×64 weight matrix and the 64×P operand tile in shared memory:
//   forward   one CTA per (chunk, head, batch): M = CB ∘ E ∘ dt_j (E the masked decay), Y = M·X
//   backward  `hsplit` CTAs per (chunk, group, batch), each looping over its share of the group's heads so that its part of
//             dCB (a sum over heads; the parts are added by the caller) stays in registers:  dM = dY·Xᵀ (masked),  dX = Mᵀ·dY,
//             dCB += dM ∘ E ∘ dt_j,  dcs_i = Σ_j dM∘M − Σ_i' (dM∘M)[i', i],  ddt_j = Σ_i dM ∘ CB ∘ E
// Layouts: x, y, dy, dx [B, Lp, H, P] (x bf16 or fp32 → templated; y, dy, dx fp32), dt [B, Lp, H] fp32, cs and dcs [B, nC, H, 64],
// ddt [B, nC, H, 64], CB [B, nC, G, 64, 64] and dCB parts [B, nC, G, hsplit, 64, 64] fp32, bc [B, nC, 64] int32 (document breaks so far inside the chunk) or null.
// Lp = nC·64; P a multiple of 64.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "api.h"

namespace b200 {

constexpr int SI_C = 64;

template <typename T> __device__ __forceinline__ float si_ld(const T* p);
template <> __device__ __forceinline__ float si_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float si_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// shared: sM[64][65], sX[64][64], s_cs[64], s_dt[64], s_bc[64]
template <typename TX>
__global__ void __launch_bounds__(256) ssd_intra_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ dt,
                                                           const float* __restrict__ cs, const float* __restrict__ CB,
                                                           const int* __restrict__ bc, float* __restrict__ y, int nC, int H, int G,
                                                           int P) {
  __shared__ float sM[SI_C][SI_C + 1];
  __shared__ float sX[SI_C][SI_C];
  __shared__ float s_cs[SI_C], s_dt[SI_C];
  __shared__ int s_bc[SI_C];
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z, g = h / (H / G);
  const int tid = threadIdx.x;
  const size_t Lp = static_cast<size_t>(nC) * SI_C;
  const size_t tok0 = static_cast<size_t>(b) * Lp + static_cast<size_t>(n) * SI_C;
  if (tid < SI_C) {
    s_cs[tid] = cs[((static_cast<size_t>(b) * nC + n) * H + h) * SI_C + tid];
    s_dt[tid] = dt[(tok0 + tid) * H + h];
    s_bc[tid] = bc ? bc[(static_cast<size_t>(b) * nC + n) * SI_C + tid] : 0;
  }
  __syncthreads();
  const float* cb = CB + ((static_cast<size_t>(b) * nC + n) * G + g) * SI_C * SI_C;
  for (int e = tid; e < SI_C * SI_C; e += 256) {
    const int i = e >> 6, j = e & 63;
    float m = 0.f;
    if (j <= i && s_bc[i] == s_bc[j]) m = cb[e] * __expf(s_cs[i] - s_cs[j]) * s_dt[j];
    sM[i][j] = m;
  }
  const int ti = tid >> 4, tp = tid & 15;                  // 4 rows × 4 columns per thread
  for (int p0 = 0; p0 < P; p0 += SI_C) {
    __syncthreads();
    for (int e = tid; e < SI_C * SI_C; e += 256) {
      const int j = e >> 6, p = e & 63;
      sX[j][p] = si_ld(x + ((tok0 + j) * H + h) * P + p0 + p);
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
    const int jmax = ti * 4 + 3;                           // lower-triangular: nothing beyond the block's last row
    for (int j = 0; j <= jmax; ++j) {
      const float4 xv = *reinterpret_cast<const float4*>(&sX[j][tp * 4]);
      float mv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) mv[a] = sM[ti * 4 + a][j];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        acc[a][0] = fmaf(mv[a], xv.x, acc[a][0]); acc[a][1] = fmaf(mv[a], xv.y, acc[a][1]);
        acc[a][2] = fmaf(mv[a], xv.z, acc[a][2]); acc[a][3] = fmaf(mv[a], xv.w, acc[a][3]);
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
      *reinterpret_cast<float4*>(y + ((tok0 + ti * 4 + a) * H + h) * P + p0 + tp * 4) =
          make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
  }
}

// shared: sM (M, then reused), sW (dM), sX, sDY tiles
template <typename TX>
__global__ void __launch_bounds__(256) ssd_intra_bwd_kernel(const TX* __restrict__ x, const float* __restrict__ dt,
                                                           const float* __restrict__ cs, const float* __restrict__ CB,
                                                           const int* __restrict__ bc, const float* __restrict__ dy,
                                                           float* __restrict__ dx, float* __restrict__ ddt, float* __restrict__ dcs,
                                                           float* __restrict__ dCB, int nC, int H, int G, int P, int hsplit) {
  extern __shared__ float si_dyn[];
  float (*sM)[SI_C + 1] = reinterpret_cast<float (*)[SI_C + 1]>(si_dyn);                 // M = CB∘E∘dt_j
  float (*sW)[SI_C + 1] = sM + SI_C;                                                     // dM (masked)
  float (*sX)[SI_C] = reinterpret_cast<float (*)[SI_C]>(&sW[SI_C][0]);
  float (*sDY)[SI_C] = sX + SI_C;
  float* s_cs = &sDY[SI_C][0];
  float* s_dt = s_cs + SI_C;
  int* s_bc = reinterpret_cast<int*>(s_dt + SI_C);
  // blockIdx.y = group · hsplit + part: the heads of a group are dealt to `hsplit` CTAs, each writes its own partial dCB
  const int n = blockIdx.x, g = blockIdx.y / hsplit, part = blockIdx.y % hsplit, b = blockIdx.z, rep = H / G;
  const int tid = threadIdx.x;
  const int ti = tid >> 4, tp = tid & 15;
  const size_t Lp = static_cast<size_t>(nC) * SI_C;
  const size_t tok0 = static_cast<size_t>(b) * Lp + static_cast<size_t>(n) * SI_C;
  const float* cb = CB + ((static_cast<size_t>(b) * nC + n) * G + g) * SI_C * SI_C;
  if (tid < SI_C) s_bc[tid] = bc ? bc[(static_cast<size_t>(b) * nC + n) * SI_C + tid] : 0;
  float dcb_acc[16];                                       // entries e = tid + 256·q of the 64×64 matrix
#pragma unroll
  for (int q = 0; q < 16; ++q) dcb_acc[q] = 0.f;
  for (int r = part; r < rep; r += hsplit) {
    const int h = g * rep + r;
    __syncthreads();
    if (tid < SI_C) {
      s_cs[tid] = cs[((static_cast<size_t>(b) * nC + n) * H + h) * SI_C + tid];
      s_dt[tid] = dt[(tok0 + tid) * H + h];
    }
    __syncthreads();
    for (int e = tid; e < SI_C * SI_C; e += 256) {
      const int i = e >> 6, j = e & 63;
      float m = 0.f;
      if (j <= i && s_bc[i] == s_bc[j]) m = cb[e] * __expf(s_cs[i] - s_cs[j]) * s_dt[j];
      sM[i][j] = m;
      sW[i][j] = 0.f;
    }
    // dM = Σ_p dY[i, p]·X[j, p] (accumulated over the P blocks), dX = Mᵀ·dY per P block
    float wacc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) wacc[a][c] = 0.f;
    for (int p0 = 0; p0 < P; p0 += SI_C) {
      __syncthreads();
      for (int e = tid; e < SI_C * SI_C; e += 256) {
        const int j = e >> 6, p = e & 63;
        sX[j][p] = si_ld(x + ((tok0 + j) * H + h) * P + p0 + p);
        sDY[j][p] = dy[((tok0 + j) * H + h) * P + p0 + p];
      }
      __syncthreads();
      // this thread's 4×4 block of dM: rows i = 4·ti + a, columns j = 4·tp + c
      if (tp <= ti) {
        for (int p = 0; p < SI_C; p += 4) {
          float4 dv[4], xv[4];
#pragma unroll
          for (int a = 0; a < 4; ++a) dv[a] = *reinterpret_cast<const float4*>(&sDY[ti * 4 + a][p]);
#pragma unroll
          for (int c = 0; c < 4; ++c) xv[c] = *reinterpret_cast<const float4*>(&sX[tp * 4 + c][p]);
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c)
              wacc[a][c] += dv[a].x * xv[c].x + dv[a].y * xv[c].y + dv[a].z * xv[c].z + dv[a].w * xv[c].w;
        }
      }
      // dX[j, p] = Σ_{i ≥ j} M[i, j]·dY[i, p]: rows j = 4·ti + a, columns p = 4·tp + c
      float xacc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) xacc[a][c] = 0.f;
      for (int i = ti * 4; i < SI_C; ++i) {
        const float4 dv = *reinterpret_cast<const float4*>(&sDY[i][tp * 4]);
        float mv[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) mv[a] = sM[i][ti * 4 + a];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          xacc[a][0] = fmaf(mv[a], dv.x, xacc[a][0]); xacc[a][1] = fmaf(mv[a], dv.y, xacc[a][1]);
          xacc[a][2] = fmaf(mv[a], dv.z, xacc[a][2]); xacc[a][3] = fmaf(mv[a], dv.w, xacc[a][3]);
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
        *reinterpret_cast<float4*>(dx + ((tok0 + ti * 4 + a) * H + h) * P + p0 + tp * 4) =
            make_float4(xacc[a][0], xacc[a][1], xacc[a][2], xacc[a][3]);
    }
    __syncthreads();
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < 4; ++c) sW[ti * 4 + a][tp * 4 + c] = wacc[a][c];
    __syncthreads();
    // per-entry products; sW becomes dM∘M (for dcs), dCB and ddt are formed on the fly
    float col_dt = 0.f;                                    // used by threads tid < 64 below
    for (int q = 0; q < 16; ++q) {
      const int e = tid + 256 * q, i = e >> 6, j = e & 63;
      const float m = sM[i][j];                            // zero outside the mask
      const float w = sW[i][j];
      const float ed = (j <= i && s_bc[i] == s_bc[j]) ? __expf(s_cs[i] - s_cs[j]) : 0.f;     // masked decay E
      dcb_acc[q] += w * ed * s_dt[j];
      sM[i][j] = w * cb[e] * ed;                           // dM ∘ CB ∘ E  (column sums → ddt)
      sW[i][j] = w * m;                                    // dM ∘ M       (row sums − column sums → dcs)
    }
    __syncthreads();
    if (tid < SI_C) {
      float row = 0.f, col = 0.f;
      for (int jj = 0; jj < SI_C; ++jj) { row += sW[tid][jj]; col += sW[jj][tid]; col_dt += sM[jj][tid]; }
      dcs[((static_cast<size_t>(b) * nC + n) * H + h) * SI_C + tid] = row - col;
      ddt[((static_cast<size_t>(b) * nC + n) * H + h) * SI_C + tid] = col_dt;
    }
  }
  float* out = dCB + (((static_cast<size_t>(b) * nC + n) * G + g) * hsplit + part) * SI_C * SI_C;
#pragma unroll
  for (int q = 0; q < 16; ++q) out[tid + 256 * q] = dcb_acc[q];
}

constexpr int SI_BWD_SMEM = (2 * SI_C * (SI_C + 1) + 2 * SI_C * SI_C + 2 * SI_C) * 4 + SI_C * 4;

}  // namespace b200

// x_dtype: 0 fp32, 1 bf16.  See the top of the file for the layouts.
extern "C" int b200_ssd_intra_fwd(const void* x, int x_dtype, const float* dt, const float* cs, const float* CB, const int* bc,
                                  float* y, int B, int nC, int H, int G, int P, cudaStream_t st) {
  using namespace b200;
  if (B <= 0 || nC <= 0) return 0;
  if (P % SI_C || H % G) return -1;
  const dim3 grid(nC, H, B);
  if (x_dtype == 1)
    ssd_intra_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), dt, cs, CB, bc, y, nC, H, G, P);
  else
    ssd_intra_fwd_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), dt, cs, CB, bc, y, nC, H, G, P);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_ssd_intra_bwd(const void* x, int x_dtype, const float* dt, const float* cs, const float* CB, const int* bc,
                                  const float* dy, float* dx, float* ddt, float* dcs, float* dCB, int B, int nC, int H, int G,
                                  int P, int hsplit, cudaStream_t st) {
  using namespace b200;
  if (B <= 0 || nC <= 0) return 0;
  if (P % SI_C || H % G || hsplit < 1 || (H / G) % hsplit) return -1;
  const dim3 grid(nC, G * hsplit, B);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ssd_intra_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SI_BWD_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(ssd_intra_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SI_BWD_SMEM) != cudaSuccess)
      return -2;
    configured = true;
  }
  if (x_dtype == 1)
    ssd_intra_bwd_kernel<__nv_bfloat16><<<grid, 256, SI_BWD_SMEM, st>>>(static_cast<const __nv_bfloat16*>(x), dt, cs, CB, bc, dy, dx,
                                                                       ddt, dcs, dCB, nC, H, G, P, hsplit);
  else
    ssd_intra_bwd_kernel<float><<<grid, 256, SI_BWD_SMEM, st>>>(static_cast<const float*>(x), dt, cs, CB, bc, dy, dx, ddt, dcs, dCB,
                                                               nC, H, G, P, hsplit);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
