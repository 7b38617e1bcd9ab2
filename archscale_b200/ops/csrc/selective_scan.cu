// Mamba-1 selective scan, forward and backward, on token-major activations (rows = tokens, channels contiguous).
//   dt_t = softplus(delta_t + bias),  h_t = exp(dt_t·A)·h_{t-1} + dt_t·B_t·u_t,  y_t = C_t·h_t + D·u_t  (·silu(z_t))
// with N = 16 states per channel and an optional per-token reset flag (start of a packed document: h_{t-1} := 0).
//
// Work decomposition: one thread per (batch, channel, state); a warp holds 2 channels × 16 states, a CTA 16 channels.
// Time runs sequentially inside the thread in tiles of 64 steps that the CTA stages through shared memory with
// 32-byte row segments; sums over the 16 states use a 15-shuffle "reduce-scatter" per 16 steps (lane n ends up with
// the total of step n), so the recurrence itself is one FMA per step and everything else has ILP across steps.
// The forward stores the state entering every 32-step half tile (fp32, L/32 × Di × 16); the backward walks the halves
// in reverse, recomputes the 32 states of a half into registers and runs the adjoint recurrence
//   G_t = C_t·dy'_t + a_{t+1}·G_{t+1}
// dB/dC (sums over channels) are reduced over the CTA's 16 channels in shared memory, written as per-CTA partial
// sums and summed over channel blocks by a second kernel (deterministic, no atomics).
#include "sm100.cuh"
#include "api.h"

namespace b200 {

constexpr int SS_T = 64;    // steps per tile (= checkpoint interval)
constexpr int SS_C = 16;    // channels per CTA
constexpr int SS_N = 16;    // states per channel
constexpr float SS_LOG2E = 1.4426950408889634f;

template <typename T> __device__ __forceinline__ float ld1(const T* p);
template <> __device__ __forceinline__ float ld1<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st1(T* p, float v);
template <> __device__ __forceinline__ void st1<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float ss_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float ss_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }

// v[s] (s = 0..15) summed over the 16 lanes of a half warp; lane n returns the total of step n.
__device__ __forceinline__ float treduce16(float (&v)[16], int n) {
#pragma unroll
  for (int w = 8; w >= 1; w >>= 1) {
    const bool hi = (n & w) != 0;
#pragma unroll
    for (int k = 0; k < w; ++k) {
      const float send = hi ? v[k] : v[k + w];
      const float keep = hi ? v[k + w] : v[k];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, w);
    }
  }
  return v[0];
}

template <typename T>
__global__ void __launch_bounds__(256)
sscan_fwd_kernel(const T* __restrict__ u, int su, const T* __restrict__ delta, int sd, const float* __restrict__ A,
                 const T* __restrict__ Bm, int sB, const T* __restrict__ Cm, int sC, const float* __restrict__ Dp,
                 const T* __restrict__ z, int sz, const float* __restrict__ dbias, const int* __restrict__ reset,
                 T* __restrict__ y, float* __restrict__ ckpt, int L, int Di, int softplus) {
  __shared__ float s_dt[SS_T][SS_C], s_dtu[SS_T][SS_C], s_B[SS_T][SS_N], s_C[SS_T][SS_N], s_y[SS_T][SS_C];
  __shared__ int s_reset[SS_T];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int cl = 2 * w + (lane >> 4), n = lane & 15;
  const int d0 = blockIdx.x * SS_C, b = blockIdx.y, d = d0 + cl;
  const int ci = tid >> 4, cj = tid & 15;           // cooperative mapping: rows ci + 16k, column cj
  const float A2 = A[d * SS_N + n] * SS_LOG2E;
  const float bias_j = dbias ? dbias[d0 + cj] : 0.f, D_j = Dp ? Dp[d0 + cj] : 0.f;
  const int nseg = (L + SS_T - 1) / SS_T;
  const size_t row0 = static_cast<size_t>(b) * L;
  float h = 0.f;
  for (int seg = 0; seg < nseg; ++seg) {
    const int t0 = seg * SS_T;
    float ur[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = ci + 16 * k, t = t0 + i;
      float dt = 0.f, uu = 0.f, bv = 0.f, cv = 0.f;
      if (t < L) {
        const size_t r = row0 + t;
        dt = ld1(delta + r * sd + d0 + cj) + bias_j;
        if (softplus) dt = ss_softplus(dt);
        uu = ld1(u + r * su + d0 + cj);
        bv = ld1(Bm + r * sB + cj);
        cv = ld1(Cm + r * sC + cj);
      }
      ur[k] = uu;
      s_dt[i][cj] = dt; s_dtu[i][cj] = dt * uu; s_B[i][cj] = bv; s_C[i][cj] = cv;
    }
    if (tid < SS_T) s_reset[tid] = (reset && t0 + tid < L) ? reset[row0 + t0 + tid] : 0;
    __syncthreads();
#pragma unroll
    for (int sb = 0; sb < SS_T / 16; ++sb) {
      if ((sb & 1) == 0 && ckpt) ckpt[((static_cast<size_t>(b) * nseg * 2 + seg * 2 + (sb >> 1)) * Di + d) * SS_N + n] = h;
      float p[16];
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        const int i = sb * 16 + s;
        float a = exp2f(s_dt[i][cl] * A2);
        if (s_reset[i]) a = 0.f;
        h = a * h + s_dtu[i][cl] * s_B[i][n];
        p[s] = h * s_C[i][n];
      }
      const float tot = treduce16(p, n);
      s_y[sb * 16 + n][cl] = tot;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = ci + 16 * k, t = t0 + i;
      if (t < L) {
        const size_t r = row0 + t;
        float yv = s_y[i][cj] + D_j * ur[k];
        if (z) { const float zz = ld1(z + r * sz + d0 + cj); yv *= zz * ss_sigmoid(zz); }
        st1(y + r * Di + d0 + cj, yv);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
sscan_bwd_kernel(const T* __restrict__ dy, int sdy, const T* __restrict__ u, int su, const T* __restrict__ delta, int sd,
                 const float* __restrict__ A, const T* __restrict__ Bm, int sB, const T* __restrict__ Cm, int sC,
                 const float* __restrict__ Dp, const T* __restrict__ z, int sz, const float* __restrict__ dbias,
                 const int* __restrict__ reset, const float* __restrict__ ckpt, T* __restrict__ du, T* __restrict__ ddelta,
                 T* __restrict__ dz, float* __restrict__ dA, float* __restrict__ dBf, float* __restrict__ dCf,
                 float* __restrict__ dD, float* __restrict__ ddbias, int L, int Di, int softplus) {
  extern __shared__ float ss_dyn[];
  typedef float (*Tile)[SS_C];
  Tile s_dt = reinterpret_cast<Tile>(ss_dyn), s_u = s_dt + SS_T, s_dyp = s_u + SS_T, s_B = s_dyp + SS_T, s_C = s_B + SS_T;
  Tile s_ypre = s_C + SS_T, s_ddt = s_ypre + SS_T, s_du = s_ddt + SS_T;
  // per-warp slabs for the channel sums of dB / dC: plain stores, summed over the 8 warps in the tile epilogue
  float (*s_dBw)[SS_T][SS_N] = reinterpret_cast<float (*)[SS_T][SS_N]>(s_du + SS_T);
  float (*s_dCw)[SS_T][SS_N] = s_dBw + 8;
  int* s_reset = reinterpret_cast<int*>(s_dCw + 8);
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int cl = 2 * w + (lane >> 4), n = lane & 15;
  const int d0 = blockIdx.x * SS_C, b = blockIdx.y, d = d0 + cl;
  const int ci = tid >> 4, cj = tid & 15;
  const float Araw = A[d * SS_N + n], A2 = Araw * SS_LOG2E;
  const float bias_j = dbias ? dbias[d0 + cj] : 0.f, D_j = Dp ? Dp[d0 + cj] : 0.f;
  const int nseg = (L + SS_T - 1) / SS_T;
  const size_t row0 = static_cast<size_t>(b) * L;
  float G = 0.f;                 // a_{t+1}·G_{t+1}: adjoint arriving from later steps
  float dA_acc = 0.f, dD_acc = 0.f, dbias_acc = 0.f;
  for (int seg = nseg - 1; seg >= 0; --seg) {
    const int t0 = seg * SS_T;
    float ur[4], sg[4], dyr[4], zr[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = ci + 16 * k, t = t0 + i;
      float dt = 0.f, uu = 0.f, bv = 0.f, cv = 0.f, dyv = 0.f, zz = 0.f, sig = 1.f;
      if (t < L) {
        const size_t r = row0 + t;
        dt = ld1(delta + r * sd + d0 + cj) + bias_j;
        if (softplus) { sig = ss_sigmoid(dt); dt = ss_softplus(dt); }
        uu = ld1(u + r * su + d0 + cj);
        bv = ld1(Bm + r * sB + cj);
        cv = ld1(Cm + r * sC + cj);
        dyv = ld1(dy + r * sdy + d0 + cj);
        if (z) zz = ld1(z + r * sz + d0 + cj);
      }
      ur[k] = uu; sg[k] = sig; dyr[k] = dyv; zr[k] = zz;
      s_dt[i][cj] = dt; s_u[i][cj] = uu; s_B[i][cj] = bv; s_C[i][cj] = cv;
      s_dyp[i][cj] = z ? dyv * zz * ss_sigmoid(zz) : dyv;
    }
    if (tid < SS_T) s_reset[tid] = (reset && t0 + tid < L) ? reset[row0 + t0 + tid] : 0;
    __syncthreads();
#pragma unroll 1
    for (int half = 1; half >= 0; --half) {      // 32-step halves: the recomputed states of a half fit in registers
      float h = ckpt[((static_cast<size_t>(b) * nseg * 2 + seg * 2 + half) * Di + d) * SS_N + n];
      float hs[32];              // state before each step of the half (0 where the step resets)
#pragma unroll
      for (int sbl = 0; sbl < 2; ++sbl) {
        const int sb = half * 2 + sbl;
        float p[16];
#pragma unroll
        for (int s = 0; s < 16; ++s) {
          const int i = sb * 16 + s;
          const float dt = s_dt[i][cl];
          float a = exp2f(dt * A2);
          if (s_reset[i]) { a = 0.f; h = 0.f; }
          hs[sbl * 16 + s] = h;
          h = a * h + dt * s_u[i][cl] * s_B[i][n];
          p[s] = h * s_C[i][n];
        }
        const float tot = treduce16(p, n);
        s_ypre[sb * 16 + n][cl] = tot;
      }
#pragma unroll
      for (int sbl = 1; sbl >= 0; --sbl) {
        const int sb = half * 2 + sbl;
        float vdt[16], vdu[16];
#pragma unroll
        for (int s = 15; s >= 0; --s) {
          const int i = sb * 16 + s;
          const float dt = s_dt[i][cl], uu = s_u[i][cl], Bv = s_B[i][n], Cv = s_C[i][n], dyp = s_dyp[i][cl];
          float a = exp2f(dt * A2);
          if (s_reset[i]) a = 0.f;
          const float hprev = hs[sbl * 16 + s];
          const float ht = a * hprev + dt * uu * Bv;
          const float g = G + Cv * dyp;
          float vC = dyp * ht, vB = g * dt * uu;
          const float daa = g * hprev * a;
          dA_acc += daa * dt;
          vdt[s] = daa * Araw + g * Bv * uu;
          vdu[s] = g * dt * Bv;
          G = g * a;
          vB += __shfl_xor_sync(0xffffffffu, vB, 16);
          vC += __shfl_xor_sync(0xffffffffu, vC, 16);
          if (lane < 16) { s_dBw[w][i][n] = vB; s_dCw[w][i][n] = vC; }
        }
        const float tdt = treduce16(vdt, n), tdu = treduce16(vdu, n);
        s_ddt[sb * 16 + n][cl] = tdt;
        s_du[sb * 16 + n][cl] = tdu;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int i = ci + 16 * k, t = t0 + i;
      if (t < L) {
        const size_t r = row0 + t;
        const float dyp = z ? dyr[k] * zr[k] * ss_sigmoid(zr[k]) : dyr[k];
        const float dd = s_ddt[i][cj] * sg[k];
        st1(ddelta + r * Di + d0 + cj, dd);
        dbias_acc += dd;
        st1(du + r * Di + d0 + cj, s_du[i][cj] + dyp * D_j);
        dD_acc += dyp * ur[k];
        if (z) {
          const float ypre = s_ypre[i][cj] + D_j * ur[k];
          const float sgz = ss_sigmoid(zr[k]);
          st1(dz + r * Di + d0 + cj, dyr[k] * ypre * sgz * (1.f + zr[k] * (1.f - sgz)));
        }
        float sb = 0.f, sc = 0.f;
#pragma unroll
        for (int ww = 0; ww < 8; ++ww) { sb += s_dBw[ww][i][cj]; sc += s_dCw[ww][i][cj]; }
        // partial sums of this 16-channel block; summed over blocks by sscan_reduce_bc_kernel
        const size_t po = (static_cast<size_t>(blockIdx.x) * gridDim.y * L + r) * SS_N + cj;
        dBf[po] = sb;
        dCf[po] = sc;
      }
    }
    __syncthreads();
  }
  atomicAdd(&dA[d * SS_N + n], dA_acc);
  if (dD) atomicAdd(&dD[d0 + cj], dD_acc);
  if (ddbias) atomicAdd(&ddbias[d0 + cj], dbias_acc);
}

// dB / dC [rows, 16] = Σ over channel blocks of the partial sums [nblk, rows, 16] written by the backward.
template <typename T>
__global__ void __launch_bounds__(256) sscan_reduce_bc_kernel(const float* __restrict__ pB, const float* __restrict__ pC,
                                                             T* __restrict__ dB, T* __restrict__ dC, size_t n, int nblk) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float sb = 0.f, sc = 0.f;
#pragma unroll 4
  for (int k = 0; k < nblk; ++k) { sb += pB[k * n + i]; sc += pC[k * n + i]; }
  st1(dB + i, sb);
  st1(dC + i, sc);
}

constexpr int SS_BWD_SMEM = (8 * SS_T * SS_C + 16 * SS_T * SS_N) * 4 + SS_T * 4;

}  // namespace b200

using namespace b200;

extern "C" int b200_selective_scan_channel_blocks(int Di) { return Di / SS_C; }

extern "C" int b200_selective_scan_ckpt_segments(int L) { return 2 * ((L + SS_T - 1) / SS_T); }

// u, delta, z: rows of `su`, `sd`, `sz` elements; Bm, Cm: [B·L, 16] with row strides sB, sC; y: dense [B, L, Di].
// reset: int32 per token (1 = h is cleared before this step) or null.  ckpt: fp32 [B, 2·ceil(L/64), Di, 16] or null.
extern "C" int b200_selective_scan_fwd(const void* u, int su, const void* delta, int sd, const float* A, const void* Bm, int sB,
                                       const void* Cm, int sC, const float* D, const void* z, int sz, const float* dbias,
                                       const int* reset, void* y, float* ckpt, int dtype, int B, int L, int Di, int softplus,
                                       cudaStream_t st) {
  if (Di % SS_C) return -1;
  if (B * L == 0) return 0;
  dim3 grid(Di / SS_C, B);
  if (dtype == 1)
    sscan_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)u, su, (const __nv_bfloat16*)delta, sd, A,
        (const __nv_bfloat16*)Bm, sB, (const __nv_bfloat16*)Cm, sC, D, (const __nv_bfloat16*)z, sz, dbias, reset,
        (__nv_bfloat16*)y, ckpt, L, Di, softplus);
  else
    sscan_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)u, su, (const float*)delta, sd, A, (const float*)Bm, sB,
        (const float*)Cm, sC, D, (const float*)z, sz, dbias, reset, (float*)y, ckpt, L, Di, softplus);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dA [Di,16], dD [Di], ddbias [Di] are fp32 accumulators that must be zero on entry.  partB / partC: fp32 scratch
// [Di/16, B·L, 16] (fully overwritten); dB / dC: [B·L, 16] in the activation dtype.
extern "C" int b200_selective_scan_bwd(const void* dy, int sdy, const void* u, int su, const void* delta, int sd, const float* A,
                                       const void* Bm, int sB, const void* Cm, int sC, const float* D, const void* z, int sz,
                                       const float* dbias, const int* reset, const float* ckpt, void* du, void* ddelta, void* dz,
                                       float* dA, float* partB, float* partC, void* dB, void* dC, float* dD, float* ddbias,
                                       int dtype, int B, int L, int Di, int softplus, cudaStream_t st) {
  if (Di % SS_C) return -1;
  if (B * L == 0) return 0;
  dim3 grid(Di / SS_C, B);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sscan_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SS_BWD_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(sscan_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SS_BWD_SMEM) != cudaSuccess)
      return -2;
    configured = true;
  }
  const size_t n = static_cast<size_t>(B) * L * SS_N;
  const unsigned rgrid = static_cast<unsigned>((n + 255) / 256);
  if (dtype == 1) {
    sscan_bwd_kernel<__nv_bfloat16><<<grid, 256, SS_BWD_SMEM, st>>>((const __nv_bfloat16*)dy, sdy, (const __nv_bfloat16*)u, su,
        (const __nv_bfloat16*)delta, sd, A, (const __nv_bfloat16*)Bm, sB, (const __nv_bfloat16*)Cm, sC, D,
        (const __nv_bfloat16*)z, sz, dbias, reset, ckpt, (__nv_bfloat16*)du, (__nv_bfloat16*)ddelta, (__nv_bfloat16*)dz, dA,
        partB, partC, dD, ddbias, L, Di, softplus);
    sscan_reduce_bc_kernel<__nv_bfloat16><<<rgrid, 256, 0, st>>>(partB, partC, (__nv_bfloat16*)dB, (__nv_bfloat16*)dC, n, Di / SS_C);
  } else {
    sscan_bwd_kernel<float><<<grid, 256, SS_BWD_SMEM, st>>>((const float*)dy, sdy, (const float*)u, su, (const float*)delta, sd, A,
        (const float*)Bm, sB, (const float*)Cm, sC, D, (const float*)z, sz, dbias, reset, ckpt, (float*)du, (float*)ddelta,
        (float*)dz, dA, partB, partC, dD, ddbias, L, Di, softplus);
    sscan_reduce_bc_kernel<float><<<rgrid, 256, 0, st>>>(partB, partC, (float*)dB, (float*)dC, n, Di / SS_C);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
