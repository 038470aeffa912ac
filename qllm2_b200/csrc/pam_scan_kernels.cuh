// fp32-math kernels of the chunked PAM scan (forward + backward), CUDA-core FFMA.
//
// These serve the complex64 path, where tensor cores cannot meet the 1e-4 bar (tcgen05 offers
// tf32/bf16 inputs only), and accept bf16 token tensors as well (fp32 accumulate).
//
// Pipeline (every sequence is tiled into chunks of CH = 64 tokens):
//   k_chunk_outer  (mode STATE)  U_c   = sum_s D[last,s] v_s (x) conj(k_s)          chunk-parallel
//   k_state_scan   (forward)     S_c+1 = g_c S_c + U_c                               HBM-bound carry
//   k_fwd_chunk                  Y     = (W .* D~) V + sum_k c_k e^{A^k} Q~ S_k^T    chunk-parallel
// backward:
//   k_chunk_outer  (mode DSTATE) G_c   = sum_t conj(c) e^{A_t} dy_t (x) conj(q~_t)
//   k_state_scan   (reverse)     dS_c  = g_c dS_c+1 + G_c
//   k_bwd_chunk                  dq, dk, dv, raw dA_t, dcoef
//   k_dgamma_finalize            dgamma_u = (sum_{t>=u} dA_t) / (gamma_u + eps)
#pragma once
#include "common.cuh"

namespace qpam {

constexpr int NT = 256;       // threads per CTA in the chunk kernels: a 16 x 16 grid
constexpr int KMAX = QPAM_MAX_STATES;
constexpr int XS = CH + 1;    // row stride (float2) of a [CH][CH] tile

// acc[r][c] += sum_kk opA(A[m_r, kk]) * opB(B[n_c, kk]),  m_r = ty + 16 r,  n_c = tx + 16 c.
// A(m,kk) = A[m*sAm + kk*sAk], B(n,kk) = B[n*sBn + kk*sBk] (float2 units).  All tiles are kept
// with an odd row stride so both the row-major and the transposed walks are bank-conflict free.
template <int RM, int RN, bool CA, bool CB>
__device__ __forceinline__ void cgemm(float2 (&acc)[RM][RN], const float2* __restrict__ A, int sAm,
                                      int sAk, const float2* __restrict__ B, int sBn, int sBk,
                                      int kdim, int ty, int tx) {
  const float2* a0 = A + ty * sAm;
  const float2* b0 = B + tx * sBn;
#pragma unroll 2
  for (int kk = 0; kk < kdim; ++kk) {
    float2 a[RM], b[RN];
#pragma unroll
    for (int r = 0; r < RM; ++r) a[r] = a0[r * 16 * sAm + kk * sAk];
#pragma unroll
    for (int c = 0; c < RN; ++c) b[c] = b0[c * 16 * sBn + kk * sBk];
#pragma unroll
    for (int r = 0; r < RM; ++r)
#pragma unroll
      for (int c = 0; c < RN; ++c) cfma<CA, CB>(acc[r][c], a[r], b[c]);
  }
}

template <int RM, int RN>
__device__ __forceinline__ void czero(float2 (&acc)[RM][RN]) {
#pragma unroll
  for (int r = 0; r < RM; ++r)
#pragma unroll
    for (int c = 0; c < RN; ++c) acc[r][c] = make_float2(0.f, 0.f);
}

// Load a [CH][D] complex token tile into shared memory (row stride D+1 float2), rows >= len
// zeroed, every element multiplied by `scale`.
template <int D, typename T>
__device__ __forceinline__ void load_tile(float2* dst, const T* __restrict__ src, int len, float scale,
                                          int tid) {
  constexpr int LD = D + 1;
  for (int e = tid; e < CH * D; e += NT) {
    const int t = e / D, j = e - t * D;
    float2 x = make_float2(0.f, 0.f);
    if (t < len) {
      x = IO<T>::ld2(src + ((size_t)t * D + j) * 2);
      x.x *= scale;
      x.y *= scale;
    }
    dst[t * LD + j] = x;
  }
}

// Inclusive cumulative sum of a_t = log(gamma_t + eps) over one chunk, done by one warp
// (two tokens per lane).  Tokens >= len contribute 0, so A[CH-1] is the chunk total.
__device__ __forceinline__ void warp_chunk_cumsum(float* A, const float* __restrict__ gamma, int len,
                                                  float eps, int lane) {
  const int t = 2 * lane;
  const float x0 = (t < len) ? logf(gamma[t] + eps) : 0.f;
  const float x1 = (t + 1 < len) ? logf(gamma[t + 1] + eps) : 0.f;
  const float s = x0 + x1;
  float incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  const float excl = incl - s;
  A[t] = excl + x0;
  A[t + 1] = excl + x0 + x1;
}

struct ScanParams {
  const void *q, *k, *v, *dy;
  const float* gamma;   // [K,B,H,T]
  const float* coef;    // [K,B,H,T,2] or null
  void *y, *dq, *dk, *dv;
  float* dgamma;        // [K,B,H,T] (raw dA first, finalised in place)
  float* dA_k;          // tensor-core backward: Re<k_t, dk_t> per token [B,H,T] (the dq and dk kernels may overlap)
  float* dcoef;         // [K,B,H,T,2] or null
  float2* states;       // [K,H,nslots,D,D]
  float2* dstates;      // [K,H,nslots,D,D]
  float* chunk_decay;   // [K,H,nslots]; entry slot0+c+1 = total decay of chunk c
  const float* s0;      // [K,S,H,D,D,2] or null
  float* s_final;       // same or null
  const float* ds_final;
  float* ds0;
  ChunkGeom geom;
  int64_t nslots;
  int32_t B, H, T, K;
  float q_scale, eps;
  int32_t y_token_major;   // tensor-core forward kernels only: y laid out [B,T,H,d,2] instead of [B,H,T,d,2]
};

__device__ __forceinline__ size_t token_base(const ScanParams& p, int b, int h, int t, int D) {
  return (((size_t)b * p.H + h) * p.T + t) * (size_t)D * 2;
}
__device__ __forceinline__ size_t gamma_base(const ScanParams& p, int k, int b, int h, int t) {
  return (((size_t)k * p.B + b) * p.H + h) * p.T + t;
}
__device__ __forceinline__ size_t state_base(const ScanParams& p, int k, int h, int64_t slot, int D) {
  return (((size_t)k * p.H + h) * p.nslots + slot) * (size_t)(D * D);
}

// ---------------------------------------------------------------------------------------------
// Chunk-local outer-product sums.  grid = (chunks, H, K).
//   DSTATE == false:  U[i][j] = sum_s w_s v_s[i] conj(k_s[j]),  w_s = exp(min(0, A_last - A_s));
//                     stored in state slot c+1, chunk decay exp(A_last) recorded.
//   DSTATE == true :  G[i][j] = sum_t f_t dy_t[i] conj(q~_t[j]), f_t = conj(c_t) exp(A_t);
//                     stored in dstate slot c.
// ---------------------------------------------------------------------------------------------
template <int D, typename T, bool DSTATE>
__global__ void __launch_bounds__(NT) k_chunk_outer(ScanParams p) {
  constexpr int LD = D + 1, RD = D / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* Xs = reinterpret_cast<float2*>(smem_raw);   // [CH][LD]  v (or dy), row-weighted
  float2* Ys = Xs + CH * LD;                           // [CH][LD]  k (or q~)
  float* A = reinterpret_cast<float*>(Ys + CH * LD);   // [CH]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y, k = blockIdx.z;
  if (tid < 32) warp_chunk_cumsum(A, p.gamma + gamma_base(p, k, L.b, h, L.t0), L.len, p.eps, tid);
  const size_t tb = token_base(p, L.b, h, L.t0, D);
  const T* xsrc = reinterpret_cast<const T*>(DSTATE ? p.dy : p.v) + tb;
  const T* ysrc = reinterpret_cast<const T*>(DSTATE ? p.q : p.k) + tb;
  load_tile<D, T>(Xs, xsrc, L.len, 1.f, tid);
  load_tile<D, T>(Ys, ysrc, L.len, DSTATE ? p.q_scale : 1.f, tid);
  __syncthreads();
  const float a_last = A[CH - 1];
  // weight the rows of X
  for (int e = tid; e < CH * D; e += NT) {
    const int t = e / D, j = e - t * D;
    float2 x = Xs[t * LD + j];
    if (DSTATE) {
      float2 c = make_float2(1.f, 0.f);
      if (p.coef != nullptr && t < L.len)
        c = *reinterpret_cast<const float2*>(p.coef + gamma_base(p, k, L.b, h, L.t0 + t) * 2);
      const float ea = expf(A[t]);
      x = cmulc(x, c);  // dy * conj(c)
      x.x *= ea;
      x.y *= ea;
    } else {
      const float w = expf(fminf(0.f, a_last - A[t]));
      x.x *= w;
      x.y *= w;
    }
    Xs[t * LD + j] = x;
  }
  __syncthreads();
  float2 acc[RD][RD];
  czero(acc);
  cgemm<RD, RD, false, true>(acc, Xs, 1, LD, Ys, 1, LD, CH, ty, tx);
  const int64_t slot = L.slot0 + L.c + (DSTATE ? 0 : 1);
  float2* dst = (DSTATE ? p.dstates : p.states) + state_base(p, k, h, slot, D);
#pragma unroll
  for (int r = 0; r < RD; ++r)
#pragma unroll
    for (int c = 0; c < RD; ++c) dst[(ty + 16 * r) * D + tx + 16 * c] = acc[r][c];
  if (!DSTATE && tid == 0)
    p.chunk_decay[((size_t)k * p.H + h) * p.nslots + L.slot0 + L.c + 1] = expf(a_last);
}

// ---------------------------------------------------------------------------------------------
// Inter-chunk carry: a first-order linear recurrence over the chunk axis, element-wise over the
// d x d complex state.  Pure HBM streaming: every thread owns one float4 (two complex entries),
// reads U_c, applies S <- g_c S + U_c and writes S back to the same slot.  Loads of the next
// chunks do not depend on the recurrence, so they are issued ahead of the FMA chain.
// grid = (S, H*K, ceil(D*D/2/256)).  REVERSE runs the adjoint recurrence for the backward pass.
// ---------------------------------------------------------------------------------------------
template <bool REVERSE>
__global__ void __launch_bounds__(256) k_state_scan(ScanParams p, int D) {
  const int seq = blockIdx.x;
  const int hk = blockIdx.y;
  const int k = hk / p.H, h = hk - k * p.H;
  const int e4 = blockIdx.z * 256 + threadIdx.x;  // float4 index within the D*D*2 floats
  const int n4 = D * D / 2;
  if (e4 >= n4) return;
  int64_t slot0;
  int nc;
  if (p.geom.cu_seqlens == nullptr) {
    nc = p.geom.nc_uniform;
    slot0 = (int64_t)seq * (nc + 1);
  } else {
    nc = p.geom.chunk_prefix[seq + 1] - p.geom.chunk_prefix[seq];
    slot0 = (int64_t)p.geom.chunk_prefix[seq] + seq;
  }
  float4* st = reinterpret_cast<float4*>((REVERSE ? p.dstates : p.states) + state_base(p, k, h, slot0, D)) + e4;
  const float* dec = p.chunk_decay + ((size_t)k * p.H + h) * p.nslots + slot0;
  const size_t ext = ((((size_t)k * p.geom.S + seq) * p.H + h) * (size_t)(D * D)) / 2 + e4;  // float4 units
  const float* init = REVERSE ? p.ds_final : p.s0;
  float4 cur = make_float4(0.f, 0.f, 0.f, 0.f);
  if (init != nullptr) cur = reinterpret_cast<const float4*>(init)[ext];
  constexpr int UN = 4;
  if (!REVERSE) {
    st[0] = cur;
    for (int c = 0; c < nc; c += UN) {
      float4 u[UN];
      float g[UN];
#pragma unroll
      for (int i = 0; i < UN; ++i)
        if (c + i < nc) {
          u[i] = st[(size_t)(c + i + 1) * n4];
          g[i] = dec[c + i + 1];
        }
#pragma unroll
      for (int i = 0; i < UN; ++i)
        if (c + i < nc) {
          cur.x = fmaf(g[i], cur.x, u[i].x);
          cur.y = fmaf(g[i], cur.y, u[i].y);
          cur.z = fmaf(g[i], cur.z, u[i].z);
          cur.w = fmaf(g[i], cur.w, u[i].w);
          st[(size_t)(c + i + 1) * n4] = cur;
        }
    }
    if (p.s_final != nullptr) reinterpret_cast<float4*>(p.s_final)[ext] = cur;
  } else {
    st[(size_t)nc * n4] = cur;
    for (int c = nc - 1; c >= 0; c -= UN) {
      float4 u[UN];
      float g[UN];
#pragma unroll
      for (int i = 0; i < UN; ++i)
        if (c - i >= 0) {
          u[i] = st[(size_t)(c - i) * n4];
          g[i] = dec[c - i + 1];
        }
#pragma unroll
      for (int i = 0; i < UN; ++i)
        if (c - i >= 0) {
          cur.x = fmaf(g[i], cur.x, u[i].x);
          cur.y = fmaf(g[i], cur.y, u[i].y);
          cur.z = fmaf(g[i], cur.z, u[i].z);
          cur.w = fmaf(g[i], cur.w, u[i].w);
          st[(size_t)(c - i) * n4] = cur;
        }
    }
    if (p.ds0 != nullptr) reinterpret_cast<float4*>(p.ds0)[ext] = cur;
  }
}

}  // namespace qpam
