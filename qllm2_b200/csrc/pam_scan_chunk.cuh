// Chunk-parallel output (forward) and gradient (backward) kernels of the fp32-math PAM scan.
#pragma once
#include "pam_scan_kernels.cuh"

namespace qpam {

// Shared bookkeeping of a chunk: per-state cumulative log-decays and read-out coefficients.
//   A[k][t]  = sum_{u<=t} log(gamma^k_u + eps)   (tokens >= len add 0)
//   cf[k][t] = coef_{k,t}  (1 when coef == nullptr, 0 for tokens >= len)
__device__ __forceinline__ void load_decay_coef(const ScanParams& p, const ChunkLoc& L, int h, float* A,
                                                float2* cf, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  for (int k = warp; k < p.K; k += NT / 32)
    warp_chunk_cumsum(A + k * CH, p.gamma + gamma_base(p, k, L.b, h, L.t0), L.len, p.eps, lane);
  for (int e = tid; e < p.K * CH; e += NT) {
    const int k = e / CH, t = e - k * CH;
    float2 c = make_float2(0.f, 0.f);
    if (t < L.len) {
      c = make_float2(1.f, 0.f);
      if (p.coef != nullptr)
        c = *reinterpret_cast<const float2*>(p.coef + gamma_base(p, k, L.b, h, L.t0 + t) * 2);
    }
    cf[e] = c;
  }
}

template <int D>
__device__ __forceinline__ void load_state(float2* dst, const float2* __restrict__ src, int tid) {
  constexpr int LD = D + 1;
  for (int e = tid; e < D * D; e += NT) {
    const int i = e / D, j = e - i * D;
    dst[i * LD + j] = src[e];
  }
}

template <int D>
constexpr size_t fwd_chunk_smem() {
  return sizeof(float2) * (3 * CH * (D + 1) + CH * XS) + sizeof(float) * KMAX * CH + sizeof(float2) * KMAX * CH;
}

// ---------------------------------------------------------------------------------------------
// Forward output of one chunk.  grid = (chunks, H).
//   W = Q~ K^H,  M = W .* D~,  D~[t,s] = sum_k c_{k,t} exp(min(0, A^k_t - A^k_s))  (s <= t)
//   Y = M V + sum_k c_{k,t} exp(A^k_t) (Q~ S_k^T)        S_k = state before the chunk
// ---------------------------------------------------------------------------------------------
template <int D, typename T>
__global__ void __launch_bounds__(NT) k_fwd_chunk(ScanParams p) {
  constexpr int LD = D + 1, RD = D / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* Qs = reinterpret_cast<float2*>(smem_raw);
  float2* Ks = Qs + CH * LD;
  float2* Vs = Ks + CH * LD;
  float2* X = Vs + CH * LD;                                   // [CH][XS] or [D][LD]
  float* A = reinterpret_cast<float*>(X + CH * XS);           // [KMAX][CH]
  float2* cf = reinterpret_cast<float2*>(A + KMAX * CH);      // [KMAX][CH]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  load_decay_coef(p, L, h, A, cf, tid);
  const size_t tb = token_base(p, L.b, h, L.t0, D);
  load_tile<D, T>(Qs, reinterpret_cast<const T*>(p.q) + tb, L.len, p.q_scale, tid);
  load_tile<D, T>(Ks, reinterpret_cast<const T*>(p.k) + tb, L.len, 1.f, tid);
  load_tile<D, T>(Vs, reinterpret_cast<const T*>(p.v) + tb, L.len, 1.f, tid);
  __syncthreads();
  {
    float2 w[4][4];
    czero(w);
    cgemm<4, 4, false, true>(w, Qs, LD, 1, Ks, LD, 1, D, ty, tx);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int t = ty + 16 * r, s = tx + 16 * c;
        float2 dt = make_float2(0.f, 0.f);
        if (s <= t)
          for (int k = 0; k < p.K; ++k) {
            const float dk = expf(fminf(0.f, A[k * CH + t] - A[k * CH + s]));
            const float2 c_ = cf[k * CH + t];
            dt.x = fmaf(c_.x, dk, dt.x);
            dt.y = fmaf(c_.y, dk, dt.y);
          }
        X[t * XS + s] = cmul(w[r][c], dt);
      }
  }
  __syncthreads();
  float2 acc[4][RD];
  czero(acc);
  cgemm<4, RD, false, false>(acc, X, XS, 1, Vs, 1, LD, CH, ty, tx);
  if (L.c > 0 || p.s0 != nullptr) {
    for (int k = 0; k < p.K; ++k) {
      __syncthreads();
      load_state<D>(X, p.states + state_base(p, k, h, L.slot0 + L.c, D), tid);
      __syncthreads();
      float2 t2[4][RD];
      czero(t2);
      cgemm<4, RD, false, false>(t2, Qs, LD, 1, X, LD, 1, D, ty, tx);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int t = ty + 16 * r;
        const float2 f = cscale(cf[k * CH + t], expf(A[k * CH + t]));
#pragma unroll
        for (int c = 0; c < RD; ++c) {
          const float2 m = cmul(f, t2[r][c]);
          acc[r][c].x += m.x;
          acc[r][c].y += m.y;
        }
      }
    }
  }
  T* y = reinterpret_cast<T*>(p.y) + tb;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = ty + 16 * r;
    if (t < L.len)
#pragma unroll
      for (int c = 0; c < RD; ++c) IO<T>::st2(y + ((size_t)t * D + tx + 16 * c) * 2, acc[r][c]);
  }
}

template <int D>
constexpr size_t bwd_chunk_smem() {
  return sizeof(float2) * (4 * CH * (D + 1) + 2 * CH * XS)   // Q K V dY, X, Z
         + sizeof(float) * KMAX * CH                          // A
         + sizeof(float2) * KMAX * CH                         // cf
         + sizeof(float2) * KMAX * CH                         // dcI
         + sizeof(float) * KMAX * CH                          // col
         + sizeof(float) * 8 * KMAX * CH;                     // per-warp column partials
}

// 16-lane (half-warp) sum; all 32 lanes take part, lanes with equal (lane & 16) form a group.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------------------
// Backward of one chunk.  grid = (chunks, H).  With P = dY V^H, cwp = conj(W) .* P:
//   dcI_k[t]  = sum_s D_k[t,s] cwp[t,s]                 (+ <dy_t, Yinter^k_t> below)
//   col_k[s]  = sum_t D_k[t,s] Re(conj(c_{k,t}) cwp[t,s])  (+ Re<v_s, dv^{k,state}_s> below)
//   M = W .* D~,  Z = conj(D~) .* P
//   dV = M^H dY + sum_k D_k[last,s] K dS_k^T      dQ~ = Z K + sum_k conj(c_k) e^{A^k} dY conj(S_k)
//   dK = Z^H Q~ + sum_k D_k[last,s] V conj(dS_k)
//   dA^k_t = Re(conj(c_{k,t}) dcI_k[t]) - col_k[t]      (raw; reverse-cumsummed afterwards)
// S_k: state before the chunk; dS_k: gradient reaching the state after the chunk.
// ---------------------------------------------------------------------------------------------
template <int D, typename T>
__global__ void __launch_bounds__(NT) k_bwd_chunk(ScanParams p) {
  constexpr int LD = D + 1, RD = D / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* Qs = reinterpret_cast<float2*>(smem_raw);
  float2* Ks = Qs + CH * LD;
  float2* Vs = Ks + CH * LD;
  float2* Gs = Vs + CH * LD;
  float2* X = Gs + CH * LD;
  float2* Z = X + CH * XS;
  float* A = reinterpret_cast<float*>(Z + CH * XS);
  float2* cf = reinterpret_cast<float2*>(A + KMAX * CH);
  float2* dcI = cf + KMAX * CH;
  float* col = reinterpret_cast<float*>(dcI + KMAX * CH);
  float* colp = col + KMAX * CH;  // [8 warps][KMAX][CH]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  load_decay_coef(p, L, h, A, cf, tid);
  const size_t tb = token_base(p, L.b, h, L.t0, D);
  load_tile<D, T>(Qs, reinterpret_cast<const T*>(p.q) + tb, L.len, p.q_scale, tid);
  load_tile<D, T>(Ks, reinterpret_cast<const T*>(p.k) + tb, L.len, 1.f, tid);
  load_tile<D, T>(Vs, reinterpret_cast<const T*>(p.v) + tb, L.len, 1.f, tid);
  load_tile<D, T>(Gs, reinterpret_cast<const T*>(p.dy) + tb, L.len, 1.f, tid);
  __syncthreads();

  // ---- scores, P, and the element-wise pass
  {
    float2 w[4][4], pp[4][4];
    czero(w);
    czero(pp);
    cgemm<4, 4, false, true>(w, Qs, LD, 1, Ks, LD, 1, D, ty, tx);
    cgemm<4, 4, false, true>(pp, Gs, LD, 1, Vs, LD, 1, D, ty, tx);
    float2 dtl[4][4];
    czero(dtl);
    for (int k = 0; k < p.K; ++k) {
      float colsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int t = ty + 16 * r;
        const float2 c_ = cf[k * CH + t];
        const float at = A[k * CH + t];
        float2 rowsum = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int s = tx + 16 * c;
          if (s <= t) {
            const float dk = expf(fminf(0.f, at - A[k * CH + s]));
            const float2 cwp = cmulc(pp[r][c], w[r][c]);  // P * conj(W)
            rowsum.x = fmaf(dk, cwp.x, rowsum.x);
            rowsum.y = fmaf(dk, cwp.y, rowsum.y);
            colsum[c] = fmaf(dk, c_.x * cwp.x + c_.y * cwp.y, colsum[c]);  // Re(conj(c) cwp)
            dtl[r][c].x = fmaf(c_.x, dk, dtl[r][c].x);
            dtl[r][c].y = fmaf(c_.y, dk, dtl[r][c].y);
          }
        }
        rowsum.x = half_warp_sum(rowsum.x);
        rowsum.y = half_warp_sum(rowsum.y);
        if (tx == 0) dcI[k * CH + t] = rowsum;
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float v2 = colsum[c] + __shfl_xor_sync(0xffffffffu, colsum[c], 16);
        if (lane < 16) colp[(warp * KMAX + k) * CH + tx + 16 * c] = v2;
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int t = ty + 16 * r, s = tx + 16 * c;
        X[t * XS + s] = cmul(w[r][c], dtl[r][c]);
        Z[t * XS + s] = cmulc(pp[r][c], dtl[r][c]);  // P * conj(D~)
      }
  }
  __syncthreads();
  for (int e = tid; e < p.K * CH; e += NT) {
    const int k = e / CH, s = e - k * CH;
    float a = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) a += colp[(w8 * KMAX + k) * CH + s];
    col[e] = a;
  }

  // ---- intra-chunk gradient products
  float2 aV[4][RD], aQ[4][RD], aK[4][RD];
  czero(aV);
  czero(aQ);
  czero(aK);
  cgemm<4, RD, true, false>(aV, X, 1, XS, Gs, 1, LD, CH, ty, tx);
  cgemm<4, RD, false, false>(aQ, Z, XS, 1, Ks, 1, LD, CH, ty, tx);
  cgemm<4, RD, true, false>(aK, Z, 1, XS, Qs, 1, LD, CH, ty, tx);

  // ---- inter-chunk terms through the carried state and its gradient
  const bool has_prev = (L.c > 0) || (p.s0 != nullptr);
  const bool has_next = (L.c < L.nc - 1) || (p.ds_final != nullptr);
  for (int k = 0; k < p.K; ++k) {
    if (!has_prev && !has_next) break;
    __syncthreads();
    if (has_prev) load_state<D>(X, p.states + state_base(p, k, h, L.slot0 + L.c, D), tid);
    if (has_next) load_state<D>(Z, p.dstates + state_base(p, k, h, L.slot0 + L.c + 1, D), tid);
    __syncthreads();
    const float a_last = A[k * CH + CH - 1];
    if (has_prev) {
      float2 t2[4][RD];
      czero(t2);
      cgemm<4, RD, false, false>(t2, Qs, LD, 1, X, LD, 1, D, ty, tx);  // Q~ S^T -> [t][i]
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int t = ty + 16 * r;
        const float ea = expf(A[k * CH + t]);
        float2 d = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < RD; ++c) {
          const float2 g = Gs[t * LD + tx + 16 * c];
          const float2 m = cmulc(g, cscale(t2[r][c], ea));  // dy * conj(Yinter)
          d.x += m.x;
          d.y += m.y;
        }
        d.x = half_warp_sum(d.x);
        d.y = half_warp_sum(d.y);
        if (tx == 0) {
          dcI[k * CH + t].x += d.x;
          dcI[k * CH + t].y += d.y;
        }
      }
      czero(t2);
      cgemm<4, RD, false, true>(t2, Gs, LD, 1, X, 1, LD, D, ty, tx);  // dY conj(S) -> [t][j]
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int t = ty + 16 * r;
        const float2 c_ = cf[k * CH + t];
        const float2 f = cscale(make_float2(c_.x, -c_.y), expf(A[k * CH + t]));
#pragma unroll
        for (int c = 0; c < RD; ++c) {
          const float2 m = cmul(f, t2[r][c]);
          aQ[r][c].x += m.x;
          aQ[r][c].y += m.y;
        }
      }
    }
    if (has_next) {
      float2 t2[4][RD];
      czero(t2);
      cgemm<4, RD, false, false>(t2, Ks, LD, 1, Z, LD, 1, D, ty, tx);  // K dS^T -> [s][i]
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int s = ty + 16 * r;
        const float wl = expf(fminf(0.f, a_last - A[k * CH + s]));
        float cs = 0.f;
#pragma unroll
        for (int c = 0; c < RD; ++c) {
          const float2 m = cscale(t2[r][c], wl);
          aV[r][c].x += m.x;
          aV[r][c].y += m.y;
          const float2 vv = Vs[s * LD + tx + 16 * c];
          cs += vv.x * m.x + vv.y * m.y;  // Re(conj(v) dv_state)
        }
        cs = half_warp_sum(cs);
        if (tx == 0) col[k * CH + s] += cs;
      }
      czero(t2);
      cgemm<4, RD, false, true>(t2, Vs, LD, 1, Z, 1, LD, D, ty, tx);  // V conj(dS) -> [s][j]
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int s = ty + 16 * r;
        const float wl = expf(fminf(0.f, a_last - A[k * CH + s]));
#pragma unroll
        for (int c = 0; c < RD; ++c) {
          aK[r][c].x += wl * t2[r][c].x;
          aK[r][c].y += wl * t2[r][c].y;
        }
      }
    }
  }
  __syncthreads();
  // ---- outputs
  for (int e = tid; e < p.K * CH; e += NT) {
    const int k = e / CH, t = e - k * CH;
    if (t < L.len) {
      const float2 c_ = cf[e], d = dcI[e];
      const size_t gi = gamma_base(p, k, L.b, h, L.t0 + t);
      p.dgamma[gi] = (c_.x * d.x + c_.y * d.y) - col[e];
      if (p.dcoef != nullptr) *reinterpret_cast<float2*>(p.dcoef + gi * 2) = d;
    }
  }
  T* dq = reinterpret_cast<T*>(p.dq) + tb;
  T* dk = reinterpret_cast<T*>(p.dk) + tb;
  T* dv = reinterpret_cast<T*>(p.dv) + tb;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = ty + 16 * r;
    if (t < L.len)
#pragma unroll
      for (int c = 0; c < RD; ++c) {
        const size_t o = ((size_t)t * D + tx + 16 * c) * 2;
        IO<T>::st2(dq + o, cscale(aQ[r][c], p.q_scale));
        IO<T>::st2(dk + o, aK[r][c]);
        IO<T>::st2(dv + o, aV[r][c]);
      }
  }
}

// ---------------------------------------------------------------------------------------------
// dgamma_u = (sum_{t >= u, same sequence} dA_t) / (gamma_u + eps), in place.  grid = (S, H, K).
// The suffix sum runs in double so that long sequences do not lose the small terms.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_dgamma_finalize(ScanParams p, int D) {
  __shared__ double wsum[8];
  const int seq = blockIdx.x, h = blockIdx.y, k = blockIdx.z;
  int b = seq, a = 0, e = p.T;
  int64_t slot_last;
  if (p.geom.cu_seqlens != nullptr) {
    b = 0;
    a = p.geom.cu_seqlens[seq];
    e = p.geom.cu_seqlens[seq + 1];
    slot_last = (int64_t)p.geom.chunk_prefix[seq + 1] + seq;
  } else {
    slot_last = (int64_t)seq * (p.geom.nc_uniform + 1) + p.geom.nc_uniform;
  }
  const size_t base = gamma_base(p, k, b, h, 0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double carry = 0.0;
  if (p.ds_final != nullptr) {
    // the total decay of the sequence also scales s_final: dA_last += Re<dS_final, S_final>
    const float* sf = reinterpret_cast<const float*>(p.states + state_base(p, k, h, slot_last, D));
    const float* dsf = p.ds_final + (((size_t)k * p.geom.S + seq) * p.H + h) * (size_t)(D * D) * 2;
    double part = 0.0;
    for (int i = tid; i < D * D * 2; i += 256) part += (double)sf[i] * (double)dsf[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) wsum[warp] = part;
    __syncthreads();
    for (int w8 = 0; w8 < 8; ++w8) carry += wsum[w8];
    __syncthreads();
  }
  for (int end = e; end > a; end -= 256) {
    const int idx = end - 1 - tid;
    double v = (idx >= a) ? (double)p.dgamma[base + idx] : 0.0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    if (lane == 31) wsum[warp] = v;
    __syncthreads();
    double off = 0.0, tot = 0.0;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) {
      if (w8 < warp) off += wsum[w8];
      tot += wsum[w8];
    }
    const double incl = v + off + carry;
    if (idx >= a) p.dgamma[base + idx] = (float)(incl / ((double)p.gamma[base + idx] + (double)p.eps));
    carry += tot;
    __syncthreads();
  }
}

}  // namespace qpam
