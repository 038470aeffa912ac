// fp32-math kernels of the fused tied-head cross-entropy (CUDA-core FFMA).
//
// These serve fp32 inputs (where the 1e-5 loss bar and fp32-exact gradients are wanted) and are
// the fall-through for shapes the tensor-core path does not take.  Vocabulary tiles of 64 columns
// stream through shared memory; each CTA keeps a running (max, sum-exp, arg-max, target logit) per
// row, so logits never reach memory.
#pragma once
#include <math.h>

#include "common.cuh"

namespace qpam {

constexpr int CE_TM = 64, CE_TN = 64, CE_TK = 32, CE_LDS = CE_TK + 1;

struct CEParams {
  const void* h;
  const void* w;
  const int64_t* targets;
  const float* mask;
  int64_t N, V, v_offset, ignore_index;
  int32_t F;
  // partial statistics [nsplit][N]
  float *pm, *ps, *pt, *pbest;
  int32_t* pidx;
  int32_t nsplit, tiles_per_split;
  // probability tiles (backward)
  void* pbuf;
  int64_t ldp, row0, rows;
  const float* lse;
  const float* grad_scale;
  const float* denom;
};

// 64x64 tile of logits z[m][n] = sum_f H[row0+m][f] W[col0+n][f]; thread (ty,tx) owns rows
// ty+16r and columns tx+16c.  Out-of-range rows/columns read as zero.
template <typename T>
__device__ __forceinline__ void logits_tile(float (&acc)[4][4], const T* __restrict__ H, const T* __restrict__ W,
                                            int64_t row0, int64_t nrows, int64_t col0, int64_t ncols, int F,
                                            float* Hs, float* Ws, int tid, int ty, int tx) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  for (int f0 = 0; f0 < F; f0 += CE_TK) {
#pragma unroll
    for (int i = 0; i < CE_TM * CE_TK / 256; ++i) {
      const int e = tid + i * 256, m = e / CE_TK, kk = e - m * CE_TK;
      const bool fk = (f0 + kk) < F;
      Hs[m * CE_LDS + kk] = (fk && row0 + m < nrows) ? IO<T>::ld(H + (row0 + m) * F + f0 + kk) : 0.f;
      Ws[m * CE_LDS + kk] = (fk && col0 + m < ncols) ? IO<T>::ld(W + (col0 + m) * F + f0 + kk) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < CE_TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = Hs[(ty + 16 * r) * CE_LDS + kk];
#pragma unroll
      for (int c = 0; c < 4; ++c) b[c] = Ws[(tx + 16 * c) * CE_LDS + kk];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
    }
    __syncthreads();
  }
}

__device__ __forceinline__ float hw_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float hw_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// (value, index) arg-max over 16 lanes; the lowest index wins ties (torch.argmax on CPU/CUDA
// returns the first maximal element for the sizes used here).
__device__ __forceinline__ void hw_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

// grid = (nsplit, row tiles).  Per-row partial statistics of one vocabulary split.
template <typename T>
__global__ void __launch_bounds__(256) k_ce_partial(CEParams p) {
  __shared__ float Hs[CE_TM * CE_LDS], Ws[CE_TN * CE_LDS];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int split = blockIdx.x;
  const int64_t row0 = (int64_t)blockIdx.y * CE_TM;
  const int64_t nvt = (p.V + CE_TN - 1) / CE_TN;
  const int64_t vt0 = (int64_t)split * p.tiles_per_split;
  const int64_t vt1 = min(nvt, vt0 + p.tiles_per_split);
  float m_run[4], s_run[4], best[4], tz[4];
  int bidx[4];
  int64_t tcol[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m_run[r] = -INFINITY;
    s_run[r] = 0.f;
    best[r] = -INFINITY;
    bidx[r] = 0x7fffffff;
    tz[r] = 0.f;
    const int64_t row = row0 + ty + 16 * r;
    tcol[r] = -1;
    if (row < p.N && p.targets != nullptr) {
      const int64_t t = p.targets[row];
      if (t != p.ignore_index) tcol[r] = t - p.v_offset;
    }
  }
  for (int64_t vt = vt0; vt < vt1; ++vt) {
    const int64_t col0 = vt * CE_TN;
    float z[4][4];
    logits_tile<T>(z, reinterpret_cast<const T*>(p.h), reinterpret_cast<const T*>(p.w), row0, p.N, col0, p.V,
                   p.F, Hs, Ws, tid, ty, tx);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float lm = -INFINITY;
      int li = 0x7fffffff;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int64_t col = col0 + tx + 16 * c;
        if (col < p.V) {
          if (z[r][c] > lm) {  // columns ascend with c, so strict > keeps the lowest index
            lm = z[r][c];
            li = (int)col;
          }
          if (col == tcol[r]) tz[r] = z[r][c];
        }
      }
      hw_argmax(lm, li);
      if (lm > best[r] || (lm == best[r] && li < bidx[r])) {
        best[r] = lm;
        bidx[r] = li;
      }
      const float m_new = fmaxf(m_run[r], lm);
      float se = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (col0 + tx + 16 * c < p.V) se += expf(z[r][c] - m_new);
      se = hw_sum(se);
      s_run[r] = s_run[r] * expf(m_run[r] - m_new) + se;
      m_run[r] = m_new;
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const float t = hw_sum(tz[r]);
    const int64_t row = row0 + ty + 16 * r;
    if (tx == 0 && row < p.N) {
      const size_t o = (size_t)split * p.N + row;
      p.pm[o] = m_run[r];
      p.ps[o] = s_run[r];
      p.pt[o] = t;
      p.pbest[o] = best[r];
      p.pidx[o] = bidx[r];
    }
  }
}

__global__ void k_ce_merge(CEParams p, float* row_max, float* row_sumexp, float* row_tgt, int64_t* row_argmax) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= p.N) return;
  float M = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) M = fmaxf(M, p.pm[(size_t)s * p.N + n]);
  float S = 0.f, tz = 0.f, best = -INFINITY;
  int bi = 0x7fffffff;
  for (int s = 0; s < p.nsplit; ++s) {
    const size_t o = (size_t)s * p.N + n;
    S += p.ps[o] * expf(p.pm[o] - M);
    tz += p.pt[o];
    const float b = p.pbest[o];
    const int i = p.pidx[o];
    if (b > best || (b == best && i < bi)) {
      best = b;
      bi = i;
    }
  }
  if (row_max) row_max[n] = M;
  if (row_sumexp) row_sumexp[n] = S;
  if (row_tgt) row_tgt[n] = tz;
  if (row_argmax) row_argmax[n] = (int64_t)bi + p.v_offset;
}

// Single CTA: lse, per-token loss and the scalar reductions (fixed summation order, double).
__global__ void __launch_bounds__(1024) k_ce_finalize(CEParams p, const float* row_max, const float* row_sumexp,
                                                      const float* row_tgt, const int64_t* row_argmax, float* lse,
                                                      float* per_token, float* loss_sum, float* denom,
                                                      float* correct, float* tokens) {
  __shared__ double red[4][32];
  double a_loss = 0.0, a_den = 0.0, a_cor = 0.0, a_tok = 0.0;
  for (int64_t n = threadIdx.x; n < p.N; n += blockDim.x) {
    const float l = row_max[n] + logf(row_sumexp[n]);
    lse[n] = l;
    const bool valid = p.targets[n] != p.ignore_index;
    const float pt = valid ? (l - row_tgt[n]) : 0.f;
    if (per_token) per_token[n] = pt;
    const float mk = p.mask ? p.mask[n] : 1.f;
    const float tm = p.mask ? p.mask[n] : (valid ? 1.f : 0.f);  // token mask of linear_ce_stats
    a_loss += (double)pt * mk;
    a_den += p.mask ? (double)mk : (valid ? 1.0 : 0.0);
    a_tok += tm;
    if (row_argmax) a_cor += (row_argmax[n] == p.targets[n]) ? (double)tm : 0.0;
  }
  double v[4] = {a_loss, a_den, a_cor, a_tok};
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[q] += __shfl_xor_sync(0xffffffffu, v[q], o);
    if (lane == 0) red[q][warp] = v[q];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double t[4] = {0, 0, 0, 0};
    for (int q = 0; q < 4; ++q)
      for (int w8 = 0; w8 < (int)(blockDim.x >> 5); ++w8) t[q] += red[q][w8];
    if (loss_sum) loss_sum[0] = (float)t[0];
    if (denom) denom[0] = (float)fmax(t[1], 1.0);
    if (correct) correct[0] = (float)t[2];
    if (tokens) tokens[0] = (float)t[3];
  }
}

// grid = (vocab tiles, row tiles of the chunk).  P = (exp(z - lse) - onehot) * scale_row,
// written to pbuf[(row-row0)][col] with leading dimension ldp.
template <typename T>
__global__ void __launch_bounds__(256) k_ce_probs(CEParams p) {
  __shared__ float Hs[CE_TM * CE_LDS], Ws[CE_TN * CE_LDS];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t col0 = (int64_t)blockIdx.x * CE_TN;
  const int64_t rloc0 = (int64_t)blockIdx.y * CE_TM;
  const int64_t row_end = p.row0 + p.rows;
  float z[4][4];
  logits_tile<T>(z, reinterpret_cast<const T*>(p.h), reinterpret_cast<const T*>(p.w), p.row0 + rloc0, row_end,
                 col0, p.V, p.F, Hs, Ws, tid, ty, tx);
  const float gs = p.grad_scale[0] / p.denom[0];
  T* P = reinterpret_cast<T*>(p.pbuf);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t rl = rloc0 + ty + 16 * r, row = p.row0 + rl;
    if (row >= row_end) continue;
    const int64_t t = p.targets[row];
    const bool valid = t != p.ignore_index;
    const float sc = valid ? gs * (p.mask ? p.mask[row] : 1.f) : 0.f;
    const float l = p.lse[row];
    const int64_t tc = t - p.v_offset;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int64_t col = col0 + tx + 16 * c;
      if (col < p.V) {
        float pr = expf(z[r][c] - l);
        if (col == tc) pr -= 1.f;
        IO<T>::st(P + rl * p.ldp + col, pr * sc);
      }
    }
  }
}

// C[M,N] = (beta ? C : 0) + sum_k A(m,k) B(k,n);  A(m,k) = TRA ? A[k*lda+m] : A[m*lda+k],
// B(k,n) = TRB ? B[n*ldb+k] : B[k*ldb+n].  64x64 tiles, fp32 accumulate.
template <typename TA, typename TB, typename TC, bool TRA, bool TRB>
__global__ void __launch_bounds__(256) k_gemm(const TA* __restrict__ A, const TB* __restrict__ B, TC* __restrict__ C,
                                              int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                              int beta) {
  __shared__ float As[CE_TM * CE_LDS], Bs[CE_TN * CE_LDS];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * CE_TM, n0 = (int64_t)blockIdx.x * CE_TN;
  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += CE_TK) {
#pragma unroll
    for (int i = 0; i < CE_TM * CE_TK / 256; ++i) {
      const int e = tid + i * 256;
      int m, kk;
      if (TRA) { kk = e / CE_TM; m = e - kk * CE_TM; } else { m = e / CE_TK; kk = e - m * CE_TK; }
      float a = 0.f;
      if (m0 + m < M && k0 + kk < K) a = IO<TA>::ld(TRA ? A + (k0 + kk) * lda + m0 + m : A + (m0 + m) * lda + k0 + kk);
      As[m * CE_LDS + kk] = a;
      int n, k2;
      if (TRB) { n = e / CE_TK; k2 = e - n * CE_TK; } else { k2 = e / CE_TN; n = e - k2 * CE_TN; }
      float b = 0.f;
      if (n0 + n < N && k0 + k2 < K) b = IO<TB>::ld(TRB ? B + (n0 + n) * ldb + k0 + k2 : B + (k0 + k2) * ldb + n0 + n);
      Bs[n * CE_LDS + k2] = b;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < CE_TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = As[(ty + 16 * r) * CE_LDS + kk];
#pragma unroll
      for (int c = 0; c < 4; ++c) b[c] = Bs[(tx + 16 * c) * CE_LDS + kk];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t m = m0 + ty + 16 * r;
    if (m >= M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int64_t n = n0 + tx + 16 * c;
      if (n >= N) continue;
      float v = acc[r][c];
      if (beta) v += IO<TC>::ld(C + m * ldc + n);
      IO<TC>::st(C + m * ldc + n, v);
    }
  }
}

template <typename T>
__global__ void k_cast_from_f32(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    IO<T>::st(dst + i, src[i]);
}

}  // namespace qpam
