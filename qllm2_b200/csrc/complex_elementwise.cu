// Fused element-wise complex operators of the V11 blocks, forward and backward, on the interleaved
// [..., C, 2] layout: magnitude-RMS norm, modSwish / modReLU, the gated-unit product, and the
// head split + rotary rotation + protect-gate scaling that feeds the PAM scan.
//
// The reference runs these as Triton kernels in the forward pass and as chains of torch operators in
// the backward pass (v11/triton_kernels.py:48-166 kernels, :209-417 autograd functions, :489-520 the
// plain arithmetic).  Here each direction is ONE pass over the tensors (HBM-bound): 16-byte vector
// loads of 4 complex channels per thread, fp32 arithmetic, per-channel parameter gradients kept in
// registers over the rows a thread walks and written as partial rows that the caller sums.
#include <algorithm>

#include "common.cuh"
#include "elementwise.cuh"

namespace qpam {
namespace {
using namespace ew;

// ------------------------------------------------------------------------------------------------
// Magnitude-RMS norm.  out = z / (|z| + e) * (|z| / rms) * scale,  |z| = sqrt(re^2 + im^2 + e),
// rms = sqrt(mean_j |z_j|^2 + eps).  One warp per row; a lane owns the same channels in every row
// it visits, so d(scale) accumulates in registers (MAXV vectors of 4 channels per lane).
// ------------------------------------------------------------------------------------------------
template <typename TI, typename TO, int MAXV, bool CACHE>
__global__ void __launch_bounds__(128) k_cnorm_fwd(const TI* __restrict__ z, const float* __restrict__ scale,
                                                   TO* __restrict__ out, int64_t N, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int groups = D >> 2;
  constexpr int NV = CACHE ? MAXV : 1;  // rows wider than the register cache are read a second time (L1/L2 hits)
  for (int64_t row = warp; row < N; row += nwarps) {
    const TI* zr = z + row * (int64_t)D * 2;
    float re[NV][4], im[NV][4], ss = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int g = v * 32 + lane, cv = CACHE ? v : 0;
      if (g < groups) {
        V4<TI>::ld(zr + g * 8, re[cv], im[cv]);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += re[cv][j] * re[cv][j] + im[cv][j] * im[cv][j] + MAG_EPS;
      }
    }
    ss = warp_sum(ss);
    const float rrms = rsqrtf(ss / (float)D + eps);
    TO* orow = out + row * (int64_t)D * 2;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int g = v * 32 + lane, cv = CACHE ? v : 0;
      if (g < groups) {
        if (!CACHE) V4<TI>::ld(zr + g * 8, re[cv], im[cv]);
        const float4 sc = *reinterpret_cast<const float4*>(scale + g * 4);
        const float s4[4] = {sc.x, sc.y, sc.z, sc.w};
        float orr[4], oi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const MagInv mag_ = mag_inv(re[cv][j] * re[cv][j] + im[cv][j] * im[cv][j] + MAG_EPS); const float mag = mag_.mag;
          const float w = mag * mag_.inv * rrms * s4[j];
          orr[j] = re[cv][j] * w;
          oi[j] = im[cv][j] * w;
        }
        V4<TO>::st(orow + g * 8, orr, oi);
      }
    }
  }
}

// With w_j = scale_j m_j / rms, m_j = |z_j| / (|z_j| + e), s_j = Re(conj(z_j) dout_j):
//   dz_j = dout_j w_j + z_j [ s_j scale_j e / (rms (|z_j|+e)^2 |z_j|) - c / (rms D) ],
//   c = sum_j s_j scale_j m_j / rms^2,    dscale_j = sum_rows s_j m_j / rms.
template <typename TI, typename TO, int MAXV, bool CACHE>
__global__ void __launch_bounds__(128) k_cnorm_bwd(const TI* __restrict__ z, const float* __restrict__ scale,
                                                   const TO* __restrict__ dout, TI* __restrict__ dz,
                                                   float* __restrict__ dscale_part, int64_t N, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int groups = D >> 2;
  constexpr int NV = CACHE ? MAXV : 1;
  float acc[MAXV][4];
#pragma unroll
  for (int v = 0; v < MAXV; ++v)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[v][j] = 0.f;
  for (int64_t row = warp; row < N; row += nwarps) {
    const TI* zr = z + row * (int64_t)D * 2;
    const TO* dr = dout + row * (int64_t)D * 2;
    float re[NV][4], im[NV][4], gr[NV][4], gi[NV][4], ss = 0.f, cs = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int g = v * 32 + lane, cv = CACHE ? v : 0;
      if (g < groups) {
        V4<TI>::ld(zr + g * 8, re[cv], im[cv]);
        V4<TO>::ld(dr + g * 8, gr[cv], gi[cv]);
        const float4 sc = *reinterpret_cast<const float4*>(scale + g * 4);
        const float s4[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float m2 = re[cv][j] * re[cv][j] + im[cv][j] * im[cv][j] + MAG_EPS;
          const MagInv mag_ = mag_inv(m2); const float mag = mag_.mag;
          ss += m2;
          cs += (gr[cv][j] * re[cv][j] + gi[cv][j] * im[cv][j]) * s4[j] * (mag * mag_.inv);
        }
      }
    }
    ss = warp_sum(ss);
    cs = warp_sum(cs);
    const float rrms = rsqrtf(ss / (float)D + eps);
    const float common = cs * rrms * rrms * rrms / (float)D;  // c / (rms D)
    TI* dzr = dz + row * (int64_t)D * 2;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int g = v * 32 + lane, cv = CACHE ? v : 0;
      if (g < groups) {
        if (!CACHE) {
          V4<TI>::ld(zr + g * 8, re[cv], im[cv]);
          V4<TO>::ld(dr + g * 8, gr[cv], gi[cv]);
        }
        const float4 sc = *reinterpret_cast<const float4*>(scale + g * 4);
        const float s4[4] = {sc.x, sc.y, sc.z, sc.w};
        float orr[4], oi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const MagInv mag_ = mag_inv(re[cv][j] * re[cv][j] + im[cv][j] * im[cv][j] + MAG_EPS); const float mag = mag_.mag;
          const float inv = mag_.inv;
          const float m = mag * inv;
          const float s = gr[cv][j] * re[cv][j] + gi[cv][j] * im[cv][j];
          const float w = m * rrms * s4[j];
          const float k = s * s4[j] * MAG_EPS * rrms * inv * inv * mag_.rmag - common;
          orr[j] = gr[cv][j] * w + re[cv][j] * k;
          oi[j] = gi[cv][j] * w + im[cv][j] * k;
          acc[v][j] += s * m * rrms;
        }
        V4<TI>::st(dzr + g * 8, orr, oi);
      }
    }
  }
  {  // every warp writes its row of partial sums (zeros when it had no rows): the caller adds all of them
    float* prow = dscale_part + warp * (int64_t)D;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int g = v * 32 + lane;
      if (g < groups) *reinterpret_cast<float4*>(prow + g * 4) = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
    }
  }
}

template <typename TI, typename TO>
int cnorm_launch(bool bwd, const void* z, const float* scale, const void* dout_or_out, void* dz, float* part,
                 int P, int64_t N, int D, float eps, cudaStream_t st) {
  const int groups = D / 4;
  const int maxv = (groups + 31) / 32;
  const int blocks = (P + 3) / 4;
#define QPAM_CNORM(MV, CA)                                                                                          \
  if (bwd)                                                                                                          \
    k_cnorm_bwd<TI, TO, MV, CA><<<blocks, 128, 0, st>>>((const TI*)z, scale, (const TO*)dout_or_out, (TI*)dz, part, \
                                                        N, D, eps);                                                 \
  else                                                                                                              \
    k_cnorm_fwd<TI, TO, MV, CA><<<blocks, 128, 0, st>>>((const TI*)z, scale, (TO*)const_cast<void*>(dout_or_out), N, D, eps);
  if (maxv <= 3) { QPAM_CNORM(3, true) }
  else if (maxv <= 6) { QPAM_CNORM(6, true) }
  else if (maxv <= 12) { QPAM_CNORM(12, false) }
  else { QPAM_CNORM(24, false) }
#undef QPAM_CNORM
  if (bwd) { QPAM_LAUNCH_CHECK("k_cnorm_bwd"); } else { QPAM_LAUNCH_CHECK("k_cnorm_fwd"); }
  return QPAM_OK;
}

// ------------------------------------------------------------------------------------------------
// modSwish  out = z / (|z|+e) * |z| sigmoid(beta |z| + bias)      (beta != nullptr)
// modReLU   out = z / (|z|+e) * relu(|z| + bias)                  (beta == nullptr)
// A thread owns one group of 4 channels and walks rows blockIdx.y, blockIdx.y + gridDim.y, ...
// ------------------------------------------------------------------------------------------------
template <typename T, bool SWISH>
__global__ void __launch_bounds__(512) k_modact_fwd(const T* __restrict__ z, const float* __restrict__ bias,
                                                    const float* __restrict__ beta, T* __restrict__ out,
                                                    int64_t N, int C) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= (C >> 2)) return;
  float b4[4], be4[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b4[j] = bias[g * 4 + j];
    be4[j] = SWISH ? beta[g * 4 + j] : 0.f;
  }
#pragma unroll 2
  for (int64_t row = blockIdx.y; row < N; row += gridDim.y) {
    float re[4], im[4];
    V4<T>::ld(z + (row * C + g * 4) * 2, re, im);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const MagInv mag_ = mag_inv(re[j] * re[j] + im[j] * im[j] + MAG_EPS); const float mag = mag_.mag;
      const float act = SWISH ? mag * sigmoidf_(be4[j] * mag + b4[j]) : fmaxf(mag + b4[j], 0.f);
      const float f = act * mag_.inv;
      re[j] *= f;
      im[j] *= f;
    }
    V4<T>::st(out + (row * C + g * 4) * 2, re, im);
  }
}

// out = z f(|z|):  dz = dout f + z s f'(|z|) / |z|,  s = Re(conj(z) dout).
template <typename T, bool SWISH>
__global__ void __launch_bounds__(512) k_modact_bwd(const T* __restrict__ z, const float* __restrict__ bias,
                                                    const float* __restrict__ beta, const T* __restrict__ dout,
                                                    T* __restrict__ dz, float* __restrict__ dbias_part,
                                                    float* __restrict__ dbeta_part, int64_t N, int C) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= (C >> 2)) return;
  float b4[4], be4[4], ab[4] = {0.f, 0.f, 0.f, 0.f}, abe[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b4[j] = bias[g * 4 + j];
    be4[j] = SWISH ? beta[g * 4 + j] : 0.f;
  }
#pragma unroll 2
  for (int64_t row = blockIdx.y; row < N; row += gridDim.y) {
    float re[4], im[4], gr[4], gi[4];
    V4<T>::ld(z + (row * C + g * 4) * 2, re, im);
    V4<T>::ld(dout + (row * C + g * 4) * 2, gr, gi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const MagInv mag_ = mag_inv(re[j] * re[j] + im[j] * im[j] + MAG_EPS); const float mag = mag_.mag;
      const float inv = mag_.inv;
      const float s = gr[j] * re[j] + gi[j] * im[j];
      float act, dact;  // act(|z|) and its derivative
      if (SWISH) {
        const float sg = sigmoidf_(be4[j] * mag + b4[j]);
        const float t = mag * sg * (1.f - sg);
        act = mag * sg;
        dact = sg + t * be4[j];
        ab[j] += s * t * inv;
        abe[j] += s * t * mag * inv;
      } else {
        const bool on = mag + b4[j] > 0.f;
        act = on ? mag + b4[j] : 0.f;
        dact = on ? 1.f : 0.f;
        ab[j] += on ? s * inv : 0.f;
      }
      const float f = act * inv;
      const float k = s * (dact * inv - act * inv * inv) * mag_.rmag;
      const float r0 = re[j], i0 = im[j];
      re[j] = gr[j] * f + r0 * k;
      im[j] = gi[j] * f + i0 * k;
    }
    V4<T>::st(dz + (row * C + g * 4) * 2, re, im);
  }
  float* pb = dbias_part + (int64_t)blockIdx.y * C + g * 4;
  *reinterpret_cast<float4*>(pb) = make_float4(ab[0], ab[1], ab[2], ab[3]);
  if (SWISH) {
    float* pe = dbeta_part + (int64_t)blockIdx.y * C + g * 4;
    *reinterpret_cast<float4*>(pe) = make_float4(abe[0], abe[1], abe[2], abe[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// Gated-unit product  out = gate/(|gate|+e) * up * sigmoid(|gate|)   (complex product).
// gate / up / dgate / dup rows may sit inside wider matrices: ld_* are row strides in scalars.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512) k_cgu_gate_fwd(const T* __restrict__ gate, int64_t ld_gate,
                                                      const T* __restrict__ up, int64_t ld_up,
                                                      T* __restrict__ out, int64_t N, int C) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= (C >> 2)) return;
#pragma unroll 2
  for (int64_t row = blockIdx.y; row < N; row += gridDim.y) {
    float ar[4], ai[4], ur[4], ui[4];
    V4<T>::ld(gate + row * ld_gate + g * 8, ar, ai);
    V4<T>::ld(up + row * ld_up + g * 8, ur, ui);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const MagInv mag_ = mag_inv(ar[j] * ar[j] + ai[j] * ai[j] + MAG_EPS); const float mag = mag_.mag;
      const float h = sigmoidf_(mag) * mag_.inv;
      const float pr = ar[j] * ur[j] - ai[j] * ui[j], pi = ar[j] * ui[j] + ai[j] * ur[j];
      ar[j] = pr * h;
      ai[j] = pi * h;
    }
    V4<T>::st(out + (row * C + g * 4) * 2, ar, ai);
  }
}

template <typename T>
__global__ void __launch_bounds__(512) k_cgu_gate_bwd(const T* __restrict__ gate, int64_t ld_gate,
                                                      const T* __restrict__ up, int64_t ld_up,
                                                      const T* __restrict__ dout, T* __restrict__ dgate,
                                                      int64_t ld_dgate, T* __restrict__ dup, int64_t ld_dup,
                                                      int64_t N, int C) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= (C >> 2)) return;
#pragma unroll 2
  for (int64_t row = blockIdx.y; row < N; row += gridDim.y) {
    float ar[4], ai[4], ur[4], ui[4], gr[4], gi[4], dur[4], dui[4];
    V4<T>::ld(gate + row * ld_gate + g * 8, ar, ai);
    V4<T>::ld(up + row * ld_up + g * 8, ur, ui);
    V4<T>::ld(dout + (row * C + g * 4) * 2, gr, gi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const MagInv mag_ = mag_inv(ar[j] * ar[j] + ai[j] * ai[j] + MAG_EPS); const float mag = mag_.mag;
      const float inv = mag_.inv;
      const float sg = sigmoidf_(mag);
      const float h = sg * inv;
      const float dh = sg * (1.f - sg) * inv - sg * inv * inv;
      const float pr = ar[j] * ur[j] - ai[j] * ui[j], pi = ar[j] * ui[j] + ai[j] * ur[j];
      const float s = gr[j] * pr + gi[j] * pi;
      // d(up) = conj(gate) dout h ;  d(gate) = conj(up) dout h + gate s h'(|gate|) / |gate|
      dur[j] = h * (ar[j] * gr[j] + ai[j] * gi[j]);
      dui[j] = h * (ar[j] * gi[j] - ai[j] * gr[j]);
      const float k = s * dh * mag_.rmag;
      const float dgr = h * (ur[j] * gr[j] + ui[j] * gi[j]) + ar[j] * k;
      const float dgi = h * (ur[j] * gi[j] - ui[j] * gr[j]) + ai[j] * k;
      ar[j] = dgr;
      ai[j] = dgi;
    }
    V4<T>::st(dgate + row * ld_dgate + g * 8, ar, ai);
    V4<T>::st(dup + row * ld_dup + g * 8, dur, dui);
  }
}


// ------------------------------------------------------------------------------------------------
// PAM input stage: the fused projection output qkv [B,T,3,H,d,2] is split into Q, K, V'
// [B,H,T,d,2]; Q and K are rotated by rope[pos] (cos,sin per channel), V' = (1-p) V with the
// protect gate's complement omp [B,T,H] (fp32).  pos = positions[b,t] when given, else offset + t.
// A thread moves one group of 4 channels of one of the three tensors; gph = d/4 groups per head.
// ------------------------------------------------------------------------------------------------
struct PrepParams {
  const void* qkv;
  const float* rope;
  const int64_t* positions;
  const float* omp;
  void *q, *k, *v;      // fwd: outputs; bwd: incoming gradients
  void* dqkv;           // bwd
  float* domp;          // bwd (may be null)
  int64_t offset, rope_len;
  int B, T, H, d;
};

constexpr int PREP_U = 2;  // tokens in flight per thread: all their loads are issued before any arithmetic or store

// A thread owns one (head, group of 4 channels) and moves q, k and v of it (the rotary factors are shared by
// q and k); d/4 consecutive lanes cover a head, so d(omp) is a shuffle sum.
template <typename T, bool BWD>
__global__ void __launch_bounds__(512) k_pam_prep(PrepParams p) {
  const int gph = p.d >> 2;
  const int per_tok = p.H * gph;
  const int per_tok_pad = (per_tok + 31) & ~31;
  const int64_t ntok = (int64_t)p.B * p.T;
  const int64_t ntile = (ntok + PREP_U - 1) / PREP_U;
  const int64_t side_stride = (int64_t)p.H * p.d * 2;  // q -> k -> v inside one token of qkv
  for (int64_t tile = blockIdx.x; tile < ntile; tile += gridDim.x) {
    for (int idx = threadIdx.x; idx < per_tok_pad; idx += blockDim.x) {
      const bool lane_on = idx < per_tok;
      const int h = lane_on ? idx / gph : 0, g = lane_on ? idx - h * gph : 0;
      float re[PREP_U][3][4], im[PREP_U][3][4], vr[PREP_U][4], vi[PREP_U][4], keep[PREP_U];
      float4 c0[PREP_U], c1[PREP_U];
      int64_t src[PREP_U], dst[PREP_U];
      bool on[PREP_U];
      // ---- all loads first
#pragma unroll
      for (int u = 0; u < PREP_U; ++u) {
        const int64_t tok = tile * PREP_U + u;
        on[u] = lane_on && tok < ntok;
        const int64_t tk = on[u] ? tok : 0;
        const int b = (int)(tk / p.T), t = (int)(tk - (int64_t)b * p.T);
        src[u] = (tk * 3 * p.H + h) * (int64_t)p.d * 2 + g * 8;
        dst[u] = (((int64_t)b * p.H + h) * p.T + t) * (int64_t)p.d * 2 + g * 8;
        keep[u] = 1.f;
        c0[u] = c1[u] = make_float4(1.f, 0.f, 1.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          vr[u][j] = vi[u][j] = 0.f;
#pragma unroll
          for (int w = 0; w < 3; ++w) re[u][w][j] = im[u][w][j] = 0.f;
        }
        if (on[u]) {
          if (!BWD) {
#pragma unroll
            for (int w = 0; w < 3; ++w) V4<T>::ld(reinterpret_cast<const T*>(p.qkv) + src[u] + w * side_stride, re[u][w], im[u][w]);
          } else {
            V4<T>::ld(reinterpret_cast<const T*>(p.q) + dst[u], re[u][0], im[u][0]);
            V4<T>::ld(reinterpret_cast<const T*>(p.k) + dst[u], re[u][1], im[u][1]);
            V4<T>::ld(reinterpret_cast<const T*>(p.v) + dst[u], re[u][2], im[u][2]);
            if (p.domp) V4<T>::ld(reinterpret_cast<const T*>(p.qkv) + src[u] + 2 * side_stride, vr[u], vi[u]);
          }
          if (p.omp) keep[u] = p.omp[tk * p.H + h];
          if (p.rope) {
            int64_t pos = p.positions ? p.positions[tk] : p.offset + t;
            pos = pos < 0 ? 0 : (pos >= p.rope_len ? p.rope_len - 1 : pos);
            c0[u] = *reinterpret_cast<const float4*>(p.rope + (pos * p.d + g * 4) * 2);
            c1[u] = *reinterpret_cast<const float4*>(p.rope + (pos * p.d + g * 4) * 2 + 4);
          }
        }
      }
      // ---- arithmetic and stores
#pragma unroll
      for (int u = 0; u < PREP_U; ++u) {
        float dot = 0.f;
        if (on[u]) {
          const float cs[4] = {c0[u].x, c0[u].z, c1[u].x, c1[u].z};
          const float sn[4] = {c0[u].y, c0[u].w, c1[u].y, c1[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            dot += vr[u][j] * re[u][2][j] + vi[u][j] * im[u][2][j];
            const float s_ = BWD ? -sn[j] : sn[j];  // the gradient rotates back
#pragma unroll
            for (int w = 0; w < 2; ++w) {
              const float r0 = re[u][w][j], i0 = im[u][w][j];
              re[u][w][j] = r0 * cs[j] - i0 * s_;
              im[u][w][j] = r0 * s_ + i0 * cs[j];
            }
            re[u][2][j] *= keep[u];
            im[u][2][j] *= keep[u];
          }
          if (!BWD) {
            V4<T>::st(reinterpret_cast<T*>(p.q) + dst[u], re[u][0], im[u][0]);
            V4<T>::st(reinterpret_cast<T*>(p.k) + dst[u], re[u][1], im[u][1]);
            V4<T>::st(reinterpret_cast<T*>(p.v) + dst[u], re[u][2], im[u][2]);
          } else {
#pragma unroll
            for (int w = 0; w < 3; ++w) V4<T>::st(reinterpret_cast<T*>(p.dqkv) + src[u] + w * side_stride, re[u][w], im[u][w]);
          }
        }
        if (BWD && p.domp) {  // sum over the head's channels: gph consecutive lanes (gph divides 32)
          for (int o = gph >> 1; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (on[u] && g == 0) p.domp[(tile * PREP_U + u) * p.H + h] = dot;
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Read-out of K phase-routed states:  y[r, :] = sum_k c_k[r] * y_k[r, :]  (complex), rows r = (b,h,t),
// coef fp32 [K, R, 2].  Backward: dy_k = conj(c_k) dy,  dc_k[r] = sum_j dy[r,j] conj(y_k[r,j]).
// d/4 consecutive lanes share a row (d a power of two <= 128).
// ------------------------------------------------------------------------------------------------
struct CombineParams {
  const void* yk[QPAM_MAX_STATES];
  void* dyk[QPAM_MAX_STATES];
  const float* coef;
  void* y;        // fwd: output; bwd: incoming gradient
  float* dcoef;   // bwd
  int64_t R;
  int d, K;
  int H, T;       // > 0: y (forward) and dy (backward) are token-major, [b, t, h, :] for row r = (b, h, t)
};

// KK: the number of states as a compile-time constant, so that the K loads of a group are all in flight before the
// first one is used
template <typename T, bool BWD, int KK>
__global__ void __launch_bounds__(256) k_state_combine(CombineParams p) {
  const int gpr = p.d >> 2;  // vector groups per row
  const int64_t total = p.R * gpr;
  const int64_t total_pad = (total + 31) & ~(int64_t)31;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_pad;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const bool on = idx < total;
    const int64_t r = on ? idx / gpr : 0;
    const int g = on ? (int)(idx - r * gpr) : 0;
    const int64_t off = (r * p.d + g * 4) * 2;
    float ar[4] = {0.f, 0.f, 0.f, 0.f}, ai[4] = {0.f, 0.f, 0.f, 0.f};
    int64_t yo = off;                                   // where this group sits in y (forward) / dy (backward)
    if (p.H > 0) {
      const int64_t bh = r / p.T, t = r - bh * p.T, b = bh / p.H, h = bh - b * p.H;
      yo = (((b * p.T + t) * p.H + h) * p.d + g * 4) * 2;
    }
    if (BWD && on) V4<T>::ld(reinterpret_cast<const T*>(p.y) + yo, ar, ai);
    float2 cs[KK];
    float yrs[KK][4], yis[KK][4];
#pragma unroll
    for (int k = 0; k < KK; ++k) {
      cs[k] = on ? *reinterpret_cast<const float2*>(p.coef + ((int64_t)k * p.R + r) * 2) : make_float2(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) yrs[k][j] = yis[k][j] = 0.f;
      if (on) V4<T>::ld(reinterpret_cast<const T*>(p.yk[k]) + off, yrs[k], yis[k]);
    }
#pragma unroll
    for (int k = 0; k < KK; ++k) {
      const float2 c = cs[k];
      const float (&yr)[4] = yrs[k];
      const float (&yi)[4] = yis[k];
      if (!BWD) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ar[j] += c.x * yr[j] - c.y * yi[j];
          ai[j] += c.x * yi[j] + c.y * yr[j];
        }
      } else {
        float dr = 0.f, di = 0.f, gr[4], gi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          dr += ar[j] * yr[j] + ai[j] * yi[j];
          di += ai[j] * yr[j] - ar[j] * yi[j];
          gr[j] = c.x * ar[j] + c.y * ai[j];
          gi[j] = c.x * ai[j] - c.y * ar[j];
        }
        for (int o = gpr >> 1; o; o >>= 1) {
          dr += __shfl_xor_sync(0xffffffffu, dr, o);
          di += __shfl_xor_sync(0xffffffffu, di, o);
        }
        if (on) {
          V4<T>::st(reinterpret_cast<T*>(p.dyk[k]) + off, gr, gi);
          if (g == 0) *reinterpret_cast<float2*>(p.dcoef + ((int64_t)k * p.R + r) * 2) = make_float2(dr, di);
        }
      }
    }
    if (!BWD && on) V4<T>::st(reinterpret_cast<T*>(p.y) + yo, ar, ai);
  }
}

inline int act_grid_y(int64_t N, int xblocks, int threads) {  // enough rows in flight to fill every SM's thread slots
  const int64_t y = std::max<int64_t>(1, (sm_count() * 2048) / ((int64_t)xblocks * threads));
  return (int)std::min<int64_t>(std::min<int64_t>(y, N), 65535);
}

}  // namespace
}  // namespace qpam

using namespace qpam;

extern "C" int qpam_cnorm_fwd(const void* z, int32_t z_dtype, const float* scale, void* out, int32_t out_dtype,
                              int64_t N, int32_t D, float eps, void* stream) {
  QPAM_REQUIRE(z && scale && out, "cnorm_fwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(z_dtype) && is_dtype(out_dtype) && !(z_dtype == QPAM_BF16 && out_dtype == QPAM_F32),
               "cnorm_fwd: dtypes must be f32->f32, f32->bf16 or bf16->bf16");
  QPAM_REQUIRE(N >= 0 && D > 0 && D % 4 == 0 && D <= 3072, "cnorm_fwd: D must be a multiple of 4 and <= 3072 (got %d)", D);
  if (N == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int P = (int)std::min<int64_t>(N, sm_count() * 32);
  if (z_dtype == QPAM_F32 && out_dtype == QPAM_F32) return cnorm_launch<float, float>(false, z, scale, out, nullptr, nullptr, P, N, D, eps, st);
  if (z_dtype == QPAM_F32) return cnorm_launch<float, __nv_bfloat16>(false, z, scale, out, nullptr, nullptr, P, N, D, eps, st);
  return cnorm_launch<__nv_bfloat16, __nv_bfloat16>(false, z, scale, out, nullptr, nullptr, P, N, D, eps, st);
}

extern "C" int qpam_cnorm_bwd(const void* z, int32_t z_dtype, const float* scale, const void* dout,
                              int32_t out_dtype, void* dz, float* dscale_partials, int32_t P, int64_t N,
                              int32_t D, float eps, void* stream) {
  QPAM_REQUIRE(z && scale && dout && dz && dscale_partials, "cnorm_bwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(z_dtype) && is_dtype(out_dtype) && !(z_dtype == QPAM_BF16 && out_dtype == QPAM_F32),
               "cnorm_bwd: dtypes must be f32->f32, f32->bf16 or bf16->bf16");
  QPAM_REQUIRE(N > 0 && D > 0 && D % 4 == 0 && D <= 3072, "cnorm_bwd: D must be a multiple of 4 and <= 3072 (got %d)", D);
  QPAM_REQUIRE(P > 0 && P % 4 == 0, "cnorm_bwd: the number of partial rows must be a positive multiple of 4");
  cudaStream_t st = (cudaStream_t)stream;
  if (z_dtype == QPAM_F32 && out_dtype == QPAM_F32) return cnorm_launch<float, float>(true, z, scale, dout, dz, dscale_partials, P, N, D, eps, st);
  if (z_dtype == QPAM_F32) return cnorm_launch<float, __nv_bfloat16>(true, z, scale, dout, dz, dscale_partials, P, N, D, eps, st);
  return cnorm_launch<__nv_bfloat16, __nv_bfloat16>(true, z, scale, dout, dz, dscale_partials, P, N, D, eps, st);
}

extern "C" int qpam_modact_fwd(const void* z, int32_t dtype, const float* bias, const float* beta, void* out,
                               int64_t N, int32_t C, void* stream) {
  QPAM_REQUIRE(z && bias && out, "modact_fwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && N >= 0 && C > 0 && C % 4 == 0, "modact_fwd: C must be a multiple of 4 (got %d)", C);
  if (N == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int groups = C / 4, threads = pick_threads(groups), xb = (groups + threads - 1) / threads;
  dim3 grid(xb, act_grid_y(N, xb, threads));
#define QPAM_ACT(T)                                                                                      \
  if (beta) k_modact_fwd<T, true><<<grid, threads, 0, st>>>((const T*)z, bias, beta, (T*)out, N, C);     \
  else k_modact_fwd<T, false><<<grid, threads, 0, st>>>((const T*)z, bias, beta, (T*)out, N, C);
  if (dtype == QPAM_F32) { QPAM_ACT(float) } else { QPAM_ACT(__nv_bfloat16) }
#undef QPAM_ACT
  QPAM_LAUNCH_CHECK("k_modact_fwd");
  return QPAM_OK;
}

extern "C" int qpam_modact_bwd(const void* z, int32_t dtype, const float* bias, const float* beta,
                               const void* dout, void* dz, float* dbias_partials, float* dbeta_partials,
                               int32_t P, int64_t N, int32_t C, void* stream) {
  QPAM_REQUIRE(z && bias && dout && dz && dbias_partials && (!beta || dbeta_partials), "modact_bwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && N > 0 && C > 0 && C % 4 == 0, "modact_bwd: C must be a multiple of 4 (got %d)", C);
  QPAM_REQUIRE(P > 0 && P <= N && P <= 65535, "modact_bwd: partial rows must be in [1, min(N, 65535)]");
  cudaStream_t st = (cudaStream_t)stream;
  const int groups = C / 4, threads = pick_threads(groups), xb = (groups + threads - 1) / threads;
  dim3 grid(xb, P);
#define QPAM_ACT(T)                                                                                              \
  if (beta) k_modact_bwd<T, true><<<grid, threads, 0, st>>>((const T*)z, bias, beta, (const T*)dout, (T*)dz,      \
                                                            dbias_partials, dbeta_partials, N, C);               \
  else k_modact_bwd<T, false><<<grid, threads, 0, st>>>((const T*)z, bias, beta, (const T*)dout, (T*)dz,          \
                                                        dbias_partials, dbeta_partials, N, C);
  if (dtype == QPAM_F32) { QPAM_ACT(float) } else { QPAM_ACT(__nv_bfloat16) }
#undef QPAM_ACT
  QPAM_LAUNCH_CHECK("k_modact_bwd");
  return QPAM_OK;
}

extern "C" int qpam_cgu_gate_fwd(const void* gate, int64_t ld_gate, const void* up, int64_t ld_up, int32_t dtype,
                                 void* out, int64_t N, int32_t C, void* stream) {
  QPAM_REQUIRE(gate && up && out, "cgu_gate_fwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && N >= 0 && C > 0 && C % 4 == 0, "cgu_gate_fwd: C must be a multiple of 4 (got %d)", C);
  const int64_t al = dtype == QPAM_F32 ? 4 : 8;  // 16-byte rows
  QPAM_REQUIRE(ld_gate >= 2 * C && ld_up >= 2 * C && ld_gate % al == 0 && ld_up % al == 0,
               "cgu_gate_fwd: row strides must cover 2*C scalars and keep rows 16-byte aligned");
  if (N == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int groups = C / 4, threads = pick_threads(groups), xb = (groups + threads - 1) / threads;
  dim3 grid(xb, act_grid_y(N, xb, threads));
  if (dtype == QPAM_F32) k_cgu_gate_fwd<float><<<grid, threads, 0, st>>>((const float*)gate, ld_gate, (const float*)up, ld_up, (float*)out, N, C);
  else k_cgu_gate_fwd<__nv_bfloat16><<<grid, threads, 0, st>>>((const __nv_bfloat16*)gate, ld_gate, (const __nv_bfloat16*)up, ld_up, (__nv_bfloat16*)out, N, C);
  QPAM_LAUNCH_CHECK("k_cgu_gate_fwd");
  return QPAM_OK;
}

extern "C" int qpam_cgu_gate_bwd(const void* gate, int64_t ld_gate, const void* up, int64_t ld_up,
                                 const void* dout, int32_t dtype, void* dgate, int64_t ld_dgate, void* dup,
                                 int64_t ld_dup, int64_t N, int32_t C, void* stream) {
  QPAM_REQUIRE(gate && up && dout && dgate && dup, "cgu_gate_bwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && N > 0 && C > 0 && C % 4 == 0, "cgu_gate_bwd: C must be a multiple of 4 (got %d)", C);
  const int64_t al = dtype == QPAM_F32 ? 4 : 8;
  QPAM_REQUIRE(ld_gate >= 2 * C && ld_up >= 2 * C && ld_dgate >= 2 * C && ld_dup >= 2 * C && ld_gate % al == 0 &&
                   ld_up % al == 0 && ld_dgate % al == 0 && ld_dup % al == 0,
               "cgu_gate_bwd: row strides must cover 2*C scalars and keep rows 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int groups = C / 4, threads = pick_threads(groups), xb = (groups + threads - 1) / threads;
  dim3 grid(xb, act_grid_y(N, xb, threads));
  if (dtype == QPAM_F32)
    k_cgu_gate_bwd<float><<<grid, threads, 0, st>>>((const float*)gate, ld_gate, (const float*)up, ld_up, (const float*)dout,
                                                    (float*)dgate, ld_dgate, (float*)dup, ld_dup, N, C);
  else
    k_cgu_gate_bwd<__nv_bfloat16><<<grid, threads, 0, st>>>((const __nv_bfloat16*)gate, ld_gate, (const __nv_bfloat16*)up, ld_up,
                                                            (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgate, ld_dgate,
                                                            (__nv_bfloat16*)dup, ld_dup, N, C);
  QPAM_LAUNCH_CHECK("k_cgu_gate_bwd");
  return QPAM_OK;
}

static int pam_prep(bool bwd, const void* qkv, int32_t dtype, const float* rope, int64_t rope_len,
                    const int64_t* positions, int64_t offset, const float* omp, void* q, void* k, void* v,
                    void* dqkv, float* domp, int32_t B, int32_t T, int32_t H, int32_t d, void* stream) {
  QPAM_REQUIRE(qkv && q && k && v && (!bwd || dqkv), "pam_prep: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && B > 0 && T > 0 && H > 0, "pam_prep: bad dtype or empty shape");
  QPAM_REQUIRE(d >= 4 && d <= 128 && (d & (d - 1)) == 0, "pam_prep: head_dim must be a power of two in [4,128] (got %d)", d);
  QPAM_REQUIRE(!rope || rope_len > 0, "pam_prep: empty rotary table");
  QPAM_REQUIRE(!rope || positions || offset + T <= rope_len, "pam_prep: rotary table shorter than offset + T");
  cudaStream_t st = (cudaStream_t)stream;
  PrepParams p{qkv, rope, positions, omp, q, k, v, dqkv, (bwd && omp) ? domp : nullptr, offset, rope_len, B, T, H, d};
  const int per_tok = H * (d / 4);
  const int threads = pick_threads(per_tok);
  const int grid = (int)std::min<int64_t>(((int64_t)B * T + PREP_U - 1) / PREP_U, (sm_count() * 2048) / threads);
  if (dtype == QPAM_F32) {
    if (bwd) k_pam_prep<float, true><<<grid, threads, 0, st>>>(p);
    else k_pam_prep<float, false><<<grid, threads, 0, st>>>(p);
  } else {
    if (bwd) k_pam_prep<__nv_bfloat16, true><<<grid, threads, 0, st>>>(p);
    else k_pam_prep<__nv_bfloat16, false><<<grid, threads, 0, st>>>(p);
  }
  if (bwd) { QPAM_LAUNCH_CHECK("k_pam_prep_bwd"); } else { QPAM_LAUNCH_CHECK("k_pam_prep_fwd"); }
  return QPAM_OK;
}

extern "C" int qpam_pam_prep_fwd(const void* qkv, int32_t dtype, const float* rope, int64_t rope_len,
                                 const int64_t* positions, int64_t offset, const float* omp, void* q, void* k,
                                 void* v, int32_t B, int32_t T, int32_t H, int32_t d, void* stream) {
  return pam_prep(false, qkv, dtype, rope, rope_len, positions, offset, omp, q, k, v, nullptr, nullptr, B, T, H, d, stream);
}

extern "C" int qpam_pam_prep_bwd(const void* qkv, int32_t dtype, const float* rope, int64_t rope_len,
                                 const int64_t* positions, int64_t offset, const float* omp, const void* dq,
                                 const void* dk, const void* dv, void* dqkv, float* domp, int32_t B, int32_t T,
                                 int32_t H, int32_t d, void* stream) {
  return pam_prep(true, qkv, dtype, rope, rope_len, positions, offset, omp, const_cast<void*>(dq),
                  const_cast<void*>(dk), const_cast<void*>(dv), dqkv, domp, B, T, H, d, stream);
}

namespace qpam {
namespace {
using namespace ew;
// ------------------------------------------------------------------------------------------------
// Residual with a learnable scalar:  out = x + s * delta  (x, out: TX; delta: TD), backward
// d(delta) = s * dout, d(s) = sum dout * delta (per-CTA partial sums), d(x) = dout.
// Block weight of a complex projection:  W[(o,c),(j,c')] with (c,c') = (re,re): Wr, (re,im): -Wi,
// (im,re): Wi, (im,im): Wr, so that interleaved y = x W^T is the complex product; and its transpose
// map for the gradient  dWr = dW[re,re] + dW[im,im],  dWi = dW[im,re] - dW[re,im].
// ------------------------------------------------------------------------------------------------
template <typename TX, typename TD>
__global__ void __launch_bounds__(256) k_scaled_residual_fwd(const TX* __restrict__ x, const TD* __restrict__ delta,
                                                             const float* __restrict__ s, TX* __restrict__ out,
                                                             int64_t n) {
  const float sv = *s;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float xv[4], dv[4];
    E4<TX>::ld(x + i, xv);
    E4<TD>::ld(delta + i, dv);
#pragma unroll
    for (int j = 0; j < 4; ++j) xv[j] = fmaf(sv, dv[j], xv[j]);
    E4<TX>::st(out + i, xv);
  }
}

template <typename TX, typename TD>
__global__ void __launch_bounds__(256) k_scaled_residual_bwd(const TX* __restrict__ dout, const TD* __restrict__ delta,
                                                             const float* __restrict__ s, TD* __restrict__ ddelta,
                                                             float* __restrict__ ds_part, int64_t n) {
  __shared__ float red[8];
  const float sv = *s;
  float acc = 0.f;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float gv[4], dv[4];
    E4<TX>::ld(dout + i, gv);
    E4<TD>::ld(delta + i, dv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc = fmaf(gv[j], dv[j], acc);
      dv[j] = sv * gv[j];
    }
    E4<TD>::st(ddelta + i, dv);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    ds_part[blockIdx.x] = t;
  }
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(256) k_block_weight_fwd(const TW* __restrict__ wr, const TW* __restrict__ wi,
                                                          TO* __restrict__ w, int out_dim, int in_dim) {
  const int64_t n = (int64_t)out_dim * in_dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = i / in_dim, j = i - o * in_dim;
    const float a = IO<TW>::ld(wr + i), b = IO<TW>::ld(wi + i);
    TO* r0 = w + (2 * o) * (int64_t)(2 * in_dim) + 2 * j;       // row (o, re)
    TO* r1 = r0 + 2 * in_dim;                                   // row (o, im)
    IO<TO>::st2(r0, make_float2(a, -b));
    IO<TO>::st2(r1, make_float2(b, a));
  }
}

template <typename TW, typename TO>
__global__ void __launch_bounds__(256) k_block_weight_bwd(const TO* __restrict__ dw, TW* __restrict__ dwr,
                                                          TW* __restrict__ dwi, int out_dim, int in_dim) {
  const int64_t n = (int64_t)out_dim * in_dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = i / in_dim, j = i - o * in_dim;
    const TO* r0 = dw + (2 * o) * (int64_t)(2 * in_dim) + 2 * j;
    const float2 a = IO<TO>::ld2(r0), b = IO<TO>::ld2(r0 + 2 * in_dim);
    IO<TW>::st(dwr + i, a.x + b.y);
    IO<TW>::st(dwi + i, b.x - a.y);
  }
}

}  // namespace
}  // namespace qpam

namespace qpam {
namespace {
using namespace ew;
// ------------------------------------------------------------------------------------------------
// Gate arithmetic of the PAM layer on [B,T,H] logits (v11/model.py:308-350, 630-655, 685-720):
//   x_k = dt + dt_bias[h] + off[k];  base_k = 1/(1+e^{x_k}) (= exp(-softplus(x_k)));  base'_k = floor + (1-floor) base_k
//   p = sigmoid(pg) (0 without the protect gate);  gamma[k,b,h,t] = base'_k (1-p) + p;  omp[b,t,h] = 1 - p
//   w = K softmax_k(score) (1 without scores);  coef[k,b,h,t] = w_k e^{i phase_k}
// One thread per (b,t,h); the backward writes d(dt), d(pg), d(phase), d(score) and per-CTA partial sums
// of d(x_k) over its tokens, [P, H, K], from which d(dt_bias) and d(off) follow.
// ------------------------------------------------------------------------------------------------
struct GateParams {
  const float *dt, *pg, *phase, *score;      // [B,T,H], [B,T,H], [B,T,H,K], [B,T,H,K] (pg/phase/score may be null)
  const float *dt_bias, *off;                // [H], [K] (off may be null)
  float *gamma, *omp, *coef;                 // fwd out: [K,B,H,T], [B,T,H] (null without pg), [K,B,H,T,2] (null if K == 1 and no phase)
  const float *dgamma, *domp, *dcoef;        // bwd in
  float *ddt, *dpg, *dphase, *dscore, *dx_part;   // bwd out; dx_part [P,H,K]
  float floor_;
  int B, T, H, K;
};

template <bool BWD>
__global__ void __launch_bounds__(256) k_pam_gates(GateParams p) {
  extern __shared__ float s_part[];          // [H*K] (backward)
  const int HK = p.H * p.K;
  if (BWD) {
    for (int i = threadIdx.x; i < HK; i += blockDim.x) s_part[i] = 0.f;
    __syncthreads();
  }
  const int64_t n = (int64_t)p.B * p.T * p.H;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    const int h = (int)(e % p.H);
    const int64_t bt = e / p.H;
    const int b = (int)(bt / p.T), t = (int)(bt - (int64_t)b * p.T);
    const float dtv = p.dt[e] + p.dt_bias[h];
    const float pr = p.pg ? sigmoidf_(p.pg[e]) : 0.f;
    float sc[QPAM_MAX_STATES], w[QPAM_MAX_STATES];
    float wmax = -INFINITY, wsum = 0.f;
    if (p.score) {
      for (int k = 0; k < p.K; ++k) { sc[k] = p.score[e * p.K + k]; wmax = fmaxf(wmax, sc[k]); }
      for (int k = 0; k < p.K; ++k) { w[k] = __expf(sc[k] - wmax); wsum += w[k]; }
      for (int k = 0; k < p.K; ++k) w[k] = w[k] / wsum * (float)p.K;
    } else {
      for (int k = 0; k < p.K; ++k) w[k] = 1.f;
    }
    float dp = 0.f, ddt = 0.f, wdw = 0.f, dw[QPAM_MAX_STATES];
    for (int k = 0; k < p.K; ++k) {
      const float x = dtv + (p.off ? p.off[k] : 0.f);
      const float base = sigmoidf_(-x);
      const float basef = p.floor_ > 0.f ? p.floor_ + (1.f - p.floor_) * base : base;
      const int64_t gi = (((int64_t)k * p.B + b) * p.H + h) * p.T + t;
      float sn = 0.f, cs = 1.f;
      const bool has_coef = p.coef != nullptr || p.dcoef != nullptr;
      if (has_coef && p.phase) sincosf(p.phase[e * p.K + k], &sn, &cs);
      if (!BWD) {
        p.gamma[gi] = basef * (1.f - pr) + pr;
        if (p.coef) *reinterpret_cast<float2*>(p.coef + gi * 2) = make_float2(w[k] * cs, w[k] * sn);
      } else {
        const float dg = p.dgamma[gi];
        dp += dg * (1.f - basef);
        const float dx = -(1.f - (p.floor_ > 0.f ? p.floor_ : 0.f)) * dg * (1.f - pr) * base * (1.f - base);
        ddt += dx;
        atomicAdd(&s_part[h * p.K + k], dx);
        dw[k] = 0.f;
        if (p.dcoef) {
          const float2 dc = *reinterpret_cast<const float2*>(p.dcoef + gi * 2);
          dw[k] = cs * dc.x + sn * dc.y;
          if (p.dphase) p.dphase[e * p.K + k] = w[k] * (cs * dc.y - sn * dc.x);
          wdw += w[k] * dw[k];
        } else if (p.dphase) {
          p.dphase[e * p.K + k] = 0.f;
        }
      }
    }
    if (!BWD) {
      if (p.omp) p.omp[e] = 1.f - pr;
    } else {
      p.ddt[e] = ddt;
      if (p.dpg) {
        if (p.domp) dp -= p.domp[e];
        p.dpg[e] = dp * pr * (1.f - pr);
      }
      if (p.dscore)
        for (int k = 0; k < p.K; ++k) p.dscore[e * p.K + k] = w[k] * (dw[k] - wdw / (float)p.K);
    }
  }
  if (BWD) {
    __syncthreads();
    for (int i = threadIdx.x; i < HK; i += blockDim.x) p.dx_part[(int64_t)blockIdx.x * HK + i] = s_part[i];
  }
}
}  // namespace
}  // namespace qpam

namespace qpam {
namespace {
using namespace ew;
// |z| = sqrt(re^2 + im^2 + 1e-8) of [n] complex values -> [n];  backward dz = dm z / |z|.
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) k_cmagnitude(const T* __restrict__ z, const T* __restrict__ dm, T* __restrict__ out, int64_t n) {
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float re[4], im[4];
    V4<T>::ld(z + i * 2, re, im);
    if (!BWD) {
      float m[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) m[j] = mag_inv(re[j] * re[j] + im[j] * im[j] + MAG_EPS).mag;
      E4<T>::st(out + i, m);
    } else {
      float g[4];
      E4<T>::ld(dm + i, g);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float s = g[j] * mag_inv(re[j] * re[j] + im[j] * im[j] + MAG_EPS).rmag;
        re[j] *= s;
        im[j] *= s;
      }
      V4<T>::st(out + i * 2, re, im);
    }
  }
}
}  // namespace
}  // namespace qpam

static int state_combine(bool bwd, const void* const* yk, void* const* dyk, const float* coef, void* y, float* dcoef,
                         int32_t dtype, int32_t K, int64_t R, int32_t d, void* stream, int32_t H = 0, int32_t T = 0) {
  QPAM_REQUIRE(yk && coef && y && (!bwd || (dyk && dcoef)), "state_combine: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && K >= 1 && K <= QPAM_MAX_STATES && R >= 0, "state_combine: bad dtype, K or row count");
  QPAM_REQUIRE(d >= 4 && d <= 128 && (d & (d - 1)) == 0, "state_combine: d must be a power of two in [4,128] (got %d)", d);
  if (R == 0) return QPAM_OK;
  CombineParams p{};
  for (int k = 0; k < K; ++k) {
    QPAM_REQUIRE(yk[k] && (!bwd || dyk[k]), "state_combine: NULL state tensor");
    p.yk[k] = yk[k];
    p.dyk[k] = bwd ? dyk[k] : nullptr;
  }
  p.coef = coef; p.y = y; p.dcoef = dcoef; p.R = R; p.d = d; p.K = K; p.H = H; p.T = T;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = R * (d / 4);
  const int grid = (int)std::min<int64_t>((total + 255) / 256, sm_count() * 16);
#define QPAM_COMBINE(TT, KK_)                                                   \
  if (K == KK_) {                                                              \
    if (bwd) k_state_combine<TT, true, KK_><<<grid, 256, 0, st>>>(p);          \
    else k_state_combine<TT, false, KK_><<<grid, 256, 0, st>>>(p);             \
  }
  if (dtype == QPAM_F32) {
    QPAM_COMBINE(float, 1) QPAM_COMBINE(float, 2) QPAM_COMBINE(float, 3) QPAM_COMBINE(float, 4)
  } else {
    QPAM_COMBINE(__nv_bfloat16, 1) QPAM_COMBINE(__nv_bfloat16, 2) QPAM_COMBINE(__nv_bfloat16, 3) QPAM_COMBINE(__nv_bfloat16, 4)
  }
#undef QPAM_COMBINE
  if (bwd) { QPAM_LAUNCH_CHECK("k_state_combine_bwd"); } else { QPAM_LAUNCH_CHECK("k_state_combine_fwd"); }
  return QPAM_OK;
}

extern "C" int qpam_state_combine_fwd(const void* const* yk, const float* coef, void* y, int32_t dtype, int32_t K,
                                      int64_t R, int32_t d, void* stream) {
  return state_combine(false, yk, nullptr, coef, y, nullptr, dtype, K, R, d, stream);
}

extern "C" int qpam_state_combine_bwd(const void* const* yk, const float* coef, const void* dy, void* const* dyk,
                                      float* dcoef, int32_t dtype, int32_t K, int64_t R, int32_t d, void* stream) {
  return state_combine(true, yk, dyk, coef, const_cast<void*>(dy), dcoef, dtype, K, R, d, stream);
}

template <typename TX, typename TD>
static int scaled_residual(bool bwd, const void* x_or_dout, const void* delta, const float* s, void* out_or_ddelta,
                           float* ds_part, int32_t P, int64_t n, cudaStream_t st) {
  if (!bwd) {
    const int grid = (int)std::min<int64_t>((n / 4 + 255) / 256 + 1, sm_count() * 8);
    k_scaled_residual_fwd<TX, TD><<<grid, 256, 0, st>>>((const TX*)x_or_dout, (const TD*)delta, s, (TX*)out_or_ddelta, n);
    QPAM_LAUNCH_CHECK("k_scaled_residual_fwd");
  } else {
    k_scaled_residual_bwd<TX, TD><<<P, 256, 0, st>>>((const TX*)x_or_dout, (const TD*)delta, s, (TD*)out_or_ddelta, ds_part, n);
    QPAM_LAUNCH_CHECK("k_scaled_residual_bwd");
  }
  return QPAM_OK;
}

extern "C" int qpam_scaled_residual_fwd(const void* x, int32_t x_dtype, const void* delta, int32_t d_dtype,
                                        const float* scale, void* out, int64_t n, void* stream) {
  QPAM_REQUIRE(x && delta && scale && out, "scaled_residual_fwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(x_dtype) && is_dtype(d_dtype) && n >= 0 && n % 4 == 0, "scaled_residual_fwd: bad dtype, or a size that is not a multiple of 4");
  if (n == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define QPAM_SR_F(TX, TD) scaled_residual<TX, TD>(false, x, delta, scale, out, nullptr, 0, n, st)
  if (x_dtype == QPAM_F32 && d_dtype == QPAM_F32) return QPAM_SR_F(float, float);
  if (x_dtype == QPAM_F32) return QPAM_SR_F(float, __nv_bfloat16);
  if (d_dtype == QPAM_BF16) return QPAM_SR_F(__nv_bfloat16, __nv_bfloat16);
  return QPAM_SR_F(__nv_bfloat16, float);
#undef QPAM_SR_F
}

extern "C" int qpam_scaled_residual_bwd(const void* dout, int32_t x_dtype, const void* delta, int32_t d_dtype,
                                        const float* scale, void* ddelta, float* dscale_partials, int32_t P,
                                        int64_t n, void* stream) {
  QPAM_REQUIRE(dout && delta && scale && ddelta && dscale_partials, "scaled_residual_bwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(x_dtype) && is_dtype(d_dtype) && n > 0 && n % 4 == 0 && P > 0 && P <= 65535, "scaled_residual_bwd: bad dtype, size (multiple of 4) or partial count");
  cudaStream_t st = (cudaStream_t)stream;
#define QPAM_SR_B(TX, TD) scaled_residual<TX, TD>(true, dout, delta, scale, ddelta, dscale_partials, P, n, st)
  if (x_dtype == QPAM_F32 && d_dtype == QPAM_F32) return QPAM_SR_B(float, float);
  if (x_dtype == QPAM_F32) return QPAM_SR_B(float, __nv_bfloat16);
  if (d_dtype == QPAM_BF16) return QPAM_SR_B(__nv_bfloat16, __nv_bfloat16);
  return QPAM_SR_B(__nv_bfloat16, float);
#undef QPAM_SR_B
}

extern "C" int qpam_block_weight_fwd(const void* wr, const void* wi, int32_t w_dtype, void* w, int32_t out_dtype,
                                     int32_t out_dim, int32_t in_dim, void* stream) {
  QPAM_REQUIRE(wr && wi && w, "block_weight_fwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(w_dtype) && is_dtype(out_dtype) && out_dim > 0 && in_dim > 0, "block_weight_fwd: bad dtype or shape");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (int)std::min<int64_t>(((int64_t)out_dim * in_dim + 255) / 256, sm_count() * 8);
#define QPAM_BW(TW, TO) k_block_weight_fwd<TW, TO><<<grid, 256, 0, st>>>((const TW*)wr, (const TW*)wi, (TO*)w, out_dim, in_dim)
  if (w_dtype == QPAM_F32 && out_dtype == QPAM_F32) QPAM_BW(float, float);
  else if (w_dtype == QPAM_F32) QPAM_BW(float, __nv_bfloat16);
  else if (out_dtype == QPAM_BF16) QPAM_BW(__nv_bfloat16, __nv_bfloat16);
  else QPAM_BW(__nv_bfloat16, float);
#undef QPAM_BW
  QPAM_LAUNCH_CHECK("k_block_weight_fwd");
  return QPAM_OK;
}

extern "C" int qpam_block_weight_bwd(const void* dw, int32_t out_dtype, void* dwr, void* dwi, int32_t w_dtype,
                                     int32_t out_dim, int32_t in_dim, void* stream) {
  QPAM_REQUIRE(dw && dwr && dwi, "block_weight_bwd: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(w_dtype) && is_dtype(out_dtype) && out_dim > 0 && in_dim > 0, "block_weight_bwd: bad dtype or shape");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (int)std::min<int64_t>(((int64_t)out_dim * in_dim + 255) / 256, sm_count() * 8);
#define QPAM_BW(TW, TO) k_block_weight_bwd<TW, TO><<<grid, 256, 0, st>>>((const TO*)dw, (TW*)dwr, (TW*)dwi, out_dim, in_dim)
  if (w_dtype == QPAM_F32 && out_dtype == QPAM_F32) QPAM_BW(float, float);
  else if (w_dtype == QPAM_F32) QPAM_BW(float, __nv_bfloat16);
  else if (out_dtype == QPAM_BF16) QPAM_BW(__nv_bfloat16, __nv_bfloat16);
  else QPAM_BW(__nv_bfloat16, float);
#undef QPAM_BW
  QPAM_LAUNCH_CHECK("k_block_weight_bwd");
  return QPAM_OK;
}

extern "C" int qpam_state_combine_tokens_fwd(const void* const* yk, const float* coef, void* y, int32_t dtype, int32_t K,
                                             int32_t B, int32_t H, int32_t T, int32_t d, void* stream) {
  QPAM_REQUIRE(B > 0 && H > 0 && T > 0, "state_combine_tokens: empty shape");
  return state_combine(false, yk, nullptr, coef, y, nullptr, dtype, K, (int64_t)B * H * T, d, stream, H, T);
}

static int pam_gates(bool bwd, GateParams& p, int32_t P, void* stream) {
  QPAM_REQUIRE(p.dt && p.dt_bias, "pam_gates: NULL pointer argument");
  QPAM_REQUIRE(p.B > 0 && p.T > 0 && p.H > 0 && p.K >= 1 && p.K <= QPAM_MAX_STATES, "pam_gates: bad shape (K in [1,%d])", QPAM_MAX_STATES);
  QPAM_REQUIRE(!p.score || p.K > 1, "pam_gates: routing scores need K > 1");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n = (int64_t)p.B * p.T * p.H;
  if (!bwd) {
    QPAM_REQUIRE(p.gamma && (!p.pg || p.omp), "pam_gates_fwd: NULL output");
    const int grid = (int)std::min<int64_t>((n + 255) / 256, sm_count() * 8);
    k_pam_gates<false><<<grid, 256, 0, st>>>(p);
    QPAM_LAUNCH_CHECK("k_pam_gates_fwd");
  } else {
    QPAM_REQUIRE(p.dgamma && p.ddt && p.dx_part && (!p.pg || p.dpg), "pam_gates_bwd: NULL pointer argument");
    QPAM_REQUIRE(P > 0 && P <= 65535, "pam_gates_bwd: partial rows must be in [1, 65535]");   // one CTA per partial row
    k_pam_gates<true><<<P, 256, sizeof(float) * p.H * p.K, st>>>(p);
    QPAM_LAUNCH_CHECK("k_pam_gates_bwd");
  }
  return QPAM_OK;
}

extern "C" int qpam_pam_gates_fwd(const float* dt, const float* pg, const float* phase, const float* score,
                                  const float* dt_bias, const float* state_dt_offset, float gamma_floor,
                                  float* gamma, float* omp, float* coef, int32_t B, int32_t T, int32_t H, int32_t K,
                                  void* stream) {
  GateParams p{};
  p.dt = dt; p.pg = pg; p.phase = phase; p.score = score; p.dt_bias = dt_bias; p.off = state_dt_offset;
  p.gamma = gamma; p.omp = omp; p.coef = coef; p.floor_ = gamma_floor; p.B = B; p.T = T; p.H = H; p.K = K;
  return pam_gates(false, p, 0, stream);
}

extern "C" int qpam_pam_gates_bwd(const float* dt, const float* pg, const float* phase, const float* score,
                                  const float* dt_bias, const float* state_dt_offset, float gamma_floor,
                                  const float* dgamma, const float* domp, const float* dcoef, float* ddt, float* dpg,
                                  float* dphase, float* dscore, float* dx_partials, int32_t P, int32_t B, int32_t T,
                                  int32_t H, int32_t K, void* stream) {
  GateParams p{};
  p.dt = dt; p.pg = pg; p.phase = phase; p.score = score; p.dt_bias = dt_bias; p.off = state_dt_offset;
  p.dgamma = dgamma; p.domp = domp; p.dcoef = dcoef; p.ddt = ddt; p.dpg = dpg; p.dphase = dphase; p.dscore = dscore;
  p.dx_part = dx_partials; p.floor_ = gamma_floor; p.B = B; p.T = T; p.H = H; p.K = K;
  return pam_gates(true, p, P, stream);
}

extern "C" int qpam_cmagnitude_fwd(const void* z, int32_t dtype, void* mag, int64_t n, void* stream) {
  QPAM_REQUIRE(z && mag && is_dtype(dtype) && n >= 0 && n % 4 == 0, "cmagnitude_fwd: NULL pointer, bad dtype or n not a multiple of 4");
  if (n == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (int)std::min<int64_t>((n / 4 + 255) / 256, sm_count() * 8);
  if (dtype == QPAM_F32) k_cmagnitude<float, false><<<grid, 256, 0, st>>>((const float*)z, nullptr, (float*)mag, n);
  else k_cmagnitude<__nv_bfloat16, false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)z, nullptr, (__nv_bfloat16*)mag, n);
  QPAM_LAUNCH_CHECK("k_cmagnitude_fwd");
  return QPAM_OK;
}

extern "C" int qpam_cmagnitude_bwd(const void* z, const void* dmag, int32_t dtype, void* dz, int64_t n, void* stream) {
  QPAM_REQUIRE(z && dmag && dz && is_dtype(dtype) && n > 0 && n % 4 == 0, "cmagnitude_bwd: NULL pointer, bad dtype or n not a multiple of 4");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = (int)std::min<int64_t>((n / 4 + 255) / 256, sm_count() * 8);
  if (dtype == QPAM_F32) k_cmagnitude<float, true><<<grid, 256, 0, st>>>((const float*)z, (const float*)dmag, (float*)dz, n);
  else k_cmagnitude<__nv_bfloat16, true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)z, (const __nv_bfloat16*)dmag, (__nv_bfloat16*)dz, n);
  QPAM_LAUNCH_CHECK("k_cmagnitude_bwd");
  return QPAM_OK;
}

extern "C" int qpam_state_combine_tokens_bwd(const void* const* yk, const float* coef, const void* dy, void* const* dyk,
                                             float* dcoef, int32_t dtype, int32_t K, int32_t B, int32_t H, int32_t T,
                                             int32_t d, void* stream) {
  QPAM_REQUIRE(B > 0 && H > 0 && T > 0, "state_combine_tokens: empty shape");
  return state_combine(true, yk, dyk, coef, const_cast<void*>(dy), dcoef, dtype, K, (int64_t)B * H * T, d, stream, H, T);
}
