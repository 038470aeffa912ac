// Forward-only fusions of a V11 block for inference (prefill and the per-token decode step), where
// no activation has to be kept for a backward pass:
//   k_act_gate_packed   modSwish/modReLU of the `up` half + the gated-unit product, from ONE
//                       projection output [N, gate | up]                (v11/model.py CGU forward)
//   k_residual_cnorm    z += s * delta  and  xn = ComplexNorm(z) (+ |xn|) in one sweep over the row
//   k_pam_front         decay / protect gate / phase-routing read-out weights AND the head split +
//                       rotary rotation + protect scaling, from the fused projection output
//                       (PhaseAssociativeLayer._project, _gamma_and_vprime, phase routing:
//                       v11/model.py:271-350, 630-655)
// The reference runs each of these as 10-30 separate torch operators per layer and token
// (v11/model.py:1206-1245 drives them once per generated token).
#include <algorithm>

#include "common.cuh"
#include "elementwise.cuh"

namespace qpam {
namespace {
using namespace ew;

template <typename T>
__device__ __forceinline__ float rnd(float x);
template <>
__device__ __forceinline__ float rnd<float>(float x) { return x; }
template <>
__device__ __forceinline__ float rnd<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// sigmoid in the precision the result is stored in
template <typename T>
__device__ __forceinline__ float sig(float x);
template <>
__device__ __forceinline__ float sig<float>(float x) { return sigmoidf_(x); }
template <>
__device__ __forceinline__ float sig<__nv_bfloat16>(float x) { return sigmoid_approx(x); }

template <typename T, bool SWISH>
__global__ void __launch_bounds__(512) k_act_gate_packed(const T* __restrict__ gu, int64_t ld,
                                                         const float* __restrict__ bias,
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
  constexpr int U = 2;  // rows in flight per thread: their four loads are issued before any arithmetic
  for (int64_t row0 = (int64_t)blockIdx.y * U; row0 < N; row0 += (int64_t)gridDim.y * U) {
    float ar[U][4], ai[U][4], ur[U][4], ui[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t row = row0 + u < N ? row0 + u : N - 1;
      V4<T>::ld(gu + row * ld + g * 8, ar[u], ai[u]);
      V4<T>::ld(gu + row * ld + 2 * C + g * 8, ur[u], ui[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (row0 + u >= N) break;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const MagInv um_ = mag_inv(ur[u][j] * ur[u][j] + ui[u][j] * ui[u][j] + MAG_EPS); const float um = um_.mag;
        const float act = SWISH ? um * sig<T>(be4[j] * um + b4[j]) : fmaxf(um + b4[j], 0.f);
        const float f = act * um_.inv;
        const MagInv gm_ = mag_inv(ar[u][j] * ar[u][j] + ai[u][j] * ai[u][j] + MAG_EPS); const float gm = gm_.mag;
        const float h = sig<T>(gm) * gm_.inv * f;
        const float pr = ar[u][j] * ur[u][j] - ai[u][j] * ui[u][j], pi = ar[u][j] * ui[u][j] + ai[u][j] * ur[u][j];
        ar[u][j] = pr * h;
        ai[u][j] = pi * h;
      }
      V4<T>::st(out + ((row0 + u) * C + g * 4) * 2, ar[u], ai[u]);
    }
  }
}

// One warp per row.  The updated row is written first and read back for the second sweep (same
// thread, L1/L2 hits), so any width works without a register cache.
template <typename T>
__global__ void __launch_bounds__(128) k_residual_cnorm(T* __restrict__ z, const T* __restrict__ delta,
                                                        const float* __restrict__ res_scale,
                                                        const float* __restrict__ norm_scale, T* __restrict__ xn,
                                                        T* __restrict__ mag_out, int64_t N, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int groups = D >> 2;
  const float s = res_scale ? *res_scale : 1.f;
  for (int64_t row = warp; row < N; row += nwarps) {
    T* zr = z + row * (int64_t)D * 2;
    float ss = 0.f;
    for (int g = lane; g < groups; g += 32) {
      float re[4], im[4];
      V4<T>::ld(zr + g * 8, re, im);
      if (delta) {
        float dr[4], di[4];
        V4<T>::ld(delta + row * (int64_t)D * 2 + g * 8, dr, di);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          re[j] = fmaf(s, dr[j], re[j]);
          im[j] = fmaf(s, di[j], im[j]);
        }
        V4<T>::st(zr + g * 8, re, im);
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // the norm sees the stored (rounded) residual stream, as the modules do
          re[j] = rnd<T>(re[j]);
          im[j] = rnd<T>(im[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += re[j] * re[j] + im[j] * im[j] + MAG_EPS;
    }
    ss = warp_sum(ss);
    if (!xn) continue;
    const float rrms = rsqrtf(ss / (float)D + eps);
    for (int g = lane; g < groups; g += 32) {
      float re[4], im[4], mg[4];
      V4<T>::ld(zr + g * 8, re, im);
      const float4 sc = *reinterpret_cast<const float4*>(norm_scale + g * 4);
      const float s4[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const MagInv m_ = mag_inv(re[j] * re[j] + im[j] * im[j] + MAG_EPS); const float m = m_.mag;
        const float w = m * m_.inv * rrms * s4[j];
        re[j] *= w;
        im[j] *= w;
      }
      V4<T>::st(xn + row * (int64_t)D * 2 + g * 8, re, im);
      if (mag_out) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // magnitude of the stored (rounded) values
          const float r0 = rnd<T>(re[j]), i0 = rnd<T>(im[j]);
          mg[j] = fsqrt_(r0 * r0 + i0 * i0 + MAG_EPS);
        }
        T* mp = mag_out + row * (int64_t)D + g * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) IO<T>::st(mp + j, mg[j]);
      }
    }
  }
}

// Few rows (a decode step): one CTA per row, one vector of 4 channels per thread, a single sweep.
template <typename T>
__global__ void __launch_bounds__(1024) k_residual_cnorm_row(T* __restrict__ z, const T* __restrict__ delta,
                                                             const float* __restrict__ res_scale,
                                                             const float* __restrict__ norm_scale,
                                                             T* __restrict__ xn, T* __restrict__ mag_out, int D,
                                                             float eps) {
  __shared__ float s_part[32];
  const int64_t row = blockIdx.x;
  const int g = threadIdx.x, groups = D >> 2;
  const bool on = g < groups;
  float re[4] = {0.f, 0.f, 0.f, 0.f}, im[4] = {0.f, 0.f, 0.f, 0.f}, ss = 0.f;
  if (on) {
    V4<T>::ld(z + row * (int64_t)D * 2 + g * 8, re, im);
    if (delta) {
      const float s = res_scale ? *res_scale : 1.f;
      float dr[4], di[4];
      V4<T>::ld(delta + row * (int64_t)D * 2 + g * 8, dr, di);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        re[j] = fmaf(s, dr[j], re[j]);
        im[j] = fmaf(s, di[j], im[j]);
      }
      V4<T>::st(z + row * (int64_t)D * 2 + g * 8, re, im);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        re[j] = rnd<T>(re[j]);
        im[j] = rnd<T>(im[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += re[j] * re[j] + im[j] * im[j] + MAG_EPS;
  }
  if (!xn) return;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
  if (!on) return;
  const float rrms = rsqrtf(tot / (float)D + eps);
  const float4 sc = *reinterpret_cast<const float4*>(norm_scale + g * 4);
  const float s4[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const MagInv m_ = mag_inv(re[j] * re[j] + im[j] * im[j] + MAG_EPS); const float m = m_.mag;
    const float w = m * m_.inv * rrms * s4[j];
    re[j] *= w;
    im[j] *= w;
  }
  V4<T>::st(xn + row * (int64_t)D * 2 + g * 8, re, im);
  if (mag_out) {
    T* mp = mag_out + row * (int64_t)D + g * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float r0 = rnd<T>(re[j]), i0 = rnd<T>(im[j]);
      IO<T>::st(mp + j, fsqrt_(r0 * r0 + i0 * i0 + MAG_EPS));
    }
  }
}

struct FrontParams {
  qpam_front_args a;
};

constexpr int FRONT_U = 1;  // tokens per tile (one keeps the streaming warps at ~64 registers, 4+ CTAs per SM)

// Threads [0, main_threads): one (head, group of 4 channels) of FRONT_U consecutive tokens each, moving q, k
// and v of it (all loads first).  Threads [main_threads, blockDim): one (head, state) pair each, writing the
// decay and the read-out weight of those tokens -- a chain of small dependent loads and transcendentals that
// runs beside the streaming warps instead of at their tail.
template <typename T>
__global__ void __launch_bounds__(512) k_pam_front(FrontParams fp, int main_threads) {
  const qpam_front_args& a = fp.a;
  const int H = a.H, K = a.K, d = a.d;
  const int gph = d >> 2;
  const int per_tok = H * gph;
  const int64_t ntok = (int64_t)a.B * a.T;
  const int64_t ntile = (ntok + FRONT_U - 1) / FRONT_U;
  const int64_t side_stride = (int64_t)H * d * 2;
  if ((int)threadIdx.x >= main_threads) {
    const int gate_threads = blockDim.x - main_threads;
    for (int64_t tile = blockIdx.x; tile < ntile; tile += gridDim.x) {
      for (int e = threadIdx.x - main_threads; e < FRONT_U * H * K; e += gate_threads) {
        const int u = e / (H * K), hk = e - u * H * K, h = hk / K, k = hk - h * K;
        const int64_t tok = tile * FRONT_U + u;
        if (tok >= ntok) continue;
        const int b = (int)(tok / a.T), t = (int)(tok - (int64_t)b * a.T);
        const float x = IO<T>::ld(reinterpret_cast<const T*>(a.dt) + tok * a.ld_dt + h) + a.dt_bias[h] +
                        (a.state_dt_offset ? a.state_dt_offset[k] : 0.f);
        const float p = a.pg ? sigmoidf_(IO<T>::ld(reinterpret_cast<const T*>(a.pg) + tok * a.ld_pg + h)) : 0.f;
        float w = 1.f, ph = 0.f;
        if (a.coef) {
          if (a.phase) ph = IO<T>::ld(reinterpret_cast<const T*>(a.phase) + tok * a.ld_phase + h * K + k);
          if (a.score) {
            const T* sc = reinterpret_cast<const T*>(a.score) + tok * a.ld_score + h * K;
            float wmax = -INFINITY, wsum = 0.f;
            for (int kk = 0; kk < K; ++kk) wmax = fmaxf(wmax, IO<T>::ld(sc + kk));
            for (int kk = 0; kk < K; ++kk) wsum += __expf(IO<T>::ld(sc + kk) - wmax);
            w = __expf(IO<T>::ld(sc + k) - wmax) / wsum * (float)K;
          }
        }
        float base = sigmoidf_(-x);   // exp(-softplus(x)) = 1 / (1 + e^x)
        if (a.gamma_floor > 0.f) base = a.gamma_floor + (1.f - a.gamma_floor) * base;
        const int64_t gi = (((int64_t)k * a.B + b) * H + h) * a.T + t;
        a.gamma[gi] = base * (1.f - p) + p;
        if (a.coef) {
          float sn_, cs_;
          sincosf(ph, &sn_, &cs_);
          *reinterpret_cast<float2*>(a.coef + gi * 2) = make_float2(w * cs_, w * sn_);
        }
      }
    }
    return;
  }
  for (int64_t tile = blockIdx.x; tile < ntile; tile += gridDim.x) {
    for (int idx = threadIdx.x; idx < per_tok; idx += main_threads) {
      const int h = idx / gph, g = idx - h * gph;
      float re[FRONT_U][3][4], im[FRONT_U][3][4], pgv[FRONT_U];
      float4 c0[FRONT_U], c1[FRONT_U];
      int64_t dst[FRONT_U];
      bool on[FRONT_U];
#pragma unroll
      for (int u = 0; u < FRONT_U; ++u) {
        const int64_t tok = tile * FRONT_U + u;
        on[u] = tok < ntok;
        const int64_t tk = on[u] ? tok : 0;
        const int b = (int)(tk / a.T), t = (int)(tk - (int64_t)b * a.T);
        const int64_t src = tk * a.ld_qkv + (int64_t)h * d * 2 + g * 8;
        dst[u] = (((int64_t)b * H + h) * a.T + t) * (int64_t)d * 2 + g * 8;
        c0[u] = c1[u] = make_float4(1.f, 0.f, 1.f, 0.f);
        pgv[u] = 0.f;
        if (on[u]) {
#pragma unroll
          for (int w = 0; w < 3; ++w) V4<T>::ld(reinterpret_cast<const T*>(a.qkv) + src + w * side_stride, re[u][w], im[u][w]);
          if (a.pg) pgv[u] = IO<T>::ld(reinterpret_cast<const T*>(a.pg) + tk * a.ld_pg + h);
          if (a.rope) {
            int64_t pos = a.positions ? a.positions[tk] : a.offset + t;
            pos = pos < 0 ? 0 : (pos >= a.rope_len ? a.rope_len - 1 : pos);
            c0[u] = *reinterpret_cast<const float4*>(a.rope + (pos * d + g * 4) * 2);
            c1[u] = *reinterpret_cast<const float4*>(a.rope + (pos * d + g * 4) * 2 + 4);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < FRONT_U; ++u) {
        if (!on[u]) continue;
        const float keep = a.pg ? 1.f - sigmoidf_(pgv[u]) : 1.f;
        const float cs[4] = {c0[u].x, c0[u].z, c1[u].x, c1[u].z};
        const float sn[4] = {c0[u].y, c0[u].w, c1[u].y, c1[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            const float mul = w == 0 ? a.q_scale : 1.f;
            const float r0 = re[u][w][j], i0 = im[u][w][j];
            re[u][w][j] = (r0 * cs[j] - i0 * sn[j]) * mul;
            im[u][w][j] = (r0 * sn[j] + i0 * cs[j]) * mul;
          }
          re[u][2][j] *= keep;
          im[u][2][j] *= keep;
        }
        V4<T>::st(reinterpret_cast<T*>(a.q) + dst[u], re[u][0], im[u][0]);
        V4<T>::st(reinterpret_cast<T*>(a.k) + dst[u], re[u][1], im[u][1]);
        V4<T>::st(reinterpret_cast<T*>(a.v) + dst[u], re[u][2], im[u][2]);
      }
    }
  }
}

}  // namespace
}  // namespace qpam

using namespace qpam;
using namespace qpam::ew;

extern "C" int qpam_act_gate_packed_fwd(const void* gate_up, int64_t ld, int32_t dtype, const float* bias,
                                        const float* beta, void* out, int64_t N, int32_t C, void* stream) {
  QPAM_REQUIRE(gate_up && bias && out, "act_gate_packed: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(dtype) && N >= 0 && C > 0 && C % 4 == 0, "act_gate_packed: C must be a multiple of 4 (got %d)", C);
  QPAM_REQUIRE(ld >= 4 * (int64_t)C && ld % (dtype == QPAM_F32 ? 4 : 8) == 0,
               "act_gate_packed: the row stride must cover 4*C scalars and keep rows 16-byte aligned");
  if (N == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int groups = C / 4, threads = pick_threads(groups), xb = (groups + threads - 1) / threads;
  dim3 grid(xb, (unsigned)std::min<int64_t>((N + 1) / 2, std::max(1, (sm_count() * 2048) / (xb * threads))));
#define QPAM_AG(T)                                                                                                  \
  if (beta) k_act_gate_packed<T, true><<<grid, threads, 0, st>>>((const T*)gate_up, ld, bias, beta, (T*)out, N, C); \
  else k_act_gate_packed<T, false><<<grid, threads, 0, st>>>((const T*)gate_up, ld, bias, beta, (T*)out, N, C);
  if (dtype == QPAM_F32) { QPAM_AG(float) } else { QPAM_AG(__nv_bfloat16) }
#undef QPAM_AG
  QPAM_LAUNCH_CHECK("k_act_gate_packed");
  return QPAM_OK;
}

extern "C" int qpam_residual_cnorm_fwd(void* z, const void* delta, const float* res_scale, const float* norm_scale,
                                       void* xn, void* mag, int32_t dtype, int64_t N, int32_t D, float eps,
                                       void* stream) {
  QPAM_REQUIRE(z && (delta || xn), "residual_cnorm: NULL pointer argument");
  QPAM_REQUIRE(!xn || norm_scale, "residual_cnorm: the norm needs its scale vector");
  QPAM_REQUIRE(!mag || xn, "residual_cnorm: magnitudes are those of the normalised rows");
  QPAM_REQUIRE(is_dtype(dtype) && N >= 0 && D > 0 && D % 4 == 0, "residual_cnorm: D must be a multiple of 4 (got %d)", D);
  if (N == 0) return QPAM_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (N <= sm_count() * 8 && D <= 4096) {  // few rows: a CTA per row keeps every SM busy
    const int threads = (D / 4 + 31) / 32 * 32;
    if (dtype == QPAM_F32)
      k_residual_cnorm_row<float><<<(unsigned)N, threads, 0, st>>>((float*)z, (const float*)delta, res_scale, norm_scale, (float*)xn, (float*)mag, D, eps);
    else
      k_residual_cnorm_row<__nv_bfloat16><<<(unsigned)N, threads, 0, st>>>((__nv_bfloat16*)z, (const __nv_bfloat16*)delta, res_scale, norm_scale,
                                                                            (__nv_bfloat16*)xn, (__nv_bfloat16*)mag, D, eps);
    QPAM_LAUNCH_CHECK("k_residual_cnorm_row");
    return QPAM_OK;
  }
  const int blocks = (int)std::min<int64_t>((N + 3) / 4, sm_count() * 8);
  if (dtype == QPAM_F32)
    k_residual_cnorm<float><<<blocks, 128, 0, st>>>((float*)z, (const float*)delta, res_scale, norm_scale, (float*)xn, (float*)mag, N, D, eps);
  else
    k_residual_cnorm<__nv_bfloat16><<<blocks, 128, 0, st>>>((__nv_bfloat16*)z, (const __nv_bfloat16*)delta, res_scale, norm_scale,
                                                            (__nv_bfloat16*)xn, (__nv_bfloat16*)mag, N, D, eps);
  QPAM_LAUNCH_CHECK("k_residual_cnorm");
  return QPAM_OK;
}

extern "C" int qpam_pam_front_fwd(const qpam_front_args* a, void* stream) {
  QPAM_REQUIRE(a, "pam_front: NULL args");
  QPAM_REQUIRE(a->qkv && a->dt && a->dt_bias && a->q && a->k && a->v && a->gamma, "pam_front: NULL pointer argument");
  QPAM_REQUIRE(is_dtype(a->io_dtype) && a->B > 0 && a->T > 0 && a->H > 0 && a->H <= 64, "pam_front: bad dtype or shape (H <= 64)");
  QPAM_REQUIRE(a->K >= 1 && a->K <= QPAM_MAX_STATES, "pam_front: K must be in [1,%d]", QPAM_MAX_STATES);
  QPAM_REQUIRE(a->d >= 4 && a->d <= 128 && (a->d & (a->d - 1)) == 0, "pam_front: head_dim must be a power of two in [4,128]");
  const int64_t al = a->io_dtype == QPAM_F32 ? 4 : 8;
  QPAM_REQUIRE(a->ld_qkv >= 6 * (int64_t)a->H * a->d && a->ld_qkv % al == 0, "pam_front: qkv row stride too small or rows not 16-byte aligned");
  QPAM_REQUIRE(!a->rope || a->rope_len > 0, "pam_front: empty rotary table");
  QPAM_REQUIRE(!a->rope || a->positions || a->offset + a->T <= a->rope_len, "pam_front: rotary table shorter than offset + T");
  QPAM_REQUIRE(a->K == 1 || a->coef, "pam_front: K > 1 needs the read-out weight output");
  QPAM_REQUIRE(!a->score || a->coef, "pam_front: scores without read-out weights");
  cudaStream_t st = (cudaStream_t)stream;
  FrontParams fp{*a};
  const int per_tok = a->H * (a->d / 4);
  const int main_threads = std::min(pick_threads(per_tok), 384);
  const int gate_threads = std::min((FRONT_U * a->H * a->K + 31) / 32 * 32, 128);
  const int threads = main_threads + gate_threads;
  const int grid = (int)std::min<int64_t>(((int64_t)a->B * a->T + FRONT_U - 1) / FRONT_U, (sm_count() * 2048) / threads);
  if (a->io_dtype == QPAM_F32) k_pam_front<float><<<grid, threads, 0, st>>>(fp, main_threads);
  else k_pam_front<__nv_bfloat16><<<grid, threads, 0, st>>>(fp, main_threads);
  QPAM_LAUNCH_CHECK("k_pam_front");
  return QPAM_OK;
}
