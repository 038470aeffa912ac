// Register-level helpers shared by the element-wise kernels: 16-byte loads/stores of 4 interleaved
// complex channels, warp sums, the guarded magnitude.
#pragma once
#include "common.cuh"

namespace qpam {
namespace ew {

constexpr float MAG_EPS = 1e-8f;  // inside the square root and beside the magnitude, as the reference

// 4 complex channels (re,im interleaved) <-> registers
template <typename T>
struct V4;
template <>
struct V4<float> {
  static __device__ __forceinline__ void ld(const float* p, float (&r)[4], float (&i)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    r[0] = a.x; i[0] = a.y; r[1] = a.z; i[1] = a.w; r[2] = b.x; i[2] = b.y; r[3] = b.z; i[3] = b.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&r)[4], const float (&i)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(r[0], i[0], r[1], i[1]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(r[2], i[2], r[3], i[3]);
  }
};
template <>
struct V4<__nv_bfloat16> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&r)[4], float (&i)[4]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      r[j] = __uint_as_float(w[j] << 16);
      i[j] = __uint_as_float(w[j] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&r)[4], const float (&i)[4]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(r[j], i[j]);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// 4 consecutive scalars <-> registers (16-byte / 8-byte accesses)
template <typename T>
struct E4;
template <>
struct E4<float> {
  static __device__ __forceinline__ void ld(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct E4<__nv_bfloat16> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Approximate reciprocal / square root (about 2 ulp): the IEEE forms cost several times more issue slots, and
// these kernels do ~10 of them per 8 bytes moved.
__device__ __forceinline__ float frcp_(float x) { return __fdividef(1.f, x); }
__device__ __forceinline__ float fsqrt_(float x) { return x * rsqrtf(x); }  // x >= 1e-8 here, never 0
// |z|, 1/(|z| + 1e-8) and 1/|z| of m2 = re^2 + im^2 + 1e-8 from ONE special-function instruction:
// with rs = rsqrt(m2):  |z| = m2 rs,  1/(|z| + e) = rs / (1 + e rs) = rs (1 - t + t^2 - ...), t = e rs <= 1e-4
// (m2 >= 1e-8), so the two kept terms leave an error below 1e-12.  These kernels are otherwise bound by the
// special-function unit (16 results per clock per SM), not by HBM.
struct MagInv {
  float mag, inv, rmag;
};
__device__ __forceinline__ MagInv mag_inv(float m2) {
  const float rs = rsqrtf(m2);
  const float t = MAG_EPS * rs;
  return {m2 * rs, rs * (1.f - t + t * t), rs};
}
// sigmoid from one special-function instruction (tanh.approx, abs. error ~5e-4): for results stored as bf16
__device__ __forceinline__ float sigmoid_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(0.5f * x));
  return fmaf(0.5f, y, 0.5f);
}
__device__ __forceinline__ float sigmoidf_(float x) { return frcp_(1.f + __expf(-x)); }

// Threads per CTA for kernels whose threads each own one group of 4 channels: the largest multiple of 32
// (up to 256) that divides the group count, so that no CTA runs mostly idle; 256 when none does.  Up to
// 512 groups get one thread each.  Kernels launched with it declare __launch_bounds__(512).
inline int pick_threads(int groups) {
  if (groups <= 512) return (groups + 31) / 32 * 32;
  for (int t = 256; t >= 64; t -= 32)
    if (groups % t == 0) return t;
  return 256;
}
inline bool is_dtype(int32_t d) { return d == QPAM_F32 || d == QPAM_BF16; }

}  // namespace ew
}  // namespace qpam
