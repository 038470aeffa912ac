// Shared device/host helpers for the PAM kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/qllm2_pam.h"

namespace qpam {

// ------------------------------------------------------------------ error reporting
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
int sm_count();   // multiprocessors of the current device

#define QPAM_REQUIRE(cond, ...)            \
  do {                                     \
    if (!(cond)) {                         \
      ::qpam::set_error(__VA_ARGS__);      \
      return QPAM_EINVAL;                  \
    }                                      \
  } while (0)

#define QPAM_CUDA(call)                                              \
  do {                                                               \
    cudaError_t e__ = (call);                                        \
    if (e__ != cudaSuccess) return ::qpam::cuda_fail(e__, #call);    \
  } while (0)

// Counts the launch and, while profiling is on, records an event behind it on `stream_`.
void note_launch(const char* name, cudaStream_t stream_);
// True while qpam_profile_begin .. qpam_profile_end is recording (entry points then keep to one stream).
bool profiling_active();

#define QPAM_LAUNCH_CHECK_ON(name, stream_)                              \
  do {                                                                   \
    cudaError_t e__ = cudaGetLastError();                                \
    if (e__ != cudaSuccess) return ::qpam::cuda_fail(e__, "launch " name); \
    ::qpam::note_launch(name, stream_);                                  \
  } while (0)
// every launch site names its stream `st`
#define QPAM_LAUNCH_CHECK(name) QPAM_LAUNCH_CHECK_ON(name, st)

// ------------------------------------------------------------------ io element access
template <typename T>
struct IO;
template <>
struct IO<float> {
  static __device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void st2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <>
struct IO<__nv_bfloat16> {
  static __device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void st2(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __float22bfloat162_rn(v);
  }
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// ------------------------------------------------------------------ complex helpers
__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
__device__ __forceinline__ float2 cmulc(float2 a, float2 b) {  // a * conj(b)
  return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
__device__ __forceinline__ float2 cscale(float2 a, float s) { return make_float2(a.x * s, a.y * s); }

// acc += opA(a) * opB(b)
template <bool CA, bool CB>
__device__ __forceinline__ void cfma(float2& acc, float2 a, float2 b) {
  const float ay = CA ? -a.y : a.y;
  const float by = CB ? -b.y : b.y;
  acc.x = fmaf(a.x, b.x, acc.x);
  acc.x = fmaf(-ay, by, acc.x);
  acc.y = fmaf(a.x, by, acc.y);
  acc.y = fmaf(ay, b.x, acc.y);
}

// ------------------------------------------------------------------ chunk geometry
// The scan tiles every sequence into chunks of CH tokens; chunks never straddle a sequence
// boundary (CH is the tile of the FFMA kernels; ChunkGeom::ch is the tile in use).  Sequence s owns state slots [slot_base(s), slot_base(s)+nchunks(s)] (one more
// slot than chunks: slot c holds the state BEFORE chunk c, the last the final state).
constexpr int CH = 64;

struct ChunkGeom {
  const int32_t* cu_seqlens;    // device, or nullptr
  const int32_t* chunk_prefix;  // device int32[S+1] (packed mode only): chunks before sequence s
  int32_t S;                    // sequences
  int32_t T;                    // tokens per sequence (batch mode) / packed total
  int32_t nc_uniform;           // chunks per sequence in batch mode
  int32_t ch;                   // tokens per chunk (64 for the FFMA kernels, 128 for the tensor-core ones)
};

struct ChunkLoc {
  int32_t seq;      // sequence index
  int32_t c;        // chunk within sequence
  int32_t nc;       // chunks in this sequence
  int32_t b;        // batch row of the token tensors (0 in packed mode)
  int32_t t0;       // first token (index along the T axis of the token tensors)
  int32_t len;      // tokens in the chunk (1..CH)
  int64_t slot0;    // state slot of the sequence's first chunk
  bool valid;
};

__device__ __forceinline__ ChunkLoc locate_chunk(const ChunkGeom& g, int32_t x) {
  ChunkLoc L;
  L.valid = false;
  if (g.cu_seqlens == nullptr) {
    const int32_t seq = x / g.nc_uniform;
    if (seq >= g.S) return L;
    L.seq = seq;
    L.c = x - seq * g.nc_uniform;
    L.nc = g.nc_uniform;
    L.b = seq;
    L.t0 = L.c * g.ch;
    L.len = min(g.ch, g.T - L.t0);
    L.slot0 = (int64_t)seq * (g.nc_uniform + 1);
    L.valid = true;
    return L;
  }
  if (x >= g.chunk_prefix[g.S]) return L;
  int lo = 0, hi = g.S;  // find the last s with prefix[s] <= x (skipping empty sequences)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (g.chunk_prefix[mid] <= x) lo = mid; else hi = mid;
  }
  L.seq = lo;
  L.c = x - g.chunk_prefix[lo];
  L.nc = g.chunk_prefix[lo + 1] - g.chunk_prefix[lo];
  L.b = 0;
  const int32_t a = g.cu_seqlens[lo], e = g.cu_seqlens[lo + 1];
  L.t0 = a + L.c * g.ch;
  L.len = min(g.ch, e - L.t0);
  L.slot0 = (int64_t)g.chunk_prefix[lo] + lo;
  L.valid = true;
  return L;
}

}  // namespace qpam
