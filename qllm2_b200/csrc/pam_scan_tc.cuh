// Tensor-core (tcgen05 / TMEM / TMA) kernels of the chunked PAM scan for bf16 token tensors,
// head dim 64, one state.  Chunks are 128 tokens, so every MMA is M = 128.
//
// This file: the chunk-local state sums (k_tc_chunk_outer).  The
// state sums run as real bf16 MMAs on the INTERLEAVED (re, im) rows as they sit in memory: a token
// row of 64 complex numbers is a 128-element real vector x = (r0, i0, r1, i1, ...); with
// cj(x) = (r0, -i0, ...) the real and imaginary parts of v (x) conj(k) come from the operand rows
// w cj(k), w (ki, kr) against the de-interleaved planes Re v, Im v.  The chunk outputs and
// gradients are in pam_scan_tc2.cuh.
#pragma once
#include "pam_scan_kernels.cuh"
#include "umma.cuh"

namespace qpam {
namespace tcs {

constexpr int TC = 128;   // tokens per chunk
constexpr int TD = 64;    // head dim (complex); a token row is 2*TD bf16 = 256 bytes

// byte offset of (row, 16-byte chunk c in 0..7) inside a [rows][128 B] block with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int c) { return (uint32_t)row * 128u + (uint32_t)((c ^ (row & 7)) << 4); }

__device__ __forceinline__ float2 unpack_bf162(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}
__device__ __forceinline__ uint32_t pack_bf162(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// inclusive cumulative sum of log(gamma + eps) over 128 tokens by one warp (4 tokens per lane)
// (two halves, so that a caller can put other loads between the request for the decays and their first use)
__device__ __forceinline__ void warp_cumsum128_load(float (&g)[4], const float* __restrict__ gamma, int len, int lane) {
  const int t = 4 * lane;
#pragma unroll
  for (int i = 0; i < 4; ++i) g[i] = (t + i < len) ? __ldg(gamma + t + i) : 1.f;
}
__device__ __forceinline__ void warp_cumsum128_finish(float* A, const float (&g)[4], int len, float eps, int lane) {
  const int t = 4 * lane;
  float x[4];
  // log(gamma + eps) without the full-precision logf (~500 clocks of the chain that the first barrier of a chunk job
  // waits for).  Decays close to 1 are the ones whose errors would add up over thousands of tokens, so they get the
  // series of log1p(u), u = x - 1 (exact by Sterbenz for x in [0.5, 2]), to fp32 rounding: |u| < 1/16, six terms,
  // truncation < u^7/7 < 6e-10.  The rest takes the hardware logarithm (absolute error <= 2^-22 per token; such a
  // sequence has forgotten a token after a few hundred steps, long before those errors add up to 1e-4).  Every
  // tensor-core kernel forms its decays here, so chunk sums, carried states and outputs agree.
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float xg = g[i] + eps, u = xg - 1.f;
    const float series = u * fmaf(u, fmaf(u, fmaf(u, fmaf(u, fmaf(u, -1.f / 6.f, 0.2f), -0.25f), 1.f / 3.f), -0.5f), 1.f);
    x[i] = (t + i < len) ? (fabsf(u) < 0.0625f ? series : __logf(xg)) : 0.f;
  }
  x[1] += x[0];
  x[2] += x[1];
  x[3] += x[2];
  float incl = x[3];
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  const float excl = incl - x[3];
#pragma unroll
  for (int i = 0; i < 4; ++i) A[t + i] = excl + x[i];
}
__device__ __forceinline__ void warp_cumsum128(float* A, const float* __restrict__ gamma, int len, float eps, int lane) {
  float g[4];
  warp_cumsum128_load(g, gamma, len, lane);
  warp_cumsum128_finish(A, g, len, eps, lane);
}

// ---------------------------------------------------------------------------------------------
// Chunk-local state sum  U[i][j] = sum_s w_s v_s[i] conj(k_s[j])  in transposed form, from the key tile AS THE TMA
// DELIVERS IT (interleaved re, im: no operand is built from it) and the value tile split into two weighted planes:
//   A  (MN-major, M = 128 interleaved key columns n' = 2j + c, K = 128 tokens): k'[s][n']   (kr_j at 2j, ki_j at 2j+1)
//   Br (MN-major, N = 64 value channels, K = 128): w_s Re v_s          D1[n'][i] = sum_s A[s][n'] Br[s][i]
//   Bi (                  the same                ): w_s Im v_s          D2[n'][i] = sum_s A[s][n'] Bi[s][i]
//   Re U[i][j] = D1[2j][i] + D2[2j+1][i],   Im U[i][j] = D2[2j][i] - D1[2j+1][i]:  neighbouring TMEM lanes, one shuffle.
// grid = (chunks, H, K); 256 threads; 66 KB shared memory, 128 TMEM columns: three CTAs per SM.
// ---------------------------------------------------------------------------------------------
constexpr size_t OUTER_SMEM = 1024 + 32768 + 32768 + 1024;

// DSTATE == true computes the gradient counterpart  G = sum_t scale e^{A_t} dy_t (x) conj(q_t)  (dy in
// place of v, q in place of k) into dstate slot c.
// The two token tiles (k and v, or q and dy; maps of [B*H*T rows][128 bf16], boxes of 64 x 128, 128-byte swizzle)
// arrive by TMA; the value tile lands in the region its planes are then built in: every thread reads its pieces, a
// barrier, and the planes are written over them.
template <bool DSTATE>
__global__ void __launch_bounds__(256, 3) k_tc_chunk_outer(const __grid_constant__ CUtensorMap mk,
                                                           const __grid_constant__ CUtensorMap mv, ScanParams p) {
  using namespace umma;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;            // key tile: [2 boxes of 64 columns][128 rows][128 B]
  unsigned char* sB = smem + 32768;    // value tile, then [256 rows][128 B]: rows s = w Re v_s, rows 128 + s = w Im v_s
  float* Acum = reinterpret_cast<float*>(smem + 65536);          // [128]
  uint64_t* bar = reinterpret_cast<uint64_t*>(Acum + TC);       // [0] MMAs  [1] token tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  const int kst = blockIdx.z;                 // state (its decay weights the rows); grid z = K
  float graw[4] = {1.f, 1.f, 1.f, 1.f};
  if (warp == 1) warp_cumsum128_load(graw, p.gamma + gamma_base(p, kst, L.b, h, L.t0), L.len, lane);
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    fence_barrier_init();
    const int row0 = (L.b * p.H + h) * p.T + L.t0;
    mbar_arrive_expect_tx(&bar[1], 4 * 16384);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(sA + kb * 16384, &mk, &bar[1], kb * 64, row0);
      tma_load_2d(sB + kb * 16384, &mv, &bar[1], kb * 64, row0);
    }
  }
  __syncwarp();
  if (warp == 0) tmem_alloc<128>(tmem_slot);
  if (warp == 1) warp_cumsum128_finish(Acum, graw, L.len, p.eps, lane);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const float a_last = Acum[TC - 1];
  const bool tiles_ok = mbar_wait(&bar[1], 0, 202);
  // this thread's 16-byte pieces of the value tile (rows past the chunk's end belong to someone else: their zeros
  // also cancel whatever the key tile holds in those rows)
  uint4 vxa[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = tid + 256 * it;
    const int row = idx >> 4, c16 = idx & 15;
    vxa[it] = make_uint4(0, 0, 0, 0);
    if (row < L.len) vxa[it] = *reinterpret_cast<const uint4*>(sB + (c16 >> 3) * 16384 + sw128(row, c16 & 7));
  }
  __syncthreads();      // every piece has been read: the planes may overwrite the tile
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = tid + 256 * it;
    const int row = idx >> 4, c16 = idx & 15;
    const uint4 vx = vxa[it];
    const float w = DSTATE ? p.q_scale * __expf(Acum[row]) : __expf(fminf(0.f, a_last - Acum[row]));
    const uint32_t vw[4] = {vx.x, vx.y, vx.z, vx.w};
    float vr[4], vi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 vv = unpack_bf162(vw[e]);
      vr[e] = w * vv.x;
      vi[e] = w * vv.y;
    }
    const uint32_t boff = (c16 & 1) * 8;
    *reinterpret_cast<uint2*>(sB + sw128(row, c16 >> 1) + boff) = make_uint2(pack_bf162(vr[0], vr[1]), pack_bf162(vr[2], vr[3]));
    *reinterpret_cast<uint2*>(sB + sw128(128 + row, c16 >> 1) + boff) = make_uint2(pack_bf162(vi[0], vi[1]), pack_bf162(vi[2], vi[3]));
  }
  fence_proxy_async();
  __syncthreads();
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16(128, 64, true, true);
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)      // D1 = A^T Br: k-step = 16 tokens = 2048 bytes in either operand
      mma_bf16(tmem, smem_desc_sw128(a0 + kk * 2048, 16384, 1024), smem_desc_sw128(b0 + kk * 2048, 16, 1024), idesc, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)      // D2 = A^T Bi
      mma_bf16(tmem + 64, smem_desc_sw128(a0 + kk * 2048, 16384, 1024), smem_desc_sw128(b0 + 16384 + kk * 2048, 16, 1024), idesc, kk > 0);
    mma_commit(&bar[0]);
  }
  __syncwarp();
  const bool ok = mbar_wait(&bar[0], 0, 201) && tiles_ok;
  tc_fence_after();
  {
    // lane n' = 2j+c of the tile holds column i: state[i][j][c] sits at float offset i*128 + n'
    float2* slot = DSTATE ? p.dstates + state_base(p, kst, h, L.slot0 + L.c, TD)
                          : p.states + state_base(p, kst, h, L.slot0 + L.c + 1, TD);
    const int q4 = warp & 3, cc = warp >> 2;   // TMEM lane quarter, column half
    float* dst = reinterpret_cast<float*>(slot) + (q4 * 32 + lane);
    float d1[32], d2[32];
    tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + cc * 32, d1);
    tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + 64 + cc * 32, d2);
    const bool even = (lane & 1) == 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, d2[i], 1);      // D2 of the neighbouring key column
      const float u = even ? d1[i] + other : other - d1[i];
      if (ok) dst[(size_t)(cc * 32 + i) * 128] = u;
    }
    if (ok && !DSTATE && tid == 0) p.chunk_decay[((size_t)kst * p.H + h) * p.nslots + L.slot0 + L.c + 1] = __expf(a_last);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<128>(tmem);
  }
}

// ---------------------------------------------------------------------------------------------
// State sums of K states from ONE load of the key / value tiles (forward only, 2 <= K <= 4).  As in k_tc_chunk_outer
// the key tile is the A operand as the TMA delivers it and the decay weights sit on the value planes, so a state costs
// one rewrite of the planes B_k = w^k_s (Re v_s ; Im v_s) from the registers that hold the value tile, its two MMA
// chains into the same 128 TMEM columns, and its epilogue; the states follow one another.
// grid = (chunks, H); 256 threads; 70 KB shared memory, 128 TMEM columns: three CTAs per SM.
// ---------------------------------------------------------------------------------------------
constexpr size_t OUTERK_SMEM = 1024 + 65536 + 4096;

__global__ void __launch_bounds__(256, 3) k_tc_chunk_outerK(const __grid_constant__ CUtensorMap mk,
                                                            const __grid_constant__ CUtensorMap mv, ScanParams p) {
  using namespace umma;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;            // key tile: [2 boxes of 64 columns][128 rows][128 B]
  unsigned char* sB = smem + 32768;    // value tile, then per state [256 rows][128 B]: w Re v_s ; w Im v_s
  float* Acum = reinterpret_cast<float*>(smem + 65536);           // [KMAX][128]
  uint64_t* bar = reinterpret_cast<uint64_t*>(Acum + KMAX * TC);  // one per state, [KMAX]: the token tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + KMAX + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  const int K = p.K;
  float graw[4] = {1.f, 1.f, 1.f, 1.f};
  if (warp >= 1 && warp <= K) warp_cumsum128_load(graw, p.gamma + gamma_base(p, warp - 1, L.b, h, L.t0), L.len, lane);
  if (tid == 0) {
    for (int k = 0; k < K; ++k) mbar_init(&bar[k], 1);
    mbar_init(&bar[KMAX], 1);
    fence_barrier_init();
    const int row0 = (L.b * p.H + h) * p.T + L.t0;
    mbar_arrive_expect_tx(&bar[KMAX], 4 * 16384);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(sA + kb * 16384, &mk, &bar[KMAX], kb * 64, row0);
      tma_load_2d(sB + kb * 16384, &mv, &bar[KMAX], kb * 64, row0);
    }
  }
  __syncwarp();
  if (warp == 0) tmem_alloc<128>(tmem_slot);
  if (warp >= 1 && warp <= K) warp_cumsum128_finish(Acum + (warp - 1) * TC, graw, L.len, p.eps, lane);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool ok = mbar_wait(&bar[KMAX], 0, 206);
  // this thread's 16-byte pieces of the value tile (rows past the chunk's end: zeros, which also cancel whatever the
  // key tile holds in those rows)
  uint4 vxa[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = tid + 256 * it;
    const int row = idx >> 4, c16 = idx & 15;
    vxa[it] = make_uint4(0, 0, 0, 0);
    if (row < L.len) vxa[it] = *reinterpret_cast<const uint4*>(sB + (c16 >> 3) * 16384 + sw128(row, c16 & 7));
  }
  const int q4 = warp & 3, cc = warp >> 2;   // epilogue: TMEM lane quarter, column half
  const bool even = (lane & 1) == 0;
  for (int k = 0; k < K; ++k) {
    // every piece has been read (k = 0) / the previous state's MMAs have read the planes and its epilogue the
    // accumulators (k > 0: every thread waited for them below)
    tc_fence_before();
    __syncthreads();
    const float a_last = Acum[k * TC + TC - 1];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int idx = tid + 256 * it;
      const int row = idx >> 4, c16 = idx & 15;
      const uint4 vx = vxa[it];
      const float w = __expf(fminf(0.f, a_last - Acum[k * TC + row]));
      const uint32_t vw[4] = {vx.x, vx.y, vx.z, vx.w};
      float vr[4], vi[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 vv = unpack_bf162(vw[e]);
        vr[e] = w * vv.x;
        vi[e] = w * vv.y;
      }
      const uint32_t boff = (c16 & 1) * 8;
      *reinterpret_cast<uint2*>(sB + sw128(row, c16 >> 1) + boff) = make_uint2(pack_bf162(vr[0], vr[1]), pack_bf162(vr[2], vr[3]));
      *reinterpret_cast<uint2*>(sB + sw128(128 + row, c16 >> 1) + boff) = make_uint2(pack_bf162(vi[0], vi[1]), pack_bf162(vi[2], vi[3]));
    }
    fence_proxy_async();
    __syncthreads();
    if (warp == 0 && elect_one()) {
      tc_fence_after();
      constexpr uint32_t idesc = idesc_bf16(128, 64, true, true);
      const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)      // D1 = A^T Br
        mma_bf16(tmem, smem_desc_sw128(a0 + kk * 2048, 16384, 1024), smem_desc_sw128(b0 + kk * 2048, 16, 1024), idesc, kk > 0);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)      // D2 = A^T Bi
        mma_bf16(tmem + 64, smem_desc_sw128(a0 + kk * 2048, 16384, 1024), smem_desc_sw128(b0 + 16384 + kk * 2048, 16, 1024), idesc, kk > 0);
      mma_commit(&bar[k]);
    }
    __syncwarp();
    ok = mbar_wait(&bar[k], 0, 205) && ok;
    tc_fence_after();
    // Re U = D1[2j] + D2[2j+1], Im U = D2[2j] - D1[2j+1]: lane n' = 2j+c holds column i, state[i][j][c] at i*128 + n'
    float2* slot = p.states + state_base(p, k, h, L.slot0 + L.c + 1, TD);
    float* dst = reinterpret_cast<float*>(slot) + (q4 * 32 + lane);
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {          // 16 columns at a time: the value tile stays in registers beside them
      float d1[16], d2[16];
      const uint32_t col = (uint32_t)(cc * 32 + hh * 16);
      tmem_ld16x2(tmem + ((uint32_t)(q4 * 32) << 16) + col, d1, tmem + ((uint32_t)(q4 * 32) << 16) + 64 + col, d2);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, d2[i], 1);
        const float u = even ? d1[i] + other : other - d1[i];
        if (ok) dst[(size_t)(col + i) * 128] = u;
      }
    }
    if (ok && tid == 0) p.chunk_decay[((size_t)k * p.H + h) * p.nslots + L.slot0 + L.c + 1] = __expf(a_last);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<128>(tmem);
  }
}

enum ChunkMode { M_FWD = 0, M_DQ = 1, M_DV = 2, M_DK = 3 };

struct ChunkMaps {
  CUtensorMap a1, b1, x2;  // [B*H*T rows][128 bf16], boxes of 64 x 128, 128-byte swizzle
  CUtensorMap out;         // the output tensor, same shape, boxes of 64 x 32 (one per epilogue warp)
};

}  // namespace tcs
}  // namespace qpam
