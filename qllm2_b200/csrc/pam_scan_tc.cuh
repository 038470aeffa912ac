// Tensor-core (tcgen05 / TMEM / TMA) kernels of the chunked PAM scan for bf16 token tensors,
// head dim 64, one state.  Chunks are 128 tokens, so every MMA is M = 128.
//
// Complex products run as real bf16 MMAs on the INTERLEAVED (re, im) rows as they sit in memory:
// a token row of 64 complex numbers is a 128-element real vector x = (r0, i0, r1, i1, ...); with
// rot(x) = (-i0, r0, -i1, r1, ...) and cj(x) = (r0, -i0, ...):
//     Re(q . conj(k)) = <q, k>            Im(q . conj(k)) = <q, rot(k)>
//     (m v)_interleaved = Re(m) v + Im(m) rot(v)
// so the real/imaginary planes are separate MMA operands (k and rot(k), v and rot(v), ...) built
// by element-wise passes over shared memory; nothing is de-interleaved in HBM.
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
__device__ __forceinline__ void warp_cumsum128(float* A, const float* __restrict__ gamma, int len, float eps, int lane) {
  const int t = 4 * lane;
  float x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = (t + i < len) ? logf(gamma[t + i] + eps) : 0.f;
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

struct TcMaps {
  CUtensorMap q, k, v;  // [B*H*T rows][128 bf16], boxes of 64 x 128, 128-byte swizzle
};

// ---------------------------------------------------------------------------------------------
// Chunk-local state sum, transposed form:  D[2j+c][i] = (Re|Im) sum_s w_s v_s[i] conj(k_s[j])
//   A (MN-major, M = 128 interleaved key columns, K = 256): rows s      : w_s * cj(k_s)
//                                                           rows 128+s  : w_s * (ki, kr)
//   B (MN-major, N = 64 value channels,          K = 256): rows s      : Re v_s
//                                                           rows 128+s  : Im v_s
// grid = (chunks, H); 128 threads; ~97 KB shared memory, 64 TMEM columns (two CTAs per SM).
// ---------------------------------------------------------------------------------------------
constexpr size_t OUTER_SMEM = 1024 + 65536 + 32768 + 1024;

__global__ void __launch_bounds__(128) k_tc_chunk_outer(ScanParams p) {
  using namespace umma;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = smem;            // [2 blocks][256 rows][128 B]
  unsigned char* sB = smem + 65536;    // [256 rows][128 B]
  float* Acum = reinterpret_cast<float*>(smem + 65536 + 32768);  // [128]
  uint64_t* bar = reinterpret_cast<uint64_t*>(Acum + TC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  if (tid == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc<64>(tmem_slot);
  if (warp == 1) warp_cumsum128(Acum, p.gamma + gamma_base(p, 0, L.b, h, L.t0), L.len, p.eps, lane);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const float a_last = Acum[TC - 1];
  const size_t tb = token_base(p, L.b, h, L.t0, TD);
  const uint4* kg = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.k) + tb);
  const uint4* vg = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.v) + tb);
#pragma unroll 4
  for (int it = 0; it < 16; ++it) {
    const int idx = tid + 128 * it;
    const int row = idx >> 4, c16 = idx & 15;
    uint4 kx = make_uint4(0, 0, 0, 0), vx = make_uint4(0, 0, 0, 0);
    if (row < L.len) {
      kx = __ldg(kg + idx);
      vx = __ldg(vg + idx);
    }
    const float w = __expf(fminf(0.f, a_last - Acum[row]));
    const uint32_t kw[4] = {kx.x, kx.y, kx.z, kx.w};
    const uint32_t vw[4] = {vx.x, vx.y, vx.z, vx.w};
    uint32_t lo[4], hi[4];
    float vr[4], vi[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 kk = unpack_bf162(kw[e]);
      lo[e] = pack_bf162(w * kk.x, -w * kk.y);
      hi[e] = pack_bf162(w * kk.y, w * kk.x);
      const float2 vv = unpack_bf162(vw[e]);
      vr[e] = vv.x;
      vi[e] = vv.y;
    }
    unsigned char* ablk = sA + (c16 >> 3) * 32768;
    *reinterpret_cast<uint4*>(ablk + sw128(row, c16 & 7)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    *reinterpret_cast<uint4*>(ablk + sw128(128 + row, c16 & 7)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
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
    for (int kk = 0; kk < 16; ++kk)
      mma_bf16(tmem, smem_desc_sw128(a0 + kk * 2048, 32768, 1024), smem_desc_sw128(b0 + kk * 2048, 16, 1024), idesc, kk > 0);
    mma_commit(bar);
  }
  __syncwarp();
  const bool ok = mbar_wait(bar, 0, 201);
  tc_fence_after();
  if (ok) {
    // lane n' = 2j+c of the tile holds column i: state[i][j][c] sits at float offset i*128 + n'
    float* dst = reinterpret_cast<float*>(p.states + state_base(p, 0, h, L.slot0 + L.c + 1, TD)) + (warp * 32 + lane);
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      float v[32];
      tmem_ld32(taddr + cc * 32, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) dst[(size_t)(cc * 32 + i) * 128] = v[i];
    }
    if (tid == 0) p.chunk_decay[(size_t)h * p.nslots + L.slot0 + L.c + 1] = __expf(a_last);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<64>(tmem);
  }
}

// ---------------------------------------------------------------------------------------------
// Forward output of one 128-token chunk.  grid = (chunks, H); 256 threads; 192 KB shared memory.
//   GEMM1  [Wr | Wi] = Q [K ; rot K]^T                      M128 N256 K128   (TMA operands)
//   epi 1  M = scale * D .* W  -> bf16 [Mr | Mi]  (overlays K),  Q <- scale * e^{A_t} Q
//   GEMM2  Y  = [Mr | Mi] [V ; rot V]                       M128 N128 K256
//   GEMM3  Y += Q' Bs^T,  Bs rows 2i: cj(S[i,:]), 2i+1: (Si, Sr)   M128 N128 K128 (carried state)
//   epi 2  Y -> bf16 -> global
// ---------------------------------------------------------------------------------------------
constexpr size_t FWD_SMEM = 1024 + 65536 + 32768 + 65536 + 32768 + 1024;

__global__ void __launch_bounds__(256, 1) k_tc_fwd_chunk(const __grid_constant__ TcMaps maps, ScanParams p) {
  using namespace umma;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* R1 = smem;                    // K | rot K : [2 kb][256 rows][128 B]; later [Mr|Mi]: [4 kb][128 rows][128 B]
  unsigned char* R2 = R1 + 65536;              // Q         : [2 kb][128 rows][128 B]
  unsigned char* R3 = R2 + 32768;              // V | rot V : [2 nb][256 rows][128 B]
  unsigned char* R4 = R3 + 65536;              // Bs        : [2 kb][128 rows][128 B]
  float* Acum = reinterpret_cast<float*>(R4 + 32768);
  uint64_t* bars = reinterpret_cast<uint64_t*>(Acum + TC);  // [0] tma, [1] gemm1, [2] gemm2+3
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  const bool has_prev = (L.c > 0) || (p.s0 != nullptr);
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc<512>(tmem_slot);
  if (warp == 1) warp_cumsum128(Acum, p.gamma + gamma_base(p, 0, L.b, h, L.t0), L.len, p.eps, lane);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int row0 = (L.b * p.H + h) * p.T + L.t0;  // row of the [B*H*T][128] token matrices
  if (tid == 0) {
    mbar_arrive_expect_tx(&bars[0], 6 * 16384);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(R2 + kb * 16384, &maps.q, &bars[0], kb * 64, row0);
      tma_load_2d(R1 + kb * 32768, &maps.k, &bars[0], kb * 64, row0);
      tma_load_2d(R3 + kb * 32768, &maps.v, &bars[0], kb * 64, row0);
    }
  }
  if (has_prev) {
    // carried state (fp32 [i][j] complex) -> bf16 K-major rows 2i = cj(S[i,:]), 2i+1 = (Si, Sr)
    const float4* sg = reinterpret_cast<const float4*>(p.states + state_base(p, 0, h, L.slot0 + L.c, TD));
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;       // (i, c16): 4 complex = 2 float4
      const int i = idx >> 4, c16 = idx & 15;
      const float4 s01 = __ldg(sg + idx * 2), s23 = __ldg(sg + idx * 2 + 1);
      const uint4 even = make_uint4(pack_bf162(s01.x, -s01.y), pack_bf162(s01.z, -s01.w), pack_bf162(s23.x, -s23.y), pack_bf162(s23.z, -s23.w));
      const uint4 odd = make_uint4(pack_bf162(s01.y, s01.x), pack_bf162(s01.w, s01.z), pack_bf162(s23.y, s23.x), pack_bf162(s23.w, s23.z));
      unsigned char* blk = R4 + (c16 >> 3) * 16384;
      *reinterpret_cast<uint4*>(blk + sw128(2 * i, c16 & 7)) = even;
      *reinterpret_cast<uint4*>(blk + sw128(2 * i + 1, c16 & 7)) = odd;
    }
  }
  bool ok = mbar_wait(&bars[0], 0, 211);
  // rot K and rot V: element-wise on the swizzled bytes, same position 128 rows further down
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int ci = tid + 256 * it;          // 2 blocks x 128 rows x 8 chunks
    const uint32_t off = (uint32_t)(ci >> 10) * 32768u + (uint32_t)(ci & 1023) * 16u;
    const uint4 kx = *reinterpret_cast<const uint4*>(R1 + off);
    const uint4 vx = *reinterpret_cast<const uint4*>(R3 + off);
    const uint32_t kw[4] = {kx.x, kx.y, kx.z, kx.w}, vw[4] = {vx.x, vx.y, vx.z, vx.w};
    uint32_t kr[4], vr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // (re, im) -> (-im, re): swap the halves and flip the sign bit of the new low half
      kr[e] = ((kw[e] >> 16) | (kw[e] << 16)) ^ 0x00008000u;
      vr[e] = ((vw[e] >> 16) | (vw[e] << 16)) ^ 0x00008000u;
    }
    *reinterpret_cast<uint4*>(R1 + off + 16384) = make_uint4(kr[0], kr[1], kr[2], kr[3]);
    *reinterpret_cast<uint4*>(R3 + off + 16384) = make_uint4(vr[0], vr[1], vr[2], vr[3]);
  }
  fence_proxy_async();
  __syncthreads();
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16(128, 256, false, false);
    const uint32_t q0 = smem_u32(R2), k0 = smem_u32(R1);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        mma_bf16(tmem, smem_desc_sw128(q0 + kb * 16384 + kk * 32, 16, 1024),
                 smem_desc_sw128(k0 + kb * 32768 + kk * 32, 16, 1024), idesc, (kb | kk) != 0);
    mma_commit(&bars[1]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[1], 0, 212) && ok;
  tc_fence_after();
  {
    // epilogue 1: decay-masked scores to bf16 [Mr | Mi] (K-major, 4 k-blocks) over the K | rot K region
    const int q4 = warp & 3, hf = warp >> 2;
    const int t = q4 * 32 + lane;
    const float a_t = Acum[t];
    const uint32_t taddr = tmem + ((uint32_t)(q4 * 32) << 16);
#pragma unroll 1
    for (int cc = 0; cc < 2; ++cc) {
      const int s0 = hf * 64 + cc * 32;
      uint32_t mr[16], mi[16];
      if (s0 > q4 * 32 + 31) {
#pragma unroll
        for (int j = 0; j < 16; ++j) mr[j] = mi[j] = 0u;
      } else {
        float wr[32], wi[32];
        tmem_ld32(taddr + s0, wr);
        tmem_ld32(taddr + 128 + s0, wi);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int s = s0 + j;
          const float d0 = (s <= t) ? p.q_scale * __expf(fminf(0.f, a_t - Acum[s])) : 0.f;
          const float d1 = (s + 1 <= t) ? p.q_scale * __expf(fminf(0.f, a_t - Acum[s + 1])) : 0.f;
          mr[j >> 1] = pack_bf162(d0 * wr[j], d1 * wr[j + 1]);
          mi[j >> 1] = pack_bf162(d0 * wi[j], d1 * wi[j + 1]);
        }
      }
      unsigned char* br = R1 + (s0 >> 6) * 16384;          // Mr: k = s
      unsigned char* bi = R1 + (2 + (s0 >> 6)) * 16384;    // Mi: k = 128 + s
      const int c0 = (s0 & 63) >> 3;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        *reinterpret_cast<uint4*>(br + sw128(t, c0 + g)) = make_uint4(mr[4 * g], mr[4 * g + 1], mr[4 * g + 2], mr[4 * g + 3]);
        *reinterpret_cast<uint4*>(bi + sw128(t, c0 + g)) = make_uint4(mi[4 * g], mi[4 * g + 1], mi[4 * g + 2], mi[4 * g + 3]);
      }
    }
    if (has_prev) {
      // Q <- scale * exp(A_t) * Q in place (the row of a 16-byte chunk follows from its offset)
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int ci = tid + 256 * it;      // 2 kb x 128 rows x 8 chunks
        const int row = (ci >> 3) & 127;
        const float f = p.q_scale * __expf(Acum[row]);
        uint4* ptr = reinterpret_cast<uint4*>(R2 + (size_t)ci * 16);
        const uint4 x = *ptr;
        const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 v2 = unpack_bf162(xw[e]);
          o[e] = pack_bf162(f * v2.x, f * v2.y);
        }
        *ptr = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t idesc2 = idesc_bf16(128, 128, false, true);
    constexpr uint32_t idesc3 = idesc_bf16(128, 128, false, false);
    const uint32_t m0 = smem_u32(R1), v0 = smem_u32(R3), q0 = smem_u32(R2), b0 = smem_u32(R4);
    const uint32_t dY = tmem + 256;
#pragma unroll
    for (int kk = 0; kk < 16; ++kk)
      mma_bf16(dY, smem_desc_sw128(m0 + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
               smem_desc_sw128(v0 + kk * 2048, 32768, 1024), idesc2, kk > 0);
    if (has_prev) {
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(dY, smem_desc_sw128(q0 + kb * 16384 + kk * 32, 16, 1024),
                   smem_desc_sw128(b0 + kb * 16384 + kk * 32, 16, 1024), idesc3, true);
    }
    mma_commit(&bars[2]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[2], 0, 213) && ok;
  tc_fence_after();
  if (ok) {
    const int q4 = warp & 3, hf = warp >> 2;
    const int t = q4 * 32 + lane;
    const uint32_t taddr = tmem + 256 + ((uint32_t)(q4 * 32) << 16) + hf * 64;
    __nv_bfloat16* yrow = reinterpret_cast<__nv_bfloat16*>(p.y) + token_base(p, L.b, h, L.t0 + t, TD) + hf * 64;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      float v[32];
      tmem_ld32(taddr + cc * 32, v);
      if (t < L.len) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(yrow + cc * 32 + g * 8) =
              make_uint4(pack_bf162(v[8 * g], v[8 * g + 1]), pack_bf162(v[8 * g + 2], v[8 * g + 3]),
                         pack_bf162(v[8 * g + 4], v[8 * g + 5]), pack_bf162(v[8 * g + 6], v[8 * g + 7]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<512>(tmem);
  }
}

}  // namespace tcs
}  // namespace qpam
