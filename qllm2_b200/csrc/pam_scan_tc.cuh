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
// grid = (chunks, H); 256 threads; ~97 KB shared memory, 64 TMEM columns (two CTAs per SM).
// ---------------------------------------------------------------------------------------------
constexpr size_t OUTER_SMEM = 1024 + 65536 + 32768 + 1024;

// DSTATE == true computes the gradient counterpart  G = sum_t scale e^{A_t} dy_t (x) conj(q_t)  (dy in
// place of v, q in place of k) into dstate slot c.
template <bool DSTATE>
__global__ void __launch_bounds__(256, 2) k_tc_chunk_outer(ScanParams p) {
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
  const size_t tb = token_base(p, L.b, h, L.t0, TD);
  const uint4* kg = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(DSTATE ? p.q : p.k) + tb);
  const uint4* vg = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(DSTATE ? p.dy : p.v) + tb);
  // every global load of this thread is in flight before the first barrier
  uint4 kxa[8], vxa[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = tid + 256 * it;
    kxa[it] = make_uint4(0, 0, 0, 0);
    vxa[it] = make_uint4(0, 0, 0, 0);
    if ((idx >> 4) < L.len) {
      kxa[it] = __ldg(kg + idx);
      vxa[it] = __ldg(vg + idx);
    }
  }
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
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = tid + 256 * it;
    const int row = idx >> 4, c16 = idx & 15;
    const uint4 kx = kxa[it], vx = vxa[it];
    const float w = DSTATE ? p.q_scale * __expf(Acum[row]) : __expf(fminf(0.f, a_last - Acum[row]));
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
    float2* slot = DSTATE ? p.dstates + state_base(p, 0, h, L.slot0 + L.c, TD)
                          : p.states + state_base(p, 0, h, L.slot0 + L.c + 1, TD);
    const int q4 = warp & 3, cc = warp >> 2;   // TMEM lane quarter, column half
    float* dst = reinterpret_cast<float*>(slot) + (q4 * 32 + lane);
    float v[32];
    tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + cc * 32, v);
#pragma unroll
    for (int i = 0; i < 32; ++i) dst[(size_t)(cc * 32 + i) * 128] = v[i];
    if (!DSTATE && tid == 0) p.chunk_decay[(size_t)h * p.nslots + L.slot0 + L.c + 1] = __expf(a_last);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<64>(tmem);
  }
}

// ---------------------------------------------------------------------------------------------
// One 128-token chunk of the forward output or of one gradient.  All four share the structure
//
//   stage 1  [Xr | Xi] = A1 [B1 ; rot B1]^T                 M128 N256 K128   X[t][s], t: A1 row, s: B1 row
//   epi 1    T = scale * D[t,s] .* X   (s <= t, D = exp(min(0, A_t - A_s)))  -> bf16 in shared memory
//   stage 2  out  = T (.) [X2 ; rot X2]                     M128 N128 K256
//   stage 3  out += A3 B3^T  through the carried state      M128 N128 K128
//   epi 2    out -> bf16 -> global (+ the decay-gradient dot product for DQ / DK)
//
//   MODE  A1  B1  X2  T used as                 A3 (row-scaled in place)   B3 (bf16 image of)
//   FWD   q   k   v   [Tr | Ti]  rows t         scale e^{A_t} q            S   rows 2i: cj(S[i,:]), 2i+1: (Si,Sr)
//   DQ    dy  v   k   [Tr | Ti]  rows t         scale e^{A_t} dy           S   rows 2j: (Sr,Si)[:,j], 2j+1: (-Si,Sr)[:,j]
//   DV    q   k   dy  [Tr ; -Ti]^T rows s       w_s k                      dS  as FWD
//   DK    dy  v   q   [Tr ; -Ti]^T rows s       w_s v                      dS  as DQ
//
// with w_s = exp(min(0, A_last - A_s)), S the state before the chunk and dS the gradient reaching
// the state after it.  grid = (chunks, H); 256 threads; 192 KB shared memory; 384 TMEM columns.
// ---------------------------------------------------------------------------------------------
enum ChunkMode { M_FWD = 0, M_DQ = 1, M_DV = 2, M_DK = 3 };

struct ChunkMaps {
  CUtensorMap a1, b1, x2;  // [B*H*T rows][128 bf16], boxes of 64 x 128, 128-byte swizzle
};

constexpr size_t CHUNK_SMEM = 1024 + 32768 + 65536 + 65536 + 32768 + 2048;

template <int MODE>
__global__ void __launch_bounds__(256, 1) k_tc_chunk(const __grid_constant__ ChunkMaps maps, ScanParams p) {
  using namespace umma;
  constexpr bool ROWS_T = (MODE == M_FWD || MODE == M_DQ);   // output rows follow A1's tokens
  constexpr bool OP_TRANSPOSED = (MODE == M_DQ || MODE == M_DK);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* RA = smem;                  // A1        : [2 kb][128 rows][128 B]
  unsigned char* RB = RA + 32768;            // B1 | rot  : [2 kb][256 rows][128 B]
  unsigned char* RC = RB + 65536;            // X2 | rot  : [2 nb][256 rows][128 B]
  unsigned char* RD = RC + 65536;            // B3        : [2 kb][128 rows][128 B]
  float* Acum = reinterpret_cast<float*>(RD + 32768);   // [128]
  float* dots = Acum + TC;                              // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(dots + 2 * TC);  // [0] tma, [1] stage 1, [2] stages 2+3
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  const bool has_state = ROWS_T ? ((L.c > 0) || (p.s0 != nullptr)) : ((L.c < L.nc - 1) || (p.ds_final != nullptr));
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
      tma_load_2d(RA + kb * 16384, &maps.a1, &bars[0], kb * 64, row0);
      tma_load_2d(RB + kb * 32768, &maps.b1, &bars[0], kb * 64, row0);
      tma_load_2d(RC + kb * 32768, &maps.x2, &bars[0], kb * 64, row0);
    }
  }
  if (has_state) {
    const float2* st = ROWS_T ? p.states + state_base(p, 0, h, L.slot0 + L.c, TD)
                              : p.dstates + state_base(p, 0, h, L.slot0 + L.c + 1, TD);
    const float4* sg = reinterpret_cast<const float4*>(st);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      // (i, c16): state[i][4*c16 .. +3].  The transposed image is written with 4-byte stores whose
      // bank follows i, so there consecutive lanes take consecutive i (conflict-free); the plain
      // image keeps consecutive lanes on consecutive c16 (coalesced 512-byte reads).
      const int idx = tid + 256 * it;
      const int i = OP_TRANSPOSED ? (idx & 63) : (idx >> 4);
      const int c16 = OP_TRANSPOSED ? (idx >> 6) : (idx & 15);
      const float4 s01 = __ldg(sg + (i * 16 + c16) * 2), s23 = __ldg(sg + (i * 16 + c16) * 2 + 1);
      if (!OP_TRANSPOSED) {
        const uint4 even = make_uint4(pack_bf162(s01.x, -s01.y), pack_bf162(s01.z, -s01.w), pack_bf162(s23.x, -s23.y), pack_bf162(s23.z, -s23.w));
        const uint4 odd = make_uint4(pack_bf162(s01.y, s01.x), pack_bf162(s01.w, s01.z), pack_bf162(s23.y, s23.x), pack_bf162(s23.w, s23.z));
        unsigned char* blk = RD + (c16 >> 3) * 16384;
        *reinterpret_cast<uint4*>(blk + sw128(2 * i, c16 & 7)) = even;
        *reinterpret_cast<uint4*>(blk + sw128(2 * i + 1, c16 & 7)) = odd;
      } else {
        // rows 2j / 2j+1, K position 2i: 4-byte words scattered along the (transposed) state
        const float sr[4] = {s01.x, s01.z, s23.x, s23.z}, si[4] = {s01.y, s01.w, s23.y, s23.w};
        unsigned char* blk = RD + (i >> 5) * 16384;
        const int c = (i & 31) >> 2;
        const uint32_t woff = (uint32_t)(i & 3) * 4u;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 4 * c16 + e;
          *reinterpret_cast<uint32_t*>(blk + sw128(2 * j, c) + woff) = pack_bf162(sr[e], si[e]);
          *reinterpret_cast<uint32_t*>(blk + sw128(2 * j + 1, c) + woff) = pack_bf162(-si[e], sr[e]);
        }
      }
    }
  }
  bool ok = mbar_wait(&bars[0], 0, 211);
  // rot B1 and rot X2: element-wise on the swizzled bytes, same position 128 rows further down
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int ci = tid + 256 * it;          // 2 blocks x 128 rows x 8 chunks
    const uint32_t off = (uint32_t)(ci >> 10) * 32768u + (uint32_t)(ci & 1023) * 16u;
    const uint4 bx = *reinterpret_cast<const uint4*>(RB + off);
    const uint4 xx = *reinterpret_cast<const uint4*>(RC + off);
    const uint32_t bw[4] = {bx.x, bx.y, bx.z, bx.w}, xw[4] = {xx.x, xx.y, xx.z, xx.w};
    uint32_t br[4], xr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // (re, im) -> (-im, re): swap the halves and flip the sign bit of the new low half
      br[e] = ((bw[e] >> 16) | (bw[e] << 16)) ^ 0x00008000u;
      xr[e] = ((xw[e] >> 16) | (xw[e] << 16)) ^ 0x00008000u;
    }
    *reinterpret_cast<uint4*>(RB + off + 16384) = make_uint4(br[0], br[1], br[2], br[3]);
    *reinterpret_cast<uint4*>(RC + off + 16384) = make_uint4(xr[0], xr[1], xr[2], xr[3]);
  }
  fence_proxy_async();
  __syncthreads();
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t idesc = idesc_bf16(128, 256, false, false);
    const uint32_t a0 = smem_u32(RA), b0 = smem_u32(RB);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        mma_bf16(tmem, smem_desc_sw128(a0 + kb * 16384 + kk * 32, 16, 1024),
                 smem_desc_sw128(b0 + kb * 32768 + kk * 32, 16, 1024), idesc, (kb | kk) != 0);
    mma_commit(&bars[1]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[1], 0, 212) && ok;
  tc_fence_after();
  const float a_last = Acum[TC - 1];
  {
    // epilogue 1: decay-masked X to bf16.  The 64-wide column blocks of Tr and Ti are four 16 KB
    // pieces [128 rows t][128 B]; where they go depends on how stage 2 reads them.
    unsigned char* piece_r0 = ROWS_T ? RB : RA;                   // Tr, s in [0,64)
    unsigned char* piece_r1 = ROWS_T ? RB + 16384 : RA + 16384;   // Tr, s in [64,128)
    unsigned char* piece_i0 = ROWS_T ? RB + 32768 : RB + 16384;   // Ti (ROWS_T) or -Ti
    unsigned char* piece_i1 = ROWS_T ? RB + 49152 : RB + 49152;
    const float isign = ROWS_T ? 1.f : -1.f;
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
          // rows past the end of a ragged chunk hold other sequences' tokens: they must not reach
          // the transposed products (DV, DK), where t is the contraction index
          const float d0 = (s <= t && t < L.len) ? p.q_scale * __expf(fminf(0.f, a_t - Acum[s])) : 0.f;
          const float d1 = (s + 1 <= t && t < L.len) ? p.q_scale * __expf(fminf(0.f, a_t - Acum[s + 1])) : 0.f;
          mr[j >> 1] = pack_bf162(d0 * wr[j], d1 * wr[j + 1]);
          mi[j >> 1] = pack_bf162(isign * d0 * wi[j], isign * d1 * wi[j + 1]);
        }
      }
      unsigned char* br = hf ? piece_r1 : piece_r0;
      unsigned char* bi = hf ? piece_i1 : piece_i0;
      const int c0 = cc * 4;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        *reinterpret_cast<uint4*>(br + sw128(t, c0 + g)) = make_uint4(mr[4 * g], mr[4 * g + 1], mr[4 * g + 2], mr[4 * g + 3]);
        *reinterpret_cast<uint4*>(bi + sw128(t, c0 + g)) = make_uint4(mi[4 * g], mi[4 * g + 1], mi[4 * g + 2], mi[4 * g + 3]);
      }
    }
    if (has_state) {
      // A3: scale the rows of A1 (FWD, DQ: scale e^{A_t}) or of the raw B1 (DV, DK: w_s) in place;
      // the row of a 16-byte chunk follows from its offset, the swizzle only permutes inside rows
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int ci = tid + 256 * it;      // 2 kb x 128 rows x 8 chunks
        const int row = (ci >> 3) & 127;
        const float f = ROWS_T ? p.q_scale * __expf(Acum[row]) : __expf(fminf(0.f, a_last - Acum[row]));
        unsigned char* base = ROWS_T ? RA + (size_t)ci * 16 : RB + (size_t)(ci >> 10) * 32768 + (size_t)(ci & 1023) * 16;
        uint4* ptr = reinterpret_cast<uint4*>(base);
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
    const uint32_t ra = smem_u32(RA), rb = smem_u32(RB), rc = smem_u32(RC), rd = smem_u32(RD);
    const uint32_t dOut = tmem + 256;
    if (ROWS_T) {
      constexpr uint32_t idesc2 = idesc_bf16(128, 128, false, true);
#pragma unroll
      for (int kk = 0; kk < 16; ++kk)
        mma_bf16(dOut, smem_desc_sw128(rb + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                 smem_desc_sw128(rc + kk * 2048, 32768, 1024), idesc2, kk > 0);
    } else {
      constexpr uint32_t idesc2 = idesc_bf16(128, 128, true, true);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)    // K = t over Tr rows, against X2 rows t
        mma_bf16(dOut, smem_desc_sw128(ra + kk * 2048, 16384, 1024), smem_desc_sw128(rc + kk * 2048, 32768, 1024),
                 idesc2, kk > 0);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)    // K = t over -Ti rows, against rot X2 rows t
        mma_bf16(dOut, smem_desc_sw128(rb + 16384 + kk * 2048, 32768, 1024),
                 smem_desc_sw128(rc + 16384 + kk * 2048, 32768, 1024), idesc2, true);
    }
    if (has_state) {
      constexpr uint32_t idesc3 = idesc_bf16(128, 128, false, false);
      const uint32_t a3 = ROWS_T ? ra : rb;
      const uint32_t a3_stride = ROWS_T ? 16384u : 32768u;
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          mma_bf16(dOut, smem_desc_sw128(a3 + kb * a3_stride + kk * 32, 16, 1024),
                   smem_desc_sw128(rd + kb * 16384 + kk * 32, 16, 1024), idesc3, true);
    }
    mma_commit(&bars[2]);
  }
  __syncwarp();
  {
    const int q4 = warp & 3, hf = warp >> 2;
    const int t = q4 * 32 + lane;
    const uint32_t taddr = tmem + 256 + ((uint32_t)(q4 * 32) << 16) + hf * 64;
    void* outp = MODE == M_FWD ? p.y : MODE == M_DQ ? p.dq : MODE == M_DV ? p.dv : p.dk;
    const size_t rb = token_base(p, L.b, h, L.t0 + t, TD) + hf * 64;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(outp) + rb;
    const __nv_bfloat16* drow = reinterpret_cast<const __nv_bfloat16*>(MODE == M_DQ ? p.q : p.k) + rb;
    uint4 dpre[8];   // q (DQ) or k (DK) row for the decay-gradient dot product, fetched under the MMAs
    if ((MODE == M_DQ || MODE == M_DK) && t < L.len) {
#pragma unroll
      for (int g = 0; g < 8; ++g) dpre[g] = __ldg(reinterpret_cast<const uint4*>(drow) + g);
    }
    ok = mbar_wait(&bars[2], 0, 213) && ok;
    tc_fence_after();
    float dot = 0.f;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      float v[32];
      tmem_ld32(taddr + cc * 32, v);
      if (ok && t < L.len) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) =
              make_uint4(pack_bf162(v[8 * g], v[8 * g + 1]), pack_bf162(v[8 * g + 2], v[8 * g + 3]),
                         pack_bf162(v[8 * g + 4], v[8 * g + 5]), pack_bf162(v[8 * g + 6], v[8 * g + 7]));
          if (MODE == M_DQ || MODE == M_DK) {
            const uint4 x = dpre[cc * 4 + g];
            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x2 = unpack_bf162(xw[e]);
              dot = fmaf(x2.x, v[8 * g + 2 * e], dot);
              dot = fmaf(x2.y, v[8 * g + 2 * e + 1], dot);
            }
          }
        }
      }
    }
    if (MODE == M_DQ || MODE == M_DK) {
      // raw decay gradient dA_t = Re<q_t, dq_t> - Re<k_t, dk_t>: DQ stores its half, DK subtracts
      dots[hf * TC + t] = dot;
      __syncthreads();
      if (tid < L.len && ok) {
        const float d2 = dots[tid] + dots[TC + tid];
        float* g = p.dgamma + gamma_base(p, 0, L.b, h, L.t0 + tid);
        if (MODE == M_DQ) *g = d2; else *g -= d2;
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
