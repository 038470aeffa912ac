// Tensor-core chunk kernel of the PAM scan (forward output and the three gradients): planar operands, two CTAs per SM.
//
// After the TMA has delivered the interleaved (re, im) token rows, each tile is de-interleaved IN
// PLACE into a real plane and an imaginary plane (each one 128-byte-swizzled K-major block), so a
// complex product is four real MMAs (one of them with the tensor core's negate-A flag) and no
// rotated operand copies exist.  The decay-masked score tile T never touches shared memory: the
// epilogue rewrites the fp32 scores in TMEM as packed bf16 pairs and the second product reads its A
// operand from TMEM.  Shared memory: 3 x 32 KB; TMEM: 256 columns.
//
// All four modes have output rows = rows of A1 (t for FWD / DQ, s for DV / DK):
//
//   MODE  A1  B1  X2  mask             row factor (stage 3)          carried operand      out
//   FWD   q   k   v   col <= row       scale e^{A_row}               S    (out = op a)    y
//   DQ    dy  v   k   col <= row       scale e^{A_row}               S^H  (out = op^H a)  dq
//   DV    k   q   dy  row <= col < len exp(min(0, A_last - A_row))   dS                   dv
//   DK    v   dy  q   row <= col < len exp(min(0, A_last - A_row))   dS^H                 dk
//
//   stage 1  X = A1 conj(B1)^T                               Xr: cols [0,128)  Xi: cols [128,256)
//   epi 1    T = mask(row, col) * colfac[col] * X -> bf16    Tr: cols [0,64)   Ti: cols [128,192)
//   stage 2  acc  = T X2        (A from TMEM)                acc_r: cols [64,128)  acc_i: cols [192,256)
//   stage 3  acc += A1 (.) (cst * carried state)
//   epi 2    out  = rowfac[row] * acc
//
// The decay D(row, col) = exp(A_row - A_col) (or its transpose) is applied in factored form around a
// mid-chunk reference A_m: for the lower-triangular modes D = e^{A_row - A_m} e^{A_m - A_col}, the row
// factor being common to the intra-chunk and the carried-state term up to the chunk constant
// cst = e^{A_m}; for the upper-triangular modes D = e^{A_m - A_row} e^{A_col - A_m}, cst = e^{A_last - A_m}.
// That leaves 256 exponentials per chunk instead of 16 K and no row-scaling pass over shared memory.
// Exponents are clamped to [-80, 80]; this only alters terms whose true weight is below e^-80.
// (Like the backward formulas, the factored form assumes gamma + eps <= 1, where the reference's
// min(., 0) clamp of the decay matrix is inactive.)
#pragma once
#include "pam_scan_tc.cuh"

namespace qpam {
namespace tcs {

constexpr size_t CHUNK2_SMEM = 1024 + 3 * 32768 + 4096;

// De-interleave one [2 blocks][128 rows][128 B] tile in place: thread (row, hb) owns block hb of its
// row (32 complex numbers).  Phase 1 reads them; after a CTA-wide barrier phase 2 writes the 32 real
// parts to the real plane (block 0) and the 32 imaginary parts to the imaginary plane (block 1).
__device__ __forceinline__ void deint_read(const unsigned char* tile, int row, int hb, uint4 (&r)[8]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) r[c] = *reinterpret_cast<const uint4*>(tile + hb * 16384 + sw128(row, c));
}
__device__ __forceinline__ void deint_write(unsigned char* tile, int row, int hb, const uint4 (&r)[8]) {
#pragma unroll
  for (int c2 = 0; c2 < 4; ++c2) {
    // two source chunks (8 complex) -> one 16-byte chunk of reals and one of imaginaries
    const uint32_t w[8] = {r[2 * c2].x, r[2 * c2].y, r[2 * c2].z, r[2 * c2].w,
                           r[2 * c2 + 1].x, r[2 * c2 + 1].y, r[2 * c2 + 1].z, r[2 * c2 + 1].w};
    uint32_t re[4], im[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      re[e] = __byte_perm(w[2 * e], w[2 * e + 1], 0x5410);   // low halves
      im[e] = __byte_perm(w[2 * e], w[2 * e + 1], 0x7632);   // high halves
    }
    const int c = hb * 4 + c2;
    *reinterpret_cast<uint4*>(tile + sw128(row, c)) = make_uint4(re[0], re[1], re[2], re[3]);
    *reinterpret_cast<uint4*>(tile + 16384 + sw128(row, c)) = make_uint4(im[0], im[1], im[2], im[3]);
  }
}

template <int MODE>
__global__ void __launch_bounds__(256, 2) k_tc_chunk2(const __grid_constant__ ChunkMaps maps, ScanParams p) {
  using namespace umma;
  constexpr bool LOWER = (MODE == M_FWD || MODE == M_DQ);       // mask col <= row
  constexpr bool OP_H = (MODE == M_DQ || MODE == M_DK);         // carried operand conj-transposed
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* RA = smem;                  // A1: real plane, imaginary plane  (2 x [128 rows][128 B])
  unsigned char* RB = RA + 32768;            // B1 planes; after stage 1: carried state planes (2 x [64 rows][128 B])
  unsigned char* RC = RB + 32768;            // X2 planes
  float* Acum = reinterpret_cast<float*>(RC + 32768);   // [128]
  float* dots = Acum + TC;                              // [2][128]
  float* colfac = dots + 2 * TC;                        // [128]
  float* rowfac = colfac + TC;                          // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(rowfac + TC);  // [0] tma, [1] stage 1, [2] stages 2+3
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  const bool has_state = LOWER ? ((L.c > 0) || (p.s0 != nullptr)) : ((L.c < L.nc - 1) || (p.ds_final != nullptr));
  const int row0 = (L.b * p.H + h) * p.T + L.t0;
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    fence_barrier_init();
    // the token tiles are requested first: the prologue below (TMEM allocation, cumulative decay, factors,
    // carried-state prefetch) runs while they are in flight
    mbar_arrive_expect_tx(&bars[0], 6 * 16384);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(RA + kb * 16384, &maps.a1, &bars[0], kb * 64, row0);
      tma_load_2d(RB + kb * 16384, &maps.b1, &bars[0], kb * 64, row0);
      tma_load_2d(RC + kb * 16384, &maps.x2, &bars[0], kb * 64, row0);
    }
  }
  __syncwarp();
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  if (warp == 1) warp_cumsum128(Acum, p.gamma + gamma_base(p, 0, L.b, h, L.t0), L.len, p.eps, lane);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const float a_mid = Acum[TC / 2 - 1], a_last = Acum[TC - 1];
  auto cexp = [](float x) { return __expf(fminf(80.f, fmaxf(-80.f, x))); };
  if (tid < TC) {
    const float a = Acum[tid];
    if (LOWER) {
      colfac[tid] = cexp(a_mid - a);
      rowfac[tid] = p.q_scale * cexp(a - a_mid);
    } else {
      colfac[tid] = (tid < L.len) ? p.q_scale * cexp(a - a_mid) : 0.f;
      rowfac[tid] = cexp(a_mid - a);
    }
  }
  const float st_cst = LOWER ? cexp(a_mid) : cexp(a_last - a_mid);
  // carried state, fetched early and kept as packed bf16 (4 complex per item, 4 items per thread)
  uint32_t st_r[4][2], st_i[4][2];
  if (has_state) {
    const float2* st = LOWER ? p.states + state_base(p, 0, h, L.slot0 + L.c, TD)
                             : p.dstates + state_base(p, 0, h, L.slot0 + L.c + 1, TD);
    const float4* sg = reinterpret_cast<const float4*>(st);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;          // (i, c16): state[i][4*c16 .. +3]
      const float4 s01 = __ldg(sg + idx * 2), s23 = __ldg(sg + idx * 2 + 1);
      st_r[it][0] = pack_bf162(st_cst * s01.x, st_cst * s01.z);
      st_r[it][1] = pack_bf162(st_cst * s23.x, st_cst * s23.z);
      st_i[it][0] = pack_bf162(st_cst * s01.y, st_cst * s01.w);
      st_i[it][1] = pack_bf162(st_cst * s23.y, st_cst * s23.w);
    }
  }
  bool ok = mbar_wait(&bars[0], 0, 221);
  {
    // de-interleave the three tiles in place (read all, barrier, write all)
    const int row = tid >> 1, hb = tid & 1;
    uint4 ra[8], rb[8], rc[8];
    deint_read(RA, row, hb, ra);
    deint_read(RB, row, hb, rb);
    deint_read(RC, row, hb, rc);
    __syncthreads();
    deint_write(RA, row, hb, ra);
    deint_write(RB, row, hb, rb);
    deint_write(RC, row, hb, rc);
  }
  fence_proxy_async();
  __syncthreads();
  const uint32_t a_r = smem_u32(RA), a_i = a_r + 16384, b_r = smem_u32(RB), b_i = b_r + 16384;
  const uint32_t x_r = smem_u32(RC), x_i = x_r + 16384;
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t id = idesc_bf16(128, 128, false, false);
    constexpr uint32_t idn = idesc_bf16_nega(128, 128, false, false);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)   // Xr = ar br^T
      mma_bf16(tmem, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)   //    + ai bi^T
      mma_bf16(tmem, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), id, true);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)   // Xi = ai br^T
      mma_bf16(tmem + 128, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)   //    - ar bi^T
      mma_bf16(tmem + 128, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), idn, true);
    mma_commit(&bars[1]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[1], 0, 222) && ok;
  tc_fence_after();
  const int q4 = warp & 3, hf = warp >> 2;
  const int r = q4 * 32 + lane;                               // this thread's row (TMEM lane)
  const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
  {
    // epilogue 1: masked, decayed scores of columns [64 hf, 64 hf + 64) as packed bf16 pairs
    uint32_t tr[32], ti[32];
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c0 = hf * 64 + cc * 16;
      const bool dead = LOWER ? (c0 > q4 * 32 + 31) : (c0 + 15 < q4 * 32);   // warp-uniform
      if (dead) {
#pragma unroll
        for (int j = 0; j < 8; ++j) tr[cc * 8 + j] = ti[cc * 8 + j] = 0u;
      } else {
        float xr[16], xi[16];
        tmem_ld16(tlane + c0, xr);
        tmem_ld16(tlane + 128 + c0, xi);
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          float d[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = c0 + j + e;
            d[e] = (LOWER ? (c <= r) : (c >= r)) ? colfac[c] : 0.f;
          }
          tr[cc * 8 + (j >> 1)] = pack_bf162(d[0] * xr[j], d[1] * xr[j + 1]);
          ti[cc * 8 + (j >> 1)] = pack_bf162(d[0] * xi[j], d[1] * xi[j + 1]);
        }
      }
    }
    tc_fence_before();
    __syncthreads();          // every warp has read its scores: their columns may be overwritten
    tc_fence_after();
    {
      uint32_t lo[16], hi[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) { lo[j] = tr[j]; hi[j] = tr[16 + j]; }
      tmem_st16(tlane + hf * 32, lo);
      tmem_st16(tlane + hf * 32 + 16, hi);
#pragma unroll
      for (int j = 0; j < 16; ++j) { lo[j] = ti[j]; hi[j] = ti[16 + j]; }
      tmem_st16(tlane + 128 + hf * 32, lo);
      tmem_st16(tlane + 128 + hf * 32 + 16, hi);
      tmem_st_wait();
    }
    if (has_state) {
      // carried state planes (already multiplied by the chunk constant) into the B1 region
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int idx = tid + 256 * it;
        const int i = idx >> 4, c16 = idx & 15;
        const uint32_t off = sw128(i, c16 >> 1) + (c16 & 1) * 8;
        *reinterpret_cast<uint2*>(RB + off) = make_uint2(st_r[it][0], st_r[it][1]);
        *reinterpret_cast<uint2*>(RB + 8192 + off) = make_uint2(st_i[it][0], st_i[it][1]);
      }
    }
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t id = idesc_bf16(128, 64, false, true);        // A: TMEM, B: MN-major plane
    constexpr uint32_t idn = idesc_bf16_nega(128, 64, false, true);
    const uint32_t Tr = tmem, Ti = tmem + 128, Or = tmem + 64, Oi = tmem + 192;
    // out_r = Tr x2r - Ti x2i ; out_i = Tr x2i + Ti x2r      (K = 128 columns = 8 steps of 16)
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      mma_bf16_ts(Or, Tr + kk * 8, smem_desc_sw128(x_r + kk * 2048, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      mma_bf16_ts(Or, Ti + kk * 8, smem_desc_sw128(x_i + kk * 2048, 16, 1024), idn, true);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      mma_bf16_ts(Oi, Tr + kk * 8, smem_desc_sw128(x_i + kk * 2048, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      mma_bf16_ts(Oi, Ti + kk * 8, smem_desc_sw128(x_r + kk * 2048, 16, 1024), id, true);
    if (has_state) {
      const uint32_t s_r = b_r, s_i = b_r + 8192;   // [64 rows i][64 j] planes
      if (!OP_H) {
        // out[r][i] += sum_j a3[r][j] S[i][j]:  B K-major (rows i, K = j)
        constexpr uint32_t k3 = idesc_bf16(128, 64, false, false), k3n = idesc_bf16_nega(128, 64, false, false);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ar = smem_desc_sw128(a_r + kk * 32, 16, 1024), ai = smem_desc_sw128(a_i + kk * 32, 16, 1024);
          const uint64_t sr = smem_desc_sw128(s_r + kk * 32, 16, 1024), si = smem_desc_sw128(s_i + kk * 32, 16, 1024);
          mma_bf16(Or, ar, sr, k3, true);    // + a3r Sr^T
          mma_bf16(Or, ai, si, k3n, true);   // - a3i Si^T
          mma_bf16(Oi, ar, si, k3, true);    // + a3r Si^T
          mma_bf16(Oi, ai, sr, k3, true);    // + a3i Sr^T
        }
      } else {
        // out[r][j] += sum_i conj(S[i][j]) a3[r][i]:  B MN-major (rows = K = i, N = j)
        constexpr uint32_t k3 = idesc_bf16(128, 64, false, true), k3n = idesc_bf16_nega(128, 64, false, true);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ar = smem_desc_sw128(a_r + kk * 32, 16, 1024), ai = smem_desc_sw128(a_i + kk * 32, 16, 1024);
          const uint64_t sr = smem_desc_sw128(s_r + kk * 2048, 16, 1024), si = smem_desc_sw128(s_i + kk * 2048, 16, 1024);
          mma_bf16(Or, ar, sr, k3, true);    // + a3r Sr
          mma_bf16(Or, ai, si, k3, true);    // + a3i Si
          mma_bf16(Oi, ai, sr, k3, true);    // + a3i Sr
          mma_bf16(Oi, ar, si, k3n, true);   // - a3r Si
        }
      }
    }
    mma_commit(&bars[2]);
  }
  __syncwarp();
  {
    void* outp = MODE == M_FWD ? p.y : MODE == M_DQ ? p.dq : MODE == M_DV ? p.dv : p.dk;
    const size_t rbase = token_base(p, L.b, h, L.t0 + r, TD) + hf * 64;   // channels [32 hf, 32 hf + 32)
    const size_t obase = (MODE == M_FWD && p.y_token_major)
                             ? (((size_t)L.b * p.T + L.t0 + r) * p.H + h) * (size_t)(TD * 2) + hf * 64 : rbase;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(outp) + obase;
    const __nv_bfloat16* drow = reinterpret_cast<const __nv_bfloat16*>(MODE == M_DQ ? p.q : p.k) + rbase;
    uint4 dpre[8];
    if ((MODE == M_DQ || MODE == M_DK) && r < L.len) {
#pragma unroll
      for (int g = 0; g < 8; ++g) dpre[g] = __ldg(reinterpret_cast<const uint4*>(drow) + g);
    }
    ok = mbar_wait(&bars[2], 0, 223) && ok;
    tc_fence_after();
    const float rf = rowfac[r];
    float dot = 0.f;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      float vr[16], vi[16];
      tmem_ld16(tlane + 64 + hf * 32 + cc * 16, vr);
      tmem_ld16(tlane + 192 + hf * 32 + cc * 16, vi);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        vr[j] *= rf;
        vi[j] *= rf;
      }
      if (ok && r < L.len) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {     // 4 complex channels -> one 16-byte store
          *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) =
              make_uint4(pack_bf162(vr[4 * g], vi[4 * g]), pack_bf162(vr[4 * g + 1], vi[4 * g + 1]),
                         pack_bf162(vr[4 * g + 2], vi[4 * g + 2]), pack_bf162(vr[4 * g + 3], vi[4 * g + 3]));
          if (MODE == M_DQ || MODE == M_DK) {
            const uint4 x = dpre[cc * 4 + g];
            const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x2 = unpack_bf162(xw[e]);
              dot = fmaf(x2.x, vr[4 * g + e], dot);
              dot = fmaf(x2.y, vi[4 * g + e], dot);
            }
          }
        }
      }
    }
    if (MODE == M_DQ || MODE == M_DK) {
      dots[hf * TC + r] = dot;
      __syncthreads();
      if (tid < L.len && ok) {
        const float d2 = dots[tid] + dots[TC + tid];
        const size_t gi = gamma_base(p, 0, L.b, h, L.t0 + tid);
        if (MODE == M_DQ) p.dgamma[gi] = d2; else p.dA_k[gi] = d2;   // combined by k_tc_dgamma_finalize
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<256>(tmem);
  }
}

}  // namespace tcs
}  // namespace qpam
