// Tensor-core chunk kernels of the PAM scan for bf16 token tensors, head dim 64, one state: the forward output
// and the three gradients (dq, dv, dk) of a 128-token chunk.  One CTA of 256 threads per (chunk, job), two CTAs
// per SM (96 KB shared memory, 256 TMEM columns each); the backward launches the three jobs of a chunk as
// neighbouring CTAs, so the token tiles they share are fetched from DRAM once and found in L2 after that.
//
// After the TMA has delivered the interleaved (re, im) token rows, each tile is de-interleaved IN PLACE into a
// real plane and an imaginary plane (each one 128-byte-swizzled K-major block), so a complex product is four
// real MMAs (one of them with the tensor core's negate-A flag) and no rotated operand copies exist.  A job is
//
//   stage 1  X   = A1 conj(B1)^T                      fp32 scores in TMEM     Xr: cols [0,128)  Xi: [128,256)
//   epi 1    T   = mask (.) D (.) X  -> bf16          written over the thread's OWN Xr columns (no barrier between)
//   stage 2  acc = T X2   (A operand read from TMEM)  acc_r: cols [128,192)   acc_i: cols [192,256)
//   stage 3  acc += A1 (.) carried state planes       (planes take the place of the B1 tile)
//   epi 2    out = rowfac (.) acc -> bf16 rows in global memory
//
//   job  A1  B1  X2  mask              carried operand                                     out
//   FWD  q   k   v   col <= row        S_c     (state entering the chunk)                  y
//   DQ   dy  v   k   col <= row        S_c^H                                               dq (+ Re<q, dq>)
//   DV   k   q   dy  row <= col < len  dS_c+1  (gradient reaching the state after it)      dv
//   DK   v   dy  q   row <= col < len  dS_c+1^H                                            dk (+ Re<k, dk>)
//
// A thread owns half a row: 64 score columns in epi 1, 32 output channels in epi 2.
//
// Decay.  D(t, s) = exp(A_t - A_s) for s <= t (A = cumulative log decay inside the chunk).  When the whole
// chunk decays by less than e^-80 the factored form  e^{A_t - A_m} e^{A_m - A_s}  around the mid-chunk
// value A_m is exact (every exponent stays inside [-80, 80]): the column factor goes into T, the row
// factor into epi 2, where it also carries the decay of the carried-state term (chunk constant folded into
// the state planes) -- 256 exponentials per chunk instead of 16 K.  (The dq and dk jobs put both factors into T
// and rescale the A1 rows for the carried-state term instead: their scores must round alike, see chunk_job.)
// A chunk that decays more strongly takes the
// slow path: every score gets its own exp(A_t - A_s), and the carried-state product is formed first, rescaled
// row by row in TMEM, and the score product accumulates onto it.  Both paths are exact for every gamma in (0, 1].
// (Like the backward formulas, both assume gamma + eps <= 1, where the reference's min(., 0) clamp of the
// decay matrix is inactive.)
#pragma once
#include "pam_scan_tc.cuh"

namespace qpam {
namespace tcs {

constexpr size_t CHUNK2_SMEM = 1024 + 3 * 32768 + 4096;
constexpr float STRONG_DECAY = -80.f;      // cumulative log decay of a chunk below which the factored form is left
constexpr int ANCHOR_PARTS = 64;           // partial sums per decay-gradient anchor left by the reverse carry

struct BwdMaps {
  CUtensorMap q, k, v, dy;   // [B*H*T rows][128 bf16], boxes of 64 x 128, 128-byte swizzle
  CUtensorMap dq, dk, dv;    // outputs, same shape, boxes of 64 x 32 (one per epilogue warp)
};

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

// ---- MMA issue (one thread) -----------------------------------------------------------------------------
// X = A1 conj(B1)^T : Xr = ar br^T + ai bi^T, Xi = ai br^T - ar bi^T  (planes K-major, K = 64)
// IMAG_SWAPPED: the two halves of Xi are accumulated in the other order, so that the job whose operands are swapped
// (dk: v dy^H against dq: dy v^H) adds the same numbers in the same order and gets the negated imaginary part bit
// for bit.
template <bool IMAG_SWAPPED = false>
__device__ __forceinline__ void bw_issue_scores(uint32_t slot, uint32_t a_r, uint32_t b_r) {
  using namespace umma;
  constexpr uint32_t id = idesc_bf16(128, 128, false, false);
  constexpr uint32_t idn = idesc_bf16_nega(128, 128, false, false);
  const uint32_t a_i = a_r + 16384, b_i = b_r + 16384;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    mma_bf16(slot, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, kk > 0);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk)
    mma_bf16(slot, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), id, true);
  if (!IMAG_SWAPPED) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(slot + 128, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(slot + 128, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), idn, true);
  } else {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(slot + 128, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), idn, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(slot + 128, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, true);
  }
}

// TMEM column of the packed bf16 scores of k-step kk (16 score columns = 8 TMEM columns): the thread that
// owns score columns [32 cq, 32 cq + 32) of a row writes  Tr(2cq) Tr(2cq+1) Ti(2cq) Ti(2cq+1)  over them.
__device__ __forceinline__ uint32_t bw_tr_col(int kk) { return (uint32_t)(32 * (kk >> 1) + 8 * (kk & 1)); }
__device__ __forceinline__ uint32_t bw_ti_col(int kk) { return bw_tr_col(kk) + 16u; }

// acc = T X2 : out_r = Tr x2r - Ti x2i, out_i = Tr x2i + Ti x2r   (X2 planes MN-major, K = 128 tokens)
__device__ __forceinline__ void bw_issue_out(uint32_t slot, uint32_t x_r, bool accumulate = false) {
  using namespace umma;
  constexpr uint32_t id = idesc_bf16(128, 64, false, true);
  constexpr uint32_t idn = idesc_bf16_nega(128, 64, false, true);
  const uint32_t x_i = x_r + 16384, Or = slot + 128, Oi = slot + 192;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    mma_bf16_ts(Or, slot + bw_tr_col(kk), smem_desc_sw128(x_r + kk * 2048, 16, 1024), id, accumulate || kk > 0);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    mma_bf16_ts(Or, slot + bw_ti_col(kk), smem_desc_sw128(x_i + kk * 2048, 16, 1024), idn, true);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    mma_bf16_ts(Oi, slot + bw_tr_col(kk), smem_desc_sw128(x_i + kk * 2048, 16, 1024), id, accumulate || kk > 0);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    mma_bf16_ts(Oi, slot + bw_ti_col(kk), smem_desc_sw128(x_r + kk * 2048, 16, 1024), id, true);
}

// acc (+)= A1 (.) state planes [64 rows i][64 j]:  OP_H == false: out[r][i] = sum_j a[r][j] S[i][j];
// OP_H == true: out[r][j] = sum_i conj(S[i][j]) a[r][i].
template <bool OP_H>
__device__ __forceinline__ void bw_issue_state(uint32_t slot, uint32_t a_r, uint32_t s_r, bool accumulate) {
  using namespace umma;
  const uint32_t a_i = a_r + 16384, s_i = s_r + 8192, Or = slot + 128, Oi = slot + 192;
  if (!OP_H) {
    constexpr uint32_t k3 = idesc_bf16(128, 64, false, false), k3n = idesc_bf16_nega(128, 64, false, false);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint64_t ar = smem_desc_sw128(a_r + kk * 32, 16, 1024), ai = smem_desc_sw128(a_i + kk * 32, 16, 1024);
      const uint64_t sr = smem_desc_sw128(s_r + kk * 32, 16, 1024), si = smem_desc_sw128(s_i + kk * 32, 16, 1024);
      mma_bf16(Or, ar, sr, k3, accumulate || kk > 0);    // + a_r S_r^T
      mma_bf16(Or, ai, si, k3n, true);                   // - a_i S_i^T
      mma_bf16(Oi, ar, si, k3, accumulate || kk > 0);    // + a_r S_i^T
      mma_bf16(Oi, ai, sr, k3, true);                    // + a_i S_r^T
    }
  } else {
    constexpr uint32_t k3 = idesc_bf16(128, 64, false, true), k3n = idesc_bf16_nega(128, 64, false, true);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint64_t ar = smem_desc_sw128(a_r + kk * 32, 16, 1024), ai = smem_desc_sw128(a_i + kk * 32, 16, 1024);
      const uint64_t sr = smem_desc_sw128(s_r + kk * 2048, 16, 1024), si = smem_desc_sw128(s_i + kk * 2048, 16, 1024);
      mma_bf16(Or, ar, sr, k3, accumulate || kk > 0);    // + a_r S_r
      mma_bf16(Or, ai, si, k3, true);                    // + a_i S_i
      mma_bf16(Oi, ai, sr, k3, accumulate || kk > 0);    // + a_i S_r
      mma_bf16(Oi, ar, si, k3n, true);                   // - a_r S_i
    }
  }
}

// ---- epilogue 1: decay-masked scores of this thread's row, columns [32 cb, 32 cb + 32), as packed bf16 ------
// fast path: T = [mask] cfac[col] X;  slow path (STRONG): T = [mask] scale exp(-|A_row - A_col|) X.
// ROWW: the row's own factor `rowf` multiplies the weight before the score is rounded (see chunk_job).
template <bool LOWER, bool STRONG, bool ROWW>
__device__ __forceinline__ void bw_epi_scores_t(uint32_t tlane_slot, int q4, int cb, int r, int len,
                                                const float* __restrict__ cfac, const float* __restrict__ Acum,
                                                float scale, float rowf) {
  using namespace umma;
  const int c0 = 32 * cb;
  const bool dead = LOWER ? (c0 > q4 * 32 + 31) : (c0 + 31 < q4 * 32);      // warp-uniform
  const bool full = LOWER ? (c0 + 31 <= q4 * 32) : (c0 >= q4 * 32 + 31);    // no triangle inside the block
  uint32_t tr[16], ti[16];
  if (dead) {
#pragma unroll
    for (int j = 0; j < 16; ++j) tr[j] = ti[j] = 0u;
  } else {
    const float a_r = STRONG ? Acum[r] : 0.f;
    uint32_t xr0[16], xr1[16], xi0[16], xi1[16];
    tmem_ld16x4(tlane_slot + c0, xr0, tlane_slot + c0 + 16, xr1, tlane_slot + 128 + c0, xi0, tlane_slot + 128 + c0 + 16, xi1);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        float d[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = c0 + 16 * hh + j + e;
          bool on = full || (LOWER ? (c <= r) : (c >= r));
          if (!LOWER && STRONG) on = on && (c < len);      // (the column factors of the fast path are zero past `len`)
          const float w = STRONG ? scale * __expf(fminf(0.f, LOWER ? a_r - Acum[c] : Acum[c] - a_r))
                                 : (ROWW ? rowf * cfac[c] : cfac[c]);
          d[e] = on ? w : 0.f;
        }
        const float r0 = __uint_as_float(hh ? xr1[j] : xr0[j]), r1 = __uint_as_float(hh ? xr1[j + 1] : xr0[j + 1]);
        const float i0 = __uint_as_float(hh ? xi1[j] : xi0[j]), i1 = __uint_as_float(hh ? xi1[j + 1] : xi0[j + 1]);
        tr[hh * 8 + (j >> 1)] = pack_bf162(d[0] * r0, d[1] * r1);
        ti[hh * 8 + (j >> 1)] = pack_bf162(d[0] * i0, d[1] * i1);
      }
    }
  }
  // every load of this thread has completed: its own 32 Xr columns take the packed scores
  tmem_st16(tlane_slot + c0, tr);
  tmem_st16(tlane_slot + c0 + 16, ti);
}
template <bool LOWER, bool ROWW = false>
__device__ __forceinline__ void bw_epi_scores(uint32_t tlane_slot, int q4, int cb, int r, int len, bool strong,
                                              const float* __restrict__ cfac, const float* __restrict__ Acum,
                                              float scale, float rowf = 1.f) {
  if (strong) bw_epi_scores_t<LOWER, true, false>(tlane_slot, q4, cb, r, len, cfac, Acum, scale, 1.f);
  else bw_epi_scores_t<LOWER, false, ROWW>(tlane_slot, q4, cb, r, len, cfac, Acum, scale, rowf);
}

// ---- epilogue 2: out[r][16 cb .. 16 cb + 16) = rf * acc -> global; optional part of Re<x_r, out_r>, x_r given as the
// four 16-byte pieces of the interleaved bf16 row that cover these channels ------------------------------------
// `stage` != nullptr: the 16-byte pieces go to this row of a 128-byte-swizzled staging block (piece index
// 4 * (cb & 1) + g, row & 7 = `sw`) instead of global memory; a TMA store moves the block afterwards.
template <bool DOT, bool ADD = false>
__device__ __forceinline__ float bw_epi_out(uint32_t tlane_slot, int cb, float rf, __nv_bfloat16* __restrict__ orow,
                                            const uint4 (&xg)[4], bool valid, unsigned char* stage = nullptr, int sw = 0) {
  using namespace umma;
  float vr[16], vi[16];
  tmem_ld16x2(tlane_slot + 128 + 16 * cb, vr, tlane_slot + 192 + 16 * cb, vi);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    vr[j] *= rf;
    vi[j] *= rf;
  }
  float dot = 0.f;
  if (valid) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {   // 4 complex channels -> one 16-byte store
      const uint4 pk = make_uint4(pack_bf162(vr[4 * g], vi[4 * g]), pack_bf162(vr[4 * g + 1], vi[4 * g + 1]),
                                  pack_bf162(vr[4 * g + 2], vi[4 * g + 2]), pack_bf162(vr[4 * g + 3], vi[4 * g + 3]));
      if (stage != nullptr) {
        *reinterpret_cast<uint4*>(stage + (((4 * (cb & 1) + g) ^ sw) << 4)) = pk;
      } else if (ADD) {          // ragged chunk of an accumulating call: read, add, write (this lane's own row)
        const uint4 o = *reinterpret_cast<const uint4*>(orow + g * 8);
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
        uint32_t nw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x2 = unpack_bf162(ow[e]);
          nw[e] = pack_bf162(x2.x + vr[4 * g + e], x2.y + vi[4 * g + e]);
        }
        *reinterpret_cast<uint4*>(orow + g * 8) = make_uint4(nw[0], nw[1], nw[2], nw[3]);
      } else {
        *reinterpret_cast<uint4*>(orow + g * 8) = pk;
      }
      if (DOT) {
        const uint32_t xw[4] = {xg[g].x, xg[g].y, xg[g].z, xg[g].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x2 = unpack_bf162(xw[e]);
          dot = fmaf(x2.x, vr[4 * g + e], dot);
          dot = fmaf(x2.y, vi[4 * g + e], dot);
        }
      }
    }
  }
  return dot;
}
// slow path: multiply this thread's share of its row's accumulators (channel blocks 2 hf, 2 hf + 1) by w in TMEM
__device__ __forceinline__ void rescale_acc_half(uint32_t tlane_slot, int hf, float w) {
  using namespace umma;
#pragma unroll 1
  for (int cb = 2 * hf; cb < 2 * hf + 2; ++cb) {
    float vr[16], vi[16];
    tmem_ld16x2(tlane_slot + 128 + 16 * cb, vr, tlane_slot + 192 + 16 * cb, vi);
    uint32_t ur[16], ui[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      ur[j] = __float_as_uint(w * vr[j]);
      ui[j] = __float_as_uint(w * vi[j]);
    }
    tmem_st16(tlane_slot + 128 + 16 * cb, ur);
    tmem_st16(tlane_slot + 192 + 16 * cb, ui);
  }
  tmem_st_wait();
}

// ---------------------------------------------------------------------------------------------
// One job of one chunk (256 threads; the caller's CTA holds nothing else).
// ---------------------------------------------------------------------------------------------
template <int MODE, bool ACC = false>      // ACC: the output is added to what the buffer holds (gradients only)
__device__ __forceinline__ void chunk_job(const CUtensorMap* __restrict__ ma1, const CUtensorMap* __restrict__ mb1,
                                          const CUtensorMap* __restrict__ mx2, const CUtensorMap* __restrict__ mout,
                                          const CUtensorMap* __restrict__ mdot, const ScanParams& p, int chunk_x, int h,
                                          unsigned char* smem) {
  using namespace umma;
  constexpr bool LOWER = (MODE == M_FWD || MODE == M_DQ);       // mask col <= row
  constexpr bool OP_H = (MODE == M_DQ || MODE == M_DK);         // carried operand conj-transposed
  constexpr bool DOT = (MODE == M_DQ || MODE == M_DK);          // also leaves Re<x_row, out_row>, x = q (dq) or k (dk): mdot
  // The decay gradient is a running sum of Re<q_t, dq_t> - Re<k_t, dk_t> over the chunk, in which the contribution of
  // every (t, s) pair cancels -- exactly only if dq and dk are built from the SAME rounded scores.  So these two jobs
  // put the whole weight e^{A_t - A_s} (row factor x column factor) into a score before it is rounded to bf16, which
  // makes the dk job's scores the conjugate transpose of the dq job's bit for bit; the carried-state term gets its row
  // factor from the A1 rows, rescaled between stage 1 and stage 3.  (With the row factor applied in epilogue 2 the two
  // jobs rounded different numbers and the noise of up to 128 tokens piled up in the sum: 1-3 % of dgamma at decays
  // around 0.5 per token.)  The forward and the dv job keep the row factor in epilogue 2.
  constexpr bool ROWW = DOT;
  unsigned char* RA = smem;                  // A1: real plane, imaginary plane  (2 x [128 rows][128 B])
  unsigned char* RB = RA + 32768;            // B1 planes; after stage 1: carried state planes (2 x [64 rows][128 B])
  unsigned char* RC = RB + 32768;            // X2 planes
  float* Acum = reinterpret_cast<float*>(RC + 32768);   // [128]
  float* dots = Acum + TC;                              // [2][128]
  float* cfac = dots + 2 * TC;                          // [128]
  float* rfac = cfac + TC;                              // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(rfac + TC);  // [0] tma, [1] scores, [2] outputs, [3] state product, [4] carried state
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  int* failed = reinterpret_cast<int*>(tmem_slot + 1);      // error word as found at the start of this CTA
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, chunk_x);
  if (!L.valid) return;
  if (tid == 64) *failed = device_error_now();     // not on warp 1: its cumulative decay is the prologue's critical path
  const bool has_state = LOWER ? ((L.c > 0) || (p.s0 != nullptr)) : ((L.c < L.nc - 1) || (p.ds_final != nullptr));
  const int row0 = (L.b * p.H + h) * p.T + L.t0;
  float graw[4] = {1.f, 1.f, 1.f, 1.f};
  if (warp == 1) warp_cumsum128_load(graw, p.gamma + gamma_base(p, 0, L.b, h, L.t0), L.len, lane);
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
    // the token tiles are requested first: the prologue below (TMEM allocation, cumulative decay, factors,
    // carried-state prefetch) runs while they are in flight
    mbar_arrive_expect_tx(&bars[0], 6 * 16384);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(RA + kb * 16384, ma1, &bars[0], kb * 64, row0);
      tma_load_2d(RB + kb * 16384, mb1, &bars[0], kb * 64, row0);
      tma_load_2d(RC + kb * 16384, mx2, &bars[0], kb * 64, row0);
    }
  }
  __syncwarp();
  if (warp == 1) warp_cumsum128_finish(Acum, graw, L.len, p.eps, lane);
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (*failed != 0) {
    // an earlier launch gave up on a wait: leave the outputs alone (the tiles still land; wait for them so that no
    // bulk copy is in flight into this CTA's shared memory when it exits)
    mbar_wait(&bars[0], 0, 225);
    __syncthreads();
    if (warp == 0) tmem_dealloc<256>(tmem);
    return;
  }
  const float a_mid = Acum[TC / 2 - 1], a_last = Acum[TC - 1];
  const bool strong = a_last < STRONG_DECAY;             // CTA-uniform
  if (tid < TC) {
    const float a = Acum[tid];
    const float up = strong ? 1.f : __expf(a_mid - a), dn = p.q_scale * (strong ? 1.f : __expf(a - a_mid));
    if (LOWER) {
      cfac[tid] = up;
      rfac[tid] = dn;
    } else {
      cfac[tid] = (tid < L.len) ? dn : 0.f;
      rfac[tid] = up;
    }
  }
  bool ok = mbar_wait(&bars[0], 0, 221);
  {
    // de-interleave the three tiles in place (read all, barrier, write all)
    const int row = tid & 127, hb = tid >> 7;      // a quarter-warp reads eight rows of one block: no bank conflict
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
  const uint32_t a_r = smem_u32(RA), b_r = smem_u32(RB), x_r = smem_u32(RC);
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    bw_issue_scores<MODE == M_DK>(tmem, a_r, b_r);
    mma_commit(&bars[1]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[1], 0, 222) && ok;
  tc_fence_after();
  if (has_state && tid == 0) {
    // stage 1 has released the B1 region: the carried state (fp32, 32 KB, contiguous) comes into it by one bulk copy
    // while epilogue 1 runs
    const float2* st = LOWER ? p.states + state_base(p, 0, h, L.slot0 + L.c, TD)
                             : p.dstates + state_base(p, 0, h, L.slot0 + L.c + 1, TD);
    mbar_arrive_expect_tx(&bars[4], 32768);
    bulk_load_1d(RB, st, 32768, &bars[4]);
  }
  const int q4 = warp & 3, hf = warp >> 2;
  const int r = q4 * 32 + lane;                               // this thread's row (TMEM lane)
  const uint32_t tl = tmem + ((uint32_t)(q4 * 32) << 16);
  // epilogue 1: masked, decayed scores of columns [64 hf, 64 hf + 64) as packed bf16 pairs
#pragma unroll 1
  for (int cb = 2 * hf; cb < 2 * hf + 2; ++cb)
    bw_epi_scores<LOWER, ROWW>(tl, q4, cb, r, L.len, strong, cfac, Acum, p.q_scale, ROWW ? rfac[r] : 1.f);
  tmem_st_wait();
  if (ROWW && has_state && !strong) {
    // stage 1 was the last reader of the unscaled A1 rows: thread (row r, plane hf) multiplies its 128 bytes by the
    // row factor f = fh + fl (two bf16 numbers; x fh + x fl in one fused multiply-add rounds x f once), eight rows of a
    // quarter-warp spread over all banks by the swizzle
    const float f = rfac[r];
    const __nv_bfloat16 fh = __float2bfloat16_rn(f), fl = __float2bfloat16_rn(f - __bfloat162float(fh));
    const __nv_bfloat162 fh2 = __bfloat162bfloat162(fh), fl2 = __bfloat162bfloat162(fl);
    unsigned char* prow = RA + hf * 16384;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4* pp = reinterpret_cast<uint4*>(prow + sw128(r, c));
      uint4 x = *pp;
      __nv_bfloat162* xs = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
      for (int e = 0; e < 4; ++e) xs[e] = __hfma2(xs[e], fh2, __hmul2(xs[e], fl2));
      *pp = x;
    }
  }
  if (has_state) {
    // the carried state has landed as fp32 [i][j] (re, im): every thread reads its four items (4 complex each; the two
    // 16-byte halves in an order that keeps a quarter-warp on distinct banks), a barrier, and the bf16 planes, times the
    // chunk constant, are written over it
    ok = mbar_wait(&bars[4], 0, 226) && ok;
    const float st_cst = strong ? 1.f : (LOWER ? __expf(a_mid) : __expf(a_last - a_mid));
    const int flip = (lane >> 2) & 1;
    uint32_t st_r[4][2], st_i[4][2];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;          // (i, c16): state[i][4*c16 .. +3]
      const float4 a = *reinterpret_cast<const float4*>(RB + idx * 32 + flip * 16);
      const float4 b = *reinterpret_cast<const float4*>(RB + idx * 32 + (flip ^ 1) * 16);
      const float4 s01 = flip ? b : a, s23 = flip ? a : b;
      st_r[it][0] = pack_bf162(st_cst * s01.x, st_cst * s01.z);
      st_r[it][1] = pack_bf162(st_cst * s23.x, st_cst * s23.z);
      st_i[it][0] = pack_bf162(st_cst * s01.y, st_cst * s01.w);
      st_i[it][1] = pack_bf162(st_cst * s23.y, st_cst * s23.w);
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;
      const int i = idx >> 4, c16 = idx & 15;
      const uint32_t off = sw128(i, c16 >> 1) + (c16 & 1) * 8;
      *reinterpret_cast<uint2*>(RB + off) = make_uint2(st_r[it][0], st_r[it][1]);
      *reinterpret_cast<uint2*>(RB + 8192 + off) = make_uint2(st_i[it][0], st_i[it][1]);
    }
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  const bool two_step = strong && has_state;            // CTA-uniform
  if (two_step) {
    // slow path: the carried-state product alone, then every row rescaled by its own decay in TMEM
    if (warp == 0 && elect_one()) {
      tc_fence_after();
      bw_issue_state<OP_H>(tmem, a_r, b_r, false);
      mma_commit(&bars[3]);
    }
    __syncwarp();
    ok = mbar_wait(&bars[3], 0, 224) && ok;
    tc_fence_after();
    const float a_row = Acum[r];
    rescale_acc_half(tl, hf, LOWER ? p.q_scale * __expf(a_row) : __expf(fminf(0.f, a_last - a_row)));
    tc_fence_before();
    __syncthreads();
  }
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    const bool state_now = has_state && !strong;
    if (state_now) {        // the carried-state product first: it is the last reader of the A1 planes
      bw_issue_state<OP_H>(tmem, a_r, b_r, false);
      if (DOT) mma_commit(&bars[3]);
    }
    bw_issue_out(tmem, x_r, two_step || state_now);
    mma_commit(&bars[2]);
    if (DOT) {
      // The rows of q (k) for the decay dots arrive by TMA in the A1 region as soon as no MMA reads it any more (a
      // per-lane global read of one's own row costs 32 cache lines per instruction).
      bool free_now = true;
      if (state_now) free_now = mbar_wait(&bars[3], 0, 227);
      if (free_now) {
        mbar_arrive_expect_tx(&bars[0], 2 * 16384);
        tma_load_2d(RA, mdot, &bars[0], 0, row0);
        tma_load_2d(RA + 16384, mdot, &bars[0], 64, row0);
      }
    }
  }
  __syncwarp();
  {
    void* outp = MODE == M_FWD ? p.y : MODE == M_DQ ? p.dq : MODE == M_DV ? p.dv : p.dk;
    const size_t rbase = token_base(p, L.b, h, L.t0 + r, TD) + hf * 64;   // channels [32 hf, 32 hf + 32)
    const size_t obase = (MODE == M_FWD && p.y_token_major)
                             ? (((size_t)L.b * p.T + L.t0 + r) * p.H + h) * (size_t)(TD * 2) + hf * 64 : rbase;
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(outp) + obase;
    const bool valid = r < L.len;
    uint4 dpre[2][4];
    ok = mbar_wait(&bars[2], 0, 223) && ok;
    tc_fence_after();
    if (DOT) {
      ok = mbar_wait(&bars[0], 1, 228) && ok;      // second use of the tile barrier: the rows for the dots
#pragma unroll
      for (int g = 0; g < 8; ++g) dpre[g >> 2][g & 3] = *reinterpret_cast<const uint4*>(RA + hf * 16384 + sw128(r, g));
    }
    const float rf = (strong || ROWW) ? 1.f : rfac[r];
    // A full chunk leaves through the X2 region, which every MMA has finished reading: each warp stages its 32 rows
    // x 128 bytes there and one TMA store moves the block (whole 128-byte lines instead of 16 bytes per lane and
    // row).  A ragged chunk (its rows past `len` belong to someone else) stores per lane.
    const bool bulk = ok && L.len == TC;                                             // CTA-uniform
    const bool tok = MODE == M_FWD && p.y_token_major;     // [B, T, H, d, 2]: the map's rows are tokens, a row holds all heads
    constexpr bool accum = ACC && MODE != M_FWD;             // gradients of several scans over the same q, k, v add up
    unsigned char* wbox = RC + hf * 16384 + q4 * 4096;                               // this warp's 32 x 128 B block
    float dot = 0.f;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc)
      dot += bw_epi_out<DOT, accum>(tl, 2 * hf + cc, rf, orow + cc * 32, dpre[cc], valid && ok,
                                    bulk ? wbox + lane * 128 : nullptr, lane & 7);
    if (bulk) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        const int ox = tok ? h * 128 + hf * 64 : hf * 64, oy = (tok ? L.b * p.T + L.t0 : row0) + q4 * 32;
        if (accum) tma_reduce_add_2d(mout, wbox, ox, oy);      // global += tile, done by the copy engine
        else tma_store_2d_keep(mout, wbox, ox, oy);
      }
    }
    if (DOT) {
      dots[hf * TC + r] = dot;
      __syncthreads();
      if (tid < L.len && ok) {
        const float d2 = dots[tid] + dots[TC + tid];
        const size_t gi = gamma_base(p, 0, L.b, h, L.t0 + tid);
        if (MODE == M_DQ) p.dgamma[gi] = d2; else p.dA_k[gi] = d2;   // combined by k_tc_dgamma_finalize
      }
    }
  }
  if (lane == 0) tma_store_wait_read();      // the staging block is read before this CTA's shared memory goes away
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<256>(tmem);
  }
}

// forward output: grid = (chunks, H)
__global__ void __launch_bounds__(256, 2) k_tc_chunk_fwd(const __grid_constant__ ChunkMaps maps, ScanParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  chunk_job<M_FWD>(&maps.a1, &maps.b1, &maps.x2, &maps.out, &maps.a1, p, blockIdx.x, blockIdx.y, smem);
}

// the three gradients: grid = (3 * chunks, H); CTA x works on chunk x / 3, job x % 3 (dq, dv, dk), so the CTAs that
// read the same q, k, v, dy tiles are scheduled together
// ACC: dq, dk, dv are added to what the buffers hold (the K states of a layer share q, k, v)
template <bool ACC>
__global__ void __launch_bounds__(256, 2) k_tc_chunk_bwd(const __grid_constant__ BwdMaps maps, ScanParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int chunk_x = blockIdx.x / 3, job = blockIdx.x - 3 * chunk_x;
  if (job == 0) chunk_job<M_DQ, ACC>(&maps.dy, &maps.v, &maps.k, &maps.dq, &maps.q, p, chunk_x, blockIdx.y, smem);
  else if (job == 1) chunk_job<M_DV, ACC>(&maps.k, &maps.q, &maps.dy, &maps.dv, &maps.k, p, chunk_x, blockIdx.y, smem);
  else chunk_job<M_DK, ACC>(&maps.v, &maps.dy, &maps.q, &maps.dk, &maps.k, p, chunk_x, blockIdx.y, smem);
}

// ---------------------------------------------------------------------------------------------
// Reverse inter-chunk carry of the tensor-core backward (d = 64, one state), with the anchors of the decay
// gradient:  dS_c = g_c dS_c+1 + G_c  in place over the chunk axis, and for every state slot the partial sums of
// Re<dS_slot, S_slot> (S: forward state of the slot) -- one value per warp, ANCHOR_PARTS per slot, summed by the
// chunk kernel.  Scaling S_c by e^x changes the loss by x Re<dS_c, S_c>, so that inner product is the exact
// value of the suffix sum da at the first token of chunk c, known from fp32 quantities.
// grid = (S, H, 8), 256 threads: every thread owns one float4 (two complex entries) of the state.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_tc_state_scan_rev(ScanParams p, float* __restrict__ anchor_parts) {
  const int seq = blockIdx.x, h = blockIdx.y;
  const int e4 = blockIdx.z * 256 + threadIdx.x;
  constexpr int n4 = TD * TD / 2;
  const int lane = threadIdx.x & 31, part = blockIdx.z * 8 + (threadIdx.x >> 5);
  int64_t slot0;
  int nc;
  if (p.geom.cu_seqlens == nullptr) {
    nc = p.geom.nc_uniform;
    slot0 = (int64_t)seq * (nc + 1);
  } else {
    nc = p.geom.chunk_prefix[seq + 1] - p.geom.chunk_prefix[seq];
    slot0 = (int64_t)p.geom.chunk_prefix[seq] + seq;
  }
  float4* st = reinterpret_cast<float4*>(p.dstates + state_base(p, 0, h, slot0, TD)) + e4;
  const float4* fs = reinterpret_cast<const float4*>(p.states + state_base(p, 0, h, slot0, TD)) + e4;
  const float* dec = p.chunk_decay + (size_t)h * p.nslots + slot0;
  float* parts = anchor_parts + ((size_t)h * p.nslots + slot0) * ANCHOR_PARTS + part;
  const size_t ext = (((size_t)seq * p.H + h) * (size_t)(TD * TD)) / 2 + e4;
  float4 cur = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.ds_final != nullptr) cur = reinterpret_cast<const float4*>(p.ds_final)[ext];
  auto anchor = [&](int slot, const float4& a, const float4& b) {
    float d = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if (lane == 0) parts[(size_t)slot * ANCHOR_PARTS] = d;
  };
  st[(size_t)nc * n4] = cur;
  anchor(nc, cur, __ldg(fs + (size_t)nc * n4));
  constexpr int UN = 4;
  for (int c = nc - 1; c >= 0; c -= UN) {
    float4 u[UN], f[UN];
    float g[UN];
#pragma unroll
    for (int i = 0; i < UN; ++i)
      if (c - i >= 0) {
        u[i] = st[(size_t)(c - i) * n4];
        f[i] = __ldg(fs + (size_t)(c - i) * n4);
        g[i] = dec[c - i + 1];
      }
#pragma unroll
    for (int i = 0; i < UN; ++i)
      if (c - i >= 0) {
        cur.x = fmaf(g[i], cur.x, u[i].x);
        cur.y = fmaf(g[i], cur.y, u[i].y);
        cur.z = fmaf(g[i], cur.z, u[i].z);
        cur.w = fmaf(g[i], cur.w, u[i].w);
        st[(size_t)(c - i) * n4] = cur;
        anchor(c - i, cur, f[i]);
      }
  }
  if (p.ds0 != nullptr) reinterpret_cast<float4*>(p.ds0)[ext] = cur;
}

// ---------------------------------------------------------------------------------------------
// Decay gradient on the tensor-core path.  The chunk kernels leave the raw per-token values
// dA_t = Re<q_t,dq_t> - Re<k_t,dk_t>; da_u = sum_{t>=u} dA_t would accumulate their bf16-level errors as a random
// walk over the whole sequence.  Instead the suffix sum is anchored at every chunk boundary with the value the
// reverse carry kernel left there; inside a chunk the raw values are summed from the next anchor and the small
// mismatch at the chunk's first token is spread linearly over its tokens.
// grid = (chunks, H); one thread per token; chunks are independent once anchored.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_tc_dgamma_finalize(ScanParams p, const float* __restrict__ anchor_parts) {
  __shared__ float wsum[4];
  __shared__ float anc[2];
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  const int h = blockIdx.y;
  const size_t base = gamma_base(p, 0, L.b, h, L.t0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int len = L.len;
  if (warp < 2) {      // warp 0: anchor at the chunk's first token, warp 1: just after the chunk
    const float* ap = anchor_parts + ((size_t)h * p.nslots + L.slot0 + L.c + warp) * ANCHOR_PARTS;
    double a = (double)ap[lane] + (double)ap[lane + 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) anc[warp] = (float)a;
  }
  const int j = TC - 1 - tid;                         // thread tid sums the tokens j .. len-1 of the chunk
  float v = (j < len) ? p.dgamma[base + j] - p.dA_k[base + j] : 0.f;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  float off = 0.f;
  for (int w4 = 0; w4 < warp; ++w4) off += wsum[w4];
  const float suffix = v + off;                        // sum of raw values over tokens j .. len-1
  const float total = wsum[0] + wsum[1] + wsum[2] + wsum[3];
  const float lo = anc[0], hi = anc[1];
  const float mismatch = total - (lo - hi);
  if (j < len) {
    const float da = hi + suffix - mismatch * (float)(len - j) / (float)len;
    p.dgamma[base + j] = da / (p.gamma[base + j] + p.eps);
  }
}

}  // namespace tcs
}  // namespace qpam
