// Forward output of the K-state (phase-routed) scan on tensor cores, all states in ONE pass over the
// token tiles (bf16, d = 64, 2 <= K <= 4):
//
//   y_t = sum_k c_{k,t} [ sum_{s<=t} D^k_{ts} (q~_t . conj(k_s)) v_s  +  e^{A^k_t} S^k_c q~_t ]
//
// The score product Q conj(K)^T and the product with V do not depend on the state (the fused form of the
// reference, v11/model.py:657-781): only the weight applied to the scores does,
//   G[t][s] = sum_k rho_k[t] cf_k[s],   rho_k[t] = c_{k,t} scale e^{A^k_t - A^k_m} (complex),  cf_k[s] = e^{A^k_m - A^k_s},
// with the decay of every state factored around its own mid-chunk reference A^k_m (a state whose chunk decays
// by more than e^-80 is taken unfactored: per-score exp(A^k_t - A^k_s), see pam_scan_tc2.cuh).  So stage 1, the TMEM
// rewrite of the weighted scores and stage 2 run once, as in the single-state kernel (pam_scan_tc2.cuh).
// The carried-state terms use the same tensor-core path as "extra score columns": for state k the rows
// T'_k[t][j] = rho_k[t] q_t[j] are written to TMEM (into the columns the scores no longer need) and multiplied
// with the state planes e^{A^k_m} S^k_c, accumulating into the same output tile -- two states per pass.
//
//   stage 1  X = Q conj(K)^T                         Xr: cols [0,128)   Xi: cols [128,256)
//   epi 1    T = [s <= t] G (.) X  -> bf16           Tr: cols [0,64)    Ti: cols [128,192)
//   stage 2  acc = T V                               acc_r: cols [64,128)  acc_i: cols [192,256)
//   pass p   T'_k -> cols [32 s, 32 s + 32) of the Tr / Ti ranges (s = slot of state k in the pass)
//            acc += T'_k (e^{A^k_m} S^k)^T
//   epi 2    y = acc
#pragma once
#include "pam_scan_tc2.cuh"

namespace qpam {
namespace tcs {

constexpr size_t CHUNKK_SMEM = 1024 + 3 * 32768 + 9216;

__global__ void __launch_bounds__(256, 2) k_tc_chunk_fwdK(const __grid_constant__ ChunkMaps maps, ScanParams p) {
  using namespace umma;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* RA = smem;                  // Q: real plane, imaginary plane  (2 x [128 rows][128 B])
  unsigned char* RB = RA + 32768;            // K planes; after stage 1: two slots of carried-state planes (2 x 16 KB)
  unsigned char* RC = RB + 32768;            // V planes
  float* Acum = reinterpret_cast<float*>(RC + 32768);        // [KMAX][128]  cumulative log-decay per state
  float* cfac = Acum + KMAX * TC;                            // [KMAX][128]  e^{A_m - A_s}
  float2* rho = reinterpret_cast<float2*>(cfac + KMAX * TC); // [KMAX][128]  c_k scale e^{A_t - A_m}
  uint64_t* bars = reinterpret_cast<uint64_t*>(rho + KMAX * TC);  // [0] tma [1] stage 1 [2] stage 2 [3],[4] state passes
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  int* failed = reinterpret_cast<int*>(tmem_slot + 1);      // error word as found at the start of this CTA
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ChunkLoc L = locate_chunk(p.geom, blockIdx.x);
  if (!L.valid) return;
  if (tid == 160) *failed = device_error_now();
  const int h = blockIdx.y;
  const int K = p.K;
  const bool has_state = (L.c > 0) || (p.s0 != nullptr);
  const int row0 = (L.b * p.H + h) * p.T + L.t0;
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
    mbar_arrive_expect_tx(&bars[0], 6 * 16384);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_2d(RA + kb * 16384, &maps.a1, &bars[0], kb * 64, row0);
      tma_load_2d(RB + kb * 16384, &maps.b1, &bars[0], kb * 64, row0);
      tma_load_2d(RC + kb * 16384, &maps.x2, &bars[0], kb * 64, row0);
    }
  }
  __syncwarp();
  // the read-out weights of this thread's (state, token) entries: requested here, used after the first barrier
  float2 craw[2] = {make_float2(1.f, 0.f), make_float2(1.f, 0.f)};
  if (p.coef != nullptr) {
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int e = tid + 256 * m, k = e / TC, t = e - k * TC;
      if (e < K * TC && t < L.len) craw[m] = __ldg(reinterpret_cast<const float2*>(p.coef + gamma_base(p, k, L.b, h, L.t0 + t) * 2));
    }
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  if (warp >= 1 && warp <= K)
    warp_cumsum128(Acum + (warp - 1) * TC, p.gamma + gamma_base(p, warp - 1, L.b, h, L.t0), L.len, p.eps, lane);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (*failed != 0) {       // an earlier launch gave up on a wait: outputs stay untouched (see pam_scan_tc2.cuh)
    mbar_wait(&bars[0], 0, 239);
    __syncthreads();
    if (warp == 0) tmem_dealloc<256>(tmem);
    return;
  }
  // a state whose chunk decays by more than e^-80 leaves the factored form (its exponents would overflow): its
  // scores get exp(A_t - A_s) one by one and its carried-state rows their own e^{A_t}
  uint32_t strong_mask = 0;
#pragma unroll
  for (int k = 0; k < KMAX; ++k)
    if (k < K && Acum[k * TC + TC - 1] < STRONG_DECAY) strong_mask |= 1u << k;
#pragma unroll
  for (int m = 0; m < 2; ++m) {          // KMAX * TC = 512 entries, two per thread
    const int e = tid + 256 * m;
    if (e < K * TC) {
      const int k = e / TC;
      const bool strong = (strong_mask >> k) & 1u;
      const float a = Acum[e], a_mid = Acum[k * TC + TC / 2 - 1];
      cfac[e] = strong ? 1.f : __expf(a_mid - a);
      const float2 c = craw[m];
      const float rf = p.q_scale * (strong ? 1.f : __expf(a - a_mid));
      rho[e] = make_float2(c.x * rf, c.y * rf);
    }
  }
  bool ok = mbar_wait(&bars[0], 0, 231);
  {
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
  const uint32_t a_r = smem_u32(RA), a_i = a_r + 16384, b_r = smem_u32(RB), b_i = b_r + 16384;
  const uint32_t x_r = smem_u32(RC), x_i = x_r + 16384;
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t id = idesc_bf16(128, 128, false, false);
    constexpr uint32_t idn = idesc_bf16_nega(128, 128, false, false);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(tmem, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(tmem, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), id, true);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(tmem + 128, smem_desc_sw128(a_i + kk * 32, 16, 1024), smem_desc_sw128(b_r + kk * 32, 16, 1024), id, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      mma_bf16(tmem + 128, smem_desc_sw128(a_r + kk * 32, 16, 1024), smem_desc_sw128(b_i + kk * 32, 16, 1024), idn, true);
    mma_commit(&bars[1]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[1], 0, 232) && ok;
  tc_fence_after();
  const int q4 = warp & 3, hf = warp >> 2;
  const int r = q4 * 32 + lane;                               // this thread's row (TMEM lane)
  const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
  float2 rk[KMAX];                                            // rho_k of this row
#pragma unroll
  for (int k = 0; k < KMAX; ++k) rk[k] = (k < K) ? rho[k * TC + r] : make_float2(0.f, 0.f);

  // carried-state planes of state k (times its chunk constant e^{A^k_m}) into slot s of the K-plane region
  auto stage_state = [&](int k, int s) {
    const float cst = ((strong_mask >> k) & 1u) ? 1.f : __expf(Acum[k * TC + TC / 2 - 1]);
    const float4* sg = reinterpret_cast<const float4*>(p.states + state_base(p, k, h, L.slot0 + L.c, TD));
    unsigned char* dstp = RB + s * 16384;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int idx = tid + 256 * it;          // (i, c16): state[i][4*c16 .. +3]
      const float4 s01 = __ldg(sg + idx * 2), s23 = __ldg(sg + idx * 2 + 1);
      const int i = idx >> 4, c16 = idx & 15;
      const uint32_t off = sw128(i, c16 >> 1) + (c16 & 1) * 8;
      *reinterpret_cast<uint2*>(dstp + off) = make_uint2(pack_bf162(cst * s01.x, cst * s01.z), pack_bf162(cst * s23.x, cst * s23.z));
      *reinterpret_cast<uint2*>(dstp + 8192 + off) = make_uint2(pack_bf162(cst * s01.y, cst * s01.w), pack_bf162(cst * s23.y, cst * s23.w));
    }
  };

  {
    // epilogue 1: weighted, masked scores of columns [64 hf, 64 hf + 64) as packed bf16 pairs
    uint32_t tr[32], ti[32];
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c0 = hf * 64 + cc * 16;
      const bool dead = c0 > q4 * 32 + 31;   // warp-uniform: the whole block lies above the diagonal
      if (dead) {
#pragma unroll
        for (int j = 0; j < 8; ++j) tr[cc * 8 + j] = ti[cc * 8 + j] = 0u;
      } else {
        float xr[16], xi[16];
        tmem_ld16(tlane + c0, xr);
        tmem_ld16(tlane + 128 + c0, xi);
        // (the two loops differ only in how a state's column factor is formed: the common case -- no state of this
        // chunk decays strongly, CTA-uniform -- keeps the exponentials out of the per-score code)
        if (strong_mask == 0u) {
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            float wr[2], wi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int c = c0 + j + e;
              float gr = 0.f, gi = 0.f;
#pragma unroll
              for (int k = 0; k < KMAX; ++k)
                if (k < K) {
                  const float cf = cfac[k * TC + c];
                  gr = fmaf(rk[k].x, cf, gr);
                  gi = fmaf(rk[k].y, cf, gi);
                }
              if (c > r) gr = gi = 0.f;
              wr[e] = xr[j + e] * gr - xi[j + e] * gi;
              wi[e] = xr[j + e] * gi + xi[j + e] * gr;
            }
            tr[cc * 8 + (j >> 1)] = pack_bf162(wr[0], wr[1]);
            ti[cc * 8 + (j >> 1)] = pack_bf162(wi[0], wi[1]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            float wr[2], wi[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int c = c0 + j + e;
              float gr = 0.f, gi = 0.f;
#pragma unroll
              for (int k = 0; k < KMAX; ++k)
                if (k < K) {
                  const float cf = ((strong_mask >> k) & 1u) ? __expf(fminf(0.f, Acum[k * TC + r] - Acum[k * TC + c]))
                                                             : cfac[k * TC + c];
                  gr = fmaf(rk[k].x, cf, gr);
                  gi = fmaf(rk[k].y, cf, gi);
                }
              if (c > r) gr = gi = 0.f;
              wr[e] = xr[j + e] * gr - xi[j + e] * gi;
              wi[e] = xr[j + e] * gi + xi[j + e] * gr;
            }
            tr[cc * 8 + (j >> 1)] = pack_bf162(wr[0], wr[1]);
            ti[cc * 8 + (j >> 1)] = pack_bf162(wi[0], wi[1]);
          }
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
    if (has_state) {          // the K planes are no longer needed: states 0 and 1 take their place
      stage_state(0, 0);
      if (K > 1) stage_state(1, 1);
    }
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  const uint32_t Tr = tmem, Ti = tmem + 128, Or = tmem + 64, Oi = tmem + 192;
  if (warp == 0 && elect_one()) {
    tc_fence_after();
    constexpr uint32_t id = idesc_bf16(128, 64, false, true);        // A: TMEM, B: MN-major plane
    constexpr uint32_t idn = idesc_bf16_nega(128, 64, false, true);
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
    mma_commit(&bars[2]);
  }
  __syncwarp();
  ok = mbar_wait(&bars[2], 0, 233) && ok;
  tc_fence_after();
  if (has_state) {
    for (int pass = 0; pass * 2 < K; ++pass) {
      const int k_mine = pass * 2 + hf;                 // the state whose rows this half of the CTA writes
      if (pass > 0) {                                   // the previous pass has finished with both slots
        stage_state(pass * 2, 0);
        if (pass * 2 + 1 < K) stage_state(pass * 2 + 1, 1);
      }
      if (k_mine < K) {
        // T'[r][j] = rho_k[r] q_r[j], j = 0..63, as packed bf16 pairs: 32 columns of reals, 32 of imaginaries
        float2 rr = rk[0];                           // (a select chain keeps rk in registers)
#pragma unroll
        for (int k = 1; k < KMAX; ++k)
          if (k_mine == k) rr = rk[k];
        if ((strong_mask >> k_mine) & 1u) {          // unfactored state: the row's own decay goes here
          const float ea = __expf(Acum[k_mine * TC + r]);
          rr.x *= ea;
          rr.y *= ea;
        }
        uint32_t wr[32], wi[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 qr = *reinterpret_cast<const uint4*>(RA + sw128(r, c));
          const uint4 qi = *reinterpret_cast<const uint4*>(RA + 16384 + sw128(r, c));
          const uint32_t qrw[4] = {qr.x, qr.y, qr.z, qr.w}, qiw[4] = {qi.x, qi.y, qi.z, qi.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a = unpack_bf162(qrw[e]), b = unpack_bf162(qiw[e]);   // two consecutive channels
            wr[c * 4 + e] = pack_bf162(a.x * rr.x - b.x * rr.y, a.y * rr.x - b.y * rr.y);
            wi[c * 4 + e] = pack_bf162(a.x * rr.y + b.x * rr.x, a.y * rr.y + b.y * rr.x);
          }
        }
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) { lo[j] = wr[j]; hi[j] = wr[16 + j]; }
        tmem_st16(tlane + hf * 32, lo);
        tmem_st16(tlane + hf * 32 + 16, hi);
#pragma unroll
        for (int j = 0; j < 16; ++j) { lo[j] = wi[j]; hi[j] = wi[16 + j]; }
        tmem_st16(tlane + 128 + hf * 32, lo);
        tmem_st16(tlane + 128 + hf * 32 + 16, hi);
        tmem_st_wait();
      }
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      if (warp == 0 && elect_one()) {
        tc_fence_after();
        constexpr uint32_t k3 = idesc_bf16(128, 64, false, false), k3n = idesc_bf16_nega(128, 64, false, false);
        for (int s = 0; s < 2 && pass * 2 + s < K; ++s) {
          const uint32_t s_r = b_r + s * 16384, s_i = s_r + 8192;   // [64 rows i][64 j] planes of this slot
          const uint32_t tr_ = Tr + s * 32, ti_ = Ti + s * 32;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t sr = smem_desc_sw128(s_r + kk * 32, 16, 1024), si = smem_desc_sw128(s_i + kk * 32, 16, 1024);
            mma_bf16_ts(Or, tr_ + kk * 8, sr, k3, true);    // + T'r Sr^T
            mma_bf16_ts(Or, ti_ + kk * 8, si, k3n, true);   // - T'i Si^T
            mma_bf16_ts(Oi, tr_ + kk * 8, si, k3, true);    // + T'r Si^T
            mma_bf16_ts(Oi, ti_ + kk * 8, sr, k3, true);    // + T'i Sr^T
          }
        }
        mma_commit(&bars[3 + pass]);
      }
      __syncwarp();
      ok = mbar_wait(&bars[3 + pass], 0, 234 + pass) && ok;
      tc_fence_after();
    }
  }
  {
    const size_t rbase = (p.y_token_major ? (((size_t)L.b * p.T + L.t0 + r) * p.H + h) * (size_t)(TD * 2)
                                          : token_base(p, L.b, h, L.t0 + r, TD)) + hf * 64;   // channels [32 hf, 32 hf + 32)
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.y) + rbase;
    // a full chunk leaves through the X2 region (no MMA reads it any more): 32 rows x 128 bytes per warp, one TMA
    // store each; a ragged chunk stores per lane
    const bool bulk = ok && L.len == TC;                                             // CTA-uniform
    unsigned char* wrow = RC + hf * 16384 + (warp & 3) * 4096 + lane * 128;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      float vr[16], vi[16];
      tmem_ld16(tlane + 64 + hf * 32 + cc * 16, vr);
      tmem_ld16(tlane + 192 + hf * 32 + cc * 16, vi);
      if (ok && r < L.len) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4 pk = make_uint4(pack_bf162(vr[4 * g], vi[4 * g]), pack_bf162(vr[4 * g + 1], vi[4 * g + 1]),
                                      pack_bf162(vr[4 * g + 2], vi[4 * g + 2]), pack_bf162(vr[4 * g + 3], vi[4 * g + 3]));
          if (bulk) *reinterpret_cast<uint4*>(wrow + (((4 * cc + g) ^ (lane & 7)) << 4)) = pk;
          else *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = pk;
        }
      }
    }
    if (bulk) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0)
        tma_store_2d_keep(&maps.out, RC + hf * 16384 + (warp & 3) * 4096, p.y_token_major ? h * 128 + hf * 64 : hf * 64,
                          (p.y_token_major ? L.b * p.T + L.t0 : (L.b * p.H + h) * p.T + L.t0) + (warp & 3) * 32);
      if (lane == 0) tma_store_wait_read();
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
