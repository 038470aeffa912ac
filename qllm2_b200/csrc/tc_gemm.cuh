// Warp-specialised bf16 GEMM on the 5th-generation tensor cores (tcgen05) for the tied-head
// cross-entropy: D[128 x BN] tiles accumulate in TMEM (fp32), operands arrive through a TMA ->
// shared-memory ring, and the epilogue reads TMEM with tcgen05.ld while the next tile's MMAs run
// into the second accumulator buffer.
//
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one elected lane)
//   warps 2..9  epilogue; warp w owns TMEM lanes 32*(w%4) .. +31 (= tile rows); warps 2..5 take the lower
//               half of a tile's columns, warps 6..9 the upper half, so every scheduler holds two epilogue
//               warps and one covers the other's tcgen05.ld latency
//
// A CTA owns one 128-row tile and walks the N tiles [n_begin, n_end) over the K blocks
// [kb_begin, kb_end).  Operands may be K-major (rows of 64 K elements) or MN-major (rows of 64
// M/N elements); both are 128-byte swizzled TMA boxes, see umma.cuh.
#pragma once
#include "common.cuh"
#include "umma.cuh"

namespace qpam {
namespace tc {

constexpr int BM = 128, BK = 64;
constexpr int EPI_WARPS = 8;
constexpr int NTHREADS = 64 + 32 * EPI_WARPS;

enum Epi { EPI_STATS = 0, EPI_PROBS = 1, EPI_STORE = 2, EPI_STORE_BF16 = 3 };   // 3: D as bf16 through tmC (boxes of 64 x 32)

constexpr float LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct GemmParams {
  // tile walk
  int32_t n_tiles;          // N tiles in total
  int32_t tiles_per_cta;    // N tiles walked by one CTA (blockIdx.x selects the range)
  int32_t kb_total;         // K blocks in total
  int32_t kb_per_split;     // K blocks per blockIdx.z
  int32_t swap_xy;          // 1: blockIdx.x walks the M tiles (neighbouring CTAs share the B tile in L2)
  int64_t M, N;             // logical extents (rows / columns of D)
  // EPI_STATS
  const int64_t* targets;
  int64_t v_offset, ignore_index;
  float *pm, *ps, *pt, *pbest;
  int32_t* pidx;
  int64_t stats_ld;         // = rows of the whole problem (partials are [split][rows])
  int64_t row_base;         // global row of tile row 0 of blockIdx.y == 0
  // EPI_PROBS
  __nv_bfloat16* pbuf;
  int64_t ldp;
  const float* lse;
  const float* mask;
  const float* grad_scale;
  const float* denom;
  // EPI_STORE
  float* c;                 // [splits][M][ldc] fp32
  int64_t ldc;
  int32_t beta;             // 1: accumulate into c
};

// MT = row tiles of one CTA.  MT == 1: one 128 x BN tile at a time, two accumulator buffers, so the epilogue of a
// tile overlaps the MMAs of the next (short-K products with heavy epilogues).  MT == 2: two 128-row tiles share
// every B block (a 256 x BN tile per CTA: a third less operand traffic from L2 per MAC, half the barrier
// hand-offs), both accumulators live at once and the epilogue runs at the end (long-K products).
// PAIR: two CTAs of a cluster (neighbouring SMs) work on one 256-row tile with cta_group::2 MMAs: each CTA loads
// its own 128 rows of A and only HALF of the B tile, so the operand traffic per MAC drops by a third while both
// accumulator buffers stay (short-K products with heavy epilogues).
template <int BN, int MT = 1, bool PAIR = false>
struct Cfg {
  static constexpr int A_BYTES = MT * BM * BK * 2;           // 16 KB per row tile
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;   // this CTA's share of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : (MT == 2) ? 3 : (BN == 256) ? 4 : 6;
  static constexpr int NBUF = (MT == 2) ? 1 : 2;             // accumulator sets in flight
  static constexpr int TMEM_COLS = 2 * BN;                   // two accumulator buffers, or two row tiles
  static constexpr int EPI_STAGE_BYTES = 4096;               // per epilogue warp: 32 rows x 64 bf16, swizzled
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  // EPI_PROBS and EPI_STORE launches add the staging blocks (EPI_STATS keeps the bytes for L1)
  static constexpr size_t SMEM_BYTES_STAGED = SMEM_BYTES + (size_t)EPI_WARPS * EPI_STAGE_BYTES;
};

template <int BN, int EPI, bool A_MN, bool B_MN, int MT = 1, bool PAIR = false>
__global__ void __launch_bounds__(NTHREADS, 1)
k_tc_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
          const __grid_constant__ CUtensorMap tmC, const GemmParams p) {   // tmC: EPI_PROBS output, boxes of 64 x 32
  using namespace umma;
  using C = Cfg<BN, MT, PAIR>;
  static_assert(MT == 1 || EPI == EPI_STORE || EPI == EPI_STORE_BF16, "two row tiles per CTA: plain stores only");
  static_assert(!PAIR || (MT == 1 && !A_MN && !B_MN), "CTA pairs: K-major operands, one row tile per CTA");
  // PAIR: launched as clusters of two CTAs along the row-tile axis; tmB's box holds BN / 2 rows
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = crank == 0u;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // [operand ring][staging blocks of the epilogue warps (1024-byte aligned: TMA stores read them)][barriers]
  unsigned char* stg_base = smem + (size_t)C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg_base + (EPI == EPI_STATS ? 0 : (size_t)EPI_WARPS * C::EPI_STAGE_BYTES));
  uint64_t* full = bars;                      // [STAGES]
  uint64_t* empty = bars + C::STAGES;         // [STAGES]
  uint64_t* tfull = bars + 2 * C::STAGES;     // [2]
  uint64_t* tempty = bars + 2 * C::STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = p.swap_xy ? blockIdx.x : blockIdx.y;
  const int n_begin = (p.swap_xy ? blockIdx.y : blockIdx.x) * p.tiles_per_cta;
  const int n_end = min(p.n_tiles, n_begin + p.tiles_per_cta);
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kb_end = min(p.kb_total, kb_begin + p.kb_per_split);
  uint32_t* err_slot = tmem_slot + 1;

  if (threadIdx.x == 0) {
    // one read of the device error word for the whole CTA: every warp must take the same side of has_work
    // (the epilogue warps meet at a named barrier), whatever another CTA writes meanwhile
    *err_slot = (uint32_t) * reinterpret_cast<volatile int*>(&g_device_error);
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], (PAIR ? 2 : 1) * EPI_WARPS);  // one arrival per epilogue warp (of both CTAs of a pair)
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair<C::TMEM_COLS>(tmem_slot);
    else tmem_alloc<C::TMEM_COLS>(tmem_slot);
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // after a failed handshake anywhere on the device, later CTAs do not start new work
  const bool has_work = (n_begin < n_end) && (kb_begin < kb_end) && (*err_slot == 0);

  if (has_work) {
    if (warp == 0) {
      // ------------------------------------------------------------- TMA producer
      if (elect_one()) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int n = n_begin; n < n_end && ok; ++n) {
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1, 101)) { ok = false; break; }
            unsigned char* sa = smem + (size_t)stage * C::STAGE_BYTES;
            unsigned char* sb = sa + C::A_BYTES;
            if constexpr (PAIR) {
              // the leader's barrier counts the bytes of both CTAs; each CTA loads its rows of A and its half of B
              if (leader) mbar_arrive_expect_tx(&full[stage], 2 * C::STAGE_BYTES);
              const uint32_t fb = cluster_map(&full[stage], 0);
              tma_load_2d_pair(sa, &tmA, fb, kb * BK, m_tile * BM);
              tma_load_2d_pair(sb, &tmB, fb, kb * BK, n * BN + (int)crank * (BN / 2));
              if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
              continue;
            }
            mbar_arrive_expect_tx(&full[stage], C::STAGE_BYTES);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              unsigned char* sam = sa + mt * (BM * BK * 2);
              const int m0 = (m_tile * MT + mt) * BM;       // rows past M arrive as zeros
              if (!A_MN) {
                tma_load_2d(sam, &tmA, &full[stage], kb * BK, m0);
              } else {
#pragma unroll
                for (int j = 0; j < BM / 64; ++j)
                  tma_load_2d(sam + j * 8192, &tmA, &full[stage], m0 + j * 64, kb * BK);
              }
            }
            if (!B_MN) {
              tma_load_2d(sb, &tmB, &full[stage], kb * BK, n * BN);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * 8192, &tmB, &full[stage], n * BN + j * 64, kb * BK);
            }
            if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------- MMA issuer (PAIR: the leader's, for both CTAs)
      if (leader && elect_one()) {
        constexpr uint32_t idesc = idesc_bf16(PAIR ? 2 * BM : BM, BN, A_MN, B_MN);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int it = 0;
        for (int n = n_begin; n < n_end && ok; ++n, ++it) {
          const int buf = it % C::NBUF;
          const uint32_t bphase = (it / C::NBUF) & 1;
          if (!mbar_wait(&tempty[buf], bphase ^ 1, 102)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (!mbar_wait(&full[stage], phase, 103)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + (size_t)stage * C::STAGE_BYTES);
            const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              const uint64_t bd = B_MN ? smem_desc_sw128(sb + kk * 2048, 8192, 1024) : smem_desc_sw128(sb + kk * 32, 16, 1024);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const uint32_t sam = sa + mt * (BM * BK * 2);
                const uint64_t ad = A_MN ? smem_desc_sw128(sam + kk * 2048, 8192, 1024) : smem_desc_sw128(sam + kk * 32, 16, 1024);
                if (PAIR) mma_bf16_pair(d_tmem + mt * BN, ad, bd, idesc, (kb > kb_begin) || (kk > 0));
                else mma_bf16(d_tmem + mt * BN, ad, bd, idesc, (kb > kb_begin) || (kk > 0));
              }
            }
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if (PAIR) mma_commit_pair(&empty[stage]);
            else mma_commit(&empty[stage]);
            if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) {
            if (PAIR) mma_commit_pair(&tfull[buf]);
            else mma_commit(&tfull[buf]);
          }
        }
      }
    } else {
      // ------------------------------------------------------------- epilogue (8 warps)
      const int quarter = warp & 3;
      const int half = (warp - 2) >> 2;                        // which half of the tile's columns
      constexpr int CC_HALF = BN / 64;                         // 32-column groups per half
      const int r_tile = quarter * 32 + lane;                  // row within the tile == TMEM lane
      const int64_t row = (int64_t)m_tile * BM + r_tile;       // row of D
      const bool row_ok = row < p.M;
      const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
      // EPI_STATS running state
      float m_run = -INFINITY, s_run = 0.f, best = -INFINITY, tz = 0.f;
      int bidx = 0x7fffffff;
      int64_t tcol = -1;
      float lse_r = 0.f, sc_r = 0.f;
      if (EPI == EPI_STATS && row_ok && p.targets != nullptr) {
        const int64_t t = p.targets[p.row_base + row];
        if (t != p.ignore_index) tcol = t - p.v_offset;
      }
      if (EPI == EPI_PROBS && row_ok) {
        const int64_t grow = p.row_base + row;
        const int64_t t = p.targets[grow];
        const bool valid = t != p.ignore_index;
        tcol = valid ? t - p.v_offset : -1;
        lse_r = p.lse[grow];
        sc_r = valid ? (p.grad_scale[0] / p.denom[0]) * (p.mask ? p.mask[grow] : 1.f) : 0.f;
      }
      // exp(v - lse) * sc = 2^(v log2e - off) with off = lse log2e - log2(sc): two instructions per element.
      // Rows whose scale is not positive (ignored rows, a negative upstream gradient) multiply instead.
      const bool sc_pos = sc_r > 0.f;
      const float off_r = sc_pos ? fmaf(lse_r, LOG2E, -__log2f(sc_r)) : lse_r * LOG2E;
      const float mul_r = sc_pos ? 1.f : sc_r;
      bool ok = true;
      int it = 0;
      for (int n = n_begin; n < n_end && ok; ++n, ++it) {
        const int buf = it % C::NBUF;
        const uint32_t bphase = (it / C::NBUF) & 1;
        if (!mbar_wait(&tfull[buf], bphase, 104)) { ok = false; break; }
        tc_fence_after();
        const int64_t col0 = (int64_t)n * BN;
        if constexpr (EPI == EPI_PROBS || EPI == EPI_STORE_BF16) {
          // Probability tiles leave through a per-warp staging block so that global stores are whole 128-byte
          // rows: a lane owns a tile row in TMEM, but 8 lanes share a row when storing.  16-byte pieces are
          // placed at (piece ^ (row & 7)) within their 128-byte row: both phases are free of bank conflicts.
          unsigned char* stg = stg_base + (size_t)(warp - 2) * C::EPI_STAGE_BYTES;
          constexpr int G_HALF = BN / 128;                                   // groups of 64 columns per half tile
#pragma unroll 1
          for (int gm = 0; gm < MT * G_HALF; ++gm) {
            const int mt = gm / G_HALF, g = half * G_HALF + gm % G_HALF;
            const int64_t row0 = ((int64_t)m_tile * MT + mt) * BM + quarter * 32;
            const int64_t cb = col0 + g * 64;
            if (cb >= p.N) continue;
            // the block may still be read by the store of the previous group
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              float v[32];
              tmem_ld32(tmem_base + lane_addr + buf * BN + mt * BN + g * 64 + hh * 32, v);
              const int64_t dt = EPI == EPI_PROBS ? tcol - (cb + hh * 32) : -1;
              if constexpr (EPI == EPI_PROBS) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = ex2_fast(fmaf(v[j], LOG2E, -off_r));
                if (!sc_pos) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] *= mul_r;
                }
              }
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                uint4 pk;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(v[g8 * 8 + 2 * j], v[g8 * 8 + 2 * j + 1]);
                *reinterpret_cast<uint4*>(stg + lane * 128 + (((hh * 4 + g8) ^ (lane & 7)) << 4)) = pk;
              }
              if (dt >= 0 && dt < 32) {
                // the target column lies in this group: (p - 1) * scale there.  The thread patches the one value it
                // has just staged (its own row), which keeps the 32 values above in registers.
                __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(
                    stg + lane * 128 + (((hh * 4 + ((int)dt >> 3)) ^ (lane & 7)) << 4)) + ((int)dt & 7);
                *e = __float2bfloat16_rn(__bfloat162float(*e) - sc_r);
              }
            }
            // one TMA store per 32 x 64 block: rows past M and columns past N are clipped by the tensor map
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && row0 < p.M) tma_store_2d(&tmC, stg, (int32_t)cb, (int32_t)row0);
          }
        } else {
#pragma unroll 1
          for (int ccm = half * CC_HALF; ccm < half * CC_HALF + MT * CC_HALF; ++ccm) {
            const int mt = (ccm - half * CC_HALF) / CC_HALF;          // row tile of this CTA (EPI_STORE only)
            const int cc = ccm - mt * CC_HALF;
            float v[32];
            tmem_ld32(tmem_base + lane_addr + buf * BN + mt * BN + cc * 32, v);
            const int64_t cbase = col0 + cc * 32;
            if (EPI == EPI_STATS) {
              if (cbase >= p.N) continue;
              const int nvalid = (int)min((int64_t)32, p.N - cbase);
              if (nvalid < 32) {             // the ragged last group: columns past N can neither win nor add
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j >= nvalid) v[j] = -INFINITY;
              }
              float cmax = v[0];
#pragma unroll
              for (int j = 1; j < 32; ++j) cmax = fmaxf(cmax, v[j]);
              if (cmax > best) {             // rarer and rarer as the walk goes on: only then is the column looked up
                best = cmax;
                int ci = 31;
#pragma unroll
                for (int j = 30; j >= 0; --j)
                  if (v[j] == cmax) ci = j;  // lowest column among equals
                bidx = (int)cbase + ci;
              }
              const float m_new = fmaxf(m_run, cmax);
              const float ml2 = m_new * LOG2E;
              float se = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) se += ex2_fast(fmaf(v[j], LOG2E, -ml2));
              s_run = s_run * ex2_fast((m_run - m_new) * LOG2E) + se;
              m_run = m_new;
              if (tcol >= cbase && tcol < cbase + nvalid) {   // a target past N belongs to another vocabulary shard
                const int tj = (int)(tcol - cbase);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j == tj) tz = v[j];
              }
            } else {  // EPI_STORE: through the staging block, whole 128-byte rows per 8 lanes
              if (cbase >= p.N) continue;
              unsigned char* stg = stg_base + (size_t)(warp - 2) * C::EPI_STAGE_BYTES;
              const int64_t row0 = ((int64_t)m_tile * MT + mt) * BM + quarter * 32;
#pragma unroll
              for (int g4 = 0; g4 < 8; ++g4)
                *reinterpret_cast<float4*>(stg + lane * 128 + ((g4 ^ (lane & 7)) << 4)) =
                    make_float4(v[g4 * 4], v[g4 * 4 + 1], v[g4 * 4 + 2], v[g4 * 4 + 3]);
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = 4 * i + (lane >> 3), c = lane & 7;
                float4 o = *reinterpret_cast<const float4*>(stg + r * 128 + ((c ^ (r & 7)) << 4));
                if (row0 + r < p.M && cbase + c * 4 + 4 <= p.N) {
                  float* dst = p.c + ((size_t)blockIdx.z * p.M + row0 + r) * p.ldc + cbase + c * 4;
                  if (p.beta) {
                    const float4 c0 = *reinterpret_cast<const float4*>(dst);
                    o.x += c0.x; o.y += c0.y; o.z += c0.z; o.w += c0.w;
                  }
                  *reinterpret_cast<float4*>(dst) = o;
                }
              }
              __syncwarp();
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR && !leader) mbar_arrive_cluster(cluster_map(&tempty[buf], 0));   // the leader issues the MMAs
          else mbar_arrive(&tempty[buf]);
        }
      }
      if (EPI == EPI_PROBS || EPI == EPI_STORE_BF16) {
        if (lane == 0) tma_store_wait_all();     // the staging block and the stores outlive no one
        __syncwarp();
      }
      if (EPI == EPI_STATS) {
        // The two warps of a row fold their running statistics through shared memory.  The ring's first
        // stage is free by now: a warp that saw the last accumulator complete has seen every load consumed.
        float* mg = reinterpret_cast<float*>(smem) + r_tile * 5;
        if (half == 1 && ok) {
          mg[0] = m_run; mg[1] = s_run; mg[2] = tz; mg[3] = best; mg[4] = __int_as_float(bidx);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
        if (half == 0 && ok) {
          const float m1 = mg[0], s1 = mg[1], b1 = mg[3];
          const int i1 = __float_as_int(mg[4]);
          const float m_new = fmaxf(m_run, m1);
          if (m_new > -INFINITY) s_run = s_run * __expf(m_run - m_new) + s1 * __expf(m1 - m_new);
          m_run = m_new;
          tz += mg[2];
          if (b1 > best || (b1 == best && i1 < bidx)) { best = b1; bidx = i1; }
        }
      }
      if (EPI == EPI_STATS && ok && row_ok && half == 0) {
        const size_t o = (size_t)(p.swap_xy ? blockIdx.y : blockIdx.x) * p.stats_ld + p.row_base + row;   // [split][row]
        p.pm[o] = m_run;
        p.ps[o] = s_run;
        p.pt[o] = tz;
        p.pbest[o] = best;
        p.pidx[o] = bidx;
      }
    }
  }
  // ------------------------------------------------------------- teardown
  tc_fence_before();
  if (PAIR) cluster_sync_all();   // no signal of the peer is still on its way to this CTA's barriers
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair<C::TMEM_COLS>(tmem_base);
    else tmem_dealloc<C::TMEM_COLS>(tmem_base);
  }
}

}  // namespace tc
}  // namespace qpam
