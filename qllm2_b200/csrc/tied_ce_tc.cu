// Tensor-core path of the fused tied-head cross-entropy (bf16 inputs): TMA descriptors, tile
// plans and launches of k_tc_gemm.
#include "tc_gemm.cuh"
#include "tma_host.cuh"
#include "tied_ce_tc.cuh"

namespace qpam {

template <typename K>
static int opt_in_smem(K kern, size_t bytes) {
  QPAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return QPAM_OK;
}

// Launch a kernel of CTA pairs: clusters of two CTAs along x (pair_axis 0) or y (pair_axis 1).
template <typename... KArgs, typename... Args>
static cudaError_t launch_pairs(void (*kern)(KArgs...), dim3 grid, int pair_axis, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(tc::NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = pair_axis == 0 ? 2 : 1;
  at[0].val.clusterDim.y = pair_axis == 1 ? 2 : 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// ------------------------------------------------------------------ plan
CETcPlan ce_tc_plan(const qpam_ce_args* a) {
  CETcPlan pl{};
  pl.enabled = a->io_dtype == QPAM_BF16 && (a->F % 8) == 0 && a->N > 0;
  pl.n_tiles = (int32_t)((a->V + 255) / 256);
  const int64_t row_tiles = (a->N + tc::BM - 1) / tc::BM;
  // vocabulary splits: fill the SMs in whole waves (one CTA per SM: the ring takes ~193 KB)
  const int sms = sm_count();
  int best = 1;
  double best_eff = -1.0;
  const int max_split = pl.n_tiles < 128 ? pl.n_tiles : 128;
  for (int s = 1; s <= max_split; ++s) {
    const int tps = (pl.n_tiles + s - 1) / s;
    const int real = (pl.n_tiles + tps - 1) / tps;
    if (real != s) continue;
    const double ctas = (double)row_tiles * s;
    const double waves = (ctas + sms - 1) / sms;
    // last factor: a CTA pays its prologue and one epilogue that no MMA overlaps (~0.7 of a tile's time)
    const double eff = ctas / ((double)(int64_t)waves * sms) * ((double)pl.n_tiles / ((double)tps * s)) *
                       (tps / (tps + 0.7));
    if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
  }
  pl.nsplit = best;
  pl.tiles_per_split = (pl.n_tiles + best - 1) / best;
  int64_t rows = ((a->N + tc::BM - 1) / tc::BM) * tc::BM;
  if (rows > 8192) rows = 8192;
  if (rows < tc::BM) rows = tc::BM;
  pl.chunk_rows = rows;
  const int64_t f_tiles = (a->F + 255) / 256;
  // split-K of dH: one CTA per SM, so the cost is (waves of CTAs) x (K blocks per split)
  const int64_t kb_total = (a->V + tc::BK - 1) / tc::BK;
  int64_t ks = 1, ks_cost = -1;
  for (int64_t s = 1; s <= 8 && s <= kb_total; ++s) {
    const int64_t ctas = f_tiles * ((rows + 2 * tc::BM - 1) / (2 * tc::BM)) * s;     // CTAs of two row tiles
    const int64_t cost = ((ctas + sms - 1) / sms) * ((kb_total + s - 1) / s + 8);   // + 8: prologue and epilogue of a CTA
    if (ks_cost < 0 || cost < ks_cost) { ks_cost = cost; ks = s; }
  }
  pl.ksplit = (int32_t)ks;
  // every row chunk (up to 4) sums its dW into a buffer of its own: adding into one buffer made the epilogue
  // of the later chunks read what it writes (+50 % on that launch); the final bf16 pass adds the buffers
  const int64_t n_chunks = (a->N + rows - 1) / rows;
  // (one row chunk needs none: its dW leaves the accumulators as bf16)
  pl.dw_bufs = (int32_t)(n_chunks <= 1 ? 0 : (n_chunks > 4 ? 4 : n_chunks));
  return pl;
}

// Vocabulary tiles one CTA of the probability pass walks for its row tile: more tiles hide the epilogue of one
// tile behind the MMAs of the next (two accumulator buffers), fewer fill the last wave better.
static int probs_tiles_per_cta(int64_t row_tiles, int n_tiles) {
  const int sms = sm_count();
  int best = 1;
  double best_eff = -1.0;
  for (int t = 1; t <= 32 && t <= n_tiles; ++t) {
    const int groups = (n_tiles + t - 1) / t;
    const double ctas = (double)row_tiles * groups;
    const double waves = (double)(int64_t)((ctas + sms - 1) / sms);
    const double eff = (ctas / (waves * sms)) * ((double)n_tiles / ((double)t * groups)) * (t / (t + 1.2));
    if (eff > best_eff + 1e-9) { best_eff = eff; best = t; }
  }
  return best;
}

// ------------------------------------------------------------------ forward statistics
int ce_tc_partial(const qpam_ce_args* a, const CETcPlan& pl, const CETcBuffers& b, cudaStream_t st) {
  CUtensorMap tmH, tmW;
  int rc = make_map(&tmH, a->h, a->F, a->N, a->F, tc::BK, tc::BM);
  if (rc) return rc;
  rc = make_map(&tmW, a->w, a->F, a->V, a->F, tc::BK, 128);     // a CTA of a pair loads half of a 256-row B tile
  if (rc) return rc;
  tc::GemmParams p{};
  p.n_tiles = pl.n_tiles;
  p.tiles_per_cta = pl.tiles_per_split;
  p.kb_total = (a->F + tc::BK - 1) / tc::BK;
  p.kb_per_split = p.kb_total;
  p.M = a->N; p.N = a->V;
  p.targets = a->targets; p.v_offset = a->v_offset; p.ignore_index = a->ignore_index;
  p.pm = b.pm; p.ps = b.ps; p.pt = b.pt; p.pbest = b.pbest; p.pidx = b.pidx;
  p.stats_ld = a->N; p.row_base = 0;
  // CTA pairs (cta_group::2): two row tiles share one 256-column B tile, each CTA loading half of it
  auto kern = tc::k_tc_gemm<256, tc::EPI_STATS, false, false, 1, true>;
  using CfgP = tc::Cfg<256, 1, true>;
  rc = opt_in_smem(kern, CfgP::SMEM_BYTES);
  if (rc) return rc;
  const unsigned row_tiles = (unsigned)((a->N + tc::BM - 1) / tc::BM);
  p.swap_xy = 1;      // blockIdx.x walks the row tiles: the two CTAs of a pair are neighbours in x
  QPAM_CUDA(launch_pairs(kern, dim3((row_tiles + 1) & ~1u, pl.nsplit, 1), 0, CfgP::SMEM_BYTES, st, tmH, tmW, tmW, p));
  QPAM_LAUNCH_CHECK("k_tc_gemm<stats>");
  return QPAM_OK;
}

// ------------------------------------------------------------------ plain logits (sampling decode head)
// out[N][ld] (bf16) = h w^T: the logits GEMM of the statistics pass with the accumulators leaving as bf16 tiles
// through TMA stores; CTA pairs, a pair walks a few vocabulary tiles of its two row tiles.
int ce_tc_logits(const qpam_ce_args* a, const CETcPlan& pl, void* out, int64_t ld, cudaStream_t st) {
  auto kern = tc::k_tc_gemm<256, tc::EPI_STORE_BF16, false, false, 1, true>;
  using CfgP = tc::Cfg<256, 1, true>;
  int rc = opt_in_smem(kern, CfgP::SMEM_BYTES_STAGED);
  if (rc) return rc;
  CUtensorMap tmH, tmW, tmO;
  if ((rc = make_map(&tmH, a->h, a->F, a->N, a->F, tc::BK, tc::BM))) return rc;
  if ((rc = make_map(&tmW, a->w, a->F, a->V, a->F, tc::BK, 128))) return rc;
  if ((rc = make_map(&tmO, out, a->V, a->N, ld, 64, 32))) return rc;
  const unsigned row_tiles = (unsigned)((a->N + tc::BM - 1) / tc::BM);
  tc::GemmParams p{};
  p.n_tiles = pl.n_tiles;
  p.tiles_per_cta = probs_tiles_per_cta(row_tiles, pl.n_tiles);
  const unsigned n_groups = (unsigned)((pl.n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta);
  p.kb_total = (a->F + tc::BK - 1) / tc::BK;
  p.kb_per_split = p.kb_total;
  p.M = a->N; p.N = a->V;
  p.swap_xy = 1;
  QPAM_CUDA(launch_pairs(kern, dim3((row_tiles + 1) & ~1u, n_groups, 1), 0, CfgP::SMEM_BYTES_STAGED, st, tmH, tmW, tmO, p));
  QPAM_LAUNCH_CHECK("k_tc_gemm<logits>");
  return QPAM_OK;
}

// ------------------------------------------------------------------ backward
__global__ void k_reduce_splits_bf16(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int64_t n,
                                     int splits, int64_t split_stride) {
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 acc = *reinterpret_cast<const float4*>(part + i);
    for (int s = 1; s < splits; ++s) {
      const float4 x = *reinterpret_cast<const float4*>(part + s * split_stride + i);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + i) = pk;
  }
}

// make `waiter` wait for everything enqueued on `st` so far
int signal_stream(cudaStream_t st, cudaStream_t waiter) {
  cudaEvent_t ev;
  QPAM_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ev, st);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(waiter, ev, 0);
  cudaEventDestroy(ev);      // released once the record has completed
  if (e != cudaSuccess) return cuda_fail(e, "signal_stream");
  return QPAM_OK;
}

int ce_tc_backward(const qpam_ce_args* a, const CETcPlan& pl, const CETcBuffers& b, const float* lse,
                   const float* grad_scale, const float* denom, void* dh, void* dw, cudaStream_t st,
                   cudaStream_t dh_ready_stream) {
  const int F = a->F;
  const int64_t V = a->V;
  auto k_probs = tc::k_tc_gemm<256, tc::EPI_PROBS, false, false, 1, true>;      // CTA pairs, as the forward pass
  using CfgP = tc::Cfg<256, 1, true>;
  // dH and dW run long K loops into few output tiles: two row tiles per CTA share every B block
  constexpr int MT = 2;
  auto k_dh = tc::k_tc_gemm<256, tc::EPI_STORE, false, true, MT>;
  auto k_dw = tc::k_tc_gemm<256, tc::EPI_STORE, true, true, MT>;
  int rc = opt_in_smem(k_probs, CfgP::SMEM_BYTES_STAGED);
  if (rc) return rc;
  rc = opt_in_smem(k_dh, tc::Cfg<256, MT>::SMEM_BYTES_STAGED);
  if (rc) return rc;
  rc = opt_in_smem(k_dw, tc::Cfg<256, MT>::SMEM_BYTES_STAGED);
  if (rc) return rc;
  // one row chunk: dW is complete after one product and leaves as bf16 straight from the accumulators
  auto k_dw16 = tc::k_tc_gemm<256, tc::EPI_STORE_BF16, true, true, MT>;
  const bool dw_direct = a->N <= pl.chunk_rows;
  rc = opt_in_smem(k_dw16, tc::Cfg<256, MT>::SMEM_BYTES_STAGED);
  if (rc) return rc;
  CUtensorMap tmWk, tmWmn;
  rc = make_map(&tmWk, a->w, F, V, F, tc::BK, 128);   // K-major B of the logits GEMM: half a tile per CTA of a pair
  if (rc) return rc;
  rc = make_map(&tmWmn, a->w, F, V, F, 64, 64);        // MN-major B of dH = P W   ([K=V][N=F])
  if (rc) return rc;
  const int f_tiles = (F + 255) / 256;
  int chunk_idx = 0;
  for (int64_t r0 = 0; r0 < a->N; r0 += pl.chunk_rows) {
    const int64_t rows = (a->N - r0 < pl.chunk_rows) ? a->N - r0 : pl.chunk_rows;
    const unsigned row_tiles = (unsigned)((rows + tc::BM - 1) / tc::BM);
    const __nv_bfloat16* hchunk = reinterpret_cast<const __nv_bfloat16*>(a->h) + r0 * F;
    CUtensorMap tmHk, tmHmn, tmPk, tmPmn;
    if ((rc = make_map(&tmHk, hchunk, F, rows, F, tc::BK, tc::BM))) return rc;       // A of logits
    if ((rc = make_map(&tmHmn, hchunk, F, rows, F, 64, 64))) return rc;              // MN-major B of dW ([K=rows][N=F])
    if ((rc = make_map(&tmPk, b.pbuf, V, rows, b.ldp, tc::BK, tc::BM))) return rc;   // K-major A of dH ([M=rows][K=V])
    if ((rc = make_map(&tmPmn, b.pbuf, V, rows, b.ldp, 64, 64))) return rc;          // MN-major A of dW ([K=rows][M=V])
    // 1) P = (softmax - onehot) * scale, bf16, 128 x 256 tiles; a CTA walks a few vocabulary tiles of its rows
    tc::GemmParams p{};
    p.n_tiles = pl.n_tiles; p.tiles_per_cta = probs_tiles_per_cta(row_tiles, pl.n_tiles);
    const unsigned n_groups = (unsigned)((pl.n_tiles + p.tiles_per_cta - 1) / p.tiles_per_cta);
    p.kb_total = (F + tc::BK - 1) / tc::BK; p.kb_per_split = p.kb_total;
    p.M = rows; p.N = V;
    p.targets = a->targets; p.v_offset = a->v_offset; p.ignore_index = a->ignore_index;
    p.row_base = r0;
    p.pbuf = reinterpret_cast<__nv_bfloat16*>(b.pbuf); p.ldp = b.ldp;
    p.lse = lse; p.mask = a->mask; p.grad_scale = grad_scale; p.denom = denom;
    p.swap_xy = 1;   // consecutive CTAs take the row tiles of one vocabulary tile: W is read from DRAM once
    CUtensorMap tmPst;                                                                 // P as the output of TMA stores
    if ((rc = make_map(&tmPst, b.pbuf, V, rows, b.ldp, 64, 32))) return rc;
    QPAM_CUDA(launch_pairs(k_probs, dim3((row_tiles + 1) & ~1u, n_groups, 1), 0, CfgP::SMEM_BYTES_STAGED, st, tmHk, tmWk, tmPst, p));
    QPAM_LAUNCH_CHECK("k_tc_gemm<probs>");
    // 2) dH[r0:r0+rows] = P W, split over the vocabulary (K) axis, fp32 partials then bf16
    tc::GemmParams g{};
    g.n_tiles = f_tiles; g.tiles_per_cta = 1;
    g.kb_total = (int32_t)((V + tc::BK - 1) / tc::BK);
    g.kb_per_split = (g.kb_total + pl.ksplit - 1) / pl.ksplit;
    const int ks = (g.kb_total + g.kb_per_split - 1) / g.kb_per_split;
    g.M = rows; g.N = F;
    g.c = b.dh_part; g.ldc = F; g.beta = 0;
    k_dh<<<dim3(f_tiles, (row_tiles + MT - 1) / MT, ks), tc::NTHREADS, tc::Cfg<256, MT>::SMEM_BYTES_STAGED, st>>>(tmPk, tmWmn, tmWmn, g);
    QPAM_LAUNCH_CHECK("k_tc_gemm<dH>");
    k_reduce_splits_bf16<<<592, 256, 0, st>>>(b.dh_part, reinterpret_cast<__nv_bfloat16*>(dh) + r0 * F, rows * F, ks,
                                             rows * F);
    QPAM_LAUNCH_CHECK("k_reduce_splits_bf16");
    if (dh_ready_stream != nullptr && r0 + rows >= a->N) {
      // dH is complete: a caller's side stream (the all-reduce of the vocabulary-parallel form) may start on it
      // while the dW products below still run
      int rc2 = signal_stream(st, dh_ready_stream);
      if (rc2) return rc2;
    }
    // 3) dW (+)= P^T H[r0:r0+rows]
    tc::GemmParams w{};
    w.n_tiles = f_tiles; w.tiles_per_cta = 1;
    w.kb_total = (int32_t)((rows + tc::BK - 1) / tc::BK); w.kb_per_split = w.kb_total;
    w.M = V; w.N = F;
    if (!dw_direct) { w.c = b.dwacc + (size_t)(chunk_idx % pl.dw_bufs) * V * F; w.beta = chunk_idx >= pl.dw_bufs ? 1 : 0; }
    w.ldc = F;
    if (dw_direct) {
      CUtensorMap tmDw;
      if ((rc = make_map(&tmDw, dw, F, V, F, 64, 32))) return rc;
      k_dw16<<<dim3(f_tiles, (unsigned)((V + MT * tc::BM - 1) / (MT * tc::BM)), 1), tc::NTHREADS,
               tc::Cfg<256, MT>::SMEM_BYTES_STAGED, st>>>(tmPmn, tmHmn, tmDw, w);
    } else {
      k_dw<<<dim3(f_tiles, (unsigned)((V + MT * tc::BM - 1) / (MT * tc::BM)), 1), tc::NTHREADS,
             tc::Cfg<256, MT>::SMEM_BYTES_STAGED, st>>>(tmPmn, tmHmn, tmHmn, w);
    }
    QPAM_LAUNCH_CHECK("k_tc_gemm<dW>");
    ++chunk_idx;
  }
  if (!dw_direct) {
    k_reduce_splits_bf16<<<1184, 256, 0, st>>>(b.dwacc, reinterpret_cast<__nv_bfloat16*>(dw), V * (int64_t)F,
                                              chunk_idx < pl.dw_bufs ? (chunk_idx > 0 ? chunk_idx : 1) : pl.dw_bufs, V * (int64_t)F);
    QPAM_LAUNCH_CHECK("k_reduce_splits_bf16");
  }
  return QPAM_OK;
}

}  // namespace qpam

namespace qpam {
int ce_tc_device_status(int* value, bool clear) {
  QPAM_CUDA(umma::read_device_error(value, clear));
  return QPAM_OK;
}
}  // namespace qpam
