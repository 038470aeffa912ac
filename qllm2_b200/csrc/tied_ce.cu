// Host side of the fused tied-head cross-entropy: argument checks, workspace carving, launches.
#include "tied_ce_kernels.cuh"
#include "tied_ce_tc.cuh"

namespace qpam {

static inline size_t ce_align(size_t x) { return (x + 255) & ~(size_t)255; }
static inline size_t dtype_size(int dt) { return dt == QPAM_BF16 ? 2 : 4; }

struct CELayout {
  int32_t nsplit, tiles_per_split;
  int64_t ldp, chunk_rows;
  size_t off_pm, off_ps, off_pt, off_pbest, off_pidx, total_fwd;
  size_t off_pbuf, off_dwacc, off_dhpart, total_bwd;
  CETcPlan tc;  // tensor-core path (bf16 inputs)
};

static CELayout ce_layout(const qpam_ce_args* a) {
  CELayout L{};
  const int64_t nvt = (a->V + CE_TN - 1) / CE_TN;
  const int64_t nrt = (a->N + CE_TM - 1) / CE_TM;
  int64_t want = nrt > 0 ? (592 + nrt - 1) / nrt : 1;  // aim at ~4 CTAs per SM
  if (want < 1) want = 1;
  if (want > nvt) want = nvt;
  if (want < 1) want = 1;
  L.tiles_per_split = (int32_t)((nvt + want - 1) / want);
  if (L.tiles_per_split < 1) L.tiles_per_split = 1;
  L.nsplit = (int32_t)((nvt + L.tiles_per_split - 1) / L.tiles_per_split);
  if (L.nsplit < 1) L.nsplit = 1;
  L.tc = ce_tc_plan(a);
  const int32_t split_cap = (L.tc.enabled && L.tc.nsplit > L.nsplit) ? L.tc.nsplit : L.nsplit;
  const size_t n = (size_t)split_cap * (size_t)(a->N > 0 ? a->N : 1);
  size_t off = 0;
  L.off_pm = off; off += ce_align(n * 4);
  L.off_ps = off; off += ce_align(n * 4);
  L.off_pt = off; off += ce_align(n * 4);
  L.off_pbest = off; off += ce_align(n * 4);
  L.off_pidx = off; off += ce_align(n * 4);
  L.total_fwd = off;
  L.ldp = (a->V + 7) & ~(int64_t)7;
  const size_t row_bytes = (size_t)L.ldp * dtype_size(a->io_dtype);
  int64_t rows = (int64_t)(((size_t)256 << 20) / row_bytes);
  rows = (rows / CE_TM) * CE_TM;
  if (rows < CE_TM) rows = CE_TM;
  const int64_t n_up = ((a->N + CE_TM - 1) / CE_TM) * CE_TM;
  if (rows > n_up) rows = n_up > 0 ? n_up : CE_TM;
  L.chunk_rows = rows;
  size_t pbuf_bytes = (size_t)rows * row_bytes;
  if (L.tc.enabled && (size_t)L.tc.chunk_rows * row_bytes > pbuf_bytes) pbuf_bytes = (size_t)L.tc.chunk_rows * row_bytes;
  L.off_pbuf = off; off += ce_align(pbuf_bytes);
  L.off_dwacc = off;
  if (a->io_dtype != QPAM_F32) off += ce_align((size_t)(L.tc.enabled ? L.tc.dw_bufs : 1) * a->V * a->F * 4);
  L.off_dhpart = off;
  if (L.tc.enabled) off += ce_align((size_t)L.tc.ksplit * L.tc.chunk_rows * a->F * 4);
  L.total_bwd = off;
  return L;
}

static int check_ce_args(const qpam_ce_args* a, bool need_targets) {
  QPAM_REQUIRE(a != nullptr, "ce: args is NULL");
  QPAM_REQUIRE(a->h && a->w, "ce: h/w must not be NULL");
  QPAM_REQUIRE(!need_targets || a->targets, "ce: targets must not be NULL");
  QPAM_REQUIRE(a->N >= 0 && a->V >= 1 && a->F >= 1, "ce: bad N/V/F = %lld/%lld/%d", (long long)a->N, (long long)a->V, a->F);
  QPAM_REQUIRE(a->V < ((int64_t)1 << 31), "ce: V too large");
  QPAM_REQUIRE(a->io_dtype == QPAM_F32 || a->io_dtype == QPAM_BF16, "ce: io_dtype %d unknown", a->io_dtype);
  QPAM_REQUIRE(a->workspace != nullptr && ((uintptr_t)a->workspace & 255) == 0, "ce: workspace NULL or not 256-byte aligned");
  return QPAM_OK;
}

static CEParams ce_params(const qpam_ce_args* a, const CELayout& L) {
  CEParams p{};
  char* ws = reinterpret_cast<char*>(a->workspace);
  p.h = a->h; p.w = a->w; p.targets = a->targets; p.mask = a->mask;
  p.N = a->N; p.V = a->V; p.v_offset = a->v_offset; p.ignore_index = a->ignore_index; p.F = a->F;
  p.pm = reinterpret_cast<float*>(ws + L.off_pm);
  p.ps = reinterpret_cast<float*>(ws + L.off_ps);
  p.pt = reinterpret_cast<float*>(ws + L.off_pt);
  p.pbest = reinterpret_cast<float*>(ws + L.off_pbest);
  p.pidx = reinterpret_cast<int32_t*>(ws + L.off_pidx);
  p.nsplit = L.nsplit; p.tiles_per_split = L.tiles_per_split;
  p.pbuf = ws + L.off_pbuf; p.ldp = L.ldp;
  return p;
}

static bool tc_usable(const qpam_ce_args* a, const CELayout& L) {
  return L.tc.enabled && (((uintptr_t)a->h | (uintptr_t)a->w) & 15) == 0;
}

static CETcBuffers tc_buffers(const qpam_ce_args* a, const CELayout& L) {
  char* ws = reinterpret_cast<char*>(a->workspace);
  CETcBuffers b{};
  b.pm = reinterpret_cast<float*>(ws + L.off_pm);
  b.ps = reinterpret_cast<float*>(ws + L.off_ps);
  b.pt = reinterpret_cast<float*>(ws + L.off_pt);
  b.pbest = reinterpret_cast<float*>(ws + L.off_pbest);
  b.pidx = reinterpret_cast<int32_t*>(ws + L.off_pidx);
  b.pbuf = ws + L.off_pbuf;
  b.ldp = L.ldp;
  b.dh_part = reinterpret_cast<float*>(ws + L.off_dhpart);
  b.dwacc = reinterpret_cast<float*>(ws + L.off_dwacc);
  return b;
}

template <typename T>
static int ce_partial_t(const qpam_ce_args* a, const CELayout& L, float* row_max, float* row_sumexp,
                        float* row_tgt, int64_t* row_argmax, cudaStream_t st) {
  CEParams p = ce_params(a, L);
  const int64_t nrt = (a->N + CE_TM - 1) / CE_TM;
  k_ce_partial<T><<<dim3(L.nsplit, (unsigned)nrt), 256, 0, st>>>(p);
  QPAM_LAUNCH_CHECK("k_ce_partial");
  k_ce_merge<<<(unsigned)((a->N + 255) / 256), 256, 0, st>>>(p, row_max, row_sumexp, row_tgt, row_argmax);
  QPAM_LAUNCH_CHECK("k_ce_merge");
  return QPAM_OK;
}

template <typename T>
static int ce_bwd_t(const qpam_ce_args* a, const CELayout& L, const float* lse, const float* grad_scale,
                    const float* denom, void* dh, void* dw, cudaStream_t st) {
  CEParams p = ce_params(a, L);
  p.lse = lse; p.grad_scale = grad_scale; p.denom = denom;
  char* ws = reinterpret_cast<char*>(a->workspace);
  constexpr bool kF32 = sizeof(T) == 4;
  float* dwacc = kF32 ? reinterpret_cast<float*>(dw) : reinterpret_cast<float*>(ws + L.off_dwacc);
  const T* P = reinterpret_cast<const T*>(p.pbuf);
  const int64_t nvt = (a->V + CE_TN - 1) / CE_TN;
  const unsigned ft = (unsigned)((a->F + CE_TN - 1) / CE_TN);
  int first = 1;
  for (int64_t r0 = 0; r0 < a->N; r0 += L.chunk_rows) {
    const int64_t rows = (a->N - r0 < L.chunk_rows) ? a->N - r0 : L.chunk_rows;
    p.row0 = r0; p.rows = rows;
    const unsigned rt = (unsigned)((rows + CE_TM - 1) / CE_TM);
    k_ce_probs<T><<<dim3((unsigned)nvt, rt), 256, 0, st>>>(p);
    QPAM_LAUNCH_CHECK("k_ce_probs");
    // dH[r0:r0+rows] = P W
    k_gemm<T, T, T, false, false><<<dim3(ft, rt), 256, 0, st>>>(
        P, reinterpret_cast<const T*>(a->w), reinterpret_cast<T*>(dh) + r0 * a->F, rows, a->F, a->V, L.ldp, a->F,
        a->F, 0);
    QPAM_LAUNCH_CHECK("k_gemm<dH>");
    // dW += P^T H[r0:r0+rows]
    k_gemm<T, T, float, true, false><<<dim3(ft, (unsigned)nvt), 256, 0, st>>>(
        P, reinterpret_cast<const T*>(a->h) + r0 * a->F, dwacc, a->V, a->F, rows, L.ldp, a->F, a->F, first ? 0 : 1);
    QPAM_LAUNCH_CHECK("k_gemm<dW>");
    first = 0;
  }
  if (a->N == 0) {
    QPAM_CUDA(cudaMemsetAsync(dw, 0, (size_t)a->V * a->F * sizeof(T), st));
  } else if (!kF32) {
    k_cast_from_f32<T><<<1184, 256, 0, st>>>(dwacc, reinterpret_cast<T*>(dw), a->V * (int64_t)a->F);
    QPAM_LAUNCH_CHECK("k_cast_from_f32");
  }
  return QPAM_OK;
}

}  // namespace qpam

using namespace qpam;

extern "C" size_t qpam_ce_workspace_bytes(const qpam_ce_args* a, int32_t with_backward) {
  if (a == nullptr || a->V < 1 || a->F < 1 || a->N < 0) return 0;
  const CELayout L = ce_layout(a);
  return with_backward ? L.total_bwd : L.total_fwd;
}

extern "C" int qpam_ce_partial(const qpam_ce_args* a, float* row_max, float* row_sumexp, float* row_tgt,
                               int64_t* row_argmax, void* stream) {
  int rc = check_ce_args(a, row_tgt != nullptr);
  if (rc) return rc;
  const CELayout L = ce_layout(a);
  if (a->workspace_bytes < L.total_fwd) {
    set_error("ce partial: workspace %zu bytes < required %zu", a->workspace_bytes, L.total_fwd);
    return QPAM_EWORKSPACE;
  }
  if (a->N == 0) return QPAM_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tc_usable(a, L)) {
    rc = ce_tc_partial(a, L.tc, tc_buffers(a, L), st);
    if (rc) return rc;
    CEParams p = ce_params(a, L);
    p.nsplit = L.tc.nsplit;
    k_ce_merge<<<(unsigned)((a->N + 255) / 256), 256, 0, st>>>(p, row_max, row_sumexp, row_tgt, row_argmax);
    QPAM_LAUNCH_CHECK("k_ce_merge");
    return QPAM_OK;
  }
  return a->io_dtype == QPAM_BF16 ? ce_partial_t<__nv_bfloat16>(a, L, row_max, row_sumexp, row_tgt, row_argmax, st)
                                  : ce_partial_t<float>(a, L, row_max, row_sumexp, row_tgt, row_argmax, st);
}

extern "C" int qpam_ce_finalize(const qpam_ce_args* a, const float* row_max, const float* row_sumexp,
                                const float* row_tgt, const int64_t* row_argmax, float* lse, float* per_token,
                                float* loss_sum, float* denom, float* correct, float* tokens, void* stream) {
  int rc = check_ce_args(a, true);
  if (rc) return rc;
  QPAM_REQUIRE(row_max && row_sumexp && row_tgt && lse, "ce finalize: row_max/row_sumexp/row_tgt/lse must not be NULL");
  QPAM_REQUIRE(correct == nullptr || row_argmax != nullptr, "ce finalize: correct needs row_argmax");
  CEParams p{};
  p.targets = a->targets; p.mask = a->mask; p.N = a->N; p.ignore_index = a->ignore_index;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  k_ce_finalize<<<1, 1024, 0, st>>>(p, row_max, row_sumexp, row_tgt, row_argmax, lse, per_token, loss_sum, denom,
                                    correct, tokens);
  QPAM_LAUNCH_CHECK("k_ce_finalize");
  return QPAM_OK;
}

extern "C" int qpam_ce_bwd(const qpam_ce_args* a, const float* lse, const float* grad_scale, const float* denom,
                           void* dh, void* dw, void* stream) {
  return qpam_ce_bwd_overlap(a, lse, grad_scale, denom, dh, dw, stream, nullptr);
}

extern "C" int qpam_ce_bwd_overlap(const qpam_ce_args* a, const float* lse, const float* grad_scale, const float* denom,
                                   void* dh, void* dw, void* stream, void* dh_ready_stream) {
  int rc = check_ce_args(a, true);
  if (rc) return rc;
  QPAM_REQUIRE(lse && grad_scale && denom && dh && dw, "ce bwd: NULL pointer argument");
  const CELayout L = ce_layout(a);
  if (a->workspace_bytes < L.total_bwd) {
    set_error("ce bwd: workspace %zu bytes < required %zu", a->workspace_bytes, L.total_bwd);
    return QPAM_EWORKSPACE;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaStream_t side = reinterpret_cast<cudaStream_t>(dh_ready_stream);
  if (a->N > 0 && tc_usable(a, L) && ((uintptr_t)dh & 15) == 0 && ((uintptr_t)dw & 15) == 0)
    return ce_tc_backward(a, L.tc, tc_buffers(a, L), lse, grad_scale, denom, dh, dw, st, side);
  rc = a->io_dtype == QPAM_BF16 ? ce_bwd_t<__nv_bfloat16>(a, L, lse, grad_scale, denom, dh, dw, st)
                                : ce_bwd_t<float>(a, L, lse, grad_scale, denom, dh, dw, st);
  if (rc == QPAM_OK && side != nullptr) rc = signal_stream(st, side);    // these kernels finish dh and dw together
  return rc;
}

extern "C" int qpam_head_logits(const qpam_ce_args* a, void* logits, int64_t ld, void* stream) {
  QPAM_REQUIRE(a != nullptr && a->h && a->w, "head logits: args / h / w must not be NULL");
  QPAM_REQUIRE(a->N >= 0 && a->V >= 1 && a->F >= 1 && a->V < ((int64_t)1 << 31), "head logits: bad N/V/F = %lld/%lld/%d",
               (long long)a->N, (long long)a->V, a->F);
  QPAM_REQUIRE(a->io_dtype == QPAM_F32 || a->io_dtype == QPAM_BF16, "head logits: io_dtype %d unknown", a->io_dtype);
  QPAM_REQUIRE(logits != nullptr, "head logits: logits must not be NULL");
  QPAM_REQUIRE(ld >= a->V && ld % 8 == 0 && ((uintptr_t)logits & 15) == 0,
               "head logits: ld must be a multiple of 8 that covers V, logits 16-byte aligned (got ld %lld)", (long long)ld);
  const CELayout L = ce_layout(a);
  if (!tc_usable(a, L)) {
    set_error("head logits: bf16 h and w with 16-byte aligned rows only (the tensor-core path)");
    return QPAM_EUNSUPPORTED;
  }
  if (a->N == 0) return QPAM_OK;
  return ce_tc_logits(a, L.tc, logits, ld, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int qpam_head_argmax(const qpam_ce_args* a, int64_t* ids, float* best, void* stream) {
  QPAM_REQUIRE(ids != nullptr, "head argmax: ids must not be NULL");
  return qpam_ce_partial(a, best, nullptr, nullptr, ids, stream);
}
