// Host side of the chunked PAM scan: argument checks, workspace carving, launches.
#include <mutex>

#include "pam_scan_chunk.cuh"
#include "pam_scan_tc.cuh"
#include "pam_scan_tc2.cuh"
#include "pam_scan_tc3.cuh"
#include "tma_host.cuh"

namespace qpam {

static inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Chunks-before-sequence prefix of the packed layout, with the descriptor checked on the way: cu_seqlens must
// start at 0, never decrease and end at or before T.  A descriptor that fails leaves an all-zero prefix (no
// kernel of the call then finds a chunk to work on, so nothing is read or written through it) and records
// QPAM_DEV_BAD_CU_SEQLENS in the device status word.
constexpr int QPAM_DEV_BAD_CU_SEQLENS = 301;
constexpr int QPAM_DEV_WAIT_SELFTEST = 299;
__global__ void __launch_bounds__(256) k_chunk_prefix_checked(const int32_t* __restrict__ cu, int32_t* __restrict__ prefix,
                                                               int S, int ch, int T) {
  // one CTA: sequences in tiles of 256, each tile an inclusive scan of the chunk counts (warp shuffles + one
  // exchange through shared memory) on top of the running total; the descriptor is checked on the way
  __shared__ int wsum[8];
  __shared__ int carry_s, bad_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { carry_s = 0; bad_s = (cu[0] != 0) ? 1 : 0; prefix[0] = 0; }
  __syncthreads();
  for (int base = 0; base < S; base += 256) {
    const int s_ = base + tid;
    int n = 0;
    bool bad = false;
    if (s_ < S) {
      const int a = cu[s_], e = cu[s_ + 1];
      bad = !(e >= a && e <= T);
      n = (max(0, e - a) + ch - 1) / ch;
    }
    int inc = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) wsum[warp] = inc;
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(&bad_s, 1);
    __syncthreads();
    int before = carry_s;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    if (s_ < S) prefix[s_ + 1] = before + inc;
    __syncthreads();
    if (tid == 255) carry_s = before + inc;
    __syncthreads();
  }
  if (bad_s) {
    for (int s_ = tid; s_ <= S; s_ += 256) prefix[s_] = 0;
    if (tid == 0) umma::record_device_error(QPAM_DEV_BAD_CU_SEQLENS);
  }
}

struct ScanLayout {
  int64_t nslots;
  int32_t ch;           // tokens per chunk of this layout
  int32_t nc_uniform;
  int32_t grid_chunks;  // upper bound on the number of chunks (grid.x of the chunk kernels)
  size_t off_prefix, off_states, off_decay, off_dstates, off_anchors, off_dak, total_fwd, total_bwd;
};

// Tensor-core kernels take bf16 token tensors with head dim 64 and a single state; their chunk is
// 128 tokens.  Everything else runs the FFMA kernels on 64-token chunks.
static bool tc_fwd_eligible(const qpam_scan_args* a) {
  return a->io_dtype == QPAM_BF16 && a->d == 64 && a->K == 1 && a->coef == nullptr &&
         (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->y) & 15) == 0 &&
         (int64_t)a->B * a->H * a->T < ((int64_t)1 << 31);
}
// bf16 / d = 64 / 2..4 phase-routed states: forward on the fused K-state tensor-core kernel
static bool tc_fwdK_eligible(const qpam_scan_args* a) {
  return a->io_dtype == QPAM_BF16 && a->d == 64 && a->K >= 2 && a->K <= QPAM_MAX_STATES &&
         (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->y) & 15) == 0 &&
         (int64_t)a->B * a->H * a->T < ((int64_t)1 << 31);
}
static int fwd_chunk_len(const qpam_scan_args* a) { return (tc_fwd_eligible(a) || tc_fwdK_eligible(a)) ? tcs::TC : CH; }

static ScanLayout scan_layout(const qpam_scan_args* a, int ch) {
  ScanLayout L{};
  const int64_t S = a->S;
  const int64_t dd = (int64_t)a->d * a->d;
  L.ch = ch;
  if (a->cu_seqlens == nullptr) {
    L.nc_uniform = (a->T + ch - 1) / ch;
    L.nslots = S * (L.nc_uniform + 1);
    L.grid_chunks = (int32_t)(S * L.nc_uniform);
  } else {
    L.nc_uniform = 0;
    L.nslots = a->T / ch + 2 * S;
    L.grid_chunks = (int32_t)(a->T / ch + S);
  }
  size_t off = 0;
  L.off_prefix = off;
  off += align256(sizeof(int32_t) * (size_t)(S + 1));
  L.off_states = off;
  off += align256(sizeof(float2) * (size_t)a->K * a->H * L.nslots * dd);
  L.off_decay = off;
  off += align256(sizeof(float) * (size_t)a->K * a->H * L.nslots);
  L.total_fwd = off;
  L.off_dstates = off;
  off += align256(sizeof(float2) * (size_t)a->K * a->H * L.nslots * dd);
  L.off_anchors = off;   // partial sums of the decay-gradient anchors (tensor-core backward)
  off += align256(sizeof(float) * (size_t)a->K * a->H * L.nslots * tcs::ANCHOR_PARTS);
  L.off_dak = off;       // Re<k_t, dk_t> per token (tensor-core backward)
  off += align256(sizeof(float) * (size_t)a->B * a->H * a->T);
  L.total_bwd = off;
  return L;
}

static int check_scan_args(const qpam_scan_args* a) {
  QPAM_REQUIRE(a != nullptr, "scan: args is NULL");
  QPAM_REQUIRE(a->d == 16 || a->d == 32 || a->d == 64, "scan: head dim d=%d not in {16,32,64}", a->d);
  QPAM_REQUIRE(a->K >= 1 && a->K <= QPAM_MAX_STATES, "scan: K=%d outside [1,%d]", a->K, QPAM_MAX_STATES);
  QPAM_REQUIRE(a->B >= 1 && a->H >= 1 && a->T >= 0, "scan: bad B/H/T = %d/%d/%d", a->B, a->H, a->T);
  QPAM_REQUIRE(a->H <= 65535 && a->H * a->K <= 65535, "scan: H*K too large for the launch grid");
  QPAM_REQUIRE(a->io_dtype == QPAM_F32 || a->io_dtype == QPAM_BF16, "scan: io_dtype %d unknown", a->io_dtype);
  if (a->cu_seqlens != nullptr) {
    QPAM_REQUIRE(a->B == 1, "scan: packed mode (cu_seqlens) needs B == 1, got %d", a->B);
    QPAM_REQUIRE(a->S >= 1, "scan: packed mode needs S >= 1");
  } else {
    QPAM_REQUIRE(a->S == a->B, "scan: without cu_seqlens S must equal B (%d vs %d)", a->S, a->B);
  }
  QPAM_REQUIRE(a->q && a->k && a->v && a->gamma, "scan: q/k/v/gamma must not be NULL");
  QPAM_REQUIRE(a->workspace != nullptr && ((uintptr_t)a->workspace & 255) == 0,
               "scan: workspace NULL or not 256-byte aligned");
  QPAM_REQUIRE((int64_t)a->B * a->H * a->T * a->d * 2 < ((int64_t)1 << 40), "scan: tensors too large");
  return QPAM_OK;
}

static ScanParams make_params(const qpam_scan_args* a, const ScanLayout& L) {
  ScanParams p{};
  char* ws = reinterpret_cast<char*>(a->workspace);
  p.q = a->q; p.k = a->k; p.v = a->v;
  p.gamma = a->gamma; p.coef = a->coef;
  p.y = a->y;
  p.states = reinterpret_cast<float2*>(ws + L.off_states);
  p.chunk_decay = reinterpret_cast<float*>(ws + L.off_decay);
  p.dstates = reinterpret_cast<float2*>(ws + L.off_dstates);
  p.s0 = a->s0; p.s_final = a->s_final;
  p.geom.cu_seqlens = a->cu_seqlens;
  p.geom.chunk_prefix = reinterpret_cast<const int32_t*>(ws + L.off_prefix);
  p.geom.S = a->S; p.geom.T = a->T; p.geom.nc_uniform = L.nc_uniform; p.geom.ch = L.ch;
  p.nslots = L.nslots;
  p.B = a->B; p.H = a->H; p.T = a->T; p.K = a->K;
  p.q_scale = a->q_scale; p.eps = a->gamma_eps;
  return p;
}

template <typename KernelT>
static int set_smem(KernelT kern, size_t bytes) {
  if (bytes > 48 * 1024) QPAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return QPAM_OK;
}

template <int D>
constexpr size_t outer_smem() { return sizeof(float2) * 2 * CH * (D + 1) + sizeof(float) * CH; }

template <int D, typename T>
static int launch_states(const ScanParams& p, const ScanLayout& L, const qpam_scan_args* a, cudaStream_t st) {
  // chunk-local state sums, then the carry over the chunk axis
  if (a->cu_seqlens != nullptr) {
    k_chunk_prefix_checked<<<1, 256, 0, st>>>(a->cu_seqlens, const_cast<int32_t*>(p.geom.chunk_prefix), a->S, L.ch, a->T);
    QPAM_LAUNCH_CHECK("k_chunk_prefix");
  }
  if (L.grid_chunks > 0) {
    auto kern = k_chunk_outer<D, T, false>;
    int rc = set_smem(kern, outer_smem<D>());
    if (rc) return rc;
    kern<<<dim3(L.grid_chunks, a->H, a->K), NT, outer_smem<D>(), st>>>(p);
    QPAM_LAUNCH_CHECK("k_chunk_outer<state>");
  }
  const int n4 = D * D / 2;
  k_state_scan<false><<<dim3(a->S, a->H * a->K, (n4 + 255) / 256), 256, 0, st>>>(p, D);
  QPAM_LAUNCH_CHECK("k_state_scan<fwd>");
  return QPAM_OK;
}

template <int D, typename T>
static int scan_fwd_t(const qpam_scan_args* a, const ScanLayout& L, cudaStream_t st) {
  ScanParams p = make_params(a, L);
  int rc = launch_states<D, T>(p, L, a, st);
  if (rc) return rc;
  if (L.grid_chunks > 0 && a->y != nullptr) {
    auto kern = k_fwd_chunk<D, T>;
    rc = set_smem(kern, fwd_chunk_smem<D>());
    if (rc) return rc;
    kern<<<dim3(L.grid_chunks, a->H), NT, fwd_chunk_smem<D>(), st>>>(p);
    QPAM_LAUNCH_CHECK("k_fwd_chunk");
  }
  return QPAM_OK;
}

// The view of ONE state k of a K-state problem as a single-state problem: every per-state array of the parameters
// and of the workspace is laid out state-major, so the kernels written for one state run on it with shifted bases.
static ScanParams one_state_view(const ScanParams& pK, const qpam_scan_args* a, const ScanLayout& L, int k) {
  ScanParams p = pK;
  const size_t per_state = (size_t)a->H * L.nslots;
  p.K = 1;
  p.gamma = pK.gamma + (size_t)k * a->B * a->H * a->T;
  p.states = pK.states + (size_t)k * per_state * 64 * 64;
  p.dstates = pK.dstates + (size_t)k * per_state * 64 * 64;
  p.chunk_decay = pK.chunk_decay + (size_t)k * per_state;
  if (pK.s0 != nullptr) p.s0 = pK.s0 + (size_t)k * a->S * a->H * 64 * 64 * 2;
  p.s_final = nullptr;      // written by the K-state carry
  p.coef = nullptr;
  return p;
}

// chunk-local state sums on tensor cores, then the carry over the chunk axis
static int tc_states(const ScanParams& p, const ScanLayout& L, const qpam_scan_args* a, cudaStream_t st) {
  if (L.grid_chunks > 0 && a->K > 1) {      // all states from one load of the key / value tiles
    int rc = set_smem(tcs::k_tc_chunk_outerK, tcs::OUTERK_SMEM);
    if (rc) return rc;
    CUtensorMap mk, mv;
    const int64_t rows = (int64_t)a->B * a->H * a->T;
    if ((rc = make_map(&mk, a->k, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&mv, a->v, 128, rows, 128, 64, 128))) return rc;
    tcs::k_tc_chunk_outerK<<<dim3(L.grid_chunks, a->H), 256, tcs::OUTERK_SMEM, st>>>(mk, mv, p);
    QPAM_LAUNCH_CHECK("k_tc_chunk_outerK");
  } else if (L.grid_chunks > 0) {
    int rc = set_smem(tcs::k_tc_chunk_outer<false>, tcs::OUTER_SMEM);
    if (rc) return rc;
    CUtensorMap mk, mv;
    const int64_t rows = (int64_t)a->B * a->H * a->T;
    if ((rc = make_map(&mk, a->k, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&mv, a->v, 128, rows, 128, 64, 128))) return rc;
    tcs::k_tc_chunk_outer<false><<<dim3(L.grid_chunks, a->H, a->K), 256, tcs::OUTER_SMEM, st>>>(mk, mv, p);
    QPAM_LAUNCH_CHECK("k_tc_chunk_outer<state>");
  }
  k_state_scan<false><<<dim3(a->S, a->H * a->K, (64 * 64 / 2 + 255) / 256), 256, 0, st>>>(p, 64);
  QPAM_LAUNCH_CHECK("k_state_scan<fwd>");
  return QPAM_OK;
}

// Output tensor as the target of the chunk kernels' TMA stores (boxes of 64 elements x 32 rows): [B*H*T rows][128], or
// for the token-major layout [B*T rows][H*128].
static int make_out_map(CUtensorMap* m, const qpam_scan_args* a, bool token_major) {
  if (token_major) return make_map(m, a->y, (int64_t)a->H * 128, (int64_t)a->B * a->T, (int64_t)a->H * 128, 64, 32);
  return make_map(m, a->y, 128, (int64_t)a->B * a->H * a->T, 128, 64, 32);
}

// bf16 / d = 64 / one state: tensor-core kernels on 128-token chunks
static int scan_fwd_tc(const qpam_scan_args* a, const ScanLayout& L, cudaStream_t st, bool token_major = false) {
  ScanParams p = make_params(a, L);
  p.y_token_major = token_major ? 1 : 0;
  if (a->cu_seqlens != nullptr) {
    k_chunk_prefix_checked<<<1, 256, 0, st>>>(a->cu_seqlens, const_cast<int32_t*>(p.geom.chunk_prefix), a->S, L.ch, a->T);
    QPAM_LAUNCH_CHECK("k_chunk_prefix");
  }
  int rc;
  rc = tc_states(p, L, a, st);
  if (rc) return rc;
  if (L.grid_chunks > 0 && a->y != nullptr) {
    tcs::ChunkMaps maps;
    const int64_t rows = (int64_t)a->B * a->H * a->T;
    if ((rc = make_map(&maps.a1, a->q, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.b1, a->k, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.x2, a->v, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_out_map(&maps.out, a, token_major))) return rc;
    if ((rc = set_smem(tcs::k_tc_chunk_fwd, tcs::CHUNK2_SMEM))) return rc;
    tcs::k_tc_chunk_fwd<<<dim3(L.grid_chunks, a->H), 256, tcs::CHUNK2_SMEM, st>>>(maps, p);
    QPAM_LAUNCH_CHECK("k_tc_chunk<fwd>");
  }
  return QPAM_OK;
}

// bf16 / d = 64 / K = 2..4 states: state sums and carry per state, then ONE fused output kernel
static int scan_fwd_tcK(const qpam_scan_args* a, const ScanLayout& L, cudaStream_t st, bool token_major = false) {
  ScanParams p = make_params(a, L);
  p.y_token_major = token_major ? 1 : 0;
  if (a->cu_seqlens != nullptr) {
    k_chunk_prefix_checked<<<1, 256, 0, st>>>(a->cu_seqlens, const_cast<int32_t*>(p.geom.chunk_prefix), a->S, L.ch, a->T);
    QPAM_LAUNCH_CHECK("k_chunk_prefix");
  }
  int rc = tc_states(p, L, a, st);
  if (rc) return rc;
  if (L.grid_chunks > 0 && a->y != nullptr) {
    tcs::ChunkMaps maps;
    const int64_t rows = (int64_t)a->B * a->H * a->T;
    if ((rc = make_map(&maps.a1, a->q, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.b1, a->k, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.x2, a->v, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_out_map(&maps.out, a, token_major))) return rc;
    if ((rc = set_smem(tcs::k_tc_chunk_fwdK, tcs::CHUNKK_SMEM))) return rc;
    tcs::k_tc_chunk_fwdK<<<dim3(L.grid_chunks, a->H), 256, tcs::CHUNKK_SMEM, st>>>(maps, p);
    QPAM_LAUNCH_CHECK("k_tc_chunk_fwdK");
  }
  return QPAM_OK;
}

// bf16 / d = 64 / K = 2..4 states, training form: the state sums of all states from ONE load of the key / value tiles
// and one carry launch, as above, then the single-state output kernel once per state into ys[k] (a backward needs
// every state's own output; the fused output kernel only leaves their weighted sum)
static int scan_fwd_tc_states(const qpam_scan_args* a, const ScanLayout& L, void* ys, cudaStream_t st) {
  ScanParams p = make_params(a, L);
  if (a->cu_seqlens != nullptr) {
    k_chunk_prefix_checked<<<1, 256, 0, st>>>(a->cu_seqlens, const_cast<int32_t*>(p.geom.chunk_prefix), a->S, L.ch, a->T);
    QPAM_LAUNCH_CHECK("k_chunk_prefix");
  }
  int rc = tc_states(p, L, a, st);
  if (rc) return rc;
  if (L.grid_chunks == 0) return QPAM_OK;
  tcs::ChunkMaps maps;
  const int64_t rows = (int64_t)a->B * a->H * a->T;
  if ((rc = make_map(&maps.a1, a->q, 128, rows, 128, 64, 128))) return rc;
  if ((rc = make_map(&maps.b1, a->k, 128, rows, 128, 64, 128))) return rc;
  if ((rc = make_map(&maps.x2, a->v, 128, rows, 128, 64, 128))) return rc;
  if ((rc = set_smem(tcs::k_tc_chunk_fwd, tcs::CHUNK2_SMEM))) return rc;
  for (int k = 0; k < a->K; ++k) {
    ScanParams pk = one_state_view(p, a, L, k);
    __nv_bfloat16* yk = reinterpret_cast<__nv_bfloat16*>(ys) + (size_t)k * rows * 128;
    pk.y = yk;
    if ((rc = make_map(&maps.out, yk, 128, rows, 128, 64, 32))) return rc;
    tcs::k_tc_chunk_fwd<<<dim3(L.grid_chunks, a->H), 256, tcs::CHUNK2_SMEM, st>>>(maps, pk);
    QPAM_LAUNCH_CHECK("k_tc_chunk<fwd>");
  }
  return QPAM_OK;
}

// bf16 / d = 64 / one state, backward: gradient state sums -> reverse carry (with the anchors of the decay
// gradient) -> ONE launch for the dq, dv, dk jobs of every chunk -> dgamma.  Everything stays on the caller's stream.
// state >= 0: `a` describes K states whose forward (qpam_scan_fwd_states) left its states in the workspace; the backward of
// that one state runs on its slices (dgamma, ds_final, ds0 are that state's arrays)
static int scan_bwd_tc(const qpam_scan_args* a, const ScanLayout& L, const void* dy, void* dq, void* dk, void* dv,
                       float* dgamma, const float* ds_final, float* ds0, int states_valid, cudaStream_t st,
                       bool accumulate = false, int state = -1) {
  ScanParams p = make_params(a, L);
  if (state >= 0) p = one_state_view(p, a, L, state);
  p.dy = dy; p.dq = dq; p.dk = dk; p.dv = dv;
  p.dgamma = dgamma; p.dcoef = nullptr; p.ds_final = ds_final; p.ds0 = ds0;
  int rc;
  if (!states_valid) {
    ScanParams pf = p;
    pf.s_final = nullptr;
    if (a->cu_seqlens != nullptr) {
      k_chunk_prefix_checked<<<1, 256, 0, st>>>(a->cu_seqlens, const_cast<int32_t*>(p.geom.chunk_prefix), a->S, L.ch, a->T);
      QPAM_LAUNCH_CHECK("k_chunk_prefix");
    }
    rc = tc_states(pf, L, a, st);
    if (rc) return rc;
  }
  float* anchors = reinterpret_cast<float*>(reinterpret_cast<char*>(a->workspace) + L.off_anchors) +
                   (state > 0 ? (size_t)state * a->H * L.nslots * tcs::ANCHOR_PARTS : 0);
  p.dA_k = reinterpret_cast<float*>(reinterpret_cast<char*>(a->workspace) + L.off_dak);
  if (L.grid_chunks > 0) {
    rc = set_smem(tcs::k_tc_chunk_outer<true>, tcs::OUTER_SMEM);
    if (rc) return rc;
    CUtensorMap mq, mdy;
    const int64_t rows = (int64_t)a->B * a->H * a->T;
    if ((rc = make_map(&mq, a->q, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&mdy, dy, 128, rows, 128, 64, 128))) return rc;
    tcs::k_tc_chunk_outer<true><<<dim3(L.grid_chunks, a->H), 256, tcs::OUTER_SMEM, st>>>(mq, mdy, p);
    QPAM_LAUNCH_CHECK("k_tc_chunk_outer<dstate>");
  }
  tcs::k_tc_state_scan_rev<<<dim3(a->S, a->H, 64 * 64 / 2 / 256), 256, 0, st>>>(p, anchors);
  QPAM_LAUNCH_CHECK("k_tc_state_scan_rev");
  if (L.grid_chunks > 0) {
    tcs::BwdMaps maps;
    const int64_t rows = (int64_t)a->B * a->H * a->T;
    if ((rc = make_map(&maps.q, a->q, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.k, a->k, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.v, a->v, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.dy, dy, 128, rows, 128, 64, 128))) return rc;
    if ((rc = make_map(&maps.dq, dq, 128, rows, 128, 64, 32))) return rc;
    if ((rc = make_map(&maps.dk, dk, 128, rows, 128, 64, 32))) return rc;
    if ((rc = make_map(&maps.dv, dv, 128, rows, 128, 64, 32))) return rc;
    if (accumulate) {
      if ((rc = set_smem(tcs::k_tc_chunk_bwd<true>, tcs::CHUNK2_SMEM))) return rc;
      tcs::k_tc_chunk_bwd<true><<<dim3(3 * L.grid_chunks, a->H), 256, tcs::CHUNK2_SMEM, st>>>(maps, p);
    } else {
      if ((rc = set_smem(tcs::k_tc_chunk_bwd<false>, tcs::CHUNK2_SMEM))) return rc;
      tcs::k_tc_chunk_bwd<false><<<dim3(3 * L.grid_chunks, a->H), 256, tcs::CHUNK2_SMEM, st>>>(maps, p);
    }
    QPAM_LAUNCH_CHECK("k_tc_chunk<dq,dv,dk>");
    tcs::k_tc_dgamma_finalize<<<dim3(L.grid_chunks, a->H), 128, 0, st>>>(p, anchors);
    QPAM_LAUNCH_CHECK("k_tc_dgamma_finalize");
  }
  return QPAM_OK;
}

template <int D, typename T>
static int scan_bwd_t(const qpam_scan_args* a, const ScanLayout& L, const void* dy, void* dq, void* dk,
                      void* dv, float* dgamma, float* dcoef, const float* ds_final, float* ds0,
                      int states_valid, cudaStream_t st) {
  ScanParams p = make_params(a, L);
  p.dy = dy; p.dq = dq; p.dk = dk; p.dv = dv;
  p.dgamma = dgamma; p.dcoef = dcoef; p.ds_final = ds_final; p.ds0 = ds0;
  int rc;
  if (!states_valid) {
    ScanParams pf = p;
    pf.s_final = nullptr;
    rc = launch_states<D, T>(pf, L, a, st);
    if (rc) return rc;
  }
  if (L.grid_chunks > 0) {
    auto kern = k_chunk_outer<D, T, true>;
    rc = set_smem(kern, outer_smem<D>());
    if (rc) return rc;
    kern<<<dim3(L.grid_chunks, a->H, a->K), NT, outer_smem<D>(), st>>>(p);
    QPAM_LAUNCH_CHECK("k_chunk_outer<dstate>");
  }
  const int n4 = D * D / 2;
  k_state_scan<true><<<dim3(a->S, a->H * a->K, (n4 + 255) / 256), 256, 0, st>>>(p, D);
  QPAM_LAUNCH_CHECK("k_state_scan<rev>");
  if (L.grid_chunks > 0) {
    auto kern = k_bwd_chunk<D, T>;
    rc = set_smem(kern, bwd_chunk_smem<D>());
    if (rc) return rc;
    kern<<<dim3(L.grid_chunks, a->H), NT, bwd_chunk_smem<D>(), st>>>(p);
    QPAM_LAUNCH_CHECK("k_bwd_chunk");
    k_dgamma_finalize<<<dim3(a->S, a->H, a->K), 256, 0, st>>>(p, D);
    QPAM_LAUNCH_CHECK("k_dgamma_finalize");
  }
  return QPAM_OK;
}

}  // namespace qpam

namespace qpam {
// one thread waits on an mbarrier nobody arrives at, with a short limit: exercises the give-up path of every
// bounded wait (status word, return) without hanging anything
__global__ void k_wait_selftest(unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    umma::mbar_init(&bar, 1);
    umma::fence_barrier_init();
    umma::mbar_wait(&bar, 0, QPAM_DEV_WAIT_SELFTEST, limit_ns);
  }
}
int scan_tc_device_status(int* value, bool clear) {
  QPAM_CUDA(umma::read_device_error(value, clear));
  return QPAM_OK;
}
}  // namespace qpam

using namespace qpam;

extern "C" int qpam_selftest_wait_expiry(int64_t limit_ns, void* stream) {
  QPAM_REQUIRE(limit_ns > 0 && limit_ns <= 100000000, "wait self-test: limit_ns=%lld outside (0, 1e8]", (long long)limit_ns);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  k_wait_selftest<<<1, 32, 0, st>>>((unsigned long long)limit_ns);
  QPAM_LAUNCH_CHECK("k_wait_selftest");
  return QPAM_OK;
}

extern "C" size_t qpam_scan_workspace_bytes(const qpam_scan_args* a, int32_t with_backward) {
  if (a == nullptr || a->d <= 0 || a->K <= 0 || a->H <= 0 || a->S <= 0 || a->T < 0) return 0;
  const ScanLayout L = scan_layout(a, CH);  // the 64-token layout is the larger one
  return with_backward ? L.total_bwd : L.total_fwd;
}

#define QPAM_DISPATCH_SCAN(FN, ...)                                                      \
  do {                                                                                   \
    const bool bf = a->io_dtype == QPAM_BF16;                                            \
    switch (a->d) {                                                                      \
      case 16: return bf ? FN<16, __nv_bfloat16>(__VA_ARGS__) : FN<16, float>(__VA_ARGS__); \
      case 32: return bf ? FN<32, __nv_bfloat16>(__VA_ARGS__) : FN<32, float>(__VA_ARGS__); \
      default: return bf ? FN<64, __nv_bfloat16>(__VA_ARGS__) : FN<64, float>(__VA_ARGS__); \
    }                                                                                    \
  } while (0)

static int scan_fwd_any(const qpam_scan_args* a, void* stream, bool token_major) {
  int rc = check_scan_args(a);
  if (rc) return rc;
  const ScanLayout L = scan_layout(a, fwd_chunk_len(a));
  if (a->workspace_bytes < L.total_fwd) {
    set_error("scan fwd: workspace %zu bytes < required %zu", a->workspace_bytes, L.total_fwd);
    return QPAM_EWORKSPACE;
  }
  QPAM_REQUIRE(a->y != nullptr || a->s_final != nullptr, "scan fwd: both y and s_final are NULL");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (L.ch == tcs::TC) return tc_fwdK_eligible(a) ? scan_fwd_tcK(a, L, st, token_major) : scan_fwd_tc(a, L, st, token_major);
  if (token_major) {
    set_error("scan fwd: the token-major output exists on the tensor-core path only (bf16, d = 64)");
    return QPAM_EUNSUPPORTED;
  }
  QPAM_DISPATCH_SCAN(scan_fwd_t, a, L, st);
}

extern "C" int qpam_scan_fwd(const qpam_scan_args* a, void* stream) { return scan_fwd_any(a, stream, false); }

extern "C" int qpam_scan_fwd_tokens(const qpam_scan_args* a, void* stream) { return scan_fwd_any(a, stream, true); }

extern "C" int qpam_scan_bwd(const qpam_scan_args* a, const void* dy, void* dq, void* dk, void* dv,
                             float* dgamma, float* dcoef, const float* ds_final, float* ds0,
                             int32_t states_valid, void* stream) {
  int rc = check_scan_args(a);
  if (rc) return rc;
  QPAM_REQUIRE(dy && dq && dk && dv && dgamma, "scan bwd: dy/dq/dk/dv/dgamma must not be NULL");
  QPAM_REQUIRE(dcoef == nullptr || a->coef != nullptr, "scan bwd: dcoef requested but coef is NULL");
  const bool tc_bwd = tc_fwd_eligible(a) && a->T > 0 && dcoef == nullptr &&
                      (((uintptr_t)dy | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv) & 15) == 0;
  const ScanLayout L = scan_layout(a, tc_bwd ? tcs::TC : CH);
  if (fwd_chunk_len(a) != L.ch) states_valid = 0;  // the forward left states of another chunking
  if (a->workspace_bytes < L.total_bwd) {
    set_error("scan bwd: workspace %zu bytes < required %zu", a->workspace_bytes, L.total_bwd);
    return QPAM_EWORKSPACE;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tc_bwd) return scan_bwd_tc(a, L, dy, dq, dk, dv, dgamma, ds_final, ds0, states_valid, st);
  QPAM_DISPATCH_SCAN(scan_bwd_t, a, L, dy, dq, dk, dv, dgamma, dcoef, ds_final, ds0, states_valid, st);
}

// The same backward with dq, dk, dv ADDED to what the buffers hold: the K phase-routed states of a layer are K
// scans over the same q, k, v, and their gradients sum.  Tensor-core path only (one state per call).
extern "C" int qpam_scan_bwd_accumulate(const qpam_scan_args* a, const void* dy, void* dq, void* dk, void* dv,
                                        float* dgamma, const float* ds_final, float* ds0, int32_t states_valid,
                                        void* stream) {
  int rc = check_scan_args(a);
  if (rc) return rc;
  QPAM_REQUIRE(dy && dq && dk && dv && dgamma, "scan bwd: dy/dq/dk/dv/dgamma must not be NULL");
  const bool tc_bwd = tc_fwd_eligible(a) && a->T > 0 &&
                      (((uintptr_t)dy | (uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv) & 15) == 0;
  if (!tc_bwd) {
    set_error("scan bwd (accumulate): offered on the tensor-core path only (bf16, d = 64, one state, 16-byte aligned tensors)");
    return QPAM_EUNSUPPORTED;
  }
  const ScanLayout L = scan_layout(a, tcs::TC);
  if (fwd_chunk_len(a) != L.ch) states_valid = 0;
  if (a->workspace_bytes < L.total_bwd) {
    set_error("scan bwd: workspace %zu bytes < required %zu", a->workspace_bytes, L.total_bwd);
    return QPAM_EWORKSPACE;
  }
  return scan_bwd_tc(a, L, dy, dq, dk, dv, dgamma, ds_final, ds0, states_valid, reinterpret_cast<cudaStream_t>(stream), true);
}

// K = 2..4 states for training (tensor-core path only): per-state outputs ys [K,B,H,T,d,2] and s_final, the state
// sums shared between the states; the workspace keeps every state's chunk states for qpam_scan_bwd_state.
extern "C" int qpam_scan_fwd_states(const qpam_scan_args* a, void* ys, void* stream) {
  int rc = check_scan_args(a);
  if (rc) return rc;
  QPAM_REQUIRE(ys != nullptr && ((uintptr_t)ys & 15) == 0, "scan fwd (states): ys must be a 16-byte aligned buffer");
  qpam_scan_args probe = *a;
  probe.y = ys;
  probe.coef = nullptr;
  if (!tc_fwdK_eligible(&probe)) {
    set_error("scan fwd (states): offered on the tensor-core path only (bf16, d = 64, 2..4 states, 16-byte aligned tensors)");
    return QPAM_EUNSUPPORTED;
  }
  const ScanLayout L = scan_layout(a, tcs::TC);
  if (a->workspace_bytes < L.total_fwd) {
    set_error("scan fwd (states): workspace %zu bytes < required %zu", a->workspace_bytes, L.total_fwd);
    return QPAM_EWORKSPACE;
  }
  return scan_fwd_tc_states(a, L, ys, reinterpret_cast<cudaStream_t>(stream));
}

// Backward of state `state` of a qpam_scan_fwd_states call (same args, same workspace): dy is that state's output
// gradient, dgamma / ds_final / ds0 that state's arrays; accumulate != 0 adds dq, dk, dv to what the buffers hold.
extern "C" int qpam_scan_bwd_state(const qpam_scan_args* a, int32_t state, const void* dy, void* dq, void* dk, void* dv,
                                   float* dgamma, const float* ds_final, float* ds0, int32_t accumulate, void* stream) {
  int rc = check_scan_args(a);
  if (rc) return rc;
  QPAM_REQUIRE(dy && dq && dk && dv && dgamma, "scan bwd (state): dy/dq/dk/dv/dgamma must not be NULL");
  QPAM_REQUIRE(state >= 0 && state < a->K, "scan bwd (state): state %d outside [0,%d)", state, a->K);
  qpam_scan_args probe = *a;
  probe.y = const_cast<void*>(dy);
  probe.coef = nullptr;
  if (!tc_fwdK_eligible(&probe) || a->T <= 0 || (((uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv) & 15) != 0) {
    set_error("scan bwd (state): offered on the tensor-core path only (bf16, d = 64, 2..4 states, 16-byte aligned tensors)");
    return QPAM_EUNSUPPORTED;
  }
  const ScanLayout L = scan_layout(a, tcs::TC);
  if (a->workspace_bytes < L.total_bwd) {
    set_error("scan bwd (state): workspace %zu bytes < required %zu", a->workspace_bytes, L.total_bwd);
    return QPAM_EWORKSPACE;
  }
  return scan_bwd_tc(a, L, dy, dq, dk, dv, dgamma, ds_final, ds0, 1, reinterpret_cast<cudaStream_t>(stream),
                     accumulate != 0, state);
}

// ---------------------------------------------------------------------------------------------
// Forward scan for callers that cannot allocate device memory.
//
// Some hosts hand the whole GPU to one memory pool at start-up (an inference server, a plugin
// sandbox) or run a latency-critical loop in which cudaMalloc -- which may synchronise the
// device -- is off limits.  Such a caller has nowhere to get the scan's workspace from.  This
// entry point keeps that workspace in a fixed array that is part of the library image itself.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_scan_static_scratch[QPAM_STATIC_SCRATCH_BYTES];

namespace qpam {
static std::mutex g_static_mu;
static void* g_static_ptr[64] = {nullptr};  // device address of the array, per device ordinal
}  // namespace qpam

extern "C" int qpam_scan_fwd_static(const qpam_scan_args* a, void* stream) {
  QPAM_REQUIRE(a != nullptr, "scan (static scratch): args is NULL");
  int dev = -1;
  QPAM_CUDA(cudaGetDevice(&dev));
  QPAM_REQUIRE(dev >= 0 && dev < 64, "scan (static scratch): device ordinal %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
      // In host code the array's name is only a handle; the kernels need its device address.
      void* ptr = nullptr;
      QPAM_CUDA(cudaGetSymbolAddress(&ptr, g_scan_static_scratch));
      g_static_ptr[dev] = ptr;
    }
    scratch = g_static_ptr[dev];
  }
  qpam_scan_args b = *a;
  b.workspace = scratch;
  b.workspace_bytes = QPAM_STATIC_SCRATCH_BYTES;
  int rc = check_scan_args(&b);
  if (rc) return rc;
  const ScanLayout L = scan_layout(&b, CH);
  if (L.total_fwd > (size_t)QPAM_STATIC_SCRATCH_BYTES) {
    set_error("scan (static scratch): this shape needs %zu bytes of workspace, the built-in scratch holds %zu; "
              "use qpam_scan_fwd with a caller-provided workspace", L.total_fwd, (size_t)QPAM_STATIC_SCRATCH_BYTES);
    return QPAM_EWORKSPACE;
  }
  return qpam_scan_fwd(&b, stream);
}
