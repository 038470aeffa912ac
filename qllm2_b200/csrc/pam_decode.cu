// O(1)-per-token recurrent PAM step over a pool of per-sequence state slots.
//
// HBM-bound: per (sequence, head, state) the kernel streams a d x d complex matrix in and out
// once (2 * d*d*2*sizeof(state) bytes) for ~22 d^2 flops.  Each thread owns 16-byte pieces of
// state rows (128-bit coalesced loads/stores, a row is covered by consecutive lanes), all loads of
// a state are issued before the first use, and the read-out y = S q is finished with warp
// shuffles.  Continuous batching: `slot_ids` picks the slot of every live sequence, so sequences
// join and leave by editing that index vector only.
#include "common.cuh"
#include "umma.cuh"

namespace qpam {

template <typename ST>
struct StateVec;
template <>
struct StateVec<float> {
  static constexpr int NC = 2;  // complex entries per 16-byte vector
  static __device__ __forceinline__ void load(const float* p, float2 (&o)[NC]) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(p));
    o[0] = make_float2(v.x, v.y);
    o[1] = make_float2(v.z, v.w);
  }
  static __device__ __forceinline__ void store(float* p, const float2 (&o)[NC]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(o[0].x, o[0].y, o[1].x, o[1].y));
  }
};
template <>
struct StateVec<__nv_bfloat16> {
  static constexpr int NC = 4;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float2 (&o)[NC]) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < NC; ++i) o[i] = __bfloat1622float2(b[i]);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float2 (&o)[NC]) {
    uint4 v;
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < NC; ++i) b[i] = __float22bfloat162_rn(o[i]);
    __stcs(reinterpret_cast<uint4*>(p), v);
  }
};

struct DecodeParams {
  void* pool;
  const int32_t* slot_ids;
  const void *q, *k, *v;
  const float* gamma;  // [K,n,H]
  const float* coef;   // [K,n,H,2] or null
  void* y;
  int64_t n_slots;
  int32_t L, layer, n, H, K;
};

// grid = n*H CTAs; block = min(256, D*D/NC) threads.
template <int D, typename ST, typename T>
__global__ void __launch_bounds__(256) k_decode_step(DecodeParams p) {
  constexpr int NC = StateVec<ST>::NC;
  constexpr int LPR = D / NC;                                  // lanes per state row
  constexpr int NTH = (D * D / NC) < 256 ? (D * D / NC) : 256;  // threads
  constexpr int RPP = NTH / LPR;                               // rows per pass
  constexpr int PASSES = D / RPP;
  __shared__ float2 sq[D], sk[D], sv[D];
  const int tid = threadIdx.x;
  const int seq = blockIdx.x / p.H, h = blockIdx.x - seq * p.H;
  const int slot = p.slot_ids[seq];
  if (slot < 0 || slot >= p.n_slots) return;  // padded / retired entry: nothing to do
  const size_t vb = ((size_t)seq * p.H + h) * D * 2;
  if (tid < D) {
    sq[tid] = IO<T>::ld2(reinterpret_cast<const T*>(p.q) + vb + 2 * tid);
    sk[tid] = IO<T>::ld2(reinterpret_cast<const T*>(p.k) + vb + 2 * tid);
    sv[tid] = IO<T>::ld2(reinterpret_cast<const T*>(p.v) + vb + 2 * tid);
  }
  __syncthreads();
  const int row0 = tid / LPR, j0 = (tid % LPR) * NC;
  float2 kq[NC], qq[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    kq[c] = sk[j0 + c];
    qq[c] = sq[j0 + c];
  }
  float2 yacc[PASSES];
#pragma unroll
  for (int r = 0; r < PASSES; ++r) yacc[r] = make_float2(0.f, 0.f);
  for (int k = 0; k < p.K; ++k) {
    ST* S = reinterpret_cast<ST*>(p.pool) +
            ((((size_t)slot * p.L + p.layer) * p.K + k) * p.H + h) * (size_t)(D * D * 2);
    const size_t gi = ((size_t)k * p.n + seq) * p.H + h;
    const float g = p.gamma[gi];
    float2 cf = make_float2(1.f, 0.f);
    if (p.coef != nullptr) cf = *reinterpret_cast<const float2*>(p.coef + gi * 2);
    float2 s[PASSES][NC];
#pragma unroll
    for (int r = 0; r < PASSES; ++r) StateVec<ST>::load(S + ((size_t)(row0 + r * RPP) * D + j0) * 2, s[r]);
#pragma unroll
    for (int r = 0; r < PASSES; ++r) {
      const float2 vi = sv[row0 + r * RPP];
      float2 part = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const float2 o = cmulc(vi, kq[c]);  // v_i conj(k_j)
        s[r][c].x = fmaf(g, s[r][c].x, o.x);
        s[r][c].y = fmaf(g, s[r][c].y, o.y);
        cfma<false, false>(part, s[r][c], qq[c]);
      }
      StateVec<ST>::store(S + ((size_t)(row0 + r * RPP) * D + j0) * 2, s[r]);
      const float2 m = cmul(cf, part);
      yacc[r].x += m.x;
      yacc[r].y += m.y;
    }
  }
#pragma unroll
  for (int r = 0; r < PASSES; ++r) {
    float2 a = yacc[r];
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
      a.x += __shfl_xor_sync(0xffffffffu, a.x, o);
      a.y += __shfl_xor_sync(0xffffffffu, a.y, o);
    }
    if ((tid % LPR) == 0) IO<T>::st2(reinterpret_cast<T*>(p.y) + vb + 2 * (row0 + r * RPP), a);
  }
}

// ------------------------------------------------------------------------------------------------
// bf16 state, d = 64: the K states of one (sequence, head) are 16 KB each.  They are brought into
// shared memory by bulk copies issued up front by one thread (all K in flight at once, independent of
// the register file), updated in place there, and written back by bulk copies.  With ~50 KB per CTA
// four CTAs fit on an SM, i.e. ~190 KB of loads in flight per SM.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(umma::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(umma::smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :
               : "l"(reinterpret_cast<uint64_t>(gdst)), "r"(umma::smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

constexpr int DEC_BULK_STATE_BYTES = 64 * 64 * 2 * 2;  // one bf16 state

template <typename T>
__global__ void __launch_bounds__(256) k_decode_step_bulk(DecodeParams p) {
  constexpr int D = 64, NC = 4, LPR = D / NC, RPP = 256 / LPR, PASSES = D / RPP;
  extern __shared__ __align__(128) unsigned char dec_smem[];
  __shared__ float2 sq[D], sk[D], sv[D];
  __shared__ __align__(8) uint64_t bar[QPAM_MAX_STATES];   // one per state: work on state k starts when it has landed
  const int tid = threadIdx.x;
  const int seq = blockIdx.x / p.H, h = blockIdx.x - seq * p.H;
  const int slot = p.slot_ids[seq];
  if (slot < 0 || slot >= p.n_slots) return;  // padded / retired entry: nothing to do (whole CTA)
  __nv_bfloat16* pool = reinterpret_cast<__nv_bfloat16*>(p.pool);
  const size_t state_elems = (size_t)D * D * 2;
  const size_t base = (((size_t)slot * p.L + p.layer) * p.K) * p.H + h;  // + k * H per state
  if (tid == 0) {
    for (int k = 0; k < p.K; ++k) umma::mbar_init(&bar[k], 1);
    umma::fence_barrier_init();
    for (int k = 0; k < p.K; ++k) {
      umma::mbar_arrive_expect_tx(&bar[k], (uint32_t)DEC_BULK_STATE_BYTES);
      bulk_load(dec_smem + (size_t)k * DEC_BULK_STATE_BYTES, pool + (base + (size_t)k * p.H) * state_elems,
                DEC_BULK_STATE_BYTES, &bar[k]);
    }
  }
  const size_t vb = ((size_t)seq * p.H + h) * D * 2;
  if (tid < D) {
    sq[tid] = IO<T>::ld2(reinterpret_cast<const T*>(p.q) + vb + 2 * tid);
    sk[tid] = IO<T>::ld2(reinterpret_cast<const T*>(p.k) + vb + 2 * tid);
    sv[tid] = IO<T>::ld2(reinterpret_cast<const T*>(p.v) + vb + 2 * tid);
  }
  __syncthreads();  // also publishes the barriers' initialisation to the waiters
  bool arrived = true;
  const int row0 = tid / LPR, j0 = (tid % LPR) * NC;
  float2 kq[NC], qq[NC], yacc[PASSES];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    kq[c] = sk[j0 + c];
    qq[c] = sq[j0 + c];
  }
#pragma unroll
  for (int r = 0; r < PASSES; ++r) yacc[r] = make_float2(0.f, 0.f);
  {
    for (int k = 0; k < p.K; ++k) {
      // on a give-up the error word is set and the arithmetic below is skipped; the barriers are not
      arrived = umma::mbar_wait(&bar[k], 0, 31) && arrived;
      __nv_bfloat16* S = reinterpret_cast<__nv_bfloat16*>(dec_smem + (size_t)k * DEC_BULK_STATE_BYTES);
      const size_t gi = ((size_t)k * p.n + seq) * p.H + h;
      const float g = p.gamma[gi];
      float2 cf = make_float2(1.f, 0.f);
      if (p.coef != nullptr) cf = *reinterpret_cast<const float2*>(p.coef + gi * 2);
#pragma unroll
      for (int r = 0; r < PASSES; ++r) {
        if (!arrived) break;
        const int row = row0 + r * RPP;
        uint4* cell = reinterpret_cast<uint4*>(S + ((size_t)row * D + j0) * 2);
        uint4 raw = *cell;
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&raw);
        const float2 vi = sv[row];
        float2 part = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float2 e = __bfloat1622float2(b[c]);
          const float2 o = cmulc(vi, kq[c]);  // v_i conj(k_j)
          e.x = fmaf(g, e.x, o.x);
          e.y = fmaf(g, e.y, o.y);
          cfma<false, false>(part, e, qq[c]);
          b[c] = __float22bfloat162_rn(e);
        }
        *cell = raw;
        const float2 m = cmul(cf, part);
        yacc[r].x += m.x;
        yacc[r].y += m.y;
      }
      umma::fence_proxy_async();  // the bulk store below reads what the generic proxy just wrote
      __syncthreads();
      if (tid == 0 && arrived) {    // state k goes back while state k+1 is being updated
        bulk_store(pool + (base + (size_t)k * p.H) * state_elems, dec_smem + (size_t)k * DEC_BULK_STATE_BYTES,
                   DEC_BULK_STATE_BYTES);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
  }
  if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the copies
#pragma unroll
  for (int r = 0; r < PASSES; ++r) {
    float2 a = yacc[r];
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
      a.x += __shfl_xor_sync(0xffffffffu, a.x, o);
      a.y += __shfl_xor_sync(0xffffffffu, a.y, o);
    }
    if ((tid % LPR) == 0) IO<T>::st2(reinterpret_cast<T*>(p.y) + vb + 2 * (row0 + r * RPP), a);
  }
}

template <typename T>
static int launch_decode_bulk(const DecodeParams& p, cudaStream_t st) {
  const size_t smem = (size_t)p.K * DEC_BULK_STATE_BYTES;
  auto kern = k_decode_step_bulk<T>;
  QPAM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<p.n * p.H, 256, smem, st>>>(p);
  QPAM_LAUNCH_CHECK("k_decode_step_bulk");
  return QPAM_OK;
}

int decode_device_status(int* value, bool clear) {
  QPAM_CUDA(umma::read_device_error(value, clear));
  return QPAM_OK;
}

template <int D, typename ST, typename T>
static int launch_decode(const DecodeParams& p, cudaStream_t st) {
  constexpr int NC = StateVec<ST>::NC;
  constexpr int NTH = (D * D / NC) < 256 ? (D * D / NC) : 256;
  k_decode_step<D, ST, T><<<p.n * p.H, NTH, 0, st>>>(p);
  QPAM_LAUNCH_CHECK("k_decode_step");
  return QPAM_OK;
}

template <typename ST>
__global__ void k_pool_store(ST* pool, const int32_t* slot_ids, const float* states, int64_t n_slots, int L,
                             int layer, int S, int H, int K, int dd2) {
  // one CTA per (k, s, h); states [K,S,H,dd2] -> pool[slot, layer, k, h, dd2]
  const int h = blockIdx.x % H, s = (blockIdx.x / H) % S, k = blockIdx.x / (H * S);
  const int slot = slot_ids[s];
  if (slot < 0 || slot >= n_slots) return;
  const float* src = states + (((size_t)k * S + s) * H + h) * dd2;
  ST* dst = pool + ((((size_t)slot * L + layer) * K + k) * H + h) * (size_t)dd2;
  for (int e = threadIdx.x; e < dd2; e += blockDim.x) IO<ST>::st(dst + e, src[e]);
}

}  // namespace qpam

using namespace qpam;

extern "C" int qpam_decode_step(void* state_pool, int32_t state_dtype, int64_t n_slots, int32_t L,
                                int32_t layer, const int32_t* slot_ids, const void* q, const void* k,
                                const void* v, const float* gamma, const float* coef, void* y, int32_t n,
                                int32_t H, int32_t d, int32_t K, int32_t io_dtype, void* stream) {
  QPAM_REQUIRE(state_pool && slot_ids && q && k && v && gamma && y, "decode: NULL pointer argument");
  QPAM_REQUIRE(d == 16 || d == 32 || d == 64, "decode: head dim d=%d not in {16,32,64}", d);
  QPAM_REQUIRE(K >= 1 && K <= QPAM_MAX_STATES, "decode: K=%d outside [1,%d]", K, QPAM_MAX_STATES);
  QPAM_REQUIRE(n >= 0 && H >= 1 && L >= 1 && layer >= 0 && layer < L, "decode: bad n/H/L/layer");
  QPAM_REQUIRE(state_dtype == QPAM_F32 || state_dtype == QPAM_BF16, "decode: state_dtype %d unknown", state_dtype);
  QPAM_REQUIRE(io_dtype == QPAM_F32 || io_dtype == QPAM_BF16, "decode: io_dtype %d unknown", io_dtype);
  QPAM_REQUIRE(((uintptr_t)state_pool & 15) == 0, "decode: state_pool must be 16-byte aligned");
  if (n == 0) return QPAM_OK;
  DecodeParams p{state_pool, slot_ids, q, k, v, gamma, coef, y, n_slots, L, layer, n, H, K};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (d == 64 && state_dtype == QPAM_BF16)   // shared-memory staged variant (bulk copies)
    return io_dtype == QPAM_F32 ? launch_decode_bulk<float>(p, st) : launch_decode_bulk<__nv_bfloat16>(p, st);
#define QPAM_DEC(DD)                                                                          \
  if (state_dtype == QPAM_F32)                                                                \
    return io_dtype == QPAM_F32 ? launch_decode<DD, float, float>(p, st)                      \
                                : launch_decode<DD, float, __nv_bfloat16>(p, st);             \
  return io_dtype == QPAM_F32 ? launch_decode<DD, __nv_bfloat16, float>(p, st)                \
                              : launch_decode<DD, __nv_bfloat16, __nv_bfloat16>(p, st);
  if (d == 16) { QPAM_DEC(16) }
  if (d == 32) { QPAM_DEC(32) }
  QPAM_DEC(64)
#undef QPAM_DEC
}

extern "C" int qpam_pool_store(void* state_pool, int32_t state_dtype, int64_t n_slots, int32_t L,
                               int32_t layer, const int32_t* slot_ids, const float* states, int32_t S,
                               int32_t H, int32_t d, int32_t K, void* stream) {
  QPAM_REQUIRE(state_pool && slot_ids && states, "pool_store: NULL pointer argument");
  QPAM_REQUIRE(S >= 0 && H >= 1 && K >= 1 && d >= 1 && L >= 1 && layer >= 0 && layer < L, "pool_store: bad sizes");
  QPAM_REQUIRE(state_dtype == QPAM_F32 || state_dtype == QPAM_BF16, "pool_store: state_dtype %d unknown", state_dtype);
  if (S == 0) return QPAM_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int dd2 = d * d * 2;
  if (state_dtype == QPAM_F32)
    k_pool_store<float><<<K * S * H, 256, 0, st>>>(reinterpret_cast<float*>(state_pool), slot_ids, states, n_slots, L, layer, S, H, K, dd2);
  else
    k_pool_store<__nv_bfloat16><<<K * S * H, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(state_pool), slot_ids, states, n_slots, L, layer, S, H, K, dd2);
  QPAM_LAUNCH_CHECK("k_pool_store");
  return QPAM_OK;
}
