// Token sampling on the device: temperature, repetition penalty, top-k, top-p (nucleus) and the draw itself,
// one CTA per row of logits, no sort and no host round trip.  Semantics of the reference's sampling block
// (v11/model.py:1221-1244):
//   x = logits / temperature
//   x[h] = x[h] > 0 ? x[h] / penalty : x[h] * penalty          for every token h already in the sequence
//   top-k : drop x < (k-th largest x)                            (ties with the k-th value stay)
//   top-p : in descending order, drop a token when the probability mass BEFORE it is >= top_p
//   draw from softmax of what is left
// The row lives in shared memory (V <= ~56k floats) or in a caller workspace; the k-th largest value and the
// nucleus threshold are found without sorting: the k-th largest value by radix selection over order-preserving
// integer keys (4 passes of 8 bits over count histograms), the nucleus threshold by a 4-way search over the bit
// patterns of the unnormalised probabilities (each probe a deterministic block reduction); the draw is the inverse
// CDF in vocabulary order of a uniform number the caller supplies.  Nothing depends on the order of atomics, so the
// same inputs give the same token on every run.  Tokens that tie with the nucleus threshold are all kept (a sort would keep an arbitrary
// subset of them).
#include "common.cuh"

namespace qpam {
namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_SMEM_EXTRA = 12288;  // histograms, scan scratch, scalars, compact list of the top-k survivors
constexpr int SAMPLE_COMPACT = 1024;       // survivors of top-k that the later stages handle one per thread

struct SampleParams {
  const void* logits;
  int64_t ldl;
  const int32_t* slot_ids;
  int64_t* history;
  int64_t ld_hist;
  int32_t* hist_len;
  const float* uniforms;
  int64_t* next_ids;
  float* stats;
  float* work;
  int32_t n, V, n_hist_rows, hist_cols, top_k, append, row_in_smem;
  float inv_temperature, top_p, penalty;
};

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Histogram update of a whole warp (every lane calls; bin < 0 = this lane adds nothing).  Lanes that hit the same
// bin are combined before the shared-memory atomic, so a row whose keys share their leading bits (the usual case
// at the first radix level) does not serialise 32 ways on one address.
__device__ __forceinline__ void warp_hist_count(uint32_t* hist, int bin) {
  const unsigned peers = __match_any_sync(0xffffffffu, bin);
  if (bin >= 0 && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
}

struct Scratch {
  uint32_t count[256];
  float mass[256];
  float warp_f[32];
  float bcast_f[4];
  uint32_t prefix;
  uint32_t remaining;
  int chosen;
  int last_kept;
};

__device__ __forceinline__ float block_max(float v, Scratch* sc) {
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sc->warp_f[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sc->warp_f[threadIdx.x & 31];
  for (int o = 16; o; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

__device__ __forceinline__ float block_sum(float v, Scratch* sc) {
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sc->warp_f[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sc->warp_f[threadIdx.x & 31];
  for (int o = 16; o; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

// exclusive prefix of v over the block (thread order); *total = sum over the block
__device__ __forceinline__ float block_exclusive_scan(float v, Scratch* sc, float* total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  float inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) sc->warp_f[w] = inc;
  __syncthreads();
  float ws = sc->warp_f[lane];
  float winc = ws;
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += t;
  }
  const float before_warp = __shfl_sync(0xffffffffu, winc - ws, w);
  *total = __shfl_sync(0xffffffffu, winc, 31);
  return before_warp + inc - v;
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS) k_sample_rows(SampleParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Scratch* sc = reinterpret_cast<Scratch*>(smem_raw);
  const int row = blockIdx.x, tid = threadIdx.x, V = p.V;
  float* w = p.row_in_smem ? reinterpret_cast<float*>(smem_raw + SAMPLE_SMEM_EXTRA) : p.work + (size_t)row * V;
  const T* lg = reinterpret_cast<const T*>(p.logits) + (size_t)row * p.ldl;

  int hrow = -1;
  if (p.history) {
    hrow = p.slot_ids ? p.slot_ids[row] : row;
    if (hrow < 0 || hrow >= p.n_hist_rows) hrow = -1;
  }
  if (p.slot_ids && hrow < 0 && p.history) {  // padded row of a captured batch: nothing to draw
    if (tid == 0) p.next_ids[row] = 0;
    return;
  }

  for (int i = tid; i < V; i += SAMPLE_THREADS) w[i] = IO<T>::ld(lg + i) * p.inv_temperature;
  __syncthreads();
  int hlen = 0;
  if (hrow >= 0) {
    hlen = p.hist_len ? p.hist_len[hrow] : p.hist_cols;
    hlen = max(0, min(hlen, p.hist_cols));
    if (p.penalty != 1.0f) {
      const int64_t* hist = p.history + (size_t)hrow * p.ld_hist;
      for (int j = tid; j < hlen; j += SAMPLE_THREADS) {
        const int64_t h = hist[j];
        if (h >= 0 && h < V) {
          const float x = IO<T>::ld(lg + h) * p.inv_temperature;  // from the ORIGINAL value: repeats write the same
          w[h] = x > 0.f ? x / p.penalty : x * p.penalty;
        }
      }
    }
  }
  __syncthreads();

  // ---- top-k: key of the k-th largest value (0 keeps everything)
  uint32_t key_k = 0;
  if (p.top_k > 0 && p.top_k < V) {
    if (tid == 0) { sc->prefix = 0; sc->remaining = (uint32_t)p.top_k; }
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) sc->count[tid] = 0;
      __syncthreads();
      const uint32_t prefix = sc->prefix;
      const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int base = 0; base < V; base += SAMPLE_THREADS) {
        const int i = base + tid;
        const uint32_t key = i < V ? order_key(w[i]) : 0u;
        const bool in = i < V && (key & himask) == prefix;
        if (__ballot_sync(0xffffffffu, in) == 0u) continue;     // below the first level few warps hold a candidate
        // first level: few distinct leading bytes, lanes are combined; deeper levels spread over the bins
        if (shift == 24) warp_hist_count(sc->count, in ? (int)((key >> shift) & 255u) : -1);
        else if (in) atomicAdd(&sc->count[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid < 32) {  // warp 0: lane l owns bins 255-8l .. 248-8l (descending order of keys)
        const uint32_t rem = sc->remaining;
        const int top = 255 - 8 * tid;
        uint32_t mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += sc->count[top - j];
        uint32_t inc = mine;
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
          if (tid >= o) inc += t;
        }
        const uint32_t before = inc - mine;
        const unsigned hit = __ballot_sync(0xffffffffu, before < rem && rem <= inc);
        const int owner = hit ? __ffs(hit) - 1 : 31;
        if (tid == owner) {
          uint32_t cum = before;
          int b = top;
          for (; b > top - 7; --b) {
            if (cum + sc->count[b] >= rem) break;
            cum += sc->count[b];
          }
          sc->remaining = rem - cum;
          sc->prefix = prefix | ((uint32_t)b << shift);
        }
      }
      __syncthreads();
    }
    key_k = sc->prefix;
  }

  // ---- what top-k left, as unnormalised probabilities e = exp(x - max) in place of the logits (0 = dropped).
  // e is monotone in x, and for non-negative floats the bit pattern orders like the value.
  float mx = -INFINITY;
  for (int i = tid; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, w[i]);
  mx = block_max(mx, sc);
  float z = 0.f;
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    const float x = w[i];
    const float e = order_key(x) >= key_k ? __expf(x - mx) : 0.f;
    w[i] = e;
    z += e;
  }
  z = block_sum(z, sc);

  // ---- a short list of survivors (top-k with a small k): the nucleus search and the draw then touch one element
  // per thread instead of the whole row.  The list keeps vocabulary order.
  float* cval = reinterpret_cast<float*>(smem_raw + sizeof(Scratch));
  int* cidx = reinterpret_cast<int*>(cval + SAMPLE_COMPACT);
  const float* ev = w;
  int n_el = V;
  if (p.top_k > 0 && p.top_k <= SAMPLE_COMPACT / 2 && p.top_k < V) {
    const int per_v = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int a0 = min(V, tid * per_v), a1 = min(V, a0 + per_v);
    int c = 0;
    for (int i = a0; i < a1; ++i) c += w[i] > 0.f ? 1 : 0;
    float tot;
    const int at = (int)block_exclusive_scan((float)c, sc, &tot);      // counts <= V: exact in float
    if ((int)tot <= SAMPLE_COMPACT) {                                    // block-uniform
      int o = at;
      for (int i = a0; i < a1; ++i) {
        const float e = w[i];
        if (e > 0.f) {
          cval[o] = e;
          cidx[o] = i;
          ++o;
        }
      }
      ev = cval;
      n_el = (int)tot;
      __syncthreads();
    }
  }
  const bool compact = ev != w;

  // ---- top-p: the largest threshold t (as a bit pattern) with mass{e >= t} >= top_p * z, i.e. the value at which
  // the descending cumulative mass first reaches the target; found by a 4-way search over the bit patterns of
  // (0, 1].  Every probe is one pass with a fixed reduction tree: no atomics, the same result on every run.
  uint32_t bits_min = 1u;                       // keeps every e > 0
  if (p.top_p > 0.f && p.top_p < 1.f && compact && n_el <= 256) {
    // a short list: one warp holds it in registers (eight per lane) and runs the same search with shuffles only
    const float target = p.top_p * z;
    if (tid < 32) {
      float e8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) e8[j] = (tid + 32 * j < n_el) ? ev[tid + 32 * j] : 0.f;
      uint32_t lo = 1u, hi = 0x3f800001u;
      while (hi - lo > 1u) {
        const uint32_t step = (hi - lo) >> 2;
        const uint32_t m2 = lo + ((hi - lo) >> 1);
        const uint32_t m1 = step ? lo + step : m2, m3 = step ? m2 + step : m2;
        float f1 = 0.f, f2 = 0.f, f3 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t eb = __float_as_uint(e8[j]);
          f1 += eb >= m1 ? e8[j] : 0.f;
          f2 += eb >= m2 ? e8[j] : 0.f;
          f3 += eb >= m3 ? e8[j] : 0.f;
        }
        for (int o = 16; o; o >>= 1) {
          f1 += __shfl_xor_sync(0xffffffffu, f1, o);
          f2 += __shfl_xor_sync(0xffffffffu, f2, o);
          f3 += __shfl_xor_sync(0xffffffffu, f3, o);
        }
        if (f3 >= target && m3 > m2) lo = m3;
        else if (f2 >= target) { lo = m2; if (m3 > m2) hi = m3; }
        else if (f1 >= target && m1 < m2) { lo = m1; hi = m2; }
        else hi = (m1 < m2) ? m1 : m2;
      }
      if (tid == 0) sc->prefix = lo;
    }
    __syncthreads();
    bits_min = sc->prefix;
  } else if (p.top_p > 0.f && p.top_p < 1.f) {
    const float target = p.top_p * z;
    uint32_t lo = 1u, hi = 0x3f800001u;         // mass{>= lo} >= target > mass{>= hi}
    while (hi - lo > 1u) {
      const uint32_t step = (hi - lo) >> 2;
      const uint32_t m2 = lo + ((hi - lo) >> 1);
      const uint32_t m1 = step ? lo + step : m2, m3 = step ? m2 + step : m2;
      float f1 = 0.f, f2 = 0.f, f3 = 0.f;
      for (int i = tid; i < n_el; i += SAMPLE_THREADS) {
        const float e = ev[i];
        const uint32_t eb = __float_as_uint(e);
        f1 += eb >= m1 ? e : 0.f;
        f2 += eb >= m2 ? e : 0.f;
        f3 += eb >= m3 ? e : 0.f;
      }
      // one reduction for the three sums
      for (int o = 16; o; o >>= 1) {
        f1 += __shfl_xor_sync(0xffffffffu, f1, o);
        f2 += __shfl_xor_sync(0xffffffffu, f2, o);
        f3 += __shfl_xor_sync(0xffffffffu, f3, o);
      }
      __syncthreads();
      if ((tid & 31) == 0) {
        sc->mass[tid >> 5] = f1;
        sc->mass[32 + (tid >> 5)] = f2;
        sc->mass[64 + (tid >> 5)] = f3;
      }
      __syncthreads();
      f1 = sc->mass[tid & 31];
      f2 = sc->mass[32 + (tid & 31)];
      f3 = sc->mass[64 + (tid & 31)];
      for (int o = 16; o; o >>= 1) {
        f1 += __shfl_xor_sync(0xffffffffu, f1, o);
        f2 += __shfl_xor_sync(0xffffffffu, f2, o);
        f3 += __shfl_xor_sync(0xffffffffu, f3, o);
      }
      if (f3 >= target && m3 > m2) lo = m3;
      else if (f2 >= target) { lo = m2; if (m3 > m2) hi = m3; }
      else if (f1 >= target && m1 < m2) { lo = m1; hi = m2; }
      else hi = (m1 < m2) ? m1 : m2;
    }
    bits_min = lo;
  }

  // ---- the draw: inverse CDF in vocabulary order over the kept tokens
  const int per = (n_el + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int i0 = min(n_el, tid * per), i1 = min(n_el, i0 + per);
  float mine = 0.f;
  int last = -1, cnt = 0;
  for (int i = i0; i < i1; ++i) {
    const float e = ev[i];
    if (__float_as_uint(e) >= bits_min) {
      mine += e;
      last = i;
      ++cnt;
    }
  }
  if (tid == 0) { sc->chosen = -1; sc->last_kept = -1; }
  float total;
  const float before = block_exclusive_scan(mine, sc, &total);
  const float kept = block_sum((float)cnt, sc);
  if (last >= 0) atomicMax(&sc->last_kept, last);
  const float target = p.uniforms[row] * total;
  if (cnt > 0 && before <= target && target < before + mine) {
    float cum = before;
    int pick = last;
    for (int i = i0; i < i1; ++i) {
      const float e = ev[i];
      if (__float_as_uint(e) >= bits_min) {
        cum += e;
        if (cum > target) { pick = i; break; }
      }
    }
    atomicMax(&sc->chosen, pick);
  }
  __syncthreads();
  if (tid == 0) {
    int pick = sc->chosen >= 0 ? sc->chosen : sc->last_kept;
    if (compact) pick = cidx[pick];
    p.next_ids[row] = pick;
    if (p.stats) {
      float* s = p.stats + 4 * (size_t)row;
      s[0] = mx;
      s[1] = total;
      s[2] = kept;
      s[3] = z;
    }
    if (p.append && hrow >= 0 && p.hist_len) {
      const int len = p.hist_len[hrow];
      if (len >= 0 && len < p.hist_cols) {
        p.history[(size_t)hrow * p.ld_hist + len] = pick;
        p.hist_len[hrow] = len + 1;
      }
    }
  }
}

}  // namespace
}  // namespace qpam

using namespace qpam;

extern "C" size_t qpam_sample_workspace_bytes(int32_t n, int32_t V) {
  if (n <= 0 || V <= 0) return 0;
  if ((size_t)V * 4 + SAMPLE_SMEM_EXTRA <= 227u * 1024u) return 0;
  return (size_t)n * V * 4;
}

extern "C" int qpam_sample_logits(const void* logits, int32_t io_dtype, int32_t n, int32_t V, int64_t ld_logits,
                                  float temperature, int32_t top_k, float top_p, float repetition_penalty,
                                  const int32_t* slot_ids, int64_t* history, int32_t n_hist_rows, int32_t hist_cols,
                                  int64_t ld_hist, int32_t* hist_len, int32_t append, const float* uniforms,
                                  int64_t* next_ids, float* stats, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  QPAM_REQUIRE(logits && uniforms && next_ids, "sample: NULL pointer argument");
  QPAM_REQUIRE(io_dtype == QPAM_F32 || io_dtype == QPAM_BF16, "sample: io_dtype %d unknown", io_dtype);
  QPAM_REQUIRE(n >= 0 && V >= 1 && ld_logits >= V, "sample: bad n=%d V=%d ld=%lld", n, V, (long long)ld_logits);
  QPAM_REQUIRE(temperature > 0.f, "sample: temperature must be positive (arg-max decoding is qpam_head_argmax)");
  QPAM_REQUIRE(repetition_penalty > 0.f, "sample: repetition_penalty must be positive");
  QPAM_REQUIRE(top_k >= 0 && top_p >= 0.f, "sample: top_k and top_p must not be negative");
  QPAM_REQUIRE(!history || (n_hist_rows >= 1 && hist_cols >= 0 && ld_hist >= hist_cols), "sample: bad history shape");
  QPAM_REQUIRE(!append || (history && hist_len), "sample: append needs history and hist_len");
  if (n == 0) return QPAM_OK;
  SampleParams p{};
  p.logits = logits; p.ldl = ld_logits; p.slot_ids = slot_ids; p.history = history; p.ld_hist = ld_hist;
  p.hist_len = hist_len; p.uniforms = uniforms; p.next_ids = next_ids; p.stats = stats;
  p.n = n; p.V = V; p.n_hist_rows = n_hist_rows; p.hist_cols = hist_cols; p.top_k = top_k; p.append = append;
  p.inv_temperature = 1.f / temperature; p.top_p = top_p; p.penalty = repetition_penalty;
  const size_t need = qpam_sample_workspace_bytes(n, V);
  p.row_in_smem = need == 0;
  size_t smem = SAMPLE_SMEM_EXTRA;
  if (p.row_in_smem) {
    smem += (size_t)V * 4;
  } else {
    QPAM_REQUIRE(workspace && workspace_bytes >= need, "sample: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    p.work = reinterpret_cast<float*>(workspace);
  }
  static_assert(sizeof(Scratch) + SAMPLE_COMPACT * 8 <= SAMPLE_SMEM_EXTRA, "scratch does not fit");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == QPAM_F32) {
    QPAM_CUDA(cudaFuncSetAttribute(k_sample_rows<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_sample_rows<float><<<n, SAMPLE_THREADS, smem, st>>>(p);
  } else {
    QPAM_CUDA(cudaFuncSetAttribute(k_sample_rows<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_sample_rows<__nv_bfloat16><<<n, SAMPLE_THREADS, smem, st>>>(p);
  }
  QPAM_LAUNCH_CHECK("k_sample_rows");
  return QPAM_OK;
}
