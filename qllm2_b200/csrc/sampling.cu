// Token sampling on the device: temperature, repetition penalty, top-k, top-p (nucleus) and the draw itself,
// one CTA per row of logits, no sort and no host round trip.  Semantics of the reference's sampling block
// (v11/model.py:1221-1244):
//   x = logits / temperature
//   x[h] = x[h] > 0 ? x[h] / penalty : x[h] * penalty          for every token h already in the sequence
//   top-k : drop x < (k-th largest x)                            (ties with the k-th value stay)
//   top-p : in descending order, drop a token when the probability mass BEFORE it is >= top_p
//   draw from softmax of what is left
// The row lives in shared memory (V <= ~56k floats) or in a caller workspace; the k-th largest value and the
// nucleus threshold are found by radix selection over order-preserving integer keys (4 passes of 8 bits, counts
// for top-k, probability mass for top-p); the draw is the inverse CDF in vocabulary order of a uniform number the
// caller supplies.  Tokens that tie with the nucleus threshold are all kept (a sort would keep an arbitrary
// subset of them).
#include "common.cuh"

namespace qpam {
namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_SMEM_EXTRA = 4096;  // histograms, scan scratch, scalars

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

// Histogram updates of a whole warp (every lane calls; bin < 0 = this lane adds nothing).  Lanes that hit the same
// bin are combined before the shared-memory atomic, so a row whose keys share their leading bits (the usual case
// at the first radix level) does not serialise 32 ways on one address.
__device__ __forceinline__ void warp_hist_count(uint32_t* hist, int bin) {
  const unsigned peers = __match_any_sync(0xffffffffu, bin);
  if (bin >= 0 && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
}
__device__ __forceinline__ void warp_hist_mass(float* hist, int bin, float val) {
  const unsigned peers = __match_any_sync(0xffffffffu, bin);
  const int lane = threadIdx.x & 31;
  const bool big = bin >= 0 && __popc(peers) >= 8;
  unsigned leaders = __ballot_sync(0xffffffffu, big && lane == __ffs(peers) - 1);   // at most four groups of >= 8
  while (leaders) {
    const int ld = __ffs(leaders) - 1;
    leaders &= leaders - 1;
    const int b = __shfl_sync(0xffffffffu, bin, ld);
    float s = (bin == b) ? val : 0.f;
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == ld) atomicAdd(&hist[b], s);
  }
  if (bin >= 0 && !big) atomicAdd(&hist[bin], val);
}

struct Scratch {
  uint32_t count[256];
  float mass[256];
  float warp_f[32];
  float bcast_f[4];
  uint32_t prefix;
  uint32_t remaining;
  float mass_above;
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
        warp_hist_count(sc->count, (i < V && (key & himask) == prefix) ? (int)((key >> shift) & 255u) : -1);
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

  // ---- softmax statistics of what top-k left
  float mx = -INFINITY;
  for (int i = tid; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, w[i]);
  mx = block_max(mx, sc);
  float z = 0.f;
  for (int i = tid; i < V; i += SAMPLE_THREADS) {
    const float x = w[i];
    if (order_key(x) >= key_k) z += __expf(x - mx);
  }
  z = block_sum(z, sc);

  // ---- top-p: the key at which the descending cumulative mass first reaches top_p * z
  uint32_t key_p = 0;
  if (p.top_p > 0.f && p.top_p < 1.f) {
    const float target = p.top_p * z;
    __syncthreads();
    if (tid == 0) { sc->prefix = 0; sc->mass_above = 0.f; }
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) sc->mass[tid] = 0.f;
      __syncthreads();
      const uint32_t prefix = sc->prefix;
      const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int base = 0; base < V; base += SAMPLE_THREADS) {
        const int i = base + tid;
        const float x = i < V ? w[i] : 0.f;
        const uint32_t key = order_key(x);
        const bool in = i < V && key >= key_k && (key & himask) == prefix;
        warp_hist_mass(sc->mass, in ? (int)((key >> shift) & 255u) : -1, __expf(x - mx));
      }
      __syncthreads();
      if (tid < 32) {  // warp 0: lane l owns bins 255-8l .. 248-8l
        const int top = 255 - 8 * tid;
        float mine = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += sc->mass[top - j];
        float inc = mine;
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, inc, o);
          if (tid >= o) inc += t;
        }
        const float before = sc->mass_above + (inc - mine);
        const unsigned hit = __ballot_sync(0xffffffffu, mine > 0.f && before + mine >= target);
        const unsigned occupied = __ballot_sync(0xffffffffu, mine > 0.f);
        // rounding can leave the whole sum just below the target: the lowest occupied bin closes the nucleus then
        const int owner = hit ? __ffs(hit) - 1 : (occupied ? 31 - __clz(occupied) : 31);
        if (tid == owner) {
          float cum = before;
          int b = top, found = -1, lowest = top - 7;
          for (; b > top - 8; --b) {
            const float m = sc->mass[b];
            if (m > 0.f) {
              lowest = b;
              if (cum + m >= target) { found = b; break; }
              cum += m;
            }
          }
          if (found < 0) {
            found = lowest;
            cum -= sc->mass[found];
          }
          sc->mass_above = cum;
          sc->prefix = prefix | ((uint32_t)found << shift);
        }
      }
      __syncthreads();
    }
    key_p = sc->prefix;
  }
  const uint32_t key_min = key_k > key_p ? key_k : key_p;

  // ---- the draw: inverse CDF in vocabulary order over the kept tokens
  const int per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int i0 = min(V, tid * per), i1 = min(V, i0 + per);
  float mine = 0.f;
  int last = -1, cnt = 0;
  for (int i = i0; i < i1; ++i) {
    const float x = w[i];
    if (order_key(x) >= key_min) {
      mine += __expf(x - mx);
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
      const float x = w[i];
      if (order_key(x) >= key_min) {
        cum += __expf(x - mx);
        if (cum > target) { pick = i; break; }
      }
    }
    atomicMax(&sc->chosen, pick);
  }
  __syncthreads();
  if (tid == 0) {
    const int pick = sc->chosen >= 0 ? sc->chosen : sc->last_kept;
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
  static_assert(sizeof(Scratch) <= SAMPLE_SMEM_EXTRA, "scratch does not fit");
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
