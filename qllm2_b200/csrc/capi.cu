// Error reporting and version string of the C ABI.
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace qpam {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return QPAM_ECUDA;
}

// SMs of the current device (grids and split heuristics are sized from it); 148 if the query fails.
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ------------------------------------------------------------------ launch accounting
static std::atomic<long long> g_launches{0};
static std::atomic<bool> g_profiling{false};
bool profiling_active() { return g_profiling.load(std::memory_order_relaxed); }
static std::mutex g_prof_mu;
struct ProfRec {
  const char* name;
  cudaEvent_t ev;
};
static std::vector<ProfRec> g_prof;  // g_prof[0] is the base mark

void note_launch(const char* name, cudaStream_t stream_) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_profiling.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  cudaEvent_t ev;
  if (cudaEventCreate(&ev) != cudaSuccess) return;
  cudaEventRecord(ev, stream_);
  g_prof.push_back({name, ev});
}

}  // namespace qpam

extern "C" long long qpam_launch_count(void) { return qpam::g_launches.load(); }

extern "C" int qpam_profile_begin(void* stream) {
  using namespace qpam;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) cudaEventDestroy(r.ev);
  g_prof.clear();
  cudaEvent_t ev;
  QPAM_CUDA(cudaEventCreate(&ev));
  QPAM_CUDA(cudaEventRecord(ev, reinterpret_cast<cudaStream_t>(stream)));
  g_prof.push_back({"<mark>", ev});
  g_profiling.store(true);
  return QPAM_OK;
}

extern "C" int qpam_profile_end(char* buf, size_t buf_bytes) {
  using namespace qpam;
  g_profiling.store(false);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  std::map<std::string, std::pair<long long, double>> agg;
  if (!g_prof.empty()) QPAM_CUDA(cudaEventSynchronize(g_prof.back().ev));
  for (size_t i = 1; i < g_prof.size(); ++i) {
    float ms = 0.f;
    QPAM_CUDA(cudaEventElapsedTime(&ms, g_prof[i - 1].ev, g_prof[i].ev));
    auto& a = agg[g_prof[i].name];
    a.first += 1;
    a.second += ms;
  }
  for (auto& r : g_prof) cudaEventDestroy(r.ev);
  g_prof.clear();
  std::string out;
  char line[256];
  for (auto& kv : agg) {
    snprintf(line, sizeof(line), "%s %lld %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
    out += line;
  }
  if (buf != nullptr && buf_bytes > 0) {
    const size_t n = out.size() < buf_bytes - 1 ? out.size() : buf_bytes - 1;
    memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return QPAM_OK;
}

namespace qpam {
// one device status word per translation unit that waits on the device
int ce_tc_device_status(int* value, bool clear);
int scan_tc_device_status(int* value, bool clear);
int decode_device_status(int* value, bool clear);
}

extern "C" int qpam_device_status(int32_t* status, int32_t clear) {
  int first = 0;
  int (*readers[])(int*, bool) = {qpam::ce_tc_device_status, qpam::scan_tc_device_status, qpam::decode_device_status};
  for (auto rd : readers) {
    int v = 0;
    const int rc = rd(&v, clear != 0);
    if (rc) return rc;
    if (first == 0) first = v;
  }
  if (status) *status = first;
  return QPAM_OK;
}

extern "C" const char* qpam_last_error(void) { return qpam::g_err; }

extern "C" const char* qpam_version(void) { return "qllm2_pam_b200 0.1 sm_100a"; }
