// C ABI glue: error reporting, version, and the thin wrappers whose kernels
// live in mn_map_keys.cu.
#include "mn_common.cuh"

#include <atomic>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace mn {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// ---- launch counter and optional per-kernel event timing -------------------
namespace {
constexpr int kMaxProfiled = 4096;
struct ProfEntry {
  const char *name;
  cudaEvent_t begin, end;
};
std::atomic<long long> g_launches{0};
std::atomic<bool> g_profiling{false};
std::mutex g_prof_mutex;
std::vector<ProfEntry> g_prof;   // completed (begin, end) pairs only
}  // namespace

// The scope owns its two events and hands the finished pair to the record under the
// lock, so a report that clears the record while a launch is in flight on another
// thread cannot leave a scope pointing at a slot that no longer exists.
LaunchScope::LaunchScope(const char *name, cudaStream_t st)
    : st_(st), name_(name), begin_(nullptr), end_(nullptr) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_profiling.load(std::memory_order_relaxed)) return;
  if (cudaEventCreate(&begin_) != cudaSuccess) { begin_ = nullptr; return; }
  if (cudaEventCreate(&end_) != cudaSuccess) {
    cudaEventDestroy(begin_);
    begin_ = end_ = nullptr;
    return;
  }
  cudaEventRecord(begin_, st);
}

LaunchScope::~LaunchScope() {
  if (begin_ == nullptr) return;
  cudaEventRecord(end_, st_);
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  if ((int)g_prof.size() < kMaxProfiled) {
    g_prof.push_back(ProfEntry{name_, begin_, end_});
  } else {
    cudaEventDestroy(begin_);
    cudaEventDestroy(end_);
  }
}

}  // namespace mn

using namespace mn;

extern "C" long long mn_launch_count(void) { return g_launches.load(); }

extern "C" void mn_profile_enable(int on) {
  g_profiling.store(on != 0);
}

// Waits for the recorded events and writes one line per distinct kernel name:
// "name launches total_ms".  Returns the number of bytes written and clears
// the record.
extern "C" int mn_profile_report(char *buf, int buf_bytes) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  std::vector<std::string> names;
  std::vector<int> counts;
  std::vector<double> totals;
  for (auto &e : g_prof) {
    float ms = 0.f;
    if (cudaEventSynchronize(e.end) == cudaSuccess) cudaEventElapsedTime(&ms, e.begin, e.end);
    cudaEventDestroy(e.begin);
    cudaEventDestroy(e.end);
    size_t i = 0;
    for (; i < names.size(); i++) if (names[i] == e.name) break;
    if (i == names.size()) { names.push_back(e.name); counts.push_back(0); totals.push_back(0.0); }
    counts[i]++;
    totals[i] += ms;
  }
  g_prof.clear();
  int used = 0;
  for (size_t i = 0; i < names.size() && buf != nullptr; i++) {
    int n = snprintf(buf + used, buf_bytes > used ? buf_bytes - used : 0, "%s %d %.6f\n",
                     names[i].c_str(), counts[i], totals[i]);
    if (n < 0 || used + n >= buf_bytes) break;
    used += n;
  }
  return used;
}

extern "C" const char *mn_last_error(void) { return g_error; }

extern "C" int mn_version(void) { return MN_ABI_VERSION; }

extern "C" mn_status mn_bbox(const int32_t *a, int64_t na, const int32_t *b, int64_t nb, int ndim,
                             int32_t *minmax_dev, void *ws_ptr, size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(ndim >= 1 && ndim <= MN_MAX_NDIM, "bbox: ndim %d not in 1..4", ndim);
  MN_CHECK_ARG(na >= 0 && nb >= 0, "bbox: negative row count");
  MN_CHECK_ARG(minmax_dev != nullptr, "bbox: null output");
  MN_CHECK_ARG((na == 0 || a != nullptr) && (nb == 0 || b != nullptr), "bbox: null input");
  Workspace ws(ws_ptr, ws_bytes);
  return launch_bbox(a, na, b, nb, ndim, minmax_dev, ws, static_cast<cudaStream_t>(stream));
}

extern "C" mn_status mn_pack_keys(const int32_t *coords, int64_t n, int ndim,
                                  const int64_t *batch_dims, int64_t num_clouds,
                                  const int32_t *tstride, const mn_keyspec *spec,
                                  uint64_t *keys_out, int32_t *status_dev, void *stream) {
  MN_CHECK_ARG(n >= 0 && ndim >= 1 && ndim <= MN_MAX_NDIM, "pack_keys: bad n/ndim");
  MN_CHECK_ARG(spec != nullptr && spec->ndim == ndim, "pack_keys: key spec missing or of another ndim");
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(coords != nullptr && keys_out != nullptr && status_dev != nullptr,
               "pack_keys: null pointer");
  return launch_pack(coords, n, ndim, batch_dims, num_clouds, tstride, *spec, keys_out, status_dev,
                     static_cast<cudaStream_t>(stream));
}
