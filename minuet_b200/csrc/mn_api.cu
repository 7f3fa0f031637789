// C ABI glue: error reporting, version, and the thin wrappers whose kernels
// live in mn_map_keys.cu.
#include "mn_common.cuh"

#include <cstring>

namespace mn {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

}  // namespace mn

using namespace mn;

extern "C" const char *mn_last_error(void) { return g_error; }

extern "C" int mn_version(void) { return 1; }

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
