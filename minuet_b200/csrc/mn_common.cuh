// Shared declarations of the CUDA side: error plumbing, launch helpers, the key
// layout and the internal (C++-linkage) launchers that mn_api.cu wraps.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/minuet_b200.h"

namespace mn {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs
constexpr int kMaxDevices = 64;
constexpr int kMaxCoopBlocks = 1024;  // upper bound of a cooperative grid (workspace sizing)

// Key layout as a kernel parameter: the host copy, or (when the layout was
// derived on the device and never read back) a pointer to the device copy.
struct SpecRef {
  mn_keyspec host;
  const mn_keyspec *dev;
};
inline SpecRef make_spec_ref(const mn_keyspec &s) {
  SpecRef r;
  r.host = s;
  r.dev = static_cast<const mn_keyspec *>(s.device_copy);
  return r;
}
#ifdef __CUDACC__
__device__ __forceinline__ const mn_keyspec &spec_of(const SpecRef &r) {
  return r.dev != nullptr ? *r.dev : r.host;
}
#endif

void set_error(const char *fmt, ...);

#define MN_CHECK_ARG(cond, ...)                      \
  do {                                               \
    if (!(cond)) {                                   \
      ::mn::set_error(__VA_ARGS__);                  \
      return MN_ERR_BAD_ARG;                         \
    }                                                \
  } while (0)

#define MN_CHECK_CUDA(expr)                                                   \
  do {                                                                        \
    cudaError_t e__ = (expr);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      ::mn::set_error("%s:%d CUDA error: %s", __FILE__, __LINE__,             \
                      cudaGetErrorString(e__));                               \
      return MN_ERR_CUDA;                                                     \
    }                                                                         \
  } while (0)

#define MN_CHECK_LAUNCH() MN_CHECK_CUDA(cudaGetLastError())

// Counts the launch and, while profiling is on (mn_profile_enable), brackets it
// with a pair of CUDA events on the launching stream.
struct LaunchScope {
  LaunchScope(const char *name, cudaStream_t st);
  ~LaunchScope();
  cudaStream_t st_;
  const char *name_;
  cudaEvent_t begin_, end_;   // both null unless this launch is being timed
};

#define MN_LAUNCH(name, st, ...)                  \
  do {                                            \
    {                                             \
      ::mn::LaunchScope scope__(name, st);        \
      __VA_ARGS__;                                \
    }                                             \
    MN_CHECK_LAUNCH();                            \
  } while (0)

// Optional phase timing of a kernel (builds with -DMN_PHASE_TIMING only): thread 0
// of the first blocks stores its SM cycle counter at numbered points into a
// file-local array that a debug entry point copies out.
#ifdef MN_PHASE_TIMING
#define MN_MARKS_DECL(name) static __device__ long long name[2048 * 16]
#define MN_MARK(name, slot)                                                          \
  do {                                                                               \
    if (threadIdx.x == 0 && blockIdx.x < 2048) name[blockIdx.x * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define MN_MARKS_DECL(name)
#define MN_MARK(name, slot) do {} while (0)
#endif

#define MN_RETURN_IF(expr)              \
  do {                                  \
    mn_status s__ = (expr);             \
    if (s__ != MN_OK) return s__;       \
  } while (0)

inline int64_t div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

// Bump allocator over the caller's workspace; never touches the driver.
struct Workspace {
  char *base;
  size_t size;
  size_t used = 0;
  bool overflow = false;
  Workspace(void *p, size_t n) : base(static_cast<char *>(p)), size(n) {}
  template <typename T>
  T *take(size_t count) {
    size_t bytes = align_up(count * sizeof(T), 256);
    if (base == nullptr || used + bytes > size) {
      overflow = true;
      used += bytes;
      return nullptr;
    }
    T *p = reinterpret_cast<T *>(base + used);
    used += bytes;
    return p;
  }
};

#define MN_CHECK_WS(ws)                                                        \
  do {                                                                         \
    if ((ws).overflow) {                                                       \
      ::mn::set_error("workspace too small: need %zu bytes, have %zu",         \
                      (ws).used, (ws).size);                                   \
      return MN_ERR_WORKSPACE;                                                 \
    }                                                                          \
  } while (0)

// Offsets regrouped for the search kernel: offsets that share every dimension
// but the last form a group, and inside a group the queries of one row grow
// with the member index, so one binary search serves the whole group.
struct OffsetTable {
  int32_t num_offsets;
  int32_t num_groups;
  int32_t ndim;
  int32_t pad_;
  int32_t off[MN_MAX_OFFSETS][MN_MAX_NDIM];  // effective (sign folded) offsets
  uint8_t member[MN_MAX_OFFSETS];            // offset indices, group by group
  uint8_t group_begin[MN_MAX_OFFSETS + 1];   // prefix into member[]
};

mn_status make_offset_table(const int32_t *offsets, int64_t O, int ndim, int sign,
                            const mn_keyspec *spec, OffsetTable *out);

// Problem table of the grouped GEMM over offsets, passed to the kernels by value.
struct GemmTable {
  int32_t num_problems;
  int32_t tile_rows;                          // rows per tile the prefix was built for
  int32_t tile_prefix[MN_MAX_OFFSETS + 2];    // prefix of row tiles over problems
  int32_t rows[MN_MAX_OFFSETS + 1];
  int32_t weight_row[MN_MAX_OFFSETS + 1];     // mask row whose weight matrix to use
  const void *a[MN_MAX_OFFSETS + 1];          // first A row of the problem
  void *c[MN_MAX_OFFSETS + 1];                // first C row of the problem
  int64_t a_row[MN_MAX_OFFSETS + 1];          // that row's index inside its operand array
  uint8_t direct[MN_MAX_OFFSETS + 1];         // 1: A is the input feature matrix, 0: gather buffer
};

// Operand arrays of the tensor-core GEMM (TMA addresses whole arrays, not rows).
struct TcOperands {
  const void *gathered = nullptr;   // [gathered_rows, c_in]
  int64_t gathered_rows = 0;
  const void *sources = nullptr;    // [source_rows, c_in]
  int64_t source_rows = 0;
  void *products = nullptr;         // [gathered_rows, c_out]: outputs of the buffered problems
  void *out = nullptr;              // [out_rows, c_out]: output of the direct problem
  int64_t out_rows = 0;
  void *weights_t = nullptr;        // scratch for the transposed weights [O, c_out, c_in]
  int num_weights = 0;              // O
  int32_t *status = nullptr;        // device status word
};

// Tensor-core grouped GEMM (mn_gemm_tc.cu); *handled = false when the shape or
// dtype is outside what it covers and the caller must use the SIMT kernel.
mn_status launch_gemm_tc(const GemmTable &tab, const TcOperands &ops, int c_in, int c_out,
                         mn_dtype dtype, const void *weights, const int32_t *order,
                         cudaStream_t st, bool *handled);
bool gemm_tc_supported(int c_in, int c_out, mn_dtype dtype);
size_t gemm_tc_workspace_bytes(int64_t O, int64_t c_in, int64_t c_out);

// ---- launchers (defined in the .cu files) ---------------------------------
mn_status launch_bbox(const int32_t *a, int64_t na, const int32_t *b, int64_t nb,
                      int ndim, int32_t *minmax_dev, Workspace &ws, cudaStream_t st);
mn_status launch_pack(const int32_t *coords, int64_t n, int ndim,
                      const int64_t *batch_dims, int64_t num_clouds,
                      const int32_t *tstride, const mn_keyspec &spec,
                      uint64_t *keys_out, int32_t *status_dev, cudaStream_t st);
// Coordinate rows a sort builds its keys from (floored to tstride when given).
struct SortSource {
  const int32_t *coords;
  const int64_t *batch_dims;
  int64_t num_clouds;
  int ndim;
  const int32_t *tstride;   // host, may be NULL
};
mn_status launch_radix_sort(uint64_t *keys, uint64_t *keys_tmp, int32_t *vals, int32_t *vals_tmp,
                            bool iota_vals, int64_t n, int begin_bit, int end_bit,
                            const mn_keyspec &spec, const SortSource *source, int32_t *ctrl,
                            int32_t *result_in_second_dev, Workspace &ws, bool *result_in_tmp,
                            cudaStream_t st);
size_t radix_sort_workspace_bytes(int64_t n);

}  // namespace mn
