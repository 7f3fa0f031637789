// Map step, part 0: bounding box and coordinate packing.
//
// Every later Map-step kernel works on one 64-bit key per voxel
//   key = cloud << cloud_shift | sum_k (c[k] - base[k]) << shift[k]
// whose unsigned order equals the tensors' sorted order (cloud-major, then
// lexicographic with dimension 0 most significant) and for which adding a
// kernel offset is a single 64-bit add: each field carries `margin` spare values
// on both sides, so target + offset never borrows from a neighbouring field.
// This replaces the reference's per-cloud flattening
// (csrc/minuet/cuda/kernels/flatten_coordinates.cuh:23-38) and its three-way
// integer comparisons (csrc/minuet/common/functions.h:94-105).
#include "mn_grid.cuh"
#include "mn_pack.cuh"

#include <algorithm>
#include <climits>

namespace mn {

namespace {

constexpr int kBBoxThreads = 256;
constexpr int kBBoxMaxBlocks = kNumSMs * 4;

__device__ __forceinline__ void fold(int v, int d, int (&mn_)[4], int (&mx_)[4]) {
#pragma unroll
  for (int k = 0; k < 4; k++) {
    if (d == k) {
      mn_[k] = min(mn_[k], v);
      mx_[k] = max(mx_[k], v);
    }
  }
}

// Min/max over a flat int32 stream (element j belongs to dim j % ndim) read with
// 128-bit loads by `nthreads` threads of which this one is `thread`; p + first
// must be 16-byte aligned for the vector path.
__device__ __forceinline__ void scan_flat(const int32_t *__restrict__ p, int64_t first,
                                          int64_t count, int ndim, int64_t thread,
                                          int64_t nthreads, int (&mn_)[4], int (&mx_)[4]) {
  const bool aligned = (reinterpret_cast<uintptr_t>(p + first) & 15) == 0;
  const int64_t nvec = aligned ? (count >> 2) : 0;
  const int4 *pv = reinterpret_cast<const int4 *>(p + first);
  for (int64_t i = thread; i < nvec; i += nthreads) {
    int4 v = __ldg(pv + i);
    int d = (int)((uint32_t)((first + (i << 2)) % (int64_t)ndim));
    fold(v.x, d, mn_, mx_); d = (d + 1 == ndim) ? 0 : d + 1;
    fold(v.y, d, mn_, mx_); d = (d + 1 == ndim) ? 0 : d + 1;
    fold(v.z, d, mn_, mx_); d = (d + 1 == ndim) ? 0 : d + 1;
    fold(v.w, d, mn_, mx_);
  }
  for (int64_t j = (nvec << 2) + thread; j < count; j += nthreads)
    fold(__ldg(p + first + j), (int)((first + j) % ndim), mn_, mx_);
}

// One partial box per block: partial[b][0..3] = min, [4..7] = max.
__global__ void __launch_bounds__(kBBoxThreads)
bbox_partial_kernel(const int32_t *__restrict__ a, int64_t na,
                    const int32_t *__restrict__ b, int64_t nb, int ndim,
                    int32_t *__restrict__ partial) {
  int mn_[4] = {INT_MAX, INT_MAX, INT_MAX, INT_MAX};
  int mx_[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  if (a != nullptr) scan_flat(a, 0, na * ndim, ndim, gid, gsz, mn_, mx_);
  if (b != nullptr) scan_flat(b, 0, nb * ndim, ndim, gid, gsz, mn_, mx_);
#pragma unroll
  for (int k = 0; k < 4; k++) {
    mn_[k] = __reduce_min_sync(0xffffffffu, mn_[k]);
    mx_[k] = __reduce_max_sync(0xffffffffu, mx_[k]);
  }
  __shared__ int s[kBBoxThreads / 32][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < 4; k++) { s[warp][k] = mn_[k]; s[warp][4 + k] = mx_[k]; }
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    int v = s[0][threadIdx.x];
    for (int w = 1; w < kBBoxThreads / 32; w++)
      v = threadIdx.x < 4 ? min(v, s[w][threadIdx.x]) : max(v, s[w][threadIdx.x]);
    partial[blockIdx.x * 8 + threadIdx.x] = v;
  }
}

__global__ void __launch_bounds__(256)
bbox_final_kernel(const int32_t *__restrict__ partial, int nblocks,
                  int32_t *__restrict__ minmax) {
  // 8 groups of 32 threads, one per output value
  const int which = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int v = which < 4 ? INT_MAX : INT_MIN;
  for (int b = lane; b < nblocks; b += 32) {
    int p = partial[b * 8 + which];
    v = which < 4 ? min(v, p) : max(v, p);
  }
  v = which < 4 ? __reduce_min_sync(0xffffffffu, v) : __reduce_max_sync(0xffffffffu, v);
  if (lane == 0) minmax[which] = v;
}

constexpr int kPackThreads = 256;
constexpr int kMaxSmemClouds = 2048;

// Keys of rows [r_begin, r_end) (r_begin a multiple of 4), the work split over
// `nthreads` threads of which this one is `thread`.  ndim == 3 fast path: 4 rows
// (48 bytes) per thread as three 128-bit loads and two 128-bit stores.
__device__ __forceinline__ void pack_rows(const int32_t *__restrict__ coords, int64_t r_begin,
                                          int64_t r_end, int ndim, const int64_t *bd,
                                          int num_clouds, const mn_keyspec &spec,
                                          const PackParams &p, uint64_t *__restrict__ keys,
                                          int64_t thread, int64_t nthreads, bool &bad) {
  if (ndim == 3) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(coords) | reinterpret_cast<uintptr_t>(keys)) & 15) == 0;
    const int64_t q_begin = r_begin >> 2;
    const int64_t q_end = aligned ? (r_end >> 2) : q_begin;
    const int4 *cv = reinterpret_cast<const int4 *>(coords);
    for (int64_t q = q_begin + thread; q < q_end; q += nthreads) {
      int4 v0 = __ldg(cv + 3 * q), v1 = __ldg(cv + 3 * q + 1), v2 = __ldg(cv + 3 * q + 2);
      int c0[4] = {v0.x, v0.y, v0.z, 0}, c1[4] = {v0.w, v1.x, v1.y, 0};
      int c2[4] = {v1.z, v1.w, v2.x, 0}, c3[4] = {v2.y, v2.z, v2.w, 0};
      const int64_t r = q << 2;
      uint64_t g0 = 0, g1 = 0, g2 = 0, g3 = 0;
      if (bd != nullptr) {
        g0 = cloud_of(bd, num_clouds, r);
        g3 = cloud_of(bd, num_clouds, r + 3);
        g1 = g0 == g3 ? g0 : cloud_of(bd, num_clouds, r + 1);
        g2 = g0 == g3 ? g0 : cloud_of(bd, num_clouds, r + 2);
      }
      ulonglong2 lo, hi;
      lo.x = pack_one(c0, 3, g0, spec, p, bad);
      lo.y = pack_one(c1, 3, g1, spec, p, bad);
      hi.x = pack_one(c2, 3, g2, spec, p, bad);
      hi.y = pack_one(c3, 3, g3, spec, p, bad);
      ulonglong2 *kv = reinterpret_cast<ulonglong2 *>(keys + r);
      kv[0] = lo;
      kv[1] = hi;
    }
    for (int64_t r = (q_end << 2) + thread; r < r_end; r += nthreads) {
      int c[4] = {coords[r * 3], coords[r * 3 + 1], coords[r * 3 + 2], 0};
      uint64_t g = bd != nullptr ? cloud_of(bd, num_clouds, r) : 0;
      keys[r] = pack_one(c, 3, g, spec, p, bad);
    }
  } else {
    for (int64_t r = r_begin + thread; r < r_end; r += nthreads) {
      int c[4] = {0, 0, 0, 0};
      for (int k = 0; k < ndim; k++) c[k] = coords[r * ndim + k];
      uint64_t g = bd != nullptr ? cloud_of(bd, num_clouds, r) : 0;
      keys[r] = pack_one(c, ndim, g, spec, p, bad);
    }
  }
}

// The cloud boundaries, staged in shared memory when they fit
__device__ __forceinline__ const int64_t *stage_batch_dims(const int64_t *batch_dims, int num_clouds,
                                                           int64_t *s_bd) {
  if (batch_dims == nullptr || num_clouds > kMaxSmemClouds) return batch_dims;
  for (int i = threadIdx.x; i <= num_clouds; i += blockDim.x) s_bd[i] = batch_dims[i];
  __syncthreads();
  return s_bd;
}

__global__ void __launch_bounds__(kPackThreads)
pack_kernel(const int32_t *__restrict__ coords, int64_t n, int ndim,
            const int64_t *__restrict__ batch_dims, int num_clouds,
            const __grid_constant__ PackParams p, uint64_t *__restrict__ keys,
            int32_t *__restrict__ status) {
  const mn_keyspec &spec = spec_of(p.spec);
  __shared__ int64_t s_bd[kMaxSmemClouds + 1];
  const int64_t *bd = stage_batch_dims(batch_dims, num_clouds, s_bd);
  bool bad = false;
  pack_rows(coords, 0, n, ndim, bd, num_clouds, spec, p, keys,
            (int64_t)blockIdx.x * blockDim.x + threadIdx.x, (int64_t)gridDim.x * blockDim.x, bad);
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(status, MN_STATUS_KEY_BOX);
}

// Bounding box, key layout and (optionally) the keys of the same rows in one
// cooperative launch: every block takes the box of its contiguous chunk of rows,
// a grid barrier later every block reduces all the partial boxes and derives the
// layout (block 0 also stores it for the kernels that follow), then packs its
// own chunk, which it has just read.  Nothing is read back by the host.
struct RootArgs {
  const int32_t *coords;
  const int64_t *batch_dims;
  int64_t n, num_clouds;
  int32_t ndim, margin;
  int32_t *partial;        // workspace [grid][8]
  mn_keyspec *spec_out;
  uint64_t *keys_out;      // may be NULL: layout only
  int32_t *ctrl;
};

__global__ void __launch_bounds__(kBBoxThreads)
root_keys_kernel(const __grid_constant__ RootArgs a) {
  __shared__ int s[kBBoxThreads / 32][8];
  __shared__ int32_t s_mm[8];
  __shared__ PackParams s_p;
  __shared__ int64_t s_bd[kMaxSmemClouds + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  // chunk of rows of this block, a multiple of 4 rows (16-byte aligned for any ndim)
  const int64_t per_block = ((a.n + G - 1) / G + 3) / 4 * 4;
  const int64_t r0 = min(a.n, (int64_t)b * per_block), r1 = min(a.n, r0 + per_block);
  int mn_[4] = {INT_MAX, INT_MAX, INT_MAX, INT_MAX};
  int mx_[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
  if (r1 > r0) scan_flat(a.coords, r0 * a.ndim, (r1 - r0) * a.ndim, a.ndim, threadIdx.x, blockDim.x, mn_, mx_);
#pragma unroll
  for (int k = 0; k < 4; k++) {
    mn_[k] = __reduce_min_sync(0xffffffffu, mn_[k]);
    mx_[k] = __reduce_max_sync(0xffffffffu, mx_[k]);
  }
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < 4; k++) { s[warp][k] = mn_[k]; s[warp][4 + k] = mx_[k]; }
  }
  __syncthreads();
  if (threadIdx.x < 8) {
    int v = s[0][threadIdx.x];
    for (int w = 1; w < kBBoxThreads / 32; w++)
      v = threadIdx.x < 4 ? min(v, s[w][threadIdx.x]) : max(v, s[w][threadIdx.x]);
    a.partial[b * 8 + threadIdx.x] = v;
  }
  grid_barrier(a.ctrl, (unsigned)G);
  {
    // 8 warps, one per output value
    const int which = warp;
    int v = which < 4 ? INT_MAX : INT_MIN;
    for (int bb = lane; bb < G; bb += 32) {
      const int p = __ldcg(a.partial + bb * 8 + which);
      v = which < 4 ? min(v, p) : max(v, p);
    }
    v = which < 4 ? __reduce_min_sync(0xffffffffu, v) : __reduce_max_sync(0xffffffffu, v);
    if (lane == 0) s_mm[which] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!compute_keyspec(s_mm, a.ndim, a.num_clouds, a.margin, &s_p.spec.host) && b == 0)
      atomicOr(a.ctrl + MN_CTRL_STATUS, MN_STATUS_KEY_BITS);
    s_p.spec.dev = nullptr;
    s_p.has_stride = 0;
    for (int k = 0; k < 4; k++) s_p.tstride[k] = 1;
    if (b == 0) *a.spec_out = s_p.spec.host;
  }
  __syncthreads();
  if (a.keys_out == nullptr) return;
  const int nc = a.batch_dims != nullptr ? (int)a.num_clouds : 1;
  const int64_t *bd = stage_batch_dims(a.batch_dims, nc, s_bd);
  bool bad = false;
  pack_rows(a.coords, r0, r1, a.ndim, bd, nc, s_p.spec.host, s_p, a.keys_out, threadIdx.x,
            blockDim.x, bad);
  if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(a.ctrl + MN_CTRL_STATUS, MN_STATUS_KEY_BOX);
}

}  // namespace

mn_status launch_bbox(const int32_t *a, int64_t na, const int32_t *b, int64_t nb,
                      int ndim, int32_t *minmax_dev, Workspace &ws, cudaStream_t st) {
  int64_t elems = (na + nb) * ndim;
  int blocks = (int)std::min<int64_t>(kBBoxMaxBlocks, std::max<int64_t>(1, div_up(elems, kBBoxThreads * 16)));
  int32_t *partial = ws.take<int32_t>((size_t)kBBoxMaxBlocks * 8);
  MN_CHECK_WS(ws);
  MN_LAUNCH("bbox_partial_kernel", st, bbox_partial_kernel<<<blocks, kBBoxThreads, 0, st>>>(na > 0 ? a : nullptr, na,
                                                       nb > 0 ? b : nullptr, nb, ndim, partial));
  MN_LAUNCH("bbox_final_kernel", st, bbox_final_kernel<<<1, 256, 0, st>>>(partial, blocks, minmax_dev));
  return MN_OK;
}

mn_status launch_pack(const int32_t *coords, int64_t n, int ndim,
                      const int64_t *batch_dims, int64_t num_clouds,
                      const int32_t *tstride, const mn_keyspec &spec,
                      uint64_t *keys_out, int32_t *status_dev, cudaStream_t st) {
  if (n == 0) return MN_OK;
  PackParams p;
  p.spec = make_spec_ref(spec);
  p.has_stride = 0;
  for (int k = 0; k < 4; k++) p.tstride[k] = 1;
  if (tstride != nullptr) {
    for (int k = 0; k < ndim; k++) {
      MN_CHECK_ARG(tstride[k] >= 1, "pack_keys: stride must be >= 1, got %d", tstride[k]);
      p.tstride[k] = tstride[k];
      if (tstride[k] != 1) p.has_stride = 1;
    }
  }
  if (batch_dims == nullptr) num_clouds = 1;
  int blocks = (int)std::min<int64_t>(kNumSMs * 8, div_up(n, kPackThreads * 4));
  MN_LAUNCH("pack_kernel", st, pack_kernel<<<blocks, kPackThreads, 0, st>>>(coords, n, ndim, batch_dims, (int)num_clouds,
                                               p, keys_out, status_dev));
  return MN_OK;
}

}  // namespace mn

extern "C" mn_status mn_keyspec_make(const int32_t *minmax_host, int ndim,
                                     int64_t num_clouds, int32_t margin,
                                     mn_keyspec *spec) {
  using namespace mn;
  MN_CHECK_ARG(minmax_host != nullptr && spec != nullptr, "keyspec_make: null pointer");
  MN_CHECK_ARG(ndim >= 1 && ndim <= MN_MAX_NDIM, "keyspec_make: ndim %d not in 1..4", ndim);
  MN_CHECK_ARG(margin >= 0, "keyspec_make: negative margin");
  MN_CHECK_ARG(num_clouds >= 1, "keyspec_make: num_clouds must be >= 1");
  *spec = mn_keyspec{};
  if (!compute_keyspec(minmax_host, ndim, num_clouds, margin, spec)) {
    set_error("keyspec_make: bounding box needs %d key bits (> 63); coordinate "
              "ranges this large are not supported", spec->total_bits);
    return MN_ERR_UNSUPPORTED;
  }
  return MN_OK;
}

extern "C" mn_status mn_keyspec_device(const int32_t *coords, int64_t n, int ndim,
                                       const int64_t *batch_dims, int64_t num_clouds,
                                       int32_t margin, void *spec_dev, mn_keyspec *spec,
                                       uint64_t *keys_out, int32_t *ctrl, void *ws_ptr,
                                       size_t ws_bytes, void *stream) {
  using namespace mn;
  MN_CHECK_ARG(ndim >= 1 && ndim <= MN_MAX_NDIM, "keyspec_device: ndim %d not in 1..4", ndim);
  MN_CHECK_ARG(n >= 0 && margin >= 0, "keyspec_device: bad arguments");
  if (batch_dims == nullptr) num_clouds = 1;
  MN_CHECK_ARG(num_clouds >= 1, "keyspec_device: num_clouds must be >= 1");
  MN_CHECK_ARG(spec_dev != nullptr && spec != nullptr && ctrl != nullptr && (n == 0 || coords != nullptr),
               "keyspec_device: null pointer");
  MN_CHECK_ARG((reinterpret_cast<uintptr_t>(spec_dev) & 15) == 0, "keyspec_device: spec_dev must be 16-byte aligned");
  static thread_local int grid_cache[kMaxDevices] = {0};
  int device = 0;
  MN_CHECK_CUDA(cudaGetDevice(&device));
  MN_CHECK_ARG(device >= 0 && device < kMaxDevices, "keyspec_device: device index %d out of range", device);
  if (grid_cache[device] == 0) {
    grid_cache[device] = std::min(kBBoxMaxBlocks, max_coresident_blocks(root_keys_kernel, kBBoxThreads, 0));
    if (grid_cache[device] <= 0) {
      grid_cache[device] = 0;
      set_error("keyspec_device: cannot size the cooperative grid");
      return MN_ERR_CUDA;
    }
  }
  const int grid = (int)std::min<int64_t>(grid_cache[device],
                                          std::max<int64_t>(1, div_up(n, kBBoxThreads * 4)));
  Workspace ws(ws_ptr, ws_bytes);
  RootArgs a{};
  a.partial = ws.take<int32_t>((size_t)kBBoxMaxBlocks * 8);
  MN_CHECK_WS(ws);
  a.coords = coords; a.batch_dims = batch_dims; a.n = n; a.num_clouds = num_clouds;
  a.ndim = ndim; a.margin = margin;
  a.spec_out = static_cast<mn_keyspec *>(spec_dev);
  a.keys_out = n > 0 ? keys_out : nullptr;
  a.ctrl = ctrl;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  void *params[] = {&a};
  {
    LaunchScope scope("root_keys_kernel", st);
    MN_CHECK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(root_keys_kernel), dim3(grid),
                                              dim3(kBBoxThreads), params, 0, st));
  }
  MN_CHECK_LAUNCH();
  *spec = mn_keyspec{};
  spec->ndim = ndim;
  spec->margin = margin;
  spec->total_bits = -1;   // only known on the device
  spec->device_copy = spec_dev;
  return MN_OK;
}
