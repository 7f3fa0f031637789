// Per-voxel feature averaging for voxelisation: the step before the hot path
// (minuet/nn/functional/voxelize.py:10-35 in the reference, which stops at the
// unique coordinates and leaves the features to the caller).
//
// After floor -> arg-sort -> unique, the points of one voxel are CONTIGUOUS in
// sorted order: run_ids[i] (the unique op's index array) is the voxel of sorted
// row i and never decreases.  One warp owns one sorted row; the warp of a run's
// first row walks the run, sums the feature rows in fp32 in sorted order (a fixed
// order: the result does not depend on scheduling, no atomics) and writes the
// mean once.  Lanes stride over channels, so a row is read with coalesced loads.
#include "mn_common.cuh"

namespace mn {
namespace {

template <typename T> __device__ __forceinline__ float vx_to_f32(T v);
template <> __device__ __forceinline__ float vx_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float vx_to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float vx_to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T vx_from_f32(float v);
template <> __device__ __forceinline__ float vx_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half vx_from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 vx_from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

constexpr int kVxThreads = 256;
constexpr int kVxChunk = 8;   // channels per lane held in registers at a time

template <typename T>
__global__ void __launch_bounds__(kVxThreads)
voxel_mean_kernel(const T *__restrict__ features, int64_t n, int channels,
                  const int64_t *__restrict__ sorted_index, const int64_t *__restrict__ run_ids,
                  T *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kVxThreads / 32);
  for (int64_t i = (int64_t)blockIdx.x * (kVxThreads / 32) + (threadIdx.x >> 5); i < n; i += warps) {
    const int64_t u = __ldg(run_ids + i);
    if (i > 0 && __ldg(run_ids + i - 1) == u) continue;   // not the first row of its voxel
    int64_t end = i + 1;
    while (end < n && __ldg(run_ids + end) == u) end++;
    const float inv = 1.0f / (float)(end - i);
    for (int c0 = lane; c0 < channels; c0 += 32 * kVxChunk) {
      float acc[kVxChunk];
#pragma unroll
      for (int k = 0; k < kVxChunk; k++) acc[k] = 0.f;
      for (int64_t j = i; j < end; j++) {
        const T *row = features + __ldg(sorted_index + j) * channels;
#pragma unroll
        for (int k = 0; k < kVxChunk; k++) {
          const int c = c0 + 32 * k;
          if (c < channels) acc[k] += vx_to_f32<T>(row[c]);
        }
      }
#pragma unroll
      for (int k = 0; k < kVxChunk; k++) {
        const int c = c0 + 32 * k;
        if (c < channels) out[u * channels + c] = vx_from_f32<T>(acc[k] * inv);
      }
    }
  }
}

template <typename T>
mn_status run_voxel_mean(const void *features, int64_t n, int64_t channels,
                         const int64_t *sorted_index, const int64_t *run_ids, void *out,
                         cudaStream_t st) {
  const int blocks = (int)std::min<int64_t>(kNumSMs * 32, div_up(n, kVxThreads / 32));
  MN_LAUNCH("voxel_mean_kernel", st,
            voxel_mean_kernel<T><<<blocks, kVxThreads, 0, st>>>(
                static_cast<const T *>(features), n, (int)channels, sorted_index, run_ids,
                static_cast<T *>(out)));
  return MN_OK;
}

}  // namespace
}  // namespace mn

using namespace mn;

extern "C" mn_status mn_voxel_mean(const void *features, int64_t n, int64_t channels, mn_dtype dtype,
                                   const int64_t *sorted_index, const int64_t *run_ids,
                                   void *means_out, void *stream) {
  MN_CHECK_ARG(n >= 0 && channels >= 1 && channels < (1 << 20), "voxel_mean: bad shape");
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(features != nullptr && sorted_index != nullptr && run_ids != nullptr &&
                   means_out != nullptr, "voxel_mean: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MN_F32: return run_voxel_mean<float>(features, n, channels, sorted_index, run_ids, means_out, st);
    case MN_F16: return run_voxel_mean<__half>(features, n, channels, sorted_index, run_ids, means_out, st);
    case MN_BF16:
      return run_voxel_mean<__nv_bfloat16>(features, n, channels, sorted_index, run_ids, means_out, st);
  }
  set_error("voxel_mean: unknown dtype %d", (int)dtype);
  return MN_ERR_BAD_ARG;
}
