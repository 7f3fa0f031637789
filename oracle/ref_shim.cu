// C entry points over the reference's own CUDA functors, so that the tests can
// run the UNMODIFIED reference implementation of the hot path on a GPU and pin
// the CPU oracle against it.  TEST INFRASTRUCTURE ONLY: this file is compiled
// by oracle/build_ref.py together with the reference's .cu files, which are
// read in place from the reference checkout (never copied into this
// repository); the result is oracle/_ref/libminuet_ref.so.
//
// Instantiations used: int32 coordinates and indices, 3 dimensions, float
// features -- the combination the benchmark configurations exercise and the
// only feature type the reference enables (csrc/minuet/enabled_arguments.h).
#include <cublas_v2.h>

#include <cstdint>
#include <cstring>
#include <optional>
#include <string>

#include "minuet/cuda/context.cuh"
#include "minuet/cuda/functions/arg_sort_coodrinates.cuh"
#include "minuet/cuda/functions/query_sorted_index.cuh"
#include "minuet/cuda/functions/scan.cuh"
#include "minuet/cuda/functions/sparse_convolution.cuh"
#include "minuet/cuda/functions/unique_coordinates.cuh"

namespace {
std::string g_error;
cublasHandle_t g_cublas = nullptr;

template <typename F>
int guarded(F f) {
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
}

minuet::cuda::Context make_context(void *stream) {
  return minuet::cuda::Context(static_cast<cudaStream_t>(stream));
}
}  // namespace

using i32 = std::int32_t;
using i64 = std::int64_t;

extern "C" {

const char *ref_last_error() { return g_error.c_str(); }

int ref_arg_sort(i64 n, const i32 *coords, i32 *index, int flatten, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    minuet::cuda::ArgSortCoordinates().operator()<3, i32, i32>(n, coords, index, flatten != 0, ctx);
    ctx.Synchronize();
  });
}

int ref_multi_arg_sort(i64 n, i64 batch, const i32 *coords, const i32 *batch_dims, i32 *index,
                       int flatten, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    minuet::cuda::MultiArgSortCoordinates().operator()<3, i32, i32>(n, batch, coords, batch_dims,
                                                                    index, flatten != 0, ctx);
    ctx.Synchronize();
  });
}

// indices: int64 [n+1]; returns the unique count through *count; out holds n rows
int ref_unique(i64 n, const i32 *coords, i64 *indices, i32 *out, i64 *count, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    std::size_t u = 0;
    minuet::cuda::UniqueCoordinates().operator()<i32, i64, 3>(n, u, coords, indices, ctx);
    minuet::cuda::FillUniqueCoordinates().operator()<i32, i64, 3>(n, coords, indices, out, ctx);
    ctx.Synchronize();
    *count = (i64)u;
  });
}

// batched form as the torch binding calls it: num_batches = len(batch_dims)
int ref_multi_unique(i64 n, i64 batch_dims_len, const i32 *coords, const i32 *batch_dims,
                     i32 *indices, i32 *out, i64 *count, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    std::size_t u = 0;
    minuet::cuda::MultiUniqueCoordinates().operator()<i32, i32, 3>(batch_dims_len, n, u, coords,
                                                                  batch_dims, indices, ctx);
    minuet::cuda::FillUniqueCoordinates().operator()<i32, i32, 3>(n, coords, indices, out, ctx);
    ctx.Synchronize();
    *count = (i64)u;
  });
}

int ref_query(i64 S, i64 T, i64 O, const i32 *sources, const i32 *targets, const i32 *offsets,
              i32 *kernel_map, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    minuet::cuda::QuerySortedIndexWithOffsets().operator()<i32, i32, 3>(S, T, O, sources, targets,
                                                                       offsets, kernel_map, ctx);
    ctx.Synchronize();
  });
}

int ref_multi_query(i64 batch, i64 O, const i32 *sbd, const i32 *tbd, const i32 *sources,
                    const i32 *targets, const i32 *offsets, i32 *kernel_map, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    minuet::cuda::MultiQuerySortedIndexWithOffsets().operator()<i32, i32, 3>(
        batch, O, sbd, tbd, sources, targets, offsets, kernel_map, ctx);
    ctx.Synchronize();
  });
}

int ref_sizes(i64 O, i64 T, const i32 *kernel_map, i32 *sizes, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    minuet::cuda::ComputeKernelMapSizes().operator()<i32>(O, T, kernel_map, sizes, ctx);
    ctx.Synchronize();
  });
}

int ref_masks(i64 O, i64 S, i64 T, const i32 *kernel_map, const i32 *sizes, i32 *source_masks,
              i32 *target_masks, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    minuet::cuda::ComputeKernelMapMasks().operator()<i32>(O, S, T, kernel_map, sizes, source_masks,
                                                          target_masks, ctx);
    ctx.Synchronize();
  });
}

// threshold_mode: 0 = number, 1 = None
int ref_conv_forward(i64 S, i64 T, i64 O, int threshold_mode, double threshold, i64 parallel,
                     int allow_shortcut, i64 c_in, i64 c_out, const i32 *source_masks,
                     const i32 *target_masks, const i32 *order, const i32 *sizes,
                     const float *sources, const float *weights, float *targets, i64 gather_tile,
                     i64 scatter_tile, void *stream) {
  return guarded([&] {
    auto ctx = make_context(stream);
    if (g_cublas == nullptr) {
      if (cublasCreate(&g_cublas) != CUBLAS_STATUS_SUCCESS) throw std::runtime_error("cublasCreate failed");
    }
    cublasSetStream(g_cublas, static_cast<cudaStream_t>(stream));
    ctx.SetCUBLASHandle(g_cublas);
    std::optional<double> th;
    if (threshold_mode == 0) th = threshold;
    minuet::cuda::SparseConvolutionForward().operator()<i32, float>(
        S, T, O, th, parallel, allow_shortcut != 0, c_in, c_out, source_masks, target_masks, order,
        sizes, sources, weights, targets, gather_tile, scatter_tile, ctx);
    ctx.Synchronize();
    cudaDeviceSynchronize();
  });
}

}  // extern "C"
