// Device helpers that turn one coordinate row into its packed 64-bit key, and
// the key layout computed from a bounding box (host and device).
#pragma once

#include "mn_common.cuh"

namespace mn {

// Key layout from a bounding box: dimension ndim-1 sits at bit 0, every field
// has `margin` spare values on both sides, the cloud id takes the top bits.
// Returns false when the layout needs more than 63 bits (the spec is still
// filled in, but keys built from it would overlap).
__host__ __device__ inline bool compute_keyspec(const int32_t *minmax, int ndim, int64_t num_clouds,
                                                int32_t margin, mn_keyspec *spec) {
  spec->ndim = ndim;
  spec->margin = margin;
  spec->device_copy = nullptr;
  for (int k = 0; k < MN_MAX_NDIM; k++) {
    spec->shift[k] = 0; spec->bits[k] = 0; spec->base[k] = 0; spec->extent[k] = 0;
  }
  int shift = 0;
  for (int k = ndim - 1; k >= 0; k--) {
    int64_t lo = minmax[k], hi = minmax[4 + k];
    if (lo > hi) { lo = 0; hi = 0; }  // empty input
    spec->base[k] = lo - margin;
    spec->extent[k] = (hi + margin) - spec->base[k];
    int bits = 0;
    for (uint64_t v = (uint64_t)spec->extent[k]; v != 0; v >>= 1) bits++;
    spec->bits[k] = bits < 1 ? 1 : bits;
    spec->shift[k] = shift;
    shift += spec->bits[k];
  }
  spec->cloud_shift = shift;
  int cloud_bits = 0;
  for (uint64_t v = (uint64_t)(num_clouds - 1); v != 0; v >>= 1) cloud_bits++;
  spec->cloud_bits = cloud_bits;
  spec->total_bits = shift + cloud_bits;
  return spec->total_bits <= 63;
}

#ifdef __CUDACC__
__device__ __forceinline__ int floor_to(int c, int s) {
  int q = c / s;
  if ((c % s != 0) && (c < 0)) q--;
  return q * s;
}

// largest g with bd[g] <= row
__device__ __forceinline__ int cloud_of(const int64_t *bd, int num_clouds, int64_t row) {
  int lo = 0, hi = num_clouds;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (bd[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

struct PackParams {
  SpecRef spec;
  int32_t tstride[4];
  int32_t has_stride;
};

__device__ __forceinline__ uint64_t pack_one(const int (&c)[4], int ndim, uint64_t cloud,
                                             const mn_keyspec &spec, const PackParams &p,
                                             bool &bad) {
  uint64_t key = cloud << spec.cloud_shift;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    if (k < ndim) {
      int v = p.has_stride ? floor_to(c[k], p.tstride[k]) : c[k];
      int64_t f = (int64_t)v - spec.base[k];
      if (f < 0 || f > spec.extent[k]) {
        bad = true;
        f = f < 0 ? 0 : spec.extent[k];
      }
      key |= (uint64_t)f << spec.shift[k];
    }
  }
  return key;
}
#endif

}  // namespace mn
