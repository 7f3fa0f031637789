// CPU oracle for the Minuet sparse-convolution hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain C++17 + OpenMP, the
// semantics of the reference's Map step (coordinate arg-sort, unique, kernel
// map query, sizes, size order, masks) and of its Gather-GEMM-Scatter forward
// pass.  It is the checker the CUDA kernels are compared against and the CPU
// baseline that the benchmark times; the product never links or calls it.
//
// The reference ships no CPU implementation of this path (every functional
// wrapper raises NotImplementedError off-GPU: minuet/nn/functional/indexing.py:56,127,
// hash.py:25,50, scan.py:24,48, convolution.py:155), and no tests or golden
// vectors of its own.  Parity status: PINNED against outputs of the reference
// itself.  The reference's unmodified CUDA sources are compiled into
// oracle/_ref/libminuet_ref.so (oracle/build_ref.py); tests/test_reference_pin.py
// runs them on a GPU against this file (arg-sort, unique, kernel map, sizes,
// masks bit-exact, fp32 forward within 1e-5), and tests/test_golden.py checks
// this file against tests/golden/reference_golden.npz, which
// tests/golden/make_reference_golden.py recorded from the same library.  The
// size order is the one stage the reference leaves undefined (torch.sort ties);
// see orc_order.
//
// All coordinates are int32 [n, D] row-major (D <= 4), clouds are delimited by
// int64 prefix offsets batch_dims[B+1] (NULL = one cloud).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// Lexicographic comparison, dimension 0 most significant
// (csrc/minuet/common/functions.h:94-105).
inline int cmp_coord(const int32_t *a, const int32_t *b, int D) {
  for (int k = 0; k < D; k++) {
    if (a[k] != b[k]) return a[k] < b[k] ? -1 : 1;
  }
  return 0;
}

inline int cmp_coord_off(const int32_t *src, const int32_t *tgt,
                         const int32_t *off, int D) {
  // sign of (src - off) - tgt, evaluated without overflow
  for (int k = 0; k < D; k++) {
    int64_t a = (int64_t)src[k] - (int64_t)off[k];
    int64_t b = tgt[k];
    if (a != b) return a < b ? -1 : 1;
  }
  return 0;
}

inline int64_t cloud_of(int64_t row, int64_t nb, const int64_t *bd) {
  // largest g with bd[g] <= row
  int64_t lo = 0, hi = nb;
  while (hi - lo > 1) {
    int64_t mid = (lo + hi) >> 1;
    if (bd[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

}  // namespace

extern "C" {

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Stable arg-sort of coordinates, cloud-major then lexicographic.
// Reference: ArgSortCoordinates / MultiArgSortCoordinates
// (csrc/minuet/cuda/functions/arg_sort_coodrinates.cu:274-360, 363-469): the
// coordinates are flattened into one unsigned key over the per-cloud bounding
// box (kernels/flatten_coordinates.cuh:23-38) and radix-sorted (a stable sort),
// the batched form adds a stable pass on the cloud id (:454-468).  A stable
// comparison sort inside each cloud yields the same permutation.
void orc_arg_sort(int64_t n, int D, const int32_t *coords, int64_t nb,
                  const int64_t *batch_dims, int64_t *index) {
  int64_t one[2] = {0, n};
  if (batch_dims == nullptr) { batch_dims = one; nb = 1; }
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t g = 0; g < nb; g++) {
    int64_t lo = batch_dims[g], hi = batch_dims[g + 1];
    // flatten when the bounding box fits 64 bits, as the reference does
    int64_t cmin[4], cmax[4];
    for (int k = 0; k < D; k++) { cmin[k] = INT64_MAX; cmax[k] = INT64_MIN; }
    for (int64_t i = lo; i < hi; i++)
      for (int k = 0; k < D; k++) {
        cmin[k] = std::min<int64_t>(cmin[k], coords[i * D + k]);
        cmax[k] = std::max<int64_t>(cmax[k], coords[i * D + k]);
      }
    __int128 room = UINT64_MAX;
    bool flat = hi > lo;
    for (int k = 0; k < D && flat; k++) {
      __int128 size = (__int128)cmax[k] - cmin[k] + 1;
      if (room < size) flat = false; else room /= size;
    }
    if (flat) {
      std::vector<std::pair<uint64_t, int64_t>> kv(hi - lo);
      for (int64_t i = lo; i < hi; i++) {
        uint64_t key = 0;
        for (int k = 0; k < D; k++)
          key = key * (uint64_t)(cmax[k] - cmin[k] + 1) +
                (uint64_t)(coords[i * D + k] - cmin[k]);
        kv[i - lo] = {key, i};
      }
      std::stable_sort(kv.begin(), kv.end(),
                       [](const auto &a, const auto &b) { return a.first < b.first; });
      for (int64_t i = lo; i < hi; i++) index[i] = kv[i - lo].second;
    } else {
      std::iota(index + lo, index + hi, lo);
      std::stable_sort(index + lo, index + hi, [&](int64_t a, int64_t b) {
        return cmp_coord(coords + a * D, coords + b * D, D) < 0;
      });
    }
  }
}

// Unique over sorted coordinates.
// Reference: UniqueCoordinates / MultiUniqueCoordinates
// (csrc/minuet/cuda/functions/unique_coordinates.cu:16-46, 57-90): flag[i] = 1
// when row i differs from row i+1 or is the last row of its cloud;
// indices[0] = 0, indices[i+1] = sum(flag[0..i]); rows with flag set are copied
// to out[indices[i]] (kernels/fill_unique_coordinate.cuh:13-19).
// Returns the number of unique rows.  `out` must hold n rows.
int64_t orc_unique(int64_t n, int D, const int32_t *coords, int64_t nb,
                   const int64_t *batch_dims, int32_t *out, int64_t *indices) {
  indices[0] = 0;
  int64_t g = 0;
  for (int64_t i = 0; i < n; i++) {
    bool last = (i + 1 == n);
    if (batch_dims != nullptr) {
      while (g + 1 < nb && batch_dims[g + 1] <= i) g++;
      if (batch_dims[g + 1] == i + 1) last = true;
    }
    bool flag = last || cmp_coord(coords + i * D, coords + (i + 1) * D, D) != 0;
    indices[i + 1] = indices[i] + (flag ? 1 : 0);
    if (flag) std::memcpy(out + indices[i] * D, coords + i * D, sizeof(int32_t) * D);
  }
  return indices[n];
}

// Target coordinates of a strided convolution.
// Reference: KernelMapCache.get_target_coordinates
// (minuet/nn/convolutions.py:85-96): (C // ts) * ts with floor division, sort,
// unique, and target batch_dims = indices[source batch_dims].
// Returns U; out_coords holds n rows; out_batch_dims holds nb+1 entries.
int64_t orc_downsample(int64_t n, int D, const int32_t *coords,
                       const int32_t *tstride, int64_t nb,
                       const int64_t *batch_dims, int32_t *out_coords,
                       int64_t *out_batch_dims) {
  std::vector<int32_t> floored((size_t)n * D), sorted((size_t)n * D);
#pragma omp parallel for
  for (int64_t i = 0; i < n; i++)
    for (int k = 0; k < D; k++) {
      int32_t c = coords[i * D + k], s = tstride[k];
      int32_t q = c / s;
      if ((c % s != 0) && ((c < 0) != (s < 0))) q--;  // floor, as torch's //
      floored[i * D + k] = q * s;
    }
  std::vector<int64_t> index(n), indices(n + 1);
  orc_arg_sort(n, D, floored.data(), nb, batch_dims, index.data());
#pragma omp parallel for
  for (int64_t i = 0; i < n; i++)
    std::memcpy(&sorted[i * D], &floored[index[i] * D], sizeof(int32_t) * D);
  int64_t U = orc_unique(n, D, sorted.data(), nb, batch_dims, out_coords, indices.data());
  if (batch_dims != nullptr && out_batch_dims != nullptr)
    for (int64_t g = 0; g <= nb; g++) out_batch_dims[g] = indices[batch_dims[g]];
  return U;
}

// Kernel map: map[o, t] = s with sources[s] == targets[t] + offsets[o] inside
// the same cloud, else -1.
// Reference: QuerySortedIndexWithOffsets / MultiQuerySortedIndexWithOffsets
// (csrc/minuet/cuda/functions/query_sorted_index.cu:14-119, 122-204; the search
// itself is kernels/query_sorted_index_with_offsets.cuh:60-76: a lower-bound
// binary search of target in the list {source - offset}, equality test).
void orc_query(int64_t S, int64_t T, int64_t O, int D, const int32_t *sources,
               const int32_t *targets, const int32_t *offsets, int64_t nb,
               const int64_t *sbd, const int64_t *tbd, int32_t *map) {
  int64_t s_one[2] = {0, S}, t_one[2] = {0, T};
  if (sbd == nullptr) { sbd = s_one; tbd = t_one; nb = 1; }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t o = 0; o < O; o++) {
    for (int64_t g = 0; g < nb; g++) {
      const int32_t *off = offsets + o * D;
      int64_t slo = sbd[g], shi = sbd[g + 1];
      int64_t hint = slo;
      for (int64_t t = tbd[g]; t < tbd[g + 1]; t++) {
        const int32_t *tg = targets + t * D;
        // queries grow with t, so resume from the previous hit (galloping)
        int64_t lo = hint, step = 1, hi = hint;
        while (hi < shi && cmp_coord_off(sources + hi * D, tg, off, D) < 0) {
          lo = hi + 1; hi += step; step <<= 1;
        }
        if (hi > shi) hi = shi;
        while (lo < hi) {
          int64_t mid = (lo + hi) >> 1;
          if (cmp_coord_off(sources + mid * D, tg, off, D) < 0) lo = mid + 1; else hi = mid;
        }
        hint = lo;
        bool hit = lo < shi && cmp_coord_off(sources + lo * D, tg, off, D) == 0;
        map[o * T + t] = hit ? (int32_t)lo : -1;
      }
    }
  }
}

// sizes[o] = #{t : map[o, t] != -1}
// (ComputeKernelMapSizes, csrc/minuet/cuda/functions/scan.cu:221-290).
void orc_sizes(int64_t O, int64_t T, const int32_t *map, int32_t *sizes) {
#pragma omp parallel for
  for (int64_t o = 0; o < O; o++) {
    int32_t c = 0;
    for (int64_t t = 0; t < T; t++) c += map[o * T + t] != -1;
    sizes[o] = c;
  }
}

// Ascending size order (minuet/nn/convolutions.py:156-161 sorts with
// torch.sort, whose tie order is unspecified; this restatement breaks ties by
// offset index, i.e. a stable sort).
void orc_order(int64_t O, const int32_t *sizes, int32_t *order, int32_t *sorted_sizes) {
  std::vector<int32_t> idx(O);
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(),
                   [&](int32_t a, int32_t b) { return sizes[a] < sizes[b]; });
  for (int64_t i = 0; i < O; i++) { order[i] = idx[i]; sorted_sizes[i] = sizes[idx[i]]; }
}

// Masks from a kernel map whose rows are already in the order the masks use.
// Reference: ComputeKernelMapMasks (csrc/minuet/cuda/functions/scan.cu:293-365)
// and kernels/generate_masks_from_kernel_map.cuh:20-29: valid entries of row o
// are ranked by increasing t; source_masks[o, s] = target_masks[o, t] = rank,
// every other entry is -1.
void orc_masks(int64_t O, int64_t S, int64_t T, const int32_t *map,
               int32_t *source_masks, int32_t *target_masks) {
#pragma omp parallel for
  for (int64_t o = 0; o < O; o++) {
    std::fill(source_masks + o * S, source_masks + (o + 1) * S, -1);
    int32_t r = 0;
    for (int64_t t = 0; t < T; t++) {
      int32_t s = map[o * T + t];
      if (s != -1) {
        source_masks[o * S + s] = r;
        target_masks[o * T + t] = r;
        r++;
      } else {
        target_masks[o * T + t] = -1;
      }
    }
  }
}

// Padding-bucket planner over size-sorted offsets.
// Reference: GeneratePaddingBuckets and ComputeCumsumKernelPaddedSizes
// (csrc/minuet/cuda/functions/sparse_convolution.cu:17-43, 273-292).
// mode: 0 = threshold is a number, 1 = threshold is None (fuse everything).
// buckets holds up to O+1 entries, cumsum_pad O+1.  Returns #buckets.
int64_t orc_plan_buckets(int64_t O, const int32_t *sizes, int mode,
                         double threshold, int64_t *buckets, int64_t *cumsum_pad) {
  int64_t nbk = 0;
  buckets[nbk++] = 0;
  for (int64_t i = 0; i < O; i++) {
    int64_t j = i;
    uint64_t actual = (uint64_t)sizes[i], summit = (uint64_t)sizes[i];
    while (i + 1 < O) {
      actual += (uint64_t)sizes[i + 1];
      summit = std::max<uint64_t>(summit, (uint64_t)sizes[i + 1]);
      uint64_t padded = summit * (uint64_t)((i + 1) - j + 1);
      double redundancy = (double)(padded - actual) / (double)actual;
      if (mode == 0 && (threshold < 0 || redundancy > threshold)) break;
      i++;
    }
    buckets[nbk++] = i + 1;
  }
  cumsum_pad[0] = 0;
  for (int64_t b = 0; b + 1 < nbk; b++) {
    int64_t summit = 0;
    for (int64_t j = buckets[b]; j < buckets[b + 1]; j++)
      summit = std::max<int64_t>(summit, sizes[j]);
    for (int64_t j = buckets[b]; j < buckets[b + 1]; j++)
      cumsum_pad[j + 1] = cumsum_pad[j] + summit;
  }
  return nbk - 1;
}

// Forward pass out[t,:] = sum_o sum_{(s,t) in map[o]} in[s,:] . W[order[o]]
// Reference: SparseConvolutionForward::operator()
// (csrc/minuet/cuda/functions/sparse_convolution.cu:505-661): offsets are
// visited in mask-row (size-sorted) order, each row's GEMM is accumulated into
// the target row (kernels/padded_scatter_warp_optimized.cuh:34-53), and when
// allow_shortcut and the last row covers every voxel it is added last as a
// dense product (:558-564, :647-660).  Accumulation is fp32 per product
// (acc64 = 0) or fp64 throughout (acc64 = 1, the tolerance reference).
void orc_conv_forward(int64_t S, int64_t T, int64_t O, int64_t Cin, int64_t Cout,
                      const int32_t *source_masks, const int32_t *target_masks,
                      const int32_t *order /* may be NULL */, const float *in,
                      const float *weights, float *out, int acc64) {
  // per mask row: rank -> source row
  std::vector<std::vector<int32_t>> src_of_rank(O);
#pragma omp parallel for
  for (int64_t o = 0; o < O; o++) {
    int32_t n = 0;
    for (int64_t s = 0; s < S; s++) n = std::max(n, source_masks[o * S + s] + 1);
    src_of_rank[o].assign(n, -1);
    for (int64_t s = 0; s < S; s++) {
      int32_t r = source_masks[o * S + s];
      if (r != -1) src_of_rank[o][r] = (int32_t)s;
    }
  }
#pragma omp parallel
  {
    std::vector<double> acc_d(Cout);
    std::vector<float> acc_f(Cout), prod(Cout);
#pragma omp for schedule(dynamic, 256)
    for (int64_t t = 0; t < T; t++) {
      if (acc64) std::fill(acc_d.begin(), acc_d.end(), 0.0);
      else std::fill(acc_f.begin(), acc_f.end(), 0.f);
      for (int64_t o = 0; o < O; o++) {
        int32_t r = target_masks[o * T + t];
        if (r == -1) continue;
        int32_t s = src_of_rank[o][r];
        const float *w = weights + (order ? order[o] : o) * Cin * Cout;
        const float *x = in + (int64_t)s * Cin;
        if (acc64) {
          for (int64_t c = 0; c < Cin; c++) {
            double xv = x[c];
            const float *wr = w + c * Cout;
            for (int64_t d = 0; d < Cout; d++) acc_d[d] += xv * (double)wr[d];
          }
        } else {
          std::fill(prod.begin(), prod.end(), 0.f);
          for (int64_t c = 0; c < Cin; c++) {
            float xv = x[c];
            const float *wr = w + c * Cout;
            for (int64_t d = 0; d < Cout; d++) prod[d] += xv * wr[d];
          }
          for (int64_t d = 0; d < Cout; d++) acc_f[d] += prod[d];
        }
      }
      float *y = out + t * Cout;
      if (acc64) for (int64_t d = 0; d < Cout; d++) y[d] = (float)acc_d[d];
      else for (int64_t d = 0; d < Cout; d++) y[d] = acc_f[d];
    }
  }
}

}  // extern "C"
