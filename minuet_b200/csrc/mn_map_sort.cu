// Map step, part 1: radix sort of packed keys, unique, and the fused target
// coordinate build of strided convolutions.
//
// The reference sorts with cub::DeviceRadixSort::SortPairs over all 8*sizeof(key)
// bits (csrc/minuet/cuda/functions/arg_sort_coodrinates.cu:346-357) and removes
// duplicates with cub::DeviceScan + a compaction kernel
// (csrc/minuet/cuda/functions/unique_coordinates.cu:16-101).  Here the sort is a
// hand-written stable LSD radix sort (9-bit digits, warp match ranking) that
// only visits the key bits the bounding box uses, and unique/compaction is one
// count + scan + compact pipeline that can also unpack keys back to coordinates.
#include "mn_common.cuh"

#include <algorithm>
#include <mutex>

namespace mn {

namespace {

// ---------------------------------------------------------------------------
// radix sort
// ---------------------------------------------------------------------------
constexpr int kRsThreads = 256;
constexpr int kRsWarps = kRsThreads / 32;
constexpr int kRsItems = 4;                       // keys per thread
constexpr int kRsTile = kRsThreads * kRsItems;    // 1024 keys per block
constexpr int kRsBits = 9;                        // digit width: 4 passes cover 36 key bits
constexpr int kRadix = 1 << kRsBits;

__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// block_hist[d * nblocks + b] = number of keys of block b whose digit is d
__global__ void __launch_bounds__(kRsThreads)
radix_hist_kernel(const uint64_t *__restrict__ keys, int64_t n, int shift,
                  uint32_t *__restrict__ block_hist, int nblocks) {
  __shared__ uint32_t hist[kRadix];
  for (int d = threadIdx.x; d < kRadix; d += kRsThreads) hist[d] = 0;
  __syncthreads();
  const int64_t tile0 = (int64_t)blockIdx.x * kRsTile;
#pragma unroll 4
  for (int c = 0; c < kRsItems; c++) {
    int64_t i = tile0 + c * kRsThreads + threadIdx.x;
    if (i < n) atomicAdd(&hist[(keys[i] >> shift) & (kRadix - 1)], 1u);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < kRadix; d += kRsThreads)
    block_hist[(size_t)d * nblocks + blockIdx.x] = hist[d];
}

// One warp per digit: exclusive scan of that digit's row over the blocks, in
// place, and the digit total.
__global__ void __launch_bounds__(kRsThreads)
radix_scan_kernel(uint32_t *__restrict__ block_hist, int nblocks,
                  uint32_t *__restrict__ digit_total) {
  const int lane = threadIdx.x & 31;
  const int d = blockIdx.x * kRsWarps + (threadIdx.x >> 5);
  uint32_t *row = block_hist + (size_t)d * nblocks;
  uint32_t carry = 0;
  for (int b0 = 0; b0 < nblocks; b0 += 32) {
    int b = b0 + lane;
    uint32_t v = b < nblocks ? row[b] : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, inc, s);
      if (lane >= s) inc += t;
    }
    if (b < nblocks) row[b] = carry + inc - v;
    carry += __shfl_sync(0xffffffffu, inc, 31);
  }
  if (lane == 0) digit_total[d] = carry;
}

// Stable scatter.  Warp w owns kRsItems*32 consecutive keys of the tile and walks
// them in chunks of 32 consecutive keys; inside a chunk lanes with equal
// digits find each other with match.any, the lowest lane bumps the warp's digit
// counter, and every lane's rank is counter + number of equal lanes below it.
template <bool kHasVals>
__global__ void __launch_bounds__(kRsThreads)
radix_scatter_kernel(const uint64_t *__restrict__ keys_in, const int32_t *__restrict__ vals_in,
                     int64_t n, int shift, const uint32_t *__restrict__ block_hist, int nblocks,
                     const uint32_t *__restrict__ digit_total,
                     uint64_t *__restrict__ keys_out, int32_t *__restrict__ vals_out) {
  __shared__ uint32_t s_cnt[kRsWarps][kRadix];
  __shared__ uint32_t s_base[kRadix];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kRsWarps * kRadix; i += kRsThreads) (&s_cnt[0][0])[i] = 0;
  {
    // exclusive scan of the digit totals by warp 0 (kRadix / 32 digits per lane)
    if (warp == 0) {
      constexpr int kPerLane = kRadix / 32;
      uint32_t v[kPerLane], sum = 0;
#pragma unroll
      for (int j = 0; j < kPerLane; j++) { v[j] = digit_total[lane * kPerLane + j]; sum += v[j]; }
      uint32_t inc = sum;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, inc, s);
        if (lane >= s) inc += t;
      }
      uint32_t run = inc - sum;
#pragma unroll
      for (int j = 0; j < kPerLane; j++) { s_base[lane * kPerLane + j] = run; run += v[j]; }
    }
  }
  __syncthreads();

  const int64_t seg0 = (int64_t)blockIdx.x * kRsTile + warp * (kRsItems * 32);
  uint64_t key[kRsItems];
  uint32_t rank[kRsItems];
  const unsigned lt = lanemask_lt();
#pragma unroll
  for (int c = 0; c < kRsItems; c++) {
    const int64_t i = seg0 + c * 32 + lane;
    const bool valid = i < n;
    key[c] = valid ? keys_in[i] : 0ull;
    const unsigned d = valid ? (unsigned)((key[c] >> shift) & (kRadix - 1)) : (unsigned)kRadix;
    const unsigned peers = __match_any_sync(0xffffffffu, d);
    const int leader = __ffs(peers) - 1;
    uint32_t old = 0;
    if (lane == leader && valid) {
      old = s_cnt[warp][d];
      s_cnt[warp][d] = old + __popc(peers);
    }
    old = __shfl_sync(0xffffffffu, old, leader);
    rank[c] = old + __popc(peers & lt);
    __syncwarp();
  }
  __syncthreads();
  for (int d = threadIdx.x; d < kRadix; d += kRsThreads) {
    uint32_t run = s_base[d] + block_hist[(size_t)d * nblocks + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kRsWarps; w++) {
      uint32_t t = s_cnt[w][d];
      s_cnt[w][d] = run;
      run += t;
    }
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < kRsItems; c++) {
    const int64_t i = seg0 + c * 32 + lane;
    if (i < n) {
      const unsigned d = (unsigned)((key[c] >> shift) & (kRadix - 1));
      const uint32_t pos = s_cnt[warp][d] + rank[c];
      keys_out[pos] = key[c];
      if (kHasVals) vals_out[pos] = vals_in != nullptr ? vals_in[i] : (int32_t)i;
    }
  }
}

__global__ void widen_index_kernel(const int32_t *__restrict__ in, int64_t n,
                                   int64_t *__restrict__ out) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gsz) out[i] = in[i];
}

__global__ void iota_index_kernel(int64_t n, int64_t *__restrict__ out) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gsz) out[i] = i;
}

// ---------------------------------------------------------------------------
// unique: count -> scan -> compact
// ---------------------------------------------------------------------------
constexpr int kUqThreads = 256;
constexpr int kUqItems = 8;
constexpr int kUqTile = kUqThreads * kUqItems;  // 2048 rows per block

struct RowsView {  // sorted coordinate rows
  const int32_t *coords;
  const int64_t *batch_dims;
  int num_clouds;
  int ndim;
  int64_t n;
  // true when row i closes a run: it differs from row i+1, is the last row, or
  // row i+1 opens a new cloud (unique_coordinates.cu:16-26, 57-70)
  __device__ __forceinline__ bool closes(int64_t i) const {
    if (i + 1 >= n) return true;
    bool same = true;
    for (int k = 0; k < ndim; k++) same &= coords[i * ndim + k] == coords[(i + 1) * ndim + k];
    if (!same) return true;
    if (batch_dims != nullptr) {
      int lo = 0, hi = num_clouds;  // is i+1 a cloud start?
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (batch_dims[mid] < i + 1) lo = mid + 1; else hi = mid;
      }
      if (batch_dims[lo] == i + 1) return true;
    }
    return false;
  }
};

struct KeysView {  // sorted packed keys; the cloud id is part of the key
  const uint64_t *keys;
  int64_t n;
  __device__ __forceinline__ bool closes(int64_t i) const {
    return i + 1 >= n || keys[i] != keys[i + 1];
  }
};

template <typename View>
__global__ void __launch_bounds__(kUqThreads)
unique_count_kernel(const View v, uint32_t *__restrict__ block_counts) {
  const int64_t base = (int64_t)blockIdx.x * kUqTile + (int64_t)threadIdx.x * kUqItems;
  uint32_t c = 0;
#pragma unroll
  for (int j = 0; j < kUqItems; j++) {
    int64_t i = base + j;
    if (i < v.n && v.closes(i)) c++;
  }
  c = __reduce_add_sync(0xffffffffu, c);
  __shared__ uint32_t s[kUqThreads / 32];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < kUqThreads / 32; w++) t += s[w];
    block_counts[blockIdx.x] = t;
  }
}

// Single block: exclusive scan of the block counts in place, total -> *total
// (and, when given, *total64).
__global__ void __launch_bounds__(1024)
scan_blocks_kernel(uint32_t *__restrict__ counts, int nblocks, uint32_t *__restrict__ total,
                   int64_t *__restrict__ total64) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nblocks; b0 += 1024) {
    const int b = b0 + threadIdx.x;
    const uint32_t v = b < nblocks ? counts[b] : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, inc, s);
      if (lane >= s) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      uint32_t w = s_warp[lane], winc = w;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, winc, s);
        if (lane >= s) winc += t;
      }
      s_warp[lane] = winc - w;
    }
    __syncthreads();
    const uint32_t carry = s_carry;
    if (b < nblocks) counts[b] = carry + s_warp[warp] + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = carry + s_warp[warp] + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    *total = s_carry;
    if (total64 != nullptr) *total64 = s_carry;
  }
}

struct CoordSink {  // reference-API unique: rows + inclusive index array
  const int32_t *coords;
  int ndim;
  int32_t *out_rows;
  int64_t *indices;  // [n+1]
  __device__ __forceinline__ void index(int64_t i, uint32_t inclusive) const {
    indices[i + 1] = inclusive;
  }
  __device__ __forceinline__ void emit(int64_t i, uint32_t pos) const {
    for (int k = 0; k < ndim; k++) out_rows[(int64_t)pos * ndim + k] = coords[i * ndim + k];
  }
};

struct KeySink {  // fused path: unique keys + unpacked coordinates
  const uint64_t *keys;
  mn_keyspec spec;
  uint64_t *out_keys;
  int32_t *out_rows;
  __device__ __forceinline__ void index(int64_t, uint32_t) const {}
  __device__ __forceinline__ void emit(int64_t i, uint32_t pos) const {
    const uint64_t key = keys[i];
    out_keys[pos] = key;
    for (int k = 0; k < spec.ndim; k++) {
      uint64_t f = (key >> spec.shift[k]) & ((1ull << spec.bits[k]) - 1ull);
      out_rows[(int64_t)pos * spec.ndim + k] = (int32_t)((int64_t)f + spec.base[k]);
    }
  }
};

template <typename View, typename Sink>
__global__ void __launch_bounds__(kUqThreads)
unique_compact_kernel(const View v, const Sink sink, const uint32_t *__restrict__ block_offsets) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t base = (int64_t)blockIdx.x * kUqTile + (int64_t)threadIdx.x * kUqItems;
  bool flag[kUqItems];
  uint32_t c = 0;
#pragma unroll
  for (int j = 0; j < kUqItems; j++) {
    int64_t i = base + j;
    flag[j] = i < v.n && v.closes(i);
    c += flag[j];
  }
  uint32_t inc = c;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, inc, s);
    if (lane >= s) inc += t;
  }
  __shared__ uint32_t s_warp[kUqThreads / 32];
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  uint32_t run = block_offsets[blockIdx.x] + inc - c;
  for (int w = 0; w < warp; w++) run += s_warp[w];
#pragma unroll
  for (int j = 0; j < kUqItems; j++) {
    int64_t i = base + j;
    if (i < v.n) {
      if (flag[j]) sink.emit(i, run);
      run += flag[j];
      sink.index(i, run);
    }
  }
}

// out_bd[g] = number of unique keys whose cloud id is < g.  One warp per cloud
// boundary: a 32-ary ballot search (4 rounds of loads for half a million keys
// instead of the 19 dependent loads of a binary search).
__global__ void __launch_bounds__(128)
cloud_starts_kernel(const uint64_t *__restrict__ keys, const int64_t *__restrict__ count,
                    int cloud_shift, int num_clouds, int64_t *__restrict__ out_bd) {
  const int lane = threadIdx.x & 31;
  const int g = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g > num_clouds) return;
  const uint64_t q = (uint64_t)g << cloud_shift;
  int64_t lo = 0, hi = *count;
  for (int round = 0; round < 16; round++) {
    const int64_t len = hi - lo;
    if (len <= 0) break;
    const int64_t stride = (len + 31) >> 5;
    const int64_t idx = lo + (int64_t)(lane + 1) * stride - 1;
    const bool pred = idx < hi && keys[idx] < q;
    const int c = __popc(__ballot_sync(0xffffffffu, pred));
    if (stride == 1) { lo += c; break; }
    const int64_t nlo = min(lo + (int64_t)c * stride, hi);
    hi = min(hi, nlo + stride - 1);
    lo = nlo;
  }
  if (lane == 0) out_bd[g] = lo;
}

__global__ void zero_index0_kernel(int64_t *indices) { indices[0] = 0; }

}  // namespace

size_t radix_sort_workspace_bytes(int64_t n) {
  int64_t nblocks = std::max<int64_t>(1, div_up(n, kRsTile));
  return align_up((size_t)nblocks * kRadix * sizeof(uint32_t), 256) + align_up(kRadix * sizeof(uint32_t), 256);
}

// Stable LSD sort of `keys` on bits [begin_bit, end_bit), ping-ponging between
// keys and keys_tmp.  With vals/vals_tmp given, int32 payloads move with the
// keys; iota_vals makes the first pass use the element index as payload instead
// of reading vals.  *result_in_tmp tells which buffers hold the result.
mn_status launch_radix_sort(uint64_t *keys, uint64_t *keys_tmp, int32_t *vals,
                            int32_t *vals_tmp, bool iota_vals, int64_t n, int begin_bit,
                            int end_bit, Workspace &ws, bool *result_in_tmp,
                            cudaStream_t st) {
  *result_in_tmp = false;
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(n < (1ll << 31), "radix sort: n = %lld exceeds 2^31-1", (long long)n);
  if (end_bit <= begin_bit) end_bit = begin_bit + 1;
  const int nblocks = (int)div_up(n, kRsTile);
  uint32_t *block_hist = ws.take<uint32_t>((size_t)nblocks * kRadix);
  uint32_t *digit_total = ws.take<uint32_t>(kRadix);
  MN_CHECK_WS(ws);
  const bool has_vals = vals != nullptr && vals_tmp != nullptr;
  uint64_t *kin = keys, *kout = keys_tmp;
  int32_t *vin = vals, *vout = vals_tmp;
  bool first = true;
  for (int shift = begin_bit; shift < end_bit; shift += kRsBits) {
    MN_LAUNCH("radix_hist_kernel", st, radix_hist_kernel<<<nblocks, kRsThreads, 0, st>>>(kin, n, shift, block_hist, nblocks));
    MN_LAUNCH("radix_scan_kernel", st, radix_scan_kernel<<<kRadix / kRsWarps, kRsThreads, 0, st>>>(block_hist, nblocks, digit_total));
    {
    LaunchScope scope("radix_scatter_kernel", st);
    if (has_vals) {
      radix_scatter_kernel<true><<<nblocks, kRsThreads, 0, st>>>(
          kin, (first && iota_vals) ? nullptr : vin, n, shift, block_hist, nblocks,
          digit_total, kout, vout);
    } else {
      radix_scatter_kernel<false><<<nblocks, kRsThreads, 0, st>>>(
          kin, nullptr, n, shift, block_hist, nblocks, digit_total, kout, nullptr);
    }
    }
    MN_CHECK_LAUNCH();
    std::swap(kin, kout);
    std::swap(vin, vout);
    *result_in_tmp = !*result_in_tmp;
    first = false;
  }
  return MN_OK;
}

}  // namespace mn

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
using namespace mn;

extern "C" mn_status mn_arg_sort_coordinates(const int32_t *coords, int64_t n, int ndim,
                                             const int64_t *batch_dims, int64_t num_clouds,
                                             const mn_keyspec *spec, int64_t *index_out,
                                             int32_t *status_dev, void *ws_ptr,
                                             size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(n >= 0 && ndim >= 1 && ndim <= MN_MAX_NDIM, "arg_sort: bad n/ndim");
  MN_CHECK_ARG(spec != nullptr && spec->ndim == ndim, "arg_sort: key spec missing or of another ndim");
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(coords != nullptr && index_out != nullptr && status_dev != nullptr,
               "arg_sort: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace ws(ws_ptr, ws_bytes);
  uint64_t *keys = ws.take<uint64_t>(n), *keys_tmp = ws.take<uint64_t>(n);
  int32_t *vals = ws.take<int32_t>(n), *vals_tmp = ws.take<int32_t>(n);
  MN_CHECK_WS(ws);
  MN_RETURN_IF(launch_pack(coords, n, ndim, batch_dims, num_clouds, nullptr, *spec, keys,
                           status_dev, st));
  bool in_tmp = false;
  MN_RETURN_IF(launch_radix_sort(keys, keys_tmp, vals, vals_tmp, true, n, 0, spec->total_bits,
                                 ws, &in_tmp, st));
  const int blocks = (int)std::min<int64_t>(kNumSMs * 8, div_up(n, 256));
  MN_LAUNCH("widen_index_kernel", st, widen_index_kernel<<<blocks, 256, 0, st>>>(in_tmp ? vals_tmp : vals, n, index_out));
  return MN_OK;
}

extern "C" mn_status mn_unique_coordinates(const int32_t *coords, int64_t n, int ndim,
                                           const int64_t *batch_dims, int64_t num_clouds,
                                           int32_t *unique_out, int64_t *indices_out,
                                           void *ws_ptr, size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(n >= 0 && ndim >= 1 && ndim <= MN_MAX_NDIM, "unique: bad n/ndim");
  MN_CHECK_ARG(indices_out != nullptr, "unique: null indices");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MN_LAUNCH("zero_index0_kernel", st, zero_index0_kernel<<<1, 1, 0, st>>>(indices_out));
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(coords != nullptr && unique_out != nullptr, "unique: null pointer");
  MN_CHECK_ARG(n < (1ll << 31), "unique: n exceeds 2^31-1");
  Workspace ws(ws_ptr, ws_bytes);
  const int nblocks = (int)div_up(n, kUqTile);
  uint32_t *counts = ws.take<uint32_t>(nblocks);
  uint32_t *total = ws.take<uint32_t>(1);
  MN_CHECK_WS(ws);
  RowsView view{coords, batch_dims, batch_dims ? (int)num_clouds : 1, ndim, n};
  CoordSink sink{coords, ndim, unique_out, indices_out};
  MN_LAUNCH("unique_count_kernel", st, unique_count_kernel<RowsView><<<nblocks, kUqThreads, 0, st>>>(view, counts));
  MN_LAUNCH("scan_blocks_kernel", st, scan_blocks_kernel<<<1, 1024, 0, st>>>(counts, nblocks, total, nullptr));
  MN_LAUNCH("unique_compact_kernel", st, unique_compact_kernel<RowsView, CoordSink><<<nblocks, kUqThreads, 0, st>>>(view, sink, counts));
  return MN_OK;
}

extern "C" mn_status mn_downsample_coordinates(
    const int32_t *coords, int64_t n, int ndim, const int64_t *batch_dims, int64_t num_clouds,
    const int32_t *tstride, const mn_keyspec *spec, int32_t *unique_out, uint64_t *keys_out,
    int64_t *out_batch_dims, int64_t *count_dev, int32_t *status_dev, void *ws_ptr,
    size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(n >= 0 && ndim >= 1 && ndim <= MN_MAX_NDIM, "downsample: bad n/ndim");
  MN_CHECK_ARG(spec != nullptr && spec->ndim == ndim, "downsample: key spec missing or of another ndim");
  MN_CHECK_ARG(tstride != nullptr && count_dev != nullptr && status_dev != nullptr,
               "downsample: null pointer");
  MN_CHECK_ARG(n < (1ll << 31), "downsample: n exceeds 2^31-1");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    MN_CHECK_CUDA(cudaMemsetAsync(count_dev, 0, sizeof(int64_t), st));
    if (batch_dims != nullptr && out_batch_dims != nullptr)
      MN_CHECK_CUDA(cudaMemsetAsync(out_batch_dims, 0, sizeof(int64_t) * (num_clouds + 1), st));
    return MN_OK;
  }
  MN_CHECK_ARG(coords != nullptr && unique_out != nullptr && keys_out != nullptr,
               "downsample: null pointer");
  for (int k = 0; k < ndim; k++)
    MN_CHECK_ARG(tstride[k] >= 1 && tstride[k] - 1 <= spec->margin,
                 "downsample: stride %d needs a key margin >= %d (have %d)", tstride[k],
                 tstride[k] - 1, spec->margin);
  Workspace ws(ws_ptr, ws_bytes);
  uint64_t *keys = ws.take<uint64_t>(n), *keys_tmp = ws.take<uint64_t>(n);
  const int nblocks = (int)div_up(n, kUqTile);
  uint32_t *counts = ws.take<uint32_t>(nblocks);
  uint32_t *total = ws.take<uint32_t>(1);
  MN_CHECK_WS(ws);
  MN_RETURN_IF(launch_pack(coords, n, ndim, batch_dims, num_clouds, tstride, *spec, keys,
                           status_dev, st));
  bool in_tmp = false;
  MN_RETURN_IF(launch_radix_sort(keys, keys_tmp, nullptr, nullptr, false, n, 0,
                                 spec->total_bits, ws, &in_tmp, st));
  const uint64_t *sorted = in_tmp ? keys_tmp : keys;
  KeysView view{sorted, n};
  KeySink sink{sorted, *spec, keys_out, unique_out};
  MN_LAUNCH("unique_count_kernel", st, unique_count_kernel<KeysView><<<nblocks, kUqThreads, 0, st>>>(view, counts));
  MN_LAUNCH("scan_blocks_kernel", st, scan_blocks_kernel<<<1, 1024, 0, st>>>(counts, nblocks, total, count_dev));
  MN_LAUNCH("unique_compact_kernel", st, unique_compact_kernel<KeysView, KeySink><<<nblocks, kUqThreads, 0, st>>>(view, sink, counts));
  if (batch_dims != nullptr && out_batch_dims != nullptr) {
    const int nb = (int)num_clouds + 1;
    MN_LAUNCH("cloud_starts_kernel", st, cloud_starts_kernel<<<(nb + 3) / 4, 128, 0, st>>>(keys_out, count_dev, spec->cloud_shift,
                                                           (int)num_clouds, out_batch_dims));
  }
  return MN_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free variant of mn_unique_coordinates
// ---------------------------------------------------------------------------
// Some hosts may not allocate device memory at the point where they need this
// op: code running inside a CUDA stream capture or under a framework that
// forbids allocator calls on its hot path, plugins handed a fixed memory
// budget at load time, or real-time loops that must not touch the driver's
// allocator.  For them the block counts and the total live in a fixed array
// inside the library image.  Every GPU that loads the library carries these
// 33 KB until the process exits.
namespace {
constexpr int64_t kStaticUniqueMaxRows = 16ll << 20;  // 16 Mi rows per call
constexpr int kStaticUniqueBlocks = (int)(kStaticUniqueMaxRows / kUqTile);  // 8192 block counts
constexpr int kStaticUniqueWords = kStaticUniqueBlocks + 64;                // + the total
constexpr int kMaxDevices = 64;
}  // namespace

static __device__ __align__(256) uint32_t g_unique_scratch[kStaticUniqueWords];

// In host code `g_unique_scratch` is only a handle for the symbol, not a device
// address, so the address is looked up once per device (with that device
// current) and cached here.
static uint32_t *g_unique_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_unique_scratch_mutex;

static mn_status unique_scratch_address(uint32_t **out) {
  int device = -1;
  MN_CHECK_CUDA(cudaGetDevice(&device));
  MN_CHECK_ARG(device >= 0 && device < kMaxDevices, "unique_static: device index %d out of range",
               device);
  std::lock_guard<std::mutex> lock(g_unique_scratch_mutex);
  if (g_unique_scratch_addr[device] == nullptr) {
    uint32_t *p = nullptr;
    MN_CHECK_CUDA(cudaGetSymbolAddress((void **)&p, g_unique_scratch));
    g_unique_scratch_addr[device] = p;
  }
  *out = g_unique_scratch_addr[device];
  return MN_OK;
}

extern "C" mn_status mn_unique_coordinates_static(const int32_t *coords, int64_t n, int ndim,
                                                  const int64_t *batch_dims, int64_t num_clouds,
                                                  int32_t *unique_out, int64_t *indices_out,
                                                  void *stream) {
  MN_CHECK_ARG(n >= 0 && ndim >= 1 && ndim <= MN_MAX_NDIM, "unique_static: bad n/ndim");
  MN_CHECK_ARG(indices_out != nullptr, "unique_static: null indices");
  if (n > kStaticUniqueMaxRows) {
    set_error("unique_static: %lld rows exceed the built-in scratch limit of %lld rows; call "
              "mn_unique_coordinates with a caller-provided workspace instead",
              (long long)n, (long long)kStaticUniqueMaxRows);
    return MN_ERR_BAD_ARG;
  }
  uint32_t *scratch = nullptr;
  MN_RETURN_IF(unique_scratch_address(&scratch));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MN_LAUNCH("zero_index0_kernel", st, zero_index0_kernel<<<1, 1, 0, st>>>(indices_out));
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(coords != nullptr && unique_out != nullptr, "unique_static: null pointer");
  const int nblocks = (int)div_up(n, kUqTile);
  uint32_t *counts = scratch;                       // [nblocks], every word written before read
  uint32_t *total = scratch + kStaticUniqueBlocks;  // [1]
  RowsView view{coords, batch_dims, batch_dims ? (int)num_clouds : 1, ndim, n};
  CoordSink sink{coords, ndim, unique_out, indices_out};
  MN_LAUNCH("unique_count_kernel", st,
            unique_count_kernel<RowsView><<<nblocks, kUqThreads, 0, st>>>(view, counts));
  MN_LAUNCH("scan_blocks_kernel", st,
            scan_blocks_kernel<<<1, 1024, 0, st>>>(counts, nblocks, total, nullptr));
  MN_LAUNCH("unique_compact_kernel", st,
            unique_compact_kernel<RowsView, CoordSink><<<nblocks, kUqThreads, 0, st>>>(view, sink, counts));
  return MN_OK;
}
