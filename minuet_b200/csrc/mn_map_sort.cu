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
#include "mn_grid.cuh"
#include "mn_pack.cuh"

#include <algorithm>
#include <mutex>

namespace mn {

namespace {

// ---------------------------------------------------------------------------
// radix sort: one cooperative kernel for all passes
// ---------------------------------------------------------------------------
// Stable LSD sort, 9-bit digits.  The work is latency bound (a few megabytes per
// pass), so the grid is small: every block (1024 threads) owns a contiguous
// chunk of about 8192 keys and every warp a contiguous slice of that chunk, so
// that "block order, then warp order, then position" is the input order.  A
// warp keeps its slice in registers for the whole pass when it fits (up to 8
// keys per lane).  Per pass:
//   A  every warp counts the digits of its slice into its own row of a
//      [32 warps][512 digits] shared-memory table (equal digits inside a group
//      of 32 keys find each other with match.any, one lane adds the group's
//      count); the block histogram goes to a [block][digit] global table
//   -- grid barrier --
//   C  every block reads the whole table (a few hundred KB in L2), derives its
//      own base position per digit, turns its per-warp counts into global
//      positions and walks its chunk again in the same order, writing every key
//      (and payload) to its place
//   -- grid barrier (the next pass reads what this one wrote) --
// The first pass can build the keys itself from coordinate rows (floor to a
// target stride and pack), so that the strided target-coordinate build needs no
// separate packing launch.  The number of passes comes from the key layout,
// which may live on the device only.
constexpr int kRsThreads = 1024;
constexpr int kRsWarps = kRsThreads / 32;
constexpr int kRsBits = 9;                        // digit width: 4 passes cover 36 key bits
constexpr int kRadix = 1 << kRsBits;
constexpr int kRsMaxBlocks = 256;                 // workspace sizing
constexpr int kRsKeysPerLane = 8;                 // register-resident slice: 256 keys per warp
constexpr int kRsChunk = kRsWarps * 32 * kRsKeysPerLane;   // 8192 keys per block
constexpr size_t kRsSmemBytes = (size_t)kRsWarps * kRadix * sizeof(uint32_t);   // 64 KB

__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

struct SortArgs {
  uint64_t *keys[2];          // ping-pong buffers; the input (or the packed keys) sits in [0]
  int32_t *vals[2];           // optional payloads
  int64_t n;
  int32_t begin_bit;
  int32_t end_bit;            // < 0: the key layout's total_bits
  int32_t has_vals;
  int32_t iota_vals;          // first pass: the payload is the element index
  uint32_t *hist;             // [grid][kRadix]
  int32_t *result_in_second;  // out (may be NULL): 1 when the result is in keys[1] / vals[1]
  int32_t *ctrl;
  // optional key construction in front of the first pass
  const int32_t *coords;      // NULL: keys[0] already holds the keys
  const int64_t *batch_dims;
  int32_t ndim, num_clouds;
  PackParams pack;
};

__global__ void __launch_bounds__(kRsThreads, 1)
radix_sort_kernel(const __grid_constant__ SortArgs a) {
  extern __shared__ __align__(16) uint32_t s_cnt[];   // [kRsWarps][kRadix]
  __shared__ uint32_t s_half[2][kRadix];
  __shared__ uint32_t s_scan[kRsWarps];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  const unsigned lt = lanemask_lt();
  const mn_keyspec &spec = spec_of(a.pack.spec);
  const int end_bit = a.end_bit >= 0 ? a.end_bit : spec.total_bits;
  int passes = (end_bit - a.begin_bit + kRsBits - 1) / kRsBits;
  passes = passes < 1 ? 1 : (passes > 8 ? 8 : passes);

  // chunk of this block and slice of this warp (multiples of 32 keys)
  const int64_t groups = (a.n + 31) >> 5;
  const int64_t g_per_block = (groups + G - 1) / G;
  const int64_t c0 = min(a.n, (int64_t)b * g_per_block * 32);
  const int64_t c1 = min(a.n, c0 + g_per_block * 32);
  const int64_t g_per_warp = (g_per_block + kRsWarps - 1) / kRsWarps;
  const int64_t w0 = min(c1, c0 + (int64_t)warp * g_per_warp * 32);
  const int64_t w1 = min(c1, w0 + g_per_warp * 32);
  const bool resident = g_per_warp <= kRsKeysPerLane;   // the slice stays in registers (uniform)

  if (a.coords != nullptr) {
    // keys of this block's chunk from the coordinate rows (the block is the only
    // reader of its chunk until the first scatter)
    bool bad = false;
    for (int64_t r = c0 + tid; r < c1; r += kRsThreads) {
      int c[4] = {0, 0, 0, 0};
      for (int k = 0; k < a.ndim; k++) c[k] = __ldg(a.coords + r * a.ndim + k);
      const uint64_t g = a.batch_dims != nullptr ? cloud_of(a.batch_dims, a.num_clouds, r) : 0;
      a.keys[0][r] = pack_one(c, a.ndim, g, spec, a.pack, bad);
    }
    if (bad) atomicOr(a.ctrl + MN_CTRL_STATUS, MN_STATUS_KEY_BOX);
    __syncthreads();
  }

  for (int p = 0; p < passes; p++) {
    const int shift = a.begin_bit + p * kRsBits;
    const uint64_t *kin = a.keys[p & 1];
    uint64_t *kout = a.keys[(p & 1) ^ 1];
    const int32_t *vin = a.vals[p & 1];
    int32_t *vout = a.vals[(p & 1) ^ 1];
    const bool iota = a.iota_vals && p == 0;
    uint32_t *mine = s_cnt + warp * kRadix;
    // ---- A: per-warp digit counts ------------------------------------------------
    {
      uint4 *z = reinterpret_cast<uint4 *>(s_cnt);
      for (int i = tid; i < kRsWarps * kRadix / 4; i += kRsThreads) z[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    uint64_t key[kRsKeysPerLane];
    if (resident) {
      // .cg loads: other blocks rewrote this buffer since this SM last read it
#pragma unroll
      for (int j = 0; j < kRsKeysPerLane; j++) {
        const int64_t i = w0 + j * 32 + lane;
        key[j] = i < w1 ? __ldcg(kin + i) : 0ull;
      }
    }
    __syncthreads();
    if (resident) {
#pragma unroll
      for (int j = 0; j < kRsKeysPerLane; j++) {
        const int64_t i = w0 + j * 32 + lane;
        const bool valid = i < w1;
        const unsigned d = valid ? (unsigned)((key[j] >> shift) & (kRadix - 1)) : (unsigned)kRadix;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        if (valid && (peers & lt) == 0u) mine[d] += __popc(peers);
        __syncwarp();
      }
    } else {
      for (int64_t i0 = w0; i0 < w1; i0 += 32) {
        const int64_t i = i0 + lane;
        const bool valid = i < w1;
        const unsigned d = valid ? (unsigned)((__ldcg(kin + i) >> shift) & (kRadix - 1)) : (unsigned)kRadix;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        if (valid && (peers & lt) == 0u) mine[d] += __popc(peers);
        __syncwarp();
      }
    }
    __syncthreads();
    for (int d = tid; d < kRadix; d += kRsThreads) {
      uint32_t sum = 0;
#pragma unroll 8
      for (int w = 0; w < kRsWarps; w++) sum += s_cnt[w * kRadix + d];
      a.hist[(size_t)b * kRadix + d] = sum;
    }
    grid_barrier(a.ctrl, (unsigned)G);
    // ---- C: positions, scatter --------------------------------------------------------
    // two threads per digit add up the table column: keys of that digit in the blocks
    // before this one, and in all blocks
    {
      const int d = tid & (kRadix - 1), half = tid >> kRsBits;
      uint32_t before = 0, all = 0;
#pragma unroll 8
      for (int bb = half; bb < G; bb += 2) {
        const uint32_t v = __ldcg(a.hist + (size_t)bb * kRadix + d);
        all += v;
        before += bb < b ? v : 0u;
      }
      if (half == 1) { s_half[0][d] = before; s_half[1][d] = all; }
      __syncthreads();
      uint32_t excl = 0;
      if (half == 0) {
        before += s_half[0][d];
        all += s_half[1][d];
        // exclusive scan of the digit totals over the first 512 threads (16 warps)
        uint32_t inc = all;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
          const uint32_t u = __shfl_up_sync(0xffffffffu, inc, s);
          if (lane >= s) inc += u;
        }
        if (lane == 31) s_scan[warp] = inc;
        excl = inc - all;
      }
      __syncthreads();
      if (half == 0) {
        uint32_t run = excl + before;
        for (int w = 0; w < warp; w++) run += s_scan[w];
#pragma unroll 8
        for (int w = 0; w < kRsWarps; w++) {
          const uint32_t c = s_cnt[w * kRadix + d];
          s_cnt[w * kRadix + d] = run;
          run += c;
        }
      }
    }
    __syncthreads();
    if (resident) {
#pragma unroll
      for (int j = 0; j < kRsKeysPerLane; j++) {
        const int64_t i = w0 + j * 32 + lane;
        const bool valid = i < w1;
        const unsigned d = valid ? (unsigned)((key[j] >> shift) & (kRadix - 1)) : (unsigned)kRadix;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        if (valid) {
          const uint32_t pos = mine[d] + __popc(peers & lt);
          kout[pos] = key[j];
          if (a.has_vals) vout[pos] = iota ? (int32_t)i : __ldcg(vin + i);
        }
        __syncwarp();
        if (valid && (peers & lt) == 0u) mine[d] += __popc(peers);
        __syncwarp();
      }
    } else {
      for (int64_t i0 = w0; i0 < w1; i0 += 32) {
        const int64_t i = i0 + lane;
        const bool valid = i < w1;
        const uint64_t k = valid ? __ldcg(kin + i) : 0ull;
        const unsigned d = valid ? (unsigned)((k >> shift) & (kRadix - 1)) : (unsigned)kRadix;
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        if (valid) {
          const uint32_t pos = mine[d] + __popc(peers & lt);
          kout[pos] = k;
          if (a.has_vals) vout[pos] = iota ? (int32_t)i : __ldcg(vin + i);
        }
        __syncwarp();
        if (valid && (peers & lt) == 0u) mine[d] += __popc(peers);
        __syncwarp();
      }
    }
    if (p + 1 < passes) grid_barrier(a.ctrl, (unsigned)G);
  }
  if (b == 0 && tid == 0 && a.result_in_second != nullptr) *a.result_in_second = passes & 1;
}

__global__ void widen_index_kernel(const int32_t *__restrict__ in, int64_t n,
                                   int64_t *__restrict__ out) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gsz) out[i] = in[i];
}

// Keys of one LSD pass of the dimension-by-dimension sort: the coordinate of
// dimension `dim` (dim >= 0; sign bit flipped, so that unsigned order is signed
// order) or the cloud (dim < 0) of the row that currently sits at position i.
__global__ void dimension_keys_kernel(const int32_t *__restrict__ coords, int64_t n, int ndim, int dim,
                                      const int32_t *__restrict__ perm,
                                      const int64_t *__restrict__ batch_dims, int num_clouds,
                                      uint64_t *__restrict__ keys) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gsz) {
    const int64_t row = perm != nullptr ? perm[i] : i;
    uint64_t k;
    if (dim >= 0) {
      k = (uint64_t)((uint32_t)__ldg(coords + row * ndim + dim) ^ 0x80000000u);
    } else {
      int lo = 0, hi = num_clouds;   // last cloud whose first row is <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(batch_dims + mid) <= row) lo = mid; else hi = mid;
      }
      k = (uint64_t)lo;
    }
    keys[i] = k;
  }
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

// ---------------------------------------------------------------------------
// unique over sorted keys (strided target coordinates): one cooperative kernel
// ---------------------------------------------------------------------------
// Every block owns a contiguous chunk of the sorted keys.  It counts the keys
// that open a run (differ from their predecessor), a grid barrier later sums
// the counts of the blocks before it, and walks the chunk again: every opening
// key goes to its rank in keys_out, is unpacked into a coordinate row, and, when
// it is the first key of its cloud, fills the cloud-start table.  The count,
// the cloud starts and a copy of the status word land in one int64 block
// (meta), so that the host needs a single small read.
constexpr int kUkThreads = 1024;
constexpr int kUkWarps = kUkThreads / 32;

struct UniqueKeysArgs {
  const uint64_t *keys[2];           // sorted keys are in keys[*which] (which may be NULL: keys[0])
  const int32_t *which;
  int64_t n;
  SpecRef spec;
  uint64_t *keys_out;                // [n]
  int32_t *rows_out;                 // [n, ndim]
  int64_t *meta;                     // [num_clouds + 3]: count, cloud starts [num_clouds + 1], status
  int32_t num_clouds;
  uint32_t *block_counts;            // workspace [grid]
  int32_t *ctrl;
};

constexpr int kUkRounds = 8;                          // keys per thread and step
constexpr int kUkStep = kUkThreads * kUkRounds;       // 8192 keys per block and step

__global__ void __launch_bounds__(kUkThreads, 1)
unique_keys_kernel(const __grid_constant__ UniqueKeysArgs a) {
  __shared__ uint32_t s_cnt[kUkRounds][kUkWarps];     // openers per (round, warp), then their prefix
  __shared__ uint32_t s_before, s_total, s_step_total;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  const unsigned lt = (1u << lane) - 1u;
  const mn_keyspec &spec = spec_of(a.spec);
  const uint64_t *keys = a.keys[a.which != nullptr ? (*a.which & 1) : 0];
  const int64_t per_block = ((a.n + G - 1) / G + kUkThreads - 1) / kUkThreads * kUkThreads;
  const int64_t c0 = min(a.n, (int64_t)b * per_block), c1 = min(a.n, c0 + per_block);

  // ---- count the run openers of this chunk (a key opens a run when it differs from
  // its predecessor); all loads of a step are issued before any is used -------------
  uint32_t mine = 0;
  for (int64_t s0 = c0; s0 < c1; s0 += kUkStep) {
    uint64_t k[kUkRounds], pk[kUkRounds];
#pragma unroll
    for (int j = 0; j < kUkRounds; j++) {
      const int64_t i = s0 + j * kUkThreads + tid;
      k[j] = i < c1 ? __ldcg(keys + i) : 0ull;
      pk[j] = (i < c1 && i > 0) ? __ldcg(keys + i - 1) : 0ull;
    }
#pragma unroll
    for (int j = 0; j < kUkRounds; j++) {
      const int64_t i = s0 + j * kUkThreads + tid;
      mine += (i < c1 && (i == 0 || k[j] != pk[j])) ? 1u : 0u;
    }
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  if (lane == 0) s_cnt[0][warp] = mine;
  __syncthreads();
  if (tid == 0) {
    uint32_t t = 0;
    for (int w = 0; w < kUkWarps; w++) t += s_cnt[0][w];
    a.block_counts[b] = t;
  }
  grid_barrier(a.ctrl, (unsigned)G);
  if (warp == 0) {
    uint32_t before = 0, all = 0;
    for (int bb = lane; bb < G; bb += 32) {
      const uint32_t v = __ldcg(a.block_counts + bb);
      all += v;
      if (bb < b) before += v;
    }
    before = __reduce_add_sync(0xffffffffu, before);
    all = __reduce_add_sync(0xffffffffu, all);
    if (lane == 0) { s_before = before; s_total = all; }
  }
  __syncthreads();
  uint32_t run = s_before;
  const uint32_t total = s_total;

  // ---- compact, unpack, cloud starts ----------------------------------------------
  for (int64_t s0 = c0; s0 < c1; s0 += kUkStep) {
    uint64_t k[kUkRounds], pk[kUkRounds];
    unsigned votes[kUkRounds];
#pragma unroll
    for (int j = 0; j < kUkRounds; j++) {
      const int64_t i = s0 + j * kUkThreads + tid;
      k[j] = i < c1 ? __ldcg(keys + i) : 0ull;
      pk[j] = (i < c1 && i > 0) ? __ldcg(keys + i - 1) : 0ull;
    }
    __syncthreads();   // the prefix table of the previous step has been read
#pragma unroll
    for (int j = 0; j < kUkRounds; j++) {
      const int64_t i = s0 + j * kUkThreads + tid;
      const bool opens = i < c1 && (i == 0 || k[j] != pk[j]);
      votes[j] = __ballot_sync(0xffffffffu, opens);
      if (lane == 0) s_cnt[j][warp] = __popc(votes[j]);
    }
    __syncthreads();
    if (warp == 0) {
      // exclusive prefix over the kUkRounds * kUkWarps counts, in (round, warp) order
      uint32_t v[kUkRounds], sum = 0;
#pragma unroll
      for (int j = 0; j < kUkRounds; j++) { v[j] = (&s_cnt[0][0])[lane * kUkRounds + j]; sum += v[j]; }
      uint32_t inc = sum;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, s);
        if (lane >= s) inc += t;
      }
      uint32_t r = inc - sum;
#pragma unroll
      for (int j = 0; j < kUkRounds; j++) { (&s_cnt[0][0])[lane * kUkRounds + j] = r; r += v[j]; }
      if (lane == 31) s_step_total = inc;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kUkRounds; j++) {
      const int64_t i = s0 + j * kUkThreads + tid;
      if ((votes[j] >> lane) & 1u) {
        const uint32_t pos = run + s_cnt[j][warp] + __popc(votes[j] & lt);
        const uint64_t key = k[j];
        a.keys_out[pos] = key;
        for (int d = 0; d < spec.ndim; d++) {
          const uint64_t f = (key >> spec.shift[d]) & ((1ull << spec.bits[d]) - 1ull);
          a.rows_out[(int64_t)pos * spec.ndim + d] = (int32_t)((int64_t)f + spec.base[d]);
        }
        // first key of cloud c: every cloud after the previous key's cloud starts here
        const int64_t c_here = (int64_t)(key >> spec.cloud_shift);
        const int64_t c_prev = i == 0 ? -1 : (int64_t)(pk[j] >> spec.cloud_shift);
        for (int64_t g = c_prev + 1; g <= c_here && g <= a.num_clouds; g++) a.meta[1 + g] = pos;
      }
    }
    run += s_step_total;
  }
  if (b == 0 && tid == 0) {
    a.meta[0] = total;
    const int64_t c_last = a.n > 0 ? (int64_t)(__ldcg(keys + a.n - 1) >> spec.cloud_shift) : -1;
    for (int64_t g = c_last + 1; g <= a.num_clouds; g++) a.meta[1 + g] = total;
    a.meta[a.num_clouds + 2] = a.ctrl[MN_CTRL_STATUS];
  }
}

__global__ void zero_index0_kernel(int64_t *indices) { indices[0] = 0; }

}  // namespace

size_t radix_sort_workspace_bytes(int64_t n) {
  (void)n;
  return align_up((size_t)kRsMaxBlocks * kRadix * sizeof(uint32_t), 256) + 256;
}

namespace {

// Grid of a cooperative kernel with one 1024-thread block per SM, cached per device.
template <typename Kernel>
mn_status coop_grid_1024(Kernel kernel, size_t smem, int *cache, int *out) {
  int device = 0;
  MN_CHECK_CUDA(cudaGetDevice(&device));
  MN_CHECK_ARG(device >= 0 && device < kMaxDevices, "device index %d out of range", device);
  if (cache[device] == 0) {
    if (smem > 48 * 1024)
      MN_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cache[device] = std::min(kRsMaxBlocks, max_coresident_blocks(kernel, 1024, smem));
    if (cache[device] <= 0) {
      cache[device] = 0;
      set_error("cannot size a cooperative grid on device %d", device);
      return MN_ERR_CUDA;
    }
  }
  *out = cache[device];
  return MN_OK;
}

}  // namespace

// Stable LSD sort of `keys` on bits [begin_bit, end_bit) (end_bit < 0: up to the
// key layout's total_bits, read on the device), ping-ponging between keys and
// keys_tmp.  With vals/vals_tmp given, int32 payloads move with the keys;
// iota_vals makes the first pass use the element index as payload.  With
// `coords` given the first pass builds the keys itself (floor to pack.tstride,
// pack).  Where the result ends up is written to *result_in_second_dev (device,
// may be NULL) and, when end_bit is known on the host, to *result_in_tmp.
mn_status launch_radix_sort(uint64_t *keys, uint64_t *keys_tmp, int32_t *vals, int32_t *vals_tmp,
                            bool iota_vals, int64_t n, int begin_bit, int end_bit,
                            const mn_keyspec &spec, const SortSource *source, int32_t *ctrl,
                            int32_t *result_in_second_dev, Workspace &ws, bool *result_in_tmp,
                            cudaStream_t st) {
  if (result_in_tmp != nullptr) *result_in_tmp = false;
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(n < (1ll << 31), "radix sort: n = %lld exceeds 2^31-1", (long long)n);
  MN_CHECK_ARG(ctrl != nullptr, "radix sort: null control block");
  static thread_local int grid_cache[kMaxDevices] = {0};
  int coresident = 0;
  MN_RETURN_IF(coop_grid_1024(radix_sort_kernel, kRsSmemBytes, grid_cache, &coresident));
  // every SM gets a block as soon as there are 2048 keys for it: the passes are latency
  // bound (two grid barriers each), so smaller chunks per block shorten them
  const int grid = (int)std::min<int64_t>(coresident, std::max<int64_t>(1, div_up(n, kRsChunk / 4)));
  SortArgs a{};
  a.keys[0] = keys; a.keys[1] = keys_tmp;
  a.vals[0] = vals; a.vals[1] = vals_tmp;
  a.n = n;
  a.begin_bit = begin_bit;
  a.end_bit = end_bit;
  a.has_vals = vals != nullptr && vals_tmp != nullptr;
  a.iota_vals = iota_vals ? 1 : 0;
  a.hist = ws.take<uint32_t>((size_t)kRsMaxBlocks * kRadix);
  MN_CHECK_WS(ws);
  a.result_in_second = result_in_second_dev;
  a.ctrl = ctrl;
  a.pack.spec = make_spec_ref(spec);
  a.pack.has_stride = 0;
  for (int k = 0; k < 4; k++) a.pack.tstride[k] = 1;
  if (source != nullptr) {
    a.coords = source->coords;
    a.batch_dims = source->batch_dims;
    a.ndim = source->ndim;
    a.num_clouds = source->batch_dims != nullptr ? (int)source->num_clouds : 1;
    for (int k = 0; k < source->ndim; k++) {
      a.pack.tstride[k] = source->tstride != nullptr ? source->tstride[k] : 1;
      if (a.pack.tstride[k] != 1) a.pack.has_stride = 1;
    }
  }
  void *params[] = {&a};
  {
    LaunchScope scope("radix_sort_kernel", st);
    MN_CHECK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(radix_sort_kernel), dim3(grid),
                                              dim3(kRsThreads), params, kRsSmemBytes, st));
  }
  MN_CHECK_LAUNCH();
  if (result_in_tmp != nullptr && end_bit >= 0) {
    int passes = (end_bit - begin_bit + kRsBits - 1) / kRsBits;
    passes = std::min(8, std::max(1, passes));
    *result_in_tmp = (passes & 1) != 0;
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
  MN_CHECK_ARG(spec->device_copy == nullptr, "arg_sort: needs a key spec whose layout is known on the host");
  SortSource source{coords, batch_dims, num_clouds, ndim, nullptr};
  bool in_tmp = false;
  MN_RETURN_IF(launch_radix_sort(keys, keys_tmp, vals, vals_tmp, true, n, 0, spec->total_bits,
                                 *spec, &source, status_dev, nullptr, ws, &in_tmp, st));
  const int blocks = (int)std::min<int64_t>(kNumSMs * 8, div_up(n, 256));
  MN_LAUNCH("widen_index_kernel", st, widen_index_kernel<<<blocks, 256, 0, st>>>(in_tmp ? vals_tmp : vals, n, index_out));
  return MN_OK;
}

extern "C" mn_status mn_arg_sort_coordinates_by_dimension(
    const int32_t *coords, int64_t n, int ndim, const int64_t *batch_dims, int64_t num_clouds,
    int64_t *index_out, int32_t *ctrl, void *ws_ptr, size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(n >= 0 && n < (1ll << 31) && ndim >= 1 && ndim <= MN_MAX_NDIM,
               "arg_sort_by_dimension: bad n/ndim");
  if (n == 0) return MN_OK;
  MN_CHECK_ARG(coords != nullptr && index_out != nullptr && ctrl != nullptr,
               "arg_sort_by_dimension: null pointer");
  if (batch_dims == nullptr) num_clouds = 1;
  MN_CHECK_ARG(num_clouds >= 1 && num_clouds < (1ll << 31), "arg_sort_by_dimension: bad num_clouds");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace ws(ws_ptr, ws_bytes);
  uint64_t *keys[2] = {ws.take<uint64_t>(n), ws.take<uint64_t>(n)};
  int32_t *vals[2] = {ws.take<int32_t>(n), ws.take<int32_t>(n)};
  MN_CHECK_WS(ws);
  const size_t fixed = ws.used;
  const mn_keyspec no_spec{};
  const int blocks = (int)std::min<int64_t>(kNumSMs * 8, div_up(n, 256));
  int cur = 0;            // vals[cur] holds the current permutation (after the first pass)
  bool first = true;
  // least significant key first: last dimension ... dimension 0, then the cloud
  for (int dim = ndim - 1; dim >= (num_clouds > 1 ? -1 : 0); dim--) {
    int bits = 32;
    if (dim < 0) {
      bits = 1;
      while ((1ll << bits) < num_clouds) bits++;
    }
    MN_LAUNCH("dimension_keys_kernel", st,
              dimension_keys_kernel<<<blocks, 256, 0, st>>>(coords, n, ndim, dim,
                                                            first ? nullptr : vals[cur], batch_dims,
                                                            (int)num_clouds, keys[cur]));
    Workspace sub(static_cast<char *>(ws_ptr) + fixed, ws_bytes - fixed);
    bool in_tmp = false;
    MN_RETURN_IF(launch_radix_sort(keys[cur], keys[cur ^ 1], vals[cur], vals[cur ^ 1], first, n, 0,
                                   bits, no_spec, nullptr, ctrl, nullptr, sub, &in_tmp, st));
    if (in_tmp) cur ^= 1;
    first = false;
  }
  MN_LAUNCH("widen_index_kernel", st, widen_index_kernel<<<blocks, 256, 0, st>>>(vals[cur], n, index_out));
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
    int64_t *meta_out, int32_t *ctrl, void *ws_ptr, size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(n >= 0 && ndim >= 1 && ndim <= MN_MAX_NDIM, "downsample: bad n/ndim");
  MN_CHECK_ARG(spec != nullptr && spec->ndim == ndim, "downsample: key spec missing or of another ndim");
  MN_CHECK_ARG(tstride != nullptr && meta_out != nullptr && ctrl != nullptr, "downsample: null pointer");
  MN_CHECK_ARG(n < (1ll << 31), "downsample: n exceeds 2^31-1");
  if (batch_dims == nullptr) num_clouds = 1;
  MN_CHECK_ARG(num_clouds >= 1, "downsample: num_clouds must be >= 1");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MN_CHECK_ARG(n == 0 || (coords != nullptr && unique_out != nullptr && keys_out != nullptr),
               "downsample: null pointer");
  for (int k = 0; k < ndim; k++)
    MN_CHECK_ARG(tstride[k] >= 1 && tstride[k] - 1 <= spec->margin,
                 "downsample: stride %d needs a key margin >= %d (have %d)", tstride[k],
                 tstride[k] - 1, spec->margin);
  Workspace ws(ws_ptr, ws_bytes);
  uint64_t *keys = ws.take<uint64_t>(std::max<int64_t>(n, 1)), *keys_tmp = ws.take<uint64_t>(std::max<int64_t>(n, 1));
  int32_t *which = ws.take<int32_t>(1);
  uint32_t *block_counts = ws.take<uint32_t>(kRsMaxBlocks);
  MN_CHECK_WS(ws);
  SortSource source{coords, batch_dims, num_clouds, ndim, tstride};
  MN_RETURN_IF(launch_radix_sort(keys, keys_tmp, nullptr, nullptr, false, n, 0,
                                 spec->device_copy != nullptr ? -1 : spec->total_bits, *spec,
                                 &source, ctrl, which, ws, nullptr, st));
  static thread_local int grid_cache[kMaxDevices] = {0};
  int coresident = 0;
  MN_RETURN_IF(coop_grid_1024(unique_keys_kernel, 0, grid_cache, &coresident));
  const int grid = (int)std::min<int64_t>(coresident, std::max<int64_t>(1, div_up(n, kUkStep)));
  UniqueKeysArgs a{};
  a.keys[0] = keys; a.keys[1] = keys_tmp;
  a.which = n > 0 ? which : nullptr;
  a.n = n;
  a.spec = make_spec_ref(*spec);
  a.keys_out = keys_out;
  a.rows_out = unique_out;
  a.meta = meta_out;
  a.num_clouds = (int)num_clouds;
  a.block_counts = block_counts;
  a.ctrl = ctrl;
  void *params[] = {&a};
  {
    LaunchScope scope("unique_keys_kernel", st);
    MN_CHECK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(unique_keys_kernel), dim3(grid),
                                              dim3(kUkThreads), params, 0, st));
  }
  MN_CHECK_LAUNCH();
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
