// Map step, part 2: kernel-map search, sizes, size order and masks.
//
// The reference builds the kernel map in two traversals
// (csrc/minuet/cuda/functions/query_sorted_index.cu:14-119): a global binary
// search per (256-source block, offset) for target borders, then a per-target
// binary search inside one source block staged in shared memory
// (kernels/query_sorted_index_with_offsets.cuh:60-76); sizes, order and masks
// follow as a reduce-by-key, a torch.sort, a DeviceSelect, two memsets and a
// scatter kernel (functions/scan.cu:221-365, minuet/nn/convolutions.py:156-170).
//
// Here both traversals live in one row-tile-stationary kernel over packed
// 64-bit keys.  A block owns 1024 consecutive rows (targets) and, for every
// group of offsets that differ only in the last dimension, (1) finds the window
// of the sorted table (sources) that can match the tile with a warp-cooperative
// 32-ary ballot search, (2) stages that window in shared memory (adjacent groups
// share one staging pass when their union fits) and (3) lets every row do ONE
// binary search per group followed by a short forward walk for the group's
// other offsets, because inside a group the queries of a row are ascending.
// The kernel either writes kernel-map rows or, for the fused build, a 32-bit
// word of per-offset hit bits per row plus per-tile hit counts; ranks and both
// masks are then produced by a scan over tile counts and one streaming kernel
// that writes every mask element exactly once (no memset, no select, no
// scatter).  For submanifold maps (sources == targets, symmetric offsets) the
// source mask of offset o is read off the hit bits of the mirrored offset.
#include "mn_common.cuh"

#include <algorithm>
#include <vector>

namespace mn {

namespace {

#ifndef MN_QTHREADS
#define MN_QTHREADS 128
#endif
constexpr int kQThreads = MN_QTHREADS;
constexpr int kQWarps = kQThreads / 32;
constexpr int kQRows = 4;                    // rows per thread
constexpr int kQTile = kQThreads * kQRows;   // 512 rows per block
constexpr int kQWindow = 2048;               // table keys staged per pass
constexpr int kQHash = 2048;                 // slots of the shared-memory hash of cells
constexpr uint32_t kHashEmpty = 0xffffffffu;
constexpr uint32_t kQPad = 4096;             // slack below/above the window in relative keys
constexpr uint64_t kKeyInf = ~0ull;

__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Warp-cooperative 32-ary search in global memory: lower bound (first index
// with t[i] >= q) or upper bound (first index with t[i] > q).  Every lane
// probes one pivot per round, a ballot narrows the range 32-fold; ~4 rounds for
// half a million keys.  All 32 lanes must call with identical arguments.
__device__ __forceinline__ int64_t warp_bound(const uint64_t *__restrict__ t, int64_t n,
                                              uint64_t q, bool upper, int lane) {
  int64_t lo = 0, hi = n;
  for (int round = 0; round < 16; round++) {
    const int64_t len = hi - lo;
    if (len <= 0) break;
    const int64_t stride = (len + 31) >> 5;
    const int64_t idx = lo + (int64_t)(lane + 1) * stride - 1;
    bool pred = false;
    if (idx < hi) {
      const uint64_t v = __ldg(t + idx);
      pred = upper ? (v <= q) : (v < q);
    }
    const int c = __popc(__ballot_sync(0xffffffffu, pred));
    if (stride == 1) return lo + c;
    const int64_t nlo = min(lo + (int64_t)c * stride, hi);
    hi = min(hi, nlo + stride - 1);
    lo = nlo;
  }
  return lo;
}

struct SearchArgs {
  const uint64_t *rows;
  const uint64_t *table;
  int64_t n_rows;
  int64_t n_table;
  int32_t *kernel_map;   // kMap:  [O, n_rows]
  uint32_t *hit_words;   // kBits: [n_rows]
  int32_t *tile_counts;  // kBits: [O, n_tiles]
  int32_t n_tiles;
  int32_t shift[4];
  int32_t fast_ok;       // every last-dimension offset is within +-kQPad
};

// One launch can serve two searches (e.g. targets->sources and sources->targets).
struct SearchPair {
  SearchArgs a[2];
  OffsetTable tab[2];
  int32_t tiles0;   // blocks of the first search
};

enum SearchMode { kMap = 0, kBits = 1 };

// lower bound of q in win[a, b); trip count depends only on b - a (uniform)
template <typename K>
__device__ __forceinline__ int lower_bound_win(const K *win, int a, int b, K q) {
  int base = a, len = b - a;
  while (len > 1) {
    const int half = len >> 1;
    base = (win[base + half - 1] < q) ? base + half : base;
    len -= half;
  }
  return (len == 1 && win[base] < q) ? base + 1 : base;
}

// One result of one (row, offset): either a kernel-map entry or a hit bit.
template <int kMode>
__device__ __forceinline__ void emit(const SearchArgs &a, int o, int64_t row, bool vec_ok,
                                     const bool (&live)[kQRows], const int32_t (&idx)[kQRows],
                                     uint32_t (&bits)[kQRows]) {
  if (kMode == kMap) {
    int32_t *dst = a.kernel_map + (int64_t)o * a.n_rows + row;
    if (vec_ok && live[kQRows - 1]) {
      *reinterpret_cast<int4 *>(dst) = make_int4(idx[0], idx[1], idx[2], idx[3]);
    } else {
#pragma unroll
      for (int j = 0; j < kQRows; j++) if (live[j]) dst[j] = idx[j];
    }
  } else {
#pragma unroll
    for (int j = 0; j < kQRows; j++) bits[j] |= (idx[j] >= 0 ? 1u : 0u) << o;
  }
}

// The hash set is kQHash / 2 buckets of two {cell, mask} slots (16 bytes).  Inserts
// fill slot 0 of a bucket first, then slot 1, then move on to the next bucket, so a
// bucket whose slot 1 is empty never overflowed.
constexpr int kQBuckets = kQHash / 2;

__device__ __forceinline__ uint32_t hash_bucket(uint32_t k) {
  return (k * 0x9E3779B1u) >> 22;  // top 10 bits: 1024 buckets
}

// Occupancy mask of cell c (0 when the cell is absent) and the slot that holds it.
// The home bucket and its successor are read up front with two 16-byte loads; only
// a cell pushed further than that (rare at these load factors) takes the loop, so
// the lanes of a warp stay converged.
__device__ __forceinline__ uint32_t find_cell(const uint2 *slots, uint32_t c, uint32_t *slot) {
  const uint4 *buckets = reinterpret_cast<const uint4 *>(slots);
  uint32_t b = hash_bucket(c);
  const uint4 a0 = buckets[b];
  const uint32_t b1 = (b + 1) & (kQBuckets - 1);
  const uint4 a1 = buckets[b1];
  if (a0.x == c) { *slot = 2 * b; return a0.y; }
  if (a0.z == c) { *slot = 2 * b + 1; return a0.w; }
  if (a0.z == kHashEmpty) { *slot = 0; return 0u; }
  if (a1.x == c) { *slot = 2 * b1; return a1.y; }
  if (a1.z == c) { *slot = 2 * b1 + 1; return a1.w; }
  if (a1.z == kHashEmpty) { *slot = 0; return 0u; }
  b = b1;
  for (int probe = 2; probe < kQBuckets; probe++) {
    b = (b + 1) & (kQBuckets - 1);
    const uint4 v = buckets[b];
    if (v.x == c) { *slot = 2 * b; return v.y; }
    if (v.z == c) { *slot = 2 * b + 1; return v.w; }
    if (v.z == kHashEmpty) break;
  }
  *slot = 0;
  return 0u;
}

// A block owns 512 consecutive rows, a thread 4 consecutive rows.
//
// Fast path (the table window that can match the tile, over ALL offsets, holds
// at most kQWindow keys spanning less than 2^32 - 4*kQPad, and no offset moves
// the last dimension by more than kQPad): two warp-cooperative 32-ary searches
// find the window of the sorted table.  The block stages that sorted block in
// shared memory as a hash set of CELLS: 32 consecutive values of the last
// dimension share one slot {cell id, 32-bit occupancy mask} (plus the position
// of the cell's first key when kernel-map entries are wanted; the rest follows
// by popcount because the table is sorted).  The offsets of a group differ only
// in the last dimension, so one probe usually answers the whole group, and the
// probes of a thread do not depend on each other.
// General path (huge or wide windows): per-group windows, 64-bit keys, staged
// when they fit, binary-searched in global memory otherwise.
template <int kMode>
__global__ void __launch_bounds__(kQThreads, 8)
search_kernel(const __grid_constant__ SearchPair sp) {
  // blocks [0, tiles0) serve direction 0, the rest direction 1 (rows and table swapped)
  const int dir = (int)blockIdx.x >= sp.tiles0 ? 1 : 0;
  const int bid = (int)blockIdx.x - dir * sp.tiles0;
  const SearchArgs &a = sp.a[dir];
  const OffsetTable &tab = sp.tab[dir];
  __shared__ __align__(16) uint64_t s_win[kQWindow + 2];          // hash slots / general path
  __shared__ uint16_t s_hpos[kMode == kMap ? kQHash : 1];         // first position of a cell
  __shared__ int64_t s_delta[MN_MAX_OFFSETS];
  __shared__ int64_t s_glo[MN_MAX_OFFSETS], s_ghi[MN_MAX_OFFSETS];
  __shared__ int32_t s_stage_gbeg[MN_MAX_OFFSETS + 1];
  __shared__ int32_t s_counts[MN_MAX_OFFSETS];
  __shared__ int32_t s_num_stages;
  static_assert(kQHash <= kQWindow + 2, "the hash slots live in s_win");

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int O = tab.num_offsets, G = tab.num_groups;
  const int last = tab.ndim - 1;
  const int64_t tile0 = (int64_t)bid * kQTile;
  const int tile_rows = (int)min((int64_t)kQTile, a.n_rows - tile0);
  const int64_t row0 = tile0 + tid * kQRows;

  for (int o = tid; o < O; o += kQThreads) {
    int64_t d = 0;
    for (int k = 0; k < tab.ndim; k++) d += (int64_t)tab.off[o][k] * ((int64_t)1 << a.shift[k]);
    s_delta[o] = d;
    s_counts[o] = 0;
  }

  uint64_t key[kQRows];
  bool live[kQRows];
  if (tid * kQRows + kQRows <= tile_rows && (reinterpret_cast<uintptr_t>(a.rows) & 15) == 0) {
    const ulonglong2 v0 = __ldg(reinterpret_cast<const ulonglong2 *>(a.rows + row0));
    const ulonglong2 v1 = __ldg(reinterpret_cast<const ulonglong2 *>(a.rows + row0) + 1);
    key[0] = v0.x; key[1] = v0.y; key[2] = v1.x; key[3] = v1.y;
#pragma unroll
    for (int j = 0; j < kQRows; j++) live[j] = true;
  } else {
#pragma unroll
    for (int j = 0; j < kQRows; j++) {
      live[j] = tid * kQRows + j < tile_rows;
      key[j] = live[j] ? __ldg(a.rows + row0 + j) : 0ull;
    }
  }
  const uint64_t kfirst = __ldg(a.rows + tile0);
  const uint64_t klast = __ldg(a.rows + tile0 + tile_rows - 1);
  const bool vec_ok = kMode == kMap && (a.n_rows & 3) == 0 &&
                      (reinterpret_cast<uintptr_t>(a.kernel_map) & 15) == 0;
  __syncthreads();

  // window of the table over all offsets: groups are ordered by delta
  __shared__ int64_t s_union[2];
  if (warp < 2) {
    const uint64_t q = warp == 0 ? kfirst + (uint64_t)s_delta[tab.member[0]]
                                 : klast + (uint64_t)s_delta[tab.member[O - 1]];
    const int64_t r = warp_bound(a.table, a.n_table, q, warp == 1, lane);
    if (lane == 0) s_union[warp] = r;
  }
  uint2 *slots = reinterpret_cast<uint2 *>(s_win);
  for (int i = tid; i < kQHash; i += kQThreads) slots[i] = make_uint2(kHashEmpty, 0u);
  __syncthreads();
  const int64_t ulo = s_union[0], uhi = max(s_union[0], s_union[1]);
  const int wn = (int)min(uhi - ulo, (int64_t)kQWindow + 1);
  bool fast = a.fast_ok && uhi - ulo <= kQWindow;
  uint64_t base = 0;
  if (fast && wn > 0) {
    base = __ldg(a.table + ulo);
    fast = __ldg(a.table + uhi - 1) - base < 0xffffffffull - 4ull * kQPad;
  }

  uint32_t bits[kQRows] = {0u, 0u, 0u, 0u};
  if (fast) {
    // keys relative to base - kQPad, so that "query below the window" needs no test
    for (int w = tid; w < wn; w += kQThreads) {
      const uint64_t tk = __ldg(a.table + ulo + w);
      const uint32_t k = (uint32_t)(tk - base) + kQPad;
      const uint32_t cell = k >> 5;
      uint32_t b = hash_bucket(cell), h = 0;
      for (int probe = 0; probe < kQBuckets; probe++) {
        uint32_t old = atomicCAS(&slots[2 * b].x, kHashEmpty, cell);
        if (old == kHashEmpty || old == cell) { h = 2 * b; break; }
        old = atomicCAS(&slots[2 * b + 1].x, kHashEmpty, cell);
        if (old == kHashEmpty || old == cell) { h = 2 * b + 1; break; }
        b = (b + 1) & (kQBuckets - 1);
      }
      atomicOr(&slots[h].y, 1u << (k & 31));
      if (kMode == kMap) {
        // the table is sorted: exactly one key of a cell has a predecessor in another cell
        const bool first = w == 0 ||
            (((uint32_t)(__ldg(a.table + ulo + w - 1) - base) + kQPad) >> 5) != cell;
        if (first) s_hpos[h] = (uint16_t)w;
      }
    }
    __syncthreads();
    int64_t rel[kQRows];
#pragma unroll
    for (int j = 0; j < kQRows; j++) rel[j] = (int64_t)(key[j] - base) + kQPad;
    for (int g = 0; g < G; g++) {
      const int mb = tab.group_begin[g], me = tab.group_begin[g + 1];
      const int o_first = tab.member[mb];
      const int e_first = tab.off[o_first][last];
      const int e_span = tab.off[tab.member[me - 1]][last] - e_first;  // >= 0, members ascend
      const int64_t dg = s_delta[o_first] - e_first;  // the last dimension sits at bit 0
      // Per row: the 64 consecutive last-dimension values starting at the cell of
      // the group's first query, as one 64-bit occupancy mask (low cell | high cell).
      uint32_t sh[kQRows], mlo[kQRows], mhi[kQRows], slo[kQRows], shi[kQRows];
      uint32_t c0[kQRows];
      bool ok[kQRows];
#pragma unroll
      for (int j = 0; j < kQRows; j++) {
        const uint64_t t = (uint64_t)(rel[j] + dg);
        ok[j] = live[j] && t < 0xffffffffull - 2ull * kQPad;  // t +- kQPad stays inside 32 bits
        const uint32_t q0 = (uint32_t)t + (uint32_t)e_first;
        c0[j] = q0 >> 5;
        sh[j] = q0 & 31;
      }
#pragma unroll
      for (int j = 0; j < kQRows; j++) {
        const uint32_t m0 = find_cell(slots, c0[j], &slo[j]);
        mlo[j] = ok[j] ? m0 : 0u;
        mhi[j] = 0u;
        shi[j] = 0u;
        if (ok[j] && (int)sh[j] + e_span > 31)   // the group reaches into the next cell
          mhi[j] = find_cell(slots, c0[j] + 1, &shi[j]);
      }
      if (kMode == kBits && e_span <= 32) {
        // hit bits only: every offset of the group is one bit of the row's 64-value
        // strip, extracted without branches so that the warp stays converged
        uint64_t strip[kQRows];
#pragma unroll
        for (int j = 0; j < kQRows; j++)
          strip[j] = (((uint64_t)mhi[j] << 32) | mlo[j]) >> sh[j];
        for (int m = mb; m < me; m++) {
          const int o = tab.member[m];
          const int de = tab.off[o][last] - e_first;   // 0..32
#pragma unroll
          for (int j = 0; j < kQRows; j++)
            bits[j] |= ((uint32_t)(strip[j] >> de) & 1u) << o;
        }
        continue;
      }
      for (int m = mb; m < me; m++) {
        const int o = tab.member[m];
        const int de = tab.off[o][last] - e_first;
        int32_t idx[kQRows];
#pragma unroll
        for (int j = 0; j < kQRows; j++) {
          const int b = (int)sh[j] + de;   // bit index into the 64-value strip (or beyond)
          idx[j] = -1;
          if (b < 32) {
            if ((mlo[j] >> b) & 1u)
              idx[j] = kMode == kMap
                  ? (int32_t)(ulo + s_hpos[slo[j]] + __popc(mlo[j] & ((1u << b) - 1u))) : 0;
          } else if (b < 64) {
            if ((mhi[j] >> (b - 32)) & 1u)
              idx[j] = kMode == kMap
                  ? (int32_t)(ulo + s_hpos[shi[j]] + __popc(mhi[j] & ((1u << (b - 32)) - 1u))) : 0;
          } else if (ok[j]) {   // offsets more than 63 apart inside one group: probe per member
            const uint32_t q = (c0[j] << 5) + (uint32_t)b;
            const uint32_t c = q >> 5;
            uint32_t h = 0;
            const uint32_t um = find_cell(slots, c, &h);
            if ((um >> (q & 31)) & 1u)
              idx[j] = kMode == kMap
                  ? (int32_t)(ulo + s_hpos[h] + __popc(um & ((1u << (q & 31)) - 1u))) : 0;
          }
        }
        emit<kMode>(a, o, row0, vec_ok, live, idx, bits);
      }
    }
  } else {
    // ---- general path -----------------------------------------------------
    for (int g = warp; g < G; g += kQWarps) {
      const int mb = tab.group_begin[g], me = tab.group_begin[g + 1];
      const uint64_t qlo = kfirst + (uint64_t)s_delta[tab.member[mb]];
      const uint64_t qhi = klast + (uint64_t)s_delta[tab.member[me - 1]];
      const int64_t lo = warp_bound(a.table, a.n_table, qlo, false, lane);
      const int64_t hi = warp_bound(a.table, a.n_table, qhi, true, lane);
      if (lane == 0) { s_glo[g] = lo; s_ghi[g] = max(lo, hi); }
    }
    __syncthreads();
    if (tid == 0) {
      int ns = 0, g = 0;
      while (g < G) {
        s_stage_gbeg[ns++] = g;
        int64_t lo = s_glo[g], hi = s_ghi[g];
        g++;
        if (hi - lo <= kQWindow) {
          while (g < G) {
            const int64_t nlo = min(lo, s_glo[g]), nhi = max(hi, s_ghi[g]);
            if (nhi - nlo > kQWindow) break;
            lo = nlo; hi = nhi; g++;
          }
        }
      }
      s_stage_gbeg[ns] = G;
      s_num_stages = ns;
    }
    __syncthreads();
    const int num_stages = s_num_stages;
    for (int st = 0; st < num_stages; st++) {
      const int gb = s_stage_gbeg[st], ge = s_stage_gbeg[st + 1];
      int64_t lo = s_glo[gb], hi = s_ghi[gb];
      for (int g = gb + 1; g < ge; g++) { lo = min(lo, s_glo[g]); hi = max(hi, s_ghi[g]); }
      const int64_t n = hi - lo;
      const bool staged = n <= kQWindow;
      if (staged) {
        for (int i = tid; i < (int)n; i += kQThreads) s_win[i] = __ldg(a.table + lo + i);
      }
      __syncthreads();
      for (int g = gb; g < ge; g++) {
        const int mb = tab.group_begin[g], me = tab.group_begin[g + 1];
        const int64_t glo = s_glo[g], ghi = s_ghi[g];
        int64_t pos[kQRows];
#pragma unroll
        for (int j = 0; j < kQRows; j++) {
          const uint64_t q0 = key[j] + (uint64_t)s_delta[tab.member[mb]];
          if (staged) {
            pos[j] = lo + lower_bound_win<uint64_t>(s_win, (int)(glo - lo), (int)(ghi - lo), q0);
          } else {
            int64_t l = glo, h = ghi;
            while (l < h) {
              const int64_t mid = (l + h) >> 1;
              if (__ldg(a.table + mid) < q0) l = mid + 1; else h = mid;
            }
            pos[j] = l;
          }
        }
        for (int m = mb; m < me; m++) {
          const int o = tab.member[m];
          int32_t idx[kQRows];
#pragma unroll
          for (int j = 0; j < kQRows; j++) {
            const uint64_t q = key[j] + (uint64_t)s_delta[o];
            int64_t p = pos[j];
            uint64_t v = kKeyInf;
            while (p < ghi) {
              v = staged ? s_win[p - lo] : __ldg(a.table + p);
              if (v >= q) break;
              p++;
              v = kKeyInf;
            }
            pos[j] = p;
            idx[j] = (live[j] && v == q) ? (int32_t)p : -1;
          }
          emit<kMode>(a, o, row0, vec_ok, live, idx, bits);
        }
      }
      __syncthreads();
    }
  }

  if (kMode == kBits) {
    if (live[kQRows - 1] && (reinterpret_cast<uintptr_t>(a.hit_words) & 15) == 0) {
      *reinterpret_cast<uint4 *>(a.hit_words + row0) = make_uint4(bits[0], bits[1], bits[2], bits[3]);
    } else {
#pragma unroll
      for (int j = 0; j < kQRows; j++) if (live[j]) a.hit_words[row0 + j] = bits[j];
    }
    // per-offset hit counts of the warp, four offsets at a time: the four bits of
    // a word are spread into four byte lanes by a multiply, summed over the rows
    // and reduced over the warp with one redux
    for (int o0 = 0; o0 < O; o0 += 4) {
      uint32_t packed = 0;
#pragma unroll
      for (int j = 0; j < kQRows; j++)
        packed += (((bits[j] >> o0) & 0xfu) * 0x00204081u) & 0x01010101u;
      packed = __reduce_add_sync(0xffffffffu, packed);  // each byte <= 128
      if (lane < 4 && o0 + lane < O) {
        const int c = (packed >> (8 * lane)) & 0xff;
        if (c != 0) atomicAdd(&s_counts[o0 + lane], c);
      }
    }
    __syncthreads();
    for (int o = tid; o < O; o += kQThreads)
      a.tile_counts[(int64_t)o * a.n_tiles + bid] = s_counts[o];
  }
}

// ---------------------------------------------------------------------------
// plan: per-offset exclusive scan of the tile counts, sizes
// ---------------------------------------------------------------------------
// Block (o, dir) turns row o of counts[dir] ([O, tiles]) into its exclusive
// prefix, in place, and writes the row total to sizes[dir * O + o].
struct ScanArgs {
  int32_t *counts[2];
  int32_t tiles[2];
  int32_t num_offsets;
  int32_t *sizes;  // [2, O]
};

__global__ void __launch_bounds__(1024) scan_tiles_kernel(const ScanArgs p) {
  __shared__ int32_t s_warp[32];
  __shared__ int32_t s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int o = blockIdx.x, dir = blockIdx.y;
  const int n = p.tiles[dir];
  int32_t *row = p.counts[dir] + (int64_t)o * n;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < n; b0 += 1024) {
    const int b = b0 + threadIdx.x;
    const int32_t v = b < n ? row[b] : 0;
    int32_t inc = v;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int32_t t = __shfl_up_sync(0xffffffffu, inc, s);
      if (lane >= s) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    int32_t before = s_carry;
    for (int w = 0; w < warp; w++) before += s_warp[w];
    if (b < n) row[b] = before + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = before + inc;
    __syncthreads();
  }
  if (threadIdx.x == 0) p.sizes[dir * p.num_offsets + o] = s_carry;
}

// order[p] = offset at mask row p (stable ascending sizes), sizes_out[p] its size
__device__ __forceinline__ void rank_offsets(const int32_t *sizes_raw, int O, int reorder,
                                             int32_t *s_pos /* shared [O] */) {
  for (int o = threadIdx.x; o < O; o += blockDim.x) {
    int pos = o;
    if (reorder) {
      const int32_t mine = sizes_raw[o];
      pos = 0;
      for (int j = 0; j < O; j++) {
        const int32_t other = sizes_raw[j];
        pos += (other < mine) || (other == mine && j < o);
      }
    }
    s_pos[o] = pos;
  }
}

__global__ void identity_order_kernel(int O, int32_t *order_out, int32_t *sizes_out) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o < O) { order_out[o] = o; sizes_out[o] = 0; }
}

// ---------------------------------------------------------------------------
// masks from hit words
// ---------------------------------------------------------------------------
struct EmitArgs {
  const uint32_t *words_t;   // [T] hit bits of target rows
  const uint32_t *words_s;   // [S] hit bits of source rows (== words_t when mirrored)
  const int32_t *prefix_t;   // [O, tiles_t] exclusive tile prefix, target direction
  const int32_t *prefix_s;   // [O, tiles_s] source direction (== prefix_t when mirrored)
  const int32_t *sizes_raw;  // [O] hits per offset (offset order)
  int32_t *order_out;        // [O] offset at mask row p
  int32_t *sizes_out;        // [O] size of mask row p
  int32_t reorder;
  int32_t *target_masks;     // [O, T]
  int32_t *source_masks;     // [O, S]
  int64_t T, S;
  int32_t tiles_t, tiles_s;
  int32_t num_offsets;
  uint8_t mirror[MN_MAX_OFFSETS];  // source direction: which offset's bit/prefix to read
};

// One block = 1024 consecutive rows of one direction; thread t owns rows
// 4t..4t+3.  For every offset the rank of a hit row is
//   tile prefix + hits in lower warps + hits in lower lanes + own earlier hits,
// and the four results leave as one 128-bit store when the row pitch allows it.
__global__ void __launch_bounds__(kQThreads)
emit_masks_kernel(const __grid_constant__ EmitArgs e) {
  __shared__ int32_t s_wtot[32][kQWarps + 1];  // offsets handled 32 at a time
  __shared__ int32_t s_pos[MN_MAX_OFFSETS];
  __shared__ int32_t s_pre[MN_MAX_OFFSETS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  rank_offsets(e.sizes_raw, e.num_offsets, e.reorder, s_pos);
  {
    // this tile's rank offset for every output row, fetched once per block
    const bool src_dir0 = blockIdx.x >= (unsigned)e.tiles_t;
    const int tile0 = src_dir0 ? blockIdx.x - e.tiles_t : blockIdx.x;
    const int32_t *prefix0 = src_dir0 ? e.prefix_s : e.prefix_t;
    const int n_tiles0 = src_dir0 ? e.tiles_s : e.tiles_t;
    for (int o = tid; o < e.num_offsets; o += kQThreads) {
      const int b = src_dir0 ? e.mirror[o] : o;
      s_pre[o] = __ldg(prefix0 + (int64_t)b * n_tiles0 + tile0);
    }
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int o = tid; o < e.num_offsets; o += kQThreads) {
      e.order_out[s_pos[o]] = o;
      e.sizes_out[s_pos[o]] = e.sizes_raw[o];
    }
  }
  const bool src_dir = blockIdx.x >= (unsigned)e.tiles_t;
  const int tile = src_dir ? blockIdx.x - e.tiles_t : blockIdx.x;
  const uint32_t *words = src_dir ? e.words_s : e.words_t;
  const int32_t *prefix = src_dir ? e.prefix_s : e.prefix_t;
  const int n_tiles = src_dir ? e.tiles_s : e.tiles_t;
  const int64_t n = src_dir ? e.S : e.T;
  int32_t *out = src_dir ? e.source_masks : e.target_masks;
  const int O = e.num_offsets;
  const unsigned lt = lanemask_lt();

  const int64_t row0 = (int64_t)tile * kQTile + tid * 4;
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  const bool vec_in = (row0 + 3 < n) && ((reinterpret_cast<uintptr_t>(words) & 15) == 0);
  if (vec_in) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(words + row0));
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++) if (row0 + i < n) w[i] = __ldg(words + row0 + i);
  }
  const bool vec_out = ((n & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);

  for (int o0 = 0; o0 < O; o0 += 32) {
    const int oc = min(32, O - o0);
    // warp totals of this chunk of offsets
    for (int oo = 0; oo < oc; oo++) {
      const int b = src_dir ? e.mirror[o0 + oo] : (o0 + oo);
      int c = ((w[0] >> b) & 1u) + ((w[1] >> b) & 1u) + ((w[2] >> b) & 1u) + ((w[3] >> b) & 1u);
      c = __reduce_add_sync(0xffffffffu, c);
      if (lane == 0) s_wtot[oo][warp] = c;
    }
    __syncthreads();
    if (tid < oc) {
      int run = 0;
#pragma unroll
      for (int ww = 0; ww < kQWarps; ww++) {
        const int t = s_wtot[tid][ww];
        s_wtot[tid][ww] = run;
        run += t;
      }
    }
    __syncthreads();
    for (int oo = 0; oo < oc; oo++) {
      const int o = o0 + oo;
      const int b = src_dir ? e.mirror[o] : o;
      const int v0 = (w[0] >> b) & 1u, v1 = (w[1] >> b) & 1u, v2 = (w[2] >> b) & 1u,
                v3 = (w[3] >> b) & 1u;
      const int mine = v0 + v1 + v2 + v3;
      // exclusive prefix of `mine` over the lanes of this warp
      int inc = mine;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, s);
        if (lane >= s) inc += t;
      }
      int r = s_pre[o] + s_wtot[oo][warp] + inc - mine;
      int4 res;
      res.x = v0 ? r : -1; r += v0;
      res.y = v1 ? r : -1; r += v1;
      res.z = v2 ? r : -1; r += v2;
      res.w = v3 ? r : -1;
      int32_t *dst = out + (int64_t)s_pos[o] * n + row0;
      if (vec_out) {
        if (row0 < n) *reinterpret_cast<int4 *>(dst) = res;
      } else {
        if (row0 + 0 < n) dst[0] = res.x;
        if (row0 + 1 < n) dst[1] = res.y;
        if (row0 + 2 < n) dst[2] = res.z;
        if (row0 + 3 < n) dst[3] = res.w;
      }
    }
    __syncthreads();
  }
  (void)lt;
}

// ---------------------------------------------------------------------------
// reference-API pieces that start from a materialised kernel map
// ---------------------------------------------------------------------------
// counts[o, tile] = valid entries of kernel_map[o, tile*1024 ...)
__global__ void __launch_bounds__(kQThreads)
map_count_kernel(const int32_t *__restrict__ kernel_map, int64_t T, int n_tiles,
                 int32_t *__restrict__ counts, int32_t *__restrict__ sizes_atomic) {
  const int o = blockIdx.y, tile = blockIdx.x;
  const int64_t t0 = (int64_t)tile * kQTile;
  int c = 0;
#pragma unroll
  for (int j = 0; j < kQRows; j++) {
    const int64_t t = t0 + j * kQThreads + threadIdx.x;
    if (t < T) c += __ldg(kernel_map + (int64_t)o * T + t) != -1;
  }
  c = __reduce_add_sync(0xffffffffu, c);
  __shared__ int s[kQWarps];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int w = 0; w < kQWarps; w++) tot += s[w];
    if (counts != nullptr) counts[(int64_t)o * n_tiles + tile] = tot;
    if (sizes_atomic != nullptr && tot != 0) atomicAdd(sizes_atomic + o, tot);
  }
}

// rank valid entries of row o by t; write the target mask densely and the
// source mask (pre-filled with -1) by scatter
__global__ void __launch_bounds__(kQThreads)
map_masks_kernel(const int32_t *__restrict__ kernel_map, int64_t S, int64_t T, int n_tiles,
                 const int32_t *__restrict__ prefix, int32_t *__restrict__ source_masks,
                 int32_t *__restrict__ target_masks) {
  const int o = blockIdx.y, tile = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t0 = (int64_t)tile * kQTile + threadIdx.x * 4;
  int32_t s_idx[4];
  int mine = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    s_idx[i] = (t0 + i < T) ? __ldg(kernel_map + (int64_t)o * T + t0 + i) : -1;
    mine += s_idx[i] != -1;
  }
  int inc = mine;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, s);
    if (lane >= s) inc += t;
  }
  __shared__ int s_w[kQWarps];
  if (lane == 31) s_w[warp] = inc;
  __syncthreads();
  int r = prefix[(int64_t)o * n_tiles + tile] + inc - mine;
  for (int w = 0; w < warp; w++) r += s_w[w];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    if (t0 + i < T) {
      const bool v = s_idx[i] != -1;
      target_masks[(int64_t)o * T + t0 + i] = v ? r : -1;
      if (v) source_masks[(int64_t)o * S + s_idx[i]] = r;
      r += v;
    }
  }
}

void fill_search_args(SearchArgs *a, const uint64_t *rows, int64_t n_rows, const uint64_t *table,
                      int64_t n_table, const OffsetTable &tab, const mn_keyspec &spec,
                      int32_t *kernel_map, uint32_t *hit_words, int32_t *tile_counts) {
  *a = SearchArgs{};
  a->rows = rows; a->table = table; a->n_rows = n_rows; a->n_table = n_table;
  a->kernel_map = kernel_map; a->hit_words = hit_words; a->tile_counts = tile_counts;
  a->n_tiles = (int)div_up(n_rows, kQTile);
  for (int k = 0; k < 4; k++) a->shift[k] = spec.shift[k];
  a->fast_ok = spec.shift[spec.ndim - 1] == 0;
  for (int o = 0; o < tab.num_offsets; o++) {
    const int e = tab.off[o][tab.ndim - 1];
    if (e > (int)kQPad || e < -(int)kQPad) a->fast_ok = 0;
  }
}

// Launches one search, or two in the same grid when `second` is given.
mn_status run_search(int mode, const SearchArgs &first, const OffsetTable &tab_first,
                     const SearchArgs *second, const OffsetTable *tab_second, cudaStream_t st) {
  thread_local static SearchPair sp;   // ~5 KB: kept off the stack; passed by value per launch
  sp.a[0] = first;
  sp.tab[0] = tab_first;
  sp.tiles0 = first.n_tiles;
  int blocks = first.n_tiles;
  if (second != nullptr) {
    sp.a[1] = *second;
    sp.tab[1] = *tab_second;
    blocks += second->n_tiles;
  }
  if (blocks == 0) return MN_OK;
  {
    LaunchScope scope(mode == kMap ? "search_kernel<map>" : "search_kernel<bits>", st);
    if (mode == kMap) search_kernel<kMap><<<blocks, kQThreads, 0, st>>>(sp);
    else search_kernel<kBits><<<blocks, kQThreads, 0, st>>>(sp);
  }
  MN_CHECK_LAUNCH();
  return MN_OK;
}

}  // namespace

mn_status make_offset_table(const int32_t *offsets, int64_t O, int ndim, int sign,
                            const mn_keyspec *spec, OffsetTable *out) {
  MN_CHECK_ARG(offsets != nullptr && spec != nullptr, "offset table: null pointer");
  MN_CHECK_ARG(O >= 1 && O <= MN_MAX_OFFSETS, "offset table: %lld offsets (supported: 1..%d)",
               (long long)O, MN_MAX_OFFSETS);
  MN_CHECK_ARG(ndim == spec->ndim, "offset table: ndim %d differs from the key spec's %d", ndim,
               spec->ndim);
  *out = OffsetTable{};
  out->num_offsets = (int32_t)O;
  out->ndim = ndim;
  for (int64_t o = 0; o < O; o++)
    for (int k = 0; k < ndim; k++) {
      const int64_t v = (int64_t)sign * offsets[o * ndim + k];
      MN_CHECK_ARG(v >= -(int64_t)spec->margin && v <= (int64_t)spec->margin,
                   "offset %lld exceeds the key margin %d", (long long)v, spec->margin);
      out->off[o][k] = (int32_t)v;
    }
  std::vector<int> idx(O);
  for (int64_t o = 0; o < O; o++) idx[o] = (int)o;
  std::stable_sort(idx.begin(), idx.end(), [&](int x, int y) {
    for (int k = 0; k < ndim; k++)
      if (out->off[x][k] != out->off[y][k]) return out->off[x][k] < out->off[y][k];
    return false;
  });
  int g = 0;
  for (int64_t i = 0; i < O; i++) {
    out->member[i] = (uint8_t)idx[i];
    bool new_group = i == 0;
    if (i > 0)
      for (int k = 0; k + 1 < ndim; k++)
        new_group |= out->off[idx[i]][k] != out->off[idx[i - 1]][k];
    if (new_group) out->group_begin[g++] = (uint8_t)i;
  }
  out->group_begin[g] = (uint8_t)O;
  out->num_groups = g;
  return MN_OK;
}

}  // namespace mn

using namespace mn;

extern "C" size_t mn_map_workspace_bytes(int64_t S, int64_t T, int64_t O) {
  const int64_t n = std::max<int64_t>(std::max(S, T), 1);
  size_t sort = 2 * align_up((size_t)n * 8, 256) + 2 * align_up((size_t)n * 4, 256) +
                radix_sort_workspace_bytes(n) + align_up((size_t)div_up(n, 2048) * 4, 256) + 512;
  const int64_t tiles = div_up(S, kQTile) + div_up(T, kQTile) + 2;
  size_t map = align_up((size_t)S * 4, 256) + align_up((size_t)T * 4, 256) +
               2 * align_up((size_t)std::max<int64_t>(O, 1) * tiles * 4, 256) + 4 * 1024;
  size_t bbox = (size_t)kNumSMs * 4 * 8 * 4 + 256;
  return std::max(std::max(sort, map), bbox) + 4096;
}

extern "C" mn_status mn_query_sorted_index_with_offsets(
    const uint64_t *source_keys, int64_t S, const uint64_t *target_keys, int64_t T,
    const int32_t *offsets, int64_t O, const mn_keyspec *spec, int32_t *kernel_map_out,
    void *stream) {
  MN_CHECK_ARG(S >= 0 && T >= 0, "query: negative size");
  MN_CHECK_ARG(spec != nullptr, "query: null key spec");
  MN_CHECK_ARG(S < (1ll << 31) && T < (1ll << 31), "query: more than 2^31-1 rows");
  OffsetTable tab;
  MN_RETURN_IF(make_offset_table(offsets, O, spec->ndim, +1, spec, &tab));
  if (T == 0) return MN_OK;
  MN_CHECK_ARG(target_keys != nullptr && kernel_map_out != nullptr && (S == 0 || source_keys != nullptr),
               "query: null pointer");
  SearchArgs a;
  fill_search_args(&a, target_keys, T, source_keys, S, tab, *spec, kernel_map_out, nullptr, nullptr);
  return run_search(kMap, a, tab, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" mn_status mn_compute_kernel_map_sizes(const int32_t *kernel_map, int64_t O, int64_t T,
                                                 int32_t *sizes_out, void *stream) {
  MN_CHECK_ARG(O >= 0 && T >= 0 && O <= 65535, "sizes: bad shape");
  if (O == 0) return MN_OK;
  MN_CHECK_ARG(sizes_out != nullptr, "sizes: null output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MN_CHECK_CUDA(cudaMemsetAsync(sizes_out, 0, sizeof(int32_t) * O, st));
  if (T == 0) return MN_OK;
  MN_CHECK_ARG(kernel_map != nullptr, "sizes: null kernel map");
  const int n_tiles = (int)div_up(T, kQTile);
  MN_LAUNCH("map_count_kernel", st, map_count_kernel<<<dim3(n_tiles, (unsigned)O), kQThreads, 0, st>>>(kernel_map, T, n_tiles, nullptr,
                                                                     sizes_out));
  return MN_OK;
}

extern "C" mn_status mn_compute_kernel_map_masks(const int32_t *kernel_map, int64_t O, int64_t S,
                                                 int64_t T, int32_t *source_masks_out,
                                                 int32_t *target_masks_out, void *ws_ptr,
                                                 size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(O >= 0 && S >= 0 && T >= 0, "masks: bad shape");
  MN_CHECK_ARG(O <= MN_MAX_OFFSETS, "masks: %lld offsets (supported: up to %d)", (long long)O,
               MN_MAX_OFFSETS);
  if (O == 0) return MN_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (S > 0) {
    MN_CHECK_ARG(source_masks_out != nullptr, "masks: null source mask");
    MN_CHECK_CUDA(cudaMemsetAsync(source_masks_out, 0xff, sizeof(int32_t) * O * S, st));
  }
  if (T == 0) return MN_OK;
  MN_CHECK_ARG(kernel_map != nullptr && target_masks_out != nullptr, "masks: null pointer");
  Workspace ws(ws_ptr, ws_bytes);
  const int n_tiles = (int)div_up(T, kQTile);
  int32_t *counts = ws.take<int32_t>((size_t)O * n_tiles);
  int32_t *scratch = ws.take<int32_t>(4 * MN_MAX_OFFSETS);
  MN_CHECK_WS(ws);
  MN_LAUNCH("map_count_kernel", st, map_count_kernel<<<dim3(n_tiles, (unsigned)O), kQThreads, 0, st>>>(kernel_map, T, n_tiles, counts,
                                                                     nullptr));
  ScanArgs p{};
  p.counts[0] = counts; p.tiles[0] = n_tiles; p.num_offsets = (int)O; p.sizes = scratch;
  MN_LAUNCH("scan_tiles_kernel", st, scan_tiles_kernel<<<dim3((unsigned)O, 1), 1024, 0, st>>>(p));
  MN_LAUNCH("map_masks_kernel", st, map_masks_kernel<<<dim3(n_tiles, (unsigned)O), kQThreads, 0, st>>>(
      kernel_map, S, T, n_tiles, counts, source_masks_out, target_masks_out));
  return MN_OK;
}

extern "C" mn_status mn_build_kernel_map(const uint64_t *source_keys, int64_t S,
                                         const uint64_t *target_keys, int64_t T,
                                         const int32_t *offsets, int64_t O,
                                         const mn_keyspec *spec, int reorder,
                                         int32_t *source_masks_out, int32_t *target_masks_out,
                                         int32_t *order_out, int32_t *sizes_out, void *ws_ptr,
                                         size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(S >= 0 && T >= 0, "build_kernel_map: negative size");
  MN_CHECK_ARG(spec != nullptr, "build_kernel_map: null key spec");
  MN_CHECK_ARG(S < (1ll << 31) && T < (1ll << 31), "build_kernel_map: more than 2^31-1 rows");
  if (O > 32) {
    set_error("build_kernel_map: the fused build handles up to 32 offsets (got %lld); use "
              "mn_query_sorted_index_with_offsets + mn_compute_kernel_map_masks", (long long)O);
    return MN_ERR_UNSUPPORTED;
  }
  MN_CHECK_ARG(order_out != nullptr && sizes_out != nullptr, "build_kernel_map: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ndim = spec->ndim;
  OffsetTable fwd;
  MN_RETURN_IF(make_offset_table(offsets, O, ndim, +1, spec, &fwd));

  // mirrored offset of every offset, if the table is symmetric
  bool symmetric = true;
  uint8_t neg[MN_MAX_OFFSETS] = {0};
  for (int64_t o = 0; o < O && symmetric; o++) {
    int found = -1;
    for (int64_t j = 0; j < O && found < 0; j++) {
      bool same = true;
      for (int k = 0; k < ndim; k++) same &= offsets[j * ndim + k] == -offsets[o * ndim + k];
      if (same) found = (int)j;
    }
    if (found < 0) symmetric = false; else neg[o] = (uint8_t)found;
  }
  const bool mirrored = symmetric && source_keys == target_keys && S == T;

  Workspace ws(ws_ptr, ws_bytes);
  const int tiles_t = (int)div_up(T, kQTile), tiles_s = (int)div_up(S, kQTile);
  uint32_t *words_t = ws.take<uint32_t>(std::max<int64_t>(T, 1));
  int32_t *counts_t = ws.take<int32_t>((size_t)O * std::max(tiles_t, 1));
  uint32_t *words_s = words_t;
  int32_t *counts_s = counts_t;
  if (!mirrored) {
    words_s = ws.take<uint32_t>(std::max<int64_t>(S, 1));
    counts_s = ws.take<int32_t>((size_t)O * std::max(tiles_s, 1));
  }
  int32_t *sizes_raw = ws.take<int32_t>(2 * MN_MAX_OFFSETS);
  MN_CHECK_WS(ws);

  if (T == 0 || S == 0) {
    // nothing can match: every mask entry is -1, every size 0
    if (S > 0 && O > 0) MN_CHECK_CUDA(cudaMemsetAsync(source_masks_out, 0xff, sizeof(int32_t) * O * S, st));
    if (T > 0 && O > 0) MN_CHECK_CUDA(cudaMemsetAsync(target_masks_out, 0xff, sizeof(int32_t) * O * T, st));
    MN_LAUNCH("identity_order_kernel", st,
              identity_order_kernel<<<1, MN_MAX_OFFSETS, 0, st>>>((int)O, order_out, sizes_out));
    return MN_OK;
  }
  MN_CHECK_ARG(source_keys != nullptr && target_keys != nullptr && source_masks_out != nullptr &&
                   target_masks_out != nullptr, "build_kernel_map: null pointer");

  SearchArgs fwd_args, bwd_args;
  fill_search_args(&fwd_args, target_keys, T, source_keys, S, fwd, *spec, nullptr, words_t, counts_t);
  if (mirrored) {
    MN_RETURN_IF(run_search(kBits, fwd_args, fwd, nullptr, nullptr, st));
  } else {
    // second direction in the same launch: sources as rows, targets as table, -offsets
    OffsetTable bwd;
    MN_RETURN_IF(make_offset_table(offsets, O, ndim, -1, spec, &bwd));
    fill_search_args(&bwd_args, source_keys, S, target_keys, T, bwd, *spec, nullptr, words_s, counts_s);
    MN_RETURN_IF(run_search(kBits, fwd_args, fwd, &bwd_args, &bwd, st));
  }
  ScanArgs p{};
  p.counts[0] = counts_t; p.tiles[0] = tiles_t;
  p.counts[1] = counts_s; p.tiles[1] = tiles_s;
  p.num_offsets = (int)O; p.sizes = sizes_raw;
  MN_LAUNCH("scan_tiles_kernel", st,
            scan_tiles_kernel<<<dim3((unsigned)O, mirrored ? 1 : 2), 1024, 0, st>>>(p));

  EmitArgs e{};
  e.words_t = words_t; e.words_s = words_s; e.prefix_t = counts_t; e.prefix_s = counts_s;
  e.sizes_raw = sizes_raw; e.order_out = order_out; e.sizes_out = sizes_out;
  e.reorder = reorder ? 1 : 0; e.target_masks = target_masks_out; e.source_masks = source_masks_out;
  e.T = T; e.S = S; e.tiles_t = tiles_t; e.tiles_s = tiles_s; e.num_offsets = (int)O;
  for (int64_t o = 0; o < O; o++) e.mirror[o] = mirrored ? neg[o] : (uint8_t)o;
  MN_LAUNCH("emit_masks_kernel", st, emit_masks_kernel<<<tiles_t + tiles_s, kQThreads, 0, st>>>(e));
  return MN_OK;
}
