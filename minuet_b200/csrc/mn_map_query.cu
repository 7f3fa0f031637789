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
// Here the map build is two launches over packed 64-bit keys.
//
// search_kernel: a block owns 512 consecutive rows (targets).  Two
// warp-cooperative 32-ary ballot searches find the window of the sorted table
// (sources) that can match the tile over all offsets; the window is staged in
// shared memory as a hash set of CELLS (32 consecutive values of the last
// dimension -> {cell id, 32-bit occupancy}, 8-byte slots, linear probing): the
// offsets that differ only in the last dimension (a "group", split so that its
// span is at most 16) are answered by ONE lookup per row, plus a second one for
// the few rows whose strip crosses a cell boundary; shared-memory bandwidth, not
// instruction issue, is what bounds this kernel, hence the 64-bit single-slot
// lookups.  Tiles whose window does not fit the hash are
// processed group range by group range, and ranges that still do not fit fall
// back to binary search in global memory.  The kernel writes kernel-map rows
// or, for the fused build, one 32-bit word of per-offset hit bits per row.
//
// emit_masks_kernel (cooperative launch, all blocks resident): every block
// owns a contiguous range of 512-row tiles.  Phase 1 counts the hits per
// offset of its range (32x32 bit-matrix transposes turn 32 hit words into 32
// per-offset row masks); one grid barrier later every block knows its rank
// offset per offset and the total sizes, hence the stable size order; phase 2
// turns each tile's row masks into ranks in a shared-memory staging tile
// (pre-filled with -1, only the hits are patched) and writes every mask row
// segment with one bulk asynchronous copy (cp.async.bulk shared -> global),
// whatever the alignment of the row pitch.  No memset, no select, no scatter,
// no separate scan kernel.  For submanifold maps (sources == targets,
// symmetric offsets) the source mask of offset o is read off the hit bits of
// the mirrored offset.
#include "mn_grid.cuh"

#include <algorithm>
#include <vector>

namespace mn {

namespace {

constexpr int kQThreads = 256;
constexpr int kQWarps = kQThreads / 32;
constexpr int kQRows = 2;                    // rows per thread
constexpr int kQTile = kQThreads * kQRows;   // 512 rows per block
constexpr int kQSlots = 4096;                // hash slots of 8 bytes: {cell, occupancy}
constexpr int kQMaxWindow = 1280;            // table keys per hashed stage (load factor <= 0.31)
constexpr int kQMaxSpan = 16;                // last-dimension span of one group
constexpr uint32_t kQPad = 64;               // relative keys start at kQPad
constexpr uint32_t kHashEmpty = 0xffffffffu;
constexpr uint64_t kRelLimit = 0xffffffffull - 4ull * kQPad;

__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Warp-cooperative 32-ary search in global memory: lower bound (first index
// with t[i] >= q) or upper bound (first index with t[i] > q) inside [lo, hi).
// Every lane probes one pivot per round, a ballot narrows the range 32-fold;
// ~4 rounds for half a million keys.  All 32 lanes must call with identical
// arguments.
__device__ __forceinline__ int64_t warp_bound(const uint64_t *__restrict__ t, int64_t lo,
                                              int64_t hi, uint64_t q, bool upper, int lane) {
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
  int32_t *kernel_map;     // kMap:  [O, n_rows]
  uint32_t *hit_words;     // kBits / kBitsRev: [n_rows]
  uint32_t *table_words;   // kBitsRev: [n_table], zeroed; bit o of entry s is set when row t hits s
  int32_t n_tiles;
};

// One launch can serve two searches (e.g. targets->sources and sources->targets).
struct SearchPair {
  SearchArgs a[2];
  OffsetTable tab[2];
  SpecRef spec;
  int32_t tiles0;   // blocks of the first search
};

// kMap: kernel-map rows; kBits: per-row hit words; kBitsRev: hit words of the rows
// and, through atomicOr at the matched table position, of the table entries
// (one search then serves both masks of a map whose two sides differ).
enum SearchMode { kMap = 0, kBits = 1, kBitsRev = 2 };

MN_MARKS_DECL(g_marks_search);
MN_MARKS_DECL(g_marks_emit);

__device__ __forceinline__ uint32_t hash_slot(uint32_t c) {
  return (c * 0x9E3779B1u) >> 20;  // top 12 bits: 4096 slots
}

// Occupancy mask of cell c (0 when absent) and the slot that holds it: linear
// probing over 8-byte {cell, mask} slots, one 64-bit shared-memory load per step.
// At the load factors used (<= 0.31) most lookups end at the first slot.
__device__ __forceinline__ uint32_t find_cell(const uint2 *slots, uint32_t c, uint32_t *slot) {
  uint32_t h = hash_slot(c);
  for (int probe = 0; probe < kQSlots; probe++) {
    const uint2 v = slots[h];
    if (v.x == c) { *slot = h; return v.y; }
    if (v.x == kHashEmpty) break;
    h = (h + 1) & (kQSlots - 1);
  }
  *slot = 0;
  return 0u;
}

__device__ __forceinline__ uint32_t insert_cell(uint2 *slots, uint32_t c, uint32_t bit) {
  uint32_t h = hash_slot(c);
  for (int probe = 0; probe < kQSlots; probe++) {
    const uint32_t old = atomicCAS(&slots[h].x, kHashEmpty, c);
    if (old == kHashEmpty || old == c) break;
    h = (h + 1) & (kQSlots - 1);
  }
  atomicOr(&slots[h].y, 1u << bit);
  return h;
}

template <int kMode>
__global__ void __launch_bounds__(kQThreads, kMode == kBits ? 5 : 4)
search_kernel(const __grid_constant__ SearchPair sp) {
  constexpr bool kPos = kMode != kBits;   // table positions are needed
  // blocks [0, tiles0) serve direction 0, the rest direction 1 (rows and table swapped)
  const int dir = (int)blockIdx.x >= sp.tiles0 ? 1 : 0;
  const int bid = (int)blockIdx.x - dir * sp.tiles0;
  const SearchArgs &a = sp.a[dir];
  const OffsetTable &tab = sp.tab[dir];
  const mn_keyspec &spec = spec_of(sp.spec);
  __shared__ __align__(16) uint2 s_slots[kQSlots];
  __shared__ uint16_t s_hpos[kPos ? kQSlots : 2];   // first position of a cell
  __shared__ int64_t s_delta[MN_MAX_OFFSETS];
  __shared__ int64_t s_gdelta[MN_MAX_OFFSETS];       // per group: delta of its first member
  __shared__ uint32_t s_gmeta[MN_MAX_OFFSETS];       // span | first offset << 8 | members << 16 | compact << 24
  __shared__ int64_t s_glo[MN_MAX_OFFSETS], s_ghi[MN_MAX_OFFSETS];
  __shared__ int64_t s_slo[MN_MAX_OFFSETS], s_shi[MN_MAX_OFFSETS];
  __shared__ uint8_t s_stage_gbeg[MN_MAX_OFFSETS + 1];
  __shared__ int32_t s_num_stages;
  __shared__ int64_t s_union[2];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int O = tab.num_offsets, G = tab.num_groups;
  const int last = tab.ndim - 1;
  const int64_t tile0 = (int64_t)bid * kQTile;
  const int tile_rows = (int)min((int64_t)kQTile, a.n_rows - tile0);
  const int64_t row0 = tile0 + tid * kQRows;
  MN_MARK(g_marks_search, 0);

  for (int o = tid; o < O; o += kQThreads) {
    int64_t d = 0;
    for (int k = 0; k < tab.ndim; k++) d += (int64_t)tab.off[o][k] * ((int64_t)1 << spec.shift[k]);
    s_delta[o] = d;
  }
  for (int g = tid; g < G; g += kQThreads) {
    const int mb = tab.group_begin[g], me = tab.group_begin[g + 1];
    const int o_first = tab.member[mb];
    int64_t d = 0;
    for (int k = 0; k < tab.ndim; k++) d += (int64_t)tab.off[o_first][k] * ((int64_t)1 << spec.shift[k]);
    s_gdelta[g] = d;
    // compact: member i is offset o_first + i and sits i values further along the last dimension
    bool compact = true;
    for (int m = mb; m < me; m++)
      compact &= tab.member[m] == o_first + (m - mb) &&
                 tab.off[tab.member[m]][last] - tab.off[o_first][last] == m - mb;
    const int span = tab.off[tab.member[me - 1]][last] - tab.off[o_first][last];
    s_gmeta[g] = (uint32_t)span | ((uint32_t)o_first << 8) | ((uint32_t)(me - mb) << 16) |
                 ((compact ? 1u : 0u) << 24);
  }

  uint64_t key[kQRows];
  bool live[kQRows];
  if (tid * kQRows + kQRows <= tile_rows && (reinterpret_cast<uintptr_t>(a.rows) & 15) == 0) {
    const ulonglong2 v = __ldg(reinterpret_cast<const ulonglong2 *>(a.rows + row0));
    key[0] = v.x; key[1] = v.y;
    live[0] = live[1] = true;
  } else {
#pragma unroll
    for (int j = 0; j < kQRows; j++) {
      live[j] = tid * kQRows + j < tile_rows;
      key[j] = live[j] ? __ldg(a.rows + row0 + j) : 0ull;
    }
  }
  const uint64_t kfirst = __ldg(a.rows + tile0);
  const uint64_t klast = __ldg(a.rows + tile0 + tile_rows - 1);
  __syncthreads();
  MN_MARK(g_marks_search, 1);

  // window of the table over all offsets: members are ordered by delta
  if (warp < 2) {
    const uint64_t q = warp == 0 ? kfirst + (uint64_t)s_delta[tab.member[0]]
                                 : klast + (uint64_t)s_delta[tab.member[O - 1]];
    const int64_t r = warp_bound(a.table, 0, a.n_table, q, warp == 1, lane);
    if (lane == 0) s_union[warp] = r;
  }
  __syncthreads();
  {
    const int64_t ulo = s_union[0], uhi = max(s_union[0], s_union[1]);
    bool one_stage = uhi - ulo <= kQMaxWindow;
    if (one_stage && uhi > ulo)
      one_stage = __ldg(a.table + uhi - 1) - __ldg(a.table + ulo) < kRelLimit;
    if (one_stage) {
      if (tid == 0) {
        s_num_stages = 1;
        s_stage_gbeg[0] = 0;
        s_stage_gbeg[1] = (uint8_t)G;
        s_slo[0] = ulo;
        s_shi[0] = uhi;
      }
    } else {
      // per-group windows inside the union window, then consecutive groups are
      // merged into stages for as long as their joint window fits the hash
      for (int g = warp; g < G; g += kQWarps) {
        const int mb = tab.group_begin[g], me = tab.group_begin[g + 1];
        const uint64_t qlo = kfirst + (uint64_t)s_delta[tab.member[mb]];
        const uint64_t qhi = klast + (uint64_t)s_delta[tab.member[me - 1]];
        const int64_t lo = warp_bound(a.table, ulo, uhi, qlo, false, lane);
        const int64_t hi = warp_bound(a.table, ulo, uhi, qhi, true, lane);
        if (lane == 0) { s_glo[g] = lo; s_ghi[g] = max(lo, hi); }
      }
      __syncthreads();
      if (tid == 0) {
        int ns = 0, g = 0;
        while (g < G) {
          s_stage_gbeg[ns] = (uint8_t)g;
          int64_t lo = s_glo[g], hi = s_ghi[g];
          g++;
          if (hi - lo <= kQMaxWindow) {
            while (g < G) {
              const int64_t nlo = min(lo, s_glo[g]), nhi = max(hi, s_ghi[g]);
              if (nhi - nlo > kQMaxWindow) break;
              lo = nlo; hi = nhi; g++;
            }
          }
          s_slo[ns] = lo;
          s_shi[ns] = hi;
          ns++;
        }
        s_stage_gbeg[ns] = (uint8_t)G;
        s_num_stages = ns;
      }
    }
  }
  __syncthreads();
  MN_MARK(g_marks_search, 2);

  uint32_t bits[kQRows] = {0u, 0u};
  const bool vec_ok = kMode == kMap && (a.n_rows & 1) == 0 &&
                      (reinterpret_cast<uintptr_t>(a.kernel_map) & 7) == 0 && live[kQRows - 1];
  const int num_stages = s_num_stages;
  for (int st = 0; st < num_stages; st++) {
    const int gb = s_stage_gbeg[st], ge = s_stage_gbeg[st + 1];
    const int64_t lo = s_slo[st], hi = s_shi[st];
    const int wn = (int)min(hi - lo, (int64_t)kQMaxWindow + 1);
    bool hashed = hi - lo <= kQMaxWindow;
    uint64_t base = 0;
    if (hashed && wn > 0) {
      base = __ldg(a.table + lo);
      hashed = __ldg(a.table + hi - 1) - base < kRelLimit;
    }
    if (hashed) {
      {
        uint4 *clear = reinterpret_cast<uint4 *>(s_slots);
        for (int i = tid; i < kQSlots / 2; i += kQThreads)
          clear[i] = make_uint4(kHashEmpty, 0u, kHashEmpty, 0u);   // two {cell, mask} slots
      }
      __syncthreads();
      MN_MARK(g_marks_search, 3);
      // relative keys start at kQPad, so that a query below the window stays non-negative
      for (int w = tid; w < wn; w += kQThreads) {
        const uint32_t k = (uint32_t)(__ldg(a.table + lo + w) - base) + kQPad;
        const uint32_t h = insert_cell(s_slots, k >> 5, k & 31u);
        if (kPos) {
          // the table is sorted: exactly one key of a cell has a predecessor in another cell
          uint32_t pk = 0;
          if (w > 0) pk = (uint32_t)(__ldg(a.table + lo + w - 1) - base) + kQPad;
          if (w == 0 || (pk >> 5) != (k >> 5)) s_hpos[h] = (uint16_t)w;
        }
      }
      __syncthreads();
      MN_MARK(g_marks_search, 4);
      int64_t rel[kQRows];
#pragma unroll
      for (int j = 0; j < kQRows; j++)   // a dead row gets a value that no window can reach
        rel[j] = live[j] ? (int64_t)(key[j] - base) + kQPad : (int64_t)1 << 62;
      for (int g = gb; g < ge; g++) {
        const int64_t dg = s_gdelta[g];
        const uint32_t meta = s_gmeta[g];
        const uint32_t e_span = meta & 0xffu, o_first = (meta >> 8) & 0xffu,
                       members = (meta >> 16) & 0xffu;
        // per row: the strip of last-dimension values [q0, q0 + 31] as one 32-bit mask, from
        // the cell of q0 and, when the group reaches past its end, the next cell
        uint32_t sh[kQRows], mlo[kQRows], mhi[kQRows], slo[kQRows], shi[kQRows];
#pragma unroll
        for (int j = 0; j < kQRows; j++) {
          const uint64_t t0 = (uint64_t)(rel[j] + dg);
          const uint32_t q0 = (uint32_t)t0;
          const bool ok = t0 < kRelLimit;
          sh[j] = q0 & 31u;
          slo[j] = shi[j] = 0u;
          mlo[j] = mhi[j] = 0u;
          if (ok) {
            mlo[j] = find_cell(s_slots, q0 >> 5, &slo[j]);
            if (sh[j] + e_span > 31u) mhi[j] = find_cell(s_slots, (q0 >> 5) + 1u, &shi[j]);
          }
        }
        if (kMode == kBits && (meta >> 24) != 0u) {
#pragma unroll
          for (int j = 0; j < kQRows; j++) {
            const uint32_t strip = (uint32_t)((((uint64_t)mhi[j] << 32) | mlo[j]) >> sh[j]);
            bits[j] |= (strip & ((1u << members) - 1u)) << o_first;
          }
          continue;
        }
        const int mb = tab.group_begin[g], me = mb + (int)members;
        const int e_first = tab.off[o_first][last];
        for (int m = mb; m < me; m++) {
          const int o = tab.member[m];
          const int de = tab.off[o][last] - e_first;
          if (kMode == kBits) {
#pragma unroll
            for (int j = 0; j < kQRows; j++) {
              const uint64_t both = ((uint64_t)mhi[j] << 32) | mlo[j];
              bits[j] |= ((uint32_t)(both >> (sh[j] + de)) & 1u) << o;
            }
          } else {
            int32_t idx[kQRows];
#pragma unroll
            for (int j = 0; j < kQRows; j++) {
              const uint32_t b = sh[j] + (uint32_t)de;   // < 48
              idx[j] = -1;
              if (b < 32u) {
                if ((mlo[j] >> b) & 1u)
                  idx[j] = (int32_t)(lo + s_hpos[slo[j]] + __popc(mlo[j] & ((1u << b) - 1u)));
              } else if ((mhi[j] >> (b - 32u)) & 1u) {
                idx[j] = (int32_t)(lo + s_hpos[shi[j]] + __popc(mhi[j] & ((1u << (b - 32u)) - 1u)));
              }
            }
            if (kMode == kBitsRev) {
#pragma unroll
              for (int j = 0; j < kQRows; j++) {
                if (idx[j] >= 0) {
                  bits[j] |= 1u << o;
                  atomicOr(a.table_words + idx[j], 1u << o);
                }
              }
            } else {
              int32_t *dst = a.kernel_map + (int64_t)o * a.n_rows + row0;
              if (vec_ok) {
                *reinterpret_cast<int2 *>(dst) = make_int2(idx[0], idx[1]);
              } else {
#pragma unroll
                for (int j = 0; j < kQRows; j++) if (live[j]) dst[j] = idx[j];
              }
            }
          }
        }
      }
      __syncthreads();
    } else {
      // ---- window too large or too wide for the hash: binary search in global memory
      for (int g = gb; g < ge; g++) {
        const int mb = tab.group_begin[g], me = tab.group_begin[g + 1];
        const int64_t glo = s_glo[g], ghi = s_ghi[g];
        int64_t pos[kQRows];
#pragma unroll
        for (int j = 0; j < kQRows; j++) {
          const uint64_t q0 = key[j] + (uint64_t)s_delta[tab.member[mb]];
          int64_t l = glo, h = ghi;
          while (l < h) {
            const int64_t mid = (l + h) >> 1;
            if (__ldg(a.table + mid) < q0) l = mid + 1; else h = mid;
          }
          pos[j] = l;
        }
        for (int m = mb; m < me; m++) {
          const int o = tab.member[m];
          int32_t idx[kQRows];
#pragma unroll
          for (int j = 0; j < kQRows; j++) {
            const uint64_t q = key[j] + (uint64_t)s_delta[o];
            int64_t p = pos[j];
            uint64_t v = ~0ull;
            while (p < ghi) {   // at most kQMaxSpan steps: the table holds distinct keys
              v = __ldg(a.table + p);
              if (v >= q) break;
              p++;
              v = ~0ull;
            }
            pos[j] = p;
            idx[j] = (live[j] && v == q) ? (int32_t)p : -1;
          }
          if (kMode == kMap) {
            int32_t *dst = a.kernel_map + (int64_t)o * a.n_rows + row0;
#pragma unroll
            for (int j = 0; j < kQRows; j++) if (live[j]) dst[j] = idx[j];
          } else {
#pragma unroll
            for (int j = 0; j < kQRows; j++) {
              if (idx[j] >= 0) {
                bits[j] |= 1u << o;
                if (kMode == kBitsRev) atomicOr(a.table_words + idx[j], 1u << o);
              }
            }
          }
        }
      }
    }
  }

  MN_MARK(g_marks_search, 5);
  if (kMode != kMap) {
    if (live[kQRows - 1] && (reinterpret_cast<uintptr_t>(a.hit_words) & 7) == 0) {
      *reinterpret_cast<uint2 *>(a.hit_words + row0) = make_uint2(bits[0], bits[1]);
    } else {
#pragma unroll
      for (int j = 0; j < kQRows; j++) if (live[j]) a.hit_words[row0 + j] = bits[j];
    }
  }
}

// ---------------------------------------------------------------------------
// masks from hit words (fused build)
// ---------------------------------------------------------------------------
constexpr int kEThreads = 512;
constexpr int kEWarps = kEThreads / 32;
constexpr int kETile = 512;           // rows per tile: one 32-row segment per warp
constexpr int kEPitch = kETile + 4;   // staging row pitch (elements), a multiple of 4
constexpr int kEBatch = 8;            // tiles whose hit words are fetched together

struct EmitArgs {
  const uint32_t *words_t;   // [T] hit bits of target rows
  const uint32_t *words_s;   // [S] hit bits of source rows (== words_t when mirrored)
  int32_t *target_masks;     // [O, T]
  int32_t *source_masks;     // [O, S]
  int32_t *order_out;        // [O] offset at mask row p
  int32_t *sizes_out;        // [O + 1] size of mask row p, then a copy of the status word
  uint32_t *bits_t;          // optional [T]: bit p set when mask row p has an entry for the target
  uint32_t *bits_s;          // optional [S]: the same for the sources
  int32_t *agg;              // workspace [64 pairs][grid]: hit counts of every block's tile
                             // range, then their exclusive prefix; pair = direction * 32 + offset
  int32_t *total;            // workspace [64]
  int32_t *ctrl;
  int64_t T, S;
  int32_t tiles_t, tiles_s;
  int32_t num_offsets;
  int32_t reorder;
  uint8_t mirror[32];        // source direction: which offset's bit to read
};

// Transpose of the 32x32 bit matrix held one row per lane: on return lane j
// holds column j (bit i = bit j of lane i's input).
__device__ __forceinline__ uint32_t transpose32(uint32_t x, int lane) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    const uint32_t low = s == 16 ? 0x0000ffffu : s == 8 ? 0x00ff00ffu : s == 4 ? 0x0f0f0f0fu
                       : s == 2 ? 0x33333333u : 0x55555555u;
    const uint32_t y = __shfl_xor_sync(0xffffffffu, x, s);
    x = (lane & s) ? ((x & ~low) | ((y & ~low) >> s)) : ((x & low) | ((y & low) << s));
  }
  return x;
}

__device__ __forceinline__ void bulk_store(void *dst_global, const void *src_shared, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_global),
               "r"((uint32_t)__cvta_generic_to_shared(src_shared)), "r"(bytes)
               : "memory");
}

__global__ void __launch_bounds__(kEThreads)
emit_masks_kernel(const __grid_constant__ EmitArgs e) {
  extern __shared__ __align__(16) int32_t s_stage[];   // [O][kEPitch]
  __shared__ int32_t s_wcnt[32][kEWarps + 1];           // per offset: warp counts, then warp bases
  __shared__ int32_t s_run[2][32];                      // rank of the next hit, per direction / offset
  __shared__ int32_t s_size[32], s_pos[32], s_ord[32];
  __shared__ int32_t s_mis[32];
  __shared__ uint32_t s_words[kEBatch][kETile];         // hit words of up to kEBatch tiles
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int O = e.num_offsets;
  const int G = (int)gridDim.x, b = (int)blockIdx.x;
  const int total_tiles = e.tiles_t + e.tiles_s;
  const int t_begin = (int)((int64_t)total_tiles * b / G);
  const int t_end = (int)((int64_t)total_tiles * (b + 1) / G);
  const unsigned lt = lanemask_lt();
  const int my_mirror = lane < O ? e.mirror[lane] : 0;

  MN_MARK(g_marks_emit, 0);
  // hit words of tiles [first, first + kEBatch) of this block's range: all loads are in
  // flight together; a thread only ever reads back the words it loaded itself
  auto fetch_words = [&](int first) {
#pragma unroll
    for (int k = 0; k < kEBatch; k++) {
      const int tile = first + k;
      uint32_t w = 0u;
      if (tile < t_end) {
        const int dir = tile >= e.tiles_t ? 1 : 0;
        const int64_t r = (int64_t)(tile - dir * e.tiles_t) * kETile + tid;
        const int64_t n = dir ? e.S : e.T;
        if (r < n) w = __ldg((dir ? e.words_s : e.words_t) + r);
      }
      s_words[k][tid] = w;
    }
  };

  // ---- phase 1: hits per offset of this block's tile range ---------------------
  int cnt0 = 0, cnt1 = 0;   // lane o: hits of offset o, per direction
  for (int first = t_begin; first < t_end; first += kEBatch) {
    fetch_words(first);
    for (int tile = first; tile < min(first + kEBatch, t_end); tile++) {
      const int dir = tile >= e.tiles_t ? 1 : 0;
      const uint32_t w = s_words[tile - first][tid];
      if (__ballot_sync(0xffffffffu, w != 0u) == 0u) continue;
      uint32_t plane = transpose32(w, lane);
      if (dir) plane = __shfl_sync(0xffffffffu, plane, my_mirror);
      if (dir) cnt1 += __popc(plane); else cnt0 += __popc(plane);
    }
  }
  for (int d = 0; d < 2; d++) {
    if (lane < O) s_wcnt[lane][warp] = d ? cnt1 : cnt0;
    __syncthreads();
    if (tid < 32) {
      int sum = 0;
      if (tid < O)
        for (int w = 0; w < kEWarps; w++) sum += s_wcnt[tid][w];
      e.agg[(int64_t)(d * 32 + tid) * G + b] = sum;
    }
    __syncthreads();
  }
  MN_MARK(g_marks_emit, 1);
  grid_barrier(e.ctrl, (unsigned)G);
  MN_MARK(g_marks_emit, 2);

  // ---- one warp per (direction, offset): exclusive prefix over the blocks ----------
  for (int pair = b * kEWarps + warp; pair < 64; pair += G * kEWarps) {
    {
      int32_t *row = e.agg + (int64_t)pair * G;
      int carry = 0;
      for (int b0 = 0; b0 < G; b0 += 32) {
        const int bb = b0 + lane;
        const int v = bb < G ? __ldcg(row + bb) : 0;
        int inc = v;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, inc, s);
          if (lane >= s) inc += t;
        }
        if (bb < G) row[bb] = carry + inc - v;
        carry += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) e.total[pair] = carry;
    }
  }
  MN_MARK(g_marks_emit, 3);
  grid_barrier(e.ctrl, (unsigned)G);
  MN_MARK(g_marks_emit, 4);

  // ---- rank offsets of this block, total sizes, size order ---------------------
  if (tid < 64) s_run[tid >> 5][tid & 31] = __ldcg(e.agg + (int64_t)tid * G + b);
  if (tid < 32) s_size[tid] = __ldcg(e.total + tid);
  __syncthreads();
  if (tid < O) {
    int pos = tid;
    if (e.reorder) {
      // stable ascending sizes: ties keep the offset order
      const int mine = s_size[tid];
      pos = 0;
      for (int j = 0; j < O; j++) {
        const int other = s_size[j];
        pos += (other < mine) || (other == mine && j < tid);
      }
    }
    s_pos[tid] = pos;
    s_ord[pos] = tid;
    if (b == 0) {
      e.order_out[pos] = tid;
      e.sizes_out[pos] = s_size[tid];
    }
  }
  if (b == 0 && tid == 0) e.sizes_out[O] = e.ctrl[MN_CTRL_STATUS];
  __syncthreads();

  MN_MARK(g_marks_emit, 5);
  // ---- phase 2: ranks, staged per tile, one bulk copy per mask row segment ------
  bool pending = false;   // threads < O: a bulk group of mine may still be reading the stage
  for (int tile = t_begin; tile < t_end; tile++) {
    // the words of the first kEBatch tiles are still in shared memory from phase 1
    if (tile != t_begin && (tile - t_begin) % kEBatch == 0) fetch_words(tile);
    if (tile == t_begin && t_end - t_begin > kEBatch) fetch_words(tile);
    const int dir = tile >= e.tiles_t ? 1 : 0;
    const int64_t tile_row0 = (int64_t)(tile - dir * e.tiles_t) * kETile;
    const int64_t n = dir ? e.S : e.T;
    int32_t *out = dir ? e.source_masks : e.target_masks;
    const int rows_here = (int)min((int64_t)kETile, n - tile_row0);
    const int seg = warp * 32;

    uint32_t plane = transpose32(s_words[(tile - t_begin) % kEBatch][tid], lane);
    if (dir) plane = __shfl_sync(0xffffffffu, plane, my_mirror);
    if (lane >= O) plane = 0u;
    {
      // hit word of every row in mask-row order (bit p <-> mask row p), for the
      // convolution kernels that walk a row's pairs without scanning the masks
      uint32_t *bits_out = dir ? e.bits_s : e.bits_t;
      if (bits_out != nullptr) {
        uint32_t by_row = __shfl_sync(0xffffffffu, plane, lane < O ? s_ord[lane] : 0);
        if (lane >= O) by_row = 0u;
        by_row = transpose32(by_row, lane);
        if (tile_row0 + seg + lane < n) bits_out[tile_row0 + seg + lane] = by_row;
      }
    }
    if (lane < O) s_wcnt[lane][warp] = __popc(plane);
    // the previous tile's copies must have read the stage before it is refilled
    if (pending) {
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      pending = false;
    }
    __syncthreads();
    if (tid < O) {
      // exclusive prefix over the warps on top of the running rank; where the
      // row segment of this offset starts relative to a 16-byte boundary
      int run = s_run[dir][tid];
#pragma unroll
      for (int w = 0; w < kEWarps; w++) {
        const int c = s_wcnt[tid][w];
        s_wcnt[tid][w] = run;
        run += c;
      }
      s_run[dir][tid] = run;
      const int64_t g0 = (int64_t)s_pos[tid] * n + tile_row0;
      s_mis[tid] = (int)(((reinterpret_cast<uintptr_t>(out) >> 2) + (uint64_t)g0) & 3u);
    }
    {
      int4 *fill = reinterpret_cast<int4 *>(s_stage);
      const int n_vec = O * kEPitch / 4;
      for (int i = tid; i < n_vec; i += kEThreads) fill[i] = make_int4(-1, -1, -1, -1);
    }
    __syncthreads();
    // sparse planes: the owning lane walks its hits; dense planes: all lanes, one row each
    {
      int base = 0;
      int32_t *row = s_stage;
      if (lane < O) {
        base = s_wcnt[lane][warp];
        row = s_stage + lane * kEPitch + s_mis[lane] + seg;
      }
      const bool dense = __popc(plane) > 6;
      uint32_t p = dense ? 0u : plane;
      int r = base;
      while (p != 0u) {
        row[__ffs(p) - 1] = r++;
        p &= p - 1u;
      }
      uint32_t todo = __ballot_sync(0xffffffffu, dense);
      while (todo != 0u) {
        const int o = __ffs(todo) - 1;
        todo &= todo - 1u;
        const uint32_t pl = __shfl_sync(0xffffffffu, plane, o);
        const int bs = __shfl_sync(0xffffffffu, base, o);
        if ((pl >> lane) & 1u) s_stage[o * kEPitch + s_mis[o] + seg + lane] = bs + __popc(pl & lt);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid < O) {
      const int mis = s_mis[tid];
      const int32_t *src = s_stage + tid * kEPitch + mis;
      int32_t *dst = out + (int64_t)s_pos[tid] * n + tile_row0;
      const int head = min((4 - mis) & 3, rows_here);
      const int body = (rows_here - head) & ~3;
      if (body > 0) {
        bulk_store(dst + head, src + head, (uint32_t)body * 4u);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        pending = true;
      }
      for (int i = 0; i < head; i++) dst[i] = src[i];
      for (int i = head + body; i < rows_here; i++) dst[i] = src[i];
    }
  }
  MN_MARK(g_marks_emit, 6);
  if (pending) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  MN_MARK(g_marks_emit, 7);
}

__global__ void identity_order_kernel(int O, int32_t *order_out, int32_t *sizes_out,
                                      const int32_t *ctrl) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o < O) { order_out[o] = o; sizes_out[o] = 0; }
  if (o == O) sizes_out[O] = ctrl[MN_CTRL_STATUS];
}

// ---------------------------------------------------------------------------
// reference-API pieces that start from a materialised kernel map
// ---------------------------------------------------------------------------
constexpr int kMTile = 1024;     // rows per tile of the kernels below
constexpr int kMThreads = 256;

// counts[o, tile] = valid entries of kernel_map[o, tile * kMTile ...)
__global__ void __launch_bounds__(kMThreads)
map_count_kernel(const int32_t *__restrict__ kernel_map, int64_t T, int n_tiles,
                 int32_t *__restrict__ counts, int32_t *__restrict__ sizes_atomic) {
  const int o = blockIdx.y, tile = blockIdx.x;
  const int64_t t0 = (int64_t)tile * kMTile;
  int c = 0;
#pragma unroll
  for (int j = 0; j < kMTile / kMThreads; j++) {
    const int64_t t = t0 + j * kMThreads + threadIdx.x;
    if (t < T) c += __ldg(kernel_map + (int64_t)o * T + t) != -1;
  }
  c = __reduce_add_sync(0xffffffffu, c);
  __shared__ int s[kMThreads / 32];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int w = 0; w < kMThreads / 32; w++) tot += s[w];
    if (counts != nullptr) counts[(int64_t)o * n_tiles + tile] = tot;
    if (sizes_atomic != nullptr && tot != 0) atomicAdd(sizes_atomic + o, tot);
  }
}

// Block o turns row o of counts ([O, tiles]) into its exclusive prefix, in place.
__global__ void __launch_bounds__(1024)
scan_tiles_kernel(int32_t *__restrict__ counts, int n) {
  __shared__ int32_t s_warp[32];
  __shared__ int32_t s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t *row = counts + (int64_t)blockIdx.x * n;
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
}

// rank valid entries of row o by t; write the target mask densely and the
// source mask (pre-filled with -1) by scatter
__global__ void __launch_bounds__(kMThreads)
map_masks_kernel(const int32_t *__restrict__ kernel_map, int64_t S, int64_t T, int n_tiles,
                 const int32_t *__restrict__ prefix, int32_t *__restrict__ source_masks,
                 int32_t *__restrict__ target_masks) {
  const int o = blockIdx.y, tile = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t0 = (int64_t)tile * kMTile + threadIdx.x * 4;
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
  __shared__ int s_w[kMThreads / 32];
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
                      int64_t n_table, int32_t *kernel_map, uint32_t *hit_words) {
  *a = SearchArgs{};
  a->rows = rows; a->table = table; a->n_rows = n_rows; a->n_table = n_table;
  a->kernel_map = kernel_map; a->hit_words = hit_words;
  a->n_tiles = (int)div_up(n_rows, kQTile);
}

// Launches one search, or two in the same grid when `second` is given.
mn_status run_search(int mode, const mn_keyspec &spec, const SearchArgs &first,
                     const OffsetTable &tab_first, const SearchArgs *second,
                     const OffsetTable *tab_second, cudaStream_t st) {
  thread_local static SearchPair sp;   // ~5 KB: kept off the stack; passed by value per launch
  sp.a[0] = first;
  sp.tab[0] = tab_first;
  sp.spec = make_spec_ref(spec);
  sp.tiles0 = first.n_tiles;
  int blocks = first.n_tiles;
  if (second != nullptr) {
    sp.a[1] = *second;
    sp.tab[1] = *tab_second;
    blocks += second->n_tiles;
  }
  if (blocks == 0) return MN_OK;
  {
    LaunchScope scope(mode == kMap ? "search_kernel<map>" : mode == kBits ? "search_kernel<bits>"
                                                                         : "search_kernel<bits,rev>", st);
    if (mode == kMap) search_kernel<kMap><<<blocks, kQThreads, 0, st>>>(sp);
    else if (mode == kBits) search_kernel<kBits><<<blocks, kQThreads, 0, st>>>(sp);
    else search_kernel<kBitsRev><<<blocks, kQThreads, 0, st>>>(sp);
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
  // a group: same offset in every dimension but the last, last-dimension span <= kQMaxSpan
  int g = 0, first = 0;
  for (int64_t i = 0; i < O; i++) {
    out->member[i] = (uint8_t)idx[i];
    bool new_group = i == 0;
    if (i > 0) {
      for (int k = 0; k + 1 < ndim; k++)
        new_group |= out->off[idx[i]][k] != out->off[idx[i - 1]][k];
      new_group |= out->off[idx[i]][ndim - 1] - out->off[first][ndim - 1] > kQMaxSpan;
    }
    if (new_group) {
      out->group_begin[g++] = (uint8_t)i;
      first = idx[i];
    }
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
  const int64_t tiles = div_up(S, kMTile) + div_up(T, kMTile) + 2;
  size_t map = align_up((size_t)S * 4, 256) + align_up((size_t)T * 4, 256) +
               2 * align_up((size_t)std::max<int64_t>(O, 1) * tiles * 4, 256) +
               align_up((size_t)kMaxCoopBlocks * 64 * 4, 256) + 4 * 1024;
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (S == 0) {
    MN_CHECK_CUDA(cudaMemsetAsync(kernel_map_out, 0xff, sizeof(int32_t) * O * T, st));
    return MN_OK;
  }
  SearchArgs a;
  fill_search_args(&a, target_keys, T, source_keys, S, kernel_map_out, nullptr);
  return run_search(kMap, *spec, a, tab, nullptr, nullptr, st);
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
  const int n_tiles = (int)div_up(T, kMTile);
  MN_LAUNCH("map_count_kernel", st,
            map_count_kernel<<<dim3(n_tiles, (unsigned)O), kMThreads, 0, st>>>(
                kernel_map, T, n_tiles, nullptr, sizes_out));
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
  const int n_tiles = (int)div_up(T, kMTile);
  int32_t *counts = ws.take<int32_t>((size_t)O * n_tiles);
  MN_CHECK_WS(ws);
  MN_LAUNCH("map_count_kernel", st,
            map_count_kernel<<<dim3(n_tiles, (unsigned)O), kMThreads, 0, st>>>(
                kernel_map, T, n_tiles, counts, nullptr));
  MN_LAUNCH("scan_tiles_kernel", st, scan_tiles_kernel<<<(unsigned)O, 1024, 0, st>>>(counts, n_tiles));
  MN_LAUNCH("map_masks_kernel", st,
            map_masks_kernel<<<dim3(n_tiles, (unsigned)O), kMThreads, 0, st>>>(
                kernel_map, S, T, n_tiles, counts, source_masks_out, target_masks_out));
  return MN_OK;
}

extern "C" mn_status mn_build_kernel_map(const uint64_t *source_keys, int64_t S,
                                         const uint64_t *target_keys, int64_t T,
                                         const int32_t *offsets, int64_t O,
                                         const mn_keyspec *spec, int reorder,
                                         int32_t *source_masks_out, int32_t *target_masks_out,
                                         int32_t *order_out, int32_t *sizes_out,
                                         uint32_t *source_bits_out, uint32_t *target_bits_out,
                                         int32_t *ctrl, void *ws_ptr, size_t ws_bytes,
                                         void *stream) {
  MN_CHECK_ARG(S >= 0 && T >= 0, "build_kernel_map: negative size");
  MN_CHECK_ARG(spec != nullptr, "build_kernel_map: null key spec");
  MN_CHECK_ARG(S < (1ll << 31) && T < (1ll << 31), "build_kernel_map: more than 2^31-1 rows");
  if (O > 32) {
    set_error("build_kernel_map: the fused build handles up to 32 offsets (got %lld); use "
              "mn_query_sorted_index_with_offsets + mn_compute_kernel_map_masks", (long long)O);
    return MN_ERR_UNSUPPORTED;
  }
  MN_CHECK_ARG(order_out != nullptr && sizes_out != nullptr && ctrl != nullptr,
               "build_kernel_map: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ndim = spec->ndim;
  OffsetTable fwd;
  MN_RETURN_IF(make_offset_table(offsets, O, ndim, +1, spec, &fwd));

  if (T == 0 || S == 0) {
    // nothing can match: every mask entry is -1, every size 0
    if (S > 0) MN_CHECK_CUDA(cudaMemsetAsync(source_masks_out, 0xff, sizeof(int32_t) * O * S, st));
    if (T > 0) MN_CHECK_CUDA(cudaMemsetAsync(target_masks_out, 0xff, sizeof(int32_t) * O * T, st));
    if (S > 0 && source_bits_out != nullptr) MN_CHECK_CUDA(cudaMemsetAsync(source_bits_out, 0, sizeof(uint32_t) * S, st));
    if (T > 0 && target_bits_out != nullptr) MN_CHECK_CUDA(cudaMemsetAsync(target_bits_out, 0, sizeof(uint32_t) * T, st));
    MN_LAUNCH("identity_order_kernel", st,
              identity_order_kernel<<<1, MN_MAX_OFFSETS + 32, 0, st>>>((int)O, order_out, sizes_out, ctrl));
    return MN_OK;
  }
  MN_CHECK_ARG(source_keys != nullptr && target_keys != nullptr && source_masks_out != nullptr &&
                   target_masks_out != nullptr, "build_kernel_map: null pointer");

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

  // grid of the cooperative emission kernel: every block resident at once
  const size_t stage_bytes = (size_t)O * kEPitch * sizeof(int32_t);
  static thread_local int coresident_for[kMaxDevices][33] = {{0}};
  int device = 0;
  MN_CHECK_CUDA(cudaGetDevice(&device));
  MN_CHECK_ARG(device >= 0 && device < kMaxDevices, "build_kernel_map: device index %d out of range", device);
  int &coresident = coresident_for[device][O];
  if (coresident == 0) {
    MN_CHECK_CUDA(cudaFuncSetAttribute(emit_masks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       32 * kEPitch * (int)sizeof(int32_t)));
    coresident = std::min(kMaxCoopBlocks, max_coresident_blocks(emit_masks_kernel, kEThreads, stage_bytes));
    if (coresident <= 0) {
      coresident = 0;
      set_error("build_kernel_map: cannot size the cooperative grid");
      return MN_ERR_CUDA;
    }
  }
  const int tiles_t = (int)div_up(T, kETile), tiles_s = (int)div_up(S, kETile);
  const int grid = std::min(tiles_t + tiles_s, coresident);

  Workspace ws(ws_ptr, ws_bytes);
  uint32_t *words_t = ws.take<uint32_t>(T);
  uint32_t *words_s = mirrored ? words_t : ws.take<uint32_t>(S);
  int32_t *agg = ws.take<int32_t>((size_t)grid * 64);
  int32_t *total = ws.take<int32_t>(64);
  MN_CHECK_WS(ws);

  SearchArgs fwd_args;
  fill_search_args(&fwd_args, target_keys, T, source_keys, S, nullptr, words_t);
  if (mirrored) {
    MN_RETURN_IF(run_search(kBits, *spec, fwd_args, fwd, nullptr, nullptr, st));
  } else {
    // one search with the targets as rows; every hit also sets its bit in the word of the
    // source it found, so the source side needs no search of its own
    MN_CHECK_CUDA(cudaMemsetAsync(words_s, 0, sizeof(uint32_t) * S, st));
    fwd_args.table_words = words_s;
    MN_RETURN_IF(run_search(kBitsRev, *spec, fwd_args, fwd, nullptr, nullptr, st));
  }

  EmitArgs e{};
  e.words_t = words_t; e.words_s = words_s;
  e.target_masks = target_masks_out; e.source_masks = source_masks_out;
  e.order_out = order_out; e.sizes_out = sizes_out; e.agg = agg; e.total = total; e.ctrl = ctrl;
  e.bits_t = target_bits_out; e.bits_s = source_bits_out;
  e.T = T; e.S = S; e.tiles_t = tiles_t; e.tiles_s = tiles_s;
  e.num_offsets = (int)O; e.reorder = reorder ? 1 : 0;
  for (int64_t o = 0; o < O; o++) e.mirror[o] = mirrored ? neg[o] : (uint8_t)o;
  void *params[] = {&e};
  {
    LaunchScope scope("emit_masks_kernel", st);
    MN_CHECK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(emit_masks_kernel), dim3(grid),
                                              dim3(kEThreads), params, stage_bytes, st));
  }
  MN_CHECK_LAUNCH();
  return MN_OK;
}

#ifdef MN_PHASE_TIMING
// Debug build only: copies the phase marks of the last search (which = 0) or mask
// emission (which = 1) launch to the host (blocking).
extern "C" int mn_debug_marks_query(int which, long long *out, int count) {
  const size_t bytes = sizeof(long long) * (size_t)std::min(count, 2048 * 16);
  cudaError_t e = which == 0 ? cudaMemcpyFromSymbol(out, g_marks_search, bytes)
                             : cudaMemcpyFromSymbol(out, g_marks_emit, bytes);
  return e == cudaSuccess ? 0 : 1;
}
#endif
