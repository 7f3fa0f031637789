// Fused (implicit-GEMM) forward pass of a sparse convolution, fp16/bf16.
//
// The reference gathers every (source, target) pair row into a padded buffer,
// multiplies bucket by bucket with cuBLAS and scatters the products back
// (csrc/minuet/cuda/functions/sparse_convolution.cu:505-661); every pair row
// crosses HBM four times.  Here one persistent kernel owns 128 consecutive TARGET
// rows at a time and accumulates ALL kernel offsets of that tile in one TMEM
// accumulator:
//   warps 0..7  producers: warp w fetches, for every active offset and k-block, the
//               128-byte slices of the source rows that feed target rows 16w..16w+15
//               (cp.async straight into the 128-byte-swizzled A tile, eight lanes per
//               row, zeros where the kernel map has no entry); thread 0 also starts
//               the TMA load of the offset's transposed weight tile
//   warp 8      allocates TMEM and issues tcgen05.mma over (offset, k-block)
//   warps 9..12 epilogue: TMEM -> registers -> optional per-channel scale/shift
//               (folded BatchNorm or bias), residual add, ReLU -> swizzled shared
//               tile -> TMA store of the output rows
// so that features are read once per pair (mostly from L2), outputs are written
// once, and no pair-row buffer exists.  Offsets with no pair inside a tile are
// skipped through a per-tile bit mask.  The neighbour table [O, T] (source row
// of target t under mask row p, or -1) is derived once per kernel map from the
// masks by mn_build_neighbor_table.  Every barrier wait is bounded (status bit 2).
#include "mn_tc.cuh"

#include <algorithm>

namespace mn {

namespace {

using namespace tc;

constexpr int kProdWarps = 8;          // producer warps: warp w owns 128 / kProdWarps rows of a sub-tile
constexpr int kProdRows = 128 / kProdWarps;
constexpr int kMmaWarp = kProdWarps;   // then the MMA issuer, then four epilogue warps
constexpr int kImThreads = (kProdWarps + 5) * 32;
constexpr int kImCtas = kProdWarps > 4 ? 2 : 3;   // CTAs per SM the register file allows
constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kMaxStages = 10;
constexpr int kMaxSub = 4;             // 128-row sub-tiles per CTA tile

struct ImArgs {
  const uint8_t *in;          // [S, K] 16-bit
  const int32_t *nbr;         // [O, T]
  const uint32_t *tile_bits;  // [tiles]
  const int32_t *order;       // [O] or NULL
  const float *scale;         // [N] or NULL
  const float *shift;         // [N] or NULL
  const uint8_t *residual;    // [T, N] 16-bit or NULL
  int32_t *status;
  int64_t T;
  int32_t K, N, n_pad, k_blocks, stages, a_bytes, stage_bytes, elem_is_bf16, num_tiles, relu;
  int32_t sub;         // 128-row sub-tiles per CTA tile (1..4): they share every weight tile
  int32_t acc_bufs;    // accumulator sets in TMEM (2 when 2 * sub * n_pad <= 512, else 1)
  int32_t n_tiles128;  // entries of tile_bits
  int32_t num_offsets; // O
  int32_t tmem_cols;   // TMEM columns this CTA allocates
  // pair mode (step 1 of the pair-list forward): the rows are PRODUCT rows, row r reads
  // source row nbr[r], every tile has exactly one "offset" whose weight matrix follows from
  // the mask row that owns the tile, and the fp32 accumulators are stored as they are
  int32_t pair_mode;
  int32_t pair_rows;                            // mask rows in pair_tile_prefix
  int32_t pair_tile_prefix[MN_MAX_PAIR_ROWS + 1];
  float *out_f32;                               // [T, N]
  const int32_t *perm;   // [T] or NULL: tile row r is target row perm[r] (nbr is in tile-row order)
  uint8_t *out16;        // [T, N] 16-bit output, addressed row by row when perm is given
};

// mask row that owns 128-row tile `tile` of the product buffer
__device__ __forceinline__ int pair_row_of_tile(const ImArgs &a, int tile) {
  int lo = 0, hi = a.pair_rows;   // last p with prefix[p] <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (a.pair_tile_prefix[mid] <= tile) lo = mid; else hi = mid;
  }
  return lo;
}

// 16-byte asynchronous copy; src_bytes = 0 writes 16 zero bytes instead (the fill
// travels the same path as the copies, so no proxy fence is needed for it)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}

template <bool kBf16>
__device__ __forceinline__ float elem_to_f32(uint16_t v) {
  if (kBf16) return __uint_as_float((uint32_t)v << 16);
  return __half2float(__ushort_as_half(v));
}

__global__ void __launch_bounds__(kImThreads, kImCtas)
conv_implicit_kernel(const __grid_constant__ ImArgs args,
                     const __grid_constant__ CUtensorMap map_b,     // weights^T [O, N, K]
                     const __grid_constant__ CUtensorMap map_out) { // output    [T, N]
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kMaxStages], bar_empty[kMaxStages];
  __shared__ uint64_t bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  uint8_t *stage_base = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = args.stages;
  const uint32_t tmem_cols = (uint32_t)args.tmem_cols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) {
      mbar_init(&bar_full[s], kProdWarps * 32 + 1);   // every producer lane + the weight tile's expect_tx
      mbar_init(&bar_empty[s], 1);
    }
    for (int a = 0; a < 2; a++) { mbar_init(&bar_acc_full[a], 1); mbar_init(&bar_acc_empty[a], 4); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&s_tmem_base)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem_base;
  volatile int *abort_flag = &s_abort;

  if (warp < kProdWarps) {
    // ------------------------------ producers ---------------------------------
    // Eight warps feed the ring; warp w owns rows 16w .. 16w+15 of every 128-row sub-tile
    // and lane l holds the source row of row 16w + (l & 15) (one coalesced load from the
    // neighbour table per offset, the next offset's requested before the current one is
    // copied).  Per stage eight lanes copy one row: a warp-wide cp.async reads four whole
    // 128-byte lines (16 bytes of 32 different lines would cost a tag lookup per lane),
    // zero fill where the kernel map has no source.  Each lane's arrival on the stage
    // barrier fires when its copies have landed.  All sub-tiles of a CTA tile share every
    // weight tile.  A stage is a serial chain per CTA (about 120 cycles per cp.async a
    // thread issues): four producer warps with eight copies each were 5-18 % slower, a
    // single producer warp 2.5x slower.
    const int sub = args.sub;
    const uint32_t b_bytes = (uint32_t)(args.stage_bytes - args.a_bytes);
    const int chunk = lane & 7;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; alive && tile < args.num_tiles; tile += gridDim.x) {
      uint32_t rest = 0u, hb[kMaxSub];   // offsets of the CTA tile and of each sub-tile
#pragma unroll
      for (int h = 0; h < kMaxSub; h++) {
        hb[h] = 0u;
        if (h < sub && tile * sub + h < args.n_tiles128)
          hb[h] = args.pair_mode ? 1u : __ldg(args.tile_bits + tile * sub + h);
        rest |= hb[h];
      }
      const int pair_row = args.pair_mode ? pair_row_of_tile(args, tile) : 0;
      int p = rest != 0u ? __ffs(rest) - 1 : -1;
      int src[kMaxSub], src_next[kMaxSub];
      auto fetch = [&](int pp, int (&dst)[kMaxSub]) {
#pragma unroll
        for (int h = 0; h < kMaxSub; h++) {
          const int64_t t = ((int64_t)tile * sub + h) * kBM + warp * kProdRows + (lane & (kProdRows - 1));
          // a sub-tile without offset pp has no table block: its rows are zero rows
          dst[h] = (pp >= 0 && ((hb[h] >> pp) & 1u) && t < args.T) ? __ldg(args.nbr + (int64_t)pp * args.T + t) : -1;
        }
      };
      fetch(p, src);
      while (alive && p >= 0) {
        rest &= rest - 1u;
        const int p_next = rest != 0u ? __ffs(rest) - 1 : -1;
        fetch(p_next, src_next);
        for (int kb = 0; kb < args.k_blocks; kb++) {
          int ok = 1;   // one lane polls the barrier, the warp follows
          if (lane == 0) ok = mbar_wait(&bar_empty[stage], phase ^ 1u, abort_flag, args.status) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { alive = false; break; }
          uint8_t *sa = stage_base + (size_t)stage * args.stage_bytes;
          if (threadIdx.x == 0) {
            const int wrow = args.pair_mode ? pair_row : p;
            const int widx = args.order != nullptr ? __ldg(args.order + wrow) : wrow;
            mbar_expect_tx(&bar_full[stage], b_bytes);
            tma_load_3d(sa + args.a_bytes, &map_b, kb * kBK, 0, widx, &bar_full[stage]);
          }
          const int kcol = kb * kBK + chunk * 8;
#pragma unroll
          for (int h = 0; h < kMaxSub; h++) {
            if (h < sub) {
#pragma unroll
              for (int i = 0; i < kProdRows / 4; i++) {
                const int owner = 4 * i + (lane >> 3);           // lane that holds this row's index
                const int s_idx = __shfl_sync(0xffffffffu, src[h], owner);
                const int rr = warp * kProdRows + owner;           // row inside the sub-tile
                const uint32_t dst = smem_u32(sa) + (uint32_t)(h * kBM + rr) * 128u +
                                     (uint32_t)((chunk ^ (rr & 7)) << 4);
                const bool valid = s_idx >= 0 && kcol < args.K;
                cp_async_16(dst, valid ? args.in + ((int64_t)s_idx * args.K + kcol) * 2 : args.in,
                            valid ? 16u : 0u);
              }
            }
          }
          // this lane's arrival fires when its copies above have landed: no stall here
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(
                           smem_u32(&bar_full[stage]))
                       : "memory");
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        p = p_next;
#pragma unroll
        for (int h = 0; h < kMaxSub; h++) src[h] = src_next[h];
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this lane is in flight at exit
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t fmt = args.elem_is_bf16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) |
                             ((uint32_t)(args.n_pad >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < args.num_tiles; tile += gridDim.x) {
        if (!mbar_wait(&bar_acc_empty[acc], acc_phase ^ 1u, abort_flag, args.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * args.sub * args.n_pad);
        uint32_t tb = 0u;
        for (int h = 0; h < args.sub; h++)
          if (tile * args.sub + h < args.n_tiles128)
            tb |= args.pair_mode ? 1u : __ldg(args.tile_bits + tile * args.sub + h);
        const int n_stage = __popc(tb) * args.k_blocks;
        uint32_t accumulate = 0u;
        for (int it = 0; it < n_stage; it++) {
          const int kb = it % args.k_blocks;
          if (!mbar_wait(&bar_full[stage], phase, abort_flag, args.status)) { alive = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(stage_base + (size_t)stage * args.stage_bytes);
          const uint32_t sb = sa + (uint32_t)args.a_bytes;
          const int nk = min(kBK / kUmmaK, (args.K - kb * kBK + kUmmaK - 1) / kUmmaK);
          for (int k = 0; k < nk; k++) {
            const uint64_t db = umma_desc(sb + k * kUmmaK * 2);   // one weight tile, all sub-tiles
            for (int h = 0; h < args.sub; h++)
              umma_f16(tmem_d + (uint32_t)(h * args.n_pad),
                       umma_desc(sa + h * (kBM * kBK * 2) + k * kUmmaK * 2), db, idesc, accumulate);
            accumulate = 1u;
          }
          umma_commit(&bar_empty[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit(&bar_acc_full[acc]);
        if (++acc == args.acc_bufs) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;
    uint8_t *cbuf = stage_base + (size_t)stages * args.stage_bytes + (size_t)(warp - kMmaWarp - 1) * 8192;
    int acc = 0, chunk = 0;   // chunk: 64-column chunks so far (parity = staging buffer)
    uint32_t acc_phase = 0;
    const int n = args.N;
    const int cps = (args.n_pad + 63) / 64;   // 64-column chunks per sub-tile
    // The residual rows of a chunk are copied into the chunk's staging buffer (eight lanes
    // per row, whole 128-byte lines, asynchronously and one chunk ahead); the lanes then add
    // them from shared memory and overwrite them with the output.  Per-lane loads of 16
    // bytes from 32 different rows cost the residual layers 15-35 % of their time.
    const bool staged_res = args.residual != nullptr && args.out_f32 == nullptr;
    auto stage_residual = [&](uint8_t *dst, int out_row, int64_t grow, int c0) {
      const int piece = lane & 7;
      const int col = c0 + piece * 8;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int rl = 4 * i + (lane >> 3);
        const int64_t drow = __shfl_sync(0xffffffffu, grow, rl);
        const bool valid = (int64_t)out_row + rl < args.T && col < n;
        cp_async_16(smem_u32(dst + rl * 128 + ((piece ^ (rl & 7)) << 4)),
                    valid ? args.residual + (drow * n + col) * 2 : args.residual, valid ? 16u : 0u);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int tile = blockIdx.x; tile < args.num_tiles; tile += gridDim.x) {
      // row of the output (and of the residual) this lane's accumulator row belongs to, per
      // sub-tile; nsub = sub-tiles of this CTA tile that have rows for this warp
      int64_t grow[kMaxSub];
      int nsub = 0;
#pragma unroll
      for (int h = 0; h < kMaxSub; h++) {
        const int64_t row = (int64_t)(tile * args.sub + h) * kBM + quarter * 32 + lane;
        grow[h] = row;
        if (h < args.sub && row - lane < args.T) {
          nsub = h + 1;
          if (args.perm != nullptr && row < args.T) grow[h] = (int64_t)__ldg(args.perm + row);
        }
      }
      auto grow_of = [&](int h) {
        int64_t g = grow[0];
#pragma unroll
        for (int k = 1; k < kMaxSub; k++) g = h == k ? grow[k] : g;
        return g;
      };
      const int total = nsub * cps;
      if (staged_res && total > 0) {
        // the first chunk's residual rows travel while the MMAs run
        if (args.perm == nullptr && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        stage_residual(cbuf + (chunk & 1) * 4096, tile * args.sub * kBM + quarter * 32, grow[0], 0);
      }
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&bar_acc_full[acc], acc_phase, abort_flag, args.status) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t tb = 0u;
      for (int h = 0; h < args.sub; h++)
        if (tile * args.sub + h < args.n_tiles128)
          tb |= args.pair_mode ? 1u : __ldg(args.tile_bits + tile * args.sub + h);
      const bool empty_tile = tb == 0u;   // no pair in the whole tile: no MMA ran, the rows are zero
      for (int q = 0; q < total; q++, chunk++) {
        const int h = q / cps;
        const int c0 = (q - h * cps) * 64;
        const int out_row = (tile * args.sub + h) * kBM + quarter * 32;
        const int64_t row = (int64_t)out_row + lane;
        const int64_t grow_h = grow_of(h);
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                               (uint32_t)((acc * args.sub + h) * args.n_pad);
        uint8_t *buf = cbuf + (chunk & 1) * 4096;
        if (args.out_f32 == nullptr) {
          // this chunk's buffer (and, with a staged residual, the next chunk's) must have
          // been read by the bulk stores that used them
          if (args.perm == nullptr && lane == 0) {
            if (staged_res) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          }
          __syncwarp();
        }
        if (staged_res) {
          if (q + 1 < total) {
            const int h2 = (q + 1) / cps;
            stage_residual(cbuf + ((chunk + 1) & 1) * 4096, (tile * args.sub + h2) * kBM + quarter * 32,
                           grow_of(h2), (q + 1 - h2 * cps) * 64);
            asm volatile("cp.async.wait_group 1;" ::: "memory");   // this chunk's rows have landed
          } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
          }
          __syncwarp();
        }
        // 32 columns at a time: the two halves fill one 64-column staging tile
        for (int half = 0; half < 2; half++) {
          const int cb = c0 + 32 * half;
          if (cb >= args.n_pad) break;
          uint32_t rr[32];
          tmem_ld_32x32(taddr + (uint32_t)cb, rr);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (args.out_f32 != nullptr) {
            // pair mode: the fp32 accumulators of this row go out as they are
            if (row < args.T) {
              float4 *dst = reinterpret_cast<float4 *>(args.out_f32 + row * n + cb);
#pragma unroll
              for (int v = 0; v < 8; v++)
                if (cb + 4 * v < n)
                  dst[v] = make_float4(__uint_as_float(rr[4 * v]), __uint_as_float(rr[4 * v + 1]),
                                       __uint_as_float(rr[4 * v + 2]), __uint_as_float(rr[4 * v + 3]));
            }
            continue;
          }
#pragma unroll
          for (int v = 0; v < 4; v++) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = empty_tile ? 0.f : __uint_as_float(rr[v * 8 + i]);
            const int c = cb + v * 8;
            const int piece = half * 4 + v;
            uint4 *slot = reinterpret_cast<uint4 *>(buf + lane * 128 + ((piece ^ (lane & 7)) << 4));
            if (c < n) {
              if (args.scale != nullptr) {   // n is a multiple of 8 here
                const float4 s0 = __ldg(reinterpret_cast<const float4 *>(args.scale + c));
                const float4 s1 = __ldg(reinterpret_cast<const float4 *>(args.scale + c) + 1);
                f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w;
                f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
              }
              if (args.shift != nullptr) {
                const float4 s0 = __ldg(reinterpret_cast<const float4 *>(args.shift + c));
                const float4 s1 = __ldg(reinterpret_cast<const float4 *>(args.shift + c) + 1);
                f[0] += s0.x; f[1] += s0.y; f[2] += s0.z; f[3] += s0.w;
                f[4] += s1.x; f[5] += s1.y; f[6] += s1.z; f[7] += s1.w;
              }
              if (staged_res) {
                const uint4 rv = *slot;      // this row's residual piece (zeros past the last row)
                const uint16_t *r16 = reinterpret_cast<const uint16_t *>(&rv);
#pragma unroll
                for (int i = 0; i < 8; i++)
                  f[i] += args.elem_is_bf16 ? elem_to_f32<true>(r16[i]) : elem_to_f32<false>(r16[i]);
              }
              if (args.relu) {
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = fmaxf(f[i], 0.f);
              }
            }
            uint4 out;
            uint32_t *o32 = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
            for (int k = 0; k < 4; k++) {
              if (args.elem_is_bf16) {
                __nv_bfloat162 pk = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
                o32[k] = *reinterpret_cast<uint32_t *>(&pk);
              } else {
                __half2 pk = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
                o32[k] = *reinterpret_cast<uint32_t *>(&pk);
              }
            }
            *slot = out;
          }
        }
        if (args.out_f32 != nullptr) continue;
        if (args.perm != nullptr) {
          // permuted rows: eight lanes store one row's 128 bytes of this chunk, four rows
          // per instruction, each row at its own place in the output
          __syncwarp();
          const int piece = lane & 7;
          const int col = c0 + piece * 8;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int rl = 4 * i + (lane >> 3);
            const int64_t drow = __shfl_sync(0xffffffffu, grow_h, rl);
            const uint4 v = *reinterpret_cast<const uint4 *>(buf + rl * 128 + ((piece ^ (rl & 7)) << 4));
            if ((int64_t)out_row + rl < args.T && col < n)
              *reinterpret_cast<uint4 *>(args.out16 + (drow * n + col) * 2) = v;
          }
          __syncwarp();
          continue;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&map_out, c0, out_row, buf);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_acc_empty[acc]);
      if (++acc == args.acc_bufs) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_abort) {
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(tmem_cols)
                 : "memory");
  }
}

// ---- neighbour table from masks --------------------------------------------------
struct CumSizes {
  int64_t cum[MN_MAX_OFFSETS + 1];
};

// src_of_rank[cum[p] + source_masks[p, s]] = s
__global__ void __launch_bounds__(256)
rank_to_source_kernel(const int32_t *__restrict__ source_masks, int64_t S, int O,
                      const __grid_constant__ CumSizes cs, int32_t *__restrict__ src_of_rank) {
  const int p = blockIdx.y;
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gsz) {
    const int m = __ldg(source_masks + (int64_t)p * S + s);
    if (m >= 0) src_of_rank[cs.cum[p] + m] = (int32_t)s;
  }
}

// the same from the sources' hit words: a source row reads only the mask entries of the
// offsets it takes part in (E entries instead of O * S)
__global__ void __launch_bounds__(256)
rank_to_source_bits_kernel(const int32_t *__restrict__ source_masks,
                           const uint32_t *__restrict__ source_bits, int64_t S,
                           const __grid_constant__ CumSizes cs, int32_t *__restrict__ src_of_rank) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gsz) {
    for (uint32_t rest = __ldg(source_bits + s); rest != 0u; rest &= rest - 1u) {
      const int p = __ffs(rest) - 1;
      const int m = __ldg(source_masks + (int64_t)p * S + s);
      if (m >= 0) src_of_rank[cs.cum[p] + m] = (int32_t)s;
    }
  }
}

// nbr[p, r] = source row feeding target perm[r] (perm == NULL: target r) under mask row p
// (or -1); bit p of tile_bits[r / 128] is set when any row of that 128-row tile has such a
// source.  With the targets' hit words (`bits`) only the (tile, p) blocks whose bit is set
// are written, and a row looks its source up only for the offsets of its own word: the rest
// of the table is never read by the forward pass, which checks tile_bits first.
__global__ void __launch_bounds__(128)
neighbor_table_kernel(const int32_t *__restrict__ target_masks, int64_t T, int O,
                      const __grid_constant__ CumSizes cs,
                      const int32_t *__restrict__ src_of_rank, const int32_t *__restrict__ perm,
                      const uint32_t *__restrict__ bits, int32_t *__restrict__ nbr,
                      uint32_t *__restrict__ tile_bits) {
  __shared__ uint32_t s_bits;
  if (threadIdx.x == 0) s_bits = 0u;
  __syncthreads();
  const int64_t r = (int64_t)blockIdx.x * 128 + threadIdx.x;
  const int64_t t = (r < T && perm != nullptr) ? (int64_t)__ldg(perm + r) : r;
  if (bits != nullptr) {
    const uint32_t mine = r < T ? __ldg(bits + t) : 0u;
    const uint32_t warp_or = __reduce_or_sync(0xffffffffu, mine);
    if ((threadIdx.x & 31) == 0 && warp_or != 0u) atomicOr(&s_bits, warp_or);
    __syncthreads();
    const uint32_t tile = s_bits;
    if (threadIdx.x == 0) tile_bits[blockIdx.x] = tile;
    if (r >= T) return;
    for (uint32_t rest = tile; rest != 0u; rest &= rest - 1u) {
      const int p = __ffs(rest) - 1;
      int v = -1;
      if ((mine >> p) & 1u)
        v = __ldg(src_of_rank + cs.cum[p] + __ldg(target_masks + (int64_t)p * T + t));
      nbr[(int64_t)p * T + r] = v;
    }
    return;
  }
  uint32_t mine = 0u;
  for (int p = 0; p < O; p++) {
    int v = -1;
    if (r < T) {
      const int m = __ldg(target_masks + (int64_t)p * T + t);
      if (m >= 0) v = __ldg(src_of_rank + cs.cum[p] + m);
      nbr[(int64_t)p * T + r] = v;
    }
    mine |= (v >= 0 ? 1u : 0u) << p;
  }
  mine = __reduce_or_sync(0xffffffffu, mine);
  if ((threadIdx.x & 31) == 0 && mine != 0u) atomicOr(&s_bits, mine);
  __syncthreads();
  if (threadIdx.x == 0) tile_bits[blockIdx.x] = s_bits;
}

// sort keys of the row permutation: the row's hit word with its bits reversed (rows with
// the same set of offsets become neighbours, so whole tiles can skip the offsets none of
// their rows has).  Mask rows are in ascending size order, so the reversal makes the RARE
// offsets the most significant key bits: the few rows that have a rare offset end up
// together instead of sprinkling it over many tiles (15 against 20 offsets per tile on a
// map with 9 pairs per row).
__global__ void hit_word_keys_kernel(const uint32_t *__restrict__ bits, int64_t n, int num_offsets,
                                     uint64_t *__restrict__ keys) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gsz) {
    // position of the reversed word in the reflected Gray sequence: neighbouring keys then
    // differ in one offset instead of many (2-5 % fewer offsets per tile than binary order)
    uint32_t r = __brev(__ldg(bits + i)) >> (32 - num_offsets);
    r ^= r >> 1; r ^= r >> 2; r ^= r >> 4; r ^= r >> 8; r ^= r >> 16;
    keys[i] = (uint64_t)r;
  }
}

}  // namespace

mn_status launch_pair_products(const PairPlan &plan, int64_t S, int64_t c_in, int64_t c_out, bool bf16,
                               const void *sources, const void *weights_t, int O,
                               const int32_t *pair_src, const int32_t *order, float *products,
                               int32_t *status_dev, cudaStream_t st) {
  (void)S;
  MN_CHECK_ARG(plan.total_rows > 0 && plan.total_rows % kBM == 0 && plan.total_rows < (1ll << 31),
               "pair products: bad product row count");
  MN_CHECK_ARG(((reinterpret_cast<uintptr_t>(sources) | reinterpret_cast<uintptr_t>(products) |
                 reinterpret_cast<uintptr_t>(weights_t)) & 15) == 0,
               "pair products: arrays must be 16-byte aligned");
  ImArgs a{};
  a.in = static_cast<const uint8_t *>(sources);
  a.nbr = pair_src;
  a.tile_bits = nullptr;
  a.order = order;
  a.status = status_dev;
  a.T = plan.total_rows;
  a.K = (int)c_in;
  a.N = (int)c_out;
  a.n_pad = (int)align_up((size_t)c_out, 16);
  a.k_blocks = (int)div_up(c_in, kBK);
  a.n_tiles128 = (int)(plan.total_rows / kBM);
  a.sub = 1;
  a.acc_bufs = 2;
  a.a_bytes = kBM * kBK * 2;
  a.stage_bytes = a.a_bytes + a.n_pad * kBK * 2;
  const TcSizing sizing = size_tc_kernel(a.stage_bytes, a.acc_bufs * a.sub * a.n_pad, kMaxStages, kImCtas);
  a.stages = sizing.stages;
  a.tmem_cols = sizing.tmem_cols;
  a.num_offsets = 1;
  a.elem_is_bf16 = bf16 ? 1 : 0;
  a.num_tiles = a.n_tiles128;
  a.pair_mode = 1;
  a.pair_rows = plan.num_rows;
  for (int p = 0; p <= MN_MAX_PAIR_ROWS; p++) a.pair_tile_prefix[p] = plan.tile_prefix[p];
  a.out_f32 = products;
  CUtensorMap map_b;
  MN_RETURN_IF(make_kmajor_map(&map_b, weights_t, bf16, c_in, c_out, O, a.n_pad));
  const size_t smem = sizing.smem_bytes;
  MN_CHECK_CUDA(cudaFuncSetAttribute(conv_implicit_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = std::min(a.num_tiles, kNumSMs * sizing.ctas_per_sm);
  // the output map is not used in pair mode; any valid map will do
  MN_LAUNCH("conv_implicit_kernel<pairs>", st,
            conv_implicit_kernel<<<grid, kImThreads, smem, st>>>(a, map_b, map_b));
  return MN_OK;
}

}  // namespace mn

using namespace mn;

extern "C" int mn_implicit_supported(int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype) {
  return (dtype == MN_F16 || dtype == MN_BF16) && O >= 1 && O <= 32 && c_in >= 8 && c_in % 8 == 0 &&
         c_out >= 8 && c_out % 8 == 0 && c_out <= 256;
}

extern "C" size_t mn_neighbor_table_workspace_bytes(const int32_t *sizes_host, int64_t O, int64_t T) {
  int64_t e = 0;
  for (int64_t p = 0; p < O; p++) e += sizes_host[p];
  const size_t n = (size_t)std::max<int64_t>(T, 1);
  const size_t sort = 2 * align_up(n * 8, 256) + 2 * align_up(n * 4, 256) + radix_sort_workspace_bytes(T);
  return align_up((size_t)std::max<int64_t>(e, 1) * sizeof(int32_t), 256) + sort + 1024;
}

extern "C" mn_status mn_build_neighbor_table(const int32_t *source_masks,
                                             const int32_t *target_masks,
                                             const int32_t *sizes_host, int64_t O, int64_t S,
                                             int64_t T, const uint32_t *source_bits,
                                             const uint32_t *target_bits,
                                             int32_t *nbr_out, uint32_t *tile_bits_out,
                                             int32_t *perm_out, int32_t *ctrl, void *ws_ptr,
                                             size_t ws_bytes, void *stream) {
  MN_CHECK_ARG(O >= 1 && O <= 32, "neighbor table: %lld offsets (supported: 1..32)", (long long)O);
  MN_CHECK_ARG(S >= 0 && T >= 0 && T < (1ll << 31) && sizes_host != nullptr,
               "neighbor table: bad arguments");
  if (T == 0) return MN_OK;
  MN_CHECK_ARG(source_masks != nullptr && target_masks != nullptr && nbr_out != nullptr &&
                   tile_bits_out != nullptr, "neighbor table: null pointer");
  MN_CHECK_ARG(perm_out == nullptr || (target_bits != nullptr && ctrl != nullptr),
               "neighbor table: a row permutation needs the targets' hit words and a control block");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CumSizes cs{};
  for (int64_t p = 0; p < O; p++) {
    MN_CHECK_ARG(sizes_host[p] >= 0 && sizes_host[p] <= std::min(S, T), "neighbor table: bad size");
    cs.cum[p + 1] = cs.cum[p] + sizes_host[p];
  }
  Workspace ws(ws_ptr, ws_bytes);
  int32_t *src_of_rank = ws.take<int32_t>((size_t)std::max<int64_t>(cs.cum[O], 1));
  MN_CHECK_WS(ws);
  if (perm_out != nullptr) {
    // stable sort of the rows by hit word: perm[r] = target row at position r
    uint64_t *keys = ws.take<uint64_t>(T), *keys_tmp = ws.take<uint64_t>(T);
    int32_t *vals = ws.take<int32_t>(T), *vals_tmp = ws.take<int32_t>(T);
    MN_CHECK_WS(ws);
    const int blocks = (int)std::min<int64_t>(kNumSMs * 8, div_up(T, 256));
    MN_LAUNCH("hit_word_keys_kernel", st,
              hit_word_keys_kernel<<<blocks, 256, 0, st>>>(target_bits, T, (int)O, keys));
    const mn_keyspec no_spec{};
    bool in_tmp = false;
    MN_RETURN_IF(launch_radix_sort(keys, keys_tmp, vals, vals_tmp, true, T, 0, (int)O, no_spec,
                                   nullptr, ctrl, nullptr, ws, &in_tmp, st));
    MN_CHECK_CUDA(cudaMemcpyAsync(perm_out, in_tmp ? vals_tmp : vals, (size_t)T * sizeof(int32_t),
                                  cudaMemcpyDeviceToDevice, st));
  }
  // a scattered 4-byte read costs a 32-byte sector: worth it while the pairs are fewer than
  // an eighth of the mask entries
  if (S > 0 && source_bits != nullptr && cs.cum[O] * 8 < O * S) {
    const int blocks = (int)std::min<int64_t>(kNumSMs * 16, div_up(S, 256));
    MN_LAUNCH("rank_to_source_bits_kernel", st,
              rank_to_source_bits_kernel<<<blocks, 256, 0, st>>>(source_masks, source_bits, S, cs,
                                                                  src_of_rank));
  } else if (S > 0) {
    const dim3 grid((unsigned)std::min<int64_t>(kNumSMs * 4, div_up(S, 256)), (unsigned)O);
    MN_LAUNCH("rank_to_source_kernel", st,
              rank_to_source_kernel<<<grid, 256, 0, st>>>(source_masks, S, (int)O, cs, src_of_rank));
  }
  MN_LAUNCH("neighbor_table_kernel", st,
            neighbor_table_kernel<<<(unsigned)div_up(T, 128), 128, 0, st>>>(
                target_masks, T, (int)O, cs, src_of_rank, perm_out, target_bits, nbr_out, tile_bits_out));
  return MN_OK;
}

extern "C" size_t mn_implicit_workspace_bytes(int64_t O, int64_t c_in, int64_t c_out) {
  return align_up((size_t)O * c_in * c_out * 2, 1024) + 1024;
}

extern "C" mn_status mn_sparse_convolution_forward_implicit(
    int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
    const void *sources, const void *weights, const void *weights_t_in, const int32_t *nbr,
    const uint32_t *tile_bits, const int32_t *perm,
    const int32_t *order, const float *scale, const float *shift, const void *residual, int relu,
    double pairs_per_row, int sub_hint, void *targets_out, int32_t *status_dev, void *ws_ptr,
    size_t ws_bytes, void *stream) {
  if (!mn_implicit_supported(O, c_in, c_out, dtype)) {
    set_error("implicit forward: needs fp16/bf16, at most 32 offsets, channels multiple of 8, "
              "c_out <= 256 (got O=%lld c_in=%lld c_out=%lld dtype=%d)", (long long)O,
              (long long)c_in, (long long)c_out, (int)dtype);
    return MN_ERR_UNSUPPORTED;
  }
  MN_CHECK_ARG(S >= 0 && T >= 0 && T < (1ll << 31) && S < (1ll << 31), "implicit forward: bad sizes");
  if (T == 0) return MN_OK;
  MN_CHECK_ARG((weights != nullptr || weights_t_in != nullptr) && nbr != nullptr && tile_bits != nullptr &&
                   targets_out != nullptr && status_dev != nullptr && (S == 0 || sources != nullptr),
               "implicit forward: null pointer");
  MN_CHECK_ARG(((reinterpret_cast<uintptr_t>(sources) | reinterpret_cast<uintptr_t>(targets_out) |
                 reinterpret_cast<uintptr_t>(residual)) & 15) == 0,
               "implicit forward: feature arrays must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == MN_BF16;
  Workspace ws(ws_ptr, ws_bytes);
  const void *weights_t = weights_t_in;
  if (weights_t == nullptr) {
    char *mine = ws.take<char>(align_up((size_t)O * c_in * c_out * 2, 1024));
    MN_CHECK_WS(ws);
    MN_RETURN_IF(launch_transpose_weights(weights, mine, (int)O, (int)c_in, (int)c_out, bf16, st));
    weights_t = mine;
  }

  ImArgs a{};
  a.in = static_cast<const uint8_t *>(sources);
  a.nbr = nbr;
  a.tile_bits = tile_bits;
  a.order = order;
  a.scale = scale;
  a.shift = shift;
  a.residual = static_cast<const uint8_t *>(residual);
  a.perm = perm;
  a.out16 = static_cast<uint8_t *>(targets_out);
  a.status = status_dev;
  a.T = T;
  a.K = (int)c_in;
  a.N = (int)c_out;
  a.n_pad = (int)align_up((size_t)c_out, 16);
  a.k_blocks = (int)div_up(c_in, kBK);
  a.n_tiles128 = (int)div_up(T, kBM);
  // Sub-tiles per CTA tile.  Every sub-tile of a CTA tile reuses the weight tile of a stage,
  // at the price of a shallower ring and, past 512 / (2 * n_pad) sub-tiles, a single
  // accumulator buffer (the epilogue then no longer overlaps the next tile's MMAs).  The
  // automatic choice is the one that measured fastest per output width on maps with two or
  // more pairs per row (1 sub-tile at 64 columns, 2 at 32, 128 and 256); sparse
  // maps keep small CTA tiles and several CTAs per SM.  Callers that have timed the layer
  // pass their own choice.
  int sub = sub_hint;
  if (sub <= 0) {
    sub = 1;
    if (pairs_per_row >= 2.0) sub = a.n_pad >= 128 ? 2 : a.n_pad >= 64 ? 1 : 2;
    while (sub > 1 && (sub * a.n_pad > 512 || a.n_tiles128 < 2 * sub * kNumSMs ||
                       2 * (sub * kBM * kBK * 2 + a.n_pad * kBK * 2) + 4 * 8192 + 2048 > 227 * 1024))
      sub--;
  }
  MN_CHECK_ARG(sub >= 1 && sub <= kMaxSub && sub * a.n_pad <= 512,
               "implicit forward: %d sub-tiles of %d columns do not fit TMEM", sub, a.n_pad);
  a.sub = sub;
  a.acc_bufs = 2 * a.sub * a.n_pad <= 512 ? 2 : 1;
  a.a_bytes = a.sub * kBM * kBK * 2;
  a.stage_bytes = a.a_bytes + a.n_pad * kBK * 2;
  const TcSizing sizing = size_tc_kernel(a.stage_bytes, a.acc_bufs * a.sub * a.n_pad, kMaxStages, kImCtas);
  a.stages = sizing.stages;
  a.tmem_cols = sizing.tmem_cols;
  a.num_offsets = (int)O;
  a.elem_is_bf16 = bf16 ? 1 : 0;
  a.num_tiles = (int)div_up(a.n_tiles128, a.sub);
  a.relu = relu ? 1 : 0;

  CUtensorMap map_b, map_out;
  MN_RETURN_IF(make_kmajor_map(&map_b, weights_t, bf16, c_in, c_out, O, a.n_pad));
  MN_RETURN_IF(make_kmajor_map(&map_out, targets_out, bf16, c_out, T, 0, 32));
  const size_t smem = sizing.smem_bytes;
  MN_CHECK_CUDA(cudaFuncSetAttribute(conv_implicit_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = std::min(a.num_tiles, kNumSMs * sizing.ctas_per_sm);
  MN_LAUNCH("conv_implicit_kernel", st,
            conv_implicit_kernel<<<grid, kImThreads, smem, st>>>(a, map_b, map_out));
  return MN_OK;
}
