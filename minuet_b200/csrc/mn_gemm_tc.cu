// Tensor-core grouped GEMM over kernel offsets: tcgen05.mma with TMEM
// accumulators, operands staged in shared memory by TMA, fp16/bf16 in, fp32
// accumulate.  One persistent launch covers every offset of a convolution (and
// its centre offset), where the reference issues one cuBLAS call per padding
// bucket on up to four streams
// (csrc/minuet/cuda/functions/sparse_convolution.cu:586-641, 647-660).
//
// Layout of one CTA (192 threads, one CTA per SM, cluster size 1, every TMA load is CTA-local):
//   warp 0      TMA producer: A tile [128 rows x 64 k] and B tile [N x 64 k] per
//               k-block into a ring of shared-memory stages (128-byte swizzle)
//   warp 1      allocates TMEM, issues tcgen05.mma (one elected lane), commits
//               stage-free and accumulator-ready barriers
//   warps 2..5  epilogue: tcgen05.ld the 128 x N fp32 accumulator (each warp its
//               own 32-lane quarter), convert, store the rows that exist
// Two accumulators (2 x N columns of TMEM) let the epilogue of tile i overlap
// the MMAs of tile i+1.  Every barrier wait is bounded: on expiry the kernel
// raises bit 2 of *status, all roles leave their loops, TMEM is freed and the
// kernel returns.
//
// B is the weight matrix of one offset TRANSPOSED to [N, K] (K contiguous), so
// that both operands are K-major; a small kernel transposes the layer's weights
// into the workspace first.
#include "mn_tc.cuh"

#include <algorithm>

namespace mn {

namespace {

using namespace tc;

constexpr int kTcThreads = 192;
constexpr int kBM = 128;            // rows per tile = UMMA M
constexpr int kBK = 64;             // k elements per stage = one 128-byte swizzle row
constexpr int kUmmaK = 16;          // k elements per tcgen05.mma (16-bit inputs)
constexpr int kMaxStages = 10;

struct TcArgs {
  int32_t k_blocks;      // ceil(c_in / 64)
  int32_t n_pad;         // c_out rounded up to 16 (UMMA N)
  int32_t c_out;
  int32_t stages;
  int32_t tmem_cols;     // TMEM columns this CTA allocates (two accumulators)
  int32_t a_bytes;       // bytes of one A stage (16 KB)
  int32_t stage_bytes;   // A + B bytes of one stage
  int32_t elem_is_bf16;
  int32_t total_tiles;
  const int32_t *order;  // device, may be NULL
  int32_t *status;       // device status word (bit 2: bounded wait expired)
  int32_t fused_epilogue; // direct problems: add product rows, scale/shift/residual/ReLU
  int32_t plain_store;    // c_out is not a multiple of 8: rows leave with plain stores, no TMA
  void *out_plain;        // [rows, c_out] output of the direct problem for plain_store
  int64_t out_rows;
};

struct TilePos {
  int problem;
  int m0;      // first row of the tile inside the problem
};

__device__ __forceinline__ TilePos locate_tile(const GemmTable &tab, int tile) {
  int lo = 0, hi = tab.num_problems;  // last p with tile_prefix[p] <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tab.tile_prefix[mid] <= tile) lo = mid; else hi = mid;
  }
  return TilePos{lo, (tile - tab.tile_prefix[lo]) * kBM};
}

template <typename T>
__global__ void __launch_bounds__(kTcThreads, 4)
gemm_tc_kernel(const __grid_constant__ GemmTable tab, const __grid_constant__ TcArgs args,
               const __grid_constant__ CUtensorMap map_a,       // gather buffer  [rows, K]
               const __grid_constant__ CUtensorMap map_direct,  // input features [S, K]
               const __grid_constant__ CUtensorMap map_b,       // weights^T      [O, N, K]
               const __grid_constant__ CUtensorMap map_c,       // product buffer [rows, N]
               const __grid_constant__ CUtensorMap map_c_direct,    // output features [T, N]
               const __grid_constant__ PairEpilogue ep) {           // fused epilogue of direct problems
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_full[kMaxStages], bar_empty[kMaxStages];
  __shared__ uint64_t bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  // dynamic shared memory is only guaranteed 16-byte aligned: round up to 1024
  uint8_t *stage_base = reinterpret_cast<uint8_t *>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = args.stages;
  const uint32_t tmem_cols = (uint32_t)args.tmem_cols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&bar_acc_full[a], 1); mbar_init(&bar_acc_empty[a], 4); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
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

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = (uint32_t)args.stage_bytes;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < args.total_tiles; tile += gridDim.x) {
        const TilePos pos = locate_tile(tab, tile);
        const int p = pos.problem;
        const bool direct = tab.direct[p] != 0;
        const int row0 = (int)tab.a_row[p] + pos.m0;
        const int wrow = tab.weight_row[p];
        const int widx = args.order != nullptr ? __ldg(args.order + wrow) : wrow;
        for (int kb = 0; kb < args.k_blocks; kb++) {
          if (!mbar_wait(&bar_empty[stage], phase ^ 1u, abort_flag, args.status)) { alive = false; break; }
          uint8_t *sa = stage_base + (size_t)stage * args.stage_bytes;
          uint8_t *sb = sa + args.a_bytes;
          mbar_expect_tx(&bar_full[stage], tx_bytes);
          tma_load_2d(sa, direct ? &map_direct : &map_a, kb * kBK, row0, &bar_full[stage]);
          tma_load_3d(sb, &map_b, kb * kBK, 0, widx, &bar_full[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, A/B format, both K-major, N, M
      const uint32_t fmt = args.elem_is_bf16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) |
                             ((uint32_t)(args.n_pad >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < args.total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&bar_acc_empty[acc], acc_phase ^ 1u, abort_flag, args.status)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * args.n_pad);
        for (int kb = 0; kb < args.k_blocks; kb++) {
          if (!mbar_wait(&bar_full[stage], phase, abort_flag, args.status)) { alive = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_u32(stage_base + (size_t)stage * args.stage_bytes);
          const uint32_t sb = sa + (uint32_t)args.a_bytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; k++) {
            const uint64_t da = umma_desc(sa + k * kUmmaK * 2);
            const uint64_t db = umma_desc(sb + k * kUmmaK * 2);
            umma_f16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bar_empty[stage]);   // the stage is free once these MMAs have read it
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit(&bar_acc_full[acc]);    // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // Each warp turns its 32 accumulator rows into 16-bit, 64 columns at a time,
    // parks them in a 128-byte-swizzled shared tile and lets TMA store the tile:
    // full 128-byte lines reach memory, rows past the end of the output array
    // are clipped by the tensor map, rows past the end of a problem land in the
    // padding of the product buffer.
    const int quarter = warp & 3;           // TMEM lanes a warp may read: 32 * (warp id % 4)
    uint8_t *cbuf = stage_base + (size_t)stages * args.stage_bytes + (size_t)(warp - 2) * 8192;
    int acc = 0, chunk = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < args.total_tiles; tile += gridDim.x) {
      const TilePos pos = locate_tile(tab, tile);
      const int p = pos.problem;
      const bool direct = tab.direct[p] != 0;
      const int out_row = (direct ? 0 : (int)tab.a_row[p]) + pos.m0 + quarter * 32;
      // the hit word of this lane's output row and the first product row it names are
      // fetched while the tile's MMAs are still in flight
      uint32_t hit_word = 0u;
      int first_hit = -1;
      int64_t first_row = 0;
      if (direct && args.fused_epilogue && ep.bits != nullptr && (int64_t)out_row + lane < ep.T) {
        const int64_t t = (int64_t)out_row + lane;
        hit_word = __ldg(ep.bits + t) & ep.keep;
        if (hit_word != 0u) {
          first_hit = __ffs(hit_word) - 1;
          first_row = ep.row_begin[first_hit] + __ldg(ep.target_masks + (int64_t)first_hit * ep.T + t);
          const char *prow = reinterpret_cast<const char *>(ep.products + first_row * args.c_out);
          for (int off = 0; off < args.c_out * 4; off += 128)
            asm volatile("prefetch.global.L1 [%0];" ::"l"(prow + off));
        }
      }
      if (direct && args.fused_epilogue && ep.residual != nullptr && (int64_t)out_row + lane < ep.T) {
        // the residual row of this lane is on its way while the MMAs run
        const char *rrow = static_cast<const char *>(ep.residual) +
                           ((int64_t)out_row + lane) * args.c_out * 2;
        for (int off = 0; off < args.c_out * 2; off += 128)
          asm volatile("prefetch.global.L1 [%0];" ::"l"(rrow + off));
      }
      int ok = 1;   // one lane polls the barrier, the warp follows
      if (lane == 0) ok = mbar_wait(&bar_acc_full[acc], acc_phase, abort_flag, args.status) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * args.n_pad);
      for (int c0 = 0; c0 < args.n_pad; c0 += 64, chunk++) {
        uint8_t *buf = cbuf + (chunk & 1) * 4096;
        bool buffer_free = false;
        // 32 columns at a time (a 64-column register tile would cap the kernel at one
        // CTA per SM); the two halves fill one 64-column staging tile
        for (int half = 0; half < 2; half++) {
          const int cb = c0 + 32 * half;
          if (cb >= args.n_pad) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + (uint32_t)cb, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (direct && args.fused_epilogue) {
            const int64_t t = (int64_t)out_row + lane;
            const int n = args.c_out;
            if (t < ep.T) {
              // the other offsets' products of this output row, named by its hit word
              uint32_t w = hit_word;
              while (w != 0u) {
                const int pr = __ffs(w) - 1;
                w &= w - 1u;
                const int64_t prow = pr == first_hit
                    ? first_row
                    : ep.row_begin[pr] + __ldg(ep.target_masks + (int64_t)pr * ep.T + t);
                const float4 *src = reinterpret_cast<const float4 *>(ep.products + prow * n + cb);
#pragma unroll
                for (int v = 0; v < 8; v++) {
                  if (cb + 4 * v < n) {
                    const float4 a = __ldg(src + v);
                    r[4 * v] = __float_as_uint(__uint_as_float(r[4 * v]) + a.x);
                    r[4 * v + 1] = __float_as_uint(__uint_as_float(r[4 * v + 1]) + a.y);
                    r[4 * v + 2] = __float_as_uint(__uint_as_float(r[4 * v + 2]) + a.z);
                    r[4 * v + 3] = __float_as_uint(__uint_as_float(r[4 * v + 3]) + a.w);
                  }
                }
              }
#pragma unroll
              for (int v = 0; v < 4; v++) {
                const int c = cb + v * 8;
                if (c < n) {
                  float f[8];
#pragma unroll
                  for (int i = 0; i < 8; i++) f[i] = __uint_as_float(r[v * 8 + i]);
                  if (ep.scale != nullptr) {
                    if (c + 8 <= n) {
                      const float4 s0 = __ldg(reinterpret_cast<const float4 *>(ep.scale + c));
                      const float4 s1 = __ldg(reinterpret_cast<const float4 *>(ep.scale + c) + 1);
                      f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w;
                      f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
                    } else {
                      for (int i = 0; i < 8 && c + i < n; i++) f[i] *= __ldg(ep.scale + c + i);
                    }
                  }
                  if (ep.shift != nullptr) {
                    if (c + 8 <= n) {
                      const float4 s0 = __ldg(reinterpret_cast<const float4 *>(ep.shift + c));
                      const float4 s1 = __ldg(reinterpret_cast<const float4 *>(ep.shift + c) + 1);
                      f[0] += s0.x; f[1] += s0.y; f[2] += s0.z; f[3] += s0.w;
                      f[4] += s1.x; f[5] += s1.y; f[6] += s1.z; f[7] += s1.w;
                    } else {
                      for (int i = 0; i < 8 && c + i < n; i++) f[i] += __ldg(ep.shift + c + i);
                    }
                  }
                  if (ep.residual != nullptr && c + 8 <= n) {
                    const uint4 rv = __ldg(reinterpret_cast<const uint4 *>(
                        static_cast<const uint8_t *>(ep.residual) + (t * n + c) * 2));
                    const uint16_t *r16 = reinterpret_cast<const uint16_t *>(&rv);
#pragma unroll
                    for (int i = 0; i < 8; i++)
                      f[i] += args.elem_is_bf16 ? __uint_as_float((uint32_t)r16[i] << 16)
                                                : __half2float(__ushort_as_half(r16[i]));
                  } else if (ep.residual != nullptr) {
                    const uint16_t *r16 = static_cast<const uint16_t *>(ep.residual) + t * n + c;
                    for (int i = 0; i < 8 && c + i < n; i++)
                      f[i] += args.elem_is_bf16 ? __uint_as_float((uint32_t)r16[i] << 16)
                                                : __half2float(__ushort_as_half(r16[i]));
                  }
                  if (ep.relu) {
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = fmaxf(f[i], 0.f);
                  }
#pragma unroll
                  for (int i = 0; i < 8; i++) r[v * 8 + i] = __float_as_uint(f[i]);
                }
              }
            }
          }
          if (args.plain_store) {
            // row pitch not a multiple of 16 bytes: no tensor map exists for this output
            const int64_t t = (int64_t)out_row + lane;
            if (t < args.out_rows) {
              uint32_t *dst = reinterpret_cast<uint32_t *>(static_cast<uint16_t *>(args.out_plain) +
                                                           t * args.c_out + cb);
#pragma unroll
              for (int h = 0; h < 16; h++) {
                if (cb + 2 * h + 1 < args.c_out) {
                  const float lo = __uint_as_float(r[2 * h]), hi = __uint_as_float(r[2 * h + 1]);
                  if (args.elem_is_bf16) {
                    __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
                    dst[h] = *reinterpret_cast<uint32_t *>(&pk);
                  } else {
                    __half2 pk = __floats2half2_rn(lo, hi);
                    dst[h] = *reinterpret_cast<uint32_t *>(&pk);
                  }
                }
              }
            }
            continue;
          }
          if (!buffer_free) {
            // the store that last read this buffer (two chunks ago) must be done with it
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            buffer_free = true;
          }
#pragma unroll
          for (int v = 0; v < 4; v++) {         // 8 outputs = one 16-byte piece of the row
            uint4 out;
            uint32_t *o32 = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
            for (int h = 0; h < 4; h++) {
              const float lo = __uint_as_float(r[v * 8 + 2 * h]);
              const float hi = __uint_as_float(r[v * 8 + 2 * h + 1]);
              if (args.elem_is_bf16) {
                __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
                o32[h] = *reinterpret_cast<uint32_t *>(&pk);
              } else {
                __half2 pk = __floats2half2_rn(lo, hi);
                o32[h] = *reinterpret_cast<uint32_t *>(&pk);
              }
            }
            // 128-byte swizzle: 16-byte piece v of row `lane` lives at piece v ^ (lane % 8)
            const int piece = half * 4 + v;
            *reinterpret_cast<uint4 *>(buf + lane * 128 + ((piece ^ (lane & 7)) << 4)) = out;
          }
        }
        if (args.plain_store) continue;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(direct ? &map_c_direct : &map_c, c0, out_row, buf);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  }

  // ------------------------------ teardown ------------------------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_abort) {
    // a role gave up: give copies and MMAs still in flight time to land before
    // shared memory and TMEM go away
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(tmem_cols)
                 : "memory");
  }
}

// wt[o][n][k] = w[o][k][n]
template <typename T>
__global__ void __launch_bounds__(256)
transpose_weights_kernel(const T *__restrict__ w, T *__restrict__ wt, int K, int N) {
  __shared__ T tile[32][33];
  const int o = blockIdx.z;
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const T *src = w + (int64_t)o * K * N;
  T *dst = wt + (int64_t)o * K * N;
  for (int i = ty; i < 32; i += 8)
    if (k0 + i < K && n0 + tx < N) tile[i][tx] = src[(int64_t)(k0 + i) * N + n0 + tx];
  __syncthreads();
  for (int i = ty; i < 32; i += 8)
    if (n0 + i < N && k0 + tx < K) dst[(int64_t)(n0 + i) * K + k0 + tx] = tile[tx][i];
}

}  // namespace

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// K-major operand map: dims (K, rows[, batch]), box (64, box_rows[, 1]), 128-byte swizzle
mn_status make_kmajor_map(CUtensorMap *map, const void *base, bool bf16, int64_t K, int64_t rows,
                   int64_t batch, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return MN_ERR_CUDA;
  }
  const cuuint32_t rank = batch > 0 ? 3 : 2;
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(batch, 1)};
  cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)K * 2 * (cuuint64_t)rows};
  cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        rank, const_cast<void *>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (K=%lld rows=%lld batch=%lld)", (int)r,
              (long long)K, (long long)rows, (long long)batch);
    return MN_ERR_CUDA;
  }
  return MN_OK;
}


mn_status launch_transpose_weights(const void *weights, void *weights_t, int O, int c_in, int c_out,
                                   bool bf16, cudaStream_t st) {
  const dim3 grid((unsigned)div_up(c_out, 32), (unsigned)div_up(c_in, 32), (unsigned)O);
  if (bf16) {
    MN_LAUNCH("transpose_weights_kernel", st,
              transpose_weights_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
                  static_cast<const __nv_bfloat16 *>(weights),
                  static_cast<__nv_bfloat16 *>(weights_t), c_in, c_out));
  } else {
    MN_LAUNCH("transpose_weights_kernel", st,
              transpose_weights_kernel<__half><<<grid, 256, 0, st>>>(
                  static_cast<const __half *>(weights), static_cast<__half *>(weights_t), c_in,
                  c_out));
  }
  return MN_OK;
}

size_t gemm_tc_workspace_bytes(int64_t O, int64_t c_in, int64_t c_out) {
  return align_up((size_t)O * c_in * c_out * 2, 1024);
}

bool gemm_tc_supported(int c_in, int c_out, mn_dtype dtype) {
  return (dtype == MN_F16 || dtype == MN_BF16) && c_in >= 8 && c_in % 8 == 0 && c_out >= 8 &&
         c_out % 8 == 0 && c_out <= 256;
}

namespace {

mn_status launch_gemm_tc_impl(const GemmTable &tab_in, const TcOperands &ops, int c_in, int c_out,
                              mn_dtype dtype, const void *weights, const int32_t *order,
                              const PairEpilogue *ep, bool weights_are_transposed, cudaStream_t st,
                              bool *handled);

}  // namespace

mn_status launch_gemm_tc(const GemmTable &tab_in, const TcOperands &ops, int c_in, int c_out,
                         mn_dtype dtype, const void *weights, const int32_t *order,
                         cudaStream_t st, bool *handled) {
  return launch_gemm_tc_impl(tab_in, ops, c_in, c_out, dtype, weights, order, nullptr, false, st,
                             handled);
}

// Dense product of `rows` input rows with the weight matrix of mask row `centre`
// (weights_t: already transposed [O, c_out, c_in]) and the fused epilogue.
mn_status launch_centre_gemm(int64_t rows, int64_t c_in, int64_t c_out, bool bf16, const void *sources,
                             const void *weights_t, int O, int centre, const int32_t *order,
                             const PairEpilogue &ep, void *out, int32_t *status_dev, cudaStream_t st) {
  GemmTable tab{};
  tab.num_problems = 1;
  tab.rows[0] = (int32_t)rows;
  tab.weight_row[0] = centre;
  tab.a[0] = sources;
  tab.c[0] = out;
  tab.a_row[0] = 0;
  tab.direct[0] = 1;
  TcOperands ops;
  ops.sources = sources;
  ops.source_rows = rows;
  ops.out = out;
  ops.out_rows = rows;
  ops.weights_t = const_cast<void *>(weights_t);
  ops.num_weights = O;
  ops.status = status_dev;
  bool handled = false;
  MN_RETURN_IF(launch_gemm_tc_impl(tab, ops, (int)c_in, (int)c_out, bf16 ? MN_BF16 : MN_F16, nullptr,
                                   order, &ep, true, st, &handled));
  if (!handled) {
    set_error("centre GEMM: shape not covered by the tensor-core kernel (c_in=%lld c_out=%lld)",
              (long long)c_in, (long long)c_out);
    return MN_ERR_UNSUPPORTED;
  }
  return MN_OK;
}

namespace {

mn_status launch_gemm_tc_impl(const GemmTable &tab_in, const TcOperands &ops, int c_in, int c_out,
                              mn_dtype dtype, const void *weights, const int32_t *order,
                              const PairEpilogue *ep, bool weights_are_transposed, cudaStream_t st,
                              bool *handled) {
  *handled = false;
  // a dense problem with the fused epilogue also takes even c_out that are not a multiple
  // of 8 (the rows then leave with plain stores instead of through a tensor map)
  const bool plain_store = ep != nullptr && c_out % 8 != 0 && c_out % 2 == 0 && c_out <= 256 &&
                           c_in >= 8 && c_in % 8 == 0 && (dtype == MN_F16 || dtype == MN_BF16);
  if ((!gemm_tc_supported(c_in, c_out, dtype) && !plain_store) || ops.weights_t == nullptr ||
      ops.status == nullptr)
    return MN_OK;
  const bool bf16 = dtype == MN_BF16;
  const int O = ops.num_weights;

  // weights [O, K, N] -> [O, N, K]
  if (!weights_are_transposed)
    MN_RETURN_IF(launch_transpose_weights(weights, ops.weights_t, O, c_in, c_out, bf16, st));

  GemmTable tab = tab_in;
  tab.tile_rows = kBM;
  tab.tile_prefix[0] = 0;
  for (int p = 0; p < tab.num_problems; p++)
    tab.tile_prefix[p + 1] = tab.tile_prefix[p] + (int)div_up(tab.rows[p], kBM);
  const int total_tiles = tab.tile_prefix[tab.num_problems];
  if (total_tiles == 0) { *handled = true; return MN_OK; }

  TcArgs args{};
  args.k_blocks = (int)div_up(c_in, kBK);
  args.n_pad = (int)align_up((size_t)c_out, 16);
  args.c_out = c_out;
  args.a_bytes = kBM * kBK * 2;
  args.stage_bytes = args.a_bytes + args.n_pad * kBK * 2;
  const TcSizing sizing = size_tc_kernel(args.stage_bytes, 2 * args.n_pad, kMaxStages, 4);
  args.stages = sizing.stages;
  args.tmem_cols = sizing.tmem_cols;
  args.elem_is_bf16 = bf16 ? 1 : 0;
  args.total_tiles = total_tiles;
  args.order = order;
  args.status = ops.status;
  args.fused_epilogue = ep != nullptr ? 1 : 0;
  args.plain_store = plain_store ? 1 : 0;
  args.out_plain = ops.out;
  args.out_rows = ops.out_rows;
  static const PairEpilogue no_epilogue{};
  const PairEpilogue &epilogue = ep != nullptr ? *ep : no_epilogue;

  CUtensorMap map_a, map_direct, map_b, map_c, map_c_direct;
  // an operand that no problem uses still needs a valid map: point it at the other one
  const void *gather_base = ops.gathered != nullptr ? ops.gathered : ops.sources;
  const int64_t gather_rows = ops.gathered != nullptr ? ops.gathered_rows : ops.source_rows;
  const void *direct_base = ops.sources != nullptr ? ops.sources : ops.gathered;
  const int64_t direct_rows = ops.sources != nullptr ? ops.source_rows : ops.gathered_rows;
  MN_CHECK_ARG(gather_base != nullptr && gather_rows > 0, "gemm_tc: no A operand");
  MN_CHECK_ARG((reinterpret_cast<uintptr_t>(gather_base) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(direct_base) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(ops.weights_t) & 15) == 0,
               "gemm_tc: operands must be 16-byte aligned");
  MN_RETURN_IF(make_kmajor_map(&map_a, gather_base, bf16, c_in, gather_rows, 0, kBM));
  MN_RETURN_IF(make_kmajor_map(&map_direct, direct_base, bf16, c_in, direct_rows, 0, kBM));
  MN_RETURN_IF(make_kmajor_map(&map_b, ops.weights_t, bf16, c_in, c_out, O, args.n_pad));
  // outputs: [rows, N], box 64 columns x 32 rows (one epilogue warp), 128-byte swizzle
  const void *prod_base = ops.products != nullptr ? ops.products : ops.out;
  const int64_t prod_rows = ops.products != nullptr ? ops.gathered_rows : ops.out_rows;
  const void *out_base = ops.out != nullptr ? ops.out : ops.products;
  const int64_t out_rows = ops.out != nullptr ? ops.out_rows : ops.gathered_rows;
  MN_CHECK_ARG(prod_base != nullptr && prod_rows > 0 &&
                   (reinterpret_cast<uintptr_t>(prod_base) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out_base) & 15) == 0,
               "gemm_tc: outputs must exist and be 16-byte aligned");
  if (plain_store) {
    map_c = map_b;          // never used: the epilogue stores the rows itself
    map_c_direct = map_b;
  } else {
    MN_RETURN_IF(make_kmajor_map(&map_c, prod_base, bf16, c_out, prod_rows, 0, 32));
    MN_RETURN_IF(make_kmajor_map(&map_c_direct, out_base, bf16, c_out, out_rows, 0, 32));
  }

  const size_t smem = sizing.smem_bytes;
  const int grid = std::min(total_tiles, kNumSMs * sizing.ctas_per_sm);
  if (bf16) {
    MN_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<__nv_bfloat16>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MN_LAUNCH("gemm_tc_kernel", st,
              gemm_tc_kernel<__nv_bfloat16><<<grid, kTcThreads, smem, st>>>(
                  tab, args, map_a, map_direct, map_b, map_c, map_c_direct, epilogue));
  } else {
    MN_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<__half>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MN_LAUNCH("gemm_tc_kernel", st,
              gemm_tc_kernel<__half><<<grid, kTcThreads, smem, st>>>(tab, args, map_a, map_direct,
                                                                    map_b, map_c, map_c_direct,
                                                                    epilogue));
  }
  *handled = true;
  return MN_OK;
}

}  // namespace

}  // namespace mn
