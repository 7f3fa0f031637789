// Gather - grouped GEMM - Scatter forward pass of a sparse convolution.
//
// Reference: SparseConvolutionForward::operator()
// (csrc/minuet/cuda/functions/sparse_convolution.cu:505-661): weights permuted
// into size order, a host bucket plan, a padded gather
// (kernels/padded_gather_warp_optimized.cuh:11-63), one cuBLAS (batched) GEMM
// per bucket on up to four streams, an output-stationary padded scatter
// (kernels/padded_scatter_warp_optimized.cuh:11-64) and a dense GEMM with beta=1
// for the centre offset.
//
// Here the GEMM over all offsets is ONE grouped launch driven by a problem
// table in kernel parameters, so no offset needs equal-size buckets: rows of
// mask row o live at [row_begin[o], row_begin[o] + size[o]) of the gather
// buffer, with row_begin aligned to the GEMM's row tile.  Weights are indexed
// through `order` on the device instead of being permuted on every call.  The
// centre offset (when the shortcut applies) is one more problem of the same
// launch that reads the input features and writes the output rows directly;
// the scatter then adds the other offsets in mask-row order and the centre
// last, which is the reference's summation order.
#include "mn_common.cuh"

#include <algorithm>
#include <vector>

namespace mn {

namespace {

constexpr int kRowAlign = 128;  // row_begin alignment = row tile of the tensor-core GEMM

template <typename T> struct VecOf;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

template <int kBytes> struct Chunk;
template <> struct Chunk<16> { using type = uint4; };
template <> struct Chunk<8> { using type = uint2; };
template <> struct Chunk<4> { using type = uint32_t; };
template <> struct Chunk<2> { using type = uint16_t; };

struct RowPlan {
  int64_t row_begin[MN_MAX_OFFSETS + 1];
};

// ---------------------------------------------------------------------------
// gather: buf[row_begin[o] + source_masks[o, s], :] = in[s, :]
// ---------------------------------------------------------------------------
struct GatherArgs {
  const char *in;              // [S, row_bytes]
  char *buf;                   // [total_rows, row_bytes]
  const int32_t *source_masks; // [O, S]
  int64_t S;
  int32_t num_offsets;         // mask rows that go through the buffer
  int32_t row_bytes;
  int32_t lanes_per_row;       // power of two <= 32
};

// A warp owns 32 consecutive source rows.  It reads the mask words of eight
// offsets at a time (eight independent coalesced 128-byte loads in flight),
// then, per offset, compacts the hit rows through shared memory and copies
// 32/lanes_per_row rows per step with 16-byte accesses; the input rows stay in
// L1 across the offsets that reuse them.
template <int kVec>
__global__ void __launch_bounds__(256)
gather_kernel(const GatherArgs g, const __grid_constant__ RowPlan plan) {
  using V = typename Chunk<kVec>::type;
  constexpr int kBatch = 8;
  __shared__ int2 s_list[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lpr = g.lanes_per_row, rpi = 32 / lpr;
  const int sub = lane / lpr, part = lane % lpr;
  const int chunks = g.row_bytes / kVec;
  const int64_t n_chunks32 = (g.S + 31) >> 5;
  for (int64_t blk = (int64_t)blockIdx.x * 8 + warp; blk < n_chunks32; blk += (int64_t)gridDim.x * 8) {
    const int64_t s = (blk << 5) + lane;
    for (int o0 = 0; o0 < g.num_offsets; o0 += kBatch) {
      int m[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; i++)
        m[i] = (s < g.S && o0 + i < g.num_offsets)
                   ? __ldg(g.source_masks + (int64_t)(o0 + i) * g.S + s) : -1;
#pragma unroll
      for (int i = 0; i < kBatch; i++) {
        const unsigned hits = __ballot_sync(0xffffffffu, m[i] >= 0);
        if (hits == 0) continue;
        const int cnt = __popc(hits);
        if (m[i] >= 0) {
          const int r = __popc(hits & ((1u << lane) - 1u));
          s_list[warp][r] = make_int2(lane, m[i]);
        }
        __syncwarp();
        for (int e0 = 0; e0 < cnt; e0 += rpi) {
          const int e = e0 + sub;
          if (e < cnt) {
            const int2 it = s_list[warp][e];
            const V *src = reinterpret_cast<const V *>(g.in + ((blk << 5) + it.x) * g.row_bytes);
            V *dst = reinterpret_cast<V *>(g.buf + (plan.row_begin[o0 + i] + it.y) * g.row_bytes);
            for (int c = part; c < chunks; c += lpr) dst[c] = __ldg(src + c);
          }
        }
        __syncwarp();
      }
    }
  }
}

// ---------------------------------------------------------------------------
// scatter: out[t, :] = sum_o buf[row_begin[o] + target_masks[o, t], :] (+ out[t, :])
// ---------------------------------------------------------------------------
template <typename T>
struct ScatterArgs {
  const T *buf;                // [total_rows, C]
  T *out;                      // [T, C]
  const int32_t *target_masks; // [O, T]
  int64_t T_rows;
  int32_t num_offsets;
  int32_t channels;
  int32_t lanes_per_row;
  int32_t add_existing;        // out already holds the centre product: add it last
};

// A warp owns 32 consecutive target rows.  Phase 1: lane r reads the mask words
// of row r for every offset (coalesced, many loads in flight), keeps a bit per
// hit and parks the words in shared memory.  Phase 2: lanes_per_row lanes share
// one row, walk only that row's hits in mask-row order, accumulate the product
// rows in fp32 registers and write the row once (adding the centre product that
// the GEMM already left in `out` last, when there is one).
template <typename T, int kVecElems, int kAcc>
__global__ void __launch_bounds__(256)
scatter_kernel(const ScatterArgs<T> a, const __grid_constant__ RowPlan plan) {
  using V = typename Chunk<kVecElems * sizeof(T)>::type;
  extern __shared__ int32_t s_masks[];   // [warps][num_offsets][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int O = a.num_offsets;
  int32_t *my = s_masks + (size_t)warp * O * 32;
  const int lpr = a.lanes_per_row, rpi = 32 / lpr;
  const int sub = lane / lpr, part = lane % lpr;
  const int chunks = a.channels / kVecElems;
  const int64_t n_blocks32 = (a.T_rows + 31) >> 5;
  for (int64_t blk = (int64_t)blockIdx.x * nwarps + warp; blk < n_blocks32;
       blk += (int64_t)gridDim.x * nwarps) {
    const int64_t t_lane = (blk << 5) + lane;
    uint32_t hits[4] = {0u, 0u, 0u, 0u};   // bit o of word o/32: offset o feeds row `lane`
#pragma unroll
    for (int w = 0; w < 4; w++) {
      if (w * 32 < O) {
        for (int o0 = w * 32; o0 < min(O, w * 32 + 32); o0 += 8) {
          int m[8];
#pragma unroll
          for (int i = 0; i < 8; i++)
            m[i] = (t_lane < a.T_rows && o0 + i < O)
                       ? __ldg(a.target_masks + (int64_t)(o0 + i) * a.T_rows + t_lane) : -1;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            if (o0 + i < O) my[(o0 + i) * 32 + lane] = m[i];
            hits[w] |= (m[i] >= 0 ? 1u : 0u) << ((o0 + i) & 31);
          }
        }
      }
    }
    __syncwarp();
    for (int r0 = 0; r0 < 32; r0 += rpi) {
      const int r = r0 + sub;
      const int64_t t = (blk << 5) + r;
      // a row without any pair keeps the centre product the GEMM already wrote
      // (all shuffles happen here, before the row groups of the warp diverge)
      uint32_t hw[4] = {0u, 0u, 0u, 0u}, any_hit = 0u;
#pragma unroll
      for (int w = 0; w < 4; w++) {
        if (w * 32 < O) hw[w] = __shfl_sync(0xffffffffu, hits[w], r);
        any_hit |= hw[w];
      }
      if (any_hit == 0u && a.add_existing) continue;
      float acc[kAcc];
#pragma unroll
      for (int i = 0; i < kAcc; i++) acc[i] = 0.f;
#pragma unroll
      for (int w = 0; w < 4; w++) {
        if (w * 32 < O) {
          uint32_t h = hw[w];
          while (h != 0u) {
            const int o = w * 32 + __ffs(h) - 1;
            h &= h - 1u;
            const int m = my[o * 32 + r];
            const V *src = reinterpret_cast<const V *>(a.buf + (plan.row_begin[o] + m) * a.channels);
#pragma unroll
            for (int i = 0; i < kAcc / kVecElems; i++) {
              const int c = part + i * lpr;
              if (c < chunks) {
                const V v = __ldg(src + c);
                const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
                for (int k = 0; k < kVecElems; k++) acc[i * kVecElems + k] += to_f32(e[k]);
              }
            }
          }
        }
      }
      if (t < a.T_rows) {
        V *dst = reinterpret_cast<V *>(a.out + t * a.channels);
#pragma unroll
        for (int i = 0; i < kAcc / kVecElems; i++) {
          const int c = part + i * lpr;
          if (c < chunks) {
            V v;
            T *e = reinterpret_cast<T *>(&v);
            if (a.add_existing) {
              const V old = dst[c];
              const T *oe = reinterpret_cast<const T *>(&old);
#pragma unroll
              for (int k = 0; k < kVecElems; k++)
                e[k] = from_f32<T>(acc[i * kVecElems + k] + to_f32(oe[k]));
            } else {
#pragma unroll
              for (int k = 0; k < kVecElems; k++) e[k] = from_f32<T>(acc[i * kVecElems + k]);
            }
            dst[c] = v;
          }
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace

namespace {

constexpr int kGemmTM = 64, kGemmTN = 64, kGemmTK = 16;

// SIMT fallback / fp32 path: 64x64 tile, 256 threads x (4x4) fp32 FFMA, any
// c_in / c_out.  fp32 features must not go through TF32 tensor cores (10-bit
// mantissa breaks the 1e-5 bound), so this is also the product path for fp32.
template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const __grid_constant__ GemmTable tab, const T *__restrict__ weights,
                 const int32_t *__restrict__ order, int c_in, int c_out) {
  __shared__ float sA[kGemmTK][kGemmTM + 4];
  __shared__ float sB[kGemmTK][kGemmTN + 4];
  __shared__ int s_prob;
  if (threadIdx.x == 0) {
    int lo = 0, hi = tab.num_problems;  // last p with tile_prefix[p] <= blockIdx.x
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tab.tile_prefix[mid] <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    s_prob = lo;
  }
  __syncthreads();
  const int p = s_prob;
  const int m0 = ((int)blockIdx.x - tab.tile_prefix[p]) * kGemmTM;
  const int n0 = blockIdx.y * kGemmTN;
  const int rows = tab.rows[p];
  const T *A = static_cast<const T *>(tab.a[p]);
  T *C = static_cast<T *>(tab.c[p]);
  const int wrow = tab.weight_row[p];
  const T *B = weights + (int64_t)(order != nullptr ? __ldg(order + wrow) : wrow) * c_in * c_out;

  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < c_in; k0 += kGemmTK) {
    for (int i = threadIdx.x; i < kGemmTM * kGemmTK; i += 256) {
      const int m = i / kGemmTK, k = i % kGemmTK;
      float v = 0.f;
      if (m0 + m < rows && k0 + k < c_in) v = to_f32(A[(int64_t)(m0 + m) * c_in + k0 + k]);
      sA[k][m] = v;
    }
    for (int i = threadIdx.x; i < kGemmTK * kGemmTN; i += 256) {
      const int k = i / kGemmTN, n = i % kGemmTN;
      float v = 0.f;
      if (k0 + k < c_in && n0 + n < c_out) v = to_f32(B[(int64_t)(k0 + k) * c_out + n0 + n]);
      sB[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kGemmTK; k++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = sA[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = sB[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < c_out) C[(int64_t)m * c_out + n] = from_f32<T>(acc[i][j]);
    }
  }
}

int pow2_floor(int v) {
  int p = 1;
  while (p * 2 <= v) p *= 2;
  return p;
}

size_t dtype_size(mn_dtype d) { return d == MN_F32 ? 4 : 2; }

struct ConvLayout {
  int n_buf;            // mask rows routed through the gather buffer
  bool shortcut;        // last mask row handled as a dense product
  RowPlan plan;
  int64_t total_rows;
};

ConvLayout make_layout(const int32_t *sizes, int64_t O, int64_t S, int64_t T, int allow_shortcut) {
  ConvLayout L{};
  L.shortcut = allow_shortcut && O > 0 && sizes[O - 1] == T && sizes[O - 1] == S;
  L.n_buf = (int)O - (L.shortcut ? 1 : 0);
  L.plan.row_begin[0] = 0;
  for (int o = 0; o < L.n_buf; o++)
    L.plan.row_begin[o + 1] = L.plan.row_begin[o] + (int64_t)align_up((size_t)sizes[o], kRowAlign);
  for (int o = L.n_buf; o < MN_MAX_OFFSETS; o++) L.plan.row_begin[o + 1] = L.plan.row_begin[L.n_buf];
  L.total_rows = L.plan.row_begin[L.n_buf];
  return L;
}

struct ConvBuffers {
  char *gathered;   // [total_rows, c_in]
  char *products;   // [total_rows, c_out]
  char *weights_t;  // [O, c_out, c_in], tensor-core path only
};

mn_status carve(const ConvLayout &L, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
                void *ws_ptr, size_t ws_bytes, ConvBuffers *b) {
  Workspace ws(ws_ptr, ws_bytes);
  const size_t e = dtype_size(dtype);
  b->gathered = ws.take<char>((size_t)std::max<int64_t>(L.total_rows, 1) * c_in * e);
  b->products = ws.take<char>((size_t)std::max<int64_t>(L.total_rows, 1) * c_out * e);
  b->weights_t = nullptr;
  if (gemm_tc_supported((int)c_in, (int)c_out, dtype))
    b->weights_t = ws.take<char>(gemm_tc_workspace_bytes(O, c_in, c_out));
  MN_CHECK_WS(ws);
  return MN_OK;
}

mn_status run_gather(const ConvLayout &L, const ConvBuffers &b, int64_t S, int64_t c_in,
                     mn_dtype dtype, const void *sources, const int32_t *source_masks, int tile,
                     cudaStream_t st) {
  if (L.n_buf == 0 || S == 0) return MN_OK;
  const int e = (int)dtype_size(dtype);
  const int row_bytes = (int)c_in * e;
  int vec = 16;
  while (vec > e && (row_bytes % vec != 0)) vec >>= 1;
  // tile = channels per lane (the reference's tunable); 1 = built-in choice
  int chunks = row_bytes / vec;
  int lpr = pow2_floor(std::min(32, chunks));
  if (tile > 1) {
    const int want_vec = std::min(16, pow2_floor(std::max(e, tile * e)));
    while (vec > want_vec) vec >>= 1;
    chunks = row_bytes / vec;
    lpr = pow2_floor(std::max(1, std::min(32, (int)(c_in / tile))));
    lpr = std::min(lpr, pow2_floor(std::min(32, chunks)));
  }
  if ((reinterpret_cast<uintptr_t>(sources) | reinterpret_cast<uintptr_t>(b.gathered)) % vec != 0) {
    vec = e; chunks = row_bytes / vec; lpr = pow2_floor(std::min(32, chunks));
  }
  GatherArgs g{};
  g.in = static_cast<const char *>(sources);
  g.buf = b.gathered;
  g.source_masks = source_masks;
  g.S = S;
  g.num_offsets = L.n_buf;
  g.row_bytes = row_bytes;
  g.lanes_per_row = lpr;
  const int blocks = (int)std::min<int64_t>(kNumSMs * 64, div_up(div_up(S, 32), 8));
  {
  LaunchScope scope("gather_kernel", st);
  switch (vec) {
    case 16: gather_kernel<16><<<blocks, 256, 0, st>>>(g, L.plan); break;
    case 8: gather_kernel<8><<<blocks, 256, 0, st>>>(g, L.plan); break;
    case 4: gather_kernel<4><<<blocks, 256, 0, st>>>(g, L.plan); break;
    default: gather_kernel<2><<<blocks, 256, 0, st>>>(g, L.plan); break;
  }
  }
  MN_CHECK_LAUNCH();
  return MN_OK;
}

template <typename T>
mn_status run_scatter_t(const ConvLayout &L, const ConvBuffers &b, int64_t T_rows, int64_t c_out,
                        const int32_t *target_masks, int tile, void *out, cudaStream_t st) {
  if (T_rows == 0) return MN_OK;
  constexpr int e = (int)sizeof(T);
  int vec_elems = 16 / e;
  while (vec_elems > 1 && (c_out % vec_elems != 0)) vec_elems >>= 1;
  if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(b.products)) % (vec_elems * e) != 0)
    vec_elems = 1;
  int chunks = (int)c_out / vec_elems;
  int lpr = pow2_floor(std::min(32, chunks));
  if (tile > 1) {
    lpr = pow2_floor(std::max(1, std::min(32, (int)(c_out / tile))));
    lpr = std::min(lpr, pow2_floor(std::min(32, chunks)));
  }
  // accumulators per lane must fit the compiled bound
  auto acc_needed = [&](int l) { return (int)div_up(chunks, l) * vec_elems; };
  while (lpr < 32 && acc_needed(lpr) > 32) lpr *= 2;
  if (acc_needed(lpr) > 32) {
    set_error("scatter: %lld output channels exceed the supported 1024 per row", (long long)c_out);
    return MN_ERR_UNSUPPORTED;
  }
  ScatterArgs<T> a{};
  a.buf = reinterpret_cast<const T *>(b.products);
  a.out = static_cast<T *>(out);
  a.target_masks = target_masks;
  a.T_rows = T_rows;
  a.num_offsets = L.n_buf;
  a.channels = (int)c_out;
  a.lanes_per_row = lpr;
  a.add_existing = L.shortcut ? 1 : 0;
  // shared memory: one 128-byte row of mask words per (warp, offset)
  const int n_off = std::max(L.n_buf, 1);
  const int warps_per_block = n_off <= 32 ? 8 : (n_off <= 64 ? 4 : 2);
  const int threads = warps_per_block * 32;
  const size_t smem = (size_t)warps_per_block * n_off * 32 * sizeof(int32_t);
  const int blocks =
      (int)std::min<int64_t>(kNumSMs * 64, div_up(div_up(T_rows, 32), warps_per_block));
  const int need = acc_needed(lpr);
#define MN_SCATTER(VE)                                                                          \
  do {                                                                                          \
    if (need <= 8) scatter_kernel<T, VE, 8><<<blocks, threads, smem, st>>>(a, L.plan);          \
    else if (need <= 16) scatter_kernel<T, VE, 16><<<blocks, threads, smem, st>>>(a, L.plan);   \
    else scatter_kernel<T, VE, 32><<<blocks, threads, smem, st>>>(a, L.plan);                   \
  } while (0)
  {
  LaunchScope scope("scatter_kernel", st);
  if (vec_elems * e == 16) { MN_SCATTER(16 / e); }
  else if (vec_elems * e == 8) { MN_SCATTER(8 / e); }
  else if (vec_elems * e == 4) { MN_SCATTER(4 / e); }
  else { MN_SCATTER(1); }
  }
#undef MN_SCATTER
  MN_CHECK_LAUNCH();
  return MN_OK;
}

mn_status run_scatter(const ConvLayout &L, const ConvBuffers &b, int64_t T_rows, int64_t c_out,
                      mn_dtype dtype, const int32_t *target_masks, int tile, void *out,
                      cudaStream_t st) {
  switch (dtype) {
    case MN_F32: return run_scatter_t<float>(L, b, T_rows, c_out, target_masks, tile, out, st);
    case MN_F16: return run_scatter_t<__half>(L, b, T_rows, c_out, target_masks, tile, out, st);
    default: return run_scatter_t<__nv_bfloat16>(L, b, T_rows, c_out, target_masks, tile, out, st);
  }
}

mn_status run_gemm(const ConvLayout &L, const ConvBuffers &b, const int32_t *sizes, int64_t O,
                   int64_t S, int64_t c_in, int64_t c_out, mn_dtype dtype, const void *sources,
                   const void *weights, const int32_t *order, void *out, int64_t out_rows,
                   int32_t *status_dev, cudaStream_t st) {
  const size_t e = dtype_size(dtype);
  GemmTable tab{};
  int np = 0;
  for (int o = 0; o < L.n_buf; o++) {
    if (sizes[o] <= 0) continue;
    tab.rows[np] = sizes[o];
    tab.weight_row[np] = o;
    tab.a[np] = b.gathered + (size_t)L.plan.row_begin[o] * c_in * e;
    tab.c[np] = b.products + (size_t)L.plan.row_begin[o] * c_out * e;
    tab.a_row[np] = L.plan.row_begin[o];
    tab.direct[np] = 0;
    np++;
  }
  if (L.shortcut && S > 0) {
    tab.rows[np] = (int32_t)S;
    tab.weight_row[np] = L.n_buf;
    tab.a[np] = sources;
    tab.c[np] = out;
    tab.a_row[np] = 0;
    tab.direct[np] = 1;
    np++;
  }
  tab.num_problems = np;
  if (np == 0) return MN_OK;

  bool handled = false;
  TcOperands ops;
  ops.gathered = L.total_rows > 0 ? b.gathered : nullptr;
  ops.gathered_rows = L.total_rows;
  ops.sources = S > 0 ? sources : nullptr;
  ops.source_rows = S;
  ops.products = L.total_rows > 0 ? b.products : nullptr;
  ops.out = out;
  ops.out_rows = out_rows;
  ops.weights_t = b.weights_t;
  ops.num_weights = (int)O;
  ops.status = status_dev;
  MN_RETURN_IF(launch_gemm_tc(tab, ops, (int)c_in, (int)c_out, dtype, weights, order, st, &handled));
  if (handled) return MN_OK;

  tab.tile_rows = kGemmTM;
  tab.tile_prefix[0] = 0;
  for (int p = 0; p < np; p++) tab.tile_prefix[p + 1] = tab.tile_prefix[p] + (int)div_up(tab.rows[p], kGemmTM);
  const dim3 grid(tab.tile_prefix[np], (unsigned)div_up(c_out, kGemmTN));
  {
  LaunchScope scope("gemm_simt_kernel", st);
  switch (dtype) {
    case MN_F32:
      gemm_simt_kernel<float><<<grid, 256, 0, st>>>(tab, static_cast<const float *>(weights), order,
                                                    (int)c_in, (int)c_out);
      break;
    case MN_F16:
      gemm_simt_kernel<__half><<<grid, 256, 0, st>>>(tab, static_cast<const __half *>(weights), order,
                                                     (int)c_in, (int)c_out);
      break;
    default:
      gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          tab, static_cast<const __nv_bfloat16 *>(weights), order, (int)c_in, (int)c_out);
      break;
  }
  }
  MN_CHECK_LAUNCH();
  return MN_OK;
}

mn_status check_conv_args(int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out,
                          mn_dtype dtype, const int32_t *sizes_host) {
  MN_CHECK_ARG(S >= 0 && T >= 0 && O >= 1 && O <= MN_MAX_OFFSETS,
               "conv: bad shape S=%lld T=%lld O=%lld", (long long)S, (long long)T, (long long)O);
  MN_CHECK_ARG(c_in >= 1 && c_out >= 1, "conv: channels must be positive");
  MN_CHECK_ARG(dtype == MN_F32 || dtype == MN_F16 || dtype == MN_BF16, "conv: unknown dtype %d", (int)dtype);
  MN_CHECK_ARG(sizes_host != nullptr, "conv: sizes_host is required");
  for (int64_t o = 0; o < O; o++)
    MN_CHECK_ARG(sizes_host[o] >= 0 && sizes_host[o] <= std::min(S, T),
                 "conv: size[%lld] = %d is outside [0, min(S, T)]", (long long)o, sizes_host[o]);
  return MN_OK;
}

}  // namespace
}  // namespace mn

using namespace mn;

namespace mn {
namespace {

// x[t, c] = relu?(x[t, c] * scale[c] + shift[c] + residual[t, c]), in place, 8 (16-bit) or 4
// (fp32) channels per thread
template <typename T, int kVecElems>
__global__ void __launch_bounds__(256)
epilogue_kernel(T *__restrict__ x, int64_t n_vec, int vec_per_row, const float *__restrict__ scale,
                const float *__restrict__ shift, const T *__restrict__ residual, int relu) {
  using V = typename Chunk<kVecElems * sizeof(T)>::type;
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += gsz) {
    const int c0 = (int)(i % vec_per_row) * kVecElems;
    V v = reinterpret_cast<V *>(x)[i];
    T *e = reinterpret_cast<T *>(&v);
    V rv{};
    if (residual != nullptr) rv = __ldg(reinterpret_cast<const V *>(residual) + i);
    const T *re = reinterpret_cast<const T *>(&rv);
#pragma unroll
    for (int k = 0; k < kVecElems; k++) {
      float f = to_f32(e[k]);
      if (scale != nullptr) f *= __ldg(scale + c0 + k);
      if (shift != nullptr) f += __ldg(shift + c0 + k);
      if (residual != nullptr) f += to_f32(re[k]);
      if (relu) f = fmaxf(f, 0.f);
      e[k] = from_f32<T>(f);
    }
    reinterpret_cast<V *>(x)[i] = v;
  }
}

template <typename T>
mn_status run_epilogue(void *x, int64_t rows, int64_t c, const float *scale, const float *shift,
                       const void *residual, int relu, cudaStream_t st) {
  constexpr int kVec = 16 / (int)sizeof(T);
  const bool vec_ok = c % kVec == 0 &&
                      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual)) & 15) == 0;
  const int64_t n = rows * c;
  if (vec_ok) {
    const int64_t n_vec = n / kVec;
    const int blocks = (int)std::min<int64_t>(kNumSMs * 16, div_up(n_vec, 256));
    MN_LAUNCH("epilogue_kernel", st,
              epilogue_kernel<T, kVec><<<blocks, 256, 0, st>>>(
                  static_cast<T *>(x), n_vec, (int)(c / kVec), scale, shift,
                  static_cast<const T *>(residual), relu));
  } else {
    const int blocks = (int)std::min<int64_t>(kNumSMs * 16, div_up(n, 256));
    MN_LAUNCH("epilogue_kernel", st,
              epilogue_kernel<T, 1><<<blocks, 256, 0, st>>>(static_cast<T *>(x), n, (int)c, scale,
                                                            shift, static_cast<const T *>(residual),
                                                            relu));
  }
  return MN_OK;
}

}  // namespace
}  // namespace mn

extern "C" mn_status mn_apply_epilogue(void *features, int64_t rows, int64_t channels,
                                       mn_dtype dtype, const float *scale, const float *shift,
                                       const void *residual, int relu, void *stream) {
  MN_CHECK_ARG(rows >= 0 && channels >= 1, "apply_epilogue: bad shape");
  if (rows == 0) return MN_OK;
  MN_CHECK_ARG(features != nullptr, "apply_epilogue: null features");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MN_F32: return run_epilogue<float>(features, rows, channels, scale, shift, residual, relu, st);
    case MN_F16: return run_epilogue<__half>(features, rows, channels, scale, shift, residual, relu, st);
    case MN_BF16:
      return run_epilogue<__nv_bfloat16>(features, rows, channels, scale, shift, residual, relu, st);
  }
  set_error("apply_epilogue: unknown dtype %d", (int)dtype);
  return MN_ERR_BAD_ARG;
}

extern "C" mn_status mn_dense_forward_simt(int64_t rows, int64_t c_in, int64_t c_out, mn_dtype dtype,
                                           const void *features, const void *weights,
                                           const float *scale, const float *shift,
                                           const void *residual, int relu, void *out,
                                           void *stream) {
  MN_CHECK_ARG(rows >= 0 && rows < (1ll << 31) && c_in >= 1 && c_out >= 1,
               "dense forward (FFMA): bad shape rows=%lld c_in=%lld c_out=%lld", (long long)rows,
               (long long)c_in, (long long)c_out);
  MN_CHECK_ARG(dtype == MN_F32 || dtype == MN_F16 || dtype == MN_BF16,
               "dense forward (FFMA): unknown dtype %d", (int)dtype);
  if (rows == 0) return MN_OK;
  MN_CHECK_ARG(features != nullptr && weights != nullptr && out != nullptr,
               "dense forward (FFMA): null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  GemmTable tab{};
  tab.num_problems = 1;
  tab.rows[0] = (int32_t)rows;
  tab.weight_row[0] = 0;
  tab.a[0] = features;
  tab.c[0] = out;
  tab.direct[0] = 1;
  tab.tile_rows = kGemmTM;
  tab.tile_prefix[0] = 0;
  tab.tile_prefix[1] = (int)div_up(rows, kGemmTM);
  const dim3 grid(tab.tile_prefix[1], (unsigned)div_up(c_out, kGemmTN));
  {
    LaunchScope scope("gemm_simt_kernel", st);
    switch (dtype) {
      case MN_F32:
        gemm_simt_kernel<float><<<grid, 256, 0, st>>>(tab, static_cast<const float *>(weights), nullptr,
                                                      (int)c_in, (int)c_out);
        break;
      case MN_F16:
        gemm_simt_kernel<__half><<<grid, 256, 0, st>>>(tab, static_cast<const __half *>(weights),
                                                       nullptr, (int)c_in, (int)c_out);
        break;
      default:
        gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
            tab, static_cast<const __nv_bfloat16 *>(weights), nullptr, (int)c_in, (int)c_out);
        break;
    }
  }
  MN_CHECK_LAUNCH();
  if (scale == nullptr && shift == nullptr && residual == nullptr && !relu) return MN_OK;
  return mn_apply_epilogue(out, rows, c_out, dtype, scale, shift, residual, relu, stream);
}

extern "C" mn_status mn_plan_buckets(const int32_t *sizes, int64_t O, int has_threshold,
                                     double threshold, int64_t *buckets_out, int64_t *cumsum_out,
                                     int64_t *num_buckets_out) {
  MN_CHECK_ARG(O >= 0 && (O == 0 || sizes != nullptr), "plan_buckets: bad sizes");
  MN_CHECK_ARG(buckets_out != nullptr && cumsum_out != nullptr && num_buckets_out != nullptr,
               "plan_buckets: null output");
  int64_t nb = 0;
  buckets_out[nb++] = 0;
  for (int64_t i = 0; i < O; i++) {
    const int64_t first = i;
    uint64_t actual = (uint64_t)sizes[i], summit = (uint64_t)sizes[i];
    for (; i + 1 < O; i++) {
      const uint64_t next = (uint64_t)sizes[i + 1];
      const uint64_t new_actual = actual + next, new_summit = std::max(summit, next);
      const uint64_t padded = new_summit * (uint64_t)(i + 2 - first);
      const double waste = (double)(padded - new_actual) / (double)new_actual;
      if (has_threshold && (threshold < 0 || waste > threshold)) break;
      actual = new_actual;
      summit = new_summit;
    }
    buckets_out[nb++] = i + 1;
  }
  cumsum_out[0] = 0;
  for (int64_t b = 0; b + 1 < nb; b++) {
    int64_t summit = 0;
    for (int64_t j = buckets_out[b]; j < buckets_out[b + 1]; j++) summit = std::max<int64_t>(summit, sizes[j]);
    for (int64_t j = buckets_out[b]; j < buckets_out[b + 1]; j++) cumsum_out[j + 1] = cumsum_out[j] + summit;
  }
  *num_buckets_out = nb - 1;
  return MN_OK;
}

extern "C" size_t mn_conv_workspace_bytes(const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                                          int64_t c_in, int64_t c_out, mn_dtype dtype,
                                          int allow_shortcut, int has_threshold, double threshold) {
  (void)has_threshold; (void)threshold;
  if (sizes_host == nullptr || O < 1 || O > MN_MAX_OFFSETS) return 0;
  const ConvLayout L = make_layout(sizes_host, O, S, T, allow_shortcut);
  const size_t e = dtype_size(dtype);
  const size_t rows = (size_t)std::max<int64_t>(L.total_rows, 1);
  size_t total = align_up(rows * c_in * e, 256) + align_up(rows * c_out * e, 256) + 1024;
  if (gemm_tc_supported((int)c_in, (int)c_out, dtype)) total += gemm_tc_workspace_bytes(O, c_in, c_out) + 256;
  return total;
}

extern "C" mn_status mn_conv_stage(int stage, int64_t S, int64_t T, int64_t O, int64_t c_in,
                                   int64_t c_out, mn_dtype dtype, const void *sources,
                                   const void *weights, const int32_t *source_masks,
                                   const int32_t *target_masks, const int32_t *order,
                                   const int32_t *sizes_host, int tile, int allow_shortcut,
                                   int has_threshold, double threshold, void *targets_out,
                                   int32_t *status_dev, void *ws_ptr, size_t ws_bytes,
                                   void *stream) {
  (void)has_threshold; (void)threshold;
  MN_RETURN_IF(check_conv_args(S, T, O, c_in, c_out, dtype, sizes_host));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const ConvLayout L = make_layout(sizes_host, O, S, T, allow_shortcut);
  ConvBuffers b{};
  MN_RETURN_IF(carve(L, O, c_in, c_out, dtype, ws_ptr, ws_bytes, &b));
  switch (stage) {
    case 0:
      MN_CHECK_ARG(sources != nullptr && source_masks != nullptr, "conv_stage: null pointer");
      return run_gather(L, b, S, c_in, dtype, sources, source_masks, tile, st);
    case 1:
      MN_CHECK_ARG(sources != nullptr && weights != nullptr && targets_out != nullptr, "conv_stage: null pointer");
      return run_gemm(L, b, sizes_host, O, S, c_in, c_out, dtype, sources, weights, order,
                      targets_out, T, status_dev, st);
    case 2:
      MN_CHECK_ARG(target_masks != nullptr && targets_out != nullptr, "conv_stage: null pointer");
      return run_scatter(L, b, T, c_out, dtype, target_masks, tile, targets_out, st);
    default:
      set_error("conv_stage: stage %d is not 0 (gather), 1 (gemm) or 2 (scatter)", stage);
      return MN_ERR_BAD_ARG;
  }
}

extern "C" mn_status mn_sparse_convolution_forward(
    int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
    const void *sources, const void *weights, const int32_t *source_masks,
    const int32_t *target_masks, const int32_t *order, const int32_t *sizes_host, int gather_tile,
    int scatter_tile, int allow_shortcut, int has_threshold, double threshold, void *targets_out,
    int32_t *status_dev, void *ws_ptr, size_t ws_bytes, void *stream) {
  (void)has_threshold; (void)threshold;
  MN_RETURN_IF(check_conv_args(S, T, O, c_in, c_out, dtype, sizes_host));
  if (T == 0) return MN_OK;
  MN_CHECK_ARG(weights != nullptr && targets_out != nullptr && source_masks != nullptr &&
                   target_masks != nullptr && (S == 0 || sources != nullptr),
               "conv: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const ConvLayout L = make_layout(sizes_host, O, S, T, allow_shortcut);
  ConvBuffers b{};
  MN_RETURN_IF(carve(L, O, c_in, c_out, dtype, ws_ptr, ws_bytes, &b));
  MN_RETURN_IF(run_gather(L, b, S, c_in, dtype, sources, source_masks, gather_tile, st));
  MN_RETURN_IF(run_gemm(L, b, sizes_host, O, S, c_in, c_out, dtype, sources, weights, order,
                        targets_out, T, status_dev, st));
  MN_RETURN_IF(run_scatter(L, b, T, c_out, dtype, target_masks, scatter_tile, targets_out, st));
  return MN_OK;
}
