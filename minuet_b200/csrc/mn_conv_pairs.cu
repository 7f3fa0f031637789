// Pair-list forward pass of a sparse convolution on SPARSE kernel maps, fp16/bf16.
//
// The reference gathers every (source, target) pair row into a padded buffer,
// multiplies bucket by bucket and scatters the products back, with one dense
// GEMM for the centre offset (csrc/minuet/cuda/functions/sparse_convolution.cu:
// 505-661); its gather and scatter kernels scan one mask row per offset for every
// source / target row (kernels/padded_gather_warp_optimized.cuh:11-63,
// padded_scatter_warp_optimized.cuh:11-64).  On the maps of outdoor scans nine
// tenths of those mask words are -1.  Here the masks are only touched where a
// pair exists: the map build leaves one hit word per row (bit p <=> mask row p
// has an entry), from which
//   pair_list_kernel   builds, once per kernel map, the source row of every
//                      product row (mask row p owns the 128-aligned block
//                      [row_begin[p], row_begin[p] + size[p]));
//   step 1             is the fused implicit-GEMM kernel run over PRODUCT rows:
//                      A rows are fetched through the pair list, the products
//                      leave in fp32;
//   step 2             is the tensor-core GEMM of the centre offset over the
//                      input rows themselves (TMA-fed), whose epilogue adds, per
//                      output row, the product rows its hit word names, then the
//                      folded BatchNorm / bias, the residual and the ReLU, and
//                      rounds ONCE to 16 bits.  Without a centre offset (strided
//                      and transposed layers) a scatter kernel plays that role.
// Pair rows cross HBM once in fp32 instead of four times in 16 bits, the output
// is written once, and no mask row is scanned.
#include "mn_tc.cuh"

#include <algorithm>

namespace mn {

namespace {

constexpr int kPairAlign = 128;   // product rows of one mask row start on a GEMM tile boundary

// pair_src[row_begin[p] + source_masks[p, s]] = s for every set bit p of bits[s]
__global__ void __launch_bounds__(256)
pair_list_kernel(const int32_t *__restrict__ source_masks, const uint32_t *__restrict__ bits,
                 int64_t S, uint32_t keep, const __grid_constant__ PairPlan plan,
                 int32_t *__restrict__ pair_src) {
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; s < S; s += gsz) {
    uint32_t w = __ldg(bits + s) & keep;
    while (w != 0u) {
      const int p = __ffs(w) - 1;
      w &= w - 1u;
      const int m = __ldg(source_masks + (int64_t)p * S + s);
      if (m >= 0) pair_src[plan.row_begin[p] + m] = (int32_t)s;
    }
  }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// out[t, :] = epilogue(sum over the set bits p of bits[t] of products[row_begin[p] +
// target_masks[p, t], :]) for layers without a centre offset.  Eight channels per
// thread, the threads of a row next to each other.
template <typename T>
__global__ void __launch_bounds__(256)
pair_scatter_kernel(const float *__restrict__ products, const int32_t *__restrict__ target_masks,
                    const uint32_t *__restrict__ bits, int64_t T_rows, int c_out, uint32_t keep,
                    const __grid_constant__ PairPlan plan, const float *__restrict__ scale,
                    const float *__restrict__ shift, const T *__restrict__ residual, int relu,
                    T *__restrict__ out) {
  const int chunks = c_out >> 3;   // c_out is a multiple of 8
  const int64_t total = T_rows * chunks;
  const int64_t gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gsz) {
    const int64_t t = i / chunks;
    const int c = (int)(i - t * chunks) << 3;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint32_t w = __ldg(bits + t) & keep;
    while (w != 0u) {
      const int p = __ffs(w) - 1;
      w &= w - 1u;
      const int m = __ldg(target_masks + (int64_t)p * T_rows + t);
      if (m < 0) continue;
      const float4 *src = reinterpret_cast<const float4 *>(products + (plan.row_begin[p] + m) * c_out + c);
      const float4 a = __ldg(src), b = __ldg(src + 1);
      f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
      f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
    }
    if (scale != nullptr) {
#pragma unroll
      for (int k = 0; k < 8; k++) f[k] *= __ldg(scale + c + k);
    }
    if (shift != nullptr) {
#pragma unroll
      for (int k = 0; k < 8; k++) f[k] += __ldg(shift + c + k);
    }
    if (residual != nullptr) {
      const uint4 rv = __ldg(reinterpret_cast<const uint4 *>(residual + t * c_out + c));
      const T *r = reinterpret_cast<const T *>(&rv);
#pragma unroll
      for (int k = 0; k < 8; k++) f[k] += to_f32<T>(r[k]);
    }
    uint4 packed;
    T *o = reinterpret_cast<T *>(&packed);
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = from_f32<T>(relu ? fmaxf(f[k], 0.f) : f[k]);
    *reinterpret_cast<uint4 *>(out + t * c_out + c) = packed;
  }
}

}  // namespace

// Which mask rows go through the product buffer and where their rows start.
PairPlan make_pair_plan(const int32_t *sizes, int64_t O, int64_t S, int64_t T, int allow_shortcut) {
  PairPlan plan{};
  plan.centre = (allow_shortcut && O > 0 && sizes[O - 1] == T && sizes[O - 1] == S) ? (int)O - 1 : -1;
  plan.num_rows = (int)O;
  int64_t row = 0;
  int tiles = 0;
  for (int p = 0; p < MN_MAX_PAIR_ROWS; p++) {
    plan.row_begin[p] = row;
    plan.tile_prefix[p] = tiles;
    if (p < O && p != plan.centre) {
      const int64_t rows = (int64_t)align_up((size_t)sizes[p], kPairAlign);
      row += rows;
      tiles += (int)(rows / kPairAlign);
    }
  }
  plan.row_begin[MN_MAX_PAIR_ROWS] = row;
  plan.tile_prefix[MN_MAX_PAIR_ROWS] = tiles;
  plan.total_rows = row;
  plan.keep = 0u;
  for (int p = 0; p < O; p++)
    if (p != plan.centre && sizes[p] > 0) plan.keep |= 1u << p;
  return plan;
}

}  // namespace mn

using namespace mn;

extern "C" int mn_pairs_supported(int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype) {
  return mn_implicit_supported(O, c_in, c_out, dtype);
}

extern "C" int64_t mn_pair_rows(const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                                int allow_shortcut) {
  if (sizes_host == nullptr || O < 1 || O > MN_MAX_PAIR_ROWS) return 0;
  return make_pair_plan(sizes_host, O, S, T, allow_shortcut).total_rows;
}

extern "C" mn_status mn_build_pair_list(const int32_t *source_masks, const uint32_t *source_bits,
                                        const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                                        int allow_shortcut, int32_t *pair_src_out, void *stream) {
  MN_CHECK_ARG(O >= 1 && O <= MN_MAX_PAIR_ROWS, "pair list: %lld offsets (supported: 1..%d)",
               (long long)O, MN_MAX_PAIR_ROWS);
  MN_CHECK_ARG(S >= 0 && T >= 0 && sizes_host != nullptr, "pair list: bad arguments");
  for (int64_t p = 0; p < O; p++)
    MN_CHECK_ARG(sizes_host[p] >= 0 && sizes_host[p] <= std::min(S, T), "pair list: bad size");
  const PairPlan plan = make_pair_plan(sizes_host, O, S, T, allow_shortcut);
  if (plan.total_rows == 0) return MN_OK;
  MN_CHECK_ARG(source_masks != nullptr && source_bits != nullptr && pair_src_out != nullptr,
               "pair list: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // padding rows read no source
  MN_CHECK_CUDA(cudaMemsetAsync(pair_src_out, 0xff, sizeof(int32_t) * plan.total_rows, st));
  const int blocks = (int)std::min<int64_t>(kNumSMs * 8, div_up(S, 256));
  MN_LAUNCH("pair_list_kernel", st,
            pair_list_kernel<<<blocks, 256, 0, st>>>(source_masks, source_bits, S, plan.keep, plan,
                                                     pair_src_out));
  return MN_OK;
}

extern "C" size_t mn_pairs_workspace_bytes(const int32_t *sizes_host, int64_t O, int64_t S, int64_t T,
                                           int64_t c_in, int64_t c_out, int allow_shortcut) {
  if (sizes_host == nullptr || O < 1 || O > MN_MAX_PAIR_ROWS) return 0;
  const PairPlan plan = make_pair_plan(sizes_host, O, S, T, allow_shortcut);
  return align_up((size_t)std::max<int64_t>(plan.total_rows, 1) * c_out * sizeof(float), 1024) +
         align_up((size_t)O * c_in * c_out * 2, 1024) + 2048;
}

extern "C" mn_status mn_sparse_convolution_forward_pairs(
    int64_t S, int64_t T, int64_t O, int64_t c_in, int64_t c_out, mn_dtype dtype,
    const void *sources, const void *weights, const void *weights_t_in,
    const int32_t *target_masks, const uint32_t *target_bits, const int32_t *pair_src,
    const int32_t *order, const int32_t *sizes_host, int allow_shortcut, const float *scale,
    const float *shift, const void *residual, int relu, void *targets_out, int32_t *status_dev,
    void *ws_ptr, size_t ws_bytes, void *stream) {
  if (!mn_pairs_supported(O, c_in, c_out, dtype)) {
    set_error("pair-list forward: needs fp16/bf16, at most 32 offsets, channels multiple of 8, "
              "c_out <= 256 (got O=%lld c_in=%lld c_out=%lld dtype=%d)", (long long)O,
              (long long)c_in, (long long)c_out, (int)dtype);
    return MN_ERR_UNSUPPORTED;
  }
  MN_CHECK_ARG(S >= 0 && T >= 0 && T < (1ll << 31) && S < (1ll << 31) && sizes_host != nullptr,
               "pair-list forward: bad sizes");
  for (int64_t p = 0; p < O; p++)
    MN_CHECK_ARG(sizes_host[p] >= 0 && sizes_host[p] <= std::min(S, T),
                 "pair-list forward: size[%lld] = %d is outside [0, min(S, T)]", (long long)p, sizes_host[p]);
  if (T == 0) return MN_OK;
  MN_CHECK_ARG((weights != nullptr || weights_t_in != nullptr) && target_masks != nullptr &&
                   target_bits != nullptr && targets_out != nullptr && status_dev != nullptr &&
                   (S == 0 || sources != nullptr), "pair-list forward: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == MN_BF16;
  const PairPlan plan = make_pair_plan(sizes_host, O, S, T, allow_shortcut);
  MN_CHECK_ARG(plan.total_rows == 0 || pair_src != nullptr, "pair-list forward: null pair list");
  Workspace ws(ws_ptr, ws_bytes);
  float *products = ws.take<float>((size_t)std::max<int64_t>(plan.total_rows, 1) * c_out);
  const void *weights_t = weights_t_in;
  if (weights_t == nullptr) {
    char *mine = ws.take<char>(align_up((size_t)O * c_in * c_out * 2, 1024));
    MN_CHECK_WS(ws);
    MN_RETURN_IF(launch_transpose_weights(weights, mine, (int)O, (int)c_in, (int)c_out, bf16, st));
    weights_t = mine;
  }
  MN_CHECK_WS(ws);

  // step 1: products of the mask rows that go through the buffer
  if (plan.total_rows > 0)
    MN_RETURN_IF(launch_pair_products(plan, S, c_in, c_out, bf16, sources, weights_t, (int)O, pair_src,
                                      order, products, status_dev, st));

  PairEpilogue ep{};
  ep.scale = scale; ep.shift = shift; ep.residual = residual; ep.relu = relu ? 1 : 0;
  ep.bits = target_bits; ep.target_masks = target_masks; ep.products = products;
  ep.T = T; ep.keep = plan.keep;
  for (int p = 0; p <= MN_MAX_PAIR_ROWS; p++) ep.row_begin[p] = plan.row_begin[p];
  if (plan.centre >= 0) {
    // step 2: centre product over the input rows, the other products added in its epilogue
    return launch_centre_gemm(S, c_in, c_out, bf16, sources, weights_t, (int)O, plan.centre, order,
                              ep, targets_out, status_dev, st);
  }
  const int64_t total = T * (c_out / 8);
  const int blocks = (int)std::min<int64_t>(kNumSMs * 16, div_up(total, 256));
  if (bf16) {
    MN_LAUNCH("pair_scatter_kernel", st,
              pair_scatter_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
                  products, target_masks, target_bits, T, (int)c_out, plan.keep, plan, scale, shift,
                  static_cast<const __nv_bfloat16 *>(residual), relu ? 1 : 0,
                  static_cast<__nv_bfloat16 *>(targets_out)));
  } else {
    MN_LAUNCH("pair_scatter_kernel", st,
              pair_scatter_kernel<__half><<<blocks, 256, 0, st>>>(
                  products, target_masks, target_bits, T, (int)c_out, plan.keep, plan, scale, shift,
                  static_cast<const __half *>(residual), relu ? 1 : 0,
                  static_cast<__half *>(targets_out)));
  }
  return MN_OK;
}

// A dense [rows, c_in] x [c_in, c_out] product with the fused epilogue on the
// tensor cores: the 1x1x1 convolution (minuet/nn/convolutions.py:448-454 uses
// torch.mm for it).
extern "C" int mn_dense_supported(int64_t c_in, int64_t c_out, mn_dtype dtype) {
  return (dtype == MN_F16 || dtype == MN_BF16) && c_in >= 8 && c_in % 8 == 0 && c_out >= 2 &&
         c_out % 2 == 0 && c_out <= 256;
}

extern "C" size_t mn_dense_workspace_bytes(int64_t c_in, int64_t c_out) {
  return align_up((size_t)c_in * c_out * 2, 1024) + 1024;
}

extern "C" mn_status mn_dense_forward(int64_t rows, int64_t c_in, int64_t c_out, mn_dtype dtype,
                                      const void *features, const void *weights,
                                      const void *weights_t_in, const float *scale,
                                      const float *shift, const void *residual, int relu,
                                      void *out, int32_t *status_dev, void *ws_ptr, size_t ws_bytes,
                                      void *stream) {
  if (!mn_dense_supported(c_in, c_out, dtype)) {
    set_error("dense forward: needs fp16/bf16, c_in a multiple of 8, c_out even and <= 256 (got "
              "c_in=%lld c_out=%lld dtype=%d)", (long long)c_in, (long long)c_out, (int)dtype);
    return MN_ERR_UNSUPPORTED;
  }
  MN_CHECK_ARG(rows >= 0 && rows < (1ll << 31), "dense forward: bad row count");
  if (rows == 0) return MN_OK;
  MN_CHECK_ARG(features != nullptr && (weights != nullptr || weights_t_in != nullptr) &&
                   out != nullptr && status_dev != nullptr, "dense forward: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == MN_BF16;
  Workspace ws(ws_ptr, ws_bytes);
  const void *weights_t = weights_t_in;
  if (weights_t == nullptr) {
    char *mine = ws.take<char>(align_up((size_t)c_in * c_out * 2, 1024));
    MN_CHECK_WS(ws);
    MN_RETURN_IF(launch_transpose_weights(weights, mine, 1, (int)c_in, (int)c_out, bf16, st));
    weights_t = mine;
  }
  PairEpilogue ep{};
  ep.scale = scale; ep.shift = shift; ep.residual = residual; ep.relu = relu ? 1 : 0;
  ep.T = rows;
  return launch_centre_gemm(rows, c_in, c_out, bf16, features, weights_t, 1, 0, nullptr, ep, out,
                            status_dev, st);
}

extern "C" mn_status mn_transpose_weights(const void *weights, int64_t O, int64_t c_in, int64_t c_out,
                                          mn_dtype dtype, void *weights_t_out, void *stream) {
  MN_CHECK_ARG(dtype == MN_F16 || dtype == MN_BF16, "transpose weights: fp16/bf16 only");
  MN_CHECK_ARG(O >= 1 && c_in >= 1 && c_out >= 1 && weights != nullptr && weights_t_out != nullptr,
               "transpose weights: bad arguments");
  return launch_transpose_weights(weights, weights_t_out, (int)O, (int)c_in, (int)c_out,
                                  dtype == MN_BF16, static_cast<cudaStream_t>(stream));
}
