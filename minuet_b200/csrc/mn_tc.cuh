// PTX wrappers shared by the tensor-core kernels: mbarrier, TMA, tcgen05.
#pragma once

#include <cuda.h>

#include <algorithm>

#include "mn_common.cuh"

namespace mn {
namespace tc {

constexpr uint32_t kSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: false when the limit expired or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int32_t *status) {
  for (uint32_t spin = 0; spin < kSpinLimit; spin++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicOr(status, 4);
  return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, const void *src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map),
               "r"(x), "r"(y), "r"(smem_u32(src))
               : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle:
// rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                         // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                         // layout: 128-byte swizzle
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}


}  // namespace tc

// Shared-memory ring depth, TMEM columns and CTAs per SM of a tensor-core kernel.
// These layers are bound by memory latency, not by the tensor pipe (a 128-row tile
// of a 32-channel layer is 16 KB of traffic and a microsecond of dependent loads),
// so as many CTAs as fit share an SM, each with a short ring and only the TMEM
// columns its accumulators need.
struct TcSizing {
  int stages;
  int tmem_cols;      // power of two >= 32
  int ctas_per_sm;
  size_t smem_bytes;  // dynamic shared memory per CTA
};
inline TcSizing size_tc_kernel(int stage_bytes, int acc_cols, int max_stages, int max_ctas,
                               int extra_bytes = 0) {
  TcSizing z{};
  z.tmem_cols = 32;
  while (z.tmem_cols < acc_cols) z.tmem_cols *= 2;
  const int extra = 4 * 8192 + 1024 + extra_bytes;   // epilogue staging tiles + alignment slack
  for (int ctas = std::min(max_ctas, 512 / z.tmem_cols); ctas >= 1; ctas--) {
    const int budget = (227 * 1024) / ctas - 2048;   // static shared memory and reserve
    const int stages = std::min(max_stages, (budget - extra) / stage_bytes);
    if (stages >= 2 || ctas == 1) {
      z.ctas_per_sm = ctas;
      z.stages = std::max(2, ctas == 1 ? stages : std::min(stages, 4));
      break;
    }
  }
  z.smem_bytes = (size_t)z.stages * stage_bytes + extra;
  return z;
}

// ---- pair-list forward (mn_conv_pairs.cu) -------------------------------------------
constexpr int MN_MAX_PAIR_ROWS = 32;

// Which mask rows of a kernel map go through the product buffer, and where.
struct PairPlan {
  int64_t row_begin[MN_MAX_PAIR_ROWS + 1];   // first product row of mask row p (128-aligned)
  int32_t tile_prefix[MN_MAX_PAIR_ROWS + 1]; // first 128-row tile of mask row p
  int64_t total_rows;
  int32_t centre;                            // mask row handled as a dense product, or -1
  int32_t num_rows;                          // O
  uint32_t keep;                             // bit p set: mask row p has product rows
};
PairPlan make_pair_plan(const int32_t *sizes, int64_t O, int64_t S, int64_t T, int allow_shortcut);

// Epilogue of the dense (centre / 1x1x1) GEMM: out = relu?((acc + sum of the product
// rows named by the row's hit word) * scale + shift + residual), rounded once.
struct PairEpilogue {
  const float *scale;
  const float *shift;
  const void *residual;          // [T, c_out], feature dtype
  const uint32_t *bits;          // [T] hit words, or NULL: nothing to add
  const int32_t *target_masks;   // [O, T]
  const float *products;         // [total_rows, c_out]
  int64_t T;
  int64_t row_begin[MN_MAX_PAIR_ROWS + 1];
  uint32_t keep;
  int32_t relu;
};

// step 1: products[r, :] = sources[pair_src[r], :] @ weights_t[order[p(r)]]^T, fp32
mn_status launch_pair_products(const PairPlan &plan, int64_t S, int64_t c_in, int64_t c_out, bool bf16,
                               const void *sources, const void *weights_t, int O,
                               const int32_t *pair_src, const int32_t *order, float *products,
                               int32_t *status_dev, cudaStream_t st);
// step 2: out = epilogue(sources @ weights_t[order[centre]]^T)
mn_status launch_centre_gemm(int64_t rows, int64_t c_in, int64_t c_out, bool bf16, const void *sources,
                             const void *weights_t, int O, int centre, const int32_t *order,
                             const PairEpilogue &ep, void *out, int32_t *status_dev, cudaStream_t st);

// K-major operand map: dims (K, rows[, batch]), box (64, box_rows[, 1]), 128-byte swizzle,
// 16-bit elements (mn_gemm_tc.cu)
mn_status make_kmajor_map(CUtensorMap *map, const void *base, bool bf16, int64_t K, int64_t rows,
                          int64_t batch, int box_rows);
// weights [O, K, N] -> weights_t [O, N, K]
mn_status launch_transpose_weights(const void *weights, void *weights_t, int O, int c_in, int c_out,
                                   bool bf16, cudaStream_t st);

}  // namespace mn
