// Grid-wide helpers for kernels whose blocks are all resident at once
// (cooperative launches): a bounded, self-resetting barrier and the launch
// helper that sizes such a grid.
//
// The barrier state lives in the caller's control block (see MN_CTRL_* in the
// public header): an arrival count and several copies of a generation word on
// cache lines of their own.  A block reads its copy of the generation, arrives
// on the count, and the last arriver resets the count and bumps every copy, so
// the state is clean again after every barrier and survives from launch to
// launch.  (With count and generation on one line, a few hundred polling blocks
// delayed the arrivals by several microseconds.)  Every wait is
// bounded: when the limit expires the block sets MN_STATUS_GRID_TIMEOUT in the
// status word and carries on (its results are then invalid, but the kernel
// ends and the context stays usable).
#pragma once

#include "mn_common.cuh"

namespace mn {

constexpr unsigned kGridSpinLimit = 1u << 21;   // polls; each backs off ~100 ns

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_u32(unsigned *p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// All threads of all blocks of a cooperative grid must call this the same
// number of times.  ctrl points at the control block.
__device__ __forceinline__ void grid_barrier(int32_t *ctrl, unsigned num_blocks) {
  unsigned *count = reinterpret_cast<unsigned *>(ctrl + MN_CTRL_BARRIER_COUNT);
  volatile unsigned *gen = reinterpret_cast<volatile unsigned *>(ctrl + MN_CTRL_BARRIER_GEN) +
                           32u * (blockIdx.x % MN_CTRL_GEN_COPIES);
  // the generation cannot advance before this block has arrived, so it can be read
  // ahead of the block-wide barrier (its latency then overlaps the stragglers)
  unsigned my_gen = 0;
  if (threadIdx.x == 0) my_gen = *gen;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();   // release: the block's writes are visible before it arrives
    const unsigned arrived = atomicAdd(count, 1u);
    if (arrived == num_blocks - 1) {
      *count = 0u;
      __threadfence();   // one fence, then plain stores: a release per copy costs a fence each
      volatile unsigned *all = reinterpret_cast<volatile unsigned *>(ctrl + MN_CTRL_BARRIER_GEN);
#pragma unroll
      for (int k = 0; k < MN_CTRL_GEN_COPIES; k++) all[32 * k] = my_gen + 1u;
    } else {
      unsigned spins = 0;
      while (*gen == my_gen) {
        if (++spins > kGridSpinLimit) {
          atomicOr(ctrl + MN_CTRL_STATUS, MN_STATUS_GRID_TIMEOUT);
          break;
        }
        __nanosleep(64);
      }
    }
    __threadfence();   // acquire: later reads of this block see what the others wrote
  }
  __syncthreads();
}

// Largest grid of `kernel` (block size `threads`, `smem` dynamic bytes) whose
// blocks are all resident at once on the current device; 0 on error.
template <typename Kernel>
inline int max_coresident_blocks(Kernel kernel, int threads, size_t smem) {
  int device = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess)
    return 0;
  return sms * per_sm;
}

}  // namespace mn
