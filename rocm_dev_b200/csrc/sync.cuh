// Bounded grid-wide barrier on a counter in global memory.
//
// Contract: every block of the grid is resident (cooperative launch), the two
// counter words start at zero, and each block calls grid_barrier the same
// number of times.  The wait is bounded: when the budget runs out the barrier
// returns false (the caller records a status and leaves) instead of spinning
// forever.  grid_barrier_exit() puts the words back to zero once the last
// block has left, so that consecutive launches may use different grid sizes.
#pragma once

#include "ptx.cuh"

namespace rdb {

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned atom_add_release_gpu(unsigned* p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

// words[0]: arrivals (monotonic within a launch), words[1]: departures.
__device__ __forceinline__ bool grid_barrier(unsigned* words, unsigned nblocks) {
    __shared__ int ok_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned old = atom_add_release_gpu(words, 1u);
        const unsigned target = old - old % nblocks + nblocks;
        bool ok = true;
        if (ld_acquire_gpu(words) < target) {
            const uint64_t t0 = globaltimer_ns(), budget = wait_budget_ns();
            unsigned spins = 0;
            while (ld_acquire_gpu(words) < target) {
                if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > budget) { ok = false; break; }
            }
        }
        ok_s = ok ? 1 : 0;
    }
    __syncthreads();
    return ok_s != 0;
}

// Call once per block after its last grid_barrier of the launch.
__device__ __forceinline__ void grid_barrier_exit(unsigned* words, unsigned nblocks) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned left = atom_add_release_gpu(words + 1, 1u);
        if (left == nblocks - 1) {          // everyone has passed every barrier: reset for the next launch
            words[0] = 0;
            words[1] = 0;
            __threadfence();
        }
    }
}

}  // namespace rdb
