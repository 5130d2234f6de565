// tiled_sum_reduce and the grid-barrier micro-kernel.
//
// tiled_sum_reduce: D[m,n] = sum_b (A[b,m,n] + B[b,m,n]) in fp32, the batch
// summed in order (bit-identical to the host loop of
// projects/tiled_sum_reduce/test.cu:13-25 in the reference project).  Replaces
// _tiled_sum_reduce_kernel (projects/tiled_sum_reduce/src.cu:11-50, one wave per
// 8x64 tile) and the producer/consumer variant _tsr_kernel
// (projects/tiled_sum_reduce_async/src.cu:99-177): the op is a pure HBM stream
// (8*b*m*n + 4*m*n bytes), so each thread owns four adjacent outputs and keeps
// eight 16-byte loads in flight; no shared-memory ring is needed to saturate
// the memory system, and the column-offset bug of the reference
// (src.cu:21, correct only for n = 64) does not carry over.
//
// globs: the reference's grid-barrier latency probe (projects/global_sync/
// src.cu:7-27): write, grid barrier, atomic decrement.  The barrier is the
// bounded one of sync.cuh instead of cooperative_groups::this_grid().sync().
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "host_util.h"
#include "sync.cuh"

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace reduce {

__device__ __forceinline__ float4 ldg_stream(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

constexpr int UNROLL = 4;

__global__ void __launch_bounds__(256) tsr_vec4_kernel(const float4* __restrict__ A, const float4* __restrict__ B,
                                                       float4* __restrict__ D, int b, size_t mn4) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < mn4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4* a = A + i;
        const float4* bb = B + i;
        int ib = 0;
        for (; ib + UNROLL <= b; ib += UNROLL) {
            float4 va[UNROLL], vb[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                va[u] = ldg_stream(a + static_cast<size_t>(u) * mn4);
                vb[u] = ldg_stream(bb + static_cast<size_t>(u) * mn4);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {   // batch order, one add per term like the host loop
                acc.x += va[u].x + vb[u].x;
                acc.y += va[u].y + vb[u].y;
                acc.z += va[u].z + vb[u].z;
                acc.w += va[u].w + vb[u].w;
            }
            a += static_cast<size_t>(UNROLL) * mn4;
            bb += static_cast<size_t>(UNROLL) * mn4;
        }
        for (; ib < b; ib++) {
            const float4 x = ldg_stream(a), y = ldg_stream(bb);
            acc.x += x.x + y.x; acc.y += x.y + y.y; acc.z += x.z + y.z; acc.w += x.w + y.w;
            a += mn4;
            bb += mn4;
        }
        D[i] = acc;
    }
}

__global__ void __launch_bounds__(256) tsr_scalar_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                         float* __restrict__ D, int b, size_t mn) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < mn;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float acc = 0.f;
        for (int ib = 0; ib < b; ib++) acc += A[static_cast<size_t>(ib) * mn + i] + B[static_cast<size_t>(ib) * mn + i];
        D[i] = acc;
    }
}

// ------------------------------------------------------------- grid barrier
__global__ void globs_kernel(unsigned* D, unsigned* words, int rounds, int* status) {
    // write, barrier, decrement - the reference's probe body, `rounds` times
    bool ok = true;
    for (int r = 0; r < rounds && ok; r++) {
        D[blockIdx.x] = 0;
        ok = grid_barrier(words, gridDim.x);
        if (ok) atomicDec(&D[blockIdx.x], 1u);
    }
    if (!ok && threadIdx.x == 0) report_timeout(status);
    grid_barrier_exit(words, gridDim.x);
}

// Barrier words, one pair per device, allocated (and zeroed) on first use.
static unsigned* barrier_words(int* err) {
    static unsigned* words[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { *err = RDB_CUDA_ERROR; return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    if (!words[dev]) {
        if (cudaMalloc(reinterpret_cast<void**>(&words[dev]), 256) != cudaSuccess ||
            cudaMemset(words[dev], 0, 256) != cudaSuccess) {
            *err = RDB_CUDA_ERROR;
            return nullptr;
        }
    }
    return words[dev];
}

int launch_globs(unsigned* D, unsigned* words, int blocks, int threads, int rounds, int* status, cudaStream_t stream) {
    void* args[] = {&D, &words, &rounds, &status};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(globs_kernel), dim3(blocks), dim3(threads),
                                                      args, 0, stream);
    if (e != cudaSuccess) {
        cudaGetLastError();      // do not leave the error for the next launch's check to trip over
        return RDB_CUDA_ERROR;
    }
    return RDB_SUCCESS;
}

// Blocks of `threads` threads of the probe kernel the current device can hold at
// once (a cooperative launch of more is refused); 0 when the query fails.
// Queries only - nothing is allocated.
static int globs_resident_blocks(int threads) {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, globs_kernel, threads, 0) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return sms * per_sm;
}

// ------------------------------------------------ allocation-free variant
// The barrier words of the probe normally sit in a buffer the library
// allocates on first use.  Some callers may not allocate at all once they are
// running: a host framework that owns every byte of device memory and hands
// plugins a fixed arena, or a latency-critical loop in which a device
// allocation (which synchronises the whole GPU) is unacceptable.  For them the
// same kernel can run on words that live in this file-scope array instead.
// Every GPU that loads the library holds these 256 bytes until the process
// exits.  Word 0/1: barrier arrivals / departures, word 2: status, rest unused.
constexpr int kNoAllocWords = 64;
constexpr int kNoAllocMaxBlocks = 1024;
constexpr long long kNoAllocMaxArrivals = 1ll << 30;   // the arrival word counts blocks x rounds per launch
static __device__ __align__(256) unsigned g_noalloc_scratch[kNoAllocWords];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a
// device address, so the address is looked up once per device (with that
// device current) and cached.  Nothing is allocated here.
static unsigned* noalloc_scratch(int* err) {
    static unsigned* ptr[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = RDB_CUDA_ERROR; return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    if (!ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            *err = RDB_CUDA_ERROR;
            return nullptr;
        }
        ptr[dev] = static_cast<unsigned*>(p);
    }
    return ptr[dev];
}

}  // namespace reduce
}  // namespace rdb

extern "C" {

int rdb_tiled_sum_reduce(const float* A, const float* B, float* D, int b, int m, int n, void* stream) {
    if (b < 0 || m < 1 || n < 1) return RDB_BAD_SHAPE;
    int err = 0;
    rdb::DeviceInfo* info = rdb::device_info(&err);
    if (!info) return err;
    const size_t mn = static_cast<size_t>(m) * n;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool vec = (mn % 4 == 0) && rdb::aligned16(A) && rdb::aligned16(B) && rdb::aligned16(D);
    const size_t work = vec ? mn / 4 : mn;
    size_t blocks = (work + 255) / 256;
    const size_t cap = static_cast<size_t>(info->sm_count) * 8;   // 8 resident blocks of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (vec)
        rdb::reduce::tsr_vec4_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(
            reinterpret_cast<const float4*>(A), reinterpret_cast<const float4*>(B), reinterpret_cast<float4*>(D), b, mn / 4);
    else
        rdb::reduce::tsr_scalar_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(A, B, D, b, mn);
    return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

int rdb_globs_n(uint32_t* D, int blocks, int threads, int rounds, void* stream) {
    if (blocks < 1 || threads < 1 || threads > 1024 || rounds < 1) return RDB_BAD_SHAPE;
    int err = 0;
    rdb::DeviceInfo* info = rdb::device_info(&err);
    if (!info) return err;
    if (blocks > info->sm_count * 8) return RDB_SIZE_ABOVE_LIMIT;
    unsigned* words = rdb::reduce::barrier_words(&err);
    if (!words) return err;
    return rdb::reduce::launch_globs(D, words, blocks, threads, rounds, info->status_dev,
                                     static_cast<cudaStream_t>(stream));
}

int rdb_globs(uint32_t* D, void* stream) { return rdb_globs_n(D, 2, 64, 1, stream); }

int rdb_globs_n_noalloc(uint32_t* D, int blocks, int threads, int rounds, void* stream) {
    using namespace rdb::reduce;
    if (blocks < 1 || threads < 1 || threads > 1024 || rounds < 1) return RDB_BAD_SHAPE;
    if (blocks > kNoAllocMaxBlocks || static_cast<long long>(blocks) * rounds > kNoAllocMaxArrivals) {
        fprintf(stderr,
                "rdb_globs_n_noalloc: %d blocks x %d rounds is beyond what the built-in scratch supports "
                "(at most %d blocks and %lld barrier arrivals per launch)\n",
                blocks, rounds, kNoAllocMaxBlocks, kNoAllocMaxArrivals);
        return RDB_SIZE_ABOVE_LIMIT;
    }
    const int resident = globs_resident_blocks(threads);
    if (resident > 0 && blocks > resident) {
        fprintf(stderr,
                "rdb_globs_n_noalloc: %d blocks of %d threads cannot be resident together on this device "
                "(at most %d): the barrier needs the whole grid on the GPU at once\n",
                blocks, threads, resident);
        return RDB_SIZE_ABOVE_LIMIT;
    }
    int err = 0;
    unsigned* words = noalloc_scratch(&err);
    if (!words) return err;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left (a timed-out barrier leaves
    // its counters mid-count): the two barrier words must start at zero.
    if (cudaMemsetAsync(words, 0, 2 * sizeof(unsigned), s) != cudaSuccess) return RDB_CUDA_ERROR;
    return launch_globs(D, words, blocks, threads, rounds, reinterpret_cast<int*>(words + 2), s);
}

int rdb_noalloc_status(void) {
    int err = 0;
    unsigned* words = rdb::reduce::noalloc_scratch(&err);
    if (!words) return err;
    if (cudaDeviceSynchronize() != cudaSuccess) return RDB_CUDA_ERROR;
    int st = 0;
    if (cudaMemcpy(&st, words + 2, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return RDB_CUDA_ERROR;
    if (st != 0 && cudaMemset(words + 2, 0, sizeof(int)) != cudaSuccess) return RDB_CUDA_ERROR;
    return st;
}

}  // extern "C"
