// Per-tensor FP8 quantiser: scale = amax/448 (1 for an all-zero tensor),
// q = e4m3fn_sat_rn(x / scale) - the step that precedes every GEMM of this
// library (the reference's drivers draw fp8 values directly and have no such
// step; the rule is the configuration text's, the conversion that of
// projects/common.cuh:103 in the reference project).  One cooperative kernel:
// every thread folds its share of |x| into a block maximum, blocks combine with
// atomicMax on the (non-negative) float bits, a bounded grid barrier follows,
// then every thread converts its share with the exact reciprocal-based
// division.  Scratch: one amax word and the two barrier words per device.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <mutex>

#include "fp8_codec.cuh"
#include "host_util.h"
#include "sync.cuh"

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace quant {

constexpr int kThreads = 256;

__device__ __forceinline__ float amax8(const uint4 v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        m = fmaxf(m, fabsf(__uint_as_float(w[j] << 16)));
        m = fmaxf(m, fabsf(__uint_as_float(w[j] & 0xFFFF0000u)));
    }
    return m;
}

__device__ __forceinline__ uint2 encode8(const uint4 v, const rdb::ar::BlockDivisor& d) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8], t[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
    d.div8(f, t);
    uint32_t o[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(t[4 * j], t[4 * j + 1]), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(make_float2(t[4 * j + 2], t[4 * j + 3]), __NV_SATFINITE, __NV_E4M3);
        o[j] = static_cast<uint32_t>(a) | (static_cast<uint32_t>(b) << 16);
    }
    return make_uint2(o[0], o[1]);
}

// The last block to leave puts the barrier words and the maximum back to zero
// for the next call (also after a timed-out barrier).
__device__ __forceinline__ void leave(unsigned* scratch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned left = atom_add_release_gpu(scratch + 1, 1u);
        if (left == gridDim.x - 1) {
            scratch[0] = 0;
            scratch[1] = 0;
            scratch[2] = 0;
            __threadfence();
        }
    }
}

__global__ void __launch_bounds__(kThreads)
quantize_per_tensor_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale_out,
                           size_t n, unsigned* scratch, int* status) {
    // scratch[0..1]: barrier words, scratch[2]: amax bits (zero at entry, reset at exit)
    const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t n8 = n / 8;
    float amax = 0.0f;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    size_t i0 = tid;
    for (; i0 + 3 * nthreads < n8; i0 += 4 * nthreads) {            // four loads in flight per thread
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = __ldg(x4 + i0 + u * nthreads);
#pragma unroll
        for (int u = 0; u < 4; u++) amax = fmaxf(amax, amax8(v[u]));
    }
    for (; i0 < n8; i0 += nthreads) amax = fmaxf(amax, amax8(__ldg(x4 + i0)));
    for (size_t i = n8 * 8 + tid; i < n; i += nthreads) amax = fmaxf(amax, fabsf(__bfloat162float(x[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0 && amax > 0.0f) atomicMax(scratch + 2, __float_as_uint(amax));   // non-negative floats order like uints
    if (!grid_barrier(scratch, gridDim.x)) {
        if (threadIdx.x == 0) report_timeout(status);
        leave(scratch);
        return;
    }
    const float s = rdb::ar::block_scale(__uint_as_float(ld_acquire_gpu(scratch + 2)));
    rdb::ar::BlockDivisor d;
    d.set(s);
    if (tid == 0) *scale_out = s;
    uint2* q2 = reinterpret_cast<uint2*>(q);
    // walk the tensor backwards: its tail is what the first pass left in L2
    size_t r = n8 / nthreads;                                  // full rounds; the partial one first
    if (r * nthreads + tid < n8) q2[r * nthreads + tid] = encode8(__ldg(x4 + r * nthreads + tid), d);
    for (; r >= 4; r -= 4) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = __ldg(x4 + (r - 1 - u) * nthreads + tid);
#pragma unroll
        for (int u = 0; u < 4; u++) q2[(r - 1 - u) * nthreads + tid] = encode8(v[u], d);
    }
    for (; r >= 1; r--) q2[(r - 1) * nthreads + tid] = encode8(__ldg(x4 + (r - 1) * nthreads + tid), d);
    for (size_t i = n8 * 8 + tid; i < n; i += nthreads) {
        const uint32_t one = static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(x)[i]);
        q[i] = static_cast<uint8_t>(encode8(make_uint4(one, 0u, 0u, 0u), d).x & 0xFF);
    }
    leave(scratch);   // everyone has read the maximum
}

static unsigned* scratch_words(int* err) {
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

}  // namespace quant
}  // namespace rdb

extern "C" int rdb_quantize_per_tensor(const uint16_t* x, uint8_t* q, float* scale, size_t n, void* stream) {
    if (n == 0) return RDB_BAD_SHAPE;
    if (!rdb::aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u)) return RDB_BAD_ALIGNMENT;
    int err = 0;
    rdb::DeviceInfo* info = rdb::device_info(&err);
    if (!info) return err;
    unsigned* scratch = rdb::quant::scratch_words(&err);
    if (!scratch) return err;
    size_t blocks = (n / 8 + rdb::quant::kThreads - 1) / rdb::quant::kThreads;
    const size_t cap = static_cast<size_t>(info->sm_count) * 4;     // co-resident: the kernel holds a grid barrier
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
    int* status = info->status_dev;
    void* args[] = {&xp, &q, &scale, &n, &scratch, &status};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(rdb::quant::quantize_per_tensor_kernel),
                                                      dim3(static_cast<unsigned>(blocks)), dim3(rdb::quant::kThreads), args, 0,
                                                      static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}
