// Source-level face of the library: the reference's launcher names and
// argument lists over the C ABI of rocm_dev_b200.h, for drivers that include a
// launcher and call it directly (the reference's test.cu / bench.cu do:
// projects/skinny_gemm/test.cu:2,82).  Header-only; compile with nvcc and link
// librocm_dev_b200.so.
//
//   reference launcher                                        file:line (reference project)
//   int  skinny_gemm_fastpath(A, B, D, scale_tensor, m, n, k) projects/skinny_gemm/skinny_gemm_caller.cu:343-346
//   int  skinny_gemm(A, B, D, scale_tensor, m, n, k, b_stride, split_k, A_producers, B_producers,
//                    consumers, b_lanes, qsize, op_m, ops, stream)        same file :20-43
//   void async_gemm<T>(A, B, D, m, n, k)                      projects/async_gemm_16x16x64/src.cu:54-62 (and the
//                                                             blanes / sparse projects' sparse_k.cu)
//   void tiled_sum_reduce(A, B, D, b, m, n)                   projects/tiled_sum_reduce/src.cu:52-59
//   void globs(uint* D)                                       projects/global_sync/src.cu:15
//
// Conventions kept: all pointers are device pointers owned by the caller, the
// calls are asynchronous on stream 0 (skinny_gemm takes a stream), the skinny
// launchers return SkinnyGemmReturnCode 0..6 with the reference's numbering and
// print a message on std::cerr, async_gemm prints the reference's message and
// exits on a shape its project's tile does not divide, tiled_sum_reduce only
// warns.  The tile rule is applied when the including file defines WARPTILE_M /
// WARPTILE_N / WARPTILE_K the way the reference's core.cu files do.
// Differences forced by the target: fp8 bytes are OCP e4m3fn, the skinny
// GEMM's D is bf16 (the reference's half) and every D is overwritten instead of
// accumulated into, so it need not be zeroed.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <iostream>
#include <type_traits>

#include "rocm_dev_b200.h"

using fp8 = unsigned char;          // the reference's __hip_fp8_storage_t (projects/common.cuh:9)
#ifndef RDB_COMPAT_NO_UINT
typedef unsigned int uint;
#endif

enum SkinnyGemmReturnCode {
    SUCCESS = 0,
    M_ABOVE_WARPTILE_M = 1,
    N_NOT_EVEN = 2,
    K_NOT_DIVISIBLE_BY_WARPTILE_K = 3,
    TOO_MANY_WARPS = 4,
    QSIZE_TOO_SMALL = 5,
    INVALID_CONFIG = 6
};

namespace rdb_compat {

// The second per-tensor scale of the new ABI: the reference has one scale, so
// the wrappers pass a device-resident 1.0f (one word per device, made on first use).
inline const float* device_one() {
    static float* one[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!one[dev]) {
        const float v = 1.0f;
        if (cudaMalloc(reinterpret_cast<void**>(&one[dev]), sizeof(float)) != cudaSuccess ||
            cudaMemcpy(one[dev], &v, sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
            return nullptr;
    }
    return one[dev];
}

inline int report(int code, const char* who) {
    if (code != 0) std::cerr << who << ": " << rdb_status_string(code) << " (" << code << ")" << std::endl;
    return code;
}

template <class T>
struct is_bf16_storage : std::integral_constant<bool, std::is_same<T, __nv_bfloat16>::value || std::is_same<T, uint16_t>::value> {};

}  // namespace rdb_compat

template <class OUT>
inline int skinny_gemm_fastpath(const fp8* __restrict__ A, const fp8* __restrict__ B, OUT* __restrict__ D,
                                const float* scale_tensor, const int m, const int n, const int k) {
    static_assert(rdb_compat::is_bf16_storage<OUT>::value,
                  "D holds bf16 here (the reference writes fp16): declare it as __nv_bfloat16 (#define OUTD __nv_bfloat16)");
    return rdb_compat::report(rdb_skinny_gemm_fp8(A, B, scale_tensor, rdb_compat::device_one(), reinterpret_cast<uint16_t*>(D),
                                                  m, n, k, k, nullptr),
                              "skinny_gemm_fastpath");
}

template <class OUT>
inline int skinny_gemm(const fp8* __restrict__ A, const fp8* __restrict__ B, OUT* __restrict__ D, const float* scale_tensor,
                       const int m, const int n, const int k, const int b_stride, const int split_k, const int A_producers,
                       const int B_producers, const int consumers, const int b_lanes, const int qsize, const int op_m,
                       const int ops, cudaStream_t stream) {
    static_assert(rdb_compat::is_bf16_storage<OUT>::value,
                  "D holds bf16 here (the reference writes fp16): declare it as __nv_bfloat16 (#define OUTD __nv_bfloat16)");
    return rdb_compat::report(
        rdb_skinny_gemm_fp8_hinted(A, B, scale_tensor, rdb_compat::device_one(), reinterpret_cast<uint16_t*>(D), m, n, k, b_stride,
                                   split_k, A_producers, B_producers, consumers, b_lanes, qsize, op_m, ops, stream),
        "skinny_gemm");
}

template <typename out_dtype>
inline void async_gemm(const fp8* __restrict__ A, const fp8* __restrict__ B, out_dtype* __restrict__ D, const int m, const int n,
                       const int k) {
#if defined(WARPTILE_M) && defined(WARPTILE_N) && defined(WARPTILE_K)
    if ((m % WARPTILE_M != 0) || (n % WARPTILE_N != 0) || (k % WARPTILE_K != 0)) {
        std::cerr << "Either m, n or k is not divisible by the corresponding WARPTILE_ :" << m << ", " << n << ", " << k << std::endl;
        exit(1);
    }
#endif
    int code;
    if (std::is_same<out_dtype, float>::value) {
        code = rdb_dense_gemm_fp8_f32(A, B, reinterpret_cast<float*>(D), m, n, k, nullptr);             // unscaled fp32
    } else {
        static_assert(std::is_same<out_dtype, float>::value || rdb_compat::is_bf16_storage<out_dtype>::value,
                      "async_gemm writes fp32 (the reference's output) or bf16");
        code = rdb_dense_gemm_fp8(A, B, rdb_compat::device_one(), rdb_compat::device_one(), reinterpret_cast<uint16_t*>(D), m, n, k,
                                  nullptr);
    }
    if (rdb_compat::report(code, "async_gemm") != 0) exit(1);
}

inline void tiled_sum_reduce(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ D, const int b,
                             const int m, const int n) {
#if defined(WARPTILE_M) && defined(WARPTILE_N)
    if ((m % WARPTILE_M != 0) || (n % WARPTILE_N != 0))
        std::cerr << "Either m or n is not divisible by the corresponding WARPTILE_" << std::endl;   // the reference goes on too
#endif
    rdb_compat::report(rdb_tiled_sum_reduce(A, B, D, b, m, n, nullptr), "tiled_sum_reduce");
}

inline void globs(uint* D) { rdb_compat::report(rdb_globs(D, nullptr), "globs"); }
