// Helpers shared by the harness drivers (test.cu / bench.cu of each project):
// error checking, host/device tensors drawn with rand() like the reference's
// drivers do (fp8 = saturating RN conversion of uniform[-1,1), float =
// uniform[-0.5,0.5); projects/common.cuh:90-105 in the reference project), an
// L2 flush between timed launches (projects/common.cuh:117-158) and the CPU
// oracle's prototypes (the checker; liboracle.so).
#pragma once

#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "rocm_dev_b200.h"

extern "C" {
uint8_t orc_e4m3fn_encode(float x);
float orc_bf16_decode(uint16_t h);
void orc_gemm_fp8_bf16(const uint8_t* A, const uint8_t* B, float scale_a, float scale_b, uint16_t* D, int M, int N, int K, int ldb);
void orc_gemm_fp8_f32(const uint8_t* A, const uint8_t* B, float* D, int M, int N, int K);
void orc_tiled_sum_reduce(const float* A, const float* B, float* D, int b, int m, int n);
void orc_deltas(const float* x, const float* ref, size_t n, float* max_delta, float* total_delta);
}

#define CUDA_CHECK(expr)                                                                          \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            fprintf(stderr, "%s failed: %s (%s:%d)\n", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(1);                                                                              \
        }                                                                                         \
    } while (0)

#define RDB_CHECK(expr)                                                                           \
    do {                                                                                          \
        int s_ = (expr);                                                                          \
        if (s_ != 0) {                                                                            \
            fprintf(stderr, "%s returned %d (%s)\n", #expr, s_, rdb_status_string(s_));           \
            exit(1);                                                                              \
        }                                                                                         \
    } while (0)

inline float unit_rand() { return static_cast<float>(rand()) / static_cast<float>(RAND_MAX); }

inline std::vector<uint8_t> random_fp8(size_t n) {
    std::vector<uint8_t> v(n);
    for (auto& x : v) x = orc_e4m3fn_encode(2.0f * (unit_rand() - 0.5f));
    return v;
}
inline std::vector<float> random_f32(size_t n) {
    std::vector<float> v(n);
    for (auto& x : v) x = unit_rand() - 0.5f;
    return v;
}

template <typename T>
T* to_device(const std::vector<T>& h) {
    T* d = nullptr;
    CUDA_CHECK(cudaMalloc(&d, h.size() * sizeof(T)));
    CUDA_CHECK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}
template <typename T>
T* device_zeros(size_t n) {
    T* d = nullptr;
    CUDA_CHECK(cudaMalloc(&d, n * sizeof(T)));
    CUDA_CHECK(cudaMemset(d, 0, n * sizeof(T)));
    return d;
}
template <typename T>
std::vector<T> to_host(const T* d, size_t n) {
    std::vector<T> h(n);
    CUDA_CHECK(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost));
    return h;
}

// Evicts L2 by writing a buffer twice its size.
struct CacheFlusher {
    char* buf = nullptr;
    size_t bytes = 0;
    CacheFlusher() {
        int dev = 0, l2 = 0;
        CUDA_CHECK(cudaGetDevice(&dev));
        CUDA_CHECK(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev));
        bytes = 2 * static_cast<size_t>(l2);
        CUDA_CHECK(cudaMalloc(&buf, bytes));
    }
    void flush() { CUDA_CHECK(cudaMemsetAsync(buf, 0, bytes)); }
    ~CacheFlusher() { cudaFree(buf); }
};

// Event-timed loop printing the reference's bench protocol: ", "-separated
// microsecond samples, "End of warmup, " before the first timed one.
template <typename F>
void bench_protocol(int warmups, int iterations, F&& launch) {
    CacheFlusher flusher;
    cudaEvent_t start, stop;
    CUDA_CHECK(cudaEventCreate(&start));
    CUDA_CHECK(cudaEventCreate(&stop));
    for (int it = 0; it < warmups + iterations; it++) {
        flusher.flush();
        CUDA_CHECK(cudaDeviceSynchronize());
        CUDA_CHECK(cudaEventRecord(start));
        launch(it);
        CUDA_CHECK(cudaEventRecord(stop));
        CUDA_CHECK(cudaEventSynchronize(stop));
        float ms = 0.f;
        CUDA_CHECK(cudaEventElapsedTime(&ms, start, stop));
        // fixed notation: the reference's parser cuts the last three characters of the output
        // (bench.py:49), which must leave a number behind
        if (it == warmups) printf("End of warmup, ");
        printf("%.4f, ", ms * 1000.0f);
    }
    int st = rdb_device_status();
    if (st != 0) { fprintf(stderr, "device status %d\n", st); exit(1); }
}

inline void print_deltas(const std::vector<float>& got, const std::vector<float>& ref) {
    float mx = 0.f, tot = 0.f;
    orc_deltas(got.data(), ref.data(), got.size(), &mx, &tot);
    printf("{\"max_delta\": %g, \"total_delta\": %g}", mx, tot);
}
