// argv: m n k.
#include "common.cuh"
// tile of this project in the reference (its core.cu): the launcher applies the reference's shape rule
#define WARPTILE_M 16
#define WARPTILE_N 16
#define WARPTILE_K 64
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int m = atoi(argv[1]), n = atoi(argv[2]), k = atoi(argv[3]);
    auto hA = random_fp8(static_cast<size_t>(m) * k), hB = random_fp8(static_cast<size_t>(n) * k);
    uint8_t *dA = to_device(hA), *dB = to_device(hB);
    float* dD = device_zeros<float>(static_cast<size_t>(m) * n);
    bench_protocol(10, 50, [&](int) { async_gemm<float>(dA, dB, dD, m, n, k); });
    return 0;
}
