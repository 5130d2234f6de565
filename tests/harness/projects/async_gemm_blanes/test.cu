// argv: m n k.  Unscaled fp32 output like the reference's driver
// (projects/async_gemm_16x16x64/test.cu in the reference project).
#include "common.cuh"
// tile of this project in the reference (its core.cu): the launcher applies the reference's shape rule
#define WARPTILE_M 16
#define WARPTILE_N 48
#define WARPTILE_K 64
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int m = atoi(argv[1]), n = atoi(argv[2]), k = atoi(argv[3]);
    srand(0);
    auto hA = random_fp8(static_cast<size_t>(m) * k), hB = random_fp8(static_cast<size_t>(n) * k);
    std::vector<float> ref(static_cast<size_t>(m) * n);
    orc_gemm_fp8_f32(hA.data(), hB.data(), ref.data(), m, n, k);
    uint8_t *dA = to_device(hA), *dB = to_device(hB);
    float* dD = device_zeros<float>(static_cast<size_t>(m) * n);
    async_gemm<float>(dA, dB, dD, m, n, k);
    CUDA_CHECK(cudaDeviceSynchronize());
    print_deltas(to_host(dD, static_cast<size_t>(m) * n), ref);
    return 0;
}
