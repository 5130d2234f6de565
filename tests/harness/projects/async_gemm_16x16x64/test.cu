// argv: m n k.  Unscaled fp32 output like the reference's driver
// (projects/async_gemm_16x16x64/test.cu in the reference project).
#include "common.cuh"

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int m = atoi(argv[1]), n = atoi(argv[2]), k = atoi(argv[3]);
    srand(0);
    auto hA = random_fp8(static_cast<size_t>(m) * k), hB = random_fp8(static_cast<size_t>(n) * k);
    std::vector<float> ref(static_cast<size_t>(m) * n);
    orc_gemm_fp8_f32(hA.data(), hB.data(), ref.data(), m, n, k);
    uint8_t *dA = to_device(hA), *dB = to_device(hB);
    float* dD = device_zeros<float>(static_cast<size_t>(m) * n);
    RDB_CHECK(rdb_dense_gemm_fp8_f32(dA, dB, dD, m, n, k, nullptr));
    CUDA_CHECK(cudaDeviceSynchronize());
    print_deltas(to_host(dD, static_cast<size_t>(m) * n), ref);
    return 0;
}
