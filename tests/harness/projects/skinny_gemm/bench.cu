// argv: m n k.  Four distinct weight matrices rotate (projects/skinny_gemm/
// bench.cu:42,53-60 in the reference), L2 flushed before every timed launch.
#include "common.cuh"
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int m = atoi(argv[1]), n = atoi(argv[2]), k = atoi(argv[3]);
    const int batch = 4;
    auto hA = random_fp8(static_cast<size_t>(m) * k), hB = random_fp8(static_cast<size_t>(batch) * n * k);
    std::vector<float> one(1, 1.0f);
    uint8_t *dA = to_device(hA), *dB = to_device(hB);
    float* dOne = to_device(one);
    uint16_t* dD = device_zeros<uint16_t>(static_cast<size_t>(m) * n);
    bench_protocol(20, 100, [&](int it) {
        if (skinny_gemm_fastpath(dA, dB + static_cast<size_t>(it % batch) * n * k, dD, dOne, m, n, k) != SUCCESS) exit(1);
    });
    return 0;
}
