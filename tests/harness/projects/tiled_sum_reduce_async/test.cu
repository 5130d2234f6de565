// argv: b m n (projects/tiled_sum_reduce/test.cu:28-76 in the reference).
#include "common.cuh"
// tile of this project in the reference (its core.cu): the launcher applies the reference's shape rule
#define WARPTILE_M 8
#define WARPTILE_N 32
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int b = atoi(argv[1]), m = atoi(argv[2]), n = atoi(argv[3]);
    const size_t mn = static_cast<size_t>(m) * n;
    auto hA = random_f32(b * mn), hB = random_f32(b * mn);
    std::vector<float> ref(mn);
    orc_tiled_sum_reduce(hA.data(), hB.data(), ref.data(), b, m, n);
    float *dA = to_device(hA), *dB = to_device(hB), *dD = device_zeros<float>(mn);
    tiled_sum_reduce(dA, dB, dD, b, m, n);
    CUDA_CHECK(cudaDeviceSynchronize());
    print_deltas(to_host(dD, mn), ref);
    return 0;
}
