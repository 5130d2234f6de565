// argv: m n k.  Random fp8 operands and one random scale (as the reference's
// driver, projects/skinny_gemm/test.cu:43-114), CPU oracle vs the library.
#include "common.cuh"
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int m = atoi(argv[1]), n = atoi(argv[2]), k = atoi(argv[3]);
    srand(0);
    auto hA = random_fp8(static_cast<size_t>(m) * k), hB = random_fp8(static_cast<size_t>(n) * k);
    std::vector<float> hs = random_f32(1), one(1, 1.0f);
    std::vector<uint16_t> ref(static_cast<size_t>(m) * n);
    orc_gemm_fp8_bf16(hA.data(), hB.data(), hs[0], 1.0f, ref.data(), m, n, k, k);
    uint8_t *dA = to_device(hA), *dB = to_device(hB);
    float *dS = to_device(hs), *dOne = to_device(one);
    uint16_t* dD = device_zeros<uint16_t>(static_cast<size_t>(m) * n);
    if (skinny_gemm_fastpath(dA, dB, dD, dS, m, n, k) != SUCCESS) return 1;
    CUDA_CHECK(cudaDeviceSynchronize());
    auto got = to_host(dD, static_cast<size_t>(m) * n);
    std::vector<float> g(got.size()), r(got.size());
    for (size_t i = 0; i < got.size(); i++) { g[i] = orc_bf16_decode(got[i]); r[i] = orc_bf16_decode(ref[i]); }
    print_deltas(g, r);
    return 0;
}
