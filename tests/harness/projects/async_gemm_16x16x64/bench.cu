// argv: m n k.
#include "common.cuh"

int main(int argc, char** argv) {
    if (argc != 4) return 2;
    const int m = atoi(argv[1]), n = atoi(argv[2]), k = atoi(argv[3]);
    auto hA = random_fp8(static_cast<size_t>(m) * k), hB = random_fp8(static_cast<size_t>(n) * k);
    uint8_t *dA = to_device(hA), *dB = to_device(hB);
    float* dD = device_zeros<float>(static_cast<size_t>(m) * n);
    bench_protocol(10, 50, [&](int) { RDB_CHECK(rdb_dense_gemm_fp8_f32(dA, dB, dD, m, n, k, nullptr)); });
    return 0;
}
