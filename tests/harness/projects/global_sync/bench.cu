// Barrier probe latency (projects/global_sync/bench.cu in the reference).
#include "common.cuh"
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int, char**) {
    uint32_t* D = device_zeros<uint32_t>(1024);
    bench_protocol(20, 200, [&](int) { globs(D); });
    return 0;
}
