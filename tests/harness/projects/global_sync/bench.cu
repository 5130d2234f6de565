// Barrier probe latency (projects/global_sync/bench.cu in the reference).
#include "common.cuh"

int main(int, char**) {
    uint32_t* D = device_zeros<uint32_t>(1024);
    bench_protocol(20, 200, [&](int) { RDB_CHECK(rdb_globs(D, nullptr)); });
    return 0;
}
