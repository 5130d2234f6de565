// No arguments needed (the reference's own test.cu for this project is a stale
// copy that does not build; this one checks the probe's visible effect): after
// the barrier every block's word has been decremented an even number of times.
#include "common.cuh"
#include "rocm_dev_b200_compat.hpp"   // the reference-named launchers

int main(int, char**) {
    std::vector<uint32_t> init(1024, 5u);
    uint32_t* D = to_device(init);
    globs(D);
    CUDA_CHECK(cudaDeviceSynchronize());
    auto got = to_host(D, 1024);
    std::vector<float> g(3), r = {0.f, 0.f, 5.f};
    for (int i = 0; i < 3; i++) g[i] = static_cast<float>(got[i]);
    print_deltas(g, r);
    return rdb_device_status();
}
