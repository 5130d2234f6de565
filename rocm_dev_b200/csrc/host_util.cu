#include "host_util.h"

#include <mutex>

namespace rdb {

namespace {
std::mutex g_mu;
DeviceInfo g_dev[kMaxDevices];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// Filled during static initialisation of the kernel source files: plain arrays
// (zero-initialised before any constructor runs), so the order does not matter.
WaitBudgetSetter g_budget_setters[16];
int g_num_budget_setters = 0;

EncodeTiledFn encode_fn() {
    if (g_encode) return g_encode;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_encode) return g_encode;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return g_encode;
}
}  // namespace

void register_wait_budget_setter(WaitBudgetSetter fn) {
    if (g_num_budget_setters < 16) g_budget_setters[g_num_budget_setters++] = fn;
}

DeviceInfo* device_info(int* err) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        if (err) *err = RDB_CUDA_ERROR;
        return nullptr;
    }
    DeviceInfo* d = &g_dev[dev];
    if (d->ready) return d;
    std::lock_guard<std::mutex> lk(g_mu);
    if (d->ready) return d;
    if (cudaDeviceGetAttribute(&d->sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaHostAlloc(reinterpret_cast<void**>(&d->status_host), sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&d->status_dev), d->status_host, 0) != cudaSuccess) {
        if (err) *err = RDB_CUDA_ERROR;
        return nullptr;
    }
    *d->status_host = 0;
    d->ready = true;
    return d;
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t rows,
                 uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle,
                 CUtensorMapL2promotion promo) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return RDB_CUDA_ERROR;
    (void)elem_bytes;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

int make_tmap_kchunks(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_bytes, uint64_t pitch_bytes,
                      uint32_t box_rows, uint32_t box_chunks) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return RDB_CUDA_ERROR;
    if (k_bytes % 128 != 0) return RDB_BAD_SHAPE;
    cuuint64_t dims[3] = {128, rows, k_bytes / 128};
    cuuint64_t strides[2] = {pitch_bytes, 128};
    cuuint32_t box[3] = {128, box_rows, box_chunks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

}  // namespace rdb

extern "C" {

const char* rdb_status_string(int status) {
    switch (status) {
        case RDB_SUCCESS: return "success";
        case RDB_M_ABOVE_WARPTILE_M: return "m is above the largest supported tile";
        case RDB_N_NOT_EVEN: return "n is not even";
        case RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K: return "k or a row pitch is not a multiple of 16 bytes";
        case RDB_TOO_MANY_WARPS: return "too many warps";
        case RDB_QSIZE_TOO_SMALL: return "qsize too small";
        case RDB_INVALID_CONFIG: return "invalid configuration";
        case RDB_BAD_ALIGNMENT: return "pointer not 16-byte aligned";
        case RDB_BAD_SHAPE: return "bad shape";
        case RDB_CUDA_ERROR: return "CUDA call failed";
        case RDB_DEVICE_TIMEOUT: return "device-side wait timed out";
        case RDB_SIZE_ABOVE_LIMIT: return "size above the supported limit";
        case RDB_IO_ERROR: return "file could not be opened, read or written";
        case RDB_BAD_FILE: return "not a valid file of this format (wrong magic or version, truncated, or corrupted)";
        default: return "unknown status";
    }
}

int rdb_device_status(void) {
    int err = 0;
    rdb::DeviceInfo* d = rdb::device_info(&err);
    if (!d) return err;
    if (cudaDeviceSynchronize() != cudaSuccess) return RDB_CUDA_ERROR;
    const int s = *reinterpret_cast<volatile int*>(d->status_host);
    *reinterpret_cast<volatile int*>(d->status_host) = 0;
    return s;
}

int rdb_set_wait_budget_ns(unsigned long long ns) {
    if (ns == 0) return RDB_BAD_SHAPE;
    if (cudaDeviceSynchronize() != cudaSuccess) return RDB_CUDA_ERROR;   // no kernel reads the word while it changes
    for (int i = 0; i < rdb::g_num_budget_setters; i++) {
        const int r = rdb::g_budget_setters[i](ns);
        if (r != RDB_SUCCESS) return r;
    }
    return RDB_SUCCESS;
}

const char* rdb_version(void) { return "rocm_dev_b200 0.1 (sm_100a)"; }

}  // extern "C"
