// Host-side helpers shared by the launchers: status codes, the per-device
// status word device code reports into, and TMA tensor-map construction
// through the driver entry point (no link-time dependency on libcuda, so the
// library also loads on a machine without a GPU driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rocm_dev_b200.h"

namespace rdb {

constexpr int kMaxDevices = 64;

struct DeviceInfo {
    bool ready = false;
    int sm_count = 0;
    int* status_host = nullptr;  // pinned, mapped host word
    int* status_dev = nullptr;   // device alias of the same word
};

// Per-device facts and the status word; created on first use with that device
// current.  Returns nullptr (and sets *err) when a CUDA call fails.
DeviceInfo* device_info(int* err);

// Encodes a 2-D tiled tensor map over a row-major [rows, cols] array of
// `elem_bytes`-sized elements with row pitch `pitch_bytes`.  box = {box_cols,
// box_rows}.  swizzle is a CUtensorMapSwizzle value.
// Byte matrix [rows][k_bytes] (k_bytes a multiple of 128) seen as [k_bytes/128][rows][128]: one box of
// (128 B, box_rows, box_chunks) lands in shared memory as box_chunks consecutive K-major SWIZZLE_128B tiles
// of box_rows rows - several k-blocks of an operand with a single TMA instruction.
int make_tmap_kchunks(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_bytes, uint64_t pitch_bytes,
                      uint32_t box_rows, uint32_t box_chunks);

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t rows,
                 uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle,
                 CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B);

// Tuning-table lookups (tuning_table.cu): measured best configurations per shape, consulted by the
// launchers when the caller gives no knobs.  Return false when the shape has no entry.
bool lookup_skinny_plan(int mpad, int N, int K, int* rows, int* split_k, int* stages);
bool lookup_dense_plan(int M, int N, int K, int* tile_rows, int* max_ctas);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The device word holding the wait budget exists once per translation unit
// (ptx.cuh).  Each kernel source file names RDB_DEFINE_WAIT_BUDGET_SETTER once
// at namespace scope: it registers a function that writes that unit's copy on
// the current device, and rdb_set_wait_budget_ns calls all of them.
typedef int (*WaitBudgetSetter)(unsigned long long ns);
void register_wait_budget_setter(WaitBudgetSetter fn);

#define RDB_DEFINE_WAIT_BUDGET_SETTER()                                                                        \
    namespace {                                                                                                \
    int set_wait_budget_of_this_unit(unsigned long long ns) {                                                  \
        return cudaMemcpyToSymbol(rdb::d_wait_budget_ns, &ns, sizeof(ns)) == cudaSuccess ? RDB_SUCCESS         \
                                                                                        : RDB_CUDA_ERROR;      \
    }                                                                                                          \
    struct WaitBudgetRegistration {                                                                            \
        WaitBudgetRegistration() { rdb::register_wait_budget_setter(&set_wait_budget_of_this_unit); }          \
    } wait_budget_registration;                                                                                \
    }

}  // namespace rdb
