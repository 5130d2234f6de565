// Skinny (decode-shaped) FP8 GEMM for sm_100a:  D[M,N] = bf16((A . B^T) * sa * sb), M <= 32.
//
// The problem is bound by streaming the weight matrix B [N,K] from HBM once.
// The weights therefore sit on the 128-row side of the tensor-core tile
// ("swap-AB"): each CTA owns 128 rows of B and a contiguous slice of K, TMA
// streams 128x128-byte weight boxes (plus the matching M x 128-byte activation
// box) into a shared-memory ring guarded by full/empty mbarriers, one thread
// issues tcgen05.mma kind::f8f6f4 (128 x MPAD x 32) into a TMEM accumulator,
// and four epilogue warps read TMEM back.  K is split across the CTAs of one
// thread-block cluster; the fp32 partials are exchanged through distributed
// shared memory and summed in rank order, so the result is deterministic and
// needs no global workspace, no atomics and no zeroed output.
//
// Replaces _skinny_gemm_kernel and its producer/consumer waves
// (projects/skinny_gemm/skinny_gemm_kernel.cu:6-110, producers/, consumers/ in
// the reference project) and the launchers of skinny_gemm_caller.cu.
#include <cuda_bf16.h>

#include "host_util.h"
#include "ptx.cuh"

namespace rdb {
namespace skinny {

constexpr int BN = 128;                    // weight rows per CTA (UMMA M)
constexpr int BK = 128;                    // K bytes per stage = one 128-byte swizzle row
constexpr int W_STAGE_BYTES = BN * BK;     // 16 KiB
constexpr int NUM_THREADS = 192;           // warp 0 TMA, warp 1 MMA + TMEM, warps 2..5 epilogue
constexpr int MAX_STAGES = 12;
constexpr int BAR_BYTES = 256;
constexpr int TMEM_COLS = 32;
constexpr int SMEM_LIMIT = 232448;         // 227 KiB opt-in maximum per CTA

template <int MPAD>
struct Cfg {
    static constexpr int A_STAGE_BYTES = MPAD * BK;
    static constexpr int STAGE_BYTES = W_STAGE_BYTES + A_STAGE_BYTES;
    // split-K exchange buffer: [src rank][row in my chunk][MPAD] fp32; the
    // chunks of a cluster of S ranks hold at most ceil(128/S) rows each.
    static constexpr int RED_BYTES = (BN + 8) * MPAD * 4;
    static constexpr int FIXED_BYTES = 1024 + RED_BYTES + BAR_BYTES;
    static constexpr int max_stages() {
        int s = (SMEM_LIMIT - FIXED_BYTES) / STAGE_BYTES;
        return s > MAX_STAGES ? MAX_STAGES : s;
    }
    static constexpr int smem_bytes(int stages) { return FIXED_BYTES + stages * STAGE_BYTES; }
};

// Owner rank of tile row `row` when 128 rows are cut into S chunks
// [128c/S, 128(c+1)/S).
__device__ __forceinline__ int chunk_of_row(int row, int S) { return (row * S + S - 1) / BN; }
__device__ __forceinline__ int chunk_begin(int c, int S) { return (BN * c) / S; }

template <int MPAD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                   __nv_bfloat16* __restrict__ D, const float* __restrict__ scale_a,
                   const float* __restrict__ scale_b, int M, int N, int num_kb, int nstages, int* status) {
    using C = Cfg<MPAD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int S = gridDim.x;               // cluster = all CTAs along x = the K splits of one tile
    const int rank = blockIdx.x;
    const int n0 = blockIdx.y * BN;
    const int kb_begin = static_cast<int>((static_cast<long long>(num_kb) * rank) / S);
    const int kb_end = static_cast<int>((static_cast<long long>(num_kb) * (rank + 1)) / S);
    const int nkb = kb_end - kb_begin;

    float* red = reinterpret_cast<float*>(smem + nstages * C::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + C::RED_BYTES);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + MAX_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * MAX_STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmA);
        for (int s = 0; s < nstages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tmem_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (S > 1) cluster_arrive_release();   // phase 1: "my shared memory is live"

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first();
            const uint64_t pol_a = l2_policy_evict_last();
            for (int i = 0; i < nkb; i++) {
                const int s = i % nstages;
                const uint32_t ph = (i / nstages) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { *abort_flag = 1; report_timeout(status); break; }
                const uint32_t dst = stage0 + s * C::STAGE_BYTES;
                mbar_arrive_expect_tx(full0 + 8 * s, C::STAGE_BYTES);
                tma_load_2d(dst, &tmW, (kb_begin + i) * BK, n0, full0 + 8 * s, pol_w);
                tma_load_2d(dst + W_STAGE_BYTES, &tmA, (kb_begin + i) * BK, 0, full0 + 8 * s, pol_a);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_e4m3_f32(BN, MPAD);
            for (int i = 0; i < nkb; i++) {
                const int s = i % nstages;
                const uint32_t ph = (i / nstages) & 1;
                if (!mbar_wait(full0 + 8 * s, ph)) { *abort_flag = 1; report_timeout(status); break; }
                tc_fence_after_sync();
                const uint32_t w = stage0 + s * C::STAGE_BYTES;
                const uint32_t a = w + W_STAGE_BYTES;
#pragma unroll
                for (int ks = 0; ks < BK / 32; ks++)
                    tc_mma_f8(tmem_base, smem_desc_k128(w + ks * 32), smem_desc_k128(a + ks * 32), idesc,
                              (i | ks) != 0);
                tc_commit(empty0 + 8 * s);   // the stage is free once these MMAs have read it
            }
            tc_commit(tmem_full);            // accumulator complete (also fires after an abort)
        }
        __syncwarp();
    }

    // ---- epilogue (warps 2..5 hold one accumulator row = one weight row each)
    const bool epi = warp >= 2;
    const int quad = warp & 3;             // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;
    float acc[MPAD];
    bool ok = true;
    if (epi) {
        ok = mbar_wait(tmem_full, 0);
        if (!ok) { *abort_flag = 1; report_timeout(status); }
        ok = ok && (*abort_flag == 0);
        tc_fence_after_sync();
        if (ok) {
#pragma unroll
            for (int c = 0; c < MPAD; c += 16) tmem_ld16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + c, acc + c);
        } else {
#pragma unroll
            for (int c = 0; c < MPAD; c++) acc[c] = 0.0f;
        }
    }
    const float sc = __ldg(scale_a) * __ldg(scale_b);

    if (S == 1) {
        if (epi && ok) {
            const int n = n0 + row;
            if (n < N) {
#pragma unroll
                for (int m = 0; m < MPAD; m++)
                    if (m < M) D[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(acc[m] * sc);
            }
        }
    } else {
        cluster_wait_acquire();            // phase 1 done: every peer's shared memory is live
        if (epi) {
            const int owner = chunk_of_row(row, S);
            const int local = row - chunk_begin(owner, S);
            const int rows_per = (BN + S - 1) / S;
            const uint32_t dst = mapa_smem(smem_u32(red + (static_cast<size_t>(rank) * rows_per + local) * MPAD), owner);
#pragma unroll
            for (int c = 0; c < MPAD; c += 4) st_cluster_v4(dst + c * 4, acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
        }
        cluster_arrive_release();          // phase 2: partials delivered
        cluster_wait_acquire();
        if (epi) {
            const int lo = chunk_begin(rank, S), hi = chunk_begin(rank + 1, S);
            const int rows_per = (BN + S - 1) / S;
            const int mine = row - lo;     // threads whose row falls in my chunk finish it
            const int n = n0 + row;
            if (row >= lo && row < hi && n < N && *abort_flag == 0) {
                float sum[MPAD];
#pragma unroll
                for (int c = 0; c < MPAD; c++) sum[c] = 0.0f;
                for (int src = 0; src < S; src++) {
                    const float4* p = reinterpret_cast<const float4*>(red + (static_cast<size_t>(src) * rows_per + mine) * MPAD);
#pragma unroll
                    for (int c = 0; c < MPAD / 4; c++) {
                        const float4 v = p[c];
                        sum[4 * c + 0] += v.x; sum[4 * c + 1] += v.y; sum[4 * c + 2] += v.z; sum[4 * c + 3] += v.w;
                    }
                }
#pragma unroll
                for (int m = 0; m < MPAD; m++)
                    if (m < M) D[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(sum[m] * sc);
            }
        }
    }

    // ---- teardown: after an abort give in-flight TMA copies time to land
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

struct Plan {
    int mpad, split_k, stages;
};

template <int MPAD>
int launch(const CUtensorMap& tmW, const CUtensorMap& tmA, uint16_t* D, const float* sa, const float* sb, int M, int N,
           int num_kb, int tiles, const Plan& p, int* status, cudaStream_t stream) {
    using C = Cfg<MPAD>;
    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = skinny_gemm_kernel<MPAD>;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem_bytes(C::max_stages())) !=
            cudaSuccess)
            return RDB_CUDA_ERROR;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.split_k, tiles, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::smem_bytes(p.stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.split_k;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmW, tmA, reinterpret_cast<__nv_bfloat16*>(D), sa, sb, M, N, num_kb,
                                       p.stages, status);
    return e == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

int run(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, uint16_t* D, int M, int N, int K, int ldb,
        int split_k_hint, int stages_hint, cudaStream_t stream) {
    if (M < 1 || N < 1 || K < 1 || ldb < K) return RDB_BAD_SHAPE;
    if (M > 32) return RDB_M_ABOVE_WARPTILE_M;
    if (N % 2 != 0) return RDB_N_NOT_EVEN;
    if (K % 16 != 0 || ldb % 16 != 0) return RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K;
    if (!aligned16(A) || !aligned16(B) || (reinterpret_cast<uintptr_t>(D) & 1u)) return RDB_BAD_ALIGNMENT;
    if (split_k_hint < 0 || split_k_hint > 8 || stages_hint < 0) return RDB_INVALID_CONFIG;
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;

    Plan p;
    p.mpad = M <= 16 ? 16 : 32;
    const int num_kb = (K + BK - 1) / BK;
    const int tiles = (N + BN - 1) / BN;
    const int max_stages = p.mpad == 16 ? Cfg<16>::max_stages() : Cfg<32>::max_stages();
    if (split_k_hint > 0) {
        p.split_k = split_k_hint;
    } else {
        p.split_k = info->sm_count / tiles;
        if (p.split_k > 8) p.split_k = 8;
        if (p.split_k < 1) p.split_k = 1;
    }
    if (p.split_k > num_kb) p.split_k = num_kb;
    if (stages_hint > 0) {
        p.stages = stages_hint < max_stages ? stages_hint : max_stages;
    } else {
        // one resident CTA per SM when the grid fits in one wave, else two
        p.stages = (tiles * p.split_k <= info->sm_count) ? max_stages : max_stages / 2;
    }
    const int kb_per = (num_kb + p.split_k - 1) / p.split_k;
    if (p.stages > kb_per) p.stages = kb_per;
    if (p.stages < 1) p.stages = 1;

    CUtensorMap tmW, tmA;
    int r = make_tmap_2d(&tmW, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != RDB_SUCCESS) return r;
    r = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BK, p.mpad, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != RDB_SUCCESS) return r;
    if (p.mpad == 16) return launch<16>(tmW, tmA, D, sa, sb, M, N, num_kb, tiles, p, info->status_dev, stream);
    return launch<32>(tmW, tmA, D, sa, sb, M, N, num_kb, tiles, p, info->status_dev, stream);
}

}  // namespace skinny
}  // namespace rdb

extern "C" {

int rdb_skinny_gemm_fp8(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b, uint16_t* D,
                        int M, int N, int K, int ldb, void* stream) {
    return rdb::skinny::run(A, B, scale_a, scale_b, D, M, N, K, ldb, 0, 0, static_cast<cudaStream_t>(stream));
}

int rdb_skinny_gemm_fp8_hinted(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b,
                               uint16_t* D, int M, int N, int K, int ldb, int split_k, int A_producers, int B_producers,
                               int consumers, int b_lanes, int qsize, int op_m, int ops, void* stream) {
    // Validation order and codes follow the reference launcher.
    if (N % 2 != 0) return RDB_N_NOT_EVEN;
    if ((op_m != 8 && op_m != 16 && op_m != 32) || ops < 1 || b_lanes < 1) return RDB_INVALID_CONFIG;
    if (K % ((512 / op_m) * ops) != 0) return RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K;
    if (A_producers + B_producers + consumers > 16) return RDB_TOO_MANY_WARPS;
    if (qsize < A_producers || qsize < B_producers / b_lanes || qsize < consumers) return RDB_QSIZE_TOO_SMALL;
    if (split_k > 8) split_k = 8;
    return rdb::skinny::run(A, B, scale_a, scale_b, D, M, N, K, ldb, split_k < 0 ? 0 : split_k, qsize,
                            static_cast<cudaStream_t>(stream));
}

}  // extern "C"
