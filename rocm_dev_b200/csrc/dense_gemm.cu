// Dense FP8 GEMM for sm_100a:  D[M,N] = (A . B^T) [* sa * sb], A [M,K], B [N,K], both e4m3 K-contiguous.
//
// One kernel replaces the three producer/consumer GEMM projects of the
// reference (projects/async_gemm_16x16x64/src.cu:5-82, projects/
// async_gemm_blanes/sparse_k.cu:5-80, projects/async_gemm_sparse/sparse_k.cu:
// 5-75 and their producer.cu / consumer.cu), whose 16x16, 16x48 and 8x64 tiles
// per block re-read the operands from L2 at 16 flop/byte.  Here a persistent
// CTA per SM walks 128 x 256 output tiles:
//   warp 0    one thread issues TMA loads (A box 128 x 128 B, B box 256 x 128 B)
//             into a 4-stage ring guarded by full/empty mbarriers;
//   warp 1    allocates all 512 TMEM columns (two 128 x 256 fp32 accumulators);
//             one thread issues tcgen05.mma kind::f8f6f4 (128 x 256 x 32), frees
//             stages with tcgen05.commit and hands finished accumulators over;
//   warps 2-5 epilogue: tcgen05.ld the accumulator (one row per thread), scale,
//             convert and store while the next tile's MMAs fill the other
//             accumulator.
// The "B lanes" of async_gemm_blanes (one A tile feeding several B tiles) are
// simply the wide UMMA N; split-K and its fp32 atomics are gone, D is
// overwritten.  Tiles are ordered in groups of 16 tile-rows so that the ~148
// tiles in flight share operand panels in L2.  When the shape allows, pairs of
// CTAs compute 256 x 256 tiles with cta_group::2 MMAs instead (second kernel
// below).
#include <cuda_bf16.h>

#include "host_util.h"
#include "ptx.cuh"

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace dense {

constexpr int BN = 256, BK = 128;
constexpr int RB_BYTES = 128 * BK, B_BYTES = BN * BK;   // one 128-row block of A, the B tile
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;

// RB = 128-row blocks of A per tile.  RB = 1: 128 x 256 tiles, 4 stages, the two
// TMEM accumulators alternate between consecutive tiles.  RB = 2: 256 x 256
// tiles - two MMA row blocks share one B tile, which cuts the operand bytes per
// MMA by a third (64 KiB per 8 MMAs instead of 48 KiB per 4) - 3 stages, and the
// two accumulators are the two row blocks of the same tile.
template <int RB>
struct Cfg {
    static constexpr int BM = 128 * RB;
    static constexpr int A_BYTES = RB * RB_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = RB == 1 ? 4 : 3;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
};

struct Params {
    void* D;
    const float* scale_a;   // nullptr: unscaled
    const float* scale_b;
    int* status;
    int M, N, num_kb, tiles_m, tiles_n;
    int out_f32;            // 1: fp32 output, 0: bf16
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& mb, int& nb) {
    const int per_group = GROUP_M * tiles_n;
    const int g = tile / per_group, r = tile - g * per_group;
    const int first = g * GROUP_M;
    const int gsize = tiles_m - first < GROUP_M ? tiles_m - first : GROUP_M;
    mb = first + r % gsize;
    nb = r / gsize;
}

// Epilogue store of 32 consecutive columns of one output row (scaled; bf16 or fp32).
// vec8: 16-byte stores are safe (aligned D, row length a multiple of 16 bytes).
__device__ __forceinline__ void store_row32(const Params& p, const float* v, float sc, int row, int col, bool vec8) {
    if (row >= p.M || col >= p.N) return;
    if (p.out_f32) {
        float* out = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.N + col;
        if (vec8 && col + 31 < p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(out + j) = make_float4(v[j] * sc, v[j + 1] * sc, v[j + 2] * sc, v[j + 3] * sc);
        } else {
            for (int j = 0; j < 32; j++)
                if (col + j < p.N) out[j] = v[j] * sc;
        }
    } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<size_t>(row) * p.N + col;
        if (vec8 && col + 31 < p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                __nv_bfloat162 b0 = __floats2bfloat162_rn(v[j] * sc, v[j + 1] * sc), b1 = __floats2bfloat162_rn(v[j + 2] * sc, v[j + 3] * sc);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(v[j + 4] * sc, v[j + 5] * sc), b3 = __floats2bfloat162_rn(v[j + 6] * sc, v[j + 7] * sc);
                uint4 o;
                o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
                o.z = *reinterpret_cast<uint32_t*>(&b2); o.w = *reinterpret_cast<uint32_t*>(&b3);
                *reinterpret_cast<uint4*>(out + j) = o;
            }
        } else {
            for (int j = 0; j < 32; j++)
                if (col + j < p.N) out[j] = __float2bfloat16_rn(v[j] * sc);
        }
    }
}

template <int RB>
__global__ void __launch_bounds__(NUM_THREADS, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
    using C = Cfg<RB>;
    constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES, A_BYTES = C::A_BYTES, BM = C::BM;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_last();   // operand panels are re-read by neighbouring tiles
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && *abort_flag == 0; tile += gridDim.x) {
                int mb, nb;
                tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
                for (int kb = 0; kb < p.num_kb; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { *abort_flag = 1; report_timeout(p.status); break; }
                    const uint32_t dst = stage0 + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
                    tma_load_2d(dst, &tmA, kb * BK, mb * BM, full0 + 8 * s, pol);
                    tma_load_2d(dst + A_BYTES, &tmB, kb * BK, nb * BN, full0 + 8 * s, pol);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_e4m3_f32(128, BN);
            int it = 0, t = 0;
            for (int tile = blockIdx.x; tile < num_tiles && *abort_flag == 0; tile += gridDim.x, t++) {
                // accumulator buffers: RB = 1 alternates them between tiles, RB = 2 uses one per row block
                const int acc0 = RB == 1 ? (t & 1) : 0;
                const uint32_t use = RB == 1 ? (t >> 1) : t;           // how often this buffer has been used before
                bool ok = true;
                for (int kb = 0; kb < p.num_kb && ok; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a = stage0 + s * STAGE_BYTES, b = a + A_BYTES;
#pragma unroll
                    for (int rb = 0; rb < RB; rb++) {
                        const int acc = acc0 + rb;
                        if (kb == 0) {
                            // the epilogue must have drained this accumulator
                            if (!mbar_wait(acc_empty0 + 8 * acc, (use & 1) ^ 1)) { ok = false; break; }
                            tc_fence_after_sync();
                        }
                        const uint32_t d = tmem_base + acc * BN;
#pragma unroll
                        for (int ks = 0; ks < BK / 32; ks++)
                            tc_mma_f8(d, smem_desc_k128(a + rb * RB_BYTES + ks * 32), smem_desc_k128(b + ks * 32), idesc, (kb | ks) != 0);
                        if (kb == p.num_kb - 1) tc_commit(acc_full0 + 8 * acc);   // this row block is complete
                    }
                    tc_commit(empty0 + 8 * s);
                }
                if (!ok) { *abort_flag = 1; report_timeout(p.status); break; }
            }
        }
        __syncwarp();
    } else {
        // epilogue warps: TMEM lane quadrant = warp % 4, one output row per thread
        const int quad = warp & 3;
        float sc = 1.0f;
        if (p.scale_a) sc = __ldg(p.scale_a) * __ldg(p.scale_b);
        // 16-byte stores need a 16-byte aligned D and rows that keep that alignment (8 bf16 or 4 fp32)
        const bool vec8 = (p.N % (p.out_f32 ? 4 : 8) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0);
        int t = 0;
        bool live = true;
        for (int tile = blockIdx.x; tile < num_tiles && live; tile += gridDim.x, t++) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
#pragma unroll 1
            for (int rb = 0; rb < RB; rb++) {
                const int acc = RB == 1 ? (t & 1) : rb;
                const uint32_t use = RB == 1 ? (t >> 1) : t;
                bool ok = mbar_wait(acc_full0 + 8 * acc, use & 1);
                if (!ok) { *abort_flag = 1; report_timeout(p.status); }
                if (*abort_flag != 0) { live = false; break; }
                tc_fence_after_sync();
                const int row = mb * BM + rb * 128 + quad * 32 + lane;
                const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    float v[32];
                    tmem_ld32(taddr + c0, v);
                    store_row32(p, v, sc, row, nb * BN + c0, vec8);
                }
                // all of this warp's TMEM reads are complete: hand the accumulator back
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
            }
        }
    }

    if (*abort_flag != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ------------------------------------------------------------- CTA pairs
// Two CTAs of a cluster compute one 256 x 256 tile with cta_group::2 MMAs: CTA
// r of the pair loads rows [128 r, 128 r + 128) of the A tile and of the B tile
// (32 KiB per k-block instead of the 64 KiB a single CTA needs for the same
// 256 x 256 tile), the even CTA issues 256 x 256 x 32 MMAs that read both
// CTAs' shared memory, and each CTA ends up with its 128 rows of the result in
// its own TMEM.  Halving the B bytes per MMA cuts the shared-memory and L2
// traffic (and with it the power) per flop.  A stage holds two 128-byte
// k-blocks per operand, fetched by one 3-D TMA box each, so that the issuing
// thread's fixed cost per stage (barrier wait, fence, commits: ~470 cycles
// measured) is spread over eight MMAs (8 x 128 cycles of tensor work); with
// four MMAs per stage the issuing thread, not the tensor pipe, set the pace.
// Barriers: `full` lives in the even CTA and counts
// the bytes of all four loads; `empty` and `acc_full` exist in both CTAs and are
// signalled in both by one tcgen05.commit with a two-CTA mask; `acc_empty`
// lives in the even CTA and collects the eight epilogue warps of the pair.
namespace pairk {
constexpr int CHUNK_BYTES = 128 * BK;           // 128 rows x 128 bytes
constexpr int PAIR_THREADS = 224;               // warp 0: A loads, 1: MMA, 2-5: epilogue, 6: B loads
// CHUNKS = k-blocks of 128 bytes per stage, fetched by one TMA box per operand
template <int CHUNKS>
struct PCfg {
    static constexpr int STAGES = 6 / CHUNKS;
    static constexpr int HALF_BYTES = CHUNKS * CHUNK_BYTES;   // this CTA's 128 rows of A (or of B) for one stage
    static constexpr int STAGE_BYTES = 2 * HALF_BYTES;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
};
}  // namespace pairk

template <int CHUNKS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pairk::PAIR_THREADS, 1)
dense_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
    using namespace pairk;
    using C = PCfg<CHUNKS>;
    constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES, HALF_BYTES = C::HALF_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0: issues the MMAs
    const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, 8);   // four epilogue warps in each CTA of the pair
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive_release();                   // both CTAs' barriers and TMEM exist before either touches the other
    cluster_wait_acquire();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int num_tiles = p.tiles_m * p.tiles_n;

    if (warp == 0 || warp == 6) {
        // two producer threads per CTA (one per operand): a single thread's wait + two TMA issues
        // per stage would be slower than the four MMAs that consume a one-chunk stage
        if (lane == 0) {
            const bool is_a = warp == 0;
            const CUtensorMap* tm = is_a ? &tmA : &tmB;
            const uint32_t off = is_a ? 0u : static_cast<uint32_t>(HALF_BYTES);
            const uint64_t pol = l2_policy_evict_last();
            const uint32_t full_even0 = mapa_smem(full0, 0);
            int it = 0;
            bool ok = true;
            for (int tile = pair_id; tile < num_tiles && ok && *abort_flag == 0; tile += num_pairs) {
                int mb, nb;
                tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
                const int row = (is_a ? mb : nb) * 256 + static_cast<int>(rank) * 128;
                for (int kb = 0; kb < p.num_kb; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { ok = false; break; }
                    if (is_a && rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                    tma_load_3d_pair(stage0 + s * STAGE_BYTES + off, tm, 0, row, kb * CHUNKS, full_even0 + 8 * s, pol);
                }
            }
            // every commit aimed at this CTA's `empty` barriers must land before the CTA may exit
            for (int i = 0; i < STAGES && ok && *abort_flag == 0; i++, it++) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) ok = false;
            }
            if (!ok) { *abort_flag = 1; report_timeout(p.status); }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = idesc_e4m3_f32(256, 256);
            int it = 0, t = 0;
            bool ok = true;
            for (int tile = pair_id; tile < num_tiles && ok && *abort_flag == 0; tile += num_pairs, t++) {
                const int acc = t & 1;
                const uint32_t use = t >> 1;
                for (int kb = 0; kb < p.num_kb && ok; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(full0 + 8 * s, ph)) { ok = false; break; }
                    if (kb == 0 && !mbar_wait_cluster(acc_empty0 + 8 * acc, (use & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a = stage0 + s * STAGE_BYTES, b = a + HALF_BYTES;
                    const uint32_t d = tmem_base + acc * 256;
#pragma unroll
                    for (int c = 0; c < CHUNKS; c++) {
#pragma unroll
                        for (int ks = 0; ks < BK / 32; ks++)
                            tc_mma_f8_pair(d, smem_desc_k128(a + c * CHUNK_BYTES + ks * 32), smem_desc_k128(b + c * CHUNK_BYTES + ks * 32),
                                           idesc, (kb | c | ks) != 0);
                    }
                    // one commit each reaches the barrier of both CTAs: the issuing thread's time per stage, not
                    // the tensor pipe, sets this kernel's pace, and a commit costs it about as much as two MMAs
                    tc_commit_pair_both(empty0 + 8 * s);
                    if (kb == p.num_kb - 1) tc_commit_pair_both(acc_full0 + 8 * acc);
                }
            }
            if (!ok) { *abort_flag = 1; report_timeout(p.status); }
        }
        __syncwarp();
    } else {
        const int quad = warp & 3;
        float sc = 1.0f;
        if (p.scale_a) sc = __ldg(p.scale_a) * __ldg(p.scale_b);
        // 16-byte stores need a 16-byte aligned D and rows that keep that alignment (8 bf16 or 4 fp32)
        const bool vec8 = (p.N % (p.out_f32 ? 4 : 8) == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0);
        const uint32_t acc_empty_even0 = mapa_smem(acc_empty0, 0);
        int t = 0;
        for (int tile = pair_id; tile < num_tiles; tile += num_pairs, t++) {
            int mb, nb;
            tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
            const int acc = t & 1;
            const uint32_t use = t >> 1;
            if (!mbar_wait(acc_full0 + 8 * acc, use & 1)) { *abort_flag = 1; report_timeout(p.status); }
            if (*abort_flag != 0) break;
            tc_fence_after_sync();
            const int row = mb * 256 + static_cast<int>(rank) * 128 + quad * 32 + lane;
            const uint32_t taddr = tmem_base + acc * 256 + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += 32) {
                float v[32];
                tmem_ld32(taddr + c0, v);
                store_row32(p, v, sc, row, nb * 256 + c0, vec8);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_even0 + 8 * acc);
        }
    }

    if (*abort_flag != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive_release();                   // neither CTA frees TMEM or exits while the other may still signal it
    cluster_wait_acquire();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

template <int RB>
static int launch(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, void* D, int out_f32, int M, int N,
                  int K, int max_ctas, DeviceInfo* info, cudaStream_t stream) {
    using C = Cfg<RB>;
    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = dense_gemm_kernel<RB>;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
            return RDB_CUDA_ERROR;
        attr_set[dev] = true;
    }
    CUtensorMap tmA, tmB;
    int r = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BK, C::BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != RDB_SUCCESS) return r;
    r = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, K, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != RDB_SUCCESS) return r;
    Params p;
    p.D = D;
    p.scale_a = sa;
    p.scale_b = sb;
    p.status = info->status_dev;
    p.M = M;
    p.N = N;
    p.num_kb = (K + BK - 1) / BK;
    p.tiles_m = (M + C::BM - 1) / C::BM;
    p.tiles_n = (N + BN - 1) / BN;
    p.out_f32 = out_f32;
    int grid = p.tiles_m * p.tiles_n;
    int cap = info->sm_count;
    if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
    if (grid > cap) grid = (grid + (grid + cap - 1) / cap - 1) / ((grid + cap - 1) / cap);   // same waves, fewest CTAs
    kernel<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

template <int CHUNKS>
static int launch_pair(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, void* D, int out_f32, int M,
                       int N, int K, int max_ctas, DeviceInfo* info, cudaStream_t stream) {
    using PC = pairk::PCfg<CHUNKS>;
    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(dense_gemm_pair_kernel<CHUNKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, PC::SMEM_BYTES) != cudaSuccess)
            return RDB_CUDA_ERROR;
        attr_set[dev] = true;
    }
    CUtensorMap tmA, tmB;
    int r = make_tmap_kchunks(&tmA, A, M, K, K, 128, CHUNKS);
    if (r != RDB_SUCCESS) return r;
    r = make_tmap_kchunks(&tmB, B, N, K, K, 128, CHUNKS);
    if (r != RDB_SUCCESS) return r;
    Params p;
    p.D = D;
    p.scale_a = sa;
    p.scale_b = sb;
    p.status = info->status_dev;
    p.M = M;
    p.N = N;
    p.num_kb = (K + CHUNKS * BK - 1) / (CHUNKS * BK);    // a stage past the end of K reads zeros
    p.tiles_m = (M + 255) / 256;
    p.tiles_n = (N + 255) / 256;
    p.out_f32 = out_f32;
    int pairs = p.tiles_m * p.tiles_n;
    int cap = info->sm_count / 2;
    if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
    // the smallest grid that still finishes in the same number of waves: 256 tiles take four waves on 74 pairs
    // and on 64, and the 64 run faster (measured 49.8 us against 54.9 us at 4096^3: fewer CTAs share L2 and power)
    if (pairs > cap) pairs = (pairs + (pairs + cap - 1) / cap - 1) / ((pairs + cap - 1) / cap);
    dense_gemm_pair_kernel<CHUNKS><<<2 * pairs, pairk::PAIR_THREADS, PC::SMEM_BYTES, stream>>>(tmA, tmB, p);
    return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

static int run(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, void* D, int out_f32, int M, int N,
               int K, int max_ctas, int tile_rows, cudaStream_t stream) {
    if (M < 1 || N < 1 || K < 1) return RDB_BAD_SHAPE;
    if (K % 16 != 0) return RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K;
    if (!aligned16(A) || !aligned16(B) || (reinterpret_cast<uintptr_t>(D) & 3u)) return RDB_BAD_ALIGNMENT;
    if ((sa == nullptr) != (sb == nullptr)) return RDB_INVALID_CONFIG;
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    if (tile_rows == 0 && max_ctas == 0) lookup_dense_plan(M, N, K, &tile_rows, &max_ctas);   // a measured entry, if any
    // 256 x 256 tiles when padding M up to a multiple of 256 wastes no more than ~12 % of the work:
    // computed by CTA pairs (K a multiple of 128 bytes; a pair uses the same two SMs as two 128-row
    // tiles would, with half the B traffic), else by single CTAs when there is at least one tile
    // per SM; 128 x 256 tiles otherwise
    const int m256 = (M + 255) / 256 * 256;
    const long long tiles256 = static_cast<long long>(m256 / 256) * ((N + BN - 1) / BN);
    const bool pad_ok = (m256 - M) * 8 <= M;
    const bool want256 = tiles256 >= info->sm_count && pad_ok;
    if (tile_rows == 2 || tile_rows == 3 || (tile_rows == 0 && pad_ok && K % 128 == 0 && info->sm_count >= 2)) {
        if (K % 128 != 0) return RDB_INVALID_CONFIG;
        // tile_rows 3: the pair kernel with three k-blocks per stage and two stages (twelve MMAs per barrier round trip)
        const int r = tile_rows == 3 ? launch_pair<3>(A, B, sa, sb, D, out_f32, M, N, K, max_ctas, info, stream)
                                     : launch_pair<2>(A, B, sa, sb, D, out_f32, M, N, K, max_ctas, info, stream);
        // a device or a partition that refuses the cluster launch: the automatic choice falls back to single CTAs
        if (r != RDB_CUDA_ERROR || tile_rows != 0) return r;
        cudaGetLastError();
    }
    const int rb = (tile_rows == 128 || (tile_rows == 0 && !want256)) ? 1 : 2;
    return rb == 1 ? launch<1>(A, B, sa, sb, D, out_f32, M, N, K, max_ctas, info, stream)
                   : launch<2>(A, B, sa, sb, D, out_f32, M, N, K, max_ctas, info, stream);
}

}  // namespace dense
}  // namespace rdb

extern "C" {

int rdb_dense_gemm_fp8(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b, uint16_t* D,
                       int M, int N, int K, void* stream) {
    if (!scale_a || !scale_b) return RDB_INVALID_CONFIG;
    return rdb::dense::run(A, B, scale_a, scale_b, D, 0, M, N, K, 0, 0, static_cast<cudaStream_t>(stream));
}

int rdb_dense_gemm_fp8_f32(const uint8_t* A, const uint8_t* B, float* D, int M, int N, int K, void* stream) {
    return rdb::dense::run(A, B, nullptr, nullptr, D, 1, M, N, K, 0, 0, static_cast<cudaStream_t>(stream));
}

int rdb_dense_gemm_fp8_tuned(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b, uint16_t* D,
                             int M, int N, int K, int tile_rows, int max_ctas, void* stream) {
    if (!scale_a || !scale_b) return RDB_INVALID_CONFIG;
    if (tile_rows != 0 && tile_rows != 128 && tile_rows != 256 && tile_rows != 2 && tile_rows != 3) return RDB_INVALID_CONFIG;
    return rdb::dense::run(A, B, scale_a, scale_b, D, 0, M, N, K, max_ctas, tile_rows, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
