// Skinny (decode-shaped) FP8 GEMM for sm_100a:  D[M,N] = bf16((A . B^T) * sa * sb), M <= 32.
//
// The problem is bound by streaming the weight matrix B [N,K] from HBM once.
// Measured on B200: one SM pulls at most ~63 GB/s through TMA, and a
// tcgen05.mma costs ~100 ns whatever its N extent.  So the weights sit on the
// wide (N <= 256) side of the MMA - 8 KiB of weights per instruction - and the
// activations on the 128-lane side, of which only the first M lanes carry data
// (the remaining lanes read whatever follows the activation box in shared
// memory and are never looked at).
//
// Work split: the N rows are cut into T tiles of R rows (R a multiple of 16,
// chosen so that T x S CTAs cover the SMs in ONE balanced wave) and K into S
// slices, the S CTAs of a tile forming one thread-block cluster.  Per CTA:
//   warp 0   one thread issues TMA loads (weights R x 128 B + activations
//            MPAD x 128 B per stage) into a ring guarded by full/empty mbarriers;
//   warp 1   allocates TMEM; one thread issues tcgen05.mma kind::f8f6f4
//            (128 x R x 32) and frees stages with tcgen05.commit;
//   warps 0,4 drain the accumulator rows from TMEM into a shared staging tile;
//   all      the split-K partials are pushed through distributed shared memory
//            with st.async (each rank owns a column chunk and waits on an
//            mbarrier for exactly the bytes it is owed), summed in rank order,
//            scaled, rounded once to bf16 and stored.
// The result is deterministic; no global workspace, atomics or zeroed output.
//
// Replaces _skinny_gemm_kernel and its producer/consumer waves
// (projects/skinny_gemm/skinny_gemm_kernel.cu:6-110, producers/, consumers/ in
// the reference project) and the launchers of skinny_gemm_caller.cu.
#include <cuda_bf16.h>

#include <cstring>
#include <mutex>

#include "host_util.h"
#include "ptx.cuh"

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace skinny {

constexpr int BK = 128;                    // K bytes per stage = one 128-byte swizzle row
constexpr int MAX_R = 256;                 // weight rows per CTA tile (UMMA N)
constexpr int NUM_THREADS = 192;
constexpr int TMEM_WARP = 4;               // warp 4 -> TMEM lane quadrant 0 (lanes 0..31 = rows m)
constexpr int MAX_STAGES = 16;
constexpr int BAR_BYTES = 512;
constexpr int A_OPERAND_SPAN = 128 * BK;   // bytes the MMA reads for its 128-row A operand
constexpr int SMEM_LIMIT = 232448;         // 227 KiB opt-in maximum per CTA

__host__ __device__ constexpr int red_bytes(int mpad, int R, int S) {
    // [src rank][m][cols per rank] fp32, cols per rank = 4 * ceil((R/4)/S)
    const int cpr = 4 * ((R / 4 + S - 1) / S);
    const int b = S * mpad * cpr * 4;
    return b < A_OPERAND_SPAN ? A_OPERAND_SPAN : b;   // also pads the last stage's A-operand read
}
__host__ __device__ constexpr int stage_bytes(int mpad, int R) { return (mpad + R) * BK; }
__host__ __device__ constexpr int smem_bytes(int mpad, int R, int S, int stages) {
    return 1024 + stages * stage_bytes(mpad, R) + red_bytes(mpad, R, S) + BAR_BYTES;
}

// Granule (4 columns) ownership when G granules are cut into S chunks [G*c/S, G*(c+1)/S).
__device__ __forceinline__ int chunk_begin(int c, int G, int S) { return (G * c) / S; }
__device__ __forceinline__ int chunk_of(int g, int G, int S) { return (g * S + S - 1) / G; }

struct Params {
    __nv_bfloat16* D;
    const float* scale_a;
    const float* scale_b;
    int* status;
    int M, N;
    int num_kb;      // ceil(K / 128)
    int R;           // rows per tile
    int nstages;
    int tmem_cols;
    int pdl;         // launched with programmatic stream serialization
    int mma_m;       // UMMA M for batches of up to 16 rows: 64 (or 128)
    unsigned long long* trace;   // optional [cta][8] %globaltimer stamps (diagnostics), else nullptr
};

// Trace slots (nanoseconds of %globaltimer), one row of 12 per CTA.
enum { TR_ENTRY = 0, TR_SETUP = 1, TR_PRIOR_DONE = 2, TR_FIRST_FULL = 3, TR_LAST_FULL = 4, TR_ACC_DONE = 5,
       TR_EXCHANGED = 6, TR_EXIT = 7, TR_EPI_READY = 8, TR_EPI_LOADED = 9, TR_EPI_STORED = 10 };
__device__ __forceinline__ void stamp(const Params& p, int slot) {
    if (p.trace) p.trace[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 12 + slot] = globaltimer_ns();
}

// Store 4 consecutive outputs of row m starting at column n (n % 4 == 0 within the tile).
__device__ __forceinline__ void store4(__nv_bfloat16* D, int N, int m, int n, float a, float b, float c, float d,
                                       bool vec_ok) {
    __nv_bfloat16* p = D + static_cast<size_t>(m) * N + n;
    if (vec_ok && n + 3 < N) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    } else {
        if (n < N) p[0] = __float2bfloat16_rn(a);
        if (n + 1 < N) p[1] = __float2bfloat16_rn(b);
        if (n + 2 < N) p[2] = __float2bfloat16_rn(c);
        if (n + 3 < N) p[3] = __float2bfloat16_rn(d);
    }
}

template <int MPAD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    if (threadIdx.x == 0) stamp(p, TR_ENTRY);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int S = gridDim.x;               // cluster = the K slices of one tile
    const int rank = blockIdx.x;
    const int R = p.R;
    const int n0 = blockIdx.y * R;
    const int nstages = p.nstages;
    const int kb_begin = static_cast<int>((static_cast<long long>(p.num_kb) * rank) / S);
    const int kb_end = static_cast<int>((static_cast<long long>(p.num_kb) * (rank + 1)) / S);
    const int nkb = kb_end - kb_begin;
    const int STAGE = stage_bytes(MPAD, R);
    constexpr int A_BYTES = MPAD * BK;

    float* red = reinterpret_cast<float*>(smem + nstages * STAGE);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + red_bytes(MPAD, R, S));
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + MAX_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * MAX_STAGES);
    const uint32_t xbar = smem_u32(bars + 2 * MAX_STAGES + 1);   // split-K partials have arrived
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile float* sc_s = reinterpret_cast<volatile float*>(tmem_slot + 2);   // scale_a * scale_b, fetched early
    const uint32_t stage0 = smem_u32(smem);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmA);
        for (int s = 0; s < nstages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(xbar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        if (S > 1) {                       // bytes this rank is owed: S ranks x M rows x its granules x 16 B
            const int G_ = R / 4;
            const int ng_ = (G_ * (rank + 1)) / S - (G_ * rank) / S;
            mbar_arrive_expect_tx(xbar, static_cast<uint32_t>(S) * p.M * ng_ * 16u);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) stamp(p, TR_SETUP);
    if (S > 1) cluster_arrive_release();   // phase 1: "my shared memory is live"
    if (p.pdl) pdl_launch_dependents();    // the next kernel in the stream may start its prologue

    if (warp == 0) {
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first();
            const uint64_t pol_a = l2_policy_evict_last();
            // Weights never depend on the preceding kernel: the first ring-full
            // of weight boxes is requested before waiting for it to finish.
            const int pre = nkb < nstages ? nkb : nstages;
            for (int i = 0; i < pre; i++) {
                mbar_arrive_expect_tx(full0 + 8 * i, STAGE);
                tma_load_2d(stage0 + i * STAGE + A_BYTES, &tmW, (kb_begin + i) * BK, n0, full0 + 8 * i, pol_w);
            }
            if (p.pdl) pdl_wait_prior();   // activations may be the preceding kernel's output
            stamp(p, TR_PRIOR_DONE);
            for (int i = 0; i < pre; i++)
                tma_load_2d(stage0 + i * STAGE, &tmA, (kb_begin + i) * BK, 0, full0 + 8 * i, pol_a);
            for (int i = pre; i < nkb; i++) {
                const int s = i % nstages;
                const uint32_t ph = (i / nstages) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { *abort_flag = 1; report_timeout(p.status); break; }
                const uint32_t dst = stage0 + s * STAGE;
                mbar_arrive_expect_tx(full0 + 8 * s, STAGE);
                tma_load_2d(dst + A_BYTES, &tmW, (kb_begin + i) * BK, n0, full0 + 8 * s, pol_w);
                tma_load_2d(dst, &tmA, (kb_begin + i) * BK, 0, full0 + 8 * s, pol_a);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // 64-row MMAs for batches of up to 16 rows: rows 0-15 of a 64-row accumulator lie in TMEM lanes 0-15, where
            // the epilogue reads them; half the padded tensor work of a 128-row MMA, hence less power
            const uint32_t idesc = idesc_e4m3_f32(MPAD == 16 ? p.mma_m : 128, R);
            for (int i = 0; i < nkb; i++) {
                const int s = i % nstages;
                const uint32_t ph = (i / nstages) & 1;
                if (!mbar_wait(full0 + 8 * s, ph)) { *abort_flag = 1; report_timeout(p.status); break; }
                tc_fence_after_sync();
                if (i == 0) stamp(p, TR_FIRST_FULL);
                if (i == nkb - 1) stamp(p, TR_LAST_FULL);
                const uint32_t a = stage0 + s * STAGE;
                const uint32_t w = a + A_BYTES;
#pragma unroll
                for (int ks = 0; ks < BK / 32; ks++)
                    tc_mma_f8(tmem_base, smem_desc_k128(a + ks * 32), smem_desc_k128(w + ks * 32), idesc,
                              (i | ks) != 0);
                tc_commit(empty0 + 8 * s);   // the stage is free once these MMAs have read it
            }
            tc_commit(tmem_full);            // accumulator complete (also fires after an abort)
        }
        __syncwarp();
    } else if (warp == 2) {
        // An otherwise idle warp fetches the two scales while the weights stream,
        // so that their global-load latency is off the epilogue's critical path.
        if (lane == 0) {
            if (p.pdl) pdl_wait_prior();   // the scales may be the preceding kernel's output
            *sc_s = __ldg(p.scale_a) * __ldg(p.scale_b);
        }
        __syncwarp();
    }

    const bool vec_ok = (p.N % 4 == 0);
    const int G = R / 4;                   // 4-column granules of the tile
    const int cpr = 4 * ((G + S - 1) / S); // columns per rank chunk (upper bound)

    // ---- epilogue.  This code runs once per CTA, so it is kept compact (small
    // loops, every thread busy): long unrolled straight-line code executed once
    // runs at instruction-cache-miss speed.
    // Step 1 - warps 0 and 4 (the two warps that may read TMEM lanes 0..31,
    // lane = output row m) move the accumulator into a staging tile stg[m][R]
    // (fp32, row pitch R+4) that reuses the drained pipeline stages.
    float* stg = reinterpret_cast<float*>(smem);
    const int pitch = R + 4;
    if ((warp & 3) == 0) {
        bool ok = mbar_wait(tmem_full, 0);
        if (!ok) { *abort_flag = 1; report_timeout(p.status); }
        ok = ok && (*abort_flag == 0);
        tc_fence_after_sync();
        if (warp == TMEM_WARP && lane == 0) stamp(p, TR_ACC_DONE);
        if (ok) {
            float* row = stg + lane * pitch;
            const int half = warp == 0 ? 0 : 1;
            for (int c0 = half * 32; c0 + 32 <= R; c0 += 64) {
                float v[32];
                tmem_ld32(tmem_base + c0, v);
                if (lane < MPAD) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<float4*>(row + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
            if ((R & 31) != 0 && ((R >> 5) & 1) == half) {   // 16-column tail (R is a multiple of 16)
                const int c0 = R & ~31;
                float v[16];
                tmem_ld16(tmem_base + c0, v);
                if (lane < MPAD) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        *reinterpret_cast<float4*>(row + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
        }
        if (warp == TMEM_WARP && lane == 0) stamp(p, TR_EPI_LOADED);
    }
    if (S > 1) cluster_wait_acquire();     // phase 1 complete: every peer's barriers and buffers are live
    if (p.pdl) pdl_wait_prior();           // D and the scales may belong to the preceding kernel
    __syncthreads();
    const float sc = *sc_s;

    if (S == 1) {
        // Step 2 - every thread converts and stores 8 consecutive outputs.
        const bool vec8 = (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.D) & 15u) == 0);
        const int groups = R >> 3;
        if (*abort_flag == 0) {
            for (int item = threadIdx.x; item < p.M * groups; item += NUM_THREADS) {
                const int m = item / groups, c = (item - m * groups) << 3;
                const float4 lo = *reinterpret_cast<const float4*>(stg + m * pitch + c);
                const float4 hi = *reinterpret_cast<const float4*>(stg + m * pitch + c + 4);
                const int n = n0 + c;
                if (vec8 && n + 7 < p.N) {
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(lo.x * sc, lo.y * sc), b1 = __floats2bfloat162_rn(lo.z * sc, lo.w * sc);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(hi.x * sc, hi.y * sc), b3 = __floats2bfloat162_rn(hi.z * sc, hi.w * sc);
                    uint4 o;
                    o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
                    o.z = *reinterpret_cast<uint32_t*>(&b2); o.w = *reinterpret_cast<uint32_t*>(&b3);
                    *reinterpret_cast<uint4*>(p.D + static_cast<size_t>(m) * p.N + n) = o;
                } else {
                    store4(p.D, p.N, m, n, lo.x * sc, lo.y * sc, lo.z * sc, lo.w * sc, vec_ok);
                    store4(p.D, p.N, m, n + 4, hi.x * sc, hi.y * sc, hi.z * sc, hi.w * sc, vec_ok);
                }
            }
        }
        if (threadIdx.x == 0) stamp(p, TR_EPI_STORED);
    } else {
        // Step 2 - thread t owns granule column g = t % 64 (4 accumulator columns)
        // and pushes rows m = t/64, t/64 + 3, ... of it to the rank that owns
        // that column, each 16-byte store signalling the owner's mbarrier.  The
        // push also runs after an abort (with whatever the staging tile holds) so
        // that no peer is left waiting for bytes.
        {
            const int g = threadIdx.x & 63;
            if (g < G) {
                const int owner = chunk_of(g, G, S);
                const int col = (g - chunk_begin(owner, G, S)) << 2;
                const uint32_t dst0 = mapa_smem(smem_u32(red + static_cast<size_t>(rank) * MPAD * cpr + col), owner);
                const uint32_t rbar = mapa_smem(xbar, owner);
                for (int m = threadIdx.x >> 6; m < p.M; m += NUM_THREADS / 64) {
                    const float4 v = *reinterpret_cast<const float4*>(stg + m * pitch + (g << 2));
                    st_async_v4(dst0 + m * cpr * 4, v.x, v.y, v.z, v.w, rbar);
                }
            }
        }
        if (threadIdx.x == 0) stamp(p, TR_EPI_STORED);
        // Step 3 - wait for the partials of my column chunk, sum them in rank order.
        if (!mbar_wait(xbar, 0)) { *abort_flag = 1; report_timeout(p.status); }
        if (threadIdx.x == 0) stamp(p, TR_EXCHANGED);
        if (*abort_flag == 0) {
            const int gb = chunk_begin(rank, G, S);
            const int ng = chunk_begin(rank + 1, G, S) - gb;
            for (int item = threadIdx.x; item < p.M * ng; item += NUM_THREADS) {
                const int m = item / ng, g = item - m * ng;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int src = 0; src < S; src++) {
                    const float4 v = *reinterpret_cast<const float4*>(red + (static_cast<size_t>(src) * MPAD + m) * cpr + g * 4);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                store4(p.D, p.N, m, n0 + (gb + g) * 4, sum.x * sc, sum.y * sc, sum.z * sc, sum.w * sc, vec_ok);
            }
        }
    }

    // ---- teardown: after an abort give in-flight TMA copies time to land
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
    if (threadIdx.x == 0) stamp(p, TR_EXIT);
}

// Diagnostics: when a trace buffer is registered, launch i writes its CTA
// stamps into slot i % slots (each slot holds up to ctas_per_slot CTAs).
static unsigned long long* g_trace = nullptr;
static int g_trace_slots = 0, g_trace_ctas = 0, g_trace_next = 0;

// How many clusters of `cluster` CTAs with `smem` bytes each can be resident
// at once on the current device (GPC placement limits make this smaller than
// SMs / cluster for the larger sizes).  Cached per (mpad, cluster, smem KiB).
template <int MPAD>
static int query_max_clusters(int cluster, int smem) {
    auto kernel = skinny_gemm_kernel<MPAD>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess) return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
    return n;
}

static int max_clusters(int mpad, int cluster, int smem) {
    static int cache[kMaxDevices][2][9][64];
    static bool init = false;
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    const int kib = (smem + 4095) / 4096;      // 4 KiB buckets
    std::lock_guard<std::mutex> lk(mu);
    if (!init) { memset(cache, 0, sizeof(cache)); init = true; }
    int& slot = cache[dev][mpad == 16 ? 0 : 1][cluster][kib < 64 ? kib : 63];
    if (slot == 0) {
        const int n = mpad == 16 ? query_max_clusters<16>(cluster, kib * 4096 > SMEM_LIMIT ? SMEM_LIMIT : kib * 4096)
                                 : query_max_clusters<32>(cluster, kib * 4096 > SMEM_LIMIT ? SMEM_LIMIT : kib * 4096);
        slot = n + 1;                          // 0 = not yet queried
    }
    return slot - 1;
}

// ------------------------------------------------------------------ planning
struct Plan {
    int mpad, R, tiles, split_k, stages, tmem_cols;
};

// Resident-cluster limits measured on B200 (148 SMs) for cluster sizes 1..8,
// used when no device is available to ask (host-only planning).
static const int kDefaultMaxClusters[9] = {0, 148, 74, 45, 33, 26, 22, 15, 15};

// Cost model from measurements on B200: TMA delivers ~60 GB/s into one SM, an
// MMA instruction costs ~74 ns whatever its N (four per 128-byte K block, plus
// ~60 ns of barrier hand-off), the whole chip streams ~6.3 TB/s, and a split-K
// exchange adds about half a microsecond.
static double plan_cost(int R, int kb_per, int S, int ctas, double total_bytes) {
    const double t_tma = R * 128.0 / 60e9, t_mma = 4 * 74e-9 + 60e-9;
    const double t_cta = kb_per * (t_tma > t_mma ? t_tma : t_mma);
    const double t_hbm = total_bytes / 6.3e12;
    // ties (HBM-bound either way) go to the plan that keeps more SMs streaming
    return (t_cta > t_hbm ? t_cta : t_hbm) + (S > 1 ? 0.5e-6 : 0.0) + 2e-9 * (ctas < 148 ? 148 - ctas : 0);
}

// max_clusters[S] = clusters of S CTAs that can be resident at once (one per SM).
static Plan make_plan(int M, int N, int K, const int* max_clusters, int split_k_hint, int stages_hint,
                      int rows_hint) {
    Plan best = {};
    best.mpad = M <= 16 ? 16 : 32;
    const int num_kb = (K + BK - 1) / BK;
    double best_cost = 1e30;
    if (split_k_hint > num_kb) split_k_hint = num_kb;
    const int s_lo = split_k_hint > 0 ? split_k_hint : 1;
    const int s_hi = split_k_hint > 0 ? split_k_hint : 8;
    const int t_min = (N + MAX_R - 1) / MAX_R;
    for (int S = s_lo; S <= s_hi; S++) {
        if (S > num_kb && S > 1) continue;
        int t_max = max_clusters[S];
        if (t_max < t_min) t_max = t_min;      // more tiles than fit at once: several waves
        for (int T = t_min; T <= t_max; T++) {
            int R = ((N + T - 1) / T + 15) / 16 * 16;
            if (rows_hint > 0) R = rows_hint;
            if (R > MAX_R) continue;
            const int tiles = (N + R - 1) / R;
            const int kb_per = (num_kb + S - 1) / S;
            const int waves = (tiles + max_clusters[S] - 1) / max_clusters[S];
            const double c = waves * plan_cost(R, kb_per, S, tiles * S, static_cast<double>(N) * K / waves);
            if (c < best_cost) {
                best_cost = c;
                best.R = R;
                best.tiles = tiles;
                best.split_k = S;
            }
            if (rows_hint > 0) break;
        }
    }
    best.tmem_cols = best.R <= 32 ? 32 : best.R <= 64 ? 64 : best.R <= 128 ? 128 : 256;
    const int kb_per = (num_kb + best.split_k - 1) / best.split_k;
    // Ring depth from a sweep on B200: with split-K (short per-CTA streams)
    // ~4 stages, small enough for the CTAs of two consecutive launches to share
    // an SM; without it (long streams) ~6 stages of bytes in flight.
    int st = best.split_k > 1 ? 4 : 6;
    if (stages_hint > 0) st = stages_hint;
    while (st > 1 && smem_bytes(best.mpad, best.R, best.split_k, st) > SMEM_LIMIT) st--;
    if (st > MAX_STAGES) st = MAX_STAGES;
    if (st > kb_per) st = kb_per;
    if (st < 1) st = 1;
    best.stages = st;
    return best;
}

template <int MPAD>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmA, const Params& prm, const Plan& pl, bool pdl,
                  cudaStream_t stream) {
    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = skinny_gemm_kernel<MPAD>;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess)
            return RDB_CUDA_ERROR;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.split_k, pl.tiles, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes(pl.mpad, pl.R, pl.split_k, pl.stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.split_k;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmW, tmA, prm);
    return e == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

static int run(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, uint16_t* D, int M, int N, int K,
               int ldb, int rows_hint, int split_k_hint, int stages_hint, unsigned flags, cudaStream_t stream) {
    if (M < 1 || N < 1 || K < 1 || ldb < K) return RDB_BAD_SHAPE;
    if (M > 32) return RDB_M_ABOVE_WARPTILE_M;
    if (N % 2 != 0) return RDB_N_NOT_EVEN;
    if (K % 16 != 0 || ldb % 16 != 0) return RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K;
    if (!aligned16(A) || !aligned16(B) || (reinterpret_cast<uintptr_t>(D) & 7u)) return RDB_BAD_ALIGNMENT;
    if (split_k_hint < 0 || split_k_hint > 8 || stages_hint < 0 || rows_hint < 0 || rows_hint > MAX_R ||
        rows_hint % 16 != 0)
        return RDB_INVALID_CONFIG;
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;

    int maxc[9] = {0};
    const int mpad = M <= 16 ? 16 : 32;
    for (int c = 1; c <= 8; c++) {
        maxc[c] = max_clusters(mpad, c, 112 * 1024);
        if (maxc[c] <= 0) maxc[c] = kDefaultMaxClusters[c] * info->sm_count / 148;
        if (maxc[c] < 1) maxc[c] = 1;
    }
    // no knobs from the caller: a measured entry of the tuning table goes before the cost model
    if (rows_hint == 0 && split_k_hint == 0 && stages_hint == 0) lookup_skinny_plan(mpad, N, K, &rows_hint, &split_k_hint, &stages_hint);
    const Plan pl = make_plan(M, N, K, maxc, split_k_hint, stages_hint, rows_hint);
    CUtensorMap tmW, tmA;
    int r = make_tmap_2d(&tmW, B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, BK, pl.R, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != RDB_SUCCESS) return r;
    r = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, K, BK, pl.mpad, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != RDB_SUCCESS) return r;
    Params prm;
    prm.D = reinterpret_cast<__nv_bfloat16*>(D);
    prm.scale_a = sa;
    prm.scale_b = sb;
    prm.status = info->status_dev;
    prm.M = M;
    prm.N = N;
    prm.num_kb = (K + BK - 1) / BK;
    prm.R = pl.R;
    prm.nstages = pl.stages;
    prm.tmem_cols = pl.tmem_cols;
    const bool pdl = (flags & RDB_SKINNY_OVERLAP_PRIOR_KERNEL) != 0;
    prm.pdl = pdl ? 1 : 0;
    static const bool force128 = [] { const char* v = getenv("RDB_SKINNY_MMA_M"); return v && v[0] == '1'; }();
    prm.mma_m = force128 ? 128 : 64;
    prm.trace = nullptr;
    if (g_trace && pl.tiles * pl.split_k <= g_trace_ctas) {
        prm.trace = g_trace + static_cast<size_t>(g_trace_next % g_trace_slots) * g_trace_ctas * 12;
        g_trace_next++;
    }
    if (pl.mpad == 16) return launch<16>(tmW, tmA, prm, pl, pdl, stream);
    return launch<32>(tmW, tmA, prm, pl, pdl, stream);
}

// Device staging of the host-buffer entry: one set of buffers per device, grown
// on demand and kept until the process exits.
struct HostStaging {
    uint8_t* a = nullptr;
    uint8_t* b = nullptr;
    uint16_t* d = nullptr;
    float* scales = nullptr;
    size_t a_cap = 0, b_cap = 0, d_cap = 0;
};

template <class T>
static bool grow(T*& ptr, size_t& cap, size_t need) {
    if (need <= cap) return true;
    if (ptr && cudaFree(ptr) != cudaSuccess) return false;
    ptr = nullptr;
    cap = 0;
    if (cudaMalloc(reinterpret_cast<void**>(&ptr), need) != cudaSuccess) { cudaGetLastError(); return false; }
    cap = need;
    return true;
}

static int run_host(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, uint16_t* D, int M, int N, int K,
                    int ldb, cudaStream_t stream) {
    if (!A || !B || !sa || !sb || !D) return RDB_INVALID_CONFIG;
    if (M < 1 || N < 1 || K < 1 || ldb < K) return RDB_BAD_SHAPE;
    static HostStaging staging[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RDB_CUDA_ERROR;
    std::lock_guard<std::mutex> lk(mu);       // one host-buffer call per process at a time: they share the staging
    HostStaging& st = staging[dev];
    const size_t a_bytes = static_cast<size_t>(M) * K, b_bytes = static_cast<size_t>(N) * K;
    const size_t d_bytes = static_cast<size_t>(M) * N * sizeof(uint16_t);
    size_t sc_cap = st.scales ? 8 : 0;
    if (!grow(st.a, st.a_cap, a_bytes) || !grow(st.b, st.b_cap, b_bytes) || !grow(st.d, st.d_cap, d_bytes) ||
        !grow(st.scales, sc_cap, 8))
        return RDB_CUDA_ERROR;
    bool ok = cudaMemcpyAsync(st.a, A, a_bytes, cudaMemcpyHostToDevice, stream) == cudaSuccess;
    // the weights land K-contiguous with pitch K whatever the host pitch was
    ok = ok && cudaMemcpy2DAsync(st.b, K, B, ldb, K, N, cudaMemcpyHostToDevice, stream) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(st.scales, sa, sizeof(float), cudaMemcpyHostToDevice, stream) == cudaSuccess;
    ok = ok && cudaMemcpyAsync(st.scales + 1, sb, sizeof(float), cudaMemcpyHostToDevice, stream) == cudaSuccess;
    if (!ok) { cudaGetLastError(); return RDB_CUDA_ERROR; }
    const int r = run(st.a, st.b, st.scales, st.scales + 1, st.d, M, N, K, K, 0, 0, 0, 0, stream);
    if (r != RDB_SUCCESS) return r;
    if (cudaMemcpyAsync(D, st.d, d_bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {
        cudaGetLastError();
        return RDB_CUDA_ERROR;
    }
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (info && *reinterpret_cast<volatile int*>(info->status_host) == RDB_DEVICE_TIMEOUT) return RDB_DEVICE_TIMEOUT;
    return RDB_SUCCESS;
}

}  // namespace skinny
}  // namespace rdb

extern "C" {

int rdb_skinny_gemm_fp8(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b, uint16_t* D,
                        int M, int N, int K, int ldb, void* stream) {
    return rdb::skinny::run(A, B, scale_a, scale_b, D, M, N, K, ldb, 0, 0, 0, 0, static_cast<cudaStream_t>(stream));
}

int rdb_skinny_gemm_fp8_host(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b, uint16_t* D,
                             int M, int N, int K, int ldb, void* stream) {
    return rdb::skinny::run_host(A, B, scale_a, scale_b, D, M, N, K, ldb, static_cast<cudaStream_t>(stream));
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
    return rdb::skinny::run(A, B, scale_a, scale_b, D, M, N, K, ldb, 0, split_k < 0 ? 0 : split_k, qsize, 0,
                            static_cast<cudaStream_t>(stream));
}

int rdb_skinny_gemm_trace(unsigned long long* device_buffer, int slots, int ctas_per_slot) {
    if (device_buffer && (slots < 1 || ctas_per_slot < 1)) return RDB_BAD_SHAPE;
    rdb::skinny::g_trace = device_buffer;
    rdb::skinny::g_trace_slots = slots;
    rdb::skinny::g_trace_ctas = ctas_per_slot;
    rdb::skinny::g_trace_next = 0;
    return RDB_SUCCESS;
}

int rdb_skinny_gemm_max_clusters(int M, int cluster_size, int smem_bytes) {
    if (M < 1 || M > 32 || cluster_size < 1 || cluster_size > 8 || smem_bytes < 0 || smem_bytes > rdb::skinny::SMEM_LIMIT)
        return -1;
    return rdb::skinny::max_clusters(M <= 16 ? 16 : 32, cluster_size, smem_bytes);
}

int rdb_skinny_gemm_plan(int M, int N, int K, int sm_count, int* rows_per_tile, int* split_k, int* stages) {
    if (M < 1 || M > 32 || N < 1 || K < 1 || sm_count < 1) return RDB_BAD_SHAPE;
    int maxc[9] = {0};
    for (int c = 1; c <= 8; c++) {
        maxc[c] = rdb::skinny::kDefaultMaxClusters[c] * sm_count / 148;
        if (maxc[c] < 1) maxc[c] = 1;
    }
    int rows_hint = 0, split_hint = 0, stages_hint = 0;
    rdb::lookup_skinny_plan(M <= 16 ? 16 : 32, N, K, &rows_hint, &split_hint, &stages_hint);     // a tuned entry wins
    const rdb::skinny::Plan pl = rdb::skinny::make_plan(M, N, K, maxc, split_hint, stages_hint, rows_hint);
    if (rows_per_tile) *rows_per_tile = pl.R;
    if (split_k) *split_k = pl.split_k;
    if (stages) *stages = pl.stages;
    return RDB_SUCCESS;
}

int rdb_skinny_gemm_fp8_tuned(const uint8_t* A, const uint8_t* B, const float* scale_a, const float* scale_b,
                              uint16_t* D, int M, int N, int K, int ldb, int rows_per_tile, int split_k, int stages,
                              unsigned flags, void* stream) {
    return rdb::skinny::run(A, B, scale_a, scale_b, D, M, N, K, ldb, rows_per_tile, split_k, stages, flags,
                            static_cast<cudaStream_t>(stream));
}

}  // extern "C"
