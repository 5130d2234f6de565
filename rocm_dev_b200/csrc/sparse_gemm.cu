// 2:4 structured-sparse FP8 GEMM for sm_100a:
//   D[M,N] = bf16( (A . W^T) * sa * sb ),  W [N,K] with two non-zeros in every aligned group of four along K.
//
// The reference's async_gemm_sparse project (projects/async_gemm_sparse/
// sparse_k.cu:5-75, consumer.cu:29-162) issues the *sparse* MFMA with constant
// fake indices as a trick to run a dense 8-row tile; it holds no pruning,
// compression or metadata code.  This file is the real thing: the weights are
// stored compressed (values [N,K/2] + 2-bit positions), halving the bytes that
// must cross HBM, and multiplied with tcgen05.mma.sp kind::f8f6f4.
//
// The sparse operand must be the MMA's A operand, so the problem is computed
// transposed ("swap-AB"): a CTA owns 128 weight rows (TMEM lanes), the padded
// batch is the MMA N extent (TMEM columns).  Per 128-byte compressed K block
// (256 logical K) a stage holds: the compressed values (128 x 128 B, TMA,
// SWIZZLE_128B), two activation boxes (NB x 128 B each), and two 2 KiB metadata
// atoms ([128 rows][16 B], bulk-copied), which an issuing thread moves into TMEM
// with tcgen05.cp.128x128b before issuing four tcgen05.mma.sp (K = 64 each).
// Two threads issue (even and odd k-blocks, an accumulator each, added in the
// epilogue): one thread's per-stage cost, not memory, had set the pace.
// K may be split over a cluster of 2 or 4 CTAs (small batches); the partials are
// exchanged through distributed shared memory with st.async and summed in rank
// order.  One launch computes a list of GEMMs that share the batch size
// (blockIdx.y walks the tiles of all of them); a single call is a list of one.
#include <cuda_bf16.h>

#include <cstring>

#include "host_util.h"
#include "ptx.cuh"

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace sparse {

constexpr int BM = 128;                 // weight rows per CTA (UMMA M)
constexpr int BKC = 128;                // compressed K bytes per stage (256 logical K elements)
constexpr int A_BYTES = BM * BKC;       // 16 KiB of compressed values
constexpr int ATOM_BYTES = 2048;        // metadata atom: 128 rows x 16 B = 128 logical K
constexpr int E_BYTES = 2 * ATOM_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_LIMIT = 232448;
// TMEM: two accumulators (even and odd k-blocks) of NB columns, a multiple of 32 apart, then 8 metadata columns per
// stage; the allocation is the next power of two, so a narrow batch leaves TMEM (and, with a short ring, shared memory) for a second CTA on the SM

__host__ __device__ constexpr int stage_bytes(int NB) { return A_BYTES + 2 * NB * 128 + E_BYTES; }
__host__ __device__ constexpr int red_bytes(int NB, int S) { return S > 1 ? BM * NB * 4 : 0; }   // [S][NB][128/S rows]
__host__ __device__ constexpr int stg_bytes(int NB) { return NB * (BM + 4) * 4; }   // [NB][128 + 4]: one line per batch row
__host__ __device__ inline int smem_bytes(int NB, int S, int stages) {
    int ring = stages * stage_bytes(NB);
    if (ring < stg_bytes(NB)) ring = stg_bytes(NB);     // the staging tile reuses the drained ring
    return 1024 + ring + red_bytes(NB, S) + BAR_BYTES;
}

struct Params {
    __nv_bfloat16* D;
    const uint8_t* meta;       // packed metadata: [N/128 tiles][K/128 atoms][128 rows][16 B]
    const float* scale_a;
    const float* scale_b;
    int* status;
    int M, N;
    int num_kb;                // K / 256
    int NB;                    // padded batch columns per CTA (UMMA N); blockIdx.z selects the batch block
    int nstages;
    int ring_bytes;
    int pdl;                   // launched with programmatic stream serialization
    int te_col, tmem_cols;     // first metadata column, allocated columns (power of two)
    int acc_stride;            // column distance between the accumulators
    int issuers;               // MMA-issuing threads (2 or 4), each with its own accumulator and every issuers-th k-block
    unsigned long long* trace; // optional: 8 %globaltimer stamps of the launch's first CTA (diagnostics), else nullptr
};

// A launch computes a LIST of GEMMs that share the batch (M) and the configuration: blockIdx.y walks the 128-row
// tiles of all problems one after the other, so the CTAs of a later problem start as SMs fall free - no launch gap,
// and set-up, first loads and epilogues of different CTAs overlap one another's streams.
constexpr int kMaxProblems = 8;
struct Prob {
    CUtensorMap tmW, tmX;
    __nv_bfloat16* D;
    const uint8_t* meta;
    const float* scale_a;
    const float* scale_b;
    int N, num_kb, tile_begin;
};
struct GParams {
    Prob prob[kMaxProblems];
    int count;
    Params common;             // D, meta, scales, N and num_kb are taken from the CTA's problem
};

// entry, set-up done, first stage full, last stage's MMAs issued, accumulator complete, partials exchanged, stores issued, exit
__device__ __forceinline__ void stamp(const Params& p, int slot) {
    if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.trace[slot] = globaltimer_ns();
}

// e4m3 x e4m3 -> f32, K-major operands, sparse A.
__host__ __device__ constexpr uint32_t idesc_sparse(int umma_m, int umma_n) {
    return (1u << 2) | (1u << 4) | (static_cast<uint32_t>(umma_n >> 3) << 17) | (static_cast<uint32_t>(umma_m >> 4) << 24);
}

// Shared-memory descriptor of one metadata atom: no swizzle, 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t smem_desc_meta(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void tmem_cp_128x128b(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void tc_mma_sp_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t tmem_e,
                                             uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.sp.cta_group::1.kind::f8f6f4 [%0], %1, %2, [%3], %4, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(tmem_e), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
        : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
sparse_gemm_kernel(const __grid_constant__ GParams g) {
    int pi = 0;
    while (pi + 1 < g.count && static_cast<int>(blockIdx.y) >= g.prob[pi + 1].tile_begin) pi++;
    const Prob& pr = g.prob[pi];
    const CUtensorMap& tmW = pr.tmW;
    const CUtensorMap& tmX = pr.tmX;
    Params p = g.common;
    p.D = pr.D;
    p.meta = pr.meta;
    p.scale_a = pr.scale_a;
    p.scale_b = pr.scale_b;
    p.N = pr.N;
    p.num_kb = pr.num_kb;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = gridDim.x, rank = blockIdx.x;      // cluster = K slices of one tile
    if (threadIdx.x == 0) stamp(p, 0);
    const int tile = static_cast<int>(blockIdx.y) - pr.tile_begin, n0 = tile * BM;
    const int m0 = blockIdx.z * p.NB;                 // first batch row of this CTA
    const int m_count = p.M - m0 < p.NB ? p.M - m0 : p.NB;
    const int NB = p.NB, nstages = p.nstages;
    const int STAGE = stage_bytes(NB);
    const int kb_begin = static_cast<int>((static_cast<long long>(p.num_kb) * rank) / S);
    const int kb_end = static_cast<int>((static_cast<long long>(p.num_kb) * (rank + 1)) / S);
    const int nkb = kb_end - kb_begin;

    float* red = reinterpret_cast<float*>(smem + p.ring_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + red_bytes(NB, S));
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + MAX_STAGES);
    const uint32_t tmem_full = smem_u32(bars + 2 * MAX_STAGES), xbar = smem_u32(bars + 2 * MAX_STAGES + 1);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* sc_slot = reinterpret_cast<float*>(tmem_slot + 2);
    const uint32_t stage0 = smem_u32(smem);
    const int rows_per = BM / S;                      // S is 1, 2 or 4

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmX);
        for (int s = 0; s < nstages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tmem_full, p.issuers);              // one commit from each issuing thread
        mbar_init(xbar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        if (S > 1) mbar_arrive_expect_tx(xbar, static_cast<uint32_t>(S) * rows_per * NB * 4u);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) stamp(p, 1);
    if (S > 1) cluster_arrive_release();              // phase 1: "my barriers and buffers are live"
    if (p.pdl) pdl_launch_dependents();               // the next kernel in the stream may start its prologue

    if (warp == 0) {
        if (lane == 0) {
            // with several batch blocks the weights are read once per block: keep them in L2 for the sibling
            const uint64_t pol_w = gridDim.z > 1 ? l2_policy_evict_last() : l2_policy_evict_first(), pol_x = l2_policy_evict_last();
            const uint8_t* meta_tile = p.meta + static_cast<size_t>(tile) * (2 * p.num_kb) * ATOM_BYTES;
            // The compressed weights and their metadata never depend on the preceding kernel: the first ring-full is
            // requested before waiting for that kernel to finish; the activations may be its output.
            const int pre = nkb < nstages ? nkb : nstages;
            for (int i = 0; i < pre; i++) {
                const int kb = kb_begin + i;
                const uint32_t dst = stage0 + i * STAGE, bar = full0 + 8 * i;
                mbar_arrive_expect_tx(bar, STAGE);
                tma_load_2d(dst, &tmW, kb * BKC, n0, bar, pol_w);
                bulk_load(dst + A_BYTES + 2 * NB * 128, meta_tile + static_cast<size_t>(2 * kb) * ATOM_BYTES, E_BYTES, bar);
            }
            if (p.pdl) pdl_wait_prior();
            for (int i = 0; i < pre; i++) {
                const int kb = kb_begin + i;
                const uint32_t dst = stage0 + i * STAGE, bar = full0 + 8 * i;
                tma_load_2d(dst + A_BYTES, &tmX, kb * 256, m0, bar, pol_x);
                tma_load_2d(dst + A_BYTES + NB * 128, &tmX, kb * 256 + 128, m0, bar, pol_x);
            }
            for (int i = pre; i < nkb; i++) {
                const int s = i % nstages;
                const uint32_t ph = (i / nstages) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { *abort_flag = 1; report_timeout(p.status); break; }
                const int kb = kb_begin + i;
                const uint32_t dst = stage0 + s * STAGE, bar = full0 + 8 * s;
                mbar_arrive_expect_tx(bar, STAGE);
                tma_load_2d(dst, &tmW, kb * BKC, n0, bar, pol_w);
                tma_load_2d(dst + A_BYTES, &tmX, kb * 256, m0, bar, pol_x);
                tma_load_2d(dst + A_BYTES + NB * 128, &tmX, kb * 256 + 128, m0, bar, pol_x);
                bulk_load(dst + A_BYTES + 2 * NB * 128, meta_tile + static_cast<size_t>(2 * kb) * ATOM_BYTES, E_BYTES, bar);
            }
        }
        __syncwarp();
    } else if (warp >= 1 && warp <= p.issuers) {
        // Several issuing threads: per stage one thread spends about half a microsecond on its barrier wait, fence, two
        // metadata copies, four MMAs and the commit - 24 KiB per 0.5 us is less than an SM can draw from HBM - so
        // lane 0 of warps 1 .. issuers (the later ones before they join the epilogue) each take every issuers-th
        // k-block into an accumulator of their own; the epilogue adds the accumulators.
        if (lane == 0) {
            const int which = warp - 1;
            if (which == p.issuers - 1) {
                // the two scales are fetched while the weights stream: their global-load latency (about a microsecond
                // when they miss L2) would otherwise sit between the last MMA and the first store
                if (p.pdl) pdl_wait_prior();               // the scales may be the preceding kernel's output
                *sc_slot = __ldg(p.scale_a) * __ldg(p.scale_b);
            }
            const uint32_t idesc = idesc_sparse(BM, NB);
            const uint32_t acc = tmem_base + which * p.acc_stride;
            for (int i = which; i < nkb; i += p.issuers) {
                const int s = i % nstages;
                const uint32_t ph = (i / nstages) & 1;
                if (!mbar_wait(full0 + 8 * s, ph)) { *abort_flag = 1; report_timeout(p.status); break; }
                tc_fence_after_sync();
                if (i == 0) stamp(p, 2);
                const uint32_t a = stage0 + s * STAGE, b = a + A_BYTES, e = b + 2 * NB * 128;
                const uint32_t te = tmem_base + p.te_col + 8 * s;
                tmem_cp_128x128b(te, smem_desc_meta(e));
                tmem_cp_128x128b(te + 4, smem_desc_meta(e + ATOM_BYTES));
#pragma unroll
                for (int j = 0; j < 4; j++)
                    tc_mma_sp_f8(acc, smem_desc_k128(a + 32 * j), smem_desc_k128(b + (j >> 1) * NB * 128 + (j & 1) * 64),
                                 te + 2 * j, idesc, (i >= p.issuers) || j != 0);
                tc_commit(empty0 + 8 * s);
            }
            tc_commit(tmem_full);                          // (also after an abort, and from a thread that had no k-block)
            if (which == 0) stamp(p, 3);
        }
        __syncwarp();
    }

    // ---- epilogue: warps 2..5 move their TMEM lane quadrant (32 weight rows each) into the staging tile in the
    // drained ring.  The tile is kept TRANSPOSED - stg[batch row m][weight row r], lines of 128 + 4 floats - because D
    // is written along n: the threads of a warp then read consecutive floats (no bank conflicts; with stg[r][m] a warp
    // that writes 128 contiguous output bytes reads 32 floats that all lie in one bank) and write whole 128-byte lines.
    float* stg = reinterpret_cast<float*>(smem);
    constexpr int pitch = BM + 4;
    if (warp >= 2) {
        bool ok = mbar_wait(tmem_full, 0);
        if (!ok) { *abort_flag = 1; report_timeout(p.status); }
        ok = ok && (*abort_flag == 0);
        tc_fence_after_sync();
        if (warp == 2 && lane == 0) stamp(p, 4);
        if (ok) {
            const int quad = warp & 3;
            float* col = stg + quad * 32 + lane;           // this thread's weight row
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < NB; c0 += 16) {
                float v[16];
                tmem_ld16(taddr + c0, v);
                for (int a = 1; a < p.issuers && a < nkb; a++) {     // the other issuers' accumulators, in order
                    float w[16];
                    tmem_ld16(taddr + a * p.acc_stride + c0, w);
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] += w[j];
                }
#pragma unroll
                for (int j = 0; j < 16; j++) col[(c0 + j) * pitch] = v[j];
            }
        }
    }
    if (S > 1) cluster_wait_acquire();
    __syncthreads();
    if (p.pdl) pdl_wait_prior();                       // D may still be read by the preceding kernel's successors
    const float sc = *sc_slot;

    // one bf16x2 store per item (batch row m, pair of weight rows); consecutive threads take consecutive pairs
    auto store_pair = [&](int m, int n, float v0, float v1) {
        if (n + 1 < p.N) {
            *reinterpret_cast<__nv_bfloat162*>(p.D + static_cast<size_t>(m0 + m) * p.N + n) = __floats2bfloat162_rn(v0 * sc, v1 * sc);
        } else if (n < p.N) {
            p.D[static_cast<size_t>(m0 + m) * p.N + n] = __float2bfloat16_rn(v0 * sc);
        }
    };
    if (S == 1) {
        if (*abort_flag == 0) {
            // six warps cannot hide the latency chain of one item per thread: four independent items per trip
#pragma unroll 4
            for (int item = threadIdx.x; item < m_count * (BM / 2); item += NUM_THREADS) {
                const int m = item / (BM / 2), r = (item - m * (BM / 2)) * 2;
                const float2 v = *reinterpret_cast<const float2*>(stg + m * pitch + r);
                store_pair(m, n0 + r, v.x, v.y);
            }
        }
    } else {
        // push: item = (batch row, granule of 4 weight rows) -> the rank that owns those rows; red[src][m][row] there
        const int rows_shift = S == 2 ? 6 : 5;              // rows_per = 128 / S, S is 2 or 4 here
#pragma unroll 4
        for (int item = threadIdx.x; item < NB * (BM / 4); item += NUM_THREADS) {
            const int m = item / (BM / 4), r = (item - m * (BM / 4)) * 4;
            const int owner = r >> rows_shift, rl = r - (owner << rows_shift);
            const float4 v = *reinterpret_cast<const float4*>(stg + m * pitch + r);
            const uint32_t dst = mapa_smem(smem_u32(red + (static_cast<size_t>(rank) * NB + m) * rows_per + rl), owner);
            st_async_v4(dst, v.x, v.y, v.z, v.w, mapa_smem(xbar, owner));
        }
        if (!mbar_wait(xbar, 0)) { *abort_flag = 1; report_timeout(p.status); }
        __syncthreads();
        if (threadIdx.x == 0) stamp(p, 5);
        if (*abort_flag == 0) {
            const int pairs = rows_per / 2, pair_shift = rows_shift - 1;
#pragma unroll 4
            for (int item = threadIdx.x; item < m_count * pairs; item += NUM_THREADS) {
                const int m = item >> pair_shift, rl = (item - (m << pair_shift)) * 2;
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int src = 0; src < 4; src++) {                 // rank order
                    if (src < S) {
                        const float2 v = *reinterpret_cast<const float2*>(red + ((src * NB + m) << rows_shift) + rl);
                        s0 += v.x;
                        s1 += v.y;
                    }
                }
                store_pair(m, n0 + rank * rows_per + rl, s0, s1);
            }
        }
    }

    if (threadIdx.x == 0) stamp(p, 6);
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
    if (threadIdx.x == 0) stamp(p, 7);
}

static unsigned long long* g_trace = nullptr;
static int g_trace_slots = 0, g_trace_next = 0;

static int run_list(const rdb_sparse_problem* pr, int count, int split_k_hint, unsigned flags, cudaStream_t stream) {
    if (flags & ~RDB_SKINNY_OVERLAP_PRIOR_KERNEL) return RDB_INVALID_CONFIG;
    if (!pr || count < 1 || count > kMaxProblems) return RDB_INVALID_CONFIG;
    if (split_k_hint != 0 && split_k_hint != 1 && split_k_hint != 2 && split_k_hint != 4) return RDB_INVALID_CONFIG;
    const int M = pr[0].M;
    int tiles = 0, min_kb = 1 << 30;
    for (int i = 0; i < count; i++) {
        const rdb_sparse_problem& q = pr[i];
        if (q.M < 1 || q.N < 1 || q.K < 1) return RDB_BAD_SHAPE;
        if (q.M > 256) return RDB_M_ABOVE_WARPTILE_M;
        if (q.M != M) return RDB_INVALID_CONFIG;             // one batch, one configuration per launch
        if (q.N % 2 != 0) return RDB_N_NOT_EVEN;
        if (q.K % 256 != 0) return RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K;
        if (!aligned16(q.A) || !aligned16(q.Wvals) || !aligned16(q.Wmeta) || (reinterpret_cast<uintptr_t>(q.D) & 3u)) return RDB_BAD_ALIGNMENT;
        if (!q.scale_a || !q.scale_b) return RDB_INVALID_CONFIG;
        tiles += (q.N + BM - 1) / BM;
        if (q.K / 256 < min_kb) min_kb = q.K / 256;
    }
    if (tiles > 65535) return RDB_SIZE_ABOVE_LIMIT;
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    // Wide batches are cut into blocks of at most 128 columns along a third grid
    // dimension: more CTAs, and each re-reads only its own part of the activations.
    const int mblocks = M > 128 ? (M + 127) / 128 : 1;
    const int NB = ((M + mblocks - 1) / mblocks + 15) / 16 * 16;
    int S = split_k_hint;
    if (S == 0) {
        // resident clusters of 2 / 4 CTAs on a 148-SM part: 74 / 33 (one per SM)
        S = 1;
        if (NB <= 64) {
            if (tiles * mblocks * 4 <= info->sm_count && tiles * mblocks <= 33 * info->sm_count / 148) S = 4;
            else if (tiles * mblocks * 2 <= info->sm_count) S = 2;
        }
        // narrow batches: up to two CTAs per SM (half rings, below), so a finer cut that fills the machine twice over
        // lets one CTA's set-up and epilogue hide behind its neighbour's stream (8192 x 8192, M = 16: four slices
        // 10.9 us against 11.3 with two, 8.6 against 10.0 when launches overlap; at M = 64 the coarser cut wins)
        if (NB <= 32) {
            if (S < 4 && tiles * mblocks * 4 <= 2 * info->sm_count) S = 4;
            else if (S < 2 && tiles * mblocks * 2 <= 2 * info->sm_count) S = 2;
        }
    }
    while (S > 1 && (S > min_kb || NB > 64)) S /= 2;
    const bool pdl = (flags & RDB_SKINNY_OVERLAP_PRIOR_KERNEL) != 0;
    // A launch that may overlap its predecessor keeps its ring to under half of an SM's shared memory (and, below,
    // its TMEM to half of the columns) when the batch is narrow: its CTAs can then become resident beside the
    // predecessor's and stream their first weights while those are still in their epilogue.
    // So does a grid of more CTAs than the machine has SMs (a list of GEMMs, a tall matrix): with two CTAs resident per
    // SM the set-up, first loads and epilogue of one overlap the other's stream (a list of 8192 x 8192 matrices at
    // M = 16 ran a quarter faster per GEMM than with one CTA per SM).
    const bool many = tiles * S * mblocks > info->sm_count && NB <= 64;
    const int ring_budget = ((pdl && NB <= 32) || many) ? 108 * 1024 : SMEM_LIMIT - 1024 - BAR_BYTES;   // wider batches: too few stages (measured slower)
    int stages = (ring_budget - red_bytes(NB, S)) / stage_bytes(NB);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const int kb_per = min_kb / S;
    if (stages > kb_per) stages = kb_per;
    if (stages < 1) stages = 1;
    while (stages > 1 && smem_bytes(NB, S, stages) > SMEM_LIMIT) stages--;
    if (smem_bytes(NB, S, stages) > SMEM_LIMIT) return RDB_SIZE_ABOVE_LIMIT;
    // Two issuing threads take alternate k-blocks, so the ring depth must be even: each thread then always meets the
    // same stages and waits for CONSECUTIVE completions of their barriers (a parity wait cannot tell completion n
    // from n + 2, which an odd depth - or a single stage - would ask of it).  A one-stage ring keeps one issuer.
    const int issuers = stages >= 2 ? 2 : 1;
    if (issuers == 2) stages -= stages % 2;

    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(sparse_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess)
            return RDB_CUDA_ERROR;
        // two half-ring CTAs of consecutive launches share an SM only if the SM is carved for shared memory
        cudaFuncSetAttribute(sparse_gemm_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        attr_set[dev] = true;
    }
    GParams g;
    memset(&g, 0, sizeof(g));
    g.count = count;
    int tile_begin = 0;
    for (int i = 0; i < count; i++) {
        const rdb_sparse_problem& q = pr[i];
        Prob& d = g.prob[i];
        int r = make_tmap_2d(&d.tmW, q.Wvals, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.N, q.K / 2, q.K / 2, BKC, BM, CU_TENSOR_MAP_SWIZZLE_128B);
        if (r != RDB_SUCCESS) return r;
        r = make_tmap_2d(&d.tmX, q.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, q.K, q.K, 128, NB, CU_TENSOR_MAP_SWIZZLE_128B);
        if (r != RDB_SUCCESS) return r;
        d.D = reinterpret_cast<__nv_bfloat16*>(q.D);
        d.meta = q.Wmeta;
        d.scale_a = q.scale_a;
        d.scale_b = q.scale_b;
        d.N = q.N;
        d.num_kb = q.K / 256;
        d.tile_begin = tile_begin;
        tile_begin += (q.N + BM - 1) / BM;
    }
    Params& p = g.common;
    p.status = info->status_dev;
    p.M = M;
    p.NB = NB;
    p.nstages = stages;
    int ring = stages * stage_bytes(NB);
    if (ring < stg_bytes(NB)) ring = stg_bytes(NB);
    p.ring_bytes = ring;
    p.pdl = pdl ? 1 : 0;
    p.trace = g_trace ? g_trace + static_cast<size_t>(g_trace_next++ % g_trace_slots) * 8 : nullptr;
    p.acc_stride = (NB + 31) / 32 * 32;
    p.issuers = issuers;       // four were measured no faster (the epilogue then adds four accumulators)
    p.te_col = p.issuers * p.acc_stride;
    p.tmem_cols = 32;
    while (p.tmem_cols < p.te_col + 8 * stages) p.tmem_cols *= 2;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S, tiles, mblocks);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes(NB, S, stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, sparse_gemm_kernel, g) == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

static int run(const uint8_t* A, const uint8_t* Wvals, const uint8_t* Wmeta, const float* sa, const float* sb, uint16_t* D,
               int M, int N, int K, int split_k_hint, unsigned flags, cudaStream_t stream) {
    rdb_sparse_problem q;
    q.A = A;
    q.Wvals = Wvals;
    q.Wmeta = Wmeta;
    q.scale_a = sa;
    q.scale_b = sb;
    q.D = D;
    q.M = M;
    q.N = N;
    q.K = K;
    return run_list(&q, 1, split_k_hint, flags, stream);
}

}  // namespace sparse
}  // namespace rdb

extern "C" {

size_t rdb_sparse_meta_bytes(int N, int K) {
    if (N < 1 || K < 1 || K % 256 != 0) return 0;
    return static_cast<size_t>((N + 127) / 128) * (K / 128) * rdb::sparse::ATOM_BYTES;
}

// Host-side packer (no GPU involved): compresses a 2:4 matrix of e4m3 bytes.
int rdb_sparse_pack_2of4(const uint8_t* Wq, int N, int K, uint8_t* vals, uint8_t* meta) {
    if (N < 1 || K < 1 || K % 256 != 0) return RDB_BAD_SHAPE;
    const int tiles = (N + 127) / 128, atoms = K / 128;
    memset(meta, 0, static_cast<size_t>(tiles) * atoms * rdb::sparse::ATOM_BYTES);
    for (int n = 0; n < N; n++) {
        const uint8_t* w = Wq + static_cast<size_t>(n) * K;
        uint8_t* v = vals + static_cast<size_t>(n) * (K / 2);
        uint8_t* mrow = meta + (static_cast<size_t>(n / 128) * atoms * 128 + (n % 128)) * 16;
        for (int c = 0; c < K / 4; c++) {
            int idx[2], cnt = 0;
            for (int i = 0; i < 4; i++) {
                if ((w[4 * c + i] & 0x7F) != 0) {          // +0 and -0 both count as zero
                    if (cnt == 2) return RDB_INVALID_CONFIG;  // more than two non-zeros: not a 2:4 matrix
                    idx[cnt++] = i;
                }
            }
            // pad with the lowest unused positions so that the pair stays strictly ascending
            for (int i = 0; i < 4 && cnt < 2; i++)
                if (cnt == 0 || idx[0] != i) idx[cnt++] = i;
            if (idx[0] > idx[1]) { const int t = idx[0]; idx[0] = idx[1]; idx[1] = t; }
            v[2 * c] = w[4 * c + idx[0]];
            v[2 * c + 1] = w[4 * c + idx[1]];
            const uint8_t nib = static_cast<uint8_t>(idx[0] | (idx[1] << 2));
            // chunk c of the row lives in atom c/32, byte (c%32)/2, low nibble first
            uint8_t* dst = mrow + static_cast<size_t>(c / 32) * 128 * 16 + (c % 32) / 2;
            *dst |= (c & 1) ? static_cast<uint8_t>(nib << 4) : nib;
        }
    }
    // rows past N in the last tile (their values are never loaded): a valid selection, positions (0, 1)
    for (int n = N; n < tiles * 128; n++)
        for (int a = 0; a < atoms; a++)
            memset(meta + ((static_cast<size_t>(n / 128) * atoms + a) * 128 + (n % 128)) * 16, 0x44, 16);
    return RDB_SUCCESS;
}

int rdb_sparse_gemm_fp8(const uint8_t* A, const uint8_t* Wvals, const uint8_t* Wmeta, const float* scale_a,
                        const float* scale_b, uint16_t* D, int M, int N, int K, void* stream) {
    return rdb::sparse::run(A, Wvals, Wmeta, scale_a, scale_b, D, M, N, K, 0, 0, static_cast<cudaStream_t>(stream));
}

int rdb_sparse_gemm_fp8_tuned(const uint8_t* A, const uint8_t* Wvals, const uint8_t* Wmeta, const float* scale_a,
                              const float* scale_b, uint16_t* D, int M, int N, int K, int split_k, void* stream) {
    return rdb::sparse::run(A, Wvals, Wmeta, scale_a, scale_b, D, M, N, K, split_k, 0, static_cast<cudaStream_t>(stream));
}

int rdb_sparse_gemm_fp8_grouped(const rdb_sparse_problem* problems, int count, unsigned flags, void* stream) {
    return rdb::sparse::run_list(problems, count, 0, flags, static_cast<cudaStream_t>(stream));
}

int rdb_sparse_gemm_trace(unsigned long long* device_buffer, int slots) {
    if (device_buffer && slots < 1) return RDB_INVALID_CONFIG;
    rdb::sparse::g_trace = device_buffer;
    rdb::sparse::g_trace_slots = slots;
    rdb::sparse::g_trace_next = 0;
    return RDB_SUCCESS;
}

int rdb_sparse_gemm_fp8_flags(const uint8_t* A, const uint8_t* Wvals, const uint8_t* Wmeta, const float* scale_a,
                              const float* scale_b, uint16_t* D, int M, int N, int K, int split_k, unsigned flags, void* stream) {
    return rdb::sparse::run(A, Wvals, Wmeta, scale_a, scale_b, D, M, N, K, split_k, flags, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
