// Grouped skinny FP8 GEMM for sm_100a: a list of independent problems
//   D_i[M_i,N_i] = bf16((A_i . B_i^T) * sa_i * sb_i),  M_i <= 32,
// computed by ONE persistent launch.
//
// A single skinny GEMM is bound by streaming its weight matrix from HBM once,
// and what a launch of it adds on top of that stream is a fixed chain - CTA
// start, barrier and TMEM set-up, the first ring of loads in flight, the
// split-K exchange, the grid draining - of several microseconds in which no
// weight byte moves.  The reference times four launches back to back on
// different weight matrices (projects/skinny_gemm/bench.cu:51-60); a decode
// step issues such a list per layer.  Here the whole list is one weight stream:
//
//   * every problem is cut into units of (R weight rows) x (128 bytes of K);
//     the units of all problems, in order, form one sequence that is split into
//     one contiguous, equally heavy range per CTA (one CTA per SM) - stream-K
//     over the concatenated problems, so the load balance does not depend on
//     how any single shape divides by the SM count;
//   * warp 1: one thread walks the CTA's range and issues the TMA loads (weights
//     R x 128 B + activations MPAD x 128 B per unit) into a 6-stage ring - the
//     ring never drains at a tile or problem boundary;
//   * warp 2: one thread issues tcgen05.mma kind::f8f6f4 (128 x R x 32, weights
//     on the wide side) into one of two TMEM accumulators, switching at every
//     tile boundary;
//   * warps 0 and 4 (the warps that may read TMEM lanes 0..31 = output rows)
//     drain finished accumulators while the next tile streams: a tile whose K
//     range lies inside the CTA's range is scaled, rounded once and stored; a
//     tile shared with other CTAs is reduced through a global workspace - the
//     CTA holding the head of the tile's K range owns the tile, the others
//     store their fp32 partial and raise a flag, and the owner adds the
//     partials in K order (deterministic) before the single rounding.
//     A CTA writes at most one partial (the first segment of its range) and
//     owns at most one shared tile (its last segment), so the exchange sits at
//     the two ends of the launch, not on the streaming path.
//
// Waits are bounded like everywhere in this library; the launch is cooperative
// so that the CTAs an owner waits for are guaranteed to be on the GPU.
// Replaces a sequence of skinny_gemm_fastpath calls
// (projects/skinny_gemm/skinny_gemm_caller.cu:343-405).
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "ar_internal.h"
#include "fp8_codec.cuh"
#include "host_util.h"
#include "ptx.cuh"

#include <cuda_fp8.h>

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace grouped {

constexpr int BK = 128;                     // K bytes per unit = one 128-byte swizzle row
constexpr int MAX_R = 256;                  // weight rows per unit (UMMA N)
constexpr int A_BYTES = 32 * BK;            // room for the activation box (up to 32 rows)
constexpr int STAGE = A_BYTES + MAX_R * BK; // 36 KiB
constexpr int STAGES = 6;
constexpr int NUM_THREADS = 160;            // warps 0, 4: epilogue; 1: TMA; 2: MMA; 3: idle
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE + 256;
constexpr int kMaxProblems = RDB_SKINNY_GROUP_MAX;
constexpr int kMaxCtas = 192;
constexpr int SLOT_FLOATS = 32 * MAX_R;     // one CTA's partial tile: [32 rows][256 columns] fp32

struct alignas(64) Problem {
    CUtensorMap tmW, tmA;
    __nv_bfloat16* D;
    const float* scale_a;
    const float* scale_b;
    int M, N, R, mpad;
    int num_kb, tiles, unit_begin, vec_ok;  // vec_ok: 16-byte stores into D are aligned
};

struct Params {
    Problem prob[kMaxProblems];
    int range_begin[kMaxCtas + 1];          // CTA c works on units [range_begin[c], range_begin[c + 1])
    int count;
    float* partial;                         // [grid][32][256] fp32
    unsigned* words;                        // [0]: launch epoch, [1]: CTAs that finished, [2]: a CTA gave up (fused
                                            // delivery), [8 + 2 c + e]: partial flags
    int* status;
    unsigned long long* trace;              // optional [grid][4] %globaltimer stamps, else nullptr
    rdb::ar::PushTarget push;               // world > 0: the result goes, block-quantised, to the allreduce staging
    int pdl;                                // launched with programmatic stream serialization (see the launcher)
    int mma_m;                              // UMMA M: 64 when no problem has more than 16 rows (half the padded work), else 128
};

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Unit u -> (problem, tile, k-block).  `pi` only moves forward.
__device__ __forceinline__ void locate(const Params& p, int u, int& pi, int& tile, int& kb) {
    while (pi + 1 < p.count && u >= p.prob[pi + 1].unit_begin) pi++;
    const int local = u - p.prob[pi].unit_begin;
    const int nkb = p.prob[pi].num_kb;
    tile = local / nkb;
    kb = local - tile * nkb;
}

__device__ __forceinline__ void stamp(const Params& p, int slot) {
    if (p.trace) p.trace[blockIdx.x * 4 + slot] = globaltimer_ns();
}

// Scales, rounds and stores 32 consecutive outputs of row m starting at tile column c0.
__device__ __forceinline__ void store_chunk(const Problem& pr, const float* v, float sc, int m, int n, int valid) {
    __nv_bfloat16* out = pr.D + static_cast<size_t>(m) * pr.N + n;
    if (pr.vec_ok && valid == 32 && n + 31 < pr.N) {
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
#pragma unroll
        for (int j = 0; j < 32; j++)            // fully unrolled: v stays in registers
            if (j < valid && n + j < pr.N) out[j] = __float2bfloat16_rn(v[j] * sc);
    }
}

// The number of the allreduce call a fused launch feeds: passed by the host, or - on a context that counts its calls on
// the device, so that the launch can be replayed from a CUDA graph - one more than the count of completed calls, which
// only the closing reduce launch of the same call advances.
__device__ __forceinline__ unsigned push_call_number(const rdb::ar::PushTarget& t) {
    return t.epoch_dev ? *reinterpret_cast<const volatile unsigned*>(t.epoch_dev) + 1u : t.epoch;
}

// GEMM -> allreduce fusion: one finished 128-column block of output row m (bf16
// values packed two per word, their maximum magnitude in `amax`) is encoded
// exactly like the allreduce's own encoder does - scale amax/448, e4m3 codes of
// x / scale - and stored into every rank's staging slot for flattened element
// `elem` of the [M,N] result.
__device__ __forceinline__ void push_block128(const rdb::ar::PushTarget& t, const unsigned call, const uint32_t* packed, float amax, size_t elem) {
    const float s = rdb::ar::block_scale(amax);
    rdb::ar::BlockDivisor d;
    d.set(s);
    const size_t g = elem / 512;
    const int blk = static_cast<int>((elem % 512) / 128);
    const size_t slot = (static_cast<size_t>(call & 1u) * t.world + t.rank) * t.slot_groups + g;
#pragma unroll 1
    for (int i = 0; i < 8; i++) {                       // 16 elements -> 16 code bytes per step
        uint32_t q[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float x[8], y[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t w = packed[8 * i + 4 * h + j];
                x[2 * j] = __uint_as_float(w << 16);
                x[2 * j + 1] = __uint_as_float(w & 0xFFFF0000u);
            }
            d.div8(x, y);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(y[4 * j], y[4 * j + 1]), __NV_SATFINITE, __NV_E4M3);
                const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(make_float2(y[4 * j + 2], y[4 * j + 3]), __NV_SATFINITE, __NV_E4M3);
                q[2 * h + j] = static_cast<uint32_t>(a) | (static_cast<uint32_t>(b) << 16);
            }
        }
        for (int k = 0; k < t.world; k++) {
            int peer = t.rank + 1 + k;
            if (peer >= t.world) peer -= t.world;
            reinterpret_cast<uint4*>(t.ws[peer] + t.off_q + slot * 512 + blk * 128)[i] = make_uint4(q[0], q[1], q[2], q[3]);
        }
    }
    for (int k = 0; k < t.world; k++)
        reinterpret_cast<float*>(t.ws[k] + t.off_s)[slot * 4 + blk] = s;
}

__global__ void __launch_bounds__(NUM_THREADS, 1) skinny_grouped_kernel(const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const int lo = p.range_begin[cta], hi = p.range_begin[cta + 1];

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(smem);

    if (threadIdx.x == 0) stamp(p, 0);
    if (threadIdx.x == 32) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(acc_full0 + 8 * a, 1);
            mbar_init(acc_empty0 + 8 * a, 2);   // the two epilogue warps
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (p.pdl) pdl_launch_dependents();     // the next kernel of the stream may take SMs as this one's CTAs leave

    if (warp == 1) {
        // ---- producer: the CTA's whole unit range through the ring, never drained
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first();   // weights are read once
            const uint64_t pol_a = l2_policy_evict_last();    // activations are re-read by every tile
            int pi = 0, last_pi = -1;
            // Weights never depend on the preceding kernel: with programmatic launch the first ring of weight boxes
            // is requested before waiting for that kernel to finish; the activations of those stages follow after.
            const int pre = p.pdl ? (hi - lo < STAGES ? hi - lo : STAGES) : 0;
            for (int pass = 0; pass < (p.pdl ? 2 : 0); pass++) {
                int pj = 0;
                if (pass == 1) pdl_wait_prior();
                for (int i = 0; i < pre; i++) {
                    int tile, kb;
                    locate(p, lo + i, pj, tile, kb);
                    const Problem& pr = p.prob[pj];
                    const uint32_t dst = stage0 + i * STAGE;
                    if (pass == 0) {
                        mbar_arrive_expect_tx(full0 + 8 * i, static_cast<uint32_t>(pr.mpad + pr.R) * BK);
                        tma_load_2d(dst + A_BYTES, &pr.tmW, kb * BK, tile * pr.R, full0 + 8 * i, pol_w);
                    } else {
                        tma_load_2d(dst, &pr.tmA, kb * BK, 0, full0 + 8 * i, pol_a);
                    }
                }
            }
            for (int u = lo + pre, i = pre; u < hi; u++, i++) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (i >= STAGES && !mbar_wait(empty0 + 8 * s, ph ^ 1)) { *abort_flag = 1; report_timeout(p.status); break; }
                int tile, kb;
                locate(p, u, pi, tile, kb);
                const Problem& pr = p.prob[pi];
                if (pi != last_pi) {
                    prefetch_tensormap(&pr.tmW);
                    prefetch_tensormap(&pr.tmA);
                    last_pi = pi;
                }
                const uint32_t dst = stage0 + s * STAGE;
                mbar_arrive_expect_tx(full0 + 8 * s, static_cast<uint32_t>(pr.mpad + pr.R) * BK);
                tma_load_2d(dst + A_BYTES, &pr.tmW, kb * BK, tile * pr.R, full0 + 8 * s, pol_w);
                tma_load_2d(dst, &pr.tmA, kb * BK, 0, full0 + 8 * s, pol_a);
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---- MMA issuer: one accumulator per segment (the part of a tile's K range inside this CTA's range)
        if (lane == 0) {
            int pi = 0, seg = 0;
            bool first = true;
            for (int u = lo, i = 0; u < hi; u++, i++) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                int tile, kb;
                locate(p, u, pi, tile, kb);
                const Problem& pr = p.prob[pi];
                const int buf = seg & 1;
                if (first) {
                    // the epilogue must have drained this accumulator (passes at once on its first two uses)
                    if (!mbar_wait(acc_empty0 + 8 * buf, ((seg >> 1) & 1) ^ 1)) { *abort_flag = 1; report_timeout(p.status); break; }
                }
                if (!mbar_wait(full0 + 8 * s, ph)) { *abort_flag = 1; report_timeout(p.status); break; }
                tc_fence_after_sync();
                if (i == 0) stamp(p, 1);
                const uint32_t a = stage0 + s * STAGE, w = a + A_BYTES;
                const uint32_t idesc = idesc_e4m3_f32(p.mma_m, pr.R);
                const uint32_t d = tmem_base + buf * MAX_R;
#pragma unroll
                for (int ks = 0; ks < BK / 32; ks++)
                    tc_mma_f8(d, smem_desc_k128(a + ks * 32), smem_desc_k128(w + ks * 32), idesc, !(first && ks == 0));
                tc_commit(empty0 + 8 * s);     // the stage is free once these MMAs have read it
                first = false;
                if (kb == pr.num_kb - 1 || u == hi - 1) {
                    tc_commit(acc_full0 + 8 * buf);
                    seg++;
                    first = true;
                }
            }
            stamp(p, 2);
        }
        __syncwarp();
    } else if ((warp & 3) == 0) {
        // ---- epilogue: warp 0 takes the even 32-column chunks of a tile, warp 4 the odd ones
        const int e = warp >> 2;
        // everything the epilogue touches - the launch epoch, the workspace, the scales, D - may still belong to the
        // preceding kernel until it has completed
        if (p.pdl) pdl_wait_prior();
        const unsigned epoch = ld_acquire_gpu_u32(p.words);
        const unsigned push_call = push_call_number(p.push);
        float* my_slot = p.partial + static_cast<size_t>(cta) * SLOT_FLOATS + lane * MAX_R;
        int pi = 0, seg = 0;
        bool live = true;
        for (int u = lo; u < hi && live; seg++) {
            int tile, kb0;
            locate(p, u, pi, tile, kb0);
            const Problem& pr = p.prob[pi];
            const int tile_end = pr.unit_begin + (tile + 1) * pr.num_kb;   // first unit after this tile
            const int seg_end = tile_end < hi ? tile_end : hi;
            const bool from_k0 = kb0 == 0, to_k_end = seg_end == tile_end;
            const int buf = seg & 1;
            // fetched now, used after the accumulator wait: the load latency hides behind the segment's MMAs
            const float sc = from_k0 ? __ldg(pr.scale_a) * __ldg(pr.scale_b) : 0.0f;
            // A tile whose head I hold (always my last segment) is mine to finish.  Its other parts were computed by
            // the following CTAs at the START of their ranges, so their flags are normally up long before my last MMA:
            // find them and poll them now, one lane per flag (each poll is an L2 round trip), while the MMAs run.
            int last_partner = cta;
            if (from_k0 && !to_k_end) {
                while (last_partner + 1 < static_cast<int>(gridDim.x) && p.range_begin[last_partner + 1] < tile_end) last_partner++;
                for (int base = cta + 1; base <= last_partner && live; base += 32) {
                    const int j = base + lane;
                    bool ok = true;
                    if (j <= last_partner && p.range_begin[j] != p.range_begin[j + 1]) {     // an empty range holds nothing
                        const unsigned* f = p.words + 8 + 2 * j + e;
                        const uint64_t t0 = globaltimer_ns(), budget = wait_budget_ns();
                        unsigned spins = 0;
                        while (static_cast<int>(ld_acquire_gpu_u32(f) - (epoch + 1)) < 0) {
                            if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > budget) { ok = false; break; }
                        }
                    }
                    if (!__all_sync(0xffffffffu, ok)) live = false;
                }
                if (!live) { *abort_flag = 1; if (lane == 0) report_timeout(p.status); }
            }
            bool ok = mbar_wait(acc_full0 + 8 * buf, (seg >> 1) & 1);
            if (!ok) { *abort_flag = 1; report_timeout(p.status); }
            if (*abort_flag != 0) { live = false; break; }
            tc_fence_after_sync();
            const int n0 = tile * pr.R;
            const uint32_t taddr = tmem_base + buf * MAX_R;
            if (!from_k0) {
                // not the owner: park the fp32 partial in this CTA's slot and raise the flag
                for (int c0 = 32 * e; c0 < pr.R; c0 += 64) {
                    float v[32];
                    tmem_ld32(taddr + c0, v);
                    if (lane < pr.M) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(my_slot + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    __threadfence();
                    st_release_gpu_u32(p.words + 8 + 2 * cta + e, epoch + 1);
                }
            } else {
                // the partners' parts of 32 columns of my row, added in K order; the loads of a part are issued
                // together (eight independent 16-byte loads per lane)
                auto add_parts = [&](int c0, float* v) {
                    if (lane < pr.M) {
                        for (int j = cta + 1; j <= last_partner; j++) {
                            if (p.range_begin[j] == p.range_begin[j + 1]) continue;
                            const float4* src = reinterpret_cast<const float4*>(p.partial + static_cast<size_t>(j) * SLOT_FLOATS + lane * MAX_R + c0);
                            float4 t[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) t[q] = __ldcg(src + q);
#pragma unroll
                            for (int q = 0; q < 8; q++) { v[4 * q] += t[q].x; v[4 * q + 1] += t[q].y; v[4 * q + 2] += t[q].z; v[4 * q + 3] += t[q].w; }
                        }
                    }
                };
                if (p.push.world > 0) {
                    // fused delivery: warp e takes whole 128-column blocks (R is a multiple of 128 here), keeps the
                    // block's bf16 values packed in registers and hands them to the encoder
                    for (int b0 = 128 * e; b0 < pr.R && n0 + b0 < pr.N; b0 += 256) {
                        uint32_t packed[64];
                        float amax = 0.0f;
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            float v[32];
                            tmem_ld32(taddr + b0 + 32 * c, v);
                            add_parts(b0 + 32 * c, v);
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j] * sc, v[2 * j + 1] * sc);
                                const uint32_t w = *reinterpret_cast<const uint32_t*>(&h2);
                                packed[16 * c + j] = w;
                                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w << 16)), fabsf(__uint_as_float(w & 0xFFFF0000u))));
                            }
                        }
                        if (lane < pr.M) push_block128(p.push, push_call, packed, amax, static_cast<size_t>(lane) * pr.N + n0 + b0);
                    }
                } else {
                    for (int c0 = 32 * e; c0 < pr.R; c0 += 64) {
                        float v[32];
                        tmem_ld32(taddr + c0, v);
                        add_parts(c0, v);
                        if (lane < pr.M) store_chunk(pr, v, sc, lane, n0 + c0, pr.R - c0 < 32 ? pr.R - c0 : 32);
                    }
                }
            }
            // this warp's TMEM reads of the segment are complete: hand the accumulator back
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
            u = seg_end;
        }
    }

    // ---- teardown: after an abort give in-flight TMA copies time to land
    if (*abort_flag != 0) {
        for (int i = 0; i < 64; i++) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, 512);
    if (threadIdx.x == 0) {
        stamp(p, 3);
        // the last CTA to finish opens the next launch's epoch (partial flags are compared with it, so
        // nothing is ever reset and a replayed CUDA graph behaves like a fresh launch)
        if (p.push.world > 0 && *abort_flag != 0) atomicOr(p.words + 2, 1u);   // a wait of this CTA ran out
        if (p.push.world > 0) __threadfence_system(); else __threadfence();   // fused: this CTA's peer stores are out
        const unsigned done = atomicAdd(p.words + 1, 1u);
        if (done == gridDim.x - 1) {
            p.words[1] = 0;
            __threadfence();
            atomicAdd(p.words, 1u);
            if (p.push.world > 0) {
                // every CTA has delivered and fenced: tell all ranks that this rank's blocks of the call are in
                // place (the allreduce's "pushed" flag of this epoch; a wait that ran out here marks it failed)
                __threadfence_system();
                const unsigned call = push_call_number(p.push);
                const unsigned word = (call << 1) | (atomicExch(p.words + 2, 0u) & 1u);
                for (int k = 0; k < p.push.world; k++) {
                    unsigned* f = reinterpret_cast<unsigned*>(p.push.ws[k] + p.push.off_flags) + (call & 1u) * 8 + p.push.rank;
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(word) : "memory");
                }
            }
        }
    }
}

// ------------------------------------------------------------------ host
struct Workspace {
    float* partial = nullptr;
    unsigned* words = nullptr;
    int grid = 0;
};

// Per-device workspace (partial tiles + flag words), allocated on first use.
static Workspace* workspace(int grid, int* err) {
    static Workspace ws[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = RDB_CUDA_ERROR; return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    Workspace& w = ws[dev];
    if (!w.partial) {
        const size_t words_bytes = (8 + 2 * kMaxCtas) * sizeof(unsigned);
        if (cudaMalloc(reinterpret_cast<void**>(&w.partial), static_cast<size_t>(kMaxCtas) * SLOT_FLOATS * sizeof(float)) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void**>(&w.words), words_bytes) != cudaSuccess ||
            cudaMemset(w.words, 0, words_bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
            cudaGetLastError();
            *err = RDB_CUDA_ERROR;
            return nullptr;
        }
        if (cudaFuncSetAttribute(skinny_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
            cudaGetLastError();
            *err = RDB_CUDA_ERROR;
            return nullptr;
        }
    }
    w.grid = grid;
    return &w;
}

static unsigned long long* g_trace = nullptr;

// Tile height and unit ranges for a list of problems on `grid` CTAs (pure host arithmetic).
// Rows per unit: 256 (8 KiB of weights per MMA instruction) unless that leaves fewer than
// eight units per CTA, in which case 128-row units balance the ranges better (an MMA instruction costs
// the same whatever its width, so narrower units would make the issuing thread the limit).
static void plan(const rdb_skinny_problem* pr, int count, int grid, int* R_out, int* unit_begin, int* range_begin) {
    int R = MAX_R;
    for (;;) {
        long long units = 0;
        for (int i = 0; i < count; i++) {
            const int r = pr[i].N < R ? (pr[i].N + 15) / 16 * 16 : R;
            units += static_cast<long long>((pr[i].N + r - 1) / r) * ((pr[i].K + BK - 1) / BK);
        }
        if (units >= 8ll * grid || R <= 128) break;
        R /= 2;
    }
    long long total_w = 0;
    int total_units = 0;
    long long w[kMaxProblems], n_units[kMaxProblems];
    for (int i = 0; i < count; i++) {
        const int r = pr[i].N < R ? (pr[i].N + 15) / 16 * 16 : R;
        R_out[i] = r;
        unit_begin[i] = total_units;
        n_units[i] = static_cast<long long>((pr[i].N + r - 1) / r) * ((pr[i].K + BK - 1) / BK);
        w[i] = r + (pr[i].M <= 16 ? 16 : 32);
        total_units += static_cast<int>(n_units[i]);
        total_w += n_units[i] * w[i];
    }
    long long acc = 0;
    int pi = 0;
    for (int c = 0; c <= grid; c++) {
        const long long target = total_w * c / grid;
        while (pi < count && acc + n_units[pi] * w[pi] <= target) { acc += n_units[pi] * w[pi]; pi++; }
        range_begin[c] = pi == count ? total_units : unit_begin[pi] + static_cast<int>((target - acc) / w[pi]);
    }
    range_begin[0] = 0;
    range_begin[grid] = total_units;
}

// `push`: nullptr for a plain grouped GEMM; else the one problem's result is delivered, block-quantised, to the
// allreduce staging it describes (D is not written).
static int run(const rdb_skinny_problem* pr, int count, cudaStream_t stream, const rdb::ar::PushTarget* push = nullptr,
               unsigned flags = 0) {
    if (flags & ~RDB_SKINNY_OVERLAP_PRIOR_KERNEL) return RDB_INVALID_CONFIG;
    if (!pr || count < 1 || count > kMaxProblems) return RDB_INVALID_CONFIG;
    if (push && (count != 1 || pr[0].N % 128 != 0)) return RDB_INVALID_CONFIG;
    long long units = 0;
    for (int i = 0; i < count; i++) {
        const rdb_skinny_problem& q = pr[i];
        if (q.M < 1 || q.N < 1 || q.K < 1 || q.ldb < q.K) return RDB_BAD_SHAPE;
        if (q.M > 32) return RDB_M_ABOVE_WARPTILE_M;
        if (q.N % 2 != 0) return RDB_N_NOT_EVEN;
        if (q.K % 16 != 0 || q.ldb % 16 != 0) return RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K;
        if (!aligned16(q.A) || !aligned16(q.B) || (reinterpret_cast<uintptr_t>(q.D) & 1u)) return RDB_BAD_ALIGNMENT;
        if (!push && !q.D) return RDB_INVALID_CONFIG;
        if (!q.scale_a || !q.scale_b) return RDB_INVALID_CONFIG;
        units += static_cast<long long>((q.N + 15) / 16) * ((q.K + BK - 1) / BK);
    }
    if (units > (1ll << 30)) return RDB_SIZE_ABOVE_LIMIT;
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    const int grid = info->sm_count < kMaxCtas ? info->sm_count : kMaxCtas;
    Workspace* ws = workspace(grid, &err);
    if (!ws) return err;

    static Params prm;                      // 11 KiB: kept off the stack; guarded by the mutex below
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    int R[kMaxProblems], unit_begin[kMaxProblems];
    plan(pr, count, grid, R, unit_begin, prm.range_begin);
    for (int i = 0; i < count; i++) {
        const rdb_skinny_problem& q = pr[i];
        Problem& d = prm.prob[i];
        d.mpad = q.M <= 16 ? 16 : 32;
        int r = make_tmap_2d(&d.tmW, q.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.N, q.K, q.ldb, BK, R[i], CU_TENSOR_MAP_SWIZZLE_128B);
        if (r != RDB_SUCCESS) return r;
        r = make_tmap_2d(&d.tmA, q.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.M, q.K, q.K, BK, d.mpad, CU_TENSOR_MAP_SWIZZLE_128B);
        if (r != RDB_SUCCESS) return r;
        d.D = reinterpret_cast<__nv_bfloat16*>(q.D);
        d.scale_a = q.scale_a;
        d.scale_b = q.scale_b;
        d.M = q.M;
        d.N = q.N;
        d.R = R[i];
        d.num_kb = (q.K + BK - 1) / BK;
        d.tiles = (q.N + R[i] - 1) / R[i];
        d.unit_begin = unit_begin[i];
        d.vec_ok = (q.N % 8 == 0 && aligned16(q.D)) ? 1 : 0;
    }
    prm.count = count;
    prm.partial = ws->partial;
    prm.words = ws->words;
    prm.status = info->status_dev;
    prm.trace = g_trace;
    if (push) prm.push = *push;
    else memset(&prm.push, 0, sizeof(prm.push));

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    // A CTA that owns a shared tile waits for parts that HIGHER-numbered CTAs compute at the very start of their
    // ranges, so those CTAs must get onto the GPU: the cooperative launch makes the runtime guarantee it (and refuse
    // a grid that cannot be resident).  RDB_GROUPED_PLAIN_LAUNCH=1 selects a plain launch, for measurements.
    // With RDB_SKINNY_OVERLAP_PRIOR_KERNEL the launch is a plain one with programmatic stream serialization instead:
    // its CTAs take SMs as the preceding kernel's CTAs leave and stream weights while that kernel drains.
    static const bool plain_launch = [] { const char* v = getenv("RDB_GROUPED_PLAIN_LAUNCH"); return v && v[0] == '1'; }();
    const bool pdl = (flags & RDB_SKINNY_OVERLAP_PRIOR_KERNEL) != 0;
    prm.pdl = pdl ? 1 : 0;
    // 64-row MMAs when every batch fits 16 rows: rows 0-15 of a 64-row accumulator lie in TMEM lanes 0-15, where the
    // epilogue warps (lanes 0-31) read them; half the padded tensor work, hence less power (RDB_SKINNY_MMA_M=128 keeps 128)
    prm.mma_m = 128;
    {
        bool narrow = true;
        for (int i = 0; i < count; i++) narrow = narrow && pr[i].M <= 16;
        static const bool force128 = [] { const char* v = getenv("RDB_SKINNY_MMA_M"); return v && v[0] == '1'; }();
        if (narrow && !force128) prm.mma_m = 64;
    }
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
    } else {
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
    }
    cfg.attrs = attr;
    cfg.numAttrs = (plain_launch && !pdl) ? 0 : 1;
    if (cudaLaunchKernelEx(&cfg, skinny_grouped_kernel, prm) != cudaSuccess) {
        cudaGetLastError();
        return RDB_CUDA_ERROR;
    }
    return RDB_SUCCESS;
}

}  // namespace grouped
}  // namespace rdb

extern "C" {

int rdb_skinny_gemm_fp8_grouped(const rdb_skinny_problem* problems, int count, unsigned flags, void* stream) {
    return rdb::grouped::run(problems, count, static_cast<cudaStream_t>(stream), nullptr, flags);
}

int rdb_skinny_gemm_fp8_allreduce_begin(void* ar_ctx, const rdb_skinny_problem* problem, void* stream) {
    if (!ar_ctx || !problem) return RDB_INVALID_CONFIG;
    if (problem->M < 1 || problem->N < 1) return RDB_BAD_SHAPE;
    if (problem->N % 128 != 0) return RDB_BAD_SHAPE;
    rdb::ar::PushTarget t;
    int r = rdb::ar::begin_prepushed(ar_ctx, static_cast<size_t>(problem->M) * problem->N, &t);
    if (r != RDB_SUCCESS) return r;
    r = rdb::grouped::run(problem, 1, static_cast<cudaStream_t>(stream), &t);
    if (r != RDB_SUCCESS) rdb::ar::cancel_prepushed(ar_ctx);     // nothing was launched: the ranks' epochs stay in step
    return r;
}

int rdb_skinny_gemm_fp8_allreduce_finish(void* ar_ctx, uint16_t* out, void* stream) {
    return rdb::ar::finish_prepushed(ar_ctx, out, static_cast<cudaStream_t>(stream));
}

int rdb_skinny_gemm_fp8_allreduce(void* ar_ctx, const rdb_skinny_problem* problem, uint16_t* out, void* stream) {
    if (!out || !rdb::aligned16(out)) return RDB_BAD_ALIGNMENT;
    const int r = rdb_skinny_gemm_fp8_allreduce_begin(ar_ctx, problem, stream);
    return r != RDB_SUCCESS ? r : rdb_skinny_gemm_fp8_allreduce_finish(ar_ctx, out, stream);
}

int rdb_skinny_gemm_grouped_plan(const rdb_skinny_problem* problems, int count, int ctas, int* rows_per_unit,
                                 int* range_begin) {
    using namespace rdb::grouped;
    if (!problems || count < 1 || count > kMaxProblems || ctas < 1 || ctas > kMaxCtas) return RDB_INVALID_CONFIG;
    for (int i = 0; i < count; i++)
        if (problems[i].M < 1 || problems[i].M > 32 || problems[i].N < 1 || problems[i].K < 1) return RDB_BAD_SHAPE;
    int R[kMaxProblems], unit_begin[kMaxProblems], ranges[kMaxCtas + 1];
    plan(problems, count, ctas, R, unit_begin, ranges);
    for (int i = 0; i < count && rows_per_unit; i++) rows_per_unit[i] = R[i];
    for (int c = 0; c <= ctas && range_begin; c++) range_begin[c] = ranges[c];
    return RDB_SUCCESS;
}

int rdb_skinny_gemm_grouped_trace(unsigned long long* device_buffer) {
    rdb::grouped::g_trace = device_buffer;
    return RDB_SUCCESS;
}

}  // extern "C"
