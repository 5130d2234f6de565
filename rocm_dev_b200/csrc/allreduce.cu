// FP8-encoded allreduce over NVLink peer memory (one process per GPU).
//
// Semantics (there is no reference code for this path; the definition is the
// configuration text restated by the CPU oracle): every rank's bf16 vector is
// encoded in blocks of 128 elements - fp32 scale s = amax/448 (1 for an
// all-zero block), q = e4m3fn_sat_rn(x / s) - and the result on every rank is
// bf16_rn( sum over ranks r = 0..W-1, in rank order, of fp32(q_r) * s_r ), the
// product and the sum rounded separately in fp32.  All ranks produce identical
// bits.
//
// Data path.  Each rank owns a workspace (cudaMalloc'd, exported through CUDA
// IPC) holding a staging area for incoming encoded blocks, a gather area for
// the bf16 result and flag words.  A call consists of three phases - run as ONE
// kernel by rdb_ar_allreduce (ar_fused_kernel), or as three launches by
// rdb_ar_phase when several ranks are emulated on one GPU:
//   phase 1  quantise the local vector and PUSH the encoded bytes and scales
//            straight into the staging slot of the rank that owns each
//            512-element group (two-shot) or of every rank (one-shot, small
//            messages): coalesced 16-byte remote stores, nothing is staged
//            locally;
//            the last block to finish publishes "my pushes are complete" to
//            every peer (release, system scope);
//   phase 2  wait (bounded) for every peer's flag, then dequantise the W copies of
//            the owned groups, accumulate in fp32 in rank order, round once to
//            bf16 and push the result into every rank's gather area (two-shot)
//            or write it straight to the output (one-shot);
//            and publish "my part of the result is delivered";
//   phase 3  (two-shot) wait for those flags and, if the caller wants the result
//            in its own buffer, copy it out of the gather area.
// Flags carry a per-call epoch, so nothing is reset between calls; the staging
// area has two sets used alternately (epoch parity) because a fast rank may
// start pushing call e+1 while a slow one still reduces call e.  Loads are
// never issued against another GPU's memory: all remote traffic is stores.
// Waits are bounded; a timeout stores RDB_DEVICE_TIMEOUT in the status word.
// When the caller supplies an NVLS multicast alias of the workspaces
// (rdb_ar_set_multicast), phase 2 delivers the bf16 result with multimem.st:
// one store per 16 bytes, replicated by the switch.
//
// The phases also exist as separate launches so that a single GPU can emulate W
// ranks legally (all phase-1 launches, then all phase-2 launches, ...): no
// launch then waits on one that has not been issued.  The fused kernel must
// never be used that way.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "ar_internal.h"
#include "fp8_codec.cuh"
#include "host_util.h"
#include "ptx.cuh"

RDB_DEFINE_WAIT_BUDGET_SETTER()

namespace rdb {
namespace ar {

constexpr int kMaxWorld = 8;
constexpr int kGroup = 512;               // elements per work item: 4 blocks of 128
constexpr size_t kOneShotMaxElems = 1u << 22;
constexpr int kThreads = 256;
constexpr int kBlocksPerSm = 4;     // resident blocks per SM the grids are sized for
// Flag-in-line transport of the encoded groups: a group of 512 elements travels as 5 lines of 128 bytes.  A line
// is written by ONE store instruction (eight lanes x 16 bytes) and read by one load instruction, so it crosses
// NVLink and is observed as a unit; its last 8 bytes hold the call's epoch twice.  The receiver polls the lines
// themselves: no separate flag, no grid-wide hand-over and no system-wide fence between the data and its "valid"
// mark - that fence, not the bytes, was what a small allreduce took its time for (~10 us per hand-over).
// Lane t of the encoder owns 16 code bytes of the group (8 of each 256-element half).  Lines 0..3: position
// t % 8 < 7 of line t / 8 holds lane t's 16 bytes; position 7 holds {two block scales (lines 0 and 1), epoch,
// epoch}.  Line 4: positions 0..3 hold the bytes of lanes 7, 15, 23, 31, position 7 the epoch pair.
constexpr int kLlLines = 5;
constexpr int kLlGroupBytes = kLlLines * 128;

struct Layout {
    size_t slot_groups;   // groups one source rank may push into one slot
    size_t off_q;         // [2][W][slot_groups * 512] bytes   (two sets, used alternately: set = epoch & 1)
    size_t off_s;         // [2][W][slot_groups * 4] floats
    size_t off_gather;    // [max_elems] bf16; the FP8 all-gather uses it as [max_elems] codes + scales at gather_scale_off
    size_t gather_scale_off;   // relative to off_gather
    size_t off_ll;        // [2][W][slot_groups][5 lines of 128 B]: staging whose every line carries its own valid mark
    size_t off_flags;     // [2 phases][2 epoch parities][kMaxWorld] uint32 flag words (epoch << 1 | failed), then 4 block
                          // counters at word 64 (low 16 bits: blocks that finished, above: blocks that gave up)
    size_t bytes;
};

__host__ __device__ inline size_t round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }

static Layout make_layout(int world, size_t max_elems) {
    Layout L;
    const size_t groups = (max_elems + kGroup - 1) / kGroup;
    const size_t shard = (groups + world - 1) / world;
    const size_t one = (kOneShotMaxElems < max_elems ? kOneShotMaxElems : max_elems) / kGroup + 1;
    L.slot_groups = shard > one ? shard : one;
    L.off_q = 0;
    L.off_s = round_up(L.off_q + 2 * static_cast<size_t>(world) * L.slot_groups * kGroup, 256);
    L.off_gather = round_up(L.off_s + 2 * static_cast<size_t>(world) * L.slot_groups * 4 * sizeof(float), 256);
    L.gather_scale_off = groups * kGroup;
    L.off_ll = round_up(L.off_gather + groups * kGroup * 2, 256);
    L.off_flags = round_up(L.off_ll + 2 * static_cast<size_t>(world) * L.slot_groups * kLlGroupBytes, 256);
    L.bytes = L.off_flags + 1024;
    return L;
}

struct Ctx {
    int rank, world;
    size_t max_elems;
    Layout L;
    uint8_t* ws[kMaxWorld];
    uint8_t* mc;          // optional NVLS multicast alias of the workspace (same layout), else nullptr
    uint8_t* reg[kMaxWorld];   // optional: every rank's registered result buffer (rank order), else nullptr
    size_t reg_bytes;
    unsigned epoch;
    bool device_epoch;    // calls are counted by the kernels (a word of the own workspace), not by the host
    unsigned long long calls;   // calls issued so far, in either mode
    int push_order;       // 0 linear, 1 rotated by rank, 2 owner-interleaved (default)
    unsigned long long* trace;   // optional: 8 globaltimer stamps of the last fused call (diagnostics)
    size_t pending_n;     // a call opened by begin_prepushed and not yet finished (0: none)
    unsigned pending_epoch;
};

struct KParams {
    uint8_t* ws[kMaxWorld];
    uint8_t* mc;         // multicast alias of every rank's workspace, or nullptr
    Layout L;
    int rank, world;
    size_t n;            // elements (multiple of 128)
    size_t groups;       // ceil(n / 512)
    unsigned epoch;      // the call's number when the host counts (epoch_dev == nullptr)
    unsigned* epoch_dev; // device-side counting: [0] completed calls of this context, [1] blocks done in the running call
    int one_shot;
    int fp8_gather;      // two-shot only: the all-gather carries re-encoded FP8 blocks instead of bf16
    int lines;           // the encoded groups travel as self-validating 128-byte lines (no flag hand-over before the reduction)
    int push_order;
    const __nv_bfloat16* x;
    __nv_bfloat16* out;  // may be nullptr (two-shot: result stays in the gather area)
    uint8_t* reg[kMaxWorld];   // direct delivery: every rank's registered result buffer, already offset to this call's
                               // position; reg[0] == nullptr means the result travels through the gather area
    int* status;
    unsigned long long* trace;
};

__device__ __forceinline__ size_t group_begin(int r, size_t groups, int world) { return groups * r / world; }

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One 16-byte store that the NVSwitch replicates into every GPU bound to the
// multicast object (the all-gather then costs one store per rank, not W).
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc_addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                   "f"(__uint_as_float(v.w))
                 : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Encodes 8 consecutive bf16 elements (one uint4) held by this lane; the 16
// lanes that share a 128-element block agree on its scale.  Elements beyond
// the end of the vector are passed as zeros.  Returns 8 bytes.
__device__ __forceinline__ uint2 encode8(const uint4 in, float& scale_out) {
    float v[8];
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = block_scale(amax);
    scale_out = s;
    BlockDivisor d;
    d.set(s);
    float t[8];
    d.div8(v, t);
    uint32_t q[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(t[4 * i], t[4 * i + 1]), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(make_float2(t[4 * i + 2], t[4 * i + 3]), __NV_SATFINITE, __NV_E4M3);
        q[i] = static_cast<uint32_t>(a) | (static_cast<uint32_t>(b) << 16);
    }
    return make_uint2(q[0], q[1]);
}

__device__ __forceinline__ void decode8(const uint2 q, float* v) {
    const uint32_t w[2] = {q.x, q.y};
#pragma unroll
    for (int i = 0; i < 2; i++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
            const __half2 hh = *reinterpret_cast<const __half2*>(&r);
            const float2 f = __half22float2(hh);
            v[4 * i + 2 * h] = f.x;
            v[4 * i + 2 * h + 1] = f.y;
        }
    }
}

// The 512 code bytes of a group: lane l holds bytes [8 l, 8 l + 8) of each 256-byte half
// (q[0], q[1]).  Returns them regrouped so that lane l holds bytes [16 l, 16 l + 16) of the
// group: remote stores of 16 bytes per lane (512 contiguous bytes per warp instruction) move
// over NVLink markedly faster than 8-byte ones.
__device__ __forceinline__ uint4 regroup16(const uint2* q, int lane) {
    const int src = (lane & 15) * 2;
    const uint32_t a0 = __shfl_sync(0xffffffffu, q[0].x, src), a1 = __shfl_sync(0xffffffffu, q[0].y, src);
    const uint32_t a2 = __shfl_sync(0xffffffffu, q[0].x, src + 1), a3 = __shfl_sync(0xffffffffu, q[0].y, src + 1);
    const uint32_t b0 = __shfl_sync(0xffffffffu, q[1].x, src), b1 = __shfl_sync(0xffffffffu, q[1].y, src);
    const uint32_t b2 = __shfl_sync(0xffffffffu, q[1].x, src + 1), b3 = __shfl_sync(0xffffffffu, q[1].y, src + 1);
    return lane < 16 ? make_uint4(a0, a1, a2, a3) : make_uint4(b0, b1, b2, b3);
}

// Work item of every kernel below: one warp per 512-element group, handled as
// two halves of 256 elements; in half h lane l owns elements [256 h + 8 l,
// 256 h + 8 l + 8).  Every load and store instruction of a warp therefore
// touches one contiguous run (512 B of bf16, 256 B of fp8): full sectors and
// full NVLink packets.  Block b of the group (128 elements) is lanes 0-15
// (b even) or 16-31 (b odd) of half b / 2.

// Called by every block at the end of a producing phase: the last block of the
// grid to get here (counted in a word of the own workspace, after a system-wide
// fence) publishes this call's flag word - (epoch << 1) | failed - in word
// [which][my rank] of every rank's flag block.  `failed` is set by any block
// whose preceding wait gave up: the data this rank was to deliver is then
// missing, and the low bit tells the peers so instead of letting them consume
// a result that was never written.  Publishing at the end of the producer - not
// at the start of the consumer - means a consumer launch never depends on a
// launch issued after it.
__device__ __forceinline__ void publish_when_grid_done(const KParams& p, const unsigned ep, int which, bool failed) {
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        unsigned word = 0;
        if (lane == 0) {
            // The block counter also carries the failure mark (bit 16 upwards), so the last block learns both from the
            // one atomic it needs anyway.  No further fence before the flag stores: every block fenced its own stores
            // before counting itself, the last block's atomic observes all those counts, and st.release orders the
            // flag after everything that happened before it.
            unsigned* cnt = reinterpret_cast<unsigned*>(p.ws[p.rank] + p.L.off_flags) + 64 + which * 2 + (ep & 1u);   // two calls may be in flight
            __threadfence_system();
            const unsigned old = atomicAdd(cnt, failed ? 0x10001u : 1u);
            if ((old & 0xFFFFu) == gridDim.x - 1) {
                *cnt = 0;                      // ready for the next launch
                word = 0x80000000u | (((old >> 16) != 0 || failed) ? 1u : 0u);
            }
        }
        word = __shfl_sync(0xffffffffu, word, 0);
        __syncwarp();
        // one lane per peer: the W release stores travel concurrently
        if (word && lane < p.world) {
            unsigned* f = reinterpret_cast<unsigned*>(p.ws[lane] + p.L.off_flags) + (which * 2 + (ep & 1u)) * kMaxWorld + p.rank;
            st_release_sys(f, (ep << 1) | (word & 1u));
        }
    }
}

// Every block waits (bounded) until all ranks have published this call's flag
// in row `which` of this rank's flag block; lane r of the first warp polls rank
// r's word, so the W acquire loads overlap.  Returns true when every rank
// arrived and none of them reported a failure; otherwise the status word gets
// RDB_DEVICE_TIMEOUT (the own wait ran out, or a peer's did and it said so).
__device__ __forceinline__ bool wait_flags(const KParams& p, const unsigned ep, int which) {
    __shared__ int ok_s;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        // one flag row per epoch parity: two calls may be in flight and may finish out of order,
        // but calls of equal parity are ordered, so each word only ever grows
        const unsigned* mine = reinterpret_cast<const unsigned*>(p.ws[p.rank] + p.L.off_flags) + (which * 2 + (ep & 1u)) * kMaxWorld;
        bool ok = true;
        if (lane < p.world) {
            // epochs only grow; a flag at or beyond this call's epoch means "arrived"
            unsigned v = ld_acquire_sys(mine + lane);
            if (static_cast<int>((v >> 1) - ep) < 0) {
                // not there yet: only now read the clock and the budget (a global load that must stay off the fast path)
                const uint64_t t0 = globaltimer_ns(), budget = wait_budget_ns();
                unsigned spins = 0;
                while (static_cast<int>(((v = ld_acquire_sys(mine + lane)) >> 1) - ep) < 0) {
                    if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > budget) { ok = false; break; }
                }
            }
            if (ok && (v >> 1) == ep && (v & 1u)) ok = false;   // that rank gave up before delivering
        }
        ok = __all_sync(0xffffffffu, ok);
        if (lane == 0) {
            if (!ok) report_timeout(p.status);
            ok_s = ok ? 1 : 0;
        }
    }
    __syncthreads();
    return ok_s != 0;
}

// The number of the call a kernel belongs to.  Ordinarily the host counts the calls and passes the number; a context
// switched to device-side counting (rdb_ar_set_device_epoch) keeps the count of completed calls in a word of its own
// workspace instead, so that a launch recorded once in a CUDA graph finds the right number on every replay.  The last
// block to finish a call stores the new count - after every block of the grid has read the old one, since a block
// counts itself only when it is done.
__device__ __forceinline__ unsigned call_epoch(const KParams& p) {
    return p.epoch_dev ? *reinterpret_cast<volatile unsigned*>(p.epoch_dev) + 1u : p.epoch;
}
__device__ __forceinline__ void call_done(const KParams& p, const unsigned ep) {
    if (p.epoch_dev == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* done = p.epoch_dev + 1;
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *done = 0;
            *reinterpret_cast<volatile unsigned*>(p.epoch_dev) = ep;
        }
    }
}

// ------------------------------------------------ flag-in-line transport
__device__ __forceinline__ void st_line16(void* addr, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_line16(const void* addr) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(addr) : "memory");
    return v;
}
// Slot of (source rank, position) in the line area of a workspace, for this call's parity.
__device__ __forceinline__ uint8_t* line_slot(const KParams& p, const unsigned ep, uint8_t* ws, int src_rank, size_t slot_g) {
    return ws + p.L.off_ll + ((static_cast<size_t>(ep & 1u) * p.world + src_rank) * p.L.slot_groups + slot_g) * kLlGroupBytes;
}

// What the two store instructions of a group carry, per lane: `a` goes to line lane / 8, position lane % 8; `b`
// (lanes 0..7 only) to line 4, position lane.  q: this lane's 8 + 8 code bytes, sc0..sc3: the group's block scales.
__device__ __forceinline__ void lines_of_group(const uint2* q, float sc0, float sc1, float sc2, float sc3, unsigned epoch, int lane,
                                               uint4& a, uint4& b) {
    const int line = lane >> 3, pos = lane & 7;
    a = make_uint4(q[0].x, q[0].y, q[1].x, q[1].y);
    // the bytes of lanes 7, 15, 23, 31 (whose position in lines 0..3 is taken by the flag) ride in line 4
    const int src = 8 * (lane & 3) + 7;
    b.x = __shfl_sync(0xffffffffu, a.x, src);
    b.y = __shfl_sync(0xffffffffu, a.y, src);
    b.z = __shfl_sync(0xffffffffu, a.z, src);
    b.w = __shfl_sync(0xffffffffu, a.w, src);
    if (pos == 7) {
        a.x = line == 0 ? __float_as_uint(sc0) : line == 1 ? __float_as_uint(sc2) : 0u;
        a.y = line == 0 ? __float_as_uint(sc1) : line == 1 ? __float_as_uint(sc3) : 0u;
        a.z = epoch;
        a.w = epoch;
    }
    if (lane >= 4) b = lane == 7 ? make_uint4(0u, 0u, epoch, epoch) : make_uint4(0u, 0u, 0u, 0u);
}

// Waits (bounded) for the five lines of one group and returns this lane's code bytes (q0: first half of the group,
// q1: second half) and the scales of its two blocks.  False when the budget ran out (decided for the whole warp).
__device__ __forceinline__ bool fetch_lines(const uint8_t* slot, unsigned epoch, int lane, uint2& q0, uint2& q1, float& s0, float& s1) {
    const int line = lane >> 3, pos = lane & 7;
    uint4 va, vb = make_uint4(0u, 0u, 0u, 0u);
    uint64_t t0 = 0, budget = 0;
    unsigned spins = 0;
    while (true) {
        va = ld_line16(slot + line * 128 + pos * 16);
        if (lane < 8) vb = ld_line16(slot + 4 * 128 + pos * 16);
        bool valid = true;
        if (pos == 7) valid = va.z == epoch && va.w == epoch && (lane != 7 || (vb.z == epoch && vb.w == epoch));
        if (__all_sync(0xffffffffu, valid)) break;
        if (spins == 0) { t0 = globaltimer_ns(); budget = wait_budget_ns(); }
        // `spins` is the same in every lane, so the whole warp takes this branch together and agrees on giving up
        if ((++spins & 0x3F) == 0 && __any_sync(0xffffffffu, globaltimer_ns() - t0 > budget)) return false;
    }
    // scales: position 7 of line 0 (lane 7) holds blocks 0, 1; of line 1 (lane 15) blocks 2, 3
    const float sc0 = __uint_as_float(__shfl_sync(0xffffffffu, va.x, 7)), sc1 = __uint_as_float(__shfl_sync(0xffffffffu, va.y, 7));
    const float sc2 = __uint_as_float(__shfl_sync(0xffffffffu, va.x, 15)), sc3 = __uint_as_float(__shfl_sync(0xffffffffu, va.y, 15));
    // lanes 7, 15, 23, 31 take their bytes from line 4 (held by lanes 0..3)
    const int src = lane >> 3;
    const uint32_t bx = __shfl_sync(0xffffffffu, vb.x, src), by = __shfl_sync(0xffffffffu, vb.y, src);
    const uint32_t bz = __shfl_sync(0xffffffffu, vb.z, src), bw = __shfl_sync(0xffffffffu, vb.w, src);
    if (pos == 7) va = make_uint4(bx, by, bz, bw);
    q0 = make_uint2(va.x, va.y);
    q1 = make_uint2(va.z, va.w);
    s0 = lane < 16 ? sc0 : sc1;
    s1 = lane < 16 ? sc2 : sc3;
    return true;
}

// ------------------------------------------------------------------ phase 1
// Loads the two 16-byte pieces this lane owns of group g (zeros past the end).
__device__ __forceinline__ void load_group(const __nv_bfloat16* x, size_t n, size_t g, int lane, uint4* in) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const size_t e = g * kGroup + 256 * h + static_cast<size_t>(lane) * 8;   // n is a multiple of 128
        in[h] = e < n ? __ldg(reinterpret_cast<const uint4*>(x + e)) : make_uint4(0, 0, 0, 0);
    }
}

// Where work item `it` of the push phase goes: the group it encodes, the slot
// position at the receiver and the receivers [first, last].  Returns false for
// an item that does not exist (a shard one group shorter than the longest).
struct PushItem {
    size_t g, slot_g;
    int first, last;
};
__device__ __forceinline__ bool push_item(const KParams& p, size_t it, size_t rot, PushItem& o) {
    if (p.one_shot) {
        o.g = o.slot_g = it;
        o.first = 0;
        o.last = p.world - 1;
        return true;
    }
    if (p.push_order == 2) {
        int owner = static_cast<int>(it % p.world) + p.rank + 1;
        while (owner >= p.world) owner -= p.world;
        o.slot_g = it / p.world;
        const size_t b = group_begin(owner, p.groups, p.world);
        if (b + o.slot_g >= group_begin(owner + 1, p.groups, p.world)) return false;   // this owner's shard is one group shorter
        o.g = b + o.slot_g;
        o.first = o.last = owner;
        return true;
    }
    size_t g = it + rot;
    if (g >= p.groups) g -= p.groups;
    int owner = static_cast<int>((g * p.world + p.world - 1) / p.groups);   // owner: largest o with begin(o) <= g
    while (owner + 1 < p.world && group_begin(owner + 1, p.groups, p.world) <= g) owner++;
    while (owner > 0 && group_begin(owner, p.groups, p.world) > g) owner--;
    o.g = g;
    o.first = o.last = owner;
    o.slot_g = g - group_begin(owner, p.groups, p.world);
    return true;
}

__device__ __forceinline__ void push_body(const KParams& p, const unsigned ep) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const size_t nwarps = (gridDim.x * static_cast<size_t>(blockDim.x)) >> 5;
    // Two-shot: group g belongs to one owner rank.  Walking the groups in linear
    // order would make every rank push to owner 0 at the same time, then to owner
    // 1, ...: one receiver's link carries all the traffic while the others idle.
    // Order 2 deals consecutive work items to consecutive owners starting after
    // this rank, so that each sender's traffic is spread evenly over all
    // receivers at every moment; order 1 walks linearly from the next rank's shard.
    const size_t shard_max = (p.groups + p.world - 1) / p.world;
    const size_t items = (p.one_shot || p.push_order != 2) ? p.groups : shard_max * p.world;
    const size_t rot = (!p.one_shot && p.push_order == 1) ? group_begin((p.rank + 1) % p.world, p.groups, p.world) : 0;
    // The loads of the next item are issued before the current one is encoded:
    // the encoder is bound by load latency (two 16-byte loads per lane and item),
    // and this keeps four of them in flight per lane.
    PushItem cur, nxt;
    uint4 in[2], in_next[2];
    bool have = warp < items && push_item(p, warp, rot, cur);
    if (have) load_group(p.x, p.n, cur.g, lane, in);
    for (size_t it = warp; it < items; it += nwarps) {
        const size_t it_next = it + nwarps;
        const bool have_next = it_next < items && push_item(p, it_next, rot, nxt);
        if (have_next) load_group(p.x, p.n, nxt.g, lane, in_next);
        if (have) {
            uint2 q[2];
            float s[2];
#pragma unroll
            for (int h = 0; h < 2; h++) q[h] = encode8(in[h], s[h]);
            // the four block scales of the group: (half 0: lanes 0, 16), (half 1: lanes 0, 16)
            const float s1 = __shfl_sync(0xffffffffu, s[0], 16), s3 = __shfl_sync(0xffffffffu, s[1], 16);
            const size_t slot = (static_cast<size_t>(ep & 1u) * p.world + p.rank) * p.L.slot_groups + cur.slot_g;
            if (p.lines) {
                const float s0b = __shfl_sync(0xffffffffu, s[0], 0), s2b = __shfl_sync(0xffffffffu, s[1], 0);
                uint4 la, lb;
                lines_of_group(q, s0b, s1, s2b, s3, ep, lane, la, lb);
                for (int k = cur.first; k <= cur.last; k++) {
                    int peer = k;
                    if (p.one_shot) {                      // start after myself: the remote lines leave first
                        peer = p.rank + 1 + k;
                        if (peer >= p.world) peer -= p.world;
                    }
                    uint8_t* dst = line_slot(p, ep, p.ws[peer], p.rank, cur.slot_g);
                    st_line16(dst + (lane >> 3) * 128 + (lane & 7) * 16, la);
                    if (lane < 8) st_line16(dst + 4 * 128 + lane * 16, lb);
                }
                have = have_next;
                cur = nxt;
                in[0] = in_next[0];
                in[1] = in_next[1];
                continue;
            }
            const uint4 q16 = regroup16(q, lane);
            for (int peer = cur.first; peer <= cur.last; peer++) {
                uint8_t* base = p.ws[peer];
                reinterpret_cast<uint4*>(base + p.L.off_q + slot * kGroup)[lane] = q16;
                if (lane == 0) {
                    float4* ds = reinterpret_cast<float4*>(base + p.L.off_s) + slot;
                    *ds = make_float4(s[0], s1, s[1], s3);
                }
            }
        }
        have = have_next;
        cur = nxt;
        in[0] = in_next[0];
        in[1] = in_next[1];
    }
}

__global__ void __launch_bounds__(kThreads) ar_push_kernel(const KParams p) {
    push_body(p, p.epoch);
    if (!p.lines) publish_when_grid_done(p, p.epoch, 0, false);
}

// ------------------------------------------------------------------ phase 2
// Returns false if a group's lines did not arrive within the budget (line transport only; with the flag-guarded
// staging the caller has already waited and passes `arrived`).
__device__ __forceinline__ bool reduce_body(const KParams& p, const unsigned ep, bool arrived) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const size_t nwarps = (gridDim.x * static_cast<size_t>(blockDim.x)) >> 5;
    const size_t gb = p.one_shot ? 0 : group_begin(p.rank, p.groups, p.world);
    const size_t ge = p.one_shot ? p.groups : group_begin(p.rank + 1, p.groups, p.world);
    uint8_t* mine = p.ws[p.rank];
    bool all_ok = true;
    for (size_t g = gb + warp; arrived && g < ge; g += nwarps) {
        const size_t slot_g = g - gb;
        float acc[2][8];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < 8; i++) acc[h][i] = 0.0f;
        bool ok = true;
        for (int r = 0; r < p.world; r++) {
            uint2 q0, q1;
            float s0, s1;
            if (p.lines) {
                if (!fetch_lines(line_slot(p, ep, mine, r, slot_g), ep, lane, q0, q1, s0, s1)) { ok = false; break; }
            } else {
                const size_t slot = (static_cast<size_t>(ep & 1u) * p.world + r) * p.L.slot_groups + slot_g;
                const uint2* src = reinterpret_cast<const uint2*>(mine + p.L.off_q + slot * kGroup) + lane;
                q0 = __ldcg(src);
                q1 = __ldcg(src + 32);
                const float* sc = reinterpret_cast<const float*>(mine + p.L.off_s) + slot * 4 + (lane >> 4);
                s0 = __ldcg(sc);
                s1 = __ldcg(sc + 2);
            }
            float v[8];
            decode8(q0, v);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[0][i] = __fadd_rn(acc[0][i], __fmul_rn(v[i], s0));   // product and sum rounded separately
            decode8(q1, v);
#pragma unroll
            for (int i = 0; i < 8; i++) acc[1][i] = __fadd_rn(acc[1][i], __fmul_rn(v[i], s1));
        }
        if (!ok) {                     // a rank's lines are missing: report, deliver nothing for this group
            if (lane == 0) report_timeout(p.status);
            all_ok = false;
            continue;
        }
        uint4 val[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const bool live = g * kGroup + 256 * h + static_cast<size_t>(lane) * 8 < p.n;
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const __nv_bfloat162 b = __floats2bfloat162_rn(acc[h][2 * i], acc[h][2 * i + 1]);
                o[i] = live ? *reinterpret_cast<const uint32_t*>(&b) : 0u;
            }
            val[h] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        if (p.fp8_gather) {
            // second variant: the bf16 result is block-quantised once more (same encoder) and travels as
            // 512 code bytes plus four scales per group; every rank decodes it in phase 3.  Blocks past
            // the end of the vector are zeros and land in the padding of the gather area.
            uint2 q[2];
            float sc[2];
#pragma unroll
            for (int h = 0; h < 2; h++) q[h] = encode8(val[h], sc[h]);
            const float s1 = __shfl_sync(0xffffffffu, sc[0], 16), s3 = __shfl_sync(0xffffffffu, sc[1], 16);
            const uint4 q16 = regroup16(q, lane);
            for (int i = 0; i < p.world; i++) {
                int peer = p.rank + 1 + i;
                if (peer >= p.world) peer -= p.world;
                uint8_t* gq = p.ws[peer] + p.L.off_gather;
                reinterpret_cast<uint4*>(gq + g * kGroup)[lane] = q16;
                if (lane == 0) reinterpret_cast<float4*>(gq + p.L.gather_scale_off)[g] = make_float4(sc[0], s1, sc[1], s3);
            }
            continue;
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t e0 = g * kGroup + 256 * h + static_cast<size_t>(lane) * 8;
            if (e0 >= p.n) continue;
            if (p.one_shot) {
                *reinterpret_cast<uint4*>(p.out + e0) = val[h];
            } else if (p.reg[0]) {
                // the ranks registered their result buffers: deliver straight into them
                for (int i = 0; i < p.world; i++) {
                    int peer = p.rank + 1 + i;
                    if (peer >= p.world) peer -= p.world;
                    *reinterpret_cast<uint4*>(p.reg[peer] + e0 * 2) = val[h];
                }
            } else if (p.mc) {
                multimem_st_v4(p.mc + p.L.off_gather + e0 * 2, val[h]);
            } else {
                for (int i = 0; i < p.world; i++) {
                    int peer = p.rank + 1 + i;
                    if (peer >= p.world) peer -= p.world;
                    *reinterpret_cast<uint4*>(p.ws[peer] + p.L.off_gather + e0 * 2) = val[h];
                }
            }
        }
    }
    return all_ok;
}

__global__ void __launch_bounds__(kThreads) ar_reduce_kernel(const KParams p) {
    const unsigned ep = call_epoch(p);
    const bool arrived = p.lines ? true : wait_flags(p, ep, 0);       // lines are waited for group by group
    const bool reduced = reduce_body(p, ep, arrived);
    // also after a timeout, so that peers are not left waiting - with the failure bit set, so that
    // they do not take the missing shard for delivered
    if (!p.one_shot) publish_when_grid_done(p, ep, 1, !arrived || !reduced);
    call_done(p, ep);                  // the closing launch of a GEMM + allreduce call on a context that counts on the device
}

// ------------------------------------------------------------------ phase 3
__device__ __forceinline__ void copy_out_body(const KParams& p) {
    if (p.out == nullptr || (p.reg[0] != nullptr && !p.fp8_gather)) return;   // nothing to copy: left in place, or delivered directly
    if (p.fp8_gather) {
        // decode: out = bf16(fp32(code) * block scale), 8 elements per thread
        const uint8_t* gq = p.ws[p.rank] + p.L.off_gather;
        const float* gs = reinterpret_cast<const float*>(gq + p.L.gather_scale_off);
        const size_t n8 = p.n / 8;
        for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
             i += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const uint2 q = __ldcg(reinterpret_cast<const uint2*>(gq) + i);
            const float s = __ldcg(gs + i / 16);
            float v[8];
            decode8(q, v);
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(v[2 * j], s), __fmul_rn(v[2 * j + 1], s));
                o[j] = *reinterpret_cast<const uint32_t*>(&b);
            }
            reinterpret_cast<uint4*>(p.out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.ws[p.rank] + p.L.off_gather);
    uint4* dst = reinterpret_cast<uint4*>(p.out);
    const size_t n16 = p.n / 8;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = __ldcg(src + i);
}

__global__ void __launch_bounds__(kThreads) ar_gather_kernel(const KParams p) {
    if (!wait_flags(p, p.epoch, 1)) return;
    copy_out_body(p);
}

// The whole call in ONE launch: every CTA pushes its share, the last one to
// finish publishes this rank's flag, every CTA then waits for all ranks' flags
// (its own included, which covers the pushes of its sibling CTAs), reduces, and
// - two-shot - repeats the publish / wait step before copying the result out.
// All CTAs must be resident together, because early CTAs wait for the last one:
// the grid is capped to what the occupancy calculator reports and the launch is
// a cooperative one, so the runtime refuses a grid that cannot be co-resident
// instead of letting part of it wait for blocks that cannot start.  Not usable when several ranks share one
// GPU: that case uses the three separate launches above.
// Diagnostics: block 0 and the last block stamp %globaltimer after each step.
__device__ __forceinline__ void stamp(const KParams& p, int slot) {
    if (p.trace && threadIdx.x == 0) {
        if (blockIdx.x == 0) p.trace[slot] = globaltimer_ns();
        if (blockIdx.x == gridDim.x - 1) p.trace[8 + slot] = globaltimer_ns();
    }
}

__global__ void __launch_bounds__(kThreads, kBlocksPerSm) ar_fused_kernel(const KParams p) {
    const unsigned ep = call_epoch(p);
    stamp(p, 0);
    push_body(p, ep);
    stamp(p, 1);
    bool arrived = true;
    if (!p.lines) {                    // flag-guarded staging: one hand-over before the reduction
        publish_when_grid_done(p, ep, 0, false);
        arrived = wait_flags(p, ep, 0);
    }
    stamp(p, 2);
    const bool reduced = reduce_body(p, ep, arrived);
    stamp(p, 3);
    if (!p.one_shot) {
        publish_when_grid_done(p, ep, 1, !arrived || !reduced);
        const bool gathered = wait_flags(p, ep, 1);
        stamp(p, 4);
        if (gathered) copy_out_body(p);
        stamp(p, 5);
    }
    call_done(p, ep);
}

// One-shot call over the line transport: a warp pushes its groups, then reduces the same groups as the lines of all
// ranks arrive.  No block waits for another block of this grid, so the launch is an ordinary one of any size.
__global__ void __launch_bounds__(kThreads) ar_oneshot_lines_kernel(const KParams p) {
    const unsigned ep = call_epoch(p);
    stamp(p, 0);
    push_body(p, ep);
    stamp(p, 1);
    reduce_body(p, ep, true);
    stamp(p, 3);
    call_done(p, ep);
}

// Standalone encoder (the quantise step alone, for bit-exact tests and callers
// that want the encoding): q [n] bytes, scales [n/128].
__global__ void __launch_bounds__(kThreads, 6) quantize_blocks128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                                     float* __restrict__ scales, size_t n, size_t groups) {
    const int lane = threadIdx.x & 31;
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const size_t nwarps = (gridDim.x * static_cast<size_t>(blockDim.x)) >> 5;
    // the loads of the next group are in flight while this one is encoded (the encoder is latency-bound)
    uint4 in[2], in_next[2];
    if (warp < groups) load_group(x, n, warp, lane, in);
    for (size_t g = warp; g < groups; g += nwarps) {
        if (g + nwarps < groups) load_group(x, n, g + nwarps, lane, in_next);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t e0 = g * kGroup + 256 * h + static_cast<size_t>(lane) * 8;
            float s;
            const uint2 enc = encode8(in[h], s);
            if (e0 < n) {
                *reinterpret_cast<uint2*>(q + e0) = enc;
                if ((lane & 15) == 0) scales[e0 / 128] = s;
            }
        }
        in[0] = in_next[0];
        in[1] = in_next[1];
    }
}

// Diagnostic: for each divisor s[i] and every bf16 bit pattern x that a block
// with that scale can hold (|x| <= 512 s, NaN included) compares the encoder's
// quotient with the IEEE quotient x / s[i]: mismatches[0] counts differing
// e4m3 bytes, mismatches[1] differing fp32 quotients among those of magnitude
// >= 2^-12 (smaller ones encode to zero whatever their last bit).  Both must be 0.
__global__ void div_check_kernel(const float* __restrict__ s, int ns, unsigned long long* mismatches) {
    for (int i = blockIdx.x; i < ns; i += gridDim.x) {
        BlockDivisor d;
        d.set(s[i]);
        unsigned bad8 = 0, bad32 = 0;
        for (unsigned b = threadIdx.x; b < 65536u; b += blockDim.x) {
            const float x = __uint_as_float(b << 16);
            if (fabsf(x) > 512.0f * s[i]) continue;         // not reachable inside a block (also drops inf)
            float xs[8] = {x, x, x, x, x, x, x, x}, q[8];
            d.div8(xs, q);
            const float a = q[0], e = __fdiv_rn(x, s[i]);
            const unsigned ca = __nv_cvt_float2_to_fp8x2(make_float2(a, a), __NV_SATFINITE, __NV_E4M3) & 0xFF;
            const unsigned ce = __nv_cvt_float2_to_fp8x2(make_float2(e, e), __NV_SATFINITE, __NV_E4M3) & 0xFF;
            if (ca != ce) bad8++;
            const bool both_nan = (a != a) && (e != e);
            if (!both_nan && fabsf(e) >= 0.000244140625f && __float_as_uint(a) != __float_as_uint(e)) bad32++;
        }
        if (bad8) atomicAdd(mismatches, static_cast<unsigned long long>(bad8));
        if (bad32) atomicAdd(mismatches + 1, static_cast<unsigned long long>(bad32));
    }
}

// Four blocks per SM: two calls issued on different streams then still fit on
// the machine together, so a kernel that waits for a peer cannot keep the
// launch that peer is waiting for off the GPU.
// The fused kernel's blocks wait on one another (through the flags of all
// ranks), so its whole grid must be resident: the cap is what the occupancy
// calculator reports for the compiled kernel, not an assumed figure.
static int fused_blocks_per_sm() {
    static int cached = 0;
    if (cached == 0) {
        int nb = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, ar_fused_kernel, kThreads, 0) != cudaSuccess || nb < 1) nb = 1;
        cached = nb < kBlocksPerSm ? nb : kBlocksPerSm;
    }
    return cached;
}

// The two words of the own flag block that hold the device-side call count and its block counter.
static unsigned* epoch_words(Ctx* c) { return reinterpret_cast<unsigned*>(c->ws[c->rank] + c->L.off_flags) + 96; }

static int grid_for(size_t warps_needed, int sm_count, int blocks_per_sm = kBlocksPerSm) {
    size_t blocks = (warps_needed * 32 + kThreads - 1) / kThreads;
    const size_t cap = static_cast<size_t>(sm_count) * blocks_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

// `prepushed`: the one-shot call's encoded input was delivered by another kernel into the flag-guarded staging area
// (GEMM epilogue), so its reduce step is the flag-waiting one; ordinary one-shot calls use the flag-in-line transport.
static int run_phase(Ctx* c, int phase, const uint16_t* x, uint16_t* out, size_t n, int algo, unsigned epoch,
                     cudaStream_t stream, bool prepushed = false) {
    int err = 0;
    DeviceInfo* info = device_info(&err);
    if (!info) return err;
    KParams p;
    memcpy(p.ws, c->ws, sizeof(p.ws));
    p.mc = c->mc;
    p.L = c->L;
    p.rank = c->rank;
    p.world = c->world;
    p.n = n;
    p.groups = (n + kGroup - 1) / kGroup;
    p.epoch = epoch;
    p.epoch_dev = (c->device_epoch && (phase == 0 || prepushed)) ? epoch_words(c) : nullptr;
    p.one_shot = algo == 1 ? 1 : 0;
    p.fp8_gather = algo == 3 ? 1 : 0;
    p.push_order = c->push_order;
    p.x = reinterpret_cast<const __nv_bfloat16*>(x);
    p.out = reinterpret_cast<__nv_bfloat16*>(out);
    p.status = info->status_dev;
    p.trace = phase == 0 ? c->trace : nullptr;
    // Direct delivery: `out` lies inside this rank's registered buffer, so the reduced shard is stored into
    // every rank's registered buffer at the same offset and nothing passes through the gather area.
    for (int i = 0; i < kMaxWorld; i++) p.reg[i] = nullptr;
    if (algo == 2 && out && c->reg[c->rank]) {
        const uintptr_t lo = reinterpret_cast<uintptr_t>(c->reg[c->rank]), o = reinterpret_cast<uintptr_t>(out);
        if (o >= lo && o + n * 2 <= lo + c->reg_bytes)
            for (int i = 0; i < c->world; i++) p.reg[i] = c->reg[i] + (o - lo);
    }
    // Transport of the FP8 leg: self-validating lines (5 lines carry 528 bytes: 21 % more wire bytes, but the first
    // hand-over disappears and the reduction starts as lines arrive - measured ahead at 16 and 64 MiB on 2 and 4 GPUs:
    // 46.9 -> 37.1 / 109.8 -> 101.6 us and 59.4 -> 48.5 / 153.1 -> 139.9 us).  RDB_AR_LINES=0 selects the flag-guarded
    // staging for two-shot calls (every rank must make the same choice); pre-pushed calls always use it.
    static const bool two_shot_lines = [] { const char* v = getenv("RDB_AR_LINES"); return !(v && v[0] == '0'); }();
    p.lines = (!prepushed && (p.one_shot || two_shot_lines)) ? 1 : 0;
    if (p.one_shot && p.lines && phase == 0) {
        ar_oneshot_lines_kernel<<<grid_for(p.groups, info->sm_count), kThreads, 0, stream>>>(p);
        return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
    }
    if (phase == 0) {
        void* args[] = {&p};
        const int grid = grid_for(p.groups, info->sm_count, fused_blocks_per_sm());
        // RDB_AR_PLAIN_LAUNCH=1: an ordinary launch of the same grid (residency then rests on the occupancy cap alone)
        static const bool plain_launch = [] { const char* v = getenv("RDB_AR_PLAIN_LAUNCH"); return v && v[0] == '1'; }();
        cudaError_t e;
        if (plain_launch) {
            ar_fused_kernel<<<grid, kThreads, 0, stream>>>(p);
            e = cudaGetLastError();
        } else {
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ar_fused_kernel), dim3(grid), dim3(kThreads), args, 0, stream);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            return RDB_CUDA_ERROR;
        }
        return RDB_SUCCESS;
    } else if (phase == 1) {
        ar_push_kernel<<<grid_for(p.groups, info->sm_count), kThreads, 0, stream>>>(p);
    } else if (phase == 2) {
        const size_t mine = p.one_shot ? p.groups : (p.groups + c->world - 1) / c->world;
        ar_reduce_kernel<<<grid_for(mine, info->sm_count), kThreads, 0, stream>>>(p);
    } else {
        if (p.one_shot) return RDB_SUCCESS;          // the one-shot result is already in `out`
        ar_gather_kernel<<<grid_for(p.out ? n / 8 / 32 + 1 : 1, info->sm_count), kThreads, 0, stream>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

static int check_call(Ctx* c, const uint16_t* x, uint16_t* out, size_t n, int& algo) {
    if (!c) return RDB_INVALID_CONFIG;
    if (n == 0 || n % 128 != 0) return RDB_BAD_SHAPE;
    if (n > c->max_elems) return RDB_SIZE_ABOVE_LIMIT;
    if (!aligned16(x) || (out && !aligned16(out))) return RDB_BAD_ALIGNMENT;
    // one-shot (every rank receives everything, flag-in-line transport, ~5 us of device time for small messages)
    // while the extra wire bytes - (W-1) x 1.25 n against (W-1)/W x 3 n for two-shot - cost less than the two
    // fenced hand-overs of two-shot: measured ahead up to 4 Mi elements on 2 and 4 GPUs (8 MiB of bf16: 20.8 us
    // against 43.6 us on 2 GPUs, 37.2 us against 50.6 us on 4); with more ranks the wire term doubles, so 2 Mi there
    if (algo == 0) algo = (out != nullptr && n <= (c->world <= 4 ? kOneShotMaxElems : kOneShotMaxElems / 2)) ? 1 : 2;
    if (algo == 1 && n > kOneShotMaxElems) return RDB_SIZE_ABOVE_LIMIT;
    if ((algo == 1 || algo == 3) && out == nullptr) return RDB_INVALID_CONFIG;
    if (algo < 1 || algo > 3) return RDB_INVALID_CONFIG;
    return RDB_SUCCESS;
}

int begin_prepushed(void* ctx, size_t n, PushTarget* t) {
    Ctx* c = static_cast<Ctx*>(ctx);
    if (!c || !t) return RDB_INVALID_CONFIG;
    if (n == 0 || n % 128 != 0) return RDB_BAD_SHAPE;
    if (n > c->max_elems || n > kOneShotMaxElems) return RDB_SIZE_ABOVE_LIMIT;
    if (c->pending_n != 0) return RDB_INVALID_CONFIG;          // one open call at a time
    for (int i = 0; i < 8; i++) t->ws[i] = i < c->world ? c->ws[i] : nullptr;
    t->off_q = c->L.off_q;
    t->off_s = c->L.off_s;
    t->off_flags = c->L.off_flags;
    t->slot_groups = c->L.slot_groups;
    t->rank = c->rank;
    t->world = c->world;
    t->epoch = ++c->epoch;
    t->epoch_dev = c->device_epoch ? epoch_words(c) : nullptr;
    c->calls++;
    c->pending_n = n;
    c->pending_epoch = t->epoch;
    return RDB_SUCCESS;
}

void cancel_prepushed(void* ctx) {
    Ctx* c = static_cast<Ctx*>(ctx);
    if (c && c->pending_n != 0) {
        c->pending_n = 0;
        c->epoch--;
        c->calls--;
    }
}

int finish_prepushed(void* ctx, uint16_t* out, cudaStream_t stream) {
    Ctx* c = static_cast<Ctx*>(ctx);
    if (!c || c->pending_n == 0) return RDB_INVALID_CONFIG;
    if (!out || !aligned16(out)) return RDB_BAD_ALIGNMENT;
    const size_t n = c->pending_n;
    c->pending_n = 0;
    // phase 2 of a one-shot call: the reduce kernel waits for every rank's "pushed" flag and writes `out`
    return run_phase(c, 2, nullptr, out, n, 1, c->pending_epoch, stream, true);
}

}  // namespace ar
}  // namespace rdb

extern "C" {

size_t rdb_ar_workspace_bytes(int world, size_t max_elems) {
    if (world < 1 || world > rdb::ar::kMaxWorld || max_elems == 0) return 0;
    return rdb::ar::make_layout(world, max_elems).bytes;
}

int rdb_ar_workspace_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return RDB_BAD_SHAPE;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) return RDB_CUDA_ERROR;
    if (cudaMemset(*ptr, 0, bytes) != cudaSuccess) return RDB_CUDA_ERROR;
    return cudaDeviceSynchronize() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

int rdb_ar_workspace_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR; }

int rdb_ar_ipc_export(void* ptr, uint8_t* handle64) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return RDB_CUDA_ERROR;
    memcpy(handle64, &h, sizeof(h));
    return RDB_SUCCESS;
}

int rdb_ar_ipc_import(const uint8_t* handle64, void** ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

int rdb_ar_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR; }

int rdb_ar_create(int rank, int world, void* const* workspaces, size_t max_elems, void** ctx) {
    if (!ctx || !workspaces || world < 1 || world > rdb::ar::kMaxWorld || rank < 0 || rank >= world || max_elems == 0)
        return RDB_INVALID_CONFIG;
    rdb::ar::Ctx* c = new rdb::ar::Ctx();
    c->rank = rank;
    c->world = world;
    c->max_elems = max_elems;
    c->L = rdb::ar::make_layout(world, max_elems);
    for (int i = 0; i < rdb::ar::kMaxWorld; i++) c->ws[i] = i < world ? static_cast<uint8_t*>(workspaces[i]) : nullptr;
    c->mc = nullptr;
    for (int i = 0; i < rdb::ar::kMaxWorld; i++) c->reg[i] = nullptr;
    c->reg_bytes = 0;
    c->epoch = 0;
    c->device_epoch = false;
    c->calls = 0;
    c->pending_n = 0;
    c->pending_epoch = 0;
    c->trace = nullptr;
    // The epoch restarts at zero, so flag words left by an earlier context over the same workspace must
    // go: this rank's flag block is cleared here.  Creation is a collective set-up step - no rank may
    // start a call before every rank's rdb_ar_create has returned.
    // ... and so must the line area, whose valid marks are epochs too (a line left by an earlier context's call of
    // the same number would otherwise pass for this context's).
    if (cudaMemset(c->ws[rank] + c->L.off_ll, 0, c->L.off_flags + 1024 - c->L.off_ll) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return RDB_CUDA_ERROR;
    }
    // tuning override for A/B measurements: RDB_AR_PUSH_ORDER = 0 (linear), 1 (rotated), 2 (interleaved, default)
    const char* po = getenv("RDB_AR_PUSH_ORDER");
    c->push_order = (po && po[0] >= '0' && po[0] <= '2' && !po[1]) ? po[0] - '0' : 2;
    *ctx = c;
    return RDB_SUCCESS;
}

int rdb_ar_set_multicast(void* ctx, void* multicast_workspace) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    if (!c) return RDB_INVALID_CONFIG;
    if (multicast_workspace && !rdb::aligned16(multicast_workspace)) return RDB_BAD_ALIGNMENT;
    c->mc = static_cast<uint8_t*>(multicast_workspace);
    return RDB_SUCCESS;
}

int rdb_ar_register_buffers(void* ctx, void* const* buffers, size_t bytes) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    if (!c) return RDB_INVALID_CONFIG;
    if (!buffers) {
        for (int i = 0; i < rdb::ar::kMaxWorld; i++) c->reg[i] = nullptr;
        c->reg_bytes = 0;
        return RDB_SUCCESS;
    }
    if (bytes == 0) return RDB_BAD_SHAPE;
    for (int i = 0; i < c->world; i++)
        if (!buffers[i] || !rdb::aligned16(buffers[i])) return RDB_BAD_ALIGNMENT;
    for (int i = 0; i < c->world; i++) c->reg[i] = static_cast<uint8_t*>(buffers[i]);
    c->reg_bytes = bytes;
    return RDB_SUCCESS;
}

int rdb_ar_set_trace(void* ctx, unsigned long long* device_buffer16) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    if (!c) return RDB_INVALID_CONFIG;
    c->trace = device_buffer16;
    return RDB_SUCCESS;
}

int rdb_ar_destroy(void* ctx) {
    delete static_cast<rdb::ar::Ctx*>(ctx);
    return RDB_SUCCESS;
}

int rdb_ar_allreduce(void* ctx, const uint16_t* x, uint16_t* out, size_t n, int algo, void* stream) {
    using namespace rdb::ar;
    Ctx* c = static_cast<Ctx*>(ctx);
    int r = check_call(c, x, out, n, algo);
    if (r != RDB_SUCCESS) return r;
    if (c->pending_n != 0) return RDB_INVALID_CONFIG;    // a fused GEMM + allreduce call is still open on this context
    // Cutting large messages into chunks on two internal streams (encoder of
    // chunk i+1 over the all-gather of chunk i) was measured slower than one
    // call (187 vs 157 us at 64 MiB on two GPUs): not done.
    const unsigned epoch = ++c->epoch;
    r = run_phase(c, 0, x, out, n, algo, epoch, static_cast<cudaStream_t>(stream));   // 0 = all phases in one launch
    if (r != RDB_SUCCESS) c->epoch--;    // nothing was launched: the ranks' epochs stay in step
    else c->calls++;
    return r;
}

int rdb_ar_set_device_epoch(void* ctx, int on) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    if (!c) return RDB_INVALID_CONFIG;
    if (c->calls != 0 || c->epoch != 0) return RDB_INVALID_CONFIG;    // the two counts would disagree from here on
    c->device_epoch = on != 0;
    return RDB_SUCCESS;
}

int rdb_ar_begin_call(void* ctx) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    if (!c || c->device_epoch) return -1;       // the separate phases take their call number from the host
    c->calls++;
    return static_cast<int>(++c->epoch);
}

int rdb_ar_phase(void* ctx, int phase, int epoch, const uint16_t* x, uint16_t* out, size_t n, int algo, void* stream) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    int r = rdb::ar::check_call(c, x, out, n, algo);
    if (r != RDB_SUCCESS) return r;
    if (phase < 1 || phase > 3 || epoch < 1 || c->device_epoch) return RDB_INVALID_CONFIG;
    return rdb::ar::run_phase(c, phase, x, out, n, algo, static_cast<unsigned>(epoch), static_cast<cudaStream_t>(stream));
}

const uint16_t* rdb_ar_result(void* ctx) {
    rdb::ar::Ctx* c = static_cast<rdb::ar::Ctx*>(ctx);
    if (!c) return nullptr;
    return reinterpret_cast<const uint16_t*>(c->ws[c->rank] + c->L.off_gather);
}

int rdb_debug_division_mismatches(const float* divisors, int count, unsigned long long* mismatches, void* stream) {
    if (count < 1) return RDB_BAD_SHAPE;
    rdb::ar::div_check_kernel<<<count < 2048 ? count : 2048, 256, 0, static_cast<cudaStream_t>(stream)>>>(divisors, count, mismatches);
    return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

int rdb_quantize_blocks128(const uint16_t* x, uint8_t* q, float* scales, size_t n, void* stream) {
    if (n == 0 || n % 128 != 0) return RDB_BAD_SHAPE;
    if (!rdb::aligned16(x) || !rdb::aligned16(q)) return RDB_BAD_ALIGNMENT;
    int err = 0;
    rdb::DeviceInfo* info = rdb::device_info(&err);
    if (!info) return err;
    const size_t groups = (n + rdb::ar::kGroup - 1) / rdb::ar::kGroup;
    // latency-bound: six resident blocks per SM (the register budget of the kernel) instead of the collectives' four
    rdb::ar::quantize_blocks128_kernel<<<rdb::ar::grid_for(groups, info->sm_count, 6), rdb::ar::kThreads, 0,
                                         static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), q, scales, n, groups);
    return cudaGetLastError() == cudaSuccess ? RDB_SUCCESS : RDB_CUDA_ERROR;
}

}  // extern "C"
