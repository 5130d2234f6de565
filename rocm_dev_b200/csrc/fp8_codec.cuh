// Exact scale and division helpers shared by the FP8 encoders (the per-block
// encoder of the allreduce and the per-tensor quantiser).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace rdb {
namespace ar {

// x / s rounded to nearest, for a divisor shared by a whole block.  With inv =
// RN(1/s), q0 = RN(x*inv), r = x - q0*s (exact, one FMA) and q = RN(q0 + r*inv)
// the result equals the IEEE quotient (Markstein's correction step) whenever
// the quotient neither overflows nor goes subnormal - and inside a block
// |x| <= amax = 448 s, so |x/s| <= 448, while quotients below 2^-10 encode to
// zero either way.  Three FMA-class instructions replace a full division,
// which had made the encoder compute-bound.  `fast` is decided once per block:
// divisors that are non-finite, tiny, huge or have an all-ones significand take
// the IEEE division.  NaN elements stay NaN on both paths.
struct BlockDivisor {
    float s, inv;
    bool fast;
    __device__ __forceinline__ void set(float scale) {
        s = scale;
        const uint32_t u = __float_as_uint(scale);
        const uint32_t e = (u >> 23) & 0xFF;
        // 2^-80 <= s < 2^100: for every quotient that can reach the e4m3 grid (|q| >= 2^-12)
        // the residual x - q0*s is then a normal number, hence exact
        fast = (e > 46) && (e < 227) && ((u & 0x7FFFFFu) != 0x7FFFFFu);
        inv = __frcp_rn(scale);
    }
    __device__ __forceinline__ float div_fast(float x) const {
        const float q0 = __fmul_rn(x, inv);
        const float r = __fmaf_rn(-q0, s, x);
        return copysignf(__fmaf_rn(r, inv, q0), x);      // s > 0; keeps the sign of a zero quotient
    }
    // 8 quotients of one lane
    __device__ __forceinline__ void div8(const float* x, float* q) const {
        if (fast) {
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = div_fast(x[i]);
        } else {
            // also unrolled: a loop with a run-time index would put x and q into local memory - for the fast path too
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = __fdiv_rn(x[i], s);
        }
    }
};

// amax / 448 rounded to nearest: the same correction step with the constant
// divisor 448 (its reciprocal is rounded at compile time); amax below 2^-100
// takes the IEEE division.
__device__ __forceinline__ float block_scale(float amax) {
    if (!(amax > 0.0f)) return 1.0f;
    if (amax < 7.888609e-31f || !(amax < 3.0e38f)) return __fdiv_rn(amax, 448.0f);
    constexpr float inv448 = 1.0f / 448.0f;
    const float q0 = __fmul_rn(amax, inv448);
    const float r = __fmaf_rn(-q0, 448.0f, amax);
    return __fmaf_rn(r, inv448, q0);
}

}  // namespace ar
}  // namespace rdb
