// What a producer kernel outside allreduce.cu needs in order to deliver encoded
// blocks itself: the GEMM -> allreduce fusion has the GEMM epilogue quantise its
// bf16 result and store codes and scales straight into every rank's staging
// slots (one-shot layout), skipping the allreduce's own "read x, encode, push"
// phase and the HBM round trip of the GEMM output.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace rdb {
namespace ar {

struct PushTarget {
    uint8_t* ws[8];            // every rank's workspace, rank order
    size_t off_q, off_s, off_flags, slot_groups;
    int rank, world;           // world == 0: no delivery (plain GEMM)
    unsigned epoch;            // the call's number when the host counts the calls ...
    const unsigned* epoch_dev; // ... else the device word holding the number of completed calls (this call: that + 1)
};

// Opens a one-shot call on `ctx` whose encoded input another kernel delivers:
// validates n (elements, multiple of 128, within the one-shot limit), advances
// the epoch and describes where group g of this rank goes:
//   codes  ws[peer] + off_q + (((epoch & 1) * world + rank) * slot_groups + g) * 512 + block * 128
//   scale  ws[peer] + off_s + ((same slot) * 4 + block) * 4
// and, once every store of the producer grid is fenced at system scope, the flag
//   ws[peer] + off_flags + ((epoch & 1) * 8 + rank) * 4  =  epoch << 1   (st.release.sys).
int begin_prepushed(void* ctx, size_t n, PushTarget* target);
// A producer launch that failed after begin_prepushed takes the epoch back.
void cancel_prepushed(void* ctx);
// Launches the consuming half of that call: wait for all ranks' flags, decode,
// sum in rank order, one bf16 rounding into `out` (n elements).
int finish_prepushed(void* ctx, uint16_t* out, cudaStream_t stream);

}  // namespace ar
}  // namespace rdb
