/*
 * C ABI of librocm_dev_b200.so - B200 (sm_100a) FP8 GEMM family, sum-reduce,
 * grid barrier and FP8-encoded allreduce.
 *
 * Conventions shared by every entry point:
 *   - all data pointers are DEVICE pointers owned by the caller; nothing is
 *     allocated per call and nothing is freed;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream, which is what the reference launchers use); calls are
 *     asynchronous and return after the launch;
 *   - the return value is an rdb_status.  Codes 0..6 keep the meaning of the
 *     reference's SkinnyGemmReturnCode (projects/skinny_gemm/
 *     skinny_gemm_caller.cu:9-17); larger codes are new.  No entry point calls
 *     exit();
 *   - fp8 means OCP e4m3fn bytes (bias 7, max 448); bf16 results are written
 *     as raw 16-bit patterns;
 *   - a device-side wait that runs out of its time budget stores
 *     RDB_DEVICE_TIMEOUT in a per-device status word read (and cleared) by
 *     rdb_device_status().
 *
 * Paths are given relative to the reference project root.
 */
#ifndef ROCM_DEV_B200_H
#define ROCM_DEV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum rdb_status {
    RDB_SUCCESS = 0,
    RDB_M_ABOVE_WARPTILE_M = 1,            /* M larger than the kernel family supports */
    RDB_N_NOT_EVEN = 2,
    RDB_K_NOT_DIVISIBLE_BY_WARPTILE_K = 3, /* K (or a row pitch) breaks the 16-byte TMA rule */
    RDB_TOO_MANY_WARPS = 4,
    RDB_QSIZE_TOO_SMALL = 5,
    RDB_INVALID_CONFIG = 6,
    RDB_BAD_ALIGNMENT = 7,                 /* a base pointer is not 16-byte aligned */
    RDB_BAD_SHAPE = 8,                     /* non-positive or unsupported extent */
    RDB_CUDA_ERROR = 9,                    /* a CUDA runtime / driver call failed */
    RDB_DEVICE_TIMEOUT = 10,               /* a bounded device-side wait ran out */
    RDB_SIZE_ABOVE_LIMIT = 11,
    RDB_IO_ERROR = 12,                     /* a file could not be opened, read or written */
    RDB_BAD_FILE = 13                      /* not a file of the expected format, truncated or corrupted */
} rdb_status;

/* Human-readable name of a status code (static storage). */
const char *rdb_status_string(int status);

/* Synchronises the current device, returns the status word device code wrote
 * since the last call (RDB_SUCCESS if none) and clears it. */
int rdb_device_status(void);

/* Time budget of every bounded device-side wait on the CURRENT device, in
 * nanoseconds (default 10^9).  Synchronises the device first.  The reference's
 * counterpart is the 100 s after which its tuner gives a run up (grid.py:125-133);
 * here a wait that runs out ends the kernel with RDB_DEVICE_TIMEOUT in the
 * status word and leaves the GPU usable.  Ranks of an allreduce may enter a call
 * up to one budget apart before the early ones give up. */
int rdb_set_wait_budget_ns(unsigned long long ns);

/* Library version string and the SM architecture the kernels were built for. */
const char *rdb_version(void);

/* ------------------------------------------------------------ skinny GEMM
 * D[M,N] = bf16( (A . B^T) * scale_a[0] * scale_b[0] ),  M <= 32.
 *   A [M,K] row-major fp8; B [N,K] fp8, K-contiguous with row pitch ldb bytes;
 *   scale_a / scale_b: device pointers to one fp32 each; D [M,N] row-major
 *   bf16, OVERWRITTEN (equals the reference result under its zeroed-D
 *   precondition).
 * Replaces skinny_gemm_fastpath (projects/skinny_gemm/skinny_gemm_caller.cu:
 * 343-405) and skinny_gemm (same file :20-340), whose output type was fp16 and
 * which took a single scale; the hint arguments of the latter are accepted by
 * rdb_skinny_gemm_fp8_hinted below. */
int rdb_skinny_gemm_fp8(const uint8_t *A, const uint8_t *B, const float *scale_a, const float *scale_b,
                        uint16_t *D, int M, int N, int K, int ldb, void *stream);

/* The same contraction for operands in HOST memory - what a caller that keeps
 * its tensors on the host does end to end (the reference's drivers do the same
 * steps around their launch: tensor_h2d, kernel, tensor_d2h of projects/
 * common.cuh:50-60).  All five pointers are host pointers (pinned memory makes
 * the copies asynchronous); A, B and the two scales are copied to device
 * staging, the kernel runs, D is copied back, all on `stream`, and the call
 * returns once D holds the result.  Exception to "nothing is allocated per
 * call": the per-device staging buffers grow when a larger operand arrives
 * and are kept until the process exits.  Returns RDB_DEVICE_TIMEOUT if the
 * device status word holds a time-out when the result has arrived. */
int rdb_skinny_gemm_fp8_host(const uint8_t *A, const uint8_t *B, const float *scale_a, const float *scale_b,
                             uint16_t *D, int M, int N, int K, int ldb, void *stream);

/* Same contraction with the reference's tuning arguments
 * (projects/skinny_gemm/skinny_gemm_caller.cu:20-43).  split_k (1..8, 0 =
 * automatic) and qsize (pipeline stages, 0 = automatic) steer the kernel; the
 * producer / consumer wave counts, b_lanes, op_m and ops are validated with
 * the reference's rules (same return codes) and otherwise ignored. */
int rdb_skinny_gemm_fp8_hinted(const uint8_t *A, const uint8_t *B, const float *scale_a, const float *scale_b,
                               uint16_t *D, int M, int N, int K, int ldb, int split_k, int A_producers,
                               int B_producers, int consumers, int b_lanes, int qsize, int op_m, int ops,
                               void *stream);

/* Tuner entry: the same contraction with the kernel's own knobs exposed.
 * rows_per_tile (multiple of 16, <= 256), split_k (1..8) and stages select
 * the tiling; 0 means automatic.  The reference tunes by rewriting #defines
 * and recompiling (grid.py:106-116 and projects/skinny_gemm/core.cu:29-38);
 * here the knobs are run-time arguments.
 * flags: RDB_SKINNY_OVERLAP_PRIOR_KERNEL launches with programmatic stream
 * serialization: the kernel starts (and prefetches WEIGHTS) while the
 * preceding kernel of the stream is still finishing, and waits for it only
 * before it reads A or writes D.  Only valid when B is not written by that
 * preceding kernel. */
#define RDB_SKINNY_OVERLAP_PRIOR_KERNEL 1u
int rdb_skinny_gemm_fp8_tuned(const uint8_t *A, const uint8_t *B, const float *scale_a, const float *scale_b,
                              uint16_t *D, int M, int N, int K, int ldb, int rows_per_tile, int split_k,
                              int stages, unsigned flags, void *stream);

/* The tiling the automatic plan picks for a shape on a device with sm_count
 * SMs (pure host arithmetic, no GPU needed).  Counterpart of the compile-time
 * knobs of projects/skinny_gemm/core.cu:29-38. */
int rdb_skinny_gemm_plan(int M, int N, int K, int sm_count, int *rows_per_tile, int *split_k, int *stages);

/* Tuning table: measured best configurations per shape, consulted by
 * rdb_skinny_gemm_fp8 / _hinted (when given no knobs), rdb_skinny_gemm_plan and
 * rdb_dense_gemm_fp8 / _f32 before their analytic plans.  Written by the tuner
 * (python -m rocm_dev_b200.tuner --table FILE), loaded from a text file - lines
 * "skinny <m_bucket 16|32> <N> <K> <rows_per_tile> <split_k> <stages>" and
 * "dense <M> <N> <K> <tile_rows 128|256|2|3> <max_ctas>", 0 = automatic for a
 * knob, '#' comments - either explicitly or, on first use, from the file the
 * environment variable RDB_TUNING_TABLE names.  Process-wide, thread-safe; a
 * later entry for the same shape replaces the earlier one; a file with a bad
 * line is refused as a whole (RDB_BAD_FILE).  The reference's counterpart is
 * the configuration its tuner compiles in (grid.py:106-116 rewriting
 * projects/<name>/core.cu). */
int rdb_tuning_table_load(const char *path);
int rdb_tuning_table_set_skinny(int M, int N, int K, int rows_per_tile, int split_k, int stages);
int rdb_tuning_table_set_dense(int M, int N, int K, int tile_rows, int max_ctas);
int rdb_tuning_table_clear(void);
int rdb_tuning_table_size(void);

/* Number of clusters of cluster_size skinny-GEMM CTAs, each with smem_bytes of
 * dynamic shared memory, that the current device can hold at once (the
 * planner keeps every launch inside one such wave); -1 on error.  The
 * reference sizes its grid from a constant instead
 * (projects/skinny_gemm/core.cu:26, skinny_gemm_caller.cu:78). */
int rdb_skinny_gemm_max_clusters(int M, int cluster_size, int smem_bytes);

/* A list of independent skinny GEMMs in ONE persistent launch - what the
 * reference's timed region is (BATCH back-to-back skinny_gemm_fastpath calls on
 * different weight matrices, projects/skinny_gemm/bench.cu:51-60) and what a
 * decode step issues per layer.  The weight matrices of all problems are
 * streamed as one sequence split evenly over the SMs, so the per-launch
 * start-up and drain of rdb_skinny_gemm_fp8 is paid once per list instead of
 * once per matrix.  Every problem follows the rules of rdb_skinny_gemm_fp8
 * (same return codes); count is 1..RDB_SKINNY_GROUP_MAX.  Results are
 * deterministic (a fixed K-order sum per shape list) but, K being cut at
 * different places, may differ from rdb_skinny_gemm_fp8's in the last bf16 bit.
 *   - flags: 0, or RDB_SKINNY_OVERLAP_PRIOR_KERNEL (defined above): the launch
 *     uses programmatic stream serialization - its CTAs take SMs as the preceding
 *     kernel's CTAs leave and stream WEIGHTS while that kernel drains; activations,
 *     scales, D and the workspace are touched only once it has completed.  Only
 *     valid when no B of the list is written by the preceding kernel.
 *   - The problems must be independent: no D of the list may be an A or B of it.
 *   - Tiles shared by several CTAs are reduced through a per-device workspace
 *     (4.7 MiB, allocated on the first call): grouped calls on one device must
 *     be ordered (same stream, or otherwise serialised), not concurrent. */
#define RDB_SKINNY_GROUP_MAX 32
typedef struct rdb_skinny_problem {
    const uint8_t *A;        /* [M,K] e4m3, row-major */
    const uint8_t *B;        /* [N,K] e4m3, K-contiguous, row pitch ldb */
    const float *scale_a;    /* one fp32 each, on the device */
    const float *scale_b;
    uint16_t *D;             /* [M,N] bf16, overwritten */
    int M, N, K, ldb;
} rdb_skinny_problem;
int rdb_skinny_gemm_fp8_grouped(const rdb_skinny_problem *problems, int count, unsigned flags, void *stream);

/* The work split of a grouped call on `ctas` CTAs (pure host arithmetic, no
 * GPU): rows_per_unit[count] weight rows per streamed unit of each problem and
 * range_begin[ctas + 1], the first unit of each CTA's contiguous range (units
 * are numbered problem by problem, tile by tile, along K).  Either output may
 * be NULL.  Counterpart of the tile arithmetic of projects/skinny_gemm/
 * skinny_gemm_kernel.cu:44-69. */
int rdb_skinny_gemm_grouped_plan(const rdb_skinny_problem *problems, int count, int ctas, int *rows_per_unit,
                                 int *range_begin);

/* Diagnostics: registers a device buffer of (SM count) x 4 uint64; while
 * registered every grouped launch stores per CTA the %globaltimer at entry, at
 * its first full stage, after its last MMA and at exit.  NULL switches it off. */
int rdb_skinny_gemm_grouped_trace(unsigned long long *device_buffer);

/* Diagnostics (the reference's counterpart is reading the saved ISA,
 * class_project.py:56-61): registers a device buffer of slots x ctas_per_slot
 * x 12 uint64.  While registered, skinny launch i writes %globaltimer stamps of
 * each CTA (entry, set-up done, prior kernel done, first/last stage full,
 * accumulator done, partials exchanged, exit, epilogue ready / first TMEM load / stores issued) into slot i % slots.  NULL
 * switches tracing off.  Not thread-safe; leave off in production. */
int rdb_skinny_gemm_trace(unsigned long long *device_buffer, int slots, int ctas_per_slot);

/* -------------------------------------------------------------- dense GEMM
 * D[M,N] = bf16( (A . B^T) * scale_a[0] * scale_b[0] ), any M, N; K % 16 == 0.
 *   A [M,K] and B [N,K] row-major fp8 (K-contiguous), D [M,N] row-major bf16,
 *   OVERWRITTEN.  One persistent tcgen05 kernel replaces the three
 *   producer/consumer projects: async_gemm<T> of
 *   projects/async_gemm_16x16x64/src.cu:54-82,
 *   projects/async_gemm_blanes/sparse_k.cu:46-80 and
 *   projects/async_gemm_sparse/sparse_k.cu:45-75 (whose output was unscaled
 *   fp32 accumulated into a zeroed D, and which exit(1) on a shape that does
 *   not divide their tile; here any shape is accepted and errors are returned). */
int rdb_dense_gemm_fp8(const uint8_t *A, const uint8_t *B, const float *scale_a, const float *scale_b,
                       uint16_t *D, int M, int N, int K, void *stream);

/* Tuner entry of the dense GEMM: tile_rows selects 128 x 256 or 256 x 256 output
 * tiles computed by one CTA (128, 256), or 256 x 256 tiles computed by pairs of
 * CTAs (2: two 128-byte k-blocks per pipeline stage, three stages; 3: three
 * k-blocks per stage, two stages; K must be a multiple of 128); 0 = automatic.  max_ctas caps the
 * persistent grid (0 = one CTA per SM).  The reference fixes its tiles with #defines (projects/
 * async_gemm_16x16x64/core.cu:21-31) and retunes by recompiling (grid.py). */
int rdb_dense_gemm_fp8_tuned(const uint8_t *A, const uint8_t *B, const float *scale_a, const float *scale_b,
                             uint16_t *D, int M, int N, int K, int tile_rows, int max_ctas, void *stream);

/* The reference's own output convention for the same projects: unscaled fp32,
 * D [M,N] OVERWRITTEN (async_gemm<float>, same citations). */
int rdb_dense_gemm_fp8_f32(const uint8_t *A, const uint8_t *B, float *D, int M, int N, int K, void *stream);

/* -------------------------------------------------------- 2:4 sparse GEMM
 * D[M,N] = bf16( (A . W^T) * scale_a[0] * scale_b[0] ), M <= 256, K % 256 == 0,
 * where W [N,K] has at most two non-zero bytes in every aligned group of four
 * along K and is passed compressed: Wvals [N, K/2] (the kept bytes, in
 * position order) and Wmeta (their 2-bit positions, rdb_sparse_meta_bytes(N,K)
 * bytes in the layout rdb_sparse_pack_2of4 writes).  The reference's
 * async_gemm_sparse (projects/async_gemm_sparse/sparse_k.cu:45-75) has the
 * signature async_gemm<T>(A, B, D, m, n, k) and multiplies a DENSE B with the
 * sparse instruction and fake indices; it has no compressed format, so the two
 * extra operands are new. */
int rdb_sparse_gemm_fp8(const uint8_t *A, const uint8_t *Wvals, const uint8_t *Wmeta, const float *scale_a,
                        const float *scale_b, uint16_t *D, int M, int N, int K, void *stream);
/* Same with the K split (1, 2 or 4 CTAs per cluster; 0 = automatic) chosen by the caller. */
int rdb_sparse_gemm_fp8_tuned(const uint8_t *A, const uint8_t *Wvals, const uint8_t *Wmeta, const float *scale_a,
                              const float *scale_b, uint16_t *D, int M, int N, int K, int split_k, void *stream);
/* Same with launch flags: RDB_SKINNY_OVERLAP_PRIOR_KERNEL lets the kernel start
 * while the preceding kernel of the stream drains - it requests its first
 * ring-full of compressed weights and metadata at once and waits for that
 * kernel only before it reads A, the scales or writes D; the preceding kernel
 * must not write Wvals or Wmeta (a decode loop). */
int rdb_sparse_gemm_fp8_flags(const uint8_t *A, const uint8_t *Wvals, const uint8_t *Wmeta, const float *scale_a,
                              const float *scale_b, uint16_t *D, int M, int N, int K, int split_k, unsigned flags,
                              void *stream);
/* Host-side packer (no GPU): Wq [N,K] e4m3 bytes that already are 2:4 ->
 * vals [N,K/2] and meta.  Returns RDB_INVALID_CONFIG if a group of four holds
 * more than two non-zero bytes.  rdb_sparse_meta_bytes gives meta's size (0 for
 * an unsupported shape). */
/* A list of sparse GEMMs that share the batch size M in ONE launch (a decode
 * layer's projections): the 128-row tiles of all problems form one grid, so the
 * CTAs of a later problem start as SMs fall free and nothing of a launch's
 * fixed chain is paid per GEMM.  All M must be equal (RDB_INVALID_CONFIG
 * otherwise); N and K may differ; 1 <= count <= RDB_SPARSE_GROUP_MAX.  flags as for
 * rdb_sparse_gemm_fp8_flags.  Same bits as the single calls with the same K
 * split (automatic from the total tile count).  No reference counterpart. */
typedef struct {
    const uint8_t *A, *Wvals, *Wmeta;
    const float *scale_a, *scale_b;
    uint16_t *D;
    int M, N, K;
} rdb_sparse_problem;
#define RDB_SPARSE_GROUP_MAX 8
int rdb_sparse_gemm_fp8_grouped(const rdb_sparse_problem *problems, int count, unsigned flags, void *stream);
/* Diagnostics: registers a device buffer of slots x 8 uint64.  While registered,
 * sparse launch i writes %globaltimer stamps of its first CTA (entry, set-up
 * done, first stage full, last stage's MMAs issued, accumulator complete,
 * partials exchanged, stores issued, exit) into slot i % slots.  NULL switches
 * it off.  Not thread-safe; leave off in production. */
int rdb_sparse_gemm_trace(unsigned long long *device_buffer, int slots);
size_t rdb_sparse_meta_bytes(int N, int K);
int rdb_sparse_pack_2of4(const uint8_t *Wq, int N, int K, uint8_t *vals, uint8_t *meta);

/* On-disk form of the compressed weights - values, metadata and the per-tensor
 * scale in one file (64-byte header with magic "RDB24W", version, N, K, scale,
 * section sizes and a checksum; then values [N,K/2]; then the metadata exactly
 * as the kernel reads it), so that weights are pruned, quantised and packed
 * once, offline.  Host code, no GPU.  The reference stores no sparse weights
 * (its "sparse" project multiplies a dense B with constant indices,
 * projects/async_gemm_sparse/consumer.cu:65,82-88), so there is no reference
 * format to follow.
 *   _write           writes vals / meta as produced by rdb_sparse_pack_2of4;
 *                    RDB_INVALID_CONFIG if a metadata entry is not an ascending
 *                    pair of positions.
 *   _pack_and_write  the same from the uncompressed 2:4 bytes Wq [N,K];
 *                    RDB_INVALID_CONFIG if Wq is not 2:4.
 *   _info            header fields only (any output may be NULL).
 *   _read            loads both sections into caller buffers of the given
 *                    capacities; RDB_BAD_FILE for a wrong magic / version /
 *                    size, a truncated or over-long file or a checksum mismatch,
 *                    RDB_INVALID_CONFIG for an intact file whose metadata is not
 *                    a 2:4 selection, RDB_SIZE_ABOVE_LIMIT if a buffer is too
 *                    small, RDB_IO_ERROR if the file cannot be opened. */
int rdb_sparse_file_write(const char *path, const uint8_t *vals, const uint8_t *meta, float scale, int N, int K);
int rdb_sparse_file_pack_and_write(const char *path, const uint8_t *Wq, float scale, int N, int K);
int rdb_sparse_file_info(const char *path, int *N, int *K, float *scale);
int rdb_sparse_file_read(const char *path, uint8_t *vals, size_t vals_capacity, uint8_t *meta, size_t meta_capacity);

/* ---------------------------------------------------------- sum reduce
 * D[m,n] = sum over the batch of (A[i,m,n] + B[i,m,n]), fp32, summed in batch
 * order (bit-identical to the host loop).  A, B [b,m,n], D [m,n], any m, n;
 * b = 0 writes zeros.  Replaces tiled_sum_reduce(A, B, D, b, m, n) of
 * projects/tiled_sum_reduce/src.cu:52-73 and projects/tiled_sum_reduce_async/
 * src.cu:179-200 (which only warn when m % 8 or n % 64 is non-zero). */
int rdb_tiled_sum_reduce(const float *A, const float *B, float *D, int b, int m, int n, void *stream);

/* ---------------------------------------------------------- grid barrier
 * The reference's barrier probe, globs(uint* D) of projects/global_sync/
 * src.cu:15-27: 2 blocks x 64 threads write D[block] = 0, meet at a grid-wide
 * barrier, then atomicDec D[block].  D needs one word per block.  The barrier
 * is a bounded counter barrier (RDB_DEVICE_TIMEOUT in the status word if it
 * runs out); its two counter words live in a per-device allocation made on the
 * first call. */
int rdb_globs(uint32_t *D, void *stream);

/* The same probe with `blocks` x `threads` and the write/barrier/decrement body
 * repeated `rounds` times (barrier latency at full-grid size).  blocks must be
 * co-resident (cooperative launch). */
int rdb_globs_n(uint32_t *D, int blocks, int threads, int rounds, void *stream);

/* ------------------------------------------------ FP8-encoded allreduce
 * out[i] = bf16( sum over ranks r = 0..world-1, in rank order, of
 * fp32(q_r[i]) * s_r[i / 128] ), where (q_r, s_r) encodes rank r's bf16 vector
 * in blocks of 128: s = amax/448 (1 for an all-zero block), q =
 * e4m3fn_sat_rn(x / s).  Identical bits on every rank.  One process per GPU;
 * encoded blocks travel as stores into peer memory over NVLink.  The reference
 * names this path (an FP8 allreduce over mscclpp) but contains no code for it,
 * so there is no reference interface to cite; tiled_sum_reduce
 * (projects/tiled_sum_reduce/src.cu:52-73) is its local reduction step.
 *
 * Set-up, once per rank: size a workspace, allocate it (it must come from
 * rdb_ar_workspace_alloc so that it can be exported), export its 64-byte IPC
 * handle, exchange handles between the processes, import the peers', then
 * create the context with the `world` workspace pointers in rank order (the
 * own one at index `rank`). */
size_t rdb_ar_workspace_bytes(int world, size_t max_elems);
int rdb_ar_workspace_alloc(size_t bytes, void **ptr);
int rdb_ar_workspace_free(void *ptr);
int rdb_ar_ipc_export(void *ptr, uint8_t *handle64);
int rdb_ar_ipc_import(const uint8_t *handle64, void **ptr);
int rdb_ar_ipc_close(void *ptr);
int rdb_ar_create(int rank, int world, void *const *workspaces, size_t max_elems, void **ctx);
int rdb_ar_destroy(void *ctx);
/* Optional: a multicast (NVLS) address that aliases EVERY rank's workspace with
 * the same layout - e.g. the multicast pointer of a symmetric-memory
 * allocation used as the workspace.  The bf16 all-gather of the two-shot
 * algorithm then uses multimem.st (one store reaches all ranks).  NULL switches
 * back to per-peer stores.  Every rank must make the same choice. */
int rdb_ar_set_multicast(void *ctx, void *multicast_workspace);
/* Optional: result buffers that peers may write.  `buffers` holds `world`
 * device pointers in rank order (the own one at index rank), each to `bytes`
 * bytes that every rank can store into - e.g. allocations of
 * rdb_ar_workspace_alloc shared through rdb_ar_ipc_export / _import, or a
 * symmetric-memory allocation.  A two-shot call (algo 2, or 0 resolving to 2)
 * whose `out` lies inside the own registered buffer then has every rank store
 * its reduced shard straight into all ranks' buffers at that offset, and the
 * copy out of the workspace disappears; every rank must pass the same offset.
 * Same result bits.  NULL unregisters.  Like rdb_ar_result, the buffer must not
 * be read by work queued after this rank's NEXT call. */
int rdb_ar_register_buffers(void *ctx, void *const *buffers, size_t bytes);
/* Optional, before the context's first call and on every rank alike: count the
 * calls on the device (a word of the own workspace that the last block of each
 * call advances) instead of on the host.  rdb_ar_allreduce and
 * rdb_skinny_gemm_fp8_allreduce launches then carry nothing that changes from
 * call to call, so they may be recorded in a CUDA graph (stream capture) and
 * replayed - with the buffers they were recorded with - any number of times,
 * mixed with direct calls.  All calls of such a context must be ordered among
 * themselves (one stream, or graph / event dependencies), and every rank must
 * issue the same sequence.  Make one call before the first capture (per-device
 * set-up allocates).  rdb_ar_phase / rdb_ar_begin_call are refused
 * (RDB_INVALID_CONFIG, -1) on such a context.  Returns RDB_INVALID_CONFIG once a
 * call has been issued. */
int rdb_ar_set_device_epoch(void *ctx, int on);
/* Diagnostics: registers a device buffer of 16 uint64.  While registered, each
 * rdb_ar_allreduce call stores %globaltimer stamps of its first CTA in words
 * 0-5 (entry, own pushes issued, all ranks' pushes arrived, own reduction and
 * all-gather stores issued, all ranks' gathers arrived, exit) and of its last
 * CTA in words 8-13.  NULL switches it off.  No reference counterpart. */
int rdb_ar_set_trace(void *ctx, unsigned long long *device_buffer16);

/* Failure behaviour: every wait is bounded (rdb_set_wait_budget_ns).  A rank
 * whose wait for its peers' encoded blocks runs out reports RDB_DEVICE_TIMEOUT
 * in its status word and still publishes its "delivered" flag, marked failed,
 * so that the others neither wait for it nor take its missing shard for
 * delivered: they report RDB_DEVICE_TIMEOUT too and leave `out` unwritten.
 * rdb_device_status() after a call tells whether `out` is valid.
 *
 * Collective: every rank calls it with the same n (a multiple of 128, at most
 * max_elems) and algo (0 automatic: one-shot up to 2^22 elements on up to four
 * ranks, 2^21 on more, when out is given, else two-shot; 1 one-shot: every rank
 * receives and reduces everything, n <= 2^22 - the encoded groups travel as
 * 128-byte lines that carry their own valid mark, so the receivers poll the
 * data itself and no fence or flag hand-over is paid; 2 two-shot: FP8 reduce-scatter
 * then bf16 all-gather; 3 two-shot with an FP8 all-gather: the reduced bf16
 * shard is block-quantised a second time before it travels, so the result is
 * decode(encode(result of algo 2)) - fewer bytes on the wire, one more
 * quantisation error; never chosen automatically).  x, out: device pointers to
 * n bf16.  out may be NULL for algo 2: the result then stays in the workspace
 * (rdb_ar_result) until this rank's next call. */
int rdb_ar_allreduce(void *ctx, const uint16_t *x, uint16_t *out, size_t n, int algo, void *stream);
const uint16_t *rdb_ar_result(void *ctx);

/* Row-parallel linear layer + allreduce in two launches instead of three and
 * without the bf16 intermediate in HBM: every rank multiplies its K slice,
 *   P_r[M,N] = bf16((A_r . B_r^T) * scale_a * scale_b)     (the problem, as for rdb_skinny_gemm_fp8_grouped),
 * and out = the FP8-encoded allreduce of the P_r as defined above (flattened
 * [M*N], blocks of 128 along N), identical bits on every rank.  The GEMM
 * epilogue quantises its result and stores codes and scales straight into
 * every rank's staging slots - the allreduce's "read x, encode, push" step and
 * the round trip of P_r through HBM disappear; the second launch waits for all
 * ranks, decodes, sums in rank order and writes `out` (M*N bf16).  problem->D
 * is not written (may be NULL).  Requires N % 128 == 0 and M*N <= 2^22 (the
 * one-shot limit) and <= the context's max_elems.  The result equals
 * rdb_ar_allreduce (one-shot) applied to the D that
 * rdb_skinny_gemm_fp8_grouped(problem, 1) writes, bit for bit.  Collective:
 * every rank calls it with the same M and N.  No reference counterpart (the
 * reference has neither collective nor fused epilogue); the epilogue it
 * replaces is projects/skinny_gemm/consumers/mfma_16x16x32_consumer.cu:111-162.
 * _begin / _finish are the two launches one by one, for drivers that emulate
 * several ranks on ONE GPU: _begin for every rank before _finish for any. */
int rdb_skinny_gemm_fp8_allreduce(void *ar_ctx, const rdb_skinny_problem *problem, uint16_t *out, void *stream);
int rdb_skinny_gemm_fp8_allreduce_begin(void *ar_ctx, const rdb_skinny_problem *problem, void *stream);
int rdb_skinny_gemm_fp8_allreduce_finish(void *ar_ctx, uint16_t *out, void *stream);

/* The three launches of a call one by one (phase 1 push, 2 reduce, 3 gather),
 * all with the epoch rdb_ar_begin_call returned.  For drivers that emulate
 * several ranks on ONE GPU: issue phase p for every rank before phase p+1 for
 * any, so that no launch waits for one that has not been issued. */
int rdb_ar_begin_call(void *ctx);
int rdb_ar_phase(void *ctx, int phase, int epoch, const uint16_t *x, uint16_t *out, size_t n, int algo,
                 void *stream);

/* The encoding step alone: q [n] e4m3fn bytes and scales [n/128] of a bf16
 * vector (n a multiple of 128), bit-exact with the definition above. */
int rdb_quantize_blocks128(const uint16_t *x, uint8_t *q, float *scales, size_t n, void *stream);

/* Per-tensor quantiser, the step before every GEMM above: scale[0] = amax/448
 * (1 for an all-zero tensor), q[i] = e4m3fn_sat_rn(x[i] / scale[0]) for a bf16
 * vector x of n elements (device pointers; x 16-byte aligned).  One cooperative
 * kernel; bit-exact with the host rule.  The maximum is combined in a small
 * per-device scratch area owned by the library: calls on one device must be
 * ordered (same stream, or otherwise serialised), not concurrent.  The reference's drivers draw fp8 values
 * directly (projects/common.cuh:97-105) and have no counterpart. */
int rdb_quantize_per_tensor(const uint16_t *x, uint8_t *q, float *scale, size_t n, void *stream);

/* Diagnostic for the encoder's division: for each of `count` fp32 divisors
 * (device array) and every bf16 bit pattern x a block with that scale can hold
 * (|x| <= 512 * divisor, NaN included) compares the encoder's quotient with
 * the IEEE quotient x / divisor.  Adds to mismatches[0] (device, two uint64
 * zeroed by the caller) the number of differing e4m3 encodings - expected 0 -
 * and to mismatches[1] the number of differing fp32 quotients of magnitude
 * >= 2^-12 - expected 0 too.  No counterpart in the reference. */
int rdb_debug_division_mismatches(const float *divisors, int count, unsigned long long *mismatches, void *stream);

/* rdb_globs_n for callers that must not allocate device memory while they
 * run - a host application that owns all GPU memory and gives its plugins a
 * fixed arena, or a latency-critical loop where a device allocation (it
 * synchronises the whole GPU) cannot be tolerated.  This entry point has no
 * counterpart in the reference.  It never calls cudaMalloc / cudaFree or any
 * other allocating routine: the two barrier counters and a status word live in
 * a 256-byte array compiled into the library (each GPU that loads the library
 * holds it until the process exits).  The caller still passes D.
 *   - Limit: at most 1024 blocks, blocks x rounds <= 2^30, and no more blocks
 *     than the device can hold at once (the barrier needs the whole grid
 *     resident: 148 SMs x the blocks of `threads` threads that fit one SM);
 *     anything larger returns RDB_SIZE_ABOVE_LIMIT and prints the reason on
 *     stderr, before anything is queued on the stream.
 *   - The first call on each device looks up the array's device address; make
 *     that first call before starting any stream capture.
 *   - All calls on one GPU share the array.  The counters are cleared (on
 *     `stream`) before every launch, so a call is independent of what the
 *     previous one left behind; two calls whose kernels overlap on the GPU
 *     (different streams) race on the counters - serialise them.
 *   - A timed-out barrier is reported through rdb_noalloc_status(), not
 *     through rdb_device_status().  The word is sticky: it keeps a time-out
 *     until rdb_noalloc_status() has returned it, also across later calls. */
int rdb_globs_n_noalloc(uint32_t *D, int blocks, int threads, int rounds, void *stream);

/* Synchronises the current device and returns (and clears) the status word of
 * the built-in scratch: RDB_SUCCESS or RDB_DEVICE_TIMEOUT.  Allocates nothing. */
int rdb_noalloc_status(void);

#ifdef __cplusplus
}
#endif

#endif /* ROCM_DEV_B200_H */
