// On-disk form of 2:4-compressed FP8 weights: the kept values, their 2-bit
// positions in the layout the sparse GEMM consumes and the per-tensor scale as
// one artefact, so that weights are pruned, quantised and packed once, offline.
// Host code only.  The reference has no counterpart: its async_gemm_sparse
// multiplies a dense matrix with fixed fake indices
// (projects/async_gemm_sparse/consumer.cu:65,82-88) and never stores metadata.
//
// Layout (little-endian):
//   bytes  0..7    magic "RDB24W\0\0"
//          8..11   format version (1)
//         12..15   header size in bytes (64)
//         16..19   N (weight rows)            20..23   K (logical columns, multiple of 256)
//         24..27   scale (fp32)               28..31   reserved, 0
//         32..39   size of the values section (N*K/2)
//         40..47   size of the metadata section (rdb_sparse_meta_bytes(N, K))
//         48..55   FNV-1a 64 checksum over values then metadata
//         56..63   reserved, 0
//   values [N, K/2], then metadata [ceil(N/128)][K/128][128 rows][16 B].
#include <cstdio>
#include <cstring>

#include "host_util.h"

namespace rdb {
namespace sparse_file {

constexpr char kMagic[8] = {'R', 'D', 'B', '2', '4', 'W', 0, 0};
constexpr uint32_t kVersion = 1;
constexpr uint32_t kHeaderBytes = 64;

struct Header {
    char magic[8];
    uint32_t version, header_bytes;
    int32_t N, K;
    float scale;
    uint32_t reserved0;
    uint64_t vals_bytes, meta_bytes, checksum, reserved1;
};
static_assert(sizeof(Header) == kHeaderBytes, "header layout");

static uint64_t fnv1a(uint64_t h, const uint8_t* p, size_t n) {
    for (size_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}
constexpr uint64_t kFnvBasis = 1469598103934665603ull;

// Every 4-bit entry of the metadata must name two different positions in
// ascending order (idx0 < idx1): anything else is not a 2:4 selection the
// tensor cores accept.
static bool meta_is_valid(const uint8_t* meta, size_t bytes) {
    for (size_t i = 0; i < bytes; i++) {
        for (int h = 0; h < 2; h++) {
            const int nib = (meta[i] >> (4 * h)) & 0xF;
            if ((nib & 3) >= (nib >> 2)) return false;
        }
    }
    return true;
}

static int read_header(FILE* f, Header* h) {
    if (fread(h, 1, sizeof(Header), f) != sizeof(Header)) return RDB_BAD_FILE;
    if (memcmp(h->magic, kMagic, 8) != 0 || h->version != kVersion || h->header_bytes != kHeaderBytes) return RDB_BAD_FILE;
    if (h->N < 1 || h->K < 1 || h->K % 256 != 0) return RDB_BAD_FILE;
    if (h->vals_bytes != static_cast<uint64_t>(h->N) * (h->K / 2) || h->meta_bytes != rdb_sparse_meta_bytes(h->N, h->K))
        return RDB_BAD_FILE;
    return RDB_SUCCESS;
}

}  // namespace sparse_file
}  // namespace rdb

extern "C" {

int rdb_sparse_file_write(const char* path, const uint8_t* vals, const uint8_t* meta, float scale, int N, int K) {
    using namespace rdb::sparse_file;
    if (!path || !vals || !meta) return RDB_INVALID_CONFIG;
    const size_t meta_bytes = rdb_sparse_meta_bytes(N, K);
    if (N < 1 || meta_bytes == 0) return RDB_BAD_SHAPE;
    if (!meta_is_valid(meta, meta_bytes)) return RDB_INVALID_CONFIG;
    Header h;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, kMagic, 8);
    h.version = kVersion;
    h.header_bytes = kHeaderBytes;
    h.N = N;
    h.K = K;
    h.scale = scale;
    h.vals_bytes = static_cast<uint64_t>(N) * (K / 2);
    h.meta_bytes = meta_bytes;
    h.checksum = fnv1a(fnv1a(kFnvBasis, vals, h.vals_bytes), meta, meta_bytes);
    FILE* f = fopen(path, "wb");
    if (!f) return RDB_IO_ERROR;
    const bool ok = fwrite(&h, 1, sizeof(h), f) == sizeof(h) && fwrite(vals, 1, h.vals_bytes, f) == h.vals_bytes &&
                    fwrite(meta, 1, meta_bytes, f) == meta_bytes;
    return (fclose(f) == 0 && ok) ? RDB_SUCCESS : RDB_IO_ERROR;
}

int rdb_sparse_file_pack_and_write(const char* path, const uint8_t* Wq, float scale, int N, int K) {
    if (!path || !Wq) return RDB_INVALID_CONFIG;
    const size_t meta_bytes = rdb_sparse_meta_bytes(N, K);
    if (N < 1 || meta_bytes == 0) return RDB_BAD_SHAPE;
    uint8_t* vals = new uint8_t[static_cast<size_t>(N) * (K / 2)];
    uint8_t* meta = new uint8_t[meta_bytes];
    int r = rdb_sparse_pack_2of4(Wq, N, K, vals, meta);        // RDB_INVALID_CONFIG when Wq is not 2:4
    if (r == RDB_SUCCESS) r = rdb_sparse_file_write(path, vals, meta, scale, N, K);
    delete[] vals;
    delete[] meta;
    return r;
}

int rdb_sparse_file_info(const char* path, int* N, int* K, float* scale) {
    using namespace rdb::sparse_file;
    if (!path) return RDB_INVALID_CONFIG;
    FILE* f = fopen(path, "rb");
    if (!f) return RDB_IO_ERROR;
    Header h;
    const int r = read_header(f, &h);
    fclose(f);
    if (r != RDB_SUCCESS) return r;
    if (N) *N = h.N;
    if (K) *K = h.K;
    if (scale) *scale = h.scale;
    return RDB_SUCCESS;
}

int rdb_sparse_file_read(const char* path, uint8_t* vals, size_t vals_capacity, uint8_t* meta, size_t meta_capacity) {
    using namespace rdb::sparse_file;
    if (!path || !vals || !meta) return RDB_INVALID_CONFIG;
    FILE* f = fopen(path, "rb");
    if (!f) return RDB_IO_ERROR;
    Header h;
    int r = read_header(f, &h);
    if (r == RDB_SUCCESS && (h.vals_bytes > vals_capacity || h.meta_bytes > meta_capacity)) r = RDB_SIZE_ABOVE_LIMIT;
    if (r == RDB_SUCCESS) {
        const bool ok = fread(vals, 1, h.vals_bytes, f) == h.vals_bytes && fread(meta, 1, h.meta_bytes, f) == h.meta_bytes;
        uint8_t extra;
        if (!ok || fread(&extra, 1, 1, f) != 0) r = RDB_BAD_FILE;                  // truncated, or trailing bytes
        else if (fnv1a(fnv1a(kFnvBasis, vals, h.vals_bytes), meta, h.meta_bytes) != h.checksum) r = RDB_BAD_FILE;
        else if (!meta_is_valid(meta, h.meta_bytes)) r = RDB_INVALID_CONFIG;       // intact file, but not a 2:4 selection
    }
    fclose(f);
    return r;
}

}  // extern "C"
