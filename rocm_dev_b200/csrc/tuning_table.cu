// Heuristic table the launchers consult before their analytic plans: measured
// best configurations per shape, written by the tuner (python -m
// rocm_dev_b200.tuner --table ...).  The reference tunes by rewriting #defines
// in a project's core.cu and recompiling the chosen configuration in
// (grid.py:106-116 in the reference project); here the chosen configuration is
// a line of a text file loaded at run time:
//   skinny <m_bucket: 16|32> <N> <K> <rows_per_tile> <split_k> <stages>
//   dense  <M> <N> <K> <tile_rows: 128|256|2|3> <max_ctas>
// '#' starts a comment.  The file named by the environment variable
// RDB_TUNING_TABLE is loaded on first use.  Host code only.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "host_util.h"

namespace rdb {
namespace {

struct SkinnyEntry { int mpad, N, K, rows, split_k, stages; };
struct DenseEntry { int M, N, K, tile_rows, max_ctas; };
std::mutex g_table_mu;
std::vector<SkinnyEntry> g_skinny;
std::vector<DenseEntry> g_dense;
bool g_env_checked = false;

bool skinny_ok(int mpad, int N, int K, int rows, int sk, int st) {
    return (mpad == 16 || mpad == 32) && N > 0 && K > 0 && rows >= 0 && rows <= 256 && rows % 16 == 0 && sk >= 0 && sk <= 8 &&
           st >= 0 && st <= 16;
}
bool dense_ok(int M, int N, int K, int tr, int mc) {
    return M > 0 && N > 0 && K > 0 && (tr == 0 || tr == 128 || tr == 256 || tr == 2 || tr == 3) && mc >= 0;
}

void put_skinny(const SkinnyEntry& e) {
    for (auto& x : g_skinny)
        if (x.mpad == e.mpad && x.N == e.N && x.K == e.K) { x = e; return; }
    g_skinny.push_back(e);
}
void put_dense(const DenseEntry& e) {
    for (auto& x : g_dense)
        if (x.M == e.M && x.N == e.N && x.K == e.K) { x = e; return; }
    g_dense.push_back(e);
}

// Parses a whole file before touching the table: a bad line leaves it unchanged.
int load_locked(const char* path) {
    FILE* f = fopen(path, "r");
    if (!f) return RDB_IO_ERROR;
    std::vector<SkinnyEntry> sk;
    std::vector<DenseEntry> de;
    char line[512];
    int status = RDB_SUCCESS;
    while (fgets(line, sizeof(line), f)) {
        char* hash = strchr(line, '#');
        if (hash) *hash = 0;
        char kind[16];
        int v[6], used = 0;
        if (sscanf(line, " %15s%n", kind, &used) != 1) continue;          // blank line
        if (strcmp(kind, "skinny") == 0) {
            if (sscanf(line + used, "%d %d %d %d %d %d", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5]) != 6 ||
                !skinny_ok(v[0], v[1], v[2], v[3], v[4], v[5])) { status = RDB_BAD_FILE; break; }
            sk.push_back({v[0], v[1], v[2], v[3], v[4], v[5]});
        } else if (strcmp(kind, "dense") == 0) {
            if (sscanf(line + used, "%d %d %d %d %d", &v[0], &v[1], &v[2], &v[3], &v[4]) != 5 ||
                !dense_ok(v[0], v[1], v[2], v[3], v[4])) { status = RDB_BAD_FILE; break; }
            de.push_back({v[0], v[1], v[2], v[3], v[4]});
        } else {
            status = RDB_BAD_FILE;
            break;
        }
    }
    fclose(f);
    if (status != RDB_SUCCESS) return status;
    for (const auto& e : sk) put_skinny(e);
    for (const auto& e : de) put_dense(e);
    return RDB_SUCCESS;
}

void check_env_locked() {
    if (g_env_checked) return;
    g_env_checked = true;
    const char* path = getenv("RDB_TUNING_TABLE");
    if (path && path[0] && load_locked(path) != RDB_SUCCESS)
        fprintf(stderr, "rocm_dev_b200: the tuning table %s could not be loaded; the analytic plans are used\n", path);
}

}  // namespace

bool lookup_skinny_plan(int mpad, int N, int K, int* rows, int* split_k, int* stages) {
    std::lock_guard<std::mutex> lk(g_table_mu);
    check_env_locked();
    for (const auto& e : g_skinny)
        if (e.mpad == mpad && e.N == N && e.K == K) {
            *rows = e.rows;
            *split_k = e.split_k;
            *stages = e.stages;
            return true;
        }
    return false;
}

bool lookup_dense_plan(int M, int N, int K, int* tile_rows, int* max_ctas) {
    std::lock_guard<std::mutex> lk(g_table_mu);
    check_env_locked();
    for (const auto& e : g_dense)
        if (e.M == M && e.N == N && e.K == K) {
            *tile_rows = e.tile_rows;
            *max_ctas = e.max_ctas;
            return true;
        }
    return false;
}

}  // namespace rdb

extern "C" {

int rdb_tuning_table_load(const char* path) {
    if (!path) return RDB_INVALID_CONFIG;
    std::lock_guard<std::mutex> lk(rdb::g_table_mu);
    return rdb::load_locked(path);
}

int rdb_tuning_table_set_skinny(int M, int N, int K, int rows_per_tile, int split_k, int stages) {
    if (M < 1 || M > 32) return RDB_M_ABOVE_WARPTILE_M;
    const int mpad = M <= 16 ? 16 : 32;
    if (!rdb::skinny_ok(mpad, N, K, rows_per_tile, split_k, stages)) return RDB_INVALID_CONFIG;
    std::lock_guard<std::mutex> lk(rdb::g_table_mu);
    rdb::put_skinny({mpad, N, K, rows_per_tile, split_k, stages});
    return RDB_SUCCESS;
}

int rdb_tuning_table_set_dense(int M, int N, int K, int tile_rows, int max_ctas) {
    if (!rdb::dense_ok(M, N, K, tile_rows, max_ctas)) return RDB_INVALID_CONFIG;
    std::lock_guard<std::mutex> lk(rdb::g_table_mu);
    rdb::put_dense({M, N, K, tile_rows, max_ctas});
    return RDB_SUCCESS;
}

int rdb_tuning_table_clear(void) {
    std::lock_guard<std::mutex> lk(rdb::g_table_mu);
    rdb::g_skinny.clear();
    rdb::g_dense.clear();
    rdb::g_env_checked = true;      // an explicit clear also drops what the environment variable named
    return RDB_SUCCESS;
}

int rdb_tuning_table_size(void) {
    std::lock_guard<std::mutex> lk(rdb::g_table_mu);
    rdb::check_env_locked();
    return static_cast<int>(rdb::g_skinny.size() + rdb::g_dense.size());
}

}  // extern "C"
