// sharding.cpp — how the path is partitioned across the GPUs of one box, behind the C ABI so that a C++ host
// (one process per GPU) takes the same decisions as the Python driver.  The reference is single-GPU
// (no cudaSetDevice, no collective anywhere in src/): nothing here has a counterpart there.
//
//   * one long sequence: contiguous page ranges per rank, sizes differing by at most one page, earlier
//     ranks taking the larger shares; every rank attends its own key range and the partials are merged;
//   * independent sequences: greedy balance of the summed cost (context length), largest unit first; a
//     family of forks (pages shared by reference count) is placed as one unit.
#include <algorithm>
#include <map>
#include <numeric>
#include <vector>

#include "../../include/drkv.h"

extern "C" {

int drkv_shard_page_range(int n_pages, int rank, int world, int* lo, int* hi) {
    if (world <= 0 || rank < 0 || rank >= world || n_pages < 0 || !lo || !hi) return DRKV_ERR_INVALID;
    const int base = n_pages / world, extra = n_pages % world;
    *lo = rank * base + std::min(rank, extra);
    *hi = *lo + base + (rank < extra ? 1 : 0);
    return DRKV_OK;
}

int drkv_shard_key_range(int seq_len, int page_size, int rank, int world, int* begin, int* end) {
    if (seq_len < 0 || page_size <= 0 || !begin || !end) return DRKV_ERR_INVALID;
    int lo = 0, hi = 0;
    const int rc = drkv_shard_page_range((seq_len + page_size - 1) / page_size, rank, world, &lo, &hi);
    if (rc != DRKV_OK) return rc;
    *begin = (int)std::min<long long>((long long)lo * page_size, seq_len);
    *end = (int)std::min<long long>((long long)hi * page_size, seq_len);
    return DRKV_OK;
}

int drkv_shard_owner_of_position(int pos, int seq_len_after, int page_size, int world) {
    if (pos < 0 || page_size <= 0 || world <= 0 || pos >= seq_len_after) return DRKV_ERR_INVALID;
    const int n_pages = (seq_len_after + page_size - 1) / page_size, page = pos / page_size;
    for (int r = 0; r < world; r++) {
        int lo = 0, hi = 0;
        drkv_shard_page_range(n_pages, r, world, &lo, &hi);
        if (lo <= page && page < hi) return r;
    }
    return DRKV_ERR_INVALID;
}

int drkv_shard_sequences(int n, const int64_t* costs, const int32_t* families, int world, int32_t* rank_of) {
    if (n < 0 || world <= 0 || (n > 0 && (!costs || !rank_of))) return DRKV_ERR_INVALID;
    // units: the members of a family in ascending order; a sequence without a family is its own unit
    std::map<long long, std::vector<int>> by_family;
    for (int i = 0; i < n; i++) by_family[families ? (long long)families[i] : (long long)i - ((long long)1 << 40)].push_back(i);
    struct Unit { std::vector<int> idx; long long cost; };
    std::vector<Unit> units;
    for (auto& kv : by_family) {
        Unit u{kv.second, 0};
        for (int i : u.idx) u.cost += costs[i];
        units.push_back(std::move(u));
    }
    std::stable_sort(units.begin(), units.end(), [](const Unit& a, const Unit& b) {
        return a.cost != b.cost ? a.cost > b.cost : a.idx[0] < b.idx[0];
    });
    std::vector<long long> load(world, 0);
    for (const Unit& u : units) {
        int r = 0;
        for (int k = 1; k < world; k++)
            if (load[k] < load[r]) r = k;          // the least loaded rank, the lowest on ties
        for (int i : u.idx) rank_of[i] = r;
        load[r] += u.cost;
    }
    return DRKV_OK;
}

}  // extern "C"
