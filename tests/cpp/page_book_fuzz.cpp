// Seeded operation mix on the host bookkeeping (PageBook: free stack, reference counts, block tables, fork,
// copy-on-write, eviction, a storage tier stub) with the invariants checked after every operation.  Built by the
// tests with -fsanitize=address,undefined: the reference's own pool has no double-free or range check
// (src/memoria/block_pool.cpp:71-74), this one must refuse bad calls with a status and never touch memory it
// does not own.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "page_book.hpp"

using namespace drkv;

namespace {

struct Rng {
    uint64_t s;
    uint64_t next() {                          // splitmix64
        uint64_t z = (s += 0x9e3779b97f4a7c15ull);
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        return z ^ (z >> 31);
    }
    int below(int n) { return (int)(next() % (uint64_t)n); }
};

// Remembers which (sequence, logical page) pairs are "stored"; fails a write now and then.
struct StubTier : TierIO {
    std::set<std::pair<int, int>> stored;
    Rng* rng;
    bool swap_out(int seq, int logical, int) override {
        if (rng->below(8) == 0) return false;
        stored.insert({seq, logical});
        return true;
    }
    bool swap_in(int seq, int logical, int) override { return stored.erase({seq, logical}) == 1; }
    void drop(int seq, int logical) override { stored.erase({seq, logical}); }
};

int check(const PageBook& b, const StubTier& tier, const std::vector<int>& held, long op) {
    const int n = b.max_pages();
    std::vector<int> refs(n, 0);
    for (int p : held) refs[p]++;
    int stored = 0;
    for (int s = 0; s < b.max_seqs(); s++) {
        const PageBook::Seq* q = b.seq(s);
        if (!q) continue;
        for (int i = 0; i < (int)q->table.size(); i++) {
            const int p = q->table[i];
            if (p >= n) return std::printf("op %ld: table entry out of range\n", op), 1;
            if (p >= 0) refs[p]++;
            if (b.seq_location(s, i) == LOC_SSD) {
                stored++;
                if (p >= 0) return std::printf("op %ld: stored page still resident\n", op), 1;
                if (!tier.stored.count({s, i})) return std::printf("op %ld: stored page unknown to the tier\n", op), 1;
            }
        }
    }
    if (stored != b.stored_pages() || stored != (int)tier.stored.size())
        return std::printf("op %ld: stored count %d / %d / %zu\n", op, stored, b.stored_pages(), tier.stored.size()), 1;
    std::vector<char> seen(n, 0);
    for (int p : b.free_stack()) {
        if (p < 0 || p >= n || seen[p]) return std::printf("op %ld: free stack corrupt\n", op), 1;
        seen[p] = 1;
        if (refs[p] != 0) return std::printf("op %ld: free page %d is referenced\n", op, p), 1;
    }
    for (int p : b.cached_lru()) {
        if (p < 0 || p >= n || seen[p]) return std::printf("op %ld: cached list corrupt\n", op), 1;
        seen[p] = 1;
        if (refs[p] != 0) return std::printf("op %ld: cached page %d is referenced\n", op, p), 1;
    }
    for (int p = 0; p < n; p++) {
        if (b.refcounts()[p] != refs[p]) return std::printf("op %ld: refcount of page %d is %d, counted %d\n", op, p, b.refcounts()[p], refs[p]), 1;
        if (!seen[p] && refs[p] == 0) return std::printf("op %ld: page %d is lost\n", op, p), 1;
    }
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    const uint64_t seed = argc > 1 ? std::strtoull(argv[1], nullptr, 10) : 1;
    const long n_ops = argc > 2 ? std::atol(argv[2]) : 20000;
    Rng rng{seed};
    PageBook book;
    std::string err;
    const int pages = 24 + rng.below(40), page = 16, seqs = 6;
    if (!book.init(pages, page, seqs, 0, rng.below(2) == 1, &err)) return std::printf("init: %s\n", err.c_str()), 1;
    StubTier tier;
    tier.rng = &rng;
    if (rng.below(2)) book.attach_tier(&tier);
    std::vector<int> held;                     // pages taken straight from the pool
    std::vector<CowJob> jobs;
    for (long op = 0; op < n_ops; op++) {
        const int s = rng.below(seqs + 2) - 1; // also -1 and an id past the end: must be refused, not crash
        jobs.clear();
        switch (rng.below(12)) {
            case 0: book.seq_create(); break;
            case 1: book.seq_release(s, rng.below(2) == 1); break;
            case 2: book.seq_fork(s); break;
            case 3: book.seq_ensure_pos(s, rng.below(3 * pages * page), &jobs); break;
            case 4: {
                const int len = book.seq_len(s);
                const int m = 1 + rng.below(3 * page);
                if (book.seq_ensure_range(s, len < 0 ? 0 : len, m, &jobs) == 0 && len >= 0) book.seq_set_len(s, len + m);
                break;
            }
            case 5: book.seq_evict(s, rng.below(4)); break;
            case 6: book.evict_cached(rng.below(4)); break;
            case 7: book.ensure_free(s, rng.below(pages + 2)); break;
            case 8: {
                const int p = book.pool_alloc();
                if (p >= 0) held.push_back(p);
                break;
            }
            case 9:
                if (!held.empty() && rng.below(2)) {
                    book.pool_free(held.back());
                    held.pop_back();
                } else {
                    // double frees, ids out of range, pages that belong to a sequence: refused; a page of `held` may go
                    const int p = rng.below(pages + 4) - 2;
                    if (book.pool_free(p) == 0) {
                        bool mine = false;
                        for (size_t i = 0; i < held.size() && !mine; i++)
                            if (held[i] == p) {
                                held.erase(held.begin() + (long)i);
                                mine = true;
                            }
                        if (!mine) return std::printf("op %ld: freed page %d that the caller did not hold\n", op, p), 1;
                    }
                }
                break;
            case 10: book.seq_set_len(s, rng.below(3 * pages * page)); break;
            default: {
                std::vector<DirtyRange> d;
                book.take_dirty(&d);
                for (const DirtyRange& r : d)
                    if (r.row < 0 || r.row >= seqs || r.lo < 0 || r.hi > book.row_width() || r.lo >= r.hi)
                        return std::printf("op %ld: bad dirty range\n", op), 1;
            }
        }
        for (const CowJob& j : jobs)
            if (j.src_page < 0 || j.src_page >= pages || j.dst_page < 0 || j.dst_page >= pages || j.n_slots < 0 || j.n_slots > page)
                return std::printf("op %ld: bad copy-on-write job\n", op), 1;
        if (check(book, tier, held, op)) return 1;
    }
    std::printf("PAGE_BOOK_FUZZ OK seed %llu ops %ld\n", (unsigned long long)seed, n_ops);
    return 0;
}
