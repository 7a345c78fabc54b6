// page_book.hpp — host bookkeeping of the paged KV cache: free stack, reference counts,
// per-sequence block tables, fork, copy-on-write, eviction.  Pure C++, no CUDA: the
// engine turns the copy jobs and dirty ranges recorded here into device work.
//
// Behaviour follows the reference where the reference has code:
//   free stack        src/memoria/block_pool.cpp:52-74   (LIFO, first pops are 0,1,2,...)
//   allocate          src/memoria/cache_manager.cpp:73-106,306-326
//   evict (stream)    src/memoria/cache_manager.cpp:118-164,185-205 (oldest allocated first,
//                     victim leaves the order list before it is examined, holes are skipped
//                     without being counted)
// and fixes the semantics the reference only describes (docs/en/architecture/02-memoria.md:25-26):
//   fork              child copies the parent's row, every shared page gets refcount + 1
//   copy-on-write     a page about to be written while refcount > 1 is replaced by a fresh
//                     page holding the sequence's valid slots of it
//   release           pages reaching refcount 0 become "cached" (contents kept) at the tail
//                     of an LRU list, or free at once when discarded
//   reclaim           when the free stack is empty the LRU head is reused; pages with
//                     refcount > 0 are never victims
#pragma once

#include <cstdint>
#include <deque>
#include <list>
#include <string>
#include <vector>

namespace drkv {

struct CowJob {
    int src_page, dst_page, n_slots;  // copy slots [0, n_slots) of K and V, every layer and head
};

struct EvictRecord {
    int32_t kind, seq, logical, page;
};

struct DirtyRange {
    int row, lo, hi;  // table[row][lo, hi) changed
};

enum class PageState : int8_t { FREE = 0, ACTIVE = 1, CACHED = 2 };

// Where a logical page of a sequence lives (BlockLocation, cache_manager.h:42-46).
enum PageLocation : int8_t { LOC_INVALID = 0, LOC_GPU = 1, LOC_SSD = 2 };

// Storage behind the pool (KVSwapper's role, kv_swapper.h:52-120).  The book decides what moves, the
// engine implements the moves; both calls are synchronous, as CacheManager's are
// (cache_manager.cpp:215-241, 243-292).
struct TierIO {
    virtual ~TierIO() = default;
    virtual bool swap_out(int seq, int logical, int page) = 0;   // page contents -> storage
    virtual bool swap_in(int seq, int logical, int page) = 0;    // storage -> page
    virtual void drop(int seq, int logical) = 0;                 // the stored copy is no longer needed
};

class PageBook {
public:
    struct Seq {
        bool live = false;
        int len = 0;
        std::vector<int32_t> table;    // logical -> page, -1 = hole / not allocated
        std::deque<int> alloc_order;   // logical indices, oldest allocation first (lru_order_)
        std::vector<int8_t> loc;       // PageLocation per logical page; only LOC_SSD is authoritative
        int dirty_lo = 0, dirty_hi = 0;
    };

    // Returns false if max_pages < 4 (block_pool.cpp:31-36).
    bool init(int max_pages, int page_size, int max_seqs, int max_pages_per_seq, bool stream_evict,
              std::string* err);

    // ---- pool (BlockPool) ----
    int pool_alloc();                 // id or -1; the caller owns the page (refcount 1)
    int pool_free(int page);          // 0 or negative status
    int free_count() const { return (int)free_stack_.size(); }
    int max_pages() const { return max_pages_; }
    int page_size() const { return page_size_; }

    // ---- sequences ----
    int seq_create();
    int seq_release(int seq, bool discard);
    int seq_fork(int parent);
    int seq_ensure_pos(int seq, int pos, std::vector<CowJob>* jobs);
    int seq_ensure_range(int seq, int pos_start, int m, std::vector<CowJob>* jobs);
    int seq_set_len(int seq, int len);
    int seq_len(int seq) const;
    int seq_num_pages(int seq) const;
    int seq_adopt(int seq, const int32_t* pages, int n_pages, int n_tokens);
    bool seq_live(int seq) const { return seq >= 0 && seq < (int)seqs_.size() && seqs_[seq].live; }
    const Seq* seq(int s) const { return seq_live(s) ? &seqs_[s] : nullptr; }

    // ---- eviction ----
    int seq_evict(int seq, int n);
    int evict_cached(int n);
    int ensure_free(int seq, int n_free);
    // Importance-guided victims (cache_manager.cpp:185-205 with importance_scorer.cu:75-87): with
    // scores attached, a sequence's victim is the resident, unshared entry of its allocation order
    // with the lowest score, the first one on ties; without candidates the oldest-first walk applies.
    // `scores` is a [max_seqs][row_width] host array the caller keeps alive; nullptr detaches.
    void attach_scores(const float* scores) { scores_ = scores; }
    // With a tier attached a sequence's own victims are written out instead of discarded, and ensure
    // on a stored page brings it back (cache_manager.cpp:84-93, 132-141).
    void attach_tier(TierIO* io) { tier_ = io; }
    int seq_location(int seq, int logical) const;
    int stored_pages() const { return n_stored_; }
    int64_t n_swap_out = 0, n_swap_in = 0;
    bool scores_attached() const { return scores_ != nullptr; }

    // ---- inspection ----
    const std::vector<int32_t>& refcounts() const { return refcount_; }
    const std::vector<int32_t>& free_stack() const { return free_stack_; }
    const std::list<int>& cached_lru() const { return lru_; }
    std::vector<EvictRecord>& evict_log() { return evict_log_; }
    int max_seqs() const { return (int)seqs_.size(); }
    int row_width() const { return row_width_; }
    int live_seqs() const { return live_; }

    // Ranges of table rows changed since the last call; clears them.
    void take_dirty(std::vector<DirtyRange>* out);

    int64_t n_evict_cached = 0, n_evict_stream = 0, n_cow = 0;

    const std::string& error() const { return err_; }

private:
    int max_pages_ = 0, page_size_ = 0, row_width_ = 0, live_ = 0;
    bool stream_evict_ = false;
    std::vector<int32_t> free_stack_;
    std::vector<int32_t> refcount_;
    std::vector<PageState> state_;
    std::vector<uint8_t> caller_owned_;                // taken by pool_alloc(): only those go back through pool_free()
    std::list<int> lru_;                               // cached pages, head = oldest release
    std::vector<std::list<int>::iterator> lru_pos_;    // valid while state == CACHED
    std::vector<Seq> seqs_;
    std::vector<EvictRecord> evict_log_;
    std::string err_;
    const float* scores_ = nullptr;
    TierIO* tier_ = nullptr;
    int n_stored_ = 0;

    int fail(int code, const std::string& msg) {
        err_ = msg;
        return code;
    }
    void mark_dirty(Seq& s, int idx) {
        if (s.dirty_lo == s.dirty_hi) {
            s.dirty_lo = idx;
            s.dirty_hi = idx + 1;
        } else {
            if (idx < s.dirty_lo) s.dirty_lo = idx;
            if (idx + 1 > s.dirty_hi) s.dirty_hi = idx + 1;
        }
    }
    // A page for `seq`: free stack, else the LRU head of the cached pages, else (stream
    // mode) after the sequence has discarded one of its own pages.  -1 when none.
    int alloc_raw();                                   // pops the free stack: the page is ACTIVE with one reference
    int take_page(int seq, bool may_store = true);
    bool evict_one_of(int seq, bool may_store = true);
    void retire(int seq, std::deque<int>::iterator it, bool may_store);
    void unref(int page, bool discard);
};

}  // namespace drkv
