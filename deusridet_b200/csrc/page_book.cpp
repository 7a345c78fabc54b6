// page_book.cpp — see page_book.hpp for the contract and the reference lines it follows.
#include "page_book.hpp"

#include "../../include/drkv.h"

#include <algorithm>

namespace drkv {

bool PageBook::init(int max_pages, int page_size, int max_seqs, int max_pages_per_seq,
                    bool stream_evict, std::string* err) {
    if (max_pages < 4) {  // block_pool.cpp:31-36
        if (err) *err = "pool too small: need at least 4 pages";
        return false;
    }
    if (page_size <= 0 || max_seqs <= 0) {
        if (err) *err = "page_size and max_seqs must be positive";
        return false;
    }
    max_pages_ = max_pages;
    page_size_ = page_size;
    // Logical space of 2 x physical pages unless told otherwise (cache_manager.cpp:39).
    row_width_ = max_pages_per_seq > 0 ? max_pages_per_seq : 2 * max_pages;
    stream_evict_ = stream_evict;
    free_stack_.resize(max_pages);
    for (int i = 0; i < max_pages; i++) free_stack_[i] = max_pages - 1 - i;  // block_pool.cpp:52-55
    refcount_.assign(max_pages, 0);
    state_.assign(max_pages, PageState::FREE);
    caller_owned_.assign(max_pages, 0);
    lru_.clear();
    lru_pos_.assign(max_pages, lru_.end());
    seqs_.assign(max_seqs, Seq());
    evict_log_.clear();
    live_ = 0;
    n_evict_cached = n_evict_stream = n_cow = 0;
    return true;
}

// ---------------------------------------------------------------------------------------
// pool
// ---------------------------------------------------------------------------------------

int PageBook::alloc_raw() {
    if (free_stack_.empty()) return -1;  // block_pool.cpp:63-69
    int id = free_stack_.back();
    free_stack_.pop_back();
    state_[id] = PageState::ACTIVE;
    refcount_[id] = 1;
    return id;
}

int PageBook::pool_alloc() {
    const int id = alloc_raw();
    if (id >= 0) caller_owned_[id] = 1;
    return id;
}

int PageBook::pool_free(int page) {
    if (page < 0 || page >= max_pages_) return fail(DRKV_ERR_INVALID, "free: page id out of range");
    if (state_[page] != PageState::ACTIVE)
        return fail(DRKV_ERR_STATE, "free: page is not allocated (double free?)");
    // The reference's free_block pushes whatever id it is given (block_pool.cpp:71-74); a page that a block table
    // still points to must not come back through this door.
    if (!caller_owned_[page]) return fail(DRKV_ERR_STATE, "free: page belongs to a sequence, not to the caller");
    if (refcount_[page] != 1) return fail(DRKV_ERR_STATE, "free: page is still shared");
    caller_owned_[page] = 0;
    refcount_[page] = 0;
    state_[page] = PageState::FREE;
    free_stack_.push_back(page);  // block_pool.cpp:71-74
    return DRKV_OK;
}

void PageBook::unref(int page, bool discard) {
    if (--refcount_[page] > 0) return;
    if (discard) {
        state_[page] = PageState::FREE;
        free_stack_.push_back(page);
    } else {
        state_[page] = PageState::CACHED;
        lru_.push_back(page);
        lru_pos_[page] = std::prev(lru_.end());
    }
}

int PageBook::evict_cached(int n) {
    int done = 0;
    while (done < n && !lru_.empty()) {
        int page = lru_.front();
        lru_.pop_front();
        lru_pos_[page] = lru_.end();
        state_[page] = PageState::FREE;
        free_stack_.push_back(page);
        evict_log_.push_back({0, -1, -1, page});
        n_evict_cached++;
        done++;
    }
    return done;
}

// The victim leaves the allocation order first (cache_manager.cpp:124-127); then its page is written to
// the tier (kind 2) when one is attached and the write succeeds, else discarded (kind 1).
void PageBook::retire(int seq, std::deque<int>::iterator it, bool may_store) {
    Seq& s = seqs_[seq];
    const int idx = *it, page = s.table[idx];
    s.alloc_order.erase(it);
    bool stored = false;
    if (tier_ != nullptr && may_store) stored = tier_->swap_out(seq, idx, page);   // cache_manager.cpp:132-141
    refcount_[page] = 0;
    state_[page] = PageState::FREE;
    free_stack_.push_back(page);  // cache_manager.cpp:144-147, 232-236
    s.table[idx] = -1;
    mark_dirty(s, idx);
    if (stored) {
        if (s.loc[idx] != LOC_SSD) n_stored_++;
        s.loc[idx] = LOC_SSD;
        n_swap_out++;
    } else {
        if (s.loc[idx] == LOC_SSD) {
            n_stored_--;
            if (tier_) tier_->drop(seq, idx);
        }
        s.loc[idx] = LOC_INVALID;
    }
    evict_log_.push_back({stored ? 2 : 1, seq, idx, page});
    n_evict_stream++;
}

bool PageBook::evict_one_of(int seq, bool may_store) {
    Seq& s = seqs_[seq];
    if (scores_ != nullptr) {
        const float* sc = scores_ + (size_t)seq * row_width_;
        auto best = s.alloc_order.end();
        for (auto it = s.alloc_order.begin(); it != s.alloc_order.end(); ++it) {
            const int page = s.table[*it];
            if (page < 0 || refcount_[page] > 1) continue;   // not resident / shared: not a candidate
            if (best == s.alloc_order.end() || sc[*it] < sc[*best]) best = it;   // strict <: first minimum
        }
        if (best != s.alloc_order.end()) {
            retire(seq, best, may_store);
            return true;
        }
    }
    for (auto it = s.alloc_order.begin(); it != s.alloc_order.end();) {
        int idx = *it;
        int page = s.table[idx];
        if (page < 0) {  // already a hole: dropped from the list, not counted (cache_manager.cpp:129-130)
            it = s.alloc_order.erase(it);
            continue;
        }
        if (refcount_[page] > 1) {  // shared with a fork: never a victim
            ++it;
            continue;
        }
        retire(seq, it, may_store);
        return true;
    }
    return false;
}

int PageBook::take_page(int seq, bool may_store) {
    int id = alloc_raw();
    if (id >= 0) return id;
    if (!lru_.empty()) {
        evict_cached(1);
        return alloc_raw();
    }
    if (stream_evict_ && seq_live(seq) && evict_one_of(seq, may_store)) return alloc_raw();  // cache_manager.cpp:310-319
    return -1;
}

int PageBook::seq_location(int seq, int logical) const {
    if (!seq_live(seq) || logical < 0 || logical >= row_width_) return DRKV_ERR_INVALID;
    const Seq& s = seqs_[seq];
    if (s.table[logical] >= 0) return LOC_GPU;
    return s.loc[logical] == LOC_SSD ? LOC_SSD : LOC_INVALID;
}

int PageBook::seq_evict(int seq, int n) {
    if (!seq_live(seq)) return fail(DRKV_ERR_STATE, "evict: unknown sequence");
    int done = 0;
    while (done < n && evict_one_of(seq)) done++;
    return done;
}

int PageBook::ensure_free(int seq, int n_free) {
    while (free_count() < n_free) {  // cache_manager.cpp:158-164
        if (evict_cached(1) == 1) continue;
        if (seq_live(seq) && evict_one_of(seq)) continue;
        return 0;
    }
    return 1;
}

// ---------------------------------------------------------------------------------------
// sequences
// ---------------------------------------------------------------------------------------

int PageBook::seq_create() {
    for (int i = 0; i < (int)seqs_.size(); i++) {
        Seq& s = seqs_[i];
        if (s.live) continue;
        s.live = true;
        s.len = 0;
        if ((int)s.table.size() != row_width_) s.table.assign(row_width_, -1);
        s.loc.assign(row_width_, LOC_INVALID);
        s.alloc_order.clear();
        live_++;
        return i;
    }
    return fail(DRKV_ERR_CAPACITY, "seq_create: all sequence slots are in use");
}

int PageBook::seq_release(int seq, bool discard) {
    if (!seq_live(seq)) return fail(DRKV_ERR_STATE, "release: unknown sequence");
    Seq& s = seqs_[seq];
    for (int idx = 0; idx < row_width_; idx++) {
        int page = s.table[idx];
        if (page < 0) {
            if (s.loc[idx] == LOC_SSD) {                   // its stored copy goes with the sequence
                if (tier_) tier_->drop(seq, idx);
                s.loc[idx] = LOC_INVALID;
                n_stored_--;
            }
            continue;
        }
        unref(page, discard);
        s.table[idx] = -1;
        mark_dirty(s, idx);
    }
    s.alloc_order.clear();
    s.len = 0;
    s.live = false;
    live_--;
    return DRKV_OK;
}

int PageBook::seq_fork(int parent) {
    if (!seq_live(parent)) return fail(DRKV_ERR_STATE, "fork: unknown sequence");
    int child = seq_create();
    if (child < 0) return child;
    Seq& p = seqs_[parent];
    Seq& c = seqs_[child];
    c.len = p.len;
    c.alloc_order = p.alloc_order;
    for (int idx = 0; idx < row_width_; idx++) {
        int page = p.table[idx];
        if (page < 0) continue;
        c.table[idx] = page;
        refcount_[page]++;
        mark_dirty(c, idx);
    }
    return child;
}

int PageBook::seq_ensure_pos(int seq, int pos, std::vector<CowJob>* jobs) {
    if (!seq_live(seq)) return fail(DRKV_ERR_STATE, "ensure: unknown sequence");
    if (pos < 0) return fail(DRKV_ERR_INVALID, "ensure: negative position");
    Seq& s = seqs_[seq];
    int idx = pos / page_size_;
    if (idx >= row_width_)  // cache_manager.cpp:77-81
        return fail(DRKV_ERR_CAPACITY, "ensure: position beyond the block table");
    int page = s.table[idx];
    if (page >= 0) {
        if (refcount_[page] == 1) return DRKV_OK;  // resident and private (cache_manager.cpp:84-86)
        // Shared with a fork: give this sequence its own copy before it writes.
        int fresh = take_page(seq);
        if (fresh < 0) return fail(DRKV_ERR_EXHAUSTED, "copy-on-write: no page available");
        int valid = s.len - idx * page_size_;
        valid = std::max(0, std::min(valid, page_size_));
        if (valid > 0 && jobs) jobs->push_back({page, fresh, valid});
        refcount_[page]--;
        s.table[idx] = fresh;
        mark_dirty(s, idx);
        n_cow++;
        return DRKV_OK;
    }
    if (s.loc[idx] == LOC_SSD && tier_ != nullptr) {
        // swap_block_from_ssd (cache_manager.cpp:243-292): a page for it, discarding (never storing) a
        // victim when the pool is empty; then the stored bytes; on failure the page goes back.
        int back = take_page(seq, /*may_store=*/false);
        if (back < 0) return fail(DRKV_ERR_EXHAUSTED, "swap-in: pool exhausted, nothing evictable");
        if (!tier_->swap_in(seq, idx, back)) {
            pool_free(back);
            return fail(DRKV_ERR_STATE, "swap-in: the stored page could not be read");
        }
        s.table[idx] = back;
        s.loc[idx] = LOC_INVALID;
        n_stored_--;
        n_swap_in++;
        s.alloc_order.push_back(idx);
        mark_dirty(s, idx);
        return DRKV_OK;
    }
    int fresh = take_page(seq);  // alloc_logical_block, cache_manager.cpp:306-326
    if (fresh < 0) return fail(DRKV_ERR_EXHAUSTED, "allocate: pool exhausted, nothing evictable");
    s.table[idx] = fresh;
    s.alloc_order.push_back(idx);
    mark_dirty(s, idx);
    return DRKV_OK;
}

int PageBook::seq_ensure_range(int seq, int pos_start, int m, std::vector<CowJob>* jobs) {
    if (!seq_live(seq)) return fail(DRKV_ERR_STATE, "ensure: unknown sequence");
    if (pos_start < 0) return fail(DRKV_ERR_INVALID, "ensure: negative position");
    if (m <= 0) return DRKV_OK;
    int first = pos_start / page_size_;
    int last = (pos_start + m - 1) / page_size_;
    for (int b = first; b <= last; b++) {  // cache_manager.cpp:97-106
        int rc = seq_ensure_pos(seq, b * page_size_, jobs);
        if (rc != DRKV_OK) return rc;
    }
    return DRKV_OK;
}

int PageBook::seq_set_len(int seq, int len) {
    if (!seq_live(seq)) return fail(DRKV_ERR_STATE, "set_len: unknown sequence");
    if (len < 0 || (int64_t)len > (int64_t)row_width_ * page_size_)
        return fail(DRKV_ERR_INVALID, "set_len: length out of range");
    seqs_[seq].len = len;
    return DRKV_OK;
}

int PageBook::seq_len(int seq) const { return seq_live(seq) ? seqs_[seq].len : DRKV_ERR_STATE; }

int PageBook::seq_num_pages(int seq) const {
    if (!seq_live(seq)) return DRKV_ERR_STATE;
    return (seqs_[seq].len + page_size_ - 1) / page_size_;  // cache_manager.cpp:114-116
}

int PageBook::seq_adopt(int seq, const int32_t* pages, int n_pages, int n_tokens) {
    if (!seq_live(seq)) return fail(DRKV_ERR_STATE, "adopt: unknown sequence");
    Seq& s = seqs_[seq];
    if (s.len != 0 || !s.alloc_order.empty()) return fail(DRKV_ERR_STATE, "adopt: sequence is not empty");
    if (n_pages < 0 || n_pages > row_width_ || n_tokens < 0 ||
        (int64_t)n_tokens > (int64_t)n_pages * page_size_)
        return fail(DRKV_ERR_INVALID, "adopt: page count does not cover the tokens");
    for (int i = 0; i < n_pages; i++) {
        int p = pages[i];
        if (p < 0 || p >= max_pages_) return fail(DRKV_ERR_INVALID, "adopt: page id out of range");
        if (state_[p] == PageState::FREE) return fail(DRKV_ERR_STATE, "adopt: page is free");
        for (int j = 0; j < i; j++)
            if (pages[j] == p) return fail(DRKV_ERR_INVALID, "adopt: page listed twice");
    }
    for (int i = 0; i < n_pages; i++) {
        int p = pages[i];
        if (state_[p] == PageState::CACHED) {
            lru_.erase(lru_pos_[p]);
            lru_pos_[p] = lru_.end();
            state_[p] = PageState::ACTIVE;
        }
        refcount_[p]++;
        s.table[i] = p;
        s.alloc_order.push_back(i);
        mark_dirty(s, i);
    }
    s.len = n_tokens;
    return DRKV_OK;
}

void PageBook::take_dirty(std::vector<DirtyRange>* out) {
    for (int i = 0; i < (int)seqs_.size(); i++) {
        Seq& s = seqs_[i];
        if (s.dirty_lo == s.dirty_hi) continue;
        out->push_back({i, s.dirty_lo, s.dirty_hi});
        s.dirty_lo = s.dirty_hi = 0;
    }
}

}  // namespace drkv
