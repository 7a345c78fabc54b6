// Storage tier behind the page pool: a page that a sequence evicts is written to a file and read
// back on its next access.  Follows KVSwapper (src/memoria/kv_swapper.h:52-120, kv_swapper.cpp:179-300)
// and CacheManager's path naming (src/memoria/cache_manager.cpp:211-213), with the page size taken from
// the engine's runtime geometry instead of compile-time constants.
//
// File of one page: for every layer, the K plane then the V plane of that page, exactly the bytes
// pool[layer][page][K|V][kv_head][slot][dim] holds (kv_swapper.cpp:183-200).  In the pool the two planes
// of a (layer, page) are adjacent, so a page is num_layers runs of page_bytes at layer_stride: one 2-D
// copy between the pool and a pinned staging buffer moves it.
#pragma once

#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include <cuda_runtime.h>

#include "page_book.hpp"

namespace drkv {

class PageStore : public TierIO {
public:
    PageStore() = default;
    ~PageStore() override;
    PageStore(const PageStore&) = delete;
    PageStore& operator=(const PageStore&) = delete;

    // pool == nullptr (an engine without a device): files are created empty, so that the bookkeeping
    // can be exercised without a GPU; nothing is copied.
    bool init(const std::string& dir, void* pool, int num_layers, size_t layer_stride_bytes, size_t page_bytes,
              std::string* err);
    void shutdown();

    // Copies out of the pool wait for work already enqueued on this stream (the stream of the engine's
    // most recent kernel launches).
    void set_order_stream(cudaStream_t s) { order_stream_ = s; }

    bool swap_out(int seq, int logical, int page) override;
    bool swap_in(int seq, int logical, int page) override;
    void drop(int seq, int logical) override;

    // Write-behind (off by default: both moves are synchronous, as CacheManager drives its swapper,
    // cache_manager.cpp:215-241).  When on, swap_out returns as soon as the page's bytes have landed in one of a few
    // pinned buffers (the pool page is free from then on) and the worker thread writes the file
    // (kv_swapper.cpp:154-177 moves pages on an I/O thread the same way); a swap-in, drop or prefetch of that page
    // waits for its write.  A write that fails is counted; the page then cannot be read back.
    void set_write_behind(bool on) { write_behind_ = on; }
    bool write_behind() const { return write_behind_; }

    // One pool page to / from a file of the caller's choosing: what a KVSwapper::submit request asks for
    // (kv_swapper.h:36-44).  Synchronous.
    bool page_to_file(int page, const std::string& path);
    bool file_to_page(const std::string& path, int page);
    void drop_prefetch(int seq, int logical);       // kv_swapper.h:88

    // Reads a stored page into host memory in the background; the next swap_in of it skips the file
    // (kv_swapper.h:78-88).  Returns false if it is not stored.
    bool prefetch(int seq, int logical);
    bool is_prefetched(int seq, int logical);
    void drain();                                   // waits for queued prefetches

    std::string path_for(int seq, int logical) const;
    size_t file_bytes() const { return (size_t)num_layers_ * page_bytes_; }
    int64_t bytes_out = 0, bytes_in = 0, prefetch_hits = 0, writes_deferred = 0, write_failures = 0;

private:
    std::string dir_;
    char* pool_ = nullptr;
    int num_layers_ = 0;
    size_t layer_stride_ = 0, page_bytes_ = 0;
    void* staging_ = nullptr;                       // pinned, one page file
    cudaStream_t copy_stream_ = nullptr, order_stream_ = nullptr;
    cudaEvent_t order_event_ = nullptr;

    static int64_t key(int seq, int logical) { return ((int64_t)seq << 32) | (uint32_t)logical; }
    std::mutex mu_;
    std::condition_variable cv_;
    struct Job {
        int64_t key;
        int wb_buf;                                 // >= 0: write this buffer to the page's file; -1: prefetch read
    };
    std::deque<Job> queue_;
    std::unordered_set<int64_t> pending_;           // prefetch reads queued or running
    static constexpr int kWriteBehindBuffers = 4;
    bool write_behind_ = false;
    void* wb_bufs_[kWriteBehindBuffers] = {};       // pinned, one page file each (allocated on first use)
    std::vector<int> wb_free_;
    std::unordered_map<int64_t, int> wb_pending_;   // page -> buffer whose file write is queued or running
    bool copy_out(int page, void* host);            // pool page -> pinned host buffer, complete on return
    bool copy_in(const void* host, int page);
    bool write_file(const std::string& path, const void* src);
    std::unordered_map<int64_t, std::vector<char>> cache_;
    std::thread worker_;
    bool running_ = false;
    void worker_loop();
    bool read_file(const std::string& path, void* dst);
};

}  // namespace drkv
