// Storage tier behind the page pool; see page_store.hpp.
#include "page_store.hpp"

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace drkv {

PageStore::~PageStore() { shutdown(); }

bool PageStore::init(const std::string& dir, void* pool, int num_layers, size_t layer_stride_bytes,
                     size_t page_bytes, std::string* err) {
    shutdown();
    struct stat st;
    if (stat(dir.c_str(), &st) != 0 && mkdir(dir.c_str(), 0755) != 0) {   // cache_manager.cpp:56-63
        *err = "cannot create the page store directory " + dir + ": " + strerror(errno);
        return false;
    }
    dir_ = dir;
    pool_ = static_cast<char*>(pool);
    num_layers_ = num_layers;
    layer_stride_ = layer_stride_bytes;
    page_bytes_ = page_bytes;
    if (pool_ != nullptr) {
        if (cudaHostAlloc(&staging_, file_bytes(), cudaHostAllocDefault) != cudaSuccess ||
            cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&order_event_, cudaEventDisableTiming) != cudaSuccess) {
            *err = "page store: pinned staging / stream allocation failed";
            shutdown();
            return false;
        }
    }
    running_ = true;
    worker_ = std::thread(&PageStore::worker_loop, this);
    return true;
}

void PageStore::shutdown() {
    {
        std::lock_guard<std::mutex> lock(mu_);
        running_ = false;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
    if (staging_) cudaFreeHost(staging_);
    if (copy_stream_) cudaStreamDestroy(copy_stream_);
    if (order_event_) cudaEventDestroy(order_event_);
    staging_ = nullptr;
    copy_stream_ = nullptr;
    order_event_ = nullptr;
    queue_.clear();
    pending_.clear();
    cache_.clear();
}

// Row 0 uses the reference's own file name (cache_manager.cpp:211-213), so a single-sequence host finds
// the files where it expects them; further sequences get a prefix.
std::string PageStore::path_for(int seq, int logical) const {
    if (seq == 0) return dir_ + "/block_" + std::to_string(logical) + ".kv";
    return dir_ + "/seq" + std::to_string(seq) + "_block_" + std::to_string(logical) + ".kv";
}

bool PageStore::swap_out(int seq, int logical, int page) {
    const std::string path = path_for(seq, logical);
    const size_t total = file_bytes();
    if (pool_ != nullptr) {
        // kernels already enqueued on the engine's stream may still be writing this page
        if (cudaEventRecord(order_event_, order_stream_) != cudaSuccess) return false;
        if (cudaStreamWaitEvent(copy_stream_, order_event_, 0) != cudaSuccess) return false;
        if (cudaMemcpy2DAsync(staging_, page_bytes_, pool_ + (size_t)page * page_bytes_, layer_stride_, page_bytes_,
                              (size_t)num_layers_, cudaMemcpyDeviceToHost, copy_stream_) != cudaSuccess)
            return false;
        if (cudaStreamSynchronize(copy_stream_) != cudaSuccess) return false;
    }
    {
        std::unique_lock<std::mutex> lock(mu_);     // a stale prefetched copy must not outlive the rewrite
        const int64_t k = key(seq, logical);
        cv_.wait(lock, [&] { return pending_.count(k) == 0; });
        cache_.erase(k);
    }
    int fd = open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return false;
    bool ok = true;
    if (pool_ != nullptr) {
        size_t done = 0;
        while (done < total) {
            ssize_t w = write(fd, static_cast<char*>(staging_) + done, total - done);
            if (w <= 0) {
                ok = false;
                break;
            }
            done += (size_t)w;
        }
        posix_fadvise(fd, 0, (off_t)total, POSIX_FADV_DONTNEED);   // kv_swapper.cpp:217-219
    }
    close(fd);
    if (!ok) {
        unlink(path.c_str());
        return false;
    }
    bytes_out += (int64_t)total;
    return true;
}

bool PageStore::read_file(const std::string& path, void* dst) {
    const size_t total = file_bytes();
    int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) return false;
    size_t done = 0;
    while (done < total) {
        ssize_t r = read(fd, static_cast<char*>(dst) + done, total - done);
        if (r <= 0) break;
        done += (size_t)r;
    }
    posix_fadvise(fd, 0, (off_t)total, POSIX_FADV_DONTNEED);
    close(fd);
    return done == total;                            // a short file is an error (kv_swapper.cpp:262-265)
}

bool PageStore::swap_in(int seq, int logical, int page) {
    const std::string path = path_for(seq, logical);
    const int64_t k = key(seq, logical);
    if (pool_ == nullptr) {
        struct stat st;
        if (stat(path.c_str(), &st) != 0) return false;
        unlink(path.c_str());
        return true;
    }
    bool hit = false;
    {
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [&] { return pending_.count(k) == 0; });   // a prefetch of this page in flight finishes first
        auto it = cache_.find(k);
        if (it != cache_.end()) {                    // kv_swapper.cpp:243-251
            memcpy(staging_, it->second.data(), file_bytes());
            cache_.erase(it);
            hit = true;
        }
    }
    if (hit)
        prefetch_hits++;
    else if (!read_file(path, staging_))
        return false;
    if (cudaEventRecord(order_event_, order_stream_) != cudaSuccess) return false;
    if (cudaStreamWaitEvent(copy_stream_, order_event_, 0) != cudaSuccess) return false;
    if (cudaMemcpy2DAsync(pool_ + (size_t)page * page_bytes_, layer_stride_, staging_, page_bytes_, page_bytes_,
                          (size_t)num_layers_, cudaMemcpyHostToDevice, copy_stream_) != cudaSuccess)
        return false;
    if (cudaStreamSynchronize(copy_stream_) != cudaSuccess) return false;
    unlink(path.c_str());                            // the pool holds the only copy again (the reference leaves the file)
    bytes_in += (int64_t)file_bytes();
    return true;
}

void PageStore::drop(int seq, int logical) {
    {
        std::unique_lock<std::mutex> lock(mu_);
        const int64_t k = key(seq, logical);
        cv_.wait(lock, [&] { return pending_.count(k) == 0; });
        cache_.erase(k);
    }
    unlink(path_for(seq, logical).c_str());
}

bool PageStore::prefetch(int seq, int logical) {
    if (pool_ == nullptr) return true;
    struct stat st;
    if (stat(path_for(seq, logical).c_str(), &st) != 0) return false;
    const int64_t k = key(seq, logical);
    {
        std::lock_guard<std::mutex> lock(mu_);
        if (cache_.count(k) || pending_.count(k)) return true;
        pending_.insert(k);
        queue_.push_back(k);
    }
    cv_.notify_all();
    return true;
}

bool PageStore::is_prefetched(int seq, int logical) {
    std::lock_guard<std::mutex> lock(mu_);
    return cache_.count(key(seq, logical)) != 0;
}

void PageStore::drain() {
    std::unique_lock<std::mutex> lock(mu_);
    cv_.wait(lock, [&] { return pending_.empty(); });
}

void PageStore::worker_loop() {
    for (;;) {
        int64_t k;
        {
            std::unique_lock<std::mutex> lock(mu_);
            cv_.wait(lock, [&] { return !running_ || !queue_.empty(); });
            if (!running_) return;
            k = queue_.front();
            queue_.pop_front();
        }
        std::vector<char> buf(file_bytes());
        const bool ok = read_file(path_for((int)(k >> 32), (int)(uint32_t)k), buf.data());
        {
            std::lock_guard<std::mutex> lock(mu_);
            if (ok) cache_[k] = std::move(buf);
            pending_.erase(k);
        }
        cv_.notify_all();
    }
}

}  // namespace drkv
