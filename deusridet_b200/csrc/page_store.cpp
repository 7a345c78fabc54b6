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
    if (running_) drain();                           // deferred writes reach their files before the worker stops
    {
        std::lock_guard<std::mutex> lock(mu_);
        running_ = false;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
    if (staging_) cudaFreeHost(staging_);
    for (void*& b : wb_bufs_) {
        if (b) cudaFreeHost(b);
        b = nullptr;
    }
    wb_free_.clear();
    wb_pending_.clear();
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

bool PageStore::copy_out(int page, void* host) {
    // kernels already enqueued on the engine's stream may still be writing this page
    if (cudaEventRecord(order_event_, order_stream_) != cudaSuccess) return false;
    if (cudaStreamWaitEvent(copy_stream_, order_event_, 0) != cudaSuccess) return false;
    if (cudaMemcpy2DAsync(host, page_bytes_, pool_ + (size_t)page * page_bytes_, layer_stride_, page_bytes_,
                          (size_t)num_layers_, cudaMemcpyDeviceToHost, copy_stream_) != cudaSuccess)
        return false;
    return cudaStreamSynchronize(copy_stream_) == cudaSuccess;
}

bool PageStore::copy_in(const void* host, int page) {
    if (cudaEventRecord(order_event_, order_stream_) != cudaSuccess) return false;
    if (cudaStreamWaitEvent(copy_stream_, order_event_, 0) != cudaSuccess) return false;
    if (cudaMemcpy2DAsync(pool_ + (size_t)page * page_bytes_, layer_stride_, host, page_bytes_, page_bytes_,
                          (size_t)num_layers_, cudaMemcpyHostToDevice, copy_stream_) != cudaSuccess)
        return false;
    return cudaStreamSynchronize(copy_stream_) == cudaSuccess;
}

bool PageStore::write_file(const std::string& path, const void* src) {
    const size_t total = file_bytes();
    int fd = open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return false;
    bool ok = true;
    if (src != nullptr) {
        size_t done = 0;
        while (done < total) {
            ssize_t w = write(fd, static_cast<const char*>(src) + done, total - done);
            if (w <= 0) {
                ok = false;
                break;
            }
            done += (size_t)w;
        }
        posix_fadvise(fd, 0, (off_t)total, POSIX_FADV_DONTNEED);   // kv_swapper.cpp:217-219
    }
    close(fd);
    if (!ok) unlink(path.c_str());
    return ok;
}

bool PageStore::swap_out(int seq, int logical, int page) {
    const std::string path = path_for(seq, logical);
    const int64_t k = key(seq, logical);
    {
        std::unique_lock<std::mutex> lock(mu_);     // neither a stale prefetched copy nor an older deferred write of
        cv_.wait(lock, [&] { return pending_.count(k) == 0 && wb_pending_.count(k) == 0; });   // this page may outlive the rewrite
        cache_.erase(k);
    }
    if (pool_ != nullptr && write_behind_) {
        int buf = -1;
        {
            std::unique_lock<std::mutex> lock(mu_);
            if (wb_free_.empty() && wb_bufs_[kWriteBehindBuffers - 1] == nullptr) {
                for (int i = 0; i < kWriteBehindBuffers; i++) {
                    if (cudaHostAlloc(&wb_bufs_[i], file_bytes(), cudaHostAllocDefault) != cudaSuccess) return false;
                    wb_free_.push_back(i);
                }
            }
            cv_.wait(lock, [&] { return !wb_free_.empty(); });     // every buffer waits for its file: back-pressure
            buf = wb_free_.back();
            wb_free_.pop_back();
        }
        if (!copy_out(page, wb_bufs_[buf])) {
            std::lock_guard<std::mutex> lock(mu_);
            wb_free_.push_back(buf);
            return false;
        }
        {
            std::lock_guard<std::mutex> lock(mu_);
            wb_pending_[k] = buf;
            queue_.push_back(Job{k, buf});
            writes_deferred++;
        }
        cv_.notify_all();
        bytes_out += (int64_t)file_bytes();
        return true;                                 // the pool page is free; the file follows
    }
    if (pool_ != nullptr && !copy_out(page, staging_)) return false;
    if (!write_file(path, pool_ != nullptr ? staging_ : nullptr)) return false;
    bytes_out += (int64_t)file_bytes();
    return true;
}

bool PageStore::page_to_file(int page, const std::string& path) {
    if (pool_ == nullptr) return write_file(path, nullptr);
    return copy_out(page, staging_) && write_file(path, staging_);
}

bool PageStore::file_to_page(const std::string& path, int page) {
    if (pool_ == nullptr) {
        struct stat st;
        return stat(path.c_str(), &st) == 0;
    }
    return read_file(path, staging_) && copy_in(staging_, page);
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
        // a prefetch of this page in flight finishes first, and so does its deferred write
        cv_.wait(lock, [&] { return pending_.count(k) == 0 && wb_pending_.count(k) == 0; });
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
    if (!copy_in(staging_, page)) return false;
    unlink(path.c_str());                            // the pool holds the only copy again (the reference leaves the file)
    bytes_in += (int64_t)file_bytes();
    return true;
}

void PageStore::drop(int seq, int logical) {
    {
        std::unique_lock<std::mutex> lock(mu_);
        const int64_t k = key(seq, logical);
        cv_.wait(lock, [&] { return pending_.count(k) == 0 && wb_pending_.count(k) == 0; });
        cache_.erase(k);
    }
    unlink(path_for(seq, logical).c_str());
}

bool PageStore::prefetch(int seq, int logical) {
    if (pool_ == nullptr) return true;
    const int64_t k = key(seq, logical);
    {
        std::lock_guard<std::mutex> lock(mu_);
        struct stat st;
        // a deferred write still queued counts as stored: the read is queued behind it
        if (wb_pending_.count(k) == 0 && stat(path_for(seq, logical).c_str(), &st) != 0) return false;
        if (cache_.count(k) || pending_.count(k)) return true;
        pending_.insert(k);
        queue_.push_back(Job{k, -1});
    }
    cv_.notify_all();
    return true;
}

bool PageStore::is_prefetched(int seq, int logical) {
    std::lock_guard<std::mutex> lock(mu_);
    return cache_.count(key(seq, logical)) != 0;
}

void PageStore::drop_prefetch(int seq, int logical) {
    std::unique_lock<std::mutex> lock(mu_);
    const int64_t k = key(seq, logical);
    cv_.wait(lock, [&] { return pending_.count(k) == 0; });
    cache_.erase(k);
}

void PageStore::drain() {
    std::unique_lock<std::mutex> lock(mu_);
    cv_.wait(lock, [&] { return pending_.empty() && wb_pending_.empty(); });
}

void PageStore::worker_loop() {
    for (;;) {
        Job job;
        {
            std::unique_lock<std::mutex> lock(mu_);
            cv_.wait(lock, [&] { return !running_ || !queue_.empty(); });
            if (!running_) return;
            job = queue_.front();
            queue_.pop_front();
        }
        const std::string path = path_for((int)(job.key >> 32), (int)(uint32_t)job.key);
        if (job.wb_buf >= 0) {                       // deferred write of a swapped-out page
            const bool ok = write_file(path, wb_bufs_[job.wb_buf]);
            {
                std::lock_guard<std::mutex> lock(mu_);
                if (!ok) write_failures++;
                wb_pending_.erase(job.key);
                wb_free_.push_back(job.wb_buf);
            }
            cv_.notify_all();
            continue;
        }
        std::vector<char> buf(file_bytes());
        const bool ok = read_file(path, buf.data());
        {
            std::lock_guard<std::mutex> lock(mu_);
            if (ok) cache_[job.key] = std::move(buf);
            pending_.erase(job.key);
        }
        cv_.notify_all();
    }
}

}  // namespace drkv
