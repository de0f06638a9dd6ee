// Host-RAM <-> NVMe tier for expert weights that fit neither in HBM nor in the pinned host arena.
// One file per (layer, expert) under `<drive>/L<layer>/E<expert>.bin`, the drive chosen as
// expert % n_drives so consecutive experts spread over all drives.  Writes go to a temporary
// name and are renamed after fsync (a crash never leaves a half-written expert).  Reads run on a
// small worker pool bounded by `queue_depth` outstanding requests and are reported through
// poll(); O_DIRECT is used when asked for and the buffer / size are 4096-aligned, otherwise the
// page cache path.  Capacity accounting refuses writes beyond the configured budget.
// Reference component: NvmeTier (src/core/memory/nvme_tier.h:24-76: per-expert files, mmap reads,
// io_uring writes, expert_idx % num_drives); io_uring is not available in this image, the worker
// pool gives the same asynchronous contract.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include "lsb_runtime.h"

namespace lsb {

struct NvmeReq { uint64_t token; int layer, expert; void* dst; int64_t bytes; };
struct NvmeDone { uint64_t token; int status; };

class NvmeTier {
public:
    NvmeTier(const std::vector<std::string>& drives, int64_t capacity_bytes, int queue_depth, bool direct_io, int workers)
        : drives_(drives), capacity_(capacity_bytes), depth_(queue_depth > 0 ? queue_depth : 64), direct_(direct_io) {
        for (int i = 0; i < (workers > 0 ? workers : 4); ++i) threads_.emplace_back([this] { run(); });
    }
    ~NvmeTier() {
        { std::lock_guard<std::mutex> g(mu_); stop_ = true; }
        cv_.notify_all();
        for (auto& t : threads_) t.join();
    }
    std::string path(int layer, int expert) const {
        const std::string& d = drives_[(size_t)expert % drives_.size()];
        return d + "/L" + std::to_string(layer) + "/E" + std::to_string(expert) + ".bin";
    }
    int write(int layer, int expert, const void* src, int64_t bytes) {
        const std::string p = path(layer, expert);
        struct stat st;
        const int64_t old = ::stat(p.c_str(), &st) == 0 ? (int64_t)st.st_size : 0;
        if (capacity_ > 0 && used_.load() - old + bytes > capacity_) return LSB_ERR_FULL;
        const std::string dir = p.substr(0, p.rfind('/'));
        ::mkdir(dir.c_str(), 0755);
        const std::string tmp = p + ".tmp";
        const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
        if (fd < 0) return LSB_ERR_IO;
        int64_t off = 0;
        while (off < bytes) {
            const ssize_t n = ::pwrite(fd, (const char*)src + off, (size_t)(bytes - off), off);
            if (n <= 0) { ::close(fd); ::unlink(tmp.c_str()); return LSB_ERR_IO; }
            off += n;
        }
        const bool ok = ::fsync(fd) == 0;
        ::close(fd);
        if (!ok || ::rename(tmp.c_str(), p.c_str()) != 0) { ::unlink(tmp.c_str()); return LSB_ERR_IO; }
        used_ += bytes - old;
        return 0;
    }
    int64_t size_of(int layer, int expert) const {
        struct stat st;
        return ::stat(path(layer, expert).c_str(), &st) == 0 ? (int64_t)st.st_size : -1;
    }
    int read_sync(int layer, int expert, void* dst, int64_t bytes) const {
        const std::string p = path(layer, expert);
        int flags = O_RDONLY;
        const bool aligned = (((uintptr_t)dst | (uintptr_t)bytes) & 4095) == 0;
        if (direct_ && aligned) flags |= O_DIRECT;
        int fd = ::open(p.c_str(), flags);
        if (fd < 0 && (flags & O_DIRECT)) fd = ::open(p.c_str(), O_RDONLY);     // file system without O_DIRECT
        if (fd < 0) return LSB_ERR_NOT_FOUND;
        int64_t off = 0;
        while (off < bytes) {
            const ssize_t n = ::pread(fd, (char*)dst + off, (size_t)(bytes - off), off);
            if (n < 0) { ::close(fd); return LSB_ERR_IO; }
            if (n == 0) break;
            off += n;
        }
        ::close(fd);
        return off == bytes ? 0 : LSB_ERR_FORMAT;
    }
    // Asynchronous read; 0 when the queue is at its depth limit.
    uint64_t read_async(int layer, int expert, void* dst, int64_t bytes) {
        std::lock_guard<std::mutex> g(mu_);
        if ((int)(queue_.size() + running_) >= depth_) return 0;
        const uint64_t tok = ++next_;
        queue_.push_back(NvmeReq{tok, layer, expert, dst, bytes});
        cv_.notify_one();
        return tok;
    }
    int poll(uint64_t* tokens, int* status, int cap) {
        std::lock_guard<std::mutex> g(mu_);
        int n = 0;
        while (n < cap && !done_.empty()) { tokens[n] = done_.front().token; status[n] = done_.front().status; done_.pop_front(); ++n; }
        return n;
    }
    int evict(int layer, int expert) {
        const int64_t sz = size_of(layer, expert);
        if (sz < 0) return LSB_ERR_NOT_FOUND;
        if (::unlink(path(layer, expert).c_str()) != 0) return LSB_ERR_IO;
        used_ -= sz;
        return 0;
    }
    int64_t used() const { return used_.load(); }
    int pending() { std::lock_guard<std::mutex> g(mu_); return (int)queue_.size() + running_; }

private:
    void run() {
        for (;;) {
            NvmeReq r;
            {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [this] { return stop_ || !queue_.empty(); });
                if (stop_ && queue_.empty()) return;
                r = queue_.front();
                queue_.pop_front();
                ++running_;
            }
            const int st = read_sync(r.layer, r.expert, r.dst, r.bytes);
            std::lock_guard<std::mutex> g(mu_);
            --running_;
            done_.push_back(NvmeDone{r.token, st});
        }
    }
    std::vector<std::string> drives_;
    int64_t capacity_;
    int depth_;
    bool direct_;
    std::atomic<int64_t> used_{0};
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<NvmeReq> queue_;
    std::deque<NvmeDone> done_;
    std::vector<std::thread> threads_;
    int running_ = 0;
    uint64_t next_ = 0;
    bool stop_ = false;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
// `drives`: directory paths separated by '\n'.
LSB_RT_API void* lsb_nvme_create(const char* drives, long long capacity_bytes, int queue_depth, int direct_io, int workers) {
    std::vector<std::string> d;
    std::string cur;
    for (const char* p = drives; p && *p; ++p) { if (*p == '\n') { if (!cur.empty()) d.push_back(cur); cur.clear(); } else cur.push_back(*p); }
    if (!cur.empty()) d.push_back(cur);
    if (d.empty()) return nullptr;
    return new NvmeTier(d, capacity_bytes, queue_depth, direct_io != 0, workers);
}
LSB_RT_API void lsb_nvme_destroy(void* h) { delete (NvmeTier*)h; }
LSB_RT_API int lsb_nvme_write(void* h, int layer, int expert, const void* src, long long bytes) { return ((NvmeTier*)h)->write(layer, expert, src, bytes); }
LSB_RT_API int lsb_nvme_read(void* h, int layer, int expert, void* dst, long long bytes) { return ((NvmeTier*)h)->read_sync(layer, expert, dst, bytes); }
LSB_RT_API unsigned long long lsb_nvme_read_async(void* h, int layer, int expert, void* dst, long long bytes) { return ((NvmeTier*)h)->read_async(layer, expert, dst, bytes); }
LSB_RT_API int lsb_nvme_poll(void* h, unsigned long long* tokens, int* status, int cap) { return ((NvmeTier*)h)->poll((uint64_t*)tokens, status, cap); }
LSB_RT_API long long lsb_nvme_size_of(void* h, int layer, int expert) { return ((NvmeTier*)h)->size_of(layer, expert); }
LSB_RT_API int lsb_nvme_evict(void* h, int layer, int expert) { return ((NvmeTier*)h)->evict(layer, expert); }
LSB_RT_API long long lsb_nvme_used(void* h) { return ((NvmeTier*)h)->used(); }
LSB_RT_API int lsb_nvme_pending(void* h) { return ((NvmeTier*)h)->pending(); }
}
