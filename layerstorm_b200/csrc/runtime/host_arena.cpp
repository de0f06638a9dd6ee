// Host-side expert storage: NUMA queries and placement, per-node budget resolution, and the
// slotted expert arena that backs the VRAM expert cache.
//
//   NumaTopology     nodes, per-node total/free memory and CPU list from sysfs; CPU-less nodes are
//                    reported as such (memory-only nodes must not receive worker threads)
//   resolve_budget   fraction_free | fraction_total | absolute_gb -> bytes for one node
//   HostArena        one slab (anonymous mmap or memfd so another process can attach), optionally
//                    bound to a NUMA node with mbind and advised for huge pages; fixed-size slots
//                    keyed by (layer, expert); LRU replacement among unreferenced slots; in-flight
//                    reference counts (a slot being read by a device copy cannot be evicted);
//                    slot states kEmpty -> kLoading -> kActive so a crash mid-load never exposes a
//                    half-written expert; optional persistence of the slot table to a meta file
//                    (written to a temporary name and renamed)
// The owner registers the slab with the CUDA driver (cudaHostRegister) - this file stays CUDA-free.
// Reference components: NumaManager / host_pool_sizing (src/core/memory/numa_manager.h:16-235),
// PinnedExpertArena + ArenaCache (src/core/memory/pinned_expert_arena.*).
#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include "lsb_runtime.h"

namespace lsb {

struct NumaNode { int id; int64_t total_bytes, free_bytes; int n_cpus; };

static int count_cpulist(const std::string& s) {
    int n = 0;
    std::stringstream ss(s);
    std::string part;
    while (std::getline(ss, part, ',')) {
        if (part.empty() || part == "\n") continue;
        int a = 0, b = 0;
        if (std::sscanf(part.c_str(), "%d-%d", &a, &b) == 2) n += b - a + 1;
        else if (std::sscanf(part.c_str(), "%d", &a) == 1) n += 1;
    }
    return n;
}

static std::vector<NumaNode> read_topology(const char* sysfs_root) {
    std::vector<NumaNode> out;
    const std::string root = sysfs_root && *sysfs_root ? sysfs_root : "/sys/devices/system/node";
    for (int id = 0; id < 1024; ++id) {
        std::ifstream mi(root + "/node" + std::to_string(id) + "/meminfo");
        if (!mi) { if (id > 64) break; else continue; }
        NumaNode n{id, 0, 0, 0};
        std::string line;
        while (std::getline(mi, line)) {
            long long kb = 0;
            const auto p = line.find("MemTotal:"), q = line.find("MemFree:");
            if (p != std::string::npos && std::sscanf(line.c_str() + p + 9, "%lld", &kb) == 1) n.total_bytes = kb * 1024;
            if (q != std::string::npos && std::sscanf(line.c_str() + q + 8, "%lld", &kb) == 1) n.free_bytes = kb * 1024;
        }
        std::ifstream cl(root + "/node" + std::to_string(id) + "/cpulist");
        std::string cpus;
        if (cl && std::getline(cl, cpus)) n.n_cpus = count_cpulist(cpus);
        out.push_back(n);
    }
    return out;
}

enum { kSizingFractionFree = 0, kSizingFractionTotal = 1, kSizingAbsoluteGb = 2 };

static int64_t resolve_budget(int mode, double value, int64_t total, int64_t free_b, int64_t reserve) {
    double b = 0;
    if (mode == kSizingFractionFree) b = value * (double)free_b;
    else if (mode == kSizingFractionTotal) b = value * (double)total;
    else b = value * (double)(1ull << 30);
    int64_t r = (int64_t)b;
    r = std::min<int64_t>(r, free_b - reserve);      // never promise more than the node can give right now
    return std::max<int64_t>(r, 0);
}

enum SlotState { kEmpty = 0, kLoading = 1, kActive = 2 };

struct ArenaSlot { int state = kEmpty; int layer = -1, expert = -1; int refs = 0; uint64_t last_use = 0; };

class HostArena {
public:
    HostArena(int64_t slot_bytes, int n_slots, int numa_node, bool use_memfd, bool thp)
        : slot_bytes_(slot_bytes), n_(n_slots), slots_(n_slots) {
        bytes_ = (size_t)slot_bytes * (size_t)n_slots;
        if (use_memfd) {
            fd_ = (int)syscall(SYS_memfd_create, "lsb-expert-arena", 0u);
            if (fd_ >= 0 && ftruncate(fd_, (off_t)bytes_) != 0) { close(fd_); fd_ = -1; }
        }
        base_ = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, fd_ >= 0 ? MAP_SHARED : (MAP_PRIVATE | MAP_ANONYMOUS), fd_, 0);
        if (base_ == MAP_FAILED) { base_ = nullptr; return; }
        if (thp) madvise(base_, bytes_, MADV_HUGEPAGE);
        if (numa_node >= 0 && numa_node < 1024) {
            unsigned long mask[16] = {0};
            mask[numa_node / (8 * sizeof(unsigned long))] |= 1ul << (numa_node % (8 * sizeof(unsigned long)));
            // MPOL_BIND = 2; failure (no NUMA support, container restrictions) is not fatal: placement is a hint
            bound_ = syscall(SYS_mbind, base_, bytes_, 2, mask, sizeof(mask) * 8, 0u) == 0;
        }
    }
    // Attach to a slab that already exists (an fd kept alive by the arena holder process): contents and, with load_meta,
    // the slot table survive an engine restart.
    HostArena(int64_t slot_bytes, int n_slots, int existing_fd)
        : slot_bytes_(slot_bytes), n_(n_slots), slots_(n_slots) {
        bytes_ = (size_t)slot_bytes * (size_t)n_slots;
        struct stat st;
        if (existing_fd < 0 || fstat(existing_fd, &st) != 0 || (size_t)st.st_size < bytes_) return;
        fd_ = dup(existing_fd);
        base_ = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0);
        if (base_ == MAP_FAILED) base_ = nullptr;
    }
    ~HostArena() {
        if (base_) munmap(base_, bytes_);
        if (fd_ >= 0) close(fd_);
    }
    bool ok() const { return base_ != nullptr; }
    void* base() const { return base_; }
    size_t bytes() const { return bytes_; }
    int fd() const { return fd_; }
    bool bound() const { return bound_; }
    int n_slots() const { return n_; }
    int64_t slot_bytes() const { return slot_bytes_; }

    int lookup(int layer, int expert) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = index_.find({layer, expert});
        if (it == index_.end() || slots_[it->second].state != kActive) return -1;
        slots_[it->second].last_use = ++clock_;
        ++hits_;
        return it->second;
    }
    // Slot to load (layer, expert) into: the existing one, a free one, or the least recently used
    // unreferenced active slot (its previous owner is returned through ev_*).  The slot enters kLoading.
    int begin_load(int layer, int expert, int* ev_layer, int* ev_expert) {
        std::lock_guard<std::mutex> g(mu_);
        *ev_layer = *ev_expert = -1;
        auto it = index_.find({layer, expert});
        if (it != index_.end()) return slots_[it->second].state == kLoading ? LSB_ERR_BUSY : it->second;
        int pick = -1;
        for (int i = 0; i < n_; ++i) if (slots_[i].state == kEmpty) { pick = i; break; }
        if (pick < 0) {
            uint64_t best = UINT64_MAX;
            for (int i = 0; i < n_; ++i)
                if (slots_[i].state == kActive && slots_[i].refs == 0 && slots_[i].last_use < best) { best = slots_[i].last_use; pick = i; }
            if (pick < 0) return LSB_ERR_FULL;
            *ev_layer = slots_[pick].layer; *ev_expert = slots_[pick].expert;
            index_.erase({slots_[pick].layer, slots_[pick].expert});
            ++evictions_;
        }
        slots_[pick] = ArenaSlot{kLoading, layer, expert, 0, ++clock_};
        index_[{layer, expert}] = pick;
        ++misses_;
        return pick;
    }
    int finish_load(int slot, bool success) {
        std::lock_guard<std::mutex> g(mu_);
        if (slot < 0 || slot >= n_ || slots_[slot].state != kLoading) return LSB_ERR_ARG;
        if (success) slots_[slot].state = kActive;
        else { index_.erase({slots_[slot].layer, slots_[slot].expert}); slots_[slot] = ArenaSlot{}; }
        return 0;
    }
    int ref(int slot, int delta) {
        std::lock_guard<std::mutex> g(mu_);
        if (slot < 0 || slot >= n_ || slots_[slot].state != kActive) return LSB_ERR_ARG;
        slots_[slot].refs = std::max(0, slots_[slot].refs + delta);
        return slots_[slot].refs;
    }
    int wipe() {
        std::lock_guard<std::mutex> g(mu_);
        for (auto& s : slots_) if (s.refs > 0) return LSB_ERR_BUSY;
        for (auto& s : slots_) s = ArenaSlot{};
        index_.clear();
        return 0;
    }
    void stats(uint64_t* hits, uint64_t* misses, uint64_t* evictions, int* active) {
        std::lock_guard<std::mutex> g(mu_);
        *hits = hits_; *misses = misses_; *evictions = evictions_;
        int a = 0;
        for (auto& s : slots_) a += s.state == kActive;
        *active = a;
    }
    int slot_info(int slot, int* state, int* layer, int* expert, int* refs) {
        std::lock_guard<std::mutex> g(mu_);
        if (slot < 0 || slot >= n_) return LSB_ERR_ARG;
        *state = slots_[slot].state; *layer = slots_[slot].layer; *expert = slots_[slot].expert; *refs = slots_[slot].refs;
        return 0;
    }
    // Persist / restore the table of ACTIVE slots (loading slots are dropped: their bytes are not trustworthy).
    int save_meta(const char* path, uint64_t content_tag) {
        std::lock_guard<std::mutex> g(mu_);
        const std::string tmp = std::string(path) + ".tmp";
        FILE* f = std::fopen(tmp.c_str(), "w");
        if (!f) return LSB_ERR_IO;
        std::fprintf(f, "lsb-arena-meta 1 %lld %d %llu\n", (long long)slot_bytes_, n_, (unsigned long long)content_tag);
        for (int i = 0; i < n_; ++i)
            if (slots_[i].state == kActive) std::fprintf(f, "%d %d %d\n", i, slots_[i].layer, slots_[i].expert);
        const bool ok = std::fflush(f) == 0 && fsync(fileno(f)) == 0;
        std::fclose(f);
        if (!ok || std::rename(tmp.c_str(), path) != 0) return LSB_ERR_IO;
        return 0;
    }
    int load_meta(const char* path, uint64_t content_tag) {
        std::lock_guard<std::mutex> g(mu_);
        FILE* f = std::fopen(path, "r");
        if (!f) return LSB_ERR_NOT_FOUND;
        long long sb = 0; int n = 0, ver = 0; unsigned long long tag = 0;
        if (std::fscanf(f, "lsb-arena-meta %d %lld %d %llu\n", &ver, &sb, &n, &tag) != 4 || ver != 1 || sb != slot_bytes_ || n != n_ || tag != content_tag) {
            std::fclose(f);
            return LSB_ERR_FORMAT;                     // different geometry or different model: start empty
        }
        for (auto& s : slots_) s = ArenaSlot{};
        index_.clear();
        int i, l, e, restored = 0;
        while (std::fscanf(f, "%d %d %d\n", &i, &l, &e) == 3)
            if (i >= 0 && i < n_) { slots_[i] = ArenaSlot{kActive, l, e, 0, ++clock_}; index_[{l, e}] = i; ++restored; }
        std::fclose(f);
        return restored;
    }

private:
    int64_t slot_bytes_; int n_;
    size_t bytes_ = 0;
    void* base_ = nullptr;
    int fd_ = -1;
    bool bound_ = false;
    std::mutex mu_;
    std::vector<ArenaSlot> slots_;
    std::map<std::pair<int, int>, int> index_;
    uint64_t clock_ = 0, hits_ = 0, misses_ = 0, evictions_ = 0;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
// out arrays hold up to `cap` nodes; returns the node count.
LSB_RT_API int lsb_numa_topology(const char* sysfs_root, int cap, int* ids, long long* total, long long* free_b, int* n_cpus) {
    const auto nodes = read_topology(sysfs_root);
    const int n = std::min<int>(cap, (int)nodes.size());
    for (int i = 0; i < n; ++i) { ids[i] = nodes[i].id; total[i] = nodes[i].total_bytes; free_b[i] = nodes[i].free_bytes; n_cpus[i] = nodes[i].n_cpus; }
    return (int)nodes.size();
}
LSB_RT_API long long lsb_host_pool_budget(int mode, double value, long long total, long long free_b, long long reserve) {
    return resolve_budget(mode, value, total, free_b, reserve);
}
LSB_RT_API void* lsb_arena_create(long long slot_bytes, int n_slots, int numa_node, int use_memfd, int thp) {
    if (slot_bytes <= 0 || n_slots <= 0) return nullptr;
    auto* a = new HostArena(slot_bytes, n_slots, numa_node, use_memfd != 0, thp != 0);
    if (!a->ok()) { delete a; return nullptr; }
    return a;
}
LSB_RT_API void* lsb_arena_attach(long long slot_bytes, int n_slots, int fd) {
    if (slot_bytes <= 0 || n_slots <= 0) return nullptr;
    auto* a = new HostArena(slot_bytes, n_slots, fd);
    if (!a->ok()) { delete a; return nullptr; }
    return a;
}
LSB_RT_API void lsb_arena_destroy(void* h) { delete (HostArena*)h; }
LSB_RT_API void* lsb_arena_base(void* h) { return ((HostArena*)h)->base(); }
LSB_RT_API unsigned long long lsb_arena_bytes(void* h) { return ((HostArena*)h)->bytes(); }
LSB_RT_API int lsb_arena_fd(void* h) { return ((HostArena*)h)->fd(); }
LSB_RT_API int lsb_arena_numa_bound(void* h) { return ((HostArena*)h)->bound() ? 1 : 0; }
LSB_RT_API int lsb_arena_lookup(void* h, int layer, int expert) { return ((HostArena*)h)->lookup(layer, expert); }
LSB_RT_API int lsb_arena_begin_load(void* h, int layer, int expert, int* ev_layer, int* ev_expert) { return ((HostArena*)h)->begin_load(layer, expert, ev_layer, ev_expert); }
LSB_RT_API int lsb_arena_finish_load(void* h, int slot, int success) { return ((HostArena*)h)->finish_load(slot, success != 0); }
LSB_RT_API int lsb_arena_ref(void* h, int slot, int delta) { return ((HostArena*)h)->ref(slot, delta); }
LSB_RT_API int lsb_arena_wipe(void* h) { return ((HostArena*)h)->wipe(); }
LSB_RT_API void lsb_arena_stats(void* h, unsigned long long* hits, unsigned long long* misses, unsigned long long* evictions, int* active) {
    uint64_t a, b, c;
    ((HostArena*)h)->stats(&a, &b, &c, active);
    *hits = a; *misses = b; *evictions = c;
}
LSB_RT_API int lsb_arena_slot_info(void* h, int slot, int* state, int* layer, int* expert, int* refs) { return ((HostArena*)h)->slot_info(slot, state, layer, expert, refs); }
LSB_RT_API int lsb_arena_save_meta(void* h, const char* path, unsigned long long tag) { return ((HostArena*)h)->save_meta(path, tag); }
LSB_RT_API int lsb_arena_load_meta(void* h, const char* path, unsigned long long tag) { return ((HostArena*)h)->load_meta(path, tag); }
}
