// Lock-free plumbing between the serving threads and the engine thread, and the tracing ring:
//   SpscRing       single-producer / single-consumer ring of fixed-size slots (command ring: 256-byte
//                  slots, completion ring: 128-byte slots) with acquire/release indices
//   StateSnapshot  seqlock-published state block: the writer bumps a sequence counter to odd, writes,
//                  bumps to even; readers retry until they see the same even value before and after
//   PerfTrace      preallocated ring of 32-byte records (ns, stage, gpu, cmd_seq, key, token) claimed
//                  with one atomic fetch_add; dumped to CSV; per-stage aggregation
// Reference components: src/daemon/spsc_ring.h:23, src/daemon/state_publisher.*, state_transaction.h,
// src/core/perf_trace.h:26-71 (LS_PERF_TRACE / LS_PERF_TRACE_OUT).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

class SpscRing {
public:
    SpscRing(uint32_t slots, uint32_t slot_bytes) : slots_(slots), slot_bytes_(slot_bytes), buf_((size_t)slots * slot_bytes) {
        // capacity must be a power of two so the indices can wrap freely
        mask_ = slots - 1;
    }
    bool valid() const { return slots_ && (slots_ & (slots_ - 1)) == 0; }
    bool push(const void* data, uint32_t n) {
        if (n > slot_bytes_) return false;
        const uint64_t h = head_.load(std::memory_order_relaxed);
        if (h - tail_.load(std::memory_order_acquire) >= slots_) return false;     // full: back-pressure
        uint8_t* dst = buf_.data() + (size_t)(h & mask_) * slot_bytes_;
        std::memcpy(dst, data, n);
        if (n < slot_bytes_) std::memset(dst + n, 0, slot_bytes_ - n);
        head_.store(h + 1, std::memory_order_release);
        return true;
    }
    bool pop(void* out) {
        const uint64_t t = tail_.load(std::memory_order_relaxed);
        if (t == head_.load(std::memory_order_acquire)) return false;
        std::memcpy(out, buf_.data() + (size_t)(t & mask_) * slot_bytes_, slot_bytes_);
        tail_.store(t + 1, std::memory_order_release);
        return true;
    }
    uint64_t size() const { return head_.load(std::memory_order_acquire) - tail_.load(std::memory_order_acquire); }
    uint32_t slot_bytes() const { return slot_bytes_; }
private:
    uint32_t slots_, slot_bytes_, mask_;
    std::vector<uint8_t> buf_;
    alignas(64) std::atomic<uint64_t> head_{0};
    alignas(64) std::atomic<uint64_t> tail_{0};
};

// The payload of a seqlock is read while it may be written: the reader throws a torn copy away, but the accesses themselves must not be
// data races, so both sides move the shared bytes with relaxed atomic accesses (words when aligned, bytes otherwise).
static inline void copy_to_shared(uint8_t* shared, const uint8_t* src, uint32_t n) {
    uint32_t i = 0;
    if (((uintptr_t)shared & 7) == 0)
        for (; i + 8 <= n; i += 8) { uint64_t v; std::memcpy(&v, src + i, 8); __atomic_store_n((uint64_t*)(shared + i), v, __ATOMIC_RELAXED); }
    for (; i < n; ++i) __atomic_store_n(shared + i, src[i], __ATOMIC_RELAXED);
}
static inline void copy_from_shared(uint8_t* dst, const uint8_t* shared, uint32_t n) {
    uint32_t i = 0;
    if (((uintptr_t)shared & 7) == 0)
        for (; i + 8 <= n; i += 8) { const uint64_t v = __atomic_load_n((const uint64_t*)(shared + i), __ATOMIC_RELAXED); std::memcpy(dst + i, &v, 8); }
    for (; i < n; ++i) dst[i] = __atomic_load_n(shared + i, __ATOMIC_RELAXED);
}

class StateSnapshot {
public:
    explicit StateSnapshot(uint32_t bytes) : data_(bytes) {}
    void begin() { if (depth_++ == 0) seq_.fetch_add(1, std::memory_order_acq_rel); }   // nested transactions publish once
    void write(uint32_t off, const void* src, uint32_t n) { if (off + n <= data_.size()) copy_to_shared(data_.data() + off, (const uint8_t*)src, n); }
    void end() { if (--depth_ == 0) seq_.fetch_add(1, std::memory_order_acq_rel); }
    // Returns the version read, or 0 when no consistent copy was obtained within `tries`.
    uint64_t read(void* out, uint32_t off, uint32_t n, int tries) const {
        for (int i = 0; i < tries; ++i) {
            const uint64_t a = seq_.load(std::memory_order_acquire);
            if (a & 1) continue;
            copy_from_shared((uint8_t*)out, data_.data() + off, n);
            std::atomic_thread_fence(std::memory_order_acquire);
            if (seq_.load(std::memory_order_acquire) == a) return a + 2;   // +2 so that version 0 can mean failure
        }
        return 0;
    }
    uint32_t size() const { return (uint32_t)data_.size(); }
private:
    std::vector<uint8_t> data_;
    std::atomic<uint64_t> seq_{0};
    int depth_ = 0;
};

struct TraceRecord { uint64_t ns; uint16_t stage; uint16_t gpu; uint32_t cmd_seq; uint64_t key; uint64_t token; };
static_assert(sizeof(TraceRecord) == 32, "trace records are 32 bytes");

class PerfTrace {
public:
    explicit PerfTrace(uint64_t capacity) : cap_(capacity), rec_(capacity) {}
    static uint64_t now_ns() { return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
    void record(uint16_t stage, uint16_t gpu, uint32_t cmd_seq, uint64_t key, uint64_t token) {
        const uint64_t i = next_.fetch_add(1, std::memory_order_relaxed);
        if (i >= cap_) { dropped_.fetch_add(1, std::memory_order_relaxed); return; }
        rec_[i] = TraceRecord{now_ns(), stage, gpu, cmd_seq, key, token};
    }
    uint64_t count() const { return std::min<uint64_t>(next_.load(), cap_); }
    uint64_t dropped() const { return dropped_.load(); }
    int dump_csv(const char* path) const {
        FILE* f = std::fopen(path, "w");
        if (!f) return LSB_ERR_IO;
        std::fprintf(f, "ns,stage,gpu,cmd_seq,key,token\n");
        for (uint64_t i = 0; i < count(); ++i)
            std::fprintf(f, "%llu,%u,%u,%u,%llu,%llu\n", (unsigned long long)rec_[i].ns, rec_[i].stage, rec_[i].gpu, rec_[i].cmd_seq,
                         (unsigned long long)rec_[i].key, (unsigned long long)rec_[i].token);
        std::fclose(f);
        return 0;
    }
    // Sum of (end - begin) over matching tokens for a begin/end stage pair, in ns; *n = pairs.
    uint64_t span_ns(uint16_t begin_stage, uint16_t end_stage, uint64_t* n) const {
        std::map<uint64_t, uint64_t> open;
        uint64_t tot = 0, cnt = 0;
        for (uint64_t i = 0; i < count(); ++i) {
            const auto& r = rec_[i];
            if (r.stage == begin_stage) open[r.token] = r.ns;
            else if (r.stage == end_stage) {
                auto it = open.find(r.token);
                if (it != open.end()) { tot += r.ns - it->second; ++cnt; open.erase(it); }
            }
        }
        if (n) *n = cnt;
        return tot;
    }
private:
    uint64_t cap_;
    std::vector<TraceRecord> rec_;
    std::atomic<uint64_t> next_{0}, dropped_{0};
};

}  // namespace lsb

using namespace lsb;
extern "C" {
LSB_RT_API void* lsb_ring_create(unsigned int slots, unsigned int slot_bytes) {
    auto* r = new SpscRing(slots, slot_bytes);
    if (!r->valid()) { delete r; return nullptr; }
    return r;
}
LSB_RT_API void lsb_ring_destroy(void* h) { delete (SpscRing*)h; }
LSB_RT_API int lsb_ring_push(void* h, const void* data, unsigned int n) { return ((SpscRing*)h)->push(data, n) ? 1 : 0; }
LSB_RT_API int lsb_ring_pop(void* h, void* out) { return ((SpscRing*)h)->pop(out) ? 1 : 0; }
LSB_RT_API unsigned long long lsb_ring_size(void* h) { return ((SpscRing*)h)->size(); }

LSB_RT_API void* lsb_snap_create(unsigned int bytes) { return new StateSnapshot(bytes); }
LSB_RT_API void lsb_snap_destroy(void* h) { delete (StateSnapshot*)h; }
LSB_RT_API void lsb_snap_begin(void* h) { ((StateSnapshot*)h)->begin(); }
LSB_RT_API void lsb_snap_write(void* h, unsigned int off, const void* src, unsigned int n) { ((StateSnapshot*)h)->write(off, src, n); }
LSB_RT_API void lsb_snap_end(void* h) { ((StateSnapshot*)h)->end(); }
LSB_RT_API unsigned long long lsb_snap_read(void* h, void* out, unsigned int off, unsigned int n, int tries) { return ((StateSnapshot*)h)->read(out, off, n, tries); }

LSB_RT_API void* lsb_trace_create(unsigned long long capacity) { return new PerfTrace(capacity); }
LSB_RT_API void lsb_trace_destroy(void* h) { delete (PerfTrace*)h; }
LSB_RT_API void lsb_trace_record(void* h, int stage, int gpu, unsigned int cmd_seq, unsigned long long key, unsigned long long token) {
    ((PerfTrace*)h)->record((uint16_t)stage, (uint16_t)gpu, cmd_seq, key, token);
}
LSB_RT_API unsigned long long lsb_trace_count(void* h) { return ((PerfTrace*)h)->count(); }
LSB_RT_API unsigned long long lsb_trace_dropped(void* h) { return ((PerfTrace*)h)->dropped(); }
LSB_RT_API int lsb_trace_dump_csv(void* h, const char* path) { return ((PerfTrace*)h)->dump_csv(path); }
LSB_RT_API unsigned long long lsb_trace_span_ns(void* h, int begin_stage, int end_stage, unsigned long long* n) {
    uint64_t c = 0;
    const uint64_t t = ((PerfTrace*)h)->span_ns((uint16_t)begin_stage, (uint16_t)end_stage, &c);
    if (n) *n = c;
    return t;
}
}
