// Bookkeeping core of the asynchronous host<->device transfer engine (expert streaming, KV
// tiering).  CUDA-free: the owner issues the actual pinned cudaMemcpyAsync on a side stream and
// reports completion (an event fired); this class decides WHAT is issued WHEN:
//   * requests are de-duplicated by key {layer, expert, gpu, direction}: a second request for a
//     transfer that is queued or in flight returns the first one's token (priority is raised)
//   * tokens increase monotonically and never repeat
//   * per-GPU staged queues by priority (0 = needed by the running layer ... levels-1 = speculative
//     prefetch), FIFO inside a level, at most `waterline` transfers in flight per GPU
//   * cancel: a queued transfer is dropped at once, one in flight is marked and reported as
//     cancelled when it completes (its destination slot must not be reused earlier)
//   * completions are handed out in completion order by poll_completions
//   * EWMA bandwidth estimate per (gpu, direction) from bytes / measured duration
// Reference component: TransferEngine (src/core/transfer/transfer_engine.h: dedup key, token,
// priority-staged queue + in-flight waterline, deferred cancel, poll_completions, BW estimate).
#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

enum TransferState { kQueued = 0, kInFlight = 1, kDone = 2, kCancelled = 3 };

struct Transfer {
    uint64_t token;
    int layer, expert, gpu, dir, priority;
    int64_t bytes;
    int state;
    bool cancel_requested;
    uint64_t issue_ns;
};

class TransferEngine {
public:
    TransferEngine(int n_gpus, int levels, int waterline) : n_gpus_(n_gpus), levels_(std::max(1, levels)), waterline_(std::max(1, waterline)),
        queues_((size_t)n_gpus * levels_), inflight_(n_gpus, 0), bw_((size_t)n_gpus * 2, 0.0) {}

    uint64_t submit(int layer, int expert, int gpu, int dir, int priority, int64_t bytes) {
        std::lock_guard<std::mutex> g(mu_);
        if (gpu < 0 || gpu >= n_gpus_ || dir < 0 || dir > 1) return 0;
        priority = std::clamp(priority, 0, levels_ - 1);
        const Key k{layer, expert, gpu, dir};
        auto it = by_key_.find(k);
        if (it != by_key_.end()) {
            Transfer& t = live_.at(it->second);
            t.cancel_requested = false;                      // a new request revives a transfer that was being cancelled
            if (t.state == kQueued && priority < t.priority) {   // raise: move between level queues
                auto& q = queue(gpu, t.priority);
                q.erase(std::find(q.begin(), q.end(), t.token));
                t.priority = priority;
                queue(gpu, priority).push_back(t.token);
            }
            ++dedup_hits_;
            return t.token;
        }
        Transfer t{++next_token_, layer, expert, gpu, dir, priority, bytes, kQueued, false, 0};
        live_.emplace(t.token, t);
        by_key_.emplace(k, t.token);
        queue(gpu, priority).push_back(t.token);
        return t.token;
    }

    // Next transfer the owner should issue on `gpu`, or 0 when the waterline is reached / nothing is queued.
    uint64_t next_to_issue(int gpu, uint64_t now_ns) {
        std::lock_guard<std::mutex> g(mu_);
        if (gpu < 0 || gpu >= n_gpus_ || inflight_[gpu] >= waterline_) return 0;
        for (int p = 0; p < levels_; ++p) {
            auto& q = queue(gpu, p);
            if (q.empty()) continue;
            const uint64_t tok = q.front();
            q.pop_front();
            Transfer& t = live_.at(tok);
            t.state = kInFlight;
            t.issue_ns = now_ns;
            ++inflight_[gpu];
            return tok;
        }
        return 0;
    }

    int info(uint64_t tok, int* layer, int* expert, int* gpu, int* dir, int* priority, int64_t* bytes, int* state) const {
        std::lock_guard<std::mutex> g(mu_);
        auto it = live_.find(tok);
        if (it == live_.end()) return LSB_ERR_NOT_FOUND;
        const Transfer& t = it->second;
        *layer = t.layer; *expert = t.expert; *gpu = t.gpu; *dir = t.dir; *priority = t.priority; *bytes = t.bytes; *state = t.state;
        return 0;
    }

    // The copy behind `tok` has finished on the device.
    int complete(uint64_t tok, uint64_t now_ns) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = live_.find(tok);
        if (it == live_.end() || it->second.state != kInFlight) return LSB_ERR_NOT_FOUND;
        Transfer& t = it->second;
        --inflight_[t.gpu];
        if (now_ns > t.issue_ns && t.bytes > 0) {
            const double gbs = (double)t.bytes / (double)(now_ns - t.issue_ns);   // bytes per ns = GB/s
            double& e = bw_[(size_t)t.gpu * 2 + t.dir];
            e = e == 0.0 ? gbs : 0.8 * e + 0.2 * gbs;
        }
        t.state = t.cancel_requested ? kCancelled : kDone;
        finished_.push_back(t);
        by_key_.erase(Key{t.layer, t.expert, t.gpu, t.dir});
        live_.erase(it);
        return 0;
    }

    // 1 = dropped now, 2 = in flight (will be reported cancelled on completion), error otherwise.
    int cancel(uint64_t tok) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = live_.find(tok);
        if (it == live_.end()) return LSB_ERR_NOT_FOUND;
        Transfer& t = it->second;
        if (t.state == kQueued) {
            auto& q = queue(t.gpu, t.priority);
            q.erase(std::find(q.begin(), q.end(), tok));
            t.state = kCancelled;
            finished_.push_back(t);
            by_key_.erase(Key{t.layer, t.expert, t.gpu, t.dir});
            live_.erase(it);
            return 1;
        }
        t.cancel_requested = true;
        return 2;
    }

    // Up to `cap` finished transfers in completion order: tokens[i], states[i] (kDone / kCancelled).
    int poll_completions(uint64_t* tokens, int* states, int* layers, int* experts, int* gpus, int cap) {
        std::lock_guard<std::mutex> g(mu_);
        int n = 0;
        while (n < cap && !finished_.empty()) {
            const Transfer& t = finished_.front();
            tokens[n] = t.token; states[n] = t.state; layers[n] = t.layer; experts[n] = t.expert; gpus[n] = t.gpu;
            finished_.pop_front();
            ++n;
        }
        return n;
    }

    int queued(int gpu) const { std::lock_guard<std::mutex> g(mu_); int n = 0; for (int p = 0; p < levels_; ++p) n += (int)queues_[(size_t)gpu * levels_ + p].size(); return n; }
    int in_flight(int gpu) const { std::lock_guard<std::mutex> g(mu_); return inflight_[gpu]; }
    double bandwidth_gbs(int gpu, int dir) const { std::lock_guard<std::mutex> g(mu_); return bw_[(size_t)gpu * 2 + dir]; }
    uint64_t dedup_hits() const { std::lock_guard<std::mutex> g(mu_); return dedup_hits_; }
    uint64_t find(int layer, int expert, int gpu, int dir) const {
        std::lock_guard<std::mutex> g(mu_);
        auto it = by_key_.find(Key{layer, expert, gpu, dir});
        return it == by_key_.end() ? 0 : it->second;
    }

private:
    using Key = std::tuple<int, int, int, int>;
    std::deque<uint64_t>& queue(int gpu, int p) { return queues_[(size_t)gpu * levels_ + p]; }
    int n_gpus_, levels_, waterline_;
    mutable std::mutex mu_;
    uint64_t next_token_ = 0, dedup_hits_ = 0;
    std::unordered_map<uint64_t, Transfer> live_;
    std::map<Key, uint64_t> by_key_;
    std::vector<std::deque<uint64_t>> queues_;
    std::vector<int> inflight_;
    std::vector<double> bw_;
    std::deque<Transfer> finished_;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
LSB_RT_API void* lsb_te_create(int n_gpus, int levels, int waterline) { return n_gpus > 0 ? new TransferEngine(n_gpus, levels, waterline) : nullptr; }
LSB_RT_API void lsb_te_destroy(void* h) { delete (TransferEngine*)h; }
LSB_RT_API unsigned long long lsb_te_submit(void* h, int layer, int expert, int gpu, int dir, int priority, long long bytes) {
    return ((TransferEngine*)h)->submit(layer, expert, gpu, dir, priority, bytes);
}
LSB_RT_API unsigned long long lsb_te_next(void* h, int gpu, unsigned long long now_ns) { return ((TransferEngine*)h)->next_to_issue(gpu, now_ns); }
LSB_RT_API int lsb_te_info(void* h, unsigned long long tok, int* layer, int* expert, int* gpu, int* dir, int* priority, long long* bytes, int* state) {
    int64_t b = 0;
    const int rc = ((TransferEngine*)h)->info(tok, layer, expert, gpu, dir, priority, &b, state);
    *bytes = b;
    return rc;
}
LSB_RT_API int lsb_te_complete(void* h, unsigned long long tok, unsigned long long now_ns) { return ((TransferEngine*)h)->complete(tok, now_ns); }
LSB_RT_API int lsb_te_cancel(void* h, unsigned long long tok) { return ((TransferEngine*)h)->cancel(tok); }
LSB_RT_API int lsb_te_poll(void* h, unsigned long long* tokens, int* states, int* layers, int* experts, int* gpus, int cap) {
    return ((TransferEngine*)h)->poll_completions((uint64_t*)tokens, states, layers, experts, gpus, cap);
}
LSB_RT_API int lsb_te_queued(void* h, int gpu) { return ((TransferEngine*)h)->queued(gpu); }
LSB_RT_API int lsb_te_in_flight(void* h, int gpu) { return ((TransferEngine*)h)->in_flight(gpu); }
LSB_RT_API double lsb_te_bandwidth_gbs(void* h, int gpu, int dir) { return ((TransferEngine*)h)->bandwidth_gbs(gpu, dir); }
LSB_RT_API unsigned long long lsb_te_dedup_hits(void* h) { return ((TransferEngine*)h)->dedup_hits(); }
LSB_RT_API unsigned long long lsb_te_find(void* h, int layer, int expert, int gpu, int dir) { return ((TransferEngine*)h)->find(layer, expert, gpu, dir); }
}
