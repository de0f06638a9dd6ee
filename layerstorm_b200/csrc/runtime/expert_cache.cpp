// VRAM expert cache bookkeeping: a fixed number of equally sized slots per GPU, split into a
// stable zone and a streaming zone (prefetch + spill), with two-phase fills (reserve ->
// mark_ready), lock/unlock pinning while kernels read a slot, explicit eviction with pluggable
// scoring, promote/demote between zones, elastic extra zones with a generation counter and
// residency listeners.  Metadata only: the caller moves the bytes.
//
// Reference component: ExpertCache (src/core/memory/expert_cache.h:29-133, eviction_policy.h:
// impact_weighted_lru | lru | lfu with +1000 duplicate and +500 streaming penalties;
// ExpertCache::reserve never evicts on its own - callers make room explicitly,
// src/daemon/moe/moe_progressive.cpp:441-453).
//
// Weighted scoring (set_weights): keep-value = -alpha*recency + beta*frequency + gamma*routing_weight +
// delta*temporal_autocorrelation + epsilon*coactivation + zeta*prefetch_score + eta*hysteresis, every
// term in [0, 1]; the lowest keep-value is evicted first.  frequency / autocorrelation are per-step
// EMAs maintained by end_step(); coactivation and prefetch score are hints from the advisers;
// hysteresis is a small per-slot state machine with asymmetric promote / demote thresholds over the
// activations of a window of steps, which keeps a briefly idle hot expert from being thrashed.
// Reference: python/orchestrator/eviction_policy.py (7-term impact-weighted score, HysteresisTracker).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <functional>
#include <unordered_map>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

enum Zone { kStable = 0, kStreaming = 1 };
enum SlotState { kFree = 0, kReserved = 1, kReady = 2 };
enum Policy { kImpactWeightedLru = 0, kLru = 1, kLfu = 2 };

struct Slot {
    int state = kFree;
    int zone = kStable;
    int64_t key = -1;        // layer * 65536 + expert
    int locks = 0;
    uint64_t last_use = 0;
    uint64_t uses = 0;
    float impact = 0.f;      // mean routing weight observed (impact-weighted LRU)
    float freq = 0.f;        // EMA over steps of "was routed in the step"
    float autocorr = 0.f;    // EMA over steps of "was routed in this step and the one before"
    float coact = 0.f;       // hint: co-activation with the experts of the current working set
    float prefetch = 0.f;    // hint: fused prefetch score (likely needed soon)
    int step_uses = 0;       // touches since the last end_step()
    int window_uses = 0;     // touches in the current hysteresis window
    int hyst = 0;            // hysteresis stage, 0 .. hyst_stages
    bool prev_step = false;  // routed in the previous step
    int elastic_gen = 0;     // 0 = permanent slot, otherwise the generation of its elastic zone
};

typedef void (*ResidencyCb)(void* user, int layer, int expert, int slot, int resident);

class ExpertCache {
public:
    ExpertCache(int stable_slots, int streaming_slots, int policy) : policy_(policy) {
        slots_.resize(stable_slots + streaming_slots);
        for (int i = 0; i < (int)slots_.size(); ++i) slots_[i].zone = i < stable_slots ? kStable : kStreaming;
        n_stable_ = stable_slots;
    }

    static int64_t make_key(int layer, int expert) { return (int64_t)layer * 65536 + expert; }

    int lookup(int layer, int expert) const {
        auto it = map_.find(make_key(layer, expert));
        return it == map_.end() ? -1 : it->second;
    }
    int is_ready(int layer, int expert) const {
        int s = lookup(layer, expert);
        return s >= 0 && slots_[s].state == kReady;
    }

    // Phase 1: claim a free slot in `zone` (streaming overflow falls back to stable when allowed).
    int reserve(int layer, int expert, int zone, bool allow_fallback) {
        if (lookup(layer, expert) >= 0) return LSB_ERR_EXISTS;
        int s = find_free(zone);
        if (s < 0 && allow_fallback) s = find_free(zone == kStable ? kStreaming : kStable);
        if (s < 0) return LSB_ERR_FULL;
        Slot& sl = slots_[s];
        sl.state = kReserved; sl.key = make_key(layer, expert); sl.locks = 0; sl.uses = 0; sl.impact = 0.f;
        sl.freq = sl.autocorr = sl.coact = sl.prefetch = 0.f;
        sl.step_uses = sl.window_uses = sl.hyst = 0; sl.prev_step = false;
        sl.last_use = ++tick_;
        map_[sl.key] = s;
        return s;
    }
    // Phase 2: the copy has landed.
    int mark_ready(int layer, int expert) {
        int s = lookup(layer, expert);
        if (s < 0) return LSB_ERR_NOT_FOUND;
        if (slots_[s].state != kReserved) return LSB_ERR_ARG;
        slots_[s].state = kReady;
        notify(slots_[s], s, 1);
        return s;
    }
    // A failed fill releases its reservation; the expert stays fetchable.
    int cancel(int layer, int expert) {
        int s = lookup(layer, expert);
        if (s < 0) return LSB_ERR_NOT_FOUND;
        if (slots_[s].state != kReserved) return LSB_ERR_ARG;
        free_slot(s);
        return 0;
    }
    int lock(int layer, int expert) {
        int s = lookup(layer, expert);
        if (s < 0 || slots_[s].state != kReady) return LSB_ERR_NOT_FOUND;
        slots_[s].locks++;
        return s;
    }
    int unlock(int layer, int expert) {
        int s = lookup(layer, expert);
        if (s < 0 || slots_[s].locks <= 0) return LSB_ERR_ARG;
        slots_[s].locks--;
        return 0;
    }
    void touch(int layer, int expert, float weight) {
        int s = lookup(layer, expert);
        if (s < 0) return;
        Slot& sl = slots_[s];
        sl.last_use = ++tick_;
        sl.uses++;
        sl.step_uses++;
        sl.window_uses++;
        sl.impact += (weight - sl.impact) / (float)std::min<uint64_t>(sl.uses, 64);
    }
    int evict(int layer, int expert) {
        int s = lookup(layer, expert);
        if (s < 0) return LSB_ERR_NOT_FOUND;
        if (slots_[s].locks > 0 || slots_[s].state == kReserved) return LSB_ERR_BUSY;
        notify(slots_[s], s, 0);
        free_slot(s);
        return s;
    }
    // Eviction score: lower = evict first.  Streaming-zone entries and duplicates (resident on
    // another GPU too) are preferred victims.
    double score(const Slot& sl, bool duplicate) const {
        double base;
        if (weighted_ && policy_ == kImpactWeightedLru) {
            double recency = (double)(tick_ - sl.last_use) / (double)(tick_ + 1);
            double hyst = hyst_stages_ > 0 ? (double)sl.hyst / hyst_stages_ : 0.0;
            base = -w_[0] * recency + w_[1] * sl.freq + w_[2] * std::min(1.f, sl.impact) + w_[3] * sl.autocorr + w_[4] * sl.coact +
                   w_[5] * sl.prefetch + w_[6] * hyst;
            if (duplicate) base -= 1000.0;
            if (sl.zone == kStreaming) base -= 500.0;
            return base;
        }
        if (policy_ == kLru) base = (double)sl.last_use;
        else if (policy_ == kLfu) base = (double)sl.uses;
        else base = (double)sl.last_use * (0.25 + (double)sl.impact);
        if (duplicate) base -= 1000.0;
        if (sl.zone == kStreaming) base -= 500.0;
        return base;
    }
    // Live-changeable: policy and the seven weights (alpha .. eta).  Switches the impact-weighted policy to the weighted score.
    void set_weights(int policy, const float* w7) {
        policy_ = policy;
        for (int i = 0; i < 7; ++i) w_[i] = w7[i];
        weighted_ = true;
    }
    void set_hysteresis(int stages, int up, int down, int window_steps, float ema) {
        hyst_stages_ = stages; hyst_up_ = up; hyst_down_ = down; hyst_window_ = std::max(1, window_steps);
        ema_ = ema;
    }
    int set_hint(int layer, int expert, float coactivation, float prefetch_score) {
        int s = lookup(layer, expert);
        if (s < 0) return LSB_ERR_NOT_FOUND;
        if (coactivation >= 0.f) slots_[s].coact = std::min(1.f, coactivation);
        if (prefetch_score >= 0.f) slots_[s].prefetch = std::min(1.f, prefetch_score);
        return 0;
    }
    // Once per decode step / prefill chunk: fold the step's touches into the per-slot statistics.
    void end_step() {
        ++steps_;
        bool close_window = steps_ % hyst_window_ == 0;
        for (auto& sl : slots_) {
            if (sl.state != kReady) continue;
            bool on = sl.step_uses > 0;
            sl.freq += ema_ * ((on ? 1.f : 0.f) - sl.freq);
            sl.autocorr += ema_ * ((on && sl.prev_step ? 1.f : 0.f) - sl.autocorr);
            sl.prev_step = on;
            sl.step_uses = 0;
            if (close_window) {
                int diff = sl.window_uses - sl.hyst;
                if (diff >= hyst_up_) sl.hyst = std::min(hyst_stages_, sl.hyst + 1);
                else if (-diff >= hyst_down_) sl.hyst = std::max(0, sl.hyst - 1);
                sl.window_uses = 0;
            }
        }
    }
    int slot_stats(int slot, float* out7) const {
        if (slot < 0 || slot >= (int)slots_.size()) return LSB_ERR_ARG;
        const Slot& sl = slots_[slot];
        out7[0] = (float)((double)(tick_ - sl.last_use) / (double)(tick_ + 1)); out7[1] = sl.freq; out7[2] = sl.impact; out7[3] = sl.autocorr;
        out7[4] = sl.coact; out7[5] = sl.prefetch; out7[6] = hyst_stages_ > 0 ? (float)sl.hyst / hyst_stages_ : 0.f;
        return 0;
    }
    // Picks an unlocked ready victim in `zone` (-1 = any); returns slot or -1 and its key.
    int pick_victim(int zone, const uint8_t* duplicate_flags, int n_flags, int* layer, int* expert) const {
        int best = -1;
        double bs = 0;
        for (int i = 0; i < (int)slots_.size(); ++i) {
            const Slot& sl = slots_[i];
            if (sl.state != kReady || sl.locks > 0) continue;
            if (zone >= 0 && sl.zone != zone) continue;
            bool dup = duplicate_flags && i < n_flags && duplicate_flags[i];
            double sc = score(sl, dup);
            if (best < 0 || sc < bs) { best = i; bs = sc; }
        }
        if (best >= 0) { *layer = (int)(slots_[best].key / 65536); *expert = (int)(slots_[best].key % 65536); }
        return best;
    }
    // Zone moves are metadata only when the slot pools share storage: swap zone labels with a free
    // slot of the target zone so the zone sizes stay constant.
    int move_zone(int layer, int expert, int to_zone) {
        int s = lookup(layer, expert);
        if (s < 0) return LSB_ERR_NOT_FOUND;
        if (slots_[s].zone == to_zone) return s;
        int f = find_free(to_zone);
        if (f < 0) return LSB_ERR_FULL;
        std::swap(slots_[s].zone, slots_[f].zone);
        return s;
    }
    // Elastic zones: extra stable slots on memory lent by the KV pool.  Returns the generation id.
    int add_elastic_zone(int n_slots) {
        int gen = ++generation_;
        for (int i = 0; i < n_slots; ++i) { Slot s; s.zone = kStable; s.elastic_gen = gen; slots_.push_back(s); }
        return gen;
    }
    // Removing a zone requires all its slots to be free (caller quiesces + evicts first).
    int remove_elastic_zone(int gen) {
        for (auto& s : slots_) if (s.elastic_gen == gen && s.state != kFree) return LSB_ERR_BUSY;
        std::vector<Slot> keep;
        std::unordered_map<int, int> remap;
        for (int i = 0; i < (int)slots_.size(); ++i)
            if (slots_[i].elastic_gen != gen) { remap[i] = (int)keep.size(); keep.push_back(slots_[i]); }
        for (auto& kv : map_) kv.second = remap[kv.second];
        slots_.swap(keep);
        ++generation_;
        return 0;
    }
    int generation() const { return generation_; }
    int n_slots() const { return (int)slots_.size(); }
    int count(int zone, int state) const {
        int c = 0;
        for (auto& s : slots_) if ((zone < 0 || s.zone == zone) && s.state == state) ++c;
        return c;
    }
    int slot_info(int slot, int* state, int* zone, int* layer, int* expert, int* locks) const {
        if (slot < 0 || slot >= (int)slots_.size()) return LSB_ERR_ARG;
        const Slot& s = slots_[slot];
        *state = s.state; *zone = s.zone; *locks = s.locks;
        *layer = s.key < 0 ? -1 : (int)(s.key / 65536); *expert = s.key < 0 ? -1 : (int)(s.key % 65536);
        return 0;
    }
    void set_listener(ResidencyCb cb, void* user) { cb_ = cb; user_ = user; }

private:
    int find_free(int zone) const {
        for (int i = 0; i < (int)slots_.size(); ++i)
            if (slots_[i].state == kFree && slots_[i].zone == zone) return i;
        return -1;
    }
    void free_slot(int s) {
        map_.erase(slots_[s].key);
        slots_[s].state = kFree; slots_[s].key = -1; slots_[s].locks = 0;
    }
    void notify(const Slot& sl, int slot, int resident) {
        if (cb_) cb_(user_, (int)(sl.key / 65536), (int)(sl.key % 65536), slot, resident);
    }
    std::vector<Slot> slots_;
    std::unordered_map<int64_t, int> map_;
    int n_stable_ = 0, policy_ = 0, generation_ = 0;
    uint64_t tick_ = 0, steps_ = 0;
    bool weighted_ = false;
    float w_[7] = {0.4f, 0.35f, 0.25f, 0.f, 0.f, 0.f, 0.f};
    int hyst_stages_ = 5, hyst_up_ = 5, hyst_down_ = 1, hyst_window_ = 16;
    float ema_ = 0.1f;
    ResidencyCb cb_ = nullptr;
    void* user_ = nullptr;
};

}  // namespace lsb

using lsb::ExpertCache;
extern "C" {
LSB_RT_API void* lsb_ec_create(int stable, int streaming, int policy) { return new ExpertCache(stable, streaming, policy); }
LSB_RT_API void lsb_ec_destroy(void* h) { delete (ExpertCache*)h; }
LSB_RT_API int lsb_ec_lookup(void* h, int layer, int expert) { return ((ExpertCache*)h)->lookup(layer, expert); }
LSB_RT_API int lsb_ec_is_ready(void* h, int layer, int expert) { return ((ExpertCache*)h)->is_ready(layer, expert); }
LSB_RT_API int lsb_ec_reserve(void* h, int layer, int expert, int zone, int fallback) { return ((ExpertCache*)h)->reserve(layer, expert, zone, fallback != 0); }
LSB_RT_API int lsb_ec_mark_ready(void* h, int layer, int expert) { return ((ExpertCache*)h)->mark_ready(layer, expert); }
LSB_RT_API int lsb_ec_cancel(void* h, int layer, int expert) { return ((ExpertCache*)h)->cancel(layer, expert); }
LSB_RT_API int lsb_ec_lock(void* h, int layer, int expert) { return ((ExpertCache*)h)->lock(layer, expert); }
LSB_RT_API int lsb_ec_unlock(void* h, int layer, int expert) { return ((ExpertCache*)h)->unlock(layer, expert); }
LSB_RT_API void lsb_ec_touch(void* h, int layer, int expert, float w) { ((ExpertCache*)h)->touch(layer, expert, w); }
LSB_RT_API int lsb_ec_evict(void* h, int layer, int expert) { return ((ExpertCache*)h)->evict(layer, expert); }
LSB_RT_API int lsb_ec_pick_victim(void* h, int zone, const uint8_t* dup, int n, int* layer, int* expert) { return ((ExpertCache*)h)->pick_victim(zone, dup, n, layer, expert); }
LSB_RT_API int lsb_ec_move_zone(void* h, int layer, int expert, int zone) { return ((ExpertCache*)h)->move_zone(layer, expert, zone); }
LSB_RT_API int lsb_ec_add_elastic_zone(void* h, int n) { return ((ExpertCache*)h)->add_elastic_zone(n); }
LSB_RT_API int lsb_ec_remove_elastic_zone(void* h, int gen) { return ((ExpertCache*)h)->remove_elastic_zone(gen); }
LSB_RT_API int lsb_ec_generation(void* h) { return ((ExpertCache*)h)->generation(); }
LSB_RT_API int lsb_ec_n_slots(void* h) { return ((ExpertCache*)h)->n_slots(); }
LSB_RT_API int lsb_ec_count(void* h, int zone, int state) { return ((ExpertCache*)h)->count(zone, state); }
LSB_RT_API int lsb_ec_slot_info(void* h, int slot, int* state, int* zone, int* layer, int* expert, int* locks) {
    return ((ExpertCache*)h)->slot_info(slot, state, zone, layer, expert, locks);
}
LSB_RT_API void lsb_ec_set_weights(void* h, int policy, const float* w7) { ((ExpertCache*)h)->set_weights(policy, w7); }
LSB_RT_API void lsb_ec_set_hysteresis(void* h, int stages, int up, int down, int window_steps, float ema) {
    ((ExpertCache*)h)->set_hysteresis(stages, up, down, window_steps, ema);
}
LSB_RT_API int lsb_ec_set_hint(void* h, int layer, int expert, float coact, float prefetch) { return ((ExpertCache*)h)->set_hint(layer, expert, coact, prefetch); }
LSB_RT_API void lsb_ec_end_step(void* h) { ((ExpertCache*)h)->end_step(); }
LSB_RT_API int lsb_ec_slot_stats(void* h, int slot, float* out7) { return ((ExpertCache*)h)->slot_stats(slot, out7); }
LSB_RT_API void lsb_ec_set_listener(void* h, lsb::ResidencyCb cb, void* user) { ((ExpertCache*)h)->set_listener(cb, user); }
}
