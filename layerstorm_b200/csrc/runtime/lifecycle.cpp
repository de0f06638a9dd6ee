// Residency state machines that sit between the routing decisions and the byte movers.
//
//   ExpertLifecycle   per (layer, expert, gpu): host tier {cold (NVMe), loading-to-RAM, warm (pinned
//                     arena)} x device tier {absent, reserved, transferring, hot, draining} with an
//                     interest count.  ensure_resident() returns the NEXT action the owner must
//                     perform (read from NVMe, reserve a cache slot, start the H2D copy, nothing) and
//                     events move the machine forward; an expert with interest > 0 is never drained.
//   ZoneRebalancer    lends runs of KV pages to the expert cache as elastic zones: pressure flows
//                     expert -> KV only; low/high water marks with hysteresis decide when to lend and
//                     when to reclaim; a reclaim first quiesces (no new placements), then waits for
//                     the zone to drain, then returns the pages.
//   KvTierTable       which KV pages of a sequence are hot (HBM) or cold (pinned host), the demotion
//                     frontier behind the retention window, refcounted cold slots shared across forks,
//                     re-promotion on rewind, and the hot-row LRU for rows fetched back for sparse
//                     attention.  Placement only: the set of rows attention reads is decided by the
//                     indexer and is the same with tiering on or off.
// Reference components: ExpertLifecycleManager (src/daemon/expert_lifecycle_manager.h:38-92),
// ExpertZoneRebalancer (src/daemon/expert_zone_rebalancer.{h,cpp}), KvTieringManager
// (src/daemon/kv_tiering_manager.h:1-260).
#include <algorithm>
#include <cstdint>
#include <list>
#include <map>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

// ------------------------------------------------------------------ expert lifecycle
enum HostTier { kCold = 0, kLoadingToRam = 1, kWarm = 2 };
enum GpuTier { kAbsent = 0, kReserved = 1, kTransferring = 2, kHot = 3, kDraining = 4 };
enum Action { kActNone = 0, kActReadNvme = 1, kActReserveSlot = 2, kActStartH2D = 3, kActWait = 4 };
enum Event { kEvNvmeDone = 0, kEvNvmeFailed = 1, kEvSlotReserved = 2, kEvSlotDenied = 3, kEvH2DStarted = 4, kEvH2DDone = 5,
             kEvH2DFailed = 6, kEvEvictRequested = 7, kEvDrained = 8, kEvHostEvicted = 9 };

struct ExpertState { int host = kCold; int gpu = kAbsent; int interest = 0; uint64_t token = 0; };

class ExpertLifecycle {
public:
    using Key = std::tuple<int, int, int>;
    void set_host_tier(int layer, int expert, int tier) {
        for (auto& kv : st_) if (std::get<0>(kv.first) == layer && std::get<1>(kv.first) == expert) kv.second.host = tier;
        host_[{layer, expert}] = tier;
    }
    ExpertState& at(int layer, int expert, int gpu) {
        auto it = st_.find({layer, expert, gpu});
        if (it == st_.end()) {
            ExpertState s;
            auto h = host_.find({layer, expert});
            s.host = h == host_.end() ? kCold : h->second;
            it = st_.emplace(Key{layer, expert, gpu}, s).first;
        }
        return it->second;
    }
    // Registers interest and says what to do next.
    int ensure_resident(int layer, int expert, int gpu, uint64_t* token) {
        ExpertState& s = at(layer, expert, gpu);
        ++s.interest;
        if (!s.token) s.token = ++next_;
        *token = s.token;
        return next_action(s);
    }
    int next_action(const ExpertState& s) const {
        if (s.gpu == kHot) return kActNone;
        if (s.gpu == kDraining) return kActWait;
        if (s.host == kCold) return kActReadNvme;
        if (s.host == kLoadingToRam) return kActWait;
        if (s.gpu == kAbsent) return kActReserveSlot;
        if (s.gpu == kReserved) return kActStartH2D;
        return kActWait;                                    // transferring
    }
    int release(int layer, int expert, int gpu) {
        ExpertState& s = at(layer, expert, gpu);
        if (s.interest > 0) --s.interest;
        return s.interest;
    }
    // Returns the next action after the event, or an error for an event that does not fit the state.
    int on_event(int layer, int expert, int gpu, int ev) {
        ExpertState& s = at(layer, expert, gpu);
        switch (ev) {
            case kEvNvmeDone: if (s.host == kCold || s.host == kLoadingToRam) set_host_tier(layer, expert, kWarm); s.host = kWarm; break;
            case kEvNvmeFailed: set_host_tier(layer, expert, kCold); s.host = kCold; break;
            case kEvSlotReserved: if (s.gpu != kAbsent) return LSB_ERR_ARG; s.gpu = kReserved; break;
            case kEvSlotDenied: if (s.gpu != kAbsent) return LSB_ERR_ARG; break;
            case kEvH2DStarted: if (s.gpu != kReserved) return LSB_ERR_ARG; s.gpu = kTransferring; break;
            case kEvH2DDone: if (s.gpu != kTransferring) return LSB_ERR_ARG; s.gpu = kHot; ++loads_; break;
            case kEvH2DFailed: if (s.gpu != kTransferring && s.gpu != kReserved) return LSB_ERR_ARG; s.gpu = kAbsent; break;
            case kEvEvictRequested:
                if (s.gpu != kHot) return LSB_ERR_ARG;
                if (s.interest > 0) return LSB_ERR_BUSY;    // somebody is about to run it
                s.gpu = kDraining; break;
            case kEvDrained: if (s.gpu != kDraining) return LSB_ERR_ARG; s.gpu = kAbsent; s.token = 0; ++evictions_; break;
            case kEvHostEvicted:
                if (s.gpu == kTransferring || s.gpu == kReserved) return LSB_ERR_BUSY;   // the copy still reads the host slot
                set_host_tier(layer, expert, kCold); s.host = kCold; break;
            default: return LSB_ERR_ARG;
        }
        if (ev == kEvNvmeDone) { auto& cur = at(layer, expert, gpu); return next_action(cur); }
        return next_action(s);
    }
    // When the host read starts, all device views of the expert see kLoadingToRam.
    void begin_host_load(int layer, int expert) { set_host_tier(layer, expert, kLoadingToRam); }
    void get(int layer, int expert, int gpu, int* host, int* gputier, int* interest) {
        const ExpertState& s = at(layer, expert, gpu);
        *host = s.host; *gputier = s.gpu; *interest = s.interest;
    }
    uint64_t loads() const { return loads_; }
    uint64_t evictions() const { return evictions_; }
private:
    std::map<Key, ExpertState> st_;
    std::map<std::pair<int, int>, int> host_;
    uint64_t next_ = 0, loads_ = 0, evictions_ = 0;
};

// ------------------------------------------------------------------ zone rebalancer
enum ZoneState { kZoneActive = 0, kZoneQuiescing = 1 };
enum RebalanceAction { kRbNone = 0, kRbLend = 1, kRbBeginReclaim = 2, kRbFinishReclaim = 3 };

struct LentZone { int gen; int pages; int state; };

class ZoneRebalancer {
public:
    ZoneRebalancer(int total_kv_pages, int pages_per_zone, double low_water, double high_water, int max_zones)
        : total_(total_kv_pages), per_zone_(pages_per_zone), low_(low_water), high_(high_water), max_zones_(max_zones) {}
    // kv_used: KV pages in use (lent pages excluded); expert_miss_rate: recent miss fraction of the expert cache;
    // zone_occupancy: resident experts in the zone being reclaimed (only read while quiescing).
    int step(int kv_used, double expert_miss_rate, int zone_occupancy, int* gen_out) {
        *gen_out = -1;
        const int lent = lent_pages();
        const double util = (double)kv_used / (double)std::max(1, total_ - lent);
        for (auto& z : zones_) {
            if (z.state == kZoneQuiescing) {
                *gen_out = z.gen;
                return zone_occupancy == 0 ? kRbFinishReclaim : kRbNone;          // wait for the drain
            }
        }
        if (util > high_ && !zones_.empty()) {                                   // KV pressure: take the newest zone back
            zones_.back().state = kZoneQuiescing;
            *gen_out = zones_.back().gen;
            return kRbBeginReclaim;
        }
        const double util_after = (double)kv_used / (double)std::max(1, total_ - lent - per_zone_);
        if (expert_miss_rate > 0.0 && util_after < low_ && (int)zones_.size() < max_zones_ && total_ - lent - per_zone_ > kv_used) {
            *gen_out = ++gen_;
            return kRbLend;
        }
        return kRbNone;
    }
    void on_lent(int gen) { zones_.push_back(LentZone{gen, per_zone_, kZoneActive}); }
    int on_reclaimed(int gen) {
        for (auto it = zones_.begin(); it != zones_.end(); ++it)
            if (it->gen == gen) { if (it->state != kZoneQuiescing) return LSB_ERR_BUSY; zones_.erase(it); return 0; }
        return LSB_ERR_NOT_FOUND;
    }
    int lent_pages() const { int n = 0; for (auto& z : zones_) n += z.pages; return n; }
    int n_zones() const { return (int)zones_.size(); }
private:
    int total_, per_zone_;
    double low_, high_;
    int max_zones_;
    int gen_ = 0;
    std::vector<LentZone> zones_;
};

// ------------------------------------------------------------------ KV tier table
struct SeqTier {
    std::vector<int> cold_slot;      // per logical page: -1 = hot (in HBM), else cold slot id
    int frontier = 0;                // pages [0, frontier) have been considered for demotion
};

class KvTierTable {
public:
    KvTierTable(int page_tokens, int hot_window_tokens, int cold_slots, int row_cache_rows)
        : page_(page_tokens), window_(hot_window_tokens), cold_refs_(cold_slots, 0), row_cap_(row_cache_rows) {
        for (int i = cold_slots - 1; i >= 0; --i) free_cold_.push_back(i);
    }
    void create(int seq) { seqs_[seq] = SeqTier{}; }
    int fork(int parent, int child, int prefix_pages) {
        auto it = seqs_.find(parent);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        SeqTier c;
        c.cold_slot.assign(it->second.cold_slot.begin(), it->second.cold_slot.begin() + std::min<size_t>(prefix_pages, it->second.cold_slot.size()));
        for (int s : c.cold_slot) if (s >= 0) ++cold_refs_[s];             // cold copies are shared, not duplicated
        c.frontier = std::min(it->second.frontier, prefix_pages);
        seqs_[child] = c;
        return 0;
    }
    int destroy(int seq) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        for (int s : it->second.cold_slot) if (s >= 0) unref_cold(s);
        seqs_.erase(it);
        return 0;
    }
    // Pages wholly behind the retention window that are still hot, oldest first (up to cap).
    int demotion_candidates(int seq, int seq_len, int* pages, int cap) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        SeqTier& s = it->second;
        const int npages = (seq_len + page_ - 1) / page_;
        if ((int)s.cold_slot.size() < npages) s.cold_slot.resize(npages, -1);
        const int last = (seq_len - window_) / page_;                     // pages [0, last) end before the window starts
        int n = 0;
        for (int p = 0; p < last && n < cap; ++p) if (s.cold_slot[p] < 0) pages[n++] = p;
        return n;
    }
    // Assign a cold slot to a page that is being demoted (the owner then copies the page D2H and frees the HBM page).
    int demote(int seq, int page) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end() || page < 0 || page >= (int)it->second.cold_slot.size()) return LSB_ERR_ARG;
        if (it->second.cold_slot[page] >= 0) return it->second.cold_slot[page];
        if (free_cold_.empty()) return LSB_ERR_FULL;
        const int slot = free_cold_.back();
        free_cold_.pop_back();
        cold_refs_[slot] = 1;
        it->second.cold_slot[page] = slot;
        it->second.frontier = std::max(it->second.frontier, page + 1);
        ++demotions_;
        return slot;
    }
    // Rewind below the frontier or a non-tierable shape: the page returns to HBM; returns the cold slot to read back.
    int promote(int seq, int page) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end() || page < 0 || page >= (int)it->second.cold_slot.size()) return LSB_ERR_ARG;
        const int slot = it->second.cold_slot[page];
        if (slot < 0) return LSB_ERR_NOT_FOUND;
        it->second.cold_slot[page] = -1;
        unref_cold(slot);
        ++promotions_;
        return slot;
    }
    int truncate(int seq, int new_len) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        const int keep = (new_len + page_ - 1) / page_;
        SeqTier& s = it->second;
        for (int p = keep; p < (int)s.cold_slot.size(); ++p) if (s.cold_slot[p] >= 0) unref_cold(s.cold_slot[p]);
        if ((int)s.cold_slot.size() > keep) s.cold_slot.resize(keep);
        s.frontier = std::min(s.frontier, keep);
        return 0;
    }
    int where(int seq, int page) const {
        auto it = seqs_.find(seq);
        if (it == seqs_.end() || page < 0 || page >= (int)it->second.cold_slot.size()) return -1;
        return it->second.cold_slot[page];
    }
    // Classify the rows selected for one attention call: hot page / hot row cache / cold fetch.
    // rows[i] = token position; out_kind[i] = 0 hot page, 1 row cache hit (out_ref = cache line), 2 cold (out_ref = cold slot).
    int classify(int seq, int layer, const int* rows, int n, int* out_kind, int* out_ref) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        int cold = 0;
        for (int i = 0; i < n; ++i) {
            const int p = rows[i] / page_;
            const int slot = p < (int)it->second.cold_slot.size() ? it->second.cold_slot[p] : -1;
            if (slot < 0) { out_kind[i] = 0; out_ref[i] = p; continue; }
            const RowKey k{seq, layer, rows[i]};
            auto rc = row_index_.find(k);
            if (rc != row_index_.end()) {
                lru_.splice(lru_.begin(), lru_, rc->second);
                out_kind[i] = 1; out_ref[i] = rc->second->line; ++row_hits_;
            } else {
                out_kind[i] = 2; out_ref[i] = slot; ++cold;
            }
        }
        cold_fetches_ += cold;
        return cold;
    }
    // Insert a fetched cold row into the hot row cache; returns the cache line to write it to.
    int cache_row(int seq, int layer, int row) {
        if (row_cap_ <= 0) return -1;
        const RowKey k{seq, layer, row};
        auto rc = row_index_.find(k);
        if (rc != row_index_.end()) { lru_.splice(lru_.begin(), lru_, rc->second); return rc->second->line; }
        int line;
        if ((int)lru_.size() < row_cap_) line = (int)lru_.size();
        else { line = lru_.back().line; row_index_.erase(lru_.back().key); lru_.pop_back(); }
        lru_.push_front(RowLine{k, line});
        row_index_[k] = lru_.begin();
        return line;
    }
    int free_cold_slots() const { return (int)free_cold_.size(); }
    void stats(uint64_t* dem, uint64_t* prom, uint64_t* cold, uint64_t* hits) const { *dem = demotions_; *prom = promotions_; *cold = cold_fetches_; *hits = row_hits_; }
private:
    using RowKey = std::tuple<int, int, int>;
    struct RowLine { RowKey key; int line; };
    void unref_cold(int slot) { if (--cold_refs_[slot] == 0) free_cold_.push_back(slot); }
    int page_, window_;
    std::vector<int> cold_refs_, free_cold_;
    int row_cap_;
    std::map<int, SeqTier> seqs_;
    std::list<RowLine> lru_;
    std::map<RowKey, std::list<RowLine>::iterator> row_index_;
    uint64_t demotions_ = 0, promotions_ = 0, cold_fetches_ = 0, row_hits_ = 0;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
LSB_RT_API void* lsb_elm_create() { return new ExpertLifecycle(); }
LSB_RT_API void lsb_elm_destroy(void* h) { delete (ExpertLifecycle*)h; }
LSB_RT_API void lsb_elm_set_host_tier(void* h, int layer, int expert, int tier) { ((ExpertLifecycle*)h)->set_host_tier(layer, expert, tier); }
LSB_RT_API void lsb_elm_begin_host_load(void* h, int layer, int expert) { ((ExpertLifecycle*)h)->begin_host_load(layer, expert); }
LSB_RT_API int lsb_elm_ensure_resident(void* h, int layer, int expert, int gpu, unsigned long long* token) {
    uint64_t t = 0;
    const int a = ((ExpertLifecycle*)h)->ensure_resident(layer, expert, gpu, &t);
    *token = t;
    return a;
}
LSB_RT_API int lsb_elm_release(void* h, int layer, int expert, int gpu) { return ((ExpertLifecycle*)h)->release(layer, expert, gpu); }
LSB_RT_API int lsb_elm_on_event(void* h, int layer, int expert, int gpu, int ev) { return ((ExpertLifecycle*)h)->on_event(layer, expert, gpu, ev); }
LSB_RT_API void lsb_elm_get(void* h, int layer, int expert, int gpu, int* host, int* gputier, int* interest) { ((ExpertLifecycle*)h)->get(layer, expert, gpu, host, gputier, interest); }
LSB_RT_API unsigned long long lsb_elm_loads(void* h) { return ((ExpertLifecycle*)h)->loads(); }
LSB_RT_API unsigned long long lsb_elm_evictions(void* h) { return ((ExpertLifecycle*)h)->evictions(); }

LSB_RT_API void* lsb_zr_create(int total_kv_pages, int pages_per_zone, double low_water, double high_water, int max_zones) {
    return new ZoneRebalancer(total_kv_pages, pages_per_zone, low_water, high_water, max_zones);
}
LSB_RT_API void lsb_zr_destroy(void* h) { delete (ZoneRebalancer*)h; }
LSB_RT_API int lsb_zr_step(void* h, int kv_used, double miss_rate, int zone_occupancy, int* gen) { return ((ZoneRebalancer*)h)->step(kv_used, miss_rate, zone_occupancy, gen); }
LSB_RT_API void lsb_zr_on_lent(void* h, int gen) { ((ZoneRebalancer*)h)->on_lent(gen); }
LSB_RT_API int lsb_zr_on_reclaimed(void* h, int gen) { return ((ZoneRebalancer*)h)->on_reclaimed(gen); }
LSB_RT_API int lsb_zr_lent_pages(void* h) { return ((ZoneRebalancer*)h)->lent_pages(); }
LSB_RT_API int lsb_zr_n_zones(void* h) { return ((ZoneRebalancer*)h)->n_zones(); }

LSB_RT_API void* lsb_kvt_create(int page_tokens, int hot_window_tokens, int cold_slots, int row_cache_rows) {
    return new KvTierTable(page_tokens, hot_window_tokens, cold_slots, row_cache_rows);
}
LSB_RT_API void lsb_kvt_destroy(void* h) { delete (KvTierTable*)h; }
LSB_RT_API void lsb_kvt_seq_create(void* h, int seq) { ((KvTierTable*)h)->create(seq); }
LSB_RT_API int lsb_kvt_seq_fork(void* h, int parent, int child, int prefix_pages) { return ((KvTierTable*)h)->fork(parent, child, prefix_pages); }
LSB_RT_API int lsb_kvt_seq_destroy(void* h, int seq) { return ((KvTierTable*)h)->destroy(seq); }
LSB_RT_API int lsb_kvt_demotion_candidates(void* h, int seq, int seq_len, int* pages, int cap) { return ((KvTierTable*)h)->demotion_candidates(seq, seq_len, pages, cap); }
LSB_RT_API int lsb_kvt_demote(void* h, int seq, int page) { return ((KvTierTable*)h)->demote(seq, page); }
LSB_RT_API int lsb_kvt_promote(void* h, int seq, int page) { return ((KvTierTable*)h)->promote(seq, page); }
LSB_RT_API int lsb_kvt_truncate(void* h, int seq, int new_len) { return ((KvTierTable*)h)->truncate(seq, new_len); }
LSB_RT_API int lsb_kvt_where(void* h, int seq, int page) { return ((KvTierTable*)h)->where(seq, page); }
LSB_RT_API int lsb_kvt_classify(void* h, int seq, int layer, const int* rows, int n, int* kind, int* ref) { return ((KvTierTable*)h)->classify(seq, layer, rows, n, kind, ref); }
LSB_RT_API int lsb_kvt_cache_row(void* h, int seq, int layer, int row) { return ((KvTierTable*)h)->cache_row(seq, layer, row); }
LSB_RT_API int lsb_kvt_free_cold_slots(void* h) { return ((KvTierTable*)h)->free_cold_slots(); }
LSB_RT_API void lsb_kvt_stats(void* h, unsigned long long* dem, unsigned long long* prom, unsigned long long* cold, unsigned long long* hits) {
    uint64_t a, b, c, d;
    ((KvTierTable*)h)->stats(&a, &b, &c, &d);
    *dem = a; *prom = b; *cold = c; *hits = d;
}
}
