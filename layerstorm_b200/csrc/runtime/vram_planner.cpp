// Device-memory plan of one GPU, the run-to-run determinism registry and the buffer-id registry.
//
//   VramPlan   carves the usable bytes of a GPU into fixed regions, in this order:
//                weights (resident shard) | workspace | KV speculation pool | indexer-K pool | KV main pool
//                (+ prefill scratch) | recurrent (KDA) state pool | expert streaming zone (prefetch + spill)
//                | expert stable zone | safety margin
//              Fixed-size regions are taken first; the expert zones share what is left by
//              `stable_zone_fraction`; every region is 2 MiB aligned.  The plan fails (naming the first
//              region that does not fit) instead of over-committing.
//   Determinism   registry of knobs behind two super-flags: run-to-run determinism, and reference-trajectory
//              identity (which implies the first).  A knob pinned by the user to a value that contradicts an
//              active super-flag is a refusal, not a silent override.
//   BufferRegistry   small integer ids for device buffers so commands and traces can name them.
// Reference components: VramAllocator (src/core/memory/vram_allocator.h:20-418), determinism
// (src/core/determinism.{h,cpp}), BufferRegistry (src/daemon/buffer_registry.*).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

enum Region { kRegWeights = 0, kRegWorkspace, kRegKvSpec, kRegIndexerK, kRegKvMain, kRegPrefillScratch, kRegRecurrent,
              kRegExpertStreaming, kRegExpertStable, kRegSafety, kRegCount };

struct VramPlanIn {
    int64_t total_bytes, weights_bytes, workspace_bytes;
    int64_t kv_bytes_per_page, kv_pages;           // main pool
    double spec_pool_fraction;                     // speculation pool = fraction of the main pool's pages
    int64_t indexer_bytes_per_page, indexer_pages;
    int64_t prefill_scratch_bytes;
    int64_t recurrent_bytes_per_seq, recurrent_seqs;
    int64_t expert_slot_bytes; int64_t expert_slots_wanted;   // total over layers
    double stable_zone_fraction;
    int64_t safety_bytes;
};

struct VramPlanOut {
    int64_t offset[kRegCount], size[kRegCount];
    int64_t kv_spec_pages, expert_stable_slots, expert_streaming_slots;
    int failed_region;                              // -1 = ok
};

static int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

static void plan_vram(const VramPlanIn& in, VramPlanOut& out) {
    constexpr int64_t A = 2ll << 20;
    std::memset(&out, 0, sizeof(out));
    out.failed_region = -1;
    int64_t want[kRegCount] = {0};
    want[kRegWeights] = in.weights_bytes;
    want[kRegWorkspace] = in.workspace_bytes;
    out.kv_spec_pages = (int64_t)(in.spec_pool_fraction * (double)in.kv_pages);
    want[kRegKvSpec] = out.kv_spec_pages * in.kv_bytes_per_page;
    want[kRegIndexerK] = in.indexer_pages * in.indexer_bytes_per_page;
    want[kRegKvMain] = in.kv_pages * in.kv_bytes_per_page;
    want[kRegPrefillScratch] = in.prefill_scratch_bytes;
    want[kRegRecurrent] = in.recurrent_bytes_per_seq * in.recurrent_seqs;
    want[kRegSafety] = in.safety_bytes;
    int64_t cur = 0;
    const int64_t usable = in.total_bytes - align_up(in.safety_bytes, A);
    for (int r = 0; r < kRegExpertStreaming; ++r) {
        out.offset[r] = cur;
        out.size[r] = align_up(want[r], A);
        cur += out.size[r];
        if (cur > usable) { out.failed_region = r; return; }
    }
    // expert zones share the remainder
    const int64_t left = usable - cur;
    int64_t slots = in.expert_slot_bytes > 0 ? left / in.expert_slot_bytes : 0;
    slots = std::min(slots, in.expert_slots_wanted);
    if (in.expert_slots_wanted > 0 && slots <= 0) { out.failed_region = kRegExpertStable; return; }
    const bool all_fit = slots >= in.expert_slots_wanted;
    // when everything fits there is nothing to stream: one stable zone
    out.expert_stable_slots = all_fit ? slots : (int64_t)(in.stable_zone_fraction * (double)slots);
    out.expert_streaming_slots = slots - out.expert_stable_slots;
    if (!all_fit && out.expert_streaming_slots < 2 && slots >= 2) { out.expert_streaming_slots = 2; out.expert_stable_slots = slots - 2; }
    out.offset[kRegExpertStreaming] = cur;
    out.size[kRegExpertStreaming] = out.expert_streaming_slots * in.expert_slot_bytes;
    cur += align_up(out.size[kRegExpertStreaming], A);
    out.offset[kRegExpertStable] = cur;
    out.size[kRegExpertStable] = out.expert_stable_slots * in.expert_slot_bytes;
    cur += out.size[kRegExpertStable];
    if (cur > usable) { out.failed_region = kRegExpertStable; return; }
    out.offset[kRegSafety] = usable;
    out.size[kRegSafety] = in.total_bytes - usable;
}

// ------------------------------------------------------------------ determinism
struct Knob { std::string name; int value; int det_value; int ident_value; bool pinned; };

class Determinism {
public:
    Determinism() {
        // name, default, value under run-to-run determinism (-1 = free), value under trajectory identity (-1 = free)
        add("deterministic_reduce", 1, 1, 1);
        add("deterministic_ep_combine", 1, 1, 1);
        add("ep_combine_fp32", 1, -1, 1);
        add("split_k_ordered", 1, 1, 1);
        add("atomic_accumulate", 0, 0, 0);
        add("spec_round_governor", 1, -1, 0);          // adaptive drafting changes the round shapes
        add("expert_batching_wait", 1, -1, 0);
        add("prefix_cache_grid_only", 1, 1, 1);
        add("async_expert_prefetch_reorder", 1, 0, 0);
        add("cuda_graphs", 1, -1, -1);
    }
    int set_flags(int deterministic, int identity, char* conflict, int cap) {
        det_ = deterministic || identity;
        ident_ = identity != 0;
        for (auto& k : knobs_) {
            const int forced = ident_ && k.ident_value >= 0 ? k.ident_value : (det_ && k.det_value >= 0 ? k.det_value : -1);
            if (forced < 0) continue;
            if (k.pinned && k.value != forced) {
                if (conflict && cap > 0) { std::strncpy(conflict, k.name.c_str(), cap - 1); conflict[cap - 1] = 0; }
                return LSB_ERR_BUSY;                     // refusal: a pin contradicts the super-flag
            }
            k.value = forced;
        }
        return 0;
    }
    int pin(const char* name, int value) {
        for (auto& k : knobs_) if (k.name == name) {
            const int forced = ident_ && k.ident_value >= 0 ? k.ident_value : (det_ && k.det_value >= 0 ? k.det_value : -1);
            if (forced >= 0 && forced != value) return LSB_ERR_BUSY;
            k.value = value; k.pinned = true;
            return 0;
        }
        return LSB_ERR_NOT_FOUND;
    }
    int get(const char* name) const {
        for (auto& k : knobs_) if (k.name == name) return k.value;
        return LSB_ERR_NOT_FOUND;
    }
    int count() const { return (int)knobs_.size(); }
    const char* name_at(int i) const { return i >= 0 && i < (int)knobs_.size() ? knobs_[i].name.c_str() : ""; }
private:
    void add(const char* n, int v, int d, int i) { knobs_.push_back(Knob{n, v, d, i, false}); }
    std::vector<Knob> knobs_;
    bool det_ = false, ident_ = false;
};

// ------------------------------------------------------------------ buffer registry
class BufferRegistry {
public:
    int add(const char* name, uint64_t ptr, uint64_t bytes, int gpu) {
        if (by_name_.count(name)) return LSB_ERR_EXISTS;
        const int id = (int)bufs_.size();
        bufs_.push_back({name, ptr, bytes, gpu});
        by_name_[name] = id;
        return id;
    }
    int find(const char* name) const { auto it = by_name_.find(name); return it == by_name_.end() ? LSB_ERR_NOT_FOUND : it->second; }
    int get(int id, uint64_t* ptr, uint64_t* bytes, int* gpu) const {
        if (id < 0 || id >= (int)bufs_.size()) return LSB_ERR_NOT_FOUND;
        *ptr = bufs_[id].ptr; *bytes = bufs_[id].bytes; *gpu = bufs_[id].gpu;
        return 0;
    }
    // Does [ptr, ptr+bytes) lie inside registered buffer `id`?  (argument check for primitive commands)
    int contains(int id, uint64_t ptr, uint64_t bytes) const {
        if (id < 0 || id >= (int)bufs_.size()) return 0;
        return ptr >= bufs_[id].ptr && ptr + bytes <= bufs_[id].ptr + bufs_[id].bytes;
    }
    int count() const { return (int)bufs_.size(); }
private:
    struct Buf { std::string name; uint64_t ptr, bytes; int gpu; };
    std::vector<Buf> bufs_;
    std::map<std::string, int> by_name_;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
// in: 16 values in the order of VramPlanIn (doubles carry the integers exactly up to 2^53);
// out: offset[10], size[10], kv_spec_pages, stable_slots, streaming_slots.  Returns -1 when ok, else the failed region.
LSB_RT_API int lsb_vram_plan(const double* in, long long* out) {
    VramPlanIn p;
    p.total_bytes = (int64_t)in[0]; p.weights_bytes = (int64_t)in[1]; p.workspace_bytes = (int64_t)in[2];
    p.kv_bytes_per_page = (int64_t)in[3]; p.kv_pages = (int64_t)in[4]; p.spec_pool_fraction = in[5];
    p.indexer_bytes_per_page = (int64_t)in[6]; p.indexer_pages = (int64_t)in[7]; p.prefill_scratch_bytes = (int64_t)in[8];
    p.recurrent_bytes_per_seq = (int64_t)in[9]; p.recurrent_seqs = (int64_t)in[10]; p.expert_slot_bytes = (int64_t)in[11];
    p.expert_slots_wanted = (int64_t)in[12]; p.stable_zone_fraction = in[13]; p.safety_bytes = (int64_t)in[14];
    VramPlanOut o;
    plan_vram(p, o);
    for (int r = 0; r < kRegCount; ++r) { out[r] = o.offset[r]; out[kRegCount + r] = o.size[r]; }
    out[2 * kRegCount] = o.kv_spec_pages; out[2 * kRegCount + 1] = o.expert_stable_slots; out[2 * kRegCount + 2] = o.expert_streaming_slots;
    return o.failed_region;
}

LSB_RT_API void* lsb_det_create() { return new Determinism(); }
LSB_RT_API void lsb_det_destroy(void* h) { delete (Determinism*)h; }
LSB_RT_API int lsb_det_set_flags(void* h, int deterministic, int identity, char* conflict, int cap) { return ((Determinism*)h)->set_flags(deterministic, identity, conflict, cap); }
LSB_RT_API int lsb_det_pin(void* h, const char* name, int value) { return ((Determinism*)h)->pin(name, value); }
LSB_RT_API int lsb_det_get(void* h, const char* name) { return ((Determinism*)h)->get(name); }
LSB_RT_API int lsb_det_count(void* h) { return ((Determinism*)h)->count(); }
LSB_RT_API const char* lsb_det_name_at(void* h, int i) { return ((Determinism*)h)->name_at(i); }

LSB_RT_API void* lsb_bufreg_create() { return new BufferRegistry(); }
LSB_RT_API void lsb_bufreg_destroy(void* h) { delete (BufferRegistry*)h; }
LSB_RT_API int lsb_bufreg_add(void* h, const char* name, unsigned long long ptr, unsigned long long bytes, int gpu) { return ((BufferRegistry*)h)->add(name, ptr, bytes, gpu); }
LSB_RT_API int lsb_bufreg_find(void* h, const char* name) { return ((BufferRegistry*)h)->find(name); }
LSB_RT_API int lsb_bufreg_get(void* h, int id, unsigned long long* ptr, unsigned long long* bytes, int* gpu) {
    uint64_t p = 0, b = 0;
    const int rc = ((BufferRegistry*)h)->get(id, &p, &b, gpu);
    *ptr = p; *bytes = b;
    return rc;
}
LSB_RT_API int lsb_bufreg_contains(void* h, int id, unsigned long long ptr, unsigned long long bytes) { return ((BufferRegistry*)h)->contains(id, ptr, bytes); }
LSB_RT_API int lsb_bufreg_count(void* h) { return ((BufferRegistry*)h)->count(); }
}
