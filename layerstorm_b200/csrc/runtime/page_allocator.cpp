// Paged KV-cache bookkeeping: page pools, per-sequence block tables, reference-counted
// sharing with copy-on-write on the frontier page, truncating forks, rewind, promotion between
// pools, headroom reservation, context-parallel token->rank routing and lending of free page
// runs to the expert cache.  Pure metadata: the caller owns device memory and performs the
// copies this allocator asks for.
//
// Reference component: PageAllocator (src/core/memory/page_allocator.h:28,98-460): pools
// kMain/kSpeculation/kIndexerK/kHca/kSwa/kKdaState, refcount CoW (cow_copy), metadata-only
// promote, headroom, dcp_rank_for_token, claim/release_expert_zone.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

struct PagePool {
    int n_pages = 0;
    std::vector<int> refcnt;        // 0 = free, -1 = lent to the expert cache
    std::vector<int> free_list;     // LIFO of free page ids
    int headroom = 0;               // pages only `privileged` allocations may take
    int lent = 0;
};

struct Seq {
    int pool = 0;
    int length = 0;                 // committed tokens
    int reserved_pages = 0;         // pre-reserved beyond the pages in use
    bool frozen = false;            // frozen holders never append
    std::vector<int> pages;
};

class PageAllocator {
public:
    PageAllocator(int n_pools, const int* pages_per_pool, int page_tokens) : page_tokens_(page_tokens) {
        pools_.resize(n_pools);
        for (int p = 0; p < n_pools; ++p) {
            auto& pl = pools_[p];
            pl.n_pages = pages_per_pool[p];
            pl.refcnt.assign(pl.n_pages, 0);
            pl.free_list.resize(pl.n_pages);
            for (int i = 0; i < pl.n_pages; ++i) pl.free_list[i] = pl.n_pages - 1 - i;   // pop gives 0,1,2,...
        }
    }

    int page_tokens() const { return page_tokens_; }

    int free_pages(int pool) const { return (int)pools_[pool].free_list.size(); }
    int total_pages(int pool) const { return pools_[pool].n_pages; }
    int lent_pages(int pool) const { return pools_[pool].lent; }
    void set_headroom(int pool, int pages) { pools_[pool].headroom = pages; }

    int create(int seq, int pool, int reserve_tokens) {
        if (seqs_.count(seq)) return LSB_ERR_EXISTS;
        if (pool < 0 || pool >= (int)pools_.size()) return LSB_ERR_ARG;
        Seq s;
        s.pool = pool;
        int need = pages_for(reserve_tokens);
        if (need > available(pool, false)) return LSB_ERR_POOL_EXHAUSTED;
        for (int i = 0; i < need; ++i) s.pages.push_back(take(pool));
        s.reserved_pages = need;
        seqs_[seq] = std::move(s);
        return 0;
    }

    // Extend the sequence to new_len tokens; newly attached pages are appended to new_pages.
    int extend(int seq, int new_len, bool privileged, std::vector<int>* new_pages) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        Seq& s = it->second;
        if (s.frozen) return LSB_ERR_FROZEN;
        if (new_len < s.length) return LSB_ERR_ARG;
        int need = pages_for(new_len) - (int)s.pages.size();
        if (need > 0) {
            if (need > available(s.pool, privileged)) return LSB_ERR_POOL_EXHAUSTED;
            for (int i = 0; i < need; ++i) {
                int pg = take(s.pool);
                s.pages.push_back(pg);
                if (new_pages) new_pages->push_back(pg);
            }
        }
        s.length = new_len;
        return 0;
    }

    // The frontier page must be private before an append touches it.  Returns 1 and fills
    // (src,dst) when a copy is required, 0 when not, <0 on error.
    int cow_frontier(int seq, int* src, int* dst) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        Seq& s = it->second;
        if (s.length % page_tokens_ == 0 || s.pages.empty()) return 0;
        int idx = s.length / page_tokens_;
        if (idx >= (int)s.pages.size()) return 0;
        auto& pl = pools_[s.pool];
        int pg = s.pages[idx];
        if (pl.refcnt[pg] <= 1) return 0;
        if (available(s.pool, true) < 1) return LSB_ERR_POOL_EXHAUSTED;
        int np = take(s.pool);
        pl.refcnt[pg] -= 1;
        s.pages[idx] = np;
        *src = pg; *dst = np;
        return 1;
    }

    // Truncating fork: the child shares pages covering [0, prefix_len).  A frozen child is a
    // holder that never appends (no frontier split is ever needed for it).
    int fork(int parent, int child, int prefix_len, bool frozen) {
        auto it = seqs_.find(parent);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        if (seqs_.count(child)) return LSB_ERR_EXISTS;
        const Seq& p = it->second;
        if (prefix_len < 0 || prefix_len > p.length) return LSB_ERR_ARG;
        Seq c;
        c.pool = p.pool;
        c.length = prefix_len;
        c.frozen = frozen;
        int n = pages_for(prefix_len);
        auto& pl = pools_[p.pool];
        for (int i = 0; i < n; ++i)
            if (p.pages[i] < 0) return LSB_ERR_ARG;         // swapped-out pages cannot be shared: promote them first
        for (int i = 0; i < n; ++i) { c.pages.push_back(p.pages[i]); pl.refcnt[p.pages[i]] += 1; }
        seqs_[child] = std::move(c);
        return 0;
    }

    int rewind(int seq, int new_len) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        Seq& s = it->second;
        if (new_len > s.length || new_len < 0) return LSB_ERR_ARG;
        int keep = std::max(pages_for(new_len), s.reserved_pages);
        while ((int)s.pages.size() > keep) { release(s.pool, s.pages.back()); s.pages.pop_back(); }
        s.length = new_len;
        return 0;
    }

    int destroy(int seq) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        for (int pg : it->second.pages) release(it->second.pool, pg);
        seqs_.erase(it);
        return 0;
    }

    // KV tiering of an ACTIVE sequence: logical page `idx` gives its HBM page back to the pool (its rows live in the cold tier
    // from now on; the block-table entry becomes -1), and takes a fresh HBM page again when it is promoted.  Only private,
    // completely filled pages behind the frontier may be swapped out.  Returns the released / newly attached physical page.
    int swap_out(int seq, int idx) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        Seq& s = it->second;
        if (idx < 0 || idx >= (int)s.pages.size() || (idx + 1) * page_tokens_ > s.length) return LSB_ERR_ARG;
        const int pg = s.pages[idx];
        if (pg < 0) return LSB_ERR_ARG;
        if (pools_[s.pool].refcnt[pg] != 1) return LSB_ERR_SHARED;
        release(s.pool, pg);
        s.pages[idx] = -1;
        return pg;
    }
    int swap_in(int seq, int idx) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        Seq& s = it->second;
        if (idx < 0 || idx >= (int)s.pages.size() || s.pages[idx] >= 0) return LSB_ERR_ARG;
        if (available(s.pool, true) < 1) return LSB_ERR_POOL_EXHAUSTED;
        s.pages[idx] = take(s.pool);
        return s.pages[idx];
    }

    // Metadata-only move of a sequence's accounting to another pool of the same geometry (the
    // speculation pool's accepted tokens become main-pool tokens).  Pools must share storage.
    int promote(int seq, int to_pool) {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return LSB_ERR_NOT_FOUND;
        Seq& s = it->second;
        if (to_pool == s.pool) return 0;
        auto& from = pools_[s.pool];
        auto& to = pools_[to_pool];
        if ((int)s.pages.size() > available(to_pool, true)) return LSB_ERR_POOL_EXHAUSTED;
        for (auto& pg : s.pages) {
            if (pg < 0) return LSB_ERR_ARG;
            if (from.refcnt[pg] != 1) return LSB_ERR_SHARED;
        }
        for (auto& pg : s.pages) {
            release(s.pool, pg);
            pg = take(to_pool);
        }
        s.pool = to_pool;
        (void)to;
        return 0;
    }

    int length(int seq) const { auto it = seqs_.find(seq); return it == seqs_.end() ? -1 : it->second.length; }
    int n_pages(int seq) const { auto it = seqs_.find(seq); return it == seqs_.end() ? -1 : (int)it->second.pages.size(); }
    int copy_pages(int seq, int* out, int cap) const {
        auto it = seqs_.find(seq);
        if (it == seqs_.end()) return -1;
        int n = std::min(cap, (int)it->second.pages.size());
        std::memcpy(out, it->second.pages.data(), n * sizeof(int));
        return n;
    }
    int refcount(int pool, int page) const { return pools_[pool].refcnt[page]; }

    // Lend a run of `n` consecutive free pages to the expert cache (elastic zone).  Returns the
    // first page id or -1.  Lent pages are invisible to sequences until released.
    int claim_zone(int pool, int n) {
        auto& pl = pools_[pool];
        if (n <= 0 || (int)pl.free_list.size() - pl.headroom < n) return -1;
        int run = 0;
        for (int i = 0; i < pl.n_pages; ++i) {
            run = pl.refcnt[i] == 0 ? run + 1 : 0;
            if (run == n) {
                int start = i - n + 1;
                for (int j = start; j <= i; ++j) pl.refcnt[j] = -1;
                pl.free_list.erase(std::remove_if(pl.free_list.begin(), pl.free_list.end(), [&](int p) { return p >= start && p <= i; }), pl.free_list.end());
                pl.lent += n;
                return start;
            }
        }
        return -1;
    }
    int release_zone(int pool, int start, int n) {
        auto& pl = pools_[pool];
        for (int j = start; j < start + n; ++j) if (j < 0 || j >= pl.n_pages || pl.refcnt[j] != -1) return LSB_ERR_ARG;
        for (int j = start + n - 1; j >= start; --j) { pl.refcnt[j] = 0; pl.free_list.push_back(j); }
        pl.lent -= n;
        return 0;
    }

private:
    int pages_for(int tokens) const { return (tokens + page_tokens_ - 1) / page_tokens_; }
    int available(int pool, bool privileged) const {
        const auto& pl = pools_[pool];
        int a = (int)pl.free_list.size();
        return privileged ? a : std::max(0, a - pl.headroom);
    }
    int take(int pool) {
        auto& pl = pools_[pool];
        int pg = pl.free_list.back();
        pl.free_list.pop_back();
        pl.refcnt[pg] = 1;
        return pg;
    }
    void release(int pool, int pg) {
        if (pg < 0) return;                 // a swapped-out page holds no HBM
        auto& pl = pools_[pool];
        if (--pl.refcnt[pg] == 0) pl.free_list.push_back(pg);
    }

    int page_tokens_;
    std::vector<PagePool> pools_;
    std::unordered_map<int, Seq> seqs_;
};

}  // namespace lsb

using lsb::PageAllocator;

extern "C" {

LSB_RT_API void* lsb_pa_create(int n_pools, const int* pages_per_pool, int page_tokens) { return new PageAllocator(n_pools, pages_per_pool, page_tokens); }
LSB_RT_API void lsb_pa_destroy(void* h) { delete (PageAllocator*)h; }
LSB_RT_API int lsb_pa_free_pages(void* h, int pool) { return ((PageAllocator*)h)->free_pages(pool); }
LSB_RT_API int lsb_pa_total_pages(void* h, int pool) { return ((PageAllocator*)h)->total_pages(pool); }
LSB_RT_API int lsb_pa_lent_pages(void* h, int pool) { return ((PageAllocator*)h)->lent_pages(pool); }
LSB_RT_API void lsb_pa_set_headroom(void* h, int pool, int pages) { ((PageAllocator*)h)->set_headroom(pool, pages); }
LSB_RT_API int lsb_pa_seq_create(void* h, int seq, int pool, int reserve_tokens) { return ((PageAllocator*)h)->create(seq, pool, reserve_tokens); }
LSB_RT_API int lsb_pa_seq_extend(void* h, int seq, int new_len, int privileged, int* new_pages, int cap, int* n_new) {
    std::vector<int> np;
    int rc = ((PageAllocator*)h)->extend(seq, new_len, privileged != 0, &np);
    if (n_new) *n_new = (int)np.size();
    for (int i = 0; i < (int)np.size() && i < cap; ++i) new_pages[i] = np[i];
    return rc;
}
LSB_RT_API int lsb_pa_cow_frontier(void* h, int seq, int* src, int* dst) { return ((PageAllocator*)h)->cow_frontier(seq, src, dst); }
LSB_RT_API int lsb_pa_fork(void* h, int parent, int child, int prefix_len, int frozen) { return ((PageAllocator*)h)->fork(parent, child, prefix_len, frozen != 0); }
LSB_RT_API int lsb_pa_rewind(void* h, int seq, int new_len) { return ((PageAllocator*)h)->rewind(seq, new_len); }
LSB_RT_API int lsb_pa_seq_destroy(void* h, int seq) { return ((PageAllocator*)h)->destroy(seq); }
LSB_RT_API int lsb_pa_promote(void* h, int seq, int to_pool) { return ((PageAllocator*)h)->promote(seq, to_pool); }
LSB_RT_API int lsb_pa_swap_out(void* h, int seq, int idx) { return ((PageAllocator*)h)->swap_out(seq, idx); }
LSB_RT_API int lsb_pa_swap_in(void* h, int seq, int idx) { return ((PageAllocator*)h)->swap_in(seq, idx); }
LSB_RT_API int lsb_pa_seq_length(void* h, int seq) { return ((PageAllocator*)h)->length(seq); }
LSB_RT_API int lsb_pa_seq_pages(void* h, int seq, int* out, int cap) { return ((PageAllocator*)h)->copy_pages(seq, out, cap); }
LSB_RT_API int lsb_pa_refcount(void* h, int pool, int page) { return ((PageAllocator*)h)->refcount(pool, page); }
LSB_RT_API int lsb_pa_claim_zone(void* h, int pool, int n) { return ((PageAllocator*)h)->claim_zone(pool, n); }
LSB_RT_API int lsb_pa_release_zone(void* h, int pool, int start, int n) { return ((PageAllocator*)h)->release_zone(pool, start, n); }
// Context-parallel routing: KV pages are dealt round-robin by chunk over the ranks
// (reference: dcp_rank_for_token, src/daemon/kv_shard_math.h).
LSB_RT_API int lsb_dcp_rank_for_token(long long token, int chunk_tokens, int ranks) { return (int)((token / chunk_tokens) % ranks); }
LSB_RT_API long long lsb_dcp_local_index(long long token, int chunk_tokens, int ranks) {
    long long chunk = token / chunk_tokens;
    return (chunk / ranks) * chunk_tokens + token % chunk_tokens;
}

}  // extern "C"
