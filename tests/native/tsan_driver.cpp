// ThreadSanitizer driver for the host-runtime components that are touched by two threads by design: the SPSC ring (one producer, one
// consumer), the seqlock state snapshot (one writer, any readers), the NVMe tier (caller + its worker pool) and the host arena (loaders).  Linked against the
// runtime sources compiled with -fsanitize=thread; exits 0 when the functional checks hold (TSAN reports make the process exit 66).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* lsb_ring_create(unsigned int slots, unsigned int slot_bytes);
void lsb_ring_destroy(void* h);
int lsb_ring_push(void* h, const void* data, unsigned int n);
int lsb_ring_pop(void* h, void* out);
void* lsb_snap_create(unsigned int bytes);
void lsb_snap_destroy(void* h);
void lsb_snap_begin(void* h);
void lsb_snap_write(void* h, unsigned int off, const void* src, unsigned int n);
void lsb_snap_end(void* h);
unsigned long long lsb_snap_read(void* h, void* out, unsigned int off, unsigned int n, int tries);
void* lsb_nvme_create(const char* drives, long long capacity_bytes, int queue_depth, int direct_io, int workers);
void lsb_nvme_destroy(void* h);
int lsb_nvme_write(void* h, int layer, int expert, const void* src, long long bytes);
unsigned long long lsb_nvme_read_async(void* h, int layer, int expert, void* dst, long long bytes);
int lsb_nvme_poll(void* h, unsigned long long* tokens, int* status, int cap);
int lsb_nvme_pending(void* h);
void* lsb_arena_create(long long slot_bytes, int n_slots, int numa_node, int use_memfd, int thp);
void lsb_arena_destroy(void* h);
void* lsb_arena_base(void* h);
int lsb_arena_lookup(void* h, int layer, int expert);
int lsb_arena_begin_load(void* h, int layer, int expert, int* ev_layer, int* ev_expert);
int lsb_arena_finish_load(void* h, int slot, int success);
int lsb_arena_ref(void* h, int slot, int delta);
void lsb_arena_stats(void* h, unsigned long long* hits, unsigned long long* misses, unsigned long long* evictions, int* active);
void* lsb_cpu_pool_create(int threads, const int* cpus, int n_cpus);
void lsb_cpu_pool_destroy(void* h);
int lsb_cpu_expert_ffn(void* pool, const void* fmt_struct, const void* slot, const float* x, int n, float limit, const float* scale, float* y,
                       int accumulate);
}

static int check(bool ok, const char* what) {
    if (!ok) { printf("FAIL %s\n", what); return 1; }
    return 0;
}

int main(int argc, char** argv) {
    int bad = 0;
    // 1. ring: 200k messages, every one arrives once and in order
    {
        void* r = lsb_ring_create(64, 16);
        const int N = 200000;
        std::thread prod([&] {
            for (int i = 0; i < N;) {
                uint64_t m[2] = {(uint64_t)i, (uint64_t)i * 3};
                if (lsb_ring_push(r, m, 16)) ++i; else std::this_thread::yield();
            }
        });
        int got = 0; bool order = true;
        while (got < N) {
            uint64_t m[2];
            if (lsb_ring_pop(r, m)) { order &= m[0] == (uint64_t)got && m[1] == (uint64_t)got * 3; ++got; } else std::this_thread::yield();
        }
        prod.join();
        bad += check(order, "ring order");
        lsb_ring_destroy(r);
    }
    // 2. seqlock snapshot: the reader never sees a torn record
    {
        void* s = lsb_snap_create(256);
        std::atomic<bool> stop{false};
        std::thread wr([&] {
            for (uint64_t v = 1; v <= 50000; ++v) {
                uint64_t rec[32];
                for (auto& x : rec) x = v;
                lsb_snap_begin(s); lsb_snap_write(s, 0, rec, sizeof(rec)); lsb_snap_end(s);
            }
            stop = true;
        });
        bool torn = false; uint64_t reads = 0;
        while (!stop) {
            uint64_t rec[32];
            if (lsb_snap_read(s, rec, 0, sizeof(rec), 64)) {
                ++reads;
                for (int i = 1; i < 32; ++i) torn |= rec[i] != rec[0];
            }
        }
        wr.join();
        bad += check(!torn && reads > 0, "snapshot consistency");
        lsb_snap_destroy(s);
    }
    // 3. NVMe tier: asynchronous reads served by the worker pool while the caller polls
    {
        std::string dir = argc > 1 ? argv[1] : "/tmp";
        void* t = lsb_nvme_create(dir.c_str(), 1LL << 30, 8, 0, 3);
        bad += check(t != nullptr, "nvme create");
        if (t) {
            const long long B = 64 * 1024;
            std::vector<std::vector<unsigned char>> src(12, std::vector<unsigned char>(B)), dst(12, std::vector<unsigned char>(B));
            for (int e = 0; e < 12; ++e) {
                for (long long i = 0; i < B; ++i) src[e][i] = (unsigned char)(e * 31 + i);
                bad += check(lsb_nvme_write(t, 0, e, src[e].data(), B) >= 0, "nvme write");
            }
            int done = 0, okc = 0, next = 0;
            for (int spin = 0; done < 12 && spin < 2000000; ++spin) {
                while (next < 12 && lsb_nvme_read_async(t, 0, next, dst[next].data(), B) != 0) ++next;      // 0 = queue full: poll first
                unsigned long long tok[16]; int st[16];
                int n = lsb_nvme_poll(t, tok, st, 16);
                for (int i = 0; i < n; ++i) { ++done; okc += st[i] == 0; }
                if (!n) std::this_thread::yield();
            }
            bad += check(done == 12 && okc == 12 && lsb_nvme_pending(t) == 0, "nvme completions");
            bool same = true;
            for (int e = 0; e < 12; ++e) same &= src[e] == dst[e];
            bad += check(same, "nvme data");
            lsb_nvme_destroy(t);
        }
    }
    // 4. host arena: four loader threads claim, fill and publish slots of a small arena (evicting each other's unreferenced experts)
    {
        const long long B = 4096;
        void* a = lsb_arena_create(B, 8, -1, 0, 0);
        bad += check(a != nullptr, "arena create");
        if (a) {
            std::atomic<int> loads{0}, wrong{0};
            auto worker = [&](int id) {
                unsigned char* base = (unsigned char*)lsb_arena_base(a);
                for (int it = 0; it < 400; ++it) {
                    const int layer = id & 1, expert = (it * 7 + id * 3) % 24;
                    int slot = lsb_arena_lookup(a, layer, expert);
                    if (slot >= 0 && lsb_arena_ref(a, slot, +1) >= 0) {
                        // (lookup and ref are two calls: the slot may have been re-used in between; the tag written below tells)
                        const unsigned char tag = base[(long long)slot * B];
                        if (lsb_arena_lookup(a, layer, expert) == slot) wrong += tag != (unsigned char)(layer * 24 + expert);
                        lsb_arena_ref(a, slot, -1);
                        continue;
                    }
                    int evl = -1, eve = -1;
                    slot = lsb_arena_begin_load(a, layer, expert, &evl, &eve);
                    if (slot < 0) continue;                                   // being loaded by another thread, or nothing evictable
                    std::memset(base + (long long)slot * B, layer * 24 + expert, B);
                    lsb_arena_finish_load(a, slot, 1);
                    ++loads;
                }
            };
            std::vector<std::thread> th;
            for (int i = 0; i < 4; ++i) th.emplace_back(worker, i);
            for (auto& t : th) t.join();
            unsigned long long hits = 0, misses = 0, ev = 0; int active = 0;
            lsb_arena_stats(a, &hits, &misses, &ev, &active);
            bad += check(loads > 0 && wrong == 0 && active <= 8, "arena consistency");
            lsb_arena_destroy(a);
        }
    }
    // 5. CPU expert kernels: the fork-join pool runs an expert FFN (bf16 slot image) over several tokens; compared with a serial evaluation
    {
        struct Raw { int fmt, H, F; long long stride, og, ou, od, sg, su, sd, tail; };
        const int H = 64, F = 96, n = 5;
        Raw f{0, H, F, (long long)3 * H * F * 2, 0, (long long)H * F * 2, (long long)2 * H * F * 2, 0, 0, 0, 0};
        std::vector<uint16_t> slot((size_t)3 * H * F);
        auto bf = [](float v) { uint32_t u; std::memcpy(&u, &v, 4); return (uint16_t)((u + 0x7FFF + ((u >> 16) & 1)) >> 16); };
        auto fb = [](uint16_t b) { uint32_t u = (uint32_t)b << 16; float v; std::memcpy(&v, &u, 4); return v; };
        uint32_t seed = 12345;
        auto rnd = [&] { seed = seed * 1664525u + 1013904223u; return ((seed >> 8) & 0xFFFF) / 65536.f - 0.5f; };
        for (auto& w : slot) w = bf(0.2f * rnd());
        std::vector<float> x((size_t)n * H), y((size_t)n * H, 0.f), ref((size_t)n * H, 0.f);
        for (auto& v : x) v = rnd();
        void* pool = lsb_cpu_pool_create(4, nullptr, 0);
        bad += check(pool && lsb_cpu_expert_ffn(pool, &f, slot.data(), x.data(), n, 0.f, nullptr, y.data(), 0) == 0, "cpu expert ffn");
        for (int t = 0; t < n; ++t) {
            std::vector<float> act(F);
            for (int j = 0; j < F; ++j) {
                float g = 0, u = 0;
                for (int k = 0; k < H; ++k) { g += fb(slot[(size_t)j * H + k]) * x[(size_t)t * H + k]; u += fb(slot[(size_t)H * F + (size_t)j * H + k]) * x[(size_t)t * H + k]; }
                act[j] = g / (1.f + expf(-g)) * u;
            }
            for (int o = 0; o < H; ++o) {
                float acc = 0;
                for (int j = 0; j < F; ++j) acc += fb(slot[(size_t)2 * H * F + (size_t)o * F + j]) * act[j];
                ref[(size_t)t * H + o] = acc;
            }
        }
        float err = 0, mx = 0;
        for (size_t i = 0; i < ref.size(); ++i) { err = std::max(err, std::fabs(ref[i] - y[i])); mx = std::max(mx, std::fabs(ref[i])); }
        bad += check(mx > 0 && err < 1e-3f * mx + 1e-6f, "cpu expert ffn values");
        if (pool) lsb_cpu_pool_destroy(pool);
    }
    printf(bad ? "TSAN_DRIVER_FAIL\n" : "TSAN_DRIVER_OK\n");
    return bad ? 1 : 0;
}
