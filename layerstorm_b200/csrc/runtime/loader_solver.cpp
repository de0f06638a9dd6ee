// Expert placement solver: for one (token batch, layer) decide on which device each routed expert
// runs, minimising the modelled step time
//     T = max( max_m device_time(m), max_bank egress(bank) ) + recon + evictions
//     device_time(m) = max(fetch(m), compute(resident on m)) + compute(fetched to m)
//     compute(m, c)  = a_m * c + b_m * ceil(c / P)            (calibrated grouped-GEMM curve)
//     fetch(m)       = sum over experts fetched to m of (latency + bytes / rate(bank(e), m))
// All arithmetic is integer nanoseconds, so the result is deterministic.  Three tiers, chosen by
// problem size: exact enumeration (M^N <= 2^22), subset dynamic programme O(M * 3^N) over the
// per-device part of the objective followed by a full re-evaluation, and greedy longest-
// processing-time placement; the best candidate under the full objective is returned.
// Reference component: LoaderSolver (src/core/gpu_loader/loader_solver.h:93-165, math in
// the reference's design document under docs/, lines 305-413): same objective shape and tiering, re-derived for NVLink-class devices.
#include <algorithm>
#include <climits>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

struct SolverConstants {
    int n_devices = 1, n_banks = 1;
    int batch_p = 64;                       // experts per grouped-GEMM batch
    std::vector<int64_t> a_ns, b_ns;        // per device compute curve
    std::vector<int64_t> rate_bpus;         // [bank][device] bytes per microsecond (0 = unreachable)
    std::vector<int64_t> lat_ns;            // [bank][device]
    std::vector<int64_t> egress_bpus;       // [bank]
    int64_t recon_ns = 0;                   // cross-device combine when more than one device is used
    int64_t evict_ns = 0;                   // per eviction needed to make room
};

struct SolveRequest {
    int n = 0;
    const int* bank;            // [n] host bank holding expert i
    const int64_t* bytes;       // [n]
    const uint8_t* resident;    // [n][M] 1 = already in device m's cache
    const int* free_slots;      // [M] free cache slots per device
};

class LoaderSolver {
public:
    explicit LoaderSolver(const SolverConstants& c) : c_(c) {}

    int64_t compute_ns(int m, int cnt) const {
        if (cnt <= 0) return 0;
        return c_.a_ns[m] * cnt + c_.b_ns[m] * ((cnt + c_.batch_p - 1) / c_.batch_p);
    }
    int64_t fetch_ns(const SolveRequest& r, int e, int m) const {
        if (r.resident[(size_t)e * c_.n_devices + m]) return 0;
        const int bk = r.bank[e];
        const int64_t rate = c_.rate_bpus[(size_t)bk * c_.n_devices + m];
        if (rate <= 0) return INT64_MAX / 4;
        return c_.lat_ns[(size_t)bk * c_.n_devices + m] + r.bytes[e] * 1000 / rate;
    }
    int64_t device_time(const SolveRequest& r, int m, const std::vector<int>& assign) const {
        int64_t f = 0; int res = 0, fet = 0;
        for (int e = 0; e < r.n; ++e) {
            if (assign[e] != m) continue;
            if (r.resident[(size_t)e * c_.n_devices + m]) ++res;
            else { ++fet; f += fetch_ns(r, e, m); }
        }
        return std::max(f, compute_ns(m, res)) + compute_ns(m, fet);
    }
    int64_t evaluate(const SolveRequest& r, const std::vector<int>& assign) const {
        const int M = c_.n_devices;
        int64_t worst = 0, evict = 0;
        std::vector<int64_t> egress(c_.n_banks, 0);
        std::vector<int> fetched(M, 0);
        int used = 0;
        for (int m = 0; m < M; ++m) {
            bool any = false;
            for (int e = 0; e < r.n; ++e) if (assign[e] == m) {
                any = true;
                if (!r.resident[(size_t)e * M + m]) { ++fetched[m]; egress[r.bank[e]] += r.bytes[e] * 1000 / std::max<int64_t>(1, c_.egress_bpus[r.bank[e]]); }
            }
            if (any) { ++used; worst = std::max(worst, device_time(r, m, assign)); }
            if (fetched[m] > r.free_slots[m]) evict += (int64_t)(fetched[m] - r.free_slots[m]) * c_.evict_ns;
        }
        for (int b = 0; b < c_.n_banks; ++b) worst = std::max(worst, egress[b]);
        return worst + (used > 1 ? c_.recon_ns : 0) + evict;
    }

    // tier: 0 auto, 1 exact, 2 dp, 3 greedy.  Returns the tier used; *cost = objective.
    int solve(const SolveRequest& r, int tier, int* out_assign, int64_t* cost) const {
        const int M = c_.n_devices, N = r.n;
        std::vector<int> best(N, 0);
        int64_t bc = INT64_MAX;
        int used = tier;
        if (tier == 0) {
            double combos = 1;
            for (int i = 0; i < N && combos <= (double)(1 << 22); ++i) combos *= M;
            used = combos <= (double)(1 << 22) ? 1 : (N <= 14 ? 2 : 3);
        }
        auto consider = [&](const std::vector<int>& a) { const int64_t v = evaluate(r, a); if (v < bc) { bc = v; best = a; } };
        if (used == 1) {
            std::vector<int> a(N, 0);
            while (true) {
                consider(a);
                int i = 0;
                while (i < N && ++a[i] == M) a[i++] = 0;
                if (i == N) break;
            }
        } else {
            consider(greedy(r));
            if (used == 2) consider(subset_dp(r));
        }
        std::copy(best.begin(), best.end(), out_assign);
        *cost = bc;
        return used;
    }

private:
    std::vector<int> greedy(const SolveRequest& r) const {
        const int M = c_.n_devices, N = r.n;
        std::vector<int> order(N), a(N, -1);
        std::iota(order.begin(), order.end(), 0);
        // hardest first: experts resident nowhere and large go first
        auto weight = [&](int e) { int64_t w = INT64_MAX; for (int m = 0; m < M; ++m) w = std::min(w, fetch_ns(r, e, m)); return w; };
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return weight(x) > weight(y); });
        for (int e : order) {
            int bm = 0; int64_t bv = INT64_MAX;
            for (int m = 0; m < M; ++m) {
                a[e] = m;
                std::vector<int> tmp = a;
                for (auto& t : tmp) if (t < 0) t = -1;
                // evaluate only over experts placed so far
                SolveRequest sub = r;
                const int64_t v = evaluate_partial(sub, tmp);
                if (v < bv) { bv = v; bm = m; }
            }
            a[e] = bm;
        }
        return a;
    }
    int64_t evaluate_partial(const SolveRequest& r, const std::vector<int>& assign) const {
        // unplaced experts carry -1 and are ignored by the == m tests of evaluate()
        return evaluate(r, assign);
    }
    std::vector<int> subset_dp(const SolveRequest& r) const {
        const int M = c_.n_devices, N = r.n;
        const uint32_t full = (1u << N) - 1;
        std::vector<int64_t> tm((size_t)M << N);
        std::vector<int> a(N, -1);
        for (int m = 0; m < M; ++m)
            for (uint32_t s = 0; s <= full; ++s) {
                for (int e = 0; e < N; ++e) a[e] = (s >> e & 1) ? m : -1;
                tm[((size_t)m << N) + s] = s ? device_time(r, m, a) : 0;
            }
        std::vector<int64_t> dp((size_t)(M + 1) << N, INT64_MAX);
        std::vector<uint32_t> choice((size_t)(M + 1) << N, 0);
        dp[0] = 0;
        for (int m = 0; m < M; ++m)
            for (uint32_t mask = 0; mask <= full; ++mask) {
                int64_t bv = INT64_MAX; uint32_t bs = 0;
                for (uint32_t sub = mask;; sub = (sub - 1) & mask) {
                    const int64_t prev = dp[((size_t)m << N) + (mask ^ sub)];
                    if (prev != INT64_MAX) {
                        const int64_t v = std::max(prev, tm[((size_t)m << N) + sub]);
                        if (v < bv) { bv = v; bs = sub; }
                    }
                    if (sub == 0) break;
                }
                dp[((size_t)(m + 1) << N) + mask] = bv;
                choice[((size_t)(m + 1) << N) + mask] = bs;
            }
        std::vector<int> out(N, 0);
        uint32_t mask = full;
        for (int m = M; m >= 1; --m) {
            const uint32_t s = choice[((size_t)m << N) + mask];
            for (int e = 0; e < N; ++e) if (s >> e & 1) out[e] = m - 1;
            mask ^= s;
        }
        return out;
    }
    SolverConstants c_;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
// a_ns/b_ns: [M]; rate_bpus/lat_ns: [banks][M]; egress_bpus: [banks]
LSB_RT_API void* lsb_solver_create(int n_devices, int n_banks, int batch_p, const long long* a_ns, const long long* b_ns,
                                   const long long* rate_bpus, const long long* lat_ns, const long long* egress_bpus,
                                   long long recon_ns, long long evict_ns) {
    SolverConstants c;
    c.n_devices = n_devices; c.n_banks = n_banks; c.batch_p = batch_p > 0 ? batch_p : 64;
    c.a_ns.assign(a_ns, a_ns + n_devices); c.b_ns.assign(b_ns, b_ns + n_devices);
    c.rate_bpus.assign(rate_bpus, rate_bpus + (size_t)n_banks * n_devices);
    c.lat_ns.assign(lat_ns, lat_ns + (size_t)n_banks * n_devices);
    c.egress_bpus.assign(egress_bpus, egress_bpus + n_banks);
    c.recon_ns = recon_ns; c.evict_ns = evict_ns;
    return new LoaderSolver(c);
}
LSB_RT_API void lsb_solver_destroy(void* h) { delete (LoaderSolver*)h; }
LSB_RT_API int lsb_solver_solve(void* h, int n, const int* bank, const long long* bytes, const unsigned char* resident, const int* free_slots,
                                int tier, int* out_assign, long long* cost) {
    if (n <= 0 || n > 24) return LSB_ERR_ARG;
    SolveRequest r;
    std::vector<int64_t> by(bytes, bytes + n);
    r.n = n; r.bank = bank; r.bytes = by.data(); r.resident = resident; r.free_slots = free_slots;
    int64_t c = 0;
    const int used = ((LoaderSolver*)h)->solve(r, tier, out_assign, &c);
    *cost = c;
    return used;
}
LSB_RT_API long long lsb_solver_evaluate(void* h, int n, const int* bank, const long long* bytes, const unsigned char* resident,
                                         const int* free_slots, const int* assign) {
    SolveRequest r;
    std::vector<int64_t> by(bytes, bytes + n);
    r.n = n; r.bank = bank; r.bytes = by.data(); r.resident = resident; r.free_slots = free_slots;
    return ((LoaderSolver*)h)->evaluate(r, std::vector<int>(assign, assign + n));
}
}
