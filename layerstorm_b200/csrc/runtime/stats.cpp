// Runtime statistics used by cache / placement policy and by speculation control:
//   ExpertStats        per-expert EWMA activation frequency, recency, mean routing weight and lag-1
//                      autocorrelation of activation (eviction scoring inputs)
//   CoactivationGraph  decayed pair counts of experts activated by the same token + greedy
//                      partition hints (which experts to co-locate)
//   WorkloadDetector   detects a shift of the expert-activation distribution (L2 distance of
//                      windowed frequency vectors against a Welford running mean / variance)
//   AcceptanceTracker  speculative-decoding acceptance: global, windowed and per-request EMAs
// Reference components: src/core/statistics/{expert_stats,coactivation_graph,workload_detector,
// acceptance_tracker}.{h,cpp}.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <numeric>
#include <unordered_map>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

class ExpertStats {
public:
    ExpertStats(int n, float alpha) : n_(n), alpha_(alpha), freq_(n, 0.f), weight_(n, 0.f), autocorr_(n, 0.f), last_(n, 0), prev_active_(n, 0) {}
    // One routing step: the set of activated experts with their routing weights.
    void observe(const int* ids, const float* w, int k) {
        ++tick_;
        std::vector<uint8_t> act(n_, 0);
        for (int i = 0; i < k; ++i) {
            const int e = ids[i];
            if (e < 0 || e >= n_) continue;
            act[e] = 1;
            weight_[e] += alpha_ * ((w ? w[i] : 1.f) - weight_[e]);
            last_[e] = tick_;
        }
        for (int e = 0; e < n_; ++e) {
            freq_[e] += alpha_ * ((float)act[e] - freq_[e]);
            const float both = (act[e] && prev_active_[e]) ? 1.f : 0.f;
            autocorr_[e] += alpha_ * (both - autocorr_[e]);
            prev_active_[e] = act[e];
        }
    }
    float frequency(int e) const { return freq_[e]; }
    float mean_weight(int e) const { return weight_[e]; }
    float autocorr(int e) const { return autocorr_[e]; }
    float recency(int e) const { return last_[e] ? 1.f / (1.f + (float)(tick_ - last_[e])) : 0.f; }
    void frequencies(float* out) const { std::memcpy(out, freq_.data(), n_ * sizeof(float)); }
    int size() const { return n_; }
private:
    int n_; float alpha_; uint64_t tick_ = 0;
    std::vector<float> freq_, weight_, autocorr_;
    std::vector<uint64_t> last_;
    std::vector<uint8_t> prev_active_;
};

class CoactivationGraph {
public:
    CoactivationGraph(int n, float decay) : n_(n), decay_(decay), m_((size_t)n * n, 0.f) {}
    void observe(const int* ids, int k) {
        if (++since_decay_ >= 64) { for (auto& v : m_) v *= decay_; since_decay_ = 0; }
        for (int i = 0; i < k; ++i)
            for (int j = i + 1; j < k; ++j) {
                const int a = ids[i], b = ids[j];
                if (a < 0 || b < 0 || a >= n_ || b >= n_ || a == b) continue;
                m_[(size_t)a * n_ + b] += 1.f; m_[(size_t)b * n_ + a] += 1.f;
            }
    }
    float weight(int a, int b) const { return m_[(size_t)a * n_ + b]; }
    // Greedy balanced partition into `parts` groups: experts in descending total weight join the
    // group (with room) they are most co-activated with.  out[e] = group.
    void partition(int parts, int* out) const {
        std::vector<float> tot(n_, 0.f);
        for (int a = 0; a < n_; ++a) for (int b = 0; b < n_; ++b) tot[a] += m_[(size_t)a * n_ + b];
        std::vector<int> order(n_);
        std::iota(order.begin(), order.end(), 0);
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return tot[a] > tot[b]; });
        const int cap = (n_ + parts - 1) / parts;
        std::vector<int> size(parts, 0);
        std::fill(out, out + n_, -1);
        for (int e : order) {
            int best = -1; float bs = -1.f;
            for (int g = 0; g < parts; ++g) {
                if (size[g] >= cap) continue;
                float s = 0.f;
                for (int o = 0; o < n_; ++o) if (out[o] == g) s += m_[(size_t)e * n_ + o];
                // prefer affinity, then the emptier group
                if (best < 0 || s > bs || (s == bs && size[g] < size[best])) { best = g; bs = s; }
            }
            out[e] = best; size[best]++;
        }
    }
private:
    int n_; float decay_; int since_decay_ = 0;
    std::vector<float> m_;
};

class WorkloadDetector {
public:
    WorkloadDetector(int n, int window, float z_threshold) : n_(n), window_(window), z_(z_threshold), ref_(n, 0.f) {}
    // Feed one frequency vector per completed window; returns 1 when a shift is detected.
    int observe(const float* freq) {
        double d = 0;
        for (int i = 0; i < n_; ++i) { const double x = freq[i] - ref_[i]; d += x * x; }
        d = std::sqrt(d);
        int shift = 0;
        if (count_ >= 4) {
            const double sd = std::sqrt(m2_ / (count_ - 1));
            if (d > mean_ + z_ * std::max(sd, 1e-6)) shift = 1;
        }
        ++count_;
        const double delta = d - mean_;
        mean_ += delta / count_;
        m2_ += delta * (d - mean_);
        for (int i = 0; i < n_; ++i) ref_[i] += (freq[i] - ref_[i]) * 0.25f;
        if (shift) { count_ = 0; mean_ = 0; m2_ = 0; std::copy(freq, freq + n_, ref_.begin()); ++shifts_; }
        return shift;
    }
    int shifts() const { return shifts_; }
    int window() const { return window_; }
private:
    int n_, window_; float z_; std::vector<float> ref_;
    int64_t count_ = 0; double mean_ = 0, m2_ = 0; int shifts_ = 0;
};

class AcceptanceTracker {
public:
    AcceptanceTracker(float alpha, int window) : alpha_(alpha), window_(window) {}
    void record(int request, int proposed, int accepted) {
        if (proposed <= 0) return;
        const float r = (float)accepted / (float)proposed;
        ema_ = n_ ? ema_ + alpha_ * (r - ema_) : r;
        ++n_;
        tot_prop_ += proposed; tot_acc_ += accepted;
        win_.push_back({proposed, accepted});
        if ((int)win_.size() > window_) win_.pop_front();
        auto& pr = per_req_[request];
        pr.first += proposed; pr.second += accepted;
    }
    float ema() const { return ema_; }
    float global_rate() const { return tot_prop_ ? (float)tot_acc_ / tot_prop_ : 0.f; }
    float windowed_rate() const {
        long p = 0, a = 0;
        for (auto& w : win_) { p += w.first; a += w.second; }
        return p ? (float)a / p : 0.f;
    }
    float request_rate(int request) const {
        auto it = per_req_.find(request);
        return (it == per_req_.end() || !it->second.first) ? 0.f : (float)it->second.second / it->second.first;
    }
    void forget(int request) { per_req_.erase(request); }
    // Expected tokens per round for depth gamma under an i.i.d. per-token acceptance rate.
    float expected_tokens(int gamma) const {
        const float a = std::min(std::max(windowed_rate(), 0.f), 0.999f);
        return (1.f - std::pow(a, gamma + 1)) / (1.f - a);
    }
private:
    float alpha_; int window_; float ema_ = 0.f; long n_ = 0, tot_prop_ = 0, tot_acc_ = 0;
    std::deque<std::pair<int, int>> win_;
    std::unordered_map<int, std::pair<long, long>> per_req_;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
LSB_RT_API void* lsb_es_create(int n, float alpha) { return new ExpertStats(n, alpha); }
LSB_RT_API void lsb_es_destroy(void* h) { delete (ExpertStats*)h; }
LSB_RT_API void lsb_es_observe(void* h, const int* ids, const float* w, int k) { ((ExpertStats*)h)->observe(ids, w, k); }
LSB_RT_API float lsb_es_frequency(void* h, int e) { return ((ExpertStats*)h)->frequency(e); }
LSB_RT_API float lsb_es_weight(void* h, int e) { return ((ExpertStats*)h)->mean_weight(e); }
LSB_RT_API float lsb_es_autocorr(void* h, int e) { return ((ExpertStats*)h)->autocorr(e); }
LSB_RT_API float lsb_es_recency(void* h, int e) { return ((ExpertStats*)h)->recency(e); }
LSB_RT_API void lsb_es_frequencies(void* h, float* out) { ((ExpertStats*)h)->frequencies(out); }

LSB_RT_API void* lsb_cg_create(int n, float decay) { return new CoactivationGraph(n, decay); }
LSB_RT_API void lsb_cg_destroy(void* h) { delete (CoactivationGraph*)h; }
LSB_RT_API void lsb_cg_observe(void* h, const int* ids, int k) { ((CoactivationGraph*)h)->observe(ids, k); }
LSB_RT_API float lsb_cg_weight(void* h, int a, int b) { return ((CoactivationGraph*)h)->weight(a, b); }
LSB_RT_API void lsb_cg_partition(void* h, int parts, int* out) { ((CoactivationGraph*)h)->partition(parts, out); }

LSB_RT_API void* lsb_wd_create(int n, int window, float z) { return new WorkloadDetector(n, window, z); }
LSB_RT_API void lsb_wd_destroy(void* h) { delete (WorkloadDetector*)h; }
LSB_RT_API int lsb_wd_observe(void* h, const float* freq) { return ((WorkloadDetector*)h)->observe(freq); }
LSB_RT_API int lsb_wd_shifts(void* h) { return ((WorkloadDetector*)h)->shifts(); }

LSB_RT_API void* lsb_at_create(float alpha, int window) { return new AcceptanceTracker(alpha, window); }
LSB_RT_API void lsb_at_destroy(void* h) { delete (AcceptanceTracker*)h; }
LSB_RT_API void lsb_at_record(void* h, int request, int proposed, int accepted) { ((AcceptanceTracker*)h)->record(request, proposed, accepted); }
LSB_RT_API float lsb_at_ema(void* h) { return ((AcceptanceTracker*)h)->ema(); }
LSB_RT_API float lsb_at_global(void* h) { return ((AcceptanceTracker*)h)->global_rate(); }
LSB_RT_API float lsb_at_windowed(void* h) { return ((AcceptanceTracker*)h)->windowed_rate(); }
LSB_RT_API float lsb_at_request(void* h, int request) { return ((AcceptanceTracker*)h)->request_rate(request); }
LSB_RT_API void lsb_at_forget(void* h, int request) { ((AcceptanceTracker*)h)->forget(request); }
LSB_RT_API float lsb_at_expected_tokens(void* h, int gamma) { return ((AcceptanceTracker*)h)->expected_tokens(gamma); }
}
