// CPU expert kernels: the routed-expert FFN  down( SiLU(gate x) * up x )  computed on the host straight from the
// same slot images the GPU uses (BF16, FP8 e4m3 + 128x128 block scales, NVFP4 + 128x4 scale atoms + per-tensor
// scale, GGUF Q4_K blocks), fp32 accumulation, optional SwiGLU clamp.  Weights are de-quantised on the fly one row
// at a time; rows are distributed over a fork-join pool of worker threads (optionally pinned to a CPU set).
// Uses: oracle for the device kernels' slot formats, timed CPU baseline of the tiny configuration, and optional
// host execution of experts that are cold in the VRAM cache.
// Reference components: deps/LayerStoRmCpuExpertKernels/csrc/compute/cpu/{nvfp4_cpu_kernel,cpu_moe_kernels,
// numa_thread_pool}.* and the NumaCpuExpertDevice (src/compute/cpu/numa_cpu_expert_device.*).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include <pthread.h>
#include <sched.h>

#include "lsb_runtime.h"

extern "C" int lsb_ggml_dequantize(int type, const void* src, float* dst, long long n);

namespace lsb {

// ------------------------------------------------------------------ fork-join pool
class ForkJoinPool {
public:
    explicit ForkJoinPool(int n, const int* cpus, int n_cpus) : n_(std::max(1, n)) {
        for (int i = 1; i < n_; ++i) {
            threads_.emplace_back([this, i] { worker(i); });
            if (cpus && n_cpus > 0) {
                cpu_set_t set;
                CPU_ZERO(&set);
                CPU_SET(cpus[i % n_cpus], &set);
                pthread_setaffinity_np(threads_.back().native_handle(), sizeof(set), &set);   // best effort
            }
        }
    }
    ~ForkJoinPool() {
        { std::lock_guard<std::mutex> g(mu_); stop_ = true; ++gen_; }
        cv_.notify_all();
        for (auto& t : threads_) t.join();
    }
    int size() const { return n_; }
    // fn(worker, n_workers) runs on every worker (the caller is worker 0); returns when all are done.
    void run(const std::function<void(int, int)>& fn) {
        {
            std::lock_guard<std::mutex> g(mu_);
            fn_ = &fn;
            pending_ = n_ - 1;
            ++gen_;
        }
        cv_.notify_all();
        fn(0, n_);
        std::unique_lock<std::mutex> g(mu_);
        done_.wait(g, [this] { return pending_ == 0; });
    }
private:
    void worker(int id) {
        uint64_t seen = 0;
        for (;;) {
            const std::function<void(int, int)>* fn;
            {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [&] { return gen_ != seen; });
                seen = gen_;
                if (stop_) return;
                fn = fn_;
            }
            (*fn)(id, n_);
            std::lock_guard<std::mutex> g(mu_);
            if (--pending_ == 0) done_.notify_one();
        }
    }
    int n_;
    std::vector<std::thread> threads_;
    std::mutex mu_;
    std::condition_variable cv_, done_;
    const std::function<void(int, int)>* fn_ = nullptr;
    uint64_t gen_ = 0;
    int pending_ = 0;
    bool stop_ = false;
};

// ------------------------------------------------------------------ scalar decoders
static inline float bf16_to_f32(uint16_t v) { uint32_t u = (uint32_t)v << 16; float f; std::memcpy(&f, &u, 4); return f; }

static float e4m3_decode(uint8_t b) {
    const int sign = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 0) v = std::ldexp((float)m, -9);                 // subnormal: m * 2^-3 * 2^-6
    else if (e == 15 && m == 7) v = NAN;
    else v = std::ldexp(1.0f + (float)m / 8.0f, e - 7);
    return sign ? -v : v;
}
// all 256 codes once: the FP8 row decoder is one table load per weight (a per-element ldexp made FP8 slots 7x slower than BF16 ones)
struct E4m3Table {
    float v[256];
    E4m3Table() { for (int i = 0; i < 256; ++i) v[i] = e4m3_decode((uint8_t)i); }
};
static const E4m3Table kE4m3;
static inline float e4m3_to_f32(uint8_t b) { return kE4m3.v[b]; }
static const float kE2M1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

struct Fmt { int fmt, H, F; int64_t stride, off_gate, off_up, off_down, off_sg, off_su, off_sd, off_tail; };

// De-quantise row n of a [N, K] matrix stored in format `fmt` at `w` (scales at `sf`, per-tensor scale `ts`).
static void dequant_row(int fmt, const uint8_t* w, const uint8_t* sf, float ts, int n, int K, float* out) {
    switch (fmt) {
        case 0: {
            const uint16_t* p = reinterpret_cast<const uint16_t*>(w) + (size_t)n * K;
            for (int k = 0; k < K; ++k) out[k] = bf16_to_f32(p[k]);
            break;
        }
        case 1: {
            const uint8_t* p = w + (size_t)n * K;
            const float* s = reinterpret_cast<const float*>(sf) + (size_t)(n >> 7) * ((K + 127) >> 7);
            for (int k = 0; k < K; ++k) out[k] = e4m3_to_f32(p[k]) * s[k >> 7];
            break;
        }
        case 2: {
            const uint8_t* p = w + (size_t)n * (K >> 1);
            const int G = K >> 4, gtiles = (G + 3) >> 2;
            for (int g = 0; g < G; ++g) {
                const size_t off = ((size_t)(n >> 7) * gtiles + (g >> 2)) * 512 + (n & 31) * 16 + ((n & 127) >> 5) * 4 + (g & 3);
                const float s = e4m3_to_f32(sf[off]) * ts;
                for (int i = 0; i < 8; ++i) {
                    const uint8_t b = p[g * 8 + i];
                    out[g * 16 + 2 * i] = kE2M1[b & 15] * s;
                    out[g * 16 + 2 * i + 1] = kE2M1[b >> 4] * s;
                }
            }
            break;
        }
        case 3:
            lsb_ggml_dequantize(12 /* Q4_K */, w + (size_t)n * (K >> 8) * 144, out, K);
            break;
    }
}

// Function multiversioning resolves through an ifunc that runs before a ThreadSanitizer runtime is initialised (the process crashes at
// start-up), so the clones are left out of -fsanitize=thread builds.
#if defined(__SANITIZE_THREAD__)
#define LSB_TARGET_CLONES
#else
#define LSB_TARGET_CLONES __attribute__((target_clones("avx512f", "avx2", "default")))
#endif

LSB_TARGET_CLONES
static float dot_f32(const float* a, const float* b, int n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
    float s = 0.f;
    for (; i < n; ++i) s += a[i] * b[i];
    for (int j = 0; j < 8; ++j) s += acc[j];
    return s;
}

static inline float silu(float x) { return x / (1.f + std::exp(-x)); }

// y[t][:] (+)= scale[t] * expert(x[t][:]) for n tokens with ONE expert slot image.
static void expert_ffn(ForkJoinPool& pool, const Fmt& f, const uint8_t* slot, const float* x, int n, float limit, const float* scale,
                       float* y, bool accumulate) {
    const int H = f.H, F = f.F;
    float tg = 1.f, tu = 1.f, td = 1.f;
    if (f.fmt == 2) { const float* tail = reinterpret_cast<const float*>(slot + f.off_tail); tg = tail[0]; tu = tail[1]; td = tail[2]; }
    std::vector<float> act((size_t)n * F);
    pool.run([&](int wk, int nw) {
        std::vector<float> rg(H), ru(H);
        for (int r = wk; r < F; r += nw) {
            dequant_row(f.fmt, slot + f.off_gate, slot + f.off_sg, tg, r, H, rg.data());
            dequant_row(f.fmt, slot + f.off_up, slot + f.off_su, tu, r, H, ru.data());
            for (int t = 0; t < n; ++t) {
                float g = dot_f32(rg.data(), x + (size_t)t * H, H), u = dot_f32(ru.data(), x + (size_t)t * H, H);
                if (limit > 0.f) { g = std::min(g, limit); u = std::min(std::max(u, -limit), limit); }
                act[(size_t)t * F + r] = silu(g) * u;
            }
        }
    });
    pool.run([&](int wk, int nw) {
        std::vector<float> rd(F);
        for (int r = wk; r < H; r += nw) {
            dequant_row(f.fmt, slot + f.off_down, slot + f.off_sd, td, r, F, rd.data());
            for (int t = 0; t < n; ++t) {
                const float v = dot_f32(rd.data(), act.data() + (size_t)t * F, F) * (scale ? scale[t] : 1.f);
                float& o = y[(size_t)t * H + r];
                o = accumulate ? o + v : v;
            }
        }
    });
}

}  // namespace lsb

using namespace lsb;
extern "C" {
LSB_RT_API void* lsb_cpu_pool_create(int threads, const int* cpus, int n_cpus) { return new ForkJoinPool(threads, cpus, n_cpus); }
LSB_RT_API void lsb_cpu_pool_destroy(void* h) { delete (ForkJoinPool*)h; }
LSB_RT_API int lsb_cpu_pool_size(void* h) { return ((ForkJoinPool*)h)->size(); }

// fmt_struct: the ExpertFmt structure shared with the GPU kernels (int fmt, H, F; int64 stride, 3 weight offsets,
// 3 scale offsets, tail offset).  x: fp32 [n, H]; y: fp32 [n, H]; scale: per-token routing weight or null.
LSB_RT_API int lsb_cpu_expert_ffn(void* pool, const void* fmt_struct, const void* slot, const float* x, int n, float limit,
                                  const float* scale, float* y, int accumulate) {
    struct Raw { int fmt, H, F; long long stride, og, ou, od, sg, su, sd, tail; };
    const Raw* r = (const Raw*)fmt_struct;
    if (!pool || !slot || n < 0 || r->fmt < 0 || r->fmt > 3) return LSB_ERR_ARG;
    if (r->fmt == 3 && (r->H % 256 || r->F % 256)) return LSB_ERR_ARG;
    Fmt f{r->fmt, r->H, r->F, r->stride, r->og, r->ou, r->od, r->sg, r->su, r->sd, r->tail};
    expert_ffn(*(ForkJoinPool*)pool, f, (const uint8_t*)slot, x, n, limit, scale, y, accumulate != 0);
    return 0;
}

// Full MoE layer on the host: out[t] = sum_s wts[t][s] * expert_{ids[t][s]}(x[t]) in slot order.  slots[e] = slot image of
// expert e (null = not available: contributes nothing).  Tokens of one expert are processed together.
LSB_RT_API int lsb_cpu_moe_layer(void* pool, const void* fmt_struct, const void* const* slots, int n_experts, const float* x, const int* ids,
                                 const float* wts, int tokens, int S, float limit, float* out) {
    struct Raw { int fmt, H, F; long long stride, og, ou, od, sg, su, sd, tail; };
    const Raw* r = (const Raw*)fmt_struct;
    if (!pool || tokens < 0 || S < 1) return LSB_ERR_ARG;
    const int H = r->H;
    std::vector<float> y((size_t)tokens * S * H, 0.f);
    std::vector<std::vector<int>> by_expert(n_experts);
    for (int i = 0; i < tokens * S; ++i) if (ids[i] >= 0 && ids[i] < n_experts && slots[ids[i]]) by_expert[ids[i]].push_back(i);
    Fmt f{r->fmt, r->H, r->F, r->stride, r->og, r->ou, r->od, r->sg, r->su, r->sd, r->tail};
    std::vector<float> xe, ye;
    for (int e = 0; e < n_experts; ++e) {
        const auto& pairs = by_expert[e];
        if (pairs.empty()) continue;
        xe.resize(pairs.size() * H); ye.resize(pairs.size() * H);
        for (size_t j = 0; j < pairs.size(); ++j) std::memcpy(&xe[j * H], x + (size_t)(pairs[j] / S) * H, (size_t)H * 4);     // permute
        expert_ffn(*(ForkJoinPool*)pool, f, (const uint8_t*)slots[e], xe.data(), (int)pairs.size(), limit, nullptr, ye.data(), false);
        for (size_t j = 0; j < pairs.size(); ++j) std::memcpy(&y[(size_t)pairs[j] * H], &ye[j * H], (size_t)H * 4);            // unpermute
    }
    for (int t = 0; t < tokens; ++t)
        for (int h = 0; h < H; ++h) {
            float a = 0.f;
            for (int s = 0; s < S; ++s) a = std::fma(wts[t * S + s], y[((size_t)t * S + s) * H + h], a);      // fixed slot order
            out[(size_t)t * H + h] = a;
        }
    return 0;
}
}
