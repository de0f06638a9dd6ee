// Runs the CUDA source of the chunk-parallel KDA kernels (csrc/kernels/kda_chunk.cuh) on the CPU: every CUDA thread of a block is an OS
// thread, __syncthreads is a barrier over the block, warp shuffles exchange through a per-warp buffer.  Blocks run one after the other.
// This checks the kernels' index arithmetic, shared-memory layout and barrier placement against the token-by-token recurrence without a
// GPU; it says nothing about performance.  Build: g++ -O1 -std=c++20 -pthread -I <csrc/kernels> kda_chunk_emu.cpp
#include <algorithm>
#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

typedef uint16_t bf16;
struct float4 { float x, y, z, w; };
static inline float4 make_float4(float x, float y, float z, float w) { return float4{x, y, z, w}; }
struct Idx3 { int x = 0, y = 0, z = 0; };
static thread_local Idx3 threadIdx, blockIdx;
#define __global__
#define __device__
#define __forceinline__ inline
#define __restrict__
#define __launch_bounds__(...)
#define __shared__
#define __align__(x)
using std::min;

alignas(16) float csm[64 * 1024];                        // dynamic shared memory of the running block (256 KB)
static std::barrier<>* g_block_bar = nullptr;
static std::barrier<>* g_warp_bar[8];
static float g_shfl[8][32];
static inline void __syncthreads() { g_block_bar->arrive_and_wait(); }
static inline float __shfl_xor_sync(unsigned, float v, int o) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    g_shfl[w][l] = v;
    g_warp_bar[w]->arrive_and_wait();
    const float r = g_shfl[w][l ^ o];
    g_warp_bar[w]->arrive_and_wait();
    return r;
}
#define __expf(x) expf(x)
static inline void pdl_wait() {}
static inline void pdl_launch_dependents() {}

#include "kda_types.cuh"
#include "kda_chunk.cuh"

template <class K>
static void launch(K kernel, int gx, int gy, int nthreads, const KdaParams& p, const KdaScratch& w, const KdaChunkWs& cw) {
    for (int by = 0; by < gy; ++by)
        for (int bx = 0; bx < gx; ++bx) {
            std::barrier<> bar(nthreads);
            g_block_bar = &bar;
            std::vector<std::unique_ptr<std::barrier<>>> wb;
            for (int i = 0; i < 8; ++i) { wb.emplace_back(new std::barrier<>(32)); g_warp_bar[i] = wb.back().get(); }
            std::vector<std::thread> th;
            for (int t = 0; t < nthreads; ++t)
                th.emplace_back([=, &p, &w, &cw] {
                    threadIdx.x = t; blockIdx.x = bx; blockIdx.y = by;
                    kernel(p, w, cw);
                });
            for (auto& x : th) x.join();
        }
}

static uint64_t g_rng = 0x1234567;
static float urand() { g_rng = g_rng * 6364136223846793005ULL + 1442695040888963407ULL; return (float)((g_rng >> 40) & 0xFFFFFF) / 16777216.f; }

int main(int argc, char** argv) {
    const int T = argc > 1 ? atoi(argv[1]) : 150, H = argc > 2 ? atoi(argv[2]) : 2, row0 = 3, slot = 1;
    const int rows = row0 + T, C = H * kD, ldp = 3 * C;
    std::vector<float> qn((size_t)rows * C), kn(qn.size()), vo(qn.size()), decay(qn.size()), gate(qn.size(), 1.f), beta((size_t)rows * H);
    std::vector<float> proj((size_t)rows * ldp), state((size_t)2 * H * kD * kD), conv((size_t)2 * 3 * C * 3);
    for (auto& x : proj) x = urand() - 0.5f;
    for (auto& x : state) x = 0.2f * (urand() - 0.5f);
    for (auto& x : conv) x = urand();
    for (int r = 0; r < rows; ++r)
        for (int h = 0; h < H; ++h) {
            double nq = 0, nk = 0;
            float* q = &qn[(size_t)r * C + h * kD]; float* k = &kn[(size_t)r * C + h * kD];
            for (int c = 0; c < kD; ++c) { q[c] = urand() - 0.5f; k[c] = urand() - 0.5f; nq += q[c] * q[c]; nk += k[c] * k[c]; }
            for (int c = 0; c < kD; ++c) {
                q[c] = (float)(q[c] / sqrt(nq + 1e-6) / sqrt((double)kD)); k[c] = (float)(k[c] / sqrt(nk + 1e-6));
                vo[(size_t)r * C + h * kD + c] = 2.f * urand() - 1.f;
                decay[(size_t)r * C + h * kD + c] = expf(-5.f * urand() * urand());          // (e^-5, 1], denser towards 1
            }
            beta[(size_t)r * H + h] = urand();
        }
    // reference: the recurrence token by token, in double
    std::vector<double> S((size_t)H * kD * kD), ref_o((size_t)T * C);
    for (int h = 0; h < H; ++h)
        for (int i = 0; i < kD * kD; ++i) S[(size_t)h * kD * kD + i] = state[((size_t)slot * H + h) * kD * kD + i];
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < H; ++h) {
            const size_t o = (size_t)(row0 + t) * C + h * kD;
            for (int v = 0; v < kD; ++v) {
                double* s = &S[((size_t)h * kD + v) * kD];
                double sk = 0;
                for (int c = 0; c < kD; ++c) { s[c] *= decay[o + c]; sk += s[c] * kn[o + c]; }
                const double err = (vo[o + v] - sk) * beta[(size_t)(row0 + t) * H + h];
                double out = 0;
                for (int c = 0; c < kD; ++c) { s[c] += err * kn[o + c]; out += s[c] * qn[o + c]; }
                ref_o[(size_t)t * C + h * kD + v] = out;
            }
        }
    std::vector<float> conv_ref = conv;
    for (int a = 0; a < 3; ++a)
        for (int ch = 0; ch < C; ++ch)
            for (int d = 0; d < 3; ++d) conv_ref[(((size_t)slot * 3 + a) * C + ch) * 3 + d] = proj[(size_t)(row0 + T - 3 + d) * ldp + a * C + ch];
    // the kernels
    int h_row0 = row0, h_nrows = T, h_slot = slot;
    KdaParams p{};
    p.proj = proj.data(); p.ldp = ldp; p.off_q = 0; p.off_k = C; p.off_v = 2 * C; p.state = state.data(); p.conv_state = conv.data();
    p.seq_row0 = &h_row0; p.seq_nrows = &h_nrows; p.seq_slot = &h_slot; p.H = H;
    KdaScratch w{qn.data(), kn.data(), vo.data(), decay.data(), gate.data(), beta.data(), nullptr, nullptr};
    const int nch = (rows + kCh - 1) / kCh;                  // the host sizes the grid from the step's row count (>= the sequence's rows)
    std::vector<float> ws((size_t)nch * H * (2 * kCh * kCh + kD), -777.f);
    KdaChunkWs cw{ws.data(), ws.data() + (size_t)nch * H * kCh * kCh, ws.data() + (size_t)2 * nch * H * kCh * kCh};
    if (kChunkPrepSmem > sizeof(csm) || kChunkScanSmem > sizeof(csm)) { printf("shared memory buffer too small\n"); return 2; }
    launch(kda_chunk_prep_kernel, nch, H, 256, p, w, cw);
    launch(kda_chunk_scan_kernel, H, kD / kCh, 256, p, w, cw);
    double eo = 0, mo = 0, es = 0, ms = 0;
    for (int t = 0; t < T; ++t)
        for (int c = 0; c < C; ++c) {
            eo = std::max(eo, fabs(vo[(size_t)(row0 + t) * C + c] - ref_o[(size_t)t * C + c]));
            mo = std::max(mo, fabs(ref_o[(size_t)t * C + c]));
        }
    for (int h = 0; h < H; ++h)
        for (int i = 0; i < kD * kD; ++i) {
            es = std::max(es, fabs(state[((size_t)slot * H + h) * kD * kD + i] - S[(size_t)h * kD * kD + i]));
            ms = std::max(ms, fabs(S[(size_t)h * kD * kD + i]));
        }
    bool conv_ok = conv == conv_ref;
    bool other_slot_untouched = true;
    for (int i = 0; i < H * kD * kD; ++i) other_slot_untouched &= fabs(state[i]) <= 0.1f;     // slot 0 keeps its initial values
    printf("out_rel=%.3e state_rel=%.3e conv_ok=%d other_slot_untouched=%d\n", eo / mo, es / ms, (int)conv_ok, (int)other_slot_untouched);
    return (eo / mo < 1e-4 && es / ms < 1e-4 && conv_ok && other_slot_untouched) ? 0 : 1;
}
