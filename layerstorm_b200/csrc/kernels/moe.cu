// Mixture-of-experts routing and the decode-shaped expert FFN.
//
//  * router_topk: scoring (sigmoid / softmax / sqrt-softplus) + selection bias + grouped
//    top-k (group score = sum of the two best biased scores in the group) + top-k by biased
//    score with ties to the LOWER index + unbiased weights renormalised and scaled; shared
//    experts appended as extra always-on slots.  Contract taken from the reference's CPU
//    oracle tests/unit/topk_gating_test.cpp:31-125 (kernel: E/sm120/gating/topk_gating.cu).
//  * moe_build_groups: counting sort of (row, slot) pairs by expert into groups of <= 4 rows
//    that share one weight stream (the role of E/smxx/permute/moe_permute.cu, without a
//    physical permute of activations).
//  * moe_gateup / moe_down: weight-streaming expert GEMVs with fused SwiGLU(+clamp); experts
//    are addressed through a slot table so the same kernel serves a fully resident model and
//    a capped VRAM expert cache.
//  * moe_combine: out[r] = sum over slots in slot order of w[r][s] * y[r][s]  (fp32, fixed
//    order => placement-invariant; reference: src/core/expert_device.h:31-52).
#include <cstdlib>
#include "gemv_core.cuh"
#include "comm.cuh"
#include "moe_fmt.cuh"
#include "router_core.cuh"

namespace lsb {

// One block per row.
__global__ void __launch_bounds__(1024) router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ ids,
                                                           float* __restrict__ wts, int E, int topk, int n_group, int topk_group, int scoring,
                                                           int norm_topk, float scale, int n_shared, int ld_logits) {
    extern __shared__ float sm[];
    pdl_wait();
    pdl_launch_dependents();
    router_topk_block<false>(logits + (size_t)blockIdx.x * ld_logits, bias, ids + (size_t)blockIdx.x * (topk + n_shared),
                             wts + (size_t)blockIdx.x * (topk + n_shared), E, topk, n_group, topk_group, scoring, norm_topk, scale, n_shared, sm);
}

// Router projection and top-k in one launch for decode-sized steps (rows <= 8): one block per expert computes its fp32 logit
// for all rows (fp32 router weights [E, H], bf16 activations, the reduction split over the block's 4 warps); the last block to
// finish runs the top-k of each row.  Saves a launch and a dependent-kernel hand-off per MoE layer.
constexpr int kRouterMaxRows = 8;
__global__ void __launch_bounds__(128) router_fused_kernel(const float* __restrict__ w, const bf16* __restrict__ x, float* __restrict__ logits,
                                                           const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ wts,
                                                           unsigned* __restrict__ done, int rows, int H, int E, int topk, int n_group,
                                                           int topk_group, int scoring, int norm_topk, float scale, int n_shared) {
    extern __shared__ float sm[];                // last block: scratch of the top-k selection
    __shared__ int s_last;
    __shared__ float s_part[4][kRouterMaxRows];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x;                    // one expert per block, the reduction split over the 4 warps
    const int kq = H >> 2;                       // columns per warp (a multiple of 4)
    const float* wr = w + (size_t)e * H + warp * kq;
    // weights do not depend on the previous kernel: have them on their way before the dependency wait
    for (int k = lane * 32; k < kq; k += 32 * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(wr + k));
    pdl_wait();
    pdl_launch_dependents();
    float acc[kRouterMaxRows];
#pragma unroll
    for (int m = 0; m < kRouterMaxRows; ++m) acc[m] = 0.f;
#pragma unroll 4
    for (int k = lane * 4; k < kq; k += 128) {
        const float4 wv = __ldg(reinterpret_cast<const float4*>(wr + k));
#pragma unroll
        for (int m = 0; m < kRouterMaxRows; ++m) {
            if (m < rows) {
                const uint2 xv = *reinterpret_cast<const uint2*>(x + (size_t)m * H + warp * kq + k);
                const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.x));
                const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.y));
                acc[m] = fmaf(wv.x, x01.x, acc[m]); acc[m] = fmaf(wv.y, x01.y, acc[m]);
                acc[m] = fmaf(wv.z, x23.x, acc[m]); acc[m] = fmaf(wv.w, x23.y, acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kRouterMaxRows; ++m) {
        if (m < rows) {
            const float v = warp_sum(acc[m]);
            if (lane == 0) s_part[warp][m] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < rows) logits[(size_t)threadIdx.x * E + e] = (s_part[0][threadIdx.x] + s_part[1][threadIdx.x]) + (s_part[2][threadIdx.x] + s_part[3][threadIdx.x]);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(done, 1u) == gridDim.x - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) *done = 0;
    __threadfence();
    for (int r = 0; r < rows; ++r)
        router_topk_block<true>(logits + (size_t)r * E, bias, ids + (size_t)r * (topk + n_shared), wts + (size_t)r * (topk + n_shared), E, topk, n_group,
                                topk_group, scoring, norm_topk, scale, n_shared, sm);
}

// Hash-layer gating (DeepSeek-V4 hash layers): the experts of a row come from a table indexed by the row's token id
// (tid2eid[token * topk + k], table order kept), the weights are the scores of exactly those experts - no selection
// bias - optionally renormalised and scaled.  A token id outside the table or a table entry outside [0, E) yields
// expert -1 with weight 0 (the slot is dropped by the expert kernels).  One warp per row.
// Reference semantics: src/compute/kernels/moe/hash_gating.h:1-16.
__global__ void __launch_bounds__(32) router_hash_kernel(const float* __restrict__ logits, const int* __restrict__ tid2eid,
                                                         const int* __restrict__ token_ids, int* __restrict__ ids, float* __restrict__ wts,
                                                         int E, int topk, int vocab, int scoring, int norm_topk, float scale, int n_shared,
                                                         int ld_logits) {
    const int r = blockIdx.x, lane = threadIdx.x;
    const float* lg = logits + (size_t)r * ld_logits;
    pdl_wait();
    pdl_launch_dependents();
    float mx = -INFINITY, den = 1.f;
    if (scoring == kScoreSoftmax) {                  // the only scoring that needs the whole row
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(lg[e] - mx);
        den = warp_sum(sum);
    }
    const int tok = token_ids[r];
    int id = -1;
    float w = 0.f;
    if (lane < topk && tok >= 0 && tok < vocab) {
        const int e = tid2eid[(size_t)tok * topk + lane];
        if (e >= 0 && e < E) {
            const float x = lg[e];
            id = e;
            if (scoring == kScoreSigmoid) w = 1.f / (1.f + expf(-x));
            else if (scoring == kScoreSoftmax) w = expf(x - mx) / den;
            else w = sqrtf(x > 20.f ? x : log1pf(expf(x)));
        }
    }
    const float tot = warp_sum(w);
    const int S = topk + n_shared;
    if (lane < topk) {
        if (norm_topk) w = w / (tot + 1e-20f);
        ids[r * S + lane] = id;
        wts[r * S + lane] = id >= 0 ? w * scale : 0.f;
    }
    if (lane < n_shared) { ids[r * S + topk + lane] = E + lane; wts[r * S + topk + lane] = 1.f; }
    pdl_launch_dependents();
}

// Groups: for every expert (routed and shared) with at least one (row,slot) pair, its pairs
// in ascending pair order are cut into groups of <= 4.  Output:
//   group_expert[g], group_n[g], group_pairs[g*4 + i] (pair = row*S + slot), n_groups[0].
// Single block; deterministic.
__global__ void moe_build_groups_kernel(const int* __restrict__ ids, int npairs, int E_total, int* __restrict__ group_expert,
                                        int* __restrict__ group_n, int* __restrict__ group_pairs, int* __restrict__ n_groups,
                                        int* __restrict__ counts /* scratch [E_total*2+1] */) {
    pdl_wait();
    pdl_launch_dependents();
    int* cnt = counts;             // [E_total]
    int* gbase = counts + E_total; // [E_total+1] first group index per expert
    for (int e = threadIdx.x; e < E_total; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E_total) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int g = 0;
        for (int e = 0; e < E_total; ++e) { gbase[e] = g; g += (cnt[e] + 3) >> 2; }
        gbase[E_total] = g;
        n_groups[0] = g;
    }
    __syncthreads();
    // one thread per expert walks the pair list in order (deterministic placement)
    for (int e = threadIdx.x; e < E_total; e += blockDim.x) {
        const int c = cnt[e];
        if (c == 0) continue;
        int g = gbase[e], k = 0;
        for (int i = 0; i < npairs && k < c; ++i) {
            if (ids[i] == e) {
                group_pairs[(g + (k >> 2)) * 4 + (k & 3)] = i;
                ++k;
            }
        }
        for (int j = 0; j < (c + 3) >> 2; ++j) {
            group_expert[g + j] = e;
            group_n[g + j] = min(4, c - j * 4);
        }
    }
    pdl_launch_dependents();
}

template <int FMT> struct RowOf;
template <> struct RowOf<0> {
    using T = WRowBf16;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t*, int n, int K) {
        return T{reinterpret_cast<const bf16*>(w) + (size_t)n * K};
    }
};
template <> struct RowOf<1> {
    using T = WRowFp8B;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t* s, int n, int K) {
        return T{w + (size_t)n * K, reinterpret_cast<const float*>(s) + (size_t)(n >> 7) * ((K + 127) >> 7)};
    }
};
template <> struct RowOf<2> {
    using T = WRowNvfp4;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t* s, int n, int K) {
        return T{w + (size_t)n * (K >> 1), s, n, ((K >> 4) + 3) >> 2};
    }
};

template <> struct RowOf<3> {
    using T = WRowQ4K;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t*, int n, int K) {
        return T{w + (size_t)n * (K >> 8) * 144};
    }
};

template <> struct RowOf<4> {
    using T = WRowQ5K;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t*, int n, int K) { return T{w + (size_t)n * (K >> 8) * 176}; }
};
template <> struct RowOf<5> {
    using T = WRowQ6K;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t*, int n, int K) { return T{w + (size_t)n * (K >> 8) * kQ6KDevBlock}; }
};
template <> struct RowOf<6> {
    using T = WRowQ80;
    static __device__ __forceinline__ T make(const uint8_t* w, const uint8_t*, int n, int K) { return T{w + (size_t)n * (K + (K >> 4)), K}; }
};

// act[pair][f] = silu(min(g,limit)) * clamp(u) ; g = x[row] . Wgate[f], u = x[row] . Wup[f]
template <int FMT>
__global__ void __launch_bounds__(256) moe_gateup_kernel(const bf16* __restrict__ x, const uint8_t* __restrict__ arena,
                                                         const int* __restrict__ slot_of, ExpertFmt ef,
                                                         const int* __restrict__ group_expert, const int* __restrict__ group_n,
                                                         const int* __restrict__ group_pairs, const int* __restrict__ n_groups,
                                                         bf16* __restrict__ act, int S, float limit, int* __restrict__ miss_flag) {
    pdl_wait();
    pdl_launch_dependents();
    const int g = blockIdx.y;
    if (g >= n_groups[0]) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f = blockIdx.x * 8 + warp;
    if (f >= ef.F) return;
    const int e = group_expert[g], n = group_n[g];
    const int slot = slot_of[e];
    if (slot < 0) { if (miss_flag && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(miss_flag, e + 1); return; }
    const uint8_t* base = arena + (size_t)slot * ef.stride;
    auto rg = RowOf<FMT>::make(base + ef.off_gate, base + ef.off_sg, f, ef.H);
    auto ru = RowOf<FMT>::make(base + ef.off_up, base + ef.off_su, f, ef.H);
    float ag[4] = {0, 0, 0, 0}, au[4] = {0, 0, 0, 0};
    int pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = group_pairs[g * 4 + min(i, n - 1)];
    // rows may be arbitrary: gather pointers instead of a fixed ldx
    constexpr int E = decltype(rg)::EPL;
#pragma unroll 2
    for (int k = lane * E; k + E <= ef.H; k += 32 * E) {
        float a[E], b[E];
        rg.load(k, a);
        ru.load(k, b);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            if (m < n) {
                const bf16* xp = x + (size_t)(pr[m] / S) * ef.H + k;
#pragma unroll
                for (int e8 = 0; e8 < E; e8 += 8) {
                    float xf[8];
                    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(xp + e8)), xf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { ag[m] = fmaf(a[e8 + i], xf[i], ag[m]); au[m] = fmaf(b[e8 + i], xf[i], au[m]); }
                }
            }
        }
    }
    float sg = 1.f, su = 1.f;
    if (FMT == 2) {
        const float* tail = reinterpret_cast<const float*>(base + ef.off_tail);
        sg = tail[0]; su = tail[1];
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        if (m < n) {
            float gv = warp_sum(ag[m]) * sg, uv = warp_sum(au[m]) * su;
            if (limit > 0.f) { gv = fminf(gv, limit); uv = fminf(fmaxf(uv, -limit), limit); }
            if (lane == 0) act[(size_t)pr[m] * ef.F + f] = __float2bfloat16(siluf_(gv) * uv);
        }
    }
    pdl_launch_dependents();
}

// y[pair][h] = act[pair] . Wdown[h]   (fp32)
template <int FMT>
__global__ void __launch_bounds__(256) moe_down_kernel(const bf16* __restrict__ act, const uint8_t* __restrict__ arena,
                                                       const int* __restrict__ slot_of, ExpertFmt ef,
                                                       const int* __restrict__ group_expert, const int* __restrict__ group_n,
                                                       const int* __restrict__ group_pairs, const int* __restrict__ n_groups,
                                                       float* __restrict__ y) {
    pdl_wait();
    pdl_launch_dependents();
    const int g = blockIdx.y;
    if (g >= n_groups[0]) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = (blockIdx.x * 8 + warp) * 2;
    if (h0 >= ef.H) return;
    const int e = group_expert[g], n = group_n[g];
    const int slot = slot_of[e];
    if (slot < 0) return;
    const uint8_t* base = arena + (size_t)slot * ef.stride;
    auto r0 = RowOf<FMT>::make(base + ef.off_down, base + ef.off_sd, h0, ef.F);
    auto r1 = RowOf<FMT>::make(base + ef.off_down, base + ef.off_sd, min(h0 + 1, ef.H - 1), ef.F);
    float a0[4] = {0, 0, 0, 0}, a1[4] = {0, 0, 0, 0};
    int pr[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = group_pairs[g * 4 + min(i, n - 1)];
    constexpr int E = decltype(r0)::EPL;
#pragma unroll 2
    for (int k = lane * E; k + E <= ef.F; k += 32 * E) {
        float a[E], b[E];
        r0.load(k, a);
        r1.load(k, b);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            if (m < n) {
                const bf16* xp = act + (size_t)pr[m] * ef.F + k;
#pragma unroll
                for (int e8 = 0; e8 < E; e8 += 8) {
                    float xf[8];
                    unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(xp + e8)), xf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { a0[m] = fmaf(a[e8 + i], xf[i], a0[m]); a1[m] = fmaf(b[e8 + i], xf[i], a1[m]); }
                }
            }
        }
    }
    float sd = 1.f;
    if (FMT == 2) sd = reinterpret_cast<const float*>(base + ef.off_tail)[2];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        if (m < n) {
            const float v0 = warp_sum(a0[m]) * sd, v1 = warp_sum(a1[m]) * sd;
            if (lane == 0) {
                y[(size_t)pr[m] * ef.H + h0] = v0;
                if (h0 + 1 < ef.H) y[(size_t)pr[m] * ef.H + h0 + 1] = v1;
            }
        }
    }
    pdl_launch_dependents();
}


// ---- NVFP4 fast path (hidden and expert width multiples of 128) -----------------------------
// Row order inside a 128-row tile follows the scale-atom layout: a block covers 8 (gate/up) or 16
// (down) consecutive values of n%32 for all four 32-row quads, so every 32-byte sector of scale
// bytes it touches is used completely.
template <int MT>
__global__ void __launch_bounds__(256) moe_gateup_fp4_kernel(const bf16* __restrict__ x, const uint8_t* __restrict__ arena,
                                                             const int* __restrict__ slot_of, ExpertFmt ef,
                                                             const int* __restrict__ group_expert, const int* __restrict__ group_n,
                                                             const int* __restrict__ group_pairs, const int* __restrict__ n_groups,
                                                             bf16* __restrict__ act, int S, float limit, int* __restrict__ miss_flag, int run) {
    extern __shared__ __align__(16) uint8_t smraw[];
    __half* xs = reinterpret_cast<__half*>(smraw);
    __shared__ const bf16* rows[4];
    pdl_wait();
    pdl_launch_dependents();
    const int g = blockIdx.y;
    if (g >= (n_groups ? n_groups[0] : (int)gridDim.y)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = group_expert[g];
    const int n = MT == 1 ? 1 : (group_n ? group_n[g] : 1);
    const int slot = (e >= 0) ? slot_of[e] : -1;
    if (slot < 0) { if (miss_flag && e >= 0 && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(miss_flag, e + 1); return; }
    int pr[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) pr[i] = group_pairs ? group_pairs[g * 4 + min(i, n - 1)] : g;
    if (threadIdx.x < MT) rows[threadIdx.x] = x + (size_t)(pr[threadIdx.x] / S) * ef.H;
    const uint8_t* base = arena + (size_t)slot * ef.stride;
    // a block covers `run` consecutive values of n % 32 for all four 32-row quads of a 128-row tile (4 * run rows, run / 2 passes of
    // one row per warp): run = 8 streams most per block, smaller runs spread an expert over more blocks and shorten the chain of
    // dependent passes when a GPU holds only a few of the step's experts
    const int bpt = 32 / run;                              // blocks per 128-row tile
    const int tile = blockIdx.x / bpt, blk = blockIdx.x - tile * bpt;
    const int gtiles = ef.H >> 6;
    const int kTS = run * 16 + 4;                          // scale bytes per K-tile + 4 pad (odd number of words: conflict-free)
    uint8_t* scg = smraw + (size_t)MT * ef.H * 2;
    uint8_t* scu = scg + (size_t)gtiles * kTS;
    stage_scales(scg, base + ef.off_sg, tile, blk, run, gtiles, kTS);
    stage_scales(scu, base + ef.off_su, tile, blk, run, gtiles, kTS);
    __syncthreads();
    stage_x_half(xs, rows, n, ef.H);
    __syncthreads();
    const float* tail = reinterpret_cast<const float*>(base + ef.off_tail);
    const float sg = tail[0], su = tail[1];
#pragma unroll 1
    for (int r = 0; r < run / 2; ++r) {
        const int j = r * 8 + warp;                       // 0 .. 4 run - 1
        const int quad = j / run, i = j - quad * run;
        const int f = tile * 128 + quad * 32 + blk * run + i;
        float ag[MT], au[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) ag[m] = au[m] = 0.f;
        const int so = i * 16 + quad * 4;
        nvfp4_row_dot2_sm<MT>(base + ef.off_gate + (size_t)f * (ef.H >> 1), scg + so,
                              base + ef.off_up + (size_t)f * (ef.H >> 1), scu + so, kTS, ef.H, xs, n, ag, au);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < n) {
                float gv = warp_sum(ag[m]) * sg, uv = warp_sum(au[m]) * su;
                if (limit > 0.f) { gv = fminf(gv, limit); uv = fminf(fmaxf(uv, -limit), limit); }
                if (lane == 0) act[(size_t)pr[m] * ef.F + f] = __float2bfloat16(siluf_(gv) * uv);
            }
        }
    }
    pdl_launch_dependents();
}

template <int MT>
__global__ void __launch_bounds__(256) moe_down_fp4_kernel(const bf16* __restrict__ act, const uint8_t* __restrict__ arena,
                                                           const int* __restrict__ slot_of, ExpertFmt ef,
                                                           const int* __restrict__ group_expert, const int* __restrict__ group_n,
                                                           const int* __restrict__ group_pairs, const int* __restrict__ n_groups,
                                                           float* __restrict__ y, int run) {
    extern __shared__ __align__(16) uint8_t smraw[];
    __half* xs = reinterpret_cast<__half*>(smraw);
    __shared__ const bf16* rows[4];
    pdl_wait();
    pdl_launch_dependents();
    const int g = blockIdx.y;
    if (g >= (n_groups ? n_groups[0] : (int)gridDim.y)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = group_expert[g];
    const int n = MT == 1 ? 1 : (group_n ? group_n[g] : 1);
    const int slot = (e >= 0) ? slot_of[e] : -1;
    if (slot < 0) return;
    int pr[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) pr[i] = group_pairs ? group_pairs[g * 4 + min(i, n - 1)] : g;
    if (threadIdx.x < MT) rows[threadIdx.x] = act + (size_t)pr[threadIdx.x] * ef.F;
    const uint8_t* base = arena + (size_t)slot * ef.stride;
    const int bpt = 32 / run;                              // see moe_gateup_fp4_kernel: 4 * run rows per block, two rows per warp and pass
    const int tile = blockIdx.x / bpt, blk = blockIdx.x - tile * bpt;
    const int gtiles = ef.F >> 6;
    const int kTS = run * 16 + 4;
    uint8_t* scd = smraw + (size_t)MT * ef.F * 2;
    stage_scales(scd, base + ef.off_sd, tile, blk, run, gtiles, kTS);
    __syncthreads();
    stage_x_half(xs, rows, n, ef.F);
    __syncthreads();
    const float sd = reinterpret_cast<const float*>(base + ef.off_tail)[2];
#pragma unroll 1
    for (int r = 0; r < run / 4; ++r) {
        const int j0 = r * 16 + warp * 2;                 // 0 .. 4 run - 2, two rows per pass
        const int quad = j0 / run, i = j0 - quad * run;
        const int h0 = tile * 128 + quad * 32 + blk * run + i;
        const int h1 = h0 + 1;
        float a0[MT], a1[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) a0[m] = a1[m] = 0.f;
        const int so = i * 16 + quad * 4;
        nvfp4_row_dot2_sm<MT>(base + ef.off_down + (size_t)h0 * (ef.F >> 1), scd + so,
                              base + ef.off_down + (size_t)h1 * (ef.F >> 1), scd + so + 16, kTS, ef.F, xs, n, a0, a1);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < n) {
                const float v0 = warp_sum(a0[m]) * sd, v1 = warp_sum(a1[m]) * sd;
                if (lane == 0) { y[(size_t)pr[m] * ef.H + h0] = v0; y[(size_t)pr[m] * ef.H + h1] = v1; }
            }
        }
    }
    pdl_launch_dependents();
}

// out[r][h] = sum_s w[r][s] * y[r*S+s][h], slots in order; experts that were not resident
// (slot < 0) contribute nothing.  mode 0: write fp32; mode 1: add into out.
__global__ void moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const float* __restrict__ wts,
                                   const int* __restrict__ ids, const int* __restrict__ slot_of, int S, int H, int accumulate,
                                   PeerComm comm) {
    constexpr int kMaxS = 16;
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int h = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    unsigned next_epoch = 0;
    if (comm.nranks) next_epoch = *comm.epoch + 1;
    const bool push = comm.nranks && !comm.xchg;      // xchg: this rank's partial stays local, the consuming kernel exchanges it
    if (comm.nranks && comm.xchg && (blockIdx.x | blockIdx.y | threadIdx.x) == 0) *comm.epoch = next_epoch;
    if (h >= H) {
        if (push) comm_signal(comm, next_epoch, gridDim.x * gridDim.y);
        return;
    }
    // routing metadata first (independent loads), then all slot rows in flight together
    int e[kMaxS];
    float w[kMaxS];
#pragma unroll
    for (int s = 0; s < kMaxS; ++s) { e[s] = s < S ? ids[r * S + s] : -1; w[s] = s < S ? wts[r * S + s] : 0.f; }
#pragma unroll
    for (int s = 0; s < kMaxS; ++s) if (e[s] >= 0 && slot_of[e[s]] < 0) e[s] = -1;
    float4 v[kMaxS];
#pragma unroll
    for (int s = 0; s < kMaxS; ++s)
        v[s] = e[s] >= 0 ? *reinterpret_cast<const float4*>(y + ((size_t)r * S + s) * H + h) : make_float4(0, 0, 0, 0);
    float4 a = make_float4(0, 0, 0, 0);
#pragma unroll
    for (int s = 0; s < kMaxS; ++s) {
        if (e[s] >= 0) { a.x = fmaf(w[s], v[s].x, a.x); a.y = fmaf(w[s], v[s].y, a.y); a.z = fmaf(w[s], v[s].z, a.z); a.w = fmaf(w[s], v[s].w, a.w); }
    }
    if (push) {
        const size_t idx = (size_t)r * H + h;
        if ((comm.cap & 3) == 0) {
            comm_push4(comm, next_epoch, idx, a);
        } else {
            comm_push(comm, next_epoch, idx, a.x); comm_push(comm, next_epoch, idx + 1, a.y);
            comm_push(comm, next_epoch, idx + 2, a.z); comm_push(comm, next_epoch, idx + 3, a.w);
        }
        comm_signal(comm, next_epoch, gridDim.x * gridDim.y);
    } else {
        float4* o = reinterpret_cast<float4*>(out + (size_t)r * H + h);
        if (accumulate) { float4 p = *o; a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w; }
        *o = a;
    }
    pdl_launch_dependents();
}

// Dense SwiGLU on a fused [rows, 2F] fp32 projection (gate | up) -> bf16 [rows, F].
__global__ void swiglu_kernel(bf16* __restrict__ out, const float* __restrict__ gu, int F, float limit) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y, f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= F) return;
    float g = gu[(size_t)r * 2 * F + f], u = gu[(size_t)r * 2 * F + F + f];
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    out[(size_t)r * F + f] = __float2bfloat16(siluf_(g) * u);
    pdl_launch_dependents();
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_router_topk(const void* logits, const void* bias, void* ids, void* wts, int rows, int E, int topk,
                            int n_group, int topk_group, int scoring, int norm_topk, float scale, int n_shared,
                            int ld_logits, void* stream) {
    if (topk > 32 || n_group > 64 || E > 4096 || n_shared > 32) return -1;
    int threads = (E + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
    launch_pdl((router_topk_kernel), rows, threads, (size_t)router_topk_smem_floats(E) * 4, (cudaStream_t)stream, (const float*)logits, (const float*)bias,
               (int*)ids, (float*)wts, E, topk, n_group, topk_group, scoring, norm_topk, scale, n_shared, ld_logits);
    LSB_CHECK_LAUNCH();
}

// Router projection + top-k in one launch (rows <= 8, H % 16 == 0).  w: fp32 [E, H]; x: bf16 [rows, H]; logits: fp32 scratch
// [rows, E]; done: one zero-initialised counter.
LSB_API int lsb_router_fused(const void* w, const void* x, void* logits, const void* bias, void* ids, void* wts, void* done, int rows, int H,
                             int E, int topk, int n_group, int topk_group, int scoring, int norm_topk, float scale, int n_shared, void* stream) {
    if (rows > kRouterMaxRows || H % 16 || topk > 32 || n_group > 64 || E > 4096 || n_shared > 32) return -1;
    const size_t smem = (size_t)router_topk_smem_floats(E) * 4;
    if (smem > 48 * 1024) return -1;
    launch_pdl((router_fused_kernel), E, 128, smem, (cudaStream_t)stream, (const float*)w, (const bf16*)x, (float*)logits, (const float*)bias,
               (int*)ids, (float*)wts, (unsigned*)done, rows, H, E, topk, n_group, topk_group, scoring, norm_topk, scale, n_shared);
    LSB_CHECK_LAUNCH();
}

// Hash-layer routing: ids[r][k] = tid2eid[token_ids[r]][k], weights from the logits of those experts.
LSB_API int lsb_router_hash(const void* logits, const void* tid2eid, const void* token_ids, void* ids, void* wts, int rows, int E, int topk,
                            int vocab, int scoring, int norm_topk, float scale, int n_shared, int ld_logits, void* stream) {
    if (topk > 32 || n_shared > 32 || E <= 0) return -1;
    launch_pdl((router_hash_kernel), rows, 32, 0, (cudaStream_t)stream, (const float*)logits, (const int*)tid2eid, (const int*)token_ids, (int*)ids,
               (float*)wts, E, topk, vocab, scoring, norm_topk, scale, n_shared, ld_logits);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_moe_build_groups(const void* ids, int npairs, int E_total, void* group_expert, void* group_n,
                                 void* group_pairs, void* n_groups, void* counts, void* stream) {
    launch_pdl((moe_build_groups_kernel), 1, 512, 0, (cudaStream_t)stream, (const int*)ids, npairs, E_total, (int*)group_expert, (int*)group_n,
                                                               (int*)group_pairs, (int*)n_groups, (int*)counts);
    LSB_CHECK_LAUNCH();
}

// Pair mode (group_n == null): every (row, slot) pair is its own group - group_expert is the
// routing id array itself, group g is pair g; used for small batches where no build pass is needed.
LSB_API int lsb_moe_gateup(const void* x, const void* arena, const void* slot_of, const void* fmt_struct,
                           const void* group_expert, const void* group_n, const void* group_pairs, const void* n_groups,
                           void* act, int S, int max_groups, float limit, void* miss_flag, int run, void* stream) {
    ExpertFmt ef = *reinterpret_cast<const ExpertFmt*>(fmt_struct);
    cudaStream_t st = (cudaStream_t)stream;
    if (ef.fmt == 2 && ef.F % 128 == 0 && ef.H % 128 == 0) {   // K % 64 == 0 follows
        // run: values of n % 32 per block (8, 4 or 2; 0 = 8) - see the kernel
        if (run != 2 && run != 4) run = 8;
        dim3 g2(ef.F / (4 * run), max_groups);
        const size_t sc_bytes = (size_t)2 * (ef.H / 64) * (run * 16 + 4);
        static bool attr = false;
        if (!attr) {
            cudaFuncSetAttribute(moe_gateup_fp4_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            cudaFuncSetAttribute(moe_gateup_fp4_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            attr = true;
        }
        if (!group_n)
            launch_pdl((moe_gateup_fp4_kernel<1>), g2, 256, (size_t)ef.H * 2 + sc_bytes, st, (const bf16*)x, (const uint8_t*)arena, (const int*)slot_of, ef, (const int*)group_expert,
                                                                        nullptr, nullptr, nullptr, (bf16*)act, S, limit, (int*)miss_flag, run);
        else
            launch_pdl((moe_gateup_fp4_kernel<4>), g2, 256, (size_t)ef.H * 8 + sc_bytes, st, (const bf16*)x, (const uint8_t*)arena, (const int*)slot_of, ef, (const int*)group_expert,
                                                                        (const int*)group_n, (const int*)group_pairs, (const int*)n_groups, (bf16*)act, S, limit,
                                                                        (int*)miss_flag, run);
        LSB_CHECK_LAUNCH();
    }
    if (!group_n) return -1;   // pair mode is only implemented for the NVFP4 fast path
    dim3 grid((ef.F + 7) / 8, max_groups);
#define ARGS (const bf16*)x, (const uint8_t*)arena, (const int*)slot_of, ef, (const int*)group_expert, (const int*)group_n, \
             (const int*)group_pairs, (const int*)n_groups, (bf16*)act, S, limit, (int*)miss_flag
    if (ef.fmt == 0) launch_pdl((moe_gateup_kernel<0>), grid, 256, 0, st, ARGS);
    else if (ef.fmt == 1) launch_pdl((moe_gateup_kernel<1>), grid, 256, 0, st, ARGS);
    else if (ef.fmt == 2) launch_pdl((moe_gateup_kernel<2>), grid, 256, 0, st, ARGS);
    else if (ef.fmt == 3) launch_pdl((moe_gateup_kernel<3>), grid, 256, 0, st, ARGS);
    else if (ef.fmt == 4) launch_pdl((moe_gateup_kernel<4>), grid, 256, 0, st, ARGS);
    else if (ef.fmt == 5) launch_pdl((moe_gateup_kernel<5>), grid, 256, 0, st, ARGS);
    else if (ef.fmt == 6) launch_pdl((moe_gateup_kernel<6>), grid, 256, 0, st, ARGS);
    else return -1;
#undef ARGS
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_moe_down(const void* act, const void* arena, const void* slot_of, const void* fmt_struct,
                         const void* group_expert, const void* group_n, const void* group_pairs, const void* n_groups,
                         void* y, int max_groups, int run, void* stream) {
    ExpertFmt ef = *reinterpret_cast<const ExpertFmt*>(fmt_struct);
    cudaStream_t st = (cudaStream_t)stream;
    if (ef.down_fmt() == 2 && ef.F % 128 == 0 && ef.H % 128 == 0) {
        if (run != 4 && run != 8) run = 16;                  // values of n % 32 per block (16, 8 or 4; 0 = 16)
        dim3 g2(ef.H / (4 * run), max_groups);
        const size_t sc_bytes = (size_t)(ef.F / 64) * (run * 16 + 4);
        static bool attr = false;
        if (!attr) {
            cudaFuncSetAttribute(moe_down_fp4_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            cudaFuncSetAttribute(moe_down_fp4_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            attr = true;
        }
        if (!group_n)
            launch_pdl((moe_down_fp4_kernel<1>), g2, 256, (size_t)ef.F * 2 + sc_bytes, st, (const bf16*)act, (const uint8_t*)arena, (const int*)slot_of, ef, (const int*)group_expert,
                                                                      nullptr, nullptr, nullptr, (float*)y, run);
        else
            launch_pdl((moe_down_fp4_kernel<4>), g2, 256, (size_t)ef.F * 8 + sc_bytes, st, (const bf16*)act, (const uint8_t*)arena, (const int*)slot_of, ef, (const int*)group_expert,
                                                                      (const int*)group_n, (const int*)group_pairs, (const int*)n_groups, (float*)y, run);
        LSB_CHECK_LAUNCH();
    }
    if (!group_n) return -1;
    dim3 grid((ef.H + 15) / 16, max_groups);
#define ARGS (const bf16*)act, (const uint8_t*)arena, (const int*)slot_of, ef, (const int*)group_expert, (const int*)group_n, \
             (const int*)group_pairs, (const int*)n_groups, (float*)y
    const int df = ef.down_fmt();
    if (df == 0) launch_pdl((moe_down_kernel<0>), grid, 256, 0, st, ARGS);
    else if (df == 1) launch_pdl((moe_down_kernel<1>), grid, 256, 0, st, ARGS);
    else if (df == 2) launch_pdl((moe_down_kernel<2>), grid, 256, 0, st, ARGS);
    else if (df == 3) launch_pdl((moe_down_kernel<3>), grid, 256, 0, st, ARGS);
    else if (df == 4) launch_pdl((moe_down_kernel<4>), grid, 256, 0, st, ARGS);
    else if (df == 5) launch_pdl((moe_down_kernel<5>), grid, 256, 0, st, ARGS);
    else if (df == 6) launch_pdl((moe_down_kernel<6>), grid, 256, 0, st, ARGS);
    else return -1;
#undef ARGS
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_moe_combine(void* out, const void* y, const void* wts, const void* ids, const void* slot_of, int rows,
                            int S, int H, int accumulate, const void* comm, void* stream) {
    PeerComm pc;
    pc.nranks = 0;
    if (comm) pc = *reinterpret_cast<const PeerComm*>(comm);
    if (H % 4 || S > 16) return -1;
    dim3 grid((H / 4 + 127) / 128, rows);
    launch_pdl((moe_combine_kernel), grid, 128, 0, (cudaStream_t)stream, (float*)out, (const float*)y, (const float*)wts, (const int*)ids,
                                                             (const int*)slot_of, S, H, accumulate, pc);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_swiglu(void* out, const void* gu, int rows, int F, float limit, void* stream) {
    dim3 grid((F + 255) / 256, rows);
    launch_pdl((swiglu_kernel), grid, 256, 0, (cudaStream_t)stream, (bf16*)out, (const float*)gu, F, limit);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_moe(void* buf) { return lsb_trace_install(buf); }
