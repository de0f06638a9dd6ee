// Router scoring + grouped top-k of one row by one warp, shared by the stand-alone router kernels (moe.cu) and the
// fused hyper-connection + router kernel (mhc_cluster.cu).
#pragma once
#include "common.cuh"

namespace lsb {

enum { kScoreSigmoid = 0, kScoreSoftmax = 1, kScoreSqrtSoftplus = 2 };

// Scores, grouped selection and top-k of ONE row (lg: its E logits; ids / wts: its topk + n_shared output slots) by ONE warp (`lane`): no block-wide barriers, the k selection rounds are
// shuffle reductions.  sm: 2 E + 64 floats of shared memory, s_keep: 64 ints, both private to the warp.
template <bool CG = true>
__device__ __forceinline__ void router_topk_row(const float* __restrict__ lg, const float* __restrict__ bias, int* __restrict__ ids,
                                                float* __restrict__ wts, int E, int topk, int n_group, int topk_group, int scoring,
                                                int norm_topk, float scale, int n_shared, int lane, float* sm, int* s_keep) {
    float* score = sm;            // [E] unbiased
    float* sel = sm + E;          // [E] biased, -inf when masked/taken
    float mx = -INFINITY;
    if (scoring == kScoreSoftmax) {
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, CG ? __ldcg(lg + e) : lg[e]);
        mx = warp_max(mx);
    }
    float ssum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float x = CG ? __ldcg(lg + e) : lg[e];
        float s;
        if (scoring == kScoreSigmoid) s = 1.f / (1.f + expf(-x));
        else if (scoring == kScoreSoftmax) s = expf(x - mx);
        else s = sqrtf(x > 20.f ? x : log1pf(expf(x)));
        score[e] = s;
        ssum += s;
    }
    if (scoring == kScoreSoftmax) {
        ssum = warp_sum(ssum);
        for (int e = lane; e < E; e += 32) score[e] /= ssum;
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) sel[e] = score[e] + (bias ? bias[e] : 0.f);
    __syncwarp();
    if (n_group > 1) {
        const int gs = E / n_group;
        // group score = sum of the two best biased scores; keep topk_group groups (ties -> lower group)
        for (int g0 = 0; g0 < n_group; g0 += 32) {
            const int g = g0 + lane;
            if (g < n_group) {
                float a = -INFINITY, b2 = -INFINITY;
                for (int i = 0; i < gs; ++i) {
                    const float v = sel[g * gs + i];
                    if (v > a) { b2 = a; a = v; } else if (v > b2) b2 = v;
                }
                s_keep[g] = 0;
                sm[2 * E + g] = a + b2;
            }
        }
        __syncwarp();
        float* gscore = sm + 2 * E;
        for (int k = 0; k < topk_group; ++k) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < n_group; g += 32) {
                if (s_keep[g]) continue;
                const float v = gscore[g];
                if (bi == 0x7fffffff || v > bv || (v == bv && g < bi)) { bv = v; bi = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if (lane == 0 && bi != 0x7fffffff) s_keep[bi] = 1;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (!s_keep[e / gs]) sel[e] = -INFINITY;
        __syncwarp();
    }
    float my_w = 0.f; int my_id = 0;     // lane k keeps the k-th pick
    float tot = 0.f;
    for (int k = 0; k < topk; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = sel[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi >= E) bi = 0;               // everything masked (cannot happen with finite logits)
        const float w = score[bi];
        tot += w;
        if (lane == (k & 31)) { my_w = w; my_id = bi; }
        if (lane == 0) sel[bi] = -INFINITY;
        __syncwarp();
    }
    if (lane < topk) {
        float w = my_w;
        if (norm_topk) w = w / (tot + 1e-20f);
        ids[lane] = my_id;
        wts[lane] = w * scale;
    }
    if (lane < n_shared) { ids[topk + lane] = E + lane; wts[topk + lane] = 1.f; }
}

}  // namespace lsb
