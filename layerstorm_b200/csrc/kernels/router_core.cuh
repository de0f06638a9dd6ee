// Router scoring + grouped top-k of one row by one thread block, shared by the stand-alone router kernels (moe.cu) and
// the fused hyper-connection + router kernel (mhc_cluster.cu).
//
// Selection is by RANK instead of k rounds of arg-max: expert e is picked when fewer than k experts beat it (higher biased
// score, or the same score and a lower index), and its output slot is that count.  Every thread ranks its experts against
// the whole row in shared memory, so the k picks cost one pass instead of k dependent reductions, and the result - order
// included - is the one the sequential selection gives (ties to the lower index).
// Contract: the reference's CPU oracle tests/unit/topk_gating_test.cpp:31-125.
#pragma once
#include "common.cuh"

namespace lsb {

enum { kScoreSigmoid = 0, kScoreSoftmax = 1, kScoreSqrtSoftplus = 2 };

// floats of shared memory router_topk_block needs for E experts
__host__ __device__ constexpr int router_topk_smem_floats(int E) { return 2 * E + 64 + 64 + 32 + 32 + 34; }

// lg: the E logits of the row (global or shared memory; CG: read through L2 because other blocks of the same kernel wrote them);
// ids / wts: the row's topk + n_shared output slots.  Whole block, any block size; contains block-wide barriers.
template <bool CG = true>
__device__ __forceinline__ void router_topk_block(const float* __restrict__ lg, const float* __restrict__ bias, int* __restrict__ ids,
                                                  float* __restrict__ wts, int E, int topk, int n_group, int topk_group, int scoring,
                                                  int norm_topk, float scale, int n_shared, float* sm) {
    float* score = sm;                         // [E] unbiased
    float* sel = sm + E;                       // [E] biased, -inf when the group is masked
    float* gscore = sel + E;                   // [64]
    int* keep = reinterpret_cast<int*>(gscore + 64);       // [64]
    int* pick_id = keep + 64;                  // [32]
    float* pick_w = reinterpret_cast<float*>(pick_id + 32);   // [32]
    float* red = pick_w + 32;                  // [34]
    const int t = threadIdx.x, nt = blockDim.x;
    float mx = 0.f, den = 1.f;
    if (scoring == kScoreSoftmax) {
        float m = -INFINITY;
        for (int e = t; e < E; e += nt) m = fmaxf(m, CG ? __ldcg(lg + e) : lg[e]);
        mx = block_max(m, red);
        float s = 0.f;
        for (int e = t; e < E; e += nt) s += expf((CG ? __ldcg(lg + e) : lg[e]) - mx);
        den = block_sum(s, red);
    }
    for (int e = t; e < E; e += nt) {
        const float x = CG ? __ldcg(lg + e) : lg[e];
        float s;
        if (scoring == kScoreSigmoid) s = 1.f / (1.f + expf(-x));
        else if (scoring == kScoreSoftmax) s = expf(x - mx) / den;
        else s = sqrtf(x > 20.f ? x : log1pf(expf(x)));
        score[e] = s;
        sel[e] = s + (bias ? bias[e] : 0.f);
    }
    if (t < 32) { pick_id[t] = 0; pick_w[t] = 0.f; }
    __syncthreads();
    if (n_group > 1) {
        const int gs = E / n_group;
        // group score = sum of the two best biased scores; keep topk_group groups (ties -> lower group)
        for (int g = t; g < n_group; g += nt) {
            float a = -INFINITY, b2 = -INFINITY;
            for (int i = 0; i < gs; ++i) {
                const float v = sel[g * gs + i];
                if (v > a) { b2 = a; a = v; } else if (v > b2) b2 = v;
            }
            gscore[g] = a + b2;
        }
        __syncthreads();
        for (int g = t; g < n_group; g += nt) {
            const float v = gscore[g];
            int rank = 0;
            for (int j = 0; j < n_group; ++j) {
                const float o = gscore[j];
                rank += (o > v || (o == v && j < g)) ? 1 : 0;
            }
            keep[g] = rank < topk_group;
        }
        __syncthreads();
        for (int e = t; e < E; e += nt)
            if (!keep[e / gs]) sel[e] = -INFINITY;
        __syncthreads();
    }
    for (int e = t; e < E; e += nt) {
        const float v = sel[e];
        int rank = 0;
#pragma unroll 8
        for (int j = 0; j < E; ++j) {
            const float o = sel[j];
            rank += (o > v || (o == v && j < e)) ? 1 : 0;
        }
        if (rank < topk) { pick_id[rank] = e; pick_w[rank] = score[e]; }
    }
    __syncthreads();
    if (t < 32) {
        float tot = 0.f;
        for (int k = 0; k < topk; ++k) tot += pick_w[k];          // same order as k sequential picks
        if (t < topk) {
            float w = pick_w[t];
            if (norm_topk) w = w / (tot + 1e-20f);
            ids[t] = pick_id[t];
            wts[t] = w * scale;
        }
        if (t < n_shared) { ids[topk + t] = E + t; wts[topk + t] = 1.f; }
    }
    __syncthreads();                            // the scratch may be reused for the next row
}

}  // namespace lsb
