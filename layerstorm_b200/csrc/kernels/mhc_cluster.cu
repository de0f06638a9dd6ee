// Hyper-connection (mHC) post -> pre pass for decode-sized steps as ONE thread-block-cluster kernel per token row.
//
// What the pass computes (reference: launchers in src/compute/kernels/mhc/mhc.h, math in tools/glm53_numpy_ref.py:128-179):
//   residual'[j] = post[j] * x + sum_i comb[i][j] * residual[i]                 (post of the previous sublayer)
//   mix[o]       = fn[o] . flatten(residual') / rms(flatten(residual'))         (24 mixing logits)
//   pre, post', comb' from mix (sigmoid gates, Sinkhorn-normalised n x n matrix)
//   out          = RMSNorm(sum_j pre[j] * residual'[j]) * norm_w                (input of the next sublayer, bf16)
//
// The hidden dimension is split over the CTAs of a cluster (16 CTAs x 256 columns at hidden 4096).  Every CTA keeps its
// slice of the new residual streams in registers, publishes 34 partial sums (24 logits + the 10 entries of the Gram matrix
// of the streams, from which both RMS values follow algebraically) in its shared memory, and after one cluster barrier every
// CTA sums all slices through distributed shared memory in CTA order - no global scratch, no atomics, no second launch.
// The mixing rows `fn` do not depend on the previous kernel and are loaded before the programmatic-launch wait.
//
// Two neighbours of the pass can be folded in (both decode-only, single GPU):
//   * in front: the fixed-order weighted sum of the routed-expert outputs (the MoE combine) replaces the read of `x`;
//   * behind:   the fp32 router projection of `out` (split over the CTAs, summed through distributed shared memory)
//               and the grouped top-k selection, so a MoE layer needs no router launches.
// With a PeerComm the kernel is the consumer half of the fused cross-rank all-reduce (see comm.cuh).
#include <cooperative_groups.h>

#include "common.cuh"
#include "comm.cuh"
#include "router_core.cuh"

namespace cg = cooperative_groups;

namespace lsb {

constexpr int kCMax = 4;                                 // residual streams
constexpr int kCOut = 2 * kCMax + kCMax * kCMax;         // 24 mixing logits
constexpr int kCGram = kCMax * (kCMax + 1) / 2;          // 10
constexpr int kCSum = kCOut + kCGram;                    // 34 partial sums per CTA
constexpr int kCPerWarp = 6;                             // mixing logits per warp
constexpr int kCMaxS = 16;                               // routing slots per row the folded combine handles
constexpr int kCMaxCluster = 16;

struct MhcClusterArgs {
    bf16* out;
    float* residual;
    const float* x;
    float* post;
    float* comb;
    const float* fn;
    const float* hc_scale;
    const float* hc_base;
    const float* norm_w;
    int hidden, n, mode, iters;
    float hc_eps, rms_eps, post_mult;
    // folded MoE combine (y != null): x = sum_s wts[s] * y[r*S+s], slots in order, non-resident experts skipped
    const float* y;
    const float* cwts;
    const int* cids;
    const int* slot_of;
    int S;
    // folded router (router_w != null)
    const float* router_w;
    const float* router_bias;
    float* logits;
    int* ids_out;
    float* wts_out;
    int E, topk, n_group, topk_group, scoring, norm_topk, n_shared;
    float scale;
    PeerComm comm;
};

// Column layout of a CTA: `groups` column groups of 128 columns (4 consecutive columns per lane); a column group is served
// by four warps, warp og of them owning mixing logits 6 og .. 6 og + 5.  The CTA's slice of the mixing rows `fn`
// (24 x n x cols fp32, 96 KB at 256 columns) is staged in shared memory by asynchronous copies issued BEFORE the dependency
// wait, and the thread count / register need is kept small (256 threads), so that the CTAs of a cluster can become resident
// next to the tail of the preceding weight-streaming kernel and have the slice in place when the dependency resolves.
constexpr int kCVec = 4;
constexpr int kCGroupCols = 32 * kCVec;                  // 128

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

__global__ void __launch_bounds__(256, 1) mhc_cluster_kernel(const __grid_constant__ MhcClusterArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned crank = cluster.block_rank(), csize = cluster.num_blocks();
    __shared__ float s_part[2][kCSum];
    __shared__ float s_all[kCMaxCluster][kCSum + 2];          // partial sums of every CTA of the cluster (pushed by their owners)
    __shared__ float mix[kCSum + 2];
    __shared__ float s_pre[8];
    __shared__ __align__(16) float xs[2 * kCGroupCols];
    extern __shared__ __align__(16) float dyn[];              // [kCOut][n][cols] mixing rows, then the router scratch
    const int t = threadIdx.x, lane = t & 31, w = t >> 5, og = w & 3, grp = w >> 2;
    const int groups = blockDim.x >> 7;
    const int r = blockIdx.y;
    const int n = a.n, hidden = a.hidden;
    const int cols = groups * kCGroupCols;                    // columns of this CTA
    const int c0 = (int)crank * cols;
    const int hl = grp * kCGroupCols + lane * kCVec;          // column inside the CTA slice
    const int h = c0 + hl;
    const int nout = 2 * n + n * n;
    float* sf = dyn;
    float* rdyn = dyn + (size_t)kCOut * kCMax * cols;

    // first half of a start-up barrier: a CTA's shared memory may be written by its peers only once it is known to run
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    // mixing rows of this CTA's columns -> shared memory; independent of the previous kernel
    {
        const int per_row = cols >> 2;                        // 16-byte pieces per (logit, stream) row
        const int total = nout * n * per_row;
        for (int idx = t; idx < total; idx += blockDim.x) {
            const int row = idx / per_row, pc = idx - row * per_row;          // row = o * n + j
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(sf + (size_t)row * cols + pc * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(a.fn + (size_t)row * hidden + c0 + pc * 4) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const float4 nw4 = __ldg(reinterpret_cast<const float4*>(a.norm_w + h));
    if (a.router_w) {
        for (int e = w; e < a.E; e += (int)(blockDim.x >> 5))
            for (int k = lane * 32; k < cols; k += 32 * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.router_w + (size_t)e * hidden + c0 + k));
    }
    pdl_wait();
    pdl_launch_dependents();

    // ---- sublayer output for this thread's columns ----
    float xv[kCVec];
    if (a.comm.nranks && a.mode == 1) {
        const unsigned epoch = *a.comm.epoch;
        comm_wait(a.comm, epoch);
#pragma unroll
        for (int u = 0; u < kCVec; ++u) xv[u] = comm_reduce(a.comm, epoch, (size_t)r * hidden + h + u);
    } else if (a.y) {
        int e[kCMaxS];
        float wt[kCMaxS];
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s) { e[s] = s < a.S ? a.cids[r * a.S + s] : -1; wt[s] = s < a.S ? a.cwts[r * a.S + s] : 0.f; }
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s) if (e[s] >= 0 && a.slot_of[e[s]] < 0) e[s] = -1;
        float4 v[kCMaxS];
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s) v[s] = e[s] >= 0 ? ld4(a.y + ((size_t)r * a.S + s) * hidden + h) : make_float4(0.f, 0.f, 0.f, 0.f);
        xv[0] = xv[1] = xv[2] = xv[3] = 0.f;
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s)
            if (e[s] >= 0) {
                xv[0] = fmaf(wt[s], v[s].x, xv[0]); xv[1] = fmaf(wt[s], v[s].y, xv[1]);
                xv[2] = fmaf(wt[s], v[s].z, xv[2]); xv[3] = fmaf(wt[s], v[s].w, xv[3]);
            }
    } else {
        const float4 q = ld4(a.x + (size_t)r * hidden + h);
        xv[0] = q.x; xv[1] = q.y; xv[2] = q.z; xv[3] = q.w;
    }

    // ---- new residual streams (every warp of a column group recomputes them; warp og 0 stores) ----
    float res[kCMax][kCVec];
    float* rp = a.residual + (size_t)r * n * hidden;
    if (a.mode == 0) {
#pragma unroll
        for (int j = 0; j < kCMax; ++j)
#pragma unroll
            for (int u = 0; u < kCVec; ++u) res[j][u] = j < n ? xv[u] : 0.f;
    } else {
        float old[kCMax][kCVec];
#pragma unroll
        for (int i = 0; i < kCMax; ++i) {
            const float4 q = i < n ? ld4(rp + (size_t)i * hidden + h) : make_float4(0.f, 0.f, 0.f, 0.f);
            old[i][0] = q.x; old[i][1] = q.y; old[i][2] = q.z; old[i][3] = q.w;
        }
#pragma unroll
        for (int j = 0; j < kCMax; ++j) {
            float acc[kCVec] = {0.f, 0.f, 0.f, 0.f};
            if (j < n) {
                const float pj = a.post[r * n + j];
#pragma unroll
                for (int u = 0; u < kCVec; ++u) acc[u] = pj * xv[u];
                for (int i = 0; i < n; ++i) {
                    const float cj = a.comb[(r * n + i) * n + j];
#pragma unroll
                    for (int u = 0; u < kCVec; ++u) acc[u] += cj * old[i][u];
                }
            }
#pragma unroll
            for (int u = 0; u < kCVec; ++u) res[j][u] = acc[u];
        }
    }

    // ---- partial mixing logits and Gram entries over this warp's columns ----
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                 // the staged mixing rows of all threads are visible
#pragma unroll
    for (int i = 0; i < kCPerWarp; ++i) {
        const int o = og * kCPerWarp + i;
        float acc = 0.f;
        if (o < nout) {
#pragma unroll
            for (int j = 0; j < kCMax; ++j)
                if (j < n) {
                    const float4 f4 = ld4(sf + (size_t)(o * n + j) * cols + hl);
                    acc = fmaf(res[j][0], f4.x, acc); acc = fmaf(res[j][1], f4.y, acc);
                    acc = fmaf(res[j][2], f4.z, acc); acc = fmaf(res[j][3], f4.w, acc);
                }
        }
        acc = warp_sum(acc);
        if (lane == 0 && o < kCOut) s_part[grp][o] = acc;
    }
    {
        int e = 0;
#pragma unroll
        for (int j = 0; j < kCMax; ++j)
#pragma unroll
            for (int k = j; k < kCMax; ++k, ++e)
                if ((e & 3) == og) {
                    float g = 0.f;
#pragma unroll
                    for (int u = 0; u < kCVec; ++u) g = fmaf(res[j][u], res[k][u], g);
                    g = warp_sum(g);
                    if (lane == 0) s_part[grp][kCOut + e] = g;
                }
    }
    __syncthreads();                                 // every warp has read the old residual; partials are in shared memory
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");      // second half: every CTA of the cluster has started (long since)
    // push this CTA's 34 sums into slot [crank] of EVERY CTA of the cluster (distributed shared memory stores)
    for (int i = t; i < kCSum * (int)csize; i += blockDim.x) {
        const int c = i / kCSum, k = i - c * kCSum;
        float acc = 0.f;
        for (int g = 0; g < groups; ++g) acc += s_part[g][k];
        *cluster.map_shared_rank(&s_all[crank][k], c) = acc;
    }
    if (og == 0) {
#pragma unroll
        for (int j = 0; j < kCMax; ++j)
            if (j < n) *reinterpret_cast<float4*>(rp + (size_t)j * hidden + h) = make_float4(res[j][0], res[j][1], res[j][2], res[j][3]);
    }
    cluster.sync();                                  // the only cluster barrier of the plain pass: all slices have arrived everywhere

    if (t < kCSum) {
        float acc = 0.f;
        for (int c = 0; c < (int)csize; ++c) acc += s_all[c][t];           // CTA order: the same bits in every CTA
        mix[t] = acc;
    }
    __syncthreads();
    if (w == 0) {
        // all lanes compute the same gates and the Sinkhorn normalisation in registers (no shuffles on the dependent chain)
        float tr = 0.f;
        { int e = 0; for (int j = 0; j < kCMax; ++j) for (int k = j; k < kCMax; ++k, ++e) if (k == j && j < n) tr += mix[kCOut + e]; }
        const float inv = rsqrtf(tr / (float)(n * hidden) + a.rms_eps);
        float cm[kCMax][kCMax];
        const float s2 = a.hc_scale[2];
#pragma unroll
        for (int i = 0; i < kCMax; ++i) {
            float v[kCMax], mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < kCMax; ++j) {
                v[j] = (i < n && j < n) ? mix[2 * n + i * n + j] * inv * s2 + a.hc_base[2 * n + i * n + j] : -INFINITY;
                mx = fmaxf(mx, v[j]);
            }
            float e[kCMax], sm = 0.f;
#pragma unroll
            for (int j = 0; j < kCMax; ++j) { e[j] = (i < n && j < n) ? expf(v[j] - mx) : 0.f; }
            sm = (e[0] + e[1]) + (e[2] + e[3]);
#pragma unroll
            for (int j = 0; j < kCMax; ++j) cm[i][j] = (i < n && j < n) ? e[j] / sm + a.hc_eps : 0.f;
        }
        // column normalise, then (iters - 1) x (row normalise, column normalise)
#pragma unroll
        for (int j = 0; j < kCMax; ++j) {
            const float cs = (cm[0][j] + cm[2][j]) + (cm[1][j] + cm[3][j]);
#pragma unroll
            for (int i = 0; i < kCMax; ++i) cm[i][j] = (i < n && j < n) ? cm[i][j] / (cs + a.hc_eps) : 0.f;
        }
        for (int it = 1; it < a.iters; ++it) {
#pragma unroll
            for (int i = 0; i < kCMax; ++i) {
                const float rs = (cm[i][0] + cm[i][1]) + (cm[i][2] + cm[i][3]);
#pragma unroll
                for (int j = 0; j < kCMax; ++j) cm[i][j] = (i < n && j < n) ? cm[i][j] / (rs + a.hc_eps) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < kCMax; ++j) {
                const float cs = (cm[0][j] + cm[2][j]) + (cm[1][j] + cm[3][j]);
#pragma unroll
                for (int i = 0; i < kCMax; ++i) cm[i][j] = (i < n && j < n) ? cm[i][j] / (cs + a.hc_eps) : 0.f;
            }
        }
        float pj[kCMax];
#pragma unroll
        for (int q = 0; q < kCMax; ++q) pj[q] = q < n ? sigmoidf_(mix[q] * inv * a.hc_scale[0] + a.hc_base[q]) + a.hc_eps : 0.f;
        if (crank == 0) {
#pragma unroll
            for (int i = 0; i < kCMax; ++i)
#pragma unroll
                for (int j = 0; j < kCMax; ++j)
                    if (lane == i * kCMax + j && i < n && j < n) a.comb[(r * n + i) * n + j] = cm[i][j];
            if (lane >= 16 && lane < 16 + kCMax && lane - 16 < n)
                a.post[r * n + (lane - 16)] = sigmoidf_(mix[n + lane - 16] * inv * a.hc_scale[1] + a.hc_base[n + lane - 16]) * a.post_mult;
        }
        if (lane == 0) {
            float quad = 0.f;
            int e = 0;
            for (int p = 0; p < kCMax; ++p)
                for (int q = p; q < kCMax; ++q, ++e) quad += (p == q ? 1.f : 2.f) * pj[p] * pj[q] * mix[kCOut + e];
#pragma unroll
            for (int q = 0; q < kCMax; ++q) s_pre[q] = pj[q];
            s_pre[4] = rsqrtf(fmaxf(quad, 0.f) / (float)hidden + a.rms_eps);
        }
    }
    __syncthreads();

    // ---- contraction + RMSNorm of this CTA's columns ----
    if (og == 0) {
        const float inv = s_pre[4];
        const float nwv[kCVec] = {nw4.x, nw4.y, nw4.z, nw4.w};
        float o[kCVec];
#pragma unroll
        for (int u = 0; u < kCVec; ++u) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < kCMax; ++j) acc = fmaf(j < n ? s_pre[j] : 0.f, res[j][u], acc);
            o[u] = acc * inv * nwv[u];
        }
        const bf162 p0 = __floats2bfloat162_rn(o[0], o[1]), p1 = __floats2bfloat162_rn(o[2], o[3]);
        uint2 pk;
        pk.x = *reinterpret_cast<const uint32_t*>(&p0); pk.y = *reinterpret_cast<const uint32_t*>(&p1);
        *reinterpret_cast<uint2*>(a.out + (size_t)r * hidden + h) = pk;
        const float2 b0 = __bfloat1622float2(p0), b1 = __bfloat1622float2(p1);
        *reinterpret_cast<float4*>(xs + hl) = make_float4(b0.x, b0.y, b1.x, b1.y);
    }
    if (!a.router_w) return;                         // nothing reads a peer's shared memory after the barrier above

    // ---- folded router: partial logits over this CTA's columns, summed over the cluster in CTA order ----
    __syncthreads();
    const int E = a.E, nwarps = blockDim.x >> 5;
    float* s_rl = rdyn;
    for (int e0 = w; e0 < E; e0 += nwarps * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nwarps;
            if (e < E) {
                const float* wr = a.router_w + (size_t)e * hidden + c0;
                for (int k = lane * 4; k < cols; k += 128) {
                    const float4 wv = __ldg(reinterpret_cast<const float4*>(wr + k));
                    acc[u] = fmaf(wv.x, xs[k], acc[u]); acc[u] = fmaf(wv.y, xs[k + 1], acc[u]);
                    acc[u] = fmaf(wv.z, xs[k + 2], acc[u]); acc[u] = fmaf(wv.w, xs[k + 3], acc[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nwarps;
            const float v = warp_sum(acc[u]);
            if (lane == 0 && e < E) s_rl[e] = v;
        }
    }
    cluster.sync();                                  // partial logits published
    float* lg = rdyn + E;                            // full logits of the row, CTA 0 only
    if (crank == 0) {
        for (int e = t; e < E; e += blockDim.x) {
            float v[kCMaxCluster];
#pragma unroll
            for (int c = 0; c < kCMaxCluster; ++c) v[c] = c < (int)csize ? *cluster.map_shared_rank(&s_rl[e], c) : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < kCMaxCluster; ++c) acc += v[c];
            lg[e] = acc;
            if (a.logits) a.logits[(size_t)r * E + e] = acc;
        }
    }
    cluster.sync();                                  // CTA 0 has read every peer's partial logits
    if (crank != 0) return;
    router_topk_block<false>(lg, a.router_bias, a.ids_out + (size_t)r * (a.topk + a.n_shared), a.wts_out + (size_t)r * (a.topk + a.n_shared), E, a.topk,
                             a.n_group, a.topk_group, a.scoring, a.norm_topk, a.scale, a.n_shared, lg + E);
}

static int g_cluster_ok[64] = {0};      // per device: 0 unknown, 1 usable, -1 not usable

// Cluster width (CTAs per row) and column groups per CTA for a hidden size, or 0 when this kernel does not cover it.
static int mhc_cluster_shape(int hidden, int* groups) {
    if (hidden % kCGroupCols) return 0;
    const int units = hidden / kCGroupCols;             // column groups in a row
    int cs = kCMaxCluster;
    while (cs > 1 && (units % cs || units / cs > 2)) cs >>= 1;
    if (units % cs || units / cs > 2) return 0;
    while (cs > 1 && units / cs < 1) cs >>= 1;
    *groups = units / cs;
    return cs;
}

static size_t mhc_cluster_smem(int groups, int E_router) {
    size_t b = (size_t)kCOut * kCMax * groups * kCGroupCols * 4;
    if (E_router) b += (size_t)(2 * E_router + router_topk_smem_floats(E_router)) * 4;
    return b;
}

}  // namespace lsb
using namespace lsb;

static cudaError_t launch_mhc_cluster(const MhcClusterArgs& a, int rows, int csize, int groups, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, rows);
    cfg.blockDim = dim3(groups * 128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = csize; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled_flag() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, mhc_cluster_kernel, a);
}

// Cluster width this device would use for `hidden` (0: not covered - use lsb_mhc_post_pre).  The first call per device asks
// the driver whether a cluster of that width can become resident (16 CTAs per cluster is beyond the portable limit of 8).
LSB_API int lsb_mhc_cluster_width(int hidden, int n) {
    int groups = 0;
    const int cs = mhc_cluster_shape(hidden, &groups);
    if (!cs || n > kCMax) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (g_cluster_ok[dev] == 0) {
        bool ok = true;
        ok = ok && cudaFuncSetAttribute(mhc_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        ok = ok && cudaFuncSetAttribute(mhc_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) == cudaSuccess;
        if (ok) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(kCMaxCluster, 1);
            cfg.blockDim = dim3(256);
            cfg.dynamicSmemBytes = mhc_cluster_smem(2, 512);
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = kCMaxCluster; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int nclusters = 0;
            ok = cudaOccupancyMaxActiveClusters(&nclusters, mhc_cluster_kernel, &cfg) == cudaSuccess && nclusters >= 1;
        }
        cudaGetLastError();
        g_cluster_ok[dev] = ok ? 1 : -1;
    }
    return g_cluster_ok[dev] > 0 ? cs : 0;
}

// One launch for the whole post -> pre pass of `rows` (< 64) token rows; argument meaning as in lsb_mhc_post_pre.
// y / cwts / cids / slot_of / S: optional folded MoE combine (x is then ignored); router_*: optional folded router
// (fp32 weights [E, hidden], logits: optional fp32 [rows, E] copy of the router logits, ids_out / wts_out [rows, topk + n_shared]).
LSB_API int lsb_mhc_cluster(void* out_x, void* residual, const void* x, void* post, void* comb, const void* fn, const void* hc_scale,
                            const void* hc_base, const void* norm_w, int rows, int hidden, int n, int mode, int iters, float hc_eps,
                            float rms_eps, float post_mult, const void* y, const void* cwts, const void* cids, const void* slot_of, int S,
                            const void* router_w, const void* router_bias, void* logits, void* ids_out, void* wts_out, int E, int topk,
                            int n_group, int topk_group, int scoring, int norm_topk, float scale, int n_shared, const void* comm,
                            void* stream) {
    int groups = 0;
    const int cs = lsb_mhc_cluster_width(hidden, n);
    if (!cs || !mhc_cluster_shape(hidden, &groups)) return -1;
    if (y && (S > kCMaxS || comm)) return -1;
    if (router_w && (topk > 32 || n_group > 64 || E > 2048 || n_shared > 32)) return -1;
    if ((((uintptr_t)fn | (uintptr_t)residual | (uintptr_t)x | (uintptr_t)y | (uintptr_t)norm_w | (uintptr_t)router_w) & 15) || ((uintptr_t)out_x & 7)) return -1;
    MhcClusterArgs a;
    a.out = (bf16*)out_x; a.residual = (float*)residual; a.x = (const float*)x; a.post = (float*)post; a.comb = (float*)comb;
    a.fn = (const float*)fn; a.hc_scale = (const float*)hc_scale; a.hc_base = (const float*)hc_base; a.norm_w = (const float*)norm_w;
    a.hidden = hidden; a.n = n; a.mode = mode; a.iters = iters; a.hc_eps = hc_eps; a.rms_eps = rms_eps; a.post_mult = post_mult;
    a.y = (const float*)y; a.cwts = (const float*)cwts; a.cids = (const int*)cids; a.slot_of = (const int*)slot_of; a.S = S;
    a.router_w = (const float*)router_w; a.router_bias = (const float*)router_bias; a.logits = (float*)logits;
    a.ids_out = (int*)ids_out; a.wts_out = (float*)wts_out;
    a.E = E; a.topk = topk; a.n_group = n_group; a.topk_group = topk_group; a.scoring = scoring; a.norm_topk = norm_topk;
    a.n_shared = n_shared; a.scale = scale;
    a.comm.nranks = 0;
    if (comm) a.comm = *reinterpret_cast<const PeerComm*>(comm);
    const size_t smem = mhc_cluster_smem(groups, router_w ? E : 0);
    if (smem > 160 * 1024) return -1;
    cudaError_t e = launch_mhc_cluster(a, rows, cs, groups, smem, (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_mhc_cluster(void* buf) { return lsb_trace_install(buf); }
