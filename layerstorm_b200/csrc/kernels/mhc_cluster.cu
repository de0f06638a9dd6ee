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

template <int VEC> struct VecT;
template <> struct VecT<1> { using T = float; };
template <> struct VecT<2> { using T = float2; };

template <int VEC> __device__ __forceinline__ typename VecT<VEC>::T vld(const float* p);
template <> __device__ __forceinline__ float vld<1>(const float* p) { return *p; }
template <> __device__ __forceinline__ float2 vld<2>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <int VEC> __device__ __forceinline__ typename VecT<VEC>::T vldg(const float* p);
template <> __device__ __forceinline__ float vldg<1>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float2 vldg<2>(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }

template <int VEC>
__global__ void __launch_bounds__(512, 1) mhc_cluster_kernel(const __grid_constant__ MhcClusterArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned crank = cluster.block_rank(), csize = cluster.num_blocks();
    __shared__ float s_part[4][kCSum];
    __shared__ float s_cta[kCSum + 2];
    __shared__ float mix[kCSum + 2];
    __shared__ float s_pre[8];
    __shared__ float xs[4 * 32 * VEC];
    extern __shared__ float dyn[];                  // router: [E] partial logits, [E] logits, top-k scratch
    const int t = threadIdx.x, lane = t & 31, w = t >> 5, og = w & 3, grp = w >> 2;
    const int groups = blockDim.x >> 7;
    const int r = blockIdx.y;
    const int n = a.n, hidden = a.hidden;
    const int cols = groups * 32 * VEC;             // columns of this CTA
    const int c0 = (int)crank * cols;
    const int hl = grp * 32 * VEC + lane * VEC;     // column inside the CTA slice
    const int h = c0 + hl;
    const int nout = 2 * n + n * n;

    // mixing rows: independent of the previous kernel
    float f[kCPerWarp][kCMax][VEC];
#pragma unroll
    for (int i = 0; i < kCPerWarp; ++i) {
        const int o = og * kCPerWarp + i;
#pragma unroll
        for (int j = 0; j < kCMax; ++j) {
            if (o < nout && j < n) {
                const typename VecT<VEC>::T v = vldg<VEC>(a.fn + ((size_t)o * n + j) * hidden + h);
                memcpy(f[i][j], &v, sizeof(v));
            } else {
#pragma unroll
                for (int u = 0; u < VEC; ++u) f[i][j][u] = 0.f;
            }
        }
    }
    float nw[VEC];
    {
        const typename VecT<VEC>::T v = vldg<VEC>(a.norm_w + h);
        memcpy(nw, &v, sizeof(v));
    }
    if (a.router_w) {
        // the router rows of this CTA's column slice: start them towards L2 under the predecessor's tail
        for (int e = w; e < a.E; e += (int)(blockDim.x >> 5))
            for (int k = lane * 32; k < cols; k += 32 * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.router_w + (size_t)e * hidden + c0 + k));
    }
    pdl_wait();
    pdl_launch_dependents();

    // ---- sublayer output for this thread's columns ----
    float xv[VEC];
    if (a.comm.nranks && a.mode == 1 && a.comm.xchg) {
        // consumer-side exchange: this CTA ships its columns of the local partial to the peers, publishes one flag and waits for
        // the same CTA of every peer - no producer-side copy, and a CTA only waits for the columns it needs
        const unsigned epoch = *a.comm.epoch;
        const typename VecT<VEC>::T q = vld<VEC>(a.x + (size_t)r * hidden + h);
        float own[VEC];
        memcpy(own, &q, sizeof(q));
        if (a.comm.xchg == 2) {
            // flag-in-data words: no fence, no flag, no barrier - every warp polls the words of its own columns
            if (og == 0) comm_ll_put<VEC>(a.comm, epoch, (size_t)r * hidden + h, own);
            comm_ll_get<VEC>(a.comm, epoch, (size_t)r * hidden + h, own, xv);
        } else {
            if (og == 0) comm_xchg_put<VEC>(a.comm, epoch, (size_t)r * hidden + h, own);
            comm_xchg_sync(a.comm, epoch, (int)(blockIdx.y * gridDim.x + blockIdx.x));
#pragma unroll
            for (int u = 0; u < VEC; ++u) xv[u] = comm_xchg_get(a.comm, epoch, (size_t)r * hidden + h + u, own[u]);
        }
    } else if (a.comm.nranks && a.mode == 1) {
        const unsigned epoch = *a.comm.epoch;
        comm_wait(a.comm, epoch);
#pragma unroll
        for (int u = 0; u < VEC; ++u) xv[u] = comm_reduce(a.comm, epoch, (size_t)r * hidden + h + u);
    } else if (a.y) {
        int e[kCMaxS];
        float wt[kCMaxS];
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s) { e[s] = s < a.S ? a.cids[r * a.S + s] : -1; wt[s] = s < a.S ? a.cwts[r * a.S + s] : 0.f; }
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s) if (e[s] >= 0 && a.slot_of[e[s]] < 0) e[s] = -1;
        float v[kCMaxS][VEC];
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s) {
            if (e[s] >= 0) {
                const typename VecT<VEC>::T q = vld<VEC>(a.y + ((size_t)r * a.S + s) * hidden + h);
                memcpy(v[s], &q, sizeof(q));
            } else {
#pragma unroll
                for (int u = 0; u < VEC; ++u) v[s][u] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < VEC; ++u) xv[u] = 0.f;
#pragma unroll
        for (int s = 0; s < kCMaxS; ++s)
            if (e[s] >= 0) {
#pragma unroll
                for (int u = 0; u < VEC; ++u) xv[u] = fmaf(wt[s], v[s][u], xv[u]);
            }
    } else {
        const typename VecT<VEC>::T q = vld<VEC>(a.x + (size_t)r * hidden + h);
        memcpy(xv, &q, sizeof(q));
    }

    // ---- new residual streams (every warp of a column group recomputes them; warp og 0 stores) ----
    float res[kCMax][VEC];
    float* rp = a.residual + (size_t)r * n * hidden;
    if (a.mode == 0) {
#pragma unroll
        for (int j = 0; j < kCMax; ++j)
#pragma unroll
            for (int u = 0; u < VEC; ++u) res[j][u] = j < n ? xv[u] : 0.f;
    } else {
        float old[kCMax][VEC];
#pragma unroll
        for (int i = 0; i < kCMax; ++i) {
            if (i < n) {
                const typename VecT<VEC>::T q = vld<VEC>(rp + (size_t)i * hidden + h);
                memcpy(old[i], &q, sizeof(q));
            } else {
#pragma unroll
                for (int u = 0; u < VEC; ++u) old[i][u] = 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < kCMax; ++j) {
            float acc[VEC];
#pragma unroll
            for (int u = 0; u < VEC; ++u) acc[u] = 0.f;
            if (j < n) {
                const float pj = a.post[r * n + j];
#pragma unroll
                for (int u = 0; u < VEC; ++u) acc[u] = pj * xv[u];
                for (int i = 0; i < n; ++i) {
                    const float cj = a.comb[(r * n + i) * n + j];
#pragma unroll
                    for (int u = 0; u < VEC; ++u) acc[u] += cj * old[i][u];
                }
            }
#pragma unroll
            for (int u = 0; u < VEC; ++u) res[j][u] = acc[u];
        }
    }

    // ---- partial mixing logits and Gram entries over this warp's columns ----
#pragma unroll
    for (int i = 0; i < kCPerWarp; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < kCMax; ++j)
#pragma unroll
            for (int u = 0; u < VEC; ++u) acc = fmaf(res[j][u], f[i][j][u], acc);
        acc = warp_sum(acc);
        const int o = og * kCPerWarp + i;
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
                    for (int u = 0; u < VEC; ++u) g = fmaf(res[j][u], res[k][u], g);
                    g = warp_sum(g);
                    if (lane == 0) s_part[grp][kCOut + e] = g;
                }
    }
    __syncthreads();                                 // every warp has read the old residual; partials are in shared memory
    if (t < kCSum) {
        float acc = 0.f;
        for (int g = 0; g < groups; ++g) acc += s_part[g][t];
        s_cta[t] = acc;
    }
    if (og == 0) {
#pragma unroll
        for (int j = 0; j < kCMax; ++j)
            if (j < n) {
                typename VecT<VEC>::T q;
                memcpy(&q, res[j], sizeof(q));
                *reinterpret_cast<typename VecT<VEC>::T*>(rp + (size_t)j * hidden + h) = q;
            }
    }
    cluster.sync();                                  // #1: all slices published

    if (t < kCSum) {
        float v[kCMaxCluster];
#pragma unroll
        for (int c = 0; c < kCMaxCluster; ++c) v[c] = c < (int)csize ? *cluster.map_shared_rank(&s_cta[t], c) : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < kCMaxCluster; ++c) acc += v[c];
        mix[t] = acc;
    }
    __syncthreads();
    if (w == 0) {
        // sum of squares of the residual streams = trace of the Gram matrix
        float tr = 0.f;
        { int e = 0; for (int j = 0; j < kCMax; ++j) for (int k = j; k < kCMax; ++k, ++e) if (k == j && j < n) tr += mix[kCOut + e]; }
        const float inv = rsqrtf(tr / (float)(n * hidden) + a.rms_eps);
        float cm = 0.f;
        const int i = (t & 15) >> 2, j = t & 3;
        const bool valid = t < 16 && i < n && j < n;
        {
            float v = valid ? mix[2 * n + i * n + j] * inv * a.hc_scale[2] + a.hc_base[2 * n + i * n + j] : -INFINITY;
            float mx = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float e = valid ? expf(v - mx) : 0.f;
            float sm = e + __shfl_xor_sync(0xffffffffu, e, 1);
            sm += __shfl_xor_sync(0xffffffffu, sm, 2);
            cm = valid ? e / sm + a.hc_eps : 0.f;
            float cs = cm + __shfl_xor_sync(0xffffffffu, cm, 4);
            cs += __shfl_xor_sync(0xffffffffu, cs, 8);
            cm = valid ? cm / (cs + a.hc_eps) : 0.f;
            for (int it = 1; it < a.iters; ++it) {
                float rs = cm + __shfl_xor_sync(0xffffffffu, cm, 1);
                rs += __shfl_xor_sync(0xffffffffu, rs, 2);
                cm = valid ? cm / (rs + a.hc_eps) : 0.f;
                cs = cm + __shfl_xor_sync(0xffffffffu, cm, 4);
                cs += __shfl_xor_sync(0xffffffffu, cs, 8);
                cm = valid ? cm / (cs + a.hc_eps) : 0.f;
            }
        }
        if (valid && crank == 0) a.comb[(r * n + i) * n + j] = cm;
        // pre gates on lanes 16..19, post gates on lanes 20..23
        float pre_v = 0.f;
        if (t >= 16 && t < 16 + kCMax && t - 16 < n) pre_v = sigmoidf_(mix[t - 16] * inv * a.hc_scale[0] + a.hc_base[t - 16]) + a.hc_eps;
        if (crank == 0 && t >= 20 && t < 20 + kCMax && t - 20 < n)
            a.post[r * n + (t - 20)] = sigmoidf_(mix[n + t - 20] * inv * a.hc_scale[1] + a.hc_base[n + t - 20]) * a.post_mult;
        float pj[kCMax];
#pragma unroll
        for (int q = 0; q < kCMax; ++q) pj[q] = __shfl_sync(0xffffffffu, pre_v, 16 + q);
        if (t == 0) {
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
        float o[VEC];
#pragma unroll
        for (int u = 0; u < VEC; ++u) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < kCMax; ++j) acc = fmaf(j < n ? s_pre[j] : 0.f, res[j][u], acc);
            o[u] = acc * inv * nw[u];
        }
        if (VEC == 2) {
            const bf162 p = __floats2bfloat162_rn(o[0], o[VEC - 1]);
            *reinterpret_cast<bf162*>(a.out + (size_t)r * hidden + h) = p;
            const float2 back = __bfloat1622float2(p);
            xs[hl] = back.x; xs[hl + VEC - 1] = back.y;
        } else {
            const bf16 p = __float2bfloat16(o[0]);
            a.out[(size_t)r * hidden + h] = p;
            xs[hl] = __bfloat162float(p);
        }
    }
    if (!a.router_w) {
        cluster.sync();                              // #2: nobody leaves while a peer may still read its partial sums
        return;
    }

    // ---- folded router: partial logits over this CTA's columns, summed over the cluster in CTA order ----
    __syncthreads();
    const int E = a.E, nwarps = blockDim.x >> 5;
    float* s_rl = dyn;
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
    cluster.sync();                                  // #2: partial logits published (and all reads of the partial sums done)
    float* lg = dyn + E;                             // full logits of the row, CTA 0 only
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
    cluster.sync();                                  // #3: CTA 0 has read every peer's partial logits
    if (crank != 0) return;
    router_topk_block<false>(lg, a.router_bias, a.ids_out + (size_t)r * (a.topk + a.n_shared), a.wts_out + (size_t)r * (a.topk + a.n_shared), E, a.topk,
                             a.n_group, a.topk_group, a.scoring, a.norm_topk, a.scale, a.n_shared, lg + E);
}

static int g_cluster_ok[64] = {0};      // per device: 0 unknown, 1 usable, -1 not usable

// Cluster width (CTAs per row) and column groups per CTA for a hidden size, or 0 when this kernel does not cover it.
static int mhc_cluster_shape(int hidden, int* groups, int* vec) {
    if (hidden % 32) return 0;
    for (int v = 2; v >= 1; --v) {
        const int unit = 32 * v;                    // columns of one column group
        if (hidden % unit) continue;
        int cs = kCMaxCluster;
        while (cs > 1 && (hidden % (cs * unit) || hidden / (cs * unit) < 1)) cs >>= 1;
        const int g = hidden / (cs * unit);
        if (hidden % (cs * unit) == 0 && g >= 1 && g <= 4) { *groups = g; *vec = v; return cs; }
    }
    return 0;
}

}  // namespace lsb
using namespace lsb;

template <int VEC>
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
    return cudaLaunchKernelEx(&cfg, mhc_cluster_kernel<VEC>, a);
}

// Cluster width this device would use for `hidden` (0: not covered - use lsb_mhc_post_pre).  The first call per device asks
// the driver whether a cluster of that width can become resident (16 CTAs per cluster is beyond the portable limit of 8).
LSB_API int lsb_mhc_cluster_width(int hidden, int n) {
    int groups = 0, vec = 0;
    const int cs = mhc_cluster_shape(hidden, &groups, &vec);
    if (!cs || n > kCMax) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (g_cluster_ok[dev] == 0) {
        bool ok = true;
        ok = ok && cudaFuncSetAttribute(mhc_cluster_kernel<1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        ok = ok && cudaFuncSetAttribute(mhc_cluster_kernel<2>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        if (ok) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(kCMaxCluster, 1);
            cfg.blockDim = dim3(512);
            cfg.dynamicSmemBytes = 16 * 1024;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = kCMaxCluster; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int nclusters = 0;
            ok = cudaOccupancyMaxActiveClusters(&nclusters, mhc_cluster_kernel<2>, &cfg) == cudaSuccess && nclusters >= 1;
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
    int groups = 0, vec = 0;
    const int cs = lsb_mhc_cluster_width(hidden, n);
    if (!cs || !mhc_cluster_shape(hidden, &groups, &vec)) return -1;
    if (y && (S > kCMaxS || comm)) return -1;
    if (router_w && (topk > 32 || n_group > 64 || E > 2048 || n_shared > 32 || (groups * 32 * vec) % 4)) return -1;
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
    const size_t smem = router_w ? (size_t)(2 * E + router_topk_smem_floats(E)) * 4 : 0;
    if (smem > 48 * 1024) return -1;
    cudaError_t e = vec == 2 ? launch_mhc_cluster<2>(a, rows, cs, groups, smem, (cudaStream_t)stream)
                             : launch_mhc_cluster<1>(a, rows, cs, groups, smem, (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_mhc_cluster(void* buf) { return lsb_trace_install(buf); }
