// RMSNorm family and the hyper-connection (mHC) residual-stream kernels.
//
// RMSNorm: plain, strided, fused residual add (reference: src/compute/kernels/sm120/norm/rmsnorm.cu:71-164).
// mHC: `hc_mult` residual streams per token; "pre" mixes them into the sublayer input
// (sigmoid gates, Sinkhorn-normalised stream-mixing matrix), "post" writes the sublayer
// output back (reference: launchers in src/compute/kernels/mhc/mhc.h, math in
// tools/glm53_numpy_ref.py:128-179).  Here post of sublayer i and pre of sublayer i+1
// are one fused pass: a partial kernel spread over the hidden dimension followed by a
// one-block-per-token finalize that also applies the sublayer's input RMSNorm.
#include "common.cuh"
#include "comm.cuh"

namespace lsb {

template <typename TIn>
__device__ __forceinline__ float ld_as_float(const TIn* p, int i);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p, int i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_as_float<bf16>(const bf16* p, int i) { return __bfloat162float(p[i]); }

// out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * w ; optional: resid[r] += x[r] first and
// normalise the sum (resid updated in place, fp32).
template <typename TIn, bool ADD>
__global__ void rmsnorm_kernel(bf16* __restrict__ out, const TIn* __restrict__ x, float* __restrict__ resid,
                               const float* __restrict__ w, int dim, int ldx, int ldo, int ldr, float eps,
                               float* __restrict__ out_f32, PeerComm comm) {
    __shared__ float red[33];
    extern __shared__ float row[];
    const int r = blockIdx.x;
    const TIn* xr = x + (size_t)r * ldx;
    pdl_wait();
    pdl_launch_dependents();
    unsigned epoch = 0;
    if (comm.nranks) {
        epoch = *comm.epoch;
        if (comm.xchg) {
            // consumer-side exchange: this block ships its row of the local partial to the peers, then waits for theirs
            for (int i = threadIdx.x; i < dim; i += blockDim.x) {
                const float v = ld_as_float<TIn>(xr, i);
                if (comm.xchg == 2) comm_ll_put<1>(comm, epoch, (size_t)r * ldx + i, &v);
                else comm_xchg_put<1>(comm, epoch, (size_t)r * ldx + i, &v);
            }
            if (comm.xchg != 2) comm_xchg_sync(comm, epoch, r);
        } else {
            comm_wait(comm, epoch);
        }
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v;
        if (comm.nranks && comm.xchg == 2) { const float own = ld_as_float<TIn>(xr, i); comm_ll_get<1>(comm, epoch, (size_t)r * ldx + i, &own, &v); }
        else v = comm.nranks ? (comm.xchg ? comm_xchg_get(comm, epoch, (size_t)r * ldx + i, ld_as_float<TIn>(xr, i)) : comm_reduce(comm, epoch, (size_t)r * ldx + i))
                             : ld_as_float<TIn>(xr, i);
        if (ADD) {
            v += resid[(size_t)r * ldr + i];
            resid[(size_t)r * ldr + i] = v;
        }
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = row[i] * inv * w[i];
        out[(size_t)r * ldo + i] = __float2bfloat16(v);
        if (out_f32) out_f32[(size_t)r * ldo + i] = v;
    }
    pdl_launch_dependents();
}

constexpr int kHcMax = 4;           // residual streams
constexpr int kHcOut = 2 * kHcMax + kHcMax * kHcMax;   // 24 mixing logits
constexpr int kHcChunk = 32;        // hidden columns per partial block
constexpr int kHcPerWarp = 6;       // mixing logits per warp (4 warps x 6 = 24)

// Pass 1 of post+pre.  mode 0: residual[j] = x (replicate, first layer);
// mode 1: residual[j] = post[j]*x + sum_i comb[i][j]*residual[i].
// Then partial mixing logits and partial sum of squares of the NEW residual over this
// block's 32 hidden columns: part[r][chunk][0..23] logits, [24] sum of squares.
// Lane = column, warp = a group of 6 mixing logits; every warp recomputes the (cheap) residual
// update, warp 0 stores it.
__global__ void __launch_bounds__(128) mhc_post_partial_kernel(float* __restrict__ residual, const float* __restrict__ x,
                                                               const float* __restrict__ post, const float* __restrict__ comb,
                                                               const float* __restrict__ fn, float* __restrict__ part,
                                                               int hidden, int n, int mode, int rows, int rows_per_block, PeerComm comm) {
    const int c = blockIdx.y, lane = threadIdx.x & 31, og = threadIdx.x >> 5;
    const int h = c * kHcChunk + lane;
    const int nout = 2 * n + n * n;
    // mixing-matrix rows do not depend on the previous kernel: fetch them before the dependency wait
    float f[kHcPerWarp][kHcMax];
#pragma unroll
    for (int i = 0; i < kHcPerWarp; ++i) {
        const int o = og * kHcPerWarp + i;
#pragma unroll
        for (int j = 0; j < kHcMax; ++j) f[i][j] = (o < nout && j < n) ? __ldg(fn + ((size_t)o * n + j) * hidden + h) : 0.f;
    }
    pdl_wait();
    pdl_launch_dependents();
    unsigned epoch = 0;
    if (comm.nranks && mode == 1) {
        epoch = *comm.epoch;
        comm_wait(comm, epoch);
    }
    // a block serves `rows_per_block` consecutive rows with the same register-resident mixing rows
    for (int r = blockIdx.x * rows_per_block; r < min(rows, (int)(blockIdx.x + 1) * rows_per_block); ++r) {
        float res[kHcMax];
        float* rp = residual + (size_t)r * n * hidden;
        const float xv = (comm.nranks && mode == 1) ? comm_reduce(comm, epoch, (size_t)r * hidden + h) : x[(size_t)r * hidden + h];
        if (mode == 0) {
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) res[j] = j < n ? xv : 0.f;
        } else {
            float old[kHcMax];
#pragma unroll
            for (int i = 0; i < kHcMax; ++i) old[i] = i < n ? rp[(size_t)i * hidden + h] : 0.f;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) {
                float a = 0.f;
                if (j < n) {
                    a = post[r * n + j] * xv;
                    for (int i = 0; i < n; ++i) a += comb[(r * n + i) * n + j] * old[i];
                }
                res[j] = a;
            }
        }
        float* po = part + ((size_t)r * gridDim.y + c) * (kHcOut + 1);
#pragma unroll
        for (int i = 0; i < kHcPerWarp; ++i) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) a = fmaf(res[j], f[i][j], a);
            a = warp_sum(a);
            const int o = og * kHcPerWarp + i;
            if (lane == 0 && o < kHcOut) po[o] = a;
        }
        __syncthreads();                              // every warp has read the old streams of this row (in-place update by warp 0)
        if (og == 0) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j)
                if (j < n) { rp[(size_t)j * hidden + h] = res[j]; ss += res[j] * res[j]; }
            ss = warp_sum(ss);
            if (lane == 0) po[kHcOut] = ss;
        }
    }
    pdl_launch_dependents();
}

// Many-row variant of the pass above: a block covers 128 hidden columns (4 consecutive columns per lane, 16-byte
// loads and stores), so the 25 warp reductions per (row, block) amortise over four times the columns - with 2048-row
// prefill chunks the narrow kernel is bound by its shuffles, not by memory.  part[r][chunk128][0..24].
constexpr int kHcWide = 128;
__global__ void __launch_bounds__(128) mhc_post_partial_wide_kernel(float* __restrict__ residual, const float* __restrict__ x,
                                                                    const float* __restrict__ post, const float* __restrict__ comb,
                                                                    const float* __restrict__ fn, float* __restrict__ part,
                                                                    int hidden, int n, int mode, int rows, int rows_per_block, PeerComm comm) {
    const int c = blockIdx.x, lane = threadIdx.x & 31, og = threadIdx.x >> 5;
    const int h = c * kHcWide + lane * 4;
    const int nout = 2 * n + n * n;
    float4 f[kHcPerWarp][kHcMax];
#pragma unroll
    for (int i = 0; i < kHcPerWarp; ++i) {
        const int o = og * kHcPerWarp + i;
#pragma unroll
        for (int j = 0; j < kHcMax; ++j)
            f[i][j] = (o < nout && j < n) ? __ldg(reinterpret_cast<const float4*>(fn + ((size_t)o * n + j) * hidden + h)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    pdl_launch_dependents();
    unsigned epoch = 0;
    if (comm.nranks && mode == 1) {
        epoch = *comm.epoch;
        comm_wait(comm, epoch);
    }
    // The rows of a block are independent but each one is a chain load -> mix -> 7 warp reductions -> store: with one row in
    // flight the block waits a DRAM round trip per row (16 per block).  The next row's operands (x, the four old streams, its
    // post / comb gates: 10 16-byte loads) are therefore requested before the current row is worked on.
    struct RowIn { float4 xv; float4 old[kHcMax]; float pj[kHcMax]; float cj[kHcMax][kHcMax]; };
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    auto load_row = [&](int r, RowIn& in) {
        const float* rp = residual + (size_t)r * n * hidden;
        if (comm.nranks && mode == 1) {
            const size_t b = (size_t)r * hidden + h;
            in.xv = make_float4(comm_reduce(comm, epoch, b), comm_reduce(comm, epoch, b + 1), comm_reduce(comm, epoch, b + 2), comm_reduce(comm, epoch, b + 3));
        } else {
            in.xv = *reinterpret_cast<const float4*>(x + (size_t)r * hidden + h);
        }
        if (mode != 0) {
#pragma unroll
            for (int i = 0; i < kHcMax; ++i) in.old[i] = i < n ? *reinterpret_cast<const float4*>(rp + (size_t)i * hidden + h) : z4;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) {
                in.pj[j] = j < n ? post[r * n + j] : 0.f;
#pragma unroll
                for (int i = 0; i < kHcMax; ++i) in.cj[i][j] = (i < n && j < n) ? comb[(r * n + i) * n + j] : 0.f;
            }
        }
    };
    const int r_begin = blockIdx.y * rows_per_block, r_end = min(rows, (int)(blockIdx.y + 1) * rows_per_block);
    RowIn cur, nxt;
    if (r_begin < r_end) load_row(r_begin, cur);
    for (int r = r_begin; r < r_end; ++r) {
        if (r + 1 < r_end) load_row(r + 1, nxt);      // (rows are disjoint: the in-place store of row r below never touches row r + 1)
        float4 res[kHcMax];
        float* rp = residual + (size_t)r * n * hidden;
        if (mode == 0) {
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) res[j] = j < n ? cur.xv : z4;
        } else {
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) {
                float4 a = z4;
                if (j < n) {
                    const float pj = cur.pj[j];
                    a = make_float4(pj * cur.xv.x, pj * cur.xv.y, pj * cur.xv.z, pj * cur.xv.w);
#pragma unroll
                    for (int i = 0; i < kHcMax; ++i) {
                        if (i < n) {
                            const float cj = cur.cj[i][j];
                            a.x += cj * cur.old[i].x; a.y += cj * cur.old[i].y; a.z += cj * cur.old[i].z; a.w += cj * cur.old[i].w;
                        }
                    }
                }
                res[j] = a;
            }
        }
        float* po = part + ((size_t)r * gridDim.x + c) * (kHcOut + 1);
#pragma unroll
        for (int i = 0; i < kHcPerWarp; ++i) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) {
                a = fmaf(res[j].x, f[i][j].x, a); a = fmaf(res[j].y, f[i][j].y, a);
                a = fmaf(res[j].z, f[i][j].z, a); a = fmaf(res[j].w, f[i][j].w, a);
            }
            a = warp_sum(a);
            const int o = og * kHcPerWarp + i;
            if (lane == 0 && o < kHcOut) po[o] = a;
        }
        // the residual is updated in place by warp 0 while every warp of the block read the old streams of this row above:
        // all of them must have done so before the store (warps drift apart over the row loop)
        __syncthreads();
        if (og == 0) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j)
                if (j < n) {
                    *reinterpret_cast<float4*>(rp + (size_t)j * hidden + h) = res[j];
                    ss += res[j].x * res[j].x + res[j].y * res[j].y + res[j].z * res[j].z + res[j].w * res[j].w;
                }
            ss = warp_sum(ss);
            if (lane == 0) po[kHcOut] = ss;
        }
        cur = nxt;
    }
    pdl_launch_dependents();
}

// Pass 2: reduce the partials in a fixed order, form pre/post gates and the Sinkhorn-
// normalised mixing matrix (one matrix element per lane, sums by shuffles), then
// out = RMSNorm(sum_j pre[j]*residual[j]) * w (bf16).
__global__ void __launch_bounds__(512) mhc_finalize_kernel(bf16* __restrict__ out, const float* __restrict__ residual, const float* __restrict__ part,
                                                           const float* __restrict__ hc_scale, const float* __restrict__ hc_base,
                                                           const float* __restrict__ norm_w, float* __restrict__ post_out, float* __restrict__ comb_out,
                                                           int hidden, int n, int nchunks, int iters, float hc_eps, float rms_eps, float post_mult) {
    __shared__ float red[33];
    __shared__ float mix[kHcOut + 1];
    __shared__ float pre[kHcMax];
    extern __shared__ float row[];
    const int r = blockIdx.x, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    {
        const int o = t >> 4, sub = t & 15;
        float a = 0.f;
        if (o <= kHcOut) {
            // batches of 8 independent loads: the adds must not serialise the memory latency
            for (int c0 = sub; c0 < nchunks; c0 += 128) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int c = c0 + u * 16;
                    v[u] = c < nchunks ? part[((size_t)r * nchunks + c) * (kHcOut + 1) + o] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) a += v[u];
            }
        }
#pragma unroll
        for (int d = 8; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d, 16);
        if (sub == 0 && o <= kHcOut) mix[o] = a;
    }
    __syncthreads();
    if (t < 32) {
        const float inv = rsqrtf(mix[kHcOut] / (float)(n * hidden) + rms_eps);
        if (t < 16) {
            const int i = t >> 2, j = t & 3;
            const bool valid = i < n && j < n;
            float v = valid ? mix[2 * n + i * n + j] * inv * hc_scale[2] + hc_base[2 * n + i * n + j] : -INFINITY;
            float mx = fmaxf(v, __shfl_xor_sync(0xffffu, v, 1, 16));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffu, mx, 2, 16));
            float e = valid ? expf(v - mx) : 0.f;
            float s = e + __shfl_xor_sync(0xffffu, e, 1, 16);
            s += __shfl_xor_sync(0xffffu, s, 2, 16);
            float cm = valid ? e / s + hc_eps : 0.f;
            // column normalise, then (iters-1) x (row normalise, column normalise)
            float cs = cm + __shfl_xor_sync(0xffffu, cm, 4, 16);
            cs += __shfl_xor_sync(0xffffu, cs, 8, 16);
            cm = valid ? cm / (cs + hc_eps) : 0.f;
            for (int it = 1; it < iters; ++it) {
                float rs = cm + __shfl_xor_sync(0xffffu, cm, 1, 16);
                rs += __shfl_xor_sync(0xffffu, rs, 2, 16);
                cm = valid ? cm / (rs + hc_eps) : 0.f;
                cs = cm + __shfl_xor_sync(0xffffu, cm, 4, 16);
                cs += __shfl_xor_sync(0xffffu, cs, 8, 16);
                cm = valid ? cm / (cs + hc_eps) : 0.f;
            }
            if (valid) comb_out[(r * n + i) * n + j] = cm;
        } else if (t < 16 + kHcMax) {
            const int j = t - 16;
            if (j < n) pre[j] = sigmoidf_(mix[j] * inv * hc_scale[0] + hc_base[j]) + hc_eps;
        } else if (t < 16 + 2 * kHcMax) {
            const int j = t - 16 - kHcMax;
            if (j < n) post_out[r * n + j] = sigmoidf_(mix[n + j] * inv * hc_scale[1] + hc_base[n + j]) * post_mult;
        }
    }
    __syncthreads();
    const float* rp = residual + (size_t)r * n * hidden;
    float ss = 0.f;
    float pj[kHcMax];
#pragma unroll
    for (int j = 0; j < kHcMax; ++j) pj[j] = j < n ? pre[j] : 0.f;
    for (int h0 = t; h0 < hidden; h0 += blockDim.x * 4) {
        float v[4][kHcMax];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int h = h0 + u * blockDim.x;
#pragma unroll
            for (int j = 0; j < kHcMax; ++j) v[u][j] = (h < hidden && j < n) ? rp[(size_t)j * hidden + h] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int h = h0 + u * blockDim.x;
            if (h < hidden) {
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < kHcMax; ++j) a += pj[j] * v[u][j];
                row[h] = a;
                ss += a * a;
            }
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + rms_eps);
    for (int h = t; h < hidden; h += blockDim.x) out[(size_t)r * hidden + h] = __float2bfloat16(row[h] * inv * norm_w[h]);
    pdl_launch_dependents();
}


// ---- few-row (decode) variant: two launches instead of partial + one-block-per-row finalize -------------------------------
// mhc_post_fused: same residual update and partial mixing logits as mhc_post_partial, plus the partial Gram matrix
// G[j][j'] = sum_h res_j[h] res_j'[h] of the new residual streams.  The last block of a row to finish (atomic counter)
// reduces the partials in chunk order, forms pre / post and the Sinkhorn-normalised mixing matrix, and gets the RMS of the
// contracted vector algebraically:  sum_h (sum_j pre_j res_j[h])^2 = pre^T G pre  - no second pass over the hidden dimension.
// mhc_contract: out[h] = inv_rms * w[h] * sum_j pre_j res_j[h], fully parallel over the hidden dimension.
constexpr int kHcGram = kHcMax * (kHcMax + 1) / 2;         // 10
constexpr int kHcPart2 = kHcOut + kHcGram + 2;             // 36 floats per (row, chunk)

__global__ void __launch_bounds__(128) mhc_post_fused_kernel(float* __restrict__ residual, const float* __restrict__ x,
                                                             float* __restrict__ post, float* __restrict__ comb,
                                                             const float* __restrict__ fn, const float* __restrict__ hc_scale,
                                                             const float* __restrict__ hc_base, float* __restrict__ part,
                                                             unsigned* __restrict__ done, float* __restrict__ prex, int hidden, int n, int mode,
                                                             int iters, float hc_eps, float rms_eps, float post_mult, PeerComm comm) {
    __shared__ float mix[kHcPart2];
    __shared__ int s_last;
    const int r = blockIdx.x, c = blockIdx.y, lane = threadIdx.x & 31, og = threadIdx.x >> 5, t = threadIdx.x;
    const int nchunks = gridDim.y;
    const int h = c * kHcChunk + lane;
    const int nout = 2 * n + n * n;
    float f[kHcPerWarp][kHcMax];
#pragma unroll
    for (int i = 0; i < kHcPerWarp; ++i) {
        const int o = og * kHcPerWarp + i;
#pragma unroll
        for (int j = 0; j < kHcMax; ++j) f[i][j] = (o < nout && j < n) ? __ldg(fn + ((size_t)o * n + j) * hidden + h) : 0.f;
    }
    pdl_wait();
    pdl_launch_dependents();
    float res[kHcMax];
    float* rp = residual + (size_t)r * n * hidden;
    float xv;
    if (comm.nranks && mode == 1) {
        const unsigned epoch = *comm.epoch;
        comm_wait(comm, epoch);
        xv = comm_reduce(comm, epoch, (size_t)r * hidden + h);
    } else {
        xv = x[(size_t)r * hidden + h];
    }
    if (mode == 0) {
#pragma unroll
        for (int j = 0; j < kHcMax; ++j) res[j] = j < n ? xv : 0.f;
    } else {
        float old[kHcMax];
#pragma unroll
        for (int i = 0; i < kHcMax; ++i) old[i] = i < n ? rp[(size_t)i * hidden + h] : 0.f;
#pragma unroll
        for (int j = 0; j < kHcMax; ++j) {
            float a = 0.f;
            if (j < n) {
                a = post[r * n + j] * xv;
                for (int i = 0; i < n; ++i) a += comb[(r * n + i) * n + j] * old[i];
            }
            res[j] = a;
        }
    }
    float* po = part + ((size_t)r * nchunks + c) * kHcPart2;
#pragma unroll
    for (int i = 0; i < kHcPerWarp; ++i) {
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < kHcMax; ++j) a = fmaf(res[j], f[i][j], a);
        a = warp_sum(a);
        const int o = og * kHcPerWarp + i;
        if (lane == 0 && o < kHcOut) po[o] = a;
    }
    // Gram entries (j <= j'), spread over the four warps: warp w takes entries w, w+4, w+8
    {
        int e = 0;
#pragma unroll
        for (int j = 0; j < kHcMax; ++j)
#pragma unroll
            for (int k = j; k < kHcMax; ++k, ++e)
                if ((e & 3) == og) {
                    const float g = warp_sum(res[j] * res[k]);
                    if (lane == 0) po[kHcOut + e] = g;
                }
    }
    __syncthreads();                                  // every warp has read the old streams (in-place update by warp 0)
    if (og == 0) {
#pragma unroll
        for (int j = 0; j < kHcMax; ++j)
            if (j < n) rp[(size_t)j * hidden + h] = res[j];
    }
    // ---- last block of this row finishes the job ----
    __threadfence();
    __syncthreads();
    if (t == 0) s_last = atomicAdd(done + r, 1u) == (unsigned)(nchunks - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (t < kHcOut + kHcGram) {                       // 34 threads, each sums one column over the chunks in chunk order
        float a = 0.f;
        for (int c0 = 0; c0 < nchunks; c0 += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = c0 + u < nchunks ? __ldcg(part + ((size_t)r * nchunks + c0 + u) * kHcPart2 + t) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) a += v[u];
        }
        mix[t] = a;
    }
    __syncthreads();
    if (t < 32) {
        // sum of squares of the residual streams = trace of the Gram matrix (diagonal entries 0, 4, 7, 9 for n = 4)
        float tr = 0.f;
        { int e = 0; for (int j = 0; j < kHcMax; ++j) for (int k = j; k < kHcMax; ++k, ++e) if (k == j && j < n) tr += mix[kHcOut + e]; }
        const float inv = rsqrtf(tr / (float)(n * hidden) + rms_eps);
        float cm = 0.f;
        const int i = (t & 15) >> 2, j = t & 3;
        const bool valid = t < 16 && i < n && j < n;
        {
            float v = valid ? mix[2 * n + i * n + j] * inv * hc_scale[2] + hc_base[2 * n + i * n + j] : -INFINITY;
            float mx = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float e = valid ? expf(v - mx) : 0.f;
            float sm = e + __shfl_xor_sync(0xffffffffu, e, 1);
            sm += __shfl_xor_sync(0xffffffffu, sm, 2);
            cm = valid ? e / sm + hc_eps : 0.f;
            float cs = cm + __shfl_xor_sync(0xffffffffu, cm, 4);
            cs += __shfl_xor_sync(0xffffffffu, cs, 8);
            cm = valid ? cm / (cs + hc_eps) : 0.f;
            for (int it = 1; it < iters; ++it) {
                float rs = cm + __shfl_xor_sync(0xffffffffu, cm, 1);
                rs += __shfl_xor_sync(0xffffffffu, rs, 2);
                cm = valid ? cm / (rs + hc_eps) : 0.f;
                cs = cm + __shfl_xor_sync(0xffffffffu, cm, 4);
                cs += __shfl_xor_sync(0xffffffffu, cs, 8);
                cm = valid ? cm / (cs + hc_eps) : 0.f;
            }
        }
        if (valid) comb[(r * n + i) * n + j] = cm;
        // pre gates on lanes 16..19, post gates on lanes 20..23
        float pre_v = 0.f;
        if (t >= 16 && t < 16 + kHcMax && t - 16 < n) pre_v = sigmoidf_(mix[t - 16] * inv * hc_scale[0] + hc_base[t - 16]) + hc_eps;
        if (t >= 20 && t < 20 + kHcMax && t - 20 < n) post[r * n + (t - 20)] = sigmoidf_(mix[n + t - 20] * inv * hc_scale[1] + hc_base[n + t - 20]) * post_mult;
        float pj[kHcMax];
#pragma unroll
        for (int q = 0; q < kHcMax; ++q) pj[q] = __shfl_sync(0xffffffffu, pre_v, 16 + q);
        if (t == 0) {
            float quad = 0.f;
            int e = 0;
            for (int a = 0; a < kHcMax; ++a)
                for (int b = a; b < kHcMax; ++b, ++e) quad += (a == b ? 1.f : 2.f) * pj[a] * pj[b] * mix[kHcOut + e];
            float* px = prex + (size_t)r * 8;
#pragma unroll
            for (int q = 0; q < kHcMax; ++q) px[q] = pj[q];
            px[4] = rsqrtf(fmaxf(quad, 0.f) / (float)hidden + rms_eps);
            done[r] = 0;
        }
    }
}

__global__ void __launch_bounds__(256) mhc_contract_kernel(bf16* __restrict__ out, const float* __restrict__ residual, const float* __restrict__ prex,
                                                           const float* __restrict__ norm_w, int hidden, int n) {
    const int r = blockIdx.x;
    const int h = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    float4 w4 = make_float4(0, 0, 0, 0);
    if (h < hidden) w4 = *reinterpret_cast<const float4*>(norm_w + h);
    pdl_wait();
    pdl_launch_dependents();
    if (h >= hidden) return;
    const float* px = prex + (size_t)r * 8;
    const float* rp = residual + (size_t)r * n * hidden + h;
    float4 a = make_float4(0, 0, 0, 0), v[kHcMax];
#pragma unroll
    for (int j = 0; j < kHcMax; ++j) v[j] = j < n ? *reinterpret_cast<const float4*>(rp + (size_t)j * hidden) : make_float4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < kHcMax; ++j) {
        const float p = j < n ? px[j] : 0.f;
        a.x = fmaf(p, v[j].x, a.x); a.y = fmaf(p, v[j].y, a.y); a.z = fmaf(p, v[j].z, a.z); a.w = fmaf(p, v[j].w, a.w);
    }
    const float inv = px[4];
    bf162 o0 = __floats2bfloat162_rn(a.x * inv * w4.x, a.y * inv * w4.y), o1 = __floats2bfloat162_rn(a.z * inv * w4.z, a.w * inv * w4.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&o0); pk.y = *reinterpret_cast<uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(out + (size_t)r * hidden + h) = pk;
}

// Last layer: out = RMSNorm(mean_j(post[j]*x + sum_i comb[i][j]*residual[i])) * w.
__global__ void mhc_contract_norm_kernel(bf16* __restrict__ out, const float* __restrict__ residual, const float* __restrict__ x,
                                         const float* __restrict__ post, const float* __restrict__ comb,
                                         const float* __restrict__ norm_w, int hidden, int n, float rms_eps, PeerComm comm) {
    __shared__ float red[33];
    extern __shared__ float row[];
    const int r = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    unsigned epoch = 0;
    if (comm.nranks) {
        epoch = *comm.epoch;
        if (comm.xchg) {
            for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
                const float v = x[(size_t)r * hidden + h];
                if (comm.xchg == 2) comm_ll_put<1>(comm, epoch, (size_t)r * hidden + h, &v);
                else comm_xchg_put<1>(comm, epoch, (size_t)r * hidden + h, &v);
            }
            if (comm.xchg != 2) comm_xchg_sync(comm, epoch, r);
        } else {
            comm_wait(comm, epoch);
        }
    }
    const float* rp = residual + (size_t)r * n * hidden;
    float pm = 0.f, cw[kHcMax];
    for (int j = 0; j < n; ++j) pm += post[r * n + j];
    for (int i = 0; i < n; ++i) {
        float s = 0.f;
        for (int j = 0; j < n; ++j) s += comb[(r * n + i) * n + j];
        cw[i] = s;
    }
    float ss = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float xs_;
        if (comm.nranks && comm.xchg == 2) { const float own = x[(size_t)r * hidden + h]; comm_ll_get<1>(comm, epoch, (size_t)r * hidden + h, &own, &xs_); }
        else xs_ = comm.nranks ? (comm.xchg ? comm_xchg_get(comm, epoch, (size_t)r * hidden + h, x[(size_t)r * hidden + h])
                                            : comm_reduce(comm, epoch, (size_t)r * hidden + h))
                               : x[(size_t)r * hidden + h];
        float a = pm * xs_;
        for (int i = 0; i < n; ++i) a += cw[i] * rp[(size_t)i * hidden + h];
        a /= (float)n;
        row[h] = a;
        ss += a * a;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + rms_eps);
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) out[(size_t)r * hidden + h] = __float2bfloat16(row[h] * inv * norm_w[h]);
    pdl_launch_dependents();
}


// Producer half of the in-kernel all-reduce for partials that a kernel without a fused epilogue has already written to
// local memory: stores x[m][n] (fp32, row stride ld) into slot[this rank] of every rank's receive buffer and publishes
// the epoch.  The consumer (add_rmsnorm / mHC kernels with `comm`) sums the slots in rank order.
__global__ void __launch_bounds__(256) comm_push_rows_kernel(const float* __restrict__ x, int ld, int N, long long total, PeerComm c) {
    pdl_wait();
    pdl_launch_dependents();
    const unsigned next_epoch = *c.epoch + 1u;
    if (c.xchg) {          // the consuming kernel exchanges the (already local) partial itself
        if ((blockIdx.x | threadIdx.x) == 0) *c.epoch = next_epoch;
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / N;
        comm_push(c, next_epoch, (size_t)i, x[m * ld + (i - m * N)]);
    }
    comm_signal(c, next_epoch, gridDim.x);
    pdl_launch_dependents();
}
}  // namespace lsb
using namespace lsb;

static PeerComm comm_from_host(const void* h) {
    PeerComm c;
    c.nranks = 0;
    if (h) c = *reinterpret_cast<const PeerComm*>(h);
    return c;
}

// Push a locally computed fp32 partial [M, N] (row stride ld) as this rank's contribution to the next all-reduce epoch.
LSB_API int lsb_comm_push_rows(const void* x, int M, int N, int ld, const void* comm, void* stream) {
    if (!comm) return -1;
    const PeerComm c = comm_from_host(comm);
    const long long total = (long long)M * N;
    if (c.nranks <= 0 || total > c.cap) return -2;
    const int grid = (int)((total + 256 * 8 - 1) / (256 * 8) < 592 ? (total + 256 * 8 - 1) / (256 * 8) : 592);
    launch_pdl((comm_push_rows_kernel), grid > 0 ? grid : 1, 256, 0, (cudaStream_t)stream, (const float*)x, ld, N, total, c);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_rmsnorm(void* out, const void* x, const void* w, int rows, int dim, int ldx, int ldo, float eps,
                        int x_is_f32, void* out_f32, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    PeerComm nocomm;
    nocomm.nranks = 0;
    const int thr = dim >= 2048 ? 512 : 256;
    const size_t sm = (size_t)dim * 4;
    if (x_is_f32)
        launch_pdl((rmsnorm_kernel<float, false>), rows, thr, sm, st, (bf16*)out, (const float*)x, nullptr, (const float*)w, dim, ldx, ldo, 0, eps, (float*)out_f32, nocomm);
    else
        launch_pdl((rmsnorm_kernel<bf16, false>), rows, thr, sm, st, (bf16*)out, (const bf16*)x, nullptr, (const float*)w, dim, ldx, ldo, 0, eps, (float*)out_f32, nocomm);
    LSB_CHECK_LAUNCH();
}

// resid (fp32, in place) += x (fp32); out = RMSNorm(resid) * w as bf16.  With `comm`, x is the
// cross-rank sum of the partials the producing kernel pushed (fused all-reduce).
LSB_API int lsb_add_rmsnorm(void* out, void* resid, const void* x, const void* w, int rows, int dim, float eps, const void* comm,
                            void* stream) {
    const int thr = dim >= 2048 ? 512 : 256;
    launch_pdl((rmsnorm_kernel<float, true>), rows, thr, (size_t)dim * 4, (cudaStream_t)stream, (bf16*)out, (const float*)x, (float*)resid,
                                                                                   (const float*)w, dim, dim, dim, dim, eps, nullptr, comm_from_host(comm));
    LSB_CHECK_LAUNCH();
}

// residual: fp32 [rows, n, hidden] updated in place; x: fp32 [rows, hidden] sublayer output
// (or the embedding when mode == 0); post/comb: state from the previous finalize (in) and
// for the next post (out, same buffers).  part: scratch fp32 [rows, hidden/32, 25].
LSB_API int lsb_mhc_post_pre(void* out_x, void* residual, const void* x, void* post, void* comb, const void* fn,
                             const void* hc_scale, const void* hc_base, const void* norm_w, void* part, int rows,
                             int hidden, int n, int mode, int iters, float hc_eps, float rms_eps, float post_mult,
                             void* done, void* prex, const void* comm, void* stream) {
    if (hidden % kHcChunk || n > kHcMax) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    const int nchunks = hidden / kHcChunk;
    if (done && prex && rows < 64 && hidden % 4 == 0) {
        // few rows: partials + finalize in one launch (last block per row), then a fully parallel contraction.
        // part must hold rows * nchunks * 36 floats, done rows zero-initialised counters, prex rows * 8 floats.
        launch_pdl((mhc_post_fused_kernel), dim3(rows, nchunks), 128, 0, st, (float*)residual, (const float*)x, (float*)post, (float*)comb,
                   (const float*)fn, (const float*)hc_scale, (const float*)hc_base, (float*)part, (unsigned*)done, (float*)prex, hidden, n, mode,
                   iters, hc_eps, rms_eps, post_mult, comm_from_host(comm));
        launch_pdl((mhc_contract_kernel), dim3(rows, (hidden / 4 + 255) / 256), 256, 0, st, (bf16*)out_x, (const float*)residual, (const float*)prex,
                   (const float*)norm_w, hidden, n);
        LSB_CHECK_LAUNCH();
    }
    const int rpb = rows >= 64 ? 16 : 1;      // many rows: amortise the mixing-matrix loads over 16 rows per block
    int nparts = nchunks;
    if (rows >= 64 && hidden % kHcWide == 0) {
        nparts = hidden / kHcWide;
        // hidden parts are the fastest grid dimension: the blocks that run together read whole rows of the residual streams (16 KB
        // runs) instead of 512-byte pieces 64 KB apart
        launch_pdl((mhc_post_partial_wide_kernel), dim3(nparts, (rows + rpb - 1) / rpb), 128, 0, st, (float*)residual, (const float*)x, (const float*)post,
                   (const float*)comb, (const float*)fn, (float*)part, hidden, n, mode, rows, rpb, comm_from_host(comm));
    } else {
        launch_pdl((mhc_post_partial_kernel), dim3((rows + rpb - 1) / rpb, nchunks), 128, 0, st, (float*)residual, (const float*)x, (const float*)post,
                   (const float*)comb, (const float*)fn, (float*)part, hidden, n, mode, rows, rpb, comm_from_host(comm));
    }
    launch_pdl((mhc_finalize_kernel), rows, 512, (size_t)hidden * 4, st, (bf16*)out_x, (const float*)residual, (const float*)part,
                                                              (const float*)hc_scale, (const float*)hc_base, (const float*)norm_w,
                                                              (float*)post, (float*)comb, hidden, n, nparts, iters, hc_eps, rms_eps, post_mult);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_mhc_contract_norm(void* out, const void* residual, const void* x, const void* post, const void* comb,
                                  const void* norm_w, int rows, int hidden, int n, float rms_eps, const void* comm, void* stream) {
    launch_pdl((mhc_contract_norm_kernel), rows, 512, (size_t)hidden * 4, (cudaStream_t)stream, (bf16*)out, (const float*)residual, (const float*)x,
                                                                                      (const float*)post, (const float*)comb,
                                                                                      (const float*)norm_w, hidden, n, rms_eps, comm_from_host(comm));
    LSB_CHECK_LAUNCH();
}

// out[r] = cos(a[r], b[r]) over `dim` bf16 elements (0 when either vector is all zero): how much a layer changed its input.
__global__ void __launch_bounds__(256) cosine_sim_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, int dim, int lda, int ldb,
                                                         float* __restrict__ out) {
    __shared__ float red[3][33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    float ab = 0.f, aa = 0.f, bb = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float x = __bfloat162float(a[(size_t)r * lda + i]), y = __bfloat162float(b[(size_t)r * ldb + i]);
        ab = fmaf(x, y, ab); aa = fmaf(x, x, aa); bb = fmaf(y, y, bb);
    }
    ab = block_sum(ab, red[0]); aa = block_sum(aa, red[1]); bb = block_sum(bb, red[2]);
    if (threadIdx.x == 0) out[r] = (aa > 0.f && bb > 0.f) ? ab * rsqrtf(aa) * rsqrtf(bb) : 0.f;
}

// Cosine similarity of `rows` pairs of bf16 vectors (layer skipping: the input of a layer against the input of the next one).
// Reference: src/compute/kernels/similarity/cosine_sim.h (one pair per call, output on the device).
LSB_API int lsb_cosine_sim(const void* a, const void* b, int rows, int dim, int lda, int ldb, void* out, void* stream) {
    if (rows <= 0 || dim <= 0) return -1;
    launch_pdl((cosine_sim_kernel), rows, 256, 0, (cudaStream_t)stream, (const bf16*)a, (const bf16*)b, dim, lda, ldb, (float*)out);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_norm(void* buf) { return lsb_trace_install(buf); }
