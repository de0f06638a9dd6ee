// Kimi Delta Attention (KDA) linear-attention layer body: depthwise causal conv(4)+SiLU on
// q/k/v, low-rank gate tails, the gated delta-rule recurrence with an fp32 [128 v x 128 k]
// state per head, and the gated RMSNorm of the output - one kernel for any number of
// consecutive tokens of a sequence (decode: 1, verify: a few, prefill: a chunk).
//
// Math order (reference: tools/glm53_numpy_ref.py:185-232, tools/gen_kda_golden.py:186-278):
//   q,k,v = SiLU(conv4(raw));  qn = q/sqrt(sum q^2 + 1e-6) * scale;  kn = k/sqrt(sum k^2 + 1e-6)
//   g_log = lower_bound * sigmoid(a_exp * (raw_g + dt_bias));  S *= exp(g_log)[None,:]   (decay first)
//   err = (v - S kn) * sigmoid(beta);  S += err (x) kn;  o = S qn                          (read after write)
//   out = o / sqrt(mean(o^2) + eps) * w_onorm * sigmoid(g2)
// The reference runs this as four external kernels (kda_conv, kda_chunk / kda_decode, gated
// RMSNorm; src/compute/kernels/sm120/attention/kda_linear.h); here thread v owns state row
// S[v][:] in registers, so the token loop needs no cross-thread reduction except the norms.
#include "common.cuh"
#include <cstdlib>

namespace lsb {

#include "kda_types.cuh"

// Shared-memory row stride (bytes) of the staged low-rank gate rows: 16 bytes of padding make the per-thread 16-byte reads
// of 32 different rows conflict-free.
__host__ __device__ constexpr int kda_gate_row_bytes(int rank) { return rank * 2 + 16; }

__global__ void __launch_bounds__(kD) kda_kernel(KdaParams p) {
    __shared__ float s_q[kD], s_k[kD], s_fa[128], s_ga[128], s_red[2][33];
    extern __shared__ __align__(16) uint8_t s_gate[];          // [2][kD] rows of rank bf16 (+ pad): f_b, g_b of this head
    const int seq = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    // everything read before the dependency wait is written by the host or by the PREVIOUS step, never by the predecessor kernel
    const int row0 = p.seq_row0[seq], nrows = p.seq_nrows[seq], slot = p.seq_slot[seq];

    const int C = p.H * kD, ch = h * kD + t;
    const int grb = kda_gate_row_bytes(p.rank);
    {
        // low-rank gate rows of this head -> shared memory (coalesced 16-byte pieces, asynchronously)
        const int per_row = p.rank / 8;                          // 16-byte pieces per row
        const uint8_t* fsrc = reinterpret_cast<const uint8_t*>(p.f_b + (size_t)h * kD * p.rank);
        const uint8_t* gsrc = reinterpret_cast<const uint8_t*>(p.g_b + (size_t)h * kD * p.rank);
        for (int idx = t; idx < kD * per_row; idx += kD) {
            const int rr = idx / per_row, pc = idx - rr * per_row;
            const uint32_t df = (uint32_t)__cvta_generic_to_shared(s_gate + (size_t)rr * grb + pc * 16);
            const uint32_t dg = (uint32_t)__cvta_generic_to_shared(s_gate + (size_t)(kD + rr) * grb + pc * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(df), "l"(fsrc + (size_t)idx * 16) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dg), "l"(gsrc + (size_t)idx * 16) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // state row (an unused sequence slot of the step: nothing to load, and the block leaves only AFTER the dependency wait - a
    // grid whose blocks all exit before it would let its successor overtake the predecessor)
    const bool live = nrows > 0 && slot >= 0;
    float S[kD];
    float* sp = p.state + (((size_t)(live ? slot : 0) * p.H + h) * kD + t) * kD;
    if (live) {
#pragma unroll
        for (int c = 0; c < kD; c += 4) {
            float4 v = *reinterpret_cast<const float4*>(sp + c);
            S[c] = v.x; S[c + 1] = v.y; S[c + 2] = v.z; S[c + 3] = v.w;
        }
    }
    const uint8_t* fb = s_gate + (size_t)t * grb;
    const uint8_t* gb = s_gate + (size_t)(kD + t) * grb;
    pdl_wait();
    pdl_launch_dependents();
    if (!live) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");     // the gate rows in flight target this block's shared memory
        return;
    }
    // conv history (3 raw taps, oldest first) and taps: small, in flight together with the first projection row
    float hq[3], hk[3], hv[3], wq[4], wk[4], wv[4];
    float* csq = p.conv_state + (((size_t)slot * 3 + 0) * C + ch) * 3;
    float* csk = p.conv_state + (((size_t)slot * 3 + 1) * C + ch) * 3;
    float* csv = p.conv_state + (((size_t)slot * 3 + 2) * C + ch) * 3;
#pragma unroll
    for (int j = 0; j < 3; ++j) { hq[j] = csq[j]; hk[j] = csk[j]; hv[j] = csv[j]; }
#pragma unroll
    for (int j = 0; j < 4; ++j) { wq[j] = p.conv_q[ch * 4 + j]; wk[j] = p.conv_k[ch * 4 + j]; wv[j] = p.conv_v[ch * 4 + j]; }
    const float a_exp = p.a_exp[h], dtb = p.dt_bias[ch], ow = p.onorm_w[t];
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    for (int i = 0; i < nrows; ++i) {
        const float* pr = p.proj + (size_t)(row0 + i) * p.ldp;
        const float rq = pr[p.off_q + ch], rk = pr[p.off_k + ch], rv = pr[p.off_v + ch];
        const float beta = sigmoidf_(pr[p.off_beta + h]);
        float q = hq[0] * wq[0]; q += hq[1] * wq[1]; q += hq[2] * wq[2]; q += rq * wq[3];
        float k = hk[0] * wk[0]; k += hk[1] * wk[1]; k += hk[2] * wk[2]; k += rk * wk[3];
        float v = hv[0] * wv[0]; v += hv[1] * wv[1]; v += hv[2] * wv[2]; v += rv * wv[3];
        hq[0] = hq[1]; hq[1] = hq[2]; hq[2] = rq;
        hk[0] = hk[1]; hk[1] = hk[2]; hk[2] = rk;
        hv[0] = hv[1]; hv[1] = hv[2]; hv[2] = rv;
        q = siluf_(q); k = siluf_(k); v = siluf_(v);
        if (t < p.rank) { s_fa[t] = pr[p.off_fa + t]; s_ga[t] = pr[p.off_ga + t]; }
        // both squared norms in one pass over the block (fixed order: warp tree, then warp 0 over the warp partials)
        float qs = warp_sum(q * q), ks = warp_sum(k * k);
        if ((t & 31) == 0) { s_red[0][t >> 5] = qs; s_red[1][t >> 5] = ks; }
        __syncthreads();                                       // also publishes s_fa / s_ga and the staged gate rows
        qs = (s_red[0][0] + s_red[0][1]) + (s_red[0][2] + s_red[0][3]);
        ks = (s_red[1][0] + s_red[1][1]) + (s_red[1][2] + s_red[1][3]);
        s_q[t] = q * rsqrtf(qs + 1e-6f) * p.scale;
        s_k[t] = k * rsqrtf(ks + 1e-6f);
        // low-rank tails: raw_g (per key channel t) and g2 (per value channel t)
        float raw_g = 0.f, g2 = 0.f;
        for (int j = 0; j < p.rank; j += 8) {
            const uint4 a = *reinterpret_cast<const uint4*>(fb + j * 2);
            const uint4 b = *reinterpret_cast<const uint4*>(gb + j * 2);
            float af[8], bfv[8];
            unpack_bf16x8(a, af); unpack_bf16x8(b, bfv);
#pragma unroll
            for (int e = 0; e < 8; ++e) { raw_g = fmaf(af[e], s_fa[j + e], raw_g); g2 = fmaf(bfv[e], s_ga[j + e], g2); }
        }
        const float decay_t = __expf(p.lower_bound * sigmoidf_(a_exp * (raw_g + dtb)));
        // broadcast decay per key channel through shared memory (reuse s_fa after sync)
        __syncthreads();
        s_fa[t] = decay_t;
        __syncthreads();
        // four independent accumulation chains per reduction (a single 128-long dependent FMA chain would bound the step)
        float sk0 = 0.f, sk1 = 0.f, sk2 = 0.f, sk3 = 0.f;
#pragma unroll
        for (int c = 0; c < kD; c += 4) {
            S[c] *= s_fa[c]; sk0 = fmaf(S[c], s_k[c], sk0);
            S[c + 1] *= s_fa[c + 1]; sk1 = fmaf(S[c + 1], s_k[c + 1], sk1);
            S[c + 2] *= s_fa[c + 2]; sk2 = fmaf(S[c + 2], s_k[c + 2], sk2);
            S[c + 3] *= s_fa[c + 3]; sk3 = fmaf(S[c + 3], s_k[c + 3], sk3);
        }
        const float err = (v - ((sk0 + sk1) + (sk2 + sk3))) * beta;
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int c = 0; c < kD; c += 4) {
            S[c] = fmaf(err, s_k[c], S[c]); o0 = fmaf(S[c], s_q[c], o0);
            S[c + 1] = fmaf(err, s_k[c + 1], S[c + 1]); o1 = fmaf(S[c + 1], s_q[c + 1], o1);
            S[c + 2] = fmaf(err, s_k[c + 2], S[c + 2]); o2 = fmaf(S[c + 2], s_q[c + 2], o2);
            S[c + 3] = fmaf(err, s_k[c + 3], S[c + 3]); o3 = fmaf(S[c + 3], s_q[c + 3], o3);
        }
        const float o = (o0 + o1) + (o2 + o3);
        float os = warp_sum(o * o);
        __syncthreads();                                       // s_red is free again
        if ((t & 31) == 0) s_red[0][t >> 5] = os;
        __syncthreads();
        os = (s_red[0][0] + s_red[0][1]) + (s_red[0][2] + s_red[0][3]);
        const float y = o * rsqrtf(os / (float)kD + p.eps) * ow * sigmoidf_(g2);
        p.out[(size_t)(row0 + i) * C + ch] = __float2bfloat16(y);
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < kD; c += 4) *reinterpret_cast<float4*>(sp + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
#pragma unroll
    for (int j = 0; j < 3; ++j) { csq[j] = hq[j]; csk[j] = hk[j]; csv[j] = hv[j]; }
}


// ---------------------------------------------------------------------------------------------
// Many-token path (prefill chunks, verify batches).  Everything that is not part of the
// recurrence is hoisted out of the token loop and runs in parallel over (row, head):
//   kda_prep    conv4+SiLU, q/k L2 norms, low-rank gate tails, decay = exp(lb * sigmoid(..)),
//               output gate sigmoid(g2), beta -> fp32 arrays [rows, C] / [rows, H]
//   kda_recur   the delta rule only: per token 4 x 128 FMAs per thread on the register-resident
//               state row; q/k/decay vectors arrive through a double-buffered cp.async pipeline
//   kda_out     gated RMSNorm of the outputs -> bf16
// The math per token is the one of kda_kernel above, in the same operation order.
constexpr int kTCH = 8;       // tokens per shared-memory pipeline stage


// fp32 low-rank activations -> bf16 (hi | lo) pairs, so that the bf16 tensor-core product with the duplicated weight
// [W | W] reproduces the fp32-activation product to ~2^-16: xs[row][which][0..rank) = hi, [rank..2 rank) = v - hi.
__global__ void __launch_bounds__(128) kda_split_kernel(const float* __restrict__ proj, int ldp, int off_fa, int off_ga, int rank,
                                                        bf16* __restrict__ xs) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const float* pr = proj + (size_t)row * ldp;
    for (int j = threadIdx.x; j < 2 * rank; j += blockDim.x) {
        const int which = j / rank, jj = j - which * rank;
        const float v = pr[(which ? off_ga : off_fa) + jj];
        const bf16 hi = __float2bfloat16(v);
        bf16* o = xs + ((size_t)row * 2 + which) * 2 * rank;
        o[jj] = hi;
        o[rank + jj] = __float2bfloat16(v - __bfloat162float(hi));
    }
    pdl_launch_dependents();
}

constexpr int kPrepRows = 16;   // rows per prep block (amortises staging the head's low-rank matrices)

__global__ void __launch_bounds__(kD) kda_prep_kernel(KdaParams p, KdaScratch w, int nseq, int total_rows) {
    extern __shared__ __align__(16) uint8_t prep_sm[];
    bf16* s_fb = reinterpret_cast<bf16*>(prep_sm);            // [rank][128] transposed: lane-contiguous reads
    bf16* s_gb = s_fb + (size_t)p.rank * kD;
    __shared__ float s_fa[128], s_ga[128], s_red[33];
    const int h = blockIdx.y, t = threadIdx.x;
    const int C = p.H * kD, ch = h * kD + t;
    float wq[4], wk[4], wv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { wq[j] = p.conv_q[ch * 4 + j]; wk[j] = p.conv_k[ch * 4 + j]; wv[j] = p.conv_v[ch * 4 + j]; }
    const float a_exp = p.a_exp[h], dtb = p.dt_bias[ch];
    const bool pre = w.rawg != nullptr;
    if (!pre) {   // weights do not depend on the previous kernel: stage them before the dependency wait
        const bf16* fb = p.f_b + (size_t)ch * p.rank;
        const bf16* gb = p.g_b + (size_t)ch * p.rank;
        for (int j = 0; j < p.rank; j += 8) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(fb + j)), b = __ldg(reinterpret_cast<const uint4*>(gb + j));
            const bf16* ap = reinterpret_cast<const bf16*>(&a);
            const bf16* bp = reinterpret_cast<const bf16*>(&b);
#pragma unroll
            for (int e = 0; e < 8; ++e) { s_fb[(size_t)(j + e) * kD + t] = ap[e]; s_gb[(size_t)(j + e) * kD + t] = bp[e]; }
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    for (int row = blockIdx.x * kPrepRows; row < min(total_rows, (int)(blockIdx.x + 1) * kPrepRows); ++row) {
        int row0 = -1, slot = 0;
        for (int s = 0; s < nseq; ++s) {
            const int r0 = p.seq_row0[s], n = p.seq_nrows[s];
            if (row >= r0 && row < r0 + n) { row0 = r0; slot = p.seq_slot[s]; }
        }
        if (row0 < 0) continue;                              // row belongs to no sequence of this step (uniform per block)
        const int i = row - row0;
        float rq[4], rk[4], rv[4];                           // raw taps, oldest first; [3] = this row
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const int back = 3 - d;                          // tap d is `back` rows before this one
            if (i - back >= 0) {
                const float* pr = p.proj + (size_t)(row - back) * p.ldp;
                rq[d] = pr[p.off_q + ch]; rk[d] = pr[p.off_k + ch]; rv[d] = pr[p.off_v + ch];
            } else {
                const int hi = 3 + i - back;                 // 0..2 in the saved history
                rq[d] = p.conv_state[(((size_t)slot * 3 + 0) * C + ch) * 3 + hi];
                rk[d] = p.conv_state[(((size_t)slot * 3 + 1) * C + ch) * 3 + hi];
                rv[d] = p.conv_state[(((size_t)slot * 3 + 2) * C + ch) * 3 + hi];
            }
        }
        const float* pr = p.proj + (size_t)row * p.ldp;
        float q = rq[0] * wq[0]; q += rq[1] * wq[1]; q += rq[2] * wq[2]; q += rq[3] * wq[3];
        float k = rk[0] * wk[0]; k += rk[1] * wk[1]; k += rk[2] * wk[2]; k += rk[3] * wk[3];
        float v = rv[0] * wv[0]; v += rv[1] * wv[1]; v += rv[2] * wv[2]; v += rv[3] * wv[3];
        q = siluf_(q); k = siluf_(k); v = siluf_(v);
        __syncthreads();                                     // previous row's readers are done with s_fa / s_ga
        if (!pre && t < p.rank) { s_fa[t] = pr[p.off_fa + t]; s_ga[t] = pr[p.off_ga + t]; }
        const float qs = block_sum(q * q, s_red);
        const float ks = block_sum(k * k, s_red);
        __syncthreads();
        const size_t o = (size_t)row * C + ch;
        float raw_g = 0.f, g2 = 0.f;
        if (pre) {
            raw_g = w.rawg[o];
            g2 = w.g2[o];
        } else {
#pragma unroll 8
            for (int j = 0; j < p.rank; ++j) {
                raw_g = fmaf(__bfloat162float(s_fb[(size_t)j * kD + t]), s_fa[j], raw_g);
                g2 = fmaf(__bfloat162float(s_gb[(size_t)j * kD + t]), s_ga[j], g2);
            }
        }
        w.qn[o] = q * rsqrtf(qs + 1e-6f) * p.scale;
        w.kn[o] = k * rsqrtf(ks + 1e-6f);
        w.vo[o] = v;
        w.decay[o] = __expf(p.lower_bound * sigmoidf_(a_exp * (raw_g + dtb)));
        w.gate[o] = sigmoidf_(g2);
        if (t == 0) w.beta[(size_t)row * p.H + h] = sigmoidf_(pr[p.off_beta + h]);
    }
    pdl_launch_dependents();
}

// Many-row prep when the gate products are precomputed: one WARP per row (lane = 4 consecutive channels of the head, 16-byte
// loads and stores, norms by warp shuffles), four rows in flight per block - no block-wide barrier per row.
__global__ void __launch_bounds__(128) kda_prep_rows_kernel(KdaParams p, KdaScratch w, int nseq, int total_rows) {
    const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = p.H * kD, ch = h * kD + lane * 4;
    float wq[4][4], wk[4][4], wv[4][4];                      // [channel][tap]
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float4 a = *reinterpret_cast<const float4*>(p.conv_q + (size_t)(ch + c) * 4);
        const float4 b = *reinterpret_cast<const float4*>(p.conv_k + (size_t)(ch + c) * 4);
        const float4 d = *reinterpret_cast<const float4*>(p.conv_v + (size_t)(ch + c) * 4);
        wq[c][0] = a.x; wq[c][1] = a.y; wq[c][2] = a.z; wq[c][3] = a.w;
        wk[c][0] = b.x; wk[c][1] = b.y; wk[c][2] = b.z; wk[c][3] = b.w;
        wv[c][0] = d.x; wv[c][1] = d.y; wv[c][2] = d.z; wv[c][3] = d.w;
    }
    const float4 dt4 = *reinterpret_cast<const float4*>(p.dt_bias + ch);
    const float dtb[4] = {dt4.x, dt4.y, dt4.z, dt4.w};
    const float a_exp = p.a_exp[h];
    pdl_wait();
    pdl_launch_dependents();
    const int row_end = min(total_rows, (int)(blockIdx.x + 1) * kPrepRows);
    for (int row = blockIdx.x * kPrepRows + warp; row < row_end; row += 4) {
        int row0 = -1, slot = 0;
        for (int s = 0; s < nseq; ++s) {
            const int r0 = p.seq_row0[s], n = p.seq_nrows[s];
            if (row >= r0 && row < r0 + n) { row0 = r0; slot = p.seq_slot[s]; }
        }
        if (row0 < 0) continue;
        const int i = row - row0;
        float q[4] = {0.f, 0.f, 0.f, 0.f}, k[4] = {0.f, 0.f, 0.f, 0.f}, v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int d = 0; d < 4; ++d) {                        // tap d is `3 - d` rows before this one (oldest first)
            const int back = 3 - d;
            float rq[4], rk[4], rv[4];
            if (i - back >= 0) {
                const float* pr = p.proj + (size_t)(row - back) * p.ldp;
                const float4 a = *reinterpret_cast<const float4*>(pr + p.off_q + ch);
                const float4 b = *reinterpret_cast<const float4*>(pr + p.off_k + ch);
                const float4 e = *reinterpret_cast<const float4*>(pr + p.off_v + ch);
                rq[0] = a.x; rq[1] = a.y; rq[2] = a.z; rq[3] = a.w;
                rk[0] = b.x; rk[1] = b.y; rk[2] = b.z; rk[3] = b.w;
                rv[0] = e.x; rv[1] = e.y; rv[2] = e.z; rv[3] = e.w;
            } else {
                const int hi = 3 + i - back;                 // 0..2 in the saved history
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    rq[c] = p.conv_state[(((size_t)slot * 3 + 0) * C + ch + c) * 3 + hi];
                    rk[c] = p.conv_state[(((size_t)slot * 3 + 1) * C + ch + c) * 3 + hi];
                    rv[c] = p.conv_state[(((size_t)slot * 3 + 2) * C + ch + c) * 3 + hi];
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) { q[c] += rq[c] * wq[c][d]; k[c] += rk[c] * wk[c][d]; v[c] += rv[c] * wv[c][d]; }
        }
        float qs = 0.f, ks = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) { q[c] = siluf_(q[c]); k[c] = siluf_(k[c]); v[c] = siluf_(v[c]); qs += q[c] * q[c]; ks += k[c] * k[c]; }
        qs = warp_sum(qs);
        ks = warp_sum(ks);
        const float qi = rsqrtf(qs + 1e-6f) * p.scale, ki = rsqrtf(ks + 1e-6f);
        const size_t o = (size_t)row * C + ch;
        const float4 rg = *reinterpret_cast<const float4*>(w.rawg + o), g2 = *reinterpret_cast<const float4*>(w.g2 + o);
        const float rgv[4] = {rg.x, rg.y, rg.z, rg.w}, g2v[4] = {g2.x, g2.y, g2.z, g2.w};
        float dec[4], gat[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) { dec[c] = __expf(p.lower_bound * sigmoidf_(a_exp * (rgv[c] + dtb[c]))); gat[c] = sigmoidf_(g2v[c]); }
        *reinterpret_cast<float4*>(w.qn + o) = make_float4(q[0] * qi, q[1] * qi, q[2] * qi, q[3] * qi);
        *reinterpret_cast<float4*>(w.kn + o) = make_float4(k[0] * ki, k[1] * ki, k[2] * ki, k[3] * ki);
        *reinterpret_cast<float4*>(w.vo + o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(w.decay + o) = make_float4(dec[0], dec[1], dec[2], dec[3]);
        *reinterpret_cast<float4*>(w.gate + o) = make_float4(gat[0], gat[1], gat[2], gat[3]);
        if (lane == 0) w.beta[(size_t)row * p.H + h] = sigmoidf_(p.proj[(size_t)row * p.ldp + p.off_beta + h]);
    }
    pdl_launch_dependents();
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(kD) kda_recur_kernel(KdaParams p, KdaScratch w) {
    __shared__ __align__(16) float sm[2][3][kTCH][kD];       // [buffer][q,k,decay][token][channel]
    const int seq = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int row0 = p.seq_row0[seq], nrows = p.seq_nrows[seq], slot = p.seq_slot[seq];

    const int C = p.H * kD, ch = h * kD + t;
    float S[kD];
    float* sp = p.state + (((size_t)slot * p.H + h) * kD + t) * kD;
#pragma unroll
    for (int c = 0; c < kD; c += 4) {
        float4 v = *reinterpret_cast<const float4*>(sp + c);
        S[c] = v.x; S[c + 1] = v.y; S[c + 2] = v.z; S[c + 3] = v.w;
    }
    const int nchunks = (nrows + kTCH - 1) / kTCH;
    auto issue = [&](int chunk, int buf) {
        // kTCH tokens x 3 arrays x 128 floats = 768 float4 -> 6 per thread; rows past the end are clamped (unused)
        for (int idx = t; idx < 3 * kTCH * (kD / 4); idx += kD) {
            const int arr = idx / (kTCH * (kD / 4)), rem = idx % (kTCH * (kD / 4));
            const int tok = rem / (kD / 4), c4 = rem % (kD / 4);
            const int row = row0 + min(chunk * kTCH + tok, nrows - 1);
            const float* src = (arr == 0 ? w.qn : (arr == 1 ? w.kn : w.decay)) + (size_t)row * C + h * kD + c4 * 4;
            cp_async_16(&sm[buf][arr][tok][c4 * 4], src);
        }
        cp_async_commit();
    };
    issue(0, 0);
    for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int buf = chunk & 1;
        if (chunk + 1 < nchunks) issue(chunk + 1, buf ^ 1); else cp_async_commit();
        // this thread's v and beta for the chunk
        float vv[kTCH], bb[kTCH];
#pragma unroll
        for (int j = 0; j < kTCH; ++j) {
            const int row = row0 + min(chunk * kTCH + j, nrows - 1);
            vv[j] = w.vo[(size_t)row * C + ch];
            bb[j] = w.beta[(size_t)row * p.H + h];
        }
        cp_async_wait<1>();
        __syncthreads();
        const int ntok = min(kTCH, nrows - chunk * kTCH);
#pragma unroll 1
        for (int j = 0; j < ntok; ++j) {
            const float4* q4 = reinterpret_cast<const float4*>(sm[buf][0][j]);
            const float4* k4 = reinterpret_cast<const float4*>(sm[buf][1][j]);
            const float4* d4 = reinterpret_cast<const float4*>(sm[buf][2][j]);
            // four independent accumulation chains per reduction: one warp per scheduler cannot hide a 128-long
            // dependent FMA chain otherwise
            float sk0 = 0.f, sk1 = 0.f, sk2 = 0.f, sk3 = 0.f;
#pragma unroll
            for (int c = 0; c < kD / 4; ++c) {
                const float4 d = d4[c], k = k4[c];
                S[4 * c] *= d.x; sk0 = fmaf(S[4 * c], k.x, sk0);
                S[4 * c + 1] *= d.y; sk1 = fmaf(S[4 * c + 1], k.y, sk1);
                S[4 * c + 2] *= d.z; sk2 = fmaf(S[4 * c + 2], k.z, sk2);
                S[4 * c + 3] *= d.w; sk3 = fmaf(S[4 * c + 3], k.w, sk3);
            }
            const float sk = (sk0 + sk1) + (sk2 + sk3);
            float vj = vv[0], bj = bb[0];
#pragma unroll
            for (int u = 1; u < kTCH; ++u) if (u == j) { vj = vv[u]; bj = bb[u]; }
            const float err = (vj - sk) * bj;
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int c = 0; c < kD / 4; ++c) {
                const float4 k = k4[c], q = q4[c];
                S[4 * c] = fmaf(err, k.x, S[4 * c]); o0 = fmaf(S[4 * c], q.x, o0);
                S[4 * c + 1] = fmaf(err, k.y, S[4 * c + 1]); o1 = fmaf(S[4 * c + 1], q.y, o1);
                S[4 * c + 2] = fmaf(err, k.z, S[4 * c + 2]); o2 = fmaf(S[4 * c + 2], q.z, o2);
                S[4 * c + 3] = fmaf(err, k.w, S[4 * c + 3]); o3 = fmaf(S[4 * c + 3], q.w, o3);
            }
            const float o = (o0 + o1) + (o2 + o3);
            w.vo[(size_t)(row0 + chunk * kTCH + j) * C + ch] = o;
        }
        __syncthreads();                                     // everyone is done with `buf` before it is refilled
    }
    cp_async_wait<0>();
#pragma unroll
    for (int c = 0; c < kD; c += 4) *reinterpret_cast<float4*>(sp + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
    kda_update_conv_history(p, row0, nrows, slot, ch);
    pdl_launch_dependents();
}

#include "kda_chunk.cuh"

__global__ void __launch_bounds__(kD) kda_out_kernel(KdaParams p, KdaScratch w) {
    __shared__ float s_red[33];
    const int row = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    const int C = p.H * kD, ch = h * kD + t;
    const float ow = p.onorm_w[t];
    pdl_wait();
    pdl_launch_dependents();
    const float o = w.vo[(size_t)row * C + ch];
    const float os = block_sum(o * o, s_red);
    p.out[(size_t)row * C + ch] = __float2bfloat16(o * rsqrtf(os / (float)kD + p.eps) * ow * w.gate[(size_t)row * C + ch]);
    pdl_launch_dependents();
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_gemm_bf16_tc(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx, int ldw,
                             int ldo, int out_bf16, void* partial, long long partial_cap, void* err, const void* comm, void* stream);

static int kda_forward_impl(const void* proj, int ldp, int off_q, int off_k, int off_v, int off_beta, int off_fa,
                            int off_ga, int rank, const void* f_b, const void* g_b, const void* f_b2, const void* g_b2, const void* conv_q,
                            const void* conv_k, const void* conv_v, const void* a_exp, const void* dt_bias,
                            const void* onorm_w, void* state, void* conv_state, const void* seq_row0,
                            const void* seq_nrows, const void* seq_slot, void* out, int nseq, int H, int head_dim,
                            float scale, float lower_bound, float eps, int total_rows, void* scratch, void* chunk_ws, long long chunk_ws_floats,
                            void* stream) {
    if (head_dim != kD || rank > 128 || rank % 8) return -1;
    KdaParams p;
    p.proj = (const float*)proj; p.ldp = ldp; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v; p.off_beta = off_beta;
    p.off_fa = off_fa; p.off_ga = off_ga; p.rank = rank; p.f_b = (const bf16*)f_b; p.g_b = (const bf16*)g_b;
    p.conv_q = (const float*)conv_q; p.conv_k = (const float*)conv_k; p.conv_v = (const float*)conv_v;
    p.a_exp = (const float*)a_exp; p.dt_bias = (const float*)dt_bias; p.onorm_w = (const float*)onorm_w;
    p.state = (float*)state; p.conv_state = (float*)conv_state; p.seq_row0 = (const int*)seq_row0;
    p.seq_nrows = (const int*)seq_nrows; p.seq_slot = (const int*)seq_slot; p.out = (bf16*)out; p.H = H;
    p.scale = scale; p.lower_bound = lower_bound; p.eps = eps;
    cudaStream_t st = (cudaStream_t)stream;
    // A decode batch (every sequence contributes exactly one row) stays on the one-kernel step whatever its size: the many-token
    // pipeline below is three launches built for long runs of rows per sequence (measured at 32 sequences: 190 us against ~35 us).
    if (scratch && total_rows >= 8 && nseq != total_rows) {
        // scratch: fp32 [5][total_rows][H*128], [total_rows][H]; with the duplicated gate weights (f_b2 / g_b2 = [W | W],
        // [C, 2 rank]) also [2][total_rows][H*128] gate products, the bf16 (hi | lo) activations [rows][2][2 rank] and an error word
        const size_t n = (size_t)total_rows * H * kD;
        float* b = (float*)scratch;
        KdaScratch w{b, b + n, b + 2 * n, b + 3 * n, b + 4 * n, b + 5 * n, nullptr, nullptr};
        if (f_b2 && g_b2 && total_rows >= 64 && rank % 8 == 0) {
            float* rawg = b + 5 * n + (((size_t)total_rows * H + 3) & ~(size_t)3);     // keep 16-byte alignment for the GEMM operands
            float* g2 = rawg + n;
            bf16* xs = reinterpret_cast<bf16*>(g2 + n);
            int* gerr = reinterpret_cast<int*>(g2 + n + (size_t)total_rows * 2 * rank);
            launch_pdl((kda_split_kernel), total_rows, 128, 0, st, (const float*)proj, ldp, off_fa, off_ga, rank, xs);
            const int C = H * kD;
            int rc = lsb_gemm_bf16_tc(rawg, xs, f_b2, nullptr, total_rows, C, 2 * rank, 4 * rank, 2 * rank, C, 0, nullptr, 0, gerr, nullptr, stream);
            if (rc) return rc;
            rc = lsb_gemm_bf16_tc(g2, xs + 2 * rank, g_b2, nullptr, total_rows, C, 2 * rank, 4 * rank, 2 * rank, C, 0, nullptr, 0, gerr, nullptr, stream);
            if (rc) return rc;
            w.rawg = rawg; w.g2 = g2;
        }
        const size_t prep_smem = (size_t)2 * rank * kD * sizeof(bf16);
        static bool prep_attr = false;
        if (!prep_attr) { cudaFuncSetAttribute(kda_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 128 * kD * (int)sizeof(bf16)); prep_attr = true; }
        // LSB_KDA_PREP_ROWS=0 keeps the block-per-16-rows prep kernel
        static const bool prep_rows = [] { const char* e = getenv("LSB_KDA_PREP_ROWS"); return e ? atoi(e) != 0 : true; }();
        if (prep_rows && w.rawg && ldp % 4 == 0 && off_q % 4 == 0 && off_k % 4 == 0 && off_v % 4 == 0 && ((uintptr_t)proj & 15) == 0)
            launch_pdl((kda_prep_rows_kernel), dim3((total_rows + kPrepRows - 1) / kPrepRows, H), 128, 0, st, p, w, nseq, total_rows);
        else
            launch_pdl((kda_prep_kernel), dim3((total_rows + kPrepRows - 1) / kPrepRows, H), kD, prep_smem, st, p, w, nseq, total_rows);
        // chunk-parallel recurrence: one sequence per step (its rows are the step's rows), a workspace for W, B and the chunk decays
        const int nch = (total_rows + kCh - 1) / kCh;
        const long long need = (long long)nch * H * (2 * kCh * kCh + kD);
        if (chunk_ws && nseq == 1 && total_rows >= 2 * kCh && need <= chunk_ws_floats && ((uintptr_t)chunk_ws & 15) == 0) {
            static bool chunk_attr = false;
            if (!chunk_attr) {
                cudaFuncSetAttribute(kda_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kChunkPrepSmem);
                cudaFuncSetAttribute(kda_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kChunkScanSmem);
                chunk_attr = true;
            }
            float* cb = (float*)chunk_ws;
            KdaChunkWs cw{cb, cb + (size_t)nch * H * kCh * kCh, cb + (size_t)2 * nch * H * kCh * kCh};
            launch_pdl((kda_chunk_prep_kernel), dim3(nch, H), 256, kChunkPrepSmem, st, p, w, cw);
            launch_pdl((kda_chunk_scan_kernel), dim3(H, kD / kCh), 256, kChunkScanSmem, st, p, w, cw);
        } else {
            launch_pdl((kda_recur_kernel), dim3(nseq, H), kD, 0, st, p, w);
        }
        launch_pdl((kda_out_kernel), dim3(total_rows, H), kD, 0, st, p, w);
    } else {
        const int gate_smem = 2 * kD * kda_gate_row_bytes(rank);
        static bool gate_attr = false;
        if (!gate_attr) { cudaFuncSetAttribute(kda_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kD * kda_gate_row_bytes(128)); gate_attr = true; }
        launch_pdl((kda_kernel), dim3(nseq, H), kD, (size_t)gate_smem, st, p);
    }
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_kda_forward(const void* proj, int ldp, int off_q, int off_k, int off_v, int off_beta, int off_fa,
                            int off_ga, int rank, const void* f_b, const void* g_b, const void* f_b2, const void* g_b2, const void* conv_q,
                            const void* conv_k, const void* conv_v, const void* a_exp, const void* dt_bias,
                            const void* onorm_w, void* state, void* conv_state, const void* seq_row0,
                            const void* seq_nrows, const void* seq_slot, void* out, int nseq, int H, int head_dim,
                            float scale, float lower_bound, float eps, int total_rows, void* scratch, void* stream) {
    return kda_forward_impl(proj, ldp, off_q, off_k, off_v, off_beta, off_fa, off_ga, rank, f_b, g_b, f_b2, g_b2, conv_q, conv_k, conv_v, a_exp,
                            dt_bias, onorm_w, state, conv_state, seq_row0, seq_nrows, seq_slot, out, nseq, H, head_dim, scale, lower_bound,
                            eps, total_rows, scratch, nullptr, 0, stream);
}

// Same, with the recurrence of single-sequence steps of >= 128 rows done chunk-parallel.  ``chunk_ws``: fp32 workspace of
// ``chunk_ws_floats`` >= ceil(rows / 64) * H * (2 * 64 * 64 + 128) floats, 16-byte aligned.
LSB_API int lsb_kda_forward_chunked(const void* proj, int ldp, int off_q, int off_k, int off_v, int off_beta, int off_fa,
                                    int off_ga, int rank, const void* f_b, const void* g_b, const void* f_b2, const void* g_b2,
                                    const void* conv_q, const void* conv_k, const void* conv_v, const void* a_exp, const void* dt_bias,
                                    const void* onorm_w, void* state, void* conv_state, const void* seq_row0,
                                    const void* seq_nrows, const void* seq_slot, void* out, int nseq, int H, int head_dim,
                                    float scale, float lower_bound, float eps, int total_rows, void* scratch, void* chunk_ws,
                                    long long chunk_ws_floats, void* stream) {
    return kda_forward_impl(proj, ldp, off_q, off_k, off_v, off_beta, off_fa, off_ga, rank, f_b, g_b, f_b2, g_b2, conv_q, conv_k, conv_v, a_exp,
                            dt_bias, onorm_w, state, conv_state, seq_row0, seq_nrows, seq_slot, out, nseq, H, head_dim, scale, lower_bound,
                            eps, total_rows, scratch, chunk_ws, chunk_ws_floats, stream);
}

LSB_API int lsb_trace_set_kda(void* buf) { return lsb_trace_install(buf); }
