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

namespace lsb {

constexpr int kD = 128;   // head dim (key and value)

struct KdaParams {
    const float* proj;      // [rows, ldp] fp32: q | k | v | beta | f_a | g_a
    int ldp, off_q, off_k, off_v, off_beta, off_fa, off_ga, rank;
    const bf16* f_b;        // [H*128, rank]
    const bf16* g_b;        // [H*128, rank]
    const float* conv_q;    // [H*128, 4]
    const float* conv_k;
    const float* conv_v;
    const float* a_exp;     // [H]
    const float* dt_bias;   // [H,128]
    const float* onorm_w;   // [128]
    float* state;           // [slots, H, 128, 128]
    float* conv_state;      // [slots, 3(qkv), H*128, 3] oldest first
    const int* seq_row0;    // [nseq] first row of each sequence in this step
    const int* seq_nrows;   // [nseq]
    const int* seq_slot;    // [nseq] state slot
    bf16* out;              // [rows, H*128]
    int H;
    float scale, lower_bound, eps;
};

__global__ void __launch_bounds__(kD) kda_kernel(KdaParams p) {
    __shared__ float s_q[kD], s_k[kD], s_fa[128], s_ga[128], s_red[33];
    const int seq = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    const int row0 = p.seq_row0[seq], nrows = p.seq_nrows[seq], slot = p.seq_slot[seq];
    if (nrows <= 0) return;
    const int C = p.H * kD, ch = h * kD + t;
    pdl_wait();
    pdl_launch_dependents();
    // state row
    float S[kD];
    float* sp = p.state + (((size_t)slot * p.H + h) * kD + t) * kD;
#pragma unroll
    for (int c = 0; c < kD; c += 4) {
        float4 v = *reinterpret_cast<const float4*>(sp + c);
        S[c] = v.x; S[c + 1] = v.y; S[c + 2] = v.z; S[c + 3] = v.w;
    }
    // conv history (3 raw taps, oldest first) and taps
    float hq[3], hk[3], hv[3], wq[4], wk[4], wv[4];
    float* csq = p.conv_state + (((size_t)slot * 3 + 0) * C + ch) * 3;
    float* csk = p.conv_state + (((size_t)slot * 3 + 1) * C + ch) * 3;
    float* csv = p.conv_state + (((size_t)slot * 3 + 2) * C + ch) * 3;
#pragma unroll
    for (int j = 0; j < 3; ++j) { hq[j] = csq[j]; hk[j] = csk[j]; hv[j] = csv[j]; }
#pragma unroll
    for (int j = 0; j < 4; ++j) { wq[j] = p.conv_q[ch * 4 + j]; wk[j] = p.conv_k[ch * 4 + j]; wv[j] = p.conv_v[ch * 4 + j]; }
    const float a_exp = p.a_exp[h], dtb = p.dt_bias[ch], ow = p.onorm_w[t];
    const bf16* fb = p.f_b + (size_t)ch * p.rank;
    const bf16* gb = p.g_b + (size_t)ch * p.rank;

    for (int i = 0; i < nrows; ++i) {
        const float* pr = p.proj + (size_t)(row0 + i) * p.ldp;
        const float rq = pr[p.off_q + ch], rk = pr[p.off_k + ch], rv = pr[p.off_v + ch];
        float q = hq[0] * wq[0]; q += hq[1] * wq[1]; q += hq[2] * wq[2]; q += rq * wq[3];
        float k = hk[0] * wk[0]; k += hk[1] * wk[1]; k += hk[2] * wk[2]; k += rk * wk[3];
        float v = hv[0] * wv[0]; v += hv[1] * wv[1]; v += hv[2] * wv[2]; v += rv * wv[3];
        hq[0] = hq[1]; hq[1] = hq[2]; hq[2] = rq;
        hk[0] = hk[1]; hk[1] = hk[2]; hk[2] = rk;
        hv[0] = hv[1]; hv[1] = hv[2]; hv[2] = rv;
        q = siluf_(q); k = siluf_(k); v = siluf_(v);
        if (t < p.rank) { s_fa[t] = pr[p.off_fa + t]; s_ga[t] = pr[p.off_ga + t]; }
        const float qs = block_sum(q * q, s_red);
        const float ks = block_sum(k * k, s_red);
        s_q[t] = q * rsqrtf(qs + 1e-6f) * p.scale;
        s_k[t] = k * rsqrtf(ks + 1e-6f);
        __syncthreads();
        // low-rank tails: raw_g (per key channel t) and g2 (per value channel t)
        float raw_g = 0.f, g2 = 0.f;
        for (int j = 0; j < p.rank; j += 8) {
            uint4 a = __ldg(reinterpret_cast<const uint4*>(fb + j));
            uint4 b = __ldg(reinterpret_cast<const uint4*>(gb + j));
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
        const float beta = sigmoidf_(pr[p.off_beta + h]);
        float sk = 0.f;
#pragma unroll
        for (int c = 0; c < kD; ++c) { S[c] *= s_fa[c]; sk = fmaf(S[c], s_k[c], sk); }
        const float err = (v - sk) * beta;
        float o = 0.f;
#pragma unroll
        for (int c = 0; c < kD; ++c) { S[c] = fmaf(err, s_k[c], S[c]); o = fmaf(S[c], s_q[c], o); }
        const float os = block_sum(o * o, s_red);
        const float y = o * rsqrtf(os / (float)kD + p.eps) * ow * sigmoidf_(g2);
        p.out[(size_t)(row0 + i) * C + ch] = __float2bfloat16(y);
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < kD; c += 4) *reinterpret_cast<float4*>(sp + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
#pragma unroll
    for (int j = 0; j < 3; ++j) { csq[j] = hq[j]; csk[j] = hk[j]; csv[j] = hv[j]; }
    pdl_launch_dependents();
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_kda_forward(const void* proj, int ldp, int off_q, int off_k, int off_v, int off_beta, int off_fa,
                            int off_ga, int rank, const void* f_b, const void* g_b, const void* conv_q,
                            const void* conv_k, const void* conv_v, const void* a_exp, const void* dt_bias,
                            const void* onorm_w, void* state, void* conv_state, const void* seq_row0,
                            const void* seq_nrows, const void* seq_slot, void* out, int nseq, int H, int head_dim,
                            float scale, float lower_bound, float eps, void* stream) {
    if (head_dim != kD || rank > 128 || rank % 8) return -1;
    KdaParams p;
    p.proj = (const float*)proj; p.ldp = ldp; p.off_q = off_q; p.off_k = off_k; p.off_v = off_v; p.off_beta = off_beta;
    p.off_fa = off_fa; p.off_ga = off_ga; p.rank = rank; p.f_b = (const bf16*)f_b; p.g_b = (const bf16*)g_b;
    p.conv_q = (const float*)conv_q; p.conv_k = (const float*)conv_k; p.conv_v = (const float*)conv_v;
    p.a_exp = (const float*)a_exp; p.dt_bias = (const float*)dt_bias; p.onorm_w = (const float*)onorm_w;
    p.state = (float*)state; p.conv_state = (float*)conv_state; p.seq_row0 = (const int*)seq_row0;
    p.seq_nrows = (const int*)seq_nrows; p.seq_slot = (const int*)seq_slot; p.out = (bf16*)out; p.H = H;
    p.scale = scale; p.lower_bound = lower_bound; p.eps = eps;
    launch_pdl((kda_kernel), dim3(nseq, H), kD, 0, (cudaStream_t)stream, p);
    LSB_CHECK_LAUNCH();
}
