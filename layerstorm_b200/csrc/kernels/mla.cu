// Multi-head latent attention (MLA), absorbed form, over a paged quantised latent cache.
//
// Layer math (reference: src/daemon/attention/arch_mla.cpp:47-312,1824-1994):
//   q_c = RMSNorm(W_qa h);  q = W_qb q_c -> [H, d_nope + d_rope]
//   q_abs[h] = [ q_nope[h] . W_UK[h] (-> d_c) | RoPE(q_rope[h]) ]
//   kv = W_kva h -> [d_c + d_rope];  c = RMSNorm(kv[:d_c]);  k_pe = RoPE(kv[d_c:]);  cache row = (c, k_pe)
//   attention in latent space (all heads share the cached row), output [H, d_c] -> W_UV per head.
// RoPE rotates interleaved adjacent pairs.
//
// Cache row formats (kv_fmt):
//   0  bf16: (d_c + d_rope) bf16
//   1  fp8 : d_c e4m3 bytes | fp32 per-token scale (+12 pad bytes) | d_rope bf16
//          (the reference's FP8+BF16-RoPE row: its design document under docs/, line 126; K/sm120/prep/fused_k_append.cu)
//   2  tq4 : d_c / 2 bytes of 4-bit codes (low nibble = even index) | fp32 row scale (+12 pad bytes) | d_rope bf16
//          TurboQuant: the latent is L2-normalised, rotated by a fixed per-layer orthogonal matrix and every coordinate
//          (times sqrt(d_c), ~N(0,1)) is replaced by the nearest of 16 Lloyd-Max centroids; row scale = norm / sqrt(d_c).
//          Attention runs in the rotated space: the rotation is folded into W_UK / W_UV when the weights are loaded, so
//          decode only swaps the row loader (reference: 386-byte TurboQuant rows, src/compute/tq_init.h, docs/INTERNALS.md:8-9).
// Pages hold `page` consecutive tokens; a sequence's pages are listed in its block table.
#include "common.cuh"
#include <cstdlib>
#include "gemv_core.cuh"

namespace lsb {

__host__ __device__ inline int kv_row_bytes(int fmt, int dl, int dr) {
    return fmt == 0 ? (dl + dr) * 2 : (fmt == 1 ? dl + 16 + dr * 2 : dl / 2 + 16 + dr * 2);
}

__device__ __forceinline__ void rope_pair(float& a, float& b, float pos, float inv_freq) {
    float s, c;
    sincosf(pos * inv_freq, &s, &c);
    const float x = a * c - b * s, y = a * s + b * c;
    a = x; b = y;
}

// One block per row: q_c = RMSNorm(q_a) (bf16 out), latent RMSNorm, RoPE on k_pe, cache append.
__global__ void mla_prep_kernel(const float* __restrict__ proj, int ldp, int off_qa, int q_lora, int off_kv, int dl, int dr,
                                const float* __restrict__ qa_norm_w, const float* __restrict__ kv_norm_w,
                                const float* __restrict__ inv_freq, bf16* __restrict__ q_c, uint8_t* __restrict__ cache,
                                const int* __restrict__ block_table, int max_pages, const int* __restrict__ row_seq,
                                const int* __restrict__ row_pos, int page, int kv_fmt, float eps,
                                const bf16* __restrict__ tq_rot_t, const float* __restrict__ tq_centroids,
                                const int* __restrict__ row_store) {
    __shared__ float red[33];
    extern __shared__ float sm[];   // [max(q_lora, dl + dr)]
    const int r = blockIdx.x, t = threadIdx.x;
    const float* pr = proj + (size_t)r * ldp;
    pdl_wait();
    pdl_launch_dependents();
    // two blocks per row (gridDim.y == 2): block y = 0 normalises the query latent, block y = 1 does the KV row - the two chains of
    // dependent reductions and memory round trips run side by side instead of back to back
    if (q_lora > 0 && (gridDim.y == 1 || blockIdx.y == 0)) {
        float ss = 0.f;
        for (int i = t; i < q_lora; i += blockDim.x) { const float v = pr[off_qa + i]; sm[i] = v; ss += v * v; }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)q_lora + eps);
        for (int i = t; i < q_lora; i += blockDim.x) q_c[(size_t)r * q_lora + i] = __float2bfloat16(sm[i] * inv * qa_norm_w[i]);
        __syncthreads();
    }
    if (gridDim.y == 2 && blockIdx.y == 0) return;
    float ss = 0.f;
    for (int i = t; i < dl; i += blockDim.x) { const float v = pr[off_kv + i]; sm[i] = v; ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)dl + eps);
    float amax = 0.f;
    for (int i = t; i < dl; i += blockDim.x) { const float v = sm[i] * inv * kv_norm_w[i]; sm[i] = v; amax = fmaxf(amax, fabsf(v)); }
    const int seq = row_seq[r], pos = row_pos[r];
    for (int i = t; i < dr / 2; i += blockDim.x) {
        float a = pr[off_kv + dl + 2 * i], b = pr[off_kv + dl + 2 * i + 1];
        rope_pair(a, b, (float)pos, inv_freq[i]);
        sm[dl + 2 * i] = a; sm[dl + 2 * i + 1] = b;
    }
    amax = block_max(amax, red);   // also orders the shared-memory writes above
    // row_store (context-parallel cache shards): index of this row inside the local shard, < 0 = another rank stores it;
    // the rotary phase above always uses the global position
    const int spos = row_store ? row_store[r] : pos;
    if (seq < 0 || spos < 0) return;
    const int pg = block_table[(size_t)seq * max_pages + spos / page];
    const int rb = kv_row_bytes(kv_fmt, dl, dr);
    uint8_t* row = cache + ((size_t)pg * page + (spos % page)) * rb;
    if (kv_fmt == 0) {
        bf16* o = reinterpret_cast<bf16*>(row);
        for (int i = t; i < dl + dr; i += blockDim.x) o[i] = __float2bfloat16(sm[i]);
    } else if (kv_fmt == 2) {
        // rotated unit vector u' = Pi (c / |c|); tq_rot_t is Pi transposed, so consecutive threads read consecutive bytes
        float n2 = 0.f;
        for (int i = t; i < dl; i += blockDim.x) n2 += sm[i] * sm[i];
        n2 = block_sum(n2, red);
        const float norm = sqrtf(fmaxf(n2, 1e-30f));
        const float up = sqrtf((float)dl) / norm;                 // coordinates of the unit vector times sqrt(d): ~N(0,1)
        float cent[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) cent[j] = tq_centroids[j];
        for (int i0 = 2 * t; i0 < dl; i0 += 2 * blockDim.x) {    // two coordinates -> one byte
            float a0 = 0.f, a1 = 0.f;
            for (int k = 0; k < dl; ++k) {
                const bf162 w2 = *reinterpret_cast<const bf162*>(tq_rot_t + (size_t)k * dl + i0);
                const float ck = sm[k];
                a0 = fmaf(__low2float(w2), ck, a0); a1 = fmaf(__high2float(w2), ck, a1);
            }
            a0 *= up; a1 *= up;
            int c0 = 0, c1 = 0;
#pragma unroll
            for (int j = 1; j < 16; ++j) {                        // centroids ascend: count the midpoints below the value
                const float mid = 0.5f * (cent[j - 1] + cent[j]);
                c0 += a0 > mid; c1 += a1 > mid;
            }
            row[i0 >> 1] = (uint8_t)(c0 | (c1 << 4));
        }
        if (t == 0) *reinterpret_cast<float*>(row + dl / 2) = norm / sqrtf((float)dl);
        bf16* o = reinterpret_cast<bf16*>(row + dl / 2 + 16);
        for (int i = t; i < dr; i += blockDim.x) o[i] = __float2bfloat16(sm[dl + i]);
    } else {
        const float scale = fmaxf(amax, 1e-10f) / 448.f;
        const float inv_s = 1.f / scale;
        for (int i = t; i < dl; i += blockDim.x) row[i] = float_to_fp8e4m3(sm[i] * inv_s);
        if (t == 0) *reinterpret_cast<float*>(row + dl) = scale;
        bf16* o = reinterpret_cast<bf16*>(row + dl + 16);
        for (int i = t; i < dr; i += blockDim.x) o[i] = __float2bfloat16(sm[dl + i]);
    }
    pdl_launch_dependents();
}

// out[m][b][n] = sum_k x[m][b][k] * W[b][n][k]; used for W_UK absorption and the W_UV up-projection.
// Optional RoPE tail: out[m][b][N + i] = RoPE(x[m][b][K + i]) for i < dr (query rope half).
template <int MT>
__global__ void __launch_bounds__(256) batched_gemv_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                           int N, int K, long long xs_m, long long xs_b, long long os_m,
                                                           long long os_b, int dr, const float* __restrict__ inv_freq,
                                                           const int* __restrict__ row_pos, int m_base) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    const int n0 = (blockIdx.x * 8 + warp) * 2;
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x == 0 && dr > 0) {
        for (int m = 0; m < MT; ++m)
            for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
                const bf16* xp = x + (size_t)m * xs_m + (size_t)b * xs_b + K;
                float a0 = __bfloat162float(xp[2 * i]), a1 = __bfloat162float(xp[2 * i + 1]);
                rope_pair(a0, a1, (float)row_pos[m_base + m], inv_freq[i]);
                bf16* o = out + (size_t)m * os_m + (size_t)b * os_b + N;
                o[2 * i] = __float2bfloat16(a0); o[2 * i + 1] = __float2bfloat16(a1);
            }
    }
    if (n0 >= N) return;
    const int n1 = min(n0 + 1, N - 1);
    const bf16* wb = w + (size_t)b * N * K;
    WRowBf16 r0{wb + (size_t)n0 * K}, r1{wb + (size_t)n1 * K};
    float a0[MT], a1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) a0[m] = a1[m] = 0.f;
    warp_dot2<WRowBf16, MT>(r0, r1, x + (size_t)b * xs_b, (int)xs_m, K, a0, a1);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float v0 = warp_sum(a0[m]), v1 = warp_sum(a1[m]);
        if (lane == 0) {
            bf16* o = out + (size_t)m * os_m + (size_t)b * os_b;
            o[n0] = __float2bfloat16(v0);
            if (n0 + 1 < N) o[n0 + 1] = __float2bfloat16(v1);
        }
    }
    pdl_launch_dependents();
}

// RoPE of the query rope half for the many-row path (the GEMM part runs on the tensor cores).
__global__ void rope_tail_kernel(bf16* __restrict__ out, const bf16* __restrict__ x, int N, int K, long long xs_m, long long xs_b,
                                 long long os_m, long long os_b, int dr, const float* __restrict__ inv_freq, const int* __restrict__ row_pos) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.x, b = blockIdx.y;
    const bf16* xp = x + (size_t)m * xs_m + (size_t)b * xs_b + K;
    bf16* o = out + (size_t)m * os_m + (size_t)b * os_b + N;
    for (int i = threadIdx.x; i < dr / 2; i += blockDim.x) {
        float a0 = __bfloat162float(xp[2 * i]), a1 = __bfloat162float(xp[2 * i + 1]);
        rope_pair(a0, a1, (float)row_pos[m], inv_freq[i]);
        o[2 * i] = __float2bfloat16(a0); o[2 * i + 1] = __float2bfloat16(a1);
    }
    pdl_launch_dependents();
}

constexpr int kHG = 16;   // heads per block
constexpr int kTK = 32;   // cache rows per tile

struct MlaDecodeParams {
    const bf16* q;            // [R, H, dl + dr]
    const uint8_t* cache;
    const int* block_table; int max_pages;
    const int* row_seq; const int* row_len;     // causal length (tokens visible) per row
    const int* sel_idx; const int* sel_cnt; int sel_ld;   // optional sparse selection (token positions)
    float* o_part; float* ml_part;              // [R,H,NS,dl], [R,H,NS,2]
    int H, dl, dr, page, kv_fmt, NS;
    float scale;
    const float* tq_centroids;   // kv_fmt 2: the 16 reconstruction levels
};

// Loads KT cache rows (token positions s_tok[0..KT), -1 = none) into the bf16 tile Ks[KT][DP]: latent part expanded
// from the cache format (bf16 copy, FP8 e4m3 -> bf16 exactly, TurboQuant codes -> centroids), rope part copied, the
// per-row latent scale into sc[].
__device__ __forceinline__ void mla_load_tile(const MlaDecodeParams& p, int seq, int rb, const int* s_tok, bf16* Ks, float* sc, int DP, int D,
                                              int t, int nthr, int KT) {
    if (p.kv_fmt == 0) {
        const int cpr = D / 8;
        for (int i = t; i < KT * cpr; i += nthr) {
            const int j = i / cpr, c = i % cpr, tok = s_tok[j];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok >= 0) {
                const int pg = p.block_table[(size_t)seq * p.max_pages + tok / p.page];
                v = *reinterpret_cast<const uint4*>(p.cache + ((size_t)pg * p.page + tok % p.page) * rb + c * 16);
            }
            *reinterpret_cast<uint4*>(Ks + j * DP + c * 8) = v;
        }
        if (t < KT) sc[t] = 1.f;
    } else if (p.kv_fmt == 2) {
        const int c32 = p.dl / 32, cr = p.dr / 8, cpr = c32 + cr;   // 16 bytes = 32 codes
        for (int i = t; i < KT * cpr; i += nthr) {
            const int j = i / cpr, c = i % cpr, tok = s_tok[j];
            const uint8_t* row = nullptr;
            if (tok >= 0) {
                const int pg = p.block_table[(size_t)seq * p.max_pages + tok / p.page];
                row = p.cache + ((size_t)pg * p.page + tok % p.page) * rb;
            }
            if (c < c32) {
                const uint4 v = row ? *reinterpret_cast<const uint4*>(row + c * 16) : make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
                const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
                bf162* o = reinterpret_cast<bf162*>(Ks + j * DP + c * 32);
#pragma unroll
                for (int b = 0; b < 16; ++b) {
                    const uint32_t byte = (wv[b >> 2] >> (8 * (b & 3))) & 0xffu;
                    o[b] = __floats2bfloat162_rn(row ? __ldg(p.tq_centroids + (byte & 15u)) : 0.f, row ? __ldg(p.tq_centroids + (byte >> 4)) : 0.f);
                }
            } else {
                const int cc = c - c32;
                uint4 v = row ? *reinterpret_cast<const uint4*>(row + p.dl / 2 + 16 + cc * 16) : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(Ks + j * DP + p.dl + cc * 8) = v;
            }
        }
        if (t < KT) {
            const int tok = s_tok[t];
            float s = 0.f;
            if (tok >= 0) {
                const int pg = p.block_table[(size_t)seq * p.max_pages + tok / p.page];
                s = *reinterpret_cast<const float*>(p.cache + ((size_t)pg * p.page + tok % p.page) * rb + p.dl / 2);
            }
            sc[t] = s;
        }
    } else {
        const int c8 = p.dl / 16, cr = p.dr / 8, cpr = c8 + cr;
        for (int i = t; i < KT * cpr; i += nthr) {
            const int j = i / cpr, c = i % cpr, tok = s_tok[j];
            const uint8_t* row = nullptr;
            if (tok >= 0) {
                const int pg = p.block_table[(size_t)seq * p.max_pages + tok / p.page];
                row = p.cache + ((size_t)pg * p.page + tok % p.page) * rb;
            }
            if (c < c8) {
                uint4 v = row ? *reinterpret_cast<const uint4*>(row + c * 16) : make_uint4(0, 0, 0, 0);
                float f[16];
                unpack_fp8x4(v.x, f); unpack_fp8x4(v.y, f + 4); unpack_fp8x4(v.z, f + 8); unpack_fp8x4(v.w, f + 12);
                bf162* o = reinterpret_cast<bf162*>(Ks + j * DP + c * 16);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);   // e4m3 -> bf16 is exact
            } else {
                const int cc = c - c8;
                uint4 v = row ? *reinterpret_cast<const uint4*>(row + p.dl + 16 + cc * 16) : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(Ks + j * DP + p.dl + cc * 8) = v;
            }
        }
        if (t < KT) {
            const int tok = s_tok[t];
            float s = 0.f;
            if (tok >= 0) {
                const int pg = p.block_table[(size_t)seq * p.max_pages + tok / p.page];
                s = *reinterpret_cast<const float*>(p.cache + ((size_t)pg * p.page + tok % p.page) * rb + p.dl);
            }
            sc[t] = s;
        }
    }
}

__global__ void __launch_bounds__(256) mla_decode_kernel(MlaDecodeParams p) {
    extern __shared__ __align__(16) uint8_t smraw[];
    const int D = p.dl + p.dr, DP = D + 8;     // padded bf16 row (16 B mod 128 B => conflict-free 128-bit reads)
    bf16* Ks = reinterpret_cast<bf16*>(smraw);                 // [kTK][DP]
    bf16* Qs = Ks + kTK * DP;                                   // [kHG][DP]
    float* Ps = reinterpret_cast<float*>(Qs + kHG * DP);        // [kTK][kHG]
    float* sc = Ps + kTK * kHG;                                 // [kTK] row scales
    float* s_m = sc + kTK;                                      // [kHG]
    float* s_l = s_m + kHG;                                     // [kHG]
    float* s_alpha = s_l + kHG;                                 // [kHG]
    int* s_tok = reinterpret_cast<int*>(s_alpha + kHG);         // [kTK]
    const int r = blockIdx.x, hg = blockIdx.y, sp = blockIdx.z;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    pdl_wait();
    pdl_launch_dependents();
    const int seq = p.row_seq[r];
    int n = p.sel_idx ? p.sel_cnt[r] : p.row_len[r];
    if (seq < 0) n = 0;
    const int per = (((n + p.NS - 1) / p.NS) + kTK - 1) / kTK * kTK;
    const int beg = sp * per, end = min(n, beg + per);
    // stage q for this head group
    for (int i = t; i < kHG * (D / 8); i += blockDim.x) {
        const int h = i / (D / 8), c = i % (D / 8);
        const int hh = hg * kHG + h;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (hh < p.H) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)r * p.H + hh) * D + c * 8);
        *reinterpret_cast<uint4*>(Qs + h * DP + c * 8) = v;
    }
    if (t < kHG) { s_m[t] = -INFINITY; s_l[t] = 0.f; }
    float acc[kHG][2];
#pragma unroll
    for (int h = 0; h < kHG; ++h) acc[h][0] = acc[h][1] = 0.f;
    const int rb = kv_row_bytes(p.kv_fmt, p.dl, p.dr);
    for (int t0 = beg; t0 < end; t0 += kTK) {
        __syncthreads();
        if (t < kTK) {
            const int i = t0 + t;
            int tok = -1;
            if (i < end) tok = p.sel_idx ? p.sel_idx[(size_t)r * p.sel_ld + i] : i;
            s_tok[t] = tok;
        }
        __syncthreads();
        mla_load_tile(p, seq, rb, s_tok, Ks, sc, DP, D, t, blockDim.x, kTK);
        __syncthreads();
        // scores: warp -> heads (2w, 2w+1); lane -> cache row
        {
            const int h0 = 2 * warp, h1 = h0 + 1;
            float s0 = 0.f, s1 = 0.f, r0 = 0.f, r1 = 0.f;
            const bf16* kr = Ks + lane * DP;
            for (int d = 0; d < p.dl; d += 8) {
                float kf[8], q0[8], q1[8];
                unpack_bf16x8(*reinterpret_cast<const uint4*>(kr + d), kf);
                unpack_bf16x8(*reinterpret_cast<const uint4*>(Qs + h0 * DP + d), q0);
                unpack_bf16x8(*reinterpret_cast<const uint4*>(Qs + h1 * DP + d), q1);
#pragma unroll
                for (int e = 0; e < 8; ++e) { s0 = fmaf(kf[e], q0[e], s0); s1 = fmaf(kf[e], q1[e], s1); }
            }
            for (int d = p.dl; d < D; d += 8) {
                float kf[8], q0[8], q1[8];
                unpack_bf16x8(*reinterpret_cast<const uint4*>(kr + d), kf);
                unpack_bf16x8(*reinterpret_cast<const uint4*>(Qs + h0 * DP + d), q0);
                unpack_bf16x8(*reinterpret_cast<const uint4*>(Qs + h1 * DP + d), q1);
#pragma unroll
                for (int e = 0; e < 8; ++e) { r0 = fmaf(kf[e], q0[e], r0); r1 = fmaf(kf[e], q1[e], r1); }
            }
            const bool valid = s_tok[lane] >= 0;
            const float rs = sc[lane];
            s0 = valid ? (s0 * rs + r0) * p.scale : -INFINITY;
            s1 = valid ? (s1 * rs + r1) * p.scale : -INFINITY;
            const float m0 = fmaxf(s_m[h0], warp_max(s0)), m1 = fmaxf(s_m[h1], warp_max(s1));
            const float p0 = valid ? __expf(s0 - m0) : 0.f, p1 = valid ? __expf(s1 - m1) : 0.f;
            const float l0 = warp_sum(p0), l1 = warp_sum(p1);
            // the value row is the scaled latent: fold the row scale into p for the PV pass
            Ps[lane * kHG + h0] = p0 * rs;
            Ps[lane * kHG + h1] = p1 * rs;
            if (lane == 0) {
                const float a0 = (m0 == -INFINITY) ? 1.f : __expf(s_m[h0] - m0), a1 = (m1 == -INFINITY) ? 1.f : __expf(s_m[h1] - m1);
                s_alpha[h0] = a0; s_alpha[h1] = a1;
                s_l[h0] = s_l[h0] * a0 + l0; s_l[h1] = s_l[h1] * a1 + l1;
                s_m[h0] = m0; s_m[h1] = m1;
            }
        }
        __syncthreads();
        // PV: thread -> latent dims (2t, 2t+1), all heads
        if (2 * t < p.dl) {
#pragma unroll
            for (int h = 0; h < kHG; ++h) { const float a = s_alpha[h]; acc[h][0] *= a; acc[h][1] *= a; }
            for (int j = 0; j < kTK; ++j) {
                const bf162 kv = *reinterpret_cast<const bf162*>(Ks + j * DP + 2 * t);
                const float k0 = __low2float(kv), k1 = __high2float(kv);
                const float4* pp = reinterpret_cast<const float4*>(Ps + j * kHG);
#pragma unroll
                for (int h4 = 0; h4 < kHG / 4; ++h4) {
                    const float4 pv = pp[h4];
                    acc[h4 * 4 + 0][0] = fmaf(pv.x, k0, acc[h4 * 4 + 0][0]); acc[h4 * 4 + 0][1] = fmaf(pv.x, k1, acc[h4 * 4 + 0][1]);
                    acc[h4 * 4 + 1][0] = fmaf(pv.y, k0, acc[h4 * 4 + 1][0]); acc[h4 * 4 + 1][1] = fmaf(pv.y, k1, acc[h4 * 4 + 1][1]);
                    acc[h4 * 4 + 2][0] = fmaf(pv.z, k0, acc[h4 * 4 + 2][0]); acc[h4 * 4 + 2][1] = fmaf(pv.z, k1, acc[h4 * 4 + 2][1]);
                    acc[h4 * 4 + 3][0] = fmaf(pv.w, k0, acc[h4 * 4 + 3][0]); acc[h4 * 4 + 3][1] = fmaf(pv.w, k1, acc[h4 * 4 + 3][1]);
                }
            }
        }
    }
    __syncthreads();
    if (2 * t < p.dl) {
#pragma unroll
        for (int h = 0; h < kHG; ++h) {
            const int hh = hg * kHG + h;
            if (hh < p.H) {
                float* o = p.o_part + (((size_t)r * p.H + hh) * p.NS + sp) * p.dl + 2 * t;
                o[0] = acc[h][0]; o[1] = acc[h][1];
            }
        }
    }
    if (t < kHG && hg * kHG + t < p.H) {
        float* ml = p.ml_part + (((size_t)r * p.H + hg * kHG + t) * p.NS + sp) * 2;
        ml[0] = s_m[t]; ml[1] = s_l[t];
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------------------
// Many-row variant (prefill chunks, verify batches, large decode batches): same contract as mla_decode_kernel
// (grid = rows x head groups x splits, same partial outputs), but the two contractions run on the tensor
// cores: warp-level mma.sync m16n8k16 (bf16 x bf16 -> fp32) with the 16 heads of the group as the M dimension.
//   scores  S[16 heads x 64 keys]  = Q[16 x D] . K^T      warp w owns keys 8w .. 8w+7 (one n-tile), all of D
//   values  O[16 heads x dl]      += P[16 x 64] . V        warp w owns dl / 8 latent columns, all 64 keys
// K tile rows double as V rows (absorbed MLA: the value is the latent itself), so a tile is gathered and
// de-quantised once.  The softmax statistics are exchanged between the warps through shared memory.
// (The 5th-generation tensor path needs M = 128 rows per instruction; with 16-64 heads per query row and a
// private key set per row that shape does not occur here.)
constexpr int kTKM = 64;   // cache rows per tile of the tensor-core variant

__device__ __forceinline__ uint32_t smem_addr_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

LSB_API int lsb_mla_decode_mma_smem_bytes(int dl, int dr) {
    const int DP = dl + dr + 8;
    return (kTKM + kHG) * DP * 2 + kHG * (kTKM + 8) * 2 + kTKM * 4 + kTKM * 4 + (3 * kHG + 2 * 8 * kHG) * 4;
}

__global__ void __launch_bounds__(256) mla_decode_mma_kernel(MlaDecodeParams p) {
    extern __shared__ __align__(16) uint8_t smraw[];
    const int D = p.dl + p.dr, DP = D + 8;     // padded bf16 row: 16 bytes past a multiple of 128 => conflict-free ldmatrix rows
    constexpr int PP = kTKM + 8;               // padded P row
    bf16* Ks = reinterpret_cast<bf16*>(smraw);                 // [kTKM][DP]
    bf16* Qs = Ks + kTKM * DP;                                  // [kHG][DP]
    bf16* Ps = Qs + kHG * DP;                                   // [kHG][PP]  probabilities (x row scale), bf16
    float* sc = reinterpret_cast<float*>(Ps + kHG * PP);        // [kTKM] row scales
    int* s_tok = reinterpret_cast<int*>(sc + kTKM);             // [kTKM]
    float* s_m = reinterpret_cast<float*>(s_tok + kTKM);        // [kHG] running max
    float* s_l = s_m + kHG;                                     // [kHG] running sum
    float* s_alpha = s_l + kHG;                                 // [kHG]
    float* s_pmax = s_alpha + kHG;                              // [8 warps][kHG]
    float* s_psum = s_pmax + 8 * kHG;                           // [8 warps][kHG]
    const int r = blockIdx.x, hg = blockIdx.y, sp = blockIdx.z;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int g = lane >> 2, tq = lane & 3;                     // fragment row / column-pair index
    pdl_wait();
    pdl_launch_dependents();
    const int seq = p.row_seq[r];
    int n = p.sel_idx ? p.sel_cnt[r] : p.row_len[r];
    if (seq < 0) n = 0;
    const int per = (((n + p.NS - 1) / p.NS) + kTKM - 1) / kTKM * kTKM;
    const int beg = sp * per, end = min(n, beg + per);
    for (int i = t; i < kHG * (D / 8); i += blockDim.x) {
        const int h = i / (D / 8), c = i % (D / 8);
        const int hh = hg * kHG + h;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (hh < p.H) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)r * p.H + hh) * D + c * 8);
        *reinterpret_cast<uint4*>(Qs + h * DP + c * 8) = v;
    }
    if (t < kHG) { s_m[t] = -INFINITY; s_l[t] = 0.f; }
    const int ncol = p.dl / 8;                 // latent columns per warp in the PV product (multiple of 8: dl % 64 == 0)
    const int ntile = ncol / 8;                // n-tiles per warp, <= 8
    float o[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const int rb = kv_row_bytes(p.kv_fmt, p.dl, p.dr);
    const uint32_t q_addr = smem_addr_u32(Qs) + (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * DP + (lane >> 4) * 8) * 2);
    const uint32_t k_addr = smem_addr_u32(Ks) + (uint32_t)(((warp * 8 + (lane & 7)) * DP + ((lane >> 3) & 1) * 8) * 2);
    const uint32_t p_addr = smem_addr_u32(Ps) + (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * PP + (lane >> 4) * 8) * 2);
    const uint32_t v_addr = smem_addr_u32(Ks) + (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * DP + warp * ncol) * 2);
    for (int t0 = beg; t0 < end; t0 += kTKM) {
        __syncthreads();                                       // previous tile fully consumed
        if (t < kTKM) {
            const int i = t0 + t;
            int tok = -1;
            if (i < end) tok = p.sel_idx ? p.sel_idx[(size_t)r * p.sel_ld + i] : i;
            s_tok[t] = tok;
        }
        __syncthreads();
        mla_load_tile(p, seq, rb, s_tok, Ks, sc, DP, D, t, blockDim.x, kTKM);
        __syncthreads();
        // ---- scores of keys 8 warp .. 8 warp + 7 for the 16 heads ----
        float cl[4] = {0.f, 0.f, 0.f, 0.f}, cr[4] = {0.f, 0.f, 0.f, 0.f};
        for (int d = 0; d < p.dl; d += 16) {
            uint32_t a0, a1, a2, a3, b0, b1;
            ldsm_x4(q_addr + d * 2, a0, a1, a2, a3);
            ldsm_x2(k_addr + d * 2, b0, b1);
            mma_bf16_16816(cl, a0, a1, a2, a3, b0, b1);
        }
        for (int d = p.dl; d < D; d += 16) {
            uint32_t a0, a1, a2, a3, b0, b1;
            ldsm_x4(q_addr + d * 2, a0, a1, a2, a3);
            ldsm_x2(k_addr + d * 2, b0, b1);
            mma_bf16_16816(cr, a0, a1, a2, a3, b0, b1);
        }
        // this thread: heads g, g + 8; keys 8 warp + 2 tq, + 1
        const int key0 = warp * 8 + 2 * tq;
        const bool v0 = s_tok[key0] >= 0, v1 = s_tok[key0 + 1] >= 0;
        const float rs0 = sc[key0], rs1 = sc[key0 + 1];
        float s00 = v0 ? (cl[0] * rs0 + cr[0]) * p.scale : -INFINITY, s01 = v1 ? (cl[1] * rs1 + cr[1]) * p.scale : -INFINITY;
        float s10 = v0 ? (cl[2] * rs0 + cr[2]) * p.scale : -INFINITY, s11 = v1 ? (cl[3] * rs1 + cr[3]) * p.scale : -INFINITY;
        float mx0 = fmaxf(s00, s01), mx1 = fmaxf(s10, s11);
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (tq == 0) { s_pmax[warp * kHG + g] = mx0; s_pmax[warp * kHG + g + 8] = mx1; }
        __syncthreads();
        float m0 = s_m[g], m1 = s_m[g + 8];
#pragma unroll
        for (int w = 0; w < 8; ++w) { m0 = fmaxf(m0, s_pmax[w * kHG + g]); m1 = fmaxf(m1, s_pmax[w * kHG + g + 8]); }
        const float p00 = v0 ? __expf(s00 - m0) : 0.f, p01 = v1 ? __expf(s01 - m0) : 0.f;
        const float p10 = v0 ? __expf(s10 - m1) : 0.f, p11 = v1 ? __expf(s11 - m1) : 0.f;
        float l0 = p00 + p01, l1 = p10 + p11;
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        if (tq == 0) { s_psum[warp * kHG + g] = l0; s_psum[warp * kHG + g + 8] = l1; }
        // the value row is the scaled latent: fold the row scale into P for the PV product
        *reinterpret_cast<bf162*>(Ps + g * PP + key0) = __floats2bfloat162_rn(p00 * rs0, p01 * rs1);
        *reinterpret_cast<bf162*>(Ps + (g + 8) * PP + key0) = __floats2bfloat162_rn(p10 * rs0, p11 * rs1);
        // every thread holds the new maxima of its two heads; rescale its accumulators
        const float al0 = (m0 == -INFINITY) ? 1.f : __expf(s_m[g] - m0), al1 = (m1 == -INFINITY) ? 1.f : __expf(s_m[g + 8] - m1);
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
        __syncthreads();                                       // P and the partial sums are complete; all reads of s_m are done
        if (t < kHG) {
            float mm = s_m[t], ll = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) { mm = fmaxf(mm, s_pmax[w * kHG + t]); ll += s_psum[w * kHG + t]; }
            const float a = (mm == -INFINITY) ? 1.f : __expf(s_m[t] - mm);
            s_l[t] = s_l[t] * a + ll;
            s_m[t] = mm;
        }
        // ---- O += P . V over this warp's latent columns ----
#pragma unroll
        for (int ks = 0; ks < kTKM / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(p_addr + ks * 32, a0, a1, a2, a3);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < ntile) {
                    uint32_t b0, b1;
                    ldsm_x2_trans(v_addr + (uint32_t)((ks * 16 * DP + j * 8) * 2), b0, b1);
                    mma_bf16_16816(o[j], a0, a1, a2, a3, b0, b1);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (j < ntile) {
            const int col = warp * ncol + j * 8 + 2 * tq;
            const int h0 = hg * kHG + g, h1 = h0 + 8;
            if (h0 < p.H) { float* op = p.o_part + (((size_t)r * p.H + h0) * p.NS + sp) * p.dl + col; op[0] = o[j][0]; op[1] = o[j][1]; }
            if (h1 < p.H) { float* op = p.o_part + (((size_t)r * p.H + h1) * p.NS + sp) * p.dl + col; op[0] = o[j][2]; op[1] = o[j][3]; }
        }
    }
    if (t < kHG && hg * kHG + t < p.H) {
        float* ml = p.ml_part + (((size_t)r * p.H + hg * kHG + t) * p.NS + sp) * 2;
        ml[0] = s_m[t]; ml[1] = s_l[t];
    }
    pdl_launch_dependents();
}

// Head-group-shared variant: one block serves NG groups of 16 heads of a query row (4 warps per group), so a K tile is
// gathered and de-quantised once per row instead of once per 16 heads.  Per group: warp s of 4 owns keys 16 s .. 16 s + 15
// (two n-tiles) in the score product and dl / 4 latent columns in the value product.
template <int NG>
__global__ void __launch_bounds__(NG * 128) mla_decode_mma_shared_kernel(MlaDecodeParams p) {
    extern __shared__ __align__(16) uint8_t smraw[];
    constexpr int NH = NG * kHG;               // heads per block
    const int D = p.dl + p.dr, DP = D + 8;
    constexpr int PP = kTKM + 8;
    bf16* Ks = reinterpret_cast<bf16*>(smraw);                 // [kTKM][DP]
    bf16* Qs = Ks + kTKM * DP;                                  // [NH][DP]
    bf16* Ps = Qs + NH * DP;                                    // [NH][PP]
    float* sc = reinterpret_cast<float*>(Ps + NH * PP);         // [kTKM]
    int* s_tok = reinterpret_cast<int*>(sc + kTKM);             // [kTKM]
    float* s_m = reinterpret_cast<float*>(s_tok + kTKM);        // [NH]
    float* s_l = s_m + NH;                                      // [NH]
    float* s_pmax = s_l + NH;                                   // [4][NH]
    float* s_psum = s_pmax + 4 * NH;                            // [4][NH]
    const int r = blockIdx.x, hb = blockIdx.y * NH, sp = blockIdx.z;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int grp = warp >> 2, sw = warp & 3;                   // head group inside the block, warp inside the group
    const int g = lane >> 2, tq = lane & 3;
    const int hl0 = grp * kHG + g, hl1 = hl0 + 8;               // this thread's two heads (block-local)
    pdl_wait();
    pdl_launch_dependents();
    const int seq = p.row_seq[r];
    int n = p.sel_idx ? p.sel_cnt[r] : p.row_len[r];
    if (seq < 0) n = 0;
    const int per = (((n + p.NS - 1) / p.NS) + kTKM - 1) / kTKM * kTKM;
    const int beg = sp * per, end = min(n, beg + per);
    for (int i = t; i < NH * (D / 8); i += blockDim.x) {
        const int h = i / (D / 8), c = i % (D / 8);
        const int hh = hb + h;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (hh < p.H) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)r * p.H + hh) * D + c * 8);
        *reinterpret_cast<uint4*>(Qs + h * DP + c * 8) = v;
    }
    if (t < NH) { s_m[t] = -INFINITY; s_l[t] = 0.f; }
    const int ncol = p.dl / 4;                 // latent columns per warp in the PV product (multiple of 16: dl % 64 == 0)
    const int ntile = ncol / 8;                // n-tiles per warp, <= 16
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    const int rb = kv_row_bytes(p.kv_fmt, p.dl, p.dr);
    const int arow = (lane & 7) + ((lane >> 3) & 1) * 8;        // ldmatrix.x4 row of an A tile
    const uint32_t q_addr = smem_addr_u32(Qs) + (uint32_t)(((grp * kHG + arow) * DP + (lane >> 4) * 8) * 2);
    const uint32_t k_addr = smem_addr_u32(Ks) + (uint32_t)(((sw * 16 + (lane & 7)) * DP + ((lane >> 3) & 1) * 8) * 2);
    const uint32_t p_addr = smem_addr_u32(Ps) + (uint32_t)(((grp * kHG + arow) * PP + (lane >> 4) * 8) * 2);
    const uint32_t v_addr = smem_addr_u32(Ks) + (uint32_t)((arow * DP + sw * ncol) * 2);
    for (int t0 = beg; t0 < end; t0 += kTKM) {
        __syncthreads();
        if (t < kTKM) {
            const int i = t0 + t;
            int tok = -1;
            if (i < end) tok = p.sel_idx ? p.sel_idx[(size_t)r * p.sel_ld + i] : i;
            s_tok[t] = tok;
        }
        __syncthreads();
        mla_load_tile(p, seq, rb, s_tok, Ks, sc, DP, D, t, blockDim.x, kTKM);
        __syncthreads();
        // ---- scores: keys 16 sw .. 16 sw + 15 (n-tiles u = 0, 1) for this group's 16 heads ----
        float cl[2][4], cr[2][4];
#pragma unroll
        for (int u = 0; u < 2; ++u) { cl[u][0] = cl[u][1] = cl[u][2] = cl[u][3] = 0.f; cr[u][0] = cr[u][1] = cr[u][2] = cr[u][3] = 0.f; }
        for (int d = 0; d < p.dl; d += 16) {
            uint32_t a0, a1, a2, a3, b0, b1;
            ldsm_x4(q_addr + d * 2, a0, a1, a2, a3);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                ldsm_x2(k_addr + (uint32_t)((u * 8 * DP + d) * 2), b0, b1);
                mma_bf16_16816(cl[u], a0, a1, a2, a3, b0, b1);
            }
        }
        for (int d = p.dl; d < D; d += 16) {
            uint32_t a0, a1, a2, a3, b0, b1;
            ldsm_x4(q_addr + d * 2, a0, a1, a2, a3);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                ldsm_x2(k_addr + (uint32_t)((u * 8 * DP + d) * 2), b0, b1);
                mma_bf16_16816(cr[u], a0, a1, a2, a3, b0, b1);
            }
        }
        float s[2][4];                                         // [n-tile][head g: keys 2tq, 2tq+1; head g+8: same keys]
        bool vld[2][2];
        float rsv[2][2];
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int key0 = sw * 16 + u * 8 + 2 * tq;
            vld[u][0] = s_tok[key0] >= 0; vld[u][1] = s_tok[key0 + 1] >= 0;
            rsv[u][0] = sc[key0]; rsv[u][1] = sc[key0 + 1];
            s[u][0] = vld[u][0] ? (cl[u][0] * rsv[u][0] + cr[u][0]) * p.scale : -INFINITY;
            s[u][1] = vld[u][1] ? (cl[u][1] * rsv[u][1] + cr[u][1]) * p.scale : -INFINITY;
            s[u][2] = vld[u][0] ? (cl[u][2] * rsv[u][0] + cr[u][2]) * p.scale : -INFINITY;
            s[u][3] = vld[u][1] ? (cl[u][3] * rsv[u][1] + cr[u][3]) * p.scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[u][0], s[u][1]));
            mx1 = fmaxf(mx1, fmaxf(s[u][2], s[u][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (tq == 0) { s_pmax[sw * NH + hl0] = mx0; s_pmax[sw * NH + hl1] = mx1; }
        __syncthreads();
        float m0 = s_m[hl0], m1 = s_m[hl1];
#pragma unroll
        for (int w = 0; w < 4; ++w) { m0 = fmaxf(m0, s_pmax[w * NH + hl0]); m1 = fmaxf(m1, s_pmax[w * NH + hl1]); }
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int key0 = sw * 16 + u * 8 + 2 * tq;
            const float p00 = vld[u][0] ? __expf(s[u][0] - m0) : 0.f, p01 = vld[u][1] ? __expf(s[u][1] - m0) : 0.f;
            const float p10 = vld[u][0] ? __expf(s[u][2] - m1) : 0.f, p11 = vld[u][1] ? __expf(s[u][3] - m1) : 0.f;
            l0 += p00 + p01; l1 += p10 + p11;
            // the value row is the scaled latent: fold the row scale into P for the PV product
            *reinterpret_cast<bf162*>(Ps + hl0 * PP + key0) = __floats2bfloat162_rn(p00 * rsv[u][0], p01 * rsv[u][1]);
            *reinterpret_cast<bf162*>(Ps + hl1 * PP + key0) = __floats2bfloat162_rn(p10 * rsv[u][0], p11 * rsv[u][1]);
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        if (tq == 0) { s_psum[sw * NH + hl0] = l0; s_psum[sw * NH + hl1] = l1; }
        const float al0 = (m0 == -INFINITY) ? 1.f : __expf(s_m[hl0] - m0), al1 = (m1 == -INFINITY) ? 1.f : __expf(s_m[hl1] - m1);
#pragma unroll
        for (int j = 0; j < 16; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
        __syncthreads();                                       // P and the partial sums are complete; all reads of s_m are done
        if (t < NH) {
            float mm = s_m[t], ll = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) { mm = fmaxf(mm, s_pmax[w * NH + t]); ll += s_psum[w * NH + t]; }
            const float a = (mm == -INFINITY) ? 1.f : __expf(s_m[t] - mm);
            s_l[t] = s_l[t] * a + ll;
            s_m[t] = mm;
        }
        // ---- O += P . V over this warp's latent columns ----
#pragma unroll
        for (int ks = 0; ks < kTKM / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(p_addr + ks * 32, a0, a1, a2, a3);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (j < ntile) {
                    uint32_t b0, b1;
                    ldsm_x2_trans(v_addr + (uint32_t)((ks * 16 * DP + j * 8) * 2), b0, b1);
                    mma_bf16_16816(o[j], a0, a1, a2, a3, b0, b1);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (j < ntile) {
            const int col = sw * ncol + j * 8 + 2 * tq;
            const int h0 = hb + hl0, h1 = hb + hl1;
            if (h0 < p.H) { float* op = p.o_part + (((size_t)r * p.H + h0) * p.NS + sp) * p.dl + col; op[0] = o[j][0]; op[1] = o[j][1]; }
            if (h1 < p.H) { float* op = p.o_part + (((size_t)r * p.H + h1) * p.NS + sp) * p.dl + col; op[0] = o[j][2]; op[1] = o[j][3]; }
        }
    }
    if (t < NH && hb + t < p.H) {
        float* ml = p.ml_part + (((size_t)r * p.H + hb + t) * p.NS + sp) * 2;
        ml[0] = s_m[t]; ml[1] = s_l[t];
    }
    pdl_launch_dependents();
}

static int mla_mma_shared_smem_bytes(int dl, int dr, int ng) {
    const int DP = dl + dr + 8, NH = ng * kHG;
    return (kTKM + NH) * DP * 2 + NH * (kTKM + 8) * 2 + kTKM * 4 + kTKM * 4 + (2 * NH + 8 * NH) * 4;
}

// Merge split partials in split order: out = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s.  NS <= 32.
// One thread per latent column with all NS partials of the column requested before the first is used (a dependent
// batch per 8 splits made this kernel a chain of L2 round trips).
__global__ void __launch_bounds__(512) mla_combine_kernel(bf16* __restrict__ out, float* __restrict__ lse, const float* __restrict__ o_part,
                                                          const float* __restrict__ ml_part, int H, int NS, int dl) {
    __shared__ float w[32];
    __shared__ float s_invL, s_lse;
    const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const float* ml = ml_part + ((size_t)r * H + h) * NS * 2;
    const float* op = o_part + ((size_t)r * H + h) * NS * dl;
    float v[32];
    const bool col = t < dl;
#pragma unroll
    for (int s = 0; s < 32; ++s) v[s] = (col && s < NS) ? op[(size_t)s * dl + t] : 0.f;
    if (t < 32) {
        const float m = t < NS ? ml[2 * t] : -INFINITY;
        const float l = t < NS ? ml[2 * t + 1] : 0.f;
        const float M = warp_max(m);
        const float e = (m > -INFINITY) ? __expf(m - M) : 0.f;
        w[t] = e;
        // fixed-order sum over splits (ascending lane by shuffle), independent of scheduling
        float L = 0.f;
        for (int s = 0; s < NS; ++s) L += __shfl_sync(0xffffffffu, e * l, s);
        if (t == 0) {
            s_invL = L > 0.f ? 1.f / L : 0.f;
            s_lse = L > 0.f ? M + logf(L) : -INFINITY;
        }
    }
    __syncthreads();
    const float invL = s_invL;
    if (col) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < 32; ++s) a = fmaf(w[s], v[s], a);      // w[s] = 0 beyond NS
        out[((size_t)r * H + h) * dl + t] = __float2bfloat16(a * invL);
    }
    for (int d = blockDim.x + t; d < dl; d += blockDim.x) {        // latent widths beyond the block size
        float a = 0.f;
        for (int s = 0; s < NS; ++s) a = fmaf(w[s], op[(size_t)s * dl + d], a);
        out[((size_t)r * H + h) * dl + d] = __float2bfloat16(a * invL);
    }
    if (lse && t == 0) lse[(size_t)r * H + h] = s_lse;
}

}  // namespace lsb
using namespace lsb;

extern "C" int lsb_gemm_bf16_tc_batched(void* out, const void* x, const void* w, int M, int N, int K, int B, int ldx, long long xs_b, int ldw,
                                        long long ws_b, int ldo, long long os_b, int out_bf16, void* err, void* stream);

LSB_API int lsb_kv_row_bytes(int fmt, int dl, int dr) { return kv_row_bytes(fmt, dl, dr); }

LSB_API int lsb_mla_prep(const void* proj, int ldp, int off_qa, int q_lora, int off_kv, int dl, int dr,
                         const void* qa_norm_w, const void* kv_norm_w, const void* inv_freq, void* q_c, void* cache,
                         const void* block_table, int max_pages, const void* row_seq, const void* row_pos, int rows,
                         int page, int kv_fmt, float eps, const void* tq_rot_t, const void* tq_centroids, const void* row_store,
                         void* stream) {
    if (kv_fmt == 2 && (!tq_rot_t || !tq_centroids || dl % 32)) return -1;
    const int n = q_lora > dl + dr ? q_lora : dl + dr;
    launch_pdl((mla_prep_kernel), dim3(rows, q_lora > 0 && rows <= 64 ? 2 : 1), 256, (size_t)n * 4, (cudaStream_t)stream, (const float*)proj, ldp, off_qa, q_lora, off_kv, dl, dr,
                                                                      (const float*)qa_norm_w, (const float*)kv_norm_w,
                                                                      (const float*)inv_freq, (bf16*)q_c, (uint8_t*)cache,
                                                                      (const int*)block_table, max_pages, (const int*)row_seq,
                                                                      (const int*)row_pos, page, kv_fmt, eps, (const bf16*)tq_rot_t,
                                                                      (const float*)tq_centroids, (const int*)row_store);
    LSB_CHECK_LAUNCH();
}

// x: bf16 rows m with stride xs_m, batch stride xs_b; W: bf16 [B, N, K]; out bf16 (strides os_m, os_b).
LSB_API int lsb_batched_gemv_bf16(void* out, const void* x, const void* w, int M, int B, int N, int K, long long xs_m,
                                  long long xs_b, long long os_m, long long os_b, int dr, const void* inv_freq,
                                  const void* row_pos, void* stream) {
    if (K % 8 || xs_m % 8 || xs_b % 8) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((N + 15) / 16, B);
    if (M >= 32 && K % 8 == 0 && xs_m % 8 == 0 && xs_b % 8 == 0 && os_b % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
        // many rows: one tensor-core GEMM per head ([M, K] x [N, K]^T), the rope tail on the side
        const int rc = lsb_gemm_bf16_tc_batched(out, x, w, M, N, K, B, (int)xs_m, xs_b, K, (long long)N * K, (int)os_m, os_b, 1, nullptr, stream);
        if (rc) return rc;
        if (dr > 0)
            launch_pdl((rope_tail_kernel), dim3(M, B), 32, 0, st, (bf16*)out, (const bf16*)x, N, K, xs_m, xs_b, os_m, os_b, dr, (const float*)inv_freq,
                       (const int*)row_pos);
        LSB_CHECK_LAUNCH();
    }
    for (int m0 = 0; m0 < M;) {
        const int rem = M - m0, mt = rem >= 4 ? 4 : (rem >= 2 ? 2 : 1);
        bf16* o = (bf16*)out + (size_t)m0 * os_m;
        const bf16* xp = (const bf16*)x + (size_t)m0 * xs_m;
#define ARGS o, xp, (const bf16*)w, N, K, xs_m, xs_b, os_m, os_b, dr, (const float*)inv_freq, (const int*)row_pos, m0
        if (mt == 4) launch_pdl((batched_gemv_kernel<4>), grid, 256, 0, st, ARGS);
        else if (mt == 2) launch_pdl((batched_gemv_kernel<2>), grid, 256, 0, st, ARGS);
        else launch_pdl((batched_gemv_kernel<1>), grid, 256, 0, st, ARGS);
#undef ARGS
        m0 += mt;
    }
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_mla_decode_smem_bytes(int dl, int dr) {
    const int DP = dl + dr + 8;
    return (kTK + kHG) * DP * 2 + kTK * kHG * 4 + kTK * 4 + 3 * kHG * 4 + kTK * 4;
}

// q: bf16 [R,H,dl+dr]; out: bf16 [R,H,dl]; o_part/ml_part: scratch fp32 [R,H,NS,dl], [R,H,NS,2].
LSB_API int lsb_mla_decode(const void* q, const void* cache, const void* block_table, int max_pages, const void* row_seq,
                           const void* row_len, const void* sel_idx, const void* sel_cnt, int sel_ld, void* out, void* lse,
                           void* o_part, void* ml_part, int R, int H, int dl, int dr, int page, int kv_fmt, int NS,
                           float scale, const void* tq_centroids, void* stream) {
    if (dl % 16 || dr % 8 || dl > 512 || NS > 32) return -1;
    if (kv_fmt == 2 && (!tq_centroids || dl % 32)) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    MlaDecodeParams p;
    p.q = (const bf16*)q; p.cache = (const uint8_t*)cache; p.block_table = (const int*)block_table; p.max_pages = max_pages;
    p.row_seq = (const int*)row_seq; p.row_len = (const int*)row_len; p.sel_idx = (const int*)sel_idx; p.sel_cnt = (const int*)sel_cnt;
    p.sel_ld = sel_ld; p.o_part = (float*)o_part; p.ml_part = (float*)ml_part; p.H = H; p.dl = dl; p.dr = dr; p.page = page;
    p.kv_fmt = kv_fmt; p.NS = NS; p.scale = scale; p.tq_centroids = (const float*)tq_centroids;
    const int smem = lsb_mla_decode_smem_bytes(dl, dr);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(mla_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(mla_decode_mma_shared_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(mla_decode_mma_shared_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set = true;
    }
    // tensor-core variant wherever the shape allows it; the CUDA-core kernel serves the remaining head sizes
    // LSB_MLA_MMA_MIN_ROWS: step size from which the tensor-core variant is used (tuning knob; default 1: it is also the faster
    // one for single decode rows, 8.01 against 8.16 ms per step on the GLM-5.3-Flash shape)
    static const int mma_min_rows = [] { const char* e = getenv("LSB_MLA_MMA_MIN_ROWS"); return e ? atoi(e) : 1; }();
    if (R >= mma_min_rows && dl % 64 == 0 && dl <= 512 && dr % 16 == 0) {
        // more than one 16-head group per query row: the groups of a row share each gathered K tile
        if (H > 2 * kHG && mla_mma_shared_smem_bytes(dl, dr, 4) <= 200 * 1024)
            launch_pdl((mla_decode_mma_shared_kernel<4>), dim3(R, (H + 4 * kHG - 1) / (4 * kHG), NS), 512, (size_t)mla_mma_shared_smem_bytes(dl, dr, 4), st, p);
        else if (H > kHG && mla_mma_shared_smem_bytes(dl, dr, 2) <= 200 * 1024)
            launch_pdl((mla_decode_mma_shared_kernel<2>), dim3(R, (H + 2 * kHG - 1) / (2 * kHG), NS), 256, (size_t)mla_mma_shared_smem_bytes(dl, dr, 2), st, p);
        else
            launch_pdl((mla_decode_mma_kernel), dim3(R, (H + kHG - 1) / kHG, NS), 256, (size_t)lsb_mla_decode_mma_smem_bytes(dl, dr), st, p);
    } else {
        launch_pdl((mla_decode_kernel), dim3(R, (H + kHG - 1) / kHG, NS), 256, smem, st, p);
    }
    // out == null: the caller merges the partials itself (context-parallel attention combines them across ranks)
    if (out) launch_pdl((mla_combine_kernel), dim3(R, H), dl >= 512 ? 512 : (dl >= 256 ? 256 : 128), 0, st, (bf16*)out, (float*)lse, (const float*)o_part, (const float*)ml_part, H, NS, dl);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_mla(void* buf) { return lsb_trace_install(buf); }
