// Parameter blocks of the KDA kernels (shared by kda.cu, kda_chunk.cuh and the host-side emulation test of the chunk kernels).
// Needs the ``bf16`` type to be defined by the includer.
#pragma once

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

struct KdaScratch {
    float* qn; float* kn; float* vo; float* decay; float* gate;   // [rows, C]  (vo: v in, o out)
    float* beta;                                                    // [rows, H]
    // optional: the two low-rank gate products of every row, computed beforehand by the tensor-core GEMM
    // (raw_g = f_a . f_b^T, g2 = g_a . g_b^T, [rows, C]); null = the prep kernel computes them itself
    const float* rawg; const float* g2;
};

// conv history of channel `ch` = the last three raw rows (older taps come from the previous history when the step was short)
__device__ __forceinline__ void kda_update_conv_history(const KdaParams& p, int row0, int nrows, int slot, int ch) {
    const int C = p.H * kD;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        float* cs = p.conv_state + (((size_t)slot * 3 + a) * C + ch) * 3;
        const int off = a == 0 ? p.off_q : (a == 1 ? p.off_k : p.off_v);
        float nh[3];
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            const int i = nrows - 3 + d;                     // row index inside the step for new tap d
            nh[d] = i >= 0 ? p.proj[(size_t)(row0 + i) * p.ldp + off + ch] : cs[3 + i];
        }
#pragma unroll
        for (int d = 0; d < 3; ++d) cs[d] = nh[d];
    }
}
