#pragma once
// ------------------------------------------------------------------------------------------------ chunk-parallel recurrence
// The same recurrence in chunks of 64 tokens (one sequence per step, prefill chunks).  With G_t = sum_{s<=t} log d_s inside a chunk:
//   A[t][s] = sum_c k_t k_s exp(G_t - G_s) (s < t),  B[t][s] = sum_c q_t k_s exp(G_t - G_s) (s <= t)    every exponent <= 0
//   W = (I + diag(beta) tril(A,-1))^-1 diag(beta),  U = W (V - Kp S0^T),  O = Qp S0^T + tril(B) U,  S = S0 diag(gC) + U^T Km
//   Kp = K exp(G), Qp = Q exp(G), Km = K exp(G_last - G), gC = exp(G_last)
// kda_chunk_prep: everything that does not depend on the state, one block per (chunk, head); rewrites qn -> Qp, decay -> Kp, kn -> Km in
// place.  kda_chunk_scan: sequential over the chunks, one block per (head, half of the value channels) - value channels are independent.
// fp32 on the CUDA cores (same precision as kda_recur); opt-in (lsb_kda_forward_chunked).
constexpr int kCh = 64;            // tokens per chunk
constexpr int kLdK = kD + 4;       // shared-memory row stride (floats) of [*, 128] tiles: 16-byte aligned rows, conflict-free float4 columns
constexpr int kLdC = kCh + 4;      // row stride of [*, 64] tiles
constexpr int kSub = 16;           // tokens per sub-chunk of the A / B factorisation
constexpr int kLdR = kD + 1;       // odd row stride of the rescaled tiles: lanes that read different rows at the same column hit different banks
constexpr size_t kChunkPrepSmem = (size_t)(3 * kCh * kLdK + 3 * kCh * kLdC + kCh + (2 * kSub + kCh - kSub) * kLdR) * sizeof(float);
constexpr size_t kChunkScanSmem = (size_t)(4 * kCh * kLdK + 4 * kCh * kLdC) * sizeof(float);

struct KdaChunkWs {
    float* W;     // [chunks, H, 64, 64]
    float* B;     // [chunks, H, 64, 64] lower triangle incl. diagonal, zero above
    float* gC;    // [chunks, H, 128]
};

__global__ void __launch_bounds__(256) kda_chunk_prep_kernel(KdaParams p, KdaScratch w, KdaChunkWs cw) {
    extern __shared__ __align__(16) float csm[];
    float* sK = csm;
    float* sQ = sK + kCh * kLdK;
    float* sG = sQ + kCh * kLdK;
    float* sA = sG + kCh * kLdK;
    float* sB = sA + kCh * kLdC;
    float* sW = sB + kCh * kLdC;
    float* sBeta = sW + kCh * kLdC;
    float* sLk = sBeta + kCh;                                 // [16][kLdR] k rows of the current sub-chunk times exp(G - G_ref)
    float* sLq = sLk + kSub * kLdR;                           // [16][kLdR] q rows, same factor
    float* sR = sLq + kSub * kLdR;                            // [48][kLdR] earlier k rows times exp(G_ref - G)
    const int chunk = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();
    const int row0 = p.seq_row0[0], nrows = p.seq_nrows[0];
    const int c0 = chunk * kCh;
    const int cc = min(kCh, nrows - c0);                     // tokens of this chunk
    if (cc <= 0) return;
    const int C = p.H * kD;
    // 1. k, q and log-decay tiles (rows past the chunk: zeros, i.e. no decay and no write)
    for (int idx = tid; idx < kCh * (kD / 4); idx += 256) {
        const int t = idx / (kD / 4), c4 = idx % (kD / 4);
        float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), q4 = k4, g4 = k4;
        if (t < cc) {
            const size_t off = (size_t)(row0 + c0 + t) * C + h * kD + c4 * 4;
            k4 = *reinterpret_cast<const float4*>(w.kn + off);
            q4 = *reinterpret_cast<const float4*>(w.qn + off);
            const float4 d = *reinterpret_cast<const float4*>(w.decay + off);
            g4 = make_float4(logf(d.x), logf(d.y), logf(d.z), logf(d.w));
        }
        *reinterpret_cast<float4*>(sK + t * kLdK + c4 * 4) = k4;
        *reinterpret_cast<float4*>(sQ + t * kLdK + c4 * 4) = q4;
        *reinterpret_cast<float4*>(sG + t * kLdK + c4 * 4) = g4;
    }
    for (int idx = tid; idx < kCh * kLdC; idx += 256) { sA[idx] = 0.f; sB[idx] = 0.f; sW[idx] = 0.f; }
    if (tid < kCh) sBeta[tid] = tid < cc ? w.beta[(size_t)(row0 + c0 + tid) * p.H + h] : 0.f;
    __syncthreads();
    // 2. cumulative log-decay per channel (non-increasing in t)
    if (tid < kD) {
        float acc = 0.f;
        for (int t = 0; t < kCh; ++t) { acc += sG[t * kLdK + tid]; sG[t * kLdK + tid] = acc; }
    }
    __syncthreads();
    // 3. A and B.  The 64 tokens are four sub-chunks of 16.  Pairs inside a sub-chunk keep the exact form (one warp per pair, one exponential
    // per channel).  Pairs (t in sub-chunk I, s before it) factor through the first token of I:
    //     exp(G_t - G_s) = exp(G_t - G_ref) * exp(G_ref - G_s),   G_ref = G[16 I]:   both exponents <= 0 (G is non-increasing),
    // so the block is a plain product of two rescaled tiles (L = rows of I times exp(G - G_ref), R = earlier rows times exp(G_ref - G))
    // with no exponential in the inner loop: 12k exponentials per block for the tiles instead of 190k for the pairs.
    for (int I = 0; I < kCh / kSub; ++I) {
        const int t0 = I * kSub;
        if (t0 >= cc) break;                                  // block-uniform
        for (int pidx = warp; pidx < kSub * (kSub + 1) / 2; pidx += 8) {
            int dt = 0, ds = pidx;
            while (ds > dt) { ds -= dt + 1; ++dt; }
            const int t = t0 + dt, s_ = t0 + ds;
            if (t >= cc) continue;                            // warp-uniform
            const float4 kt = *reinterpret_cast<const float4*>(sK + t * kLdK + lane * 4);
            const float4 qt = *reinterpret_cast<const float4*>(sQ + t * kLdK + lane * 4);
            const float4 gt = *reinterpret_cast<const float4*>(sG + t * kLdK + lane * 4);
            const float4 ks = *reinterpret_cast<const float4*>(sK + s_ * kLdK + lane * 4);
            const float4 gs = *reinterpret_cast<const float4*>(sG + s_ * kLdK + lane * 4);
            const float e0 = __expf(fminf(gt.x - gs.x, 0.f)), e1 = __expf(fminf(gt.y - gs.y, 0.f));
            const float e2 = __expf(fminf(gt.z - gs.z, 0.f)), e3 = __expf(fminf(gt.w - gs.w, 0.f));
            const float k0 = ks.x * e0, k1 = ks.y * e1, k2 = ks.z * e2, k3 = ks.w * e3;
            float a = kt.x * k0 + kt.y * k1 + kt.z * k2 + kt.w * k3;
            float b = qt.x * k0 + qt.y * k1 + qt.z * k2 + qt.w * k3;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
            }
            if (lane == 0) { sA[t * kLdC + s_] = a; sB[t * kLdC + s_] = b; }
        }
        if (I == 0) continue;
        const float* gref = sG + t0 * kLdK;
        for (int idx = tid; idx < kSub * kD; idx += 256) {
            const int tt = idx / kD, c = idx % kD;
            const float e = __expf(fminf(sG[(t0 + tt) * kLdK + c] - gref[c], 0.f));
            sLk[tt * kLdR + c] = sK[(t0 + tt) * kLdK + c] * e;
            sLq[tt * kLdR + c] = sQ[(t0 + tt) * kLdK + c] * e;
        }
        for (int idx = tid; idx < t0 * kD; idx += 256) {
            const int s_ = idx / kD, c = idx % kD;
            sR[s_ * kLdR + c] = sK[s_ * kLdK + c] * __expf(fminf(gref[c] - sG[s_ * kLdK + c], 0.f));
        }
        __syncthreads();
        // one thread per (t, s): consecutive lanes take consecutive s (odd row stride: conflict free), t is warp-uniform or nearly
        for (int o = tid; o < kSub * t0; o += 256) {
            const int tt = o / t0, s_ = o - tt * t0;
            const float* lk = sLk + tt * kLdR;
            const float* lq = sLq + tt * kLdR;
            const float* rr = sR + s_ * kLdR;
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll 8
            for (int c = 0; c < kD; c += 2) {
                const float r0 = rr[c], r1 = rr[c + 1];
                a0 = fmaf(lk[c], r0, a0); a1 = fmaf(lk[c + 1], r1, a1);
                b0 = fmaf(lq[c], r0, b0); b1 = fmaf(lq[c + 1], r1, b1);
            }
            if (t0 + tt < cc) { sA[(t0 + tt) * kLdC + s_] = a0 + a1; sB[(t0 + tt) * kLdC + s_] = b0 + b1; }
        }
        __syncthreads();                                      // the tiles are rebuilt for the next sub-chunk
    }
    __syncthreads();
    // 4. W row by row (forward substitution): W[t][j] = beta_t ((j == t) - sum_{j <= s < t} A[t][s] W[s][j]); thread j owns column j
    // (column j depends on column j only, so each thread walks down its own column; entries above the diagonal stay zero)
    if (tid < kCh) {
        const int j = tid;
        for (int t = j; t < kCh; ++t) {
            float acc = j == t ? 1.f : 0.f;
            for (int s = j; s < t; ++s) acc = fmaf(-sA[t * kLdC + s], sW[s * kLdC + j], acc);
            sW[t * kLdC + j] = sBeta[t] * acc;
        }
    }
    __syncthreads();
    // 5. results: W, tril(B), the rescaled tiles in place, the chunk's total decay
    float* Wg = cw.W + ((size_t)chunk * p.H + h) * kCh * kCh;
    float* Bg = cw.B + ((size_t)chunk * p.H + h) * kCh * kCh;
    for (int idx = tid; idx < kCh * kCh; idx += 256) {
        const int t = idx / kCh, s = idx % kCh;
        Wg[idx] = sW[t * kLdC + s];
        Bg[idx] = sB[t * kLdC + s];
    }
    const float* gl = sG + (cc - 1) * kLdK;
    for (int idx = tid; idx < cc * (kD / 4); idx += 256) {
        const int t = idx / (kD / 4), c4 = idx % (kD / 4);
        const float4 k4 = *reinterpret_cast<const float4*>(sK + t * kLdK + c4 * 4);
        const float4 q4 = *reinterpret_cast<const float4*>(sQ + t * kLdK + c4 * 4);
        const float4 g4 = *reinterpret_cast<const float4*>(sG + t * kLdK + c4 * 4);
        const float4 l4 = *reinterpret_cast<const float4*>(gl + c4 * 4);
        const float4 eg = make_float4(expf(g4.x), expf(g4.y), expf(g4.z), expf(g4.w));
        const float4 el = make_float4(expf(fminf(l4.x - g4.x, 0.f)), expf(fminf(l4.y - g4.y, 0.f)), expf(fminf(l4.z - g4.z, 0.f)),
                                      expf(fminf(l4.w - g4.w, 0.f)));
        const size_t off = (size_t)(row0 + c0 + t) * C + h * kD + c4 * 4;
        *reinterpret_cast<float4*>(w.qn + off) = make_float4(q4.x * eg.x, q4.y * eg.y, q4.z * eg.z, q4.w * eg.w);
        *reinterpret_cast<float4*>(w.decay + off) = make_float4(k4.x * eg.x, k4.y * eg.y, k4.z * eg.z, k4.w * eg.w);
        *reinterpret_cast<float4*>(w.kn + off) = make_float4(k4.x * el.x, k4.y * el.y, k4.z * el.z, k4.w * el.w);
    }
    if (tid < kD) cw.gC[((size_t)chunk * p.H + h) * kD + tid] = expf(gl[tid]);
}

// acc[ii][jj] += sum_k A[ty + 16 ii][k] B[tx + 16 jj][k]  (both operands row-major with k contiguous, K a multiple of 4)
template <int K>
__device__ __forceinline__ void kda_mm_nt(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, float (&acc)[4][4],
                                          int tx, int ty) {
#pragma unroll 2
    for (int k = 0; k < K; k += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            a[i] = *reinterpret_cast<const float4*>(A + (ty + 16 * i) * lda + k);
            b[i] = *reinterpret_cast<const float4*>(B + (tx + 16 * i) * ldb + k);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                acc[i][j] = fmaf(a[i].x, b[j].x, fmaf(a[i].y, b[j].y, fmaf(a[i].z, b[j].z, fmaf(a[i].w, b[j].w, acc[i][j]))));
    }
}

__global__ void __launch_bounds__(256) kda_chunk_scan_kernel(KdaParams p, KdaScratch w, KdaChunkWs cw) {
    extern __shared__ __align__(16) float csm[];
    float* sS = csm;                         // [64 value channels][128 key channels] state slice
    float* sKp = sS + kCh * kLdK;            // [t][k]
    float* sQp = sKp + kCh * kLdK;
    float* sKm = sQp + kCh * kLdK;
    float* sW = sKm + kCh * kLdK;            // [t][s]
    float* sBm = sW + kCh * kLdC;
    float* sX = sBm + kCh * kLdC;            // (V - Kp S^T)^T : [v][t]
    float* sU = sX + kCh * kLdC;             // U^T : [v][t]
    const int h = blockIdx.x, vs = blockIdx.y, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    pdl_wait();
    pdl_launch_dependents();
    const int row0 = p.seq_row0[0], nrows = p.seq_nrows[0], slot = p.seq_slot[0];
    if (nrows <= 0) return;
    const int C = p.H * kD, vbase = h * kD + vs * kCh;
    float* sp = p.state + (((size_t)slot * p.H + h) * kD + vs * kCh) * kD;
    for (int idx = tid; idx < kCh * (kD / 4); idx += 256) {
        const int v = idx / (kD / 4), c4 = idx % (kD / 4);
        *reinterpret_cast<float4*>(sS + v * kLdK + c4 * 4) = *reinterpret_cast<const float4*>(sp + (size_t)v * kD + c4 * 4);
    }
    const int nchunks = (nrows + kCh - 1) / kCh;
    for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int c0 = chunk * kCh, cc = min(kCh, nrows - c0);
        for (int idx = tid; idx < kCh * (kD / 4); idx += 256) {
            const int t = idx / (kD / 4), c4 = idx % (kD / 4);
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a, c = a;
            if (t < cc) {
                const size_t off = (size_t)(row0 + c0 + t) * C + h * kD + c4 * 4;
                a = *reinterpret_cast<const float4*>(w.decay + off);     // Kp
                b = *reinterpret_cast<const float4*>(w.qn + off);        // Qp
                c = *reinterpret_cast<const float4*>(w.kn + off);        // Km
            }
            *reinterpret_cast<float4*>(sKp + t * kLdK + c4 * 4) = a;
            *reinterpret_cast<float4*>(sQp + t * kLdK + c4 * 4) = b;
            *reinterpret_cast<float4*>(sKm + t * kLdK + c4 * 4) = c;
        }
        const float* Wg = cw.W + ((size_t)chunk * p.H + h) * kCh * kCh;
        const float* Bg = cw.B + ((size_t)chunk * p.H + h) * kCh * kCh;
        for (int idx = tid; idx < kCh * (kCh / 4); idx += 256) {
            const int t = idx / (kCh / 4), c4 = idx % (kCh / 4);
            *reinterpret_cast<float4*>(sW + t * kLdC + c4 * 4) = *reinterpret_cast<const float4*>(Wg + t * kCh + c4 * 4);
            *reinterpret_cast<float4*>(sBm + t * kLdC + c4 * 4) = *reinterpret_cast<const float4*>(Bg + t * kCh + c4 * 4);
        }
        float vreg[4][4], gc[8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int t = ty + 16 * i;
                vreg[i][j] = t < cc ? w.vo[(size_t)(row0 + c0 + t) * C + vbase + tx + 16 * j] : 0.f;
            }
#pragma unroll
        for (int j = 0; j < 8; ++j) gc[j] = cw.gC[((size_t)chunk * p.H + h) * kD + tx + 16 * j];
        __syncthreads();
        float acc[4][4];
        // a. X = V - Kp S^T, stored transposed
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        kda_mm_nt<kD>(sKp, kLdK, sS, kLdK, acc, tx, ty);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) sX[(tx + 16 * j) * kLdC + ty + 16 * i] = vreg[i][j] - acc[i][j];
        __syncthreads();
        // b. U = W X, stored transposed
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        kda_mm_nt<kCh>(sW, kLdC, sX, kLdC, acc, tx, ty);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) sU[(tx + 16 * j) * kLdC + ty + 16 * i] = acc[i][j];
        __syncthreads();
        // c. O = Qp S^T + tril(B) U
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        kda_mm_nt<kD>(sQp, kLdK, sS, kLdK, acc, tx, ty);
        kda_mm_nt<kCh>(sBm, kLdC, sU, kLdC, acc, tx, ty);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = ty + 16 * i;
            if (t < cc) {
#pragma unroll
                for (int j = 0; j < 4; ++j) w.vo[(size_t)(row0 + c0 + t) * C + vbase + tx + 16 * j] = acc[i][j];
            }
        }
        __syncthreads();                                     // every thread has read S before it changes
        // d. S = S diag(gC) + U^T Km : value rows ty + 16 i, key columns tx + 16 j
        float a2[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) a2[i][j] = 0.f;
#pragma unroll 2
        for (int t = 0; t < kCh; ++t) {
            float u[4], km[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) u[i] = sU[(ty + 16 * i) * kLdC + t];
#pragma unroll
            for (int j = 0; j < 8; ++j) km[j] = sKm[t * kLdK + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) a2[i][j] = fmaf(u[i], km[j], a2[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int idx = (ty + 16 * i) * kLdK + tx + 16 * j;
                sS[idx] = fmaf(sS[idx], gc[j], a2[i][j]);
            }
        __syncthreads();
    }
    for (int idx = tid; idx < kCh * (kD / 4); idx += 256) {
        const int v = idx / (kD / 4), c4 = idx % (kD / 4);
        *reinterpret_cast<float4*>(sp + (size_t)v * kD + c4 * 4) = *reinterpret_cast<const float4*>(sS + v * kLdK + c4 * 4);
    }
    if (vs == 0 && tid < kD) kda_update_conv_history(p, row0, nrows, slot, h * kD + tid);
    pdl_launch_dependents();
}
