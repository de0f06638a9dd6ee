// Sparse-attention "lightning" indexer: a cheap single-key-head scorer that picks the
// top-k cache rows each query attends to.
//
//   k_n   = Hadamard(RoPE(LayerNorm(W_k h_n)))  stored as e4m3 + per-entry scale
//   q_h   = Hadamard(RoPE(W_qb q_c))            h = 1..IH index heads
//   score[n] = sum_h w_h * ReLU(q_h . k_n),     w = W_w h * IH^-1/2 * ID^-1/2
//   selection = top-k over causal entries, ties to the lower index, returned ascending.
// IndexPool ("kpool", P tokens per entry): P consecutive LayerNormed keys are pooled by a
// per-dimension softmax over (gate + position-embedding) before the rotation; only complete
// pools are scored (budget = topk / P pools, expanded to token rows) and the incomplete tail
// of the sequence is always selected.
// Reference behaviour: src/compute/kernels/sm120/indexer/indexer_prep.cu:16-89,
// indexer_hadamard.cu:18, external lightning_score / lightning_topk / kpool_compress and the
// CPU specification tests/unit/kpool_reference.h.
#include "common.cuh"

namespace lsb {

constexpr int kID = 128;      // index head dim
constexpr int kIdxRow = 144;  // bytes per cached entry: 128 e4m3 + fp32 scale + pad

__device__ __forceinline__ float fwht128(float v, float* buf) {
    const int t = threadIdx.x;
    for (int s = 1; s < kID; s <<= 1) {
        buf[t] = v;
        __syncthreads();
        const float o = buf[t ^ s];
        v = (t & s) ? (o - v) : (v + o);
        __syncthreads();
    }
    return v * 0.08838834764831845f;
}

__device__ __forceinline__ void rope_first(float& v, float* buf, int dr, float pos, const float* inv_freq) {
    // interleaved pairs over the first dr dims
    const int t = threadIdx.x;
    buf[t] = v;
    __syncthreads();
    if (t < dr) {
        const int i = t >> 1;
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        const float a = buf[t & ~1], b = buf[t | 1];
        v = (t & 1) ? (a * s + b * c) : (a * c - b * s);
    }
    __syncthreads();
}

// Quantise one 128-vector (one element per thread) and store [e4m3 x128 | scale].
__device__ __forceinline__ void store_entry(uint8_t* row, float v, float* red, bool pow2) {
    const float amax = block_max(fabsf(v), red);
    float scale;
    if (pow2) scale = exp2f(ceilf(log2f(fmaxf(amax, 1e-4f) / 448.f)));
    else scale = fmaxf(amax, 1e-10f) / 448.f;
    row[threadIdx.x] = float_to_fp8e4m3(fminf(fmaxf(v / scale, -448.f), 448.f));
    if (threadIdx.x == 0) *reinterpret_cast<float*>(row + kID) = scale;
}

struct IdxAppendParams {
    const float* proj; int ldp, off_k, off_gate;   // fp32 projections of the row
    const float* ln_w; const float* ln_b; const float* ape;   // ape [P,128] (kpool only)
    const float* inv_freq; int dr;
    uint8_t* cache; const int* block_table; int max_pages, page;   // entries per page = `page`
    const bf16* tail;         // [slots, P, 2, 128] LayerNormed key | gate of the open pool (kpool only);
                              // read-only here: written by indexer_q_prep, which runs after every
                              // block of this kernel has finished (no in-launch read/write race)
    bf16* kstash;             // [rows, 128] this launch's LayerNormed keys (kpool only)
    const int* row_seq; const int* row_pos; const int* row_slot;
    int P; float ln_eps;
};

// LayerNorm + RoPE of one row's raw indexer key (one element per thread).
__device__ __forceinline__ float idx_key_of_row(const IdxAppendParams& p, int row, int pos, float* buf, float* red) {
    const int t = threadIdx.x;
    float v = p.proj[(size_t)row * p.ldp + p.off_k + t];
    const float mean = block_sum(v, red) / (float)kID;
    const float dv = v - mean;
    const float var = block_sum(dv * dv, red) / (float)kID;
    v = dv * rsqrtf(var + p.ln_eps) * p.ln_w[t] + p.ln_b[t];
    if (p.dr > 0) rope_first(v, buf, p.dr, (float)pos, p.inv_freq);
    return v;
}

__global__ void __launch_bounds__(kID) indexer_k_append_kernel(IdxAppendParams p) {
    __shared__ float buf[kID];
    __shared__ float red[33];
    const int r = blockIdx.x, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int seq = p.row_seq[r], pos = p.row_pos[r];
    if (seq < 0) return;
    const float* pr = p.proj + (size_t)r * p.ldp;
    float v = idx_key_of_row(p, r, pos, buf, red);
    if (p.P <= 1) {
        v = fwht128(__bfloat162float(__float2bfloat16(v)), buf);
        const int pg = p.block_table[(size_t)seq * p.max_pages + pos / p.page];
        store_entry(p.cache + ((size_t)pg * p.page + pos % p.page) * kIdxRow, __bfloat162float(__float2bfloat16(v)), red, false);
    } else {
        const int slot = p.row_slot[r], j = pos % p.P;
        p.kstash[(size_t)r * kID + t] = __float2bfloat16(v);
        if (j == p.P - 1) {
            // Compose the pooled entry: two-pass softmax over the P slots per dimension.  Slots
            // written by earlier rows of THIS launch are recomputed from their projections (other
            // blocks may not have stored them yet); older slots come from the tail buffer.
            const bf16* t0 = p.tail + (size_t)slot * p.P * 2 * kID;
            float kk[8], s[8];
            float m = -INFINITY;
            for (int jj = 0; jj < p.P; ++jj) {
                const int d = j - jj, rr = r - d;
                float kv, gv;
                if (d == 0) {
                    kv = v; gv = pr[p.off_gate + t];
                } else if (rr >= 0 && p.row_seq[rr] == seq && p.row_pos[rr] == pos - d) {
                    kv = idx_key_of_row(p, rr, pos - d, buf, red);
                    gv = p.proj[(size_t)rr * p.ldp + p.off_gate + t];
                } else {
                    kv = __bfloat162float(t0[(size_t)jj * 2 * kID + t]);
                    gv = __bfloat162float(t0[(size_t)jj * 2 * kID + kID + t]);
                }
                kk[jj] = __bfloat162float(__float2bfloat16(kv));
                s[jj] = __bfloat162float(__float2bfloat16(gv)) + p.ape[jj * kID + t];
                m = fmaxf(m, s[jj]);
            }
            float Z = 0.f, acc = 0.f;
            for (int jj = 0; jj < p.P; ++jj) {
                const float e = expf(s[jj] - m);
                Z += e; acc += e * kk[jj];
            }
            float x = __bfloat162float(__float2bfloat16(acc / Z));
            x = __bfloat162float(__float2bfloat16(fwht128(x, buf)));
            const int entry = pos / p.P;
            const int pg = p.block_table[(size_t)seq * p.max_pages + entry / p.page];
            store_entry(p.cache + ((size_t)pg * p.page + entry % p.page) * kIdxRow, x, red, true);
        }
    }
    pdl_launch_dependents();
}

// q rows: [R, IH, 128] from the fused q_b projection (bf16, stride ldq, offset off_q);
// weights from the fused input projection.  Out: q_idx bf16 [R,IH,128], w fp32 [R,IH].
__global__ void __launch_bounds__(kID) indexer_q_prep_kernel(const bf16* __restrict__ qproj, int ldq, int off_q,
                                                              const float* __restrict__ proj, int ldp, int off_w, int IH, int dr,
                                                              const float* __restrict__ inv_freq, const int* __restrict__ row_pos,
                                                              bf16* __restrict__ q_idx, float* __restrict__ w_out,
                                                              const bf16* __restrict__ kstash, int off_gate, bf16* __restrict__ tail,
                                                              const int* __restrict__ row_seq, const int* __restrict__ row_slot, int P, int R) {
    __shared__ float buf[kID];
    const int r = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    if (h == 0 && P > 1 && row_seq[r] >= 0) {
        // publish this row's key | gate to the sequence's open-pool tail unless the pool is
        // completed by a later row of this same launch (then nobody will read it)
        const int ipos = row_pos[r], j = ipos % P, rc = r + (P - 1 - j);
        const bool completes_here = (j == P - 1) || (rc < R && row_seq[rc] == row_seq[r] && row_pos[rc] == ipos + (P - 1 - j));
        if (!completes_here) {
            bf16* tl = tail + ((size_t)row_slot[r] * P + j) * 2 * kID;
            tl[t] = kstash[(size_t)r * kID + t];
            tl[kID + t] = __float2bfloat16(proj[(size_t)r * ldp + off_gate + t]);
        }
    }
    const float pos = (float)row_pos[r];
    {
        float v = __bfloat162float(qproj[(size_t)r * ldq + off_q + h * kID + t]);
        if (dr > 0) rope_first(v, buf, dr, pos, inv_freq);
        v = fwht128(__bfloat162float(__float2bfloat16(v)), buf);
        q_idx[((size_t)r * IH + h) * kID + t] = __float2bfloat16(v);
    }
    if (h == 0 && t < IH) w_out[(size_t)r * IH + t] = proj[(size_t)r * ldp + off_w + t] * rsqrtf((float)IH) * rsqrtf((float)kID);
    pdl_launch_dependents();
}

// scores[r][n] for n < n_entries[r]; one thread per entry, q staged in shared memory.
__global__ void __launch_bounds__(128) indexer_score_kernel(const bf16* __restrict__ q_idx, const float* __restrict__ w, int IH,
                                                            const uint8_t* __restrict__ cache, const int* __restrict__ block_table,
                                                            int max_pages, int page, const int* __restrict__ row_seq,
                                                            const int* __restrict__ n_entries, float* __restrict__ scores, int ld_scores) {
    extern __shared__ __align__(16) uint8_t smraw[];
    bf16* qs = reinterpret_cast<bf16*>(smraw);                 // [IH][128]
    float* ws = reinterpret_cast<float*>(qs + IH * kID);       // [IH]
    const int r = blockIdx.y, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int seq = row_seq[r];
    const int ne = seq < 0 ? 0 : n_entries[r];
    if ((int)(blockIdx.x * blockDim.x) >= ne) return;
    for (int i = t; i < IH * kID / 8; i += blockDim.x)
        reinterpret_cast<uint4*>(qs)[i] = reinterpret_cast<const uint4*>(q_idx + (size_t)r * IH * kID)[i];
    if (t < IH) ws[t] = w[(size_t)r * IH + t];
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + t;
    if (n >= ne) return;
    const int pg = block_table[(size_t)seq * max_pages + n / page];
    const uint8_t* row = cache + ((size_t)pg * page + n % page) * kIdxRow;
    float k[kID];
#pragma unroll
    for (int c = 0; c < kID / 16; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(row + c * 16);
        unpack_fp8x4(v.x, k + c * 16); unpack_fp8x4(v.y, k + c * 16 + 4);
        unpack_fp8x4(v.z, k + c * 16 + 8); unpack_fp8x4(v.w, k + c * 16 + 12);
    }
    const float ks = *reinterpret_cast<const float*>(row + kID);
    float acc = 0.f;
    for (int h = 0; h < IH; ++h) {
        float d = 0.f;
#pragma unroll
        for (int c = 0; c < kID; c += 8) {
            float qf[8];
            unpack_bf16x8(*reinterpret_cast<const uint4*>(qs + h * kID + c), qf);
#pragma unroll
            for (int e = 0; e < 8; ++e) d = fmaf(qf[e], k[c + e], d);
        }
        acc = fmaf(fmaxf(d * ks, 0.f), ws[h], acc);
    }
    scores[(size_t)r * ld_scores + n] = acc;
    pdl_launch_dependents();
}

__device__ __forceinline__ uint32_t sortable(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Per row: radix-select the `budget` best of n_elig entries (ties to the lower index), emit
// them in ascending order expanded by P, then append the always-selected tail tokens.
//   n_elig = complete, causal entries; tail = [n_elig*P, len).  If n_elig <= budget all are taken.
__global__ void __launch_bounds__(1024) indexer_topk_kernel(const float* __restrict__ scores, int ld_scores,
                                                            const int* __restrict__ n_entries, const int* __restrict__ row_len,
                                                            const int* __restrict__ row_seq, int budget, int P,
                                                            int* __restrict__ sel_idx, int* __restrict__ sel_cnt, int sel_ld) {
    __shared__ int hist[256];
    __shared__ int s_scan[33];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need, s_base, s_eqbase;
    const int r = blockIdx.x, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int len = row_seq[r] < 0 ? 0 : row_len[r];
    const int ne = row_seq[r] < 0 ? 0 : n_entries[r];
    const float* sc = scores + (size_t)r * ld_scores;
    int* out = sel_idx + (size_t)r * sel_ld;
    int nsel_entries;
    if (ne <= budget) {
        for (int i = t; i < ne * P; i += blockDim.x) out[i] = i;
        nsel_entries = ne;
    } else {
        // Keys live in registers when the row has at most 8 entries per thread (context up to 8k
        // pooled entries); longer rows re-read the scores from memory in every pass.
        constexpr int KPT = 8;
        const bool in_regs = ne <= 1024 * KPT;
        uint32_t key[KPT];
        if (in_regs) {
#pragma unroll
            for (int u = 0; u < KPT; ++u) { const int i = t + u * 1024; key[u] = i < ne ? sortable(sc[i]) : 0u; }
        }
        // find the key of the budget-th largest element, 8 bits at a time
        if (t == 0) { s_prefix = 0; s_need = budget; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = t; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix;
            const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            if (in_regs) {
#pragma unroll
                for (int u = 0; u < KPT; ++u)
                    if (t + u * 1024 < ne && (key[u] & mask) == prefix) atomicAdd(&hist[(key[u] >> shift) & 255], 1);
            } else {
                for (int i = t; i < ne; i += blockDim.x) {
                    const uint32_t k = sortable(sc[i]);
                    if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1);
                }
            }
            __syncthreads();
            if (t < 32) {
                // bucket search from the top by one warp: each lane sums 8 buckets, then a serial walk over 32 + 8 items
                int part = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) part += hist[255 - (t * 8 + j)];
                int need = s_need, grp = 31;
                for (int l = 0; l < 32; ++l) {
                    const int pl = __shfl_sync(0xffffffffu, part, l);
                    if (pl >= need) { grp = l; break; }
                    need -= pl;
                }
                if (t == 0) {
                    int b = 255 - grp * 8;
                    for (int j = 0; j < 8; ++j, --b) {
                        if (hist[b] >= need || b == 0 || j == 7) break;
                        need -= hist[b];
                    }
                    s_need = need;
                    s_prefix = prefix | ((uint32_t)b << shift);
                }
            }
            __syncthreads();
        }
        const uint32_t T = s_prefix;   // threshold key; s_need = how many equal-to-T to take
        const int quota = s_need;
        if (t == 0) { s_base = 0; s_eqbase = 0; }
        __syncthreads();
        const int lane = t & 31, w = t >> 5;
        auto emit_chunk = [&](int i, uint32_t k) {
            const int gt = (i < ne && k > T) ? 1 : 0, eq = (i < ne && k == T) ? 1 : 0;
            // block exclusive scan of eq
            int v = eq;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int n = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += n; }
            if (lane == 31) s_scan[w] = v;
            __syncthreads();
            if (w == 0) {
                int x = s_scan[lane];
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const int n = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += n; }
                s_scan[lane] = x;
            }
            __syncthreads();
            const int eq_rank = s_eqbase + (w ? s_scan[w - 1] : 0) + v - eq;
            const int eq_total = s_scan[31];
            const int take = gt | (eq && eq_rank < quota);
            __syncthreads();
            int uu = take;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int n = __shfl_up_sync(0xffffffffu, uu, o); if (lane >= o) uu += n; }
            if (lane == 31) s_scan[w] = uu;
            __syncthreads();
            if (w == 0) {
                int x = s_scan[lane];
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const int n = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += n; }
                s_scan[lane] = x;
            }
            __syncthreads();
            const int posn = s_base + (w ? s_scan[w - 1] : 0) + uu - take;
            if (take && posn < budget)
                for (int j = 0; j < P; ++j) out[posn * P + j] = i * P + j;
            const int tot = s_scan[31];
            __syncthreads();
            if (t == 0) { s_base += tot; s_eqbase += eq_total; }
            __syncthreads();
        };
        if (in_regs) {
#pragma unroll
            for (int u = 0; u < KPT; ++u)
                if (u * 1024 < ne) emit_chunk(u * 1024 + t, key[u]);
        } else {
            for (int c0 = 0; c0 < ne; c0 += blockDim.x) emit_chunk(c0 + t, (c0 + t < ne) ? sortable(sc[c0 + t]) : 0u);
        }
        nsel_entries = budget;
    }
    const int tail0 = ne * P;
    for (int i = tail0 + t; i < len; i += blockDim.x) out[nsel_entries * P + (i - tail0)] = i;
    if (t == 0) sel_cnt[r] = nsel_entries * P + max(0, len - tail0);
    pdl_launch_dependents();
}


// ---- the same selection spread over many blocks (few rows, long rows) ------------------------------------------------------
// One block per row walks a 262k-entry row (a 1M-token context pooled by 4) in ~600 us: four passes over the row and 256
// emit rounds of six block barriers each.  Here every block owns 2048 consecutive entries of a row and the row's blocks meet in
// global memory: three histogram launches (11 + 11 + 10 key bits; the block that arrives last picks the bucket and leaves the
// histogram and the ticket zeroed for the next launch), one counting launch (entries above / equal to the threshold per block;
// the last block turns the counts into output offsets) and one emit launch.  Integer atomics only: the result does not depend on
// the order in which blocks run, and it is the single-block kernel's result entry for entry (ascending, ties to the lower index).
constexpr int kTkChunk = 2048;
constexpr int kTkThreads = 256;
constexpr int kTkBins = 2048;
struct TopkSplitRow {
    int hist[kTkBins];
    uint32_t prefix;      // the key bits decided so far
    int need;             // how many entries are still to be taken from the bucket of `prefix`
    unsigned ticket;
    int pad;
};

// Exclusive prefix sum over the block's 256 threads; `total` = the block's sum.  s_w: 8 ints of shared memory.
__device__ __forceinline__ int block_excl_scan_256(int v, int* s_w, int& total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int n = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += n; }
    __syncthreads();                       // s_w may still be read from a previous scan
    if (lane == 31) s_w[w] = x;
    __syncthreads();
    int base = 0, tot = 0;
#pragma unroll
    for (int j = 0; j < kTkThreads / 32; ++j) { const int sw = s_w[j]; if (j < w) base += sw; tot += sw; }
    total = tot;
    return base + x - v;
}

// true in exactly one block of the row: the one that took the last of `nb` tickets (all its threads return the same value)
__device__ __forceinline__ bool last_block_of_row(unsigned* ticket, int nb, int* s_flag) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *s_flag = (atomicAdd(ticket, 1u) == (unsigned)(nb - 1)) ? 1 : 0;
    __syncthreads();
    const bool last = *s_flag != 0;
    if (last) __threadfence();
    return last;
}

template <int LEVEL>
__global__ void __launch_bounds__(kTkThreads) indexer_topk_hist_kernel(const float* __restrict__ scores, int ld_scores,
                                                                       const int* __restrict__ n_entries, const int* __restrict__ row_seq,
                                                                       int budget, TopkSplitRow* __restrict__ st_all) {
    constexpr int shift = LEVEL == 0 ? 21 : (LEVEL == 1 ? 10 : 0);
    constexpr int nbins = LEVEL == 2 ? 1024 : 2048;
    __shared__ int hist[kTkBins];
    __shared__ int s_w[kTkThreads / 32];
    __shared__ int s_flag;
    const int r = blockIdx.y, b = blockIdx.x, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int ne = row_seq[r] < 0 ? 0 : n_entries[r];
    if (ne <= budget || b * kTkChunk >= ne) return;            // short rows are taken whole by the emit kernel
    TopkSplitRow& st = st_all[r];
    const int nb = (ne + kTkChunk - 1) / kTkChunk;
    for (int i = t; i < nbins; i += kTkThreads) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = LEVEL == 0 ? 0u : st.prefix;
    const int need_in = LEVEL == 0 ? budget : st.need;
    const float* sc = scores + (size_t)r * ld_scores;
#pragma unroll
    for (int u = 0; u < kTkChunk / kTkThreads; ++u) {
        const int i = b * kTkChunk + u * kTkThreads + t;
        if (i < ne) {
            const uint32_t k = sortable(sc[i]);
            if (LEVEL == 0 || (k >> (shift + (LEVEL == 1 ? 11 : 10))) == (prefix >> (shift + (LEVEL == 1 ? 11 : 10))))
                atomicAdd(&hist[(k >> shift) & (nbins - 1)], 1);
        }
    }
    __syncthreads();
    for (int i = t; i < nbins; i += kTkThreads) { const int h = hist[i]; if (h) atomicAdd(&st.hist[i], h); }
    if (!last_block_of_row(&st.ticket, nb, &s_flag)) return;
    // the row's histogram is complete: find the bucket that holds the need_in-th largest key, walking from the top
    int part = 0, mine[8];
    constexpr int per = nbins / kTkThreads;                     // 8 or 4 buckets per thread, thread 0 owns the top ones
#pragma unroll
    for (int j = 0; j < per; ++j) {
        const int bin = nbins - 1 - (t * per + j);
        mine[j] = __ldcg(&st.hist[bin]);
        st.hist[bin] = 0;                                       // left zeroed for the next launch
        part += mine[j];
    }
    int total;
    const int before = block_excl_scan_256(part, s_w, total);
    if (before < need_in && before + part >= need_in) {
        int need = need_in - before, bin = nbins - 1 - t * per;
#pragma unroll
        for (int j = 0; j < per; ++j, --bin) {
            if (mine[j] >= need || j == per - 1) break;
            need -= mine[j];
        }
        st.prefix = prefix | ((uint32_t)bin << shift);
        st.need = need;
    }
    if (t == 0) st.ticket = 0;
}

// Per block: how many of its entries lie above / on the threshold; the last block turns the counts into the blocks' first output
// position (blk[2 * nblk + b]) and the number of threshold-equal entries in front of the block (blk[3 * nblk + b]).
__global__ void __launch_bounds__(kTkThreads) indexer_topk_count_kernel(const float* __restrict__ scores, int ld_scores,
                                                                        const int* __restrict__ n_entries, const int* __restrict__ row_seq,
                                                                        int budget, TopkSplitRow* __restrict__ st_all, int* __restrict__ blk_all,
                                                                        int nblk) {
    __shared__ int s_w[kTkThreads / 32];
    __shared__ int s_flag;
    const int r = blockIdx.y, b = blockIdx.x, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int ne = row_seq[r] < 0 ? 0 : n_entries[r];
    if (ne <= budget || b * kTkChunk >= ne) return;
    TopkSplitRow& st = st_all[r];
    int* blk = blk_all + (size_t)r * 4 * nblk;
    const int nb = (ne + kTkChunk - 1) / kTkChunk;
    const uint32_t T = st.prefix;
    const int quota = st.need;
    const float* sc = scores + (size_t)r * ld_scores;
    int gt = 0, eq = 0;
#pragma unroll
    for (int u = 0; u < kTkChunk / kTkThreads; ++u) {
        const int i = b * kTkChunk + u * kTkThreads + t;
        if (i < ne) { const uint32_t k = sortable(sc[i]); gt += k > T; eq += k == T; }
    }
    int tot_gt, tot_eq;
    block_excl_scan_256(gt, s_w, tot_gt);
    block_excl_scan_256(eq, s_w, tot_eq);
    if (t == 0) { blk[b] = tot_gt; blk[nblk + b] = tot_eq; }
    if (!last_block_of_row(&st.ticket, nb, &s_flag)) return;
    // thread t owns blocks [t * per, (t + 1) * per): equal entries in front first, then the taken entries in front
    const int per = (nb + kTkThreads - 1) / kTkThreads;
    int sum_eq = 0;
    for (int j = 0; j < per; ++j) { const int bb = t * per + j; if (bb < nb) sum_eq += __ldcg(&blk[nblk + bb]); }
    int dummy;
    int eq_before = block_excl_scan_256(sum_eq, s_w, dummy);
    int sum_take = 0;
    for (int j = 0; j < per; ++j) {
        const int bb = t * per + j;
        if (bb < nb) {
            const int e = __ldcg(&blk[nblk + bb]);
            blk[3 * nblk + bb] = eq_before;
            sum_take += __ldcg(&blk[bb]) + min(e, max(0, quota - eq_before));
            eq_before += e;
        }
    }
    int pos = block_excl_scan_256(sum_take, s_w, dummy);
    for (int j = 0; j < per; ++j) {
        const int bb = t * per + j;
        if (bb < nb) {
            blk[2 * nblk + bb] = pos;
            pos += __ldcg(&blk[bb]) + min(__ldcg(&blk[nblk + bb]), max(0, quota - blk[3 * nblk + bb]));
        }
    }
    if (t == 0) st.ticket = 0;
}

__global__ void __launch_bounds__(kTkThreads) indexer_topk_emit_kernel(const float* __restrict__ scores, int ld_scores,
                                                                       const int* __restrict__ n_entries, const int* __restrict__ row_len,
                                                                       const int* __restrict__ row_seq, int budget, int P,
                                                                       const TopkSplitRow* __restrict__ st_all, const int* __restrict__ blk_all, int nblk,
                                                                       int* __restrict__ sel_idx, int* __restrict__ sel_cnt, int sel_ld) {
    constexpr int per = kTkChunk / kTkThreads;                  // 8 consecutive entries per thread: output order = index order
    __shared__ uint32_t s_key[kTkChunk + kTkThreads];           // padded: thread t reads words t * 9 ..
    __shared__ int s_w[kTkThreads / 32];
    const int r = blockIdx.y, b = blockIdx.x, t = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int len = row_seq[r] < 0 ? 0 : row_len[r];
    const int ne = row_seq[r] < 0 ? 0 : n_entries[r];
    int* out = sel_idx + (size_t)r * sel_ld;
    const int nsel_entries = ne <= budget ? ne : budget;
    if (b == 0) {                                               // the always-selected tail and the count
        const int tail0 = ne * P;
        for (int i = tail0 + t; i < len; i += kTkThreads) out[nsel_entries * P + (i - tail0)] = i;
        if (t == 0) sel_cnt[r] = nsel_entries * P + max(0, len - tail0);
    }
    if (b * kTkChunk >= ne) return;
    if (ne <= budget) {
        const int hi = min(ne, (b + 1) * kTkChunk) * P;
        for (int i = b * kTkChunk * P + t; i < hi; i += kTkThreads) out[i] = i;
        return;
    }
    const TopkSplitRow& st = st_all[r];
    const int* blk = blk_all + (size_t)r * 4 * nblk;
    const uint32_t T = st.prefix;
    const int quota = st.need;
    const float* sc = scores + (size_t)r * ld_scores;
#pragma unroll
    for (int u = 0; u < per; ++u) {
        const int j = u * kTkThreads + t, i = b * kTkChunk + j;
        s_key[j + j / per] = i < ne ? sortable(sc[i]) : 0u;      // entry j of the block sits at word j + j / 8
    }
    __syncthreads();
    uint32_t key[per];
    int n_eq = 0;
#pragma unroll
    for (int u = 0; u < per; ++u) {
        key[u] = s_key[t * (per + 1) + u];
        n_eq += (b * kTkChunk + t * per + u < ne) && key[u] == T;
    }
    int dummy;
    int eq_rank = blk[3 * nblk + b] + block_excl_scan_256(n_eq, s_w, dummy);
    unsigned take = 0;
#pragma unroll
    for (int u = 0; u < per; ++u) {
        const bool in = b * kTkChunk + t * per + u < ne;
        if (in && key[u] > T) take |= 1u << u;
        else if (in && key[u] == T) { if (eq_rank < quota) take |= 1u << u; ++eq_rank; }
    }
    int pos = blk[2 * nblk + b] + block_excl_scan_256(__popc(take), s_w, dummy);
#pragma unroll
    for (int u = 0; u < per; ++u) {
        if ((take >> u) & 1u) {
            if (pos < budget) {
                const int i = b * kTkChunk + t * per + u;
                for (int j = 0; j < P; ++j) out[pos * P + j] = i * P + j;
            }
            ++pos;
        }
    }
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_indexer_row_bytes() { return kIdxRow; }

LSB_API int lsb_indexer_k_append(const void* proj, int ldp, int off_k, int off_gate, const void* ln_w, const void* ln_b,
                                 const void* ape, const void* inv_freq, int dr, void* cache, const void* block_table,
                                 int max_pages, int page, const void* tail, void* kstash, const void* row_seq,
                                 const void* row_pos, const void* row_slot, int rows, int P, float ln_eps, void* stream) {
    if (P > 8) return -1;
    IdxAppendParams p;
    p.proj = (const float*)proj; p.ldp = ldp; p.off_k = off_k; p.off_gate = off_gate; p.ln_w = (const float*)ln_w;
    p.ln_b = (const float*)ln_b; p.ape = (const float*)ape; p.inv_freq = (const float*)inv_freq; p.dr = dr;
    p.cache = (uint8_t*)cache; p.block_table = (const int*)block_table; p.max_pages = max_pages; p.page = page;
    p.tail = (const bf16*)tail; p.kstash = (bf16*)kstash; p.row_seq = (const int*)row_seq; p.row_pos = (const int*)row_pos; p.row_slot = (const int*)row_slot;
    p.P = P; p.ln_eps = ln_eps;
    launch_pdl((indexer_k_append_kernel), rows, kID, 0, (cudaStream_t)stream, p);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_indexer_q_prep(const void* qproj, int ldq, int off_q, const void* proj, int ldp, int off_w, int IH, int dr,
                               const void* inv_freq, const void* row_pos, void* q_idx, void* w_out, const void* kstash,
                               int off_gate, void* tail, const void* row_seq, const void* row_slot, int P, int rows, void* stream) {
    if (IH > kID) return -1;
    launch_pdl((indexer_q_prep_kernel), dim3(rows, IH), kID, 0, (cudaStream_t)stream, (const bf16*)qproj, ldq, off_q, (const float*)proj, ldp, off_w, IH, dr,
                                                                 (const float*)inv_freq, (const int*)row_pos, (bf16*)q_idx, (float*)w_out,
                                                                 (const bf16*)kstash, off_gate, (bf16*)tail, (const int*)row_seq,
                                                                 (const int*)row_slot, P, rows);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_indexer_score(const void* q_idx, const void* w, int IH, const void* cache, const void* block_table,
                              int max_pages, int page, const void* row_seq, const void* n_entries, void* scores,
                              int ld_scores, int rows, int max_entries, void* stream) {
    if (max_entries <= 0) return 0;
    dim3 grid((max_entries + 127) / 128, rows);
    launch_pdl((indexer_score_kernel), grid, 128, (size_t)IH * kID * 2 + IH * 4, (cudaStream_t)stream, (const bf16*)q_idx, (const float*)w, IH, (const uint8_t*)cache,
                                                                                            (const int*)block_table, max_pages, page, (const int*)row_seq,
                                                                                            (const int*)n_entries, (float*)scores, ld_scores);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_indexer_topk(const void* scores, int ld_scores, const void* n_entries, const void* row_len,
                             const void* row_seq, int budget, int P, void* sel_idx, void* sel_cnt, int sel_ld, int rows,
                             void* stream) {
    launch_pdl((indexer_topk_kernel), rows, 1024, 0, (cudaStream_t)stream, (const float*)scores, ld_scores, (const int*)n_entries, (const int*)row_len,
                                                               (const int*)row_seq, budget, P, (int*)sel_idx, (int*)sel_cnt, sel_ld);
    LSB_CHECK_LAUNCH();
}

// Bytes of zero-initialised scratch the split selection needs for `rows` rows of up to `max_entries` entries.
LSB_API int lsb_indexer_topk_split_scratch(int rows, int max_entries) {
    const long long nblk = (max_entries + kTkChunk - 1) / kTkChunk;
    const long long n = (long long)rows * (long long)sizeof(TopkSplitRow) + (long long)rows * 4 * nblk * 4;
    return n > 0x7fffffffLL ? -1 : (int)n;
}

// The selection of lsb_indexer_topk with every row spread over ceil(max_entries / 2048) blocks (five launches); meant for steps of
// few rows over long rows.  scratch: lsb_indexer_topk_split_scratch bytes, zeroed once (every launch leaves it zeroed where needed).
LSB_API int lsb_indexer_topk_split(const void* scores, int ld_scores, const void* n_entries, const void* row_len, const void* row_seq,
                                   int budget, int P, void* sel_idx, void* sel_cnt, int sel_ld, int rows, int max_entries, void* scratch,
                                   void* stream) {
    if (rows <= 0 || max_entries <= 0) return 0;
    const int nblk = (max_entries + kTkChunk - 1) / kTkChunk;
    TopkSplitRow* st = (TopkSplitRow*)scratch;
    int* blk = (int*)((char*)scratch + (size_t)rows * sizeof(TopkSplitRow));
    const dim3 grid(nblk, rows);
    cudaStream_t s = (cudaStream_t)stream;
    launch_pdl((indexer_topk_hist_kernel<0>), grid, kTkThreads, 0, s, (const float*)scores, ld_scores, (const int*)n_entries, (const int*)row_seq, budget, st);
    launch_pdl((indexer_topk_hist_kernel<1>), grid, kTkThreads, 0, s, (const float*)scores, ld_scores, (const int*)n_entries, (const int*)row_seq, budget, st);
    launch_pdl((indexer_topk_hist_kernel<2>), grid, kTkThreads, 0, s, (const float*)scores, ld_scores, (const int*)n_entries, (const int*)row_seq, budget, st);
    launch_pdl((indexer_topk_count_kernel), grid, kTkThreads, 0, s, (const float*)scores, ld_scores, (const int*)n_entries, (const int*)row_seq, budget, st, blk, nblk);
    launch_pdl((indexer_topk_emit_kernel), grid, kTkThreads, 0, s, (const float*)scores, ld_scores, (const int*)n_entries, (const int*)row_len,
               (const int*)row_seq, budget, P, (const TopkSplitRow*)st, (const int*)blk, nblk, (int*)sel_idx, (int*)sel_cnt, sel_ld);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_indexer(void* buf) { return lsb_trace_install(buf); }
