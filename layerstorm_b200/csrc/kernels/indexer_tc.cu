// Lightning-indexer scores of a prefill chunk on the tensor cores.
//
//   scores[r][n] = ks[n] * sum_h w[r][h] * relu(q[r][h] . k[n])        r = query row of the chunk, n = pooled index entry, h = index head
//
// All rows of a prefill chunk belong to one sequence and share its index keys, so the inner products are one GEMM:
// keys are the 128-row UMMA "A" operand (M), the (row, head) pairs of 256 / IH consecutive query rows the "B" operand
// (N = 256), the reduction is the 128-wide index head dimension (two TMA stages of 64 bf16).  With the keys on the
// tensor-memory lanes, one thread owns one key and finds all heads of a query row in consecutive accumulator columns:
// the ReLU, the head weights and the sum over heads run in registers with no cross-lane traffic, and the scores of a row
// are stored coalesced over the keys.
//   indexer_keys_bf16   gathers the sequence's FP8 index entries through the page table into a dense bf16 [entries, 128]
//                       operand (E4M3 values are exact in bf16) and their fp32 scales into a vector
//   indexer_score_tc    one CTA per (128 keys, 256 / IH rows): warp 0 TMA, warp 1 tcgen05.mma (kind::f16, bf16, fp32
//                       accumulate in tensor memory), warps 2-5 epilogue.  Tiles above the causal frontier of their rows exit.
// The CUDA-core kernel (indexer.cu, one thread per (row, entry)) stays for decode steps and mixed batches; it costs
// 1.5 ms per layer and 2048-row chunk at 8k context and grows linearly with the context.
// Reference seam replaced: lightning_indexer score kernels (src/compute/kernels/sm120/attention/lightning_indexer*.cu).
#include "tc_common.cuh"

namespace lsb {
using namespace tc;

int cached_map_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, int esize, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t br, uint32_t bc);

constexpr int kScD = 128;        // index head dimension
constexpr int kScEntry = 144;    // bytes per cached entry: 128 e4m3 + fp32 scale + pad (indexer.cu)
constexpr int kScKeys = 128;     // keys per tile (UMMA M)
constexpr int kScN = 256;        // (row, head) pairs per tile (UMMA N)

// kbf[n][0..127] = bf16(e4m3 key n), kscale[n] = its scale, for n < n_entries[rows - 1]; 16 threads per entry.
__global__ void __launch_bounds__(256) indexer_keys_bf16_kernel(const uint8_t* __restrict__ cache, const int* __restrict__ block_table, int max_pages,
                                                                int page, const int* __restrict__ row_seq, const int* __restrict__ n_entries, int rows,
                                                                bf16* __restrict__ kbf, float* __restrict__ kscale) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x * 16 + (threadIdx.x >> 4), part = threadIdx.x & 15;
    const int seq = row_seq[0];
    if (seq < 0 || n >= n_entries[rows - 1]) return;
    const int pg = block_table[(size_t)seq * max_pages + n / page];
    const uint8_t* row = cache + ((size_t)pg * page + n % page) * kScEntry;
    const uint2 v = *reinterpret_cast<const uint2*>(row + part * 8);
    float f[8];
    unpack_fp8x4(v.x, f);
    unpack_fp8x4(v.y, f + 4);
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(kbf + (size_t)n * kScD + part * 8) = *reinterpret_cast<uint4*>(h);
    if (part == 0) kscale[n] = *reinterpret_cast<const float*>(row + kScD);
}

struct ScoreTcParams {
    const float* w;            // [rows, IH]
    const float* kscale;       // [entries]
    const int* n_entries;      // [rows], non-decreasing over the chunk
    const int* row_seq;
    float* scores; int ld_scores;
    int rows, IH;
    int* err;
};

constexpr int kScStage = kScKeys * 128 + kScN * 128;     // one 64-element reduction stage: keys 16 KB + (row, head) pairs 32 KB
constexpr int kScSmem = 2 * kScStage + 1024 /*align*/ + 256 /*barriers*/ + kScN * 4 /*head weights*/ + 64 * 4 /*entries per row*/;

__global__ void __launch_bounds__(192) indexer_score_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_q,
                                                               ScoreTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + 2 * kScStage);      // [2]
    uint64_t* acc_full = full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);
    float* wsm = reinterpret_cast<float*>(smem + 2 * kScStage + 256);       // [256] head weight of every accumulator column
    int* nes = reinterpret_cast<int*>(wsm + kScN);                           // [rows per tile]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rpt = kScN / p.IH;                                            // query rows per tile
    const int k0 = blockIdx.x * kScKeys, r0 = blockIdx.y * rpt;

    if (threadIdx.x == 0) {
        mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_init(acc_full, 1);
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_q);
    }
    if (warp == 1) tmem_alloc(tmem_holder, kScN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_holder;
    pdl_wait();
    pdl_launch_dependents();
    // causal frontier of this tile's rows (entries visible to the last of them); the whole CTA takes the same branch
    const int r_last = min(r0 + rpt, p.rows) - 1;
    const int ne_tile = (p.row_seq[0] < 0 || r_last < r0) ? 0 : p.n_entries[r_last];
    const bool live = k0 < ne_tile;
    if (live) {
        for (int i = threadIdx.x; i < kScN; i += blockDim.x) {
            const int r = r0 + i / p.IH;
            wsm[i] = r < p.rows ? p.w[(size_t)r * p.IH + i % p.IH] : 0.f;
        }
        for (int i = threadIdx.x; i < rpt; i += blockDim.x) nes[i] = r0 + i < p.rows ? p.n_entries[r0 + i] : 0;
    }
    __syncthreads();
    if (live) {
        if (warp == 0 && lane == 0) {
            for (int s = 0; s < 2; ++s) {
                uint8_t* st = smem + s * kScStage;
                mbar_expect_tx(&full[s], kScStage);
                tma_load_2d(st, &map_k, &full[s], s * 64, k0);
                tma_load_2d(st + kScKeys * 128, &map_q, &full[s], s * 64, r0 * p.IH);
            }
        } else if (warp == 1 && lane == 0) {
            constexpr uint32_t idesc = idesc_f16(kScKeys, kScN, 1);
            bool ok = true;
            for (int s = 0; s < 2 && ok; ++s) {
                ok = mbar_wait(&full[s], 0, p.err, 31);
                if (!ok) break;
                tc_fence_after();
                const uint8_t* st = smem + s * kScStage;
                const uint64_t da = smem_desc_sw128(st), db = smem_desc_sw128(st + kScKeys * 128);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (s > 0 || k > 0) ? 1u : 0u);
            }
            if (ok) umma_commit(acc_full);
            else {
                // a load that did not arrive: wait (bounded, no second error code) so that nothing lands after the CTA has gone
                mbar_wait(&full[1], 0, nullptr, 0);
            }
        } else if (warp >= 2) {
            const int q = warp & 3;
            const int n = k0 + q * 32 + lane;                               // this thread's key
            const bool ok = mbar_wait_relaxed(acc_full, 0, p.err, 32);
            tc_fence_after();
            if (ok) {
                const float ks = n < ne_tile ? p.kscale[n] : 0.f;
                float sum = 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < kScN; c0 += 16) {
                    float v[16];
                    tmem_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int col = c0 + j;
                        sum = fmaf(fmaxf(v[j] * ks, 0.f), wsm[col], sum);
                        if ((col + 1) % p.IH == 0) {
                            const int ri = col / p.IH;
                            if (n < nes[ri]) p.scores[(size_t)(r0 + ri) * p.ld_scores + n] = sum;
                            sum = 0.f;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_d, kScN);
    pdl_launch_dependents();
}


// ---- few-row steps over long index rows: FP8 x FP8 straight over the cached keys ------------------------------------------------
// A decode row scores every cached entry of its sequence: 262k entries at a 1M-token context, 88 us per indexer layer on the CUDA
// cores (compute-bound: entries x heads x 128 FMAs).  Here the keys stay E4M3 as they sit in the paged cache - one TMA box per
// cache page lands them in a 128-byte-swizzled [128 keys][128 bytes] tile, no gather, no conversion - the row's IH query heads are
// quantised to E4M3 with one scale per head inside the CTA (written in the same swizzle by hand), and
//   S[key][head] = k_fp8 . q_fp8     (tcgen05.mma kind::f8f6f4, M = 128 keys, N = IH, K = 128 in four instructions)
// lands in tensor memory; the epilogue applies key scale x head scale, ReLU, the head weights and the sum over heads, one thread
// per key.  One CTA per (128 entries, row); tiles above the row's fill exit at once, so a CUDA graph can size the grid for the
// row's capacity.  The query loses mantissa (3 bits) against the bf16 form: the scores move by about a percent, which is the
// precision FP8 indexers run at.
constexpr int kF8MaxIH = 64;
constexpr int kF8Smem = kScKeys * 128 + kF8MaxIH * 128 + 1024 /*align*/ + 64 /*barriers*/ + 2 * kF8MaxIH * 4;

struct ScoreF8Params {
    const bf16* q; const float* w;       // [rows, IH, 128], [rows, IH]
    const uint8_t* cache; const int* block_table; int max_pages; int page; int total_pages;
    const int* row_seq; const int* n_entries;
    float* scores; int ld_scores; int rows; int IH; int npad;
    int* err;
};

__global__ void __launch_bounds__(192) indexer_score_f8_kernel(const __grid_constant__ CUtensorMap map_c, ScoreF8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* ktile = smem;                                   // [128 keys][128 B], 128-byte swizzle (written by TMA)
    uint8_t* qtile = smem + kScKeys * 128;                   // [npad heads][128 B], same swizzle (written below)
    uint64_t* full = reinterpret_cast<uint64_t*>(qtile + kF8MaxIH * 128);
    uint64_t* acc_full = full + 1;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);
    float* qs = reinterpret_cast<float*>(qtile + kF8MaxIH * 128 + 64);      // [IH] head scale
    float* wsm = qs + kF8MaxIH;                                             // [IH] head weight
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.y, k0 = blockIdx.x * kScKeys;
    const uint32_t ncols = p.npad <= 32 ? 32u : 64u;        // tensor-memory allocations are powers of two

    if (threadIdx.x == 0) {
        mbar_init(full, 1); mbar_init(acc_full, 1);
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_c);
    }
    if (warp == 1) tmem_alloc(tmem_holder, ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_holder;
    pdl_wait();
    pdl_launch_dependents();
    const int seq = p.row_seq[r];
    const int ne = seq < 0 ? 0 : p.n_entries[r];
    const bool live = k0 < ne;                               // the whole CTA takes the same branch
    if (live) {
        // the row's heads -> E4M3 with one scale per head, in the operand's swizzle: 16-byte chunk c of row h sits at chunk c ^ (h & 7)
        for (int h = warp; h < p.npad; h += 6) {
            uint32_t packed = 0;
            if (h < p.IH) {
                const bf16* src = p.q + ((size_t)r * p.IH + h) * kScD + lane * 4;
                const uint2 raw = *reinterpret_cast<const uint2*>(src);
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
                float m = fmaxf(fmaxf(fabsf(fa.x), fabsf(fa.y)), fmaxf(fabsf(fb.x), fabsf(fb.y)));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                const float sc = m > 0.f ? m * (1.f / 448.f) : 1.f, inv = 1.f / sc;
                uint16_t lo, hi;
                asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(fa.y * inv), "f"(fa.x * inv));
                asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(fb.y * inv), "f"(fb.x * inv));
                packed = (uint32_t)lo | ((uint32_t)hi << 16);
                if (lane == 0) { qs[h] = sc; wsm[h] = p.w[(size_t)r * p.IH + h]; }
            }
            const int c = lane >> 2;
            *reinterpret_cast<uint32_t*>(qtile + h * 128 + ((c ^ (h & 7)) << 4) + (lane & 3) * 4) = packed;
        }
        fence_proxy_async();                                 // the tensor core reads the tile through the async proxy
    }
    __syncthreads();
    if (live) {
        if (warp == 0 && lane == 0) {
            // one box per cache page: `page` consecutive entries of 144 bytes, their first 128 bytes
            mbar_expect_tx(full, kScKeys * 128);
            const int boxes = kScKeys / p.page;
            for (int j = 0; j < boxes; ++j) {
                const int n = k0 + j * p.page;
                int pg = n < ne ? p.block_table[(size_t)seq * p.max_pages + n / p.page] : 0;        // pages above the fill: any valid page, masked below
                pg = pg < 0 ? 0 : (pg >= p.total_pages ? p.total_pages - 1 : pg);
                tma_load_2d(ktile + j * p.page * 128, &map_c, full, 0, pg * p.page);
            }
        } else if (warp == 1 && lane == 0) {
            const uint32_t idesc = idesc_f8(kScKeys, p.npad);
            if (mbar_wait(full, 0, p.err, 33)) {
                tc_fence_after();
                const uint64_t da = smem_desc_sw128(ktile), db = smem_desc_sw128(qtile);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_f8(tmem_d, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
                umma_commit(acc_full);
            }
        } else if (warp >= 2) {
            const int q = warp & 3;
            const int n = k0 + q * 32 + lane;                                   // this thread's entry
            float ks = 0.f;
            if (n < ne) {
                const int pg = p.block_table[(size_t)seq * p.max_pages + n / p.page];
                ks = *reinterpret_cast<const float*>(p.cache + ((size_t)pg * p.page + n % p.page) * kScEntry + kScD);
            }
            const bool ok = mbar_wait_relaxed(acc_full, 0, p.err, 34);
            tc_fence_after();
            if (ok) {
                float sum = 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < p.npad; c0 += 16) {
                    float v[16];
                    tmem_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < p.IH) sum = fmaf(fmaxf(v[j] * ks * qs[c0 + j], 0.f), wsm[c0 + j], sum);
                }
                if (n < ne) p.scores[(size_t)r * p.ld_scores + n] = sum;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_d, ncols);
    pdl_launch_dependents();
}

}  // namespace lsb
using namespace lsb;

// Scores of a single-sequence chunk (every row of the step belongs to row_seq[0], n_entries non-decreasing).  entries_hint: an upper
// bound of n_entries[rows - 1] known to the host (sizes the grids); kbf: bf16 scratch of kbf_rows x 128 (kbf_rows a multiple of 128, at
// least entries_hint), kscale: fp32 scratch of as many floats; q_idx: [rows, IH, 128] bf16 (16-byte aligned), IH a divisor of 256.
LSB_API int lsb_indexer_score_tc(const void* q_idx, const void* w, int IH, const void* cache, const void* block_table, int max_pages,
                                 int page, const void* row_seq, const void* n_entries, void* scores, int ld_scores, int rows,
                                 int entries_hint, void* kbf, int kbf_rows, void* kscale, void* err, void* stream) {
    if (IH <= 0 || kScN % IH || rows <= 0 || ((uintptr_t)q_idx & 15) || ((uintptr_t)kbf & 127)) return -1;
    if (entries_hint <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int ne_pad = (entries_hint + kScKeys - 1) / kScKeys * kScKeys;
    if (kbf_rows % kScKeys || ne_pad > kbf_rows) return -1;
    launch_pdl((indexer_keys_bf16_kernel), (entries_hint + 15) / 16, 256, 0, st, (const uint8_t*)cache, (const int*)block_table, max_pages, page,
               (const int*)row_seq, (const int*)n_entries, rows, (bf16*)kbf, (float*)kscale);
    CUtensorMap mk, mq;
    int rc = cached_map_2d(&mk, kbf, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)kbf_rows, kScD, kScD, kScKeys, 64);     // one map for the whole scratch
    if (rc) return rc;
    rc = cached_map_2d(&mq, q_idx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)rows * IH, kScD, kScD, kScN, 64);
    if (rc) return rc;
    ScoreTcParams p;
    p.w = (const float*)w; p.kscale = (const float*)kscale; p.n_entries = (const int*)n_entries; p.row_seq = (const int*)row_seq;
    p.scores = (float*)scores; p.ld_scores = ld_scores; p.rows = rows; p.IH = IH; p.err = (int*)err;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(indexer_score_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScSmem); attr = true; }
    const int rpt = kScN / IH;
    launch_pdl((indexer_score_tc_kernel), dim3(ne_pad / kScKeys, (rows + rpt - 1) / rpt), 192, kScSmem, st, mk, mq, p);
    LSB_CHECK_LAUNCH();
}

// Scores of few-row steps (decode rows, each with its own sequence) over long index rows, FP8 x FP8 on the tensor cores (see
// indexer_score_f8_kernel).  cache: [total_pages, page, 144] bytes; page (entries per page) in {8, 16, 32, 64, 128}; IH <= 64;
// q_idx 8-byte aligned.  max_entries sizes the grid (a row's capacity); tiles above a row's fill exit.
LSB_API int lsb_indexer_score_f8(const void* q_idx, const void* w, int IH, const void* cache, int total_pages, const void* block_table,
                                 int max_pages, int page, const void* row_seq, const void* n_entries, void* scores, int ld_scores, int rows,
                                 int max_entries, void* err, void* stream) {
    if (IH <= 0 || IH > kF8MaxIH || rows <= 0 || total_pages <= 0 || ((uintptr_t)q_idx & 7) || ((uintptr_t)cache & 15)) return -1;
    if (page < 8 || page > kScKeys || (page & (page - 1))) return -1;
    if (max_entries <= 0) return 0;
    CUtensorMap mc;
    int rc = cached_map_2d(&mc, cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)total_pages * page, kScD, kScEntry, (uint32_t)page, kScD);
    if (rc) return rc;
    ScoreF8Params p;
    p.q = (const bf16*)q_idx; p.w = (const float*)w; p.cache = (const uint8_t*)cache; p.block_table = (const int*)block_table;
    p.max_pages = max_pages; p.page = page; p.total_pages = total_pages; p.row_seq = (const int*)row_seq; p.n_entries = (const int*)n_entries;
    p.scores = (float*)scores; p.ld_scores = ld_scores; p.rows = rows; p.IH = IH; p.npad = (IH + 15) / 16 * 16; p.err = (int*)err;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(indexer_score_f8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem); attr = true; }
    launch_pdl((indexer_score_f8_kernel), dim3((max_entries + kScKeys - 1) / kScKeys, rows), 192, kF8Smem, (cudaStream_t)stream, mc, p);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_indexer_tc(void* buf) { return lsb_trace_install(buf); }
