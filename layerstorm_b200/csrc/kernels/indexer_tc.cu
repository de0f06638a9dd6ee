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

LSB_API int lsb_trace_set_indexer_tc(void* buf) { return lsb_trace_install(buf); }
