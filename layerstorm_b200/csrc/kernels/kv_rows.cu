// Row-granular movement of latent KV rows for KV tiering of an active sequence.
//
// A sequence whose older pages live in pinned host memory ("cold") still attends to single rows of them: the sparse-attention
// indexer selects at most top-k positions per query row.  Per attention layer the engine materialises exactly those rows in a
// dense per-query buffer and runs the ordinary attention kernel over it:
//   kv_row_gather   copies the selected rows that are still in HBM pages (block-table entry >= 0) into the buffer,
//   kv_row_scatter  places the rows that came from the cold tier (staged host -> device in one pinned copy) at their slots.
// The bytes are moved verbatim (whatever the cache format), so attention over the materialised buffer sees the same rows as
// attention over the untiered cache: tiered and untiered decoding agree bit for bit.
// Reference kernels: src/compute/kernels/smxx/kv/kv_row_copy.cu:35,50; manager: src/daemon/kv_tiering_manager.h:66-127.
#include "common.cuh"

namespace lsb {

// grid (ceil(sel_ld / 8), rows), 256 threads: a warp moves one row, 16 bytes per lane and pass
__global__ void __launch_bounds__(256) kv_row_gather_kernel(const uint8_t* __restrict__ cache, const int* __restrict__ block_table, int max_pages,
                                                            const int* __restrict__ row_seq, const int* __restrict__ sel_idx,
                                                            const int* __restrict__ sel_cnt, int sel_ld, uint8_t* __restrict__ out, int out_rows,
                                                            int page, int row_bytes) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y, j = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (j >= sel_cnt[r] || j >= out_rows) return;
    const int seq = row_seq[r], pos = sel_idx[(size_t)r * sel_ld + j];
    if (seq < 0 || pos < 0) return;
    const int pg = block_table[(size_t)seq * max_pages + pos / page];
    if (pg < 0) return;                                  // cold page: the row arrives through kv_row_scatter
    const uint4* src = reinterpret_cast<const uint4*>(cache + ((size_t)pg * page + pos % page) * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)r * out_rows + j) * row_bytes);
    for (int i = lane; i < row_bytes / 16; i += 32) dst[i] = src[i];
}

// staging: n rows of row_bytes; dst_row[i]: row index inside `out` (r * out_rows + j)
__global__ void __launch_bounds__(256) kv_row_scatter_kernel(const uint8_t* __restrict__ staging, const int* __restrict__ dst_row, int n,
                                                             uint8_t* __restrict__ out, int row_bytes) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n) return;
    const uint4* src = reinterpret_cast<const uint4*>(staging + (size_t)i * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)dst_row[i] * row_bytes);
    for (int k = lane; k < row_bytes / 16; k += 32) dst[k] = src[k];
}

// Identity selection / page table of the materialised buffer: sel_m[r][j] = j, bt_m[r][p] = r * pages_per_row + p, seq_m[r] = r.
__global__ void kv_rows_identity_kernel(int* __restrict__ sel_m, int sel_ld, int* __restrict__ bt_m, int pages_per_row, int* __restrict__ seq_m,
                                        int rows) {
    const int r = blockIdx.x;
    for (int j = threadIdx.x; j < sel_ld; j += blockDim.x) sel_m[(size_t)r * sel_ld + j] = j;
    for (int p = threadIdx.x; p < pages_per_row; p += blockDim.x) bt_m[(size_t)r * pages_per_row + p] = r * pages_per_row + p;
    if (threadIdx.x == 0) seq_m[r] = r;
}

}  // namespace lsb
using namespace lsb;

// out: [rows, out_rows, row_bytes] bytes; row_bytes a multiple of 16, all buffers 16-byte aligned.
LSB_API int lsb_kv_row_gather(const void* cache, const void* block_table, int max_pages, const void* row_seq, const void* sel_idx,
                              const void* sel_cnt, int sel_ld, void* out, int out_rows, int rows, int page, int row_bytes, void* stream) {
    if (row_bytes % 16 || (((uintptr_t)cache | (uintptr_t)out) & 15) || rows <= 0) return -1;
    launch_pdl((kv_row_gather_kernel), dim3((sel_ld + 7) / 8, rows), 256, 0, (cudaStream_t)stream, (const uint8_t*)cache, (const int*)block_table,
               max_pages, (const int*)row_seq, (const int*)sel_idx, (const int*)sel_cnt, sel_ld, (uint8_t*)out, out_rows, page, row_bytes);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_kv_row_scatter(const void* staging, const void* dst_row, int n, void* out, int row_bytes, void* stream) {
    if (row_bytes % 16 || (((uintptr_t)staging | (uintptr_t)out) & 15)) return -1;
    if (n <= 0) return 0;
    launch_pdl((kv_row_scatter_kernel), (n + 7) / 8, 256, 0, (cudaStream_t)stream, (const uint8_t*)staging, (const int*)dst_row, n, (uint8_t*)out,
               row_bytes);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_kv_rows_identity(void* sel_m, int sel_ld, void* bt_m, int pages_per_row, void* seq_m, int rows, void* stream) {
    kv_rows_identity_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>((int*)sel_m, sel_ld, (int*)bt_m, pages_per_row, (int*)seq_m, rows);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_kv_rows(void* buf) { return lsb_trace_install(buf); }
