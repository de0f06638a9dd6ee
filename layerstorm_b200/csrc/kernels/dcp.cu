// Context-parallel ("DCP", sharded KV) absorbed-MLA attention over peer-mapped memory.
//
// The latent KV cache of a sequence is sharded by token position over the ranks (round-robin in chunks of
// `chunk` tokens); every rank keeps only its own tokens, compacted, in its local paged cache.  The query heads
// stay tensor-parallel (rank r owns heads [r * Hh, (r + 1) * Hh)).  One attention call:
//
//   dcp_gather_q     every rank stores its absorbed query heads into EVERY rank's q_all buffer (P2P stores),
//                    flag phase 0                                                     [all-gather in the head dim]
//   dcp_localize     (sparse layers) the indexer's selected global positions -> the owned ones as local indices
//   mla_decode       the ordinary split-KV attention kernels over the LOCAL cache shard for ALL heads; they leave
//                    un-normalised partials (o, m, l) per (row, head, split)            [lsb_mla_decode, out = null]
//   dcp_scatter      every rank stores the partials of head h straight into the buffer of the rank that owns h,
//                    flag phase 1                                                   [reduce-scatter by P2P stores]
//   dcp_combine      the head owner merges the nranks x NS partials of its heads by their log-sum-exp weights
//
// No collective library call; every wait is bounded (2 s) and reports through an error word.  Buffers are reused
// across calls: a rank starts call k + 1 only after its own combine of call k, which waited for every peer's phase 1
// of call k, i.e. for every peer to have finished reading q_all of call k.
// Reference behaviour replaced: all-gather Q + all-gather LSE + lse-correct + all-reduce of [B, H, D_c] + slice
// (src/daemon/attention/arch_mla.cpp:2555-2574, src/parallelism/dcp_communicator.cpp C1-C3).
#include "comm.cuh"

namespace lsb {

struct DcpComm {
    int nranks, rank, H, Hh;         // heads in total / per rank
    int D, dl, NS, max_rows;         // q row width (dl + dr), latent width, splits per rank, rows per call
    bf16* q_all[kMaxRanks];          // rank p's gathered queries [max_rows][H][D]
    float* part[kMaxRanks];          // rank p's incoming partials [nranks][max_rows][Hh][NS][dl + 4]  (o, m, l, pad: rows stay 16-byte aligned)
    unsigned* flags[kMaxRanks];      // rank p's flag words [2][nranks]
    unsigned* epoch;                 // local: calls completed
    unsigned* cta_done;              // local: [2] finished-block counters
    int* err;
};

__device__ __forceinline__ void dcp_signal(const DcpComm& c, int phase, unsigned epoch, unsigned total_blocks) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(c.cta_done + phase, 1u);
        if (prev == total_blocks - 1) {
            c.cta_done[phase] = 0;
            __threadfence_system();
            for (int p = 0; p < c.nranks; ++p) st_release_sys(c.flags[p] + phase * c.nranks + c.rank, epoch);
        }
    }
}

// Whole block; false = gave up (err = 300 + 10 * phase + missing rank).
__device__ __forceinline__ bool dcp_wait(const DcpComm& c, int phase, unsigned epoch) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < (unsigned)c.nranks) {
        const unsigned* f = c.flags[c.rank] + phase * c.nranks + threadIdx.x;
        if ((int)(ld_acquire_sys(f) - epoch) < 0) {
            const unsigned long long t0 = comm_now_ns();
            unsigned it = 0;
            while ((int)(ld_acquire_sys(f) - epoch) < 0) {
                if ((++it & 1023u) == 0 && comm_now_ns() - t0 > 2000000000ull) {
                    atomicCAS(c.err, 0, 300 + 10 * phase + (int)threadIdx.x);
                    s_ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// q_local: bf16 [R][Hh][D].  grid = R, 256 threads.
__global__ void __launch_bounds__(256) dcp_gather_q_kernel(const bf16* __restrict__ q_local, int R, DcpComm c) {
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    const int r = blockIdx.x;
    const int n16 = c.Hh * c.D / 8;                               // 16-byte pieces of this rank's heads of one row
    const uint4* src = reinterpret_cast<const uint4*>(q_local + (size_t)r * c.Hh * c.D);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) {
        const uint4 v = src[i];
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
            if (p < c.nranks) reinterpret_cast<uint4*>(c.q_all[p] + ((size_t)r * c.H + (size_t)c.rank * c.Hh) * c.D)[i] = v;
    }
    dcp_signal(c, 0, epoch, gridDim.x);
}

// One block: wait for a phase (used in front of kernels that have no wait prologue of their own).
__global__ void __launch_bounds__(32) dcp_wait_kernel(int phase, DcpComm c) {
    pdl_wait();
    pdl_launch_dependents();
    dcp_wait(c, phase, *c.epoch + 1u);
}

// Global selected positions -> owned positions as local cache indices.  Token position t belongs to rank
// (t / chunk) % nranks and sits at local index (t / (chunk * nranks)) * chunk + t % chunk.  Order is preserved.
// grid = R, one warp.
__global__ void __launch_bounds__(32) dcp_localize_kernel(const int* __restrict__ sel_idx, const int* __restrict__ sel_cnt, int sel_ld,
                                                          int* __restrict__ loc_idx, int* __restrict__ loc_cnt, int chunk, int nranks, int rank) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x, lane = threadIdx.x;
    const int n = sel_cnt[r];
    int base = 0;
    for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        const int t = i < n ? sel_idx[(size_t)r * sel_ld + i] : -1;
        const bool mine = t >= 0 && (t / chunk) % nranks == rank;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) loc_idx[(size_t)r * sel_ld + base + __popc(m & ((1u << lane) - 1u))] = (t / (chunk * nranks)) * chunk + t % chunk;
        base += __popc(m);
    }
    if (lane == 0) loc_cnt[r] = base;
}

// Per step row: where this rank stores the new token (index inside its shard, -1 = not its token) and how many of the
// visible positions [0, len) it owns.
__global__ void dcp_rows_kernel(const int* __restrict__ row_pos, const int* __restrict__ row_len, int* __restrict__ row_store,
                                int* __restrict__ row_len_local, int R, int chunk, int nranks, int rank) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int pos = row_pos[r], len = row_len[r];
    row_store[r] = (pos >= 0 && (pos / chunk) % nranks == rank) ? (pos / (chunk * nranks)) * chunk + pos % chunk : -1;
    const int span = chunk * nranks, full = len / span, rem = len - full * span;
    row_len_local[r] = full * chunk + min(max(rem - rank * chunk, 0), chunk);
}

// o_part: fp32 [R][H][NS][dl], ml_part: fp32 [R][H][NS][2] (local partials of all heads).  grid = (R, H), 128 threads.
__global__ void __launch_bounds__(128) dcp_scatter_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, int R, DcpComm c) {
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    const int r = blockIdx.x, h = blockIdx.y;
    const int owner = h / c.Hh, hl = h - owner * c.Hh;
    const int W = c.dl + 4;
    float* dst = c.part[owner] + ((((size_t)c.rank * c.max_rows + r) * c.Hh + hl) * c.NS) * W;
    for (int s = 0; s < c.NS; ++s) {
        const float* o = o_part + (((size_t)r * c.H + h) * c.NS + s) * c.dl;
        for (int d = threadIdx.x * 4; d < c.dl; d += blockDim.x * 4)
            *reinterpret_cast<float4*>(dst + (size_t)s * W + d) = *reinterpret_cast<const float4*>(o + d);
        if (threadIdx.x < 2) dst[(size_t)s * W + c.dl + threadIdx.x] = ml_part[(((size_t)r * c.H + h) * c.NS + s) * 2 + threadIdx.x];
    }
    dcp_signal(c, 1, epoch, gridDim.x * gridDim.y);
}

// out: bf16 [R][Hh][dl]; lse (optional): fp32 [R][Hh].  grid = (R, Hh), 128 threads.  The last block closes the call.
__global__ void __launch_bounds__(128) dcp_combine_kernel(bf16* __restrict__ out, float* __restrict__ lse, int R, DcpComm c) {
    __shared__ float w[kMaxRanks * 32];
    __shared__ float s_inv, s_lse;
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    const bool ok = dcp_wait(c, 1, epoch);
    const int r = blockIdx.x, hl = blockIdx.y, t = threadIdx.x;
    const int W = c.dl + 4, NP = c.nranks * c.NS;
    auto slot = [&](int i) {                                      // partial i = (source rank, split)
        const int src = i / c.NS, s = i - src * c.NS;
        return c.part[c.rank] + ((((size_t)src * c.max_rows + r) * c.Hh + hl) * c.NS + s) * W;
    };
    if (ok) {
        if (t < 32) {
            // NP <= 256: each lane handles partials t, t + 32, ...
            float mx = -INFINITY;
            for (int i = t; i < NP; i += 32) mx = fmaxf(mx, __ldcg(slot(i) + c.dl));
            mx = warp_max(mx);
            float L = 0.f;
            for (int i = t; i < NP; i += 32) {
                const float m = __ldcg(slot(i) + c.dl), l = __ldcg(slot(i) + c.dl + 1);
                const float e = (m > -INFINITY) ? __expf(m - mx) : 0.f;
                w[i] = e;
                L += e * l;
            }
            L = warp_sum(L);
            if (t == 0) { s_inv = L > 0.f ? 1.f / L : 0.f; s_lse = L > 0.f ? mx + __logf(L) : -INFINITY; }
        }
        __syncthreads();
        for (int d = t; d < c.dl; d += blockDim.x) {
            float a = 0.f;
            for (int i = 0; i < NP; ++i) a = fmaf(w[i], __ldcg(slot(i) + d), a);       // rank-major, split-minor: a fixed order on every rank
            out[((size_t)r * c.Hh + hl) * c.dl + d] = __float2bfloat16(a * s_inv);
        }
        if (lse && t == 0) lse[(size_t)r * c.Hh + hl] = s_lse;
    }
    __syncthreads();
    if (t == 0) {
        __threadfence();
        if (atomicAdd(c.cta_done + 1, 1u) == gridDim.x * gridDim.y - 1) {             // counter 1 is idle between scatter and the next call
            c.cta_done[1] = 0;
            *c.epoch = epoch;
        }
    }
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_dcp_comm_bytes() { return (int)sizeof(DcpComm); }

LSB_API int lsb_dcp_gather_q(const void* q_local, int R, const void* comm, void* stream) {
    const DcpComm c = *reinterpret_cast<const DcpComm*>(comm);
    if (R > c.max_rows || (c.Hh * c.D) % 8) return -1;
    launch_pdl((dcp_gather_q_kernel), R, 256, 0, (cudaStream_t)stream, (const bf16*)q_local, R, c);
    launch_pdl((dcp_wait_kernel), 1, 32, 0, (cudaStream_t)stream, 0, c);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_dcp_localize(const void* sel_idx, const void* sel_cnt, int sel_ld, void* loc_idx, void* loc_cnt, int R, int chunk,
                             int nranks, int rank, void* stream) {
    if (chunk <= 0 || nranks <= 0) return -1;
    launch_pdl((dcp_localize_kernel), R, 32, 0, (cudaStream_t)stream, (const int*)sel_idx, (const int*)sel_cnt, sel_ld, (int*)loc_idx, (int*)loc_cnt,
               chunk, nranks, rank);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_dcp_rows(const void* row_pos, const void* row_len, void* row_store, void* row_len_local, int R, int chunk, int nranks,
                         int rank, void* stream) {
    if (chunk <= 0 || nranks <= 0) return -1;
    launch_pdl((dcp_rows_kernel), (R + 127) / 128, 128, 0, (cudaStream_t)stream, (const int*)row_pos, (const int*)row_len, (int*)row_store,
               (int*)row_len_local, R, chunk, nranks, rank);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_dcp_scatter_combine(const void* o_part, const void* ml_part, void* out, void* lse, int R, const void* comm, void* stream) {
    const DcpComm c = *reinterpret_cast<const DcpComm*>(comm);
    if (R > c.max_rows || c.dl % 4 || c.nranks * c.NS > kMaxRanks * 32) return -1;
    launch_pdl((dcp_scatter_kernel), dim3(R, c.H), 128, 0, (cudaStream_t)stream, (const float*)o_part, (const float*)ml_part, R, c);
    launch_pdl((dcp_combine_kernel), dim3(R, c.Hh), 128, 0, (cudaStream_t)stream, (bf16*)out, (float*)lse, R, c);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_dcp(void* buf) { return lsb_trace_install(buf); }
