// Expert-parallel MoE without a collective library: token dispatch and result combine are plain
// loads / stores into peer memory issued from inside the kernels that produce and consume the data.
//
//   ep_count     per-expert pair counts of this rank -> stored into every peer's count matrix (phase 0)
//   ep_layout    waits for all count vectors; every rank derives the same global placement: in the staging
//                buffer of expert-owner o the rows are ordered by expert, then by source rank.  Outputs this
//                rank's write offsets per expert (as a source) and its tile list (as an owner).
//   ep_dispatch  converts each (token, slot) pair's activation row to fp16 and stores it straight into the
//                owner's staging buffer together with its return address (phase 1)
//   [moe_tc_ffn  gate/up + SwiGLU on the owner - waits for phase 1 in its prologue; down projection - its
//                epilogue stores every output row into the token owner's per-pair buffer (phase 2)]
//   ep_combine   waits for phase 2 and sums the top-k slots of every local token in slot order (fp32,
//                deterministic), optionally adding a local (shared-expert) term
// Replaces the reference's NCCL broadcast / all-reduce based expert-parallel exchange
// (src/daemon/moe/moe_ranks.cpp:682-832, call sites C5/C6 and P1/P2) and the NCCL all-to-all baseline.
#include "common.cuh"
#include "ep_comm.cuh"

#include <cstring>

namespace lsb {

__global__ void __launch_bounds__(1024) ep_count_kernel(const int* __restrict__ ids, int npairs, EpComm c) {
    extern __shared__ int cnt[];
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    for (int e = threadIdx.x; e < c.E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < c.E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < c.E * c.nranks; idx += blockDim.x) {
        const int p = idx / c.E, e = idx % c.E;
        c.cnt_all[p][(size_t)c.rank * c.E + e] = cnt[e];
    }
    ep_signal(c, 0, epoch, 1);
}

// dst_off[e]: first row in the owner's staging buffer for this rank's pairs of expert e; cursor[e] zeroed;
// tiles for the experts this rank owns; counters[0] = tiles, counters[1] = rows received.
__global__ void __launch_bounds__(1024) ep_layout_kernel(EpComm c, int BN, int* __restrict__ dst_off, int* __restrict__ cursor,
                                                         int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ tile_n,
                                                         int* __restrict__ counters, int max_tiles) {
    extern __shared__ int sm[];
    int* tot = sm;                  // [E] rows of expert e over all sources
    int* base = sm + c.E;           // [E] first row of expert e in its owner's buffer
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    const bool ok = ep_wait(c, 0, epoch);
    const int* cnt = c.cnt_all[c.rank];
    for (int e = threadIdx.x; e < c.E; e += blockDim.x) {
        int t = 0;
        for (int s = 0; s < c.nranks; ++s) t += cnt[(size_t)s * c.E + e];
        tot[e] = ok ? t : 0;
        cursor[e] = 0;
    }
    __syncthreads();
    if (threadIdx.x < (unsigned)c.nranks) {                  // one thread per owner scans that owner's experts
        int o = 0;
        for (int e = threadIdx.x; e < c.E; e += c.nranks) { base[e] = o; o += tot[e]; }
        if (o > c.cap_rows) atomicCAS(c.err, 0, 260 + (int)threadIdx.x);      // staging buffer of owner `threadIdx.x` too small
    }
    __syncthreads();
    for (int e = threadIdx.x; e < c.E; e += blockDim.x) {
        int before = 0;
        for (int s = 0; s < c.rank; ++s) before += cnt[(size_t)s * c.E + e];
        dst_off[e] = base[e] + before;
    }
    if (threadIdx.x == 0) {
        int t = 0, rows = 0;
        for (int e = c.rank; e < c.E; e += c.nranks) {
            for (int j = 0; j < tot[e] && t < max_tiles; j += BN, ++t) { tile_expert[t] = e; tile_row0[t] = base[e] + j; tile_n[t] = min(BN, tot[e] - j); }
            rows += tot[e];
        }
        const bool fits = rows <= c.cap_rows && *c.err == 0;
        counters[0] = fits ? t : 0;                          // on overflow nothing is computed; the error word says why
        counters[1] = rows;
    }
    pdl_launch_dependents();
}

__global__ void __launch_bounds__(128) ep_dispatch_kernel(const bf16* __restrict__ x, const int* __restrict__ ids, int S,
                                                          const int* __restrict__ dst_off, int* __restrict__ cursor, EpComm c) {
    __shared__ int s_pos;
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    const int i = blockIdx.x;
    const int e = ids[i];
    if (e >= 0 && e < c.E && *c.err == 0) {
        const int o = e % c.nranks;
        if (threadIdx.x == 0) {
            s_pos = dst_off[e] + atomicAdd(&cursor[e], 1);
            c.ret[o][s_pos] = make_int2(c.rank, i);
        }
        __syncthreads();
        const int pos = s_pos;
        const bf16* src = x + (size_t)(i / S) * c.H;
        __half* dst = c.xs[o] + (size_t)pos * c.H;
        for (int k = threadIdx.x * 8; k < c.H; k += blockDim.x * 8) {
            float f[8];
            unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src + k)), f);
            __half2 h[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
            *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<uint4*>(h);       // 16-byte store over NVLink when o != rank
        }
    }
    ep_signal(c, 1, epoch, gridDim.x);
}

// out[r][h] (+)= sum_s wts[r][s] * y[r*S+s][h]; the last block closes the call (epoch += 1).
__global__ void __launch_bounds__(128) ep_combine_kernel(float* __restrict__ out, const float* __restrict__ wts, const int* __restrict__ ids,
                                                         int S, int accumulate, EpComm c) {
    constexpr int kMaxS = 16;
    pdl_wait();
    pdl_launch_dependents();
    const unsigned epoch = *c.epoch + 1u;
    ep_wait(c, 2, epoch);
    const int r = blockIdx.y, H = c.H;
    const int h = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (h < H) {
        const float* y = c.y[c.rank];
        float w[kMaxS];
        bool on[kMaxS];
#pragma unroll
        for (int s = 0; s < kMaxS; ++s) { on[s] = s < S && ids[r * S + s] >= 0 && ids[r * S + s] < c.E; w[s] = s < S ? wts[r * S + s] : 0.f; }
        float4 v[kMaxS];
#pragma unroll
        for (int s = 0; s < kMaxS; ++s)
            v[s] = on[s] ? __ldcg(reinterpret_cast<const float4*>(y + ((size_t)r * S + s) * H + h)) : make_float4(0, 0, 0, 0);   // L2: peers wrote these lines
        float4 a = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int s = 0; s < kMaxS; ++s)
            if (on[s]) { a.x = fmaf(w[s], v[s].x, a.x); a.y = fmaf(w[s], v[s].y, a.y); a.z = fmaf(w[s], v[s].z, a.z); a.w = fmaf(w[s], v[s].w, a.w); }
        float4* o = reinterpret_cast<float4*>(out + (size_t)r * H + h);
        if (accumulate) { const float4 q = *o; a.x += q.x; a.y += q.y; a.z += q.z; a.w += q.w; }
        *o = a;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(c.cta_done + 3, 1u);
        if (prev == gridDim.x * gridDim.y - 1) { c.cta_done[3] = 0; *c.epoch = epoch; }
    }
    pdl_launch_dependents();
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_ep_comm_bytes() { return (int)sizeof(EpComm); }

// ids [npairs] (expert per pair, < 0 = none); x bf16 [rows, H]; dst_off / cursor: int [E]; tile arrays: max_tiles ints.
LSB_API int lsb_ep_dispatch(const void* x, const void* ids, int npairs, int S, int BN, void* dst_off, void* cursor, void* tile_expert,
                            void* tile_row0, void* tile_n, void* counters, int max_tiles, const void* ep, void* stream) {
    EpComm c = *(const EpComm*)ep;
    if (c.nranks < 1 || c.nranks > kMaxRanks || c.E > 8192 || c.H % 8 || (BN != 32 && BN != 64 && BN != 128) || npairs < 1) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    launch_pdl((ep_count_kernel), 1, 1024, (size_t)c.E * 4, st, (const int*)ids, npairs, c);
    launch_pdl((ep_layout_kernel), 1, 1024, (size_t)c.E * 8, st, c, BN, (int*)dst_off, (int*)cursor, (int*)tile_expert, (int*)tile_row0,
               (int*)tile_n, (int*)counters, max_tiles);
    launch_pdl((ep_dispatch_kernel), npairs, 128, 0, st, (const bf16*)x, (const int*)ids, S, (const int*)dst_off, (int*)cursor, c);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_ep_combine(void* out, const void* wts, const void* ids, int rows, int S, int accumulate, const void* ep, void* stream) {
    EpComm c = *(const EpComm*)ep;
    if (c.H % 4 || S > 16 || rows < 1) return -1;
    launch_pdl((ep_combine_kernel), dim3((c.H / 4 + 127) / 128, rows), 128, 0, (cudaStream_t)stream, (float*)out, (const float*)wts,
               (const int*)ids, S, accumulate, c);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_trace_set_ep_moe(void* buf) { return lsb_trace_install(buf); }
