// Expert-parallel exchange over peer-mapped memory (NVLink / NVSwitch), used by the fused
// dispatch -> grouped GEMM -> combine path.  Expert e lives on rank e % nranks.
//
// One MoE call runs three flag phases, all numbered by the same epoch:
//   phase 0  every rank has stored its per-expert pair counts into every peer's count matrix
//   phase 1  every rank has stored its token rows (fp16) and return addresses into the expert owners'
//            staging buffers
//   phase 2  every expert owner has stored the down-projection rows straight into the token owners'
//            per-pair output buffers
// A phase flag is written with st.release.sys after a system-scope fence by the last block of the
// producing kernel; consumers poll with ld.acquire.sys under a 2 s bound and report through `err`
// instead of hanging.  Buffers are safe to reuse across calls because a rank can only start call
// k+1 after its own combine of call k, which waited for every peer's phase 2 of call k, i.e. for
// every peer to have finished reading the staging buffers of call k.
#pragma once
#include "comm.cuh"

namespace lsb {

struct EpComm {
    int nranks, rank, E;             // E = routed experts in total
    long long cap_rows;              // rows of xs / ret on every rank
    long long max_pairs;             // rows of y on every rank
    int H;
    int* cnt_all[kMaxRanks];         // rank p's count matrix [nranks][E]
    __half* xs[kMaxRanks];           // rank p's token staging [cap_rows][H]
    int2* ret[kMaxRanks];            // rank p's return addresses [cap_rows] = (source rank, pair index)
    float* y[kMaxRanks];             // rank p's per-pair outputs [max_pairs][H]
    unsigned* flags[kMaxRanks];      // rank p's flag words [3][nranks]
    unsigned* epoch;                 // local: calls completed
    unsigned* cta_done;              // local: [3] finished-block counters, one per phase
    int* err;                        // local error word
};

// Whole block: the last block of the grid publishes `epoch` for `phase` to every rank.
__device__ __forceinline__ void ep_signal(const EpComm& c, int phase, unsigned epoch, unsigned total_blocks) {
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

// Whole block: wait until every rank has published `epoch` for `phase`.  false = gave up (err = 200 + 10*phase + rank).
__device__ __forceinline__ bool ep_wait(const EpComm& c, int phase, unsigned epoch) {
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
                    atomicCAS(c.err, 0, 200 + 10 * phase + (int)threadIdx.x);
                    s_ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

}  // namespace lsb
