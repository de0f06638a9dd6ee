// In-kernel NVLink collectives over peer-mapped symmetric buffers (no NCCL on these paths).
//
// All-reduce of a [rows, hidden] fp32 partial, split between the kernel that PRODUCES the
// partial and the kernel that CONSUMES the sum:
//   producer epilogue  every block stores its part of the partial into slot[my_rank] of the
//                      receive buffer of EVERY rank (plain st.global to peer memory); the last block to
//                      finish publishes the new epoch to every rank's flag word (st.release.sys).
//   consumer prologue  waits (bounded) until all ranks' flags carry the epoch, then sums the
//                      slots in rank order - identical bits on every rank.
// Receive buffers are double-buffered by epoch parity; a rank can never run two reductions
// ahead of a peer, because producing epoch e+2 requires having consumed e+1, which requires
// every rank to have produced e+1 and therefore consumed e.
//
// This is the B200 replacement for the reference's per-layer NCCL all-reduces after o_proj and
// after the expert / dense FFN down projection (src/daemon/attention/arch_mla.cpp:2055,
// src/daemon/moe/moe_ranks.cpp:682-832; call sites C4-C6 of src/parallelism/dcp_communicator.cpp).
#pragma once
#include "common.cuh"

namespace lsb {

constexpr int kMaxRanks = 8;

struct PeerComm {
    int nranks, rank;
    long long cap;                   // floats per (parity, source-rank) slot
    float* recv[kMaxRanks];          // recv[p] = rank p's receive buffer [2][nranks][cap]
    unsigned* flags[kMaxRanks];      // flags[p] = rank p's flag words [2][nranks]
    unsigned* epoch;                 // local: reductions completed so far
    unsigned* cta_done;              // local: blocks of the current producer that have finished
    int* err;                        // local error word (0 = ok)
    int xchg;                        // few-row step: producers keep their partial local and only count the epoch, the consuming
                                     //    kernel exchanges it - 1: data + one flag per CTA (comm_xchg_*), 2: flag-in-data words
                                     //    (comm_ll_*); 0: producers push
    long long ll_cap;                // elements per (parity, source-rank) slot of the flag-in-data buffers
    unsigned long long* ll[kMaxRanks];   // ll[p] = rank p's flag-in-data receive buffer [2][nranks][ll_cap] of (value, epoch) pairs
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long comm_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Producer side, step 1 (any thread): store one partial value into every rank's slot.
__device__ __forceinline__ void comm_push(const PeerComm& c, unsigned next_epoch, size_t idx, float v) {
    const size_t off = ((size_t)(next_epoch & 1u) * c.nranks + c.rank) * (size_t)c.cap + idx;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
        if (p < c.nranks) c.recv[p][off] = v;
}

// Four consecutive values with one 16-byte store per rank (idx and cap multiples of 4).
__device__ __forceinline__ void comm_push4(const PeerComm& c, unsigned next_epoch, size_t idx, float4 v) {
    const size_t off = ((size_t)(next_epoch & 1u) * c.nranks + c.rank) * (size_t)c.cap + idx;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
        if (p < c.nranks) *reinterpret_cast<float4*>(c.recv[p] + off) = v;
}

// Producer side for few-row partials (whole block, instead of per-element pushes + comm_signal): every block has stored
// its part of the [M, N] partial to LOCAL memory `buf` (row stride ld == the consumer's row stride); the last block to
// arrive copies the whole partial into every rank's slot with 16-byte stores and publishes the epoch.  One
// system-scope fence per collective instead of one per block, and NVLink sees full 128-byte packets instead of
// thousands of 4-byte stores.
__device__ __forceinline__ void comm_finish_local(const PeerComm& c, unsigned next_epoch, unsigned total_blocks, const float* buf, int M, int N,
                                                  int ld) {
    if (c.xchg) {      // consumer-side exchange: the partial stays where it is; one thread of the grid counts the reduction
        if ((blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x) == 0) *c.epoch = next_epoch;
        return;
    }
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();                                   // this block's local stores before its arrival
        s_last = atomicAdd(c.cta_done, 1u) == total_blocks - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();                                       // the other blocks' stores are visible to this block
    const size_t off = ((size_t)(next_epoch & 1u) * c.nranks + c.rank) * (size_t)c.cap;
    if (((N | ld) & 3) == 0 && (c.cap & 3) == 0) {
        const int n4 = N >> 2;
        for (int i = threadIdx.x; i < M * n4; i += blockDim.x) {
            const int m = i / n4, n = (i - m * n4) << 2;
            const float4 v = __ldcg(reinterpret_cast<const float4*>(buf + (size_t)m * ld + n));
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
                if (p < c.nranks) *reinterpret_cast<float4*>(c.recv[p] + off + (size_t)m * ld + n) = v;
        }
    } else {
        for (int i = threadIdx.x; i < M * N; i += blockDim.x) {
            const int m = i / N, n = i - m * N;
            const float v = __ldcg(buf + (size_t)m * ld + n);
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
                if (p < c.nranks) c.recv[p][off + (size_t)m * ld + n] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        *c.cta_done = 0;
        for (int p = 0; p < c.nranks; ++p) st_release_sys(c.flags[p] + (next_epoch & 1u) * c.nranks + c.rank, next_epoch);
        *c.epoch = next_epoch;
    }
}

// Producer side, step 2 (whole block, after its pushes): the last block publishes the epoch.
__device__ __forceinline__ void comm_signal(const PeerComm& c, unsigned next_epoch, unsigned total_blocks) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(c.cta_done, 1u);
        if (prev == total_blocks - 1) {
            *c.cta_done = 0;
            __threadfence_system();
            for (int p = 0; p < c.nranks; ++p) st_release_sys(c.flags[p] + (next_epoch & 1u) * c.nranks + c.rank, next_epoch);
            *c.epoch = next_epoch;
        }
    }
}

// Consumer side (whole block): wait for every rank's contribution to `epoch`.  Gives up after
// ~2 s, records error 100 + missing rank and lets the kernel finish on whatever is there.
__device__ __forceinline__ void comm_wait(const PeerComm& c, unsigned epoch) {
    if (threadIdx.x < (unsigned)c.nranks) {
        const unsigned* f = c.flags[c.rank] + (epoch & 1u) * c.nranks + threadIdx.x;
        if ((int)(ld_acquire_sys(f) - epoch) < 0) {
            const unsigned long long t0 = comm_now_ns();
            unsigned it = 0;
            while ((int)(ld_acquire_sys(f) - epoch) < 0) {
                if ((++it & 1023u) == 0 && comm_now_ns() - t0 > 2000000000ull) { atomicCAS(c.err, 0, 100 + (int)threadIdx.x); break; }
            }
        }
    }
    __syncthreads();
}

// ---- consumer-side exchange (few rows) ---------------------------------------------------------------------------------
// For decode-sized steps the producer's push costs more than the data movement: every block of a weight-streaming kernel
// arrives on one atomic counter and the last one copies the whole partial to every peer.  In this mode the producer keeps
// its partial in LOCAL memory and the kernel that consumes the sum does the exchange itself, slice by slice: each of its
// CTAs stores the slice it is about to use into every peer's slot, publishes ONE flag per CTA, waits for the same CTA of
// every peer and sums in rank order.  No atomics, no serial copy; a CTA only waits for the columns it needs.
// Flag words: flags[p][(parity * nranks + src) * kXchgCtas + cta]  (the first 2 * nranks words are the producer-push flags).
constexpr int kXchgCtas = 128;
__device__ __forceinline__ unsigned* comm_xchg_flag(const PeerComm& c, int peer, unsigned epoch, int src, int cta) {
    return c.flags[peer] + 2 * kMaxRanks + ((epoch & 1u) * c.nranks + src) * kXchgCtas + cta;
}
// Phase 1 (every thread that owns values): store VEC consecutive values of this rank's partial into every peer's slot.
template <int VEC>
__device__ __forceinline__ void comm_xchg_put(const PeerComm& c, unsigned epoch, size_t idx, const float* v) {
    const size_t off = ((size_t)(epoch & 1u) * c.nranks + c.rank) * (size_t)c.cap + idx;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
        if (p < c.nranks && p != c.rank) {
            if (VEC == 4) *reinterpret_cast<float4*>(c.recv[p] + off) = make_float4(v[0], v[1], v[2], v[3]);
            else if (VEC == 2) *reinterpret_cast<float2*>(c.recv[p] + off) = make_float2(v[0], v[VEC > 1 ? 1 : 0]);
            else c.recv[p][off] = v[0];
        }
    }
}
// Phase 2 (whole block): publish this CTA's flag to every peer, then wait (bounded, ~2 s) for the same CTA of every peer.
__device__ __forceinline__ void comm_xchg_sync(const PeerComm& c, unsigned epoch, int cta) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int p = 0; p < c.nranks; ++p)
            if (p != c.rank) st_release_sys(comm_xchg_flag(c, p, epoch, c.rank, cta), epoch);
    }
    if (threadIdx.x < (unsigned)c.nranks && (int)threadIdx.x != c.rank) {
        const unsigned* f = comm_xchg_flag(c, c.rank, epoch, (int)threadIdx.x, cta);
        if ((int)(ld_acquire_sys(f) - epoch) < 0) {
            const unsigned long long t0 = comm_now_ns();
            unsigned it = 0;
            while ((int)(ld_acquire_sys(f) - epoch) < 0) {
                if ((++it & 1023u) == 0 && comm_now_ns() - t0 > 2000000000ull) { atomicCAS(c.err, 0, 100 + (int)threadIdx.x); break; }
            }
        }
    }
    __syncthreads();
}
// Phase 3: the sum over ranks in rank order of element idx; this rank's own value comes from the caller (same bits on every rank).
__device__ __forceinline__ float comm_xchg_get(const PeerComm& c, unsigned epoch, size_t idx, float own) {
    const float* base = c.recv[c.rank] + (size_t)(epoch & 1u) * c.nranks * (size_t)c.cap + idx;
    float v[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) v[p] = (p < c.nranks && p != c.rank) ? __ldcg(base + (size_t)p * c.cap) : 0.f;
    float a = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) a += (p == c.rank) ? own : v[p];
    return a;
}

// ---- flag-in-data exchange (lowest latency) ------------------------------------------------------------------------------
// Every element travels as one 8-byte word (fp32 value, epoch): the store that delivers the value also announces it, so the
// receiver needs no fence, no separate flag and no block-wide barrier - it polls the words it is about to use until they carry
// the current epoch.  8-byte stores arrive whole over NVLink; the epoch never repeats, so a stale word cannot be mistaken.
template <int VEC>
__device__ __forceinline__ void comm_ll_put(const PeerComm& c, unsigned epoch, size_t idx, const float* v) {
    const size_t off = ((size_t)(epoch & 1u) * c.nranks + c.rank) * (size_t)c.ll_cap + idx;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
        if (p < c.nranks && p != c.rank) {
            unsigned long long* d = c.ll[p] + off;
            if (VEC == 2) {
                asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(d), "r"(__float_as_uint(v[0])), "r"(epoch),
                             "r"(__float_as_uint(v[VEC > 1 ? 1 : 0])), "r"(epoch) : "memory");
            } else {
#pragma unroll
                for (int u = 0; u < VEC; ++u)
                    asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(d + u), "r"(__float_as_uint(v[u])), "r"(epoch) : "memory");
            }
        }
    }
}
// VEC consecutive elements: out[u] = sum over ranks in rank order (own[u] at this rank's position).  Polls (bounded, ~2 s).
template <int VEC>
__device__ __forceinline__ void comm_ll_get(const PeerComm& c, unsigned epoch, size_t idx, const float* own, float* out) {
    const unsigned long long* base = c.ll[c.rank] + (size_t)(epoch & 1u) * c.nranks * (size_t)c.ll_cap + idx;
    float v[kMaxRanks][VEC];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
#pragma unroll
        for (int u = 0; u < VEC; ++u) v[p][u] = 0.f;
        if (p < c.nranks && p != c.rank) {
            const unsigned long long* src = base + (size_t)p * c.ll_cap;
            unsigned long long t0 = 0;
            unsigned it = 0;
            while (true) {
                bool ok = true;
                if (VEC == 2) {
                    unsigned a, ea, b, eb;
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(ea), "=r"(b), "=r"(eb) : "l"(src) : "memory");
                    ok = ea == epoch && eb == epoch;
                    v[p][0] = __uint_as_float(a); v[p][VEC > 1 ? 1 : 0] = __uint_as_float(b);
                } else {
#pragma unroll
                    for (int u = 0; u < VEC; ++u) {
                        unsigned a, ea;
                        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(ea) : "l"(src + u) : "memory");
                        ok = ok && ea == epoch;
                        v[p][u] = __uint_as_float(a);
                    }
                }
                if (ok) break;
                if ((++it & 255u) == 0) {
                    const unsigned long long now = comm_now_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > 2000000000ull) { atomicCAS(c.err, 0, 100 + p); break; }
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
        float a = 0.f;
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p) a += (p == c.rank) ? own[u] : v[p][u];
        out[u] = a;
    }
}

// Sum of the ranks' slots for element idx, in rank order.
__device__ __forceinline__ float comm_reduce(const PeerComm& c, unsigned epoch, size_t idx) {
    const float* base = c.recv[c.rank] + (size_t)(epoch & 1u) * c.nranks * (size_t)c.cap + idx;
    float v[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) v[p] = p < c.nranks ? __ldcg(base + (size_t)p * c.cap) : 0.f;   // L2 read: peers wrote these lines
    float a = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) a += v[p];
    return a;
}

}  // namespace lsb
