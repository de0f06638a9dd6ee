// Token-level kernels: embedding gather, argmax, temperature / top-k / top-p sampling with a
// counter-based Philox generator, confidence (top-1 probability + normalised entropy) and
// speculative-verify acceptance.
// Reference behaviour: src/compute/kernels/sm120/sampling/sampling.cu:229-269 (one block per token,
// inline Philox-4x32-10), confidence.cu:88, embedding.cu:28, and the orchestrator's acceptance
// rules (python/orchestrator/orchestrator.py:289-303, 3781-3818).
#include <atomic>
#include "common.cuh"
#include "comm.cuh"

namespace lsb {

__device__ __forceinline__ uint32_t sortable_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// out[r] = table[ids[r]] (bf16 table; rows outside [vocab_lo, vocab_hi) give zeros, which is
// what a vocabulary-sharded table contributes before the cross-rank sum).
__global__ void embedding_kernel(float* __restrict__ out_f32, bf16* __restrict__ out_bf16, const bf16* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab_lo, int vocab_hi) {
    const int r = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int id = ids[r];
    const bool own = id >= vocab_lo && id < vocab_hi;
    const bf16* src = table + (size_t)(own ? id - vocab_lo : 0) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const bf16 v = own ? src[i] : __float2bfloat16(0.f);
        if (out_f32) out_f32[(size_t)r * hidden + i] = __bfloat162float(v);
        if (out_bf16) out_bf16[(size_t)r * hidden + i] = v;
    }
    pdl_launch_dependents();
}

// packed (key, ~index): larger value wins, equal values -> lower index wins
__device__ __forceinline__ unsigned long long pack_vi(float v, int i) {
    return ((unsigned long long)sortable_key(v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
}

__global__ void argmax_partial_kernel(const float* __restrict__ logits, int ld, int V, unsigned long long* __restrict__ part) {
    __shared__ unsigned long long sm[32];
    const int r = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    unsigned long long best = 0ull;
    const float* lg = logits + (size_t)r * ld;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
        const unsigned long long k = pack_vi(lg[i], i);
        best = k > best ? k : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const unsigned long long k = __shfl_xor_sync(0xffffffffu, best, o); best = k > best ? k : best; }
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = sm[w] > best ? sm[w] : best;
        part[(size_t)r * gridDim.x + blockIdx.x] = best;
    }
    pdl_launch_dependents();
}

// Final reduction over the per-block partials.  With `comm` (vocabulary-parallel LM head) the
// local winner - packed with its GLOBAL token id - is stored into every rank's receive slot and
// the winners of all ranks are merged, so only 8 bytes per row cross NVLink instead of the
// logits (the reference all-gathers [B, vocab/tp] fp32 logits: src/daemon/dispatch_forward.cpp:538).
__global__ void argmax_final_kernel(const unsigned long long* __restrict__ part, int nblk, int* __restrict__ out_ids,
                                    float* __restrict__ out_val, int base, PeerComm comm) {
    __shared__ unsigned long long s_best;
    const int r = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    unsigned next_epoch = 0;
    if (comm.nranks) next_epoch = *comm.epoch + 1;
    if (threadIdx.x == 0) {
        unsigned long long best = 0ull;
        for (int i = 0; i < nblk; ++i) { const unsigned long long k = part[(size_t)r * nblk + i]; best = k > best ? k : best; }
        // re-pack with the global index
        const uint32_t idx = 0xffffffffu - (uint32_t)(best & 0xffffffffull) + (uint32_t)base;
        best = (best & 0xffffffff00000000ull) | (unsigned long long)(0xffffffffu - idx);
        s_best = best;
        if (comm.nranks) {
            const size_t off = ((size_t)(next_epoch & 1u) * comm.nranks + comm.rank) * (size_t)comm.cap + (size_t)r * 2;
            for (int p = 0; p < comm.nranks; ++p) *reinterpret_cast<unsigned long long*>(comm.recv[p] + off) = best;
        }
    }
    if (comm.nranks) {
        comm_signal(comm, next_epoch, gridDim.x);
        comm_wait(comm, next_epoch);
    } else {
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        unsigned long long best = s_best;
        if (comm.nranks) {
            best = 0ull;
            for (int p = 0; p < comm.nranks; ++p) {
                const size_t off = ((size_t)(next_epoch & 1u) * comm.nranks + p) * (size_t)comm.cap + (size_t)r * 2;
                const unsigned long long k = __ldcg(reinterpret_cast<const unsigned long long*>(comm.recv[comm.rank] + off));
                best = k > best ? k : best;
            }
        }
        out_ids[r] = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
        if (out_val) {
            const uint32_t key = (uint32_t)(best >> 32);
            const uint32_t bits = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
            out_val[r] = __uint_as_float(bits);
        }
    }
    pdl_launch_dependents();
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t* out) {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// One block per row.  Keeps tokens with logit >= max(k-th largest logit, nucleus threshold),
// then draws from the renormalised kept set with one Philox uniform keyed by (seed, offset[r]).
__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, int ld, int V, float temperature, int top_k,
                                                      float top_p, unsigned long long seed, const long long* __restrict__ offsets,
                                                      int* __restrict__ out_ids) {
    __shared__ float red[33];
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_need;
    __shared__ float s_carry;
    __shared__ int s_found;
    const int r = blockIdx.x, t = threadIdx.x;
    const float* lg = logits + (size_t)r * ld;
    pdl_wait();
    pdl_launch_dependents();
    float mx = -INFINITY;
    for (int i = t; i < V; i += blockDim.x) mx = fmaxf(mx, lg[i]);
    mx = block_max(mx, red);
    const float invT = 1.f / fmaxf(temperature, 1e-6f);
    float thr = -INFINITY;
    if (top_k > 0 && top_k < V) {
        if (t == 0) { s_prefix = 0; s_need = top_k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = t; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = t; i < V; i += blockDim.x) {
                const uint32_t k = sortable_key(lg[i]);
                if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1);
            }
            __syncthreads();
            if (t == 0) {
                int need = s_need, b = 255;
                for (; b > 0; --b) { if (hist[b] >= need) break; need -= hist[b]; }
                s_need = need; s_prefix = prefix | ((uint32_t)b << shift);
            }
            __syncthreads();
        }
        const uint32_t key = s_prefix;
        const uint32_t bits = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
        thr = __uint_as_float(bits);
    }
    // total mass above thr
    float Z = 0.f;
    for (int i = t; i < V; i += blockDim.x) if (lg[i] >= thr) Z += __expf((lg[i] - mx) * invT);
    Z = block_sum(Z, red);
    if (top_p > 0.f && top_p < 1.f) {
        // bisection on the logit threshold: largest theta with mass(theta) >= top_p * Z
        float lo = fmaxf(thr, mx - 80.f / invT), hi = mx;
        for (int it = 0; it < 24; ++it) {
            const float mid = 0.5f * (lo + hi);
            float m = 0.f;
            for (int i = t; i < V; i += blockDim.x) if (lg[i] >= mid && lg[i] >= thr) m += __expf((lg[i] - mx) * invT);
            m = block_sum(m, red);
            if (m >= top_p * Z) lo = mid; else hi = mid;
        }
        thr = fmaxf(thr, lo);
        float z2 = 0.f;
        for (int i = t; i < V; i += blockDim.x) if (lg[i] >= thr) z2 += __expf((lg[i] - mx) * invT);
        Z = block_sum(z2, red);
    }
    uint32_t rnd[4];
    const unsigned long long off = offsets ? (unsigned long long)offsets[r] : (unsigned long long)r;
    philox4x32_10((uint32_t)off, (uint32_t)(off >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), rnd);
    const float u = (float)(rnd[0] >> 8) * (1.0f / 16777216.0f);
    const float target = u * Z;
    if (t == 0) { s_carry = 0.f; s_found = -1; }
    __syncthreads();
    const int lane = t & 31, w = t >> 5;
    int last_kept = -1;
    for (int c0 = 0; c0 < V && s_found < 0; c0 += blockDim.x) {
        const int i = c0 + t;
        float p = 0.f;
        if (i < V && lg[i] >= thr) p = __expf((lg[i] - mx) * invT);
        float v = p;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float n = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += n; }
        __syncthreads();
        if (lane == 31) red[w] = v;
        __syncthreads();
        if (w == 0) {
            float x = red[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const float n = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += n; }
            red[lane] = x;
        }
        __syncthreads();
        const float incl = s_carry + (w ? red[w - 1] : 0.f) + v;
        if (p > 0.f && incl > target && incl - p <= target) atomicMax(&s_found, i);
        if (p > 0.f) last_kept = i;
        const float tot = red[31];
        __syncthreads();
        if (t == 0) s_carry += tot;
        __syncthreads();
    }
    // rounding fallback: the last kept token
    if (s_found < 0) {
        __shared__ int s_last;
        if (t == 0) s_last = -1;
        __syncthreads();
        if (last_kept >= 0) atomicMax(&s_last, last_kept);
        __syncthreads();
        if (t == 0) s_found = s_last < 0 ? 0 : s_last;
        __syncthreads();
    }
    if (t == 0) out_ids[r] = s_found;
    pdl_launch_dependents();
}

__global__ void confidence_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ top1, float* __restrict__ entropy) {
    __shared__ float red[33];
    const int r = blockIdx.x, t = threadIdx.x;
    const float* lg = logits + (size_t)r * ld;
    pdl_wait();
    pdl_launch_dependents();
    float mx = -INFINITY;
    for (int i = t; i < V; i += blockDim.x) mx = fmaxf(mx, lg[i]);
    mx = block_max(mx, red);
    float z = 0.f, s = 0.f;
    for (int i = t; i < V; i += blockDim.x) { const float d = lg[i] - mx, e = __expf(d); z += e; s += e * d; }
    z = block_sum(z, red);
    s = block_sum(s, red);
    if (t == 0) {
        top1[r] = 1.f / z;
        const float H = logf(z) - s / z;   // -sum p log p
        entropy[r] = H / logf((float)V);
    }
    pdl_launch_dependents();
}

// Greedy / equality-coupled acceptance: n_acc = longest prefix with draft[k] == target[k];
// next token = target[n_acc] (the correction or the bonus).  out = {n_acc, next_token}.
__global__ void spec_verify_kernel(const int* __restrict__ draft, const int* __restrict__ target, int gamma, int* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int n = 0;
        while (n < gamma && draft[n] == target[n]) ++n;
        out[0] = n;
        out[1] = target[n];
    }
    pdl_launch_dependents();
}

}  // namespace lsb
using namespace lsb;

LSB_API int lsb_embedding(void* out_f32, void* out_bf16, const void* table, const void* ids, int rows, int hidden,
                          int vocab_lo, int vocab_hi, void* stream) {
    launch_pdl((embedding_kernel), rows, 256, 0, (cudaStream_t)stream, (float*)out_f32, (bf16*)out_bf16, (const bf16*)table, (const int*)ids,
                                                           hidden, vocab_lo, vocab_hi);
    LSB_CHECK_LAUNCH();
}

// part: scratch u64 [rows, 64].  out_val may be null.  `base` is added to the index (vocab shard offset).
LSB_API int lsb_argmax(const void* logits, int ld, int rows, int V, void* part, void* out_ids, void* out_val, int base,
                       const void* comm, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    PeerComm pc;
    pc.nranks = 0;
    if (comm) pc = *reinterpret_cast<const PeerComm*>(comm);
    launch_pdl((argmax_partial_kernel), dim3(64, rows), 256, 0, st, (const float*)logits, ld, V, (unsigned long long*)part);
    launch_pdl((argmax_final_kernel), rows, 32, 0, st, (const unsigned long long*)part, 64, (int*)out_ids, (float*)out_val, base, pc);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_sample(const void* logits, int ld, int rows, int V, float temperature, int top_k, float top_p,
                       unsigned long long seed, const void* offsets, void* out_ids, void* stream) {
    launch_pdl((sample_kernel), rows, 1024, 0, (cudaStream_t)stream, (const float*)logits, ld, V, temperature, top_k, top_p, seed,
                                                         (const long long*)offsets, (int*)out_ids);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_confidence(const void* logits, int ld, int rows, int V, void* top1, void* entropy, void* stream) {
    launch_pdl((confidence_kernel), rows, 1024, 0, (cudaStream_t)stream, (const float*)logits, ld, V, (float*)top1, (float*)entropy);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_spec_verify(const void* draft, const void* target, int gamma, void* out, void* stream) {
    launch_pdl((spec_verify_kernel), 1, 32, 0, (cudaStream_t)stream, (const int*)draft, (const int*)target, gamma, (int*)out);
    LSB_CHECK_LAUNCH();
}

// Process-wide switch for programmatic dependent launch (1 = on, the default).
LSB_API int lsb_set_pdl(int enabled) {
    lsb::pdl_enabled_flag() = enabled ? 1 : 0;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free argmax (declared in csrc/include/lsb_noalloc.h).
//
// Some callers cannot allocate device memory at all: code running while a CUDA memory pool is
// frozen, plug-ins inside a host process that owns every byte of the device heap, and latency
// paths where a cudaMalloc (an implicit device synchronisation) is not acceptable.  For them the
// per-block partial winners live in the fixed file-scope array below instead of a caller buffer.
// The array costs kNoAllocMaxRows * 64 * 8 bytes = 128 KiB on every GPU that loads this library,
// for the lifetime of the process.
constexpr int kNoAllocMaxRows = 256;
static __device__ __align__(256) unsigned long long g_argmax_scratch[kNoAllocMaxRows * 64];

// The array's name is only a host-side handle; the device address is looked up once per device.
// The per-device cache is atomic: first calls for the same device may come from several host threads at once (they all
// store the same value).
static unsigned long long* noalloc_scratch_for_current_device(int* rc) {
    static std::atomic<unsigned long long*> ptrs[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) { *rc = e != cudaSuccess ? (int)e : -3; return nullptr; }
    unsigned long long* p = ptrs[dev].load(std::memory_order_acquire);
    if (!p) {
        void* q = nullptr;
        e = cudaGetSymbolAddress(&q, g_argmax_scratch);
        if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
        p = (unsigned long long*)q;
        ptrs[dev].store(p, std::memory_order_release);
    }
    *rc = 0;
    return p;
}

LSB_API int lsb_argmax_noalloc(const float* logits, int ld, int rows, int V, int* out_ids, float* out_val, int base, void* stream) {
    if (rows <= 0 || V <= 0 || ld < V || !logits || !out_ids) return -1;     // ld < V would read past the end of a row
    if (rows > kNoAllocMaxRows) return -2;          // larger batches must use lsb_argmax with a caller-provided buffer
    int rc = 0;
    unsigned long long* part = noalloc_scratch_for_current_device(&rc);
    if (!part) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    PeerComm pc;
    pc.nranks = 0;
    // every [row][block] partial is rewritten by the first kernel before the second reads it, so
    // nothing left over from an earlier call can leak into this one
    launch_pdl((argmax_partial_kernel), dim3(64, rows), 256, 0, st, logits, ld, V, part);
    launch_pdl((argmax_final_kernel), rows, 32, 0, st, (const unsigned long long*)part, 64, out_ids, out_val, base, pc);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_argmax_noalloc_max_rows() { return kNoAllocMaxRows; }

LSB_API int lsb_trace_set_sampling(void* buf) { return lsb_trace_install(buf); }
