// Tensor-core routed-expert FFN for many tokens (prefill chunks, verify batches, large decode
// batches): a grouped GEMM over expert-sorted token rows with the weight de-quantisation fused
// into the operand pipeline.
//
//   moe_tc_sort     counting sort of (row, slot) pairs by expert + list of [expert, first row, rows]
//                   token tiles of at most BN rows (device-side, no host round trip)
//   moe_tc_gather   xs[pos] = fp16(x[pair / S]) in sorted order (the TMA-loadable "B" operand)
//   moe_tc_ffn      one CTA per (token tile, 128 weight rows):
//        warp 0      TMA producer for the token tile (cp.async.bulk.tensor, 128-byte swizzle)
//        warp 1      tensor-memory owner and tcgen05.mma issuer (kind::f16, fp16 x fp16 -> fp32 in TMEM)
//        warps 2-9   weight converters: stream the expert's NVFP4 / FP8-block / BF16 rows from HBM
//                    exactly once, expand them to fp16 (group / block scale folded in) and store them
//                    straight into the 128-byte-swizzled shared-memory tile the MMA reads; warps 2-5
//                    then run the epilogue (tcgen05.ld -> SwiGLU(+clamp) -> fp16, or -> fp32 rows)
//     gate and up tiles share one token tile and accumulate into two TMEM regions, so SwiGLU is
//     fused and the [tokens, 2F] intermediate never exists.
// Per-tensor NVFP4 scales are applied in the epilogue in fp32.  Every wait is bounded and reports
// through an error word.
// Reference seams replaced: moe_permute + external grouped GEMM + fused SwiGLU + unpermute
// (src/core/expert_device.h:31-52, E/smxx/permute/moe_permute.cu, G/sm120/gemm/grouped).
#include "tc_common.cuh"
#include <cstring>
#include "gemv_core.cuh"
#include "moe_fmt.cuh"
#include "ep_comm.cuh"

namespace lsb {
using namespace tc;

int cached_map_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, int esize, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t br, uint32_t bc);

constexpr int kTBM = 128;   // weight rows per UMMA
constexpr int kTBK = 64;    // fp16 elements per stage row (128 bytes = one swizzle span)

// ------------------------------------------------------------------------------------------ sort
// Single block.  ids[npairs] = expert of pair i (or < 0 / >= E_total: ignored).
__global__ void __launch_bounds__(1024) moe_tc_sort_kernel(const int* __restrict__ ids, int npairs, int E_total, int BN,
                                                           int* __restrict__ sorted_pair, int* __restrict__ tile_expert,
                                                           int* __restrict__ tile_row0, int* __restrict__ tile_n,
                                                           int* __restrict__ counters /* [0]=tiles [1]=sorted pairs */) {
    extern __shared__ int sm[];
    int* cnt = sm;                  // [E_total]
    int* off = sm + E_total;        // [E_total + 1]
    int* tb = off + E_total + 1;    // [E_total + 1]
    pdl_wait();
    pdl_launch_dependents();
    for (int e = threadIdx.x; e < E_total; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E_total) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int e = 0; e < E_total; ++e) { off[e] = o; tb[e] = t; o += cnt[e]; t += (cnt[e] + BN - 1) / BN; }
        off[E_total] = o; tb[E_total] = t;
        counters[0] = t; counters[1] = o;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E_total; e += blockDim.x) {
        const int c = cnt[e];
        for (int j = 0, t = tb[e]; j < c; j += BN, ++t) { tile_expert[t] = e; tile_row0[t] = off[e] + j; tile_n[t] = min(BN, c - j); }
        cnt[e] = 0;                 // reused as the placement cursor
    }
    __syncthreads();
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E_total) sorted_pair[off[e] + atomicAdd(&cnt[e], 1)] = i;
    }
    pdl_launch_dependents();
}

// xs[pos][:] = fp16(x[sorted_pair[pos] / S][:])
__global__ void __launch_bounds__(128) moe_tc_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ sorted_pair,
                                                            const int* __restrict__ counters, __half* __restrict__ xs, int S, int H) {
    pdl_wait();
    pdl_launch_dependents();
    const int pos = blockIdx.x;
    if (pos >= counters[1]) return;
    const bf16* src = x + (size_t)(sorted_pair[pos] / S) * H;
    __half* dst = xs + (size_t)pos * H;
    for (int k = threadIdx.x * 8; k < H; k += blockDim.x * 8) {
        float f[8];
        unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src + k)), f);
        __half2 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<uint4*>(h);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------ converters
// Address of 16-byte chunk `c` (0..7) of row `r` in a [rows x 64 fp16] tile with 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128_chunk(uint32_t tile, int r, int c) {
    return tile + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}
__device__ __forceinline__ void st_shared_16(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return *reinterpret_cast<__half2*>(&r);
}

// Weight conversion works in 16-byte "pieces" of raw weight bytes.  Consecutive converter threads take consecutive
// pieces along a weight row and then the next row, so every 32-byte memory sector a warp touches is consumed
// completely by that one load instruction (a row-per-thread mapping would fetch each sector twice).  A piece
// expands to 8..32 fp16 values = 1..4 sixteen-byte chunks of the swizzled operand tile.
//   Conv<FMT>::PPR   pieces per weight row per 64-element pipeline stage
//   load(raw, w, sf, n, K, k0, c)   fetch piece c of matrix row n at reduction offset k0 (issued early)
//   emit(raw, tile, row, c, k0)     expand and store it into row `row` of the operand tile
template <int FMT> struct Conv;
constexpr float kFp8Unscale = 1.f / 256.f;

// Raw weight bytes travel HBM -> shared memory with cp.async (no registers held while they are in flight, so the ring can be
// deep enough to cover DRAM latency); the thread that issued a piece's copy is the one that later expands it.
__device__ __forceinline__ void cpa16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cpa4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <> struct Conv<2> {                  // NVFP4: 32 bytes per row-stage; 4 group scales in one word
    static constexpr int PPR = 2;
    struct Raw { uint4 v; uint32_t sc; };
    static constexpr int AUX = 4;             // bytes of side data per piece in the raw ring (the scale word)
    static __device__ __forceinline__ void issue(void* a, void* b, const uint8_t* w, const uint8_t* sf, int n, int K, int k0, int c) {
        cpa16(a, w + (size_t)n * (K >> 1) + (k0 >> 1) + 16 * c);
        const int gtiles = ((K >> 4) + 3) >> 2;
        cpa4(b, sf + ((size_t)(n >> 7) * gtiles + (k0 >> 6)) * 512 + (n & 31) * 16 + ((n & 127) >> 5) * 4);
    }
    static __device__ __forceinline__ float side(const uint8_t*, int, int, int) { return 0.f; }
    static __device__ __forceinline__ void fetch(Raw& r, const void* a, const void* b, float) {
        r.v = *reinterpret_cast<const uint4*>(a);
        r.sc = *reinterpret_cast<const uint32_t*>(b);
    }
    static __device__ __forceinline__ void emit(const Raw& r, uint32_t tile, int row, int c, int) {
        const uint32_t wv[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {                 // 8 elements = one 16-byte fp16 chunk
            __half2 h[4];
            fp4x8_to_half2x4(wv[j], h);
            // both halves of s2 = the e4m3 scale of this chunk's 16-group (byte 2c + j/2 of the scale word)
            const __half2 s2 = e4m3x2_to_half2((uint16_t)(((r.sc >> ((2 * c + (j >> 1)) * 8)) & 0xffu) * 0x0101u));
#pragma unroll
            for (int q = 0; q < 4; ++q) h[q] = __hmul2(h[q], s2);
            st_shared_16(sw128_chunk(tile, row, 4 * c + j), *reinterpret_cast<uint4*>(h));
        }
    }
};

template <> struct Conv<1> {                  // FP8 e4m3 with 128x128 block scales: 64 bytes per row-stage
    static constexpr int PPR = 4;
    struct Raw { uint4 v; float sc; };
    static constexpr int AUX = 0;
    static __device__ __forceinline__ void issue(void* a, void*, const uint8_t* w, const uint8_t*, int n, int K, int k0, int c) {
        cpa16(a, w + (size_t)n * K + k0 + 16 * c);
    }
    // one float per 128 x 128 block: read (a cache hit) one stage before it is needed, so no load sits in the conversion
    static __device__ __forceinline__ float side(const uint8_t* sf, int n, int K, int k0) {
        return __ldg(reinterpret_cast<const float*>(sf) + (size_t)(n >> 7) * ((K + 127) >> 7) + (k0 >> 7));
    }
    static __device__ __forceinline__ void fetch(Raw& r, const void* a, const void*, float sd) {
        r.v = *reinterpret_cast<const uint4*>(a);
        r.sc = sd;
    }
    static __device__ __forceinline__ void emit(const Raw& r, uint32_t tile, int row, int c, int) {
        // block scales of small weights sit near the bottom of the fp16 range: carry them times 2^8 (exact)
        // and take the factor out again in the fp32 epilogue (kFp8Unscale)
        const __half2 s2 = __float2half2_rn(r.sc * 256.f);
        const uint32_t wv[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
        for (int j = 0; j < 2; ++j) {                 // 8 bytes -> 8 fp16
            __half2 h[4];
            h[0] = __hmul2(e4m3x2_to_half2((uint16_t)(wv[2 * j] & 0xffffu)), s2);
            h[1] = __hmul2(e4m3x2_to_half2((uint16_t)(wv[2 * j] >> 16)), s2);
            h[2] = __hmul2(e4m3x2_to_half2((uint16_t)(wv[2 * j + 1] & 0xffffu)), s2);
            h[3] = __hmul2(e4m3x2_to_half2((uint16_t)(wv[2 * j + 1] >> 16)), s2);
            st_shared_16(sw128_chunk(tile, row, 2 * c + j), *reinterpret_cast<uint4*>(h));
        }
    }
};

template <> struct Conv<3> {                  // GGUF Q4_K: 32 quant bytes per row-stage = one (low, high) nibble pair of sub-blocks
    static constexpr int PPR = 2;
    struct Raw { uint4 hdr; uint4 q; };
    static constexpr int AUX = 16;            // the super-block header (d, dmin, 12 scale bytes)
    static __device__ __forceinline__ void issue(void* a, void* b, const uint8_t* w, const uint8_t*, int n, int K, int k0, int c) {
        const uint8_t* blk = w + ((size_t)n * (K >> 8) + (k0 >> 8)) * 144;
        cpa16(b, blk);
        cpa16(a, blk + 16 + ((k0 & 255) >> 6) * 32 + 16 * c);
    }
    static __device__ __forceinline__ float side(const uint8_t*, int, int, int) { return 0.f; }
    static __device__ __forceinline__ void fetch(Raw& r, const void* a, const void* b, float) {
        r.q = *reinterpret_cast<const uint4*>(a);
        r.hdr = *reinterpret_cast<const uint4*>(b);
    }
    static __device__ __forceinline__ void emit(const Raw& r, uint32_t tile, int row, int c, int k0) {
        const __half2 dd = *reinterpret_cast<const __half2*>(&r.hdr.x);
        const float d = __low2float(dd), dmin = __high2float(dd);
        uint8_t sc12[12];
        const uint32_t hw[3] = {r.hdr.y, r.hdr.z, r.hdr.w};
#pragma unroll
        for (int i = 0; i < 12; ++i) sc12[i] = (uint8_t)(hw[i >> 2] >> (8 * (i & 3)));
        const uint32_t wv[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
        const int j2 = ((k0 & 255) >> 6) * 2;                      // first sub-block of this stage
#pragma unroll
        for (int half_i = 0; half_i < 2; ++half_i) {               // low nibbles: sub-block j2, high nibbles: j2 + 1
            float sc, mn;
            q4k_scale_min(sc12, j2 + half_i, sc, mn);
            const __half2 a2 = __float2half2_rn(d * sc), b2 = __float2half2_rn(-dmin * mn);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {                       // bytes 8cc..8cc+7 of the piece -> elements 16c + 8cc ..
                __half2 h[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t wq = wv[2 * cc + (q >> 1)] >> ((q & 1) * 16 + half_i * 4);
                    // two consecutive bytes -> two 4-bit values as exact fp16 integers (1024 + v) - 1024
                    const uint32_t bits = 0x64006400u | (wq & 0xFu) | (((wq >> 8) & 0xFu) << 16);
                    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&bits), __float2half2_rn(1024.f));
                    h[q] = __hfma2(v, a2, b2);
                }
                st_shared_16(sw128_chunk(tile, row, half_i * 4 + 2 * c + cc), *reinterpret_cast<uint4*>(h));
            }
        }
    }
};

template <> struct Conv<0> {                  // BF16: 128 bytes per row-stage
    static constexpr int PPR = 8;
    struct Raw { uint4 v; };
    static constexpr int AUX = 0;
    static __device__ __forceinline__ void issue(void* a, void*, const uint8_t* w, const uint8_t*, int n, int K, int k0, int c) {
        cpa16(a, w + ((size_t)n * K + k0 + 8 * c) * 2);
    }
    static __device__ __forceinline__ float side(const uint8_t*, int, int, int) { return 0.f; }
    static __device__ __forceinline__ void fetch(Raw& r, const void* a, const void*, float) {
        r.v = *reinterpret_cast<const uint4*>(a);
    }
    static __device__ __forceinline__ void emit(const Raw& r, uint32_t tile, int row, int c, int) {
        float f[8];
        unpack_bf16x8(r.v, f);
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
        st_shared_16(sw128_chunk(tile, row, c), *reinterpret_cast<uint4*>(h));
    }
};

// ------------------------------------------------------------------------------------------ main kernel
struct MoeTcParams {
    const uint8_t* arena; const int* slot_of; ExpertFmt ef;
    const int* tile_expert; const int* tile_row0; const int* tile_n; const int* counters;
    const int* sorted_pair;
    __half* act;          // gate/up output, [pairs, F] fp16 in sorted order
    float* y;             // down output, [npairs, H] fp32 in pair order
    float limit;
    int* miss_flag; int* err;
    // expert-parallel mode (ep.nranks > 0): the gate/up kernel waits for the peers' token rows (phase 1) before its
    // first load, the down kernel stores its rows straight into the token owners' buffers and publishes phase 2
    EpComm ep;
    // dense-linear mode of the down kernel (one "expert" = the whole matrix): row stride and type of the output and the
    // per-tensor scale (0 = read it from the slot tail)
    int ldo, out_bf16; float down_scale;
};

template <int FMT, int BN, bool GATEUP> struct MoeTcCfg {
    static constexpr int A_TILES = GATEUP ? 2 : 1;
    static constexpr int A_BYTES = A_TILES * kTBM * kTBK * 2;
    static constexpr int B_BYTES = BN * kTBK * 2;
    // Two operand rings with their own barriers: converted weight tiles (SA stages, filled by the converter warps)
    // and token tiles (SB stages, TMA).  The token ring runs further ahead, so a TMA round trip never sits between
    // the MMA freeing a weight stage and the converters refilling it.
    static constexpr int SA = GATEUP ? 2 : 3;
    static constexpr int SB = 4;
    static constexpr int OP_BYTES = SA * A_BYTES + SB * B_BYTES;
    static constexpr int ACC_COLS = A_TILES * BN;                         // one accumulator set (gate [+ up])
    static constexpr int TMEM_COLS = (2 * ACC_COLS) < 32 ? 32 : 2 * ACC_COLS;   // double-buffered: epilogue of tile i overlaps tile i+1
#ifndef LSB_MOE_RELAX
#define LSB_MOE_RELAX 1
#endif
#ifndef LSB_MOE_CONV_WARPS
#define LSB_MOE_CONV_WARPS 8
#endif
    static constexpr int PIECES = (GATEUP ? 2 : 1) * kTBM * Conv<FMT>::PPR;   // 16-byte pieces per stage
    static constexpr int CONV_WARPS = (PIECES / 32) < LSB_MOE_CONV_WARPS ? (PIECES / 32) : LSB_MOE_CONV_WARPS;
    static constexpr int EPI_WARPS = 4;
    static constexpr int THREADS = (2 + CONV_WARPS + EPI_WARPS) * 32;
    static constexpr int CONV_THREADS = CONV_WARPS * 32;
    static constexpr int ROWS = A_TILES * kTBM;                           // weight rows per stage (gate rows, then up rows)
    // raw ring: RD stages of not yet converted weight bytes in flight per CTA (up to ~128 KB)
    static constexpr int NP = ROWS * Conv<FMT>::PPR / CONV_THREADS;       // 16-byte pieces per converter thread per stage
    static constexpr int RAW_STAGE = NP * CONV_THREADS * (16 + Conv<FMT>::AUX);
    static constexpr int RAW_BUDGET = 227 * 1024 - 1024 - 256 - OP_BYTES > 128 * 1024 ? 128 * 1024 : 227 * 1024 - 1024 - 256 - OP_BYTES;
    static constexpr int RD_FIT = RAW_BUDGET / RAW_STAGE;
    static constexpr int RD = RD_FIT > 12 ? 12 : (RD_FIT < 3 ? 3 : RD_FIT);
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM = OP_BYTES + BAR_BYTES + RD * RAW_STAGE + 1024;
    static_assert(SMEM <= 227 * 1024, "shared memory budget");
};

// Work item w -> (token tile t, weight tile j).  Items are grouped by kTileGroup consecutive token tiles (tiles are sorted
// by expert, so a group mostly belongs to one expert); inside a group the token tile runs fastest, so the CTAs that
// are in flight together read the same 128 weight rows and all but the first hit L2.
constexpr int kTileGroup = 8;
__device__ __forceinline__ void work_item(int w, int ntiles, int NT, int& t, int& j) {
    const int per = kTileGroup * NT;
    const int gi = w / per, r = w % per;
    const int t0 = gi * kTileGroup;
    const int gsz = min(kTileGroup, ntiles - t0);
    t = t0 + r % gsz;
    j = r / gsz;
}

// Persistent kernel: one CTA per SM walks the work list (token tile x 128-row weight tile, weight tile fastest so
// that concurrently running CTAs share a token tile); the shared-memory ring, its barrier phases and the two TMEM
// accumulator sets carry over from one work item to the next.
template <int FMT, int BN, bool GATEUP>
__global__ void __launch_bounds__(MoeTcCfg<FMT, BN, GATEUP>::THREADS) moe_tc_ffn_kernel(const __grid_constant__ CUtensorMap map_b, MoeTcParams p) {
    using C = MoeTcCfg<FMT, BN, GATEUP>;
    using CV = Conv<FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;                                   // [SA] converted weight tiles (gate [+ up])
    uint8_t* smem_b = smem + C::SA * C::A_BYTES;              // [SB] token tiles
    uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + C::OP_BYTES);
    uint64_t* empty_a = full_a + C::SA;
    uint64_t* full_b = empty_a + C::SA;
    uint64_t* empty_b = full_b + C::SB;
    uint64_t* acc_full = empty_b + C::SB;        // [2]
    uint64_t* acc_empty = acc_full + 2;          // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = GATEUP ? p.ef.H : p.ef.F;          // reduction length
    const int NOUT = GATEUP ? p.ef.F : p.ef.H;       // weight rows
    const int NT = NOUT / kTBM;
    const int nkb = K / kTBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::SA; ++s) { mbar_init(&full_a[s], C::CONV_WARPS); mbar_init(&empty_a[s], 1); }
        for (int s = 0; s < C::SB; ++s) { mbar_init(&full_b[s], 1); mbar_init(&empty_b[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], C::EPI_WARPS); }
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) tmem_alloc(tmem_holder, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_holder;
    pdl_wait();
    pdl_launch_dependents();
    const bool ep_mode = p.ep.nranks > 0;
    const unsigned ep_epoch = ep_mode ? *p.ep.epoch + 1u : 0u;
    if (ep_mode && GATEUP) {
        ep_wait(p.ep, 1, ep_epoch);                  // peers' rows have landed in this rank's staging buffer
        asm volatile("fence.proxy.async;" ::: "memory");   // ... and are ordered before the TMA (async proxy) reads
    }
    const int ntiles = p.counters[0];
    const int total = ntiles * NT;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer: token tiles ----------------
            uint32_t g = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                work_item(w, ntiles, NT, t, jn);
                const int e = p.tile_expert[t];
                if (p.slot_of[e] < 0) {              // expert not resident on this GPU: every role skips the item
                    if (GATEUP && p.miss_flag && jn == 0) atomicExch(p.miss_flag, e + 1);
                    continue;
                }
                const int row0 = p.tile_row0[t];
                for (int it = 0; it < nkb; ++it, ++g) {
                    const int s = g % C::SB;
                    ok = mbar_wait(&empty_b[s], ((g / C::SB) & 1) ^ 1, p.err, 11);
                    if (!ok) break;
                    mbar_expect_tx(&full_b[s], C::B_BYTES);
                    tma_load_2d(smem_b + s * C::B_BYTES, &map_b, &full_b[s], it * kTBK, row0);
                }
            }
            if (!ok) {
                // loads in flight still write this CTA's shared memory: let them land (bounded, no error code)
                for (uint32_t i = g > (uint32_t)C::SB ? g - C::SB : 0; i < g; ++i) mbar_wait(&full_b[i % C::SB], (i / C::SB) & 1, nullptr, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc = idesc_f16(kTBM, BN, 0);
            uint32_t g = 0, lt = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                work_item(w, ntiles, NT, t, jn);
                if (p.slot_of[p.tile_expert[t]] < 0) continue;
                const uint32_t buf = lt & 1u;
                ok = mbar_wait(&acc_empty[buf], ((lt >> 1) & 1u) ^ 1u, p.err, 15);     // epilogue has drained this accumulator set
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_d + buf * C::ACC_COLS;
                for (int it = 0; it < nkb; ++it, ++g) {
                    const int sa = g % C::SA, sb = g % C::SB;
                    ok = mbar_wait(&full_b[sb], (g / C::SB) & 1, p.err, 12) && mbar_wait(&full_a[sa], (g / C::SA) & 1, p.err, 12);
                    if (!ok) break;
                    tc_fence_after();
                    const uint8_t* a = smem_a + sa * C::A_BYTES;
                    const uint64_t da0 = smem_desc_sw128(a), db = smem_desc_sw128(smem_b + sb * C::B_BYTES);
#pragma unroll
                    for (int k = 0; k < kTBK / 16; ++k) {
                        const uint32_t accum = (it > 0 || k > 0) ? 1u : 0u;
                        umma_f16(acc, da0 + 2 * k, db + 2 * k, idesc, accum);
                        if (GATEUP) umma_f16(acc + BN, smem_desc_sw128(a + kTBM * kTBK * 2) + 2 * k, db + 2 * k, idesc, accum);
                    }
                    umma_commit(&empty_a[sa]);
                    umma_commit(&empty_b[sb]);
                }
                if (ok) umma_commit(&acc_full[buf]);
                ++lt;
            }
        }
    } else if (warp < 2 + C::CONV_WARPS) {
        // ---------------- weight converters ----------------
        const int ct = threadIdx.x - 64;                       // converter thread index
        constexpr int NP = C::NP, RD = C::RD;
        uint8_t* rawA = smem + C::OP_BYTES + C::BAR_BYTES;                                 // [RD][NP][threads] x 16 bytes
        uint8_t* rawB = rawA + (size_t)RD * NP * C::CONV_THREADS * 16;                     // [RD][NP][threads] x AUX bytes
        int prow[NP], pc[NP];                                  // piece -> row inside the stage tile, piece inside the row
#pragma unroll
        for (int i = 0; i < NP; ++i) { const int pid = i * C::CONV_THREADS + ct; prow[i] = pid / CV::PPR; pc[i] = pid % CV::PPR; }
        uint32_t g = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            int t, jn;
            work_item(w, ntiles, NT, t, jn);
            const int slot = p.slot_of[p.tile_expert[t]];
            if (slot < 0) continue;
            const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
            const uint8_t* wp[NP];
            const uint8_t* sfp[NP];
            int wrow[NP];
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                const bool up = GATEUP && prow[i] >= kTBM;
                wp[i] = base + (GATEUP ? (up ? p.ef.off_up : p.ef.off_gate) : p.ef.off_down);
                sfp[i] = base + (GATEUP ? (up ? p.ef.off_su : p.ef.off_sg) : p.ef.off_sd);
                wrow[i] = jn * kTBM + (prow[i] & (kTBM - 1));   // weight row in the expert matrix
            }
            auto issue_stage = [&](int it) {
                const int ring = it % RD;
#pragma unroll
                for (int i = 0; i < NP; ++i) {
                    const size_t idx = (size_t)(ring * NP + i) * C::CONV_THREADS + ct;
                    CV::issue(rawA + idx * 16, rawB + idx * CV::AUX, wp[i], sfp[i], wrow[i], K, it * kTBK, pc[i]);
                }
            };
            float sd[NP];
#pragma unroll
            for (int i = 0; i < NP; ++i) sd[i] = CV::side(sfp[i], wrow[i], K, 0);
            // prologue: RD - 1 stages in flight (one commit group per stage, empty groups keep the count uniform)
#pragma unroll 1
            for (int j = 0; j < RD - 1; ++j) {
                if (j < nkb) issue_stage(j);
                cpa_commit();
            }
#pragma unroll 1
            for (int it = 0; it < nkb && ok; ++it) {
                float sdn[NP];
#pragma unroll
                for (int i = 0; i < NP; ++i) sdn[i] = (it + 1 < nkb) ? CV::side(sfp[i], wrow[i], K, (it + 1) * kTBK) : 0.f;
                cpa_wait<RD - 2>();                            // this thread's pieces of stage `it` have landed
                const int s = g % C::SA;
                // one lane polls the barrier, the warp sleeps at the sync: waiting warps leave the issue slots alone
                int okw = 1;
                if (lane == 0) okw = mbar_wait(&empty_a[s], ((g / C::SA) & 1) ^ 1, p.err, 13) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
                if (ok) {
                    const uint32_t st_base = smem_u32(smem_a + s * C::A_BYTES);
                    const int ring = it % RD;
#pragma unroll
                    for (int i = 0; i < NP; ++i) {
                        const size_t idx = (size_t)(ring * NP + i) * C::CONV_THREADS + ct;
                        typename CV::Raw raw;
                        CV::fetch(raw, rawA + idx * 16, rawB + idx * CV::AUX, sd[i]);
                        const uint32_t tile = st_base + ((GATEUP && prow[i] >= kTBM) ? kTBM * kTBK * 2 : 0);
                        CV::emit(raw, tile, prow[i] & (kTBM - 1), pc[i], it * kTBK);
                    }
                    // refill the ring slot that was consumed one iteration ago
                    if (it + RD - 1 < nkb) issue_stage(it + RD - 1);
                    cpa_commit();
                    fence_proxy_async();                       // generic-proxy stores -> visible to the MMA's async-proxy reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_a[s]);
                    ++g;
#pragma unroll
                    for (int i = 0; i < NP; ++i) sd[i] = sdn[i];
                }
            }
            cpa_wait<0>();                                     // nothing of this item is left in flight
        }
    } else {
        // ---------------- epilogue (4 warps: one TMEM lane quarter each) ----------------
        const int q = warp & 3;
        uint32_t lt = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            int t, jn;
            work_item(w, ntiles, NT, t, jn);
            const int e = p.tile_expert[t];
            const int slot = p.slot_of[e];
            if (slot < 0) continue;
            const int row0 = p.tile_row0[t], ncols = p.tile_n[t];
            const int n = jn * kTBM + q * 32 + lane;
            const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
            const uint32_t buf = lt & 1u;
            int okw = 1;
            if (lane == 0) okw = (LSB_MOE_RELAX ? mbar_wait_relaxed(&acc_full[buf], (lt >> 1) & 1u, p.err, 14) : mbar_wait(&acc_full[buf], (lt >> 1) & 1u, p.err, 14)) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            tc_fence_after();
            if (ok) {
                float sg = 1.f, su = 1.f;
                if (FMT == 2 && (GATEUP || p.down_scale == 0.f)) {
                    const float* tail = reinterpret_cast<const float*>(base + p.ef.off_tail);
                    if (GATEUP) { sg = tail[0]; su = tail[1]; } else sg = tail[2];
                } else if (FMT == 2) {
                    sg = p.down_scale;
                } else if (FMT == 1) {
                    sg = su = kFp8Unscale;
                }
                const uint32_t lane_addr = tmem_d + buf * C::ACC_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (c0 >= ncols) break;
                    float gq[16], uq[16];
                    tmem_ld16(lane_addr + (uint32_t)c0, gq);
                    if (GATEUP) tmem_ld16(lane_addr + (uint32_t)(BN + c0), uq);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c0 + j < ncols && n < NOUT) {
                            if (GATEUP) {
                                float gv = gq[j] * sg, uv = uq[j] * su;
                                if (p.limit > 0.f) { gv = fminf(gv, p.limit); uv = fminf(fmaxf(uv, -p.limit), p.limit); }
                                p.act[(size_t)(row0 + c0 + j) * NOUT + n] = __float2half_rn(siluf_(gv) * uv);
                            } else if (ep_mode) {
                                const int2 ra = p.ep.ret[p.ep.rank][row0 + c0 + j];      // (token owner, pair index there)
                                p.ep.y[ra.x][(size_t)ra.y * NOUT + n] = gq[j] * sg;       // NVLink store into the owner's buffer
                            } else if (p.out_bf16) {
                                reinterpret_cast<bf16*>(p.y)[(size_t)p.sorted_pair[row0 + c0 + j] * p.ldo + n] = __float2bfloat16(gq[j] * sg);
                            } else {
                                p.y[(size_t)p.sorted_pair[row0 + c0 + j] * p.ldo + n] = gq[j] * sg;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);       // the MMA issuer may overwrite this accumulator set
            ++lt;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_d, C::TMEM_COLS);
    if (ep_mode && !GATEUP) ep_signal(p.ep, 2, ep_epoch, gridDim.x);
    pdl_launch_dependents();
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int FMT, int BN, bool GATEUP>
static int launch_moe_tc(const CUtensorMap& mb, const MoeTcParams& p, int nout, int max_tiles, cudaStream_t st) {
    using C = MoeTcCfg<FMT, BN, GATEUP>;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(moe_tc_ffn_kernel<FMT, BN, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM); attr = true; }
    const long long work = (long long)(nout / kTBM) * max_tiles;
    const int grid = (int)(work < sm_count() ? (work > 0 ? work : 1) : sm_count());
    launch_pdl((moe_tc_ffn_kernel<FMT, BN, GATEUP>), grid, C::THREADS, C::SMEM, st, mb, p);
    return (int)cudaGetLastError();
}

template <int BN, bool GATEUP>
static int dispatch_fmt(int fmt, const CUtensorMap& mb, const MoeTcParams& p, int nout, int max_tiles, cudaStream_t st) {
    switch (fmt) {
        case 0: return launch_moe_tc<0, BN, GATEUP>(mb, p, nout, max_tiles, st);
        case 1: return launch_moe_tc<1, BN, GATEUP>(mb, p, nout, max_tiles, st);
        case 2: return launch_moe_tc<2, BN, GATEUP>(mb, p, nout, max_tiles, st);
        case 3: return launch_moe_tc<3, BN, GATEUP>(mb, p, nout, max_tiles, st);
    }
    return -1;
}

}  // namespace lsb
using namespace lsb;

// Tiles of at most `BN` (32, 64 or 128) sorted rows.  tile_* arrays hold npairs / BN + E_total + 1 entries,
// counters 2 ints, sorted_pair npairs ints.
LSB_API int lsb_moe_tc_sort(const void* ids, int npairs, int E_total, int BN, void* sorted_pair, void* tile_expert, void* tile_row0,
                            void* tile_n, void* counters, void* stream) {
    if (E_total > 4000 || (BN != 32 && BN != 64 && BN != 128)) return -1;
    launch_pdl((moe_tc_sort_kernel), 1, 1024, (size_t)(3 * E_total + 2) * 4, (cudaStream_t)stream, (const int*)ids, npairs, E_total, BN,
               (int*)sorted_pair, (int*)tile_expert, (int*)tile_row0, (int*)tile_n, (int*)counters);
    LSB_CHECK_LAUNCH();
}

LSB_API int lsb_moe_tc_gather(const void* x, const void* sorted_pair, const void* counters, void* xs, int npairs, int S, int H, void* stream) {
    if (H % 8) return -1;
    launch_pdl((moe_tc_gather_kernel), npairs, 128, 0, (cudaStream_t)stream, (const bf16*)x, (const int*)sorted_pair, (const int*)counters,
               (__half*)xs, S, H);
    LSB_CHECK_LAUNCH();
}

// gateup != 0: act[pos][f] = SwiGLU(xs[pos] . Wgate[f], xs[pos] . Wup[f]) for every sorted position (fp16, [cap_rows, F]).
// gateup == 0: y[pair][h] = act[pos] . Wdown[h]  (fp32, [npairs, H], rows in pair order).
// `b` is the fp16 token operand ([cap_rows, K], K = H for gate/up and F for down), 16-byte aligned.
LSB_API int lsb_moe_tc_ffn(int gateup, const void* b, int cap_rows, const void* arena, const void* slot_of, const void* fmt_struct,
                           const void* tile_expert, const void* tile_row0, const void* tile_n, const void* counters,
                           const void* sorted_pair, void* out, int BN, int max_tiles, float limit, void* miss_flag, void* err,
                           const void* ep, void* stream) {
    const ExpertFmt* ef = (const ExpertFmt*)fmt_struct;
    const int K = gateup ? ef->H : ef->F, nout = gateup ? ef->F : ef->H;
    if (K % kTBK || nout % kTBM || ((uintptr_t)b & 15)) return -1;
    if (ef->fmt == 1 && (K % 128)) return -1;
    if (ef->fmt == 3 && (K % 256)) return -1;
    CUtensorMap mb;
    int rc = cached_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)cap_rows, (uint64_t)K, (uint64_t)K, (uint32_t)BN, kTBK);
    if (rc) return rc;
    MoeTcParams p;
    p.arena = (const uint8_t*)arena; p.slot_of = (const int*)slot_of; p.ef = *ef;
    p.tile_expert = (const int*)tile_expert; p.tile_row0 = (const int*)tile_row0; p.tile_n = (const int*)tile_n;
    p.counters = (const int*)counters; p.sorted_pair = (const int*)sorted_pair;
    p.act = gateup ? (__half*)out : nullptr; p.y = gateup ? nullptr : (float*)out;
    p.limit = limit; p.miss_flag = (int*)miss_flag; p.err = (int*)err;
    if (ep) p.ep = *(const EpComm*)ep; else { memset(&p.ep, 0, sizeof(p.ep)); }
    p.ldo = nout; p.out_bf16 = 0; p.down_scale = 0.f;
    cudaStream_t st = (cudaStream_t)stream;
    if (gateup) {
        switch (BN) {
            case 32: return dispatch_fmt<32, true>(ef->fmt, mb, p, nout, max_tiles, st);
            case 64: return dispatch_fmt<64, true>(ef->fmt, mb, p, nout, max_tiles, st);
            case 128: return dispatch_fmt<128, true>(ef->fmt, mb, p, nout, max_tiles, st);
        }
    } else {
        switch (BN) {
            case 32: return dispatch_fmt<32, false>(ef->fmt, mb, p, nout, max_tiles, st);
            case 64: return dispatch_fmt<64, false>(ef->fmt, mb, p, nout, max_tiles, st);
            case 128: return dispatch_fmt<128, false>(ef->fmt, mb, p, nout, max_tiles, st);
        }
    }
    return -1;
}

// Dense linear layer with quantised weights on the tensor cores: out[m][n] = alpha * sum_k x16[m][k] * W[n][k].
// x16: fp16 [M, K] contiguous; W in storage format `fmt` (0 bf16, 1 fp8 e4m3 + 128x128 block scales, 2 nvfp4 + group-scale
// atoms) with `scales`; out fp32 or bf16 with row stride ldo.  The caller provides the (constant per M) tile description:
// tile_expert = 0, tile_row0 = t*BN, tile_n, counters = {tiles, M}, ident[m] = m, slot0 = {0}.
LSB_API int lsb_gemm_q_tc(void* out, const void* x16, const void* w, const void* scales, int fmt, int M, int N, int K, int ldo, int out_bf16,
                          float alpha, const void* tile_expert, const void* tile_row0, const void* tile_n, const void* counters,
                          const void* ident, const void* slot0, int BN, int n_tiles, void* err, void* stream) {
    if (K % kTBK || N % kTBM || ((uintptr_t)x16 & 15) || fmt < 0 || fmt > 3) return -1;
    if ((fmt == 1 && (K % 128)) || (fmt == 3 && (K % 256))) return -1;
    CUtensorMap mb;
    int rc = cached_map_2d(&mb, x16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)K, (uint32_t)BN, kTBK);
    if (rc) return rc;
    MoeTcParams p;
    memset(&p, 0, sizeof(p));
    p.arena = (const uint8_t*)w; p.slot_of = (const int*)slot0;
    p.ef.fmt = fmt; p.ef.H = N; p.ef.F = K; p.ef.stride = 0; p.ef.off_down = 0;
    p.ef.off_sd = scales ? (long long)((const uint8_t*)scales - (const uint8_t*)w) : 0;
    p.tile_expert = (const int*)tile_expert; p.tile_row0 = (const int*)tile_row0; p.tile_n = (const int*)tile_n;
    p.counters = (const int*)counters; p.sorted_pair = (const int*)ident;
    p.y = (float*)out; p.err = (int*)err; p.ldo = ldo; p.out_bf16 = out_bf16;
    p.down_scale = fmt == 2 ? alpha : 0.f;
    if (fmt != 2 && alpha != 1.0f) return -1;
    cudaStream_t st = (cudaStream_t)stream;
    switch (BN) {
        case 32: return dispatch_fmt<32, false>(fmt, mb, p, N, n_tiles, st);
        case 64: return dispatch_fmt<64, false>(fmt, mb, p, N, n_tiles, st);
        case 128: return dispatch_fmt<128, false>(fmt, mb, p, N, n_tiles, st);
    }
    return -1;
}
