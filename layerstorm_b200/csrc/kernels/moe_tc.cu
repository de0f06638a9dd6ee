// Tensor-core routed-expert FFN for many tokens (prefill chunks, verify batches, large decode
// batches): a grouped GEMM over expert-sorted token rows with the weight de-quantisation fused
// into the operand pipeline.
//
//   moe_tc_sort     counting sort of (row, slot) pairs by expert + list of [expert, first row, rows]
//                   token tiles of at most BN rows (device-side, no host round trip)
//   moe_tc_gather   xs[pos] = fp16(x[pair / S]) in sorted order (the TMA-loadable "B" operand)
//   moe_tc_ffn      persistent, one CTA per SM walking (token tile, 128 weight rows) work items:
//        warp 0      TMA producer for the token tiles (cp.async.bulk.tensor, 128-byte swizzle, 8-stage ring)
//        warp 1      tensor-memory owner and tcgen05.mma issuer (kind::f16, fp16 x fp16 -> fp32 in TMEM,
//                    A = weights read from tensor memory, B = tokens read from shared memory)
//        warps 2-9   weight converters: stream the expert's NVFP4 / FP8-block / Q4_K / BF16 rows from HBM
//                    exactly once into registers, expand them to fp16 (group / block scale folded in) and
//                    write them with tcgen05.st into a ring of operand stages in tensor memory
//        warps 10-13 epilogue (tcgen05.ld -> SwiGLU(+clamp) -> fp16, or -> fp32 / bf16 rows, or NVLink stores)
//     gate and up tiles share one token tile and accumulate into two TMEM regions, so SwiGLU is
//     fused and the [tokens, 2F] intermediate never exists.
// Per-tensor NVFP4 scales are applied in the epilogue in fp32.  Every wait is bounded and reports
// through an error word.
// Reference seams replaced: moe_permute + external grouped GEMM + fused SwiGLU + unpermute
// (src/core/expert_device.h:31-52, E/smxx/permute/moe_permute.cu, G/sm120/gemm/grouped).
#include "tc_common.cuh"
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
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
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return *reinterpret_cast<__half2*>(&r);
}
__device__ __forceinline__ uint32_t h2_bits(const __half2& h) { return *reinterpret_cast<const uint32_t*>(&h); }

// Weight path of the grouped GEMM:  HBM --TMA--> raw ring in shared memory --ld.shared--> registers --convert-->
// tcgen05.st --> operand ring in tensor memory --> tcgen05.mma (A from TMEM).
// A pipeline stage is 64 reduction elements of 128 weight rows per matrix = one TMA box of SBYTES x 128 bytes of the
// [slot][row][byte] view of the arena, written with the swizzle mode of width SBYTES.  One converter thread owns one
// weight row (TMEM lane = row) and 64 / NH consecutive elements of the stage: it reads its 16-byte chunks from the
// swizzled box (conflict free: the 8 lanes of a quarter-warp phase hit 8 different 16-byte bank groups), expands
// them to fp16 pairs with the group / block scale folded in and writes them into its TMEM lane with one tcgen05.st.
// The converted operand never exists in shared memory, which carries only raw bytes (once in, once out) and the
// token tiles; staging fp16 weight tiles there would cost about four times the shared-memory bandwidth.
//   RowConv<FMT, NH>::SBYTES                   raw bytes per row and stage
//   stage_x(it)                                byte offset of stage `it` inside a weight row
//   fetch(raw, tile, r, h)                     read this thread's chunks of row r (part h of NH) from the box at `tile`
//   convert(raw, out, k0, h)                   expand to 32 / NH packed fp16 pairs
constexpr float kFp8Unscale = 1.f / 256.f;
template <int SBYTES> __device__ __forceinline__ uint32_t swz_chunk(uint32_t tile, int r, int c) {
    if (SBYTES == 128) return tile + (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4));
    if (SBYTES == 64) return tile + (uint32_t)(r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
    return tile + (uint32_t)(r * 32 + ((c ^ ((r >> 2) & 1)) << 4));
}
template <int FMT, int NH> struct RowConv;

template <int NH> struct RowConv<2, NH> {     // NVFP4: 32 bytes per row-stage; 4 group scales in one word
    static constexpr int SBYTES = 32, NV = 2 / NH, AUX = 512;              // AUX: the stage's 128 x 4 scale atom
    struct Raw { uint4 v[NV]; uint32_t sc; };
    static __device__ __forceinline__ int pitch(int K) { return K >> 1; }
    static __device__ __forceinline__ int stage_x(int it) { return it * 32; }
    static __device__ __forceinline__ void fetch(Raw& r, uint32_t tile, int row, int h) {
#pragma unroll
        for (int i = 0; i < NV; ++i) r.v[i] = ld_shared_16(swz_chunk<32>(tile, row, h * NV + i));
    }
    static __device__ __forceinline__ void convert(const Raw& r, uint32_t* out, int, int h) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t wv[4] = {r.v[i].x, r.v[i].y, r.v[i].z, r.v[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {             // one word = 8 elements; 16-group index = word / 2
                __half2 hh[4];
                fp4x8_to_half2x4(wv[j], hh);
                const int word = (NH == 1 ? 0 : 4 * h) + 4 * i + j;
                const __half2 s2 = e4m3x2_to_half2((uint16_t)(((r.sc >> ((word >> 1) * 8)) & 0xffu) * 0x0101u));
#pragma unroll
                for (int q = 0; q < 4; ++q) out[(4 * i + j) * 4 + q] = h2_bits(__hmul2(hh[q], s2));
            }
        }
    }
};

template <int NH> struct RowConv<1, NH> {     // FP8 e4m3 with 128 x 128 block scales: 64 bytes per row-stage
    static constexpr int SBYTES = 64, NV = 4 / NH, AUX = 0;
    struct Raw { uint4 v[NV]; float sc; };
    static __device__ __forceinline__ int pitch(int K) { return K; }
    static __device__ __forceinline__ int stage_x(int it) { return it * 64; }
    static __device__ __forceinline__ void fetch(Raw& r, uint32_t tile, int row, int h) {
#pragma unroll
        for (int i = 0; i < NV; ++i) r.v[i] = ld_shared_16(swz_chunk<64>(tile, row, h * NV + i));
    }
    static __device__ __forceinline__ void convert(const Raw& r, uint32_t* out, int, int) {
        // block scales of small weights sit near the bottom of the fp16 range: carry them times 2^8 (exact)
        // and take the factor out again in the fp32 epilogue (kFp8Unscale)
        const __half2 s2 = __float2half2_rn(r.sc * 256.f);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t wv[4] = {r.v[i].x, r.v[i].y, r.v[i].z, r.v[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                out[(4 * i + j) * 2 + 0] = h2_bits(__hmul2(e4m3x2_to_half2((uint16_t)(wv[j] & 0xffffu)), s2));
                out[(4 * i + j) * 2 + 1] = h2_bits(__hmul2(e4m3x2_to_half2((uint16_t)(wv[j] >> 16)), s2));
            }
        }
    }
};

template <int NH> struct RowConv<3, NH> {     // GGUF Q4_K: a stage = 32 quant bytes: low nibbles = sub-block 2s, high nibbles = 2s + 1
    static constexpr int SBYTES = 32, AUX = 0;
    struct Raw { uint4 hdr; uint4 q[2]; };
    static __device__ __forceinline__ int pitch(int K) { return (K >> 8) * 144; }
    static __device__ __forceinline__ int stage_x(int it) { return (it >> 2) * 144 + 16 + (it & 3) * 32; }
    static __device__ __forceinline__ void fetch(Raw& r, uint32_t tile, int row, int) {
        r.q[0] = ld_shared_16(swz_chunk<32>(tile, row, 0));
        r.q[1] = ld_shared_16(swz_chunk<32>(tile, row, 1));
    }
    static __device__ __forceinline__ void convert(const Raw& r, uint32_t* out, int k0, int h) {
        const __half2 dd = *reinterpret_cast<const __half2*>(&r.hdr.x);
        const float d = __low2float(dd), dmin = __high2float(dd);
        uint8_t sc12[12];
        const uint32_t hw[3] = {r.hdr.y, r.hdr.z, r.hdr.w};
#pragma unroll
        for (int i = 0; i < 12; ++i) sc12[i] = (uint8_t)(hw[i >> 2] >> (8 * (i & 3)));
        const uint32_t wv[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
        const int j2 = ((k0 & 255) >> 6) * 2;                      // first sub-block of this stage
#pragma unroll
        for (int hi = 0; hi < 2 / NH; ++hi) {                      // which nibble: elements 32 * nib .. 32 * nib + 31
            const int nib = NH == 1 ? hi : h;
            float sc, mn;
            q4k_scale_min(sc12, j2 + nib, sc, mn);
            const __half2 a2 = __float2half2_rn(d * sc), b2 = __float2half2_rn(-dmin * mn);
#pragma unroll
            for (int pr = 0; pr < 16; ++pr) {                      // byte pair (2 pr, 2 pr + 1) -> two consecutive elements
                const uint32_t wq = wv[pr >> 1] >> ((pr & 1) * 16 + nib * 4);
                // two 4-bit values as exact fp16 integers (1024 + v) - 1024
                const uint32_t bits = 0x64006400u | (wq & 0xFu) | (((wq >> 8) & 0xFu) << 16);
                const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&bits), __float2half2_rn(1024.f));
                out[hi * 16 + pr] = h2_bits(__hfma2(v, a2, b2));
            }
        }
    }
};

template <int NH> struct RowConv<0, NH> {     // BF16: 128 bytes per row-stage
    static constexpr int SBYTES = 128, NV = 8 / NH, AUX = 0;
    struct Raw { uint4 v[NV]; };
    static __device__ __forceinline__ int pitch(int K) { return K * 2; }
    static __device__ __forceinline__ int stage_x(int it) { return it * 128; }
    static __device__ __forceinline__ void fetch(Raw& r, uint32_t tile, int row, int h) {
#pragma unroll
        for (int i = 0; i < NV; ++i) r.v[i] = ld_shared_16(swz_chunk<128>(tile, row, h * NV + i));
    }
    static __device__ __forceinline__ void convert(const Raw& r, uint32_t* out, int, int) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float f[8];
            unpack_bf16x8(r.v[i], f);
#pragma unroll
            for (int q = 0; q < 4; ++q) out[4 * i + q] = h2_bits(__floats2half2_rn(f[2 * q], f[2 * q + 1]));
        }
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
    static constexpr int NH = GATEUP ? 1 : 2;                             // converter threads per (row, stage): gate/up = one per matrix
    using CV = RowConv<FMT, NH>;
    static constexpr int B_BYTES = BN * kTBK * 2;

    static constexpr int ACC_COLS = A_TILES * BN;                         // one accumulator set (gate [+ up])
    // Tensor memory (512 columns): accumulator sets first, then the ring of converted weight stages
    // (32 columns = 64 fp16 per matrix and stage).  Two accumulator sets let the epilogue of one item overlap the
    // main loop of the next; at ACC_COLS = 256 only one fits beside the weight ring.
#ifndef LSB_MOE_NBUF1_COLS
#define LSB_MOE_NBUF1_COLS 128
#endif
    static constexpr int NBUF = ACC_COLS > LSB_MOE_NBUF1_COLS ? 1 : 2;
    static constexpr int A_COLS = 32 * A_TILES;
    static constexpr int A_BASE = NBUF * ACC_COLS;
    static constexpr int SA_FIT = (512 - A_BASE) / A_COLS;
    static constexpr int SA = SA_FIT > 8 ? 8 : SA_FIT;                    // converted weight stages in TMEM
    static constexpr int SB = 4;                                          // token-tile ring (shared memory, TMA)
    static constexpr int TMEM_COLS = 512;
    // 8 converter warps cover one stage (4 lane quarters x 2 parts); CONV_GROUPS such sets take the stages round-robin, so
    // a warp has CONV_GROUPS stage times for its serial wait -> read -> convert -> store -> signal chain.
#ifndef LSB_MOE_CONV_GROUPS
#define LSB_MOE_CONV_GROUPS 1
#endif
    static constexpr int CONV_GROUPS = LSB_MOE_CONV_GROUPS;
    static constexpr int STAGE_WARPS = 8;
    static constexpr int CONV_WARPS = STAGE_WARPS * CONV_GROUPS;
    static constexpr int EPI_WARPS = 4;
    static constexpr int RAW_WARP = 2 + CONV_WARPS + EPI_WARPS;           // last warp: TMA producer of the raw weight ring
    static constexpr int THREADS = (RAW_WARP + 1) * 32;
    // raw weight ring (shared memory): per stage one SBYTES x 128 box per matrix (+ the NVFP4 scale atoms)
    static constexpr int W_TILE = kTBM * CV::SBYTES;
    static constexpr int RAW_STAGE = A_TILES * (W_TILE + CV::AUX);
    static constexpr int BAR_BYTES = 512;
    static constexpr int RAW_BUDGET = 224 * 1024 - SB * B_BYTES - BAR_BYTES - 1024;
    static constexpr int RD_FIT = (RAW_BUDGET > 144 * 1024 ? 144 * 1024 : RAW_BUDGET) / RAW_STAGE;
    static constexpr int RD = RD_FIT > 12 ? 12 : RD_FIT;
    // One CTA per SM by construction (the CTA owns all of tensor memory): ask for more than half of the SM's shared memory.
    static constexpr int SMEM_NEED = SB * B_BYTES + RD * RAW_STAGE + BAR_BYTES + 1024;
    static constexpr int SMEM = SMEM_NEED < 120 * 1024 ? 120 * 1024 : SMEM_NEED;
    static_assert(SA >= 3 && A_BASE + SA * A_COLS <= 512, "tensor memory budget");
    static_assert(RD >= 3 && SMEM <= 227 * 1024, "shared memory budget");
    static_assert((2 * SA + 2 * SB + 2 * RD + 4) * 8 + 8 <= BAR_BYTES, "barrier area");
};
constexpr int kMaxSlots = 1 << 16;
// Role-level time breakdown for tuning builds (-DLSB_MOE_PROFILE): block 0 accumulates the cycles each role spends
// waiting on each barrier and working; lsb_moe_tc_prof_read copies the table out.
#ifdef LSB_MOE_PROFILE
__device__ unsigned long long g_moe_prof[32];
#define PROF_DECL() long long _pacc[4] = {0, 0, 0, 0}; const long long _pt0 = clock64()
#define PROF_SCOPE(j, stmt) do { const long long _t = clock64(); stmt; _pacc[j] += clock64() - _t; } while (0)
#define PROF_FLUSH(j, i) do { if (blockIdx.x == 0) g_moe_prof[i] += (unsigned long long)_pacc[j]; } while (0)
#define PROF_TOTAL(i) do { if (blockIdx.x == 0) g_moe_prof[i] += (unsigned long long)(clock64() - _pt0); } while (0)
#else
#define PROF_DECL()
#define PROF_SCOPE(j, stmt) do { stmt; } while (0)
#define PROF_FLUSH(j, i)
#define PROF_TOTAL(i)
#endif               // slot extent of the weight tensor maps

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

// Persistent kernel: one CTA per SM walks the work list (token tile x 128-row weight tile); the rings, their barrier
// phases and the accumulator sets carry over from one work item to the next, so the producers run ahead across
// item boundaries.
template <int FMT, int BN, bool GATEUP>
__global__ void __launch_bounds__(MoeTcCfg<FMT, BN, GATEUP>::THREADS) moe_tc_ffn_kernel(const __grid_constant__ CUtensorMap map_b,
                                                                                       const __grid_constant__ CUtensorMap map_w0,
                                                                                       const __grid_constant__ CUtensorMap map_w1, MoeTcParams p) {
    using C = MoeTcCfg<FMT, BN, GATEUP>;
    using CV = typename C::CV;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_b = smem;                                   // [SB] token tiles
    uint8_t* smem_r = smem + C::SB * C::B_BYTES;              // [RD] raw weight stages
    uint64_t* full_a = reinterpret_cast<uint64_t*>(smem_r + C::RD * C::RAW_STAGE);
    uint64_t* empty_a = full_a + C::SA;
    uint64_t* full_b = empty_a + C::SA;
    uint64_t* empty_b = full_b + C::SB;
    uint64_t* full_r = empty_b + C::SB;
    uint64_t* empty_r = full_r + C::RD;
    uint64_t* acc_full = empty_r + C::RD;        // [NBUF]
    uint64_t* acc_empty = acc_full + 2;          // [NBUF]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = GATEUP ? p.ef.H : p.ef.F;          // reduction length
    const int NOUT = GATEUP ? p.ef.F : p.ef.H;       // weight rows
    const int NT = NOUT / kTBM;
    const int nkb = K / kTBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::SA; ++s) { mbar_init(&full_a[s], C::STAGE_WARPS); mbar_init(&empty_a[s], 1); }
        for (int s = 0; s < C::SB; ++s) { mbar_init(&full_b[s], 1); mbar_init(&empty_b[s], 1); }
        for (int s = 0; s < C::RD; ++s) { mbar_init(&full_r[s], 1); mbar_init(&empty_r[s], C::STAGE_WARPS); }
        for (int b = 0; b < C::NBUF; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], C::EPI_WARPS); }
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_b);
        tma_prefetch_desc(&map_w0);
        if (GATEUP) tma_prefetch_desc(&map_w1);
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
    // an expert that is not resident on this GPU (or a slot the weight maps do not cover): every role skips the item
    auto slot_ok = [&](int slot) { return slot >= 0 && slot < kMaxSlots; };

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer: token tiles ----------------
            uint32_t g = 0;
            bool ok = true;
            PROF_DECL();
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                work_item(w, ntiles, NT, t, jn);
                const int e = p.tile_expert[t];
                if (!slot_ok(p.slot_of[e])) {
                    if (GATEUP && p.miss_flag && jn == 0) atomicExch(p.miss_flag, e + 1);
                    continue;
                }
                const int row0 = p.tile_row0[t];
                for (int it = 0; it < nkb; ++it, ++g) {
                    const int s = g % C::SB;
                    PROF_SCOPE(0, ok = mbar_wait(&empty_b[s], ((g / C::SB) & 1) ^ 1, p.err, 11));
                    if (!ok) break;
                    mbar_expect_tx(&full_b[s], C::B_BYTES);
                    tma_load_2d(smem_b + s * C::B_BYTES, &map_b, &full_b[s], it * kTBK, row0);
                }
            }
            PROF_FLUSH(0, 1);
            if (!ok) {
                // loads in flight still write this CTA's shared memory: let them land (bounded, no error code)
                for (uint32_t i = g > (uint32_t)C::SB ? g - C::SB : 0; i < g; ++i) mbar_wait(&full_b[i % C::SB], (i / C::SB) & 1, nullptr, 0);
            }
        }
    } else if (warp == C::RAW_WARP) {
        if (lane == 0) {
            // ---------------- TMA producer: raw weight bytes (and NVFP4 scale atoms) ----------------
            uint32_t g = 0;
            bool ok = true;
            PROF_DECL();
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                work_item(w, ntiles, NT, t, jn);
                const int slot = p.slot_of[p.tile_expert[t]];
                if (!slot_ok(slot)) continue;
                const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
                const uint8_t* sf0 = base + (GATEUP ? p.ef.off_sg : p.ef.off_sd);
                const uint8_t* sf1 = base + p.ef.off_su;
                const int gtiles = ((K >> 4) + 3) >> 2;        // NVFP4: 512-byte scale atoms per 128-row tile
                for (int it = 0; it < nkb; ++it, ++g) {
                    const int s = g % C::RD;
                    PROF_SCOPE(0, ok = mbar_wait(&empty_r[s], ((g / C::RD) & 1) ^ 1, p.err, 16));
                    if (!ok) break;
                    uint8_t* dst = smem_r + s * C::RAW_STAGE;
                    mbar_expect_tx(&full_r[s], C::RAW_STAGE);
                    const int x = CV::stage_x(it);
                    tma_load_3d(dst, &map_w0, &full_r[s], x, jn * kTBM, slot);
                    if (GATEUP) tma_load_3d(dst + C::W_TILE, &map_w1, &full_r[s], x, jn * kTBM, slot);
                    if (CV::AUX) {
                        const size_t so = ((size_t)jn * gtiles + it) * 512;
                        bulk_load_1d(dst + C::A_TILES * C::W_TILE, sf0 + so, 512, &full_r[s]);
                        if (GATEUP) bulk_load_1d(dst + C::A_TILES * C::W_TILE + 512, sf1 + so, 512, &full_r[s]);
                    }
                }
            }
            PROF_FLUSH(0, 0);
            if (!ok) {
                for (uint32_t i = g > (uint32_t)C::RD ? g - C::RD : 0; i < g; ++i) mbar_wait(&full_r[i % C::RD], (i / C::RD) & 1, nullptr, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer: A (weights) from tensor memory, B (tokens) from shared memory ----------------
            constexpr uint32_t idesc = idesc_f16(kTBM, BN, 0);
            uint32_t g = 0, lt = 0;
            bool ok = true;
            PROF_DECL();
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                work_item(w, ntiles, NT, t, jn);
                if (!slot_ok(p.slot_of[p.tile_expert[t]])) continue;
                const uint32_t buf = lt % C::NBUF;
                PROF_SCOPE(0, ok = mbar_wait(&acc_empty[buf], ((lt / C::NBUF) & 1u) ^ 1u, p.err, 15));   // epilogue has drained this accumulator set
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_d + buf * C::ACC_COLS;
                for (int it = 0; it < nkb; ++it, ++g) {
                    const int sa = g % C::SA, sb = g % C::SB;
                    PROF_SCOPE(1, ok = mbar_wait(&full_b[sb], (g / C::SB) & 1, p.err, 12));
                    if (ok) PROF_SCOPE(2, ok = mbar_wait(&full_a[sa], (g / C::SA) & 1, p.err, 12));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_t = tmem_d + C::A_BASE + sa * C::A_COLS;
                    const uint64_t db = smem_desc_sw128(smem_b + sb * C::B_BYTES);
                    PROF_SCOPE(3, {
#pragma unroll
                    for (int k = 0; k < kTBK / 16; ++k) {
                        const uint32_t accum = (it > 0 || k > 0) ? 1u : 0u;
                        umma_f16_ts(acc, a_t + 8 * k, db + 2 * k, idesc, accum);
                        if (GATEUP) umma_f16_ts(acc + BN, a_t + 32 + 8 * k, db + 2 * k, idesc, accum);
                    }
                    umma_commit(&empty_a[sa]);
                    umma_commit(&empty_b[sb]); });
                }
                if (ok) umma_commit(&acc_full[buf]);
                ++lt;
            }
            PROF_FLUSH(0, 4); PROF_FLUSH(1, 2); PROF_FLUSH(2, 3); PROF_FLUSH(3, 14); PROF_TOTAL(5);
        }
    } else if (warp < 2 + C::CONV_WARPS) {
        // ---------------- weight converters ----------------
        constexpr int NC = 32 / C::NH;
        const int q = warp & 3;                                // TMEM lane quarter this warp may access
        const int part = ((warp - 2) >> 2) & 1;                // gate/up: matrix (0 gate, 1 up); down: half of the stage's K range
        const int grp = (warp - 2) >> 3;                       // this warp converts the stages with g % CONV_GROUPS == grp
        const int row = q * 32 + lane;                         // row of the 128-row weight tile = TMEM lane
        const int h = GATEUP ? 0 : part;
        const int mat = GATEUP ? part : 0;
        const uint32_t t_lane = tmem_d + C::A_BASE + ((uint32_t)(q * 32) << 16) + (GATEUP ? part * 32 : part * NC);
        uint32_t g = 0;
        bool ok = true;
        PROF_DECL();
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            int t, jn;
            work_item(w, ntiles, NT, t, jn);
            const int slot = p.slot_of[p.tile_expert[t]];
            if (!slot_ok(slot)) continue;
            const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
            const uint8_t* wm = base + (GATEUP ? (part ? p.ef.off_up : p.ef.off_gate) : p.ef.off_down);
            const uint8_t* sf = base + (GATEUP ? (part ? p.ef.off_su : p.ef.off_sg) : p.ef.off_sd);
            const int n = jn * kTBM + row;                     // weight row in the expert matrix
            // side data that does not travel through the ring: the FP8 block scale (one float per 128 x 128 block, the
            // same for the whole tile) and the Q4_K super-block header (16 bytes per row and 256 elements), both read
            // one handled stage ahead of their use
            const float* fsc = reinterpret_cast<const float*>(sf) + (size_t)(n >> 7) * ((K + 127) >> 7);
            const uint8_t* qrow = wm + (size_t)n * CV::pitch(K);
            const int it_first = (int)((grp + C::CONV_GROUPS - g % C::CONV_GROUPS) % C::CONV_GROUPS);   // first stage of this item that is ours
            float sc_next = 0.f;
            uint4 hdr_next = make_uint4(0, 0, 0, 0);
            if (FMT == 1 && it_first < nkb) sc_next = __ldg(fsc + (it_first >> 1));
            if (FMT == 3 && it_first < nkb) hdr_next = __ldg(reinterpret_cast<const uint4*>(qrow + (size_t)(it_first >> 2) * 144));
#pragma unroll 1
            for (int it = 0; it < nkb && ok; ++it) {
                if ((int)(g % C::CONV_GROUPS) != grp) { ++g; continue; }
                typename CV::Raw raw;
                const int itn = it + C::CONV_GROUPS;               // next stage of this item that is ours
                if constexpr (FMT == 1) {
                    raw.sc = sc_next;
                    if (itn < nkb) sc_next = __ldg(fsc + (itn >> 1));
                }
                if constexpr (FMT == 3) {
                    raw.hdr = hdr_next;
                    if (itn < nkb) hdr_next = __ldg(reinterpret_cast<const uint4*>(qrow + (size_t)(itn >> 2) * 144));
                }
                const int rs = g % C::RD, s = g % C::SA;
                // one lane polls the barrier, the warp sleeps at the sync: waiting warps leave the issue slots alone
                int okw = 1;
                if (lane == 0) { if (warp == 2) PROF_SCOPE(0, okw = mbar_wait(&full_r[rs], (g / C::RD) & 1, p.err, 17) ? 1 : 0); else okw = mbar_wait(&full_r[rs], (g / C::RD) & 1, p.err, 17) ? 1 : 0; }
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
                if (!ok) break;
                const uint32_t stage = smem_u32(smem_r + rs * C::RAW_STAGE);
                CV::fetch(raw, stage + mat * C::W_TILE, row, h);
                if constexpr (FMT == 2) {
                    // scale atom of the 128-row tile: word (row % 32) * 4 + row / 32
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(raw.sc) : "r"(stage + C::A_TILES * C::W_TILE + mat * 512 + lane * 16 + q * 4) : "memory");
                }
                uint32_t out[NC];
                CV::convert(raw, out, it * kTBK, h);           // consumes every byte read above
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&empty_r[rs]);                 // the raw stage may be refilled
                    if (warp == 2) PROF_SCOPE(1, okw = mbar_wait(&empty_a[s], ((g / C::SA) & 1) ^ 1, p.err, 13) ? 1 : 0); else okw = mbar_wait(&empty_a[s], ((g / C::SA) & 1) ^ 1, p.err, 13) ? 1 : 0;
                }
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
                if (!ok) break;
                tc_fence_after();                              // the MMAs that read this operand stage have completed
                PROF_SCOPE(3, {
                    if (NC == 32) tmem_st32(t_lane + s * C::A_COLS, out);
                    else tmem_st16(t_lane + s * C::A_COLS, out);
                    tmem_wait_st(); });
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_a[s]);
                ++g;
            }
        }
        if (warp == 2 && lane == 0) { PROF_FLUSH(0, 6); PROF_FLUSH(1, 8); PROF_FLUSH(2, 7); PROF_FLUSH(3, 9); PROF_TOTAL(10); }
    } else {
        // ---------------- epilogue (4 warps: one TMEM lane quarter each) ----------------
        const int q = warp & 3;
        uint32_t lt = 0;
        bool ok = true;
        PROF_DECL();
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            int t, jn;
            work_item(w, ntiles, NT, t, jn);
            const int e = p.tile_expert[t];
            const int slot = p.slot_of[e];
            if (!slot_ok(slot)) continue;
            const int row0 = p.tile_row0[t], ncols = p.tile_n[t];
            const int n = jn * kTBM + q * 32 + lane;
            const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
            const uint32_t buf = lt % C::NBUF;
            int okw = 1;
            if (lane == 0) { if (q == 0) PROF_SCOPE(0, okw = mbar_wait_relaxed(&acc_full[buf], (lt / C::NBUF) & 1u, p.err, 14) ? 1 : 0); else okw = mbar_wait_relaxed(&acc_full[buf], (lt / C::NBUF) & 1u, p.err, 14) ? 1 : 0; }
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
        if (q == 0 && lane == 0) { PROF_FLUSH(0, 11); PROF_TOTAL(13); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_d, C::TMEM_COLS);
    if (ep_mode && !GATEUP) ep_signal(p.ep, 2, ep_epoch, gridDim.x);
    pdl_launch_dependents();
}

int make_map_bytes_3d(CUtensorMap* map, const void* ptr, uint64_t pitch, uint64_t rows, uint64_t slot_stride, uint64_t nslots,
                      uint32_t box_bytes, uint32_t box_rows);
static int cached_map_w(CUtensorMap* out, const void* ptr, uint64_t pitch, uint64_t rows, uint64_t sstride, uint64_t nslots, int sbytes) {
    struct Key {
        const void* p; uint64_t pitch, rows, ss, ns; int sb;
        bool operator<(const Key& o) const { return std::tie(p, pitch, rows, ss, ns, sb) < std::tie(o.p, o.pitch, o.rows, o.ss, o.ns, o.sb); }
    };
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> g(mu);
    const Key k{ptr, pitch, rows, sstride, nslots, sbytes};
    auto it = cache.find(k);
    if (it != cache.end()) { *out = it->second; return 0; }
    CUtensorMap m;
    const int rc = make_map_bytes_3d(&m, ptr, pitch, rows, sstride, nslots, (uint32_t)sbytes, (uint32_t)kTBM);
    if (rc) return rc;
    if (cache.size() > 65536) cache.clear();
    cache[k] = m;
    *out = m;
    return 0;
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
    using CVt = typename MoeTcCfg<FMT, BN, GATEUP>::CV;
    const int Kred = GATEUP ? p.ef.H : p.ef.F;
    CUtensorMap mw0, mw1;
    {
        // byte views of the weight matrices over every slot of the arena (dense mode: one "slot")
        const uint64_t pitch = (uint64_t)(FMT == 0 ? Kred * 2 : FMT == 1 ? Kred : FMT == 2 ? Kred / 2 : Kred / 256 * 144);
        const bool dense = p.ef.stride == 0;
        const uint64_t sstride = dense ? pitch * (uint64_t)nout : (uint64_t)p.ef.stride;
        const uint64_t nslots = dense ? 1 : (uint64_t)kMaxSlots;
        int rc = cached_map_w(&mw0, p.arena + (GATEUP ? p.ef.off_gate : p.ef.off_down), pitch, (uint64_t)nout, sstride, nslots, CVt::SBYTES);
        if (rc) return rc;
        if (GATEUP) { rc = cached_map_w(&mw1, p.arena + p.ef.off_up, pitch, (uint64_t)nout, sstride, nslots, CVt::SBYTES); if (rc) return rc; }
        else mw1 = mw0;
    }
    using C = MoeTcCfg<FMT, BN, GATEUP>;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(moe_tc_ffn_kernel<FMT, BN, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM); attr = true; }
    const long long work = (long long)(nout / kTBM) * max_tiles;
    const int grid = (int)(work < sm_count() ? (work > 0 ? work : 1) : sm_count());
    launch_pdl((moe_tc_ffn_kernel<FMT, BN, GATEUP>), grid, C::THREADS, C::SMEM, st, mb, mw0, mw1, p);
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

// Role-level cycle table of tuning builds (see PROF_SCOPE); -1 in a normal build.
LSB_API int lsb_moe_tc_prof_read(void* out32, int reset, void* stream) {
    (void)stream;
#ifdef LSB_MOE_PROFILE
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out32, g_moe_prof, sizeof(unsigned long long) * 32);
    if (reset) { unsigned long long z[32] = {0}; cudaMemcpyToSymbol(g_moe_prof, z, sizeof(z)); }
    return 0;
#else
    (void)out32; (void)reset;
    return -1;
#endif
}

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

LSB_API int lsb_trace_set_moe_tc(void* buf) { return lsb_trace_install(buf); }
