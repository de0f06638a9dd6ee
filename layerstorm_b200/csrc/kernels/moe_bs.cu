// Block-scaled tensor-core path for NVFP4 experts and NVFP4 dense matrices: both operands stay 4-bit all the way
// into the tensor core (tcgen05.mma kind::mxf4nvf4 with block scaling, one UE4M3 scale per 16 reduction elements of
// either operand), no de-quantisation to fp16 anywhere.
//
//   quant_nvfp4_tiles   bf16 / fp16 activation rows -> packed E2M1 + UE4M3 group scales in the 128 x 4 scale-atom
//                       layout + one fp32 scale per row, written in token-tile order (tile t owns rows t*BN ..)
//   moe_bs_ffn          persistent grouped GEMM, one CTA per SM walking (token tile, 128 weight rows) work items
//        warp 0      TMA producer: weight tiles (128 rows x 128 bytes = 256 reduction elements, 128-byte swizzle),
//                    the token tile, and both operands' scale atoms (cp.async.bulk, 2 KB per 128 rows and stage)
//        warp 1      tensor-memory owner; one thread copies the stage's scale atoms shared memory -> tensor memory
//                    (tcgen05.cp 32x128b.warpx4: 128 rows x 4 group scales become 4 columns, replicated over the four
//                    lane quarters) and issues 4 (gate/up: 8) block-scaled MMAs of K = 64 per stage
//        warps 2-9   epilogue (two warps per lane quarter, half of the token columns each): tcgen05.ld, per-tensor weight
//                    scale x per-row activation scale, SwiGLU(+clamp) -> fp16 rows in tile order, or fp32 rows scattered
//                    back to pair order
// The same kernel runs FP8 (E4M3) operands with one UE8M0 scale per 32 reduction elements (kind::mxf8f6f4, template FMT = 1):
// a 128-byte swizzle span then holds 128 elements = four MMAs of K = 32 that share ONE scale atom (the instruction descriptor's
// scale-factor ids pick the byte), the activations are quantised by quant_fp8_tiles, and the weights' scale atoms come from a side
// buffer the host derives from the checkpoint's 128 x 128 block scales (which must be powers of two, as DeepSeek-V3.1+ stores them).
// The weight bytes and their scale atoms are used exactly as they sit in the expert arena (the arena's NVFP4 scale layout
// is the tensor core's).  Every wait is bounded and reports through an error word.
// Reference seams replaced: BF16 -> NVFP4 activation quantisation + NVFP4 grouped GEMM over scattered expert pointers +
// fused SiLU*mul (src/core/expert_device.h:48-232, src/daemon/moe/moe_driver.cpp:1599-1677; scale-factor atom layout
// src/model/weight_loader/nvfp4_sfb_reformat.h:10-50).
#include "tc_common.cuh"
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include "moe_fmt.cuh"

namespace lsb {
using namespace tc;

int make_map_bytes_3d(CUtensorMap* map, const void* ptr, uint64_t pitch, uint64_t rows, uint64_t slot_stride, uint64_t nslots,
                      uint32_t box_bytes, uint32_t box_rows);

constexpr int kBsM = 128;        // weight rows per MMA (tensor-memory lanes)
constexpr int kBsStageK = 256;   // reduction elements per pipeline stage = 128 bytes of packed E2M1 = one swizzle span

constexpr int kBsMaxSlots = 1 << 16;

// ------------------------------------------------------------------------------------------ activation quantisation
__device__ __forceinline__ uint32_t pack_e2m1x8(const float* v) {       // v[0] -> bits 0-3 (low nibble = even element)
    uint32_t r;
    asm("{ .reg .b8 b0, b1, b2, b3;\n cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        " cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n mov.b32 %0, {b0, b1, b2, b3};\n}"
        : "=r"(r) : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return r;
}
__device__ __forceinline__ uint8_t float_to_ue4m3(float f) {            // f >= 0
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(f));
    return (uint8_t)(r & 0xffu);
}

// One block per padded tile row.  Row j of tile t reads
//   src_kind 0: bf16 x[sorted_pair[tile_row0[t] + j] / S]   (gather from the layer input)
//   src_kind 1: fp16 src[t * BN + j]                         (already in tile order: the SwiGLU output)
//   src_kind 2: bf16 src[t * BN + j]                         (dense operand in row order)
// and writes q[t * BN + j][K / 2], the row's group scales into atom row (t * max(BN, 128) + j) and alpha[t * BN + j]:
// value ~= e2m1 * ue4m3(group) * alpha(row).
__global__ void __launch_bounds__(128) quant_nvfp4_tiles_kernel(const void* __restrict__ src, int src_kind, const int* __restrict__ sorted_pair,
                                                                const int* __restrict__ tile_row0, const int* __restrict__ tile_n,
                                                                const int* __restrict__ counters, int S, int K, int BN,
                                                                uint8_t* __restrict__ q, uint8_t* __restrict__ sf, float* __restrict__ alpha) {
    constexpr int kMaxPer = 4;                               // groups per thread: K <= 128 * 16 * 4 = 8192
    __shared__ float red[4];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x / BN, j = blockIdx.x - t * BN;
    if (t >= counters[0] || j >= tile_n[t]) return;
    const size_t drow = (size_t)t * BN + j;
    const int G = K >> 4;
    float v[kMaxPer][16];
    float gmax[kMaxPer];
    float rmax = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
        const int g = threadIdx.x + i * 128;
        gmax[i] = 0.f;
        if (g < G) {
            if (src_kind == 1) {
                const __half* s = reinterpret_cast<const __half*>(src) + drow * K + g * 16;
                const uint4 a = *reinterpret_cast<const uint4*>(s), b = *reinterpret_cast<const uint4*>(s + 8);
                const __half2* ha = reinterpret_cast<const __half2*>(&a);
                const __half2* hb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 fa = __half22float2(ha[e]), fb = __half22float2(hb[e]);
                    v[i][2 * e] = fa.x; v[i][2 * e + 1] = fa.y; v[i][8 + 2 * e] = fb.x; v[i][8 + 2 * e + 1] = fb.y;
                }
            } else {
                const size_t srow = src_kind == 0 ? (size_t)(sorted_pair[tile_row0[t] + j] / S) : drow;
                const bf16* s = reinterpret_cast<const bf16*>(src) + srow * K + g * 16;
                unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(s)), v[i]);
                unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(s + 8)), v[i] + 8);
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) gmax[i] = fmaxf(gmax[i], fabsf(v[i][e]));
            rmax = fmaxf(rmax, gmax[i]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = rmax;
    __syncthreads();
    rmax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    // the largest group scale of the row lands on 448 (the top of UE4M3), the largest value on 6 (the top of E2M1)
    const float a = fmaxf(rmax, 1e-30f) * (1.f / (6.f * 448.f));
    const float inv_a = 1.f / a;
    if (threadIdx.x == 0) alpha[drow] = a;
    const int gt = (G + 3) >> 2;
    const size_t arow = (size_t)t * (BN > 128 ? BN : 128) + j;
    uint8_t* sf_row = sf + (arow >> 7) * (size_t)gt * 512 + (arow & 31) * 16 + ((arow & 127) >> 5) * 4;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
        const int g = threadIdx.x + i * 128;
        if (g < G) {
            const uint8_t s8 = float_to_ue4m3(gmax[i] * (1.f / 6.f) * inv_a);
            const float sv = fp8e4m3_to_float(s8);
            const float inv = sv > 0.f ? 1.f / (sv * a) : 0.f;
#pragma unroll
            for (int e = 0; e < 16; ++e) v[i][e] *= inv;
            uint2 w;
            w.x = pack_e2m1x8(v[i]);
            w.y = pack_e2m1x8(v[i] + 8);
            *reinterpret_cast<uint2*>(q + drow * (size_t)(K >> 1) + g * 8) = w;
            sf_row[(size_t)(g >> 2) * 512 + (g & 3)] = s8;
        }
    }
}

// FP8 variant of the quantiser: E4M3 values with one UE8M0 (power-of-two) scale per 32 elements, scale atoms in the same
// 128 x 4 layout (an atom row's four bytes = four consecutive groups = 128 elements), alpha = 1.  Same sources and tile order.
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {       // a -> byte 0
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return (uint32_t)lo | ((uint32_t)hi << 16);
}
__global__ void __launch_bounds__(128) quant_fp8_tiles_kernel(const void* __restrict__ src, int src_kind, const int* __restrict__ sorted_pair,
                                                              const int* __restrict__ tile_row0, const int* __restrict__ tile_n,
                                                              const int* __restrict__ counters, int S, int K, int BN,
                                                              uint8_t* __restrict__ q, uint8_t* __restrict__ sf, float* __restrict__ alpha) {
    constexpr int kMaxPer = 2;                               // 32-element groups per thread: K <= 128 * 32 * 2 = 8192
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x / BN, j = blockIdx.x - t * BN;
    if (t >= counters[0] || j >= tile_n[t]) return;
    const size_t drow = (size_t)t * BN + j;
    const int G = K >> 5;
    if (threadIdx.x == 0) alpha[drow] = 1.f;
    const int gt = (G + 3) >> 2;
    const size_t arow = (size_t)t * (BN > 128 ? BN : 128) + j;
    uint8_t* sf_row = sf + (arow >> 7) * (size_t)gt * 512 + (arow & 31) * 16 + ((arow & 127) >> 5) * 4;
#pragma unroll
    for (int i = 0; i < kMaxPer; ++i) {
        const int g = threadIdx.x + i * 128;
        if (g >= G) continue;
        float v[32];
        if (src_kind == 1) {
            const __half* sp = reinterpret_cast<const __half*>(src) + drow * K + g * 32;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 a = *reinterpret_cast<const uint4*>(sp + c * 8);
                const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(h[e]); v[c * 8 + 2 * e] = f.x; v[c * 8 + 2 * e + 1] = f.y; }
            }
        } else {
            const size_t srow = src_kind == 0 ? (size_t)(sorted_pair[tile_row0[t] + j] / S) : drow;
            const bf16* sp = reinterpret_cast<const bf16*>(src) + srow * K + g * 32;
#pragma unroll
            for (int c = 0; c < 4; ++c) unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(sp + c * 8)), v + c * 8);
        }
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(v[e]));
        // smallest power of two 2^ex with amax / 2^ex <= 448 (the top of E4M3)
        int ex = -127;
        if (amax > 0.f) {
            const float m = frexpf(amax * (1.f / 448.f), &ex);
            if (m == 0.5f) --ex;
            ex = max(-127, min(127, ex));
        }
        const float inv = exp2f((float)-ex);
        uint32_t w[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) w[c] = pack_e4m3x4(v[4 * c] * inv, v[4 * c + 1] * inv, v[4 * c + 2] * inv, v[4 * c + 3] * inv);
        uint4* dst = reinterpret_cast<uint4*>(q + drow * (size_t)K + g * 32);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        sf_row[(size_t)(g >> 2) * 512 + (g & 3)] = (uint8_t)(ex + 127);
    }
}

// Per operand format: reduction elements of one 128-byte swizzle span (= one pipeline stage), bytes of scale atoms per 128 rows
// and stage, tensor-memory columns they occupy.
template <int FMT> struct BsFmt;
template <> struct BsFmt<0> { static constexpr int STAGE_K = 256, SF_BYTES = 2048, SF_COLS_OP = 16, ATOM_K = 64; };     // NVFP4, UE4M3 / 16
template <> struct BsFmt<1> { static constexpr int STAGE_K = 128, SF_BYTES = 512, SF_COLS_OP = 4, ATOM_K = 128; };      // FP8 E4M3, UE8M0 / 32

// ------------------------------------------------------------------------------------------ grouped block-scaled GEMM
// Instruction descriptor of kind::mxf4nvf4 with block scaling: E2M1 x E2M1 (format code 1 of this kind), UE4M3 scales
// (scale-format bit 0), both operands K-major, fp32 accumulate, K = 64 per instruction, scale-factor ids 0 (the four
// group scales of one MMA fill the whole 32-bit column).
__host__ __device__ constexpr uint32_t idesc_mxf4nvf4(int umma_m, int umma_n) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(umma_m >> 4) << 24);
}
__device__ __forceinline__ void umma_mxf4nvf4(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
// kind::mxf8f6f4 with block scaling: E4M3 x E4M3 (format code 0), UE8M0 scales (scale-format bit 23), K = 32 per instruction; the
// scale-factor ids (bits 4-5 for B, 29-30 for A) select which byte of the 32-bit scale column this instruction uses.
__host__ __device__ constexpr uint32_t idesc_mxf8(int umma_m, int umma_n) {
    return ((uint32_t)(umma_n >> 3) << 17) | (1u << 23) | ((uint32_t)(umma_m >> 4) << 24);
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
// Shared-memory descriptor of one scale atom: 32 rows of 16 bytes, no swizzle (core matrices of 8 rows x 16 bytes,
// 128 bytes apart).
__device__ __forceinline__ uint64_t smem_desc_atom(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// 32 rows x 128 bits of shared memory -> 4 columns of tensor memory, the same 32 rows in each of the four lane quarters
__device__ __forceinline__ void tmem_cp_atom(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

struct MoeBsParams {
    const uint8_t* arena; const int* slot_of; ExpertFmt ef;      // ef.stride == 0: dense mode, one matrix at arena + off_down
    const uint8_t* xsf; const float* xalpha;                      // token operand: scale atoms and per-row scales (tile order)
    const int* tile_expert; const int* tile_row0; const int* tile_n; const int* counters; const int* sorted_pair;
    __half* act;          // gate/up output, [tiles * BN, F] fp16 in tile order
    void* y;              // down output, [npairs, ldo] fp32 (or bf16) in pair order
    float limit; float down_scale;                                // down_scale != 0: per-tensor weight scale given by the caller
    int ldo, out_bf16;
    int* miss_flag; int* err;
    // FP8: the weights' scale atoms live outside the arena (derived from the 128 x 128 block scales): slot s at wsf + s * wsf_stride,
    // this launch's matrix (gate / down) at + wsf_off0, the up matrix at + wsf_off1
    const uint8_t* wsf; long long wsf_stride, wsf_off0, wsf_off1;
};

template <int BN, bool GATEUP, int FMT> struct MoeBsCfg {
    static constexpr int A_TILES = GATEUP ? 2 : 1;
    static constexpr int A_BYTES = kBsM * 128;                    // one weight tile: 128 rows x 128 bytes
    static constexpr int B_BYTES = BN * 128;
    static constexpr int SF_BYTES = BsFmt<FMT>::SF_BYTES;         // scale atoms of 128 rows x one stage's reduction elements
    static constexpr int TX = A_TILES * (A_BYTES + SF_BYTES) + B_BYTES + SF_BYTES;      // bytes the producer loads per stage
    static constexpr int STAGE = (TX + 1023) / 1024 * 1024;       // tiles of the next stage start on a swizzle-atom boundary
    static constexpr int STAGES_FIT = (220 * 1024) / STAGE;
    static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
    static constexpr int ACC_COLS = A_TILES * BN;
    static constexpr int NBUF = ACC_COLS > 128 ? 1 : 2;
    static constexpr int SF_OP = BsFmt<FMT>::SF_COLS_OP;          // scale columns per operand and stage
    static constexpr int SF_COLS = (A_TILES + 1) * SF_OP;
    static constexpr int SF_BASE = NBUF * ACC_COLS;
    static constexpr int TMEM_COLS = 512;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM = STAGES * STAGE + BAR_BYTES + 1024;
    static constexpr int EPI_WARPS = 8;                          // two per tensor-memory lane quarter, half of the columns each
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;
    static_assert(SF_BASE + 2 * SF_COLS <= 512, "tensor memory budget");
    static_assert(STAGES >= 3 && SMEM <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ void bs_work_item(int w, int ntiles, int NT, int& t, int& j) {
    constexpr int kGroup = 8;            // consecutive token tiles (mostly one expert) share a weight tile in flight
    const int per = kGroup * NT;
    const int gi = w / per, r = w % per;
    const int t0 = gi * kGroup;
    const int gsz = min(kGroup, ntiles - t0);
    t = t0 + r % gsz;
    j = r / gsz;
}

template <int BN, bool GATEUP, int FMT>
__global__ void __launch_bounds__(MoeBsCfg<BN, GATEUP, FMT>::THREADS) moe_bs_ffn_kernel(const __grid_constant__ CUtensorMap map_b,
                                                                                   const __grid_constant__ CUtensorMap map_w0,
                                                                                   const __grid_constant__ CUtensorMap map_w1, MoeBsParams p) {
    using C = MoeBsCfg<BN, GATEUP, FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;      // [2]
    uint64_t* acc_empty = acc_full + 2;          // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = GATEUP ? p.ef.H : p.ef.F;
    const int NOUT = GATEUP ? p.ef.F : p.ef.H;
    const int NT = NOUT / kBsM;
    const int nst = K / BsFmt<FMT>::STAGE_K;
    const int gt = K / BsFmt<FMT>::ATOM_K;       // scale atoms per 128 rows
    const bool dense = p.ef.stride == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], C::EPI_WARPS); }
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
    const int ntiles = p.counters[0];
    const int total = ntiles * NT;
    auto slot_of = [&](int t) { return dense ? 0 : p.slot_of[p.tile_expert[t]]; };
    auto slot_ok = [&](int slot) { return slot >= 0 && slot < kBsMaxSlots; };

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer: weight tiles, token tile, scale atoms of both ----------------
            uint32_t g = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                bs_work_item(w, ntiles, NT, t, jn);
                const int slot = slot_of(t);
                if (!slot_ok(slot)) {
                    if (GATEUP && p.miss_flag && jn == 0) atomicExch(p.miss_flag, p.tile_expert[t] + 1);
                    continue;
                }
                const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
                const uint8_t* wsf = FMT ? p.wsf + (size_t)slot * p.wsf_stride : base;
                const uint8_t* sf0 = wsf + (FMT ? p.wsf_off0 : (GATEUP ? p.ef.off_sg : p.ef.off_sd)) + (size_t)jn * gt * 512;
                const uint8_t* sf1 = wsf + (FMT ? p.wsf_off1 : p.ef.off_su) + (size_t)jn * gt * 512;
                // token scale atoms: tile t owns atom rows t * max(BN, 128) .. (one 128-row atom row for BN <= 128)
                const uint8_t* sfx = p.xsf + (size_t)t * gt * 512;
                for (int it = 0; it < nst; ++it, ++g) {
                    const int s = g % C::STAGES;
                    ok = mbar_wait(&empty[s], ((g / C::STAGES) & 1) ^ 1, p.err, 21);
                    if (!ok) break;
                    uint8_t* st = smem + s * C::STAGE;
                    mbar_expect_tx(&full[s], C::TX);
                    tma_load_3d(st, &map_w0, &full[s], it * 128, jn * kBsM, slot);
                    if (GATEUP) tma_load_3d(st + C::A_BYTES, &map_w1, &full[s], it * 128, jn * kBsM, slot);
                    tma_load_3d(st + C::A_TILES * C::A_BYTES, &map_b, &full[s], it * 128, t * BN, 0);
                    uint8_t* sfs = st + C::A_TILES * C::A_BYTES + C::B_BYTES;
                    bulk_load_1d(sfs, sf0 + (size_t)it * C::SF_BYTES, C::SF_BYTES, &full[s]);
                    if (GATEUP) bulk_load_1d(sfs + C::SF_BYTES, sf1 + (size_t)it * C::SF_BYTES, C::SF_BYTES, &full[s]);
                    bulk_load_1d(sfs + C::A_TILES * C::SF_BYTES, sfx + (size_t)it * C::SF_BYTES, C::SF_BYTES, &full[s]);
                }
            }
            if (!ok) {
                // loads in flight still write this CTA's shared memory: let them land (bounded, no error code)
                for (uint32_t i = g > (uint32_t)C::STAGES ? g - C::STAGES : 0; i < g; ++i) mbar_wait(&full[i % C::STAGES], (i / C::STAGES) & 1, nullptr, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- scale copies + MMA issue ----------------
            constexpr uint32_t idesc = FMT ? idesc_mxf8(kBsM, BN) : idesc_mxf4nvf4(kBsM, BN);
            constexpr int OP = C::SF_OP;
            uint32_t g = 0, lt = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
                int t, jn;
                bs_work_item(w, ntiles, NT, t, jn);
                if (!slot_ok(slot_of(t))) continue;
                const uint32_t buf = lt % C::NBUF;
                ok = mbar_wait(&acc_empty[buf], ((lt / C::NBUF) & 1u) ^ 1u, p.err, 22);      // the epilogue has drained this accumulator set
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_d + buf * C::ACC_COLS;
                for (int it = 0; it < nst; ++it, ++g) {
                    const int s = g % C::STAGES;
                    ok = mbar_wait(&full[s], (g / C::STAGES) & 1, p.err, 23);
                    if (!ok) break;
                    tc_fence_after();
                    const uint8_t* st = smem + s * C::STAGE;
                    const uint32_t sfs = smem_u32(st + C::A_TILES * C::A_BYTES + C::B_BYTES);
                    const uint32_t sft = tmem_d + C::SF_BASE + (g & 1u) * C::SF_COLS;          // [A0 | (A1) | B] scale columns, OP each
                    const uint64_t da0 = smem_desc_sw128(st), da1 = smem_desc_sw128(st + C::A_BYTES);
                    const uint64_t db = smem_desc_sw128(st + C::A_TILES * C::A_BYTES);
                    if (FMT == 0) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            tmem_cp_atom(sft + 4 * k, smem_desc_atom(sfs + k * 512));
                            if (GATEUP) tmem_cp_atom(sft + OP + 4 * k, smem_desc_atom(sfs + C::SF_BYTES + k * 512));
                            tmem_cp_atom(sft + C::A_TILES * OP + 4 * k, smem_desc_atom(sfs + C::A_TILES * C::SF_BYTES + k * 512));
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t accum = (it > 0 || k > 0) ? 1u : 0u;
                            umma_mxf4nvf4(acc, da0 + 2 * k, db + 2 * k, idesc, sft + 4 * k, sft + C::A_TILES * OP + 4 * k, accum);
                            if (GATEUP) umma_mxf4nvf4(acc + BN, da1 + 2 * k, db + 2 * k, idesc, sft + OP + 4 * k, sft + C::A_TILES * OP + 4 * k, accum);
                        }
                    } else {
                        // one atom per operand covers the stage: byte k of a row's scale column belongs to the stage's k-th MMA
                        tmem_cp_atom(sft, smem_desc_atom(sfs));
                        if (GATEUP) tmem_cp_atom(sft + OP, smem_desc_atom(sfs + C::SF_BYTES));
                        tmem_cp_atom(sft + C::A_TILES * OP, smem_desc_atom(sfs + C::A_TILES * C::SF_BYTES));
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t accum = (it > 0 || k > 0) ? 1u : 0u;
                            const uint32_t idk = idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4);
                            umma_mxf8(acc, da0 + 2 * k, db + 2 * k, idk, sft, sft + C::A_TILES * OP, accum);
                            if (GATEUP) umma_mxf8(acc + BN, da1 + 2 * k, db + 2 * k, idk, sft + OP, sft + C::A_TILES * OP, accum);
                        }
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
                ++lt;
            }
        }
    } else {
        // ---------------- epilogue (4 warps: one tensor-memory lane quarter each) ----------------
        const int q = warp & 3;
        const int chalf = (warp - 2) >> 2;                 // which half of the token columns this warp drains
        constexpr int CH = BN >= 32 ? BN / 2 : BN;
        uint32_t lt = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
            int t, jn;
            bs_work_item(w, ntiles, NT, t, jn);
            const int slot = slot_of(t);
            if (!slot_ok(slot)) continue;
            const int row0 = p.tile_row0[t], ncols = p.tile_n[t];
            const int n = jn * kBsM + q * 32 + lane;
            const uint8_t* base = p.arena + (size_t)slot * p.ef.stride;
            const uint32_t buf = lt % C::NBUF;
            int okw = 1;
            if (lane == 0) okw = mbar_wait_relaxed(&acc_full[buf], (lt / C::NBUF) & 1u, p.err, 24) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
            tc_fence_after();
            if (ok) {
                float sg, su = 1.f;
                if (p.down_scale != 0.f) sg = p.down_scale;
                else {
                    const float* tail = reinterpret_cast<const float*>(base + p.ef.off_tail);
                    if (GATEUP) { sg = tail[0]; su = tail[1]; } else sg = tail[2];
                }
                const uint32_t lane_addr = tmem_d + buf * C::ACC_COLS + ((uint32_t)(q * 32) << 16);
                const float* xa = p.xalpha + (size_t)t * BN;
#pragma unroll 1
                for (int c0 = chalf * CH; c0 < (chalf + 1) * CH; c0 += 16) {
                    if (c0 >= ncols) break;
                    // the 16 columns' row scales and output rows: one lane each, handed round by shuffles (the stores below
                    // may alias anything as far as the compiler knows, so loads inside the store loop would serialise)
                    const int cl = c0 + (lane & 15);
                    const float ax_l = cl < ncols ? xa[cl] : 0.f;
                    int orow_l = row0 + cl;
                    if (!GATEUP && p.sorted_pair && cl < ncols) orow_l = p.sorted_pair[row0 + cl];
                    float gq[16], uq[16];
                    tmem_ld16(lane_addr + (uint32_t)c0, gq);
                    if (GATEUP) tmem_ld16(lane_addr + (uint32_t)(BN + c0), uq);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float ax = __shfl_sync(0xffffffffu, ax_l, j);
                        const int orow = __shfl_sync(0xffffffffu, orow_l, j);
                        if (c0 + j < ncols && n < NOUT) {
                            if (GATEUP) {
                                float gv = gq[j] * sg * ax, uv = uq[j] * su * ax;
                                if (p.limit > 0.f) { gv = fminf(gv, p.limit); uv = fminf(fmaxf(uv, -p.limit), p.limit); }
                                p.act[((size_t)t * BN + c0 + j) * NOUT + n] = __float2half_rn(siluf_(gv) * uv);
                            } else {
                                if (p.out_bf16) reinterpret_cast<bf16*>(p.y)[(size_t)orow * p.ldo + n] = __float2bfloat16(gq[j] * sg * ax);
                                else reinterpret_cast<float*>(p.y)[(size_t)orow * p.ldo + n] = gq[j] * sg * ax;
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
    pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------ host side
static int bs_cached_map(CUtensorMap* out, const void* ptr, uint64_t pitch, uint64_t rows, uint64_t sstride, uint64_t nslots, uint32_t box_rows) {
    struct Key {
        const void* p; uint64_t pitch, rows, ss, ns; uint32_t br;
        bool operator<(const Key& o) const { return std::tie(p, pitch, rows, ss, ns, br) < std::tie(o.p, o.pitch, o.rows, o.ss, o.ns, o.br); }
    };
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> g(mu);
    const Key k{ptr, pitch, rows, sstride, nslots, box_rows};
    auto it = cache.find(k);
    if (it != cache.end()) { *out = it->second; return 0; }
    CUtensorMap m;
    const int rc = make_map_bytes_3d(&m, ptr, pitch, rows, sstride, nslots, 128, box_rows);
    if (rc) return rc;
    if (cache.size() > 65536) cache.clear();
    cache[k] = m;
    *out = m;
    return 0;
}

static int bs_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, bool GATEUP, int FMT>
static int launch_moe_bs(const void* xq, int cap_rows, const MoeBsParams& p, int max_tiles, cudaStream_t st) {
    using C = MoeBsCfg<BN, GATEUP, FMT>;
    const int K = GATEUP ? p.ef.H : p.ef.F, nout = GATEUP ? p.ef.F : p.ef.H;
    const uint64_t pitch = FMT ? (uint64_t)K : (uint64_t)K / 2;
    const bool dense = p.ef.stride == 0;
    const uint64_t sstride = dense ? pitch * (uint64_t)nout : (uint64_t)p.ef.stride;
    const uint64_t nslots = dense ? 1 : (uint64_t)kBsMaxSlots;
    CUtensorMap mb, mw0, mw1;
    int rc = bs_cached_map(&mb, xq, pitch, (uint64_t)cap_rows, pitch * (uint64_t)cap_rows, 1, (uint32_t)BN);
    if (rc) return rc;
    rc = bs_cached_map(&mw0, p.arena + (GATEUP ? p.ef.off_gate : p.ef.off_down), pitch, (uint64_t)nout, sstride, nslots, (uint32_t)kBsM);
    if (rc) return rc;
    if (GATEUP) { rc = bs_cached_map(&mw1, p.arena + p.ef.off_up, pitch, (uint64_t)nout, sstride, nslots, (uint32_t)kBsM); if (rc) return rc; }
    else mw1 = mw0;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(moe_bs_ffn_kernel<BN, GATEUP, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM); attr = true; }
    const long long work = (long long)(nout / kBsM) * max_tiles;
    const int grid = (int)(work < bs_sm_count() ? (work > 0 ? work : 1) : bs_sm_count());
    launch_pdl((moe_bs_ffn_kernel<BN, GATEUP, FMT>), grid, C::THREADS, C::SMEM, st, mb, mw0, mw1, p);
    return (int)cudaGetLastError();
}

template <bool GATEUP, int FMT>
static int dispatch_bs(int BN, const void* xq, int cap_rows, const MoeBsParams& p, int max_tiles, cudaStream_t st) {
    switch (BN) {
        case 32: return launch_moe_bs<32, GATEUP, FMT>(xq, cap_rows, p, max_tiles, st);
        case 64: return launch_moe_bs<64, GATEUP, FMT>(xq, cap_rows, p, max_tiles, st);
        case 128: return launch_moe_bs<128, GATEUP, FMT>(xq, cap_rows, p, max_tiles, st);
    }
    return -1;
}

}  // namespace lsb
using namespace lsb;

// Quantise activation rows to NVFP4 in token-tile order (see quant_nvfp4_tiles_kernel).  `q` holds max_tiles * BN rows of
// K / 2 bytes, `sf` max_tiles * (K / 64) * 512 bytes, `alpha` max_tiles * BN floats.  K % 64 == 0, K <= 8192.
LSB_API int lsb_quant_nvfp4_tiles(const void* src, int src_kind, const void* sorted_pair, const void* tile_row0, const void* tile_n,
                                  const void* counters, int S, int K, int BN, int max_tiles, void* q, void* sf, void* alpha, void* stream) {
    if (K % 64 || K > 8192 || (BN != 32 && BN != 64 && BN != 128) || max_tiles <= 0) return -1;
    if (src_kind < 0 || src_kind > 2 || (src_kind == 0 && !sorted_pair)) return -1;
    launch_pdl((quant_nvfp4_tiles_kernel), max_tiles * BN, 128, 0, (cudaStream_t)stream, src, src_kind, (const int*)sorted_pair,
               (const int*)tile_row0, (const int*)tile_n, (const int*)counters, S, K, BN, (uint8_t*)q, (uint8_t*)sf, (float*)alpha);
    LSB_CHECK_LAUNCH();
}

// Grouped NVFP4 x NVFP4 expert GEMM on the block-scaled tensor-core path.
// gateup != 0: act[t * BN + j][f] = SwiGLU(x . Wgate[f], x . Wup[f]) for row j of token tile t (fp16, [max_tiles * BN, F]).
// gateup == 0: y[pair][h] = act . Wdown[h] (fp32, [npairs, H], rows in pair order through sorted_pair).
// xq / xsf / xalpha: the token operand as written by lsb_quant_nvfp4_tiles with the same BN.  Hidden and expert widths must
// be multiples of 256 (reduction) and 128 (rows).
LSB_API int lsb_moe_bs_ffn(int gateup, const void* xq, const void* xsf, const void* xalpha, const void* arena, const void* slot_of,
                           const void* fmt_struct, const void* tile_expert, const void* tile_row0, const void* tile_n, const void* counters,
                           const void* sorted_pair, void* out, int BN, int max_tiles, float limit, void* miss_flag, void* err, void* stream) {
    const ExpertFmt* ef = (const ExpertFmt*)fmt_struct;
    const int K = gateup ? ef->H : ef->F, nout = gateup ? ef->F : ef->H;
    if (ef->fmt != 2 || K % kBsStageK || nout % kBsM || ((uintptr_t)xq & 127) || ((uintptr_t)xsf & 15)) return -1;
    if ((ef->stride & 15) || (ef->off_sg & 15) || (ef->off_su & 15) || (ef->off_sd & 15)) return -1;
    MoeBsParams p;
    memset(&p, 0, sizeof(p));
    p.arena = (const uint8_t*)arena; p.slot_of = (const int*)slot_of; p.ef = *ef;
    p.xsf = (const uint8_t*)xsf; p.xalpha = (const float*)xalpha;
    p.tile_expert = (const int*)tile_expert; p.tile_row0 = (const int*)tile_row0; p.tile_n = (const int*)tile_n;
    p.counters = (const int*)counters; p.sorted_pair = (const int*)sorted_pair;
    p.act = gateup ? (__half*)out : nullptr; p.y = gateup ? nullptr : out;
    p.limit = limit; p.down_scale = 0.f; p.ldo = nout; p.out_bf16 = 0;
    p.miss_flag = (int*)miss_flag; p.err = (int*)err;
    cudaStream_t st = (cudaStream_t)stream;
    const int rc = gateup ? dispatch_bs<true, 0>(BN, xq, max_tiles * BN, p, max_tiles, st) : dispatch_bs<false, 0>(BN, xq, max_tiles * BN, p, max_tiles, st);
    return rc;
}

// Dense linear layer with NVFP4 weights on the same kernel: out[m][n] = alpha * sum_k x[m][k] * W[n][k] for M rows quantised
// by lsb_quant_nvfp4_tiles (src_kind 2, tiles of BN consecutive rows: tile_row0[t] = t * BN).  w: [N, K / 2] packed E2M1,
// wsf: its scale atoms, N % 128 == 0, K % 256 == 0.
LSB_API int lsb_gemm_nvfp4_bs(void* out, const void* xq, const void* xsf, const void* xalpha, const void* w, const void* wsf, float alpha,
                              int N, int K, int ldo, int out_bf16, const void* tile_row0, const void* tile_n, const void* counters, int BN,
                              int ntiles, void* err, void* stream) {
    if (K % kBsStageK || N % kBsM || ((uintptr_t)xq & 127) || ((uintptr_t)xsf & 15) || ((uintptr_t)w & 15) || ((uintptr_t)wsf & 15) || alpha == 0.f) return -1;
    MoeBsParams p;
    memset(&p, 0, sizeof(p));
    p.arena = (const uint8_t*)w;
    p.ef.fmt = 2; p.ef.H = N; p.ef.F = K; p.ef.stride = 0; p.ef.off_down = 0;
    p.ef.off_sd = (long long)((const uint8_t*)wsf - (const uint8_t*)w);
    p.xsf = (const uint8_t*)xsf; p.xalpha = (const float*)xalpha;
    p.tile_row0 = (const int*)tile_row0; p.tile_n = (const int*)tile_n; p.counters = (const int*)counters;
    p.y = out; p.down_scale = alpha; p.ldo = ldo; p.out_bf16 = out_bf16; p.err = (int*)err;
    return dispatch_bs<false, 0>(BN, xq, ntiles * BN, p, ntiles, (cudaStream_t)stream);
}

// ---- FP8 (E4M3 values, UE8M0 scales per 32) on the same kernel -------------------------------------------------------------
// Quantise activation rows to FP8 in token-tile order: `q` max_tiles * BN rows of K bytes, `sf` max_tiles * (K / 128) * 512 bytes,
// `alpha` max_tiles * BN floats (all 1).  K % 128 == 0, K <= 8192.
LSB_API int lsb_quant_fp8_tiles(const void* src, int src_kind, const void* sorted_pair, const void* tile_row0, const void* tile_n,
                                const void* counters, int S, int K, int BN, int max_tiles, void* q, void* sf, void* alpha, void* stream) {
    if (K % 128 || K > 8192 || (BN != 32 && BN != 64 && BN != 128) || max_tiles <= 0) return -1;
    if (src_kind < 0 || src_kind > 2 || (src_kind == 0 && !sorted_pair)) return -1;
    launch_pdl((quant_fp8_tiles_kernel), max_tiles * BN, 128, 0, (cudaStream_t)stream, src, src_kind, (const int*)sorted_pair,
               (const int*)tile_row0, (const int*)tile_n, (const int*)counters, S, K, BN, (uint8_t*)q, (uint8_t*)sf, (float*)alpha);
    LSB_CHECK_LAUNCH();
}

// Grouped FP8 x FP8 expert GEMM (arena format 1).  wsf: the weights' UE8M0 scale atoms, slot s at wsf + s * wsf_stride with the gate,
// up and down matrices' atoms at the three offsets ((rows / 128) * (K / 128) atoms of 512 equal bytes each: the exponent of the
// 128 x 128 block's power-of-two scale).  Hidden and expert widths must be multiples of 128.
LSB_API int lsb_moe_bs_ffn_fp8(int gateup, const void* xq, const void* xsf, const void* xalpha, const void* arena, const void* slot_of,
                               const void* fmt_struct, const void* wsf, long long wsf_stride, long long wsf_off_gate, long long wsf_off_up,
                               long long wsf_off_down, const void* tile_expert, const void* tile_row0, const void* tile_n, const void* counters,
                               const void* sorted_pair, void* out, int BN, int max_tiles, float limit, void* miss_flag, void* err, void* stream) {
    const ExpertFmt* ef = (const ExpertFmt*)fmt_struct;
    const int K = gateup ? ef->H : ef->F, nout = gateup ? ef->F : ef->H;
    if (ef->fmt != 1 || K % 128 || nout % kBsM || ((uintptr_t)xq & 127) || ((uintptr_t)xsf & 15) || ((uintptr_t)wsf & 15)) return -1;
    if ((ef->stride & 15) || (wsf_stride & 15) || (wsf_off_gate & 15) || (wsf_off_up & 15) || (wsf_off_down & 15)) return -1;
    MoeBsParams p;
    memset(&p, 0, sizeof(p));
    p.arena = (const uint8_t*)arena; p.slot_of = (const int*)slot_of; p.ef = *ef;
    p.xsf = (const uint8_t*)xsf; p.xalpha = (const float*)xalpha;
    p.tile_expert = (const int*)tile_expert; p.tile_row0 = (const int*)tile_row0; p.tile_n = (const int*)tile_n;
    p.counters = (const int*)counters; p.sorted_pair = (const int*)sorted_pair;
    p.act = gateup ? (__half*)out : nullptr; p.y = gateup ? nullptr : out;
    p.limit = limit; p.down_scale = 1.f; p.ldo = nout; p.out_bf16 = 0;
    p.miss_flag = (int*)miss_flag; p.err = (int*)err;
    p.wsf = (const uint8_t*)wsf; p.wsf_stride = wsf_stride; p.wsf_off0 = gateup ? wsf_off_gate : wsf_off_down; p.wsf_off1 = wsf_off_up;
    cudaStream_t st = (cudaStream_t)stream;
    return gateup ? dispatch_bs<true, 1>(BN, xq, max_tiles * BN, p, max_tiles, st) : dispatch_bs<false, 1>(BN, xq, max_tiles * BN, p, max_tiles, st);
}

// Dense linear layer with FP8 weights: out[m][n] = sum_k x[m][k] * W[n][k] for M rows quantised by lsb_quant_fp8_tiles (src_kind 2).
// w: [N, K] E4M3, wsf: its UE8M0 scale atoms ((N / 128) * (K / 128) atoms), N % 128 == 0, K % 128 == 0.
LSB_API int lsb_gemm_fp8_bs(void* out, const void* xq, const void* xsf, const void* xalpha, const void* w, const void* wsf,
                            int N, int K, int ldo, int out_bf16, const void* tile_row0, const void* tile_n, const void* counters, int BN,
                            int ntiles, void* err, void* stream) {
    if (K % 128 || N % kBsM || ((uintptr_t)xq & 127) || ((uintptr_t)xsf & 15) || ((uintptr_t)w & 15) || ((uintptr_t)wsf & 15)) return -1;
    MoeBsParams p;
    memset(&p, 0, sizeof(p));
    p.arena = (const uint8_t*)w;
    p.ef.fmt = 1; p.ef.H = N; p.ef.F = K; p.ef.stride = 0; p.ef.off_down = 0;
    p.xsf = (const uint8_t*)xsf; p.xalpha = (const float*)xalpha;
    p.tile_row0 = (const int*)tile_row0; p.tile_n = (const int*)tile_n; p.counters = (const int*)counters;
    p.y = out; p.down_scale = 1.f; p.ldo = ldo; p.out_bf16 = out_bf16; p.err = (int*)err;
    p.wsf = (const uint8_t*)wsf; p.wsf_stride = 0; p.wsf_off0 = 0; p.wsf_off1 = 0;
    return dispatch_bs<false, 1>(BN, xq, ntiles * BN, p, ntiles, (cudaStream_t)stream);
}

LSB_API int lsb_trace_set_moe_bs(void* buf) { return lsb_trace_install(buf); }
