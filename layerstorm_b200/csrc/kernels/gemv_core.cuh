// Warp-level weight-streaming dot products shared by the dense GEMV kernels and the
// MoE expert kernels.  One warp owns two weight rows and MT activation rows; lanes
// stride over K in 16-byte weight vectors.  Everything accumulates in fp32.
//
// Weight formats (struct = a view of ONE weight row):
//   WRowBf16   bf16 [K]
//   WRowF32    fp32 [K]
//   WRowFp8B   e4m3 [K] with one fp32 scale per 128 columns (the row's slice of the
//              128x128 block-scale grid)
//   WRowNvfp4  packed E2M1 [K/2] (low nibble = even k), e4m3 scales per 16 columns
//              stored in the 128x4 "scale atom" layout used by block-scaled tensor-core
//              MMAs on this architecture family:
//                 tile   = (n/128) * ceil(G/4) + g/4          (G = K/16 groups)
//                 within = (n%32)*16 + ((n%128)/32)*4 + g%4   (bytes, 512 per tile)
//              and one fp32 per-tensor scale applied by the caller.
#pragma once
#include "common.cuh"

namespace lsb {

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

struct WRowBf16 {
    static constexpr int EPL = 8;
    const bf16* w;
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + k); }
    __device__ __forceinline__ void load(int k, float* f) const {
        uint4 v = ldg_stream(w + k);
        unpack_bf16x8(v, f);
    }
};

struct WRowF32 {
    static constexpr int EPL = 4;
    const float* w;
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + k); }
    __device__ __forceinline__ void load(int k, float* f) const {
        uint4 v = ldg_stream(w + k);
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
};

struct WRowFp8B {
    static constexpr int EPL = 16;
    const uint8_t* w;     // row start
    const float* scale;   // scale for column block 0 of this row; stride 1 per 128 cols
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + k); }
    __device__ __forceinline__ void load(int k, float* f) const {
        uint4 v = ldg_stream(w + k);
        const float s = __ldg(scale + (k >> 7));
        unpack_fp8x4(v.x, f); unpack_fp8x4(v.y, f + 4);
        unpack_fp8x4(v.z, f + 8); unpack_fp8x4(v.w, f + 12);
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] *= s;
    }
};

__device__ __forceinline__ void unpack_fp4x8(uint32_t v, float s, float* f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = fp4_to_float((v >> (4 * i)) & 0xfu) * s;
}

struct WRowNvfp4 {
    static constexpr int EPL = 32;
    const uint8_t* w;    // row start of packed fp4 (K/2 bytes per row)
    const uint8_t* sf;   // base of the scale-atom array for this matrix
    int n;               // row index inside the matrix (selects the atom lane)
    int gtiles;          // ceil(G/4)
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + (k >> 1)); }
    __device__ __forceinline__ void load(int k, float* f) const {
        uint4 v = ldg_stream(w + (k >> 1));
        const int g = k >> 4;  // even
        const size_t off = ((size_t)(n >> 7) * gtiles + (g >> 2)) * 512 + (n & 31) * 16 + ((n & 127) >> 5) * 4 + (g & 3);
        const uint16_t s2 = __ldg(reinterpret_cast<const uint16_t*>(sf + off));
        const float s0 = fp8e4m3_to_float((uint8_t)(s2 & 0xff));
        const float s1 = fp8e4m3_to_float((uint8_t)(s2 >> 8));
        unpack_fp4x8(v.x, s0, f); unpack_fp4x8(v.y, s0, f + 8);
        unpack_fp4x8(v.z, s1, f + 16); unpack_fp4x8(v.w, s1, f + 24);
    }
};

// GGUF Q4_K: super-blocks of 256 weights in 144 bytes: fp16 d, fp16 dmin, 12 bytes of packed 6-bit (scale, min) pairs for 8
// sub-blocks of 32, then 128 bytes of 4-bit quants (bytes 32j..32j+31: low nibbles = sub-block 2j, high nibbles = 2j+1).
// w = d * scale_s * q - dmin * min_s.  Layout reference: src/model/quantization/gguf_kquant.h:49-57 (block sizes) and the
// ggml k-quant definition; the container reader's CPU codec (csrc/runtime/gguf.cpp) is the oracle for this decoder.
__device__ __forceinline__ void q4k_scale_min(const uint8_t* q, int j, float& sc, float& mn) {
    if (j < 4) { sc = (float)(q[j] & 63); mn = (float)(q[j + 4] & 63); }
    else { sc = (float)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); mn = (float)((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}
struct Q4KHeader { float d, dmin; uint8_t sc[12]; };
__device__ __forceinline__ Q4KHeader q4k_header(const uint8_t* blk) {
    const uint4 h = __ldg(reinterpret_cast<const uint4*>(blk));
    Q4KHeader o;
    const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
    o.d = __low2float(dd); o.dmin = __high2float(dd);
    const uint32_t w[3] = {h.y, h.z, h.w};
#pragma unroll
    for (int i = 0; i < 12; ++i) o.sc[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
    return o;
}
struct WRowQ4K {
    static constexpr int EPL = 32;
    const uint8_t* w;    // row start: K/256 blocks of 144 bytes
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + (size_t)(k >> 8) * 144); }
    __device__ __forceinline__ void load(int k, float* f) const {
        const uint8_t* blk = w + (size_t)(k >> 8) * 144;
        const int sub = (k & 255) >> 5;
        const Q4KHeader h = q4k_header(blk);
        float sc, mn;
        q4k_scale_min(h.sc, sub, sc, mn);
        const float a = h.d * sc, b = h.dmin * mn;
        const uint8_t* qs = blk + 16 + (sub >> 1) * 32;
        const uint4 v0 = ldg_stream(qs), v1 = ldg_stream(qs + 16);
        const uint32_t wv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const int sh = (sub & 1) * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) f[4 * i + c] = a * (float)((wv[i] >> (8 * c + sh)) & 0xFu) - b;
    }
};

// GGUF Q5_K: 176-byte super-blocks of 256 weights: fp16 d, fp16 dmin, 12 bytes of packed 6-bit (scale, min) pairs (as Q4_K),
// 32 bytes of fifth bits (bit s of byte l belongs to element l of sub-block s), 128 bytes of low nibbles (as Q4_K).
// w = d * scale_s * (q4 + 16 * bit) - dmin * min_s.  The block is a multiple of 16 bytes: used as it sits in the file.
struct WRowQ5K {
    static constexpr int EPL = 32;
    const uint8_t* w;    // row start: K/256 blocks of 176 bytes
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + (size_t)(k >> 8) * 176); }
    __device__ __forceinline__ void load(int k, float* f) const {
        const uint8_t* blk = w + (size_t)(k >> 8) * 176;
        const int sub = (k & 255) >> 5;
        const Q4KHeader h = q4k_header(blk);
        float sc, mn;
        q4k_scale_min(h.sc, sub, sc, mn);
        const float a = h.d * sc, b = h.dmin * mn;
        const uint4 h0 = ldg_stream(blk + 16), h1 = ldg_stream(blk + 32);
        const uint8_t* qs = blk + 48 + (sub >> 1) * 32;
        const uint4 v0 = ldg_stream(qs), v1 = ldg_stream(qs + 16);
        const uint32_t wv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const uint32_t hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const int sh = (sub & 1) * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t q = ((wv[i] >> (8 * c + sh)) & 0xFu) | (((hv[i] >> (8 * c + sub)) & 1u) << 4);
                f[4 * i + c] = a * (float)q - b;
            }
    }
};

// GGUF Q6_K, device layout: the file's 210-byte super-block (128 bytes of low nibbles, 64 bytes of 2-bit high parts, 16 int8
// scales of 16 weights each, fp16 d) padded to 224 bytes so that every field is 16-byte aligned; values are untouched.
// Element y = 128 h + 32 j + l (h half, j quarter, l 0..31): low nibble of ql[64 h + 32 (j & 1) + l] (high nibble for j >= 2),
// bits 2j, 2j+1 of qh[32 h + l]; w = d * scale[8 h + 2 j + l / 16] * (q - 32).
constexpr int kQ6KDevBlock = 224;
struct WRowQ6K {
    static constexpr int EPL = 32;
    const uint8_t* w;    // row start: K/256 blocks of 224 bytes
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + (size_t)(k >> 8) * kQ6KDevBlock); }
    __device__ __forceinline__ void load(int k, float* f) const {
        const uint8_t* blk = w + (size_t)(k >> 8) * kQ6KDevBlock;
        const int h = (k & 255) >> 7, j = (k & 127) >> 5;
        const uint8_t* ql = blk + h * 64 + (j & 1) * 32;
        const uint8_t* qh = blk + 128 + h * 32;
        const uint4 l0 = ldg_stream(ql), l1 = ldg_stream(ql + 16);
        const uint4 h0 = ldg_stream(qh), h1 = ldg_stream(qh + 16);
        const uint4 tail = __ldg(reinterpret_cast<const uint4*>(blk + 192));              // 16 int8 scales
        const __half dh = __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(blk + 208)));
        const float d = __half2float(dh);
        const uint32_t scw[4] = {tail.x, tail.y, tail.z, tail.w};
        const int si = h * 8 + j * 2;
        const float s0 = d * (float)(int8_t)((scw[si >> 2] >> (8 * (si & 3))) & 0xffu);
        const float s1 = d * (float)(int8_t)((scw[(si + 1) >> 2] >> (8 * ((si + 1) & 3))) & 0xffu);
        const uint32_t lv[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const uint32_t hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const int nsh = (j >> 1) * 4, hsh = j * 2;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int q = (int)(((lv[i] >> (8 * c + nsh)) & 0xFu) | (((hv[i] >> (8 * c + hsh)) & 3u) << 4)) - 32;
                f[4 * i + c] = (i < 4 ? s0 : s1) * (float)q;
            }
    }
};

// GGUF Q8_0, device layout per row: K int8 quants, then K/32 fp16 block scales (the file interleaves a scale in front of every
// 32 quants, which leaves the quants 2-byte aligned; values are untouched).  K % 32 == 0, row pitch K + K/16.
struct WRowQ80 {
    static constexpr int EPL = 32;
    const uint8_t* w;    // row start
    int K;
    __device__ __forceinline__ void prefetch(int k) const { prefetch_l2(w + k); }
    __device__ __forceinline__ void load(int k, float* f) const {
        const uint4 v0 = ldg_stream(w + k), v1 = ldg_stream(w + k + 16);
        const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(w + K) + (k >> 5))));
        const uint32_t wv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) f[4 * i + c] = d * (float)(int8_t)((wv[i] >> (8 * c)) & 0xffu);
    }
};

// ---- fast NVFP4 path -------------------------------------------------------------------
// Two E2M1 values per byte convert to an f16x2 with one cvt instruction; products with fp16
// activations are exact (2 x 8 significant bits), are summed 8 at a time in fp16 and then
// scaled and accumulated in fp32 per 16-element scale group.
__device__ __forceinline__ void fp4x8_to_half2x4(uint32_t v, __half2* h) {
    uint32_t r0, r1, r2, r3;
    asm("{ .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(v));
    h[0] = *reinterpret_cast<__half2*>(&r0); h[1] = *reinterpret_cast<__half2*>(&r1);
    h[2] = *reinterpret_cast<__half2*>(&r2); h[3] = *reinterpret_cast<__half2*>(&r3);
}

// Activation rows staged in shared memory as fp16 in a "part-major" layout so that the 16-byte
// reads of a warp are bank-conflict free: element k lives at ((k%32)/8 * nchunks + k/32)*8 + k%8.
__device__ __forceinline__ int xs_index(int k, int nchunks) { return (((k & 31) >> 3) * nchunks + (k >> 5)) * 8 + (k & 7); }

// Stage `nrows` bf16 rows (gathered through row pointers) of length K into xs[m][K] (fp16).
__device__ __forceinline__ void stage_x_half(__half* xs, const bf16* const* rows, int nrows, int K) {
    const int nchunks = K >> 5;
    for (int m = 0; m < nrows; ++m) {
        const bf16* src = rows[m];
        for (int k8 = threadIdx.x; k8 < (K >> 3); k8 += blockDim.x) {
            float f[8];
            unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(src + k8 * 8)), f);
            __half2 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            const int k = k8 * 8;
            *reinterpret_cast<uint4*>(xs + (size_t)m * K + xs_index(k, nchunks)) = *reinterpret_cast<uint4*>(h);
        }
    }
}

// One 32-element chunk (16 bytes of fp4, two scale groups) of one weight row against MT staged rows.
template <int MT>
__device__ __forceinline__ void nvfp4_chunk_dot(const uint4& v, float s0, float s1, const __half* xs, int K, int nchunks, int c, int nvalid,
                                                float* acc) {
    __half2 w[16];
    fp4x8_to_half2x4(v.x, w); fp4x8_to_half2x4(v.y, w + 4); fp4x8_to_half2x4(v.z, w + 8); fp4x8_to_half2x4(v.w, w + 12);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        if (m < nvalid) {
            const __half* xb = xs + (size_t)m * K + c * 8;
            __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
            for (int part = 0; part < 4; ++part) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xb + (size_t)part * nchunks * 8);
                const __half2* x2 = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (part < 2) a0 = __hfma2(w[part * 4 + i], x2[i], a0);
                    else a1 = __hfma2(w[part * 4 + i], x2[i], a1);
                }
            }
            const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
            acc[m] = fmaf(s0, f0.x + f0.y, acc[m]);
            acc[m] = fmaf(s1, f1.x + f1.y, acc[m]);
        }
    }
}

// Full row: weight row pointer (K/2 bytes), scale-atom base, row index n.
template <int MT>
__device__ __forceinline__ void nvfp4_row_dot(const uint8_t* __restrict__ wrow, const uint8_t* __restrict__ sf, int n, int K,
                                              const __half* xs, int nvalid, float* acc) {
    const int lane = threadIdx.x & 31, nchunks = K >> 5, gtiles = ((K >> 4) + 3) >> 2;
    const size_t sf_row = (size_t)(n >> 7) * gtiles * 512 + (n & 31) * 16 + ((n & 127) >> 5) * 4;
#pragma unroll 2
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 v = ldg_stream(wrow + c * 16);
        const int g = c * 2;
        const uint16_t s2 = __ldg(reinterpret_cast<const uint16_t*>(sf + sf_row + (size_t)(g >> 2) * 512 + (g & 3)));
        nvfp4_chunk_dot<MT>(v, fp8e4m3_to_float((uint8_t)(s2 & 0xff)), fp8e4m3_to_float((uint8_t)(s2 >> 8)), xs, K, nchunks, c, nvalid, acc);
    }
}

// Two rows (A, B) in one pass so both rows' loads are in flight together.
template <int MT>
__device__ __forceinline__ void nvfp4_row_dot2(const uint8_t* __restrict__ wa, const uint8_t* __restrict__ sfa, int na,
                                               const uint8_t* __restrict__ wb, const uint8_t* __restrict__ sfb, int nb, int K,
                                               const __half* xs, int nvalid, float* acca, float* accb) {
    const int lane = threadIdx.x & 31, nchunks = K >> 5, gtiles = ((K >> 4) + 3) >> 2;
    const size_t ra = (size_t)(na >> 7) * gtiles * 512 + (na & 31) * 16 + ((na & 127) >> 5) * 4;
    const size_t rb = (size_t)(nb >> 7) * gtiles * 512 + (nb & 31) * 16 + ((nb & 127) >> 5) * 4;
#pragma unroll 2
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 va = ldg_stream(wa + c * 16);
        const uint4 vb = ldg_stream(wb + c * 16);
        const int g = c * 2;
        const size_t go = (size_t)(g >> 2) * 512 + (g & 3);
        const uint16_t sa = __ldg(reinterpret_cast<const uint16_t*>(sfa + ra + go));
        const uint16_t sb = __ldg(reinterpret_cast<const uint16_t*>(sfb + rb + go));
        nvfp4_chunk_dot<MT>(va, fp8e4m3_to_float((uint8_t)(sa & 0xff)), fp8e4m3_to_float((uint8_t)(sa >> 8)), xs, K, nchunks, c, nvalid, acca);
        nvfp4_chunk_dot<MT>(vb, fp8e4m3_to_float((uint8_t)(sb & 0xff)), fp8e4m3_to_float((uint8_t)(sb >> 8)), xs, K, nchunks, c, nvalid, accb);
    }
}

// Same, with the rows' scale bytes pre-staged in shared memory: `sca`/`scb` point at the row's
// first scale pair; K-tile t (64 columns) is `tile_stride` bytes further (stride chosen odd in
// words so a warp's reads are bank-conflict free).
template <int MT>
__device__ __forceinline__ void nvfp4_row_dot2_sm(const uint8_t* __restrict__ wa, const uint8_t* sca, const uint8_t* __restrict__ wb,
                                                  const uint8_t* scb, int tile_stride, int K, const __half* xs, int nvalid,
                                                  float* acca, float* accb) {
    const int lane = threadIdx.x & 31, nchunks = K >> 5;
#pragma unroll 2
    for (int c = lane; c < nchunks; c += 32) {
        const uint4 va = ldg_stream(wa + c * 16);
        const uint4 vb = ldg_stream(wb + c * 16);
        const int so = (c >> 1) * tile_stride + (c & 1) * 2;
        const uint16_t sa = *reinterpret_cast<const uint16_t*>(sca + so);
        const uint16_t sb = *reinterpret_cast<const uint16_t*>(scb + so);
        nvfp4_chunk_dot<MT>(va, fp8e4m3_to_float((uint8_t)(sa & 0xff)), fp8e4m3_to_float((uint8_t)(sa >> 8)), xs, K, nchunks, c, nvalid, acca);
        nvfp4_chunk_dot<MT>(vb, fp8e4m3_to_float((uint8_t)(sb & 0xff)), fp8e4m3_to_float((uint8_t)(sb >> 8)), xs, K, nchunks, c, nvalid, accb);
    }
}

// Cooperative copy of the scale bytes of `rows_per_blk` consecutive n%32 values (all four 32-row
// quads) of one 128-row tile: per K-tile a contiguous run of rows_per_blk*16 bytes.
__device__ __forceinline__ void stage_scales(uint8_t* dst, const uint8_t* __restrict__ sf, int tile_n, int blk, int rows_per_blk, int gtiles,
                                             int tile_stride) {
    const int parts = rows_per_blk;          // 16-byte pieces per K-tile
    for (int idx = threadIdx.x; idx < gtiles * parts; idx += blockDim.x) {
        const int t = idx / parts, part = idx % parts;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(sf + ((size_t)tile_n * gtiles + t) * 512 + (size_t)(blk * rows_per_blk + part) * 16));
        uint32_t* d = reinterpret_cast<uint32_t*>(dst + (size_t)t * tile_stride + part * 16);
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
}

// acc0[m] += sum_k w0[k]*x[m][k], acc1 likewise for w1, over k in [k0, k1).  x is bf16 [MT][ldx].
// Lane `tid` of `nthr` cooperating threads; partial sums stay per-thread (reduce afterwards).
// The weight vectors of UNR iterations (both rows) are requested before any of them is used,
// so each thread keeps 2*UNR 16-byte loads in flight.
template <class WF, int MT, int UNR = 4>
__device__ __forceinline__ void warp_dot2(const WF& w0, const WF& w1, const bf16* __restrict__ x, int ldx, int K,
                                          float* acc0, float* acc1, int tid = -1, int nthr = 32, int k0 = 0, int k1 = -1) {
    constexpr int E = WF::EPL;
    const int lane = tid < 0 ? (threadIdx.x & 31) : tid;
    if (k1 < 0 || k1 > K) k1 = K;
    const int step = nthr * E;
    int k = k0 + lane * E;
    for (; k + (UNR - 1) * step + E <= k1; k += UNR * step) {
        float a[UNR][E], b[UNR][E];
#pragma unroll
        for (int u = 0; u < UNR; ++u) { w0.load(k + u * step, a[u]); w1.load(k + u * step, b[u]); }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const bf16* xp = x + (size_t)m * ldx + k + u * step;
#pragma unroll
                for (int e = 0; e < E; e += 8) {
                    float xf[8];
                    if constexpr (E >= 8) {
                        uint4 xv = __ldg(reinterpret_cast<const uint4*>(xp + e));
                        unpack_bf16x8(xv, xf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) { acc0[m] = fmaf(a[u][e + i], xf[i], acc0[m]); acc1[m] = fmaf(b[u][e + i], xf[i], acc1[m]); }
                    } else {
                        uint2 xv = __ldg(reinterpret_cast<const uint2*>(xp + e));
                        xf[0] = bf16_lo(xv.x); xf[1] = bf16_hi(xv.x); xf[2] = bf16_lo(xv.y); xf[3] = bf16_hi(xv.y);
#pragma unroll
                        for (int i = 0; i < 4; ++i) { acc0[m] = fmaf(a[u][e + i], xf[i], acc0[m]); acc1[m] = fmaf(b[u][e + i], xf[i], acc1[m]); }
                    }
                }
            }
        }
    }
    for (; k + E <= k1; k += step) {
        float a[E], b[E];
        w0.load(k, a);
        w1.load(k, b);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const bf16* xp = x + (size_t)m * ldx + k;
#pragma unroll
            for (int e = 0; e < E; e += 8) {
                float xf[8];
                if constexpr (E >= 8) {
                    uint4 xv = __ldg(reinterpret_cast<const uint4*>(xp + e));
                    unpack_bf16x8(xv, xf);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { acc0[m] = fmaf(a[e + i], xf[i], acc0[m]); acc1[m] = fmaf(b[e + i], xf[i], acc1[m]); }
                } else {
                    uint2 xv = __ldg(reinterpret_cast<const uint2*>(xp + e));
                    xf[0] = bf16_lo(xv.x); xf[1] = bf16_hi(xv.x); xf[2] = bf16_lo(xv.y); xf[3] = bf16_hi(xv.y);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { acc0[m] = fmaf(a[e + i], xf[i], acc0[m]); acc1[m] = fmaf(b[e + i], xf[i], acc1[m]); }
                }
            }
        }
    }
}

}  // namespace lsb
