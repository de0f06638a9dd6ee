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

struct WRowBf16 {
    static constexpr int EPL = 8;
    const bf16* w;
    __device__ __forceinline__ void load(int k, float* f) const {
        uint4 v = ldg_stream(w + k);
        unpack_bf16x8(v, f);
    }
};

struct WRowF32 {
    static constexpr int EPL = 4;
    const float* w;
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

// acc0[m] += sum_k w0[k]*x[m][k], acc1 likewise for w1.  x is bf16 [MT][ldx].
// Partial sums stay per-lane; call warp_sum on them afterwards.
template <class WF, int MT>
__device__ __forceinline__ void warp_dot2(const WF& w0, const WF& w1, const bf16* __restrict__ x, int ldx, int K,
                                          float* acc0, float* acc1) {
    constexpr int E = WF::EPL;
    const int lane = threadIdx.x & 31;
#pragma unroll 2
    for (int k = lane * E; k + E <= K; k += 32 * E) {
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
                    for (int i = 0; i < 8; ++i) {
                        acc0[m] = fmaf(a[e + i], xf[i], acc0[m]);
                        acc1[m] = fmaf(b[e + i], xf[i], acc1[m]);
                    }
                } else {
                    uint2 xv = __ldg(reinterpret_cast<const uint2*>(xp + e));
                    xf[0] = bf16_lo(xv.x); xf[1] = bf16_hi(xv.x); xf[2] = bf16_lo(xv.y); xf[3] = bf16_hi(xv.y);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc0[m] = fmaf(a[e + i], xf[i], acc0[m]);
                        acc1[m] = fmaf(b[e + i], xf[i], acc1[m]);
                    }
                }
            }
        }
    }
}

}  // namespace lsb
