// Shared device helpers for every kernel in this directory (sm_100a only).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <utility>

#define LSB_API extern "C" __attribute__((visibility("default")))

#define LSB_CHECK_LAUNCH()                       \
    do {                                         \
        cudaError_t e__ = cudaGetLastError();    \
        return (int)e__;                         \
    } while (0)

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

namespace lsb {

constexpr int kWarp = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; `red` must hold >= 33 floats. Result broadcast to all threads.
// The reduction order is fixed (warp tree, then warp 0 over warp partials), so the
// result does not depend on scheduling.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// 8 bf16 (one 16-byte vector) -> 8 floats
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float* f) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
    f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
    f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

__device__ __forceinline__ float fp8e4m3_to_float(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}
// 4 packed e4m3 -> 4 floats
__device__ __forceinline__ void unpack_fp8x4(uint32_t v, float* f) {
    __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffffu), __NV_E4M3);
    __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3);
    float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
    float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint8_t float_to_fp8e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// E2M1 (FP4) magnitude table: index = low 3 bits, bit 3 = sign.
__device__ __forceinline__ float fp4_to_float(uint32_t nib) {
    // values {0, .5, 1, 1.5, 2, 3, 4, 6}
    const uint32_t m = nib & 7u;
    float v = (m < 2u) ? 0.5f * (float)m : ((m & 1u) ? 1.5f : 1.0f) * (float)(1u << ((m >> 1) - 1u));
    return (nib & 8u) ? -v : v;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }

// 128-bit streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// Programmatic dependent launch: let the next kernel's prologue start early, and
// wait for the previous kernel's memory before touching its outputs.
// Optional step trace: when a trace buffer is installed (lsb_trace_set_* of every translation unit, see utils/step_trace.py), thread 0
// of block (0,0,0) of EVERY kernel records the time it reached its dependency wait and the time the wait returned - the moment the
// previous kernel in the stream has completed.  Consecutive "wait returned" stamps are the critical path of a step kernel by kernel,
// measured inside the CUDA graph with programmatic dependent launch active.  buf[0] = records so far, buf[1] = capacity, then 4
// words per record: t_reached_wait, t_wait_returned, gridDim.x | gridDim.y << 32, blockDim.x | gridDim.z << 32.
static __device__ unsigned long long* lsb_trace_buf = nullptr;

__device__ __forceinline__ void pdl_wait() {
    unsigned long long* tb = nullptr;
    unsigned long long t0 = 0;
    if ((blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x | threadIdx.y) == 0) {
        tb = lsb_trace_buf;
        if (tb) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tb) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        const unsigned long long i = atomicAdd(tb, 1ull);
        if (i < tb[1]) {
            unsigned long long* r = tb + 2 + 4 * i;
            r[0] = t0; r[1] = t1;
            r[2] = (unsigned long long)gridDim.x | ((unsigned long long)gridDim.y << 32);
            r[3] = (unsigned long long)blockDim.x | ((unsigned long long)gridDim.z << 32);
        }
    }
}
// Installs the trace buffer of this translation unit (every .cu file exports one setter built from this).
static inline int lsb_trace_install(void* buf) {
    unsigned long long* p = reinterpret_cast<unsigned long long*>(buf);
    return (int)cudaMemcpyToSymbol(lsb_trace_buf, &p, sizeof(p));
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Kernel launch with programmatic dependent launch: the kernel may become resident while its
// predecessor in the stream is still running and executes everything up to its
// griddepcontrol.wait (weight prefetch, barrier set-up) under the predecessor's tail.  Every
// kernel in this library reads its predecessor's output only after pdl_wait() and performs no
// global store before it, which is what makes the early start safe.
inline int& pdl_enabled_flag() { static int v = 1; return v; }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled_flag() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace lsb
