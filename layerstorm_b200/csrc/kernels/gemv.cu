// Dense weight-streaming GEMV / skinny GEMM for decode-shaped work (M <= 4 rows per
// pass): out[m][n] = sum_k x[m][k] * W[n][k].  A warp owns (a K slice of) two weight rows, so
// every weight byte is read exactly once per pass and the kernel runs at HBM speed.
// Replaces the reference's CUDA-core GEMV family (src/compute/kernels/sm120/gemm/bf16_gemm.cu:41-156,
// wq_gemm.cu:84-158) with one templated kernel over four weight formats.
#include <cstdlib>
#include <type_traits>
#include "gemv_core.cuh"
#include "tc_common.cuh"
#include "comm.cuh"

namespace lsb {

struct MatBf16 {
    const bf16* w; int ldw;
    __device__ __forceinline__ WRowBf16 row(int n) const { return WRowBf16{w + (size_t)n * ldw}; }
};
struct MatF32 {
    const float* w; int ldw;
    __device__ __forceinline__ WRowF32 row(int n) const { return WRowF32{w + (size_t)n * ldw}; }
};
struct MatFp8B {
    const uint8_t* w; int ldw; const float* scales; int kblocks;
    __device__ __forceinline__ WRowFp8B row(int n) const {
        return WRowFp8B{w + (size_t)n * ldw, scales + (size_t)(n >> 7) * kblocks};
    }
};
struct MatQ4K {
    const uint8_t* w; int K;
    __device__ __forceinline__ WRowQ4K row(int n) const { return WRowQ4K{w + (size_t)n * (K >> 8) * 144}; }
};
struct MatQ5K {
    const uint8_t* w; int K;
    __device__ __forceinline__ WRowQ5K row(int n) const { return WRowQ5K{w + (size_t)n * (K >> 8) * 176}; }
};
struct MatQ6K {
    const uint8_t* w; int K;
    __device__ __forceinline__ WRowQ6K row(int n) const { return WRowQ6K{w + (size_t)n * (K >> 8) * kQ6KDevBlock}; }
};
struct MatQ80 {
    const uint8_t* w; int K;
    __device__ __forceinline__ WRowQ80 row(int n) const { return WRowQ80{w + (size_t)n * (K + (K >> 4)), K}; }
};
struct MatNvfp4 {
    const uint8_t* w; int K; const uint8_t* sf; int gtiles;
    __device__ __forceinline__ WRowNvfp4 row(int n) const {
        return WRowNvfp4{w + (size_t)n * (K >> 1), sf, n, gtiles};
    }
};

// One block = 8 warps = (8 / KS) pairs of weight rows x KS slices of K.  KS = 1 streams whole
// rows per warp (large N); larger KS splits K across warps so that matrices with few rows still
// put enough warps - and enough bytes in flight - on every SM.  Slice partials are combined
// through shared memory in slice order, so the result is deterministic.
template <class Mat, int MT, bool OUT_BF16, int KS>
__global__ void __launch_bounds__(256) gemv_kernel(Mat mat, const bf16* __restrict__ x, int ldx, void* __restrict__ out,
                                                   int ldo, int N, int K, float alpha, const float* __restrict__ bias, PeerComm comm) {
    __shared__ float red[8][2 * MT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int PAIRS = 8 / KS;
    const int pair = warp / KS, ks = warp % KS;
    int n0 = (blockIdx.x * PAIRS + pair) * 2;
    const bool active = n0 < N;
    if (!active) n0 = 0;
    const int n1 = min(n0 + 1, N - 1);
    using Row = decltype(mat.row(0));
    constexpr int E = Row::EPL;
    const int kper = ((K + KS - 1) / KS + 32 * E - 1) / (32 * E) * (32 * E);
    const int k0 = ks * kper, k1 = min(K, k0 + kper);
    float acc0[MT], acc1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc0[m] = acc1[m] = 0.f;
    auto r0 = mat.row(n0);
    auto r1 = mat.row(n1);
    if (active) {   // weights do not depend on the previous kernel: pull the head of both rows into L2 while it finishes
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int k = k0 + (lane + 32 * it) * E;
            if (k + E <= k1) { r0.prefetch(k); r1.prefetch(k); }
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    unsigned next_epoch = 0;
    if (comm.nranks) next_epoch = *comm.epoch + 1;
    constexpr int UNR = E <= 8 ? (MT == 1 ? 4 : 2) : (E == 16 ? (MT == 1 ? 2 : 1) : 1);
    if (active) warp_dot2<Row, MT, UNR>(r0, r1, x, ldx, K, acc0, acc1, lane, 32, k0, k1);
    float va[MT], vb[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) { va[m] = warp_sum(acc0[m]); vb[m] = warp_sum(acc1[m]); }
    if (KS > 1) {
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) { red[warp][2 * m] = va[m]; red[warp][2 * m + 1] = vb[m]; }
        }
        __syncthreads();
        if (ks == 0 && lane == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float a = 0.f, b2 = 0.f;
#pragma unroll
                for (int j = 0; j < KS; ++j) { a += red[pair * KS + j][2 * m]; b2 += red[pair * KS + j][2 * m + 1]; }
                va[m] = a; vb[m] = b2;
            }
        }
    }
    if (lane == 0 && ks == 0 && active) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float a = va[m] * alpha, b2 = vb[m] * alpha;
            if (bias) { a += bias[n0]; b2 += bias[n1]; }
            if (OUT_BF16 && !comm.nranks) {
                bf16* o = reinterpret_cast<bf16*>(out) + (size_t)m * ldo;
                o[n0] = __float2bfloat16(a);
                if (n0 + 1 < N) o[n0 + 1] = __float2bfloat16(b2);
            } else {
                float* o = reinterpret_cast<float*>(out) + (size_t)m * ldo;
                o[n0] = a;
                if (n0 + 1 < N) o[n0 + 1] = b2;
            }
        }
    }
    // cross-rank reduction: the partial is in local memory now; the last block ships it to the peers
    if (comm.nranks) comm_finish_local(comm, next_epoch, gridDim.x, reinterpret_cast<const float*>(out), MT, N, ldo);
}

// A bf16 weight-row slice that a bulk copy has placed in shared memory; `w + k` addresses column k of the row.
struct WRowBf16S {
    static constexpr int EPL = 8;
    const bf16* w;
    __device__ __forceinline__ void load(int k, float* f) const {
        const uint4 v = tc::ld_shared_16((uint32_t)__cvta_generic_to_shared(w + k));
        unpack_bf16x8(v, f);
    }
};

static __device__ int g_gemv_err = 0;      // first bulk-copy wait that ran out (0 = none); read through lsb_gemv_error

// bf16 weights, same work split as gemv_kernel, but every warp asks the copy engine for its two row slices (<= 4 KB each) with
// one bulk copy per row BEFORE the dependency wait and computes out of shared memory.  Blocks that become resident under the
// predecessor's tail therefore hold their weights on chip when the activations arrive, and a resident block keeps
// 8 x 8 KB of the stream in flight without spending registers on it.
template <int MT, bool OUT_BF16, int KS>
__global__ void __launch_bounds__(256) gemv_bf16_bulk_kernel(MatBf16 mat, const bf16* __restrict__ x, int ldx, void* __restrict__ out,
                                                             int ldo, int N, int K, int kper, float alpha, const float* __restrict__ bias,
                                                             PeerComm comm) {
    __shared__ float red[8][2 * MT];
    __shared__ __align__(8) uint64_t bars[8];
    extern __shared__ __align__(128) uint8_t slices[];       // [8 warps][2 rows][kper] bf16
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int PAIRS = 8 / KS;
    const int pair = warp / KS, ks = warp % KS;
    int n0 = (blockIdx.x * PAIRS + pair) * 2;
    const bool active = n0 < N;
    if (!active) n0 = 0;
    const int n1 = min(n0 + 1, N - 1);
    const int k0 = ks * kper, k1 = min(K, k0 + kper);
    const bool work = active && k0 < k1;
    bf16* s0 = reinterpret_cast<bf16*>(slices) + (size_t)warp * 2 * kper;
    bf16* s1 = s0 + kper;
    if (work && lane == 0) {
        const uint32_t bytes = (uint32_t)(k1 - k0) * 2u;
        tc::mbar_init(&bars[warp], 1);
        tc::fence_barrier_init();
        tc::mbar_expect_tx(&bars[warp], 2u * bytes);
        tc::bulk_load_1d(s0, mat.w + (size_t)n0 * mat.ldw + k0, bytes, &bars[warp]);
        tc::bulk_load_1d(s1, mat.w + (size_t)n1 * mat.ldw + k0, bytes, &bars[warp]);
    }
    __syncwarp();
    pdl_wait();
    pdl_launch_dependents();
    unsigned next_epoch = 0;
    if (comm.nranks) next_epoch = *comm.epoch + 1;
    float acc0[MT], acc1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc0[m] = acc1[m] = 0.f;
    if (work) {
        // the copies always complete (static, valid weights); the bounded wait only guards against a protocol error
        if (!tc::mbar_wait(&bars[warp], 0, &g_gemv_err, 1)) tc::mbar_wait(&bars[warp], 0, &g_gemv_err, 2);
        constexpr int UNR = MT == 1 ? 4 : 2;
        warp_dot2<WRowBf16S, MT, UNR>(WRowBf16S{s0 - k0}, WRowBf16S{s1 - k0}, x, ldx, K, acc0, acc1, lane, 32, k0, k1);
    }
    float va[MT], vb[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) { va[m] = warp_sum(acc0[m]); vb[m] = warp_sum(acc1[m]); }
    if (KS > 1) {
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) { red[warp][2 * m] = va[m]; red[warp][2 * m + 1] = vb[m]; }
        }
        __syncthreads();
        if (ks == 0 && lane == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float a = 0.f, b2 = 0.f;
#pragma unroll
                for (int j = 0; j < KS; ++j) { a += red[pair * KS + j][2 * m]; b2 += red[pair * KS + j][2 * m + 1]; }
                va[m] = a; vb[m] = b2;
            }
        }
    }
    if (lane == 0 && ks == 0 && active) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float a = va[m] * alpha, b2 = vb[m] * alpha;
            if (bias) { a += bias[n0]; b2 += bias[n1]; }
            if (OUT_BF16 && !comm.nranks) {
                bf16* o = reinterpret_cast<bf16*>(out) + (size_t)m * ldo;
                o[n0] = __float2bfloat16(a);
                if (n0 + 1 < N) o[n0 + 1] = __float2bfloat16(b2);
            } else {
                float* o = reinterpret_cast<float*>(out) + (size_t)m * ldo;
                o[n0] = a;
                if (n0 + 1 < N) o[n0 + 1] = b2;
            }
        }
    }
    if (comm.nranks) comm_finish_local(comm, next_epoch, gridDim.x, reinterpret_cast<const float*>(out), MT, N, ldo);
}

template <int MT, bool OB, int KS>
static void launch_bulk_one(MatBf16 mat, const bf16* xp, int ldx, void* op, int ldo, int N, int K, int kper, float alpha, const float* bias,
                            PeerComm comm, cudaStream_t st) {
    const int rows_per_block = (8 / KS) * 2;
    static bool once = false;
    if (!once) {
        cudaFuncSetAttribute(gemv_bf16_bulk_kernel<MT, OB, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        cudaFuncSetAttribute(gemv_bf16_bulk_kernel<MT, OB, KS>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        once = true;
    }
    // LSB_GEMV_BULK_PAD_KB: extra shared memory requested by the 64 KB variant, to keep it two blocks deep per SM so that a
    // follower which stages ~70 KB itself can become resident under this kernel's tail.  Default 0: measured on the
    // GLM-5.3-Flash decode step, two blocks per SM cost the GEMVs more (130 us per step) than the KDA step gained.
    static const int pad_kb = [] { const char* e = getenv("LSB_GEMV_BULK_PAD_KB"); return e ? atoi(e) : 0; }();
    size_t smem = (size_t)16 * kper * 2;
    if (smem >= 64 * 1024) smem += (size_t)pad_kb * 1024;
    launch_pdl((gemv_bf16_bulk_kernel<MT, OB, KS>), (N + rows_per_block - 1) / rows_per_block, 256, smem, st, mat, xp, ldx, op, ldo,
               N, K, kper, alpha, bias, comm);
}

template <int MT, bool OB>
static void launch_bulk_ks(int ks, MatBf16 mat, const bf16* xp, int ldx, void* op, int ldo, int N, int K, int kper, float alpha, const float* bias,
                           PeerComm comm, cudaStream_t st) {
    if (ks == 1) launch_bulk_one<MT, OB, 1>(mat, xp, ldx, op, ldo, N, K, kper, alpha, bias, comm, st);
    else if (ks == 2) launch_bulk_one<MT, OB, 2>(mat, xp, ldx, op, ldo, N, K, kper, alpha, bias, comm, st);
    else if (ks == 4) launch_bulk_one<MT, OB, 4>(mat, xp, ldx, op, ldo, N, K, kper, alpha, bias, comm, st);
    else launch_bulk_one<MT, OB, 8>(mat, xp, ldx, op, ldo, N, K, kper, alpha, bias, comm, st);
}

// LSB_GEMV_BULK=0: bf16 GEMVs keep the register-streaming kernel
static bool gemv_bulk_enabled() {
    static const bool b = [] { const char* e = getenv("LSB_GEMV_BULK"); return e ? atoi(e) != 0 : true; }();
    return b;
}

template <class Mat, int MT, bool OB, int KS>
static void launch_one(Mat mat, const bf16* xp, int ldx, void* op, int ldo, int N, int K, float alpha, const float* bias, PeerComm comm,
                       cudaStream_t st) {
    const int rows_per_block = (8 / KS) * 2;
    // The kernel streams its weights past L1 (no-allocate loads) and keeps only the activation row there, so it asks for the
    // largest shared-memory carve-out: a following kernel that stages tens of KB in shared memory (the KDA step) can then become
    // resident on an SM that still runs the tail of this one (measured: KDA step 14.4 -> 9.6 us).  LSB_GEMV_CARVEOUT=-1: leave the default.
    static bool once = false;
    if (!once) {
        static const int carve = [] { const char* e = getenv("LSB_GEMV_CARVEOUT"); return e ? atoi(e) : 100; }();
        if (carve >= 0) cudaFuncSetAttribute(gemv_kernel<Mat, MT, OB, KS>, cudaFuncAttributePreferredSharedMemoryCarveout, carve);
        once = true;
    }
    launch_pdl((gemv_kernel<Mat, MT, OB, KS>), (N + rows_per_block - 1) / rows_per_block, 256, 0, st, mat, xp, ldx, op, ldo, N, K, alpha, bias, comm);
}

template <class Mat, int MT, bool OB>
static void launch_ks(int ks, Mat mat, const bf16* xp, int ldx, void* op, int ldo, int N, int K, float alpha, const float* bias, PeerComm comm,
                      cudaStream_t st) {
    if (ks == 1) launch_one<Mat, MT, OB, 1>(mat, xp, ldx, op, ldo, N, K, alpha, bias, comm, st);
    else if (ks == 2) launch_one<Mat, MT, OB, 2>(mat, xp, ldx, op, ldo, N, K, alpha, bias, comm, st);
    else if (ks == 4) launch_one<Mat, MT, OB, 4>(mat, xp, ldx, op, ldo, N, K, alpha, bias, comm, st);
    else launch_one<Mat, MT, OB, 8>(mat, xp, ldx, op, ldo, N, K, alpha, bias, comm, st);
}

// K-split so that the grid is at least ~two full waves (148 SMs x 8 resident blocks) while every
// slice still has a few 32-lane iterations.
static int choose_ks(int N, int K, int epl) {
    int ks = 1;
    while (ks < 8 && (long long)((N + 1) / 2) * ks / 8 < 2368 && K / (ks * 2) >= 32 * epl * 2) ks *= 2;
    return ks;
}

template <class Mat>
static int launch_gemv(Mat mat, const bf16* x, int ldx, void* out, int ldo, int M, int N, int K, float alpha,
                       const float* bias, int out_bf16, cudaStream_t st, const void* comm_host = nullptr) {
    PeerComm comm;
    comm.nranks = 0;
    if (comm_host) {
        comm = *reinterpret_cast<const PeerComm*>(comm_host);
        if ((M != 1 && M != 2 && M != 4) || out_bf16) return -1;   // the fused epilogue covers one single-pass launch of fp32 rows
    }
    const size_t osz = out_bf16 ? 2 : 4;
    int ks = choose_ks(N, K, decltype(mat.row(0))::EPL);
    int bulk_kper = 0;
    if constexpr (std::is_same<Mat, MatBf16>::value) {
        // bulk-copy variant: a warp's row slice must fit 4 KB of shared memory; split K further when it does not
        if (gemv_bulk_enabled() && K % 8 == 0 && mat.ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(mat.w) & 15) == 0) {
            int kb = ks;
            while (kb < 8 && (K + kb - 1) / kb > 2048) kb *= 2;
            const int kper = ((K + kb - 1) / kb + 255) / 256 * 256;
            if (kper <= 2048) { ks = kb; bulk_kper = kper; }
        }
    }
    for (int m0 = 0; m0 < M;) {
        const int rem = M - m0;
        const int mt = rem >= 4 ? 4 : (rem >= 2 ? 2 : 1);
        const bf16* xp = x + (size_t)m0 * ldx;
        void* op = reinterpret_cast<char*>(out) + (size_t)m0 * ldo * osz;
#define LSB_GEMV_CASE(MT_)                                                                              \
    if constexpr (std::is_same<Mat, MatBf16>::value) {                                                  \
        if (bulk_kper) {                                                                                \
            if (out_bf16) launch_bulk_ks<MT_, true>(ks, mat, xp, ldx, op, ldo, N, K, bulk_kper, alpha, bias, comm, st);  \
            else launch_bulk_ks<MT_, false>(ks, mat, xp, ldx, op, ldo, N, K, bulk_kper, alpha, bias, comm, st);          \
            m0 += mt;                                                                                   \
            continue;                                                                                   \
        }                                                                                               \
    }                                                                                                   \
    if (out_bf16) launch_ks<Mat, MT_, true>(ks, mat, xp, ldx, op, ldo, N, K, alpha, bias, comm, st);  \
    else launch_ks<Mat, MT_, false>(ks, mat, xp, ldx, op, ldo, N, K, alpha, bias, comm, st);
        if (mt == 4) { LSB_GEMV_CASE(4) } else if (mt == 2) { LSB_GEMV_CASE(2) } else { LSB_GEMV_CASE(1) }
#undef LSB_GEMV_CASE
        m0 += mt;
    }
    return (int)cudaGetLastError();
}

}  // namespace lsb

using namespace lsb;

// First bulk-copy wait of the bf16 GEMV that gave up since the library was loaded on the current device (0 = none).
LSB_API int lsb_gemv_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_err, sizeof(v)) != cudaSuccess) return -1;
    return v;
}

// x: bf16 [M, ldx]; W: bf16 [N, ldw]; out fp32 or bf16 [M, ldo]. K % 8 == 0, 16-byte aligned rows.
// comm: host pointer to a PeerComm (fused all-reduce push of the fp32 output) or null.
LSB_API int lsb_gemv_bf16(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx,
                          int ldw, int ldo, float alpha, int out_bf16, const void* comm, void* stream) {
    if (K % 8 || ldw % 8 || ldx % 8) return -1;
    return launch_gemv(MatBf16{(const bf16*)w, ldw}, (const bf16*)x, ldx, out, ldo, M, N, K, alpha, (const float*)bias,
                       out_bf16, (cudaStream_t)stream, comm);
}

namespace lsb {
// Many-row product with fp32 weights (router logits of a prefill chunk): out[m][n] = alpha * sum_k x[m][k] * W[n][k] + bias[n].
// 64 x 64 output tile per block, 4 x 4 outputs per thread, K in steps of 16 through shared memory; fp32 FMAs in a fixed
// k order (the routing decision must not depend on the launch shape).
__global__ void __launch_bounds__(256) sgemm_f32w_kernel(void* __restrict__ out, const bf16* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ bias, int M, int N, int K, int ldx, int ldw, int ldo,
                                                         float alpha, int out_bf16) {
    __shared__ float xs[16][64 + 4], ws[16][64 + 4];
    pdl_wait();
    pdl_launch_dependents();
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64, t = threadIdx.x;
    const int tm = (t >> 4) * 4, tn = (t & 15) * 4;
    const int lr = t >> 2, lk = (t & 3) * 4;                 // loader: row lr (0..63), 4 consecutive k
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        {
            const int m = m0 + lr, n = n0 + lr;
            float xv[4] = {0, 0, 0, 0}, wv[4] = {0, 0, 0, 0};
            if (m < M && k0 + lk < K) {
                const uint2 u = *reinterpret_cast<const uint2*>(x + (size_t)m * ldx + k0 + lk);
                xv[0] = bf16_lo(u.x); xv[1] = bf16_hi(u.x); xv[2] = bf16_lo(u.y); xv[3] = bf16_hi(u.y);
            }
            if (n < N && k0 + lk < K) {
                const float4 f = *reinterpret_cast<const float4*>(w + (size_t)n * ldw + k0 + lk);
                wv[0] = f.x; wv[1] = f.y; wv[2] = f.z; wv[3] = f.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) { xs[lk + i][lr] = xv[i]; ws[lk + i][lr] = wv[i]; }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[k][tm]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[k][tn]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            const float v = acc[i][j] * alpha + (bias ? bias[n] : 0.f);
            if (out_bf16) reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16(v);
            else reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v;
        }
    }
    pdl_launch_dependents();
}
}  // namespace lsb

// W: fp32 [N, ldw] (router / hyper-connection mixing matrices). K % 4 == 0.
LSB_API int lsb_gemv_f32w(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx,
                          int ldw, int ldo, float alpha, int out_bf16, void* stream) {
    if (K % 4 || ldw % 4 || ldx % 4) return -1;
    // The tiled SGEMM pays off from about a hundred rows; below that (decode batches, verify steps) its grid is a handful of
    // blocks (5 blocks for 288 router rows and 32 tokens: 378 us measured), while passes of the weight-streaming kernel over
    // four rows at a time keep the whole GPU busy (about 3 us per pass).
    if (M >= 128) {
        launch_pdl((sgemm_f32w_kernel), dim3((N + 63) / 64, (M + 63) / 64), 256, 0, (cudaStream_t)stream, out, (const bf16*)x, (const float*)w,
                   (const float*)bias, M, N, K, ldx, ldw, ldo, alpha, out_bf16);
        LSB_CHECK_LAUNCH();
    }
    return launch_gemv(MatF32{(const float*)w, ldw}, (const bf16*)x, ldx, out, ldo, M, N, K, alpha, (const float*)bias,
                       out_bf16, (cudaStream_t)stream);
}

// W: e4m3 [N, K] with fp32 scales [ceil(N/128), ceil(K/128)] (128x128 blocks). K % 16 == 0.
LSB_API int lsb_gemv_fp8b(void* out, const void* x, const void* w, const void* scales, const void* bias, int M, int N,
                          int K, int ldx, int ldo, float alpha, int out_bf16, const void* comm, void* stream) {
    if (K % 16 || ldx % 8) return -1;
    return launch_gemv(MatFp8B{(const uint8_t*)w, K, (const float*)scales, (K + 127) / 128}, (const bf16*)x, ldx, out,
                       ldo, M, N, K, alpha, (const float*)bias, out_bf16, (cudaStream_t)stream, comm);
}

// W: packed E2M1 [N, K/2] + e4m3 group scales in the 128x4 atom layout; alpha carries the
// per-tensor scale (weight_scale_2). K % 32 == 0.
LSB_API int lsb_gemv_nvfp4(void* out, const void* x, const void* w, const void* sf, const void* bias, int M, int N,
                           int K, int ldx, int ldo, float alpha, int out_bf16, const void* comm, void* stream) {
    if (K % 32 || ldx % 8) return -1;
    const int G = K / 16;
    return launch_gemv(MatNvfp4{(const uint8_t*)w, K, (const uint8_t*)sf, (G + 3) / 4}, (const bf16*)x, ldx, out, ldo,
                       M, N, K, alpha, (const float*)bias, out_bf16, (cudaStream_t)stream, comm);
}

// W: GGUF Q4_K blocks, [N] rows of K/256 x 144 bytes.  K % 256 == 0.
LSB_API int lsb_gemv_q4k(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx, int ldo, float alpha,
                         int out_bf16, const void* comm, void* stream) {
    if (K % 256 || ldx % 8) return -1;
    return launch_gemv(MatQ4K{(const uint8_t*)w, K}, (const bf16*)x, ldx, out, ldo, M, N, K, alpha, (const float*)bias, out_bf16,
                       (cudaStream_t)stream, comm);
}

// out[n][k] = bf16(W[n][k]) for a GGUF block-type matrix in its device layout: one thread per 32 consecutive elements.
template <class Mat>
__global__ void __launch_bounds__(256) gguf_dequant_bf16_kernel(Mat mat, bf16* __restrict__ out, int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.y;
    const int k = (blockIdx.x * blockDim.x + threadIdx.x) * 32;
    if (n >= N || k >= K) return;
    float f[32];
    mat.row(n).load(k, f);
    bf16* o = out + (size_t)n * K + k;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        __nv_bfloat162 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[i + 2 * j], f[i + 2 * j + 1]);
        *reinterpret_cast<uint4*>(o + i) = *reinterpret_cast<uint4*>(h);
    }
}

LSB_API int lsb_gguf_dequant_bf16(void* out, const void* w, int ggml_type, int N, int K, void* stream) {
    if (K % 256 || ((uintptr_t)w & 15) || ((uintptr_t)out & 15)) return -1;
    dim3 grid((K / 32 + 255) / 256, N);
    cudaStream_t st = (cudaStream_t)stream;
    switch (ggml_type) {
        case 12: launch_pdl((gguf_dequant_bf16_kernel<MatQ4K>), grid, 256, 0, st, MatQ4K{(const uint8_t*)w, K}, (bf16*)out, N, K); break;
        case 13: launch_pdl((gguf_dequant_bf16_kernel<MatQ5K>), grid, 256, 0, st, MatQ5K{(const uint8_t*)w, K}, (bf16*)out, N, K); break;
        case 14: launch_pdl((gguf_dequant_bf16_kernel<MatQ6K>), grid, 256, 0, st, MatQ6K{(const uint8_t*)w, K}, (bf16*)out, N, K); break;
        case 8: launch_pdl((gguf_dequant_bf16_kernel<MatQ80>), grid, 256, 0, st, MatQ80{(const uint8_t*)w, K}, (bf16*)out, N, K); break;
        default: return -1;
    }
    LSB_CHECK_LAUNCH();
}

// W: another GGUF block type in its device layout (see gemv_core.cuh): ggml_type 13 = Q5_K (176-byte blocks as in the file),
// 14 = Q6_K (blocks padded to 224 bytes), 8 = Q8_0 (per row: K quants, then K/32 fp16 scales).  K % 256 == 0.
LSB_API int lsb_gemv_gguf(void* out, const void* x, const void* w, int ggml_type, const void* bias, int M, int N, int K, int ldx, int ldo,
                          float alpha, int out_bf16, const void* comm, void* stream) {
    if (K % 256 || ldx % 8 || ((uintptr_t)w & 15)) return -1;
    const bf16* xb = (const bf16*)x;
    const float* bs = (const float*)bias;
    cudaStream_t st = (cudaStream_t)stream;
    switch (ggml_type) {
        case 12: return launch_gemv(MatQ4K{(const uint8_t*)w, K}, xb, ldx, out, ldo, M, N, K, alpha, bs, out_bf16, st, comm);
        case 13: return launch_gemv(MatQ5K{(const uint8_t*)w, K}, xb, ldx, out, ldo, M, N, K, alpha, bs, out_bf16, st, comm);
        case 14: return launch_gemv(MatQ6K{(const uint8_t*)w, K}, xb, ldx, out, ldo, M, N, K, alpha, bs, out_bf16, st, comm);
        case 8: return launch_gemv(MatQ80{(const uint8_t*)w, K}, xb, ldx, out, ldo, M, N, K, alpha, bs, out_bf16, st, comm);
    }
    return -1;
}

LSB_API int lsb_trace_set_gemv(void* buf) { return lsb_trace_install(buf); }
