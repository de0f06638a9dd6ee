// Tensor-core GEMM for sm_100a: Y[m][n] = sum_k X[m][k] * W[n][k]  (both operands K-major).
//
// The weight matrix is the 128-row UMMA "A" operand and the activations are the "B" operand
// (swap-AB), so any token count from 16 to thousands maps onto full 128-row tcgen05.mma
// instructions: N_umma = the token tile (16..256).  One CTA computes one [128 x BN] output
// tile (optionally one K split of it):
//     warp 0   one thread issues TMA tile loads (cp.async.bulk.tensor, 128-byte swizzle) into a
//              multi-stage shared-memory ring, completion on mbarriers
//     warp 1   allocates tensor memory; one thread issues tcgen05.mma (kind::f16, fp32 accumulate
//              in TMEM) and tcgen05.commit to release stages / publish the accumulator
//     warps 2-5 epilogue: tcgen05.ld the accumulator (one TMEM lane = one output column n),
//              optional bias, fp32 or bf16 store, coalesced over n
// This replaces the reference's CUDA-core tiled GEMM (src/compute/kernels/sm120/gemm/bf16_gemm.cu:156)
// and the external FP8 GEMM launcher (G/sm120/gemm/fp8/fp8_gemm.h) for every M > 4.
#include "tc_common.cuh"
#include "comm.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace lsb {
using namespace tc;

constexpr int BM = 128;   // weight rows per tile (UMMA M)
constexpr int BK = 64;    // bf16 elements per stage row = 128 bytes = one swizzle span

struct GemmTcParams {
    void* out; int ldo;            // [M, ldo] fp32 or bf16
    float* partial;                // [splits, M, N] fp32 when splits > 1
    const float* bias;             // [N] or null
    int M, N, K, out_bf16, splits, kb_per_split;
    int* err;
    long long out_bs;              // batched mode: elements between consecutive batches of `out` (blockIdx.z = batch)
    // fused all-reduce epilogue (row-parallel layers under tensor parallelism): instead of a local store, every tile of
    // the fp32 partial is stored into this rank's slot of every peer's receive buffer over NVLink; the last CTA
    // publishes the epoch.  The consuming kernel sums the slots in rank order.
    PeerComm comm;
};

template <int BN> struct TcCfg {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool BATCHED = false>
__global__ void __launch_bounds__(192) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmTcParams p) {
    using C = TcCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // token-row tiles are the fastest grid dimension: the blocks that share a weight tile run together, so the weight
    // matrix streams from DRAM once and the (much smaller) activation tiles stay in L2
    const int n0 = blockIdx.y * BM, m0 = blockIdx.x * BN;
    const int split = BATCHED ? 0 : blockIdx.z, batch = BATCHED ? blockIdx.z : 0;
    const int nkb_total = (p.K + BK - 1) / BK;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(nkb_total, kb0 + p.kb_per_split);
    const int nkb = max(0, kb1 - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_x);
    }
    if (warp == 1) tmem_alloc(tmem_holder, C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_holder;
    pdl_wait();
    pdl_launch_dependents();
    const unsigned next_epoch = p.comm.nranks ? *p.comm.epoch + 1u : 0u;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        int issued = 0;
        bool ok = true;
        for (int it = 0; it < nkb && ok; ++it) {
            const int s = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1;
            ok = mbar_wait(&empty[s], ph ^ 1, p.err, 1);
            if (!ok) break;
            uint8_t* a = smem + s * C::STAGE_BYTES;
            mbar_expect_tx(&full[s], C::STAGE_BYTES);
            if (BATCHED) {
                tma_load_3d(a, &map_w, &full[s], (kb0 + it) * BK, n0, batch);
                tma_load_3d(a + C::A_BYTES, &map_x, &full[s], (kb0 + it) * BK, m0, batch);
            } else {
                tma_load_2d(a, &map_w, &full[s], (kb0 + it) * BK, n0);
                tma_load_2d(a + C::A_BYTES, &map_x, &full[s], (kb0 + it) * BK, m0);
            }
            ++issued;
        }
        if (!ok) {
            // error path: let the loads already in flight land before this CTA's shared memory is released
            for (int it = max(0, issued - C::STAGES); it < issued; ++it) mbar_wait(&full[it % C::STAGES], (it / C::STAGES) & 1, nullptr, 0);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t idesc = idesc_f16(BM, BN, 1);
        bool ok = true;
        for (int it = 0; it < nkb; ++it) {
            const int s = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1;
            ok = mbar_wait(&full[s], ph, p.err, 2);
            if (!ok) break;
            tc_fence_after();
            const uint8_t* a = smem + s * C::STAGE_BYTES;
            const uint64_t da = smem_desc_sw128(a), db = smem_desc_sw128(a + C::A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) umma_f16(tmem_d, da + 2 * k, db + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
            umma_commit(&empty[s]);
        }
        if (ok) umma_commit(acc_full);
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        const int q = warp & 3;
        const int n = n0 + q * 32 + lane;
        bool ok = nkb > 0 ? mbar_wait(acc_full, 0, p.err, 3) : true;
        tc_fence_after();
        if (ok) {
            const float b = (p.bias && n < p.N && p.splits == 1) ? p.bias[n] : 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                if (nkb > 0) tmem_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.f;
                }
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c0 + j;
                        if (m < p.M) {
                            if (p.comm.nranks) comm_push(p.comm, next_epoch, (size_t)m * p.ldo + n, v[j]);
                            else if (p.splits > 1) p.partial[((size_t)split * p.M + m) * p.N + n] = v[j];
                            else if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[(size_t)batch * p.out_bs + (size_t)m * p.ldo + n] = __float2bfloat16(v[j] + b);
                            else reinterpret_cast<float*>(p.out)[(size_t)batch * p.out_bs + (size_t)m * p.ldo + n] = v[j] + b;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_d, C::TMEM_COLS);
    if (p.comm.nranks) comm_signal(p.comm, next_epoch, gridDim.x * gridDim.y * gridDim.z);
    pdl_launch_dependents();
}

// Sum K-split partials in split order (deterministic), add bias, convert.
__global__ void splitk_reduce_kernel(void* __restrict__ out, int ldo, const float* __restrict__ partial, const float* __restrict__ bias,
                                     int M, int N, int splits, int out_bf16) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (n >= N) return;
    float a = 0.f;
    for (int s = 0; s < splits; ++s) a += partial[((size_t)s * M + m) * N + n];
    if (bias) a += bias[n];
    if (out_bf16) reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16(a);
    else reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = a;
    pdl_launch_dependents();
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)f;
    }
    return fn;
}

// 2-D row-major tensor [rows, cols] of `esize`-byte elements, box [box_rows, box_cols], 128B swizzle.
int make_map_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, int esize, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return -2;
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstr[1] = {ld_elems * (uint64_t)esize};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D view [batch][rows][cols] with element strides (batch_stride, ld, 1); box [1][box_rows][box_cols].
int make_map_3d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, int esize, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                uint64_t batch, uint64_t batch_stride_elems, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return -2;
    cuuint64_t gdim[3] = {cols, rows, batch};
    cuuint64_t gstr[2] = {ld_elems * (uint64_t)esize, batch_stride_elems * (uint64_t)esize};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, dt, 3, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D byte view [slot][row][byte] of quantised weight matrices that sit at the same offset in every slot of an arena
// (strides: slot_stride, pitch, 1 bytes); box [1][box_rows][box_bytes] with the swizzle mode that matches box_bytes
// (32, 64 or 128), so that a thread reading its own row of the box hits every bank once.
int make_map_bytes_3d(CUtensorMap* map, const void* ptr, uint64_t pitch, uint64_t rows, uint64_t slot_stride, uint64_t nslots,
                      uint32_t box_bytes, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return -2;
    if (((uintptr_t)ptr & 15) || (pitch & 15) || (slot_stride & 15)) return -4;
    cuuint64_t gdim[3] = {pitch, rows, nslots};
    cuuint64_t gstr[2] = {pitch, slot_stride};
    cuuint32_t box[3] = {box_bytes, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -3;
}

struct MapKey {
    const void* p; uint64_t rows, cols, ld; uint32_t br, bc; int dt;
    bool operator<(const MapKey& o) const { return std::tie(p, rows, cols, ld, br, bc, dt) < std::tie(o.p, o.rows, o.cols, o.ld, o.br, o.bc, o.dt); }
};
static std::map<MapKey, CUtensorMap> g_maps;
static std::mutex g_maps_mu;

int cached_map_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, int esize, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t br, uint32_t bc) {
    std::lock_guard<std::mutex> g(g_maps_mu);
    MapKey k{ptr, rows, cols, ld, br, bc, (int)dt};
    auto it = g_maps.find(k);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    CUtensorMap m;
    int rc = make_map_2d(&m, ptr, dt, esize, rows, cols, ld, br, bc);
    if (rc) return rc;
    if (g_maps.size() > 65536) g_maps.clear();
    g_maps[k] = m;
    *out = m;
    return 0;
}

template <int BN>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcParams& p, cudaStream_t st) {
    using C = TcCfg<BN>;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM); attr = true; }
    dim3 grid((p.M + BN - 1) / BN, (p.N + BM - 1) / BM, p.splits);
    launch_pdl((gemm_tc_kernel<BN>), grid, 192, C::SMEM, st, mw, mx, p);
    return (int)cudaGetLastError();
}

template <int BN>
static int launch_tc_batched(const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcParams& p, int batch, cudaStream_t st) {
    using C = TcCfg<BN>;
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(gemm_tc_kernel<BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM); attr = true; }
    dim3 grid((p.M + BN - 1) / BN, (p.N + BM - 1) / BM, batch);
    launch_pdl((gemm_tc_kernel<BN, true>), grid, 192, C::SMEM, st, mw, mx, p);
    return (int)cudaGetLastError();
}

}  // namespace lsb
using namespace lsb;

// Batched product for b in [0, B): out[b][m][n] = sum_k x[b][m][k] * w[b][n][k] with element strides
// x: (xs_b, ldx, 1), w: (ws_b, ldw, 1), out: (os_b, ldo, 1).  One launch, grid.z = batch.  Strides % 8 == 0.
LSB_API int lsb_gemm_bf16_tc_batched(void* out, const void* x, const void* w, int M, int N, int K, int B, int ldx, long long xs_b, int ldw,
                                     long long ws_b, int ldo, long long os_b, int out_bf16, void* err, void* stream) {
    if (K % 8 || ldx % 8 || ldw % 8 || xs_b % 8 || ws_b % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || B < 1 || B > 65535) return -1;
    int BN = 16;
    while (BN < 256 && BN < M) BN <<= 1;
    static std::map<std::tuple<const void*, int, int, int, long long, int, int>, CUtensorMap> cache;      // per (ptr, rows, cols, ld, batch stride, B, box rows)
    static std::mutex mu;
    auto get = [&](const void* ptr, int rows, int cols, int ld, long long bs, int box_rows, CUtensorMap* o) -> int {
        std::lock_guard<std::mutex> g(mu);
        const auto key = std::make_tuple(ptr, rows, cols, ld, bs, B, box_rows);
        auto it = cache.find(key);
        if (it != cache.end()) { *o = it->second; return 0; }
        CUtensorMap m;
        const int rc = make_map_3d(&m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, cols, ld, B, bs, box_rows, BK);
        if (rc) return rc;
        if (cache.size() > 4096) cache.clear();
        cache[key] = m;
        *o = m;
        return 0;
    };
    CUtensorMap mw, mx;
    int rc = get(w, N, K, ldw, ws_b, BM, &mw);
    if (rc) return rc;
    rc = get(x, M, K, ldx, xs_b, BN, &mx);
    if (rc) return rc;
    GemmTcParams p;
    p.out = out; p.ldo = ldo; p.partial = nullptr; p.bias = nullptr; p.M = M; p.N = N; p.K = K; p.out_bf16 = out_bf16; p.err = (int*)err;
    p.splits = 1; p.kb_per_split = (K + BK - 1) / BK; p.out_bs = os_b; p.comm.nranks = 0;
    cudaStream_t st = (cudaStream_t)stream;
    switch (BN) {
        case 16: return launch_tc_batched<16>(mw, mx, p, B, st);
        case 32: return launch_tc_batched<32>(mw, mx, p, B, st);
        case 64: return launch_tc_batched<64>(mw, mx, p, B, st);
        case 128: return launch_tc_batched<128>(mw, mx, p, B, st);
        default: return launch_tc_batched<256>(mw, mx, p, B, st);
    }
}

LSB_API int lsb_gemm_tc_workspace_floats(int M, int N, int K) {
    // upper bound on split-K partial storage: at most 16 splits
    return 16 * M * N;
}

// x bf16 [M, ldx], w bf16 [N, ldw], out fp32/bf16 [M, ldo]; K % 8 == 0; ldx, ldw % 8 == 0; pointers 16-byte aligned.
// partial: fp32 scratch of partial_cap floats (split-K is limited to what fits) or null to disable split-K.
// err: int error word (0 = ok; 1-3 = a bounded pipeline wait gave up).
LSB_API int lsb_gemm_bf16_tc(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx, int ldw,
                             int ldo, int out_bf16, void* partial, long long partial_cap, void* err, const void* comm, void* stream) {
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return -1;
    if (comm) { partial = nullptr; if (out_bf16 || bias || (long long)M * ldo > ((const PeerComm*)comm)->cap) return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    int BN = 16;
    while (BN < 256 && BN < M) BN <<= 1;
    CUtensorMap mw, mx;
    int rc = cached_map_2d(&mw, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, BM, BK);
    if (rc) return rc;
    rc = cached_map_2d(&mx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, ldx, BN, BK);
    if (rc) return rc;
    GemmTcParams p;
    p.out = out; p.ldo = ldo; p.partial = (float*)partial; p.bias = (const float*)bias; p.M = M; p.N = N; p.K = K;
    p.out_bf16 = out_bf16; p.err = (int*)err; p.out_bs = 0;
    if (comm) p.comm = *(const PeerComm*)comm; else p.comm.nranks = 0;
    const int nkb = (K + BK - 1) / BK;
    const int tiles = ((N + BM - 1) / BM) * ((M + BN - 1) / BN);
    int splits = 1;
    if (partial && tiles < 148) {
        splits = (148 + tiles - 1) / tiles;
        if (splits > 16) splits = 16;
        if (splits > nkb / 4) splits = nkb / 4 > 0 ? nkb / 4 : 1;
        while (splits > 1 && (long long)splits * M * N > partial_cap) --splits;
    }
    p.kb_per_split = (nkb + splits - 1) / splits;
    p.splits = (nkb + p.kb_per_split - 1) / p.kb_per_split;
    switch (BN) {
        case 16: rc = launch_tc<16>(mw, mx, p, st); break;
        case 32: rc = launch_tc<32>(mw, mx, p, st); break;
        case 64: rc = launch_tc<64>(mw, mx, p, st); break;
        case 128: rc = launch_tc<128>(mw, mx, p, st); break;
        default: rc = launch_tc<256>(mw, mx, p, st); break;
    }
    if (rc) return rc;
    if (p.splits > 1) {
        launch_pdl((splitk_reduce_kernel), dim3((N + 255) / 256, M), 256, 0, st, out, ldo, (const float*)partial, (const float*)bias, M, N, p.splits, out_bf16);
        return (int)cudaGetLastError();
    }
    return 0;
}

LSB_API int lsb_trace_set_gemm_tc(void* buf) { return lsb_trace_install(buf); }
