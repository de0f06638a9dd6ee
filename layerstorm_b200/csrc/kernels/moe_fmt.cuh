// Byte layout of one expert slot in the expert arena, shared by the weight-streaming MoE kernels
// (moe.cu) and the tensor-core grouped GEMM (moe_tc.cu).  Mirrors the ctypes structure of the same
// name on the Python side.
#pragma once

namespace lsb {

struct ExpertFmt {
    int fmt;                 // gate / up: 0 bf16, 1 fp8 block-128, 2 nvfp4, 3 GGUF Q4_K, 4 Q5_K, 5 Q6_K (224-byte blocks), 6 Q8_0 (planar rows)
    int H, F;                // hidden, expert intermediate
    long long stride;        // bytes between slots
    long long off_gate, off_up, off_down;        // weights
    long long off_sg, off_su, off_sd;            // scales (fp8: fp32 block scales; nvfp4: atoms)
    long long off_tail;                           // nvfp4: 3 fp32 per-tensor scales (gate, up, down)
    int fmt_down1;                                // format of the down matrix + 1 when it differs from `fmt` (GGUF files mix block
                                                  // types per tensor), 0 = same as `fmt`
    __host__ __device__ int down_fmt() const { return fmt_down1 ? fmt_down1 - 1 : fmt; }
};

}  // namespace lsb
