// Byte layout of one expert slot in the expert arena, shared by the weight-streaming MoE kernels
// (moe.cu) and the tensor-core grouped GEMM (moe_tc.cu).  Mirrors the ctypes structure of the same
// name on the Python side.
#pragma once

namespace lsb {

struct ExpertFmt {
    int fmt;                 // 0 bf16, 1 fp8 block-128, 2 nvfp4, 3 GGUF Q4_K
    int H, F;                // hidden, expert intermediate
    long long stride;        // bytes between slots
    long long off_gate, off_up, off_down;        // weights
    long long off_sg, off_su, off_sd;            // scales (fp8: fp32 block scales; nvfp4: atoms)
    long long off_tail;                           // nvfp4: 3 fp32 per-tensor scales (gate, up, down)
};

}  // namespace lsb
