// Entry points of liblsb200_kernels.so that never allocate memory.
//
// This header has no counterpart in the reference engine; it exists for embedders of this
// library that are not allowed to call cudaMalloc (or any allocating routine) where the kernel
// runs - for example code executing while the device memory pool is frozen, or a host
// application that hands out every device byte itself.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Row-wise argmax of fp32 logits [rows, ld] over the first V columns, ties to the lower index.
//   out_ids[r] = base + argmax, out_val[r] = the maximum (out_val may be null).
// Same kernels and same results as lsb_argmax, but the per-block partial results are kept in a
// fixed 128 KiB array inside the library instead of a caller-provided buffer.
//
//  * rows must not exceed lsb_argmax_noalloc_max_rows() (256); more rows return -2 and nothing
//    is launched.  -1 = bad argument (null pointer, rows or V <= 0, ld < V), -3 = the current device
//    index is beyond the 64 devices this entry point keeps an address for, > 0 = a CUDA error
//    code, 0 = launched.
//  * The first call on each device looks up the array's device address (with that device
//    current).  Make that first call before any CUDA stream capture begins.
//  * All calls on a device share the one array.  Two calls whose kernels can overlap on the GPU
//    (different streams without ordering between them) race on it; serialise them.
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
int lsb_argmax_noalloc(const float* logits, int ld, int rows, int V, int* out_ids, float* out_val, int base, void* stream);
int lsb_argmax_noalloc_max_rows(void);

#ifdef __cplusplus
}
#endif
