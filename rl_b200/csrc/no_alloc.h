// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (NVIDIA-NeMo/RL ships no native code); it exists for users of
// this library.
//
// Who needs it. Some hosts of this library own all device memory themselves: a serving process that sized its KV cache
// from "whatever is free", or a runtime that reserved one arena at start-up and hands out slices of it. In such a
// process a cudaMalloc issued on the library's behalf can fail although the caller budgeted correctly, and it also
// synchronises the device, which a latency-critical step cannot afford. The regular entry point, rlb_rmsnorm_bwd,
// asks the caller for a scratch buffer (the per-CTA partial sums of the weight gradient), which in practice means an
// allocation per call. rlb_rmsnorm_bwd_static needs none: its scratch lives in a fixed array inside the library image.
//
// Cost and limits.
//  * Every GPU that loads the library holds the array (RLB_RMSNORM_STATIC_MAX_PARTS x RLB_RMSNORM_STATIC_MAX_D floats,
//    about 9.7 MB) from load until the process exits, whether or not this entry point is ever called.
//  * d must be a multiple of 8 and at most RLB_RMSNORM_STATIC_MAX_D; larger shapes are refused with
//    RLB_STATIC_ERR_TOO_LARGE (nothing is launched). rlb_rmsnorm_bwd_static_strerror turns a code into text.
//  * dy, x, w and dx must be non-null and 16-byte aligned, the strides multiples of 8 and at least d, rows below 2^31,
//    rstd and dw_f32 non-null fp32 pointers: anything else returns RLB_STATIC_ERR_BAD_SHAPE and launches nothing.
//  * The first call on each device looks up the array's device address (with that device current). Make that first
//    call from ordinary, non-capturing code before any stream capture is started on the device.
//  * All calls share the one array and it keeps the previous call's contents. Each call overwrites every element it
//    later reads, so nothing has to be cleared; but two calls whose kernels can overlap on the GPU (different streams,
//    or different host threads on one device) race on it. Serialise them on one stream.
//  * No cudaMalloc, cudaFree or allocating library routine is called, here or in the kernels.
//
// Arguments are those of rlb_rmsnorm_bwd without the scratch pointer: dy, x, w are bf16; rstd is the per-row
// reciprocal RMS saved by the forward pass; dx receives the input gradient (bf16, rows x d, dense); dw_f32 receives
// (dw_accumulate == 0) or accumulates (!= 0) the weight gradient in fp32. Strides are in elements.
// Returns 0 on success, a positive CUDA error code, or a negative RLB_STATIC_ERR_* code.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RLB_RMSNORM_STATIC_MAX_D 8192
#define RLB_RMSNORM_STATIC_MAX_PARTS 296

#define RLB_STATIC_ERR_BAD_SHAPE (-2)   /* d, a stride or a pointer breaks the 16-byte alignment rule */
#define RLB_STATIC_ERR_TOO_LARGE (-5)   /* d exceeds RLB_RMSNORM_STATIC_MAX_D */
#define RLB_STATIC_ERR_NO_SYMBOL (-6)   /* the scratch array's device address could not be resolved */

int rlb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_f32,
                           int dw_accumulate, long long rows, int d, long long x_stride, long long dy_stride,
                           void* stream);

const char* rlb_rmsnorm_bwd_static_strerror(int code);

#ifdef __cplusplus
}
#endif
