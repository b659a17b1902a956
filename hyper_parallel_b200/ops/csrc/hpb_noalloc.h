// Entry points of libhpb200.so that allocate no device memory.
//
// This header has no counterpart in the reference project (which contains no CUDA code at
// all); it exists for embedders of this library whose host process may not allocate on the
// GPU once it is running -- for example a serving or RL process that has given all of HBM
// to its own memory pool, so that a cudaMalloc issued by a library would fail or
// synchronise the device.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Negative return codes of the entry points below (positive values are cudaError_t).
#define HPB_NOALLOC_E_TOO_LARGE (-100)   // H above hpb_noalloc_max_h()
#define HPB_NOALLOC_E_BAD_SHAPE (-101)   // H not a positive multiple of 8, or T < 0
#define HPB_NOALLOC_E_DEVICE (-102)      // current device unknown, or its index is 64 or more
#define HPB_NOALLOC_E_SYMBOL (-103)      // the device address of the scratch array could not be resolved

#ifdef __cplusplus
extern "C" {
#endif

// RMSNorm backward, same math and argument meaning as hpb_rmsnorm_bwd(), but the fp32
// scratch for the partial weight gradients is a fixed 4 MiB array inside the library
// instead of a caller buffer:
//   dx[T,H]  = rstd * (dy * w) - x * rstd^3 / H * sum(dy * w * x)   (+ dres_in when given)
//   dw[H]    (+)= sum_t dy[t] * x[t] * rstd[t]      (bf16, or fp32 when dw_f32 != 0)
// dy, x, w, dres_in (may be NULL), dx are bf16; rstd is fp32 [T].
//
// * H must be a multiple of 8 and at most hpb_noalloc_max_h() (8192); larger H returns
//   HPB_NOALLOC_E_TOO_LARGE (-100).  Use hpb_noalloc_strerror() for a message.
// * Calls no cudaMalloc / cudaFree.  The first call on a device resolves the array's device
//   address with cudaGetSymbolAddress; make it before any stream capture starts.
// * All calls on a device share the array; calls that overlap on the GPU race.  Nothing in
//   the array needs clearing between calls.
// Returns 0, a negative HPB_NOALLOC_E_* code, or a positive cudaError_t from the launch.
int hpb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                            const void* dres_in, void* dx, void* dw, int dw_f32, int dw_accumulate,
                            int64_t T, int H, cudaStream_t stream);

int hpb_noalloc_max_h(void);
const char* hpb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
