// A linear-layer entry point for callers that must not allocate device memory.
// (This entry point has no counterpart in the reference project.)
//
// Who needs it: code that is loaded into a process whose device memory is already
// spoken for -- a serving engine that has handed every free byte to its KV cache,
// or a host application with its own pool -- so that a cudaMalloc made on its
// behalf could fail, or would stall all streams while the driver synchronises;
// and plain C callers that have no tensor library to allocate with.
//
// ab200_linear_bf16 (api.h) asks its caller for an fp32 scratch buffer in which
// the split-K partial sums of small-batch GEMMs are kept. This variant brings its
// own: a fixed array that lives inside the library image
// (AB200_NOALLOC_SCRATCH_BYTES, held by every GPU that loads the library until
// the process exits). Inputs and the output are still the caller's.
//
//   * Nothing is allocated or freed, on the device or through any library.
//   * Problems whose worst-case scratch need exceeds the array are refused with
//     AB200_ERR_SCRATCH_TOO_SMALL before anything is launched;
//     ab200_linear_bf16_noalloc_fits() tells in advance, and
//     ab200_noalloc_last_error() returns a readable reason for the last refusal
//     on the calling thread.
//   * The first call on each device looks up the array's device address (once per
//     device, with that device current). Make that first call before any stream
//     capture begins on the device.
//   * All calls on one device share the array and it keeps whatever the last call
//     left in it. Nothing in it has to start at zero: every element that is read
//     is written first by the same call. Two calls whose kernels may overlap on
//     the GPU (different streams without an ordering between them) race on it.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AB200_NOALLOC_SCRATCH_BYTES (32u << 20)
#define AB200_ERR_SCRATCH_TOO_SMALL (-6)
#define AB200_ERR_SYMBOL_LOOKUP (-7)

// 1 if (M, N, K) can be served from the built-in scratch array, else 0.
int ab200_linear_bf16_noalloc_fits(int M, int N, int K);

// Same contract as ab200_linear_bf16 without the workspace arguments:
// out[M,N] = act(x[M,K] * w[N,K]^T + bias) + residual, bf16 in and out.
int ab200_linear_bf16_noalloc(const void* x, long long ldx, const void* w, long long ldw,
                              void* out, long long ldo, int M, int N, int K, const void* bias,
                              const void* residual, long long ldr, int act, int force_splits,
                              int* status, cudaStream_t stream);

const char* ab200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
