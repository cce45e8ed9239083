// fl_gemm_tc_static_scratch: the split-K tensor-core product for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in codemk8/fastllm-py; it exists for
// users of this library only.
//
// Who needs it.  fl_gemm_tc splits K over several CTAs when a product has too
// few output tiles to occupy the GPU, and the partial sums pass through a float
// workspace that the CALLER allocates and hands in.  Some callers have no way to
// get such a buffer: a host program that has already given all of the device's
// memory to a pool of its own (a later cudaMalloc would fail, or would have to
// be carved out of that pool by code that knows nothing of this library); a
// plug-in that runs under a rule that forbids the CUDA allocation calls; a loop
// that must not stall, for which cudaMalloc and cudaFree are unusable because
// they synchronise the whole device.  For them the workspace lives inside the
// library: a file-scope `static __device__` array of
// FL_TC_STATIC_SCRATCH_FLOATS floats (8 MiB), which every GPU that loads the
// library holds from load until the process exits.  Inputs and the output are
// still the caller's.
//
// What it does.  The same kernels as fl_gemm_tc, with the partial sums in that
// array.  It calls no cudaMalloc, no cudaFree and no allocating library routine.
//
// Set-up.  The first call on a device looks up the array's device address (with
// that device current) and keeps it; make that first call outside any stream
// capture, once per device, before relying on later calls.  The address is kept
// in a plain table without a lock: the first call on a device must not run at
// the same time as another call on that device from a second host thread.
//
// Limits.  A problem fits when splits * M * round_up(N, 4) <=
// FL_TC_STATIC_SCRATCH_FLOATS.  Anything larger is refused: the function
// returns FL_TC_ERR_SCRATCH_TOO_SMALL, launches nothing, and writes a sentence
// with both numbers into `error_text` when that is not null.
//
// Sharing.  Every call on a device uses the same array, and the array keeps
// what the last call left in it.  Nothing has to start at zero: each split
// writes every partial sum before the reduction reads it.  Two calls that may
// run on the GPU at the same time (different streams, no ordering between them)
// race on the array and give wrong results; order them, or use fl_gemm_tc with
// separate workspaces.
#pragma once

#include <cuda_runtime.h>

#define FL_TC_STATIC_SCRATCH_FLOATS (1l << 21)
#define FL_TC_ERR_SCRATCH_TOO_SMALL (-2)
#define FL_TC_ERR_BAD_DEVICE (-3)

#ifdef __cplusplus
extern "C" {
#endif

// C[M, N] = A[M, K] * W[N, K]^T; A and W bfloat16 (row pitches lda, ldw multiples
// of 8 elements, bases 16-byte aligned), C bfloat16 (c_dtype 1) or float (0).
// bn / splits: the token-tile width and the number of K splits as fl_gemm_tc takes
// them; bn = 0 lets the library choose both (fl_gemm_tc_plan), and a given bn
// needs splits >= 1 (anything else returns cudaErrorInvalidValue).  status: a device int that receives a
// code if a bounded wait inside the kernel gives up.  Returns 0 when launched, a
// cudaError_t value when a CUDA call failed, or one of the FL_TC_ERR_* codes.
int fl_gemm_tc_static_scratch(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype,
                              long ldc, int M, int N, int K, int bn, int splits, int num_sms,
                              int* status, cudaStream_t stream, char* error_text,
                              int error_text_bytes);

#ifdef __cplusplus
}
#endif
