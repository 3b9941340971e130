// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in smallbard/kapel: it exists for users of this library whose code
// runs where cudaMalloc is off limits. Two examples: a plugin inside a host application that
// owns the whole device heap and hands the plugin fixed input and output buffers only, and
// code that runs inside a region (a recorded stream, a real-time loop) in which a call that
// may synchronise the device, as an allocation may, is not allowed. Such callers can still
// multiply a few rows of bfloat16 activations by a weight matrix, the product that decoding
// spends its time in, through the function below. It is implemented at the end of
// gemm_bf16.cu.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// The most float32 values of scratch one call may need: 4 Mi values (16 MiB). The array of
// this size is part of the library's image, so every GPU that loads the library holds it
// until the process exits.
#define KB_NO_ALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

// c[m, n] = a[m, k] . w[n, k]^T for m <= 64, with the same kernels, the same split of K and
// therefore the same bits as kb_gemm_bf16, but with the split-K partial sums kept in a scratch
// array that is built into the library instead of in memory the caller allocates.
//
//   c         bfloat16 or float32 (c_dt: 1 or 0), written in full
//   a, w      bfloat16, 16-byte aligned, k a multiple of 8
//   epilogue  0: none; 1: cap * tanh(x / cap)
//   stream    a cudaStream_t
//
// Returns 0, or 1 after storing a message for kb_last_error(). It refuses, without launching
// anything, m > 64 and any product whose partial sums (splits x m x n values; see
// kb_gemm_bf16_scratch_floats) exceed KB_NO_ALLOC_SCRATCH_FLOATS.
//
// It calls no cudaMalloc, cudaFree or any other allocating routine. The first call on a device
// looks up the device address of the built-in array (cudaGetSymbolAddress) and keeps it; make
// that first call before any stream capture begins. Every call on a device shares the one
// array: the kernels overwrite every value they later read, so nothing left by an earlier call
// is ever used, but two calls that overlap on the GPU (different streams, no ordering between
// them) race on it. Order them, or use kb_gemm_bf16 with scratch of your own for one of them.
int kb_gemm_bf16_no_alloc(void* c, int c_dt, const void* a, const void* w, int m, int n, int k, int epilogue,
                          float cap, void* stream);

#ifdef __cplusplus
}
#endif
