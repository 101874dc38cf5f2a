// Allocation-free C entry point of the bf16 tensor-core GEMM.
//
// This entry point has no counterpart in the reference framework (which ships no
// native code); it exists for callers of this library that must not allocate
// device memory when they call into it:
//   * code running while a CUDA memory pool is frozen or owned by someone else
//     (an inference server that pre-partitioned the whole device, a plugin that
//     is handed raw pointers by a host application);
//   * real-time / latency-critical loops where cudaMalloc's implicit device
//     synchronisation is unacceptable;
//   * C or other non-PyTorch hosts that have no caching allocator to ask.
// The regular entry point (gemm_bf16_nt, PyTorch binding) obtains its output and
// its split-K workspace from the PyTorch allocator; this one takes the output
// buffer from the caller and keeps the split-K partial sums in a fixed array that
// lives in the library image.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem accepted: the split-K planes must fit in the built-in scratch
// array, i.e.  splits * M * N <= CLB200_NOALLOC_SCRATCH_FLOATS  with splits >= 2.
// The array (16 MiB) is part of the loaded library on every GPU that uses it and
// stays resident until the process exits.
#define CLB200_NOALLOC_SCRATCH_FLOATS (4ll << 20)

// C[M,N] = A[M,K] * B[N,K]^T, bf16 inputs, fp32 accumulation.
//   a, b      device pointers, 16-byte aligned, K contiguous; lda/ldb = row strides in
//             elements (multiples of 8); K a multiple of 8; N a multiple of 8
//   c         device pointer to M*N outputs (row stride N): bf16, or fp32 if out_fp32
//   stream    cudaStream_t to launch on (0 = default stream)
// Returns 0 on success, non-zero on rejection or launch failure; the reason is
// available from clb200_gemm_noalloc_last_error() (thread-local string).
//
// * Calls no cudaMalloc / cudaFree / allocating library routine.
// * The FIRST call on each device performs a one-time set-up with that device
//   current (it resolves the device address of the scratch array and raises the
//   kernel's dynamic shared-memory limit).  Make that first call before any stream
//   capture begins.  Host threads that make their first call at the same time are
//   safe: the set-up runs once per device and the others wait for it.
// * All calls share one scratch array per device.  Its contents are overwritten by
//   every call (each k-slice rewrites its whole plane, so nothing needs clearing),
//   which means two calls that overlap on the GPU - different streams, or different
//   host threads - race on it.  Serialise calls per device.
int clb200_gemm_bf16_nt_noalloc(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb,
                                int out_fp32, void* stream);

const char* clb200_gemm_noalloc_last_error(void);

// A return value of 0 above means "launched".  The kernel itself never spins without a
// limit: if one of its internal waits runs out (about two seconds) it records a code,
// leaves the output unfinished and returns.  This function reads that code for the
// current device and clears it: 0 = every GEMM since the last read completed, 1 / 2 / 3 =
// the load, tensor-core or store stage gave up, -1 = the code could not be read.  It
// synchronises the device, so call it after the work you care about, not inside a
// latency-critical loop.  The code is shared with the regular entry point.
int clb200_gemm_noalloc_device_status(void);

#ifdef __cplusplus
}
#endif
