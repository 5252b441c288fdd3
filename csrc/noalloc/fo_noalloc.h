// A C entry point that never allocates device memory.  It has no counterpart in the reference.
//
// Who needs it: code that runs where cudaMalloc / cudaFree are not an option - inside another
// allocator's callback (calling back into the allocator would deadlock or recurse), in a process
// whose device memory has been handed over in full to a serving runtime's own pool, or from a
// plain C host that links this library without PyTorch and its caching allocator.  The fused
// GEMM+collective kernel needs scratch (the per-rank staging buffers its partial tiles are
// pushed into, the arrival counters and the status words); every other entry point takes that
// scratch from cudaMalloc.  This one keeps it in a fixed array inside the library image.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Scratch limits of fo_fused_loopback_noalloc: ranks * M * N * 2 bytes of staging and one
// arrival counter per output tile.
#define FO_NOALLOC_MAX_STAGING_BYTES (16u << 20)
#define FO_NOALLOC_MAX_TILES 4096
#define FO_NOALLOC_MAX_RANKS 4

// Runs all `ranks` ranks of the fused GEMM + all-reduce (comm_op 0) or GEMM + reduce-scatter
// (comm_op 1) on the current device in one cooperative launch - the single-GPU emulation that
// torch.ops.flashoverlap_op.fused_loopback offers - without allocating anything.
//
//   A, B, out   host arrays of `ranks` device pointers: A[r] is [M,K], B[r] is [N,K] (16-bit,
//               row-major), out[r] is [M,N] (all-reduce) or [M/ranks,N] (reduce-scatter), all
//               row-major; the caller owns them.
//   bf16        1: bfloat16, 0: float16.      algo: a single-CTA Algo index ((Algo & 1) == 0).
//   M, N, K     positive; M a multiple of 128, N of the Algo's tile width, K of 8.
//   strided_rows 1: rank r owns rows i with i % ranks == r, 0: contiguous blocks per tile.
//
// Returns 0 on success, a positive device status code (fo_status.h) if a bounded device wait
// gave up, a negative value for a rejected argument or a CUDA error; `err` (may be NULL)
// receives a message.  Sizes beyond the limits above are rejected, never truncated.
//
// The scratch is a file-scope __device__ array of FO_NOALLOC_MAX_STAGING_BYTES + 128 KiB that
// every GPU that loads this library holds until the process exits.  The first call on a device
// looks up its device address (cudaGetSymbolAddress) and raises the kernel's shared-memory
// limit; that first call should come before any stream capture is begun.  All calls share the
// array, which keeps the previous call's contents: each call clears the counters and status
// words it needs (stream-ordered), but two calls that overlap on the GPU - different streams,
// different host threads - race on it.  The function is synchronous: it reads the status words
// back and waits for its own work (cudaStreamSynchronize on `stream`) before it returns.
int fo_fused_loopback_noalloc(int comm_op, int ranks, const void* const* A, const void* const* B,
                              void* const* out, int M, int N, int K, int bf16, int algo,
                              int strided_rows, cudaStream_t stream, char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
