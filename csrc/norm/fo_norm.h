// Host launchers of the row kernels (RMSNorm, un-reorder + RMSNorm, reorder / un-reorder).
// Reference counterparts: reorder_rmsnorm / rmsnorm host wrappers, src/rmsnorm/rmsnorm.cu:14-45.
#pragma once
#include <cuda_runtime.h>

namespace fo {

// Y[rows, dim] = RMSNorm(X[rows, dim]) * W[dim]; 16-bit storage (bf16 or fp16), fp32 math.
cudaError_t rmsnorm_launch(const void* X, void* Y, const void* W, int rows, int dim, float eps,
                           bool bf16, int sm_count, cudaStream_t stream);

// X holds the logical [rows, dim] matrix as BM x BN tiles, tile t stored at position RA[t]
// (rldn tiles side by side per reordered row); Y is row-major.
cudaError_t reorder_rmsnorm_launch(const void* X, void* Y, const void* W, int rows, int dim, int BM,
                                   int BN, int rldn, const int* RA, float eps, bool bf16,
                                   int sm_count, cudaStream_t stream);

// to_reordered: Y(tile-contiguous) = X(row-major); otherwise the inverse.
cudaError_t reorder_launch(const void* X, void* Y, int rows, int dim, int BM, int BN, int rldn,
                           const int* RA, bool to_reordered, int sm_count, cudaStream_t stream);

}  // namespace fo
