// Memory-bound row kernels: RMSNorm, fused tile-un-reorder + RMSNorm, and the standalone
// row-major <-> tile-contiguous reorder.  Counterparts of the reference's
// reorder_rmsnorm_kernel / rmsnorm_kernel (src/rmsnorm/rmsnorm.cuh:14-117); the standalone
// reorder has no counterpart there (its layout change only ever happens inside the GEMM
// epilogue and the norm kernel).
//
// Differences from the reference kernels, on purpose: eps is an argument (it is hard-coded
// to 1e-5 at src/rmsnorm/rmsnorm.cuh:102), launches take a stream (the reference launches
// on the legacy default stream, src/rmsnorm/rmsnorm.cu:23), bf16 as well as fp16, and each
// thread keeps several 16-byte vectors in flight so that a B200 SM can cover HBM3e latency.
#include "fo_norm.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace fo {

namespace {

constexpr int kNormThreads = 256;

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
}

// y = round16(round16(x * scale) * w): the normalised value is rounded to the storage type
// before the weight multiply, as in the reference (src/rmsnorm/rmsnorm.cuh:108-113) and in
// the usual `norm(x.float()).type_as(x) * weight` module.
template <bool BF16>
__device__ __forceinline__ uint32_t scale_mul2(uint32_t x, uint32_t w, float scale) {
  const float2 xf = unpack2<BF16>(x);
  if constexpr (BF16) {
    __nv_bfloat162 n = __floats2bfloat162_rn(xf.x * scale, xf.y * scale);
    __nv_bfloat162 r = __hmul2(n, *reinterpret_cast<__nv_bfloat162*>(&w));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __half2 n = __floats2half2_rn(xf.x * scale, xf.y * scale);
    __half2 r = __hmul2(n, *reinterpret_cast<__half2*>(&w));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protects `red` against the previous row's readers
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < kNormThreads / 32) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

// Element offset, in the tile-contiguous buffer, of logical (row b, column col).
__device__ __forceinline__ size_t reordered_offset(int b, int col, int dim, int BM, int BN,
                                                   int rldn, const int* __restrict__ RA) {
  const int t = (b / BM) * (dim / BN) + col / BN;
  const int r = RA[t];
  const size_t ld = static_cast<size_t>(rldn) * BN;
  return (static_cast<size_t>(r / rldn) * BM + (b % BM)) * ld + static_cast<size_t>(r % rldn) * BN +
         (col % BN);
}

// Each CTA takes a contiguous block of rows; each thread owns VPT 16-byte vectors of a row
// (VPT * 256 * 8 >= dim).  Two things keep HBM busy: the next row's vectors are requested
// before the current row is reduced (register double buffer), and in the reordered case the
// tile look-up through RA - a dependent load in front of every data load - is done only when
// the block of rows crosses into another row panel, not per row.
template <bool BF16, bool REORDER, int VPT>
__global__ void __launch_bounds__(kNormThreads, (VPT <= 2 ? 6 : (VPT <= 4 ? 4 : 2)))
    rmsnorm_kernel(const uint16_t* __restrict__ X, uint16_t* __restrict__ Y,
                   const uint16_t* __restrict__ W, int rows, int dim, int BM, int BN, int rldn,
                   const int* __restrict__ RA, float eps) {
  __shared__ float red[kNormThreads / 32];
  const int nvec = dim / 8;
  const int per_cta = (rows + gridDim.x - 1) / gridDim.x;
  const int row_begin = blockIdx.x * per_cta;
  const int row_end = min(rows, row_begin + per_cta);
  if (row_begin >= row_end) return;

  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int j = threadIdx.x + i * kNormThreads;
    if (j < nvec) wv[i] = *reinterpret_cast<const uint4*>(W + static_cast<size_t>(j) * 8);
  }

  // Offset, in 16-byte vectors, of (row 0 of the current panel, this thread's column) per vector;
  // 32 bits cover 64 GiB of 16-bit elements.
  uint32_t panel_off[VPT];
  int panel = -1;
  const size_t ld = REORDER ? static_cast<size_t>(rldn) * BN : static_cast<size_t>(dim);
  auto load_row = [&](int b, uint4 (&dst)[VPT]) {
    if constexpr (REORDER) {
      const int pb = b / BM;
      if (pb != panel) {
        panel = pb;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int j = threadIdx.x + i * kNormThreads;
          if (j < nvec)
            panel_off[i] = static_cast<uint32_t>(reordered_offset(pb * BM, j * 8, dim, BM, BN, rldn, RA) >> 3);
        }
      }
      const uint4* row = reinterpret_cast<const uint4*>(X + static_cast<size_t>(b - pb * BM) * ld);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int j = threadIdx.x + i * kNormThreads;
        if (j < nvec) dst[i] = __ldcs(row + panel_off[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int j = threadIdx.x + i * kNormThreads;
        if (j < nvec)
          dst[i] = __ldcs(reinterpret_cast<const uint4*>(X + static_cast<size_t>(b) * dim +
                                                         static_cast<size_t>(j) * 8));
      }
    }
  };

  uint4 cur[VPT], nxt[VPT];
  load_row(row_begin, cur);
  for (int b = row_begin; b < row_end; ++b) {
    if (b + 1 < row_end) load_row(b + 1, nxt);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < nvec) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(&cur[i]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack2<BF16>(u[k]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < nvec) {
        uint4 y;
        y.x = scale_mul2<BF16>(cur[i].x, wv[i].x, scale);
        y.y = scale_mul2<BF16>(cur[i].y, wv[i].y, scale);
        y.z = scale_mul2<BF16>(cur[i].z, wv[i].z, scale);
        y.w = scale_mul2<BF16>(cur[i].w, wv[i].w, scale);
        __stcs(reinterpret_cast<uint4*>(Y + static_cast<size_t>(b) * dim + static_cast<size_t>(j) * 8), y);
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) cur[i] = nxt[i];
  }
}

// TO_REORDERED: Y[reordered] = X[natural]; otherwise Y[natural] = X[reordered].
// Same shape as the norm kernel: each CTA takes a contiguous block of rows, each thread owns VPT
// 16-byte vectors of a row, the tile look-up through RA is done only when the block of rows
// crosses into another row panel, and two rows (2 * VPT vectors per thread) are in flight.
// (The first version walked the vectors with a grid stride and paid a 64-bit division and a
// dependent RA load per vector: 0.66 of the measured copy bandwidth.)
template <bool TO_REORDERED, int VPT>
__global__ void __launch_bounds__(kNormThreads, (VPT <= 2 ? 6 : (VPT <= 4 ? 4 : 2)))
    reorder_kernel(const uint16_t* __restrict__ X, uint16_t* __restrict__ Y, int rows, int dim,
                   int BM, int BN, int rldn, const int* __restrict__ RA) {
  const int nvec = dim / 8;
  const int per_cta = (rows + gridDim.x - 1) / gridDim.x;
  const int row_begin = blockIdx.x * per_cta;
  const int row_end = min(rows, row_begin + per_cta);
  if (row_begin >= row_end) return;
  const uint4* __restrict__ x = reinterpret_cast<const uint4*>(X);
  uint4* __restrict__ y = reinterpret_cast<uint4*>(Y);
  const size_t ldv = static_cast<size_t>(rldn) * BN / 8;  // row pitch of the reordered view, in vectors

  uint32_t panel_off[VPT];  // vector offset of (row 0 of the current panel, this thread's columns)
  int panel = -1;
  auto offsets = [&](int b, size_t (&nat)[VPT], size_t (&reo)[VPT]) {
    const int pb = b / BM;
    if (pb != panel) {
      panel = pb;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int j = threadIdx.x + i * kNormThreads;
        if (j < nvec) panel_off[i] = static_cast<uint32_t>(reordered_offset(pb * BM, j * 8, dim, BM, BN, rldn, RA) >> 3);
      }
    }
    const size_t row_reo = static_cast<size_t>(b - pb * BM) * ldv;
    const size_t row_nat = static_cast<size_t>(b) * nvec;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      nat[i] = row_nat + threadIdx.x + i * kNormThreads;
      reo[i] = row_reo + panel_off[i];
    }
  };

  for (int b = row_begin; b < row_end; b += 2) {
    size_t nat0[VPT], reo0[VPT], nat1[VPT], reo1[VPT];
    uint4 v0[VPT], v1[VPT];
    const bool two = b + 1 < row_end;
    offsets(b, nat0, reo0);
    if (two) offsets(b + 1, nat1, reo1);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (threadIdx.x + i * kNormThreads < nvec) {
        v0[i] = __ldcs(x + (TO_REORDERED ? nat0[i] : reo0[i]));
        if (two) v1[i] = __ldcs(x + (TO_REORDERED ? nat1[i] : reo1[i]));
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (threadIdx.x + i * kNormThreads < nvec) {
        __stcs(y + (TO_REORDERED ? reo0[i] : nat0[i]), v0[i]);
        if (two) __stcs(y + (TO_REORDERED ? reo1[i] : nat1[i]), v1[i]);
      }
    }
  }
}

template <bool BF16, bool REORDER>
cudaError_t launch_norm(const void* X, void* Y, const void* W, int rows, int dim, int BM, int BN,
                        int rldn, const int* RA, float eps, int sm_count, cudaStream_t stream) {
  const int nvec = dim / 8;
  const int vpt = (nvec + kNormThreads - 1) / kNormThreads;
  // contiguous row blocks: enough CTAs to fill the machine several times over, yet a few
  // rows per CTA so that the prefetch and the cached tile look-ups pay off
  int grid = rows < sm_count * 8 ? rows : sm_count * 8;
  if (rows >= sm_count * 32) grid = (rows + 3) / 4 < sm_count * 16 ? (rows + 3) / 4 : sm_count * 16;
  if (grid < 1) grid = 1;
  const uint16_t* x = static_cast<const uint16_t*>(X);
  uint16_t* y = static_cast<uint16_t*>(Y);
  const uint16_t* w = static_cast<const uint16_t*>(W);
#define FO_LAUNCH_NORM(V)                                                                      \
  rmsnorm_kernel<BF16, REORDER, V><<<grid, kNormThreads, 0, stream>>>(x, y, w, rows, dim, BM, BN, \
                                                                       rldn, RA, eps)
  if (vpt <= 1) {
    FO_LAUNCH_NORM(1);
  } else if (vpt <= 2) {
    FO_LAUNCH_NORM(2);
  } else if (vpt <= 4) {
    FO_LAUNCH_NORM(4);
  } else if (vpt <= 8) {
    FO_LAUNCH_NORM(8);
  } else {
    return cudaErrorInvalidValue;  // dim > 16384
  }
#undef FO_LAUNCH_NORM
  return cudaGetLastError();
}

}  // namespace

cudaError_t rmsnorm_launch(const void* X, void* Y, const void* W, int rows, int dim, float eps,
                           bool bf16, int sm_count, cudaStream_t stream) {
  if (dim % 8 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  return bf16 ? launch_norm<true, false>(X, Y, W, rows, dim, 1, 1, 1, nullptr, eps, sm_count, stream)
              : launch_norm<false, false>(X, Y, W, rows, dim, 1, 1, 1, nullptr, eps, sm_count, stream);
}

cudaError_t reorder_rmsnorm_launch(const void* X, void* Y, const void* W, int rows, int dim, int BM,
                                   int BN, int rldn, const int* RA, float eps, bool bf16,
                                   int sm_count, cudaStream_t stream) {
  if (dim % 8 != 0 || BN % 8 != 0 || dim % BN != 0 || rows % BM != 0 || rldn < 1)
    return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  return bf16 ? launch_norm<true, true>(X, Y, W, rows, dim, BM, BN, rldn, RA, eps, sm_count, stream)
              : launch_norm<false, true>(X, Y, W, rows, dim, BM, BN, rldn, RA, eps, sm_count, stream);
}

cudaError_t reorder_launch(const void* X, void* Y, int rows, int dim, int BM, int BN, int rldn,
                           const int* RA, bool to_reordered, int sm_count, cudaStream_t stream) {
  if (dim % 8 != 0 || BN % 8 != 0 || dim % BN != 0 || rows % BM != 0 || rldn < 1)
    return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  const int nvec = dim / 8;
  const int vpt = (nvec + kNormThreads - 1) / kNormThreads;
  // contiguous row blocks, as for the norm kernels: a few rows per CTA so that the cached tile
  // look-ups pay off, enough CTAs to fill the machine several times over
  int grid = rows < sm_count * 8 ? rows : sm_count * 8;
  if (rows >= sm_count * 32) grid = (rows + 3) / 4 < sm_count * 16 ? (rows + 3) / 4 : sm_count * 16;
  if (grid < 1) grid = 1;
  const uint16_t* x = static_cast<const uint16_t*>(X);
  uint16_t* y = static_cast<uint16_t*>(Y);
#define FO_LAUNCH_REORDER(V)                                                                              \
  do {                                                                                                    \
    if (to_reordered) {                                                                                   \
      reorder_kernel<true, V><<<grid, kNormThreads, 0, stream>>>(x, y, rows, dim, BM, BN, rldn, RA);      \
    } else {                                                                                              \
      reorder_kernel<false, V><<<grid, kNormThreads, 0, stream>>>(x, y, rows, dim, BM, BN, rldn, RA);     \
    }                                                                                                     \
  } while (0)
  if (vpt <= 1) {
    FO_LAUNCH_REORDER(1);
  } else if (vpt <= 2) {
    FO_LAUNCH_REORDER(2);
  } else if (vpt <= 4) {
    FO_LAUNCH_REORDER(4);
  } else if (vpt <= 8) {
    FO_LAUNCH_REORDER(8);
  } else {
    return cudaErrorInvalidValue;  // dim > 16384
  }
#undef FO_LAUNCH_REORDER
  return cudaGetLastError();
}

}  // namespace fo
