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
// Four vectors per thread per round, all loads issued before the first store: the tile look-up
// through RA is a dependent load in front of every data load, so one vector at a time leaves
// the memory system idle.
template <bool TO_REORDERED>
__global__ void __launch_bounds__(256)
    reorder_kernel(const uint16_t* __restrict__ X, uint16_t* __restrict__ Y, int rows, int dim,
                   int BM, int BN, int rldn, const int* __restrict__ RA) {
  constexpr int U = 4;
  const int nvec = dim / 8;
  const size_t total = static_cast<size_t>(rows) * nvec;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < total; v0 += stride * U) {
    size_t src[U], dst[U];
    uint4 val[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t v = v0 + u * stride;
      if (v < total) {
        const int b = static_cast<int>(v / nvec);
        const int col = static_cast<int>(v % nvec) * 8;
        const size_t nat = static_cast<size_t>(b) * dim + col;
        const size_t reo = reordered_offset(b, col, dim, BM, BN, rldn, RA);
        src[u] = TO_REORDERED ? nat : reo;
        dst[u] = TO_REORDERED ? reo : nat;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + u * stride < total) val[u] = __ldcs(reinterpret_cast<const uint4*>(X + src[u]));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + u * stride < total) __stcs(reinterpret_cast<uint4*>(Y + dst[u]), val[u]);
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
  const size_t total = static_cast<size_t>(rows) * (dim / 8);
  size_t want = (total + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count) * 16;
  const int grid = static_cast<int>(want < cap ? want : cap);
  const uint16_t* x = static_cast<const uint16_t*>(X);
  uint16_t* y = static_cast<uint16_t*>(Y);
  if (to_reordered) {
    reorder_kernel<true><<<grid, 256, 0, stream>>>(x, y, rows, dim, BM, BN, rldn, RA);
  } else {
    reorder_kernel<false><<<grid, 256, 0, stream>>>(x, y, rows, dim, BM, BN, rldn, RA);
  }
  return cudaGetLastError();
}

}  // namespace fo
