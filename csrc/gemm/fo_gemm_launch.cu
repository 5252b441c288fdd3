// Instantiations and host launch code of the tcgen05 GEMM family.
#include "fo_gemm.h"
#include "fo_gemm_sm100.cuh"

#include <mutex>

namespace fo {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(f);
    }
  });
  return fn;
}

template <int BN, int STAGES, bool BF16, bool FUSED>
cudaError_t launch_one(const GemmTensorMaps& maps, const GemmParams& p, int grid_x, int nvr,
                       bool cooperative, cudaStream_t stream) {
  auto kernel = fo_gemm_kernel<BN, STAGES, BF16, FUSED>;
  constexpr int smem = GemmSmem<BN, STAGES>::kTotalBytes;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_x, nvr, 1);
  cfg.blockDim = dim3(FUSED ? kThreadsFused : kThreadsPlain, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  cfg.numAttrs = 0;
  if (cooperative) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, maps, p);
}

template <bool BF16, bool FUSED>
cudaError_t launch_kernel_index(int kidx, const GemmTensorMaps& maps, const GemmParams& p,
                                int grid_x, int nvr, bool coop, cudaStream_t s) {
  switch (kidx) {
    case 0: return launch_one<256, 4, BF16, FUSED>(maps, p, grid_x, nvr, coop, s);
    case 1: return launch_one<256, 3, BF16, FUSED>(maps, p, grid_x, nvr, coop, s);
    case 2: return launch_one<128, 6, BF16, FUSED>(maps, p, grid_x, nvr, coop, s);
    default: return launch_one<128, 4, BF16, FUSED>(maps, p, grid_x, nvr, coop, s);
  }
}

}  // namespace

std::string encode_tmap_16bit(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                              uint32_t box_rows) {
  EncodeFn fn = get_encode_fn();
  if (fn == nullptr) return "cuTensorMapEncodeTiled is not available from this driver";
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return "operand is not 16-byte aligned";
  if ((cols * 2) % 16 != 0) return "row pitch is not a multiple of 16 bytes";
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), box_rows};
  cuuint32_t estr[2] = {1, 1};
  // 16-bit payload: the MMA instruction descriptor decides bf16 vs fp16, TMA only moves bits.
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r));
  return "";
}

std::string prepare_tiling(int algo, GemmParams* p) {
  if (algo < 0 || algo >= kNumAlgos) return "Algo index out of range";
  const AlgoConfig c = algo_config(algo);
  if (p->M % c.bm != 0) return "M must be a multiple of 128";
  if (p->N % c.bn != 0) return "N must be a multiple of the tile width BN of this Algo";
  if (p->K % 8 != 0) return "K must be a multiple of 8";
  p->tiles_m = p->M / c.bm;
  p->tiles_n = p->N / c.bn;
  p->num_tiles = p->tiles_m * p->tiles_n;
  int sw = c.raster_sw <= 0 ? p->tiles_n : c.raster_sw;
  if (sw > p->tiles_n) sw = p->tiles_n;
  p->raster_sw = sw;
  return "";
}

int gemm_smem_bytes(int algo) {
  switch (algo & 3) {
    case 0: return GemmSmem<256, 4>::kTotalBytes;
    case 1: return GemmSmem<256, 3>::kTotalBytes;
    case 2: return GemmSmem<128, 6>::kTotalBytes;
    default: return GemmSmem<128, 4>::kTotalBytes;
  }
}

cudaError_t launch_gemm(int algo, bool bf16, bool fused, const GemmTensorMaps& maps,
                        const GemmParams& p, int grid_x, int nvr, bool cooperative,
                        cudaStream_t stream) {
  const int kidx = algo & 3;
  if (bf16) {
    if (fused) return launch_kernel_index<true, true>(kidx, maps, p, grid_x, nvr, cooperative, stream);
    return launch_kernel_index<true, false>(kidx, maps, p, grid_x, nvr, cooperative, stream);
  }
  if (fused) return launch_kernel_index<false, true>(kidx, maps, p, grid_x, nvr, cooperative, stream);
  return launch_kernel_index<false, false>(kidx, maps, p, grid_x, nvr, cooperative, stream);
}

}  // namespace fo
