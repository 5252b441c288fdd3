// Instantiations and host launch code of the tcgen05 GEMM family.
#include "fo_gemm.h"
#include "fo_gemm_sm100.cuh"

#include <mutex>

namespace fo {

// Both blocks travel as kernel parameters; stay inside the classic 4 KB parameter space.
static_assert(sizeof(GemmTensorMaps) + sizeof(GemmParams) <= 4096, "kernel parameters exceed 4 KB");

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

// query != nullptr: do not launch, report the largest co-resident grid instead.
template <int BN, int STAGES, bool BF16, bool FUSED, bool CTA2, int MT = 1, bool A2A = false, bool NORM = false,
          bool TRACE = false, int EPI = 2>
cudaError_t launch_one(const GemmTensorMaps* maps, const GemmParams* p, int grid_x, int nvr,
                       bool cooperative, cudaStream_t stream, int* query) {
  auto kernel = fo_gemm_kernel<BN, STAGES, BF16, FUSED, CTA2, MT, A2A, NORM, TRACE, EPI>;
  constexpr int smem = GemmSmem<BN, STAGES, CTA2, MT, EPI>::kTotalBytes;
  static_assert(smem <= 227 * 1024, "shared memory of this configuration exceeds 227 KB");
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(FUSED ? kThreadsFused : kThreadsPlain, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = 0;
  if (CTA2) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[cfg.numAttrs].val.clusterDim.x = 2;
    attr[cfg.numAttrs].val.clusterDim.y = 1;
    attr[cfg.numAttrs].val.clusterDim.z = 1;
    ++cfg.numAttrs;
  }
  if (query != nullptr) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return e;
    if (!CTA2) {
      *query = prop.multiProcessorCount;  // shared memory admits exactly one CTA per SM
      return cudaSuccess;
    }
    cfg.gridDim = dim3(prop.multiProcessorCount & ~1, 1, 1);
    int clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    if (e != cudaSuccess) return e;
    *query = 2 * clusters;
    return cudaSuccess;
  }
  if (CTA2) grid_x &= ~1;
  if (grid_x < (CTA2 ? 2 : 1)) grid_x = CTA2 ? 2 : 1;
  cfg.gridDim = dim3(grid_x, nvr, 1);
  if (cooperative) {
    attr[cfg.numAttrs].id = cudaLaunchAttributeCooperative;
    attr[cfg.numAttrs].val.cooperative = 1;
    ++cfg.numAttrs;
  }
  return cudaLaunchKernelEx(&cfg, kernel, *maps, *p);
}

// One case per kernel of gemm/fo_gemm_instances.inc.
template <bool BF16, bool FUSED, bool A2A = false, bool NORM = false, bool TRACE = false>
cudaError_t launch_kernel_index(int kidx, const GemmTensorMaps* maps, const GemmParams* p,
                                int grid_x, int nvr, bool coop, cudaStream_t s, int* query) {
  switch (kidx) {
#define FO_GEMM_KERNEL(idx, bn, stages, cta2, mt, stages_epi4) \
  case idx:                                                    \
    return launch_one<bn, stages, BF16, FUSED, cta2, mt, A2A, NORM, TRACE>(maps, p, grid_x, nvr, coop, s, query);
#include "fo_gemm_instances.inc"
#undef FO_GEMM_KERNEL
    default: return cudaErrorInvalidValue;
  }
}

// Fused kernels with four epilogue chunk buffers, paid for with operand stages.
template <bool BF16>
cudaError_t launch_epi4(int kidx, const GemmTensorMaps* maps, const GemmParams* p, int grid_x, int nvr,
                        bool coop, cudaStream_t s, int* query) {
  switch (kidx) {
#define FO_GEMM_KERNEL(idx, bn, stages, cta2, mt, stages_epi4) \
  case idx:                                                    \
    return launch_one<bn, stages_epi4, BF16, true, cta2, mt, false, false, false, 4>(maps, p, grid_x, nvr, coop, s, query);
#include "fo_gemm_instances.inc"
#undef FO_GEMM_KERNEL
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t dispatch(int algo, bool bf16, bool fused, const GemmTensorMaps* maps, const GemmParams* p,
                     int grid_x, int nvr, bool coop, cudaStream_t s, int* query) {
  const int kidx = algo_kernel(algo);
  if (fused && p != nullptr && p->epi_bufs == 4 && p->norm_w == nullptr && p->trace == nullptr) {
    return bf16 ? launch_epi4<true>(kidx, maps, p, grid_x, nvr, coop, s, query)
                : launch_epi4<false>(kidx, maps, p, grid_x, nvr, coop, s, query);
  }
  if (p != nullptr && p->comm == kCommFusedA2A) {
    if (bf16) return launch_kernel_index<true, false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
    return launch_kernel_index<false, false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
  }
  if (fused && p != nullptr && p->norm_w != nullptr) {  // reduce-scatter with the RMSNorm tail
    if (bf16) return launch_kernel_index<true, true, false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
    return launch_kernel_index<false, true, false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
  }
  if (fused && p != nullptr && p->trace != nullptr) {  // timeline-recording build of the fused kernel
    if (bf16) return launch_kernel_index<true, true, false, false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
    return launch_kernel_index<false, true, false, false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
  }
  if (bf16) {
    if (fused) return launch_kernel_index<true, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
    return launch_kernel_index<true, false>(kidx, maps, p, grid_x, nvr, coop, s, query);
  }
  if (fused) return launch_kernel_index<false, true>(kidx, maps, p, grid_x, nvr, coop, s, query);
  return launch_kernel_index<false, false>(kidx, maps, p, grid_x, nvr, coop, s, query);
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
  if (c.cta2 && p->M % (2 * c.mt * c.bm) != 0)
    return c.mt == 2 ? "M must be a multiple of 512 for this Algo (CTA pairs, two row halves per CTA)"
                     : "M must be a multiple of 256 for a CTA-pair Algo";
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

void set_l2_hints(GemmParams* p, bool enable) {
  p->l2_hint_a = ptx::kL2EvictNormal;
  p->l2_hint_b = ptx::kL2EvictNormal;
  if (!enable) return;
  if (p->raster_sw >= p->tiles_n) {
    p->l2_hint_a = ptx::kL2EvictLast;
    p->l2_hint_b = ptx::kL2EvictFirst;
  } else {
    p->l2_hint_a = ptx::kL2EvictFirst;
    p->l2_hint_b = ptx::kL2EvictLast;
  }
}

int gemm_smem_bytes(int algo) {
  switch (algo_kernel(algo)) {
#define FO_GEMM_KERNEL(idx, bn, stages, cta2, mt, stages_epi4) \
  case idx: return GemmSmem<bn, stages, cta2, mt>::kTotalBytes;
#include "fo_gemm_instances.inc"
#undef FO_GEMM_KERNEL
    default: return 0;
  }
}

int gemm_max_resident_ctas(int algo, bool bf16, bool fused) {
  static int cache[16][kNumKernels][2][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  int& slot = cache[dev][algo_kernel(algo)][bf16 ? 1 : 0][fused ? 1 : 0];
  if (slot == 0) {
    int q = 0;
    if (dispatch(algo, bf16, fused, nullptr, nullptr, 0, 1, false, nullptr, &q) != cudaSuccess || q <= 0) {
      cudaGetLastError();
      q = 2;  // conservative: a single CTA pair
    }
    slot = q;
  }
  return slot;
}

cudaError_t launch_gemm(int algo, bool bf16, bool fused, const GemmTensorMaps& maps,
                        const GemmParams& p, int grid_x, int nvr, bool cooperative,
                        cudaStream_t stream) {
  if (algo_config(algo).cta2 && (cooperative || nvr != 1)) return cudaErrorInvalidConfiguration;
  return dispatch(algo, bf16, fused, &maps, &p, grid_x, nvr, cooperative, stream, nullptr);
}

}  // namespace fo
