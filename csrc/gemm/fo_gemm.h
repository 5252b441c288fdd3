// Host entry points of the tcgen05 GEMM family (plain, signalling and fused-collective
// epilogues).  Counterpart of the reference's three launcher templates
// cutlass_gemm_splitk / cutlass_gemm_signal / cutlass_gemm_scatter
// (src/gemm/gemm.h:3-5, src/overlap/gemm_signal.h:3-5, src/overlap/gemm_scatter.h:3-5).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <string>

#include "fo_gemm_params.h"

namespace fo {

// Builds a 2-D tiled tensor map over a row-major [rows, cols] matrix of 16-bit elements with
// a (box_rows x 64) box and the 128-byte swizzle.  `ptr` must be 16-byte aligned and
// cols * 2 a multiple of 16.  Returns an empty string on success, else a message.
std::string encode_tmap_16bit(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                              uint32_t box_rows);

// Fills tiles_m / tiles_n / num_tiles / raster_sw of `p` for `algo` and checks divisibility.
std::string prepare_tiling(int algo, GemmParams* p);

// Launches the kernel for `algo`.  grid_x CTAs per virtual rank, nvr virtual ranks
// (gridDim.y).  `cooperative` requests a cooperative launch, which fails instead of
// deadlocking when the grid cannot be co-resident (needed when CTAs of different virtual
// ranks wait on one another on one GPU).
cudaError_t launch_gemm(int algo, bool bf16, bool fused, const GemmTensorMaps& maps,
                        const GemmParams& p, int grid_x, int nvr, bool cooperative,
                        cudaStream_t stream);

// Sets the L2 eviction priorities of the operand loads for the tiling already in `p`: with
// column strips swept M-major the B strip is re-read by every wave of the strip (keep it: evict
// last) while A streams through (evict first); with full row panels it is the other way round.
// `enable == false` leaves both at normal priority.
void set_l2_hints(GemmParams* p, bool enable);

int gemm_smem_bytes(int algo);

// Tiles whose pushes the fused kernel keeps in flight before signalling their arrival: with a
// long main loop (large K) the previous tile's stores are complete by the time the next tile
// is pushed, with a short one the completion latency of NVLink writes must be covered by
// letting several tiles overlap.
inline int default_push_lag(int K) { return K >= 4096 ? 1 : (K >= 2048 ? 2 : 4); }

// Largest grid (CTAs per virtual rank) of this Algo's kernel that is co-resident on the
// current device: one CTA per SM, or two per schedulable cluster for the CTA-pair kernels.
// Fused launches must not exceed it, since their CTAs wait for the same CTAs on the peers.
int gemm_max_resident_ctas(int algo, bool bf16, bool fused);

}  // namespace fo
