// Single-GPU emulation of the fused GEMM+collective kernels: all `ws` ranks' CTAs run in ONE
// cooperative launch on the current device (rank = blockIdx.y), each rank with its own
// operands, staging, flags and outputs.  The code path inside the kernel is the one the
// multi-GPU launch uses; only the addresses in the per-rank tables differ.  This is how the
// cross-rank protocol is tested where a single GPU is available.  (Separate launches, one
// per rank, must never be used for this: kernels that wait on one another are not
// guaranteed to be co-resident.)  The reference has no counterpart.
#pragma once
#include <ATen/ATen.h>

#include <string>
#include <vector>

namespace fo {

// comm_op: "all_reduce", "reduce_scatter" or "all_to_all".  A[r] is [M,K], B[r] is [N,K]; out[r]
// is [M,N] (all_reduce), [M/ws,N] (reduce_scatter) or the receive buffer of rank r (all_to_all,
// whose row counts come in the int32 host tensor mlen [ws, ws]).  With norm_w (reduce_scatter,
// natural_out) the reducers apply the RMSNorm tail: out[r] = rmsnorm(shard) * norm_w.  trace: int64
// CUDA tensor of ws * tiles * 8 elements that receives the timeline of the (last) call.  epi_bufs:
// 2 (default build) or 4 (four epilogue chunk buffers, one operand stage fewer).  RA / cseg_gpu may be None
// (identity order / one flag per tile).  natural_out selects row-major results instead of
// the tile-contiguous layout.  The call is repeated `repeat` times back to back to exercise
// the call-to-call handshake.  stage_local selects the pull protocol (partials staged in the
// producing rank's own memory, owners fetch them; here without a multicast mapping, so with one
// load per rank); pull_direct != 0 with it: the epilogue threads store the partial tiles themselves
// instead of handing them to the push warp's TMA stores.  norm_res / norm_out (with norm_w): per-rank
// residual added to the reduced rows before they are stored in out[r] and normalised, and per-rank
// destination of the normalised rows (default: over out[r]).  Returns ws * kStatusWords status words.
std::vector<int64_t> fused_loopback(std::string comm_op, std::vector<at::Tensor> A,
                                    std::vector<at::Tensor> B, std::vector<at::Tensor> out,
                                    c10::optional<at::Tensor> RA,
                                    c10::optional<at::Tensor> cseg_gpu, int64_t algo,
                                    bool strided_rows, bool natural_out, int64_t repeat,
                                    int64_t timeout_ms, bool stage_local,
                                    c10::optional<at::Tensor> mlen,
                                    c10::optional<at::Tensor> norm_w, double norm_eps,
                                    c10::optional<at::Tensor> trace, int64_t epi_bufs, int64_t pull_direct,
                                    c10::optional<std::vector<at::Tensor>> norm_res,
                                    c10::optional<std::vector<at::Tensor>> norm_out);

}  // namespace fo
