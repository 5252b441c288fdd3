// Host runtime of the overlap path: owns the NCCL communicator, the streams, the symmetric
// staging/flag memory and launches the tcgen05 GEMM family.
//
// The method set and argument orders follow the reference class (src/overlap_impl.h:12-43,
// bound at src/pybind.cpp:129-144) so that its callers run unchanged.  What differs is the
// mechanism behind gemm_allreduce_overlap / gemm_reducescatter_overlap: by default they run
// ONE kernel that computes the tiles and performs the collective over NVLink peer memory.
// The reference's mechanism - signalling GEMM on one stream, counting wait kernel plus one
// NCCL call per wave group on a second stream (src/overlap_impl.cu:214-321) - is kept as
// mode "gated" and serves as a baseline.
#pragma once
#include <ATen/ATen.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <torch/custom_class.h>

#include <memory>
#include <string>
#include <vector>

#include "../comm/symmetric_heap.h"
#include "../gemm/fo_gemm_params.h"

namespace fo {

class OverlapImpl : public torch::CustomClassHolder {
 public:
  OverlapImpl();
  ~OverlapImpl() override;

  // ---- reference API (names as bound in Python; see binding.cpp) ----
  void NcclInit(int64_t rank, int64_t world, std::vector<int64_t> id);
  void CutlassInit();  // name kept for compatibility: captures torch's current stream
  void OverlapInit();  // creates the high-priority communication stream
  void Gemm(at::Tensor A, at::Tensor B, at::Tensor C, int64_t Algo);
  void GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C, int64_t Algo);
  void GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t Algo);
  void GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t Algo,
                   at::Tensor mLen_CPU);
  void NcclAllReduce(at::Tensor C);
  void SegAllReduce(at::Tensor C, at::Tensor cSEG_CPU, int64_t SegNum);
  void NcclReduceScatter(at::Tensor C);
  void NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU);
  void GemmAllReduceOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor MM, at::Tensor RA,
                            int64_t rLDN, at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t Algo,
                            bool if_monitor);
  void GemmReduceScatterOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D,
                                at::Tensor MM, at::Tensor RA, at::Tensor RE, int64_t rLDN,
                                at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t Algo,
                                bool if_monitor);

  // ---- additions ----
  // Fused collectives with row-major results and one flag per tile: no RA / cSeg needed.
  void GemmAllReduceFused(at::Tensor A, at::Tensor B, at::Tensor C, int64_t Algo);
  void GemmReduceScatterFused(at::Tensor A, at::Tensor B, at::Tensor D, int64_t Algo);
  // Fused GEMM + ReduceScatter + RMSNorm: Y [M/world, N] row-major receives
  // rmsnorm(reduce_scatter(A * B^T)) * W.  The reducers gather each row's sum of squares while
  // they reduce, and whichever CTA reduces the last tile of a 128-row panel normalises the
  // panel's rows in place while they are still in L2 - no separate norm kernel, no second pass
  // over HBM.  Same arithmetic as reduce-scatter followed by `flashoverlap_op.rmsnorm`.
  void GemmReduceScatterRmsNormFused(at::Tensor A, at::Tensor B, at::Tensor Y, at::Tensor W, double eps,
                                     int64_t Algo);
  // The same with the residual connection of a pre-norm transformer block in between:
  //   R <- R + reduce_scatter(A * B^T)   (R [M / world, N]: the rank's rows of the residual stream, updated in place)
  //   Y <- rmsnorm(R) * W
  // i.e. what follows a sequence-parallel o_proj or down_proj, in the kernel that computes it.
  void GemmReduceScatterAddRmsNormFused(at::Tensor A, at::Tensor B, at::Tensor R, at::Tensor Y, at::Tensor W,
                                        double eps, int64_t Algo);
  // GEMM whose epilogue stores every row of A * B^T straight into the receive buffer D of the
  // rank it is bound for, over NVLink; same row bookkeeping as gemm_all2all (mLen_CPU[r][i]
  // rows go from rank r to rank i, runs packed in rank order, own run excluded), no C and no
  // separate collective.  Rows of the product past the last run are dropped.  D needs room for
  // the rows this rank receives; a D from symm_empty is written in place, any other D through
  // a symmetric scratch buffer and one copy.  The reference has no overlapped all-to-all.
  void GemmAll2AllFused(at::Tensor A, at::Tensor B, at::Tensor D, int64_t Algo, at::Tensor mLen_CPU);
  // Options: "mode" (0 fused, 1 gated), "strided_rows" (reduce-scatter row ownership:
  // 1 = rank r owns rows i % world == r as in the reference, 0 = contiguous blocks),
  // "sm_margin" (SMs left to NCCL in gated mode), "timeout_ms" (bound of device waits),
  // "l2_hints" (1: operand loads carry L2 eviction priorities matched to the tile sweep),
  // "nvls" (1: broadcast AllReduce results through a registered multicast mapping),
  // "push_lag" (tiles of pushes kept in flight before their arrival is signalled; 0 = from K),
  // "stage_local" (1: pull protocol - partials stay in the producing rank's staging buffer and
  // the owners fetch them, through the switch's reduction when the buffer has a multicast mapping),
  // "pull_direct" (pull protocol only; 1: the epilogue threads store the partial tile into the
  // local staging themselves and the push warp only announces it, 0: chunks go through the push
  // warp's TMA stores, -1, the default: direct for the 256 x 256-per-CTA kernels),
  // "epi_bufs" (2 | 4: fused kernels with four epilogue chunk buffers and one operand stage fewer;
  // their push warp keeps three chunks of stores in flight instead of waiting for each),
  // "wait_sleep_ns" (nanoseconds the kernel's waiting roles sleep between mbarrier polls; 0, the
  // default = poll continuously: 64 and 256 ns changed neither the instruction count nor the time),
  // "validate" (1: overlap calls also check the values of RA / RE / cSEG_GPU - permutation, range,
  // sum - at the price of a device-to-host copy per call; on by default in a -DFO_DEBUG build),
  // "tma_out" (1: plain GEMMs with a row-major or tile-contiguous output store finished chunks
  // with TMA tensor stores; 0: per-thread 16-byte stores; -1, the default: TMA for the kernels
  // whose epilogue overlaps the next main loop, per-thread stores for the 256 x 256-per-CTA ones),
  // "diag" (timing studies only - results are wrong: 1 skips the reducers' memory traffic, 2 the
  // push stores, 4 the reducers' arrival waits; shows which part of the collective is exposed.
  // After runs with bit 4, synchronise all ranks and call reset_status() before normal calls:
  // late arrivals may have been counted after the counters were cleared).
  void SetOption(std::string name, int64_t value);
  int64_t GetOption(std::string name);
  // Collective allocation of a tensor in symmetric memory.  AllReduce results written into
  // such a tensor need no extra copy.
  at::Tensor SymmEmpty(std::vector<int64_t> sizes, std::string dtype);
  // Registers symmetric memory allocated elsewhere (for instance by
  // torch.distributed._symmetric_memory): peer_ptrs[r] is rank r's copy as addressable from
  // this process, multicast_ptr the NVSwitch multicast mapping of the same buffer or 0.
  // AllReduce results written into such a tensor are broadcast with one multimem store per
  // vector (the switch replicates it) instead of one peer store per rank.  The caller keeps
  // the memory alive for as long as this object may use it.
  void RegisterSymmetric(at::Tensor local, std::vector<int64_t> peer_ptrs, int64_t multicast_ptr);
  // Staging buffer for the pull protocol (option "stage_local"): a whole symmetric buffer of at
  // least M*N*2 bytes.  When it carries a multicast mapping the owners' reducers sum the
  // partials with one switch-side reduction per vector (multimem.ld_reduce).  Same call on every rank.
  void UseStage(at::Tensor buffer);
  // Timeline recording: while `buffer` (int64 CUDA tensor, at least tiles * 8 elements; an empty
  // tensor switches recording off) is set, fused AllReduce / ReduceScatter calls run a build of
  // the kernel that stamps, per 128-row tile, when its accumulator was complete, when the
  // epilogue, the pushes and their completion signal were done and when the owner's reducer
  // waited for, got and reduced it (layout: TraceSlot in gemm/fo_gemm_params.h;
  // flashoverlap_b200/utils/trace.py turns it into a summary or a Chrome trace).
  void SetTrace(at::Tensor buffer);
  // Status words written by device-side waits that gave up (all zero when healthy).
  std::vector<int64_t> ReadStatus();
  void CheckStatus();  // throws with a description when the status is not ok
  // Clears the status words and this rank's own arrival counters after a reported failure that
  // stayed local (a bounded wait inside one GPU).  It does not touch the cross-rank state: after a
  // failure in which the ranks fell out of step (a peer skipped a call, a cross-GPU wait gave
  // up) call resync() on every rank instead.
  void ResetStatus();
  // Waits on the caller's stream until MM[index] == target and resets it to 0 (the gated path's
  // wait kernel as a call of its own); after "timeout_ms" it gives up and this object's status
  // words say so (check_status then raises).
  void WaitFlag(int64_t target, at::Tensor MM, int64_t index);
  // Collective: every rank waits for its stream, all ranks meet (NCCL), each clears its whole
  // signal region (arrival, done and ready counters) and status words, all meet again, and the
  // call numbering restarts.  Brings a group of objects back in step after a fused call that
  // some rank missed or gave up in; no fused call may be in flight on any rank.
  void Resync();

 private:
  struct FusedArgs;
  void run_plain(const at::Tensor& A, const at::Tensor& B, void* out, int out_mode,
                 const int* RA, const int* RE, int rldn, int* MM, int mm_stride, bool signal,
                 bool monitor, const int* cseg, int num_groups, int algo, int grid_cap);
  void run_fused(int comm, const at::Tensor& A, const at::Tensor& B, at::Tensor out, int out_mode,
                 const int* RA, int rldn, int* MM, int mm_stride, bool monitor, const int* cseg,
                 int num_groups, int algo, const at::Tensor* norm_w = nullptr, double norm_eps = 0.0,
                 const at::Tensor* norm_res = nullptr, const at::Tensor* norm_out = nullptr);
  void gated_overlap(int comm, at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D,
                     at::Tensor MM, at::Tensor RA, at::Tensor RE, int64_t rLDN,
                     at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t Algo, bool monitor);
  void ensure_fused_buffers(size_t stage_bytes, size_t nflags, bool pull);
  void check_overlap_args(const char* what, int M, int N, int algo, const at::Tensor& MM, const at::Tensor& RA,
                          const at::Tensor* RE, int64_t rLDN, const at::Tensor& cSEG_CPU, const at::Tensor& cSEG_GPU,
                          bool monitor, bool needs_counters) const;
  void ensure_comm_stream();
  cudaStream_t stream() const;
  ncclDataType_t nccl_dtype(const at::Tensor& t) const;

  int rank_ = 0;
  int world_ = 1;
  int device_ = 0;
  int sm_count_ = 148;
  ncclComm_t comm_ = nullptr;
  bool have_gemm_stream_ = false;
  cudaStream_t gemm_stream_ = nullptr;
  cudaStream_t comm_stream_ = nullptr;
  cudaEvent_t comm_done_ = nullptr;
  cudaEvent_t gemm_start_ = nullptr;

  std::shared_ptr<SymmetricHeap> heap_;  // shared with the tensors handed out by symm_empty
  SymmetricRegion* stage_ = nullptr;
  SymmetricRegion* signal_ = nullptr;
  SymmetricRegion* out_ = nullptr;  // symmetric AllReduce output when the caller's is not
  const SymmetricRegion* user_stage_ = nullptr;  // staging handed in through UseStage
  uint32_t epoch_ = 0;
  uint32_t a2a_epoch_ = 0;  // fused all-to-all calls so far (start-of-call handshake)
  at::Tensor a2a_tab_;      // device copy of the current call's row tables
  at::Tensor trace_;        // timeline buffer set by SetTrace, or undefined
  at::Tensor norm_ssq_;     // fp32 [rows of the shard]: per-row sums of squares, zero between calls
  at::Tensor norm_cnt_;     // int32 [row panels]: reduced tiles per panel, zero between calls
  at::Tensor status_;  // int32[kStatusWords] on the device

  int64_t opt_mode_ = 0;
  int64_t opt_strided_rows_ = 1;
  int64_t opt_sm_margin_ = 16;
  int64_t opt_timeout_ms_ = 2000;
  int64_t opt_nvls_ = 1;      // use a registered multicast mapping when there is one
  int64_t opt_push_lag_ = 0;  // 0: chosen from K
  int64_t opt_diag_ = 0;         // timing studies only (results are wrong): see GemmParams::diag
  int64_t opt_epi_bufs_ = 2;     // epilogue chunk buffers of the fused kernels (2 or 4)
#ifdef FO_DEBUG
  int64_t opt_validate_ = 1;     // debug builds check the values of RA / RE / cSEG on every overlap call
#else
  int64_t opt_validate_ = 0;     // 1: also check the VALUES of RA / RE / cSEG_GPU (a device-to-host copy per call)
#endif
  int64_t opt_tma_out_ = -1;     // plain kernels' stores: 1 TMA tensor stores, 0 per-thread stores, -1 by kernel
  int64_t opt_pull_direct_ = -1;  // pull protocol: epilogue threads store the partials themselves (1), TMA (0), by kernel (-1)
  int64_t opt_wait_sleep_ns_ = 0;   // back-off of the kernel roles that wait with slack (0: poll continuously; measured: no gain)
  int64_t opt_stage_local_ = 0;  // 1: pull protocol (partials staged locally, owners fetch them)
  int64_t opt_l2_hints_ = 0;  // measured: priorities raise DRAM traffic on B200, off by default
};

}  // namespace fo
