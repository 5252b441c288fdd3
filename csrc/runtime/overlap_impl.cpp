#include "overlap_impl.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <algorithm>
#include <cstring>

#include "../comm/nccl_utils.h"
#include "../common/fo_nvtx.h"
#include "../flags/fo_wait.h"
#include "../norm/fo_norm.h"
#include "fused_common.h"

namespace fo {

OverlapImpl::OverlapImpl() {}

OverlapImpl::~OverlapImpl() {
  // Streams and events first, then the symmetric memory, then the communicator.
  if (comm_done_ != nullptr) cudaEventDestroy(comm_done_);
  if (gemm_start_ != nullptr) cudaEventDestroy(gemm_start_);
  if (comm_stream_ != nullptr) cudaStreamDestroy(comm_stream_);
  // Tensors from symm_empty may keep the heap (and its memory) alive beyond this point; the heap
  // needs the communicator only for collective calls, which nobody can make any more.
  if (heap_ != nullptr) heap_->detach_comm();
  heap_.reset();
  if (comm_ != nullptr) ncclCommDestroy(comm_);  // the reference never destroys its communicator
}

cudaStream_t OverlapImpl::stream() const {
  // The stream current in torch at call time.  (The reference freezes the stream that was
  // current when cutlass_init ran, src/overlap_impl.cu:31-33; following the caller's stream
  // context is what torch users expect, and is identical for callers on the default stream.)
  return c10::cuda::getCurrentCUDAStream().stream();
}

ncclDataType_t OverlapImpl::nccl_dtype(const at::Tensor& t) const {
  if (t.scalar_type() == at::kBFloat16) return ncclBfloat16;
  if (t.scalar_type() == at::kHalf) return ncclFloat16;
  if (t.scalar_type() == at::kFloat) return ncclFloat32;
  FO_CHECK(false, "unsupported dtype for a collective");
  return ncclFloat16;
}

void OverlapImpl::NcclInit(int64_t rank, int64_t world, std::vector<int64_t> id) {
  FO_CHECK(world >= 1 && world <= kMaxRanks, "world size must be in [1, ", kMaxRanks, "]");
  FO_CHECK(rank >= 0 && rank < world, "rank out of range");
  FO_CHECK(comm_ == nullptr && heap_ == nullptr, "nccl_init was already called");
  rank_ = static_cast<int>(rank);
  world_ = static_cast<int>(world);
  cuda_check(cudaGetDevice(&device_), "cudaGetDevice");
  cudaDeviceProp prop;
  cuda_check(cudaGetDeviceProperties(&prop, device_), "cudaGetDeviceProperties");
  sm_count_ = prop.multiProcessorCount;
  if (world_ > 1) {
    ncclUniqueId uid = unpack_nccl_id(id);
    FO_NCCL_CHECK(ncclCommInitRank(&comm_, world_, uid, rank_));
  }
  heap_ = std::make_shared<SymmetricHeap>(rank_, world_, comm_, false);
  status_ = at::zeros({kStatusWords}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device_));
}

void OverlapImpl::CutlassInit() {
  if (heap_ == nullptr) NcclInit(0, 1, {});
}

void OverlapImpl::ensure_comm_stream() {
  if (comm_stream_ != nullptr) return;
  int lo = 0, hi = 0;
  cuda_check(cudaDeviceGetStreamPriorityRange(&lo, &hi), "cudaDeviceGetStreamPriorityRange");
  cuda_check(cudaStreamCreateWithPriority(&comm_stream_, cudaStreamNonBlocking, hi),
             "cudaStreamCreateWithPriority");
  cuda_check(cudaEventCreateWithFlags(&comm_done_, cudaEventDisableTiming), "cudaEventCreate");
  cuda_check(cudaEventCreateWithFlags(&gemm_start_, cudaEventDisableTiming), "cudaEventCreate");
}

void OverlapImpl::OverlapInit() {
  if (heap_ == nullptr) NcclInit(0, 1, {});
  ensure_comm_stream();
}

void OverlapImpl::SetOption(std::string name, int64_t value) {
  if (name == "mode") {
    FO_CHECK(value == 0 || value == 1, "mode must be 0 (fused) or 1 (gated)");
    opt_mode_ = value;
  } else if (name == "strided_rows") {
    opt_strided_rows_ = value ? 1 : 0;
  } else if (name == "sm_margin") {
    FO_CHECK(value >= 0 && value < sm_count_, "sm_margin out of range");
    opt_sm_margin_ = value;
  } else if (name == "timeout_ms") {
    FO_CHECK(value > 0, "timeout_ms must be positive");
    opt_timeout_ms_ = value;
  } else if (name == "l2_hints") {
    opt_l2_hints_ = value ? 1 : 0;
  } else if (name == "nvls") {
    opt_nvls_ = value ? 1 : 0;
  } else if (name == "push_lag") {
    FO_CHECK(value >= 0 && value <= 4, "push_lag must be 0 (automatic) or 1..4");
    opt_push_lag_ = value;
  } else if (name == "stage_local") {
    opt_stage_local_ = value ? 1 : 0;
  } else if (name == "diag") {
    FO_CHECK(value >= 0 && value <= 7, "diag is a bit mask of 1 | 2 | 4");
    opt_diag_ = value;
  } else if (name == "pull_direct") {
    FO_CHECK(value >= -1 && value <= 1, "pull_direct must be -1 (automatic), 0 or 1");
    opt_pull_direct_ = value;
  } else if (name == "wait_sleep_ns") {
    FO_CHECK(value >= 0 && value <= 10000, "wait_sleep_ns must be in [0, 10000]");
    opt_wait_sleep_ns_ = value;
  } else if (name == "validate") {
    opt_validate_ = value ? 1 : 0;
  } else if (name == "tma_out") {
    FO_CHECK(value >= -1 && value <= 1, "tma_out must be -1 (automatic), 0 or 1");
    opt_tma_out_ = value;
  } else if (name == "epi_bufs") {
    FO_CHECK(value == 2 || value == 4, "epi_bufs must be 2 or 4");
    opt_epi_bufs_ = value;
  } else {
    FO_CHECK(false, "unknown option '", name, "'");
  }
}

int64_t OverlapImpl::GetOption(std::string name) {
  if (name == "mode") return opt_mode_;
  if (name == "strided_rows") return opt_strided_rows_;
  if (name == "sm_margin") return opt_sm_margin_;
  if (name == "timeout_ms") return opt_timeout_ms_;
  if (name == "l2_hints") return opt_l2_hints_;
  if (name == "nvls") return opt_nvls_;
  if (name == "push_lag") return opt_push_lag_;
  if (name == "stage_local") return opt_stage_local_;
  if (name == "epi_bufs") return opt_epi_bufs_;
  if (name == "tma_out") return opt_tma_out_;
  if (name == "validate") return opt_validate_;
  if (name == "wait_sleep_ns") return opt_wait_sleep_ns_;
  if (name == "pull_direct") return opt_pull_direct_;
  if (name == "diag") return opt_diag_;
  if (name == "sm_count") return sm_count_;
  if (name == "rank") return rank_;
  if (name == "world") return world_;
  if (name == "num_algos") return kNumAlgos;
  FO_CHECK(false, "unknown option '", name, "'");
  return 0;
}

at::Tensor OverlapImpl::SymmEmpty(std::vector<int64_t> sizes, std::string dtype) {
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  at::ScalarType st;
  if (dtype == "bfloat16" || dtype == "bf16") {
    st = at::kBFloat16;
  } else if (dtype == "float16" || dtype == "fp16" || dtype == "half") {
    st = at::kHalf;
  } else if (dtype == "float32" || dtype == "fp32") {
    st = at::kFloat;
  } else {
    FO_CHECK(false, "unsupported dtype '", dtype, "'");
    st = at::kHalf;
  }
  int64_t numel = 1;
  for (int64_t s : sizes) {
    FO_CHECK(s >= 0, "negative size");
    numel *= s;
  }
  const size_t bytes = std::max<size_t>(static_cast<size_t>(numel) * c10::elementSize(st), 256);
  SymmetricRegion* reg = heap_->allocate(bytes, stream());
  // The memory belongs to the heap, and the tensor shares ownership of the heap: it stays valid
  // even if it outlives this object (the heap then goes with the last such tensor).
  std::shared_ptr<SymmetricHeap> keep = heap_;
  return at::from_blob(reg->local(), sizes, [keep](void*) {},
                       at::TensorOptions().dtype(st).device(at::kCUDA, device_));
}

void OverlapImpl::RegisterSymmetric(at::Tensor local, std::vector<int64_t> peer_ptrs, int64_t multicast_ptr) {
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  FO_CHECK(local.is_cuda() && local.is_contiguous(), "local must be a contiguous CUDA tensor");
  FO_CHECK(static_cast<int>(peer_ptrs.size()) == world_, "peer_ptrs must have one address per rank");
  FO_CHECK(reinterpret_cast<int64_t>(local.data_ptr()) == peer_ptrs[rank_],
           "peer_ptrs[rank] must be the address of the local tensor");
  std::vector<void*> ptrs(world_);
  for (int r = 0; r < world_; ++r) ptrs[r] = reinterpret_cast<void*>(peer_ptrs[r]);
  heap_->adopt(local.nbytes(), ptrs, reinterpret_cast<void*>(multicast_ptr));
}

void OverlapImpl::UseStage(at::Tensor buffer) {
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  FO_CHECK(buffer.is_cuda() && buffer.is_contiguous(), "the staging buffer must be a contiguous CUDA tensor");
  const SymmetricRegion* reg = heap_->find(buffer.data_ptr(), buffer.nbytes());
  FO_CHECK(reg != nullptr && reg->local() == buffer.data_ptr(),
           "use_stage needs a whole symmetric buffer (from symm_empty, or registered with register_symmetric)");
  user_stage_ = reg;
}

void OverlapImpl::SetTrace(at::Tensor buffer) {
  if (!buffer.defined() || buffer.numel() == 0) {
    trace_ = at::Tensor();
    return;
  }
  FO_CHECK(buffer.is_cuda() && buffer.is_contiguous() && buffer.scalar_type() == at::kLong,
           "the trace buffer must be a contiguous int64 CUDA tensor");
  trace_ = buffer;
}

std::vector<int64_t> OverlapImpl::ReadStatus() {
  FO_CHECK(status_.defined(), "call nccl_init first");
  at::Tensor h = status_.cpu();
  std::vector<int64_t> out(kStatusWords);
  for (int i = 0; i < kStatusWords; ++i) out[i] = h.data_ptr<int>()[i];
  return out;
}

void OverlapImpl::CheckStatus() {
  const std::vector<int64_t> s = ReadStatus();
  FO_CHECK(s[kStatusWordCode] == kStatusOk, status_message(s.data(), rank_));
}

void OverlapImpl::ResetStatus() {
  FO_CHECK(status_.defined(), "call nccl_init first");
  status_.zero_();
  if (norm_ssq_.defined()) norm_ssq_.zero_();  // an aborted call may have left partial statistics
  if (norm_cnt_.defined()) norm_cnt_.zero_();
  if (signal_ != nullptr) {
    char* base = static_cast<char*>(signal_->local());
    cuda_check(cudaMemsetAsync(base + kSignalLocalCntOffset, 0, 128, stream()), "cudaMemsetAsync");
    cuda_check(cudaMemsetAsync(base + kSignalFlagsOffset, 0, kSignalMaxFlags * sizeof(uint32_t),
                               stream()),
               "cudaMemsetAsync");
  }
}

void OverlapImpl::WaitFlag(int64_t target, at::Tensor MM, int64_t index) {
  // The bounded counting wait of the gated path as a call of its own, on the caller's stream
  // (reference: kernel_wait_flag, src/wait.cuh:5-9, which spins without a limit).  Gives up
  // after "timeout_ms" and records that in this object's status words.
  FO_CHECK(status_.defined(), "call nccl_init first");
  FO_CHECK(MM.is_cuda() && MM.scalar_type() == at::kInt && MM.is_contiguous(), "MM must be a contiguous int32 CUDA tensor");
  FO_CHECK(index >= 0 && index < MM.numel(), "counter index ", index, " outside MM (", MM.numel(), " entries)");
  FO_CHECK(target > 0, "target must be positive");
  cuda_check(wait_flag_launch(static_cast<int>(target), MM.data_ptr<int>() + index, static_cast<int>(index),
                              static_cast<uint64_t>(opt_timeout_ms_) * 1000000ull, status_.data_ptr<int>(), stream()),
             "wait kernel launch");
}

void OverlapImpl::Resync() {
  // Collective re-alignment after a failed or skipped fused call.  A rank that missed a call
  // (or gave up in one) disagrees with its peers about the call number and the `done` counters,
  // and every later fused call would time out.  All ranks: finish what is in flight, agree that
  // everybody has stopped (first barrier), clear the local counters, agree that everybody has
  // cleared (second barrier), restart the call numbering.
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  cudaStream_t s = stream();
  cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  at::Tensor token = at::zeros({1}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device_));
  auto barrier = [&]() {
    if (world_ > 1) {
      FO_NCCL_CHECK(ncclAllReduce(token.data_ptr(), token.data_ptr(), 1, ncclFloat32, ncclSum, comm_, s));
    }
    cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  };
  barrier();
  if (signal_ != nullptr) cuda_check(cudaMemsetAsync(signal_->local(), 0, kSignalBytes, s), "cudaMemsetAsync");
  status_.zero_();
  if (norm_ssq_.defined()) norm_ssq_.zero_();
  if (norm_cnt_.defined()) norm_cnt_.zero_();
  barrier();
  epoch_ = 0;
  a2a_epoch_ = 0;
}

// ---------------------------------------------------------------------------- plain GEMM

void OverlapImpl::run_plain(const at::Tensor& A, const at::Tensor& B, void* out, int out_mode,
                            const int* RA, const int* RE, int rldn, int* MM, int mm_stride,
                            bool signal, bool monitor, const int* cseg, int num_groups, int algo,
                            int grid_cap) {
  if (heap_ == nullptr) NcclInit(0, 1, {});
  c10::cuda::CUDAGuard guard(A.device());
  GemmTensorMaps maps;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  bool bf16 = true;
  setup_problem(algo, A, B, 0, &maps, &p, &bf16);
  set_l2_hints(&p, opt_l2_hints_ != 0);
  p.out_mode = out_mode;
  p.rldn = rldn < 1 ? 1 : rldn;
  p.signal = signal ? 1 : 0;
  p.monitor = monitor ? 1 : 0;
  p.mm_stride = mm_stride;
  p.num_groups = num_groups;
  p.comm = kCommNone;
  p.ws = 1;
  p.rank_base = rank_;
  p.timeout_ns = static_cast<uint64_t>(opt_timeout_ms_) * 1000000ull;
  p.wait_sleep_ns = static_cast<uint32_t>(opt_wait_sleep_ns_);
  p.RA = RA;
  p.RE = RE;
  p.cseg = cseg;
  p.out[0] = out;
  p.MM[0] = MM;
  p.status[0] = status_.data_ptr<int>();
  // TMA tensor stores pay where the epilogue runs under the next tile's main loop; the kernels
  // whose two accumulators fill TMEM (mt == 2) expose their epilogue and are faster with the
  // fire-and-forget per-thread stores (measured: 4-15 % of the step at K per rank <= 28672).
  const bool tma_out = opt_tma_out_ > 0 || (opt_tma_out_ < 0 && algo_config(algo).mt == 1);
  if (tma_out) setup_out_map(&maps, 0, out, &p, algo_config(algo).bn);
  const int resident = gemm_max_resident_ctas(algo, bf16, false);
  const int grid = std::max(1, std::min(std::min(grid_cap, resident), p.num_tiles));
  cuda_check(launch_gemm(algo, bf16, false, maps, p, grid, 1, false, stream()), "GEMM launch");
}

void OverlapImpl::Gemm(at::Tensor A, at::Tensor B, at::Tensor C, int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::cutlass_gemm");
  const GemmShape s = check_operands(A, B);
  check_out(C, A, static_cast<int64_t>(s.M) * s.N, "C");
  run_plain(A, B, C.data_ptr(), kOutNatural, nullptr, nullptr, 1, nullptr, 0, false, false, nullptr,
            0, static_cast<int>(Algo), sm_count_);
}

// ---------------------------------------------------------------------------- bare collectives

void OverlapImpl::NcclAllReduce(at::Tensor C) {
  NvtxRange nvtx_range("flashoverlap::nccl_allreduce");
  if (world_ == 1) return;
  FO_NCCL_CHECK(ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_dtype(C), ncclSum, comm_,
                              stream()));
}

void OverlapImpl::SegAllReduce(at::Tensor C, at::Tensor cSEG_CPU, int64_t SegNum) {
  NvtxRange nvtx_range("flashoverlap::seg_allreduce");
  // Equal units of numel / SegNum elements; segment s covers cSEG_CPU[s] units
  // (reference: src/overlap_impl.cu:153-168).
  if (world_ == 1) return;
  FO_CHECK(!cSEG_CPU.is_cuda() && cSEG_CPU.scalar_type() == at::kInt, "cSEG_CPU: int32 host tensor");
  const int* seg = cSEG_CPU.data_ptr<int>();
  const int64_t unit = C.numel() / SegNum;
  char* base = static_cast<char*>(C.data_ptr());
  const size_t es = C.element_size();
  int64_t acc = 0;
  int64_t units = 0;
  for (int64_t s = 0; s < cSEG_CPU.numel() && units < SegNum; ++s) {
    const int64_t n = unit * seg[s];
    FO_NCCL_CHECK(ncclAllReduce(base + acc * es, base + acc * es, n, nccl_dtype(C), ncclSum, comm_,
                                stream()));
    acc += n;
    units += seg[s];
  }
}

void OverlapImpl::NcclReduceScatter(at::Tensor C) {
  NvtxRange nvtx_range("flashoverlap::nccl_reducescatter");
  // In place: rank r's shard of the sum lands in its own slice of C
  // (reference: src/overlap_impl.cu:170-179).
  if (world_ == 1) return;
  const int64_t recv = C.numel() / world_;
  char* base = static_cast<char*>(C.data_ptr());
  FO_NCCL_CHECK(ncclReduceScatter(base, base + rank_ * recv * C.element_size(), recv, nccl_dtype(C),
                                  ncclSum, comm_, stream()));
}

void OverlapImpl::NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU) {
  NvtxRange nvtx_range("flashoverlap::nccl_all2all");
  // Variable-size all-to-all on packed rows: rank r sends mLen[r][i] rows to rank i and
  // receives mLen[i][r] rows from it; a rank's own rows are not part of C or D
  // (reference: src/overlap_impl.cu:181-212).
  if (world_ == 1) return;
  FO_CHECK(!mLen_CPU.is_cuda() && mLen_CPU.scalar_type() == at::kInt &&
                  mLen_CPU.numel() == static_cast<int64_t>(world_) * world_,
              "mLen_CPU must be an int32 host tensor of shape [world, world]");
  const int* ml = mLen_CPU.data_ptr<int>();
  const int64_t N = C.size(-1);
  const size_t es = C.element_size();
  char* src = static_cast<char*>(C.data_ptr());
  char* dst = static_cast<char*>(D.data_ptr());
  int64_t so = 0, ro = 0;
  FO_NCCL_CHECK(ncclGroupStart());
  for (int i = 0; i < world_; ++i) {
    if (i == rank_) continue;
    const int64_t sc = static_cast<int64_t>(ml[rank_ * world_ + i]) * N;
    const int64_t rc = static_cast<int64_t>(ml[i * world_ + rank_]) * N;
    FO_NCCL_CHECK(ncclSend(src + so * es, sc, nccl_dtype(C), i, comm_, stream()));
    FO_NCCL_CHECK(ncclRecv(dst + ro * es, rc, nccl_dtype(C), i, comm_, stream()));
    so += sc;
    ro += rc;
  }
  FO_NCCL_CHECK(ncclGroupEnd());
}

// ---------------------------------------------------------------------------- non-overlapped

void OverlapImpl::GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C, int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::gemm_allreduce");
  Gemm(A, B, C, Algo);
  NcclAllReduce(C);
}

void OverlapImpl::GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D,
                                    int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::gemm_reducescatter");
  Gemm(A, B, C, Algo);
  const int64_t recv = C.numel() / world_;
  check_out(D, A, recv, "D");
  if (world_ == 1) {
    cuda_check(cudaMemcpyAsync(D.data_ptr(), C.data_ptr(), recv * C.element_size(),
                               cudaMemcpyDeviceToDevice, stream()),
               "cudaMemcpyAsync");
    return;
  }
  FO_NCCL_CHECK(ncclReduceScatter(C.data_ptr(), D.data_ptr(), recv, nccl_dtype(C), ncclSum, comm_,
                                  stream()));
}

void OverlapImpl::GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, int64_t Algo,
                              at::Tensor mLen_CPU) {
  NvtxRange nvtx_range("flashoverlap::gemm_all2all");
  Gemm(A, B, C, Algo);
  NcclAll2All(C, D, mLen_CPU);
}

// ---------------------------------------------------------------------------- fused path

void OverlapImpl::ensure_fused_buffers(size_t stage_bytes, size_t nflags, bool pull) {
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  FO_CHECK(nflags <= kSignalMaxFlags, "too many tiles/groups for the flag region: ", nflags);
  if (signal_ == nullptr) signal_ = heap_->allocate(kSignalBytes, stream());
  const bool user_stage = pull && user_stage_ != nullptr && user_stage_->bytes >= stage_bytes;
  if (!user_stage && (stage_ == nullptr || stage_->bytes < stage_bytes)) {
    // A larger shape than any seen so far: take a new region, then give the old one back.  The
    // new region's handle exchange is a stream-ordered collective followed by a synchronise, so
    // every rank's earlier fused calls - the last users of the old region - have finished.
    SymmetricRegion* old = stage_;
    stage_ = heap_->allocate(stage_bytes, stream());
    if (old != nullptr) heap_->release(old, stream());
  }
}

void OverlapImpl::run_fused(int comm, const at::Tensor& A, const at::Tensor& B, at::Tensor out,
                            int out_mode, const int* RA, int rldn, int* MM, int mm_stride,
                            bool monitor, const int* cseg, int num_groups, int algo,
                            const at::Tensor* norm_w, double norm_eps, const at::Tensor* norm_res,
                            const at::Tensor* norm_out) {
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  c10::cuda::CUDAGuard guard(A.device());
  FO_CHECK(kBM % world_ == 0, "world size must divide the tile height 128");
  GemmTensorMaps maps;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  bool bf16 = true;
  setup_problem(algo, A, B, 0, &maps, &p, &bf16);
  FO_CHECK(rldn == 1 || comm == kCommFusedAR, "reduce-scatter requires rLDN == 1");

  const size_t full_bytes = static_cast<size_t>(p.M) * p.N * 2;
  const size_t nflags = (num_groups > 0 && cseg != nullptr) ? num_groups : p.num_tiles;
  // Pull protocol: partials stay in the producing rank's staging; a staging buffer with a
  // multicast mapping (use_stage) lets the switch do the summation.
  const bool pull = opt_stage_local_ != 0;
  ensure_fused_buffers(full_bytes, nflags, pull);

  const size_t out_bytes = comm == kCommFusedAR ? full_bytes : full_bytes / world_;
  check_out(out, A, static_cast<int64_t>(out_bytes / 2), comm == kCommFusedAR ? "C" : "D");
  bool copy_back = false;
  if (comm == kCommFusedAR) {
    const SymmetricRegion* reg = heap_->find(out.data_ptr(), out_bytes);
    if (reg != nullptr) {
      const size_t off = static_cast<char*>(out.data_ptr()) - static_cast<char*>(reg->local());
      for (int r = 0; r < world_; ++r) p.dst[r] = static_cast<char*>(reg->ptr[r]) + off;
      if (reg->multicast != nullptr && opt_nvls_ != 0) p.mc_dst = static_cast<char*>(reg->multicast) + off;
    } else {
      // The caller's tensor is ordinary device memory that peers cannot address: reduce into
      // a symmetric buffer and copy.  Allocate outputs with symm_empty to avoid the copy.
      if (out_ == nullptr || out_->bytes < out_bytes) {
        SymmetricRegion* old = out_;
        out_ = heap_->allocate(out_bytes, stream());
        if (old != nullptr) heap_->release(old, stream());
      }
      for (int r = 0; r < world_; ++r) p.dst[r] = out_->ptr[r];
      copy_back = true;
    }
  } else {
    p.dst[rank_] = out.data_ptr();
  }

  // The call number enters the kernel's handshakes; it is advanced only once nothing can
  // reject the call any more (directly before the launch, and taken back if the launch fails):
  // a call that throws must leave the object in step with its peers.
  const uint32_t epoch = epoch_ + 1;
  set_l2_hints(&p, opt_l2_hints_ != 0);
  p.out_mode = out_mode;
  p.rldn = rldn < 1 ? 1 : rldn;
  p.monitor = monitor ? 1 : 0;
  p.mm_stride = mm_stride;
  p.num_groups = (cseg != nullptr) ? num_groups : 0;
  p.comm = comm;
  p.ws = world_;
  p.rank_base = rank_;
  p.strided_rows = static_cast<int>(opt_strided_rows_);
  p.push_lag = opt_push_lag_ > 0 ? static_cast<int>(opt_push_lag_) : default_push_lag(p.K);
  p.epoch_done_prev = static_cast<uint32_t>(world_) * (epoch - 1);
  p.epoch_done = static_cast<uint32_t>(world_) * epoch;
  p.timeout_ns = static_cast<uint64_t>(opt_timeout_ms_) * 1000000ull;
  p.wait_sleep_ns = static_cast<uint32_t>(opt_wait_sleep_ns_);
  p.RA = RA;
  p.cseg = cseg;
  p.MM[0] = MM;
  p.status[0] = status_.data_ptr<int>();
  p.local_cnt[0] =
      reinterpret_cast<uint32_t*>(static_cast<char*>(signal_->local()) + kSignalLocalCntOffset);
  if (norm_w != nullptr) {
    FO_CHECK(comm == kCommFusedRS && out_mode == kOutNatural, "the RMSNorm tail needs a row-major reduce-scatter");
    FO_CHECK(norm_w->is_cuda() && norm_w->is_contiguous() && norm_w->scalar_type() == A.scalar_type() &&
                 norm_w->numel() == p.N,
             "W must be a contiguous CUDA tensor of N elements in the operands' dtype");
    const int64_t rows = p.M / world_;
    const auto f32 = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, device_);
    const auto i32 = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device_);
    if (!norm_ssq_.defined() || norm_ssq_.numel() < rows) norm_ssq_ = at::zeros({rows}, f32);
    if (!norm_cnt_.defined() || norm_cnt_.numel() < p.tiles_m) norm_cnt_ = at::zeros({p.tiles_m}, i32);
    p.norm_w = norm_w->data_ptr();
    p.norm_eps = static_cast<float>(norm_eps);
    if (norm_res != nullptr) {
      check_out(*norm_res, A, static_cast<int64_t>(out_bytes / 2), "R");
      p.norm_res[rank_] = norm_res->data_ptr();
    }
    if (norm_out != nullptr) {
      check_out(*norm_out, A, static_cast<int64_t>(out_bytes / 2), "Y");
      FO_CHECK(norm_out->data_ptr() != out.data_ptr(), "Y must not alias the residual stream");
      p.norm_out[rank_] = norm_out->data_ptr();
    }
    p.row_ssq = norm_ssq_.data_ptr<float>();
    p.panel_cnt = norm_cnt_.data_ptr<int>();
  }
  if (trace_.defined() && norm_w == nullptr) {
    FO_CHECK(trace_.numel() >= static_cast<int64_t>(p.num_tiles) * kTraceSlots,
             "the trace buffer needs ", static_cast<int64_t>(p.num_tiles) * kTraceSlots, " elements for this shape");
    p.trace = reinterpret_cast<unsigned long long*>(trace_.data_ptr<int64_t>());
  }
  const SymmetricRegion* stage =
      (pull && user_stage_ != nullptr && user_stage_->bytes >= full_bytes) ? user_stage_ : stage_;
  p.stage_local = pull ? 1 : 0;
  // Direct stores pay where the epilogue is exposed (the 256 x 256-per-CTA kernels, whose
  // accumulators fill TMEM); elsewhere the TMA hand-over costs fewer issue slots.
  p.pull_direct = (pull && (opt_pull_direct_ > 0 || (opt_pull_direct_ < 0 && algo_config(algo).mt == 2))) ? 1 : 0;
  p.epi_bufs = static_cast<int>(opt_epi_bufs_);
  p.diag = static_cast<int>(opt_diag_);
  if (pull && stage->multicast != nullptr && opt_nvls_ != 0) p.mc_stage = stage->multicast;
  for (int r = 0; r < world_; ++r) {
    p.stage[r] = stage->ptr[r];
    setup_stage_map(&maps, r, stage->ptr[r], p, world_, algo_config(algo).bn, pull);
    char* sig = static_cast<char*>(signal_->ptr[r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(sig + kSignalFlagsOffset);
    p.done[r] = reinterpret_cast<uint32_t*>(sig + kSignalDoneOffset);
  }
  const int grid = std::max(1, std::min(gemm_max_resident_ctas(algo, bf16, true), p.num_tiles));
  epoch_ = epoch;
  const cudaError_t launched = launch_gemm(algo, bf16, true, maps, p, grid, 1, false, stream());
  if (launched != cudaSuccess) epoch_ = epoch - 1;
  cuda_check(launched, "fused GEMM launch");
  if (copy_back) {
    cuda_check(cudaMemcpyAsync(out.data_ptr(), out_->local(), out_bytes, cudaMemcpyDeviceToDevice,
                               stream()),
               "cudaMemcpyAsync");
  }
}

void OverlapImpl::GemmAllReduceFused(at::Tensor A, at::Tensor B, at::Tensor C, int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::gemm_allreduce_fused");
  if (world_ == 1) {
    Gemm(A, B, C, Algo);
    return;
  }
  run_fused(kCommFusedAR, A, B, C, kOutNatural, nullptr, 1, nullptr, 0, false, nullptr, 0,
            static_cast<int>(Algo));
}

void OverlapImpl::GemmReduceScatterFused(at::Tensor A, at::Tensor B, at::Tensor D, int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::gemm_reducescatter_fused");
  if (world_ == 1) {
    Gemm(A, B, D, Algo);
    return;
  }
  run_fused(kCommFusedRS, A, B, D, kOutNatural, nullptr, 1, nullptr, 0, false, nullptr, 0,
            static_cast<int>(Algo));
}

void OverlapImpl::GemmReduceScatterRmsNormFused(at::Tensor A, at::Tensor B, at::Tensor Y, at::Tensor W,
                                                double eps, int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::gemm_reducescatter_rmsnorm_fused");
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  if (world_ == 1) {
    // One rank: nothing to reduce; GEMM, then the stand-alone RMSNorm.
    const GemmShape s = check_operands(A, B);
    FO_CHECK(W.is_cuda() && W.is_contiguous() && W.scalar_type() == A.scalar_type() && W.numel() == s.N,
             "W must be a contiguous CUDA tensor of N elements in the operands' dtype");
    check_out(Y, A, static_cast<int64_t>(s.M) * s.N, "Y");
    at::Tensor tmp = at::empty({s.M, s.N}, A.options());
    Gemm(A, B, tmp, Algo);
    cuda_check(rmsnorm_launch(tmp.data_ptr(), Y.data_ptr(), W.data_ptr(), s.M, s.N, static_cast<float>(eps), s.bf16,
                              sm_count_, stream()),
               "rmsnorm");
    return;
  }
  run_fused(kCommFusedRS, A, B, Y, kOutNatural, nullptr, 1, nullptr, 0, false, nullptr, 0,
            static_cast<int>(Algo), &W, eps);
}

void OverlapImpl::GemmReduceScatterAddRmsNormFused(at::Tensor A, at::Tensor B, at::Tensor R, at::Tensor Y,
                                                   at::Tensor W, double eps, int64_t Algo) {
  NvtxRange nvtx_range("flashoverlap::gemm_reducescatter_add_rmsnorm_fused");
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  if (world_ == 1) {
    // One rank: nothing to reduce; GEMM, residual add, then the stand-alone RMSNorm.
    const GemmShape s = check_operands(A, B);
    FO_CHECK(W.is_cuda() && W.is_contiguous() && W.scalar_type() == A.scalar_type() && W.numel() == s.N,
             "W must be a contiguous CUDA tensor of N elements in the operands' dtype");
    check_out(R, A, static_cast<int64_t>(s.M) * s.N, "R");
    check_out(Y, A, static_cast<int64_t>(s.M) * s.N, "Y");
    at::Tensor tmp = at::empty({s.M, s.N}, A.options());
    Gemm(A, B, tmp, Algo);
    at::Tensor r2 = R.view({s.M, s.N});
    r2.add_(tmp);
    cuda_check(rmsnorm_launch(r2.data_ptr(), Y.data_ptr(), W.data_ptr(), s.M, s.N, static_cast<float>(eps), s.bf16,
                              sm_count_, stream()),
               "rmsnorm");
    return;
  }
  run_fused(kCommFusedRS, A, B, R, kOutNatural, nullptr, 1, nullptr, 0, false, nullptr, 0,
            static_cast<int>(Algo), &W, eps, &R, &Y);
}

void OverlapImpl::GemmAll2AllFused(at::Tensor A, at::Tensor B, at::Tensor D, int64_t Algo,
                                   at::Tensor mLen_CPU) {
  NvtxRange nvtx_range("flashoverlap::gemm_all2all_fused");
  FO_CHECK(heap_ != nullptr, "call nccl_init first");
  FO_CHECK(!mLen_CPU.is_cuda() && mLen_CPU.scalar_type() == at::kInt && mLen_CPU.is_contiguous() &&
               mLen_CPU.numel() == static_cast<int64_t>(world_) * world_,
           "mLen_CPU must be a contiguous int32 host tensor of shape [world, world]");
  if (world_ == 1) return;  // a rank's own rows are not part of the exchange
  c10::cuda::CUDAGuard guard(A.device());
  const int algo = static_cast<int>(Algo);
  GemmTensorMaps maps;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  bool bf16 = true;
  setup_problem(algo, A, B, 0, &maps, &p, &bf16);

  const int* ml = mLen_CPU.data_ptr<int>();
  for (int i = 0; i < world_ * world_; ++i) FO_CHECK(ml[i] >= 0, "mLen_CPU holds a negative row count");
  const All2AllPlan plan = all2all_plan(ml, world_, rank_);
  FO_CHECK(plan.send_rows <= p.M, "mLen_CPU sends ", plan.send_rows, " rows but A has only ", p.M);
  check_out(D, A, plan.recv_rows * p.N, "D");

  // Destination addresses.  Every rank must take the same branch: D comes from symm_empty on
  // all ranks or on none.
  const size_t recv_bytes = static_cast<size_t>(plan.recv_rows) * p.N * 2;
  const SymmetricRegion* reg = heap_->find(D.data_ptr(), std::max<size_t>(recv_bytes, 1));
  bool copy_back = false;
  if (reg != nullptr) {
    const size_t off = static_cast<char*>(D.data_ptr()) - static_cast<char*>(reg->local());
    for (int r = 0; r < world_; ++r) p.dst[r] = static_cast<char*>(reg->ptr[r]) + off;
  } else {
    int64_t max_recv = 0;  // the scratch is one collective allocation: same size everywhere
    for (int r = 0; r < world_; ++r) max_recv = std::max(max_recv, all2all_plan(ml, world_, r).recv_rows);
    const size_t bytes = std::max<size_t>(static_cast<size_t>(max_recv) * p.N * 2, 256);
    if (out_ == nullptr || out_->bytes < bytes) {
      SymmetricRegion* old = out_;
      out_ = heap_->allocate(bytes, stream());
      if (old != nullptr) heap_->release(old, stream());
    }
    for (int r = 0; r < world_; ++r) p.dst[r] = out_->ptr[r];
    copy_back = true;
  }
  if (signal_ == nullptr) signal_ = heap_->allocate(kSignalBytes, stream());

  at::Tensor tab = at::zeros({2 * kMaxRanks}, at::TensorOptions().dtype(at::kInt));
  for (int d = 0; d < kMaxRanks; ++d) {
    tab.data_ptr<int>()[d] = plan.row_end[d];
    tab.data_ptr<int>()[kMaxRanks + d] = plan.dst_row[d];
  }
  a2a_tab_ = tab.to(at::Device(at::kCUDA, device_));

  set_l2_hints(&p, opt_l2_hints_ != 0);
  p.out_mode = kOutAll2All;
  p.rldn = 1;
  p.comm = kCommFusedA2A;
  p.ws = world_;
  p.rank_base = rank_;
  p.epoch_done = static_cast<uint32_t>(world_) * (epoch_ + 1);
  p.epoch_ready = static_cast<uint32_t>(world_) * (a2a_epoch_ + 1);
  p.timeout_ns = static_cast<uint64_t>(opt_timeout_ms_) * 1000000ull;
  p.wait_sleep_ns = static_cast<uint32_t>(opt_wait_sleep_ns_);
  p.a2a_tab = a2a_tab_.data_ptr<int>();
  p.status[0] = status_.data_ptr<int>();
  p.local_cnt[0] =
      reinterpret_cast<uint32_t*>(static_cast<char*>(signal_->local()) + kSignalLocalCntOffset);
  for (int r = 0; r < world_; ++r) {
    char* sig = static_cast<char*>(signal_->ptr[r]);
    p.done[r] = reinterpret_cast<uint32_t*>(sig + kSignalDoneOffset);
    p.ready[r] = reinterpret_cast<uint32_t*>(sig + kSignalReadyOffset);
  }
  const int grid = std::max(1, std::min(gemm_max_resident_ctas(algo, bf16, false), p.num_tiles));
  // the call numbers advance only with a launch that happened (see run_fused)
  ++epoch_;
  ++a2a_epoch_;
  const cudaError_t launched = launch_gemm(algo, bf16, false, maps, p, grid, 1, false, stream());
  if (launched != cudaSuccess) {
    --epoch_;
    --a2a_epoch_;
  }
  cuda_check(launched, "all-to-all GEMM launch");
  if (copy_back && recv_bytes > 0) {
    cuda_check(cudaMemcpyAsync(D.data_ptr(), out_->local(), recv_bytes, cudaMemcpyDeviceToDevice, stream()),
               "cudaMemcpyAsync");
  }
}

// ---------------------------------------------------------------------------- reference API

namespace {
int* mm_ptr(const at::Tensor& MM) {
  FO_CHECK(MM.is_cuda() && MM.scalar_type() == at::kInt && MM.is_contiguous(),
              "MM must be a contiguous int32 CUDA tensor");
  return MM.data_ptr<int>();
}
}  // namespace

// Sizes of the index arrays of an overlap call.  Every one of them is used as an address
// offset by the kernel, so a short array is an out-of-bounds access on the device: refuse it
// here.  With option "validate" the values are checked too (one device-to-host copy each).
void OverlapImpl::check_overlap_args(const char* what, int M, int N, int algo, const at::Tensor& MM,
                                     const at::Tensor& RA, const at::Tensor* RE, int64_t rLDN,
                                     const at::Tensor& cSEG_CPU, const at::Tensor& cSEG_GPU,
                                     bool monitor, bool needs_counters) const {
  FO_CHECK(algo >= 0 && algo < kNumAlgos, what, ": Algo ", algo, " out of range [0, ", kNumAlgos, ")");
  const AlgoConfig c = algo_config(algo);
  FO_CHECK(M % c.bm == 0 && N % c.bn == 0, what, ": M and N must be multiples of the tile (", c.bm, " x ", c.bn, ")");
  const int64_t tn = N / c.bn;
  const int64_t tiles = static_cast<int64_t>(M / c.bm) * tn;
  FO_CHECK(rLDN >= 1, what, ": rLDN must be at least 1");
  if (RA.defined() && RA.numel() > 0) {
    FO_CHECK(RA.numel() >= tiles, what, ": RA has ", RA.numel(), " entries, the shape has ", tiles, " tiles");
  }
  int64_t groups = 0;
  if (cSEG_GPU.defined() && cSEG_GPU.numel() > 0) {
    groups = cSEG_GPU.numel();
    FO_CHECK(groups <= tiles, what, ": more wave groups (", groups, ") than tiles (", tiles, ")");
    if (cSEG_CPU.defined() && cSEG_CPU.numel() > 0) {
      FO_CHECK(!cSEG_CPU.is_cuda() && cSEG_CPU.scalar_type() == at::kInt && cSEG_CPU.is_contiguous(),
               what, ": cSEG_CPU must be a contiguous int32 host tensor");
      FO_CHECK(cSEG_CPU.numel() == groups, what, ": cSEG_CPU and cSEG_GPU differ in length");
      const int* seg = cSEG_CPU.data_ptr<int>();
      int64_t sum = 0;
      for (int64_t i = 0; i < groups; ++i) {
        FO_CHECK(seg[i] > 0, what, ": cSEG_CPU[", i, "] = ", seg[i], " (groups hold at least one tile)");
        sum += seg[i];
      }
      FO_CHECK(sum == tiles, what, ": cSEG_CPU sums to ", sum, ", the shape has ", tiles, " tiles");
    }
  }
  if (monitor) {
    // row 0: counters (the completion counter is its last word), rows 1..: one word per tile
    FO_CHECK(MM.defined() && MM.numel() >= tn + tiles, what, ": in monitor mode MM needs (TM + 1) * TN = ",
             tn + tiles, " entries, it has ", MM.defined() ? MM.numel() : 0);
    FO_CHECK(!needs_counters || groups < tn, what, ": in monitor mode the group counters (", groups,
             ") must leave the last word of MM's first row (TN = ", tn, ") to the completion counter");
  } else if (needs_counters) {
    FO_CHECK(MM.defined() && MM.numel() >= std::max<int64_t>(groups, 1), what, ": MM has fewer counters (",
             MM.defined() ? MM.numel() : 0, ") than there are wave groups (", groups, ")");
  }
  if (RE != nullptr) {
    const int64_t rows = static_cast<int64_t>(M) * tn;  // rows of the [M * N / BN, BN] view
    FO_CHECK(RE->defined() && RE->numel() >= rows, what, ": RE needs M * N / BN = ", rows, " entries, it has ",
             RE->defined() ? RE->numel() : 0);
  }
  if (opt_validate_ == 0) return;
  // Deep validation (debug builds switch it on by default): the values, read back from the device.
  if (RA.defined() && RA.numel() > 0) {
    const at::Tensor h = RA.reshape({-1}).slice(0, 0, tiles).cpu();
    std::vector<char> seen(static_cast<size_t>(tiles), 0);
    const int* v = h.data_ptr<int>();
    for (int64_t t = 0; t < tiles; ++t) {
      FO_CHECK(v[t] >= 0 && v[t] < tiles, what, ": RA[", t, "] = ", v[t], " is not a tile position in [0, ", tiles, ")");
      FO_CHECK(!seen[v[t]], what, ": RA is not a permutation (position ", v[t], " appears twice)");
      seen[v[t]] = 1;
    }
  }
  if (groups > 0) {
    const at::Tensor h = cSEG_GPU.cpu();
    const int* v = h.data_ptr<int>();
    int64_t sum = 0;
    for (int64_t i = 0; i < groups; ++i) {
      FO_CHECK(v[i] > 0, what, ": cSEG_GPU[", i, "] = ", v[i]);
      sum += v[i];
    }
    FO_CHECK(sum == tiles, what, ": cSEG_GPU sums to ", sum, ", the shape has ", tiles, " tiles");
    if (cSEG_CPU.defined() && cSEG_CPU.numel() == groups) {
      const int* c = cSEG_CPU.data_ptr<int>();
      for (int64_t i = 0; i < groups; ++i) FO_CHECK(c[i] == v[i], what, ": cSEG_CPU and cSEG_GPU differ at ", i);
    }
  }
  if (RE != nullptr) {
    const int64_t rows = static_cast<int64_t>(M) * tn;
    const at::Tensor h = RE->reshape({-1}).slice(0, 0, rows).cpu();
    const int* v = h.data_ptr<int>();
    for (int64_t i = 0; i < rows; ++i) {
      FO_CHECK(v[i] >= 0 && v[i] < rows, what, ": RE[", i, "] = ", v[i], " is not a row in [0, ", rows, ")");
    }
  }
}

void OverlapImpl::GemmAllReduceOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor MM,
                                       at::Tensor RA, int64_t rLDN, at::Tensor cSEG_CPU,
                                       at::Tensor cSEG_GPU, int64_t Algo, bool if_monitor) {
  NvtxRange nvtx_range("flashoverlap::gemm_allreduce_overlap");
  const GemmShape s = check_operands(A, B);
  check_out(C, A, static_cast<int64_t>(s.M) * s.N, "C");
  check_overlap_args("gemm_allreduce_overlap", s.M, s.N, static_cast<int>(Algo), MM, RA, nullptr, rLDN, cSEG_CPU,
                     cSEG_GPU, if_monitor, opt_mode_ == 1 && world_ > 1);
  const AlgoConfig c = algo_config(static_cast<int>(Algo));
  const int tn = s.N / c.bn;
  const int* ra = int_ptr_or_null(RA, "RA");
  const int* cseg = int_ptr_or_null(cSEG_GPU, "cSEG_GPU");
  const int ngroups = cseg != nullptr ? static_cast<int>(cSEG_GPU.numel()) : 0;
  if (opt_mode_ == 1 && world_ > 1) {
    gated_overlap(kCommFusedAR, A, B, C, at::Tensor(), MM, RA, at::Tensor(), rLDN, cSEG_CPU,
                  cSEG_GPU, Algo, if_monitor);
    return;
  }
  if (world_ == 1) {
    // AllReduce over one rank is the identity: the reordered GEMM alone.
    run_plain(A, B, C.data_ptr(), kOutReorder, ra, nullptr, static_cast<int>(rLDN),
              if_monitor ? mm_ptr(MM) : nullptr, tn, false, if_monitor, cseg, ngroups,
              static_cast<int>(Algo), sm_count_);
    return;
  }
  run_fused(kCommFusedAR, A, B, C, kOutReorder, ra, static_cast<int>(rLDN),
            if_monitor ? mm_ptr(MM) : nullptr, tn, if_monitor, cseg, ngroups,
            static_cast<int>(Algo));
}

void OverlapImpl::GemmReduceScatterOverlap(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D,
                                           at::Tensor MM, at::Tensor RA, at::Tensor RE,
                                           int64_t rLDN, at::Tensor cSEG_CPU, at::Tensor cSEG_GPU,
                                           int64_t Algo, bool if_monitor) {
  NvtxRange nvtx_range("flashoverlap::gemm_reducescatter_overlap");
  const GemmShape s = check_operands(A, B);
  check_out(D, A, static_cast<int64_t>(s.M) * s.N / world_, "D");
  const bool gated = opt_mode_ == 1 && world_ > 1;
  check_overlap_args("gemm_reducescatter_overlap", s.M, s.N, static_cast<int>(Algo), MM, RA, gated ? &RE : nullptr,
                     rLDN, cSEG_CPU, cSEG_GPU, if_monitor, gated);
  const AlgoConfig c = algo_config(static_cast<int>(Algo));
  const int tn = s.N / c.bn;
  const int* ra = int_ptr_or_null(RA, "RA");
  const int* cseg = int_ptr_or_null(cSEG_GPU, "cSEG_GPU");
  const int ngroups = cseg != nullptr ? static_cast<int>(cSEG_GPU.numel()) : 0;
  FO_CHECK(rLDN == 1, "reduce-scatter requires rLDN == 1");
  if (opt_mode_ == 1 && world_ > 1) {
    gated_overlap(kCommFusedRS, A, B, C, D, MM, RA, RE, rLDN, cSEG_CPU, cSEG_GPU, Algo, if_monitor);
    return;
  }
  if (world_ == 1) {
    run_plain(A, B, D.data_ptr(), kOutReorder, ra, nullptr, 1, if_monitor ? mm_ptr(MM) : nullptr, tn,
              false, if_monitor, cseg, ngroups, static_cast<int>(Algo), sm_count_);
    return;
  }
  // C (the reference's full-size scratch) is not needed: partial tiles go straight to the
  // owners' staging memory.
  run_fused(kCommFusedRS, A, B, D, kOutReorder, ra, 1, if_monitor ? mm_ptr(MM) : nullptr, tn,
            if_monitor, cseg, ngroups, static_cast<int>(Algo));
}

// The reference's mechanism on our GEMM: signalling GEMM on the caller's stream; on the
// communication stream one bounded counting wait plus one NCCL call per wave group
// (src/overlap_impl.cu:247-263, :303-320).  Baseline for the fused kernels.
void OverlapImpl::gated_overlap(int comm, at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D,
                                at::Tensor MM, at::Tensor RA, at::Tensor RE, int64_t rLDN,
                                at::Tensor cSEG_CPU, at::Tensor cSEG_GPU, int64_t Algo,
                                bool monitor) {
  ensure_comm_stream();
  const GemmShape s = check_operands(A, B);
  check_out(C, A, static_cast<int64_t>(s.M) * s.N, "C");
  const AlgoConfig c = algo_config(static_cast<int>(Algo));
  const int tn = s.N / c.bn;
  const int tiles = (s.M / c.bm) * tn;
  FO_CHECK(!cSEG_CPU.is_cuda() && cSEG_CPU.scalar_type() == at::kInt, "cSEG_CPU: int32 host tensor");
  const int* seg = cSEG_CPU.data_ptr<int>();
  const int ngroups = static_cast<int>(cSEG_CPU.numel());
  const int* cseg_gpu = int_ptr_or_null(cSEG_GPU, "cSEG_GPU");
  FO_CHECK(ngroups > 0 && cseg_gpu != nullptr && cSEG_GPU.numel() == ngroups,
           "the counter-gated mode needs wave groups: cSEG_CPU and its device copy cSEG_GPU");
  int* mm = mm_ptr(MM);
  FO_CHECK(MM.numel() >= ngroups, "MM has fewer counters than there are groups");
  const bool rs = comm == kCommFusedRS;
  const int* re = rs ? int_ptr_or_null(RE, "RE") : nullptr;
  FO_CHECK(!rs || re != nullptr, "RE is required for reduce-scatter");

  cudaStream_t gs = stream();
  // Counters are consumed by this call only once the GEMM stream has reached this point
  // (the reference lets the two streams race from the start and relies on the counters
  // alone; ordering the streams also makes MM zeroing by earlier work safe).
  cuda_check(cudaEventRecord(gemm_start_, gs), "cudaEventRecord");
  cuda_check(cudaStreamWaitEvent(comm_stream_, gemm_start_, 0), "cudaStreamWaitEvent");

  run_plain(A, B, C.data_ptr(), rs ? kOutScatterRows : kOutReorder, int_ptr_or_null(RA, "RA"), re,
            static_cast<int>(rLDN), mm, tn, true, monitor, cseg_gpu, ngroups,
            static_cast<int>(Algo), sm_count_ - static_cast<int>(opt_sm_margin_));

  const size_t es = C.element_size();
  const int64_t tile_elems = static_cast<int64_t>(c.bm) * c.bn;
  char* cb = static_cast<char*>(C.data_ptr());
  char* db = rs ? static_cast<char*>(D.data_ptr()) : nullptr;
  const uint64_t timeout_ns = static_cast<uint64_t>(opt_timeout_ms_) * 1000000ull;
  int64_t acc = 0;
  int covered = 0;
  for (int g = 0; g < ngroups && covered < tiles; ++g) {
    const int64_t n = tile_elems * seg[g];
    cuda_check(wait_flag_launch(seg[g], mm + g, g, timeout_ns, status_.data_ptr<int>(), comm_stream_),
               "wait kernel launch");
    if (rs) {
      FO_NCCL_CHECK(ncclReduceScatter(cb + acc * es, db + (acc / world_) * es, n / world_,
                                      nccl_dtype(C), ncclSum, comm_, comm_stream_));
    } else {
      FO_NCCL_CHECK(ncclAllReduce(cb + acc * es, cb + acc * es, n, nccl_dtype(C), ncclSum, comm_,
                                  comm_stream_));
    }
    acc += n;
    covered += seg[g];
  }
  cuda_check(cudaEventRecord(comm_done_, comm_stream_), "cudaEventRecord");
  cuda_check(cudaStreamWaitEvent(gs, comm_done_, 0), "cudaStreamWaitEvent");
}

}  // namespace fo
