// Torch registration: torch.classes.flashoverlap_class.{OverlapImpl,BaselineImpl} and
// torch.ops.flashoverlap_op.*, with the reference's method names and argument orders
// (src/pybind.cpp:114-150) plus the additions this library makes (marked below).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/library.h>

#include "common/fo_check.h"
#include "comm/nccl_utils.h"
#include "flags/fo_wait.h"
#include "norm/fo_norm.h"
#include "runtime/baseline_impl.h"
#include "runtime/fused_common.h"
#include "runtime/loopback.h"
#include "runtime/overlap_impl.h"

namespace {

using fo::BaselineImpl;
using fo::OverlapImpl;

int sm_count_of_current_device() {
  return at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
}

bool is_bf16(const at::Tensor& t, const char* name) {
  FO_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  FO_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf, name,
              " must be bfloat16 or float16");
  return t.scalar_type() == at::kBFloat16;
}

std::vector<int64_t> generate_nccl_id() { return fo::generate_nccl_id(); }

// X: tile-contiguous [rows*dim]; RX: row-major output [rows, dim]; RW: [dim].
void reorder_rmsnorm_eps(at::Tensor X, at::Tensor RX, at::Tensor RW, int64_t BM, int64_t BN,
                         int64_t rldn, at::Tensor RA, double eps) {
  const bool bf = is_bf16(X, "X");
  FO_CHECK(RX.scalar_type() == X.scalar_type() && RW.scalar_type() == X.scalar_type(),
              "X, RX and RW must share a dtype");
  FO_CHECK(RX.dim() == 2 && RX.is_contiguous() && RX.is_cuda(), "RX must be [rows, dim]");
  const int rows = static_cast<int>(RX.size(0));
  const int dim = static_cast<int>(RX.size(1));
  FO_CHECK(X.numel() >= RX.numel() && RW.numel() == dim, "shape mismatch");
  FO_CHECK(RA.is_cuda() && RA.scalar_type() == at::kInt && RA.is_contiguous() &&
                  RA.numel() >= static_cast<int64_t>(rows / BM) * (dim / BN),
              "RA must be an int32 CUDA tensor with one entry per tile");
  c10::cuda::CUDAGuard guard(X.device());
  fo::cuda_check(fo::reorder_rmsnorm_launch(X.data_ptr(), RX.data_ptr(), RW.data_ptr(), rows, dim,
                                            static_cast<int>(BM), static_cast<int>(BN),
                                            static_cast<int>(rldn), RA.data_ptr<int>(),
                                            static_cast<float>(eps), bf, sm_count_of_current_device(),
                                            c10::cuda::getCurrentCUDAStream().stream()),
                 "reorder_rmsnorm");
}

// Reference signature (src/pybind.cpp:149): eps fixed at 1e-5 as in src/rmsnorm/rmsnorm.cuh:102.
void reorder_rmsnorm(at::Tensor X, at::Tensor RX, at::Tensor RW, int64_t BM, int64_t BN,
                     int64_t rldn, at::Tensor RA) {
  reorder_rmsnorm_eps(X, RX, RW, BM, BN, rldn, RA, 1e-5);
}

void rmsnorm(at::Tensor X, at::Tensor RX, at::Tensor RW, double eps) {
  const bool bf = is_bf16(X, "X");
  FO_CHECK(RX.scalar_type() == X.scalar_type() && RW.scalar_type() == X.scalar_type(),
              "X, RX and RW must share a dtype");
  FO_CHECK(X.dim() == 2 && RX.sizes() == X.sizes() && RX.is_contiguous() && RX.is_cuda(),
              "X and RX must be [rows, dim]");
  const int rows = static_cast<int>(X.size(0));
  const int dim = static_cast<int>(X.size(1));
  FO_CHECK(RW.numel() == dim, "RW must have dim elements");
  c10::cuda::CUDAGuard guard(X.device());
  fo::cuda_check(fo::rmsnorm_launch(X.data_ptr(), RX.data_ptr(), RW.data_ptr(), rows, dim,
                                    static_cast<float>(eps), bf, sm_count_of_current_device(),
                                    c10::cuda::getCurrentCUDAStream().stream()),
                 "rmsnorm");
}

void reorder_impl(at::Tensor X, at::Tensor Y, int64_t rows, int64_t dim, int64_t BM, int64_t BN,
                  int64_t rldn, at::Tensor RA, bool to_reordered) {
  is_bf16(X, "X");
  FO_CHECK(Y.scalar_type() == X.scalar_type() && Y.is_cuda() && Y.is_contiguous(),
              "Y must match X's dtype");
  FO_CHECK(X.numel() == rows * dim && Y.numel() == rows * dim, "X and Y must hold rows*dim elements");
  FO_CHECK(RA.is_cuda() && RA.scalar_type() == at::kInt && RA.is_contiguous() &&
                  RA.numel() >= (rows / BM) * (dim / BN),
              "RA must be an int32 CUDA tensor with one entry per tile");
  c10::cuda::CUDAGuard guard(X.device());
  fo::cuda_check(fo::reorder_launch(X.data_ptr(), Y.data_ptr(), static_cast<int>(rows),
                                    static_cast<int>(dim), static_cast<int>(BM), static_cast<int>(BN),
                                    static_cast<int>(rldn), RA.data_ptr<int>(), to_reordered,
                                    sm_count_of_current_device(),
                                    c10::cuda::getCurrentCUDAStream().stream()),
                 "reorder");
}

// Y (tile-contiguous) <- X (row-major [rows, dim]).
void reorder(at::Tensor X, at::Tensor Y, int64_t BM, int64_t BN, int64_t rldn, at::Tensor RA) {
  FO_CHECK(X.dim() == 2, "X must be [rows, dim]");
  reorder_impl(X, Y, X.size(0), X.size(1), BM, BN, rldn, RA, true);
}

// Y (row-major [rows, dim]) <- X (tile-contiguous).
void unreorder(at::Tensor X, at::Tensor Y, int64_t BM, int64_t BN, int64_t rldn, at::Tensor RA) {
  FO_CHECK(Y.dim() == 2, "Y must be [rows, dim]");
  reorder_impl(X, Y, Y.size(0), Y.size(1), BM, BN, rldn, RA, false);
}

// Bounded counting wait on MM[index] (see flags/fo_wait.h); status: int32[8] CUDA tensor.
void wait_flag(int64_t target, at::Tensor MM, int64_t index, int64_t timeout_ms, at::Tensor status) {
  FO_CHECK(MM.is_cuda() && MM.scalar_type() == at::kInt && MM.is_contiguous() &&
                  index >= 0 && index < MM.numel(),
              "MM must be an int32 CUDA tensor and index in range");
  FO_CHECK(status.is_cuda() && status.scalar_type() == at::kInt &&
                  status.numel() >= fo::kStatusWords,
              "status must be an int32 CUDA tensor with 8 words");
  c10::cuda::CUDAGuard guard(MM.device());
  fo::cuda_check(fo::wait_flag_launch(static_cast<int>(target), MM.data_ptr<int>() + index,
                                      static_cast<int>(index),
                                      static_cast<uint64_t>(timeout_ms) * 1000000ull,
                                      status.data_ptr<int>(),
                                      c10::cuda::getCurrentCUDAStream().stream()),
                 "wait_flag");
}

// Flattened Algo table: for each Algo index (BM, BN, BK, stages, raster strip width, CTA pair,
// row halves per CTA).
std::vector<int64_t> algo_table() {
  std::vector<int64_t> t;
  for (int a = 0; a < fo::kNumAlgos; ++a) {
    const fo::AlgoConfig c = fo::algo_config(a);
    t.insert(t.end(), {c.bm, c.bn, c.bk, c.stages, c.raster_sw, c.cta2, c.mt});
  }
  return t;
}

// Row tables of the fused all-to-all for one rank: row_end[8], dst_row[8], rows sent, rows
// received (see all2all_plan in runtime/fused_common.h).  Host only.
std::vector<int64_t> all2all_plan(at::Tensor mLen_CPU, int64_t rank) {
  FO_CHECK(!mLen_CPU.is_cuda() && mLen_CPU.scalar_type() == at::kInt && mLen_CPU.is_contiguous() &&
               mLen_CPU.dim() == 2 && mLen_CPU.size(0) == mLen_CPU.size(1) &&
               mLen_CPU.size(0) <= fo::kMaxRanks,
           "mLen_CPU must be a contiguous square int32 host tensor of at most 8 x 8");
  const int ws = static_cast<int>(mLen_CPU.size(0));
  FO_CHECK(rank >= 0 && rank < ws, "rank out of range");
  const fo::All2AllPlan plan = fo::all2all_plan(mLen_CPU.data_ptr<int>(), ws, static_cast<int>(rank));
  std::vector<int64_t> out;
  for (int d = 0; d < fo::kMaxRanks; ++d) out.push_back(plan.row_end[d]);
  for (int d = 0; d < fo::kMaxRanks; ++d) out.push_back(plan.dst_row[d]);
  out.push_back(plan.send_rows);
  out.push_back(plan.recv_rows);
  return out;
}

// The exception text check_status() produces for a block of status words (host only).
std::string status_message(std::vector<int64_t> words, int64_t rank) {
  FO_CHECK(static_cast<int>(words.size()) >= fo::kStatusWords, "a status block has ", fo::kStatusWords, " words");
  if (words[fo::kStatusWordCode] == fo::kStatusOk) return "";
  return fo::status_message(words.data(), static_cast<int>(rank));
}

}  // namespace

TORCH_LIBRARY(flashoverlap_class, m) {
  m.class_<BaselineImpl>("BaselineImpl")
      .def(torch::init())
      .def("nccl_init", &BaselineImpl::NcclInit)
      .def("cublas_init", &BaselineImpl::CublasInit)
      .def("gemm_allreduce", &BaselineImpl::GemmAllReduce)
      .def("gemm_reducescatter", &BaselineImpl::GemmReduceScatter)
      .def("gemm_all2all", &BaselineImpl::GemmAll2All)
      .def("cublas_gemm", &BaselineImpl::Gemm)
      .def("nccl_allreduce", &BaselineImpl::NcclAllReduce)
      .def("nccl_reducescatter", &BaselineImpl::NcclReduceScatter)
      .def("nccl_all2all", &BaselineImpl::NcclAll2All);
  m.class_<OverlapImpl>("OverlapImpl")
      .def(torch::init())
      .def("cutlass_init", &OverlapImpl::CutlassInit)
      .def("cutlass_gemm", &OverlapImpl::Gemm)
      .def("gemm_allreduce_overlap", &OverlapImpl::GemmAllReduceOverlap)
      .def("gemm_reducescatter_overlap", &OverlapImpl::GemmReduceScatterOverlap)
      .def("nccl_init", &OverlapImpl::NcclInit)
      .def("gemm_allreduce", &OverlapImpl::GemmAllReduce)
      .def("gemm_reducescatter", &OverlapImpl::GemmReduceScatter)
      .def("gemm_all2all", &OverlapImpl::GemmAll2All)
      .def("overlap_init", &OverlapImpl::OverlapInit)
      .def("nccl_allreduce", &OverlapImpl::NcclAllReduce)
      .def("nccl_reducescatter", &OverlapImpl::NcclReduceScatter)
      .def("nccl_all2all", &OverlapImpl::NcclAll2All)
      .def("seg_allreduce", &OverlapImpl::SegAllReduce)
      // additions
      .def("gemm_allreduce_fused", &OverlapImpl::GemmAllReduceFused)
      .def("gemm_reducescatter_fused", &OverlapImpl::GemmReduceScatterFused)
      .def("gemm_all2all_fused", &OverlapImpl::GemmAll2AllFused)
      .def("gemm_reducescatter_rmsnorm_fused", &OverlapImpl::GemmReduceScatterRmsNormFused)
      .def("gemm_reducescatter_add_rmsnorm_fused", &OverlapImpl::GemmReduceScatterAddRmsNormFused)
      .def("set_option", &OverlapImpl::SetOption)
      .def("get_option", &OverlapImpl::GetOption)
      .def("symm_empty", &OverlapImpl::SymmEmpty)
      .def("register_symmetric", &OverlapImpl::RegisterSymmetric)
      .def("use_stage", &OverlapImpl::UseStage)
      .def("set_trace", &OverlapImpl::SetTrace)
      .def("read_status", &OverlapImpl::ReadStatus)
      .def("check_status", &OverlapImpl::CheckStatus)
      .def("reset_status", &OverlapImpl::ResetStatus)
      .def("resync", &OverlapImpl::Resync)
      .def("wait_flag", &OverlapImpl::WaitFlag);
}

TORCH_LIBRARY(flashoverlap_op, m) {
  m.def("generate_nccl_id", &generate_nccl_id);
  m.def("reorder_rmsnorm", &reorder_rmsnorm);
  // additions
  m.def("reorder_rmsnorm_eps", &reorder_rmsnorm_eps);
  m.def("rmsnorm", &rmsnorm);
  m.def("reorder", &reorder);
  m.def("unreorder", &unreorder);
  m.def("wait_flag", &wait_flag);
  m.def("algo_table", &algo_table);
  m.def("fused_loopback", &fo::fused_loopback);
  m.def("all2all_plan", &all2all_plan);
  m.def("status_message", &status_message);
}
