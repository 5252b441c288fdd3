#include "baseline_impl.h"

#include <c10/cuda/CUDAStream.h>

#include "../comm/nccl_utils.h"
#include "fused_common.h"

namespace fo {

namespace {
ncclDataType_t nccl_dtype(const at::Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return ncclBfloat16;
  if (t.scalar_type() == at::kHalf) return ncclFloat16;
  if (t.scalar_type() == at::kFloat) return ncclFloat32;
  FO_CHECK(false, "unsupported dtype for a collective");
  return ncclFloat16;
}
}  // namespace

BaselineImpl::BaselineImpl() {}

BaselineImpl::~BaselineImpl() {
  if (comm_ != nullptr) ncclCommDestroy(comm_);
}

cudaStream_t BaselineImpl::stream() const { return c10::cuda::getCurrentCUDAStream().stream(); }

void BaselineImpl::NcclInit(int64_t rank, int64_t world, std::vector<int64_t> id) {
  FO_CHECK(world >= 1 && rank >= 0 && rank < world, "bad rank/world");
  FO_CHECK(comm_ == nullptr, "nccl_init was already called");
  rank_ = static_cast<int>(rank);
  world_ = static_cast<int>(world);
  if (world_ > 1) {
    ncclUniqueId uid = unpack_nccl_id(id);
    FO_NCCL_CHECK(ncclCommInitRank(&comm_, world_, uid, rank_));
  }
}

void BaselineImpl::CublasInit() {
  // ATen's cuBLAS handle is already bound to the current stream with tensor-op math; the
  // reference has to do this by hand (src/baseline_impl.cu:184-190).
}

void BaselineImpl::Gemm(at::Tensor A, at::Tensor B, at::Tensor C) {
  const GemmShape s = check_operands(A, B);
  check_out(C, A, static_cast<int64_t>(s.M) * s.N, "C");
  at::Tensor c2 = C.view({s.M, s.N});
  at::mm_out(c2, A, B.t());  // cuBLAS / cuBLASLt, 16-bit in and out, fp32 accumulate
}

void BaselineImpl::NcclAllReduce(at::Tensor C) {
  if (world_ == 1) return;
  FO_NCCL_CHECK(ncclAllReduce(C.data_ptr(), C.data_ptr(), C.numel(), nccl_dtype(C), ncclSum, comm_,
                              stream()));
}

void BaselineImpl::NcclReduceScatter(at::Tensor C) {
  if (world_ == 1) return;
  const int64_t recv = C.numel() / world_;
  char* base = static_cast<char*>(C.data_ptr());
  FO_NCCL_CHECK(ncclReduceScatter(base, base + rank_ * recv * C.element_size(), recv, nccl_dtype(C),
                                  ncclSum, comm_, stream()));
}

void BaselineImpl::NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU) {
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

void BaselineImpl::GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C) {
  Gemm(A, B, C);
  NcclAllReduce(C);
}

void BaselineImpl::GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D) {
  Gemm(A, B, C);
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

void BaselineImpl::GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D,
                               at::Tensor mLen_CPU) {
  Gemm(A, B, C);
  NcclAll2All(C, D, mLen_CPU);
}

}  // namespace fo
