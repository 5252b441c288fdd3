// Vendor baseline: library GEMM (cuBLAS through ATen, fp32 accumulation) followed on the same
// stream by one NCCL collective.  Same method set as the reference class
// (src/baseline_impl.h:10-34, bound at src/pybind.cpp:117-128).  Never used by product paths.
#pragma once
#include <ATen/ATen.h>
#include <cuda_runtime.h>
#include <nccl.h>
#include <torch/custom_class.h>

#include <vector>

namespace fo {

class BaselineImpl : public torch::CustomClassHolder {
 public:
  BaselineImpl();
  ~BaselineImpl() override;
  void NcclInit(int64_t rank, int64_t world, std::vector<int64_t> id);
  void CublasInit();
  void GemmAllReduce(at::Tensor A, at::Tensor B, at::Tensor C);
  void GemmReduceScatter(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D);
  void GemmAll2All(at::Tensor A, at::Tensor B, at::Tensor C, at::Tensor D, at::Tensor mLen_CPU);
  void Gemm(at::Tensor A, at::Tensor B, at::Tensor C);
  void NcclAllReduce(at::Tensor C);
  void NcclReduceScatter(at::Tensor C);
  void NcclAll2All(at::Tensor C, at::Tensor D, at::Tensor mLen_CPU);

 private:
  cudaStream_t stream() const;
  int rank_ = 0;
  int world_ = 1;
  ncclComm_t comm_ = nullptr;
};

}  // namespace fo
