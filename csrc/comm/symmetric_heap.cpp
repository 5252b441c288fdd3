#include "symmetric_heap.h"

#include <cstring>
#include <stdexcept>
#include <string>

#include "nccl_utils.h"

namespace fo {

namespace {
void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("CUDA failure in ") + what + ": " + cudaGetErrorString(e));
  }
}
}  // namespace

SymmetricHeap::SymmetricHeap(int rank, int world, ncclComm_t comm, bool loopback)
    : rank_(rank), world_(world), comm_(comm), loopback_(loopback) {
  if (world_ > 1 && !loopback_ && comm_ == nullptr) {
    throw std::runtime_error("SymmetricHeap needs an NCCL communicator to exchange IPC handles");
  }
}

SymmetricHeap::~SymmetricHeap() {
  for (auto& r : regions_) {
    if (!r->owned) continue;
    for (int i = 0; i < static_cast<int>(r->ptr.size()); ++i) {
      if (r->ptr[i] == nullptr) continue;
      if (r->loopback || i == r->rank) {
        cudaFree(r->ptr[i]);
      } else {
        cudaIpcCloseMemHandle(r->ptr[i]);
      }
    }
  }
}

SymmetricRegion* SymmetricHeap::allocate(size_t bytes, cudaStream_t stream) {
  auto region = std::make_unique<SymmetricRegion>();
  region->bytes = bytes;
  region->rank = rank_;
  region->loopback = loopback_;
  region->ptr.assign(world_, nullptr);

  if (loopback_ || world_ == 1) {
    for (int r = 0; r < world_; ++r) {
      cuda_check(cudaMalloc(&region->ptr[r], bytes), "cudaMalloc(symmetric loopback)");
      cuda_check(cudaMemsetAsync(region->ptr[r], 0, bytes, stream), "cudaMemsetAsync");
    }
    cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    regions_.push_back(std::move(region));
    return regions_.back().get();
  }

  void* local = nullptr;
  cuda_check(cudaMalloc(&local, bytes), "cudaMalloc(symmetric)");
  region->ptr[rank_] = local;
  cuda_check(cudaMemsetAsync(local, 0, bytes, stream), "cudaMemsetAsync");

  cudaIpcMemHandle_t mine;
  cuda_check(cudaIpcGetMemHandle(&mine, local), "cudaIpcGetMemHandle");

  // All-gather the handles through the communicator (device buffers, then back to host).
  const size_t hs = sizeof(cudaIpcMemHandle_t);
  char* dev = nullptr;
  cuda_check(cudaMalloc(reinterpret_cast<void**>(&dev), hs * (world_ + 1)), "cudaMalloc(handles)");
  cuda_check(cudaMemcpyAsync(dev, &mine, hs, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync");
  FO_NCCL_CHECK(ncclAllGather(dev, dev + hs, hs, ncclChar, comm_, stream));
  std::vector<cudaIpcMemHandle_t> all(world_);
  cuda_check(cudaMemcpyAsync(all.data(), dev + hs, hs * world_, cudaMemcpyDeviceToHost, stream),
             "cudaMemcpyAsync");
  cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
  cudaFree(dev);

  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    void* p = nullptr;
    cuda_check(cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess),
               "cudaIpcOpenMemHandle");
    region->ptr[r] = p;
  }
  // Nobody may touch a peer's copy before that peer has finished zero-filling it: the
  // all-gather above ran after each rank's memset on the same stream, and every rank has
  // synchronised that stream, so all copies are cleared by now.
  regions_.push_back(std::move(region));
  return regions_.back().get();
}

void SymmetricHeap::release(SymmetricRegion* region, cudaStream_t stream) {
  size_t idx = regions_.size();
  for (size_t i = 0; i < regions_.size(); ++i) {
    if (regions_[i].get() == region) idx = i;
  }
  if (idx == regions_.size()) return;  // not ours
  if (region->owned) {
    if (region->loopback || world_ == 1) {
      for (void* p : region->ptr) {
        if (p != nullptr) cudaFree(p);
      }
    } else {
      for (int r = 0; r < world_; ++r) {
        if (r != rank_ && region->ptr[r] != nullptr) cudaIpcCloseMemHandle(region->ptr[r]);
      }
      // nobody frees before everybody has unmapped
      int* token = nullptr;
      cuda_check(cudaMalloc(reinterpret_cast<void**>(&token), sizeof(int)), "cudaMalloc(token)");
      cuda_check(cudaMemsetAsync(token, 0, sizeof(int), stream), "cudaMemsetAsync");
      FO_NCCL_CHECK(ncclAllReduce(token, token, 1, ncclInt, ncclSum, comm_, stream));
      cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
      cudaFree(token);
      cudaFree(region->ptr[rank_]);
    }
  }
  regions_.erase(regions_.begin() + static_cast<long>(idx));
}

SymmetricRegion* SymmetricHeap::adopt(size_t bytes, const std::vector<void*>& ptrs, void* multicast) {
  auto region = std::make_unique<SymmetricRegion>();
  region->bytes = bytes;
  region->rank = rank_;
  region->ptr = ptrs;
  region->owned = false;
  region->multicast = multicast;
  regions_.push_back(std::move(region));
  return regions_.back().get();
}

const SymmetricRegion* SymmetricHeap::find(const void* p, size_t n) const {
  for (const auto& r : regions_) {
    if (r->contains(p, n)) return r.get();
  }
  return nullptr;
}

}  // namespace fo
