#include "loopback.h"

#include <c10/cuda/CUDAGuard.h>

#include <cstdlib>
#include <cstring>

#include "fused_common.h"

namespace fo {

std::vector<int64_t> fused_loopback(std::string comm_op, std::vector<at::Tensor> A,
                                    std::vector<at::Tensor> B, std::vector<at::Tensor> out,
                                    c10::optional<at::Tensor> RA_opt,
                                    c10::optional<at::Tensor> cseg_opt, int64_t algo,
                                    bool strided_rows, bool natural_out, int64_t repeat,
                                    int64_t timeout_ms, bool stage_local) {
  const at::Tensor RA = RA_opt.has_value() ? *RA_opt : at::Tensor();
  const at::Tensor cseg_gpu = cseg_opt.has_value() ? *cseg_opt : at::Tensor();
  const int ws = static_cast<int>(A.size());
  FO_CHECK(ws >= 2 && ws <= kMaxVirtualRanks, "loopback supports 2..", kMaxVirtualRanks, " ranks");
  FO_CHECK(static_cast<int>(B.size()) == ws && static_cast<int>(out.size()) == ws,
              "A, B and out must have one tensor per rank");
  FO_CHECK(kBM % ws == 0, "rank count must divide 128");
  int comm;
  if (comm_op == "all_reduce") {
    comm = kCommFusedAR;
  } else if (comm_op == "reduce_scatter") {
    comm = kCommFusedRS;
  } else {
    FO_CHECK(false, "comm_op must be 'all_reduce' or 'reduce_scatter'");
    comm = kCommFusedAR;
  }
  c10::cuda::CUDAGuard guard(A[0].device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
  int dev = 0;
  cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  cudaDeviceProp prop;
  cuda_check(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties");

  FO_CHECK(!algo_config(static_cast<int>(algo)).cta2,
           "the loopback emulation runs single-CTA Algos only (Algo & 3 != 1)");
  GemmTensorMaps maps;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  bool bf16 = true;
  for (int r = 0; r < ws; ++r) setup_problem(static_cast<int>(algo), A[r], B[r], r, &maps, &p, &bf16);

  const int* cseg = int_ptr_or_null(cseg_gpu, "cseg_gpu");
  const int ngroups = cseg != nullptr ? static_cast<int>(cseg_gpu.numel()) : 0;
  const size_t nflags = ngroups > 0 ? ngroups : p.num_tiles;
  FO_CHECK(nflags <= kSignalMaxFlags, "too many flags");
  const size_t full_bytes = static_cast<size_t>(p.M) * p.N * 2;
  const int64_t out_elems = comm == kCommFusedAR ? static_cast<int64_t>(p.M) * p.N
                                                 : static_cast<int64_t>(p.M) * p.N / ws;
  for (int r = 0; r < ws; ++r) check_out(out[r], A[r], out_elems, "out");

  SymmetricHeap heap(0, ws, nullptr, /*loopback=*/true);
  SymmetricRegion* stage = heap.allocate(full_bytes, stream);
  SymmetricRegion* signal = heap.allocate(kSignalBytes, stream);
  at::Tensor status =
      at::zeros({ws * kStatusWords}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev));

  set_l2_hints(&p, false);
  p.out_mode = natural_out ? kOutNatural : kOutReorder;
  p.rldn = 1;
  p.num_groups = ngroups;
  p.comm = comm;
  p.ws = ws;
  p.rank_base = 0;
  p.strided_rows = strided_rows ? 1 : 0;
  p.push_lag = default_push_lag(p.K);
  p.stage_local = stage_local ? 1 : 0;
  if (const char* d = std::getenv("FLASHOVERLAP_DIAG")) p.diag = std::atoi(d);  // timing studies only
  p.timeout_ns = static_cast<uint64_t>(timeout_ms) * 1000000ull;
  p.RA = int_ptr_or_null(RA, "RA");
  p.cseg = cseg;
  for (int r = 0; r < ws; ++r) {
    p.status[r] = status.data_ptr<int>() + r * kStatusWords;
    char* sig = static_cast<char*>(signal->ptr[r]);
    p.local_cnt[r] = reinterpret_cast<uint32_t*>(sig + kSignalLocalCntOffset);
    p.stage[r] = stage->ptr[r];
    setup_stage_map(&maps, r, stage->ptr[r], p, ws, algo_config(static_cast<int>(algo)).bn, stage_local);
    p.flags[r] = reinterpret_cast<uint32_t*>(sig + kSignalFlagsOffset);
    p.done[r] = reinterpret_cast<uint32_t*>(sig + kSignalDoneOffset);
    p.dst[r] = out[r].data_ptr();
  }
  const int per_rank = std::max(1, std::min(prop.multiProcessorCount / ws, p.num_tiles));
  for (int64_t it = 1; it <= repeat; ++it) {
    p.epoch_done_prev = static_cast<uint32_t>(ws) * static_cast<uint32_t>(it - 1);
    p.epoch_done = static_cast<uint32_t>(ws) * static_cast<uint32_t>(it);
    cuda_check(launch_gemm(static_cast<int>(algo), bf16, true, maps, p, per_rank, ws,
                           /*cooperative=*/true, stream),
               "loopback fused launch");
  }
  cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
  at::Tensor h = status.cpu();
  std::vector<int64_t> res(ws * kStatusWords);
  for (int i = 0; i < ws * kStatusWords; ++i) res[i] = h.data_ptr<int>()[i];
  return res;
}

}  // namespace fo
