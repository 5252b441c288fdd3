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
                                    int64_t timeout_ms, bool stage_local,
                                    c10::optional<at::Tensor> mlen_opt,
                                    c10::optional<at::Tensor> norm_w, double norm_eps,
                                    c10::optional<at::Tensor> trace, int64_t epi_bufs, int64_t pull_direct,
                                    c10::optional<std::vector<at::Tensor>> norm_res,
                                    c10::optional<std::vector<at::Tensor>> norm_out) {
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
  } else if (comm_op == "all_to_all") {
    comm = kCommFusedA2A;
  } else {
    FO_CHECK(false, "comm_op must be 'all_reduce', 'reduce_scatter' or 'all_to_all'");
    comm = kCommFusedAR;
  }
  c10::cuda::CUDAGuard guard(A[0].device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
  int dev = 0;
  cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  cudaDeviceProp prop;
  cuda_check(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties");

  FO_CHECK(!algo_config(static_cast<int>(algo)).cta2,
           "the loopback emulation runs single-CTA Algos only (no CTA-pair kernels)");
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
  const bool a2a = comm == kCommFusedA2A;
  at::Tensor tab;  // all-to-all row tables of every virtual rank
  if (a2a) {
    FO_CHECK(mlen_opt.has_value(), "all_to_all needs mlen");
    const at::Tensor& mlen = *mlen_opt;
    FO_CHECK(!mlen.is_cuda() && mlen.scalar_type() == at::kInt && mlen.is_contiguous() &&
                 mlen.numel() == static_cast<int64_t>(ws) * ws,
             "mlen must be a contiguous int32 host tensor of shape [ranks, ranks]");
    at::Tensor host = at::zeros({ws * 2 * kMaxRanks}, at::TensorOptions().dtype(at::kInt));
    for (int r = 0; r < ws; ++r) {
      const All2AllPlan plan = all2all_plan(mlen.data_ptr<int>(), ws, r);
      FO_CHECK(plan.send_rows <= p.M, "mlen sends more rows than A has");
      check_out(out[r], A[r], plan.recv_rows * p.N, "out");
      for (int d = 0; d < kMaxRanks; ++d) {
        host.data_ptr<int>()[(r * 2 + 0) * kMaxRanks + d] = plan.row_end[d];
        host.data_ptr<int>()[(r * 2 + 1) * kMaxRanks + d] = plan.dst_row[d];
      }
    }
    tab = host.to(at::Device(at::kCUDA, dev));
  } else {
    const int64_t out_elems = comm == kCommFusedAR ? static_cast<int64_t>(p.M) * p.N
                                                   : static_cast<int64_t>(p.M) * p.N / ws;
    for (int r = 0; r < ws; ++r) check_out(out[r], A[r], out_elems, "out");
  }

  SymmetricHeap heap(0, ws, nullptr, /*loopback=*/true);
  SymmetricRegion* stage = heap.allocate(a2a ? 256 : full_bytes, stream);
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
  p.pull_direct = (stage_local && pull_direct != 0) ? 1 : 0;
  FO_CHECK(epi_bufs == 2 || epi_bufs == 4, "epi_bufs must be 2 or 4");
  p.epi_bufs = static_cast<int>(epi_bufs);
  if (a2a) {
    p.out_mode = kOutAll2All;
    p.a2a_tab = tab.data_ptr<int>();
  }
  if (trace.has_value() && trace->numel() > 0) {
    FO_CHECK(!a2a && !norm_w.has_value(), "the timeline is recorded by the fused AllReduce / ReduceScatter kernels");
    FO_CHECK(trace->is_cuda() && trace->is_contiguous() && trace->scalar_type() == at::kLong &&
                 trace->numel() >= static_cast<int64_t>(ws) * p.num_tiles * kTraceSlots,
             "trace must be a contiguous int64 CUDA tensor of ranks * tiles * 8 elements");
    p.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr<int64_t>());
  }
  at::Tensor row_ssq, panel_cnt;  // RMSNorm tail: statistics of every virtual rank
  if (norm_w.has_value()) {
    FO_CHECK(comm == kCommFusedRS && natural_out, "the RMSNorm tail needs a row-major reduce-scatter");
    FO_CHECK(norm_w->is_cuda() && norm_w->is_contiguous() && norm_w->scalar_type() == A[0].scalar_type() &&
                 norm_w->numel() == p.N,
             "norm_w must be a contiguous CUDA tensor of N elements in the operands' dtype");
    row_ssq = at::zeros({static_cast<int64_t>(p.M)}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, dev));
    panel_cnt = at::zeros({static_cast<int64_t>(ws) * p.tiles_m},
                          at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev));
    p.norm_w = norm_w->data_ptr();
    p.norm_eps = static_cast<float>(norm_eps);
    p.row_ssq = row_ssq.data_ptr<float>();
    p.panel_cnt = panel_cnt.data_ptr<int>();
    const int64_t shard = static_cast<int64_t>(p.M / ws) * p.N;
    if (norm_res.has_value()) {
      FO_CHECK(static_cast<int>(norm_res->size()) == ws, "norm_res needs one tensor per rank");
      for (int r = 0; r < ws; ++r) {
        check_out((*norm_res)[r], A[0], shard, "norm_res");
        p.norm_res[r] = (*norm_res)[r].data_ptr();
      }
    }
    if (norm_out.has_value()) {
      FO_CHECK(static_cast<int>(norm_out->size()) == ws, "norm_out needs one tensor per rank");
      for (int r = 0; r < ws; ++r) {
        check_out((*norm_out)[r], A[0], shard, "norm_out");
        p.norm_out[r] = (*norm_out)[r].data_ptr();
      }
    }
  } else {
    FO_CHECK(!norm_res.has_value() && !norm_out.has_value(), "norm_res / norm_out belong to the RMSNorm tail (norm_w)");
  }
  if (const char* d = std::getenv("FLASHOVERLAP_DIAG")) p.diag = std::atoi(d);  // timing studies only
  p.timeout_ns = static_cast<uint64_t>(timeout_ms) * 1000000ull;
  p.wait_sleep_ns = 0;
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
    p.ready[r] = reinterpret_cast<uint32_t*>(sig + kSignalReadyOffset);
    p.dst[r] = out[r].data_ptr();
  }
  const int per_rank = std::max(1, std::min(prop.multiProcessorCount / ws, p.num_tiles));
  for (int64_t it = 1; it <= repeat; ++it) {
    p.epoch_done_prev = static_cast<uint32_t>(ws) * static_cast<uint32_t>(it - 1);
    p.epoch_done = static_cast<uint32_t>(ws) * static_cast<uint32_t>(it);
    p.epoch_ready = p.epoch_done;
    cuda_check(launch_gemm(static_cast<int>(algo), bf16, /*fused=*/!a2a, maps, p, per_rank, ws,
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
