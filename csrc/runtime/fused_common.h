// Pieces shared by the runtime classes and the single-GPU loopback driver: the layout of the
// symmetric "signal" region, operand checks and the GemmParams set-up of one call.
#pragma once
#include <ATen/ATen.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>

#include <string>

#include "../comm/symmetric_heap.h"
#include "../common/fo_check.h"
#include "../common/fo_status.h"
#include "../gemm/fo_gemm.h"

namespace fo {

// Signal region layout (bytes).  `done` and `local_cnt` sit on separate 128-byte lines so
// that remote atomics on one never contend with local atomics on the other.
constexpr size_t kSignalDoneOffset = 0;
constexpr size_t kSignalLocalCntOffset = 128;
constexpr size_t kSignalReadyOffset = 256;  // all-to-all: ranks that have entered the current call
constexpr size_t kSignalFlagsOffset = 1024;
constexpr size_t kSignalMaxFlags = 65536;
constexpr size_t kSignalBytes = kSignalFlagsOffset + kSignalMaxFlags * sizeof(uint32_t);

inline void cuda_check(cudaError_t e, const char* what) {
  FO_CHECK(e == cudaSuccess, "CUDA failure in ", what, ": ", cudaGetErrorString(e));
}

struct GemmShape {
  int M, N, K;
  bool bf16;
};

// A [M,K], B [N,K] (weight layout), both contiguous, same 16-bit floating type.
inline GemmShape check_operands(const at::Tensor& A, const at::Tensor& B) {
  FO_CHECK(A.is_cuda() && B.is_cuda(), "A and B must be CUDA tensors");
  FO_CHECK(A.dim() == 2 && B.dim() == 2, "A must be [M,K] and B must be [N,K]");
  FO_CHECK(A.is_contiguous() && B.is_contiguous(), "A and B must be contiguous");
  FO_CHECK(A.scalar_type() == B.scalar_type(), "A and B must have the same dtype");
  FO_CHECK(A.scalar_type() == at::kBFloat16 || A.scalar_type() == at::kHalf,
              "only bfloat16 and float16 operands are supported");
  FO_CHECK(A.size(1) == B.size(1), "A [M,K] and B [N,K] disagree on K");
  GemmShape s;
  s.M = static_cast<int>(A.size(0));
  s.K = static_cast<int>(A.size(1));
  s.N = static_cast<int>(B.size(0));
  s.bf16 = A.scalar_type() == at::kBFloat16;
  return s;
}

inline void check_out(const at::Tensor& C, const at::Tensor& A, int64_t numel, const char* name) {
  FO_CHECK(C.is_cuda() && C.is_contiguous(), name, " must be a contiguous CUDA tensor");
  FO_CHECK(C.scalar_type() == A.scalar_type(), name, " must have the operands' dtype");
  FO_CHECK(C.numel() >= numel, name, " is too small: needs ", numel, " elements");
}

inline const int* int_ptr_or_null(const at::Tensor& t, const char* name) {
  if (!t.defined() || t.numel() == 0) return nullptr;
  FO_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), name,
              " must be a contiguous int32 CUDA tensor");
  return t.data_ptr<int>();
}

// Shape, tiling and tensor maps for virtual rank `vr` of a launch.
inline void setup_problem(int algo, const at::Tensor& A, const at::Tensor& B, int vr,
                          GemmTensorMaps* maps, GemmParams* p, bool* bf16) {
  const GemmShape s = check_operands(A, B);
  if (vr == 0) {
    p->M = s.M;
    p->N = s.N;
    p->K = s.K;
    const std::string err = prepare_tiling(algo, p);
    FO_CHECK(err.empty(), err, " (M=", s.M, " N=", s.N, " K=", s.K, " Algo=", algo, ")");
    *bf16 = s.bf16;
  } else {
    FO_CHECK(p->M == s.M && p->N == s.N && p->K == s.K && *bf16 == s.bf16,
                "all ranks of a loopback launch must use the same shape and dtype");
  }
  const AlgoConfig c = algo_config(algo);
  std::string e = encode_tmap_16bit(&maps->a[vr], A.data_ptr(), s.M, s.K, kBM);
  FO_CHECK(e.empty(), "A: ", e);
  e = encode_tmap_16bit(&maps->b[vr], B.data_ptr(), s.N, s.K, c.cta2 ? c.bn / 2 : c.bn);
  FO_CHECK(e.empty(), "B: ", e);
}

// Tensor map over one rank's staging buffer for the push warp's TMA stores.
// Push protocol: [ws * tiles * rows_owned, BN] 16-bit elements, box rows_owned x 64 (one owner's
// slice of a chunk).  Pull protocol (`stage_local`): [tiles * 128, BN], box 128 x 64 (a whole chunk).
inline void setup_stage_map(GemmTensorMaps* maps, int rank, void* stage, const GemmParams& p, int ws, int bn,
                            bool stage_local = false) {
  const int rows_owned = kBM / ws;
  const std::string e =
      stage_local ? encode_tmap_16bit(&maps->st[rank], stage, static_cast<uint64_t>(p.num_tiles) * kBM, bn, kBM)
                  : encode_tmap_16bit(&maps->st[rank], stage,
                                      static_cast<uint64_t>(ws) * p.num_tiles * rows_owned, bn, rows_owned);
  FO_CHECK(e.empty(), "staging map: ", e);
}

// Output map of a plain kernel for virtual rank `vr`: the row-major [M, N] output, or the
// tile-contiguous layout viewed as [M * N / (rldn * BN), rldn * BN], box 128 x 64.  Sets
// p->tma_out when the layout can be described that way; otherwise the kernel keeps its
// per-thread stores (row-scatter and all-to-all outputs, a tile count that rldn does not divide,
// an output whose address is not 16-byte aligned).
inline void setup_out_map(GemmTensorMaps* maps, int vr, void* out, GemmParams* p, int bn) {
  if (vr == 0) p->tma_out = 0;
  uint64_t cols = 0;
  if (p->out_mode == kOutNatural) {
    cols = static_cast<uint64_t>(p->N);
  } else if (p->out_mode == kOutReorder && p->rldn >= 1 && p->num_tiles % p->rldn == 0) {
    cols = static_cast<uint64_t>(p->rldn) * bn;
  } else {
    return;
  }
  const uint64_t rows = static_cast<uint64_t>(p->M) * p->N / cols;
  const std::string e = encode_tmap_16bit(&maps->st[vr], out, rows, cols, kBM);
  if (e.empty()) {
    if (vr == 0) p->tma_out = 1;
  } else {
    p->tma_out = 0;
  }
}

// Send/receive plan of the variable-size all-to-all on packed rows for rank `me`
// (reference semantics, src/overlap_impl.cu:181-212): mlen is the row-major [ws, ws] matrix of
// row counts, rank r sends mlen[r][i] rows to rank i, the runs for the other ranks are packed in
// rank order in C, the runs received from the other ranks are packed in rank order in D, and a
// rank's own run is part of neither.
struct All2AllPlan {
  int row_end[kMaxRanks];  // end (exclusive) of the run of C rows bound for each rank
  int dst_row[kMaxRanks];  // first row of that rank's D that this rank's run lands on
  int64_t send_rows;       // C rows that go anywhere
  int64_t recv_rows;       // D rows that arrive here
};

inline All2AllPlan all2all_plan(const int* mlen, int ws, int me) {
  All2AllPlan plan;
  int64_t acc = 0;
  for (int d = 0; d < kMaxRanks; ++d) {
    if (d < ws && d != me) acc += mlen[me * ws + d];
    FO_CHECK(acc < (1ll << 31), "all-to-all row counts overflow 32 bits");
    plan.row_end[d] = static_cast<int>(acc);
    int64_t before = 0;
    for (int j = 0; j < me && d < ws; ++j) {
      if (j != d) before += mlen[j * ws + d];
    }
    plan.dst_row[d] = static_cast<int>(before);
  }
  plan.send_rows = acc;
  plan.recv_rows = 0;
  for (int j = 0; j < ws; ++j) {
    if (j != me) plan.recv_rows += mlen[j * ws + me];
  }
  return plan;
}

}  // namespace fo
