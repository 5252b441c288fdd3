// fo_fused_loopback_noalloc: the fused GEMM+collective emulation with its scratch in a static
// device array instead of cudaMalloc'd memory (see fo_noalloc.h for who needs that and why).
#include "fo_noalloc.h"

#include <cstdio>
#include <cstring>

#include "../common/fo_status.h"
#include "../gemm/fo_gemm.h"

namespace {

constexpr size_t kSignalFlagsOffset = 1024;  // done counter at +0, finished-CTA counter at +128
constexpr size_t kSignalBytesPerRank = kSignalFlagsOffset + FO_NOALLOC_MAX_TILES * sizeof(uint32_t);
constexpr size_t kControlBytes = 128u << 10;  // counters + status words of all ranks
constexpr size_t kStatusOffset = FO_NOALLOC_MAX_RANKS * kSignalBytesPerRank;
constexpr size_t kScratchBytes = FO_NOALLOC_MAX_STAGING_BYTES + kControlBytes;
static_assert(kStatusOffset + FO_NOALLOC_MAX_RANKS * fo::kStatusWords * sizeof(int32_t) <= kControlBytes,
              "control block too small");

// Layout: [control block | staging of rank 0 | staging of rank 1 | ...].  In host code this
// name is only a handle for cudaGetSymbolAddress, never an address to hand to a kernel.
static __device__ __align__(256) unsigned char fo_noalloc_scratch[kScratchBytes];

unsigned char* g_scratch[16] = {};

int fail(int code, char* err, size_t n, const char* msg) {
  if (err != nullptr && n > 0) std::snprintf(err, n, "%s", msg);
  return code;
}

}  // namespace

extern "C" int fo_fused_loopback_noalloc(int comm_op, int ranks, const void* const* A,
                                         const void* const* B, void* const* out, int M, int N,
                                         int K, int bf16, int algo, int strided_rows,
                                         cudaStream_t stream, char* err, size_t err_len) {
  using namespace fo;
  if (err != nullptr && err_len > 0) err[0] = 0;
  if (comm_op != 0 && comm_op != 1) return fail(-1, err, err_len, "comm_op must be 0 (all_reduce) or 1 (reduce_scatter)");
  if (ranks < 2 || ranks > FO_NOALLOC_MAX_RANKS || kBM % ranks != 0)
    return fail(-1, err, err_len, "ranks must be 2 or 4");
  if (A == nullptr || B == nullptr || out == nullptr) return fail(-1, err, err_len, "null pointer table");
  if (algo < 0 || algo >= kNumAlgos || algo_config(algo).cta2)
    return fail(-1, err, err_len, "algo must be a single-CTA Algo index ((Algo & 1) == 0)");
  if (M <= 0 || N <= 0 || K <= 0) return fail(-1, err, err_len, "M, N and K must be positive");

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K = K;
  const std::string tiling_err = prepare_tiling(algo, &p);
  if (!tiling_err.empty()) return fail(-1, err, err_len, tiling_err.c_str());
  const size_t stage_per_rank = static_cast<size_t>(M) * N * 2;
  if (stage_per_rank * ranks > FO_NOALLOC_MAX_STAGING_BYTES)
    return fail(-2, err, err_len, "ranks * M * N * 2 bytes exceeds the built-in staging scratch (16 MiB)");
  if (p.num_tiles > FO_NOALLOC_MAX_TILES)
    return fail(-2, err, err_len, "more output tiles than built-in arrival counters (4096)");

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16)
    return fail(-3, err, err_len, "cudaGetDevice failed or device index >= 16");
  if (g_scratch[dev] == nullptr) {
    // One-time set-up for this device, with this device current.
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, fo_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) return fail(-3, err, err_len, cudaGetErrorString(e));
    g_scratch[dev] = static_cast<unsigned char*>(ptr);
  }
  unsigned char* control = g_scratch[dev];
  unsigned char* staging = control + kControlBytes;

  GemmTensorMaps maps;
  const AlgoConfig cfg = algo_config(algo);
  for (int r = 0; r < ranks; ++r) {
    if (A[r] == nullptr || B[r] == nullptr || out[r] == nullptr) return fail(-1, err, err_len, "null operand");
    std::string e = encode_tmap_16bit(&maps.a[r], A[r], M, K, kBM);
    if (e.empty()) e = encode_tmap_16bit(&maps.b[r], B[r], N, K, cfg.bn);
    if (!e.empty()) return fail(-1, err, err_len, e.c_str());
  }

  // Counters and status words must start at zero; the staging contents need no clearing
  // (every slice is written before its arrival counter lets anyone read it).
  cudaError_t ce = cudaMemsetAsync(control, 0, kControlBytes, stream);
  if (ce != cudaSuccess) return fail(-3, err, err_len, cudaGetErrorString(ce));

  set_l2_hints(&p, false);
  p.out_mode = kOutNatural;
  p.rldn = 1;
  p.comm = comm_op == 0 ? kCommFusedAR : kCommFusedRS;
  p.ws = ranks;
  p.rank_base = 0;
  p.strided_rows = strided_rows ? 1 : 0;
  p.push_lag = default_push_lag(K);
  p.epoch_done_prev = 0;
  p.epoch_done = static_cast<uint32_t>(ranks);
  p.timeout_ns = 2000000000ull;
  for (int r = 0; r < ranks; ++r) {
    unsigned char* sig = control + r * kSignalBytesPerRank;
    p.done[r] = reinterpret_cast<uint32_t*>(sig);
    p.local_cnt[r] = reinterpret_cast<uint32_t*>(sig + 128);
    p.flags[r] = reinterpret_cast<uint32_t*>(sig + kSignalFlagsOffset);
    p.status[r] = reinterpret_cast<int32_t*>(control + kStatusOffset) + r * kStatusWords;
    p.stage[r] = staging + r * stage_per_rank;
    {
      const std::string e = encode_tmap_16bit(&maps.st[r], p.stage[r],
                                              static_cast<uint64_t>(ranks) * p.num_tiles * (kBM / ranks), cfg.bn,
                                              kBM / ranks);
      if (!e.empty()) return fail(-1, err, err_len, e.c_str());
    }
    p.dst[r] = out[r];
  }
  cudaDeviceProp prop;
  ce = cudaGetDeviceProperties(&prop, dev);
  if (ce != cudaSuccess) return fail(-3, err, err_len, cudaGetErrorString(ce));
  int per_rank = prop.multiProcessorCount / ranks;
  if (per_rank > p.num_tiles) per_rank = p.num_tiles;
  if (per_rank < 1) per_rank = 1;
  ce = launch_gemm(algo, bf16 != 0, /*fused=*/true, maps, p, per_rank, ranks, /*cooperative=*/true, stream);
  if (ce != cudaSuccess) return fail(-3, err, err_len, cudaGetErrorString(ce));

  int32_t host_status[FO_NOALLOC_MAX_RANKS * kStatusWords] = {};
  ce = cudaMemcpyAsync(host_status, control + kStatusOffset, sizeof(int32_t) * ranks * kStatusWords,
                       cudaMemcpyDeviceToHost, stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(stream);
  if (ce != cudaSuccess) return fail(-3, err, err_len, cudaGetErrorString(ce));
  for (int r = 0; r < ranks; ++r) {
    const int32_t code = host_status[r * kStatusWords + kStatusWordCode];
    if (code != kStatusOk) return fail(code, err, err_len, status_name(code));
  }
  return 0;
}
