// Host/device-shared parameter block of the tcgen05 GEMM family and the table of tile
// configurations ("Algo" indices) that the JSON configs and the tuner refer to.
// The reference indexes 102 CUTLASS instantiations by an integer Algo
// (src/tiling/gemm_dispatcher.h:7-27, tool/generate_instances.py:5-45); here an Algo names a
// (BN, pipeline depth, CTA-pair mode, raster strip width) tuple of one hand-written kernel.
#pragma once
#include <cuda.h>
#include <cstdint>

namespace fo {

constexpr int kBM = 128;  // tile rows = UMMA M (one TMEM lane per row)
constexpr int kBK = 64;   // 64 x 16-bit = one 128-byte swizzle atom along K
constexpr int kMaxRanks = 8;
constexpr int kMaxVirtualRanks = 8;

enum OutMode : int {
  kOutNatural = 0,      // row-major [M, N]
  kOutReorder = 1,      // tile-contiguous, tile t at position RA[t] (reference layout)
  kOutScatterRows = 2,  // reorder + per-row remap through RE (reduce-scatter staging layout)
  kOutAll2All = 3,      // row m goes to the rank and row that a2a_tab assigns to it (all-to-all kernels)
};

enum CommMode : int {
  kCommNone = 0,
  kCommFusedAR = 2,
  kCommFusedRS = 3,
  kCommFusedA2A = 4,  // rows of C stored straight into the destination ranks' receive buffers
};

// One tensor map per virtual rank.  A launch normally carries one rank (gridDim.y == 1);
// the single-GPU emulation used by the tests runs several ranks' CTAs in one cooperative
// launch, each rank with its own operands.
struct GemmTensorMaps {
  CUtensorMap a[kMaxVirtualRanks];
  CUtensorMap b[kMaxVirtualRanks];
  // fused kernels: every rank's staging buffer viewed as [ws * tiles * rows_owned, BN], box
  // (rows_owned x 64): the epilogue's pushes are TMA stores through these.  Pull variant: this
  // rank's own staging viewed as [tiles * 128, BN], box (128 x 64).  Plain kernels: st[virtual
  // rank] is the output map of that rank (GemmParams::tma_out), box (128 x 64).
  CUtensorMap st[kMaxRanks];
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, num_tiles;
  int raster_sw;     // strip width (in N tiles) of the tile sweep
  int out_mode;      // OutMode
  int rldn;          // reordered layout: tiles per reordered row (reference rLDN, 1 in practice)
  int signal;        // bump MM[group] after each tile (counter-gated NCCL path)
  int monitor;       // record per-tile completion order in MM rows 1..TM
  int mm_stride;     // row length of MM (= tiles_n in the reference's callers)
  int num_groups;    // entries of cseg; 0 => one group per tile
  int comm;          // CommMode
  int ws;            // ranks taking part in the fused collective
  int rank_base;     // rank of virtual rank 0 of this launch
  int strided_rows;  // 1: row i of a tile belongs to rank i % ws (reference), 0: contiguous
  int diag;          // diagnostic switches (timing studies only): 1 skip the reduction's memory
                     // traffic, 2 skip the push stores, 4 skip the reducers' flag waits
  int push_lag;      // tiles whose pushes may be in flight before their arrival is signalled (1..4)
  uint32_t epoch_done_prev;  // value `done` must have reached before the first push
  uint32_t epoch_done;       // value `done` reaches when this call is complete everywhere
  uint64_t timeout_ns;       // bound for every cross-GPU wait
  uint64_t l2_hint_a;        // L2 eviction-priority policy of the A / B operand loads
  uint64_t l2_hint_b;
  const int* RA;             // [num_tiles] natural tile id -> reordered position (nullptr: identity)
  const int* RE;             // [M*N/BN] row remap for kOutScatterRows
  const int* cseg;           // [num_groups] tiles per group (device)
  // indexed by virtual rank
  void* out[kMaxVirtualRanks];          // plain/signalling output
  int* MM[kMaxVirtualRanks];            // counters / monitor matrix
  int32_t* status[kMaxVirtualRanks];    // status words
  uint32_t* local_cnt[kMaxVirtualRanks];  // CTAs of this rank that finished reducing
  // indexed by rank (peer-mapped addresses valid on the launching GPU)
  void* stage[kMaxRanks];      // staging: [src rank][tile][rows owned][BN] (pull variant: see stage_local)
  uint32_t* flags[kMaxRanks];  // per tile / per group arrival counters
  uint32_t* done[kMaxRanks];   // per-call completion counter
  void* dst[kMaxRanks];        // AllReduce: every rank's output; ReduceScatter: dst[rank] only
  void* mc_dst;                // AllReduce: multicast mapping of the output (NVLS), or nullptr
  // Pull variant of the fused collective: every rank keeps its partial tiles in its OWN staging
  // buffer, laid out [tile][owner][rows owned][BN], and the owners fetch them - with one
  // switch-side reduction per vector when the staging has a multicast mapping (mc_stage), else
  // with one peer load per rank.
  int stage_local;
  void* mc_stage;
  // Pull variant only: 1 = the epilogue threads store the partial tile into the local staging
  // themselves (16-byte stores, as the plain kernels do) and the push warp only announces it;
  // 0 = every chunk is handed to the push warp, which stores it with TMA.
  int pull_direct;
  // All-to-all kernels: [virtual rank][2][kMaxRanks] ints on the device.  Row 0: end (exclusive)
  // of the run of C rows bound for each rank, runs packed in rank order; row 1: the row of that
  // rank's receive buffer where this rank's run starts.  C rows past the last run go nowhere.
  const int* a2a_tab;
  // All-to-all kernels: ready[r] counts the ranks that have entered the current call (their
  // receive buffers may be overwritten from then on); nobody stores before it reaches epoch_ready.
  uint32_t* ready[kMaxRanks];
  uint32_t epoch_ready;
  // ReduceScatter with the RMSNorm tail fused into the reducers (row-major shard only): weight
  // [N] in the operands' type, per-row sums of squares [virtual rank][M / ws] (fp32, zero between
  // calls), per-row-panel counters of reduced tiles [virtual rank][tiles_m] (zero between calls).
  // norm_res (optional): residual [M / ws, N] added to the reduced rows before they are stored
  // and normalised (the stored rows are then the new residual stream; may alias the shard).
  // norm_out (optional): where the normalised rows go; nullptr = over the shard itself.
  float norm_eps;
  const void* norm_w;
  const void* norm_res[kMaxRanks];  // indexed by rank, like dst
  void* norm_out[kMaxRanks];
  float* row_ssq;
  int* panel_cnt;
  // Timeline of the fused kernels (tracing builds of the kernel only): [virtual rank][tile]
  // [kTraceSlots] nanosecond stamps, see TraceSlot.  nullptr: no tracing.
  unsigned long long* trace;
  // Fused kernels: 4 selects the build with four epilogue chunk buffers (and one operand stage
  // fewer), whose push warp keeps three chunks of stores in flight; anything else the default (2).
  int epi_bufs;
  // Plain kernels: 1 = GemmTensorMaps::st[virtual rank] describes the output as a 2-D tensor
  // (row-major [M, N], or the tile-contiguous layout as [M * N / (rldn * BN), rldn * BN]) and
  // finished chunks leave shared memory as TMA tensor stores; 0 = per-thread 16-byte stores.
  int tma_out;
  // Back-off of the roles that wait on mbarriers with slack (TMA producer, MMA issuer, push warp;
  // four times as long for the epilogue's wait for its accumulator): nanoseconds slept between
  // polls once a wait has turned out to be a long one.  0 = poll continuously.
  uint32_t wait_sleep_ns;
};

constexpr int kTraceSlots = 8;
enum TraceSlot : int {
  kTraceAccReady = 0,     // epilogue: the tile's accumulator is complete (main loop done)
  kTraceEpilogueDone = 1, // epilogue: last chunk handed to the push warp
  kTracePushIssued = 2,   // push warp: last store of the tile issued
  kTraceSignalled = 3,    // push warp: stores complete, owners' arrival counters bumped
  kTraceWaitBegin = 4,    // reducer: starts waiting for the tile's arrivals
  kTraceWaitEnd = 5,      // reducer: every rank's slice has arrived
  kTraceReduced = 6,      // reducer: reduction of the tile issued completely
  kTraceWhere = 7,        // (SM id << 32) | CTA index
};

// ------------------------------------------------------------------ Algo table
//
// Kernels (tile configurations that are template instantiations) and Algos ((kernel, raster
// strip) pairs) come from gemm/fo_gemm_instances.inc, which tool/generate_instances.py writes
// from tool/instances.json.  Adding a kernel or a raster there appends Algo numbers; existing
// numbers never change.

struct AlgoConfig {
  int bm, bn, bk;
  int stages;
  int raster_sw;  // 0 => full row panels (strip = all N tiles)
  int cta2;       // 1: CTA pairs share 256-row tiles through tcgen05.mma.cta_group::2
  int mt;         // 128-row halves per CTA (2: a pair covers 512 x 256, accumulators fill TMEM)
  int kernel;     // index of the kernel (template instantiation set) this Algo runs
};

struct KernelEntry {
  int bn, stages, cta2, mt, stages_epi4;
};
struct AlgoEntry {
  int kernel, raster_sw;
};

constexpr KernelEntry kKernelTable[] = {
#define FO_GEMM_KERNEL(idx, bn, stages, cta2, mt, stages_epi4) {bn, stages, (cta2) ? 1 : 0, mt, stages_epi4},
#include "fo_gemm_instances.inc"
#undef FO_GEMM_KERNEL
};
constexpr AlgoEntry kAlgoTable[] = {
#define FO_GEMM_ALGO(algo, kernel, raster) {kernel, raster},
#include "fo_gemm_instances.inc"
#undef FO_GEMM_ALGO
};
constexpr int kNumKernels = static_cast<int>(sizeof(kKernelTable) / sizeof(kKernelTable[0]));
constexpr int kNumAlgos = static_cast<int>(sizeof(kAlgoTable) / sizeof(kAlgoTable[0]));

inline int algo_kernel(int algo) {
  if (algo < 0 || algo >= kNumAlgos) algo = 0;
  return kAlgoTable[algo].kernel;
}

inline AlgoConfig algo_config(int algo) {
  if (algo < 0 || algo >= kNumAlgos) algo = 0;
  const AlgoEntry a = kAlgoTable[algo];
  const KernelEntry k = kKernelTable[a.kernel];
  AlgoConfig c;
  c.bm = kBM;
  c.bk = kBK;
  c.bn = k.bn;
  c.stages = k.stages;
  c.raster_sw = a.raster_sw;
  c.cta2 = k.cta2;
  c.mt = k.mt;
  c.kernel = a.kernel;
  return c;
}

}  // namespace fo
