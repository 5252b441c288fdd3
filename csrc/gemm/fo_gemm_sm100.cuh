// Persistent, warp-specialised tcgen05 GEMM for B200 (sm_100a) with three kinds of epilogue:
//
//   * plain      C = A * B^T written row-major, tile-contiguous ("reordered") or row-scattered;
//   * signalling the same plus a per-wave-group counter bump (and an optional completion-order
//                monitor) once a tile is globally visible - the producer half of the
//                counter-gated NCCL path the reference is built around
//                (reference: src/overlap/gemm_with_signal.h:210-256, :338-361);
//   * fused      the tile's bf16/fp16 partial sums are pushed, row slice by row slice, straight
//                into the owning peer GPU's staging buffer over NVLink, the owner's reducer
//                warps (in the same kernel) sum the `ws` partials in fp32 as soon as every
//                rank's slice has landed, and write the result to every rank's output
//                (AllReduce) or to the local shard (ReduceScatter).  This replaces the
//                reference's GEMM + wait kernel + NCCL call (src/overlap_impl.cu:214-321).
//
// Roles inside a CTA (one CTA per SM, 128 x BN output tiles, BK = 64):
//   warp 0      TMA producer: 2-D tiled loads (128-byte swizzle, one CTA per copy) into a
//               STAGES-deep shared-memory ring, completion counted on mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma.kind::f16 (fp32 accumulate in TMEM),
//               tcgen05.commit releases ring slots and publishes finished accumulators;
//               this warp also owns the TMEM allocation (2 accumulators of BN columns);
//               (warps 0 and 1 walk their loops with all lanes, waits included, and a lane
//               chosen by elect.sync issues: warp-uniform control flow lets the compiler keep
//               counters, addresses and descriptors in uniform registers)
//   warps 2-5   epilogue: tcgen05.ld -> convert -> swizzled shared-memory transpose ->
//               128-byte coalesced global (local or peer) stores, then the signal;
//   warps 6-9   (fused only) reducer for the row slices this rank owns;
//   warp 10     (fused only) push: one thread turns every finished shared-memory chunk into TMA
//               stores to the owning ranks' staging memory (or this rank's own, pull protocol)
//               and, once a tile's stores have completed, hands the tile to the signal warp.
//               Waiting for remote completion happens here, off the epilogue's critical path;
//   warp 11     (fused only) signal: one thread publishes finished tiles - a system-scope
//               release fence, then relaxed atomics on the owners' arrival counters.  The fence
//               waits for every remote write the SM has in flight, which is why it has a warp
//               of its own: on the push warp it stalled the epilogue for a whole tile period.
// The two TMEM accumulators let tile i's epilogue run under tile i+1's main loop.
//
// CTA2 variant: two CTAs of a cluster (adjacent SMs) share one 256 x 256 tile through
// tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A and its own 128 of the 256
// rows of B, the leader CTA's MMA thread issues for both, and each CTA ends up with the
// accumulators of its own 128 x 256 half, so epilogue, signalling and reducer are unchanged.
// Halving the B traffic per SM is what lifts the kernel to library-GEMM throughput.
//
// MT = 2 (with CTA2): each CTA owns TWO 128-row halves that share its B tile - a 512 x 256 tile
// per pair, 256 x 256 per CTA.  Operand bytes per FLOP drop by a quarter and the number of
// waves halves (less DRAM re-reading), which buys clock under the power cap; the price is that
// the two accumulators fill TMEM, so a tile's epilogue no longer overlaps the next main loop.
// Worth it when the main loop is long (K per rank in the several thousands).
//
// Compile-time variants (template flags; the default builds contain none of their code):
//   A2A    plain kernel whose epilogue stores each row into the receive buffer of the rank it
//          is bound for (fused GEMM + all-to-all), with start- and end-of-call handshakes;
//   NORM   fused reduce-scatter whose reducers also gather each row's sum of squares and
//          normalise a 128-row panel when its last tile has been reduced (RMSNorm tail);
//   TRACE  fused kernels that stamp the life cycle of every tile for a timeline;
//   EPI    number of epilogue chunk buffers of the fused kernels (2, or 4 with one operand
//          stage fewer and three chunks of push stores in flight).
// Run-time variant: the pull protocol (GemmParams::stage_local), where partial tiles stay in
// the producing rank's staging buffer and the owners fetch them - with one multimem.ld_reduce
// per vector when the staging has an NVSwitch multicast mapping.
//
// Every wait is bounded: on expiry the role records a status code, raises a CTA-wide abort
// flag, the producer drains its TMA loads in flight, TMEM is freed and the kernel returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/fo_ptx.cuh"
#include "fo_gemm_params.h"

namespace fo {

// Tiles that the push warp may have handed to the signal warp without their arrival having been
// announced yet (fused kernels).
constexpr int kSigRing = 8;

template <int BN, int STAGES, bool CTA2 = false, int MT = 1, int EPI = 2>
struct GemmSmem {
  static constexpr int kAHalfBytes = kBM * kBK * 2;
  static constexpr int kABytes = MT * kAHalfBytes;
  static constexpr int kBRows = CTA2 ? BN / 2 : BN;  // B rows this CTA loads per k-block
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiBufBytes = kBM * 128;  // 128 rows x 64 16-bit columns
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kEpiOffset = kRingBytes;
  static constexpr int kBarOffset = kEpiOffset + EPI * kEpiBufBytes;  // EPI epilogue chunk buffers
  // + chunk_ready[EPI], chunk_free[EPI], sig_full[kSigRing], sig_empty[kSigRing]
  static constexpr int kNumBars = 2 * STAGES + 4 + 2 * EPI + 2 * kSigRing;
  static constexpr int kMiscOffset = kBarOffset + kNumBars * 8;
  static constexpr int kMiscBytes = 128;
  // +1024: the ring is aligned up to 1024 B at run time (128-byte swizzle atom).
  static constexpr int kTotalBytes = kMiscOffset + kMiscBytes + 1024;
};

struct TileCoord {
  int m, n;
};

// Position in the launch order -> tile coordinates.  Tiles are swept in column strips
// `sw` tiles wide, M-major inside a strip; sw == tiles_n gives row-panel-major order.
__device__ __forceinline__ TileCoord tile_of_position(int pos, int tiles_m, int tiles_n, int sw) {
  const int per_strip = tiles_m * sw;
  const int s = pos / per_strip;
  const int q = pos - s * per_strip;
  const int w = min(sw, tiles_n - s * sw);
  TileCoord c;
  c.m = q / w;
  c.n = s * sw + (q - c.m * w);
  return c;
}

// Wave group of reordered position r: groups are runs of cseg[g] consecutive positions.
__device__ __forceinline__ void group_of_position(const GemmParams& p, int r, int* g, int* need) {
  // No grouping, or as many groups as tiles (every group then holds exactly one tile).
  if (p.num_groups <= 0 || p.cseg == nullptr || p.num_groups == p.num_tiles) {
    *g = r;
    *need = 1;
    return;
  }
  int acc = 0, i = 0, n = 1;
  for (; i < p.num_groups; ++i) {
    n = p.cseg[i];
    acc += n;
    if (r < acc) break;
  }
  if (i >= p.num_groups) i = p.num_groups - 1;
  *g = i;
  *need = n;
}

// Reordered position of natural tile t.  A value outside [0, tiles) - a corrupted RA, or one
// built for another shape - would become an out-of-range address and counter index: it is
// reported (kStatusBadArgument) and replaced by t, so the kernel stays inside its buffers;
// the result is then wrong and the status words say why.
__device__ __forceinline__ int tile_position(const GemmParams& p, int t, int32_t* status) {
  if (p.RA == nullptr) return t;
  const int r = p.RA[t];
  if (static_cast<unsigned>(r) >= static_cast<unsigned>(p.num_tiles)) {
    ptx::report_status(status, kStatusBadArgument, 1, t, r);
    return t;
  }
  return r;
}

constexpr int kEpilogueThreads = 128;
constexpr int kReducerThreads = 128;
constexpr int kThreadsPlain = 64 + kEpilogueThreads;
constexpr int kThreadsFused = kThreadsPlain + kReducerThreads + 64;  // + push warp + signal warp

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool BF16>
__device__ __forceinline__ void unpack_add(uint32_t w, float& lo, float& hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
    float2 f = __bfloat1622float2(v);
    lo += f.x;
    hi += f.y;
  } else {
    __half2 v = *reinterpret_cast<__half2*>(&w);
    float2 f = __half22float2(v);
    lo += f.x;
    hi += f.y;
  }
}


// y = round16(round16(x * scale) * w), the arithmetic of the stand-alone RMSNorm kernels.
template <bool BF16>
__device__ __forceinline__ uint32_t norm_scale_mul2(uint32_t x, uint32_t w, float scale) {
  float lo = 0.f, hi = 0.f;
  unpack_add<BF16>(x, lo, hi);
  if constexpr (BF16) {
    __nv_bfloat162 n = __floats2bfloat162_rn(lo * scale, hi * scale);
    __nv_bfloat162 r = __hmul2(n, *reinterpret_cast<__nv_bfloat162*>(&w));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __half2 n = __floats2half2_rn(lo * scale, hi * scale);
    __half2 r = __hmul2(n, *reinterpret_cast<__half2*>(&w));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}

// round16(a + b) per 16-bit pair, added in fp32: what `a + b` on 16-bit tensors computes.
template <bool BF16>
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
  float lo = 0.f, hi = 0.f;
  unpack_add<BF16>(a, lo, hi);
  unpack_add<BF16>(b, lo, hi);
  return pack2<BF16>(lo, hi);
}

// Where the reduced vectors of one tile go.  AllReduce: every rank's output (one multimem.st
// when the output has an NVSwitch multicast mapping, else one peer store per rank).
// ReduceScatter: the local shard.  With NORM (reduce-scatter into the row-major shard) the sink
// also adds the optional residual and gathers each row's sum of squares of the stored values,
// as a separate norm kernel would see them.  Vector v of a tile slice is its bytes
// [16 v, 16 v + 16): rows of the slice are BN * 2 bytes long.
template <int BN, bool BF16, int WS, bool NORM>
struct TileSink {
  static constexpr int kVecPerRow = BN / 8;
  static constexpr int kRowsOwned = kBM / WS;
  const GemmParams& p;
  int me;
  size_t out_base;  // element offset of (tile row 0, col 0) in the destination
  size_t out_ld;
  float* row_ssq;   // NORM: sums of squares of the rows this tile's slice belongs to
  int lane;

  __device__ __forceinline__ void put(int v, uint4 y) const {
    const int q = v / kVecPerRow;
    const int c8 = v - q * kVecPerRow;
    if (p.comm == kCommFusedAR) {
      const int lr = p.strided_rows ? (q * WS + me) : (me * kRowsOwned + q);
      const size_t off = (out_base + static_cast<size_t>(lr) * out_ld + c8 * 8) * 2;
      if (p.mc_dst != nullptr) {
        // NVLS: one store, replicated by the switch into every rank's output
        ptx::multimem_st_v4(reinterpret_cast<uint8_t*>(p.mc_dst) + off, y);
      } else {
#pragma unroll
        for (int d = 0; d < WS; ++d) {
          const int dd = (me + d) % WS;  // start with the local copy, then fan out
          ptx::st_v4(reinterpret_cast<uint8_t*>(p.dst[dd]) + off, y);
        }
      }
      return;
    }
    const size_t off = (out_base + static_cast<size_t>(q) * out_ld + c8 * 8) * 2;
    if constexpr (NORM) {
      if (p.norm_res[me] != nullptr) {
        const uint4 r = ptx::ld_cg_v4(reinterpret_cast<const uint8_t*>(p.norm_res[me]) + off);
        y.x = add2<BF16>(y.x, r.x);
        y.y = add2<BF16>(y.y, r.y);
        y.z = add2<BF16>(y.z, r.z);
        y.w = add2<BF16>(y.w, r.w);
      }
    }
    ptx::st_v4(reinterpret_cast<uint8_t*>(p.dst[me]) + off, y);
    if constexpr (NORM) {
      static_assert(kVecPerRow == 32 || kVecPerRow == 16, "a row must be a warp or half a warp of vectors");
      float r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) r[i] = 0.f;
      unpack_add<BF16>(y.x, r[0], r[1]);
      unpack_add<BF16>(y.y, r[2], r[3]);
      unpack_add<BF16>(y.z, r[4], r[5]);
      unpack_add<BF16>(y.w, r[6], r[7]);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += r[i] * r[i];
#pragma unroll
      for (int o = kVecPerRow / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((lane & (kVecPerRow - 1)) == 0) atomicAdd(row_ssq + q, ss);
    }
  }
};

template <bool BF16, int WS>
__device__ __forceinline__ uint4 sum_partials(const uint4 (&x)[WS]) {
  float a[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = 0.f;
#pragma unroll
  for (int s = 0; s < WS; ++s) {
    unpack_add<BF16>(x[s].x, a[0], a[1]);
    unpack_add<BF16>(x[s].y, a[2], a[3]);
    unpack_add<BF16>(x[s].z, a[4], a[5]);
    unpack_add<BF16>(x[s].w, a[6], a[7]);
  }
  uint4 y;
  y.x = pack2<BF16>(a[0], a[1]);
  y.y = pack2<BF16>(a[2], a[3]);
  y.z = pack2<BF16>(a[4], a[5]);
  y.w = pack2<BF16>(a[6], a[7]);
  return y;
}

// Reduction of the row slices this rank owns of one tile: for every 16-byte vector the WS
// partials are summed in fp32 and the rounded result is handed to the sink.  WS is a template
// parameter so that the loads of several vectors (about 16 in flight per thread) can be issued
// before the first sum: the loop is latency bound otherwise.
//
// Where the partials are: push protocol - WS slices in THIS rank's staging, `stride` bytes
// apart, starting at src0; pull protocol - the same offset `tile_off` of EVERY rank's staging:
// with a multicast mapping of the staging one multimem.ld_reduce per vector lets the NVSwitch
// fetch and sum all ranks' copies (fp32 accumulation), so only the result crosses this GPU's
// links; otherwise each vector is loaded from every rank over NVLink and summed here.
template <int BN, bool BF16, int WS, bool NORM>
__device__ __forceinline__ void reduce_tile(const GemmParams& p, int me, int rt, const uint8_t* src0, size_t stride,
                                            size_t tile_off, const TileSink<BN, BF16, WS, NORM>& sink) {
  constexpr int kVecPerRow = BN / 8;
  constexpr int kRowsOwned = kBM / WS;
  constexpr int kTotalVec = kRowsOwned * kVecPerRow;
  constexpr int kPerThread = kTotalVec / kReducerThreads;
  constexpr int U = (16 / WS) < 1 ? 1 : (16 / WS);  // vectors per thread per round (WS loads each)
  // vectors per thread per round of the switch-side reduction (measured at 2 GPUs: 8 in flight
  // per thread were slower than 4 on a communication-bound shape)
  constexpr int UM = kPerThread >= 4 ? 4 : kPerThread;
  static_assert(kTotalVec % (kReducerThreads * U) == 0 && kTotalVec % (kReducerThreads * UM) == 0,
                "tile slice must split evenly over the reducer threads");

  if (p.stage_local && p.mc_stage != nullptr) {
    const uint8_t* mc = reinterpret_cast<const uint8_t*>(p.mc_stage) + tile_off;
    for (int v0 = rt; v0 < kTotalVec; v0 += kReducerThreads * UM) {
      uint4 y[UM];
#pragma unroll
      for (int u = 0; u < UM; ++u) {
        y[u] = ptx::multimem_ld_reduce_add_v4<BF16>(mc + static_cast<size_t>(v0 + u * kReducerThreads) * 16);
      }
#pragma unroll
      for (int u = 0; u < UM; ++u) sink.put(v0 + u * kReducerThreads, y[u]);
    }
    return;
  }

  const uint8_t* src[WS];
#pragma unroll
  for (int s = 0; s < WS; ++s) {
    src[s] = p.stage_local ? reinterpret_cast<const uint8_t*>(p.stage[(me + s) % WS]) + tile_off
                           : src0 + static_cast<size_t>(s) * stride;
  }
  for (int v0 = rt; v0 < kTotalVec; v0 += kReducerThreads * U) {
    uint4 x[U][WS];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t voff = static_cast<size_t>(v0 + u * kReducerThreads) * 16;
#pragma unroll
      for (int s = 0; s < WS; ++s) x[u][s] = ptx::ld_cg_v4(src[s] + voff);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) sink.put(v0 + u * kReducerThreads, sum_partials<BF16, WS>(x[u]));
  }
}

// RMSNorm of the `rows` shard rows starting at `row0` (all their tiles have been reduced and
// their sums of squares are complete): reads the rows from the shard and writes the normalised
// rows to `out` (the shard itself, or a second buffer when the un-normalised rows are kept as
// the residual stream).  A thread keeps kJV weight vectors in registers and walks down the rows
// two at a time, so 2 * kJV loads are in flight per thread; the rows were written moments ago
// and come from L2.
template <bool BF16>
__device__ __forceinline__ void normalise_panel(const GemmParams& p, int me, int rt, int row0, int rows,
                                                const float* row_ssq) {
  constexpr int kJV = 4;
  const int nvec = p.N / 8;
  const uint8_t* base = reinterpret_cast<const uint8_t*>(p.dst[me]) + static_cast<size_t>(row0) * p.N * 2;
  uint8_t* obase = reinterpret_cast<uint8_t*>(p.norm_out[me] != nullptr ? p.norm_out[me] : p.dst[me]) +
                   static_cast<size_t>(row0) * p.N * 2;
  const uint8_t* w = reinterpret_cast<const uint8_t*>(p.norm_w);
  const size_t pitch = static_cast<size_t>(p.N) * 2;
  const float inv_n = 1.f / static_cast<float>(p.N);
  for (int j0 = rt; j0 < nvec; j0 += kReducerThreads * kJV) {
    uint4 wv[kJV];
#pragma unroll
    for (int i = 0; i < kJV; ++i) {
      const int j = j0 + i * kReducerThreads;
      if (j < nvec) wv[i] = __ldg(reinterpret_cast<const uint4*>(w + static_cast<size_t>(j) * 16));
    }
    for (int q = 0; q < rows; q += 2) {  // rows is 128 / ws: even
      uint4 x[2][kJV];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
#pragma unroll
        for (int i = 0; i < kJV; ++i) {
          const int j = j0 + i * kReducerThreads;
          if (j < nvec) x[r][i] = ptx::ld_cg_v4(base + (q + r) * pitch + static_cast<size_t>(j) * 16);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float scale = rsqrtf(__ldcg(row_ssq + q + r) * inv_n + p.norm_eps);
#pragma unroll
        for (int i = 0; i < kJV; ++i) {
          const int j = j0 + i * kReducerThreads;
          if (j < nvec) {
            uint4 y;
            y.x = norm_scale_mul2<BF16>(x[r][i].x, wv[i].x, scale);
            y.y = norm_scale_mul2<BF16>(x[r][i].y, wv[i].y, scale);
            y.z = norm_scale_mul2<BF16>(x[r][i].z, wv[i].z, scale);
            y.w = norm_scale_mul2<BF16>(x[r][i].w, wv[i].w, scale);
            ptx::st_v4(obase + (q + r) * pitch + static_cast<size_t>(j) * 16, y);
          }
        }
      }
    }
  }
}

// One tile's reduction for a world size known at compile time, followed (NORM) by the
// normalisation of the tile's row panel when this was the panel's last tile.
template <int BN, bool BF16, int WS, bool NORM>
__device__ __forceinline__ void reduce_one_tile(const GemmParams& p, int me, int vr, int rt, int t, int tile_m,
                                                size_t out_base, size_t out_ld, const uint8_t* src0, size_t stride,
                                                size_t tile_off, volatile int* s_is_last) {
  constexpr int kRowsOwned = kBM / WS;
  TileSink<BN, BF16, WS, NORM> sink{p, me, out_base, out_ld, nullptr, rt & 31};
  if constexpr (NORM) {
    // Reduce into the row-major shard while gathering each row's sum of squares; whoever
    // reduces the last tile of a row panel normalises the panel, whose rows were written
    // moments ago and are still in L2.
    float* ssq = p.row_ssq + static_cast<size_t>(vr) * (p.M / WS) + static_cast<size_t>(tile_m) * kRowsOwned;
    int* cnt = p.panel_cnt + vr * p.tiles_m + tile_m;
    sink.row_ssq = ssq;
    reduce_tile<BN, BF16, WS, NORM>(p, me, rt, src0, stride, tile_off, sink);
    ptx::named_bar_sync(2, kReducerThreads);  // every thread's stores and atomics are issued
    if (rt == 0) {
      __threadfence();
      const int old = atomicAdd(cnt, 1);
      *s_is_last = (old == p.tiles_n - 1) ? 1 : 0;
      if (old == p.tiles_n - 1) __threadfence();
    }
    ptx::named_bar_sync(2, kReducerThreads);
    if (*s_is_last) {
      normalise_panel<BF16>(p, me, rt, tile_m * kRowsOwned, kRowsOwned, ssq);
      ptx::named_bar_sync(2, kReducerThreads);
      if (rt < kRowsOwned) ssq[rt] = 0.f;
      if (rt == 0) *cnt = 0;
    }
    ptx::named_bar_sync(2, kReducerThreads);  // s_is_last is reused by the next tile
  } else {
    reduce_tile<BN, BF16, WS, NORM>(p, me, rt, src0, stride, tile_off, sink);
  }
}

template <int BN, int STAGES, bool BF16, bool FUSED, bool CTA2, int MT, bool A2A = false, bool NORM = false,
          bool TRACE = false, int EPI = 2>
__global__ void __launch_bounds__(FUSED ? kThreadsFused : kThreadsPlain, 1)
    fo_gemm_kernel(const __grid_constant__ GemmTensorMaps maps,
                   const __grid_constant__ GemmParams p) {
  static_assert(!NORM || FUSED, "the RMSNorm tail belongs to the fused reduce-scatter");
  static_assert(!TRACE || (FUSED && !NORM), "the timeline is recorded by the fused AR/RS kernels");
  // Stamp slot `slot` of natural tile t (tracing builds only).
  auto stamp = [&](int t, int slot) {
    if constexpr (TRACE) {
      p.trace[(static_cast<size_t>(blockIdx.y) * p.num_tiles + t) * kTraceSlots + slot] = ptx::globaltimer_ns();
    }
  };
  static_assert(MT == 1 || (MT == 2 && CTA2 && BN == 256), "two row halves need CTA pairs and BN = 256");
  static_assert(!(A2A && FUSED), "the all-to-all epilogue is a variant of the plain kernel");
  static_assert(EPI == 2 || (FUSED && EPI >= 3), "more than two chunk buffers only pay in the fused kernels");
  using L = GemmSmem<BN, STAGES, CTA2, MT, EPI>;
  // Accumulator slots in TMEM: two tiles in flight (MT = 1) or the two halves of one (MT = 2).
  constexpr int kAccStages = MT == 2 ? 1 : 2;
  extern __shared__ uint8_t smem_raw[];
  // The ring must start on a 1024-byte boundary of the shared window.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
  uint64_t* chunk_ready_bar = bars + 2 * STAGES + 4;  // epilogue -> push warp: chunk written
  uint64_t* chunk_free_bar = chunk_ready_bar + EPI;   // push warp -> epilogue: chunk buffer reusable
  uint64_t* sig_full_bar = chunk_free_bar + EPI;      // push warp -> signal warp: a tile's stores have landed
  uint64_t* sig_empty_bar = sig_full_bar + kSigRing;  // signal warp -> push warp: ring slot reusable
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + L::kMiscOffset);
  uint32_t* s_tmem_base = misc;                                   // written by tcgen05.alloc
  volatile int* s_abort = reinterpret_cast<volatile int*>(misc + 1);
  volatile int* s_ep_ok = reinterpret_cast<volatile int*>(misc + 2);
  volatile int* s_is_last = reinterpret_cast<volatile int*>(misc + 3);
  // two slots, alternated per tile: a slow reader of tile i never sees tile i+1's verdict
  volatile int* s_red_ok = reinterpret_cast<volatile int*>(misc + 4);
  // ring between the push warp and the signal warp: wave group and tile id of each handed-over tile
  volatile int* s_sig_g = reinterpret_cast<volatile int*>(misc + 8);
  volatile int* s_sig_t = reinterpret_cast<volatile int*>(misc + 8 + kSigRing);

  // broadcast from lane 0 so that the compiler knows the role index is the same in every lane and
  // can keep the role loops' counters and addresses in uniform registers
  const int warp_idx = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int vr = blockIdx.y;           // virtual rank of this CTA inside the launch
  const int me = p.rank_base + vr;     // rank this CTA acts as
  const int num_kb = (p.K + kBK - 1) / kBK;
  constexpr uint32_t kTmemCols = 2 * BN;
  // Scheduling unit: a CTA (128-row tiles) or a CTA pair (256-row tiles, this CTA's half).
  const uint32_t cta_rank = CTA2 ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  const int unit = CTA2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_units = CTA2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int kRowsPerUnit = (CTA2 ? 2 : 1) * MT;  // 128-row tiles of one scheduling unit
  const int sched_tiles_m = p.tiles_m / kRowsPerUnit;
  const int sched_tiles = sched_tiles_m * p.tiles_n;
  auto my_tile = [&](int pos) {
    TileCoord tc = tile_of_position(pos, sched_tiles_m, p.tiles_n, p.raster_sw);
    tc.m = kRowsPerUnit * tc.m + MT * static_cast<int>(cta_rank);  // first half; halves follow
    return tc;
  };
  int32_t* status = p.status[vr];
  // Pipeline waits inside the CTA can legitimately last as long as a cross-GPU wait that
  // another role is sitting in, so their bound is a multiple of it.
  const uint64_t pipe_timeout = 4ull * p.timeout_ns + 1000000000ull;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tmem_full_bar[i], 1);
      // one arrival per epilogue warp, from both CTAs of a pair
      ptx::mbar_init(&tmem_empty_bar[i], CTA2 ? 8 : 4);
    }
    for (int i = 0; i < EPI; ++i) {
      ptx::mbar_init(&chunk_ready_bar[i], kEpilogueThreads);
      ptx::mbar_init(&chunk_free_bar[i], 1);
    }
    for (int i = 0; i < kSigRing; ++i) {
      ptx::mbar_init(&sig_full_bar[i], 1);
      ptx::mbar_init(&sig_empty_bar[i], 1);
    }
    *s_abort = 0;
    *s_ep_ok = 1;
    s_red_ok[0] = 1;
    s_red_ok[1] = 1;
    *s_is_last = 0;
    ptx::mbar_fence_init();
  }
  if (warp_idx == 0 && lane == 0) {
    ptx::prefetch_tmap(&maps.a[vr]);
    ptx::prefetch_tmap(&maps.b[vr]);
  }
  if (warp_idx == 1) {
    if constexpr (CTA2) {
      ptx::tmem_alloc_pair(s_tmem_base, kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(s_tmem_base, kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  if constexpr (CTA2) {
    // Both CTAs' barriers must be initialised before either receives a remote signal.
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;

  if (warp_idx == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the loops (so their control flow is warp-uniform) and one elected
    // lane issues the copies.
    {
      const bool elected = ptx::elect_one();
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;
      bool ok = true;
      for (int pos = unit; ok && pos < sched_tiles; pos += num_units) {
        const TileCoord tc = my_tile(pos);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, s_abort, pipe_timeout, p.wait_sleep_ns)) {
            if (elected) ptx::report_status(status, kStatusTimeoutSmemEmpty, pos, kb, stage);
            *s_abort = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          if (elected) {
            if constexpr (CTA2) {
              // The leader's barrier collects the bytes of both CTAs.
              if (leader) ptx::mbar_arrive_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
#pragma unroll
              for (int h = 0; h < MT; ++h) {
                ptx::tma_load_2d_pair(sa + h * L::kAHalfBytes, &maps.a[vr], &full_bar[stage], kb * kBK,
                                      (tc.m + h) * kBM, p.l2_hint_a);
              }
              ptx::tma_load_2d_pair(sb, &maps.b[vr], &full_bar[stage], kb * kBK,
                                    tc.n * BN + static_cast<int>(cta_rank) * L::kBRows, p.l2_hint_b);
            } else {
              ptx::mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
              ptx::tma_load_2d(sa, &maps.a[vr], &full_bar[stage], kb * kBK, tc.m * kBM, p.l2_hint_a);
              ptx::tma_load_2d(sb, &maps.b[vr], &full_bar[stage], kb * kBK, tc.n * BN, p.l2_hint_b);
            }
          }
          __syncwarp();
          ++issued;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Drain: do not leave the CTA while a bulk copy may still write its shared memory.
      // For each ring slot wait (bounded) for the last load issued into it.
      // (In a pair the follower's loads are counted on the leader's barriers, which the
      // follower cannot poll; it relies on the cluster-wide barrier at the end instead: the
      // leader reaches it only after draining the barriers that count both CTAs' bytes.)
      for (int s = 0; elected && s < STAGES && (!CTA2 || leader); ++s) {
        if (issued <= static_cast<uint32_t>(s)) continue;
        const uint32_t last = ((issued - 1 - s) / STAGES) * STAGES + s;  // last issue index on slot s
        const uint32_t par = (last / STAGES) & 1u;
        for (uint32_t it = 0; it < ptx::kMbarDrainPolls; ++it) {
          if (ptx::mbar_try_wait(&full_bar[s], par)) break;
        }
      }
    }
  } else if (warp_idx == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The leader's whole warp walks the loops; one elected lane issues the MMAs and commits.
    if (leader) {
      const bool elected = ptx::elect_one();
      constexpr uint32_t idesc = ptx::make_idesc_f16(BF16, CTA2 ? 2 * kBM : kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int pos = unit; ok && pos < sched_tiles; pos += num_units) {
        if (!ptx::mbar_wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1u, s_abort, pipe_timeout, p.wait_sleep_ns)) {
          if (elected) ptx::report_status(status, kStatusTimeoutTmemEmpty, pos, acc, 0);
          *s_abort = 1;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait_bounded(&full_bar[stage], phase, s_abort, pipe_timeout, p.wait_sleep_ns)) {
            if (elected) ptx::report_status(status, kStatusTimeoutSmemFull, pos, kb, stage);
            *s_abort = 1;
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t sa = ptx::smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = ptx::make_smem_desc_sw128_kmajor(sa);
          const uint64_t db = ptx::make_smem_desc_sw128_kmajor(sa + L::kABytes);
          if (elected) {
            // advance 16 elements (32 B) along K inside the swizzle atom: +2 in 16-byte units
            if constexpr (CTA2) {
#pragma unroll
              for (int h = 0; h < MT; ++h) {
                // half h: its A rows sit h * 16 KB further in the stage, its accumulator BN
                // columns further in TMEM; both halves multiply the same B tile.  The four MMAs
                // of a half are issued back to back so that consecutive instructions accumulate
                // into the same TMEM columns.
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                  ptx::umma_f16_ss_pair(tmem_d + static_cast<uint32_t>(h * BN),
                                        da + static_cast<uint64_t>(h * (L::kAHalfBytes >> 4) + 2 * k),
                                        db + static_cast<uint64_t>(2 * k), idesc,
                                        (kb > 0 || k > 0) ? 1u : 0u);
                }
              }
            } else {
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k) {
                ptx::umma_f16_ss(tmem_d, da + static_cast<uint64_t>(2 * k),
                                 db + static_cast<uint64_t>(2 * k), idesc,
                                 (kb > 0 || k > 0) ? 1u : 0u);
              }
            }
            // slot reusable (in both CTAs of a pair) once these MMAs have read it
            if constexpr (CTA2) {
              ptx::umma_commit_pair(&empty_bar[stage], 3);
            } else {
              ptx::umma_commit(&empty_bar[stage]);
            }
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (elected) {
          if constexpr (CTA2) {
            ptx::umma_commit_pair(&tmem_full_bar[acc], 3);  // accumulators complete in both CTAs
          } else {
            ptx::umma_commit(&tmem_full_bar[acc]);
          }
        }
        __syncwarp();
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp_idx < 6) {
    // ------------------------------------------------------------------ epilogue
    const int et = threadIdx.x - 64;           // 0..127
    const int quad = warp_idx & 3;             // TMEM lane quadrant this warp may read
    const int my_row = quad * 32 + lane;       // tile row held by this thread after tcgen05.ld
    uint8_t* epi = smem + L::kEpiOffset;
    const int rows_owned = kBM / p.ws;
    const size_t elem = 2;
    int acc = 0;
    uint32_t acc_phase = 0;

    // Fused push: rows are grouped by owning rank in the shared-memory chunk so that each
    // owner's slice is one contiguous (rows_owned x 128 B) box for a TMA store.
    int smem_row = my_row;
    if constexpr (FUSED) {
      const int o = p.strided_rows ? (my_row % p.ws) : (my_row / rows_owned);
      const int q = p.strided_rows ? (my_row / p.ws) : (my_row % rows_owned);
      smem_row = o * rows_owned + q;
    }
    uint32_t chunk_no = 0;  // running chunk count: buffer = chunk_no & 1, use count = chunk_no >> 1

    // tmem_empty lives in the leader CTA of a pair
    const uint32_t tmem_empty_addr0 =
        CTA2 ? ptx::mapa_shared(ptx::smem_u32(&tmem_empty_bar[0]), 0u) : ptx::smem_u32(&tmem_empty_bar[0]);

    // Plain kernels store finished chunks with TMA (one tensor store per 128 x 64 chunk through
    // the output map in maps.st[vr]) when the host could describe the output as a 2-D tensor
    // (row-major and tile-contiguous layouts); the row-scatter and all-to-all modes, whose rows
    // go to unrelated addresses, keep the per-thread 16-byte stores.
    const bool use_tma = !FUSED && !A2A && p.tma_out != 0;
    // Fused kernels, pull protocol with direct stores: the partial tile goes to this rank's own
    // staging buffer, so the epilogue threads can store it themselves (as the plain kernels do)
    // instead of handing every chunk to the push warp for a TMA store; the push warp then only
    // announces the finished tile.  chunk_ready / chunk_free count tiles in this mode.
    const bool direct = FUSED && p.stage_local != 0 && p.pull_direct != 0;

    bool go = true;
    if constexpr (A2A) {
      // Start-of-call handshake of the all-to-all: a rank's receive buffer may be overwritten
      // only after that rank has entered this call (its readers of the previous call's rows
      // come earlier in its stream).  CTA 0 announces this rank; every CTA waits, before its
      // first store, until all ranks have announced themselves.  The main loop runs meanwhile.
      if (et == 0) {
        if (blockIdx.x == 0) {
          ptx::fence_acq_rel_sys();
          for (int d = 0; d < p.ws; ++d) ptx::red_relaxed_sys_add(p.ready[(me + d) % p.ws], 1u);
        }
        uint32_t obs;
        int ok = ptx::wait_counter_ge<true>(p.ready[me], p.epoch_ready, p.timeout_ns, s_abort, &obs) ? 1 : 0;
        if (!ok) {
          ptx::report_status(status, kStatusTimeoutStartFlag, me, obs, p.epoch_ready);
          *s_abort = 1;
        }
        *s_ep_ok = ok;
      }
      ptx::named_bar_sync(1, kEpilogueThreads);
      go = *s_ep_ok != 0;
      ptx::named_bar_sync(1, kEpilogueThreads);  // everybody has read the verdict before it is reused
    }

    for (int pos = unit; go && pos < sched_tiles; pos += num_units) {
      const TileCoord tc0 = my_tile(pos);

      if (et == 0) {
        int ok = ptx::mbar_wait_bounded(&tmem_full_bar[acc], acc_phase, s_abort, pipe_timeout, 4u * p.wait_sleep_ns) ? 1 : 0;
        if (!ok) {
          ptx::report_status(status, kStatusTimeoutTmemFull, pos, acc, 0);
          *s_abort = 1;
        }
        *s_ep_ok = ok;
      }
      ptx::named_bar_sync(1, kEpilogueThreads);
      if (!*s_ep_ok) break;
      ptx::tc_fence_after_sync();

#pragma unroll 1
      for (int h = 0; h < MT; ++h) {  // the 128-row halves of this CTA's tile (one unless MT = 2)
      TileCoord tc = tc0;
      tc.m += h;
      const int t = tc.m * p.tiles_n + tc.n;
      const int r = tile_position(p, t, status);
      if constexpr (TRACE) {
        if (et == 0) {
          stamp(t, kTraceAccReady);
          p.trace[(static_cast<size_t>(blockIdx.y) * p.num_tiles + t) * kTraceSlots + kTraceWhere] =
              (static_cast<unsigned long long>(ptx::sm_id()) << 32) | blockIdx.x;
        }
      }

      // Per-thread destinations for the cooperative store phase: thread `et` stores the
      // 16-byte piece (et & 7) of rows (et >> 3) + 16 * i, i = 0..7.
      uint8_t* row_ptr[8];
      uint32_t row_valid = 0xffu;  // all-to-all: bit i clear = row i has no destination
      // TMA stores: coordinates of the tile's first chunk in the output's 2-D view
      int tma_x0 = 0, tma_y0 = 0;
      if (use_tma) {
        if (p.out_mode == kOutNatural) {
          tma_x0 = tc.n * BN;
          tma_y0 = tc.m * kBM;
        } else {  // tile-contiguous: [M * N / (rldn * BN)] rows of rldn * BN elements
          tma_x0 = (r % p.rldn) * BN;
          tma_y0 = (r / p.rldn) * kBM;
        }
      }
#pragma unroll
      for (int i = 0; i < 8 && !use_tma; ++i) {
        const int lr = (et >> 3) + 16 * i;
        size_t off = 0;  // element offset of (row lr, tile column 0)
        uint8_t* base = nullptr;
        if constexpr (A2A) {
          // Row m of C belongs to the run of the first rank whose run ends after it.
          const int m = tc.m * kBM + lr;
          const int* tab = p.a2a_tab + vr * 2 * kMaxRanks;
          int d = 0, start = 0;
          while (d < p.ws) {
            const int end = __ldg(tab + d);
            if (m < end) break;
            start = end;
            ++d;
          }
          if (d < p.ws) {
            base = reinterpret_cast<uint8_t*>(p.dst[d]);
            off = (static_cast<size_t>(__ldg(tab + kMaxRanks + d)) + static_cast<size_t>(m - start)) * p.N +
                  static_cast<size_t>(tc.n) * BN;
          } else {
            row_valid &= ~(1u << i);
          }
        } else if constexpr (!FUSED) {
          base = reinterpret_cast<uint8_t*>(p.out[vr]);
          if (p.out_mode == kOutNatural) {
            off = (static_cast<size_t>(tc.m) * kBM + lr) * p.N + static_cast<size_t>(tc.n) * BN;
          } else if (p.out_mode == kOutReorder) {
            const size_t ld = static_cast<size_t>(p.rldn) * BN;
            off = static_cast<size_t>(r / p.rldn) * kBM * ld + static_cast<size_t>(r % p.rldn) * BN +
                  static_cast<size_t>(lr) * ld;
          } else {  // kOutScatterRows: rows of the [M*N/BN, BN] view are remapped through RE
            const size_t row_id = static_cast<size_t>(r) * kBM + lr;
            const int re = p.RE[row_id];
            if (static_cast<unsigned>(re) >= static_cast<unsigned>(p.M) * static_cast<unsigned>(p.tiles_n)) {
              // a row index outside the buffer: report it and drop the row
              ptx::report_status(status, kStatusBadArgument, 2, static_cast<int32_t>(row_id), re);
              row_valid &= ~(1u << i);
            } else {
              off = static_cast<size_t>(re) * BN;
            }
          }
        }
        row_ptr[i] = base + off * elem + (et & 7) * 16;
      }

      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>((MT == 2 ? h : acc) * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v0[32], v1[32];
        ptx::tmem_ld_32x32b_x32(t_row + c * 64, v0);
        ptx::tmem_ld_32x32b_x32(t_row + c * 64 + 32, v1);
        ptx::tmem_ld_wait();
        if (c == BN / 64 - 1 && h == MT - 1) {
          // Accumulator(s) fully read by this warp: hand it back to the (leader's) MMA warp.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(tmem_empty_addr0 + static_cast<uint32_t>(acc) * 8u);
        }
        if constexpr (FUSED) {
          // The buffer is free once the push warp's stores of its previous use have read it.
          // A failed wait raises the abort flag but the thread stays in step with the others:
          // everybody leaves together at the next tile boundary.
          if (!direct && !ptx::mbar_wait_bounded(&chunk_free_bar[chunk_no % EPI], ((chunk_no / EPI) & 1u) ^ 1u,
                                                 s_abort, pipe_timeout)) {
            *s_abort = 1;
          }
        }
        if constexpr (!FUSED && !A2A) {
          if (use_tma) {
            // The store issued from this buffer two chunks ago must have read it.
            if (et == 0) ptx::bulk_wait_group_read<1>();
            ptx::named_bar_sync(1, kEpilogueThreads);
          }
        }
        const int bsel = (FUSED && !direct) ? static_cast<int>(chunk_no % EPI) : (c & 1);
        uint8_t* buf = epi + bsel * L::kEpiBufBytes + smem_row * 128;
        const int sw = smem_row & 7;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = pack2<BF16>(__uint_as_float(v0[8 * j + 0]), __uint_as_float(v0[8 * j + 1]));
          w.y = pack2<BF16>(__uint_as_float(v0[8 * j + 2]), __uint_as_float(v0[8 * j + 3]));
          w.z = pack2<BF16>(__uint_as_float(v0[8 * j + 4]), __uint_as_float(v0[8 * j + 5]));
          w.w = pack2<BF16>(__uint_as_float(v0[8 * j + 6]), __uint_as_float(v0[8 * j + 7]));
          *reinterpret_cast<uint4*>(buf + ((j ^ sw) * 16)) = w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = pack2<BF16>(__uint_as_float(v1[8 * j + 0]), __uint_as_float(v1[8 * j + 1]));
          w.y = pack2<BF16>(__uint_as_float(v1[8 * j + 2]), __uint_as_float(v1[8 * j + 3]));
          w.z = pack2<BF16>(__uint_as_float(v1[8 * j + 4]), __uint_as_float(v1[8 * j + 5]));
          w.w = pack2<BF16>(__uint_as_float(v1[8 * j + 6]), __uint_as_float(v1[8 * j + 7]));
          *reinterpret_cast<uint4*>(buf + (((j + 4) ^ sw) * 16)) = w;
        }
        if constexpr (FUSED) {
          if (direct) {
            // rows are grouped by owner in shared memory exactly as in the staging layout
            // [tile][owner][rows owned][BN]: shared row lr is staging row t * 128 + lr
            ptx::named_bar_sync(1, kEpilogueThreads);
            const uint8_t* rbuf = epi + (c & 1) * L::kEpiBufBytes;
            uint8_t* srow = reinterpret_cast<uint8_t*>(p.stage[me]) +
                            ((static_cast<size_t>(t) * kBM + (et >> 3)) * BN + c * 64) * 2 + (et & 7) * 16;
#pragma unroll
            for (int i = 0; i < 8 && !(p.diag & 2); ++i) {
              const int lr = (et >> 3) + 16 * i;
              const uint4 w = *reinterpret_cast<const uint4*>(rbuf + lr * 128 + (((et & 7) ^ (lr & 7)) * 16));
              ptx::st_v4(srow + static_cast<size_t>(16 * i) * BN * 2, w);
            }
          } else {
            // Hand the chunk to the push warp (generic-proxy writes ordered before its TMA reads).
            ptx::fence_proxy_async_smem();
            ptx::mbar_arrive(&chunk_ready_bar[chunk_no % EPI]);
            ++chunk_no;
          }
        } else if (use_tma) {
          ptx::fence_proxy_async_smem();  // generic-proxy writes before the async-proxy read
          ptx::named_bar_sync(1, kEpilogueThreads);
          if (et == 0) {
            ptx::tma_store_2d(&maps.st[vr], epi + (c & 1) * L::kEpiBufBytes, tma_x0 + c * 64, tma_y0);
            ptx::bulk_commit_group();
          }
        } else {
          ptx::named_bar_sync(1, kEpilogueThreads);
          const uint8_t* rbuf = epi + (c & 1) * L::kEpiBufBytes;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int lr = (et >> 3) + 16 * i;
            const uint4 w =
                *reinterpret_cast<const uint4*>(rbuf + lr * 128 + (((et & 7) ^ (lr & 7)) * 16));
            if ((row_valid >> i) & 1u) ptx::st_v4(row_ptr[i] + c * 128, w);
          }
        }
      }

      if constexpr (FUSED) {
        // arrival counters are bumped by the push warp
        if (et == 0) stamp(t, kTraceEpilogueDone);
        if (direct) {
          // The tile's stores have been issued by this thread: hand the tile to the push warp
          // (release at CTA scope; its system-scope fence then covers these stores).  The slot
          // is free once the push warp has announced the tile that used it EPI tiles ago.
          if (!ptx::mbar_wait_bounded(&chunk_free_bar[chunk_no % EPI], ((chunk_no / EPI) & 1u) ^ 1u, s_abort,
                                      pipe_timeout)) {
            *s_abort = 1;
          }
          ptx::mbar_arrive(&chunk_ready_bar[chunk_no % EPI]);
          ++chunk_no;
        }
      } else {
        // All of this tile's stores have been issued by every epilogue thread.
        if (!use_tma) ptx::named_bar_sync(1, kEpilogueThreads);
        if (et == 0 && p.MM[vr] != nullptr) {
          int* mm = p.MM[vr];
          if (use_tma && (p.signal || p.monitor)) {
            // The tile may be announced only once its tensor stores have been written.
            ptx::bulk_wait_group<0>();
            ptx::fence_proxy_async_all();
          }
          if (p.signal) {
            int g, need;
            group_of_position(p, r, &g, &need);
            ptx::fence_acq_rel_gpu();
            ptx::red_release_gpu_add(reinterpret_cast<uint32_t*>(mm + g), 1u);
          }
          if (p.monitor) {
            const int order = atomicAdd(mm + p.mm_stride - 1, 1);
            mm[p.mm_stride + r] = order;
          }
        }
      }
      if (FUSED && et == 0 && p.monitor && p.MM[vr] != nullptr) {
        int* mm = p.MM[vr];
        const int order = atomicAdd(mm + p.mm_stride - 1, 1);
        mm[p.mm_stride + r] = order;
      }
      }  // halves
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    // No tensor store may still read this CTA's shared memory when the CTA exits.
    if (use_tma && et == 0) ptx::bulk_wait_group<0>();
    if constexpr (A2A) {
      // End-of-call handshake of the all-to-all: once every CTA of this rank has issued its
      // stores, the last one tells every rank that this rank's rows have been sent and waits
      // until every rank has said the same - this rank's receive buffer is then complete.
      ptx::named_bar_sync(1, kEpilogueThreads);
      if (et == 0) {
        ptx::fence_acq_rel_sys();
        const uint32_t old = atomicAdd(p.local_cnt[vr], 1u);
        if (old == gridDim.x - 1) {
          *p.local_cnt[vr] = 0u;
          ptx::fence_acq_rel_sys();
          for (int d = 0; d < p.ws; ++d) ptx::red_relaxed_sys_add(p.done[(me + d) % p.ws], 1u);
          uint32_t obs;
          if (!ptx::wait_counter_ge<true>(p.done[me], p.epoch_done, p.timeout_ns, nullptr, &obs)) {
            ptx::report_status(status, kStatusTimeoutDoneFlag, me, obs, p.epoch_done);
          }
        }
      }
    }
  } else if (warp_idx < 10) {
    // ------------------------------------------------------------------ reducer (fused)
    if constexpr (FUSED) {
      const int rt = threadIdx.x - kThreadsPlain;  // 0..127
      const int ws = p.ws;
      const int rows_owned = kBM / ws;
      const size_t src_stride = static_cast<size_t>(p.num_tiles) * rows_owned * BN;  // elements
      const uint8_t* stage_me = reinterpret_cast<const uint8_t*>(p.stage[me]);

      int slot = 0;
      for (int pos = unit, hh = 0; pos < sched_tiles; slot ^= 1) {
        TileCoord tc = my_tile(pos);
        tc.m += hh;  // halves of a unit are reduced one after the other
        if (++hh == MT) {
          hh = 0;
          pos += num_units;
        }
        const int t = tc.m * p.tiles_n + tc.n;
        const int r = tile_position(p, t, status);
        if (rt == 0) {
          int g, need;
          group_of_position(p, r, &g, &need);
          uint32_t obs;
          stamp(t, kTraceWaitBegin);
          const uint32_t target = (p.diag & 4) ? 0u : static_cast<uint32_t>(need * ws);
          int ok = ptx::wait_counter_ge<true>(p.flags[me] + g, target, p.timeout_ns, s_abort, &obs)
                       ? 1
                       : 0;
          if (!ok) {
            ptx::report_status(status, kStatusTimeoutGroupFlag, g, obs, target);
            *s_abort = 1;
          }
          s_red_ok[slot] = ok;
          stamp(t, kTraceWaitEnd);
        }
        ptx::named_bar_sync(2, kReducerThreads);
        if (!s_red_ok[slot]) break;

        // Output addressing of this tile.
        size_t out_base;  // element offset of (tile row 0, col 0) in the destination
        size_t out_ld;
        if (p.comm == kCommFusedAR) {
          if (p.out_mode == kOutNatural) {
            out_ld = p.N;
            out_base = static_cast<size_t>(tc.m) * kBM * p.N + static_cast<size_t>(tc.n) * BN;
          } else {
            out_ld = static_cast<size_t>(p.rldn) * BN;
            out_base = static_cast<size_t>(r / p.rldn) * kBM * out_ld +
                       static_cast<size_t>(r % p.rldn) * BN;
          }
        } else {  // ReduceScatter: local shard [M/ws, N]
          if (p.out_mode == kOutNatural) {
            out_ld = p.N;
            out_base = static_cast<size_t>(tc.m) * rows_owned * p.N + static_cast<size_t>(tc.n) * BN;
          } else {  // tiles of rows_owned x BN in reordered order
            out_ld = BN;
            out_base = static_cast<size_t>(r) * rows_owned * BN;
          }
        }
        const uint8_t* src_tile = stage_me + static_cast<size_t>(t) * rows_owned * BN * 2;

        const size_t stride_b = src_stride * 2;
        if (p.diag & 1) continue;
        // pull protocol: rows of owner `me` inside tile t's [owner][rows owned][BN] block of any rank's staging
        const size_t tile_off = (static_cast<size_t>(t) * kBM + static_cast<size_t>(me) * rows_owned) * BN * 2;
        switch (ws) {
          case 2:
            reduce_one_tile<BN, BF16, 2, NORM>(p, me, vr, rt, t, tc.m, out_base, out_ld, src_tile, stride_b, tile_off, s_is_last);
            break;
          case 4:
            reduce_one_tile<BN, BF16, 4, NORM>(p, me, vr, rt, t, tc.m, out_base, out_ld, src_tile, stride_b, tile_off, s_is_last);
            break;
          default:
            reduce_one_tile<BN, BF16, 8, NORM>(p, me, vr, rt, t, tc.m, out_base, out_ld, src_tile, stride_b, tile_off, s_is_last);
            break;
        }
        if (rt == 0) stamp(t, kTraceReduced);
      }

      // End-of-call handshake.  The last CTA of this rank to finish clears the group flags
      // (nobody on this rank reads them any more and peers cannot push again before they
      // have seen our `done` signal), tells every rank that this rank has consumed its
      // staging, and - for AllReduce - waits until every rank's results have landed here.
      ptx::named_bar_sync(2, kReducerThreads);
      if (rt == 0) {
        ptx::fence_acq_rel_sys();
        const uint32_t old = atomicAdd(p.local_cnt[vr], 1u);
        *s_is_last = (old == gridDim.x - 1) ? 1 : 0;
      }
      ptx::named_bar_sync(2, kReducerThreads);
      if (*s_is_last) {
        const int nflags = (p.num_groups > 0 && p.cseg != nullptr) ? p.num_groups : p.num_tiles;  // same count either way when equal
        for (int i = rt; i < nflags; i += kReducerThreads) p.flags[me][i] = 0u;
        ptx::named_bar_sync(2, kReducerThreads);
        if (rt == 0) {
          *p.local_cnt[vr] = 0u;
          ptx::fence_acq_rel_sys();
          for (int d = 0; d < ws; ++d) ptx::red_relaxed_sys_add(p.done[(me + d) % ws], 1u);
          if (p.comm == kCommFusedAR) {
            uint32_t obs;
            if (!ptx::wait_counter_ge<true>(p.done[me], p.epoch_done, p.timeout_ns, nullptr,
                                            &obs)) {
              ptx::report_status(status, kStatusTimeoutDoneFlag, me, obs, p.epoch_done);
            }
          }
        }
      }
    }
  } else if (warp_idx == 10) {
    // ------------------------------------------------------------------ push warp (fused)
    if constexpr (FUSED) {
      if (lane == 0) {
        constexpr int kChunks = BN / 64;
        constexpr int kMaxLag = 4;
        const int rows_owned = kBM / p.ws;
        const uint8_t* epi = smem + L::kEpiOffset;
        // Tiles of stores kept in flight before the oldest one's completion is awaited.  Stores
        // into the local staging (pull protocol) complete within a microsecond or two: no lag.
        const int lag = p.stage_local ? 0 : (p.push_lag < 1 ? 1 : (p.push_lag > kMaxLag ? kMaxLag : p.push_lag));
        int ring[kMaxLag];       // wave groups of the tiles whose pushes may still be in flight
        int ring_t[kMaxLag];     // their tile ids
        int ring_head = 0, ring_count = 0;
        uint32_t chunk_no = 0;
        uint32_t sig_no = 0;     // tiles handed to the signal warp
        bool ok = true;

        // A tile's stores have completed (bulk wait): hand it to the signal warp, which
        // publishes it to the owners.  The system-scope release fence that publication needs
        // waits for every remote write this SM has in flight - tens of microseconds once the
        // reducers are storing results through the switch - and the chunk buffers give the
        // epilogue only two chunks of slack, so it must not run on this thread.
        auto signal_group = [&](int g, int t) {
          const uint32_t slot = sig_no % kSigRing;
          if (!ptx::mbar_wait_bounded(&sig_empty_bar[slot], ((sig_no / kSigRing) & 1u) ^ 1u, s_abort, pipe_timeout)) {
            *s_abort = 1;
            return;
          }
          s_sig_g[slot] = g;
          s_sig_t[slot] = t;
          ptx::fence_proxy_async_all();          // the bulk stores before the hand-over
          ptx::mbar_arrive(&sig_full_bar[slot]);  // release at CTA scope
          ++sig_no;
        };

        // Peers may still be reading the staging slices of the previous call.
        {
          uint32_t obs;
          if (!ptx::wait_counter_ge<true>(p.done[me], p.epoch_done_prev, p.timeout_ns, s_abort, &obs)) {
            ptx::report_status(status, kStatusTimeoutStartFlag, me, obs, p.epoch_done_prev);
            *s_abort = 1;
            ok = false;
          }
        }
        for (int pos = unit, hh = 0; ok && pos < sched_tiles;) {
          TileCoord tc = my_tile(pos);
          tc.m += hh;
          if (++hh == MT) {
            hh = 0;
            pos += num_units;
          }
          const int t = tc.m * p.tiles_n + tc.n;
          const int r = tile_position(p, t, status);
          const int row0 = (me * p.num_tiles + t) * rows_owned;
          if (p.stage_local != 0 && p.pull_direct != 0) {
            // The epilogue threads stored the tile into the local staging themselves; announce it.
            const int b = static_cast<int>(chunk_no % EPI);
            if (!ptx::mbar_wait_bounded(&chunk_ready_bar[b], (chunk_no / EPI) & 1u, s_abort, pipe_timeout, p.wait_sleep_ns)) {
              ptx::report_status(status, kStatusTimeoutTmemFull, pos, 0, 2);
              *s_abort = 1;
              ok = false;
              break;
            }
            stamp(t, kTracePushIssued);
            int g, need;
            group_of_position(p, r, &g, &need);
            signal_group(g, t);
            ptx::mbar_arrive(&chunk_free_bar[b]);
            ++chunk_no;
            continue;
          }
          for (int c = 0; c < kChunks; ++c, ++chunk_no) {
            const int b = static_cast<int>(chunk_no % EPI);
            if (!ptx::mbar_wait_bounded(&chunk_ready_bar[b], (chunk_no / EPI) & 1u, s_abort, pipe_timeout, p.wait_sleep_ns)) {
              ptx::report_status(status, kStatusTimeoutTmemFull, pos, c, 1);
              *s_abort = 1;
              ok = false;
              break;
            }
            const uint8_t* cbuf = epi + b * L::kEpiBufBytes;
            if (p.stage_local) {
              // pull variant: the whole chunk (rows already grouped by owner) stays on this GPU
              if (!(p.diag & 2)) ptx::tma_store_2d(&maps.st[me], cbuf, c * 64, t * kBM);
            } else {
              for (int o = 0; o < p.ws && !(p.diag & 2); ++o) {
                const int oo = (me + o) % p.ws;  // stagger the first target over the peers
                ptx::tma_store_2d(&maps.st[oo], cbuf + oo * rows_owned * 128, c * 64, row0);
              }
            }
            ptx::bulk_commit_group();
            if constexpr (EPI == 2) {
              ptx::bulk_wait_group_read<0>();     // sources read: the epilogue may refill the buffer
              ptx::mbar_arrive(&chunk_free_bar[b]);
            } else {
              // More buffers: keep EPI - 1 chunks of stores in flight and hand back the buffer of
              // the chunk issued EPI - 1 chunks ago, whose stores have read their source by now.
              ptx::bulk_wait_group_read<EPI - 1>();
              if (chunk_no >= static_cast<uint32_t>(EPI - 1)) {
                ptx::mbar_arrive(&chunk_free_bar[(chunk_no - static_cast<uint32_t>(EPI - 1)) % EPI]);
              }
            }
          }
          if (!ok) break;
          stamp(t, kTracePushIssued);
          int g, need;
          group_of_position(p, r, &g, &need);
          if (lag == 0) {
            ptx::bulk_wait_group<0>();
            signal_group(g, t);
            continue;
          }
          if (ring_count == lag) {
            // The oldest tile in flight was issued `lag` tiles ago; with a main loop between
            // tiles its stores have long completed and this wait returns at once.
            switch (lag) {
              case 1: ptx::bulk_wait_group<kChunks * 1>(); break;
              case 2: ptx::bulk_wait_group<kChunks * 2>(); break;
              case 3: ptx::bulk_wait_group<kChunks * 3>(); break;
              default: ptx::bulk_wait_group<kChunks * 4>(); break;
            }
            signal_group(ring[ring_head], ring_t[ring_head]);
            ring_head = (ring_head + 1) % kMaxLag;
            --ring_count;
          }
          ring[(ring_head + ring_count) % kMaxLag] = g;
          ring_t[(ring_head + ring_count) % kMaxLag] = t;
          ++ring_count;
        }
        // Flush: every push must have landed before it is announced, and no bulk copy may
        // still read this CTA's shared memory when it exits.
        ptx::bulk_wait_group<0>();
        while (ring_count > 0) {
          signal_group(ring[ring_head], ring_t[ring_head]);
          ring_head = (ring_head + 1) % kMaxLag;
          --ring_count;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ signal warp (fused)
    // Publishes finished tiles to their owners: ONE system-scope release fence for every tile
    // that is waiting in the ring, then a batch of relaxed atomics on the owners' arrival
    // counters that travel concurrently.  (A chain of red.release.sys would make every atomic
    // wait for the previous one's NVLink round trip.)
    if constexpr (FUSED) {
      if (lane == 0) {
        uint32_t total = 0;  // tiles this CTA computes
        for (int pos = unit; pos < sched_tiles; pos += num_units) total += MT;
        uint32_t n = 0;
        while (n < total) {
          if (!ptx::mbar_wait_bounded(&sig_full_bar[n % kSigRing], (n / kSigRing) & 1u, s_abort, pipe_timeout)) break;
          uint32_t m = 1;  // further tiles that are already waiting share the fence
          while (n + m < total && m < static_cast<uint32_t>(kSigRing) &&
                 ptx::mbar_try_wait(&sig_full_bar[(n + m) % kSigRing], ((n + m) / kSigRing) & 1u)) {
            ++m;
          }
          ptx::fence_proxy_async_all();
          ptx::fence_acq_rel_sys();
          for (uint32_t j = 0; j < m; ++j) {
            const uint32_t slot = (n + j) % kSigRing;
            const int g = s_sig_g[slot];
            for (int o = 0; o < p.ws; ++o) ptx::red_relaxed_sys_add(p.flags[(me + o) % p.ws] + g, 1u);
            if constexpr (TRACE) stamp(s_sig_t[slot], kTraceSignalled);
            ptx::mbar_arrive(&sig_empty_bar[slot]);
          }
          n += m;
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  if constexpr (CTA2) {
    // Neither CTA may free TMEM or leave while the other can still signal its barriers or
    // its MMAs read this CTA's shared memory.
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
    if (warp_idx == 1) {
      ptx::tc_fence_after_sync();
      ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
  } else {
    __syncthreads();
    if (warp_idx == 1) {
      ptx::tc_fence_after_sync();
      ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
  }
}

}  // namespace fo
