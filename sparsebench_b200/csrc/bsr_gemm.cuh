// The tensor-core core shared by the two block-sparse matmuls of the MoE layer (SDD and DSD).
//
// One output tile = one 128-row block x kTileN columns, accumulated in fp32 in TMEM by
// tcgen05.mma (M = 128, N = kTileN, K = 16 per instruction, four per 64-wide K step).
// The kernel is persistent: grid = number of SMs, every CTA walks tiles blockIdx.x, +gridDim.x, ...
// over the WORST-CASE tile count and reads from device memory (row_offsets) which row blocks are
// live, so the host never needs the real row count and dead tiles cost two loads.
//
// Warp roles (warp-specialised, nothing but mbarriers between them):
//   warp 0      lane 0: TMA producer. B tiles (weights, MN-major: [k rows][64 n] boxes, 128-byte
//               swizzle) for both ops, A tiles (H blocks, K-major) for DSD.
//   warp 1      lane 0: MMA issuer; the warp also owns the TMEM allocation (2 accumulators).
//   warps 2-9   epilogue: tcgen05.ld of the finished accumulator (lane quarter = warp % 4, column
//               half = (warp - 2) / 4), GELU for SDD, bf16 pack into a per-warp swizzled staging tile
//               (32 rows x 128 B) and one TMA store per 64 columns. Runs on accumulator i while
//               the MMA warp fills accumulator i^1.
//   warps 10-13 SDD only: A gather. Per K step each thread issues 8 cp.async of 16 bytes straight
//               from x[row_token] into the swizzled K-major stage; eight lanes share a row, so a warp
//               instruction moves four whole 128-byte row segments. Padding rows use the zero-fill
//               form (no global read). An asynchronous mbarrier arrive reports completion, so the
//               threads run the full pipeline depth ahead without ever waiting for their data.
//   warps 14-19 expert-parallel dispatch instance of SDD only (kDispatch): this rank's pushes as a source
//               of token rows (ep_dispatch.cuh).
//   warp 20     dispatch instance only: waits, ahead of the gather warps, for the 256-row segments each
//               tile's rows lie in to have arrived, and counts the complete tiles in shared memory; the
//               gather warps start a tile when that count covers it. Tiles follow the arrival order.
//
// Shared-memory stage layout (all 1024-byte aligned, as the 128-byte swizzle needs):
//   A: 128 rows x 128 B; 16-byte chunk c of row r is stored at chunk c ^ (r & 7)      (16 KB)
//   B: kTileN/64 slabs of [64 k rows x 128 B], same swizzle                          (kTileN*128 B)
//
// Options (GemmParams): skip_padding leaves out the stores (both ops) and loads (DSD) of 32-row groups
// that hold only padding; raster_rows walks the tiles in bands of row blocks for L2 reuse of the
// weights; peer_out makes the DSD epilogue store each row into another rank's buffer instead of y.
//
// Every wait is bounded; on expiry the role records a bit in *dev_status, raises the CTA's abort
// flag and all roles fall through to the common exit, where TMEM is released.
#pragma once

#include <cuda_bf16.h>

#include <atomic>
#include <cstdlib>

#include "ep_dispatch.cuh"
#include "ptx_sm100.cuh"
#include "sb_common.cuh"

namespace sb {

enum class GemmOp { kSdd, kDsd };

struct GemmParams {
  const int32_t* row_offsets;       // [num_row_blocks + 1]
  int32_t num_row_blocks;           // worst case
  int32_t num_slices;               // N / kTileN
  int32_t* dev_status;              // may be null
  // SDD
  const __nv_bfloat16* x;           // [T, D]
  const int32_t* row_token;         // [num_row_blocks * 128]
  const int32_t* row_block_expert;  // [num_row_blocks]
  __nv_bfloat16* h_out;             // [nnz, 128, 128]
  int32_t apply_gelu;
  // DSD
  const int32_t* col_indices;       // [nnz]
  __nv_bfloat16* y;                 // [num_row_blocks * 128, D]
  int32_t zero_dead_rows;
  int32_t block_rows;               // BSR block size: 128, or 64 (the tile's upper 64 rows then idle)
  // both
  int32_t d_model;
  // Padding rows sit at the END of every row block (the layout routing writes). When set, a group of
  // 32 rows that is all padding is not stored by either op and not loaded by DSD: SDD needs
  // row_token anyway, DSD reads it (same array) only for this.
  int32_t skip_padding;
  int32_t raster_rows;              // >= 1: row blocks per band of the tile walk
  // Weight tiles are read by several row blocks of the same expert at about the same time (experts with many row
  // blocks): keep them in L2 with the normal policy. Otherwise (about one reader per tile) they are marked
  // evict-first, so that the once-read weight stream does not push H or x out of L2.
  int32_t reuse_weights;
  // DSD as the last step of an expert-parallel owner: instead of y, row r of the layout (receive slot
  // j = row_token[r] = src * capacity + i) is stored into rank src's return buffer peer_out[src] at
  // row my_rank * capacity + i, straight from the epilogue (peer memory over NVLink). Null = off.
  void* const* peer_out;
  int32_t my_rank;
  int32_t capacity;
  // SDD as the first step of an expert-parallel owner whose rows are still arriving (kDispatch instance).
  DispatchParams dispatch;
};

template <GemmOp kOp, int kTileN, int kDispatch = 0>
struct GemmConfig {
  static constexpr int kTileM = 128;
  static constexpr int kTileK = 64;
  static constexpr int kUmmaK = 16;
  static constexpr int kABytes = kTileM * kTileK * 2;          // 16 KB
  static constexpr int kBSlabBytes = kTileK * 128;             // 64 k rows x 128 B = 8 KB
  static constexpr int kBSlabs = kTileN / 64;
  static constexpr int kBBytes = kBSlabs * kBSlabBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // Dispatch instances (expert-parallel owner whose rows are still arriving): 1 = this rank's rows are pushed by
  // warps (loads and stores through registers), 2 = by bulk copies through a ring in shared memory that one thread
  // drives; the ring takes the place of one pipeline stage.
  static constexpr bool kBulkPush = kDispatch == 2;
  static constexpr int kPushRingBytes = kBulkPush ? 48 * 1024 : 0;
  static constexpr int kStages = kTileN == 256 ? (kBulkPush ? 3 : 4) : 6;
  static constexpr int kEpilogueWarps = 8;
  static constexpr int kGatherWarps = kOp == GemmOp::kSdd ? 4 : 0;
  static constexpr int kFirstEpilogueWarp = 2;
  static constexpr int kFirstGatherWarp = kFirstEpilogueWarp + kEpilogueWarps;
  static constexpr int kPushWarps = kDispatch == 1 ? 6 : (kDispatch == 2 ? 1 : 0);
  static constexpr int kFirstPushWarp = kFirstGatherWarp + kGatherWarps;
  static constexpr int kArrivalWarp = kFirstPushWarp + kPushWarps;  // dispatch instance only
  static constexpr int kThreads = 32 * (kArrivalWarp + (kDispatch ? 1 : 0));
  static_assert(!kDispatch || kOp == GemmOp::kSdd, "only SDD has a dispatch instance");
  static constexpr int kTmemColumns = 2 * kTileN;              // two accumulators; 256 or 512
  static constexpr int kBarrierBytes = 256;
  static constexpr int kStagingBytes = 32 * 128;               // per epilogue warp: 32 rows x 64 bf16
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kPushRingBytes + kEpilogueWarps * kStagingBytes + kBarrierBytes;
  static constexpr uint32_t kFullArrivals = kOp == GemmOp::kSdd ? 1 + 32 * kGatherWarps : 1;
  static constexpr uint32_t kTxBytes = kOp == GemmOp::kSdd ? kBBytes : kStageBytes;
  static_assert(kTileN == 128 || kTileN == 256, "tile width");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// GELU in its erf form, 0.5 v (1 + erf(v / sqrt 2)), like the reference (csrc/sdd.cu:41), not the tanh form.
// erf is evaluated with the Abramowitz-Stegun 7.1.26 rational form, 1 - (a1 t + ... + a5 t^5) exp(-x^2),
// t = 1 / (1 + p |x|): absolute error below 1.5e-7 (5e-7 for the whole GELU in fp32), four orders below
// the bf16 rounding that follows, at about half the instructions of erff(). The epilogue applies it
// to 128 x 256 values per tile and would otherwise be issue-bound at full tensor rate.
__device__ __forceinline__ float gelu_erf(float v) {
  const float x = v * 0.70710678118654752f;
  const float a = fabsf(x);
  float t;  // 1 / (1 + p |x|): the hardware's approximate reciprocal (1 ulp) is ample here
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, a, 1.0f)));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float tail = poly * t * __expf(-a * a);  // 1 - erf(|x|)
  const float erf_abs = 1.0f - tail;
  return 0.5f * v * (1.0f + copysignf(erf_abs, x));
}

// The source side of the overlapped dispatch as bulk copies, driven by ONE thread of the thread block: a chunk of
// up to four rows is fetched from x into one of three buffers of a shared-memory ring (bulk loads counted on the
// buffer's mbarrier) and sent from there into its owner's receive buffer (bulk stores, one bulk group per chunk).
// No registers carry data and nothing waits for a load to come back before the next is issued, so one thread keeps
// 48 KB per SM in flight, in order: chunk j is stored while chunks j+1 and j+2 load. A chunk is counted towards its
// segment (ep_dispatch.cuh) once its group is complete, two chunks later, so the thread never waits for a store that
// it has only just issued. Chunk positions are walked like push_chunks walks them (slot-major, round-robin over the
// destinations), worker w of num_workers taking every num_workers-th. Returns false if a load did not arrive in time.
constexpr int kBulkMaxChunkRows = 4;

template <int kRingBytes>
__device__ inline bool push_rows_bulk(const DispatchParams& dp, uint32_t ring_base, uint32_t ring_bar, int worker,
                                      int num_workers, const volatile uint32_t* abort) {
  constexpr int kBufferBytes = kRingBytes / 3;
  const int32_t row_bytes = dp.vecs_per_row * 16;
  const int32_t chunk_rows = min(kBulkMaxChunkRows, kBufferBytes / row_bytes);  // 4, 2 or 1 (the host checks >= 1)
  const int32_t seg_chunks = kSegmentRows / chunk_rows;
  const int32_t ranks = dp.num_ranks;
  const int32_t total = dp.segments * seg_chunks * ranks;
  const uint32_t epoch = *dp.epoch_word;
  const char* x = reinterpret_cast<const char*>(dp.x);

  struct Chunk { int32_t d, slot0, rows, kept, token[kBulkMaxChunkRows]; };
  Chunk ring[16];  // descriptors of the chunks in flight: oldest not yet counted .. the one whose tokens are being read
  int32_t next_idx = worker;
  // The next position of this worker that holds rows; its tokens are read here and first used an iteration later.
  auto fetch = [&](Chunk& out) {
    for (; next_idx < total; next_idx += num_workers) {
      const int32_t c = next_idx / ranks;
      const int32_t d = (next_idx - c * ranks + dp.my_rank + c) % ranks;
      const int32_t base = __ldg(dp.expert_offsets + d * dp.experts_local);
      const int32_t kept = min(dp.capacity, __ldg(dp.expert_offsets + (d + 1) * dp.experts_local) - base);
      const int32_t slot0 = c * chunk_rows;
      if (slot0 >= kept) continue;
      out.d = d; out.slot0 = slot0; out.rows = min(chunk_rows, kept - slot0); out.kept = kept;
#pragma unroll
      for (int r = 0; r < kBulkMaxChunkRows; ++r)
        out.token[r] = r < out.rows ? __ldg(dp.sorted_token + base + slot0 + r) : 0;
      next_idx += num_workers;
      return true;
    }
    return false;
  };
  auto issue_loads = [&](int32_t j, const Chunk& ch) {
    const uint32_t buffer = ring_base + static_cast<uint32_t>(j % 3) * kBufferBytes;
    const uint32_t bar = ring_bar + 8u * static_cast<uint32_t>(j % 3);
    ptx::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ch.rows * row_bytes));
    for (int32_t r = 0; r < ch.rows; ++r)
      ptx::bulk_load(buffer + static_cast<uint32_t>(r * row_bytes), x + static_cast<int64_t>(ch.token[r]) * row_bytes,
                     static_cast<uint32_t>(row_bytes), bar);
  };
  // Chunks [from, to) are complete in their owners' memory: count them towards their segments. One fence for all of
  // them, the counters' round trips side by side.
  auto signal = [&](int32_t from, int32_t to) {
    if (from >= to) return;
    fence_acq_rel_sys();
    for (int32_t j0 = from; j0 < to; j0 += 4) {
      uint32_t before[4];
      uint32_t* counter[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const Chunk& ch = ring[(j0 + q) & 15];
        counter[q] = dp.done + ch.d * dp.segments + ch.slot0 / kSegmentRows;
        if (j0 + q < to) before[q] = atomicAdd(counter[q], 1u);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (j0 + q >= to) continue;
        const Chunk& ch = ring[(j0 + q) & 15];
        const int32_t g = ch.slot0 / kSegmentRows;
        const int32_t seg_rows = min(ch.kept, (g + 1) * kSegmentRows) - g * kSegmentRows;
        if (before[q] + 1u == static_cast<uint32_t>((seg_rows + chunk_rows - 1) / chunk_rows)) {
          *counter[q] = 0u;
          fence_acq_rel_sys();  // the other chunks of the segment (counted after their fences) before the flag
          st_relaxed_sys_u32(dp.peer_flags[ch.d] + dp.my_rank * dp.segments + g, epoch);
        }
      }
    }
  };

  // Chunks 0 and 1 are loading, the tokens of chunk 2 are on their way, before the first store is issued.
  int32_t fetched = 0, loading = 0;
  for (; fetched < 3 && fetch(ring[fetched & 15]); ++fetched) {}
  for (; loading < 2 && loading < fetched; ++loading) issue_loads(loading, ring[loading & 15]);
  bool ok = true;
  int32_t stored = 0, counted = 0;
  for (; stored < loading; ++stored) {
    const Chunk& ch = ring[stored & 15];
    if (!ptx::mbar_wait_bounded(ring_bar + 8u * static_cast<uint32_t>(stored % 3), static_cast<uint32_t>(stored / 3) & 1u,
                                abort)) {
      ok = false;
      break;
    }
    ptx::fence_proxy_async_shared();
    const uint32_t buffer = ring_base + static_cast<uint32_t>(stored % 3) * kBufferBytes;
    char* dst = reinterpret_cast<char*>(dp.peer_recv[ch.d]) +
                (static_cast<int64_t>(dp.my_rank) * dp.capacity + ch.slot0) * row_bytes;
    for (int32_t r = 0; r < ch.rows; ++r)
      ptx::bulk_store(dst + static_cast<int64_t>(r) * row_bytes, buffer + static_cast<uint32_t>(r * row_bytes),
                      static_cast<uint32_t>(row_bytes));
    ptx::bulk_commit();
    // The buffer of the chunk before this one is free once that chunk's group has read it.
    ptx::bulk_wait_read_but<1>();
    if (loading < fetched) {
      issue_loads(loading, ring[loading & 15]);
      ++loading;
    }
    if (fetched == loading && fetch(ring[fetched & 15])) ++fetched;  // tokens for the iteration after this one
    if (stored + 1 - 2 - counted >= 4) {  // four chunks (all but the two most recent groups) wait to be counted
      ptx::bulk_wait_but<2>();
      signal(counted, stored - 1);
      counted = stored - 1;
    }
  }
  ptx::bulk_wait_all();  // also on the way out after a failed wait: nothing of this block may still read the ring
  signal(counted, stored);
  return ok;
}

template <GemmOp kOp, int kTileN, int kDispatch = 0>
__global__ void __launch_bounds__(GemmConfig<kOp, kTileN, kDispatch>::kThreads, 1)
bsr_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_rows32,
                const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
                const __grid_constant__ GemmParams p) {
  using Cfg = GemmConfig<kOp, kTileN, kDispatch>;
  constexpr bool kIsSdd = kOp == GemmOp::kSdd;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = smem_base + Cfg::kStages * Cfg::kABytes;
  const uint32_t ring_base = smem_base + Cfg::kStages * Cfg::kStageBytes;     // bulk-push instance: three chunk buffers
  const uint32_t staging_base = ring_base + Cfg::kPushRingBytes;              // 1024-byte aligned
  const uint32_t bar_base = staging_base + Cfg::kEpilogueWarps * Cfg::kStagingBytes;
  const uint32_t full_bar = bar_base;                              // [kStages]
  const uint32_t empty_bar = bar_base + 8 * Cfg::kStages;          // [kStages]
  const uint32_t acc_full_bar = bar_base + 16 * Cfg::kStages;      // [2]
  const uint32_t acc_empty_bar = acc_full_bar + 16;                // [2]
  const uint32_t tmem_slot = acc_empty_bar + 16;                   // uint32
  const uint32_t abort_slot = tmem_slot + 4;                       // uint32
  const uint32_t arrived_slot = abort_slot + 4;                    // uint32, dispatch instance
  const uint32_t ring_bar = (arrived_slot + 4 + 7) & ~7u;          // [3], bulk-push instance
  // Generic pointers to the two words the threads read directly.
  uint8_t* smem_aligned = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
  volatile uint32_t* tmem_word = reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));
  // Dispatch instance: how many of this CTA's tiles (in walk order) have all their rows in the receive buffer.
  uint32_t* arrived_word = reinterpret_cast<uint32_t*>(smem_aligned + (arrived_slot - smem_base));

  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int lane = static_cast<int>(threadIdx.x & 31);

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      ptx::mbar_init(full_bar + 8 * s, Cfg::kFullArrivals);
      ptx::mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(acc_full_bar + 8 * a, 1);
      ptx::mbar_init(acc_empty_bar + 8 * a, 32 * Cfg::kEpilogueWarps);
    }
    *abort_word = 0u;
    *arrived_word = 0u;
    if (Cfg::kBulkPush)
      for (int b = 0; b < 3; ++b) ptx::mbar_init(ring_bar + 8 * b, 1);
    ptx::fence_barrier_init();
    if (!kIsSdd) ptx::prefetch_tensormap(&map_a);
    if (!kIsSdd && p.skip_padding) ptx::prefetch_tensormap(&map_a_rows32);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemColumns);
    ptx::tmem_relinquish();
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_word;

  const int32_t total_tiles = p.num_row_blocks * p.num_slices;
  auto give_up = [&](int bit) {
    *abort_word = 1u;
    if (p.dev_status != nullptr) atomicOr(p.dev_status, bit);
  };

  // What a role needs to know about a tile before it can start on it. Every role fetches the next
  // tile's record while it works on the current one, so these dependent global loads (row_offsets,
  // then the expert) are off the critical path at every tile boundary.
  struct TileInfo {
    int32_t begin, end, expert;
    int32_t groups;  // DSD with skip_padding: leading 32-row groups of the row block that hold real rows
  };
  // Tile order. Tiles are walked in bands of `raster_rows` row blocks: inside a band the row block
  // changes fastest, then the column slice (1 = plain row-block-major order). With a band of 8 the
  // CTAs that run at the same time work on the same ~18 column slices of (mostly) one expert's
  // weights for 8 row blocks at once, so a weight tile is fetched from HBM once and served from L2
  // to the other row blocks. That matters when an expert has many row blocks and many column
  // slices (SDD at F = 14336: a row-block-major wave covers only 2.6 row blocks, and W1 would be
  // streamed from HBM once per 2.6 row blocks); with ~2 row blocks per expert the plain order
  // already has both in flight together and is a little faster.
  const int32_t band_tiles = p.raster_rows * p.num_slices;
  auto row_block_of = [&](int32_t tile) {
    const int32_t band = tile / band_tiles;
    const int32_t first = band * p.raster_rows;
    const int32_t height = min(p.raster_rows, p.num_row_blocks - first);
    const int32_t position = first + (tile - band * band_tiles) % height;
    // Dispatch instance: the walk follows the order the rows arrive in, not the order of the layout.
    if (kDispatch && p.dispatch.row_block_order != nullptr) return __ldg(p.dispatch.row_block_order + position);
    return position;
  };
  auto slice_of = [&](int32_t tile) {
    const int32_t band = tile / band_tiles;
    const int32_t height = min(p.raster_rows, p.num_row_blocks - band * p.raster_rows);
    return (tile - band * band_tiles) / height;
  };
  auto load_tile_info = [&](int32_t tile) {
    const int32_t rb = row_block_of(tile);
    TileInfo info;
    info.begin = __ldg(p.row_offsets + rb);
    info.end = __ldg(p.row_offsets + rb + 1);
    info.expert = kIsSdd ? __ldg(p.row_block_expert + rb) : 0;
    info.groups = 0;
    if (!kIsSdd && p.skip_padding) {
      const int32_t* rows = p.row_token + static_cast<int64_t>(rb) * p.block_rows;
      for (int32_t g = 0; g < p.block_rows / 32; ++g) info.groups += __ldg(rows + 32 * g) >= 0 ? 1 : 0;
    }
    return info;
  };
  const int32_t tile_step = static_cast<int32_t>(gridDim.x);
  // DSD: K steps of 64 per BSR block (block size 128 -> 2, 64 -> 1), as a shift and a mask.
  const int32_t steps_shift = (!kIsSdd && p.block_rows == 64) ? 0 : 1;
  const int32_t steps_mask = (1 << steps_shift) - 1;
  const int32_t out_rows = kIsSdd ? Cfg::kTileM : p.block_rows;  // rows of the tile that are stored

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      // Weights and H blocks are each read once per launch: mark them first to go, so that the
      // streaming weights do not push H (written by SDD, read back by DSD) or x out of the L2.
      const uint64_t stream_once = ptx::policy_evict_first();
      const uint64_t weight_policy = p.reuse_weights ? ptx::policy_evict_normal() : stream_once;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int32_t tile = blockIdx.x;
      TileInfo cur = tile < total_tiles ? load_tile_info(tile) : TileInfo{0, 0, 0, 0};
      int32_t first_col = (!kIsSdd && cur.begin != cur.end) ? __ldg(p.col_indices + cur.begin) : 0;
      for (; ok && tile < total_tiles; tile += tile_step) {
        const int32_t next_tile = tile + tile_step;
        const TileInfo next = next_tile < total_tiles ? load_tile_info(next_tile) : TileInfo{0, 0, 0, 0};
        int32_t next_first_col = 0;
        const int32_t rb = row_block_of(tile);
        const int32_t n0 = slice_of(tile) * kTileN;
        const int32_t begin = cur.begin;
        const int32_t end = cur.end;
        const int32_t k_steps = begin == end ? 0 : (kIsSdd ? p.d_model / Cfg::kTileK : (end - begin) << steps_shift);
        const int32_t b_row_base = kIsSdd ? cur.expert * p.d_model : 0;
        int32_t col_block = 0;
        int32_t col_block_next = first_col;
        for (int32_t ks = 0; ks < k_steps; ++ks) {
          // A few steps in, the next tile's record has arrived: fetch its first column index too.
          if (!kIsSdd && ks == 4 && next.begin != next.end) next_first_col = __ldg(p.col_indices + next.begin);
          if (!ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, abort_word)) {
            give_up(SB_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t bar = full_bar + 8 * stage;
          const int32_t a_rows = (!kIsSdd && p.skip_padding) ? cur.groups * 32 : p.block_rows;
          ptx::mbar_arrive_expect_tx(bar, kIsSdd ? Cfg::kTxBytes : Cfg::kBBytes + a_rows * Cfg::kTileK * 2);
          int32_t b_row;
          if (kIsSdd) {
            b_row = b_row_base + ks * Cfg::kTileK;
          } else {
            // A 128-row block spans two 64-wide K steps, a 64-row block one.
            const int32_t blk = begin + (ks >> steps_shift);
            const int32_t k_half = (ks & steps_mask) * Cfg::kTileK;
            if (p.skip_padding && a_rows < p.block_rows) {
              // A row block that ends in padding: only its 32-row groups with real rows are fetched
              // (map_a_rows32 is map_a with a 32-row box). The rest of the stage keeps whatever it
              // held; those accumulator rows are never stored.
              for (int32_t g = 0; g < cur.groups; ++g)
                ptx::tma_load_2d_hint(a_base + stage * Cfg::kABytes + g * (32 * 128), &map_a_rows32, k_half,
                                      blk * p.block_rows + g * 32, bar, stream_once);
            } else {
              ptx::tma_load_2d_hint(a_base + stage * Cfg::kABytes, &map_a, k_half, blk * p.block_rows, bar, stream_once);
            }
            if ((ks & steps_mask) == 0) {
              // The next block's column index is fetched one block ahead to keep it off the issue path.
              col_block = col_block_next;
              if (blk + 1 < end) col_block_next = p.col_indices[blk + 1];
            }
            b_row = col_block * p.block_rows + k_half;
          }
          const uint32_t b_dst = b_base + stage * Cfg::kBBytes;
#pragma unroll
          for (int j = 0; j < Cfg::kBSlabs; ++j)
            ptx::tma_load_2d_hint(b_dst + j * Cfg::kBSlabBytes, &map_b, n0 + j * 64, b_row, bar, weight_policy);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!kIsSdd && k_steps <= 4 && next.begin != next.end) next_first_col = __ldg(p.col_indices + next.begin);
        cur = next;
        first_col = next_first_col;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t kIdesc = ptx::make_idesc_bf16(Cfg::kTileM, kTileN, /*b_mn_major=*/true);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      int32_t tile = blockIdx.x;
      TileInfo cur = tile < total_tiles ? load_tile_info(tile) : TileInfo{0, 0, 0, 0};
      for (; ok && tile < total_tiles; tile += tile_step) {
        const int32_t next_tile = tile + tile_step;
        const TileInfo next = next_tile < total_tiles ? load_tile_info(next_tile) : TileInfo{0, 0, 0, 0};
        const int32_t begin = cur.begin;
        const int32_t end = cur.end;
        cur = next;
        if (begin == end) continue;
        const int32_t k_steps = kIsSdd ? p.d_model / Cfg::kTileK : (end - begin) << steps_shift;
        if (!ptx::mbar_wait_bounded(acc_empty_bar + 8 * acc, acc_phase ^ 1u, abort_word)) {
          give_up(SB_DEV_TIMEOUT_MMA);
          break;
        }
        ptx::tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        for (int32_t ks = 0; ks < k_steps; ++ks) {
          if (!ptx::mbar_wait_bounded(full_bar + 8 * stage, phase, abort_word)) {
            give_up(SB_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          // The gathered A rows were written through the generic proxy (cp.async); order them
          // before the tensor core's async-proxy reads.
          if (kIsSdd) ptx::fence_proxy_async_shared();
          ptx::tcgen05_fence_after_sync();
          const uint32_t a_addr = a_base + stage * Cfg::kABytes;
          const uint32_t b_addr = b_base + stage * Cfg::kBBytes;
#pragma unroll
          for (int kk = 0; kk < Cfg::kTileK / Cfg::kUmmaK; ++kk) {
            // A: 16 K elements = 32 bytes along the swizzled 128-byte row.
            const uint64_t desc_a = ptx::make_smem_desc(a_addr + kk * 32, 16, 1024);
            // B: 16 k rows = two 1024-byte groups; slabs of 64 n are kBSlabBytes apart.
            const uint64_t desc_b = ptx::make_smem_desc(b_addr + kk * 2048, Cfg::kBSlabBytes, 1024);
            ptx::umma_bf16(d_tmem, desc_a, desc_b, kIdesc, (ks | kk) != 0);
          }
          ptx::umma_commit(empty_bar + 8 * stage);  // frees the stage once these MMAs have read it
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(acc_full_bar + 8 * acc);  // accumulator complete
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < Cfg::kFirstGatherWarp) {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes this warp may read: quarter*32 .. +31
    const int half = (warp - Cfg::kFirstEpilogueWarp) >> 2;
    const int row = quarter * 32 + lane;
    constexpr int kHalfCols = kTileN / 2;
    const uint32_t staging = staging_base + static_cast<uint32_t>(warp - Cfg::kFirstEpilogueWarp) * Cfg::kStagingBytes;
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
    const uint32_t stage_row = staging + static_cast<uint32_t>(lane) * 128u;
    uint32_t acc = 0, acc_phase = 0;
    for (int32_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int32_t rb = row_block_of(tile);
      const int32_t n0 = slice_of(tile) * kTileN;
      const int32_t begin = p.row_offsets[rb];
      const int32_t end = p.row_offsets[rb + 1];
      if (begin == end) {
        if (!kIsSdd && p.zero_dead_rows) {
          uint4* dst = reinterpret_cast<uint4*>(p.y + (static_cast<int64_t>(rb) * out_rows + row) * p.d_model + n0 +
                                                half * kHalfCols);
          if (row < out_rows) {
#pragma unroll
            for (int q = 0; q < kHalfCols / 8; ++q) dst[q] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        continue;
      }
      // This warp's 32 rows are all padding iff their first row is (padding sits at the end). Read
      // before the wait, so that the load is not on the path from "accumulator ready" to the stores.
      const bool rows_live = !p.skip_padding ||
                             (quarter * 32 < out_rows &&
                              __ldg(p.row_token + static_cast<int64_t>(rb) * out_rows + quarter * 32) >= 0);
      // Expert-parallel return: where this lane's row goes (0 = nowhere: a padding row).
      uint64_t row_dst = 0;
      if (!kIsSdd && p.peer_out != nullptr && quarter * 32 < out_rows) {
        const int32_t slot = __ldg(p.row_token + static_cast<int64_t>(rb) * out_rows + row);
        if (slot >= 0) {
          const int32_t src_rank = slot / p.capacity;
          const int64_t dst_row = static_cast<int64_t>(p.my_rank) * p.capacity + (slot - src_rank * p.capacity);
          row_dst = reinterpret_cast<uint64_t>(p.peer_out[src_rank]) + static_cast<uint64_t>(dst_row) * p.d_model * 2u;
        }
      }
      if (!ptx::mbar_wait_bounded(acc_full_bar + 8 * acc, acc_phase, abort_word)) {
        give_up(SB_DEV_TIMEOUT_EPILOGUE);
        break;
      }
      ptx::tcgen05_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kTileN + half * kHalfCols;
      // 64 columns at a time: TMEM -> registers -> (GELU) -> bf16 -> this warp's swizzled staging
      // tile [32 rows x 128 B] -> one TMA store, so global memory sees whole 128-byte row segments
      // instead of 32 scattered 16-byte pieces per instruction.
#pragma unroll 1
      for (int g = 0; rows_live && g < kHalfCols / 64; ++g) {
        uint32_t packed[32];  // this lane's row: 64 columns as bf16 pairs
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(t_addr + g * 64 + part * 32, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            float f0 = __uint_as_float(v[2 * h]);
            float f1 = __uint_as_float(v[2 * h + 1]);
            if (kIsSdd && p.apply_gelu) {
              f0 = gelu_erf(f0);
              f1 = gelu_erf(f1);
            }
            const __nv_bfloat162 pair = __floats2bfloat162_rn(f0, f1);
            packed[part * 16 + h] = *reinterpret_cast<const uint32_t*>(&pair);
          }
        }
        if (lane == 0) ptx::bulk_wait_read();  // the previous store has finished reading the staging tile
        __syncwarp();
#pragma unroll
        for (uint32_t c = 0; c < 8; ++c)
          ptx::st_shared_v4(stage_row + ((c ^ swz) << 4), packed[4 * c], packed[4 * c + 1], packed[4 * c + 2],
                            packed[4 * c + 3]);
        if (!kIsSdd && p.peer_out != nullptr) {
          // Eight lanes per row: every warp instruction stores four whole 128-byte row segments into
          // the buffers of the ranks the rows came from.
          __syncwarp();
          const int32_t col = n0 + half * kHalfCols + g * 64;
          const uint32_t chunk = static_cast<uint32_t>(lane & 7);
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3);
            const uint64_t dst = __shfl_sync(0xffffffffu, row_dst, r);
            const uint4 val = ptx::ld_shared_v4(staging + static_cast<uint32_t>(r) * 128u + ((chunk ^ static_cast<uint32_t>(r & 7)) << 4));
            if (dst != 0) *reinterpret_cast<uint4*>(dst + static_cast<uint64_t>(col + chunk * 8) * 2u) = val;
          }
          __syncwarp();  // the staging tile is free again
          continue;
        }
        ptx::fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0 && quarter * 32 < out_rows) {
          const int32_t col = n0 + half * kHalfCols + g * 64;  // first of 64 output columns
          if (kIsSdd) {
            // FFN column f lives in block begin + f/128, column f%128; 64 columns never straddle a block.
            ptx::tma_store_2d(&map_out, staging, col & 127, (begin + (col >> 7)) * Cfg::kTileM + quarter * 32);
          } else {
            ptx::tma_store_2d(&map_out, staging, col, rb * out_rows + quarter * 32);
          }
          ptx::bulk_commit();
        }
      }
      ptx::tcgen05_fence_before_sync();
      ptx::mbar_arrive(acc_empty_bar + 8 * acc);
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) ptx::bulk_wait_all();  // this warp's stores are complete before the CTA retires
  } else if (kIsSdd && warp < Cfg::kFirstPushWarp) {
    // ---------------------------------------------------------------- A gather (SDD)
    // Lane l = (g, c): g = l >> 3 picks one of four rows, c = l & 7 the 16-byte chunk of the 128-byte
    // K step, so one warp instruction moves four whole 128-byte row segments (coalesced in global
    // memory, conflict-free in shared memory). Warp gw covers rows j*16 + gw*4 + g, j = 0..7.
    const int gw = warp - Cfg::kFirstGatherWarp;
    const int row0 = gw * 4 + (lane >> 3);  // row for j = 0; rows for other j differ by multiples of 16
    const uint32_t chunk = static_cast<uint32_t>(lane & 7);
    const uint32_t dst_off = static_cast<uint32_t>(row0) * 128u + ((chunk ^ static_cast<uint32_t>(row0 & 7)) << 4);
    auto load_tokens = [&](int32_t tile, int32_t (&tok)[8]) {
      const int32_t* rows = p.row_token + static_cast<int64_t>(row_block_of(tile)) * Cfg::kTileM + row0;
#pragma unroll
      for (int j = 0; j < 8; ++j) tok[j] = __ldg(rows + j * 16);
    };
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    int32_t tile = blockIdx.x;
    int32_t tok[8];
    TileInfo cur = TileInfo{0, 0, 0, 0};
    if (tile < total_tiles) {
      load_tokens(tile, tok);
      cur = load_tile_info(tile);
    }
    uint32_t tiles_done = 0;  // dispatch instance: this CTA's tiles before the current one
    while (ok && tile < total_tiles) {
      // The next tile's record and row -> token table are fetched while this tile is gathered.
      const int32_t next = tile + tile_step;
      int32_t tok_next[8];
      TileInfo next_info = TileInfo{0, 0, 0, 0};
      if (next < total_tiles) {
        load_tokens(next, tok_next);
        next_info = load_tile_info(next);
      }
      const bool live = cur.begin != cur.end;
      cur = next_info;
      if (kDispatch) {
        // The rows of this tile may still be on their way: the arrival warp (below) watches the flags, several
        // tiles ahead, and counts the tiles that are complete in shared memory.
        while (ptx::ld_acquire_cta_u32(arrived_word) <= tiles_done && *abort_word == 0u) __nanosleep(20);
        if (*abort_word != 0u) break;
        ++tiles_done;
      }
      if (live) {
        const __nv_bfloat16* src[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // Padding rows still pass a valid address; the zero-fill form reads nothing from it.
          src[j] = p.x + (tok[j] >= 0 ? static_cast<int64_t>(tok[j]) * p.d_model : 0) + chunk * 8;
        }
        const int32_t k_steps = p.d_model / Cfg::kTileK;
        for (int32_t ks = 0; ks < k_steps; ++ks) {
          if (!ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, abort_word)) {
            give_up(SB_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t dst = a_base + stage * Cfg::kABytes + dst_off;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            ptx::cp_async_16_zfill(dst + j * 2048, src[j] + ks * Cfg::kTileK, tok[j] >= 0);
          ptx::cp_async_mbar_arrive_noinc(full_bar + 8 * stage);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) tok[j] = tok_next[j];
      tile = next;
    }
    ptx::cp_async_wait_all();
  } else if (kDispatch && warp == Cfg::kArrivalWarp) {
    // ---------------------------------------------------------------- dispatch arrivals (this rank as an owner)
    // Walks this CTA's tiles in order and waits, bounded, until the arrival flags of each tile's rows carry this
    // step's epoch; then raises the count the gather warps watch. The acquire loads that take a trip to L2 each are
    // thereby off the gather warps' path: once the rows are in, this warp is tiles ahead.
    const uint32_t dispatch_epoch = *p.dispatch.epoch_word;
    uint32_t tiles_done = 0;
    for (int32_t tile = blockIdx.x; tile < total_tiles; tile += tile_step) {
      const int32_t rb = row_block_of(tile);
      bool arrived = true;
      if (__ldg(p.row_offsets + rb) != __ldg(p.row_offsets + rb + 1)) {
        if (p.dispatch.row_block_order != nullptr) {
          const int32_t* list = p.dispatch.row_block_order + p.num_row_blocks + static_cast<int64_t>(rb) * kWaitStride;
          const int32_t count = __ldg(list);
          const int32_t flag_a = lane < count ? __ldg(list + 1 + lane) : 0;
          const int32_t flag_b = lane + 32 < count ? __ldg(list + 33 + lane) : 0;
          arrived = wait_list_arrived(p.dispatch, count, flag_a, flag_b, dispatch_epoch, lane, abort_word);
        } else {
          // No schedule: the flags are worked out from the rows' receive slots, 4 rows per lane.
          const int32_t* rows = p.row_token + static_cast<int64_t>(rb) * Cfg::kTileM;
          int32_t slot[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) slot[j] = j < 4 ? __ldg(rows + j * 32 + lane) : -1;
          arrived = wait_rows_arrived(p.dispatch, slot, dispatch_epoch, abort_word);
        }
      }
      if (!arrived) {
        if (lane == 0) give_up(SB_DEV_TIMEOUT_DISPATCH);
        break;
      }
      __syncwarp();  // every lane's acquire before the count
      ++tiles_done;
      if (lane == 0) ptx::st_release_cta_u32(arrived_word, tiles_done);
    }
  } else if (kDispatch) {
    // ---------------------------------------------------------------- dispatch pushes (this rank as a source)
    // Chunk position c of the slot-major walk goes to worker c mod (6 * grid): consecutive chunks to
    // different thread blocks, so that the segments every owner needs first are complete first. These warps
    // wait for nothing and run to the end of their list even if another role of the block has given up.
    if (Cfg::kBulkPush) {
      if (lane == 0 && !push_rows_bulk<Cfg::kPushRingBytes>(p.dispatch, ring_base, ring_bar, static_cast<int>(blockIdx.x),
                                                           static_cast<int>(gridDim.x), abort_word))
        give_up(SB_DEV_TIMEOUT_PRODUCER);
    } else {
    const int push_warp = warp - Cfg::kFirstPushWarp;
    // Fewer warps than there are finish the early chunks sooner (less queueing on the link) at a lower total rate.
    const int active = min(max(p.dispatch.push_warps, 0), Cfg::kPushWarps);  // 0: another launch pushes
    if (push_warp < active)
      push_chunks(p.dispatch, push_warp * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x),
                  active * static_cast<int>(gridDim.x), lane);
    }
  }

  // Common exit: every role is done (or has given up); release TMEM.
  if (*abort_word != 0u) {
    // Gave up mid-pipeline: leave bulk copies that are still in flight time to land in this CTA's
    // shared memory before it is handed back.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tcgen05_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemColumns);
  }
}

// ---- host side -----------------------------------------------------------------------------------

// Encodes a 2-D bf16 row-major tensor map [rows, cols] with a {64 x box_rows} box and 128-byte
// swizzle. Host only, no synchronisation. Returns SB_OK or records the failure.
int encode_bf16_2d_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       const char* what);

// Which L2 policy the weight tiles get. Evict-first everywhere unless SB_WEIGHT_POLICY=1 asks for the normal policy
// (an A/B knob): on the Mixtral-like shape, where eight row blocks share a weight tile, the normal policy raised the
// L2 hit rate from 63 % to 77 % and cut SDD's DRAM reads from 2.27 GB to 1.93 GB, but the kernels were not faster
// (SDD 942 us against 811-920 us over a run in which the power state drifted more than that), and on shapes with
// about one reader per tile it costs 5-7 %.
inline bool weights_reused_in_l2(int32_t /*num_row_blocks*/, int32_t /*num_experts*/) {
  const char* mode = std::getenv("SB_WEIGHT_POLICY");
  return mode != nullptr && mode[0] == '1';
}

// Opt-in to the large dynamic shared memory of one kernel instance, once per device. Two host threads
// may both find the flag clear and both set the attribute (harmless: same value); the flag itself is atomic.
template <GemmOp kOp, int kTileN, int kDispatch = 0>
int prepare_gemm_kernel(int device) {
  static std::atomic<bool> done[kMaxDevices] = {};
  if (done[device].load(std::memory_order_acquire)) return SB_OK;
  const cudaError_t err =
      cudaFuncSetAttribute(bsr_gemm_kernel<kOp, kTileN, kDispatch>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           GemmConfig<kOp, kTileN, kDispatch>::kSmemBytes);
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "shared memory opt-in: %s", cudaGetErrorString(err));
  done[device].store(true, std::memory_order_release);
  return SB_OK;
}

template <GemmOp kOp, int kTileN, int kDispatch = 0>
int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_a_rows32, const CUtensorMap& map_b,
                const CUtensorMap& map_out, const GemmParams& params, cudaStream_t stream, const char* what) {
  int device = 0;
  const DeviceInfo* info = current_device_info(&device);
  if (info == nullptr) return SB_ERR_CUDA;
  if (int rc = prepare_gemm_kernel<kOp, kTileN, kDispatch>(device)) return rc;
  using Cfg = GemmConfig<kOp, kTileN, kDispatch>;
  GemmParams launch_params = params;
  if (launch_params.raster_rows < 1) launch_params.raster_rows = 1;
  const int64_t tiles = static_cast<int64_t>(params.num_row_blocks) * params.num_slices;
  const unsigned grid = static_cast<unsigned>(tiles < info->sm_count ? tiles : info->sm_count);
  bsr_gemm_kernel<kOp, kTileN, kDispatch><<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_a, map_a_rows32, map_b,
                                                                                             map_out, launch_params);
  return check_launch(what);
}

}  // namespace sb
