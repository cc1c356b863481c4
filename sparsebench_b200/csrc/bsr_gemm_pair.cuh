// The two block-sparse matmuls of the MoE layer on PAIRS of thread blocks (clusters of two CTAs, tcgen05
// cta_group::2), for layouts whose experts have many row blocks (few large experts: the tensor-bound regime).
//
// One tile = two consecutive row blocks of ONE expert x 256 columns. CTA r of the pair owns row block
// rb0 + r: it stages that row block's A (128 x 64 per K step: gathered rows for SDD, an H block for DSD) and
// only HALF of the weight tile B (columns 128 r .. 128 r + 127 of the 256), and gets its 128 x 256 fp32
// accumulator in its own TMEM. A single tcgen05.mma of the pair (M = 256, N = 256, K = 16), issued by the
// even CTA, reads both halves of A and B from the two CTAs' shared memory. Against the one-CTA kernel
// (bsr_gemm.cuh) each SM takes in 32 KB per K step instead of 48 KB and every weight tile is fetched once per
// 256 rows instead of once per 128: less L2 and shared-memory traffic, which is what runs out first when the
// tensor cores are the roof.
//
// Pairs never straddle experts: expert e with n row blocks has ceil(n / 2) pairs starting at its first row
// block; an odd last row block forms a pair whose second half is idle (its CTA still supplies its half of B).
// The pair list is not materialised: every CTA builds the per-expert prefix of pair counts from
// padded_offsets (the routing kernel's output, on the device) in shared memory at start, so the host still
// never learns a size, and the tile loop runs over the REAL number of pairs (no dead tiles).
//
// Warp roles in each CTA (same as the one-CTA kernel unless said):
//   warp 0      lane 0: TMA producer. Plain per-CTA loads (its B half, its H block); their byte counts go to
//               the full barrier of the stage in the LEADER's shared memory.
//   warp 1      TMEM allocation (both CTAs); lane 0 of the leader issues the MMAs and commits: one commit
//               arrives on the barrier of the same name in both CTAs (stage free, accumulator ready).
//   warps 2-9   epilogue on the CTA's own accumulator; "accumulator drained" goes to the leader's barrier.
//   warps 10-13 SDD: A gather into the CTA's own stage, completion counted on a local barrier;
//   warp 14     SDD: lane 0 forwards "this CTA's A rows of the stage are in" to the leader's full barrier
//               (cp.async completion can only be counted on a barrier of the same CTA).
// All waits are bounded as in the one-CTA kernel. The padding-row skipping, the banded tile walk and the
// expert-parallel peer-store epilogue of the one-CTA kernel are kept.
#pragma once

#include <cstdlib>

#include "bsr_gemm.cuh"

namespace sb {

constexpr int kMaxPairExperts = 128;

template <GemmOp kOp>
struct PairConfig {
  static constexpr int kTileM = 128;  // per CTA
  static constexpr int kTileN = 256;
  static constexpr int kTileK = 64;
  static constexpr int kUmmaK = 16;
  static constexpr int kABytes = kTileM * kTileK * 2;      // 16 KB
  static constexpr int kBSlabBytes = kTileK * 128;         // 64 k rows x 128 B = 8 KB
  static constexpr int kBSlabs = kTileN / 2 / 64;          // this CTA's half: 2 slabs
  static constexpr int kBBytes = kBSlabs * kBSlabBytes;    // 16 KB
  static constexpr int kStageBytes = kABytes + kBBytes;    // 32 KB
  static constexpr int kStages = 6;
  static constexpr int kEpilogueWarps = 8;
  static constexpr int kFirstEpilogueWarp = 2;
  static constexpr int kFirstGatherWarp = kFirstEpilogueWarp + kEpilogueWarps;
  static constexpr int kGatherWarps = kOp == GemmOp::kSdd ? 4 : 0;
  static constexpr int kRelayWarp = kFirstGatherWarp + kGatherWarps;
  static constexpr int kThreads = 32 * (kRelayWarp + (kOp == GemmOp::kSdd ? 1 : 0));
  static constexpr int kTmemColumns = 2 * kTileN;  // two accumulators
  static constexpr int kStagingBytes = 32 * 128;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kTableBytes = 2 * (kMaxPairExperts + 1) * 4;  // pair_start and first_rb
  static constexpr int kSmemBytes =
      1024 + kStages * kStageBytes + kEpilogueWarps * kStagingBytes + kBarrierBytes + ((kTableBytes + 15) / 16) * 16;
  // Arrivals per phase on the leader's full barrier: the two producers (with their byte counts) and, for SDD,
  // the two forwarding lanes.
  static constexpr uint32_t kFullArrivals = kOp == GemmOp::kSdd ? 4 : 2;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct PairParams {
  GemmParams g;                    // as in the one-CTA kernel (row_block_expert is not used)
  const int32_t* padded_offsets;   // [num_experts + 1] first padded row of every expert, [E] = rows in use
  int32_t num_experts;
};

template <GemmOp kOp>
__global__ void __launch_bounds__(PairConfig<kOp>::kThreads, 1)
bsr_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_rows32,
                     const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
                     const __grid_constant__ PairParams pp) {
  using Cfg = PairConfig<kOp>;
  constexpr bool kIsSdd = kOp == GemmOp::kSdd;
  constexpr int kTileN = Cfg::kTileN;
  const GemmParams& p = pp.g;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = smem_base + Cfg::kStages * Cfg::kABytes;
  const uint32_t staging_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
  const uint32_t bar_base = staging_base + Cfg::kEpilogueWarps * Cfg::kStagingBytes;
  const uint32_t full_bar = bar_base;                               // [kStages]  used in the leader
  const uint32_t empty_bar = full_bar + 8 * Cfg::kStages;           // [kStages]  both CTAs
  const uint32_t a_ready_bar = empty_bar + 8 * Cfg::kStages;        // [kStages]  both CTAs (SDD)
  const uint32_t acc_full_bar = a_ready_bar + 8 * Cfg::kStages;     // [2]        both CTAs
  const uint32_t acc_empty_bar = acc_full_bar + 16;                 // [2]        used in the leader
  const uint32_t tmem_slot = acc_empty_bar + 16;
  const uint32_t abort_slot = tmem_slot + 4;
  const uint32_t table_base = bar_base + Cfg::kBarrierBytes;        // int32 [num_experts + 1]
  uint8_t* smem_aligned = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
  volatile uint32_t* tmem_word = reinterpret_cast<volatile uint32_t*>(smem_aligned + (tmem_slot - smem_base));
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_aligned + (abort_slot - smem_base));
  int32_t* pair_start = reinterpret_cast<int32_t*>(smem_aligned + (table_base - smem_base));  // [E + 1]
  int32_t* first_rb = pair_start + (kMaxPairExperts + 1);                                     // [E + 1]

  const int warp = static_cast<int>(threadIdx.x >> 5);
  const int lane = static_cast<int>(threadIdx.x & 31);
  const uint32_t rank = ptx::cluster_cta_rank();  // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      ptx::mbar_init(full_bar + 8 * s, Cfg::kFullArrivals);
      ptx::mbar_init(empty_bar + 8 * s, 1);
      ptx::mbar_init(a_ready_bar + 8 * s, 32 * Cfg::kGatherWarps > 0 ? 32 * Cfg::kGatherWarps : 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(acc_full_bar + 8 * a, 1);
      ptx::mbar_init(acc_empty_bar + 8 * a, 2 * 32 * Cfg::kEpilogueWarps);
    }
    *abort_word = 0u;
    ptx::fence_barrier_init();
    if (!kIsSdd) ptx::prefetch_tensormap(&map_a);
    if (!kIsSdd && p.skip_padding) ptx::prefetch_tensormap(&map_a_rows32);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_out);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, Cfg::kTmemColumns);
    ptx::tmem_relinquish_pair();
  }
  if (warp == 2) {
    // Prefix of pair counts per expert: pair_start[e] = pairs of experts before e. One warp, 32 experts a step.
    int32_t carry = 0;
    for (int32_t e0 = 0; e0 < pp.num_experts; e0 += 32) {
      const int32_t e = e0 + lane;
      int32_t pairs = 0;
      if (e < pp.num_experts) {
        const int32_t blocks = (__ldg(pp.padded_offsets + e + 1) - __ldg(pp.padded_offsets + e)) / Cfg::kTileM;
        pairs = (blocks + 1) >> 1;
      }
      int32_t inclusive = pairs;
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t below = __shfl_up_sync(0xffffffffu, inclusive, d);
        if (lane >= d) inclusive += below;
      }
      if (e < pp.num_experts) {
        pair_start[e] = carry + inclusive - pairs;
        first_rb[e] = __ldg(pp.padded_offsets + e) / Cfg::kTileM;
      }
      carry += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    if (lane == 0) {
      pair_start[pp.num_experts] = carry;
      first_rb[pp.num_experts] = __ldg(pp.padded_offsets + pp.num_experts) / Cfg::kTileM;
    }
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // the peer's barriers are initialised before anything is sent to them
  ptx::tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_word;

  // Barriers that live in the leader, by their shared::cluster address (the leader's own included).
  const uint32_t full_bar_leader = ptx::map_to_cta(full_bar, 0);
  const uint32_t acc_empty_bar_leader = ptx::map_to_cta(acc_empty_bar, 0);

  auto give_up = [&](int bit) {
    *abort_word = 1u;
    if (p.dev_status != nullptr) atomicOr(p.dev_status, bit);
  };

  const int32_t total_pairs = pair_start[pp.num_experts];
  const int32_t total_tiles = total_pairs * p.num_slices;
  const int32_t band_tiles = p.raster_rows * p.num_slices;  // raster_rows counts PAIRS here
  const int32_t cluster_id = static_cast<int32_t>(blockIdx.x >> 1);
  const int32_t tile_step = static_cast<int32_t>(gridDim.x >> 1);

  // What every role needs to know about a tile. The two row blocks of a pair belong to one expert, whose
  // row blocks all have the same list of column blocks (the layout routing writes), so the K loop and the
  // weight rows are the pair's, while A, the padding groups and the output rows are each CTA's own.
  struct TileInfo {
    int32_t rb;        // this CTA's row block
    int32_t valid;     // 0: the pair's second half does not exist (odd last row block), this CTA only feeds B
    int32_t expert;
    int32_t n0;        // first of the tile's 256 output columns
    int32_t begin0;    // row_offsets of the pair's first row block (DSD: column list of the pair)
    int32_t blocks;    // DSD: blocks per row block (K = 128 * blocks)
    int32_t begin;     // row_offsets of this CTA's row block (first output / input block)
    int32_t groups;    // skip_padding: leading 32-row groups of this CTA's row block that hold real rows
  };
  auto load_tile_info = [&](int32_t tile) {
    if (tile >= total_tiles) return TileInfo{0, 0, 0, 0, 0, 0, 0, 0};
    const int32_t band = tile / band_tiles;
    const int32_t first = band * p.raster_rows;
    const int32_t height = min(p.raster_rows, total_pairs - first);
    const int32_t in_band = tile - band * band_tiles;
    const int32_t pair = first + in_band % height;
    TileInfo info;
    info.n0 = (in_band / height) * kTileN;
    int32_t lo = 0, hi = pp.num_experts - 1;  // last expert whose first pair is <= pair and that has pairs
    while (lo < hi) {
      const int32_t mid = (lo + hi + 1) >> 1;
      if (pair_start[mid] <= pair) lo = mid; else hi = mid - 1;
    }
    info.expert = lo;
    // Everything up to here comes from shared memory; the global loads below depend on nothing but rb0, so a
    // role can fetch the next tile's record while it works on the current one.
    const int32_t rb0 = first_rb[lo] + 2 * (pair - pair_start[lo]);
    info.rb = rb0 + static_cast<int32_t>(rank);
    info.valid = info.rb < first_rb[lo + 1] ? 1 : 0;
    info.begin0 = __ldg(p.row_offsets + rb0);
    info.blocks = __ldg(p.row_offsets + rb0 + 1) - info.begin0;
    info.begin = info.valid ? __ldg(p.row_offsets + info.rb) : info.begin0;
    info.groups = 4;
    if (p.skip_padding && info.valid) {
      const int32_t* rows = p.row_token + static_cast<int64_t>(info.rb) * Cfg::kTileM;
      info.groups = 0;
      for (int32_t g = 0; g < 4; ++g) info.groups += __ldg(rows + 32 * g) >= 0 ? 1 : 0;
    }
    return info;
  };
  auto k_steps_of = [&](const TileInfo& info) { return kIsSdd ? p.d_model / Cfg::kTileK : info.blocks * 2; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      const uint64_t stream_once = ptx::policy_evict_first();
      const uint64_t weight_policy = p.reuse_weights ? ptx::policy_evict_normal() : stream_once;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      TileInfo upcoming = load_tile_info(cluster_id);
      for (int32_t tile = cluster_id; ok && tile < total_tiles; tile += tile_step) {
        const TileInfo info = upcoming;
        upcoming = load_tile_info(tile + tile_step);
        const int32_t k_steps = k_steps_of(info);
        const int32_t a_rows = (kIsSdd || !info.valid) ? 0 : (p.skip_padding ? info.groups * 32 : Cfg::kTileM);
        const int32_t b_col = info.n0 + static_cast<int32_t>(rank) * (kTileN / 2);
        // DSD: the column index of block j + 1 is fetched while block j is issued, off the issue path.
        int32_t col_block = 0;
        int32_t col_block_next = (!kIsSdd && info.blocks > 0) ? __ldg(p.col_indices + info.begin0) : 0;
        for (int32_t ks = 0; ks < k_steps; ++ks) {
          {
            const bool free_stage = ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, abort_word);
            if (!free_stage) {
              give_up(SB_DEV_TIMEOUT_PRODUCER);
              ok = false;
              break;
            }
          }
          const uint32_t bar = full_bar_leader + 8 * stage;
          ptx::mbar_arrive_expect_tx_cluster(bar, Cfg::kBBytes + a_rows * Cfg::kTileK * 2);
          int32_t b_row;
          if (kIsSdd) {
            b_row = info.expert * p.d_model + ks * Cfg::kTileK;
          } else {
            const int32_t j = ks >> 1;
            const int32_t k_half = (ks & 1) * Cfg::kTileK;
            if (a_rows == Cfg::kTileM) {
              ptx::tma_load_2d_hint_pair(a_base + stage * Cfg::kABytes, &map_a, k_half, (info.begin + j) * Cfg::kTileM, bar,
                                         stream_once);
            } else {
              for (int32_t g = 0; g * 32 < a_rows; ++g)
                ptx::tma_load_2d_hint_pair(a_base + stage * Cfg::kABytes + g * (32 * 128), &map_a_rows32, k_half,
                                           (info.begin + j) * Cfg::kTileM + g * 32, bar, stream_once);
            }
            if ((ks & 1) == 0) {
              col_block = col_block_next;
              if (j + 1 < info.blocks) col_block_next = __ldg(p.col_indices + info.begin0 + j + 1);
            }
            b_row = col_block * Cfg::kTileM + k_half;
          }
          const uint32_t b_dst = b_base + stage * Cfg::kBBytes;
#pragma unroll
          for (int j = 0; j < Cfg::kBSlabs; ++j)
            ptx::tma_load_2d_hint_pair(b_dst + j * Cfg::kBSlabBytes, &map_b, b_col + j * 64, b_row, bar, weight_policy);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t kIdesc = ptx::make_idesc_bf16(2 * Cfg::kTileM, kTileN, /*b_mn_major=*/true);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      TileInfo upcoming = load_tile_info(cluster_id);
      for (int32_t tile = cluster_id; ok && tile < total_tiles; tile += tile_step) {
        const TileInfo info = upcoming;
        upcoming = load_tile_info(tile + tile_step);
        const int32_t k_steps = k_steps_of(info);
        {
          const bool drained = ptx::mbar_wait_bounded(acc_empty_bar + 8 * acc, acc_phase ^ 1u, abort_word);
          if (!drained) {
            give_up(SB_DEV_TIMEOUT_MMA);
            break;
          }
        }
        ptx::tcgen05_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        for (int32_t ks = 0; ks < k_steps; ++ks) {
          {
            const bool filled = ptx::mbar_wait_bounded(full_bar + 8 * stage, phase, abort_word);
            if (!filled) {
              give_up(SB_DEV_TIMEOUT_MMA);
              ok = false;
              break;
            }
          }
          if (kIsSdd) ptx::fence_proxy_async_shared();
          ptx::tcgen05_fence_after_sync();
          const uint32_t a_addr = a_base + stage * Cfg::kABytes;
          const uint32_t b_addr = b_base + stage * Cfg::kBBytes;
#pragma unroll
          for (int kk = 0; kk < Cfg::kTileK / Cfg::kUmmaK; ++kk) {
            const uint64_t desc_a = ptx::make_smem_desc(a_addr + kk * 32, 16, 1024);
            const uint64_t desc_b = ptx::make_smem_desc(b_addr + kk * 2048, Cfg::kBSlabBytes, 1024);
            ptx::umma_bf16_pair(d_tmem, desc_a, desc_b, kIdesc, (ks | kk) != 0);
          }
          ptx::umma_commit_pair(empty_bar + 8 * stage);  // the stage is free in both CTAs
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit_pair(acc_full_bar + 8 * acc);  // both CTAs' accumulators are complete
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < Cfg::kFirstGatherWarp) {
    // ---------------------------------------------------------------- epilogue (both CTAs, own accumulator)
    const int quarter = warp & 3;
    const int half = (warp - Cfg::kFirstEpilogueWarp) >> 2;
    const int row = quarter * 32 + lane;
    constexpr int kHalfCols = kTileN / 2;
    const uint32_t staging = staging_base + static_cast<uint32_t>(warp - Cfg::kFirstEpilogueWarp) * Cfg::kStagingBytes;
    const uint32_t swz = static_cast<uint32_t>(lane & 7);
    const uint32_t stage_row = staging + static_cast<uint32_t>(lane) * 128u;
    uint32_t acc = 0, acc_phase = 0;
    TileInfo upcoming = load_tile_info(cluster_id);
    for (int32_t tile = cluster_id; tile < total_tiles; tile += tile_step) {
      const TileInfo info = upcoming;
      upcoming = load_tile_info(tile + tile_step);
      const int32_t rb = info.rb;
      const int32_t n0 = info.n0;
      const bool rows_live = info.valid && quarter < info.groups;  // groups = 4 without skip_padding
      uint64_t row_dst = 0;
      if (!kIsSdd && p.peer_out != nullptr && info.valid) {
        const int32_t slot = __ldg(p.row_token + static_cast<int64_t>(rb) * Cfg::kTileM + row);
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
#pragma unroll 1
      for (int g = 0; rows_live && g < kHalfCols / 64; ++g) {
        uint32_t packed[32];
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
        if (lane == 0) ptx::bulk_wait_read();
        __syncwarp();
#pragma unroll
        for (uint32_t c = 0; c < 8; ++c)
          ptx::st_shared_v4(stage_row + ((c ^ swz) << 4), packed[4 * c], packed[4 * c + 1], packed[4 * c + 2],
                            packed[4 * c + 3]);
        if (!kIsSdd && p.peer_out != nullptr) {
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
          __syncwarp();
          continue;
        }
        ptx::fence_proxy_async_shared();
        __syncwarp();
        if (lane == 0) {
          const int32_t col = n0 + half * kHalfCols + g * 64;
          if (kIsSdd) {
            ptx::tma_store_2d(&map_out, staging, col & 127, (info.begin + (col >> 7)) * Cfg::kTileM + quarter * 32);
          } else {
            ptx::tma_store_2d(&map_out, staging, col, rb * Cfg::kTileM + quarter * 32);
          }
          ptx::bulk_commit();
        }
      }
      ptx::tcgen05_fence_before_sync();
      ptx::mbar_arrive_cluster(acc_empty_bar_leader + 8 * acc);
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) ptx::bulk_wait_all();
  } else if (kIsSdd && warp < Cfg::kRelayWarp) {
    // ---------------------------------------------------------------- A gather (SDD, both CTAs, own rows)
    const int gw = warp - Cfg::kFirstGatherWarp;
    const int row0 = gw * 4 + (lane >> 3);
    const uint32_t chunk = static_cast<uint32_t>(lane & 7);
    const uint32_t dst_off = static_cast<uint32_t>(row0) * 128u + ((chunk ^ static_cast<uint32_t>(row0 & 7)) << 4);
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    auto load_tokens = [&](const TileInfo& info, int32_t (&tok)[8]) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        tok[j] = info.valid ? __ldg(p.row_token + static_cast<int64_t>(info.rb) * Cfg::kTileM + row0 + j * 16) : -1;
    };
    TileInfo upcoming = load_tile_info(cluster_id);
    int32_t tok_upcoming[8];
    load_tokens(upcoming, tok_upcoming);
    for (int32_t tile = cluster_id; ok && tile < total_tiles; tile += tile_step) {
      int32_t tok[8];
      const __nv_bfloat16* src[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        tok[j] = tok_upcoming[j];
        src[j] = p.x + (tok[j] >= 0 ? static_cast<int64_t>(tok[j]) * p.d_model : 0) + chunk * 8;
      }
      // The next tile's record and row -> token table are fetched while this tile is gathered.
      upcoming = load_tile_info(tile + tile_step);
      load_tokens(upcoming, tok_upcoming);
      const int32_t k_steps = p.d_model / Cfg::kTileK;
      for (int32_t ks = 0; ks < k_steps; ++ks) {
        if (!ptx::mbar_wait_bounded(empty_bar + 8 * stage, phase ^ 1u, abort_word)) {
          give_up(SB_DEV_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        const uint32_t dst = a_base + stage * Cfg::kABytes + dst_off;
#pragma unroll
        for (int j = 0; j < 8; ++j) ptx::cp_async_16_zfill(dst + j * 2048, src[j] + ks * Cfg::kTileK, tok[j] >= 0);
        ptx::cp_async_mbar_arrive_noinc(a_ready_bar + 8 * stage);
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    ptx::cp_async_wait_all();
  } else if (kIsSdd && warp == Cfg::kRelayWarp) {
    // ---------------------------------------------------------------- "A rows are in" -> leader's full barrier
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int32_t tile = cluster_id; ok && tile < total_tiles; tile += tile_step) {
        const int32_t k_steps = p.d_model / Cfg::kTileK;
        for (int32_t ks = 0; ks < k_steps; ++ks) {
          if (!ptx::mbar_wait_bounded(a_ready_bar + 8 * stage, phase, abort_word)) {
            give_up(SB_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          // The rows were written by cp.async (generic proxy); the tensor core reads them through the async proxy.
          ptx::fence_proxy_async_shared();
          ptx::mbar_arrive_cluster(full_bar_leader + 8 * stage);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }

  if (*abort_word != 0u) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  ptx::tcgen05_fence_before_sync();
  __syncthreads();
  ptx::cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the pair's MMAs may still read its memory
  if (warp == 1) {
    ptx::tcgen05_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, Cfg::kTmemColumns);
  }
}

// ---- host side -----------------------------------------------------------------------------------

template <GemmOp kOp>
int prepare_pair_kernel(int device) {
  static std::atomic<bool> done[kMaxDevices] = {};
  if (done[device].load(std::memory_order_acquire)) return SB_OK;
  cudaError_t err = cudaFuncSetAttribute(bsr_gemm_pair_kernel<kOp>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PairConfig<kOp>::kSmemBytes);
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "shared memory opt-in (pair kernel): %s", cudaGetErrorString(err));
  done[device].store(true, std::memory_order_release);
  return SB_OK;
}

// Should a layout of `num_row_blocks` (worst case) over `num_experts` experts run on CTA pairs? Only where
// experts have several row blocks each (otherwise most pairs would be half idle) and the table fits.
inline bool pair_kernel_pays(int32_t num_row_blocks, int32_t num_experts) {
  return num_experts <= kMaxPairExperts && num_row_blocks >= 4 * num_experts;
}

// The decision for one launch: needs the routing kernel's padded_offsets (without it the kernel cannot
// pair row blocks by expert). SB_GEMM_PAIRS=0 turns the pair kernel off, =2 forces it wherever it can run
// (for A/B measurements), =1 uses it where pair_kernel_pays says so; unset, it stays off (see below).
inline bool use_pair_kernel(const int32_t* padded_offsets, int32_t num_row_blocks, int32_t num_experts) {
  if (padded_offsets == nullptr || num_experts > kMaxPairExperts || num_row_blocks < 1) return false;
  const char* mode = std::getenv("SB_GEMM_PAIRS");
  if (mode != nullptr && mode[0] == '0') return false;
  if (mode != nullptr && mode[0] == '2') return true;
  if (mode != nullptr && mode[0] == '1') return pair_kernel_pays(num_row_blocks, num_experts);
  // Off unless asked for: on the Mixtral-like shape (8 experts, D = 4096, F = 14336) the pair kernels measured
  // 849 / 918 us (SDD / DSD) against 813 / 849 us for the one-CTA kernels, and the layer 1.83 ms against 1.74 ms.
  return false;
}

// How many pairs of this kernel can be resident at once on `device`. The tile walk is static (tile, tile +
// clusters, ...), so every launched cluster must be resident together: a pair needs two free SMs of one GPC, and
// not every SM of the chip can be paired. Asked once per device (a host-side query, no synchronisation).
template <GemmOp kOp>
int pair_resident_clusters(int device, int sm_count, int* out) {
  static std::atomic<int> cached[kMaxDevices] = {};
  int fit = cached[device].load(std::memory_order_acquire);
  if (fit == 0) {
    if (int rc = prepare_pair_kernel<kOp>(device)) return rc;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(sm_count / 2 * 2));
    config.blockDim = dim3(PairConfig<kOp>::kThreads);
    config.dynamicSmemBytes = PairConfig<kOp>::kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    const cudaError_t occ = cudaOccupancyMaxActiveClusters(&fit, bsr_gemm_pair_kernel<kOp>, &config);
    if (occ != cudaSuccess || fit < 1)
      return fail(SB_ERR_CUDA, "pair kernel: cudaOccupancyMaxActiveClusters: %s", cudaGetErrorString(occ));
    cached[device].store(fit, std::memory_order_release);
  }
  *out = fit;
  return SB_OK;
}

template <GemmOp kOp>
int launch_gemm_pair(const CUtensorMap& map_a, const CUtensorMap& map_a_rows32, const CUtensorMap& map_b,
                     const CUtensorMap& map_out, const GemmParams& params, const int32_t* padded_offsets,
                     int32_t num_experts, cudaStream_t stream, const char* what) {
  int device = 0;
  const DeviceInfo* info = current_device_info(&device);
  if (info == nullptr) return SB_ERR_CUDA;
  if (int rc = prepare_pair_kernel<kOp>(device)) return rc;
  using Cfg = PairConfig<kOp>;
  PairParams pp{};
  pp.g = params;
  if (pp.g.raster_rows < 1) pp.g.raster_rows = 1;
  pp.padded_offsets = padded_offsets;
  pp.num_experts = num_experts;
  // Worst case number of pair tiles: every expert may end in a half pair.
  const int64_t tiles = static_cast<int64_t>((params.num_row_blocks + num_experts + 1) / 2) * params.num_slices;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(info->sm_count / 2 * 2));
  config.blockDim = dim3(Cfg::kThreads);
  config.dynamicSmemBytes = Cfg::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  int fit = 0;
  if (int rc = pair_resident_clusters<kOp>(device, info->sm_count, &fit)) return rc;
  int64_t clusters = fit;
  if (clusters > info->sm_count / 2) clusters = info->sm_count / 2;
  if (tiles < clusters) clusters = tiles;
  if (clusters < 1) clusters = 1;
  config.gridDim = dim3(static_cast<unsigned>(2 * clusters));
  const cudaError_t err = cudaLaunchKernelEx(&config, bsr_gemm_pair_kernel<kOp>, map_a, map_a_rows32, map_b, map_out, pp);
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "%s (pair kernel): %s", what, cudaGetErrorString(err));
  return check_launch(what);
}

}  // namespace sb
