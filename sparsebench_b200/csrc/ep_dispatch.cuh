// Expert-parallel dispatch fused with the owner's first matmul: the device side shared by the SDD
// kernel's push warps, its gather warps and the stand-alone push kernel.
//
// Every rank is a SOURCE of token rows (its T*k copies, sorted by global expert) and an OWNER of
// E_local experts. Instead of "push all rows, barrier, then compute", rows travel while the owner's
// tensor cores already work:
//
//   source   its copies bound for destination d are one contiguous run of the sort (d's experts are
//            consecutive), and copy j of that run goes to slot j of this source's region of d's receive
//            buffer (what exceeds the capacity is cut). The slot space is cut into chunks of 8 rows and
//            segments of 256 rows. Chunks are walked slot-major and round-robin over the destinations
//            (chunk 0 of every destination, then chunk 1, ...), so every destination's slots fill from
//            the front at about the same pace. A warp stores a chunk's rows straight into d's memory
//            (plain stores through the peer mapping, i.e. over NVLink), fences, and counts the chunk;
//            whoever completes a segment's last chunk publishes the step's epoch in d's flag
//            [source][segment] with a system-scope release store.
//   owner    before a gather warp of SDD reads the rows of a tile it waits, bounded, until the flags
//            of the segments those rows lie in carry this step's epoch. The owner walks its row blocks
//            in the order their last row's slot arrives (sb_ep_owner_layout writes that order), so the
//            tensor cores follow the arrivals instead of waiting for the last row of the first expert.
//
// Nothing here waits for anything that itself waits: push warps never block, so two ranks' kernels
// cannot wait for each other in a circle. Flags carry a monotonically growing epoch (the value of the
// exchange's barrier counter in this step), so they are never reset.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

namespace sb {

constexpr int kPushChunkRows = 8;
constexpr int kSegmentRows = 256;  // rows per arrival flag
constexpr int kSegmentChunks = kSegmentRows / kPushChunkRows;

// The owner's schedule (sb_ep_owner_layout writes it): after the num_row_blocks entries of the arrival order, one
// wait list of kWaitStride ints per row block: [0] = how many flags its rows depend on, [1 ...] = their indices
// into the owner's flag array (source * segments + segment). A row block of at most 256 rows touches at most two
// segments per source, so the list holds up to 31 sources.
constexpr int kWaitStride = 64;
constexpr int kMaxDispatchRanks = (kWaitStride - 1) / 2;
__host__ __device__ inline int64_t dispatch_schedule_ints(int64_t num_row_blocks) {
  return num_row_blocks * (1 + kWaitStride);
}

// Arrival flags (and the sender's chunk counters) per rank pair: one per segment of the capacity.
__host__ __device__ inline int32_t dispatch_segments(int32_t capacity) {
  return (capacity + kSegmentRows - 1) / kSegmentRows;
}

struct DispatchParams {
  // Source side.
  const uint4* x;                 // [T, D] this rank's token rows
  const int32_t* sorted_token;    // [T*k] token of every sorted position (sort by global expert)
  const int32_t* expert_offsets;  // [N * E_local + 1] first sorted position of every global expert
  uint4* const* peer_recv;        // [N] every rank's receive buffer [N * capacity, D]
  uint32_t* const* peer_flags;    // [N] every rank's arrival flags [N * segments]
  uint32_t* done;                 // [N * segments] chunk counters of this rank, zero between kernels
  // Owner side.
  const uint32_t* my_flags;       // [N * segments], flag [s][g]: rows g*256 .. of source s are here
  const int32_t* row_block_order; // the owner's schedule: [num_row_blocks] row blocks in the order to work on them,
                                  // then [num_row_blocks][kWaitStride] wait lists; or null (layout order, per-row waits)
  // Both: the word whose current value is this step's epoch (the exchange's barrier counter).
  const uint32_t* epoch_word;
  int32_t my_rank;
  int32_t num_ranks;
  int32_t experts_local;
  int32_t capacity;
  int32_t segments;               // dispatch_segments(capacity)
  int32_t vecs_per_row;           // D * 2 / 16
  int32_t push_warps;             // push warps per thread block that take part (inside the SDD kernel)
  int32_t bulk_engine;            // host side: take the SDD instance that pushes with bulk copies instead of warps
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t dispatch_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// One warp copies one row of `vecs` 16-byte vectors. Up to eight loads per lane are issued before the first
// store: written as "d[v] = s[v]" in a loop, every load would wait for the store before it (the two pointers
// may alias as far as the compiler knows), one memory latency per 512 bytes.
__device__ __forceinline__ void copy_row_warp(const uint4* __restrict__ src, uint4* __restrict__ dst, int32_t vecs,
                                              int lane) {
  for (int32_t v0 = lane; v0 < vecs; v0 += 32 * 8) {
    uint4 held[8];
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (v0 + 32 * q < vecs) held[q] = __ldg(src + v0 + 32 * q);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (v0 + 32 * q < vecs) dst[v0 + 32 * q] = held[q];
  }
}

// The same for TWO rows at once, for rows of whole groups of 256 vectors (2048 elements; the caller checks): sixteen
// loads per lane in flight, no predicates. Inside a matmul kernel, whose TMA traffic keeps
// the memory pipeline full, a load takes several microseconds to come back and a push warp is limited by the bytes
// it has in flight (4 KB per warp gave 33 MB in about 95 us over the chip; 8 KB halves that).
__device__ __forceinline__ void copy_two_rows_warp(const uint4* __restrict__ src0, const uint4* __restrict__ src1,
                                                   uint4* __restrict__ dst0, uint4* __restrict__ dst1, int32_t vecs,
                                                   int lane) {
  for (int32_t v0 = lane; v0 < vecs; v0 += 32 * 8) {
    uint4 a[8], b[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) a[q] = __ldg(src0 + v0 + 32 * q);
#pragma unroll
    for (int q = 0; q < 8; ++q) b[q] = __ldg(src1 + v0 + 32 * q);
#pragma unroll
    for (int q = 0; q < 8; ++q) dst0[v0 + 32 * q] = a[q];
#pragma unroll
    for (int q = 0; q < 8; ++q) dst1[v0 + 32 * q] = b[q];
  }
}

// One warp's share of the source side: chunks worker, worker + num_workers, ... of the slot-major, destination-
// round-robin walk. Nothing is looked up but two sort offsets per chunk; a chunk's tokens come with one coalesced
// load, and two rows' loads are in flight before their stores.
__device__ __forceinline__ void push_chunks(const DispatchParams& dp, int worker, int num_workers, int lane) {
  const int32_t ranks = dp.num_ranks;
  const int32_t total = dp.segments * kSegmentChunks * ranks;  // chunk positions, most of them past the rows
  const uint32_t epoch = *dp.epoch_word;
  for (int32_t idx = worker; idx < total; idx += num_workers) {
    const int32_t c = idx / ranks;  // chunk of the slot space: slots 8c .. 8c+7
    // Rotated by the rank (sources start at different destinations) and by the chunk (a worker whose stride is a
    // multiple of the rank count still visits every destination).
    const int32_t d = (idx - c * ranks + dp.my_rank + c) % ranks;
    const int32_t base = __ldg(dp.expert_offsets + d * dp.experts_local);
    const int32_t kept = min(dp.capacity, __ldg(dp.expert_offsets + (d + 1) * dp.experts_local) - base);
    const int32_t j0 = c * kPushChunkRows;
    if (j0 >= kept) continue;
    const int32_t rows = min(kPushChunkRows, kept - j0);
    const int32_t my_token = lane < rows ? __ldg(dp.sorted_token + base + j0 + lane) : 0;
    uint4* dst = dp.peer_recv[d] + (static_cast<int64_t>(dp.my_rank) * dp.capacity + j0) * dp.vecs_per_row;
    int32_t r = 0;
    for (; (dp.vecs_per_row & 255) == 0 && r + 1 < rows; r += 2) {
      const int32_t token0 = __shfl_sync(0xffffffffu, my_token, r);
      const int32_t token1 = __shfl_sync(0xffffffffu, my_token, r + 1);
      copy_two_rows_warp(dp.x + static_cast<int64_t>(token0) * dp.vecs_per_row,
                         dp.x + static_cast<int64_t>(token1) * dp.vecs_per_row,
                         dst + static_cast<int64_t>(r) * dp.vecs_per_row,
                         dst + static_cast<int64_t>(r + 1) * dp.vecs_per_row, dp.vecs_per_row, lane);
    }
    for (; r < rows; ++r) {
      const int32_t token = __shfl_sync(0xffffffffu, my_token, r);
      copy_row_warp(dp.x + static_cast<int64_t>(token) * dp.vecs_per_row, dst + static_cast<int64_t>(r) * dp.vecs_per_row,
                    dp.vecs_per_row, lane);
    }
    fence_acq_rel_sys();  // this lane's rows are in the destination's memory before the count below
    __syncwarp();
    if (lane == 0) {
      const int32_t g = c / kSegmentChunks;
      const int32_t seg_rows = min(kept, (g + 1) * kSegmentRows) - g * kSegmentRows;
      const uint32_t chunks = static_cast<uint32_t>((seg_rows + kPushChunkRows - 1) / kPushChunkRows);
      uint32_t* counter = dp.done + d * dp.segments + g;
      if (atomicAdd(counter, 1u) + 1u == chunks) {
        *counter = 0u;        // ready for the next step
        fence_acq_rel_sys();  // the other chunks' rows (fenced before their counts) before the flag: with the
                              // relaxed store below this is the release pattern
        st_relaxed_sys_u32(dp.peer_flags[d] + dp.my_rank * dp.segments + g, epoch);
      }
    }
  }
}

// Owner side, whole warp: until the eight receive slots this lane is about to gather (slot[j] < 0: a padding row,
// nothing to wait for) lie in segments whose flag carries this step's epoch. The polls are relaxed loads (eight
// acquire loads would each wait for the one before); one acquire fence after the last of them orders the gathers
// behind the flags. Returns false when the wait ran out (1 s) or `*abort` was raised.
__device__ __forceinline__ bool wait_rows_arrived(const DispatchParams& dp, const int32_t (&slot)[8], uint32_t epoch,
                                                  const volatile uint32_t* abort) {
  const uint32_t* flag[8];
  uint32_t pending = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int32_t source = slot[j] >= 0 ? slot[j] / dp.capacity : 0;
    const int32_t within = slot[j] >= 0 ? slot[j] - source * dp.capacity : 0;
    flag[j] = dp.my_flags + source * dp.segments + within / kSegmentRows;
    if (slot[j] >= 0) pending |= 1u << j;
  }
  const uint64_t start = dispatch_timer_ns();
  for (uint32_t poll = 0;; ++poll) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if ((pending >> j & 1u) && static_cast<int32_t>(ld_relaxed_sys_u32(flag[j]) - epoch) >= 0) pending &= ~(1u << j);
    if (__all_sync(0xffffffffu, pending == 0u)) break;
    if ((poll & 31u) == 31u) {
      const bool stop = *abort != 0u || dispatch_timer_ns() - start > 1000ull * 1000ull * 1000ull;
      if (__any_sync(0xffffffffu, stop)) return false;
    }
    __nanosleep(100);
  }
  fence_acq_rel_sys();
  return true;
}

// The same from a row block's wait list: lane i watches the list's flags i and i + 32 with acquire loads, all lanes
// at once (one round trip instead of one per flag, and no fence: the fence above also waits for everything this SM
// has in flight, about 12 us per tile next to a running matmul). The caller's __syncwarp() after it carries the
// lanes' acquires over to the whole warp.
__device__ __forceinline__ bool wait_list_arrived(const DispatchParams& dp, int32_t count, int32_t flag_a, int32_t flag_b,
                                                  uint32_t epoch, int lane, const volatile uint32_t* abort) {
  const uint32_t* a = lane < count ? dp.my_flags + flag_a : nullptr;
  const uint32_t* b = lane + 32 < count ? dp.my_flags + flag_b : nullptr;
  const uint64_t start = dispatch_timer_ns();
  for (uint32_t poll = 0;; ++poll) {
    if (a != nullptr && static_cast<int32_t>(ld_acquire_sys_u32(a) - epoch) >= 0) a = nullptr;
    if (b != nullptr && static_cast<int32_t>(ld_acquire_sys_u32(b) - epoch) >= 0) b = nullptr;
    if (__all_sync(0xffffffffu, a == nullptr && b == nullptr)) return true;
    if ((poll & 31u) == 31u) {
      const bool stop = *abort != 0u || dispatch_timer_ns() - start > 1000ull * 1000ull * 1000ull;
      if (__any_sync(0xffffffffu, stop)) return false;
    }
    __nanosleep(100);
  }
}

}  // namespace sb
