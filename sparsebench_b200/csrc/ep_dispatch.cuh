// Expert-parallel dispatch fused with the owner's first matmul: the device side shared by the SDD
// kernel's push warps, its gather warps and the stand-alone push kernel.
//
// Every rank is a SOURCE of token rows (its T*k copies, sorted by global expert) and an OWNER of
// E_local experts. Instead of "push all rows, barrier, then compute", rows travel while the owner's
// tensor cores already work:
//
//   source   walks its copies expert-major (local expert 0 of every destination first, then 1, ...),
//            in chunks of a few rows of one (destination d, local expert e) pair; a warp stores a
//            chunk's rows straight into d's receive buffer (plain stores through the peer mapping,
//            i.e. over NVLink), fences, and counts the chunk; whoever completes a pair's last chunk
//            publishes the step's epoch in d's flag [source][e] with a system-scope release store.
//   owner    before a gather warp of SDD reads the rows of a tile of local expert e it waits, bounded,
//            until the flags [s][e] of all sources s carry this step's epoch (acquire loads). Tiles
//            are walked expert-major too, so the first tiles need what arrives first.
//
// Nothing here waits for anything that itself waits: push warps never block, so two ranks' kernels
// cannot wait for each other in a circle. Flags carry a monotonically growing epoch (the value of the
// exchange's barrier counter in this step), so they are never reset.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

namespace sb {

constexpr int kPushChunkRows = 8;

// Upper bound of the chunks in a push plan: every (destination, expert) pair may end in a partial chunk, and an
// empty pair still has one (it only signals).
__host__ __device__ inline int64_t push_plan_max_chunks(int64_t n_copies, int32_t num_pairs) {
  return (n_copies + kPushChunkRows - 1) / kPushChunkRows + num_pairs;
}
// Ints in a push plan: four arrays of num_pairs + 1, then one int4 per chunk (16-byte aligned).
__host__ __device__ inline int64_t push_plan_ints(int64_t n_copies, int32_t num_pairs) {
  const int64_t head = (4 * static_cast<int64_t>(num_pairs + 1) + 3) / 4 * 4;
  return head + 4 * push_plan_max_chunks(n_copies, num_pairs);
}

struct DispatchParams {
  // Source side.
  const uint4* x;                // [T, D] this rank's token rows
  const int32_t* sorted_token;   // [T*k] token of every sorted position (sort by global expert)
  // Push plan, pair q = e * num_ranks + d. Four arrays of num_pairs + 1 ints back to back:
  //   chunk_prefix | first_pos (sorted position of the run) | slot_start (first slot i at d) | kept (rows)
  // then (at the next multiple of four ints) one int4 per chunk, in the order the chunks are pushed:
  //   x = sorted position of its first row, y = its first row in the destination's buffer,
  //   z = pair q, w = rows (low 8 bits) | chunks of the pair << 8.
  const int32_t* plan;
  uint4* const* peer_recv;       // [N] every rank's receive buffer [N * capacity, D]
  uint32_t* const* peer_flags;   // [N] every rank's arrival flags [N * E_local]
  uint32_t* done;                // [num_pairs] chunk counters of this rank, zero between kernels
  // Owner side.
  const uint32_t* my_flags;      // [N * E_local]
  // Both: the word whose current value is this step's epoch (the exchange's barrier counter).
  const uint32_t* epoch_word;
  int32_t my_rank;
  int32_t num_ranks;
  int32_t experts_local;
  int32_t capacity;
  int32_t vecs_per_row;          // D * 2 / 16
  int32_t num_pairs;             // N * E_local
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
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

// One warp's share of the source side: chunks worker, worker + num_workers, ... of the push plan. A chunk is one
// 16-byte record away (no search), its rows' tokens come with one coalesced load, and a row's loads are all in
// flight before its stores: what is left per chunk is one memory latency per row and one system fence.
__device__ __forceinline__ void push_chunks(const DispatchParams& dp, int worker, int num_workers, int lane) {
  const int32_t pairs = dp.num_pairs;
  const int32_t total = __ldg(dp.plan + pairs);  // chunk_prefix[pairs]
  const int4* table = reinterpret_cast<const int4*>(dp.plan + (4 * (pairs + 1) + 3) / 4 * 4);
  const uint32_t epoch = *dp.epoch_word;
  for (int32_t c = worker; c < total; c += num_workers) {
    const int4 chunk = __ldg(table + c);
    const int32_t q = chunk.z;
    const int32_t rows = chunk.w & 0xff;  // 0: the one chunk of an empty pair, which only signals
    const int32_t e = q / dp.num_ranks;
    const int32_t d = q - e * dp.num_ranks;
    if (rows > 0) {
      const int32_t my_token = lane < rows ? __ldg(dp.sorted_token + chunk.x + lane) : 0;
      uint4* dst = dp.peer_recv[d] + static_cast<int64_t>(chunk.y) * dp.vecs_per_row;
      for (int32_t r = 0; r < rows; ++r) {
        const int32_t token = __shfl_sync(0xffffffffu, my_token, r);
        copy_row_warp(dp.x + static_cast<int64_t>(token) * dp.vecs_per_row, dst + static_cast<int64_t>(r) * dp.vecs_per_row,
                      dp.vecs_per_row, lane);
      }
      __threadfence_system();  // this lane's rows are in the destination's memory before the count below
    }
    __syncwarp();
    if (lane == 0) {
      const uint32_t chunks = static_cast<uint32_t>(chunk.w) >> 8;
      if (atomicAdd(dp.done + q, 1u) + 1u == chunks) {
        dp.done[q] = 0u;          // ready for the next step
        __threadfence_system();   // the other chunks' rows (fenced before their counts) before the flag
        st_release_sys_u32(dp.peer_flags[d] + dp.my_rank * dp.experts_local + e, epoch);
      }
    }
  }
}

// Owner side, whole warp: until every source has delivered its rows for local expert e in this step.
// Lane s watches source s. Returns false when the wait ran out (1 s) or `*abort` was raised.
__device__ __forceinline__ bool wait_expert_arrived(const DispatchParams& dp, int32_t e, uint32_t epoch, int lane,
                                                    const volatile uint32_t* abort) {
  const uint32_t* flag = dp.my_flags + (lane < dp.num_ranks ? lane : 0) * dp.experts_local + e;
  const uint64_t start = dispatch_timer_ns();
  for (uint32_t poll = 0;; ++poll) {
    const bool here = lane >= dp.num_ranks || static_cast<int32_t>(ld_acquire_sys_u32(flag) - epoch) >= 0;
    if (__all_sync(0xffffffffu, here)) return true;
    if ((poll & 31u) == 31u) {
      const bool stop = *abort != 0u || dispatch_timer_ns() - start > 1000ull * 1000ull * 1000ull;
      if (__any_sync(0xffffffffu, stop)) return false;
    }
    __nanosleep(100);
  }
}

}  // namespace sb
