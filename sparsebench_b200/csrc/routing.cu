// Routing -> block-sparse layout on the device, with no host sync and no atomics.
//
// The T*k token copies (copy c = t*k + j) are sorted by expert with a stable counting sort and each
// expert's group is padded to a multiple of block_size. The result is bit-exact to the reference's
// topology.build_topology (sparsebench/topology.py:53-118) and build_topology_cuda
// (csrc/routing.cu:197-281), including the -1 / flat tails of the worst-case sized buffers.
//
// How order is kept without atomics: a warp walks a contiguous run of copies 32 at a time, in copy
// order. Inside one step every lane learns which lanes hold the same expert (one ballot per bit of
// the id; the same mask __match_any_sync gives, which was measured far slower here); the number of
// those below it is its rank, and the lowest of them alone updates that warp's private per-expert
// counter. Runs are laid out in copy order (block 0 warp 0 first), so an exclusive scan of the
// counters over (block, warp) for each expert gives every run its base, and base + running count +
// rank is the copy's position inside its expert. Nothing depends on which thread wins a race, so
// two launches always agree.
//
// Two launch shapes:
//   cluster (n <= 131072 copies): ONE launch of a thread-block cluster (1-8 blocks of 1024 threads)
//       does count, scan, scatter and the layout arrays; the blocks share their per-expert counts
//       through distributed shared memory. This is the hot-path shape (8192 copies per layer call).
//   large: chunk histograms -> one-block scan -> scatter + layout, three launches and a scratch
//       buffer of chunks x (E + 1) ints.
// Padding rows and rows past the real end get row_token = -1 from the layout pass itself (a row
// is written exactly once, by the scatter or by the fill), so no memset is needed.

#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <atomic>

#include "ep_dispatch.cuh"
#include "sb_common.cuh"

namespace sb {
namespace {

namespace cg = cooperative_groups;

constexpr int kMaxExperts = 1024;  // one thread per expert in the scan block (reference: csrc/routing.cu:31)
constexpr unsigned kFullMask = 0xffffffffu;
constexpr int kClusterThreads = 1024;
constexpr int kMaxClusterBlocks = 8;    // the portable cluster size limit
constexpr int kMaxRunSteps = 16;        // 32-copy steps a warp keeps in registers (more would spill at 1024 threads)
constexpr int64_t kClusterMaxCopies = static_cast<int64_t>(kMaxClusterBlocks) * kClusterThreads * kMaxRunSteps;  // 131072
constexpr int kChunkThreads = 256;
constexpr int kChunkWarps = kChunkThreads / 32;
constexpr int kChunkCopies = 2048;  // copies per block in the large shape

template <typename index_t>
__device__ __forceinline__ int32_t read_expert(const index_t* __restrict__ expert_idx, int64_t c, int64_t end,
                                               int32_t num_experts, bool& bad) {
  if (c >= end) return -1;
  const index_t v = expert_idx[c];
  if (v >= 0 && v < static_cast<index_t>(num_experts)) return static_cast<int32_t>(v);
  bad = true;  // skipped: nothing is written for it except copy_row = -1
  return -1;
}

// A warp's run of copies is read up front, kIters x 32 ids into registers, so that the loads are all
// in flight together instead of one memory latency per step. Returns true if a bad id was seen.
template <typename index_t, int kIters>
__device__ __forceinline__ bool load_run(const index_t* __restrict__ expert_idx, int64_t begin, int64_t end,
                                         int32_t num_experts, int lane, int32_t (&ids)[kIters]) {
  bool bad = false;
#pragma unroll
  for (int it = 0; it < kIters; ++it) ids[it] = read_expert(expert_idx, begin + it * 32 + lane, end, num_experts, bad);
  return bad;
}

// Lanes of the warp that hold the same expert as this lane (0 for a lane without a valid copy).
// Same mask __match_any_sync(active, e) returns, built from one ballot per bit of the expert id:
// on B200 the match instruction took about 65 cycles per DISTINCT value in the warp (1740 cycles
// per step with 64 uniformly used experts), log2(E) ballots take a small constant.
__device__ __forceinline__ unsigned same_expert_lanes(int32_t e, bool valid, int id_bits) {
  unsigned peers = __ballot_sync(kFullMask, valid);
  for (int b = 0; b < id_bits; ++b) {
    const bool bit = (e >> b) & 1;
    const unsigned with_bit = __ballot_sync(kFullMask, bit);
    peers &= bit ? with_bit : ~with_bit;
  }
  return valid ? peers : 0u;
}

// Where a warp's run of expert ids comes from. IndexSource reads the caller's expert_idx. LogitSource is the
// router itself: it reads the tokens' router logits, picks the k largest per token (ties to the lower id, NaN
// above everything, as torch.topk orders them), writes expert_idx and the softmax of the k picked logits
// (reference: sparsebench/reference.py:19-29) and hands the ids on in registers, so that logits -> layout is ONE
// launch and the ids never make a round trip through memory before they are sorted.
template <typename index_t>
struct IndexSource {
  const index_t* expert_idx;
  int32_t num_experts;
  template <int kIters>
  __device__ __forceinline__ bool load(int64_t begin, int64_t end, int lane, int32_t (&ids)[kIters]) const {
    return load_run<index_t, kIters>(expert_idx, begin, end, num_experts, lane, ids);
  }
};

constexpr int kRouterMaxK = 8;

__device__ __forceinline__ bool logit_ranks_before(float a, float b) {
  // a strictly before b in torch.topk's order: NaN above everything, then the larger value. Equal values keep
  // the order they were met in (the lower expert id first).
  const bool an = a != a, bn = b != b;
  if (an != bn) return an;
  return !an && a > b;
}

template <typename logit_t>
struct LogitSource {
  const logit_t* logits;   // [T, E]
  int64_t* expert_idx;     // [T, k] out
  logit_t* expert_weight;  // [T, k] out
  int32_t num_experts;
  int32_t k;               // a power of two <= 8, so that a 32-copy step holds whole tokens

  static __device__ __forceinline__ float to_float(float v) { return v; }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

  // A 32-copy step holds 32 / k whole tokens, k consecutive lanes per token (one per copy). The k lanes of a token
  // share its E logits (lane p scans experts p, p + k, ...: adjacent addresses), each keeps the k best of its share
  // in registers (insertion into a short sorted list), and a butterfly of shuffles merges the k lists, after which
  // every lane of the token holds the token's k best and takes the one of its copy. k is a template argument of
  // the worker below: the lists are unrolled k deep, not 8 deep with predicates (every warp of the few routing
  // blocks issues these instructions, so their count is the kernel's time).
  template <int kIters>
  __device__ __forceinline__ bool load(int64_t begin, int64_t end, int lane, int32_t (&ids)[kIters]) const {
    switch (k) {
      case 1: return load_k<kIters, 1>(begin, end, lane, ids);
      case 2: return load_k<kIters, 2>(begin, end, lane, ids);
      case 4: return load_k<kIters, 4>(begin, end, lane, ids);
      default: return load_k<kIters, 8>(begin, end, lane, ids);
    }
  }

  // (v, id) goes in front of the first entry it beats: a larger logit (NaN above everything), or an equal one with
  // a lower expert id (torch.topk's order); everything from there on moves down, what falls off the end is dropped.
  template <int K>
  static __device__ __forceinline__ void insert(float (&best)[K], int32_t (&best_id)[K], float v, int32_t id) {
    bool shifting = false;
#pragma unroll
    for (int r = 0; r < K; ++r) {
      const bool beats = best_id[r] < 0 || logit_ranks_before(v, best[r]) ||
                         (!logit_ranks_before(best[r], v) && id < best_id[r]);
      if (id >= 0 && (shifting || beats)) {
        shifting = true;
        const float tv = best[r];
        const int32_t ti = best_id[r];
        best[r] = v;
        best_id[r] = id;
        v = tv;
        id = ti;
      }
    }
  }

  template <int kIters, int K>
  __device__ __forceinline__ bool load_k(int64_t begin, int64_t end, int lane, int32_t (&ids)[kIters]) const {
    const int pick = lane % K;
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      ids[it] = -1;
      const int64_t step_begin = begin + it * 32;
      if (step_begin >= end) continue;  // uniform across the warp
      const int64_t copy = step_begin + lane;
      const bool live = copy < end;  // the n copies are whole tokens, so a token's k lanes are live together
      float best[K];
      int32_t best_id[K];
#pragma unroll
      for (int r = 0; r < K; ++r) {
        best[r] = -INFINITY;
        best_id[r] = -1;
      }
      if (live) {
        const logit_t* row = logits + (copy / K) * num_experts;
        // Eight loads in flight before the first is used: one at a time, the walk is a chain of memory latencies
        // (a 32-byte sector lasts the token's lanes four steps at k = 2) on the few SMs this kernel runs on.
        for (int32_t e0 = pick; e0 < num_experts; e0 += 8 * K) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = e0 + u * K < num_experts ? to_float(__ldg(row + e0 + u * K)) : 0.0f;
#pragma unroll
          for (int u = 0; u < 8; ++u) insert<K>(best, best_id, v[u], e0 + u * K < num_experts ? e0 + u * K : -1);
        }
      }
#pragma unroll
      for (int d = 1; d < K; d <<= 1) {  // the partner's list is merged entry by entry (an id of -1 is no entry)
        float theirs[K];
        int32_t their_id[K];
#pragma unroll
        for (int r = 0; r < K; ++r) {
          theirs[r] = __shfl_xor_sync(kFullMask, best[r], d);
          their_id[r] = __shfl_xor_sync(kFullMask, best_id[r], d);
        }
#pragma unroll
        for (int r = 0; r < K; ++r) insert<K>(best, best_id, theirs[r], their_id[r]);
      }
      if (live) {
        float denom = 0.0f;
#pragma unroll
        for (int r = 0; r < K; ++r) denom += __expf(best[r] - best[0]);
        float mine = best[0];
        int32_t mine_id = best_id[0];
#pragma unroll
        for (int r = 1; r < K; ++r)
          if (r == pick) {
            mine = best[r];
            mine_id = best_id[r];
          }
        expert_idx[copy] = mine_id;
        store(expert_weight + copy, __expf(mine - best[0]) / denom);
        ids[it] = mine_id;
      }
    }
    return false;
  }
};

// One warp walks its run 32 copies per step, in copy order, and adds it to its private counters.
// For every copy it also finds pos = the number of copies of the same expert that come earlier in
// this run: the lanes holding the same expert below this one count towards pos, and the lowest of
// them alone reads and advances the counter (one writer per expert per step) and hands the old
// value to its peers. Nothing here depends on timing, so the order is stable.
// The result replaces the id in place: ids[it] becomes pos << 16 | (id & 0xffff) (an id is < 1024 or -1,
// a pos is < the run length <= 1024), so that a long run costs one register per copy, not two.
__device__ __forceinline__ int32_t packed_id(int32_t packed) {
  const int32_t low = packed & 0xffff;
  return low == 0xffff ? -1 : low;
}
__device__ __forceinline__ int32_t packed_pos(int32_t packed) { return static_cast<int32_t>(static_cast<uint32_t>(packed) >> 16); }

template <int kIters>
__device__ __forceinline__ void rank_run(int32_t (&ids)[kIters], int64_t begin, int64_t end, int id_bits,
                                         int32_t* counters, int lane) {
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int32_t e = ids[it];
    ids[it] = e & 0xffff;
    if (begin + it * 32 >= end) continue;  // uniform across the warp
    const unsigned peers = same_expert_lanes(e, e >= 0, id_bits);
    int32_t before = 0;
    if (peers != 0 && (peers & ((1u << lane) - 1u)) == 0) {
      before = counters[e];
      counters[e] = before + __popc(peers);
    }
    const int leader = peers != 0 ? __ffs(peers) - 1 : lane;
    before = __shfl_sync(kFullMask, before, leader);
    ids[it] |= (before + __popc(peers & ((1u << lane) - 1u))) << 16;
    __syncwarp();
  }
}

// Places a run. bases[e] = copies of expert e before this run (earlier chunks and warps).
template <int kIters>
__device__ __forceinline__ void scatter_run(const int32_t (&ranked)[kIters], int64_t begin, int64_t end, int32_t k,
                                            const int32_t* bases, const int32_t* padded_offsets,
                                            int32_t* __restrict__ copy_row, int32_t* __restrict__ row_token, int lane) {
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int64_t c = begin + it * 32 + lane;
    if (c >= end) continue;
    const int32_t e = packed_id(ranked[it]);
    if (e >= 0) {
      const int32_t row = padded_offsets[e] + bases[e] + packed_pos(ranked[it]);
      copy_row[c] = row;
      row_token[row] = static_cast<int32_t>(static_cast<uint32_t>(c) / static_cast<uint32_t>(k));
    } else {
      copy_row[c] = -1;  // bad id: skipped
    }
  }
}

// Exclusive scan of one value per thread over the whole block (blockDim.x <= 1024, multiple of 32).
__device__ int32_t block_exclusive_scan(int32_t value, int32_t* warp_sums /* [32] shared */, int32_t* total) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int32_t inclusive = value;
  for (int d = 1; d < 32; d <<= 1) {
    const int32_t below = __shfl_up_sync(kFullMask, inclusive, d);
    if (lane >= d) inclusive += below;
  }
  if (lane == 31) warp_sums[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    const int num_warps = blockDim.x >> 5;
    int32_t s = lane < num_warps ? warp_sums[lane] : 0;
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t below = __shfl_up_sync(kFullMask, s, d);
      if (lane >= d) s += below;
    }
    warp_sums[lane] = s;  // inclusive over warps
  }
  __syncthreads();
  const int32_t base = warp > 0 ? warp_sums[warp - 1] : 0;
  if (total != nullptr) *total = warp_sums[(blockDim.x >> 5) - 1];
  return base + inclusive - value;
}

struct LayoutOut {
  int32_t* row_token;
  int32_t* row_block_expert;
  int32_t* row_offsets;
  int32_t* col_indices;
};

// Fills every worst-case slot the scatter does not write. `warp_index` of `warp_count` warps share
// the row blocks. offsets[E+1] and counts[E] may be in shared or global memory. With null BSR
// pointers (a caller that only wants the sort) just the -1 rows are written.
__device__ void fill_layout(const int32_t* offsets, const int32_t* counts, int32_t num_experts, int32_t block_size,
                            int32_t ffn_blocks, int32_t max_row_blocks, const LayoutOut& out, int warp_index,
                            int warp_count, int lane) {
  const int32_t num_row_blocks = offsets[num_experts] / block_size;
  const bool want_bsr = out.col_indices != nullptr;
  if (block_size == 1 && !want_bsr) {
    // No padding inside an expert's group: only the rows past the real end are -1.
    for (int32_t r = num_row_blocks + warp_index * 32 + lane; r < max_row_blocks; r += warp_count * 32)
      out.row_token[r] = -1;
    return;
  }
  for (int32_t rb = warp_index; rb < max_row_blocks; rb += warp_count) {
    int32_t expert = -1;
    int32_t real_rows = 0;
    if (rb < num_row_blocks) {
      // Last expert whose range starts at or before this row block: skips empty experts, which
      // share a start with their successor (reference: csrc/routing.cu:181-189).
      const int32_t row0 = rb * block_size;
      int32_t lo = 0, hi = num_experts - 1;
      while (lo < hi) {
        const int32_t mid = (lo + hi + 1) >> 1;
        if (offsets[mid] <= row0) lo = mid; else hi = mid - 1;
      }
      expert = lo;
      real_rows = counts[expert] - (row0 - offsets[expert]);
      real_rows = max(0, min(block_size, real_rows));
    }
    const int64_t row_base = static_cast<int64_t>(rb) * block_size;
    for (int32_t j = real_rows + lane; j < block_size; j += 32) out.row_token[row_base + j] = -1;
    if (!want_bsr) continue;
    const int64_t col_base = static_cast<int64_t>(rb) * ffn_blocks;
    for (int32_t j = lane; j < ffn_blocks; j += 32)
      out.col_indices[col_base + j] = expert < 0 ? -1 : expert * ffn_blocks + j;
    if (lane == 0) {
      out.row_block_expert[rb] = expert;
      out.row_offsets[rb] = min(rb, num_row_blocks) * ffn_blocks;
    }
  }
  if (want_bsr && warp_index == 0 && lane == 0)
    out.row_offsets[max_row_blocks] = min(max_row_blocks, num_row_blocks) * ffn_blocks;
}

// ---------------------------------------------------------------------------------------------
// Cluster shape: ONE launch of a thread-block cluster of up to 8 blocks x 1024 threads does count,
// scan, scatter and the layout arrays. Block b of the cluster owns the b-th contiguous slice of the
// copies; the blocks exchange their per-expert counts through distributed shared memory (each block
// reads the others' cta_counts[] directly), so the only global traffic is the input and the outputs,
// and the scattered row_token stores are spread over as many SMs as the cluster has blocks.
// Shared memory per block: counters[32][E+1] | cta_counts[E] | offsets[E+1] | counts[E] | cta_base[E]
//                          | warp_sums[32] | bad[1].   (E+1: conflict-free column walks.)
template <typename Source, int kIters>
__global__ void __launch_bounds__(kClusterThreads, 1)
route_cluster_kernel(const Source source, int32_t n, int32_t k, int32_t num_experts, int32_t id_bits,
                     int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks,
                     int32_t* __restrict__ tokens_per_expert, int32_t* __restrict__ padded_offsets,
                     int32_t* __restrict__ copy_row, LayoutOut layout, int32_t* __restrict__ error) {
  cg::cluster_group cluster = cg::this_cluster();
  const int cta = static_cast<int>(cluster.block_rank());
  const int num_ctas = static_cast<int>(cluster.num_blocks());
  extern __shared__ int32_t smem[];
  constexpr int kWarps = kClusterThreads / 32;
  const int stride = num_experts + 1;
  int32_t* counters = smem;                         // [kWarps][stride]
  int32_t* cta_counts = counters + kWarps * stride; // [E]   read by the other blocks of the cluster
  int32_t* offsets = cta_counts + num_experts;      // [E + 1]
  int32_t* counts = offsets + num_experts + 1;      // [E]   totals over the cluster
  int32_t* cta_base = counts + num_experts;         // [E]   copies of e in earlier blocks
  int32_t* warp_sums = cta_base + num_experts;      // [32]
  int32_t* cta_bad = warp_sums + 32;                // [1]   read by block 0

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  // Runs of equal length over all warps of the cluster, a multiple of 32, in copy order.
  const int64_t run = static_cast<int64_t>((n + num_ctas * kClusterThreads - 1) / (num_ctas * kClusterThreads)) * 32;
  const int64_t begin = min(static_cast<int64_t>(n), (static_cast<int64_t>(cta) * kWarps + warp) * run);
  const int64_t end = min(static_cast<int64_t>(n), begin + run);
  int32_t ids[kIters];
  const bool bad = source.template load<kIters>(begin, end, lane, ids);
  for (int i = threadIdx.x; i < kWarps * stride; i += kClusterThreads) counters[i] = 0;
  __syncthreads();
  rank_run<kIters>(ids, begin, end, id_bits, counters + warp * stride, lane);
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (threadIdx.x == 0) *cta_bad = any_bad;

  // Per expert: exclusive scan of this block's 32 warp counters, in place. Warp w takes experts
  // w, w + 32, ...; lane l holds warp l's counter, so the scan is five shuffles.
  for (int e = warp; e < num_experts; e += kWarps) {
    int32_t* slot = counters + lane * stride + e;
    const int32_t mine = *slot;
    int32_t inclusive = mine;
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t below = __shfl_up_sync(kFullMask, inclusive, d);
      if (lane >= d) inclusive += below;
    }
    *slot = inclusive - mine;
    if (lane == 31) cta_counts[e] = inclusive;
  }
  cluster.sync();  // every block's cta_counts and cta_bad are published

  const int e = threadIdx.x;
  int32_t total = 0;
  if (e < num_experts) {
    int32_t before = 0;
    for (int b = 0; b < num_ctas; ++b) {
      const int32_t c = cluster.map_shared_rank(cta_counts, b)[e];
      if (b < cta) before += c;
      total += c;
    }
    cta_base[e] = before;
    counts[e] = total;
  }
  const int32_t padded = e < num_experts ? (total + block_size - 1) / block_size * block_size : 0;
  int32_t all_rows = 0;
  const int32_t start = block_exclusive_scan(padded, warp_sums, &all_rows);
  if (e < num_experts) offsets[e] = start;
  if (e == 0) offsets[num_experts] = all_rows;
  if (cta == 0) {
    if (e < num_experts) {
      tokens_per_expert[e] = total;
      padded_offsets[e] = start;
    }
    if (e == 0) {
      padded_offsets[num_experts] = all_rows;
      int any = 0;
      for (int b = 0; b < num_ctas; ++b) any |= *cluster.map_shared_rank(cta_bad, b);
      error[0] = any ? 1 : 0;
    }
  }
  __syncthreads();

  // This warp's base per expert = copies in earlier blocks + in earlier warps of this block.
  int32_t* bases = counters + warp * stride;
  for (int i = lane; i < num_experts; i += 32) bases[i] += cta_base[i];
  __syncwarp();
  scatter_run<kIters>(ids, begin, end, k, bases, offsets, copy_row, layout.row_token, lane);
  fill_layout(offsets, counts, num_experts, block_size, ffn_blocks, max_row_blocks, layout, cta * kWarps + warp,
              num_ctas * kWarps, lane);
  cluster.sync();  // no block may exit while another still reads its shared memory
}

// ---------------------------------------------------------------------------------------------
// Large shape, launch 1: per-chunk histograms. chunk_counts[chunk][e], chunk_error[chunk].
template <typename index_t>
__global__ void __launch_bounds__(kChunkThreads)
route_chunk_count_kernel(const index_t* __restrict__ expert_idx, int64_t n, int32_t num_experts, int32_t id_bits,
                         int32_t* __restrict__ chunk_counts, int32_t* __restrict__ chunk_error) {
  extern __shared__ int32_t smem[];  // counters[kChunkWarps][E]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kChunkWarps * num_experts; i += kChunkThreads) smem[i] = 0;
  __syncthreads();

  constexpr int64_t kRun = kChunkCopies / kChunkWarps;
  constexpr int kIters = static_cast<int>(kRun / 32);
  const int64_t begin = min(n, static_cast<int64_t>(blockIdx.x) * kChunkCopies + warp * kRun);
  const int64_t end = min(n, begin + kRun);
  int32_t ids[kIters];
  const bool bad = load_run<index_t, kIters>(expert_idx, begin, end, num_experts, lane, ids);
  rank_run<kIters>(ids, begin, end, id_bits, smem + warp * num_experts, lane);
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (threadIdx.x == 0) chunk_error[blockIdx.x] = any_bad;

  int32_t* out = chunk_counts + static_cast<int64_t>(blockIdx.x) * num_experts;
  for (int e = threadIdx.x; e < num_experts; e += kChunkThreads) {
    int32_t total = 0;
#pragma unroll
    for (int w = 0; w < kChunkWarps; ++w) total += smem[w * num_experts + e];
    out[e] = total;
  }
}

// Large shape, launch 2: one block, one thread per expert. chunk_counts becomes, in place, the
// number of copies of each expert in all earlier chunks.
__global__ void __launch_bounds__(kMaxExperts, 1)
route_scan_kernel(int32_t* __restrict__ chunk_counts, const int32_t* __restrict__ chunk_error, int32_t num_chunks,
                  int32_t num_experts, int32_t block_size, int32_t* __restrict__ tokens_per_expert,
                  int32_t* __restrict__ padded_offsets, int32_t* __restrict__ error) {
  __shared__ int32_t warp_sums[32];
  const int e = threadIdx.x;
  int32_t total = 0;
  if (e < num_experts) {
    for (int32_t b = 0; b < num_chunks; ++b) {
      int32_t* slot = chunk_counts + static_cast<int64_t>(b) * num_experts + e;
      const int32_t c = *slot;
      *slot = total;
      total += c;
    }
    tokens_per_expert[e] = total;
  }
  int bad = 0;
  for (int32_t b = threadIdx.x; b < num_chunks; b += blockDim.x) bad |= chunk_error[b];
  const int any_bad = __syncthreads_or(bad);
  if (threadIdx.x == 0) error[0] = any_bad ? 1 : 0;

  const int32_t padded = e < num_experts ? (total + block_size - 1) / block_size * block_size : 0;
  int32_t all_rows = 0;
  const int32_t start = block_exclusive_scan(padded, warp_sums, &all_rows);
  if (e < num_experts) padded_offsets[e] = start;
  if (e == 0) padded_offsets[num_experts] = all_rows;
}

// Large shape, launch 3: blocks [0, num_chunks) place their chunk; the remaining blocks fill the
// layout arrays and the -1 rows.
template <typename index_t>
__global__ void __launch_bounds__(kChunkThreads)
route_scatter_layout_kernel(const index_t* __restrict__ expert_idx, int64_t n, int32_t k, int32_t num_experts,
                            int32_t id_bits,
                            int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int32_t num_chunks,
                            const int32_t* __restrict__ chunk_base, const int32_t* __restrict__ tokens_per_expert,
                            const int32_t* __restrict__ padded_offsets, int32_t* __restrict__ copy_row,
                            LayoutOut layout) {
  extern __shared__ int32_t smem[];  // counters[kChunkWarps][E]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  if (static_cast<int32_t>(blockIdx.x) >= num_chunks) {
    const int part = static_cast<int>(blockIdx.x) - num_chunks;
    const int parts = static_cast<int>(gridDim.x) - num_chunks;
    fill_layout(padded_offsets, tokens_per_expert, num_experts, block_size, ffn_blocks, max_row_blocks, layout,
                part * kChunkWarps + warp, parts * kChunkWarps, lane);
    return;
  }

  constexpr int64_t kRun = kChunkCopies / kChunkWarps;
  constexpr int kIters = static_cast<int>(kRun / 32);
  const int64_t begin = min(n, static_cast<int64_t>(blockIdx.x) * kChunkCopies + warp * kRun);
  const int64_t end = min(n, begin + kRun);
  int32_t ids[kIters];
  load_run<index_t, kIters>(expert_idx, begin, end, num_experts, lane, ids);
  for (int i = threadIdx.x; i < kChunkWarps * num_experts; i += kChunkThreads) smem[i] = 0;
  __syncthreads();
  rank_run<kIters>(ids, begin, end, id_bits, smem + warp * num_experts, lane);
  __syncthreads();
  const int32_t* base = chunk_base + static_cast<int64_t>(blockIdx.x) * num_experts;
  for (int e = threadIdx.x; e < num_experts; e += kChunkThreads) {
    int32_t running = base[e];
#pragma unroll
    for (int w = 0; w < kChunkWarps; ++w) {
      int32_t* slot = smem + w * num_experts + e;
      const int32_t c = *slot;
      *slot = running;
      running += c;
    }
  }
  __syncthreads();
  scatter_run<kIters>(ids, begin, end, k, smem + warp * num_experts, padded_offsets, copy_row, layout.row_token,
                      lane);
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel owner: the layout over this rank's receive slots straight from the exchanged
// counts, without ever looking at the slots. Slot j = s * capacity + i holds the i-th copy that
// source rank s sent here; a source sends its copies sorted by expert, so the copies of local expert
// e from source s occupy slots s * capacity + [start_s(e), start_s(e) + counts[s][e]) with start_s the
// exclusive scan of counts[s][.] (what does not fit in `capacity` is cut off, as the sender cut it).
// Sorting the slots by expert with a stable sort (what sb_route does when it is handed one expert id
// per slot, -1 for the empty ones) puts expert e's rows in (source, i) order; this kernel writes
// exactly those arrays, bit for bit, from N * E_local counts instead of N * capacity ids, in one
// launch. Every block recomputes the small tables in shared memory and takes a share of the rows.
// Needs N * E_local <= 1024 (one thread per (source, expert) pair).
//
// row_block_order (optional): the owner's schedule for a dispatch that is still in flight (ep_dispatch.cuh).
// First the row blocks sorted by when their rows are complete if every source fills its slots from the front
// at the same pace, i.e. by the largest slot index i among the block's rows (ties in layout order, blocks
// without rows last); then, per row block, the arrival flags its rows wait for. Block 0 computes the keys
// into shared memory and ranks them by counting (at most 4096 row blocks: a few hundred in practice).
constexpr int kOwnerThreads = 1024;
constexpr int kMaxOrderedRowBlocks = 4096;

__global__ void __launch_bounds__(kOwnerThreads, 1)
ep_owner_layout_kernel(const int32_t* __restrict__ recv_counts, int32_t num_ranks, int32_t experts_local,
                       int32_t capacity, int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks,
                       int32_t* __restrict__ tokens_per_expert, int32_t* __restrict__ padded_offsets,
                       int32_t* __restrict__ copy_row, LayoutOut layout, int32_t* __restrict__ row_block_order,
                       int32_t* __restrict__ error) {
  __shared__ int32_t arrival_key[kMaxOrderedRowBlocks];
  __shared__ int32_t kept[kMaxExperts];        // [s][e] copies of e from s that fit the capacity
  __shared__ int32_t slot_start[kMaxExperts];  // [s][e] first slot index i of that run
  __shared__ int32_t row_start[kMaxExperts];   // [s][e] first row of that run in the layout
  __shared__ int32_t source_total[kMaxExperts];  // [s] slots of source s in use
  __shared__ int32_t counts[kMaxExperts];      // [e]
  __shared__ int32_t offsets[kMaxExperts + 1]; // [e] padded start row
  __shared__ int32_t warp_sums[32];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int pairs = num_ranks * experts_local;
  if (tid < num_ranks) {  // one thread per source: scan its counts over the experts, cut at the capacity
    int32_t running = 0;
    for (int32_t e = 0; e < experts_local; ++e) {
      const int32_t c = max(0, recv_counts[tid * experts_local + e]);
      const int32_t begin = min(capacity, running);
      const int32_t end = min(capacity, running + c);
      running = min(capacity, running + c);
      kept[tid * experts_local + e] = end - begin;
      slot_start[tid * experts_local + e] = begin;
    }
    source_total[tid] = running;
  }
  __syncthreads();
  int32_t total = 0;
  if (tid < experts_local) {  // one thread per expert: the sources' runs follow one another
    for (int32_t src = 0; src < num_ranks; ++src) {
      row_start[src * experts_local + tid] = total;  // relative to the expert's first row for now
      total += kept[src * experts_local + tid];
    }
    counts[tid] = total;
  }
  const int32_t padded = tid < experts_local ? (total + block_size - 1) / block_size * block_size : 0;
  int32_t all_rows = 0;
  const int32_t start = block_exclusive_scan(padded, warp_sums, &all_rows);
  if (tid < experts_local) offsets[tid] = start;
  if (tid == 0) offsets[experts_local] = all_rows;
  __syncthreads();
  if (tid < pairs) row_start[tid] += offsets[tid % experts_local];
  if (blockIdx.x == 0) {
    if (tid < experts_local) {
      tokens_per_expert[tid] = counts[tid];
      padded_offsets[tid] = offsets[tid];
    }
    if (tid == 0) {
      padded_offsets[experts_local] = all_rows;
      error[0] = 0;
    }
  }
  __syncthreads();

  const int warps_per_block = kOwnerThreads / 32;
  const int warp_index = static_cast<int>(blockIdx.x) * warps_per_block + (tid >> 5);
  const int warp_count = static_cast<int>(gridDim.x) * warps_per_block;
  // Real rows: one warp per (source, expert) run.
  for (int pair = warp_index; pair < pairs; pair += warp_count) {
    const int32_t src = pair / experts_local;
    const int32_t first_slot = src * capacity + slot_start[pair];
    const int32_t first_row = row_start[pair];
    for (int32_t j = lane; j < kept[pair]; j += 32) {
      layout.row_token[first_row + j] = first_slot + j;
      copy_row[first_slot + j] = first_row + j;
    }
  }
  // Empty slots.
  const int64_t slots = static_cast<int64_t>(num_ranks) * capacity;
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * kOwnerThreads + tid; j < slots;
       j += static_cast<int64_t>(gridDim.x) * kOwnerThreads) {
    const int32_t src = static_cast<int32_t>(j / capacity);
    if (static_cast<int32_t>(j - static_cast<int64_t>(src) * capacity) >= source_total[src]) copy_row[j] = -1;
  }
  // Padding rows, rows past the end and the block-sparse arrays.
  fill_layout(offsets, counts, experts_local, block_size, ffn_blocks, max_row_blocks, layout, warp_index, warp_count,
              lane);
  if (row_block_order == nullptr || blockIdx.x != 0) return;
  const int32_t segments = dispatch_segments(capacity);
  for (int32_t rb = tid; rb < max_row_blocks; rb += kOwnerThreads) {
    const int32_t first = rb * block_size;
    int32_t key = INT32_MAX;
    int32_t* wait_list = row_block_order + max_row_blocks + static_cast<int64_t>(rb) * kWaitStride;
    int32_t waits = 0;
    if (first < offsets[experts_local]) {
      int32_t lo = 0, hi = experts_local;  // the expert e with offsets[e] <= first < offsets[e + 1]
      while (hi - lo > 1) {
        const int32_t mid = (lo + hi) >> 1;
        if (offsets[mid] <= first) lo = mid; else hi = mid;
      }
      const int32_t e = lo;
      const int32_t end = min(first + block_size, offsets[e] + counts[e]);
      key = -1;
      for (int32_t src = 0; src < num_ranks; ++src) {
        const int32_t run = row_start[src * experts_local + e];
        const int32_t from = max(first, run);
        const int32_t to = min(end, run + kept[src * experts_local + e]);
        if (from >= to) continue;
        const int32_t first_slot = slot_start[src * experts_local + e] + (from - run);
        const int32_t last_slot = slot_start[src * experts_local + e] + (to - 1 - run);
        key = max(key, last_slot);
        // The flags this block's rows from `src` wait for (consecutive segments of its block of slots).
        for (int32_t g = first_slot / kSegmentRows; g <= last_slot / kSegmentRows && waits < kWaitStride - 1; ++g)
          wait_list[++waits] = src * segments + g;
      }
    }
    wait_list[0] = waits;
    arrival_key[rb] = key;
  }
  __syncthreads();
  for (int32_t rb = tid; rb < max_row_blocks; rb += kOwnerThreads) {
    const int32_t key = arrival_key[rb];
    int32_t rank = 0;
    for (int32_t other = 0; other < max_row_blocks; ++other) {
      const int32_t k2 = arrival_key[other];
      rank += (k2 < key || (k2 == key && other < rb)) ? 1 : 0;
    }
    row_block_order[rank] = rb;
  }
}

size_t cluster_smem_bytes(int32_t num_experts) {
  const size_t e = static_cast<size_t>(num_experts);
  return ((kClusterThreads / 32) * (e + 1) + e + (e + 1) + e + e + 32 + 1) * sizeof(int32_t);
}

int64_t num_chunks_for(int64_t n) { return (n + kChunkCopies - 1) / kChunkCopies; }

// Bits needed to tell expert ids 0 .. num_experts-1 apart.
int32_t id_bits_for(int32_t num_experts) {
  int32_t bits = 0;
  while ((1 << bits) < num_experts) ++bits;
  return bits;
}

template <typename Source, int kIters>
int launch_cluster(int device, int blocks, size_t smem, cudaStream_t stream, const Source& source, int32_t n,
                   int32_t k, int32_t num_experts, int32_t id_bits, int32_t ffn_blocks, int32_t block_size,
                   int32_t max_row_blocks, int32_t* tokens_per_expert, int32_t* padded_offsets, int32_t* copy_row,
                   LayoutOut layout, int32_t* error) {
  static std::atomic<bool> attr_done[kMaxDevices] = {};  // a lost race only repeats the same attribute call
  auto kernel = route_cluster_kernel<Source, kIters>;
  if (!attr_done[device].load(std::memory_order_acquire)) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(cluster_smem_bytes(kMaxExperts)));
    if (err != cudaSuccess) return fail(SB_ERR_CUDA, "routing: shared memory opt-in: %s", cudaGetErrorString(err));
    attr_done[device].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(blocks));
  config.blockDim = dim3(kClusterThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(blocks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, source, n, k, num_experts, id_bits, ffn_blocks,
                                             block_size, max_row_blocks, tokens_per_expert, padded_offsets, copy_row,
                                             layout, error);
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "routing (cluster): %s", cudaGetErrorString(err));
  return check_launch("routing (cluster)");
}

template <typename index_t>
int launch_route(const index_t* expert_idx, int64_t n, int32_t k, int32_t num_experts, int32_t ffn_blocks,
                 int32_t block_size, int32_t max_row_blocks, int32_t* tokens_per_expert, int32_t* padded_offsets,
                 int32_t* copy_row, const LayoutOut& layout, int32_t* error, void* workspace, cudaStream_t stream) {
  int device = 0;
  const DeviceInfo* info = current_device_info(&device);
  if (info == nullptr) return SB_ERR_CUDA;
  const int32_t id_bits = id_bits_for(num_experts);

  if (n <= kClusterMaxCopies) {
    // One block per 1024 copies up to the cluster limit, then longer runs per warp.
    int blocks = static_cast<int>((n + kClusterThreads - 1) / kClusterThreads);
    if (blocks > kMaxClusterBlocks) blocks = kMaxClusterBlocks;
    const int64_t steps = (n + static_cast<int64_t>(blocks) * kClusterThreads - 1) / (static_cast<int64_t>(blocks) * kClusterThreads);
    const size_t smem = cluster_smem_bytes(num_experts);
    const int32_t n32 = static_cast<int32_t>(n);
    const IndexSource<index_t> source{expert_idx, num_experts};
#define SB_ROUTE_CLUSTER(ITERS)                                                                                     \
  return launch_cluster<IndexSource<index_t>, ITERS>(device, blocks, smem, stream, source, n32, k, num_experts,      \
                                                     id_bits, ffn_blocks, block_size, max_row_blocks,                \
                                                     tokens_per_expert, padded_offsets, copy_row, layout, error)
    if (steps <= 1) SB_ROUTE_CLUSTER(1);
    if (steps <= 4) SB_ROUTE_CLUSTER(4);
    SB_ROUTE_CLUSTER(kMaxRunSteps);
#undef SB_ROUTE_CLUSTER
  }

  const int64_t num_chunks = num_chunks_for(n);
  int32_t* chunk_counts = static_cast<int32_t*>(workspace);
  int32_t* chunk_error = chunk_counts + num_chunks * num_experts;
  const size_t smem = static_cast<size_t>(kChunkWarps) * num_experts * sizeof(int32_t);  // <= 32 KB

  route_chunk_count_kernel<index_t><<<static_cast<unsigned>(num_chunks), kChunkThreads, smem, stream>>>(
      expert_idx, n, num_experts, id_bits, chunk_counts, chunk_error);
  if (int rc = check_launch("routing (chunk count)")) return rc;

  route_scan_kernel<<<1, kMaxExperts, 0, stream>>>(chunk_counts, chunk_error, static_cast<int32_t>(num_chunks),
                                                   num_experts, block_size, tokens_per_expert, padded_offsets,
                                                   error);
  if (int rc = check_launch("routing (scan)")) return rc;

  // Enough layout blocks to cover the row blocks a few per warp, at most a few waves.
  int64_t layout_blocks = (static_cast<int64_t>(max_row_blocks) + kChunkWarps * 4 - 1) / (kChunkWarps * 4);
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 8;
  if (layout_blocks > cap) layout_blocks = cap;
  if (layout_blocks < 1) layout_blocks = 1;
  route_scatter_layout_kernel<index_t>
      <<<static_cast<unsigned>(num_chunks + layout_blocks), kChunkThreads, smem, stream>>>(
          expert_idx, n, k, num_experts, id_bits, ffn_blocks, block_size, max_row_blocks,
          static_cast<int32_t>(num_chunks), chunk_counts, tokens_per_expert, padded_offsets, copy_row, layout);
  return check_launch("routing (scatter + layout)");
}

// Router + routing in one cluster launch. Only where a 32-copy step holds whole tokens (k a power of two) and
// the runs stay short (T*k <= 32768); any number of experts the routing kernel takes.
constexpr int64_t kFusedRouterMaxCopies = static_cast<int64_t>(kMaxClusterBlocks) * kClusterThreads * 4;

bool fused_router_fits(int64_t n_copies, int32_t k, int32_t num_experts) {
  return n_copies <= kFusedRouterMaxCopies && num_experts <= kMaxExperts && k >= 1 && k <= kRouterMaxK &&
         (k & (k - 1)) == 0;
}

template <typename logit_t>
int launch_route_logits(const logit_t* logits, int64_t num_tokens, int32_t k, int32_t num_experts, int32_t ffn_blocks,
                        int32_t block_size, int32_t max_row_blocks, int64_t* expert_idx, logit_t* expert_weight,
                        int32_t* tokens_per_expert, int32_t* padded_offsets, int32_t* copy_row, const LayoutOut& layout,
                        int32_t* error, cudaStream_t stream) {
  int device = 0;
  if (current_device_info(&device) == nullptr) return SB_ERR_CUDA;
  const int64_t n = num_tokens * k;
  int blocks = static_cast<int>((n + kClusterThreads - 1) / kClusterThreads);
  if (blocks > kMaxClusterBlocks) blocks = kMaxClusterBlocks;
  const int64_t steps = (n + static_cast<int64_t>(blocks) * kClusterThreads - 1) / (static_cast<int64_t>(blocks) * kClusterThreads);
  const LogitSource<logit_t> source{logits, expert_idx, expert_weight, num_experts, k};
  const size_t smem = cluster_smem_bytes(num_experts);
  const int32_t id_bits = id_bits_for(num_experts);
  if (steps <= 1)
    return launch_cluster<LogitSource<logit_t>, 1>(device, blocks, smem, stream, source, static_cast<int32_t>(n), k,
                                                   num_experts, id_bits, ffn_blocks, block_size, max_row_blocks,
                                                   tokens_per_expert, padded_offsets, copy_row, layout, error);
  return launch_cluster<LogitSource<logit_t>, 4>(device, blocks, smem, stream, source, static_cast<int32_t>(n), k,
                                                 num_experts, id_bits, ffn_blocks, block_size, max_row_blocks,
                                                 tokens_per_expert, padded_offsets, copy_row, layout, error);
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch for sb_route_static_scratch: the chunk histograms of the three-launch shape live
// in this array instead of a caller-provided workspace. Every GPU that loads the library carries
// these SB_ROUTE_STATIC_SCRATCH_BYTES until the process exits. In host code the array's name is only
// a stand-in for the symbol; the device address is asked for once per device below.
constexpr size_t kStaticScratchBytes = SB_ROUTE_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) int32_t g_route_static_scratch[kStaticScratchBytes / sizeof(int32_t)];

// Device address of the array on the calling thread's current device. The first call on a device
// asks the runtime for it (cudaGetSymbolAddress, with that device current); later calls read a table.
int static_scratch_address(void** out) {
  static std::atomic<void*> address[kMaxDevices] = {};  // two threads racing here ask twice and store the same value
  int device = 0;
  if (current_device_info(&device) == nullptr) return SB_ERR_CUDA;
  void* ptr = address[device].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_route_static_scratch);
    if (err != cudaSuccess || ptr == nullptr)
      return fail(SB_ERR_CUDA, "routing (static scratch): cudaGetSymbolAddress: %s", cudaGetErrorString(err));
    address[device].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return SB_OK;
}

}  // namespace
}  // namespace sb

extern "C" {

int sb_route_sizes(int64_t n_copies, int32_t num_experts, int64_t ffn_dim, int64_t block_size,
                   int64_t* max_row_blocks, int64_t* max_rows, int64_t* ffn_blocks) {
  sb::clear_error();
  constexpr int64_t kI32Max = INT32_MAX;
  if (n_copies <= 0) return sb::fail(SB_ERR_INVALID_ARGUMENT, "expert_idx must be [T, k] with T, k > 0");
  if (num_experts <= 0 || num_experts > sb::kMaxExperts)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "num_experts must be in [1, %d], got %d", sb::kMaxExperts, num_experts);
  if (block_size <= 0 || block_size > kI32Max)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "block_size must be in [1, 2^31)");
  if (ffn_dim <= 0 || ffn_dim % block_size != 0)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "ffn_dim (%lld) must be a positive multiple of block_size (%lld)",
                    (long long)ffn_dim, (long long)block_size);
  // Worst case: every expert wastes block_size - 1 rows of padding (reference: csrc/routing.cu:213-216).
  const int64_t rb = (n_copies + static_cast<int64_t>(num_experts) * (block_size - 1)) / block_size;
  const int64_t rows = rb * block_size;
  const int64_t fb = ffn_dim / block_size;
  if (n_copies > kI32Max || rows > kI32Max / ffn_dim || rb * fb >= kI32Max)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "problem too large for int32 indexing");
  if (max_row_blocks != nullptr) *max_row_blocks = rb;
  if (max_rows != nullptr) *max_rows = rows;
  if (ffn_blocks != nullptr) *ffn_blocks = fb;
  return SB_OK;
}

size_t sb_route_workspace_bytes(int64_t n_copies, int32_t num_experts) {
  if (n_copies <= sb::kClusterMaxCopies || num_experts <= 0) return 0;
  const int64_t chunks = sb::num_chunks_for(n_copies);
  return static_cast<size_t>(chunks) * (static_cast<size_t>(num_experts) + 1) * sizeof(int32_t);
}

int sb_route(const void* expert_idx, int idx_is_i64, int64_t n_copies, int32_t k, int32_t num_experts,
             int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int32_t* tokens_per_expert,
             int32_t* padded_offsets, int32_t* row_token, int32_t* copy_row, int32_t* row_block_expert,
             int32_t* row_offsets, int32_t* col_indices, int32_t* error, void* workspace, sb_stream_t stream) {
  sb::clear_error();
  if (k <= 0 || ffn_blocks <= 0) return sb::fail(SB_ERR_INVALID_ARGUMENT, "routing: k and ffn_blocks must be positive");
  int64_t want_rb = 0;
  if (int rc = sb_route_sizes(n_copies, num_experts, static_cast<int64_t>(ffn_blocks) * block_size, block_size,
                              &want_rb, nullptr, nullptr))
    return rc;
  if (want_rb != max_row_blocks)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "routing: max_row_blocks is %d, worst case needs %lld", max_row_blocks,
                    (long long)want_rb);
  if (!expert_idx || !tokens_per_expert || !padded_offsets || !row_token || !copy_row || !error)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "routing: NULL buffer");
  const int bsr_given = (row_block_expert != nullptr) + (row_offsets != nullptr) + (col_indices != nullptr);
  if (bsr_given != 0 && bsr_given != 3)
    return sb::fail(SB_ERR_INVALID_ARGUMENT,
                    "routing: row_block_expert, row_offsets and col_indices must be all given or all NULL");
  if (workspace == nullptr && sb_route_workspace_bytes(n_copies, num_experts) != 0)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "routing: workspace is NULL but %zu bytes are needed",
                    sb_route_workspace_bytes(n_copies, num_experts));

  const sb::LayoutOut layout{row_token, row_block_expert, row_offsets, col_indices};
  const cudaStream_t s = sb::as_stream(stream);
  if (idx_is_i64)
    return sb::launch_route(static_cast<const int64_t*>(expert_idx), n_copies, k, num_experts, ffn_blocks, block_size,
                            max_row_blocks, tokens_per_expert, padded_offsets, copy_row, layout, error, workspace, s);
  return sb::launch_route(static_cast<const int32_t*>(expert_idx), n_copies, k, num_experts, ffn_blocks, block_size,
                          max_row_blocks, tokens_per_expert, padded_offsets, copy_row, layout, error, workspace, s);
}

int sb_route_from_logits_fused(int64_t num_tokens, int32_t k, int32_t num_experts) {
  return sb::fused_router_fits(num_tokens * k, k, num_experts) ? 1 : 0;
}

int sb_route_from_logits(const void* logits, int logits_dtype, int64_t num_tokens, int32_t k, int32_t num_experts,
                         int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int64_t* expert_idx,
                         void* expert_weight, int32_t* tokens_per_expert, int32_t* padded_offsets, int32_t* row_token,
                         int32_t* copy_row, int32_t* row_block_expert, int32_t* row_offsets, int32_t* col_indices,
                         int32_t* error, sb_stream_t stream) {
  sb::clear_error();
  if (!logits || !expert_idx || !expert_weight)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "route_from_logits: NULL buffer");
  if (logits_dtype != 0 && logits_dtype != 1)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "route_from_logits: logits_dtype must be 0 (bf16) or 1 (fp32)");
  if (num_tokens <= 0 || k <= 0 || k > num_experts)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "route_from_logits: need [T, E] logits with 0 < k <= E");
  if (!sb::fused_router_fits(num_tokens * k, k, num_experts))
    return sb::fail(SB_ERR_UNSUPPORTED,
                    "route_from_logits: the one-launch form needs k in {1, 2, 4, 8}, E <= %d and T*k <= %lld; "
                    "use sb_router_topk followed by sb_route",
                    sb::kMaxExperts, (long long)sb::kFusedRouterMaxCopies);
  int64_t want_rb = 0;
  if (int rc = sb_route_sizes(num_tokens * k, num_experts, static_cast<int64_t>(ffn_blocks) * block_size, block_size,
                              &want_rb, nullptr, nullptr))
    return rc;
  if (ffn_blocks <= 0 || want_rb != max_row_blocks)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "route_from_logits: max_row_blocks is %d, worst case needs %lld",
                    max_row_blocks, (long long)want_rb);
  if (!tokens_per_expert || !padded_offsets || !row_token || !copy_row || !row_block_expert || !row_offsets ||
      !col_indices || !error)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "route_from_logits: NULL buffer");
  const sb::LayoutOut layout{row_token, row_block_expert, row_offsets, col_indices};
  const cudaStream_t s = sb::as_stream(stream);
  if (logits_dtype == 0)
    return sb::launch_route_logits(static_cast<const __nv_bfloat16*>(logits), num_tokens, k, num_experts, ffn_blocks,
                                   block_size, max_row_blocks, expert_idx, static_cast<__nv_bfloat16*>(expert_weight),
                                   tokens_per_expert, padded_offsets, copy_row, layout, error, s);
  return sb::launch_route_logits(static_cast<const float*>(logits), num_tokens, k, num_experts, ffn_blocks, block_size,
                                 max_row_blocks, expert_idx, static_cast<float*>(expert_weight), tokens_per_expert,
                                 padded_offsets, copy_row, layout, error, s);
}

int sb_ep_owner_layout(const int32_t* recv_counts, int32_t num_ranks, int32_t experts_local, int32_t capacity,
                       int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int32_t* tokens_per_expert,
                       int32_t* padded_offsets, int32_t* row_token, int32_t* copy_row, int32_t* row_block_expert,
                       int32_t* row_offsets, int32_t* col_indices, int32_t* row_block_order, int32_t* error,
                       sb_stream_t stream) {
  sb::clear_error();
  if (row_block_order != nullptr && (max_row_blocks > sb::kMaxOrderedRowBlocks || num_ranks > sb::kMaxDispatchRanks ||
                                     block_size > sb::kSegmentRows))
    return sb::fail(SB_ERR_INVALID_ARGUMENT,
                    "ep_owner_layout: the schedule is built for at most %d row blocks of at most %d rows and %d ranks",
                    sb::kMaxOrderedRowBlocks, sb::kSegmentRows, sb::kMaxDispatchRanks);
  if (num_ranks <= 0 || experts_local <= 0 || static_cast<int64_t>(num_ranks) * experts_local > sb::kMaxExperts)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "ep_owner_layout: need 0 < ranks * local experts <= %d", sb::kMaxExperts);
  if (capacity <= 0 || ffn_blocks <= 0) return sb::fail(SB_ERR_INVALID_ARGUMENT, "ep_owner_layout: capacity and ffn_blocks must be positive");
  int64_t want_rb = 0;
  if (int rc = sb_route_sizes(static_cast<int64_t>(num_ranks) * capacity, experts_local,
                              static_cast<int64_t>(ffn_blocks) * block_size, block_size, &want_rb, nullptr, nullptr))
    return rc;
  if (want_rb != max_row_blocks)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "ep_owner_layout: max_row_blocks is %d, worst case needs %lld", max_row_blocks,
                    (long long)want_rb);
  if (!recv_counts || !tokens_per_expert || !padded_offsets || !row_token || !copy_row || !row_block_expert ||
      !row_offsets || !col_indices || !error)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "ep_owner_layout: NULL buffer");
  const sb::DeviceInfo* info = sb::current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  // Enough blocks that the fills (a few hundred KB) spread over the GPU; every block redoes the small tables.
  int64_t blocks = (static_cast<int64_t>(num_ranks) * capacity + 8 * sb::kOwnerThreads - 1) / (8 * sb::kOwnerThreads);
  if (blocks < 1) blocks = 1;
  if (blocks > info->sm_count) blocks = info->sm_count;
  const sb::LayoutOut layout{row_token, row_block_expert, row_offsets, col_indices};
  sb::ep_owner_layout_kernel<<<static_cast<unsigned>(blocks), sb::kOwnerThreads, 0, sb::as_stream(stream)>>>(
      recv_counts, num_ranks, experts_local, capacity, ffn_blocks, block_size, static_cast<int32_t>(max_row_blocks),
      tokens_per_expert, padded_offsets, copy_row, layout, row_block_order, error);
  return sb::check_launch("ep_owner_layout");
}

int sb_route_static_scratch(const void* expert_idx, int idx_is_i64, int64_t n_copies, int32_t k,
                            int32_t num_experts, int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks,
                            int32_t* tokens_per_expert, int32_t* padded_offsets, int32_t* row_token,
                            int32_t* copy_row, int32_t* row_block_expert, int32_t* row_offsets,
                            int32_t* col_indices, int32_t* error, sb_stream_t stream) {
  sb::clear_error();
  const size_t needed = sb_route_workspace_bytes(n_copies, num_experts);
  if (needed > sb::kStaticScratchBytes)
    return sb::fail(SB_ERR_INVALID_ARGUMENT,
                    "routing (static scratch): %lld copies over %d experts need %zu bytes of scratch, the built-in "
                    "array holds %zu; use sb_route with a workspace of your own",
                    (long long)n_copies, num_experts, needed, sb::kStaticScratchBytes);
  void* scratch = nullptr;
  if (int rc = sb::static_scratch_address(&scratch)) return rc;
  // Nothing in the array has to start at zero: every chunk writes all of its counters and its
  // error word before the scan reads them, so the previous call's contents are simply overwritten.
  return sb_route(expert_idx, idx_is_i64, n_copies, k, num_experts, ffn_blocks, block_size, max_row_blocks,
                  tokens_per_expert, padded_offsets, row_token, copy_row, row_block_expert, row_offsets,
                  col_indices, error, scratch, stream);
}

}  // extern "C"
