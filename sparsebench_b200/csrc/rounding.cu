// Token rounding on the device, with no host sync: top-k routing whose per-expert token counts are moved
// to the NEAREST multiple of the tile, so that the block-sparse layout needs (almost) no padding rows.
// Same result as the reference's host-synchronising PyTorch version (sparsebench/token_rounding.py:58-81,
// SonicMoE's Algorithm 4): expert e with f picks gets target(f) rows (nearest multiple of `tile`, ties
// down, at most the largest multiple that fits in T); if target < f its lowest-scoring picks are dropped,
// if target > f the highest-scoring tokens that did not pick it are added; among equal scores the
// earlier token ranks first. Every token's weights are its kept scores renormalised to sum to 1.
//
// The reference returns a flat assignment list whose length it learns with a host sync (nonzero). Here
// the list has its worst-case length T*k + E*(tile/2) and unused entries carry expert -1, which the routing
// kernel skips, so the list feeds moe_forward_assigned as it is and the host never learns a count.
//
//   rounding_topk_kernel     one warp per token: its k best experts (ties to the lower id), per-expert counts
//   rounding_select_kernel   one block per expert: target count, then the rank threshold among the
//                            candidates (its picks when shrinking, the other tokens when growing) by a
//                            4-pass radix select on the scores, ties resolved in token order; writes keep[t][e]
//   rounding_count_kernel    one warp per token: kept experts per token and the sum of their scores
//   rounding_scan_kernel     one block: exclusive scan of those counts = every token's place in the list
//   rounding_emit_kernel     one warp per token: (token, expert, weight) in token-major, expert-ascending order
//                            (the order of the reference's nonzero); the unused tail gets expert -1

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kTopkThreads = 256;
constexpr int kSelectThreads = 1024;
constexpr int kEmitThreads = 1024;
constexpr int kMaxK = 8;
constexpr int kMaxPerLane = 32;  // E <= 1024

// Order-preserving map of a float onto unsigned integers (larger float -> larger key).
__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__global__ void __launch_bounds__(kTopkThreads)
rounding_topk_kernel(const float* __restrict__ scores, int64_t num_tokens, int32_t num_experts, int32_t k,
                     int32_t* __restrict__ picks, int32_t* __restrict__ counts) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); t < num_tokens; t += warps) {
    const float* row = scores + t * num_experts;
    uint32_t retired = 0;
    for (int r = 0; r < k; ++r) {
      float best = -INFINITY;
      int32_t best_id = INT32_MAX;
      for (int q = 0; q * 32 + lane < num_experts; ++q) {
        const int32_t e = lane + 32 * q;
        const float v = __ldg(row + e);
        if (!((retired >> q) & 1u) && (v > best || (v == best && e < best_id) || best_id == INT32_MAX)) {
          best = v;
          best_id = e;
        }
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, d);
        const int32_t other_id = __shfl_xor_sync(0xffffffffu, best_id, d);
        if (other_id != INT32_MAX && (best_id == INT32_MAX || other > best || (other == best && other_id < best_id))) {
          best = other;
          best_id = other_id;
        }
      }
      if ((best_id & 31) == lane) retired |= 1u << (best_id >> 5);
      if (lane == 0) {
        picks[t * k + r] = best_id;
        atomicAdd(counts + best_id, 1);
      }
    }
  }
}

__device__ __forceinline__ bool is_pick(const int32_t* __restrict__ picks, int64_t t, int32_t k, int32_t e) {
  bool hit = false;
  for (int r = 0; r < k; ++r) hit |= __ldg(picks + t * k + r) == e;
  return hit;
}

__global__ void __launch_bounds__(kSelectThreads, 1)
rounding_select_kernel(const float* __restrict__ scores, const int32_t* __restrict__ picks,
                       const int32_t* __restrict__ counts, int64_t num_tokens, int32_t num_experts, int32_t k,
                       int32_t tile, int32_t cached, uint8_t* __restrict__ keep) {
  // With `cached` the expert's column (every token's key and whether it picked the expert) is read once into
  // shared memory; the four select passes and the two walks after them then stay on chip. The column is strided
  // by E in global memory, so every pass over it costs a sector per token otherwise.
  extern __shared__ uint32_t column_keys[];                                         // [T] when cached
  uint8_t* column_picks = reinterpret_cast<uint8_t*>(column_keys + (cached ? num_tokens : 0));  // [T]
  __shared__ int32_t histogram[256];
  __shared__ int32_t scratch[33];
  __shared__ uint32_t chosen_prefix;
  __shared__ int32_t chosen_remaining;
  const int32_t e = blockIdx.x;
  const int32_t f = counts[e];
  // Nearest multiple of the tile, ties down, never above the largest multiple that fits in T.
  const int32_t low = f / tile * tile;
  const int32_t high = low + (f % tile > 0 ? tile : 0);
  int32_t target = (high - f < f - low) ? high : low;
  const int32_t most = static_cast<int32_t>(num_tokens / tile) * tile;
  if (target > most) target = most;

  const bool shrinking = target < f;
  const int32_t wanted = shrinking ? target : target - f;  // how many CANDIDATES to keep
  // Candidates: this expert's picks when shrinking, the tokens that did not pick it when growing.
  if (target == f || (!shrinking && wanted == 0)) {
    for (int64_t t = threadIdx.x; t < num_tokens; t += kSelectThreads) keep[t * num_experts + e] = is_pick(picks, t, k, e);
    return;
  }
  if (cached) {
    for (int64_t t = threadIdx.x; t < num_tokens; t += kSelectThreads) {
      column_keys[t] = order_key(__ldg(scores + t * num_experts + e));
      column_picks[t] = is_pick(picks, t, k, e) ? 1 : 0;
    }
    __syncthreads();
  }
  auto pick_of = [&](int64_t t) { return cached ? column_picks[t] != 0 : is_pick(picks, t, k, e); };
  auto key_of = [&](int64_t t) { return cached ? column_keys[t] : order_key(__ldg(scores + t * num_experts + e)); };
  // Radix select: the `wanted`-th largest key among the candidates, one byte per pass from the top.
  uint32_t prefix = 0, prefix_mask = 0;
  int32_t remaining = wanted;  // rank still to be found inside the current prefix class
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kSelectThreads) histogram[i] = 0;
    __syncthreads();
    for (int64_t t = threadIdx.x; t < num_tokens; t += kSelectThreads) {
      if (pick_of(t) != shrinking) continue;
      const uint32_t key = key_of(t);
      if ((key & prefix_mask) == prefix) atomicAdd(&histogram[(key >> shift) & 0xffu], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int32_t need = remaining;
      int bin = 255;
      for (; bin > 0; --bin) {  // from the largest digit down
        if (histogram[bin] >= need) break;
        need -= histogram[bin];
      }
      chosen_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
      chosen_remaining = need;
    }
    __syncthreads();
    prefix = chosen_prefix;
    remaining = chosen_remaining;
    prefix_mask |= 0xffu << shift;
    __syncthreads();
  }
  // prefix is now the threshold key; `remaining` of the candidates that equal it are kept, earliest tokens first.
  // Tokens are walked in contiguous slices per thread so that "earlier" is a prefix sum over threads.
  const int64_t per_thread = (num_tokens + kSelectThreads - 1) / kSelectThreads;
  const int64_t t_begin = min(num_tokens, static_cast<int64_t>(threadIdx.x) * per_thread);
  const int64_t t_end = min(num_tokens, t_begin + per_thread);
  int32_t equal_here = 0;
  for (int64_t t = t_begin; t < t_end; ++t) {
    if (pick_of(t) != shrinking) continue;
    equal_here += key_of(t) == prefix ? 1 : 0;
  }
  // Exclusive scan of equal_here over the threads (two-level, through shared memory).
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t inclusive = equal_here;
  for (int d = 1; d < 32; d <<= 1) {
    const int32_t below = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d) inclusive += below;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    int32_t s = scratch[lane];
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t below = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += below;
    }
    scratch[lane] = s;
  }
  __syncthreads();
  int32_t equal_before = (warp > 0 ? scratch[warp - 1] : 0) + inclusive - equal_here;
  for (int64_t t = t_begin; t < t_end; ++t) {
    const bool pick = pick_of(t);
    bool kept;
    if (pick != shrinking) {
      kept = pick;  // not a candidate: picks stay when growing, non-picks stay out when shrinking
    } else {
      const uint32_t key = key_of(t);
      if (key > prefix) kept = true;
      else if (key < prefix) kept = false;
      else kept = equal_before++ < remaining;
    }
    keep[t * num_experts + e] = kept ? 1 : 0;
  }
}

// One warp per token: how many experts kept it and the sum of their scores (fp32, ascending expert order, the
// order in which the reference's index_add_ sums them on the CPU).
__global__ void __launch_bounds__(kTopkThreads)
rounding_count_kernel(const float* __restrict__ scores, const uint8_t* __restrict__ keep, int64_t num_tokens,
                      int32_t num_experts, int32_t* __restrict__ kept_per_token, float* __restrict__ kept_sum) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); t < num_tokens; t += warps) {
    int32_t count = 0;
    float sum = 0.0f;
    for (int32_t e0 = 0; e0 < num_experts; e0 += 32) {
      const int32_t e = e0 + lane;
      const bool kept = e < num_experts && keep[t * num_experts + e] != 0;
      const float v = kept ? __ldg(scores + t * num_experts + e) : 0.0f;
      const unsigned mask = __ballot_sync(0xffffffffu, kept);
      count += __popc(mask);
      // Add this step's kept scores in lane (= expert) order, one after the other, to keep the summation order.
      for (unsigned rest = mask; rest != 0; rest &= rest - 1) sum += __shfl_sync(0xffffffffu, v, __ffs(rest) - 1);
    }
    if (lane == 0) {
      kept_per_token[t] = count;
      kept_sum[t] = sum;
    }
  }
}

// One block: kept_per_token becomes its exclusive scan, *num_copies the total (cut at the capacity).
__global__ void __launch_bounds__(kEmitThreads, 1)
rounding_scan_kernel(int32_t* __restrict__ kept_per_token, int64_t num_tokens, int64_t capacity,
                     int32_t* __restrict__ num_copies) {
  __shared__ int32_t scratch[32];
  const int64_t per_thread = (num_tokens + kEmitThreads - 1) / kEmitThreads;
  const int64_t t_begin = min(num_tokens, static_cast<int64_t>(threadIdx.x) * per_thread);
  const int64_t t_end = min(num_tokens, t_begin + per_thread);
  int32_t mine = 0;
  for (int64_t t = t_begin; t < t_end; ++t) mine += kept_per_token[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t inclusive = mine;
  for (int d = 1; d < 32; d <<= 1) {
    const int32_t below = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d) inclusive += below;
  }
  if (lane == 31) scratch[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    int32_t v = scratch[lane];
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t below = __shfl_up_sync(0xffffffffu, v, d);
      if (lane >= d) v += below;
    }
    scratch[lane] = v;
  }
  __syncthreads();
  int32_t running = (warp > 0 ? scratch[warp - 1] : 0) + inclusive - mine;
  for (int64_t t = t_begin; t < t_end; ++t) {
    const int32_t n = kept_per_token[t];
    kept_per_token[t] = running;
    running += n;
  }
  if (threadIdx.x == 0) {
    const int64_t total = scratch[31];
    *num_copies = static_cast<int32_t>(total < capacity ? total : capacity);
  }
}

// One warp per token writes its entries (expert ascending) at its offset; the warps past the last token fill
// the unused tail of the worst-case sized list with expert -1.
__global__ void __launch_bounds__(kTopkThreads)
rounding_emit_kernel(const float* __restrict__ scores, const uint8_t* __restrict__ keep,
                     const int32_t* __restrict__ offsets, const float* __restrict__ kept_sum,
                     const int32_t* __restrict__ num_copies, int64_t num_tokens, int32_t num_experts, int64_t capacity,
                     int32_t* __restrict__ token_of_copy, int32_t* __restrict__ expert_of_copy,
                     float* __restrict__ weight_of_copy) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  for (int64_t t = warp_id; t < num_tokens; t += warps) {
    int64_t out = offsets[t];
    const float sum = kept_sum[t];
    for (int32_t e0 = 0; e0 < num_experts; e0 += 32) {
      const int32_t e = e0 + lane;
      const bool kept = e < num_experts && keep[t * num_experts + e] != 0;
      const unsigned mask = __ballot_sync(0xffffffffu, kept);
      const int64_t mine = out + __popc(mask & ((1u << lane) - 1u));
      if (kept && mine < capacity) {
        token_of_copy[mine] = static_cast<int32_t>(t);
        expert_of_copy[mine] = e;
        weight_of_copy[mine] = __ldg(scores + t * num_experts + e) / sum;
      }
      out += __popc(mask);
    }
  }
  const int64_t first_unused = *num_copies;
  for (int64_t i = first_unused + warp_id * 32 + lane; i < capacity; i += warps * 32) {
    token_of_copy[i] = 0;
    expert_of_copy[i] = -1;
    weight_of_copy[i] = 0.0f;
  }
}

}  // namespace
}  // namespace sb

extern "C" {

int64_t sb_token_rounding_capacity(int64_t num_tokens, int32_t num_experts, int32_t k, int32_t tile) {
  if (num_tokens <= 0 || num_experts <= 0 || k <= 0 || tile <= 0) return 0;
  return num_tokens * k + static_cast<int64_t>(num_experts) * (tile / 2);
}

size_t sb_token_rounding_workspace_bytes(int64_t num_tokens, int32_t num_experts, int32_t k) {
  if (num_tokens <= 0 || num_experts <= 0 || k <= 0) return 0;
  // picks [T*k] int32 | counts [E] int32 | kept_per_token [T] int32 | kept_sum [T] fp32 | keep [T*E] bytes
  const size_t words = static_cast<size_t>(num_tokens) * k + static_cast<size_t>(num_experts) + 2 * static_cast<size_t>(num_tokens);
  return words * sizeof(int32_t) + static_cast<size_t>(num_tokens) * num_experts;
}

int sb_token_rounding(const float* scores, int64_t num_tokens, int32_t num_experts, int32_t k, int32_t tile,
                      int32_t* token_of_copy, int32_t* expert_of_copy, float* weight_of_copy, int32_t* num_copies,
                      void* workspace, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!scores || !token_of_copy || !expert_of_copy || !weight_of_copy || !num_copies || !workspace)
    return fail(SB_ERR_INVALID_ARGUMENT, "token_rounding: NULL buffer");
  if (num_tokens <= 0 || num_tokens > INT32_MAX / 2 || num_experts <= 0 || num_experts > 32 * kMaxPerLane)
    return fail(SB_ERR_INVALID_ARGUMENT, "token_rounding: need [T, E] scores with T > 0 and 0 < E <= %d", 32 * kMaxPerLane);
  if (k <= 0 || k > kMaxK || k > num_experts || tile <= 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "token_rounding: need 0 < k <= min(E, %d) and tile > 0", kMaxK);
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  const cudaStream_t s = as_stream(stream);
  int32_t* picks = static_cast<int32_t*>(workspace);
  int32_t* counts = picks + num_tokens * k;
  int32_t* kept_per_token = counts + num_experts;
  float* kept_sum = reinterpret_cast<float*>(kept_per_token + num_tokens);
  uint8_t* keep = reinterpret_cast<uint8_t*>(kept_sum + num_tokens);
  cudaError_t err = cudaMemsetAsync(counts, 0, static_cast<size_t>(num_experts) * sizeof(int32_t), s);
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "token_rounding: memset: %s", cudaGetErrorString(err));
  int64_t blocks = (num_tokens + kTopkThreads / 32 - 1) / (kTopkThreads / 32);
  if (blocks > static_cast<int64_t>(info->sm_count) * 8) blocks = static_cast<int64_t>(info->sm_count) * 8;
  rounding_topk_kernel<<<static_cast<unsigned>(blocks), kTopkThreads, 0, s>>>(scores, num_tokens, num_experts, k, picks, counts);
  if (int rc = check_launch("token_rounding (top-k)")) return rc;
  // The expert's column in shared memory (5 bytes per token) where it fits beside the static arrays.
  const size_t column_bytes = static_cast<size_t>(num_tokens) * 5;
  const int32_t cached = column_bytes <= 46 * 1024 ? 1 : 0;
  rounding_select_kernel<<<static_cast<unsigned>(num_experts), kSelectThreads, cached ? column_bytes : 0, s>>>(
      scores, picks, counts, num_tokens, num_experts, k, tile, cached, keep);
  if (int rc = check_launch("token_rounding (select)")) return rc;
  const int64_t capacity = sb_token_rounding_capacity(num_tokens, num_experts, k, tile);
  rounding_count_kernel<<<static_cast<unsigned>(blocks), kTopkThreads, 0, s>>>(scores, keep, num_tokens, num_experts,
                                                                              kept_per_token, kept_sum);
  if (int rc = check_launch("token_rounding (count)")) return rc;
  rounding_scan_kernel<<<1, kEmitThreads, 0, s>>>(kept_per_token, num_tokens, capacity, num_copies);
  if (int rc = check_launch("token_rounding (scan)")) return rc;
  rounding_emit_kernel<<<static_cast<unsigned>(blocks), kTopkThreads, 0, s>>>(scores, keep, kept_per_token, kept_sum,
                                                                             num_copies, num_tokens, num_experts, capacity,
                                                                             token_of_copy, expert_of_copy, weight_of_copy);
  return check_launch("token_rounding (emit)");
}

}  // extern "C"
