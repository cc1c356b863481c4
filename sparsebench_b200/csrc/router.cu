// Router front end on the device: top-k experts per token and a softmax over the k picked logits
// only (Mixtral style), what the reference does with torch.topk + torch.softmax on the host side of
// its benchmarks and tests (sparsebench/reference.py:19-29). Feeds sb_route directly, so a layer can
// go from router logits to output without the host ever seeing an expert id.
//
// One warp per token. Lane l keeps logits l, l+32, ... (up to 32 of them, E <= 1024) in registers;
// each of the k rounds takes the warp-wide maximum (lowest expert id on equal values) by shuffles and
// retires it. The softmax runs in fp32 on the k winners and is rounded to the logits' type.
//
// Order of the values is torch.topk's: NaN ranks above everything (a NaN logit is picked first and
// makes the token's weights NaN, as torch.softmax does), -inf is an ordinary smallest value. The k
// picks are always k DIFFERENT valid expert ids, also for a row of all -inf or all NaN (lowest ids
// first there; torch leaves that order unspecified).

#include <cuda_bf16.h>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxK = 8;
constexpr int kMaxPerLane = 32;  // E <= 1024

template <typename T>
__device__ __forceinline__ float load_logit(const T* p);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(__ldg(p)); }

template <typename T>
__device__ __forceinline__ void store_weight(T* p, float w);
template <>
__device__ __forceinline__ void store_weight<float>(float* p, float w) { *p = w; }
template <>
__device__ __forceinline__ void store_weight<__nv_bfloat16>(__nv_bfloat16* p, float w) { *p = __float2bfloat16_rn(w); }

// Does candidate (a, ia) rank before (b, ib)? NaN first, then larger value, then lower id.
__device__ __forceinline__ bool ranks_before(float a, int32_t ia, float b, int32_t ib) {
  const bool an = a != a, bn = b != b;
  if (an != bn) return an;
  if (!an && a != b) return a > b;
  return ia < ib;
}

template <typename logit_t, typename index_t, int kPerLane>
__global__ void __launch_bounds__(kThreads)
router_topk_kernel(const logit_t* __restrict__ logits, int64_t num_tokens, int32_t num_experts, int32_t k,
                   index_t* __restrict__ expert_idx, logit_t* __restrict__ expert_weight) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); t < num_tokens;
       t += warps) {
    const logit_t* row = logits + t * num_experts;
    float v[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < num_experts ? load_logit<logit_t>(row + e) : -INFINITY;
    }
    float picked[kMaxK];
    int32_t picked_id[kMaxK];
    uint32_t retired = 0;  // bit j: this lane's j-th logit has been picked
    for (int r = 0; r < k; ++r) {
      // Best of this lane (lowest id among equals: ids grow with j), then of the warp.
      float best = -INFINITY;
      int32_t best_id = INT32_MAX;
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        const int32_t e = lane + 32 * j;
        if (e < num_experts && !((retired >> j) & 1u) && ranks_before(v[j], e, best, best_id)) {
          best = v[j];
          best_id = e;
        }
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, d);
        const int32_t other_id = __shfl_xor_sync(0xffffffffu, best_id, d);
        if (ranks_before(other, other_id, best, best_id)) {
          best = other;
          best_id = other_id;
        }
      }
      picked[r] = best;
      picked_id[r] = best_id;
      if ((best_id & 31) == lane) retired |= 1u << (best_id >> 5);
    }
    // Softmax over the k winners, fp32; picked[0] is the maximum.
    float denom = 0.0f;
    for (int r = 0; r < k; ++r) denom += __expf(picked[r] - picked[0]);
    if (lane < k) {
      float mine = 0.0f;
      int32_t mine_id = 0;
      for (int r = 0; r < k; ++r)
        if (r == lane) {
          mine = picked[r];
          mine_id = picked_id[r];
        }
      expert_idx[t * k + lane] = static_cast<index_t>(mine_id);
      store_weight<logit_t>(expert_weight + t * k + lane, __expf(mine - picked[0]) / denom);
    }
  }
}

template <typename logit_t, typename index_t>
int launch_router(const void* logits, int64_t num_tokens, int32_t num_experts, int32_t k, void* expert_idx,
                  void* expert_weight, cudaStream_t stream) {
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  int64_t blocks = (num_tokens + kThreads / 32 - 1) / (kThreads / 32);
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 8;
  if (blocks > cap) blocks = cap;
  const auto* in = static_cast<const logit_t*>(logits);
  auto* idx = static_cast<index_t*>(expert_idx);
  auto* w = static_cast<logit_t*>(expert_weight);
  const unsigned grid = static_cast<unsigned>(blocks);
  const int per_lane = (num_experts + 31) / 32;
  if (per_lane <= 2)
    router_topk_kernel<logit_t, index_t, 2><<<grid, kThreads, 0, stream>>>(in, num_tokens, num_experts, k, idx, w);
  else if (per_lane <= 8)
    router_topk_kernel<logit_t, index_t, 8><<<grid, kThreads, 0, stream>>>(in, num_tokens, num_experts, k, idx, w);
  else
    router_topk_kernel<logit_t, index_t, kMaxPerLane><<<grid, kThreads, 0, stream>>>(in, num_tokens, num_experts, k,
                                                                                    idx, w);
  return check_launch("router_topk");
}

}  // namespace
}  // namespace sb

extern "C" int sb_router_topk(const void* logits, int logits_dtype, int64_t num_tokens, int32_t num_experts, int32_t k,
                              void* expert_idx, int idx_is_i64, void* expert_weight, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!logits || !expert_idx || !expert_weight) return fail(SB_ERR_INVALID_ARGUMENT, "router_topk: NULL buffer");
  if (num_tokens <= 0 || num_experts <= 0 || num_experts > 32 * kMaxPerLane)
    return fail(SB_ERR_INVALID_ARGUMENT, "router_topk: need T > 0 and 0 < E <= %d", 32 * kMaxPerLane);
  if (k <= 0 || k > kMaxK || k > num_experts)
    return fail(SB_ERR_INVALID_ARGUMENT, "router_topk: need [T, E] logits with 0 < k <= min(E, %d), got k=%d", kMaxK, k);
  if (logits_dtype != 0 && logits_dtype != 1)
    return fail(SB_ERR_INVALID_ARGUMENT, "router_topk: logits_dtype must be 0 (bf16) or 1 (fp32)");
  const cudaStream_t s = as_stream(stream);
  if (logits_dtype == 0) {
    return idx_is_i64 ? launch_router<__nv_bfloat16, int64_t>(logits, num_tokens, num_experts, k, expert_idx, expert_weight, s)
                      : launch_router<__nv_bfloat16, int32_t>(logits, num_tokens, num_experts, k, expert_idx, expert_weight, s);
  }
  return idx_is_i64 ? launch_router<float, int64_t>(logits, num_tokens, num_experts, k, expert_idx, expert_weight, s)
                    : launch_router<float, int32_t>(logits, num_tokens, num_experts, k, expert_idx, expert_weight, s);
}
