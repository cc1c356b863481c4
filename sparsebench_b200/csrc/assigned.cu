// Kernels for the layer on a flat assignment list (copy c sends token token_of_copy[c] to expert
// expert_of_copy[c] with weight weight_of_copy[c]; a token may have any number of copies). The
// reference does these two steps with PyTorch ops (sparsebench/moe.py:78-81 and :87-91):
//
//   sb_remap_rows        routing ran with k = 1, so its row_token holds COPY indices; turn them
//                        into token indices: out[r] = row_copy[r] >= 0 ? token_of_copy[row_copy[r]] : -1.
//                        A token id outside [0, num_tokens) also becomes -1 (the row is computed as
//                        padding and the copy contributes nothing), so that SDD never gathers past x;
//                        the reference's PyTorch indexing raises a device-side assert there instead.
//   sb_combine_assigned  out[token_of_copy[c]] += float(y[copy_row[c]]) * weight[c] in an fp32
//                        accumulator (atomic adds, like index_add_), then one rounding to bf16.

#include <cuda_bf16.h>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kThreads = 256;

template <typename index_t>
__global__ void __launch_bounds__(kThreads)
remap_rows_kernel(const int32_t* __restrict__ row_copy, const index_t* __restrict__ token_of_copy,
                  int32_t* __restrict__ row_token, int64_t num_rows, int64_t num_copies, int64_t num_tokens) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < num_rows; r += stride) {
    const int32_t c = row_copy[r];
    int64_t token = -1;
    if (c >= 0 && c < num_copies) token = static_cast<int64_t>(token_of_copy[c]);
    row_token[r] = (token >= 0 && token < num_tokens) ? static_cast<int32_t>(token) : -1;
  }
}

template <typename index_t, typename weight_t>
__global__ void __launch_bounds__(kThreads)
scatter_add_kernel(const uint2* __restrict__ y, const int32_t* __restrict__ copy_row,
                   const index_t* __restrict__ token_of_copy, const weight_t* __restrict__ weight,
                   float* __restrict__ acc, int64_t num_copies, int64_t num_tokens, int32_t quads_per_row) {
  // One thread per (copy, 4 columns): 8 bytes of y in, four float atomics out.
  const int64_t total = num_copies * quads_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t c = i / quads_per_row;
    const int32_t q = static_cast<int32_t>(i - c * quads_per_row);
    const int32_t row = __ldg(copy_row + c);
    const int64_t token = static_cast<int64_t>(__ldg(token_of_copy + c));
    if (row < 0 || token < 0 || token >= num_tokens) continue;
    const float w = static_cast<float>(__ldg(weight + c));
    const uint2 raw = __ldg(y + static_cast<int64_t>(row) * quads_per_row + q);
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 lo = __bfloat1622float2(pairs[0]);
    const float2 hi = __bfloat1622float2(pairs[1]);
    float* dst = acc + (token * quads_per_row + q) * 4;
    atomicAdd(dst + 0, lo.x * w);
    atomicAdd(dst + 1, lo.y * w);
    atomicAdd(dst + 2, hi.x * w);
    atomicAdd(dst + 3, hi.y * w);
  }
}

__global__ void __launch_bounds__(kThreads)
round_rows_kernel(const float4* __restrict__ acc, uint2* __restrict__ out, int64_t num_quads) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < num_quads; i += stride) {
    const float4 v = acc[i];
    uint2 packed;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
    o[0] = __floats2bfloat162_rn(v.x, v.y);
    o[1] = __floats2bfloat162_rn(v.z, v.w);
    out[i] = packed;
  }
}

unsigned blocks_for(int64_t items, const DeviceInfo* info) {
  int64_t blocks = (items + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  return static_cast<unsigned>(blocks < 1 ? 1 : blocks);
}

}  // namespace
}  // namespace sb

extern "C" {

int sb_remap_rows(const int32_t* row_copy, const void* token_of_copy, int token_is_i64, int32_t* row_token,
                  int64_t num_rows, int64_t num_copies, int64_t num_tokens, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!row_copy || !token_of_copy || !row_token) return fail(SB_ERR_INVALID_ARGUMENT, "remap_rows: NULL buffer");
  if (num_rows <= 0 || num_copies <= 0 || num_tokens <= 0 || num_tokens > INT32_MAX)
    return fail(SB_ERR_INVALID_ARGUMENT, "remap_rows: sizes must be positive and the token count fit int32");
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  const unsigned blocks = blocks_for(num_rows, info);
  if (token_is_i64)
    remap_rows_kernel<int64_t><<<blocks, kThreads, 0, as_stream(stream)>>>(
        row_copy, static_cast<const int64_t*>(token_of_copy), row_token, num_rows, num_copies, num_tokens);
  else
    remap_rows_kernel<int32_t><<<blocks, kThreads, 0, as_stream(stream)>>>(
        row_copy, static_cast<const int32_t*>(token_of_copy), row_token, num_rows, num_copies, num_tokens);
  return check_launch("remap_rows");
}

int sb_combine_assigned(const void* y, const int32_t* copy_row, const void* token_of_copy, int token_is_i64,
                        const void* weight, int weight_dtype, float* accumulator, void* out, int64_t num_copies,
                        int64_t num_tokens, int32_t d_model, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!y || !copy_row || !token_of_copy || !weight || !accumulator || !out)
    return fail(SB_ERR_INVALID_ARGUMENT, "combine_assigned: NULL buffer");
  if (num_copies <= 0 || num_tokens <= 0) return fail(SB_ERR_INVALID_ARGUMENT, "combine_assigned: sizes must be positive");
  if (d_model <= 0 || d_model % 4 != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "combine_assigned: D (%d) must be a positive multiple of 4", d_model);
  if (weight_dtype != 0 && weight_dtype != 1)
    return fail(SB_ERR_INVALID_ARGUMENT, "combine_assigned: weight_dtype must be 0 (bf16) or 1 (fp32)");
  if (!aligned16(accumulator) || (reinterpret_cast<uintptr_t>(y) & 7u) || (reinterpret_cast<uintptr_t>(out) & 7u))
    return fail(SB_ERR_INVALID_ARGUMENT, "combine_assigned: buffers must be aligned (y/out 8 bytes, accumulator 16)");
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  const cudaStream_t s = as_stream(stream);
  const int32_t quads = d_model / 4;
  const cudaError_t err = cudaMemsetAsync(accumulator, 0, static_cast<size_t>(num_tokens) * d_model * sizeof(float), s);
  if (err != cudaSuccess) return fail(SB_ERR_CUDA, "combine_assigned: memset: %s", cudaGetErrorString(err));
  const unsigned blocks = blocks_for(num_copies * quads, info);
  const uint2* yy = static_cast<const uint2*>(y);
#define SB_SCATTER(INDEX_T, WEIGHT_T)                                                                              \
  scatter_add_kernel<INDEX_T, WEIGHT_T><<<blocks, kThreads, 0, s>>>(yy, copy_row,                                  \
      static_cast<const INDEX_T*>(token_of_copy), static_cast<const WEIGHT_T*>(weight), accumulator, num_copies,   \
      num_tokens, quads)
  if (token_is_i64) {
    if (weight_dtype == 0) SB_SCATTER(int64_t, __nv_bfloat16); else SB_SCATTER(int64_t, float);
  } else {
    if (weight_dtype == 0) SB_SCATTER(int32_t, __nv_bfloat16); else SB_SCATTER(int32_t, float);
  }
#undef SB_SCATTER
  if (int rc = check_launch("combine_assigned (scatter)")) return rc;
  round_rows_kernel<<<blocks_for(num_tokens * quads, info), kThreads, 0, s>>>(
      reinterpret_cast<const float4*>(accumulator), static_cast<uint2*>(out), num_tokens * quads);
  return check_launch("combine_assigned (round)");
}

}  // extern "C"
