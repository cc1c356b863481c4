// Gate-weighted combine of each token's k expert rows: the last stage of the MoE layer.
//
//   out[t][:] = bf16( sum_j float(y[copy_row[t*k + j]][:]) * float(gate[t][j]) )
//
// Same arithmetic as the reference's PyTorch lines (sparsebench/moe.py:51-55): every product is
// rounded to fp32, the k products are added in order j = 0..k-1, and the sum is rounded once to
// bf16. Bandwidth-bound: each thread owns 8 consecutive columns of one token, reads k 16-byte
// vectors through the read-only path and writes one 16-byte vector, so a warp moves 512 contiguous
// bytes per row it touches. A copy whose expert id was rejected by routing (copy_row < 0)
// contributes nothing and is never dereferenced.

#include <cuda_bf16.h>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kCombineThreads = 256;

template <typename gate_t>
__device__ __forceinline__ float gate_to_float(gate_t g);
template <>
__device__ __forceinline__ float gate_to_float<float>(float g) { return g; }
template <>
__device__ __forceinline__ float gate_to_float<__nv_bfloat16>(__nv_bfloat16 g) { return __bfloat162float(g); }

template <typename gate_t>
__global__ void __launch_bounds__(kCombineThreads)
combine_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ copy_row, const gate_t* __restrict__ gate,
               uint4* __restrict__ out, int64_t num_tokens, int32_t k, int32_t vecs_per_row) {
  const int64_t total = num_tokens * vecs_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t t = i / vecs_per_row;
    const int32_t v = static_cast<int32_t>(i - t * vecs_per_row);
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
    for (int32_t j = 0; j < k; ++j) {
      const int32_t row = __ldg(copy_row + t * k + j);
      if (row < 0) continue;
      const float g = gate_to_float<gate_t>(__ldg(gate + t * k + j));
      const uint4 raw = __ldg(y + static_cast<int64_t>(row) * vecs_per_row + v);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(pairs[q]);
        // Separate multiply and add (no fused multiply-add) to round like the reference does.
        acc[2 * q] = __fadd_rn(acc[2 * q], __fmul_rn(f.x, g));
        acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], __fmul_rn(f.y, g));
      }
    }
    uint4 packed;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    out[i] = packed;
  }
}

}  // namespace
}  // namespace sb

extern "C" int sb_combine(const void* y, const int32_t* copy_row, const void* gate, int gate_dtype, void* out,
                          int64_t num_tokens, int32_t k, int32_t d_model, sb_stream_t stream) {
  sb::clear_error();
  if (!y || !copy_row || !gate || !out) return sb::fail(SB_ERR_INVALID_ARGUMENT, "combine: NULL buffer");
  if (num_tokens <= 0 || k <= 0) return sb::fail(SB_ERR_INVALID_ARGUMENT, "combine: T and k must be positive");
  if (d_model <= 0 || d_model % 8 != 0)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "combine: D (%d) must be a positive multiple of 8", d_model);
  if (!sb::aligned16(y) || !sb::aligned16(out))
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "combine: y and out must be 16-byte aligned");
  if (gate_dtype != 0 && gate_dtype != 1)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "combine: gate_dtype must be 0 (bf16) or 1 (fp32)");
  const sb::DeviceInfo* info = sb::current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;

  const int32_t vecs = d_model / 8;
  const int64_t total = num_tokens * vecs;
  int64_t blocks = (total + sb::kCombineThreads - 1) / sb::kCombineThreads;
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 16;  // a few waves, then grid-stride
  if (blocks > cap) blocks = cap;
  const cudaStream_t s = sb::as_stream(stream);
  if (gate_dtype == 0) {
    sb::combine_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), sb::kCombineThreads, 0, s>>>(
        static_cast<const uint4*>(y), copy_row, static_cast<const __nv_bfloat16*>(gate), static_cast<uint4*>(out),
        num_tokens, k, vecs);
  } else {
    sb::combine_kernel<float><<<static_cast<unsigned>(blocks), sb::kCombineThreads, 0, s>>>(
        static_cast<const uint4*>(y), copy_row, static_cast<const float*>(gate), static_cast<uint4*>(out), num_tokens,
        k, vecs);
  }
  return sb::check_launch("combine");
}
