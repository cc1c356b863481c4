// SDD entry point: the first MoE matmul, H = (gelu)(gather(x) @ W1[expert]), written straight into
// the block-sparse (BSR) block list. Argument rules follow the reference host function
// sparsebench::sdd_cuda (csrc/sdd.cu:123-170); the kernel is bsr_gemm_kernel<kSdd, 256>.

#include <cstdlib>

#include "bsr_gemm_pair.cuh"

namespace sb {
namespace {

// dispatch == nullptr: the plain kernel. Otherwise the expert-parallel instance whose extra warps push
// this rank's rows to their owners and whose gather warps wait for the rows of each tile's expert.
int sdd_launch(const void* x, const void* w1, const int32_t* row_token, const int32_t* row_block_expert,
               const int32_t* row_offsets, void* h_blocks, int64_t num_tokens, int32_t d_model, int32_t ffn_dim,
               int32_t num_experts, int32_t num_row_blocks, int apply_gelu, int skip_padding_rows,
               const int32_t* padded_offsets, const DispatchParams* dispatch, int32_t* dev_status, sb_stream_t stream) {
  if (!x || !w1 || !row_token || !row_block_expert || !row_offsets)
    return fail(SB_ERR_INVALID_ARGUMENT, "sdd: NULL buffer");
  if (num_tokens <= 0 || num_experts <= 0 || num_row_blocks < 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "sdd: x must be [T, D] and w1 [E, D, F] with T, E > 0");
  if (d_model <= 0 || d_model % 64 != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "sdd needs D (%d) to be a multiple of 64", d_model);
  if (ffn_dim <= 0 || ffn_dim % 256 != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "sdd needs F (%d) to be a multiple of 256", ffn_dim);
  if (!aligned16(x) || !aligned16(w1) || !aligned16(h_blocks))
    return fail(SB_ERR_INVALID_ARGUMENT, "x, w1 and the output blocks must be 16-byte aligned");
  const int64_t w_rows = static_cast<int64_t>(num_experts) * d_model;
  if (w_rows > INT32_MAX || static_cast<int64_t>(ffn_dim) * d_model > INT32_MAX ||
      static_cast<int64_t>(num_row_blocks) * (ffn_dim / 256) > INT32_MAX)
    return fail(SB_ERR_INVALID_ARGUMENT, "sdd: problem too large");
  if (num_row_blocks == 0 && dispatch == nullptr) return SB_OK;
  if (num_row_blocks == 0) return fail(SB_ERR_INVALID_ARGUMENT, "sdd (dispatch): the owner needs at least one row block");
  if (!h_blocks) return fail(SB_ERR_INVALID_ARGUMENT, "sdd: NULL output");

  CUtensorMap map_a{};  // unused by SDD: its A rows are gathered by cp.async
  CUtensorMap map_b;
  if (int rc = encode_bf16_2d_map(&map_b, w1, static_cast<uint64_t>(w_rows), static_cast<uint64_t>(ffn_dim), 64,
                                  "sdd (w1)"))
    return rc;

  // Output: the block list [nnz, 128, 128] seen as [nnz*128, 128]; the epilogue stores 32 x 64 boxes.
  CUtensorMap map_out;
  const uint64_t nnz = static_cast<uint64_t>(num_row_blocks) * (ffn_dim / 128);
  if (int rc = encode_bf16_2d_map(&map_out, h_blocks, nnz * 128, 128, 32, "sdd (blocks)")) return rc;

  GemmParams params{};
  params.row_offsets = row_offsets;
  params.num_row_blocks = num_row_blocks;
  params.num_slices = ffn_dim / 256;
  params.dev_status = dev_status;
  params.x = static_cast<const __nv_bfloat16*>(x);
  params.row_token = row_token;
  params.row_block_expert = row_block_expert;
  params.h_out = static_cast<__nv_bfloat16*>(h_blocks);
  params.apply_gelu = apply_gelu ? 1 : 0;
  params.skip_padding = skip_padding_rows ? 1 : 0;
  params.d_model = d_model;
  params.block_rows = 128;
  // Experts with many row blocks (worst case >= 4 per expert): walk the tiles in bands of 8 row blocks,
  // so that a W1 tile is read from HBM once per band instead of once per wave (measured on the
  // Mixtral-like shape: 1027 -> 861 us; shapes with ~2 row blocks per expert lose 3-5 % and stay plain).
  params.raster_rows = num_row_blocks >= 4 * num_experts ? 8 : 1;
  params.reuse_weights = weights_reused_in_l2(num_row_blocks, num_experts) ? 1 : 0;
  if (dispatch == nullptr && use_pair_kernel(padded_offsets, num_row_blocks, num_experts)) {
    params.raster_rows = 4;  // bands of 4 pairs = 8 row blocks
    return launch_gemm_pair<GemmOp::kSdd>(map_a, map_a, map_b, map_out, params, padded_offsets, num_experts,
                                          as_stream(stream), "sdd");
  }
  if (dispatch != nullptr) {
    params.dispatch = *dispatch;
    // A row must fit a third of the bulk-push ring; wider rows go through the push warps.
    if (dispatch->bulk_engine != 0 && d_model * 2 <= GemmConfig<GemmOp::kSdd, 256, 2>::kPushRingBytes / 3)
      return launch_gemm<GemmOp::kSdd, 256, 2>(map_a, map_a, map_b, map_out, params, as_stream(stream),
                                               "sdd (dispatch, bulk pushes)");
    return launch_gemm<GemmOp::kSdd, 256, 1>(map_a, map_a, map_b, map_out, params, as_stream(stream),
                                             "sdd (dispatch)");
  }
  return launch_gemm<GemmOp::kSdd, 256>(map_a, map_a, map_b, map_out, params, as_stream(stream), "sdd");
}

}  // namespace
}  // namespace sb

extern "C" int sb_sdd(const void* x, const void* w1, const int32_t* row_token, const int32_t* row_block_expert,
                      const int32_t* row_offsets, void* h_blocks, int64_t num_tokens, int32_t d_model,
                      int32_t ffn_dim, int32_t num_experts, int32_t num_row_blocks, int apply_gelu,
                      int skip_padding_rows, const int32_t* padded_offsets, int32_t* dev_status, sb_stream_t stream) {
  sb::clear_error();
  return sb::sdd_launch(x, w1, row_token, row_block_expert, row_offsets, h_blocks, num_tokens, d_model, ffn_dim,
                        num_experts, num_row_blocks, apply_gelu, skip_padding_rows, padded_offsets, nullptr, dev_status,
                        stream);
}

extern "C" int sb_ep_sdd_dispatch(const void* recv_rows, const void* w1, const int32_t* row_slot,
                                  const int32_t* row_block_expert, const int32_t* row_offsets, void* h_blocks,
                                  int32_t d_model, int32_t ffn_dim, int32_t num_row_blocks, const void* x,
                                  const int32_t* sorted_token, const int32_t* expert_offsets,
                                  const int32_t* row_block_order, void* const* peer_recv,
                                  uint32_t* const* peer_flags, const uint32_t* my_flags, uint32_t* done,
                                  const uint32_t* epoch_word, int32_t my_rank, int32_t num_ranks,
                                  int32_t experts_local, int32_t capacity, int32_t push_warps, int32_t* dev_status,
                                  sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!x || !sorted_token || !expert_offsets || !peer_recv || !peer_flags || !my_flags || !done || !epoch_word)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_sdd_dispatch: NULL buffer");
  if (num_ranks <= 0 || num_ranks > kMaxDispatchRanks || my_rank < 0 || my_rank >= num_ranks || experts_local <= 0 ||
      capacity <= 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_sdd_dispatch: need 0 <= rank < ranks <= %d, local experts > 0, capacity > 0",
                kMaxDispatchRanks);
  if (!aligned16(x)) return fail(SB_ERR_INVALID_ARGUMENT, "ep_sdd_dispatch: x must be 16-byte aligned");
  DispatchParams dp{};
  dp.x = static_cast<const uint4*>(x);
  dp.sorted_token = sorted_token;
  dp.expert_offsets = expert_offsets;
  dp.peer_recv = reinterpret_cast<uint4* const*>(peer_recv);
  dp.peer_flags = peer_flags;
  dp.done = done;
  dp.my_flags = my_flags;
  dp.row_block_order = row_block_order;
  dp.epoch_word = epoch_word;
  dp.my_rank = my_rank;
  dp.num_ranks = num_ranks;
  dp.experts_local = experts_local;
  dp.capacity = capacity;
  dp.segments = dispatch_segments(capacity);
  dp.push_warps = push_warps;
  if (push_warps < 0) {
    dp.push_warps = 6;
    if (const char* v = std::getenv("SB_PUSH_WARPS")) dp.push_warps = std::atoi(v);
  }
  dp.bulk_engine = 0;
  if (push_warps != 0)
    if (const char* v = std::getenv("SB_PUSH_ENGINE")) dp.bulk_engine = std::atoi(v);
  dp.vecs_per_row = d_model / 8;
  return sdd_launch(recv_rows, w1, row_slot, row_block_expert, row_offsets, h_blocks,
                    static_cast<int64_t>(num_ranks) * capacity, d_model, ffn_dim, experts_local, num_row_blocks, 1, 1, nullptr,
                    &dp, dev_status, stream);
}

extern "C" int sb_gemm_pair_clusters(void) {
  using namespace sb;
  clear_error();
  int device = 0;
  const DeviceInfo* info = current_device_info(&device);
  if (info == nullptr) return -1;
  int fit = 0;
  if (pair_resident_clusters<GemmOp::kSdd>(device, info->sm_count, &fit) != SB_OK) return -1;
  return fit;
}
