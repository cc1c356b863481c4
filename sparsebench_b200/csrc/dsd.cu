// DSD entry point: the second MoE matmul, Y = BSR(H) @ W (general block-sparse x dense). Argument
// rules follow the reference's sparsebench::dsd_cuda (csrc/dsd.cpp:27-80); the kernel is
// bsr_gemm_kernel<kDsd, 256> when D is a multiple of 256 and the 128-wide instance otherwise.

#include "bsr_gemm_pair.cuh"

namespace sb {
namespace {

// Where the result rows go when they do not go to y: the expert-parallel return (see GemmParams).
struct PeerReturn {
  void* const* peer_out = nullptr;
  int32_t my_rank = 0;
  int32_t capacity = 0;
};

int dsd_launch(const void* h_blocks, int64_t num_blocks, const void* w, int64_t w_rows, int32_t d_model,
               const int32_t* row_offsets, const int32_t* col_indices, int32_t num_row_blocks, int32_t block_size,
               int zero_dead_rows, const int32_t* row_token, void* y, const PeerReturn& peer,
               const int32_t* padded_offsets, int32_t num_experts, int32_t* dev_status, sb_stream_t stream) {
  if (block_size != 64 && block_size != 128)
    return fail(SB_ERR_INVALID_ARGUMENT, "block size must be 64 or 128, got %d", block_size);
  if (d_model <= 0 || d_model % 128 != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "D (%d) must be a positive multiple of 128", d_model);
  if (w_rows <= 0 || w_rows % block_size != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "w rows (%lld) must be a multiple of the block size (%d)", (long long)w_rows,
                block_size);
  if (num_row_blocks < 0 || num_blocks < 0) return fail(SB_ERR_INVALID_ARGUMENT, "dsd: negative size");
  if (!w || !row_offsets || !col_indices) return fail(SB_ERR_INVALID_ARGUMENT, "dsd: NULL buffer");
  if (!aligned16(h_blocks) || !aligned16(w) || !aligned16(y))
    return fail(SB_ERR_INVALID_ARGUMENT, "blocks, w and the output must be 16-byte aligned");
  if (num_blocks * block_size > INT32_MAX || w_rows > INT32_MAX ||
      static_cast<int64_t>(num_row_blocks) * block_size > INT32_MAX)
    return fail(SB_ERR_INVALID_ARGUMENT, "dsd: problem too large");
  if (num_row_blocks == 0) return SB_OK;
  if (!y && peer.peer_out == nullptr) return fail(SB_ERR_INVALID_ARGUMENT, "dsd: NULL output");

  CUtensorMap map_a, map_b;
  // H blocks [nnz, bs, bs] seen as [nnz*bs, bs], one box = 64 K columns of one block; with no blocks
  // at all every row block is dead and the map is never used, but it still has to be a valid
  // descriptor.
  const void* a_base = (num_blocks > 0 && h_blocks) ? h_blocks : w;
  const uint64_t a_rows = num_blocks > 0 ? static_cast<uint64_t>(num_blocks) * block_size : block_size;
  if (int rc = encode_bf16_2d_map(&map_a, a_base, a_rows, block_size, block_size, "dsd (blocks)")) return rc;
  // With row_token given, row blocks that end in padding are fetched in 32-row boxes, only the
  // groups that hold real rows.
  CUtensorMap map_a_rows32 = map_a;
  if (row_token != nullptr) {
    if (int rc = encode_bf16_2d_map(&map_a_rows32, a_base, a_rows, block_size, 32, "dsd (blocks, 32 rows)")) return rc;
  }
  if (int rc = encode_bf16_2d_map(&map_b, w, static_cast<uint64_t>(w_rows), static_cast<uint64_t>(d_model), 64,
                                  "dsd (w)"))
    return rc;

  CUtensorMap map_out = map_b;  // y [num_row_blocks*bs, D]; the epilogue stores 32 x 64 boxes (unused with a peer return)
  if (y != nullptr) {
    if (int rc = encode_bf16_2d_map(&map_out, y, static_cast<uint64_t>(num_row_blocks) * block_size,
                                    static_cast<uint64_t>(d_model), 32, "dsd (y)"))
      return rc;
  }

  GemmParams params{};
  params.row_offsets = row_offsets;
  params.num_row_blocks = num_row_blocks;
  params.dev_status = dev_status;
  params.col_indices = col_indices;
  params.y = static_cast<__nv_bfloat16*>(y);
  params.zero_dead_rows = zero_dead_rows ? 1 : 0;
  params.block_rows = block_size;
  params.peer_out = peer.peer_out;
  params.my_rank = peer.my_rank;
  params.capacity = peer.capacity;
  params.raster_rows = 1;  // row-block-major: D/256 slices per row block keep an expert's row blocks in one wave
  // Experts in the matrix, from its shape: w rows / (blocks per row block * block size). Several row blocks per
  // expert (worst case) means a weight tile has several readers close in time.
  if (num_blocks > 0 && num_blocks % num_row_blocks == 0) {
    const int64_t rows_per_expert = num_blocks / num_row_blocks * block_size;
    if (rows_per_expert > 0 && w_rows % rows_per_expert == 0)
      params.reuse_weights = weights_reused_in_l2(num_row_blocks, static_cast<int32_t>(w_rows / rows_per_expert)) ? 1 : 0;
  }
  params.row_token = row_token;
  params.skip_padding = row_token != nullptr ? 1 : 0;
  params.d_model = d_model;
  if (d_model % 256 == 0 && block_size == 128 && !zero_dead_rows &&
      use_pair_kernel(padded_offsets, num_row_blocks, num_experts)) {
    // Layout made by the routing kernel (every row block of an expert has the same column blocks): two row
    // blocks of one expert per tile, on a pair of thread blocks.
    params.num_slices = d_model / 256;
    return launch_gemm_pair<GemmOp::kDsd>(map_a, map_a_rows32, map_b, map_out, params, padded_offsets, num_experts,
                                          as_stream(stream), "dsd");
  }
  if (d_model % 256 == 0) {
    params.num_slices = d_model / 256;
    return launch_gemm<GemmOp::kDsd, 256>(map_a, map_a_rows32, map_b, map_out, params, as_stream(stream), "dsd");
  }
  params.num_slices = d_model / 128;
  return launch_gemm<GemmOp::kDsd, 128>(map_a, map_a_rows32, map_b, map_out, params, as_stream(stream), "dsd");
}

}  // namespace
}  // namespace sb

extern "C" int sb_dsd(const void* h_blocks, int64_t num_blocks, const void* w, int64_t w_rows, int32_t d_model,
                      const int32_t* row_offsets, const int32_t* col_indices, int32_t num_row_blocks,
                      int32_t block_size, int zero_dead_rows, const int32_t* row_token, void* y,
                      const int32_t* padded_offsets, int32_t num_experts, int32_t* dev_status, sb_stream_t stream) {
  sb::clear_error();
  if (padded_offsets != nullptr && num_experts <= 0)
    return sb::fail(SB_ERR_INVALID_ARGUMENT, "dsd: padded_offsets given without the number of experts");
  return sb::dsd_launch(h_blocks, num_blocks, w, w_rows, d_model, row_offsets, col_indices, num_row_blocks, block_size,
                        zero_dead_rows, row_token, y, sb::PeerReturn{}, padded_offsets, num_experts, dev_status, stream);
}

extern "C" int sb_ep_dsd_push(const void* h_blocks, int64_t num_blocks, const void* w, int64_t w_rows, int32_t d_model,
                              const int32_t* row_offsets, const int32_t* col_indices, int32_t num_row_blocks,
                              const int32_t* row_slot, void* const* peer_base, int32_t my_rank, int32_t num_ranks,
                              int32_t capacity, int32_t* dev_status, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!row_slot || !peer_base) return fail(SB_ERR_INVALID_ARGUMENT, "ep_dsd_push: NULL buffer");
  if (num_ranks <= 0 || my_rank < 0 || my_rank >= num_ranks || capacity <= 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_dsd_push: need 0 <= rank < ranks and capacity > 0");
  PeerReturn peer;
  peer.peer_out = peer_base;
  peer.my_rank = my_rank;
  peer.capacity = capacity;
  return dsd_launch(h_blocks, num_blocks, w, w_rows, d_model, row_offsets, col_indices, num_row_blocks, 128, 0, row_slot,
                    nullptr, peer, nullptr, 0, dev_status, stream);
}
