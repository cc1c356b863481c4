/*
 * sparsebench_b200 -- C ABI of the sync-free block-sparse MoE forward path for NVIDIA B200 (sm_100a).
 *
 * Every entry point
 *   - takes plain device pointers, sizes and a CUDA stream (no torch types),
 *   - only enqueues work on that stream: it never synchronises, never reads device memory back
 *     to the host and never calls cudaMalloc/cudaFree (all buffers belong to the caller),
 *   - works on the calling thread's current CUDA device,
 *   - returns SB_OK (0) or one of the sb_status codes; sb_last_error() gives the text of the
 *     calling thread's last failure.
 *
 * Buffers are sized for the worst case on the host; the real padded row count stays in
 * padded_offsets[num_experts] on the device and the kernels read it (or the flat tail of
 * row_offsets) from there. That is what makes the layer capturable in a CUDA graph and replayable
 * with new tokens and new routing.
 *
 * "Reference" below is the SparseBench source tree; each declaration cites the interface it
 * replaces as path:line inside that tree.
 */
#ifndef SPARSEBENCH_B200_H_
#define SPARSEBENCH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A cudaStream_t. Declared opaquely so that the header needs no CUDA include. */
typedef struct CUstream_st* sb_stream_t;

enum sb_status {
  SB_OK = 0,
  SB_ERR_INVALID_ARGUMENT = 1, /* a size/alignment/range rule of the entry point is violated */
  SB_ERR_UNSUPPORTED = 2,      /* legal for the reference, not built here (see sb_last_error) */
  SB_ERR_CUDA = 3,             /* a CUDA runtime/driver call failed (launch, attribute, ...) */
  SB_ERR_TENSOR_MAP = 4        /* cuTensorMapEncodeTiled rejected a descriptor */
};

/* Bits of the device-side status word the GEMM kernels write when a bounded wait gives up. */
enum sb_device_status {
  SB_DEV_OK = 0,
  SB_DEV_TIMEOUT_PRODUCER = 1, /* TMA/gather producer waited too long for a free stage */
  SB_DEV_TIMEOUT_MMA = 2,      /* MMA issuer waited too long for a full stage or a free accumulator */
  SB_DEV_TIMEOUT_EPILOGUE = 4, /* epilogue waited too long for a finished accumulator */
  SB_DEV_TIMEOUT_DISPATCH = 8  /* expert-parallel owner waited too long for a source rank's rows */
};

/* Text of the calling thread's last failure ("" if none). Never NULL. */
const char* sb_last_error(void);
/* Short name of a status code. Never NULL. */
const char* sb_status_string(int code);
/* Library version, "major.minor.patch". */
const char* sb_version(void);

/*
 * Fills out[0..n) with __CUDA_ARCH__ of the device code that actually ran (1000 on B200).
 * Replaces sparsebench::arch_probe (csrc/smoke.cu:23-38, csrc/ops.hpp:7-11). n must be > 0.
 */
int sb_arch_probe(int32_t* out, int64_t n, sb_stream_t stream);

/*
 * Worst-case sizes of the routing outputs, computed the way the reference host code does
 * (csrc/routing.cu:213-224): max_row_blocks = (n_copies + num_experts*(block_size-1)) / block_size,
 * max_rows = max_row_blocks * block_size. Returns SB_ERR_INVALID_ARGUMENT where the reference
 * raises ("num_experts must be in [1, 1024]", "ffn_dim must be a positive multiple of block_size",
 * "problem too large for int32 indexing").
 */
int sb_route_sizes(int64_t n_copies, int32_t num_experts, int64_t ffn_dim, int64_t block_size,
                   int64_t* max_row_blocks, int64_t* max_rows, int64_t* ffn_blocks);

/* Bytes of scratch sb_route needs for (n_copies, num_experts). May be 0. */
size_t sb_route_workspace_bytes(int64_t n_copies, int32_t num_experts);

/*
 * Routing -> block-sparse layout: a stable counting sort of the n_copies = T*k token copies by
 * expert (copy c = t*k + j keeps ascending c inside an expert), every expert group padded to a
 * multiple of block_size, plus the BSR arrays the two matmuls consume. Bit-exact to the
 * reference's topology.build_topology (sparsebench/topology.py:53-118) and to its CUDA version
 * build_topology_cuda (csrc/routing.cu:197-281), including the tails of the worst-case buffers:
 *   row_token[r]       = source token, -1 for padding rows and for rows past the real end
 *   copy_row[c]        = padded row of copy c, -1 if its expert id was outside [0, num_experts)
 *   row_block_expert[] = expert of each row block, -1 past the real end
 *   row_offsets[i]     = min(i, real_row_blocks) * ffn_blocks
 *   col_indices[]      = expert * ffn_blocks + j, -1 past the real end
 *   error[0]           = 1 if any expert id was out of range, else 0 (written, not OR-ed)
 * expert_idx is int32 (idx_is_i64 == 0) or int64. workspace must hold
 * sb_route_workspace_bytes() bytes (may be NULL when that is 0). A caller that only wants the sort
 * (the expert-parallel dispatch, at block_size 1) passes NULL for row_block_expert, row_offsets
 * and col_indices together; those three arrays are then not produced.
 */
int sb_route(const void* expert_idx, int idx_is_i64, int64_t n_copies, int32_t k, int32_t num_experts,
             int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int32_t* tokens_per_expert,
             int32_t* padded_offsets, int32_t* row_token, int32_t* copy_row, int32_t* row_block_expert,
             int32_t* row_offsets, int32_t* col_indices, int32_t* error, void* workspace,
             sb_stream_t stream);

/*
 * Routing for callers that cannot allocate device memory. No counterpart in the reference, whose
 * host code takes its scratch from PyTorch's allocator (csrc/routing.cu:238); this library's own
 * sb_route leaves the scratch to the caller instead. Some callers have no allocator to ask: a
 * language binding that only passes pointers through, a serving process that forbids cudaMalloc
 * after start-up (it synchronises the whole device, which is exactly what this path exists to
 * avoid), or code that runs where allocating would break the surrounding framework's rules.
 * For them this entry point does what sb_route does, with the same inputs, outputs and results,
 * and keeps the chunk histograms of the large launch shape in an array built into the library:
 * SB_ROUTE_STATIC_SCRATCH_BYTES of device memory that every GPU which loads the library holds
 * until the process exits. It calls no cudaMalloc, cudaFree or other allocating routine.
 *   - Sizes whose scratch (sb_route_workspace_bytes) exceeds the array are rejected with
 *     SB_ERR_INVALID_ARGUMENT and a message that names both numbers; 1 MiB covers e.g. 500 000
 *     copies over 1024 experts, or 8 million copies over 64 experts. Up to 131072 copies the
 *     routing is a single launch and no scratch is touched at all.
 *   - The first call on a device looks the array's device address up (once per device, with that
 *     device current). Make that first call outside of any stream capture.
 *   - All calls share the one array, which simply keeps whatever the last call left in it; nothing
 *     in it needs to start at zero. Two calls whose kernels can overlap on the GPU (different
 *     streams, no dependency) would race on it: order them.
 */
#define SB_ROUTE_STATIC_SCRATCH_BYTES (1u << 20)
int sb_route_static_scratch(const void* expert_idx, int idx_is_i64, int64_t n_copies, int32_t k,
                            int32_t num_experts, int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks,
                            int32_t* tokens_per_expert, int32_t* padded_offsets, int32_t* row_token,
                            int32_t* copy_row, int32_t* row_block_expert, int32_t* row_offsets,
                            int32_t* col_indices, int32_t* error, sb_stream_t stream);

/*
 * SDD: h_blocks[row_offsets[rb] + f/128][r][f%128] = (gelu)(x[row_token[rb*128+r]] . w1[e][:, f])
 * for every live row block rb (e = row_block_expert[rb]); padding rows (row_token < 0) are
 * zero-filled inside the load and come out exactly 0. Replaces sparsebench::sdd_cuda
 * (csrc/sdd.cu:123-170; kernel csrc/sdd.cu:43-114). bf16 in/out, fp32 accumulation on the
 * tcgen05 tensor cores, exact-erf GELU. Block size is 128; d_model % 64 == 0; ffn_dim % 256 == 0;
 * x, w1 and h_blocks 16-byte aligned. Row blocks with row_offsets[rb] == row_offsets[rb+1] are
 * skipped and their blocks left unwritten. dev_status (may be NULL) receives sb_device_status
 * bits if a bounded device-side wait expires; it is only ever OR-ed into.
 * skip_padding_rows (no reference counterpart; 0 gives the reference's output): for layouts whose
 * padding rows sit at the end of each row block, as sb_route writes them, a group of 32 rows that is
 * all padding is not stored (those rows of the blocks stay unwritten instead of 0), which saves
 * their share of the H traffic. Pair it with sb_dsd's row_token argument.
 * padded_offsets (no reference counterpart; NULL = never): sb_route's [num_experts + 1] array for this
 * layout. With it, layouts whose experts have several row blocks each (worst case >= 4 per expert, at
 * most 128 experts) run two row blocks of one expert per tile on a pair of thread blocks (tcgen05
 * cta_group::2), each of which loads only half of every weight tile. Same results.
 */
int sb_sdd(const void* x, const void* w1, const int32_t* row_token, const int32_t* row_block_expert,
           const int32_t* row_offsets, void* h_blocks, int64_t num_tokens, int32_t d_model, int32_t ffn_dim,
           int32_t num_experts, int32_t num_row_blocks, int apply_gelu, int skip_padding_rows,
           const int32_t* padded_offsets, int32_t* dev_status, sb_stream_t stream);

/*
 * Diagnostic: how many pairs of thread blocks of the cta_group::2 matmul kernel can be resident at once on the
 * current device (its launches use exactly that many), or -1 after recording an error. Host-side query.
 */
int sb_gemm_pair_clusters(void);

/*
 * DSD: y[rb*bs + r][:] = sum over p in [row_offsets[rb], row_offsets[rb+1]) of
 * h_blocks[p][r][:] . w[col_indices[p]*bs .. +bs][:], a general BSR x dense product.
 * Replaces sparsebench::dsd_cuda (csrc/dsd.cpp:27-80) and its version-5 kernel
 * (csrc/dsd_v5.cu:42-123). bf16 in/out, fp32 accumulation. block_size is 128 or 64 (a 64-row
 * block uses the lower half of the 128-row tensor-core tile) and d_model % 128 == 0.
 * Rows of row blocks without blocks are left unwritten, or zeroed when zero_dead_rows != 0
 * (what the reference's versions 1-3 do).
 * row_token (no reference counterpart; NULL gives the reference's behaviour): the layout's
 * [num_row_blocks * block_size] row -> token table with padding rows (< 0) at the end of each row
 * block. When given, a group of 32 rows that is all padding is neither read from h_blocks nor
 * written to y (those rows of y stay unwritten).
 * padded_offsets / num_experts (no reference counterpart; NULL / 0 = never): only for a layout made by
 * sb_route, where all row blocks of an expert have the same column blocks; as for sb_sdd, such a layout
 * with several row blocks per expert then runs on pairs of thread blocks. A general BSR matrix must
 * pass NULL.
 */
int sb_dsd(const void* h_blocks, int64_t num_blocks, const void* w, int64_t w_rows, int32_t d_model,
           const int32_t* row_offsets, const int32_t* col_indices, int32_t num_row_blocks, int32_t block_size,
           int zero_dead_rows, const int32_t* row_token, void* y, const int32_t* padded_offsets, int32_t num_experts,
           int32_t* dev_status, sb_stream_t stream);

/*
 * Combine: out[t][:] = bf16( sum_j float(y[copy_row[t*k+j]][:]) * float(gate[t][j]) ), products and
 * sums rounded separately in fp32 in the order j = 0..k-1. Replaces the PyTorch lines
 * sparsebench/moe.py:51-55. gate_dtype: 0 = bf16, 1 = fp32. A copy with copy_row < 0 contributes 0.
 * d_model % 8 == 0; y and out 16-byte aligned.
 */
int sb_combine(const void* y, const int32_t* copy_row, const void* gate, int gate_dtype, void* out,
               int64_t num_tokens, int32_t k, int32_t d_model, sb_stream_t stream);

/*
 * Router front end: for every token the k largest of its num_experts logits (descending; the lower
 * expert id wins among equal values) and a softmax over those k logits only, computed in fp32 and
 * rounded to the logits' type. Replaces what the reference does on the host side with torch.topk +
 * torch.softmax (sparsebench/reference.py:19-29); its outputs are exactly the expert_idx /
 * expert_weight inputs of the layer. logits_dtype: 0 = bf16, 1 = fp32; expert_weight has the same
 * type; expert_idx is int32 or int64 [T, k]. num_experts <= 1024, k <= min(num_experts, 8).
 */
int sb_router_topk(const void* logits, int logits_dtype, int64_t num_tokens, int32_t num_experts, int32_t k,
                   void* expert_idx, int idx_is_i64, void* expert_weight, sb_stream_t stream);

/*
 * Router and routing in ONE launch: what sb_router_topk followed by sb_route leaves (expert_idx int64
 * [T, k], expert_weight in the logits' type, and the eight layout arrays of sb_route), computed by one
 * thread-block cluster that never writes the ids out before sorting them. Replaces the host-side
 * torch.topk + softmax of sparsebench/reference.py:19-29 AND sparsebench::build_topology_cuda
 * (csrc/routing.cu:197-281) together. Available where sb_route_from_logits_fused(T, k, E) returns 1
 * (k in {1, 2, 4, 8}, E <= 256, T*k <= 32768); elsewhere it returns SB_ERR_UNSUPPORTED and the two
 * separate calls give the same result.
 */
int sb_route_from_logits_fused(int64_t num_tokens, int32_t k, int32_t num_experts);
int sb_route_from_logits(const void* logits, int logits_dtype, int64_t num_tokens, int32_t k, int32_t num_experts,
                         int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int64_t* expert_idx,
                         void* expert_weight, int32_t* tokens_per_expert, int32_t* padded_offsets, int32_t* row_token,
                         int32_t* copy_row, int32_t* row_block_expert, int32_t* row_offsets, int32_t* col_indices,
                         int32_t* error, sb_stream_t stream);

/*
 * The layer on a flat assignment list: copy c sends token token_of_copy[c] to expert
 * expert_of_copy[c] with weight weight_of_copy[c]; a token may have any number of copies,
 * including none. Replaces the PyTorch steps of sparsebench::moe_forward_assigned
 * (sparsebench/moe.py:59-91). The copies go through sb_route as a k = 1 problem, then:
 *
 * sb_remap_rows: row_token[r] = row_copy[r] >= 0 ? token_of_copy[row_copy[r]] : -1, turning the
 * copy indices k = 1 routing leaves in row_token into token indices (moe.py:78-81). May run in
 * place (row_token == row_copy). token_of_copy is int32 or int64. A token id outside
 * [0, num_tokens) becomes -1: its row is treated as padding and SDD never reads past x (the
 * reference's PyTorch indexing raises a device-side assert for such an id).
 *
 * sb_combine_assigned: out[t][:] = bf16( sum over copies c of token t of
 * float(y[copy_row[c]][:]) * float(weight[c]) ), zero for a token without copies (moe.py:87-91).
 * accumulator is caller-provided fp32 scratch [num_tokens * d_model] (cleared here); the sum uses
 * atomic adds like the reference's index_add_, so its last bits can depend on the order.
 * weight_dtype: 0 = bf16, 1 = fp32. d_model % 4 == 0.
 */
int sb_remap_rows(const int32_t* row_copy, const void* token_of_copy, int token_is_i64, int32_t* row_token,
                  int64_t num_rows, int64_t num_copies, int64_t num_tokens, sb_stream_t stream);
int sb_combine_assigned(const void* y, const int32_t* copy_row, const void* token_of_copy, int token_is_i64,
                        const void* weight, int weight_dtype, float* accumulator, void* out, int64_t num_copies,
                        int64_t num_tokens, int32_t d_model, sb_stream_t stream);

/*
 * Token rounding on the device: top-k routing whose per-expert token counts are moved to the nearest
 * multiple of `tile` (ties down, at most the largest multiple that fits in T) by dropping an expert's
 * lowest-scoring picks or adding the best-scoring tokens that did not pick it; equal scores rank in token
 * order; a token's weights are its kept scores renormalised to sum to 1. Replaces the reference's
 * host-synchronising sparsebench/token_rounding.py:58-81 (its nonzero() learns the list length on the
 * host). Here the list has the fixed length sb_token_rounding_capacity = T*k + E*(tile/2), is written in
 * the reference's order (token-major, expert ascending), and entries past *num_copies carry expert -1,
 * token 0, weight 0: sb_route skips them, so the list feeds the assignment-list layer as it is.
 * scores: fp32 [T, E] (router probabilities), E <= 1024, k <= 8. workspace:
 * sb_token_rounding_workspace_bytes bytes of device memory.
 */
int64_t sb_token_rounding_capacity(int64_t num_tokens, int32_t num_experts, int32_t k, int32_t tile);
size_t sb_token_rounding_workspace_bytes(int64_t num_tokens, int32_t num_experts, int32_t k);
int sb_token_rounding(const float* scores, int64_t num_tokens, int32_t num_experts, int32_t k, int32_t tile,
                      int32_t* token_of_copy, int32_t* expert_of_copy, float* weight_of_copy, int32_t* num_copies,
                      void* workspace, sb_stream_t stream);

/*
 * ---- Expert-parallel plumbing (no counterpart in the reference, which is single-GPU) ----------
 *
 * N ranks, E experts in total, rank d owns experts [d*experts_per_rank, (d+1)*experts_per_rank).
 * A rank first sorts its n copies by GLOBAL expert with sb_route at block_size 1 (no padding):
 * padded_offsets then is the exclusive scan of the per-expert counts, row_token the source token
 * of every sorted position, copy_row the sorted position of every copy. Exchange buffers have a
 * fixed capacity of `capacity` rows per (source, destination) pair, so no size depends on a count
 * the host does not know. The exchanges themselves are all-to-alls of the caller's choosing (NCCL).
 */
enum sb_ep_status {
  SB_EP_OK = 0,
  SB_EP_OVERFLOW = 1, /* a pair's run exceeded `capacity`: copies dropped */
  SB_EP_TIMEOUT = 2   /* sb_ep_barrier gave up waiting for a peer */
};

/*
 * send_index[d*capacity + i] = source token of the i-th copy bound for rank d, -1 past the run;
 * return_row[c] = d*capacity + i, the slot in which copy c's result comes back, -1 if it was
 * dropped (overflow, or an expert id the sort rejected). status is OR-ed with SB_EP_OVERFLOW.
 */
int sb_ep_plan(const int32_t* expert_offsets, const int32_t* sorted_token, const int32_t* copy_pos,
               int64_t n_copies, int32_t num_ranks, int32_t experts_per_rank, int32_t capacity,
               int32_t* send_index, int32_t* return_row, int32_t* status, sb_stream_t stream);

/*
 * recv_counts[s*experts_per_rank + e] = copies rank s sent for local expert e (its slice of
 * tokens_per_expert after the count all-to-all). slot_expert[s*capacity + i] = local expert of
 * receive slot (s, i), -1 past what rank s sent. Feeding slot_expert to sb_route as a k = 1
 * problem gives the owner's layout; -1 slots are skipped by it (its error flag then only says
 * that empty slots exist).
 */
int sb_ep_slot_experts(const int32_t* recv_counts, int32_t num_ranks, int32_t experts_per_rank, int32_t capacity,
                       int32_t* slot_expert, sb_stream_t stream);

/*
 * out[j][:] = src[index[j]][:] for every j in [0, num_out_rows) with index[j] >= 0; other rows of
 * out are left untouched. row_bytes % 16 == 0, both buffers 16-byte aligned. Packs the dispatch
 * buffer (src = x, index = send_index) and the return buffer (src = y, index = the owner's copy_row).
 */
int sb_gather_rows(const void* src, const int32_t* index, void* out, int64_t num_out_rows, int32_t row_bytes,
                   sb_stream_t stream);

/*
 * Exchange over peer memory (NVLink / NVSwitch) instead of a collective library: every rank maps
 * the others' exchange buffers (e.g. CUDA VMM / symmetric memory; mapping them is the caller's job)
 * and passes device arrays of the N base pointers.
 *
 * sb_ep_push_rows: for every slot j = peer*capacity + i with index[j] >= 0, stores row
 * src[index[j]] into peer_base[peer] at row my_rank*capacity + i. Only real rows cross the link, so
 * the traffic is the payload, whatever the capacity. Dispatch: src = x, index = send_index; return:
 * src = y, index = the owner's copy_row over its receive slots.
 * sb_ep_push_counts: counts[d*experts_per_rank + e] -> peer_counts[d][my_rank*experts_per_rank + e].
 * sb_ep_barrier: all ranks wait for each other on the device. peer_pads[p] is rank p's pad of
 * num_ranks words (zeroed once before the first call), my_pad this rank's own, epoch_word a local
 * device counter the kernel advances (so a captured graph stays valid across replays). Stores
 * issued before the barrier, remote ones included, are visible to every rank after it. The wait
 * is bounded (2 s): on expiry SB_EP_TIMEOUT is OR-ed into *status and the kernel returns.
 * Every rank must call it the same number of times.
 */
int sb_ep_push_rows(const void* src, const int32_t* index, void* const* peer_base, int32_t my_rank,
                    int32_t num_ranks, int32_t capacity, int32_t row_bytes, sb_stream_t stream);
int sb_ep_push_counts(const int32_t* counts, int32_t* const* peer_counts, int32_t my_rank, int32_t num_ranks,
                      int32_t experts_per_rank, sb_stream_t stream);
int sb_ep_barrier(uint32_t* const* peer_pads, uint32_t* my_pad, uint32_t* epoch_word, int32_t my_rank,
                  int32_t num_ranks, int32_t* status, sb_stream_t stream);

/*
 * The owner's DSD and the return of its rows in ONE kernel (no reference counterpart: the reference
 * is single-GPU). Same product as sb_dsd at block size 128, but row r of the layout is not written
 * to a local y: with j = row_slot[r] = src * capacity + i (the receive slot the row was computed
 * for; the owner's routing with k = 1 leaves exactly this table as row_token, < 0 for padding), the
 * epilogue stores it into rank src's return buffer, peer_base[src] + (my_rank * capacity + i) *
 * d_model elements, as whole 128-byte segments over NVLink while the tensor cores work on the next
 * tile. Replaces sb_dsd + sb_ep_push_rows on the return leg; follow it with sb_ep_barrier. Groups of
 * 32 rows that are all padding are neither loaded nor stored.
 */
int sb_ep_dsd_push(const void* h_blocks, int64_t num_blocks, const void* w, int64_t w_rows, int32_t d_model,
                   const int32_t* row_offsets, const int32_t* col_indices, int32_t num_row_blocks,
                   const int32_t* row_slot, void* const* peer_base, int32_t my_rank, int32_t num_ranks,
                   int32_t capacity, int32_t* dev_status, sb_stream_t stream);

/*
 * Dispatch overlapped with the owner's first matmul (no reference counterpart). Instead of "push all
 * rows, barrier, compute", only the per-expert COUNTS are exchanged up front; the rows travel while
 * the owners' tensor cores already work on what has arrived.
 *
 * A source's copies bound for destination rank d are one contiguous run of its sort by global expert
 * (expert_offsets [N * experts_local + 1]); copy j of that run goes to row my_rank * capacity + j of d's
 * receive buffer (copies past the capacity are cut, as sb_ep_plan cuts them). The rows are pushed in
 * chunks of 8, slot-major and round-robin over the destinations, so every owner's slots fill from the
 * front; arrival is signalled per SEGMENT of 256 slots: sb_ep_dispatch_segments(capacity) flags per
 * rank pair. Per step: sb_ep_push_counts, sb_ep_barrier (after it every owner knows how many rows to
 * expect from whom), sb_ep_owner_layout, sb_ep_sdd_dispatch.
 *
 * sb_ep_owner_layout: the owner's block-sparse layout over its N * capacity receive slots from those
 * counts alone (recv_counts [N][experts_local]), in one launch: the arrays sb_route writes when it is
 * handed sb_ep_slot_experts' output as a k = 1 problem, bit for bit (row_token holds receive-slot
 * indices; error is always 0). N * experts_local <= 1024. max_row_blocks as sb_route_sizes gives for
 * N * capacity copies. row_block_order (NULL: not wanted; needs max_row_blocks <= 4096, N <= 31, block_size <= 256):
 * the owner's schedule, sb_ep_dispatch_schedule_ints(max_row_blocks) ints. First max_row_blocks entries: the row
 * blocks sorted by the largest slot index (within its source's region) among their rows, ties in layout order,
 * row blocks without rows last: the order in which their rows become complete when every source fills its slots
 * from the front. Then 64 ints per row block: how many arrival flags its rows depend on, followed by their
 * indices source * segments + segment.
 *
 * sb_ep_push_rows_flagged: the source side as a kernel of its own. When the last chunk of segment g of
 * destination d is in, peer_flags[d][my_rank * segments + g] is set to the current value of *epoch_word
 * with a system-scope release store. done: N * segments zeroed counters (left zeroed). epoch_word:
 * the counter sb_ep_barrier advances, read AFTER the counts barrier of the step, so that every rank
 * uses the same value; flags never need clearing.
 *
 * sb_ep_sdd_dispatch: sb_sdd over the receive buffer with both sides of that protocol inside the
 * matmul kernel: six extra warps per thread block do this rank's pushes (as a source), and the
 * gather warps wait, per tile, until the segments that hold the tile's rows have arrived (as an owner:
 * my_flags, this rank's flag array [N * segments]). row_block_order: sb_ep_owner_layout's schedule; tiles
 * are walked in its order and wait for the flags of its lists (NULL: layout order, flags worked out per row). The wait is bounded (1 s): on expiry SB_DEV_TIMEOUT_DISPATCH is
 * OR-ed into *dev_status and the kernel winds down. recv_rows [N * capacity, D] is this rank's receive
 * buffer, row_slot the owner layout's row_token. Padding-only groups of 32 rows are not stored.
 * Every rank must launch it once per step (an owner without rows still has rows to push).
 * push_warps: how many of the six push warps per thread block take part (-1: all). 0: none, this rank's rows
 * are pushed by sb_ep_push_rows_flagged, launched BEFORE this kernel on another stream so that the two run side by
 * side (the push kernel waits for nothing; this kernel's waits are bounded as above).
 */
int32_t sb_ep_dispatch_segments(int32_t capacity);
int64_t sb_ep_dispatch_schedule_ints(int64_t num_row_blocks);
int sb_ep_owner_layout(const int32_t* recv_counts, int32_t num_ranks, int32_t experts_local, int32_t capacity,
                       int32_t ffn_blocks, int32_t block_size, int32_t max_row_blocks, int32_t* tokens_per_expert,
                       int32_t* padded_offsets, int32_t* row_token, int32_t* copy_row, int32_t* row_block_expert,
                       int32_t* row_offsets, int32_t* col_indices, int32_t* row_block_order, int32_t* error,
                       sb_stream_t stream);
int sb_ep_push_rows_flagged(const void* x, const int32_t* sorted_token, const int32_t* expert_offsets,
                            void* const* peer_recv, uint32_t* const* peer_flags, uint32_t* done,
                            const uint32_t* epoch_word, int32_t my_rank, int32_t num_ranks, int32_t experts_local,
                            int32_t capacity, int32_t row_bytes, sb_stream_t stream);
int sb_ep_sdd_dispatch(const void* recv_rows, const void* w1, const int32_t* row_slot, const int32_t* row_block_expert,
                       const int32_t* row_offsets, void* h_blocks, int32_t d_model, int32_t ffn_dim,
                       int32_t num_row_blocks, const void* x, const int32_t* sorted_token,
                       const int32_t* expert_offsets, const int32_t* row_block_order, void* const* peer_recv,
                       uint32_t* const* peer_flags, const uint32_t* my_flags, uint32_t* done,
                       const uint32_t* epoch_word, int32_t my_rank, int32_t num_ranks, int32_t experts_local,
                       int32_t capacity, int32_t push_warps, int32_t* dev_status, sb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARSEBENCH_B200_H_ */
