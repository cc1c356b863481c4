// Expert-parallel plumbing kernels: everything between the local sort of a rank's copies and the
// all-to-all exchanges, kept on the device so that the step stays free of host syncs.
//
// Setting: N ranks, E experts in total, rank d owns experts [d*Epr, (d+1)*Epr). A rank sorts its
// n = T*k copies by GLOBAL expert id with the routing kernel at block_size 1 (no padding), which
// makes the copies bound for rank d one contiguous run [off_d, off_d + cnt_d) of sorted positions.
// Exchange buffers have a fixed capacity of C rows per (source, destination) pair, so their size
// never depends on a count the host does not know:
//   send[d][i]   i-th copy bound for rank d      recv[s][i]   i-th copy received from rank s
// The owner treats its N*C receive slots as "tokens" of a local k = 1 routing problem; slots past
// the received count carry expert id -1 and are skipped by the routing kernel.
//
// sb_ep_plan         send_index[d*C+i] = source token of slot (d, i) or -1;
//                    return_row[c] = slot d*C+i in which copy c's result comes back, or -1 if the
//                    pair's run overflowed C (then status |= SB_EP_OVERFLOW).
// sb_ep_slot_experts slot_expert[s*C+i] = local expert of the i-th copy from rank s, or -1.
// sb_gather_rows     out[j][:] = src[index[j]][:] where index[j] >= 0 (16-byte vectors).
//
// Dispatch overlapped with the owner's first matmul (ep_dispatch.cuh has the protocol):
// sb_ep_dispatch_segments  arrival flags (and chunk counters) per rank pair for a capacity.
// sb_ep_push_rows_flagged  the source side alone, as a kernel of its own: rows into the owners'
//                       receive buffers, one arrival flag per (source, 256-row segment) at the owner. The
//                       same device code runs inside the SDD kernel's push warps (sb_ep_sdd_dispatch).

#include <cuda_bf16.h>

#include "ep_dispatch.cuh"
#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kThreads = 256;

// Rank whose run contains sorted position `pos`: the last d with rank_start(d) <= pos.
__device__ __forceinline__ int owner_of(const int32_t* __restrict__ expert_offsets, int32_t experts_per_rank,
                                        int32_t num_ranks, int32_t pos) {
  int lo = 0, hi = num_ranks - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (expert_offsets[mid * experts_per_rank] <= pos) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(kThreads)
ep_plan_kernel(const int32_t* __restrict__ expert_offsets, const int32_t* __restrict__ sorted_token,
               const int32_t* __restrict__ copy_pos, int32_t n_copies, int32_t num_ranks, int32_t experts_per_rank,
               int32_t capacity, int32_t* __restrict__ send_index, int32_t* __restrict__ return_row,
               int32_t* __restrict__ status) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // Slots: which token fills slot (d, i).
  const int64_t slots = static_cast<int64_t>(num_ranks) * capacity;
  for (int64_t s = first; s < slots; s += stride) {
    const int32_t d = static_cast<int32_t>(s / capacity);
    const int32_t i = static_cast<int32_t>(s - static_cast<int64_t>(d) * capacity);
    const int32_t begin = expert_offsets[d * experts_per_rank];
    const int32_t end = expert_offsets[(d + 1) * experts_per_rank];
    send_index[s] = i < end - begin ? sorted_token[begin + i] : -1;
    if (i == 0 && end - begin > capacity) atomicOr(status, SB_EP_OVERFLOW);
  }
  // Copies: in which slot copy c's result returns. A copy the local sort skipped (bad id) has
  // copy_pos < 0 and contributes nothing.
  for (int64_t c = first; c < n_copies; c += stride) {
    const int32_t pos = copy_pos[c];
    int32_t slot = -1;
    if (pos >= 0) {
      const int d = owner_of(expert_offsets, experts_per_rank, num_ranks, pos);
      const int32_t i = pos - expert_offsets[d * experts_per_rank];
      if (i < capacity) slot = d * capacity + i;
    }
    return_row[c] = slot;
  }
}

// grid = (ceil(C / kThreads), N). recv_counts[s][e] = copies rank s sent for local expert e.
__global__ void __launch_bounds__(kThreads)
ep_slot_experts_kernel(const int32_t* __restrict__ recv_counts, int32_t experts_per_rank, int32_t capacity,
                       int32_t* __restrict__ slot_expert) {
  extern __shared__ int32_t ends[];  // inclusive prefix of this source's counts, [experts_per_rank]
  const int32_t s = blockIdx.y;
  if (threadIdx.x == 0) {
    int32_t running = 0;
    for (int32_t e = 0; e < experts_per_rank; ++e) {
      running += max(0, recv_counts[s * experts_per_rank + e]);
      ends[e] = running;
    }
  }
  __syncthreads();
  const int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= capacity) return;
  int32_t expert = -1;
  if (i < ends[experts_per_rank - 1]) {
    int32_t lo = 0, hi = experts_per_rank - 1;  // first e with ends[e] > i
    while (lo < hi) {
      const int32_t mid = (lo + hi) >> 1;
      if (ends[mid] > i) hi = mid; else lo = mid + 1;
    }
    expert = lo;
  }
  slot_expert[static_cast<int64_t>(s) * capacity + i] = expert;
}

// One warp per output row; lanes copy 16-byte vectors.
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index, uint4* __restrict__ out,
                   int64_t num_out_rows, int32_t vecs_per_row) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); j < num_out_rows;
       j += warps) {
    const int32_t row = __ldg(index + j);
    if (row < 0) continue;
    copy_row_warp(src + static_cast<int64_t>(row) * vecs_per_row, out + j * vecs_per_row, vecs_per_row, lane);
  }
}

// One warp per slot; lanes copy 16-byte vectors into ANOTHER rank's memory (plain stores through
// the peer mapping, i.e. over NVLink). Slot j = (peer, i) with peer = j / capacity: the row lands in
// the peer's buffer at [my_rank][i]. Only real rows travel; empty slots cost one index read.
__global__ void __launch_bounds__(kThreads)
push_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index, uint4* const* __restrict__ peer_base,
                 int32_t my_rank, int32_t capacity, int64_t num_slots, int32_t vecs_per_row) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t j = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); j < num_slots;
       j += warps) {
    const int32_t row = __ldg(index + j);
    if (row < 0) continue;
    const int32_t peer = static_cast<int32_t>(j / capacity);
    const int64_t i = j - static_cast<int64_t>(peer) * capacity;
    copy_row_warp(src + static_cast<int64_t>(row) * vecs_per_row,
                  peer_base[peer] + (static_cast<int64_t>(my_rank) * capacity + i) * vecs_per_row, vecs_per_row, lane);
  }
}

// counts[d*Epr + e] -> peer d's table at [my_rank*Epr + e].
__global__ void push_counts_kernel(const int32_t* __restrict__ counts, int32_t* const* __restrict__ peer_counts,
                                   int32_t my_rank, int32_t num_ranks, int32_t experts_per_rank) {
  const int32_t total = num_ranks * experts_per_rank;
  for (int32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int32_t d = i / experts_per_rank;
    peer_counts[d][my_rank * experts_per_rank + (i - d * experts_per_rank)] = counts[i];
  }
}

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// All-ranks barrier over peer memory. One block, thread p talks to rank p: it publishes this rank's
// new epoch in p's pad (release, system scope: everything this GPU wrote before the kernel, remote
// stores included, is visible to whoever sees the epoch) and waits until p's epoch shows up in this
// rank's own pad. The wait is bounded; on expiry it sets SB_EP_TIMEOUT in *status and goes on.
constexpr uint64_t kBarrierLimitNs = 2000ull * 1000ull * 1000ull;
__global__ void ep_barrier_kernel(uint32_t* const* __restrict__ peer_pads, uint32_t* __restrict__ my_pad,
                                  uint32_t* __restrict__ epoch_word, int32_t my_rank, int32_t num_ranks,
                                  int32_t* __restrict__ status) {
  const int p = threadIdx.x;
  const uint32_t epoch = *epoch_word + 1u;
  __threadfence_system();
  if (p < num_ranks) {
    uint32_t* remote = peer_pads[p] + my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* mine = my_pad + p;
    const uint64_t start = now_ns();
    uint32_t poll = 0;
    while (true) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (static_cast<int32_t>(seen - epoch) >= 0) break;
      if ((++poll & 255u) == 0u && now_ns() - start > kBarrierLimitNs) {
        atomicOr(status, SB_EP_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  if (p == 0) *epoch_word = epoch;
}

constexpr int kPushThreads = 256;
__global__ void __launch_bounds__(kPushThreads)
ep_push_rows_flagged_kernel(const DispatchParams dp) {
  const int warps = kPushThreads / 32;
  // Consecutive chunks go to different blocks, so the first pairs finish (and signal) first.
  push_chunks(dp, (threadIdx.x >> 5) * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x),
              warps * static_cast<int>(gridDim.x), threadIdx.x & 31);
}

int64_t capped_blocks(int64_t items, int per_block, const DeviceInfo* info) {
  int64_t blocks = (items + per_block - 1) / per_block;
  const int64_t cap = static_cast<int64_t>(info->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : blocks;
}

}  // namespace
}  // namespace sb

extern "C" {

int sb_ep_plan(const int32_t* expert_offsets, const int32_t* sorted_token, const int32_t* copy_pos,
               int64_t n_copies, int32_t num_ranks, int32_t experts_per_rank, int32_t capacity,
               int32_t* send_index, int32_t* return_row, int32_t* status, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!expert_offsets || !sorted_token || !copy_pos || !send_index || !return_row || !status)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_plan: NULL buffer");
  if (n_copies <= 0 || n_copies > INT32_MAX || num_ranks <= 0 || experts_per_rank <= 0 || capacity <= 0 ||
      static_cast<int64_t>(num_ranks) * capacity > INT32_MAX)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_plan: sizes must be positive and fit int32");
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  const int64_t items = std::max<int64_t>(n_copies, static_cast<int64_t>(num_ranks) * capacity);
  ep_plan_kernel<<<static_cast<unsigned>(capped_blocks(items, kThreads, info)), kThreads, 0, as_stream(stream)>>>(
      expert_offsets, sorted_token, copy_pos, static_cast<int32_t>(n_copies), num_ranks, experts_per_rank, capacity,
      send_index, return_row, status);
  return check_launch("ep_plan");
}

int sb_ep_slot_experts(const int32_t* recv_counts, int32_t num_ranks, int32_t experts_per_rank, int32_t capacity,
                       int32_t* slot_expert, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!recv_counts || !slot_expert) return fail(SB_ERR_INVALID_ARGUMENT, "ep_slot_experts: NULL buffer");
  if (num_ranks <= 0 || num_ranks > 65535 || experts_per_rank <= 0 || experts_per_rank > 1024 || capacity <= 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_slot_experts: need 0 < ranks < 65536, 0 < experts per rank <= 1024");
  const dim3 grid(static_cast<unsigned>((capacity + kThreads - 1) / kThreads), static_cast<unsigned>(num_ranks));
  ep_slot_experts_kernel<<<grid, kThreads, experts_per_rank * sizeof(int32_t), as_stream(stream)>>>(
      recv_counts, experts_per_rank, capacity, slot_expert);
  return check_launch("ep_slot_experts");
}

int sb_gather_rows(const void* src, const int32_t* index, void* out, int64_t num_out_rows, int32_t row_bytes,
                   sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!src || !index || !out) return fail(SB_ERR_INVALID_ARGUMENT, "gather_rows: NULL buffer");
  if (num_out_rows <= 0 || row_bytes <= 0 || row_bytes % 16 != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "gather_rows: row size (%d bytes) must be a positive multiple of 16", row_bytes);
  if (!aligned16(src) || !aligned16(out)) return fail(SB_ERR_INVALID_ARGUMENT, "gather_rows: buffers must be 16-byte aligned");
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  gather_rows_kernel<<<static_cast<unsigned>(capped_blocks(num_out_rows, kThreads / 32, info)), kThreads, 0,
                       as_stream(stream)>>>(static_cast<const uint4*>(src), index, static_cast<uint4*>(out),
                                            num_out_rows, row_bytes / 16);
  return check_launch("gather_rows");
}

int sb_ep_push_rows(const void* src, const int32_t* index, void* const* peer_base, int32_t my_rank,
                    int32_t num_ranks, int32_t capacity, int32_t row_bytes, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!src || !index || !peer_base) return fail(SB_ERR_INVALID_ARGUMENT, "ep_push_rows: NULL buffer");
  if (num_ranks <= 0 || my_rank < 0 || my_rank >= num_ranks || capacity <= 0 || row_bytes <= 0 || row_bytes % 16 != 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_push_rows: need 0 <= rank < ranks, capacity > 0, row bytes a multiple of 16");
  if (!aligned16(src)) return fail(SB_ERR_INVALID_ARGUMENT, "ep_push_rows: src must be 16-byte aligned");
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  const int64_t slots = static_cast<int64_t>(num_ranks) * capacity;
  push_rows_kernel<<<static_cast<unsigned>(capped_blocks(slots, kThreads / 32, info)), kThreads, 0, as_stream(stream)>>>(
      static_cast<const uint4*>(src), index, reinterpret_cast<uint4* const*>(peer_base), my_rank, capacity, slots,
      row_bytes / 16);
  return check_launch("ep_push_rows");
}

int32_t sb_ep_dispatch_segments(int32_t capacity) { return capacity > 0 ? sb::dispatch_segments(capacity) : 0; }

int64_t sb_ep_dispatch_schedule_ints(int64_t num_row_blocks) {
  return num_row_blocks > 0 ? sb::dispatch_schedule_ints(num_row_blocks) : 0;
}

int sb_ep_push_rows_flagged(const void* x, const int32_t* sorted_token, const int32_t* expert_offsets,
                            void* const* peer_recv,
                            uint32_t* const* peer_flags, uint32_t* done, const uint32_t* epoch_word, int32_t my_rank,
                            int32_t num_ranks, int32_t experts_local, int32_t capacity, int32_t row_bytes,
                            sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!x || !sorted_token || !expert_offsets || !peer_recv || !peer_flags || !done || !epoch_word)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_push_rows_flagged: NULL buffer");
  if (num_ranks <= 0 || num_ranks > 32 || experts_local <= 0 || my_rank < 0 || my_rank >= num_ranks || capacity <= 0 ||
      row_bytes <= 0 || row_bytes % 16 != 0 || !aligned16(x))
    return fail(SB_ERR_INVALID_ARGUMENT,
                "ep_push_rows_flagged: need 0 <= rank < ranks <= 32, capacity > 0, 16-byte aligned rows of a multiple of 16 bytes");
  const DeviceInfo* info = current_device_info();
  if (info == nullptr) return SB_ERR_CUDA;
  DispatchParams dp{};
  dp.x = static_cast<const uint4*>(x);
  dp.sorted_token = sorted_token;
  dp.expert_offsets = expert_offsets;
  dp.peer_recv = reinterpret_cast<uint4* const*>(peer_recv);
  dp.peer_flags = peer_flags;
  dp.done = done;
  dp.epoch_word = epoch_word;
  dp.my_rank = my_rank;
  dp.num_ranks = num_ranks;
  dp.experts_local = experts_local;
  dp.capacity = capacity;
  dp.segments = dispatch_segments(capacity);
  dp.vecs_per_row = row_bytes / 16;
  ep_push_rows_flagged_kernel<<<static_cast<unsigned>(info->sm_count * 2), kPushThreads, 0, as_stream(stream)>>>(dp);
  return check_launch("ep_push_rows_flagged");
}

int sb_ep_push_counts(const int32_t* counts, int32_t* const* peer_counts, int32_t my_rank, int32_t num_ranks,
                      int32_t experts_per_rank, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!counts || !peer_counts) return fail(SB_ERR_INVALID_ARGUMENT, "ep_push_counts: NULL buffer");
  if (num_ranks <= 0 || my_rank < 0 || my_rank >= num_ranks || experts_per_rank <= 0)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_push_counts: bad rank or size");
  const int total = num_ranks * experts_per_rank;
  push_counts_kernel<<<(total + kThreads - 1) / kThreads, kThreads, 0, as_stream(stream)>>>(counts, peer_counts, my_rank,
                                                                                         num_ranks, experts_per_rank);
  return check_launch("ep_push_counts");
}

int sb_ep_barrier(uint32_t* const* peer_pads, uint32_t* my_pad, uint32_t* epoch_word, int32_t my_rank,
                  int32_t num_ranks, int32_t* status, sb_stream_t stream) {
  using namespace sb;
  clear_error();
  if (!peer_pads || !my_pad || !epoch_word || !status) return fail(SB_ERR_INVALID_ARGUMENT, "ep_barrier: NULL buffer");
  if (num_ranks <= 0 || num_ranks > 1024 || my_rank < 0 || my_rank >= num_ranks)
    return fail(SB_ERR_INVALID_ARGUMENT, "ep_barrier: need 0 <= rank < ranks <= 1024");
  const int threads = (num_ranks + 31) / 32 * 32;
  ep_barrier_kernel<<<1, threads, 0, as_stream(stream)>>>(peer_pads, my_pad, epoch_word, my_rank, num_ranks, status);
  return check_launch("ep_barrier");
}

}  // extern "C"
