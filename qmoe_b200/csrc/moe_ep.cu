// Dispatch metadata of the top-1 MoE layer in three launches: the capacity rule, the packing of rows
// into fixed-size exchange slots (with each row's local expert id in a 16-byte trailer) and the plan
// of the receiving side (tokens per local expert, their offsets and which received row feeds which
// slot of the grouped FFN).  The reference has no counterpart: FasterMLP.forward (sub1.py:306-321)
// loops over the active experts on the host with nonzero() and boolean masks, and hops whole
// activations between GPUs (sub1.py:307-309,320) instead of exchanging rows.
//
// Nothing here copies a row twice: the grouped FFN reads its input rows through the plan's row list
// and writes its output rows back to the same places, so there is no permute / un-permute pass.
//
// Exchange over peer memory: with `blocks` (one pointer per destination rank, each the part of that
// rank's receive buffer reserved for rows from this rank, as mapped into this GPU's address space)
// k_ep_keep and k_ep_pack store rows straight into the destinations' memory, and k_ep_plan can emit
// for every slot the address of its output row in the source rank's return buffer, which the
// grouped FFN then stores to.  k_peer_barrier orders the two sides: every rank raises one flag per
// peer in the peer's memory and waits for the peers' flags in its own, with a time limit.
#include "common.cuh"

namespace qmoe {

__device__ __forceinline__ int block_sum(int v, int *s_warp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) s_warp[warp] = v;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < nwarps; w++) total += s_warp[w];
  return total;
}

// Warp t < n_tokens: the router's capacity rule (kept iff fewer than `capacity` earlier tokens of the
// same sequence chose the same expert: cumsum(one_hot) <= expert_capacity; the lanes share out the
// earlier tokens).  expert[t] = choice or -1, dest[t] = the rank that owns the expert or -1.
// Thread i < n_slots: the trailer of exchange slot i is reset to "empty" (-1).
__global__ void k_ep_keep(const int32_t *__restrict__ choice, int32_t *__restrict__ expert,
                          int32_t *__restrict__ dest, int n_tokens, int n_experts, int local_experts,
                          int seq_len, int capacity, __nv_bfloat16 *__restrict__ send,
                          __nv_bfloat16 *const *__restrict__ blocks, int cap, int n_slots,
                          long long row_stride, int d_model) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_slots) {
    __nv_bfloat16 *row = blocks != nullptr ? blocks[i / cap] + (long long)(i % cap) * row_stride
                                           : send + (long long)i * row_stride;
    *reinterpret_cast<int32_t *>(row + d_model) = -1;
  }
  const int t = (int)(i >> 5), lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  const int c = choice[t];
  int keep = c >= 0 && c < n_experts;
  if (keep && capacity < seq_len) {
    const int s0 = (t / seq_len) * seq_len;
    int before = 0;
    for (int u = s0 + lane; u < t; u += 32) before += (choice[u] == c);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    keep = before < capacity;
  }
  if (lane == 0) {
    expert[t] = keep ? c : -1;
    dest[t] = keep ? c / local_experts : -1;
  }
}

// One CTA per token: rank of the token among the earlier kept tokens with the same destination
// (stable: token order), its exchange slot dest * cap + rank, the copy of its row and its trailer.
// A token whose rank does not fit the pair capacity is not sent: slot -1 (it passes through the
// layer like a token dropped by the capacity rule) and *overflow is incremented (never cleared here).
__global__ void __launch_bounds__(128) k_ep_pack(const int32_t *__restrict__ expert, const int32_t *__restrict__ dest,
                                                 const __nv_bfloat16 *__restrict__ hidden, long long hidden_stride,
                                                 __nv_bfloat16 *__restrict__ send,
                                                 __nv_bfloat16 *const *__restrict__ blocks, long long row_stride,
                                                 int32_t *__restrict__ slot, int *overflow, int d_model,
                                                 int local_experts, int cap) {
  __shared__ int s_warp[4];
  const int t = blockIdx.x;
  const int dst = dest[t];
  if (dst < 0) {
    if (threadIdx.x == 0) slot[t] = -1;
    return;
  }
  int mine = 0;
  for (int u = threadIdx.x; u < t; u += blockDim.x) mine += (dest[u] == dst);
  const int rank = block_sum(mine, s_warp);
  if (rank >= cap) {
    if (threadIdx.x == 0) {
      slot[t] = -1;
      atomicAdd(overflow, 1);
    }
    return;
  }
  const int s = dst * cap + rank;
  __nv_bfloat16 *row = blocks != nullptr ? blocks[dst] + (long long)rank * row_stride : send + (long long)s * row_stride;
  const __nv_bfloat16 *src = hidden + (long long)t * hidden_stride;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(row)) & 15u) == 0 && (d_model & 7) == 0) {
    for (int i = threadIdx.x; i < d_model / 8; i += blockDim.x)
      reinterpret_cast<uint4 *>(row)[i] = reinterpret_cast<const uint4 *>(src)[i];
  } else {
    for (int i = threadIdx.x; i < d_model; i += blockDim.x) row[i] = src[i];
  }
  if (threadIdx.x == 0) {
    slot[t] = s;
    *reinterpret_cast<int32_t *>(row + d_model) = expert[t] - dst * local_experts;
  }
}

// One CTA.  The bucket of row i (-1 = no row) is read from the trailers of received rows (rows !=
// nullptr) or from an int32 array.  Produces offsets[n_buckets + 1] (exclusive prefix sums of the
// bucket sizes), slot_of_row[i] = offsets[bucket] + stable rank (or -1) and row_of_slot[slot] = i.
// Every pass is parallel over the rows: (1) bucket sizes by shared-memory atomics, each row keeping
// the position it arrived at; (2) offsets by a block scan; (3) the members of every bucket written
// to the bucket's slots in arrival order; (4) the stable rank of a row = the members of its bucket
// with a smaller row index (buckets hold a handful of rows under a balanced router; a bucket of m
// rows costs m * m compares); (5) the final lists.
__global__ void __launch_bounds__(1024) k_ep_plan(const __nv_bfloat16 *__restrict__ rows, long long row_stride,
                                                  int d_model, const int32_t *__restrict__ meta_in, int n_rows,
                                                  int n_buckets, int32_t *__restrict__ offsets,
                                                  int32_t *__restrict__ slot_of_row, int32_t *__restrict__ row_of_slot,
                                                  const unsigned long long *__restrict__ out_blocks, int rows_per_block,
                                                  long long out_row_bytes, unsigned long long *__restrict__ out_ptr_of_slot) {
  extern __shared__ int s_count[];  // size of every bucket, later its first slot; then the sizes again
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  int *s_size = s_count + n_buckets;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto bucket_of = [&](int i) {
    const int b = rows != nullptr ? *reinterpret_cast<const int32_t *>(rows + (long long)i * row_stride + d_model)
                                  : meta_in[i];
    return (b >= 0 && b < n_buckets) ? b : -1;
  };
  for (int b = tid; b < n_buckets; b += blockDim.x) s_count[b] = 0;
  __syncthreads();
  for (int i = tid; i < n_rows; i += blockDim.x) {
    const int b = bucket_of(i);
    slot_of_row[i] = b >= 0 ? atomicAdd(&s_count[b], 1) : -1;  // arrival position, replaced in pass 4
  }
  if (tid == 0) {
    s_carry = 0;
    offsets[0] = 0;
  }
  __syncthreads();
  for (int b0 = 0; b0 < n_buckets; b0 += blockDim.x) {
    const int b = b0 + tid;
    const int v = b < n_buckets ? s_count[b] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += u;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int incl_all = s_carry + (warp ? s_warp[warp - 1] : 0) + incl;
    if (b < n_buckets) {
      offsets[1 + b] = incl_all;
      s_count[b] = incl_all - v;  // now the bucket's first slot
      s_size[b] = v;
    }
    __syncthreads();
    if (tid == 0) s_carry += s_warp[31];
    __syncthreads();
  }
  for (int i = tid; i < n_rows; i += blockDim.x) {
    const int pos = slot_of_row[i];
    if (pos >= 0) row_of_slot[s_count[bucket_of(i)] + pos] = i;
  }
  __syncthreads();
  for (int i = tid; i < n_rows; i += blockDim.x) {
    if (slot_of_row[i] < 0) continue;
    const int b = bucket_of(i);
    const int first = s_count[b], size = s_size[b];
    int rank = 0;
    for (int k = 0; k < size; k++) rank += (row_of_slot[first + k] < i);
    slot_of_row[i] = first + rank;
  }
  __syncthreads();
  for (int i = tid; i < n_rows; i += blockDim.x) {
    const int s = slot_of_row[i];
    if (s < 0) continue;
    row_of_slot[s] = i;
    // row i came from rank i / rows_per_block; its result goes to the same place of that rank's block
    if (out_ptr_of_slot != nullptr)
      out_ptr_of_slot[s] = out_blocks[i / rows_per_block] + (unsigned long long)(i % rows_per_block) * out_row_bytes;
  }
}

// One CTA, one thread per rank.  Thread p raises flag [channel][rank] in rank p's flag block (waiting
// first, if need be, until the flag of the previous round was taken) and then takes flag [channel][p]
// from this rank's own block.  Before the flags all earlier stores of this GPU (rows written into
// peers' memory by the kernels launched before) are made visible system-wide.  Both waits end after
// `limit_ns`: the kernel then adds 1 to *status and returns, and the exchange buffers must not be
// trusted any more.
__global__ void k_peer_barrier(int32_t *const *__restrict__ flag_blocks, int rank, int n_ranks, int channel,
                               unsigned long long limit_ns, int *status) {
  const int p = threadIdx.x;
  __threadfence_system();
  if (p < n_ranks && p != rank) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    auto expired = [&]() {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      return t - t0 > limit_ns;
    };
    int32_t *theirs = flag_blocks[p] + channel * n_ranks + rank;
    int32_t *mine = flag_blocks[rank] + channel * n_ranks + p;
    bool ok = true;
    while (atomicCAS_system(theirs, 0, 1) != 0) {
      if (expired()) {
        ok = false;
        break;
      }
      __nanosleep(200);
    }
    while (ok && atomicCAS_system(mine, 1, 0) != 1) {
      if (expired()) {
        ok = false;
        break;
      }
      __nanosleep(100);
    }
    if (!ok) atomicAdd(status, 1);
  }
  __threadfence_system();
}

int launch_ep_dispatch(const int32_t *choice, const void *hidden, int64_t hidden_stride, int32_t *expert,
                       int32_t *dest, int32_t *slot, void *send, void *const *blocks, int *overflow, int n_tokens,
                       int n_experts, int local_experts, int seq_len, int capacity, int n_ranks, int cap, int d_model,
                       cudaStream_t stream) {
  const int n_slots = n_ranks * cap;
  const long long row_stride = d_model + 8;
  const int threads = 256;
  const long long n = (long long)n_tokens * 32 > n_slots ? (long long)n_tokens * 32 : n_slots;
  QMOE_LAUNCH(k_ep_keep, (unsigned)((n + threads - 1) / threads), threads, 0, stream, choice, expert, dest, n_tokens, n_experts,
              local_experts, seq_len, capacity, reinterpret_cast<__nv_bfloat16 *>(send),
              reinterpret_cast<__nv_bfloat16 *const *>(blocks), cap > 0 ? cap : 1, n_slots, row_stride, d_model);
  QMOE_CUDA(cudaGetLastError());
  if (n_tokens > 0) {
    QMOE_LAUNCH(k_ep_pack, n_tokens, 128, 0, stream, expert, dest, reinterpret_cast<const __nv_bfloat16 *>(hidden),
                (long long)hidden_stride, reinterpret_cast<__nv_bfloat16 *>(send),
                reinterpret_cast<__nv_bfloat16 *const *>(blocks), row_stride, slot, overflow, d_model, local_experts, cap);
    QMOE_CUDA(cudaGetLastError());
  }
  return QMOE_OK;
}

int launch_ep_plan(const void *rows, int64_t row_stride, int d_model, const int32_t *meta, int n_rows, int n_buckets,
                   int32_t *offsets, int32_t *slot_of_row, int32_t *row_of_slot, const uint64_t *out_blocks,
                   int rows_per_block, int64_t out_row_bytes, uint64_t *out_ptr_of_slot, cudaStream_t stream) {
  QMOE_LAUNCH(k_ep_plan, 1, 1024, 2 * sizeof(int) * (size_t)n_buckets, stream,
              reinterpret_cast<const __nv_bfloat16 *>(rows), (long long)row_stride, d_model, meta, n_rows, n_buckets,
              offsets, slot_of_row, row_of_slot, reinterpret_cast<const unsigned long long *>(out_blocks),
              rows_per_block > 0 ? rows_per_block : 1, (long long)out_row_bytes,
              reinterpret_cast<unsigned long long *>(out_ptr_of_slot));
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_peer_barrier(int32_t *const *flag_blocks, int rank, int n_ranks, int channel, uint64_t limit_ns,
                        int *status, cudaStream_t stream) {
  QMOE_LAUNCH(k_peer_barrier, 1, (unsigned)((n_ranks + 31) / 32 * 32), 0, stream, flag_blocks, rank, n_ranks, channel,
              (unsigned long long)limit_ns, status);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
