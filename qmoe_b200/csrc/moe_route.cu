// Routing, grouping and combine kernels of the top-1 MoE layer (FasterMLP.forward, sub1.py:306-321,
// around the Switch router the reference calls at sub1.py:310).  Everything stays on the device: no
// nonzero(), no boolean-mask indexing, no host synchronisation.
#include "common.cuh"

namespace qmoe {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_min(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One warp per token.  softmax in fp32, probabilities rounded to bf16, first index of the largest
// bf16 probability (argmax over the bf16 probabilities, as the router does after its dtype cast).
__global__ void k_route_choose(const float *__restrict__ logits, int32_t *__restrict__ choice,
                               __nv_bfloat16 *__restrict__ prob, int n_tokens, int n_experts) {
  const int token = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (token >= n_tokens) return;
  const float *l = logits + (size_t)token * n_experts;
  float m = -INFINITY;
  for (int i = lane; i < n_experts; i += 32) m = fmaxf(m, l[i]);
  m = warp_max(m);
  float s = 0.f;
  for (int i = lane; i < n_experts; i += 32) s += expf(l[i] - m);
  s = warp_sum(s);
  const __nv_bfloat16 pmax = __float2bfloat16_rn(1.f / s);
  const unsigned short pmax_bits = __bfloat16_as_ushort(pmax);
  int first = n_experts;
  for (int i = lane; i < n_experts; i += 32) {
    const __nv_bfloat16 p = __float2bfloat16_rn(expf(l[i] - m) / s);
    if (__bfloat16_as_ushort(p) >= pmax_bits && i < first) first = i;
  }
  first = warp_min(first);
  if (lane == 0) {
    choice[token] = first < n_experts ? first : 0;
    prob[token] = pmax;
  }
}

// The same by a whole CTA of 256 threads, for the few tokens of a decode step (a single warp
// walking 2048 logits three times is pure latency).  Every thread returns the result.
__device__ __forceinline__ void route_token_block(const float *__restrict__ l, int n_experts, float *s_f, int *s_i,
                                                  int &first_out, __nv_bfloat16 &pmax_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float m = -INFINITY;
  for (int i = tid; i < n_experts; i += 256) m = fmaxf(m, l[i]);
  m = warp_max(m);
  __syncthreads();  // s_f / s_i may still be read from the previous token
  if (lane == 0) s_f[warp] = m;
  __syncthreads();
  m = s_f[0];
  for (int w = 1; w < 8; w++) m = fmaxf(m, s_f[w]);
  __syncthreads();
  float s = 0.f;
  for (int i = tid; i < n_experts; i += 256) s += expf(l[i] - m);
  s = warp_sum(s);
  if (lane == 0) s_f[warp] = s;
  __syncthreads();
  s = 0.f;
  for (int w = 0; w < 8; w++) s += s_f[w];
  const __nv_bfloat16 pmax = __float2bfloat16_rn(1.f / s);
  const unsigned short pmax_bits = __bfloat16_as_ushort(pmax);
  int first = n_experts;
  for (int i = tid; i < n_experts; i += 256) {
    const __nv_bfloat16 p = __float2bfloat16_rn(expf(l[i] - m) / s);
    if (__bfloat16_as_ushort(p) >= pmax_bits && i < first) first = i;
  }
  first = warp_min(first);
  if (lane == 0) s_i[warp] = first;
  __syncthreads();
  first = s_i[0];
  for (int w = 1; w < 8; w++) first = min(first, s_i[w]);
  first_out = first < n_experts ? first : 0;
  pmax_out = pmax;
}

__global__ void __launch_bounds__(256) k_route_choose_block(const float *__restrict__ logits,
                                                            int32_t *__restrict__ choice,
                                                            __nv_bfloat16 *__restrict__ prob, int n_experts) {
  __shared__ float s_f[8];
  __shared__ int s_i[8];
  int first;
  __nv_bfloat16 pmax;
  route_token_block(logits + (size_t)blockIdx.x * n_experts, n_experts, s_f, s_i, first, pmax);
  if (threadIdx.x == 0) {
    choice[blockIdx.x] = first;
    prob[blockIdx.x] = pmax;
  }
}

// Route, capacity rule, stable ranks, bucket offsets and the permutation of the rows, for at most
// 32 tokens of one sequence, in one launch of one CTA: what k_route_choose, k_capacity, k_rank,
// k_exclusive_scan and k_permute do for a full layer, for the single-token steps of generation.
constexpr int kSmallTokens = 32;
__global__ void __launch_bounds__(256) k_route_small(const float *__restrict__ logits,
                                                     const __nv_bfloat16 *__restrict__ hidden, int n_tokens,
                                                     int n_experts, int d_model, int capacity,
                                                     __nv_bfloat16 *__restrict__ prob, int32_t *__restrict__ offsets,
                                                     int32_t *__restrict__ slot, __nv_bfloat16 *__restrict__ xs) {
  __shared__ float s_f[8];
  __shared__ int s_i[8];
  __shared__ int s_choice[kSmallTokens], s_rank[kSmallTokens], s_slot[kSmallTokens];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int t = 0; t < n_tokens; t++) {
    int first;
    __nv_bfloat16 pmax;
    route_token_block(logits + (size_t)t * n_experts, n_experts, s_f, s_i, first, pmax);
    if (tid == 0) {
      s_choice[t] = first;
      prob[t] = pmax;
    }
  }
  __syncthreads();
  if (tid < n_tokens) {
    int before = 0;
    for (int u = 0; u < tid; u++) before += (s_choice[u] == s_choice[tid]);
    s_rank[tid] = before < capacity ? before : -1;  // -1: dropped by the capacity rule
  }
  if (tid == 0) s_carry = 0;
  __syncthreads();
  // offsets = exclusive prefix sum over the experts of their kept tokens
  for (int e0 = 0; e0 < n_experts; e0 += 256) {
    const int e = e0 + tid;
    int count = 0;
    if (e < n_experts)
      for (int t = 0; t < n_tokens; t++) count += (s_choice[t] == e && s_rank[t] >= 0);
    int incl = count;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    if (lane == 31) s_i[warp] = incl;
    __syncthreads();
    int base = s_carry;
    for (int w = 0; w < warp; w++) base += s_i[w];
    if (e < n_experts) offsets[e] = base + incl - count;
    if (e < n_experts && count > 0) {
      for (int t = 0; t < n_tokens; t++)
        if (s_choice[t] == e && s_rank[t] >= 0) s_slot[t] = base + incl - count + s_rank[t];
    }
    __syncthreads();
    if (tid == 255) s_carry = base + incl;
    __syncthreads();
  }
  if (tid == 0) offsets[n_experts] = s_carry;
  if (tid < n_tokens) {
    if (s_rank[tid] < 0) s_slot[tid] = -1;
    slot[tid] = s_slot[tid];
  }
  __syncthreads();
  for (int t = 0; t < n_tokens; t++) {
    const int sl = s_slot[t];
    if (sl < 0) continue;
    for (int i = tid; i < d_model; i += 256) xs[(size_t)sl * d_model + i] = hidden[(size_t)t * d_model + i];
  }
}

// Capacity rule: kept iff fewer than `capacity` earlier tokens of the same sequence chose the same
// expert (cumsum(one_hot, dim=-2) <= expert_capacity in the router).
// One warp per token: the lanes share out the earlier tokens of the sequence.
__global__ void k_capacity(const int32_t *__restrict__ choice, int32_t *__restrict__ bucket, int n_tokens,
                           int n_buckets, int seq_len, int capacity) {
  const int t = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  const int c = choice[t];
  int keep = c >= 0 && c < n_buckets;
  if (keep && capacity < seq_len) {
    const int s0 = (t / seq_len) * seq_len;
    int before = 0;
    for (int u = s0 + lane; u < t; u += 32) before += (choice[u] == c);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    keep = before < capacity;
  }
  if (lane == 0) bucket[t] = keep ? c : -1;
}

// rank[t] = number of earlier tokens in the same bucket; counts[b] = bucket sizes.  O(n^2) compares,
// all lanes of a warp reading the same address: a few microseconds for the thousands of tokens a
// layer sees, and the order is the token order by construction.
__global__ void k_rank(const int32_t *__restrict__ bucket, int32_t *__restrict__ rank,
                       int32_t *__restrict__ counts, int n_tokens) {
  __shared__ int s_b[1024];
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = t < n_tokens ? bucket[t] : -1;
  int before = 0;
  const int t_end = min(n_tokens, (int)((blockIdx.x + 1) * blockDim.x));
  for (int u0 = 0; u0 < t_end; u0 += blockDim.x) {
    const int u = u0 + threadIdx.x;
    __syncthreads();
    s_b[threadIdx.x] = u < n_tokens ? bucket[u] : -1;
    __syncthreads();
    const int lim = min((int)blockDim.x, t - u0);
    if (b >= 0) {
      for (int k = 0; k < lim; k++) before += (s_b[k] == b);
    }
  }
  if (t < n_tokens) {
    rank[t] = before;
    if (b >= 0) atomicAdd(counts + b, 1);
  }
}

__global__ void __launch_bounds__(1024) k_exclusive_scan(const int32_t *__restrict__ counts,
                                                         int32_t *__restrict__ offsets, int n) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_carry = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {
    const int i = i0 + tid;
    const int v = i < n ? counts[i] : 0;
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
    const int excl = s_carry + (warp ? s_warp[warp - 1] : 0) + incl - v;
    if (i < n) offsets[i] = excl;
    __syncthreads();
    if (tid == 0) s_carry += s_warp[31];
    __syncthreads();
  }
  if (tid == 0) offsets[n] = s_carry;
}

__device__ __forceinline__ void copy_row_bf16(const __nv_bfloat16 *__restrict__ src,
                                              __nv_bfloat16 *__restrict__ dst, int n) {
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0 && (n & 7) == 0) {
    const uint4 *s = reinterpret_cast<const uint4 *>(src);
    uint4 *d = reinterpret_cast<uint4 *>(dst);
    for (int i = threadIdx.x; i < n / 8; i += blockDim.x) d[i] = s[i];
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
}

// One CTA per token: slot = offsets[bucket] + rank, xs[slot] = hidden[token].
__global__ void k_permute(const int32_t *__restrict__ bucket, const int32_t *__restrict__ rank,
                          const int32_t *__restrict__ offsets, int32_t *__restrict__ slot,
                          const __nv_bfloat16 *__restrict__ hidden, __nv_bfloat16 *__restrict__ xs, int d_model,
                          long long hidden_stride, long long xs_stride) {
  const int t = blockIdx.x;
  const int b = bucket[t];
  const int s = b >= 0 ? offsets[b] + rank[t] : -1;
  if (threadIdx.x == 0) slot[t] = s;
  if (s >= 0) copy_row_bf16(hidden + (size_t)t * hidden_stride, xs + (size_t)s * xs_stride, d_model);
}

__global__ void k_unpermute(const __nv_bfloat16 *__restrict__ ys, const int32_t *__restrict__ slot,
                            __nv_bfloat16 *__restrict__ out, int d_model, long long ys_stride,
                            long long out_stride) {
  const int t = blockIdx.x;
  const int s = slot[t];
  __nv_bfloat16 *dst = out + (size_t)t * out_stride;
  if (s >= 0) {
    copy_row_bf16(ys + (size_t)s * ys_stride, dst, d_model);
  } else {
    for (int i = threadIdx.x; i < d_model; i += blockDim.x) dst[i] = __float2bfloat16_rn(0.f);
  }
}

// out[t] = bf16(prob[t] * (slot >= 0 ? ys[slot] : hidden[t]))   (sub1.py:312,317-318)
__global__ void k_combine(const __nv_bfloat16 *__restrict__ ys, const __nv_bfloat16 *__restrict__ hidden,
                          const int32_t *__restrict__ slot, const __nv_bfloat16 *__restrict__ prob,
                          __nv_bfloat16 *__restrict__ out, int d_model) {
  const int t = blockIdx.x;
  const int s = slot[t];
  const float p = __bfloat162float(prob[t]);
  const __nv_bfloat16 *src = s >= 0 ? ys + (size_t)s * d_model : hidden + (size_t)t * d_model;
  __nv_bfloat16 *dst = out + (size_t)t * d_model;
  if ((d_model & 7) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
    for (int i = threadIdx.x; i < d_model / 8; i += blockDim.x) {
      uint4 v = reinterpret_cast<const uint4 *>(src)[i];
      __nv_bfloat16 *h = reinterpret_cast<__nv_bfloat16 *>(&v);
#pragma unroll
      for (int k = 0; k < 8; k++) h[k] = __float2bfloat16_rn(p * __bfloat162float(h[k]));
      reinterpret_cast<uint4 *>(dst)[i] = v;
    }
    return;
  }
  for (int i = threadIdx.x; i < d_model; i += blockDim.x)
    dst[i] = __float2bfloat16_rn(p * __bfloat162float(src[i]));
}

// out[t] = bf16(residual[t] + bf16(prob[t] * (slot >= 0 ? ys[slot] : hidden[t]))): k_combine followed
// by the block's residual addition in bf16.
__global__ void k_combine_add(const __nv_bfloat16 *__restrict__ ys, const __nv_bfloat16 *__restrict__ hidden,
                              const int32_t *__restrict__ slot, const __nv_bfloat16 *__restrict__ prob,
                              const __nv_bfloat16 *__restrict__ residual, __nv_bfloat16 *__restrict__ out,
                              int d_model) {
  const int t = blockIdx.x;
  const int s = slot[t];
  const float p = __bfloat162float(prob[t]);
  const __nv_bfloat16 *src = s >= 0 ? ys + (size_t)s * d_model : hidden + (size_t)t * d_model;
  for (int i = threadIdx.x; i < d_model; i += blockDim.x) {
    const float moe = __bfloat162float(__float2bfloat16_rn(p * __bfloat162float(src[i])));
    out[(size_t)t * d_model + i] = __float2bfloat16_rn(__bfloat162float(residual[(size_t)t * d_model + i]) + moe);
  }
}

// ---- launchers ----------------------------------------------------------------------------------
int launch_route(const float *logits, int32_t *choice, void *prob, int n_tokens, int n_experts,
                 cudaStream_t stream) {
  if (n_tokens == 0) return QMOE_OK;
  // A CTA per token for wide routers (a warp walking 2048 logits three times is latency: 9.7 us
  // for 256 tokens); the choice of kernel depends on the router's width only, so that a token gets
  // the same probability bits whatever batch it arrives in.
  if (n_experts >= 512) {
    QMOE_LAUNCH(k_route_choose_block, (unsigned)n_tokens, 256, 0, stream, logits, choice,
                reinterpret_cast<__nv_bfloat16 *>(prob), n_experts);
    QMOE_CUDA(cudaGetLastError());
    return QMOE_OK;
  }
  const int threads = 128;
  const long long total = (long long)n_tokens * 32;
  QMOE_LAUNCH(k_route_choose, (unsigned)((total + threads - 1) / threads), threads, 0, stream, logits, choice, reinterpret_cast<__nv_bfloat16 *>(prob), n_tokens, n_experts);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_rank(const int32_t *choice, int32_t *bucket, int32_t *rank, int32_t *counts, int n_tokens,
                int n_buckets, int seq_len, int capacity, cudaStream_t stream) {
  QMOE_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * (size_t)n_buckets, stream));
  if (n_tokens == 0) return QMOE_OK;
  const int threads = 256;
  const int blocks = (n_tokens + threads - 1) / threads;
  QMOE_LAUNCH(k_capacity, (unsigned)(((long long)n_tokens * 32 + threads - 1) / threads), threads, 0, stream, choice,
              bucket, n_tokens, n_buckets, seq_len, capacity);
  QMOE_CUDA(cudaGetLastError());
  QMOE_LAUNCH(k_rank, blocks, threads, 0, stream, bucket, rank, counts, n_tokens);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_keep(const int32_t *choice, int32_t *expert, int n_tokens, int n_experts, int seq_len, int capacity,
                cudaStream_t stream) {
  const int threads = 256;
  QMOE_LAUNCH(k_capacity, (unsigned)(((long long)n_tokens * 32 + threads - 1) / threads), threads, 0, stream, choice,
              expert, n_tokens, n_experts, seq_len, capacity);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_scan(const int32_t *counts, int32_t *offsets, int n, cudaStream_t stream) {
  QMOE_LAUNCH(k_exclusive_scan, 1, 1024, 0, stream, counts, offsets, n);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_permute(const int32_t *bucket, const int32_t *rank, const int32_t *offsets, int32_t *slot,
                   const void *hidden, void *xs, int n_tokens, int d_model, int64_t hidden_stride,
                   int64_t xs_stride, cudaStream_t stream) {
  if (n_tokens == 0) return QMOE_OK;
  QMOE_LAUNCH(k_permute, n_tokens, 128, 0, stream, bucket, rank, offsets, slot, reinterpret_cast<const __nv_bfloat16 *>(hidden), reinterpret_cast<__nv_bfloat16 *>(xs), d_model, hidden_stride, xs_stride);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_unpermute(const void *ys, const int32_t *slot, void *out, int n_tokens, int d_model,
                     int64_t ys_stride, int64_t out_stride, cudaStream_t stream) {
  if (n_tokens == 0) return QMOE_OK;
  QMOE_LAUNCH(k_unpermute, n_tokens, 128, 0, stream, reinterpret_cast<const __nv_bfloat16 *>(ys), slot, reinterpret_cast<__nv_bfloat16 *>(out), d_model, ys_stride, out_stride);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_combine(const void *ys, const void *hidden, const int32_t *slot, const void *prob, void *out,
                   int n_tokens, int d_model, cudaStream_t stream) {
  QMOE_LAUNCH(k_combine, n_tokens, 128, 0, stream, reinterpret_cast<const __nv_bfloat16 *>(ys), reinterpret_cast<const __nv_bfloat16 *>(hidden), slot, reinterpret_cast<const __nv_bfloat16 *>(prob), reinterpret_cast<__nv_bfloat16 *>(out), d_model);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_route_small(const float *logits, const void *hidden, int n_tokens, int n_experts, int d_model,
                       int capacity, void *prob, int32_t *offsets, int32_t *slot, void *xs, cudaStream_t stream) {
  QMOE_LAUNCH(k_route_small, 1, 256, 0, stream, logits, reinterpret_cast<const __nv_bfloat16 *>(hidden), n_tokens,
              n_experts, d_model, capacity, reinterpret_cast<__nv_bfloat16 *>(prob), offsets, slot,
              reinterpret_cast<__nv_bfloat16 *>(xs));
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_combine_add(const void *ys, const void *hidden, const int32_t *slot, const void *prob,
                       const void *residual, void *out, int n_tokens, int d_model, cudaStream_t stream) {
  QMOE_LAUNCH(k_combine_add, n_tokens, 256, 0, stream, reinterpret_cast<const __nv_bfloat16 *>(ys),
              reinterpret_cast<const __nv_bfloat16 *>(hidden), slot, reinterpret_cast<const __nv_bfloat16 *>(prob),
              reinterpret_cast<const __nv_bfloat16 *>(residual), reinterpret_cast<__nv_bfloat16 *>(out), d_model);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
