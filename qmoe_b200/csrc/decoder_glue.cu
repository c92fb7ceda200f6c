// Small fused kernels for the batch-1 decode step of the generation harness (decoder.py).  The
// reference leaves these parts to HuggingFace's Switch Transformers modules (called through
// model.generate at sub1.py:373-379); at one token per step they are pure launch overhead, so each
// group of element-wise torch kernels becomes one launch here.
#include "common.cuh"

namespace qmoe {

constexpr int kMaxHeadDim = 256;
constexpr int kAttentionThreads = 1024;  // 32 warps share the cached positions of a head

__device__ __forceinline__ float block_sum(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarps; w++) t += scratch[w];
  return t;
}

__device__ __forceinline__ float block_max(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = scratch[0];
  for (int w = 1; w < nwarps; w++) t = fmaxf(t, scratch[w]);
  return t;
}

// out[r] = bf16(bf16(x[r] * rsqrt(mean(x[r]^2) + eps)) * w), one CTA per row: the T5 layer norm
// (no mean subtraction, no bias) with the roundings of its bf16 torch formulation.
__global__ void k_rms_norm(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ w,
                           __nv_bfloat16 *__restrict__ out, int d, float eps) {
  __shared__ float scratch[32];
  const __nv_bfloat16 *row = x + (size_t)blockIdx.x * d;
  float ss = 0.f;
  if ((d & 1) == 0 && (reinterpret_cast<uintptr_t>(row) & 3u) == 0) {
    const __nv_bfloat162 *row2 = reinterpret_cast<const __nv_bfloat162 *>(row);
    for (int i = threadIdx.x; i < d / 2; i += blockDim.x) {
      const float2 v = __bfloat1622float2(row2[i]);
      ss += v.x * v.x + v.y * v.y;
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float v = __bfloat162float(row[i]);
      ss += v * v;
    }
  }
  const float r = rsqrtf(block_sum(ss, scratch) / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float y = __bfloat162float(__float2bfloat16_rn(__bfloat162float(row[i]) * r));
    out[(size_t)blockIdx.x * d + i] = __float2bfloat16_rn(y * __bfloat162float(w[i]));
  }
}

// One new token of causal self-attention, one CTA per head.  qkv: [3][heads][hd] of the token;
// caches: [heads][max_len][hd].  Writes the token's key and value at position *pos, then
// out[head] = softmax(q . K[0..pos] / sqrt(hd)) V[0..pos], fp32 arithmetic, bf16 result.
// Every warp runs a running-maximum softmax over its share of the positions (up to four at a
// time, their key and value rows loaded together) and the warps' partial results are merged once.
template <int J>  // ceil(head_dim / 32): values of a cache row per lane
__global__ void __launch_bounds__(kAttentionThreads) k_decode_attention(const __nv_bfloat16 *__restrict__ qkv,
                                   __nv_bfloat16 *__restrict__ k_cache,
                                   __nv_bfloat16 *__restrict__ v_cache, const long long *__restrict__ pos_ptr,
                                   __nv_bfloat16 *__restrict__ out, int heads, int hd, int max_len,
                                   float scale_in, const float *__restrict__ bias, int *status) {
  extern __shared__ float smem[];
  constexpr int kWarps = kAttentionThreads / 32;
  float *q = smem;                     // hd
  float *partial = smem + hd;          // [kWarps][hd]
  float *part_m = partial + kWarps * hd;  // [kWarps]
  float *part_s = part_m + kWarps;        // [kWarps]
  const int head = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long pos = *pos_ptr;
  if (pos < 0 || pos >= max_len) {
    // With a status word the call is refused (counted, nothing written); without one the position is
    // clamped, which overwrites the last cache slot.
    if (status != nullptr) {
      if (tid == 0 && head == 0) atomicAdd(status, 1);
      return;
    }
    pos = pos < 0 ? 0 : max_len - 1;
  }
  __nv_bfloat16 *kc = k_cache + (size_t)head * max_len * hd;
  __nv_bfloat16 *vc = v_cache + (size_t)head * max_len * hd;
  for (int i = tid; i < hd; i += blockDim.x) {
    q[i] = __bfloat162float(qkv[(size_t)head * hd + i]);
    kc[pos * hd + i] = qkv[(size_t)(heads + head) * hd + i];
    vc[pos * hd + i] = qkv[(size_t)(2 * heads + head) * hd + i];
  }
  __syncthreads();
  // scale_in <= 0: 1 / sqrt(head_dim); T5 / Switch attention is unscaled (scale 1) with a position bias
  const float scale = scale_in > 0.f ? scale_in : rsqrtf((float)hd);
  const float *hb = bias != nullptr ? bias + (size_t)head * max_len : nullptr;  // added to the score of position t
  // 2 * U * J cache values per lane stay in registers (64 registers per thread at 1024 threads)
  constexpr int U = J <= 3 ? 4 : (J <= 4 ? 2 : 1);
  float m = -INFINITY, ssum = 0.f, acc[J];
#pragma unroll
  for (int j = 0; j < J; j++) acc[j] = 0.f;
  for (int t0 = warp * U; t0 <= pos; t0 += kWarps * U) {
    float kv[U][J], vv[U][J];
#pragma unroll
    for (int u = 0; u < U; u++) {
#pragma unroll
      for (int j = 0; j < J; j++) {
        const int i = lane + 32 * j;
        const bool ok = t0 + u <= pos && i < hd;
        kv[u][j] = ok ? __bfloat162float(kc[(size_t)(t0 + u) * hd + i]) : 0.f;
        vv[u][j] = ok ? __bfloat162float(vc[(size_t)(t0 + u) * hd + i]) : 0.f;
      }
    }
    float sc[U], round_max = -INFINITY;
#pragma unroll
    for (int u = 0; u < U; u++) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < J; j++) {
        const int i = lane + 32 * j;
        if (i < hd) d += q[i] * kv[u][j];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      sc[u] = t0 + u <= pos ? d * scale + (hb != nullptr ? hb[t0 + u] : 0.f) : -INFINITY;  // the same in every lane
      round_max = fmaxf(round_max, sc[u]);
    }
    // t0 <= pos: at least one score of the round is finite
    const float m_new = fmaxf(m, round_max);
    const float rescale = __expf(m - m_new);  // 0 on the first round (m = -inf)
    ssum *= rescale;
#pragma unroll
    for (int j = 0; j < J; j++) acc[j] *= rescale;
    m = m_new;
#pragma unroll
    for (int u = 0; u < U; u++) {
      const float p = __expf(sc[u] - m);
      ssum += p;
#pragma unroll
      for (int j = 0; j < J; j++) acc[j] += p * vv[u][j];
    }
  }
#pragma unroll
  for (int j = 0; j < J; j++) {
    const int i = lane + 32 * j;
    if (i < hd) partial[warp * hd + i] = acc[j];
  }
  if (lane == 0) {
    part_m[warp] = m;   // -inf for a warp without positions: weight 0 below
    part_s[warp] = ssum;
  }
  __syncthreads();
  float top = -INFINITY;
  for (int w = 0; w < kWarps; w++) top = fmaxf(top, part_m[w]);
  float denom = 0.f;
  for (int w = 0; w < kWarps; w++) denom += part_s[w] * __expf(part_m[w] - top);
  for (int i = tid; i < hd; i += blockDim.x) {
    float total = 0.f;
    for (int w = 0; w < kWarps; w++) total += partial[w * hd + i] * __expf(part_m[w] - top);
    out[(size_t)head * hd + i] = __float2bfloat16_rn(total / denom);
  }
}

int launch_rms_norm(const void *x, const void *w, void *out, int rows, int d, float eps, cudaStream_t stream) {
  if (rows == 0) return QMOE_OK;
  QMOE_LAUNCH(k_rms_norm, (unsigned)rows, 512, 0, stream, reinterpret_cast<const __nv_bfloat16 *>(x),
              reinterpret_cast<const __nv_bfloat16 *>(w), reinterpret_cast<__nv_bfloat16 *>(out), d, eps);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_decode_attention(const void *qkv, void *k_cache, void *v_cache, const int64_t *pos, void *out,
                            int heads, int hd, int max_len, float scale, const float *bias, int *status,
                            cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)hd + (size_t)(kAttentionThreads / 32) * (hd + 2));
  static bool limit_set[64][kMaxHeadDim / 32 + 1] = {};  // per device and instantiation
  int device = 0;
  QMOE_CUDA(cudaGetDevice(&device));
  const int chunk_count = (hd + 31) / 32;
  auto run = [&](auto kernel) -> int {
    if (device < 64 && !limit_set[device][chunk_count]) {
      QMOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
      limit_set[device][chunk_count] = true;
    } else if (device >= 64) {
      QMOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    }
    QMOE_LAUNCH(kernel, (unsigned)heads, kAttentionThreads, smem, stream, reinterpret_cast<const __nv_bfloat16 *>(qkv),
                reinterpret_cast<__nv_bfloat16 *>(k_cache), reinterpret_cast<__nv_bfloat16 *>(v_cache),
                reinterpret_cast<const long long *>(pos), reinterpret_cast<__nv_bfloat16 *>(out), heads, hd, max_len,
                scale, bias, status);
    QMOE_CUDA(cudaGetLastError());
    return QMOE_OK;
  };
  switch (chunk_count) {
    case 1: return run(k_decode_attention<1>);
    case 2: return run(k_decode_attention<2>);
    case 3: return run(k_decode_attention<3>);
    case 4: return run(k_decode_attention<4>);
    default: return run(k_decode_attention<kMaxHeadDim / 32>);
  }
}

}  // namespace qmoe

namespace qmoe {

// y = W x for one token (a matrix-vector product streams W once: HBM-bound), optionally with the
// T5 RMS norm of x fused in front (every CTA normalises x for itself: 4 KB against the megabytes
// of W it reads) and a residual added behind.  W bf16 [n][k] row-major, k a multiple of 8, rows
// 16-byte aligned; one warp per output row with 128-bit loads; fp32 accumulation.
//   NORM: x := bf16(bf16(x * rsqrt(mean(x^2) + eps)) * ln_w); CTA 0 also stores it to normed_out.
//   F32OUT: y fp32 (router logits, vocabulary logits), else bf16.
//   ADD: y := bf16(residual + y).
constexpr int kGemvThreads = 256;
constexpr int kGemvRowsPerCta = 16;

template <bool NORM, bool F32OUT, bool ADD>
__global__ void __launch_bounds__(kGemvThreads) k_gemv(const __nv_bfloat16 *__restrict__ x,
                                                       const __nv_bfloat16 *__restrict__ ln_w,
                                                       const __nv_bfloat16 *__restrict__ w,
                                                       const __nv_bfloat16 *__restrict__ residual, void *y,
                                                       __nv_bfloat16 *normed_out, int n, int k, float eps) {
  extern __shared__ __align__(16) float xs[];  // k
  __shared__ float scratch[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (NORM) {
    float ss = 0.f;
    for (int i = tid; i < k; i += kGemvThreads) {
      const float v = __bfloat162float(x[i]);
      xs[i] = v;
      ss += v * v;
    }
    const float r = rsqrtf(block_sum(ss, scratch) / (float)k + eps);
    for (int i = tid; i < k; i += kGemvThreads) {
      const __nv_bfloat16 a = __float2bfloat16_rn(xs[i] * r);
      const __nv_bfloat16 b = __float2bfloat16_rn(__bfloat162float(a) * __bfloat162float(ln_w[i]));
      xs[i] = __bfloat162float(b);
      if (blockIdx.x == 0 && normed_out != nullptr) normed_out[i] = b;
    }
  } else {
    for (int i = tid; i < k; i += kGemvThreads) xs[i] = __bfloat162float(x[i]);
  }
  __syncthreads();
  const int row_end = min(n, (int)(blockIdx.x + 1) * kGemvRowsPerCta);
  for (int row0 = blockIdx.x * kGemvRowsPerCta + warp * 2; row0 < row_end; row0 += 2 * (kGemvThreads / 32)) {
    // two rows per warp at a time: twice the loads in flight
    const bool two = row0 + 1 < row_end;
    const uint4 *wa = reinterpret_cast<const uint4 *>(w + (size_t)row0 * k);
    const uint4 *wb = reinterpret_cast<const uint4 *>(w + (size_t)(row0 + (two ? 1 : 0)) * k);
    float sa = 0.f, sb = 0.f;
#pragma unroll 4
    for (int c = lane; c < k / 8; c += 32) {
      const uint4 qa = __ldg(wa + c), qb = __ldg(wb + c);
      const float4 x0 = *reinterpret_cast<const float4 *>(xs + 8 * c);
      const float4 x1 = *reinterpret_cast<const float4 *>(xs + 8 * c + 4);
      const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
      const uint32_t ua[4] = {qa.x, qa.y, qa.z, qa.w}, ub[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        sa += xv[2 * j] * __uint_as_float(ua[j] << 16) + xv[2 * j + 1] * __uint_as_float(ua[j] & 0xffff0000u);
        sb += xv[2 * j] * __uint_as_float(ub[j] << 16) + xv[2 * j + 1] * __uint_as_float(ub[j] & 0xffff0000u);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sa += __shfl_xor_sync(0xffffffffu, sa, o);
      sb += __shfl_xor_sync(0xffffffffu, sb, o);
    }
    if (lane < (two ? 2 : 1)) {
      const int row = row0 + lane;
      float v = lane == 0 ? sa : sb;
      if (ADD) v = __bfloat162float(residual[row]) + __bfloat162float(__float2bfloat16_rn(v));
      if (F32OUT) reinterpret_cast<float *>(y)[row] = v;
      else reinterpret_cast<__nv_bfloat16 *>(y)[row] = __float2bfloat16_rn(v);
    }
  }
}

int launch_gemv(const void *x, const void *ln_w, const void *w, const void *residual, void *y, void *normed_out,
                int n, int k, float eps, int f32_out, cudaStream_t stream) {
  const unsigned grid = (unsigned)((n + kGemvRowsPerCta - 1) / kGemvRowsPerCta);
  const size_t smem = sizeof(float) * (size_t)k;
  const __nv_bfloat16 *xb = reinterpret_cast<const __nv_bfloat16 *>(x), *lb = reinterpret_cast<const __nv_bfloat16 *>(ln_w);
  const __nv_bfloat16 *wb = reinterpret_cast<const __nv_bfloat16 *>(w), *rb = reinterpret_cast<const __nv_bfloat16 *>(residual);
  __nv_bfloat16 *nb = reinterpret_cast<__nv_bfloat16 *>(normed_out);
  if (ln_w != nullptr && f32_out)
    QMOE_LAUNCH((k_gemv<true, true, false>), grid, kGemvThreads, smem, stream, xb, lb, wb, rb, y, nb, n, k, eps);
  else if (ln_w != nullptr)
    QMOE_LAUNCH((k_gemv<true, false, false>), grid, kGemvThreads, smem, stream, xb, lb, wb, rb, y, nb, n, k, eps);
  else if (residual != nullptr)
    QMOE_LAUNCH((k_gemv<false, false, true>), grid, kGemvThreads, smem, stream, xb, lb, wb, rb, y, nb, n, k, eps);
  else if (f32_out)
    QMOE_LAUNCH((k_gemv<false, true, false>), grid, kGemvThreads, smem, stream, xb, lb, wb, rb, y, nb, n, k, eps);
  else
    QMOE_LAUNCH((k_gemv<false, false, false>), grid, kGemvThreads, smem, stream, xb, lb, wb, rb, y, nb, n, k, eps);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
