// Encoder kernels: greedy longest-match walk of the dictionary trie over ternary pairs.
// Replaces Sub1PreparePack / Sub1Pack and the host glue of sub1pack_cuda
// (sub1_cuda_kernel.cu:92-126, 211-250).  The greedy walk of one row is a serial chain (the trie
// node after pair i depends on pair i-1), so rows are the unit of parallelism here as well; what
// changes against the reference is that the prefix sum runs on the device, any height is accepted,
// and a batched uint8 variant encodes many matrices per launch without a host round trip.
#include "common.cuh"

namespace qmoe {

__device__ __forceinline__ int trie_next(const int32_t *__restrict__ trie, int node, int pair) {
  return __ldg(trie + 9 * node + pair);
}

// One thread per row; the row's codes overwrite the head of the row (sub1_cuda_kernel.cu:231,236).
__global__ void k_pack_prepare(const int32_t *__restrict__ trie, int32_t *__restrict__ w_tern,
                               int32_t *__restrict__ row_len, int height, int width) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= height) return;
  int32_t *w = w_tern + (size_t)row * width;
  int node = QMOE_TRIE_ROOT;
  int n = 0;
  for (int i = 0; i < width; i += 2) {
    int pair = w[i];  // pair = 3 * second + first (sub1_cuda_kernel.cu:223-228)
    if (i + 1 < width) pair += 3 * w[i + 1];
    pair = min(max(pair, 0), 8);
    int next = trie_next(trie, node, pair);
    if (next < 0) {
      w[n++] = node;
      next = trie_next(trie, QMOE_TRIE_ROOT, pair);
    }
    node = next;
  }
  w[n++] = node;
  row_len[row] = n;
}

// In-place exclusive scan by one CTA: on entry a[1..n] holds the lengths, on exit a[0..n] holds the
// offsets (a[0] = 0).  Replaces row_off.cumsum(0) (sub1_cuda_kernel.cu:112).
__global__ void __launch_bounds__(1024) k_offsets_from_lengths(int32_t *a, int n) {
  __shared__ int s_warp[32];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    s_carry = 0;
    a[0] = 0;
  }
  __syncthreads();
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {
    const int i = i0 + tid;
    const int v = i < n ? a[i + 1] : 0;
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
    const int total = s_carry + (warp ? s_warp[warp - 1] : 0) + incl;
    if (i < n) a[i + 1] = total;
    __syncthreads();
    if (tid == 0) s_carry += s_warp[31];
    __syncthreads();
  }
}

// One warp per row: w_comp[row_off[row] + i] = codes at the head of the row (Sub1Pack, :241-250).
__global__ void k_pack_emit(const int32_t *__restrict__ w_prep, const int32_t *__restrict__ row_off,
                            uint16_t *__restrict__ w_comp, int height, int width) {
  const int row = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= height) return;
  const int off = row_off[row];
  int n = row_off[row + 1] - off;
  n = min(n, (width + 1) / 2);
  const int32_t *src = w_prep + (size_t)row * width;
  for (int i = lane; i < n; i += 32) w_comp[off + i] = (uint16_t)src[i];
}

// Batched uint8 encoder: one thread per row of [n_mat * height]; 16 symbols per load when the row
// is 16-byte aligned.
__global__ void k_pack_u8_count(const int32_t *__restrict__ trie, const uint8_t *__restrict__ sym,
                                uint16_t *__restrict__ codes_tmp, int32_t *__restrict__ row_len,
                                long long n_rows, int width) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n_rows) return;
  const uint8_t *s = sym + (size_t)row * width;
  uint16_t *out = codes_tmp + (size_t)row * (width / 2);
  int node = QMOE_TRIE_ROOT;
  int n = 0;
  auto step = [&](int pair) {
    pair = min(pair, 8);
    int next = trie_next(trie, node, pair);
    if (next < 0) {
      out[n++] = (uint16_t)node;
      next = trie_next(trie, QMOE_TRIE_ROOT, pair);
    }
    node = next;
  };
  int i = 0;
  if ((reinterpret_cast<uintptr_t>(s) & 15u) == 0) {
    for (; i + 16 <= width; i += 16) {
      const uint4 q = __ldg(reinterpret_cast<const uint4 *>(s + i));
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const uint32_t h = (w[k >> 1] >> (16 * (k & 1))) & 0xffffu;
        step((int)((h & 0xffu) + 3u * (h >> 8)));
      }
    }
  }
  for (; i < width; i += 2) step((int)s[i] + 3 * (int)s[i + 1]);
  out[n++] = (uint16_t)node;
  row_len[row] = n;
}

// One warp per row: out[mat_base[m] + row_off[m*(height+1) + r] + i] = codes_tmp[row][i].
__global__ void k_pack_u8_gather(const uint16_t *__restrict__ codes_tmp, const int32_t *__restrict__ row_off,
                                 const int64_t *__restrict__ mat_base, uint16_t *__restrict__ out,
                                 long long n_rows, int height, int width) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const long long m = row / height;
  const int r = (int)(row - m * height);
  const int32_t *ro = row_off + m * (height + 1);
  const int off = ro[r];
  int n = ro[r + 1] - off;
  n = min(max(n, 0), width / 2);
  const uint16_t *src = codes_tmp + (size_t)row * (width / 2);
  uint16_t *dst = out + mat_base[m] + off;
  for (int i = lane; i < n; i += 32) dst[i] = src[i];
}

// Counter-based generator: splitmix64 of (seed, index / 4) yields four 16-bit uniforms; u < t0 -> 0,
// the remaining range is split evenly between 1 and 2.
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void k_synth_ternary(uint8_t *__restrict__ sym, long long count, uint64_t seed,
                                uint64_t first_index, uint32_t t0, uint32_t t1) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // group of 4 symbols
  const long long i0 = g * 4;
  if (i0 >= count) return;
  const uint64_t idx = first_index + (uint64_t)i0;
  // first_index is a multiple of 4, so a group never straddles two hash inputs.
  const uint64_t h = splitmix64(seed * 0xD1342543DE82EF95ull + (idx >> 2));
  uint32_t packed = 0;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const uint32_t u = (uint32_t)(h >> (16 * k)) & 0xffffu;
    const uint32_t s = u < t0 ? 0u : (u < t1 ? 1u : 2u);
    packed |= s << (8 * k);
  }
  if (i0 + 4 <= count && (reinterpret_cast<uintptr_t>(sym + i0) & 3u) == 0) {
    *reinterpret_cast<uint32_t *>(sym + i0) = packed;
  } else {
    for (int k = 0; k < 4 && i0 + k < count; k++) sym[i0 + k] = (uint8_t)(packed >> (8 * k));
  }
}

// ---- launchers ----------------------------------------------------------------------------------
int launch_pack_prepare(const int32_t *trie, int32_t *w_tern, int32_t *row_off, int height, int width,
                        cudaStream_t stream) {
  const int threads = 64;
  QMOE_LAUNCH(k_pack_prepare, (height + threads - 1) / threads, threads, 0, stream, trie, w_tern, row_off + 1, height, width);
  QMOE_CUDA(cudaGetLastError());
  QMOE_LAUNCH(k_offsets_from_lengths, 1, 1024, 0, stream, row_off, height);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_pack_emit(const int32_t *w_tern, const int32_t *row_off, uint16_t *w_comp, int height, int width,
                     cudaStream_t stream) {
  const int threads = 256;
  const long long total = (long long)height * 32;
  QMOE_LAUNCH(k_pack_emit, (unsigned)((total + threads - 1) / threads), threads, 0, stream, w_tern, row_off, w_comp, height, width);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_pack_u8_count(const int32_t *trie, const uint8_t *sym, uint16_t *codes_tmp, int32_t *row_len,
                         int n_mat, int height, int width, cudaStream_t stream) {
  const long long n_rows = (long long)n_mat * height;
  const int threads = 64;
  QMOE_LAUNCH(k_pack_u8_count, (unsigned)((n_rows + threads - 1) / threads), threads, 0, stream, trie, sym, codes_tmp, row_len, n_rows, width);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_pack_u8_gather(const uint16_t *codes_tmp, const int32_t *row_off, const int64_t *mat_base,
                          uint16_t *out, int n_mat, int height, int width, cudaStream_t stream) {
  const long long n_rows = (long long)n_mat * height;
  const int threads = 256;
  const long long total = n_rows * 32;
  QMOE_LAUNCH(k_pack_u8_gather, (unsigned)((total + threads - 1) / threads), threads, 0, stream, codes_tmp, row_off, mat_base, out, n_rows, height, width);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_synth_ternary(uint8_t *sym, int64_t count, uint64_t seed, uint64_t first_index, float p_zero,
                         cudaStream_t stream) {
  if (first_index & 3u) {
    set_error("qmoe_synth_ternary: first_index must be a multiple of 4");
    return QMOE_ERR_INVALID_ARG;
  }
  const uint32_t t0 = (uint32_t)(p_zero * 65536.0 + 0.5);
  const uint32_t t1 = t0 + (65536u - (t0 > 65536u ? 65536u : t0)) / 2u;
  const long long groups = (count + 3) / 4;
  const int threads = 256;
  QMOE_LAUNCH(k_synth_ternary, (unsigned)((groups + threads - 1) / threads), threads, 0, stream, sym, count, seed, first_index, t0, t1);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
