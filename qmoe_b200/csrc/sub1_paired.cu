// Grouped decode-matvec for stores that carry a paired-lane copy of their code streams: the kernel
// behind qmoe_moe_grouped_ffn for a whole MoE layer per launch.  Replaces Sub1MatVec
// (sub1_cuda_kernel.cu:129-202) and the per-expert, per-token launch loop around it
// (sub1.py:139-142,315-317).
//
// What limits a decode-matvec on this GPU is not HBM but the SM itself: every 2-byte code costs one
// random dictionary lookup, up to three random gathers from the activation vector and the
// instructions around them, and both the instruction issue slots and the shared-memory pipe fill up
// long before the memory system does.  The design therefore minimises instructions per code:
//
//  * one THREAD per row, up to 1024 rows per CTA, one persistent CTA per SM, a work list of (matrix,
//    row block, group of up to four tokens) items; the activations of the item's tokens sit in
//    shared memory interleaved by token, so one decode serves up to four tokens;
//  * the store's streams are re-tokenised when the copy is built: the 40 447 most frequent dictionary
//    entries are renumbered 0 .. 40 446 and sit in shared memory (4 bytes each); every rarer code is
//    replaced by the two or three frequent codes whose sequences concatenate to its own (the
//    dictionary contains the prefixes and suffixes of its entries), so there is no second, slower
//    lookup path and no range test;
//  * two codes per 32-bit word, word k of row l of a 32-row block at index k * 32 + l (a warp's stream
//    loads are 128 contiguous bytes), every row of a block padded with a null code to the block's
//    longest row: the 32 lanes of a warp run the same number of iterations, so the loop has no
//    divergence and no per-code bounds test;
//  * a table entry is laid out so that every field costs two or three instructions: the digits of
//    its (at most three) non-zeros are 2-bit fields that one multiply-add turns into the selector of
//    a byte permute, which picks the row's min or max out of the packed bf16 pair, and one compare
//    of the same field predicates the gather and its multiply-adds away where there is no non-zero
//    (a gather that is not issued cannot collide with another lane's in a shared-memory bank).
//
// The copy decodes to exactly the same weights as the reference's streams (tested bit for bit); the
// reference's tensors stay what the C ABI takes and what checkpoints hold.
#include "common.cuh"

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

namespace qmoe {

constexpr int kPairedThreads = 1024;
constexpr int kPairedTab = QMOE_PAIRED_TABLE;            // table entries in shared memory, the last one null
constexpr uint32_t kPairedNull = kPairedTab - 1;
constexpr uint32_t kPairedNullWord = kPairedNull | (kPairedNull << 16);
// The kernel requests stream words without a range test, three words ahead of the one it consumes,
// and prefetches into L2 kPairedPrefetch words ahead: the copy ends with this many null words.
constexpr int kPairedPrefetch = 8;
constexpr int kPairedTailWords = (kPairedPrefetch + 4) * 32;
static_assert(kPairedTailWords == QMOE_PAIRED_TAIL_WORDS, "the header promises this many null words");
// A code advances the position by at most 28 weights and the position is clamped once per word (two
// codes), so the activations in shared memory are followed by this many zero columns.
constexpr int kPairedPad = 2 * 28 + 32;

// Table entry of this kernel, laid out for the fewest instructions in its inner loop:
//   bits  0..1   digit of the first non-zero: 0 = row min, 1 = row max, 2 = there is none
//   bits  2..6   its position (0..27) inside the code
//   bits  7..8   digit of the second non-zero, bits 9..10 of the third
//   bits 11..15  position of the second, bits 16..20 of the third
//   bits 21..25  weights the code covers (2 * length in pairs, 2..28)
// The null entry (covers nothing, contributes nothing) has the three digits 2 and zeros elsewhere.
constexpr uint32_t kPairedNullEntry = 2u | (2u << 7) | (2u << 9);
__host__ __device__ inline uint32_t paired_entry_digit(uint32_t e, int k) {  // 1 / 2 as in the reference, 0 = none
  const uint32_t d = (e >> (k == 0 ? 0 : (5 + 2 * k))) & 3u;
  return d == 2u ? 0u : d + 1u;
}
__host__ __device__ inline uint32_t paired_entry_pos(uint32_t e, int k) {
  return (e >> (k == 0 ? 2 : (6 + 5 * k))) & 31u;
}
__host__ __device__ inline uint32_t paired_entry_weights(uint32_t e) { return (e >> 21) & 31u; }

__host__ __device__ inline uint32_t paired_entry_from_words(uint32_t w0, uint32_t w1, bool *ok) {
  const int len = (int)(w0 & 15u);
  *ok = len >= 1 && len <= 14 && (int)(w1 & 15u) == len;
  uint32_t e = kPairedNullEntry | ((uint32_t)(2 * len) << 21);
  int nz = 0;
  for (int t = 0; t < 28; t++) {
    const uint32_t w = t < 14 ? w0 : w1;
    const uint32_t digit = (w >> (4 + 2 * (t % 14))) & 3u;
    if (digit == 0u) continue;
    if (t >= 2 * len || digit == 3u || nz == 3) {
      *ok = false;
      return kPairedNullEntry;
    }
    const int dshift = nz == 0 ? 0 : (5 + 2 * nz), pshift = nz == 0 ? 2 : (6 + 5 * nz);
    e &= ~(3u << dshift);
    e |= (digit - 1u) << dshift;
    e |= (uint32_t)t << pshift;
    nz++;
  }
  return *ok ? e : kPairedNullEntry;
}

// ---- host side: renumbering, tables and the replacement lists of rare codes ------------------------
// dec: the reference table (host copy); hist: how often each code occurs in a sample of the store.
// Outputs (host vectors): remap[code] = new number; hot_tab[kPairedTab]; tab_v1[65536] = the 4-byte
// table of the row-per-warp kernel in the new numbering (null at kPairedNull); split_off / split_codes:
// code c of the reference stream becomes split_codes[split_off[c] .. split_off[c + 1]).
// Returns false when the table cannot be served by this kernel (an entry with more than three
// non-zeros, or a rare code that cannot be cut into frequent ones).
static bool paired_plan(const int32_t *dec, const uint64_t *hist, std::vector<uint32_t> &remap,
                      std::vector<uint32_t> &hot_tab, std::vector<uint32_t> &tab_v1,
                      std::vector<uint32_t> &split_off, std::vector<uint16_t> &split_codes) {
  const int N = QMOE_DICT_COUNT;
  std::vector<std::string> seq((size_t)N);
  std::vector<uint32_t> paired_entry((size_t)N);
  std::unordered_map<std::string, int> by_seq;
  by_seq.reserve((size_t)N * 2);
  for (int c = 0; c < N; c++) {
    const uint32_t w0 = (uint32_t)dec[2 * c], w1 = (uint32_t)dec[2 * c + 1];
    bool ok;
    paired_entry[c] = paired_entry_from_words(w0, w1, &ok);
    if (!ok) return false;
    const int len = (int)(w0 & 15u);
    std::string s((size_t)len, '\0');
    for (int j = 0; j < len; j++) {
      const uint32_t nib = ((j < 7 ? w0 : w1) >> (4 + 4 * (j % 7))) & 15u;
      s[(size_t)j] = (char)((nib & 3u) + 3u * (nib >> 2));
    }
    seq[c] = s;
    by_seq.emplace(s, c);  // the first code of a sequence wins
  }
  // Most frequent first; the one-pair codes are kept among the frequent ones whatever their count,
  // so that every sequence can be cut into frequent codes.
  std::vector<int> order((size_t)N);
  for (int c = 0; c < N; c++) order[c] = c;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
    const bool fa = seq[a].size() == 1, fb = seq[b].size() == 1;
    if (fa != fb) return fa;
    return hist[a] > hist[b];
  });
  remap.assign((size_t)N, 0u);
  for (int r = 0; r < N; r++) remap[order[r]] = (uint32_t)r;
  const uint32_t n_hot = kPairedNull;  // numbers 0 .. n_hot - 1 are served from shared memory

  hot_tab.assign((size_t)kPairedTab, kPairedNullEntry);
  tab_v1.assign((size_t)N, kEntryNull);
  for (int c = 0; c < N; c++) {
    const uint32_t r = remap[c];
    if (r < n_hot) hot_tab[r] = paired_entry[c];
    // 4-byte form of common.cuh for the row-per-warp kernel
    const uint32_t e = paired_entry[c];
    uint32_t v1 = kEntryNull | (paired_entry_weights(e) >> 1);
    for (int k = 0; k < 3; k++) {
      const uint32_t digit = paired_entry_digit(e, k);
      if (digit == 0u) continue;
      v1 &= ~(0xffu << (8 + 8 * k));
      v1 |= paired_entry_pos(e, k) << (8 + 8 * k);
      if (digit == 2u) v1 |= 0x10u << k;
    }
    if (r != kPairedNull) tab_v1[r] = v1;
  }
  tab_v1[kPairedNull] = kEntryNull;  // that number means "nothing" in a paired-lane stream

  split_off.assign((size_t)N + 1, 0u);
  split_codes.clear();
  split_codes.reserve((size_t)N * 2);
  for (int c = 0; c < N; c++) {
    split_off[c] = (uint32_t)split_codes.size();
    if (remap[c] < n_hot) {
      split_codes.push_back((uint16_t)remap[c]);
      continue;
    }
    const std::string &s = seq[c];
    size_t pos = 0;
    while (pos < s.size()) {
      size_t take = 0;
      uint32_t number = 0;
      for (size_t l = s.size() - pos; l >= 1; l--) {  // longest frequent piece first
        auto it = by_seq.find(s.substr(pos, l));
        if (it != by_seq.end() && remap[it->second] < n_hot) {
          take = l;
          number = remap[it->second];
          break;
        }
      }
      if (take == 0) return false;
      split_codes.push_back((uint16_t)number);
      pos += take;
    }
  }
  split_off[N] = (uint32_t)split_codes.size();
  return true;
}

// ---- building the paired-lane copy -------------------------------------------------------------------
// One warp per 32-row block, one lane per row.  count: words the block needs (longest row after the
// replacement of rare codes, two codes per word).  emit: word k of row l at first + k * 32 + l, rows
// padded with the null code.
__global__ void k_paired_count(const uint16_t *__restrict__ codes, const int32_t *__restrict__ row_off,
                             const qmoe_matrix_desc *__restrict__ descs, const uint32_t *__restrict__ split_off,
                             int32_t *__restrict__ blk_units) {
  const qmoe_matrix_desc d = descs[blockIdx.y];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int32_t *ro = row_off + d.rowoff_base;
  const uint16_t *src = codes + d.code_base;
  for (int blk = blockIdx.x * nwarps + warp; blk < d.height / 32; blk += gridDim.x * nwarps) {
    long long b = ro[blk * 32 + lane], e = ro[blk * 32 + lane + 1];
    b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
    e = e < b ? b : (e > d.n_codes ? d.n_codes : e);
    int n = 0;
    for (long long i = b; i < e; i++) {
      const uint32_t c = src[i];
      n += (int)(__ldg(split_off + c + 1) - __ldg(split_off + c));
    }
    int words = (n + 1) >> 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) words = max(words, __shfl_xor_sync(0xffffffffu, words, o));
    if (lane == 0) blk_units[d.minmax_base / 32 + blk] = words * 32;
  }
}

__global__ void k_paired_emit(const uint16_t *__restrict__ codes, const int32_t *__restrict__ row_off,
                            const qmoe_matrix_desc *__restrict__ descs, const long long *__restrict__ blk_base,
                            const uint32_t *__restrict__ split_off, const uint16_t *__restrict__ split_codes,
                            uint32_t *__restrict__ il) {
  const qmoe_matrix_desc d = descs[blockIdx.y];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int32_t *ro = row_off + d.rowoff_base;
  const uint16_t *src = codes + d.code_base;
  for (int blk = blockIdx.x * nwarps + warp; blk < d.height / 32; blk += gridDim.x * nwarps) {
    const long long gblk = d.minmax_base / 32 + blk;
    const long long first = blk_base[gblk];
    const int words = (int)((blk_base[gblk + 1] - first) >> 5);
    long long b = ro[blk * 32 + lane], e = ro[blk * 32 + lane + 1];
    b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
    e = e < b ? b : (e > d.n_codes ? d.n_codes : e);
    uint32_t *dst = il + first + lane;
    int k = 0;
    uint32_t half = 0;
    bool have = false;
    for (long long i = b; i < e; i++) {
      const uint32_t c = src[i];
      const uint32_t s0 = __ldg(split_off + c), s1 = __ldg(split_off + c + 1);
      for (uint32_t s = s0; s < s1; s++) {
        const uint32_t piece = __ldg(split_codes + s);
        if (!have) {
          half = piece;
          have = true;
        } else {
          if (k < words) dst[(long long)k * 32] = half | (piece << 16);
          k++;
          have = false;
        }
      }
    }
    if (have) {
      if (k < words) dst[(long long)k * 32] = half | (kPairedNull << 16);
      k++;
    }
    for (; k < words; k++) dst[(long long)k * 32] = kPairedNullWord;
  }
}

int launch_paired_count(const uint16_t *codes, const int32_t *row_off, const qmoe_matrix_desc *descs, int n_matrices,
                      const uint32_t *split_off, int32_t *blk_units, cudaStream_t stream) {
  const int per_pass = 32768;  // grid.y limit is 65535
  for (int m0 = 0; m0 < n_matrices; m0 += per_pass) {
    const int n = n_matrices - m0 < per_pass ? n_matrices - m0 : per_pass;
    QMOE_LAUNCH(k_paired_count, dim3(8, (unsigned)n), 256, 0, stream, codes, row_off, descs + m0, split_off, blk_units);
    QMOE_CUDA(cudaGetLastError());
  }
  return QMOE_OK;
}

int launch_paired_emit(const uint16_t *codes, const int32_t *row_off, const qmoe_matrix_desc *descs, int n_matrices,
                     const int64_t *blk_base, const uint32_t *split_off, const uint16_t *split_codes, void *il,
                     cudaStream_t stream) {
  const int per_pass = 32768;
  for (int m0 = 0; m0 < n_matrices; m0 += per_pass) {
    const int n = n_matrices - m0 < per_pass ? n_matrices - m0 : per_pass;
    QMOE_LAUNCH(k_paired_emit, dim3(8, (unsigned)n), 256, 0, stream, codes, row_off, descs + m0,
                reinterpret_cast<const long long *>(blk_base), split_off, split_codes,
                reinterpret_cast<uint32_t *>(il));
    QMOE_CUDA(cudaGetLastError());
  }
  return QMOE_OK;
}

// Decode one matrix of a paired-lane copy to ternary symbols (one thread per row), with the table
// and the walk the grouped kernel uses: the parity vehicle of the copy.  status counts rows whose codes
// do not cover the width exactly.
__global__ void k_paired_decode(const uint32_t *__restrict__ tab, const uint32_t *__restrict__ il,
                              const long long *__restrict__ blk_base, qmoe_matrix_desc d,
                              uint8_t *__restrict__ sym, int32_t *status) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= d.height) return;
  const long long gblk = (d.minmax_base + row) >> 5;
  const long long first = blk_base[gblk];
  const int n_words = (int)((blk_base[gblk + 1] - first) >> 5);
  const uint32_t *wp = il + first + (row & 31);
  const int wlim = (d.width + 1) & ~1;
  uint8_t *out = sym + (size_t)row * d.width;
  int pos = 0;
  bool bad = false;
  for (int k = 0; k < n_words; k++) {
    const uint32_t w = wp[(long long)k * 32];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint32_t code = h ? (w >> 16) : (w & 0xffffu);
      if (code > kPairedNull) bad = true;
      const uint32_t e = tab[min(code, kPairedNull)];
#pragma unroll
      for (int j = 0; j < 3; j++) {
        const uint32_t digit = paired_entry_digit(e, j);
        const int p = pos + (int)paired_entry_pos(e, j);
        if (digit != 0u && p < d.width) out[p] = (uint8_t)digit;
      }
      pos += (int)paired_entry_weights(e);
      if (pos > wlim) bad = true;
      pos = pos > wlim ? wlim : pos;
    }
  }
  if (status != nullptr && (bad || pos != wlim)) atomicAdd(status, 1);
}

int launch_paired_decode(const uint32_t *hot_table, const void *il, const int64_t *blk_base,
                       const qmoe_matrix_desc &desc, uint8_t *sym, int32_t *status, cudaStream_t stream) {
  QMOE_CUDA(cudaMemsetAsync(sym, 0, (size_t)desc.height * desc.width, stream));
  if (status != nullptr) QMOE_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  QMOE_LAUNCH(k_paired_decode, (desc.height + 127) / 128, 128, 0, stream, hot_table,
              reinterpret_cast<const uint32_t *>(il), reinterpret_cast<const long long *>(blk_base), desc, sym, status);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

// qmoe_moe_paired_plan_host: the plan alone, host memory in and out (no device needed).
int paired_plan_host(const int32_t *dec, const uint64_t *hist, uint32_t *remap_out, uint32_t *hot_table_out,
                   uint32_t *table_out, uint32_t *split_off_out, uint16_t *split_codes_out, int64_t split_capacity,
                   int64_t *split_total_out) {
  std::vector<uint32_t> remap, hot_tab, tab_v1, split_off;
  std::vector<uint16_t> split_codes;
  if (!paired_plan(dec, hist, remap, hot_tab, tab_v1, split_off, split_codes)) {
    set_error("this decoder table cannot be served by the paired-lane kernel (an entry with more than three "
              "non-zeros, or a rare code that cannot be cut into frequent ones)");
    return QMOE_ERR_UNSUPPORTED;
  }
  if ((int64_t)split_codes.size() > split_capacity) {
    set_error("%lld replacement codes do not fit the %lld provided", (long long)split_codes.size(),
              (long long)split_capacity);
    return QMOE_ERR_INVALID_ARG;
  }
  *split_total_out = (int64_t)split_codes.size();
  std::copy(remap.begin(), remap.end(), remap_out);
  std::copy(hot_tab.begin(), hot_tab.end(), hot_table_out);
  std::copy(tab_v1.begin(), tab_v1.end(), table_out);
  std::copy(split_off.begin(), split_off.end(), split_off_out);
  std::copy(split_codes.begin(), split_codes.end(), split_codes_out);
  return QMOE_OK;
}

// Host part of qmoe_moe_paired_prepare: reads dec and the histogram back, plans, uploads.
int paired_prepare(const int32_t *dec_dev, const uint64_t *hist_dev, uint32_t *remap_out_dev,
                 uint32_t *hot_table_out_dev, uint32_t *table_out_dev, uint32_t *split_off_out_dev,
                 uint16_t *split_codes_out_dev, int64_t split_capacity, int64_t *split_total_out,
                 cudaStream_t stream) {
  std::vector<int32_t> dec((size_t)2 * QMOE_DICT_COUNT);
  std::vector<uint64_t> hist((size_t)QMOE_DICT_COUNT);
  QMOE_CUDA(cudaMemcpyAsync(dec.data(), dec_dev, dec.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  QMOE_CUDA(cudaMemcpyAsync(hist.data(), hist_dev, hist.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost, stream));
  QMOE_CUDA(cudaStreamSynchronize(stream));
  std::vector<uint32_t> remap((size_t)QMOE_DICT_COUNT), hot_tab((size_t)kPairedTab), tab_v1((size_t)QMOE_DICT_COUNT),
      split_off((size_t)QMOE_DICT_COUNT + 1);
  std::vector<uint16_t> split_codes((size_t)split_capacity);
  int rc = paired_plan_host(dec.data(), hist.data(), remap.data(), hot_tab.data(), tab_v1.data(), split_off.data(),
                          split_codes.data(), split_capacity, split_total_out);
  if (rc) return rc;
  QMOE_CUDA(cudaMemcpyAsync(remap_out_dev, remap.data(), remap.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(hot_table_out_dev, hot_tab.data(), hot_tab.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(table_out_dev, tab_v1.data(), tab_v1.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(split_off_out_dev, split_off.data(), split_off.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(split_codes_out_dev, split_codes.data(), (size_t)*split_total_out * 2,
                            cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaStreamSynchronize(stream));  // the host vectors go out of scope
  return QMOE_OK;
}

// ---- the kernel ------------------------------------------------------------------------------------------
struct PairedArgs {
  const uint32_t *tab;         // this kernel's table [kPairedTab]
  const uint32_t *il;          // paired-lane stream
  const long long *blk_base;   // first word of every 32-row block, plus the end
  const uint32_t *minmax;      // (min, max) bf16 pair of every row as one 32-bit word (min in the low half)
  const qmoe_matrix_desc *descs;
  const __nv_bfloat16 *x;
  __nv_bfloat16 *y;
  long long x_stride, y_stride;
  const int32_t *x_rows, *y_rows;  // token t reads row x_rows[t] / writes row y_rows[t] (null: t)
  const int4 *items;  // {matrix, first row, first token, rows | tokens << 16}
  int *header;        // header[0] = item count, header[1] = fetch counter
  int flags;
};

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void lds_u64(uint32_t addr, uint32_t &lo, uint32_t &hi) {
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
}
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// Both 16-bit halves of a word clamped to the null code: a stream that was damaged after it was
// built must never index past the table in shared memory.
__device__ __forceinline__ uint32_t clamp_codes(uint32_t w) {
  uint32_t r;
  asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(w), "r"(kPairedNullWord));
  return r;
}

// One non-zero slot of a code: if the slot's digit field `d` differs from `none` (the field's value
// for "no non-zero"), gather the activations at `addr` and add weight * activation to the sums.
// Gather and multiply-adds are predicated together: a slot without a non-zero costs no shared-memory
// bandwidth (and no bank conflicts), which matters because that pipe is the busiest unit of the SM.
template <uint32_t NONE>
__device__ __forceinline__ void paired_slot1(float &a0, float w, uint32_t addr, uint32_t d) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .f32 v;\n\t"
      "setp.ne.u32 p, %3, %4;\n\t"
      "@p ld.shared.f32 v, [%2];\n\t"
      "@p fma.rn.f32 %0, %1, v, %0;\n\t}"
      : "+f"(a0) : "f"(w), "r"(addr), "r"(d), "n"(NONE));
}
template <uint32_t NONE>
__device__ __forceinline__ void paired_slot2(float &a0, float &a1, float w, uint32_t addr, uint32_t d) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 v, lo, hi;\n\t"
      "setp.ne.u32 p, %4, %5;\n\t"
      "@p ld.shared.b32 v, [%3];\n\t"
      "@p shl.b32 lo, v, 16;\n\t"
      "@p and.b32 hi, v, 0xffff0000;\n\t"
      "@p fma.rn.f32 %0, %2, lo, %0;\n\t"
      "@p fma.rn.f32 %1, %2, hi, %1;\n\t}"
      : "+f"(a0), "+f"(a1) : "f"(w), "r"(addr), "r"(d), "n"(NONE));
}
template <uint32_t NONE>
__device__ __forceinline__ void paired_slot4(float &a0, float &a1, float &a2, float &a3, float w, uint32_t addr,
                                             uint32_t d) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 v0, v1, t0, t1, t2, t3;\n\t"
      "setp.ne.u32 p, %6, %7;\n\t"
      "@p ld.shared.v2.b32 {v0, v1}, [%5];\n\t"
      "@p shl.b32 t0, v0, 16;\n\t"
      "@p and.b32 t1, v0, 0xffff0000;\n\t"
      "@p shl.b32 t2, v1, 16;\n\t"
      "@p and.b32 t3, v1, 0xffff0000;\n\t"
      "@p fma.rn.f32 %0, %4, t0, %0;\n\t"
      "@p fma.rn.f32 %1, %4, t1, %1;\n\t"
      "@p fma.rn.f32 %2, %4, t2, %2;\n\t"
      "@p fma.rn.f32 %3, %4, t3, %3;\n\t}"
      : "+f"(a0), "+f"(a1), "+f"(a2), "+f"(a3) : "f"(w), "r"(addr), "r"(d), "n"(NONE));
}

// One code for T tokens.  pa: shared-memory address of the activations at the row's position
// (advanced by the code's width); mm: the row's (min, max) as packed bf16; acc: fp32 sums.
// Per non-zero: its position (a masked field, already scaled to bytes), one gather, the weight
// {min, max} picked by a byte permute whose selector is digit * 0x2200 + 0x1044, and one
// multiply-add per token (the reference's fp32 multiply-add per weight, sub1_cuda_kernel.cu:188-192).
template <int T>
__device__ __forceinline__ void paired_code(uint32_t e, uint32_t &pa, uint32_t mm, float (&acc)[T]) {
  constexpr int kBytes = T == 4 ? 8 : 4;               // bytes per column in shared memory
  uint32_t off[3];
  if (kBytes == 4) {
    off[0] = e & 0x7cu;
    off[1] = (e >> 9) & 0x7cu;
    off[2] = (e >> 14) & 0x7cu;
  } else {
    off[0] = (e & 0x7cu) << 1;
    off[1] = (e >> 8) & 0xf8u;
    off[2] = (e >> 13) & 0xf8u;
  }
  const uint32_t d0 = e & 3u, d1 = e & 0x180u, d2 = e & 0x600u;   // digit fields in place; "none" = 2, 0x100, 0x400
  const float w0 = __uint_as_float(__byte_perm(mm, 0u, d0 * 0x2200u + 0x1044u));
  const float w1 = __uint_as_float(__byte_perm(mm, 0u, d1 * 0x44u + 0x1044u));
  const float w2 = __uint_as_float(__byte_perm(mm, 0u, d2 * 0x11u + 0x1044u));
  if constexpr (T == 1) {
    paired_slot1<2u>(acc[0], w0, pa + off[0], d0);
    paired_slot1<0x100u>(acc[0], w1, pa + off[1], d1);
    paired_slot1<0x400u>(acc[0], w2, pa + off[2], d2);
  } else if constexpr (T == 2) {
    paired_slot2<2u>(acc[0], acc[1], w0, pa + off[0], d0);
    paired_slot2<0x100u>(acc[0], acc[1], w1, pa + off[1], d1);
    paired_slot2<0x400u>(acc[0], acc[1], w2, pa + off[2], d2);
  } else {
    paired_slot4<2u>(acc[0], acc[1], acc[2], acc[3], w0, pa + off[0], d0);
    paired_slot4<0x100u>(acc[0], acc[1], acc[2], acc[3], w1, pa + off[1], d1);
    paired_slot4<0x400u>(acc[0], acc[1], acc[2], acc[3], w2, pa + off[2], d2);
  }
  pa += kBytes == 4 ? ((e >> 19) & 0x7cu) : ((e >> 18) & 0xf8u);
}

// One work item: rows [row0, row0 + nrows) of matrix d against tokens tok0 .. tok0 + ntok - 1, one row
// per thread.  xs: T activations per column in shared memory (T = 1: fp32; T = 2, 4: bf16), followed
// by kPairedPad zero columns.
template <int T>
__device__ __noinline__ void paired_item(const PairedArgs &a, const qmoe_matrix_desc &d, int row0, int nrows,
                                          int tok0, int ntok, uint32_t tab_addr, uint32_t *xs) {
  constexpr int kBytes = T == 4 ? 8 : 4;
  const int tid = threadIdx.x, lane = tid & 31;
  const int W = d.width;
  const int wlim = (W + 1) & ~1;

  // stage the tokens: xs[c] = {x[token 0][c], ...}, zero beyond the width / token count
  {
    const __nv_bfloat16 *xp[T];
#pragma unroll
    for (int t = 0; t < T; t++) {
      const int tok = tok0 + (t < ntok ? t : 0);
      xp[t] = a.x + (a.x_rows != nullptr ? (long long)a.x_rows[tok] : (long long)tok) * a.x_stride;
    }
    for (int c = tid; c < wlim + kPairedPad; c += blockDim.x) {
      uint32_t h[T];
#pragma unroll
      for (int t = 0; t < T; t++) h[t] = (c < W && t < ntok) ? (uint32_t)__bfloat16_as_ushort(xp[t][c]) : 0u;
      if (T == 1) xs[c] = h[0] << 16;                     // the fp32 value of a bf16
      else if (T == 2) xs[c] = h[0] | (h[1] << 16);
      else reinterpret_cast<uint2 *>(xs)[c] = make_uint2(h[0] | (h[1 % T] << 16), h[2 % T] | (h[3 % T] << 16));
    }
  }
  __syncthreads();

  if (tid < nrows) {
    const int row = row0 + tid;
    // this lane's stream: word k at wp[k * 32]; every row of the block has n_words words
    const long long gblk = (d.minmax_base + row) >> 5;
    const long long first = a.blk_base[gblk];
    const int n_words = (int)((a.blk_base[gblk + 1] - first) >> 5);
    const uint32_t *wp = a.il + first + lane;
    const uint32_t mm = a.minmax[d.minmax_base + row];
    float acc[T];
#pragma unroll
    for (int t = 0; t < T; t++) acc[t] = 0.f;
    const uint32_t xs_addr = (uint32_t)__cvta_generic_to_shared(xs);
    const uint32_t pa_limit = xs_addr + (uint32_t)wlim * kBytes;
    uint32_t pa = xs_addr;

    // software pipeline: the entries of the current word are looked up while the previous word is
    // consumed, the next two words are in flight, and the stream is prefetched into L2 further
    // ahead; no range tests (the copy ends with kPairedTailWords null words)
    uint32_t w1 = clamp_codes(__ldg(wp + 32)), w2 = clamp_codes(__ldg(wp + 64));
    uint32_t e0, e1;
    {
      const uint32_t w0 = clamp_codes(__ldg(wp));
      e0 = lds_u32(tab_addr + ((w0 & 0xffffu) << 2));
      e1 = lds_u32(tab_addr + ((w0 >> 16) << 2));
    }
    const uint32_t *wnext = wp + 96;
#pragma unroll 1
    for (int k = 0; k < n_words; k++) {
      const uint32_t w = w1;
      w1 = w2;
      w2 = clamp_codes(__ldg(wnext));
      prefetch_l2(wnext + kPairedPrefetch * 32);
      wnext += 32;
      const uint32_t f0 = e0, f1 = e1;
      e0 = lds_u32(tab_addr + ((w & 0xffffu) << 2));
      e1 = lds_u32(tab_addr + ((w >> 16) << 2));
      paired_code<T>(f0, pa, mm, acc);
      paired_code<T>(f1, pa, mm, acc);
      pa = min(pa, pa_limit);
    }

#pragma unroll
    for (int t = 0; t < T; t++) {
      if (t < ntok) {
        // fp32 accumulate, round to bf16, then add in bf16 (sub1_cuda_kernel.cu:197-200)
        float v = __bfloat162float(__float2bfloat16_rn(acc[t]));
        const long long out_row = a.y_rows != nullptr ? a.y_rows[tok0 + t] : tok0 + t;
        __nv_bfloat16 *yp = a.y + out_row * a.y_stride + row;
        if (a.flags & QMOE_FLAG_ACCUMULATE) v = __bfloat162float(__float2bfloat16_rn(__bfloat162float(*yp) + v));
        if (a.flags & QMOE_FLAG_RELU) v = fmaxf(v, 0.f);
        *yp = __float2bfloat16_rn(v);
      }
    }
  }
}

static size_t paired_smem_bytes(int width) {
  const int wlim = (width + 1) & ~1;
  return sizeof(uint32_t) * (size_t)kPairedTab + (size_t)(wlim + kPairedPad) * 8;
}

__global__ void __launch_bounds__(kPairedThreads, 1) k_matmul_paired(const PairedArgs a) {
  extern __shared__ __align__(16) uint32_t paired_smem[];
  __shared__ int s_item;
  uint32_t *tab_s = paired_smem;
  uint32_t *xs = paired_smem + kPairedTab;
  const int n_items = a.header[0];
  if (n_items <= 0) return;
  for (uint32_t i = threadIdx.x; i < kPairedTab / 4; i += blockDim.x)
    reinterpret_cast<uint4 *>(tab_s)[i] = __ldg(reinterpret_cast<const uint4 *>(a.tab) + i);
  const uint32_t tab_addr = (uint32_t)__cvta_generic_to_shared(tab_s);
  for (;;) {
    if (threadIdx.x == 0) s_item = atomicAdd(a.header + 1, 1);
    __syncthreads();  // also orders the table fill before the first lookups
    const int i = s_item;
    if (i >= n_items) break;
    const int4 it = a.items[i];
    const qmoe_matrix_desc d = a.descs[it.x];
    const int nrows = it.w & 0x7fff, ntok = it.w >> 16;
    if (ntok <= 1) paired_item<1>(a, d, it.y, nrows, it.z, ntok, tab_addr, xs);
    else if (ntok == 2) paired_item<2>(a, d, it.y, nrows, it.z, ntok, tab_addr, xs);
    else paired_item<4>(a, d, it.y, nrows, it.z, ntok, tab_addr, xs);
    __syncthreads();  // the activations and s_item are rewritten by the next round
  }
}

int launch_paired_phase(const uint32_t *hot_table, const void *il, const int64_t *blk_base, const void *minmax,
                      const qmoe_matrix_desc *descs, const void *x, void *y, long long x_stride, long long y_stride,
                      const int32_t *x_rows, const int32_t *y_rows, const int4 *items, int *header, int flags,
                      int width, int device, cudaStream_t stream) {
  static bool configured[64] = {false};
  if (device < 0 || device >= 64) {
    set_error("device index %d out of range", device);
    return QMOE_ERR_INVALID_ARG;
  }
  {
    std::lock_guard<std::mutex> lock(setup_mutex());
    if (!configured[device]) {
      QMOE_CUDA(cudaFuncSetAttribute(k_matmul_paired, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)paired_smem_bytes(QMOE_MAX_WIDTH)));
      configured[device] = true;
    }
  }
  PairedArgs a{};
  a.tab = hot_table;
  a.il = reinterpret_cast<const uint32_t *>(il);
  a.blk_base = reinterpret_cast<const long long *>(blk_base);
  a.minmax = reinterpret_cast<const uint32_t *>(minmax);
  a.descs = descs;
  a.x = reinterpret_cast<const __nv_bfloat16 *>(x);
  a.y = reinterpret_cast<__nv_bfloat16 *>(y);
  a.x_stride = x_stride;
  a.y_stride = y_stride;
  a.x_rows = x_rows;
  a.y_rows = y_rows;
  a.items = items;
  a.header = header;
  a.flags = flags;
  QMOE_LAUNCH(k_matmul_paired, (unsigned)sm_count(device), kPairedThreads, paired_smem_bytes(width), stream, a);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
