// Grouped decode-matvec over a lane-private activation window ("ring"), the kernel behind
// qmoe_moe_grouped_ffn for stores that carry a paired-lane copy of their code streams.  Replaces
// Sub1MatVec (sub1_cuda_kernel.cu:129-202) for a whole MoE layer per launch.
//
// Where the time of a decode-matvec goes on this GPU is the shared-memory pipe, not HBM: every 2-byte
// code costs one random dictionary lookup and up to three random gathers from the activation vector,
// and 32 random addresses over 32 banks take 3.4 cycles instead of one.  This kernel removes the
// conflicts of the gathers altogether and halves what is left:
//
//  * one THREAD per row, 1024 rows per CTA, one persistent CTA per SM (as before);
//  * the activations live in shared memory as ring[column mod 512][lane]: every lane of a warp owns a
//    private copy of the current 512-column window in its own bank, so a warp's 32 gathers are one
//    conflict-free wavefront wherever the 32 rows happen to stand.  One copy per bank costs 128 bytes
//    per column, which is why the window is a ring that follows the rows: no row may run more than
//    456 columns ahead of the slowest row of the CTA (it waits, the others catch up), and the CTA
//    re-fills the columns the slowest row has left behind once every eight codes, with one barrier;
//  * the store's streams are re-tokenised when the copy is built: the 40 447 most frequent dictionary
//    entries are renumbered 0 .. 40 446 and sit in shared memory (4 bytes each); every rarer code is
//    replaced by the two or three frequent codes whose sequences concatenate to its own (the
//    dictionary is prefix- and suffix-closed), so the kernel never looks a code up in global memory
//    and needs no range test; rows of a 32-row block are padded with a null code;
//  * two codes per 32-bit word, word k of row l of a block at index k * 32 + l: a warp's stream loads
//    are 128 contiguous bytes.
//
// The copy decodes to exactly the same weights as the reference's streams (tested bit for bit); the
// reference's tensors stay what the C ABI takes and what checkpoints hold.
#include "common.cuh"

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

namespace qmoe {

constexpr int kRingCols = 512;                       // columns of the window (power of two)
constexpr int kRingMirror = 32;                      // first columns repeated behind the last (no wrap test)
constexpr int kRingAhead = 56;                       // columns past the gate that a pair of codes may touch
constexpr int kRingBand = kRingCols - kRingAhead;    // a row may start a pair of codes below slowest + band
constexpr int kRingGroups = 4;                       // pairs of codes per row between two barriers
constexpr int kRingThreads = 1024;
constexpr int kRingTab = QMOE_RING_TABLE;            // table entries in shared memory, the last one null
constexpr uint32_t kRingNull = kRingTab - 1;
constexpr uint32_t kRingNullWord = kRingNull | (kRingNull << 16);
constexpr uint32_t kDone = 0xffffffffu;

// Ring-format table entry: bits 0..3 length in pairs; byte 1 + k describes the k-th non-zero:
// bits 0..4 its position inside the code, bit 5 set = digit 2 (row max), bit 6 set = present.
// The null entry is 0.
__host__ __device__ inline uint32_t ring_entry_from_words(uint32_t w0, uint32_t w1, bool *ok) {
  const int len = (int)(w0 & 15u);
  *ok = len >= 1 && len <= 14 && (int)(w1 & 15u) == len;
  uint32_t e = (uint32_t)len;
  int nz = 0;
  for (int t = 0; t < 28; t++) {
    const uint32_t w = t < 14 ? w0 : w1;
    const uint32_t digit = (w >> (4 + 2 * (t % 14))) & 3u;
    if (digit == 0u) continue;
    if (t >= 2 * len || digit == 3u || nz == 3) {
      *ok = false;
      return 0u;
    }
    e |= ((uint32_t)t | (digit == 2u ? 0x20u : 0u) | 0x40u) << (8 + 8 * nz);
    nz++;
  }
  return *ok ? e : 0u;
}

// ---- host side: renumbering, tables and the replacement lists of rare codes ------------------------
// dec: the reference table (host copy); hist: how often each code occurs in a sample of the store.
// Outputs (host vectors): remap[code] = new number; ring_tab[kRingTab]; tab_v1[65536] = the 4-byte
// table of the row-per-warp kernel in the new numbering (null at kRingNull); split_off / split_codes:
// code c of the reference stream becomes split_codes[split_off[c] .. split_off[c + 1]).
// Returns false when the table cannot be served by this kernel (an entry with more than three
// non-zeros, or a rare code that cannot be cut into frequent ones).
static bool ring_plan(const int32_t *dec, const uint64_t *hist, std::vector<uint32_t> &remap,
                      std::vector<uint32_t> &ring_tab, std::vector<uint32_t> &tab_v1,
                      std::vector<uint32_t> &split_off, std::vector<uint16_t> &split_codes) {
  const int N = QMOE_DICT_COUNT;
  std::vector<std::string> seq((size_t)N);
  std::vector<uint32_t> ring_entry((size_t)N);
  std::unordered_map<std::string, int> by_seq;
  by_seq.reserve((size_t)N * 2);
  for (int c = 0; c < N; c++) {
    const uint32_t w0 = (uint32_t)dec[2 * c], w1 = (uint32_t)dec[2 * c + 1];
    bool ok;
    ring_entry[c] = ring_entry_from_words(w0, w1, &ok);
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
  const uint32_t n_hot = kRingNull;  // numbers 0 .. n_hot - 1 are served from shared memory

  ring_tab.assign((size_t)kRingTab, 0u);
  tab_v1.assign((size_t)N, kEntryNull);
  for (int c = 0; c < N; c++) {
    const uint32_t r = remap[c];
    if (r < n_hot) ring_tab[r] = ring_entry[c];
    // 4-byte form of common.cuh for the row-per-warp kernel
    const uint32_t e = ring_entry[c];
    uint32_t v1 = kEntryNull | (e & 15u);
    for (int k = 0; k < 3; k++) {
      const uint32_t b = (e >> (8 + 8 * k)) & 0xffu;
      if (!(b & 0x40u)) continue;
      v1 &= ~(0xffu << (8 + 8 * k));
      v1 |= (b & 31u) << (8 + 8 * k);
      if (b & 0x20u) v1 |= 0x10u << k;
    }
    if (r != kRingNull) tab_v1[r] = v1;
  }
  tab_v1[kRingNull] = kEntryNull;  // that number means "nothing" in a paired-lane stream

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
__global__ void k_ring_count(const uint16_t *__restrict__ codes, const int32_t *__restrict__ row_off,
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

__global__ void k_ring_emit(const uint16_t *__restrict__ codes, const int32_t *__restrict__ row_off,
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
      if (k < words) dst[(long long)k * 32] = half | (kRingNull << 16);
      k++;
    }
    for (; k < words; k++) dst[(long long)k * 32] = kRingNullWord;
  }
}

int launch_ring_count(const uint16_t *codes, const int32_t *row_off, const qmoe_matrix_desc *descs, int n_matrices,
                      const uint32_t *split_off, int32_t *blk_units, cudaStream_t stream) {
  const int per_pass = 32768;  // grid.y limit is 65535
  for (int m0 = 0; m0 < n_matrices; m0 += per_pass) {
    const int n = n_matrices - m0 < per_pass ? n_matrices - m0 : per_pass;
    QMOE_LAUNCH(k_ring_count, dim3(8, (unsigned)n), 256, 0, stream, codes, row_off, descs + m0, split_off, blk_units);
    QMOE_CUDA(cudaGetLastError());
  }
  return QMOE_OK;
}

int launch_ring_emit(const uint16_t *codes, const int32_t *row_off, const qmoe_matrix_desc *descs, int n_matrices,
                     const int64_t *blk_base, const uint32_t *split_off, const uint16_t *split_codes, void *il,
                     cudaStream_t stream) {
  const int per_pass = 32768;
  for (int m0 = 0; m0 < n_matrices; m0 += per_pass) {
    const int n = n_matrices - m0 < per_pass ? n_matrices - m0 : per_pass;
    QMOE_LAUNCH(k_ring_emit, dim3(8, (unsigned)n), 256, 0, stream, codes, row_off, descs + m0,
                reinterpret_cast<const long long *>(blk_base), split_off, split_codes,
                reinterpret_cast<uint32_t *>(il));
    QMOE_CUDA(cudaGetLastError());
  }
  return QMOE_OK;
}

// Decode one matrix of a paired-lane copy to ternary symbols (one thread per row), with the table
// and the walk the ring kernel uses: the parity vehicle of the copy.  status counts rows whose codes
// do not cover the width exactly.
__global__ void k_ring_decode(const uint32_t *__restrict__ tab, const uint32_t *__restrict__ il,
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
      if (code > kRingNull) bad = true;
      const uint32_t e = tab[min(code, kRingNull)];
#pragma unroll
      for (int j = 0; j < 3; j++) {
        const uint32_t b = (e >> (8 + 8 * j)) & 0xffu;
        const int p = pos + (int)(b & 31u);
        if ((b & 0x40u) && p < d.width) out[p] = (b & 0x20u) ? 2 : 1;
      }
      pos += 2 * (int)(e & 15u);
      if (pos > wlim) bad = true;
      pos = pos > wlim ? wlim : pos;
    }
  }
  if (status != nullptr && (bad || pos != wlim)) atomicAdd(status, 1);
}

int launch_ring_decode(const uint32_t *ring_table, const void *il, const int64_t *blk_base,
                       const qmoe_matrix_desc &desc, uint8_t *sym, int32_t *status, cudaStream_t stream) {
  QMOE_CUDA(cudaMemsetAsync(sym, 0, (size_t)desc.height * desc.width, stream));
  if (status != nullptr) QMOE_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  QMOE_LAUNCH(k_ring_decode, (desc.height + 127) / 128, 128, 0, stream, ring_table,
              reinterpret_cast<const uint32_t *>(il), reinterpret_cast<const long long *>(blk_base), desc, sym, status);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

// qmoe_moe_ring_plan_host: the plan alone, host memory in and out (no device needed).
int ring_plan_host(const int32_t *dec, const uint64_t *hist, uint32_t *remap_out, uint32_t *ring_table_out,
                   uint32_t *table_out, uint32_t *split_off_out, uint16_t *split_codes_out, int64_t split_capacity,
                   int64_t *split_total_out) {
  std::vector<uint32_t> remap, ring_tab, tab_v1, split_off;
  std::vector<uint16_t> split_codes;
  if (!ring_plan(dec, hist, remap, ring_tab, tab_v1, split_off, split_codes)) {
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
  std::copy(ring_tab.begin(), ring_tab.end(), ring_table_out);
  std::copy(tab_v1.begin(), tab_v1.end(), table_out);
  std::copy(split_off.begin(), split_off.end(), split_off_out);
  std::copy(split_codes.begin(), split_codes.end(), split_codes_out);
  return QMOE_OK;
}

// Host part of qmoe_moe_ring_prepare: reads dec and the histogram back, plans, uploads.
int ring_prepare(const int32_t *dec_dev, const uint64_t *hist_dev, uint32_t *remap_out_dev,
                 uint32_t *ring_table_out_dev, uint32_t *table_out_dev, uint32_t *split_off_out_dev,
                 uint16_t *split_codes_out_dev, int64_t split_capacity, int64_t *split_total_out,
                 cudaStream_t stream) {
  std::vector<int32_t> dec((size_t)2 * QMOE_DICT_COUNT);
  std::vector<uint64_t> hist((size_t)QMOE_DICT_COUNT);
  QMOE_CUDA(cudaMemcpyAsync(dec.data(), dec_dev, dec.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  QMOE_CUDA(cudaMemcpyAsync(hist.data(), hist_dev, hist.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost, stream));
  QMOE_CUDA(cudaStreamSynchronize(stream));
  std::vector<uint32_t> remap((size_t)QMOE_DICT_COUNT), ring_tab((size_t)kRingTab), tab_v1((size_t)QMOE_DICT_COUNT),
      split_off((size_t)QMOE_DICT_COUNT + 1);
  std::vector<uint16_t> split_codes((size_t)split_capacity);
  int rc = ring_plan_host(dec.data(), hist.data(), remap.data(), ring_tab.data(), tab_v1.data(), split_off.data(),
                          split_codes.data(), split_capacity, split_total_out);
  if (rc) return rc;
  QMOE_CUDA(cudaMemcpyAsync(remap_out_dev, remap.data(), remap.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(ring_table_out_dev, ring_tab.data(), ring_tab.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(table_out_dev, tab_v1.data(), tab_v1.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(split_off_out_dev, split_off.data(), split_off.size() * 4, cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaMemcpyAsync(split_codes_out_dev, split_codes.data(), (size_t)*split_total_out * 2,
                            cudaMemcpyHostToDevice, stream));
  QMOE_CUDA(cudaStreamSynchronize(stream));  // the host vectors go out of scope
  return QMOE_OK;
}

// ---- the kernel ------------------------------------------------------------------------------------------
struct RingArgs {
  const uint32_t *tab;         // ring-format table [kRingTab]
  const uint32_t *il;          // paired-lane stream
  const long long *blk_base;   // first word of every 32-row block, plus the end
  const __nv_bfloat162 *minmax;
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

// acc2 += c * v2 on a pair of floats with one packed instruction (fma.rn.f32x2).
__device__ __forceinline__ void ring_fma_pair(float &a0, float &a1, float c, float v0, float v1) {
  asm("{\n\t.reg .b64 ra, rc, rv;\n\t"
      "mov.b64 ra, {%0, %1};\n\tmov.b64 rc, {%2, %2};\n\tmov.b64 rv, {%3, %4};\n\t"
      "fma.rn.f32x2 ra, rc, rv, ra;\n\t"
      "mov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(c), "f"(v0), "f"(v1));
}

// One work item: rows [row0, row0 + nrows) of matrix d against tokens tok0 .. tok0 + ntok - 1 (T = 1:
// the window holds fp32 activations; T = 2: bf16 pairs of two tokens, one 4-byte word per column).
template <int T>
__device__ __forceinline__ void ring_item(const RingArgs &a, const qmoe_matrix_desc &d, int row0, int nrows,
                                          int tok0, int ntok, const uint32_t *tab_s, uint32_t *ring,
                                          uint32_t *wmin) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = d.width;
  const uint32_t wlim = (uint32_t)((W + 1) & ~1);
  const bool has_row = tid < nrows;
  const int row = row0 + (has_row ? tid : 0);

  // this lane's stream: word k at wp[k * 32]
  const long long gblk = (d.minmax_base + row) >> 5;
  const long long first = a.blk_base[gblk];
  const int n_words = has_row ? (int)((a.blk_base[gblk + 1] - first) >> 5) : 0;
  const uint32_t *wp = a.il + first + lane;
  auto load_word = [&](int k) -> uint32_t { return k < n_words ? __ldg(wp + (long long)k * 32) : kRingNullWord; };
  auto entry_of = [&](uint32_t code) -> uint32_t { return tab_s[min(code, kRingNull)]; };

  float mn = 0.f, mx = 0.f;
  if (has_row) {
    const __nv_bfloat162 mm = a.minmax[d.minmax_base + row];
    mn = __bfloat162float(mm.x);
    mx = __bfloat162float(mm.y);
  }
  float acc0 = 0.f, acc1 = 0.f;

  // activations of the item's tokens; columns at and beyond the width read as zero
  const int tok1 = tok0 + (ntok > 1 ? 1 : 0);
  const __nv_bfloat16 *x0 = a.x + (a.x_rows != nullptr ? (long long)a.x_rows[tok0] : (long long)tok0) * a.x_stride;
  const __nv_bfloat16 *x1 = a.x + (a.x_rows != nullptr ? (long long)a.x_rows[tok1] : (long long)tok1) * a.x_stride;
  auto x_word = [&](uint32_t c) -> uint32_t {
    if (c >= (uint32_t)W) return 0u;
    if (T == 1) return __float_as_uint(__bfloat162float(x0[c]));
    const uint32_t lo = __bfloat16_as_ushort(x0[c]);
    const uint32_t hi = ntok > 1 ? __bfloat16_as_ushort(x1[c]) : 0u;
    return lo | (hi << 16);
  };
  // column c of the window: 32 copies, one per bank; thread (tid & 7) writes four of them
  uint4 *ring4 = reinterpret_cast<uint4 *>(ring);
  auto put_column = [&](uint32_t c, uint32_t v) {
    const uint32_t slot = c & (kRingCols - 1);
    const uint4 vv = make_uint4(v, v, v, v);
    ring4[slot * 8 + (tid & 7)] = vv;
    if (slot < kRingMirror) ring4[(kRingCols + slot) * 8 + (tid & 7)] = vv;
  };
  for (uint32_t c = (uint32_t)(tid >> 3); c < (uint32_t)kRingCols; c += kRingThreads / 8) put_column(c, x_word(c));

  // software pipeline: entries of the current word, the next two words in flight
  uint32_t w_n1 = load_word(1), w_n2 = load_word(2);
  uint32_t e0, e1;
  {
    const uint32_t w0 = load_word(0);
    e0 = entry_of(w0 & 0xffffu);
    e1 = entry_of(w0 >> 16);
  }
  int k_next = 3;  // next word to request
  uint32_t pos = has_row && n_words > 0 ? 0u : kDone;  // column position of the row; kDone when finished
  const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring) + 4u * (uint32_t)lane;

  auto consume = [&](uint32_t e) {
    const uint32_t base = ring_addr + ((pos & (kRingCols - 1)) << 7);
#pragma unroll
    for (int k = 0; k < 3; k++) {
      const uint32_t o = (e >> (8 + 8 * k)) & 31u;
      const uint32_t v = lds_u32(base + (o << 7));  // unconditional: slot 0 of the code when absent
      const bool present = (e & (0x40u << (8 + 8 * k))) != 0u;
      const float w = (e & (0x20u << (8 + 8 * k))) ? mx : mn;
      if (T == 1) {
        if (present) acc0 = fmaf(w, __uint_as_float(v), acc0);
      } else {
        if (present) ring_fma_pair(acc0, acc1, w, __uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
      }
    }
    pos += (e & 15u) << 1;
  };

  __syncthreads();  // the window holds columns [0, 512)
  uint32_t f_prev2 = 0u, f_prev1 = 0u;  // slowest row of the CTA after the block before last / the last block
  for (int block = 0;; block++) {
    const uint32_t gate = f_prev2 + (uint32_t)kRingBand;
    // Columns the slowest row has left behind since the block before last make room for
    // [f_prev2 + 512, f_prev1 + 512); the loads are issued now and stored after the codes.
    const uint32_t fill_end = min(f_prev1 + (uint32_t)kRingCols, wlim);
    const uint32_t fill_c0 = f_prev2 + (uint32_t)kRingCols + (uint32_t)(tid >> 3);
    const uint32_t fill_c1 = fill_c0 + kRingThreads / 8;
    uint32_t fill_v0 = 0u, fill_v1 = 0u;
    if (fill_c0 < fill_end) fill_v0 = x_word(fill_c0);
    if (fill_c1 < fill_end) fill_v1 = x_word(fill_c1);

#pragma unroll
    for (int g = 0; g < kRingGroups; g++) {
      if (pos < gate) {  // finished rows hold kDone
        consume(e0);
        consume(e1);
        const uint32_t w = w_n1;
        w_n1 = w_n2;
        w_n2 = load_word(k_next);
        k_next++;
        e0 = entry_of(w & 0xffffu);
        e1 = entry_of(w >> 16);
        if (pos >= wlim || k_next > n_words + 2) pos = kDone;
      }
    }

    if (fill_c0 < fill_end) put_column(fill_c0, fill_v0);
    if (fill_c1 < fill_end) put_column(fill_c1, fill_v1);
    const uint32_t warp_min = __reduce_min_sync(0xffffffffu, pos);
    if (lane == 0) wmin[(block & 1) * 32 + warp] = warp_min;
    __syncthreads();
    const uint32_t f = __reduce_min_sync(0xffffffffu, wmin[(block & 1) * 32 + lane]);
    if (f == kDone) break;
    f_prev2 = f_prev1;
    f_prev1 = f;
  }

  if (has_row) {
#pragma unroll
    for (int t = 0; t < T; t++) {
      if (t < ntok) {
        // fp32 accumulate, round to bf16, then add in bf16 (sub1_cuda_kernel.cu:197-200)
        float v = __bfloat162float(__float2bfloat16_rn(t == 0 ? acc0 : acc1));
        const long long out_row = a.y_rows != nullptr ? a.y_rows[tok0 + t] : tok0 + t;
        __nv_bfloat16 *yp = a.y + out_row * a.y_stride + row;
        if (a.flags & QMOE_FLAG_ACCUMULATE) v = __bfloat162float(__float2bfloat16_rn(__bfloat162float(*yp) + v));
        if (a.flags & QMOE_FLAG_RELU) v = fmaxf(v, 0.f);
        *yp = __float2bfloat16_rn(v);
      }
    }
  }
}

constexpr size_t kRingSmemBytes = sizeof(uint32_t) * ((size_t)kRingTab + (size_t)(kRingCols + kRingMirror) * 32 + 64);

__global__ void __launch_bounds__(kRingThreads, 1) k_matmul_ring(const RingArgs a) {
  extern __shared__ __align__(16) uint32_t ring_smem[];
  __shared__ int s_item;
  uint32_t *ring = ring_smem;                                   // 16-byte aligned: the window first
  uint32_t *wmin = ring + (kRingCols + kRingMirror) * 32;
  uint32_t *tab_s = wmin + 64;
  const int n_items = a.header[0];
  if (n_items <= 0) return;
  for (uint32_t i = threadIdx.x; i < kRingTab / 4; i += blockDim.x)
    reinterpret_cast<uint4 *>(tab_s)[i] = __ldg(reinterpret_cast<const uint4 *>(a.tab) + i);
  for (;;) {
    if (threadIdx.x == 0) s_item = atomicAdd(a.header + 1, 1);
    __syncthreads();  // also orders the table fill before the first lookups
    const int i = s_item;
    if (i >= n_items) break;
    const int4 it = a.items[i];
    const qmoe_matrix_desc d = a.descs[it.x];
    const int nrows = it.w & 0x7fff, ntok = it.w >> 16;
    if (ntok <= 1) ring_item<1>(a, d, it.y, nrows, it.z, ntok, tab_s, ring, wmin);
    else ring_item<2>(a, d, it.y, nrows, it.z, ntok, tab_s, ring, wmin);
    __syncthreads();  // the window and s_item are rewritten by the next round
  }
}

int launch_ring_phase(const uint32_t *ring_table, const void *il, const int64_t *blk_base, const void *minmax,
                      const qmoe_matrix_desc *descs, const void *x, void *y, long long x_stride, long long y_stride,
                      const int32_t *x_rows, const int32_t *y_rows, const int4 *items, int *header, int flags,
                      int device, cudaStream_t stream) {
  static bool configured[64] = {false};
  if (device < 0 || device >= 64) {
    set_error("device index %d out of range", device);
    return QMOE_ERR_INVALID_ARG;
  }
  {
    std::lock_guard<std::mutex> lock(setup_mutex());
    if (!configured[device]) {
      QMOE_CUDA(cudaFuncSetAttribute(k_matmul_ring, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingSmemBytes));
      configured[device] = true;
    }
  }
  RingArgs a{};
  a.tab = ring_table;
  a.il = reinterpret_cast<const uint32_t *>(il);
  a.blk_base = reinterpret_cast<const long long *>(blk_base);
  a.minmax = reinterpret_cast<const __nv_bfloat162 *>(minmax);
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
  QMOE_LAUNCH(k_matmul_ring, (unsigned)sm_count(device), kRingThreads, kRingSmemBytes, stream, a);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
