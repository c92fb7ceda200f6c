// Row walker shared by the decode, matvec and grouped kernels.
//
// One thread owns one row of a compressed matrix.  Rows are encoded independently and their codes
// cover the row exactly (sub1_cuda_kernel.cu:211-239), so a thread needs only its row's span
// [row_off[r], row_off[r+1]) of the code stream: it streams the span with aligned 128-bit loads
// (8 codes), looks every code up in the sparse table and keeps a running column position.  There
// is no cross-lane dependency, no shuffle and no barrier inside a row.
//
// The inner loop is written for instruction count: a code costs one table load, one position
// update and, per possible non-zero, one byte extract, one predicated shared load, one select of the
// row's weight value and one multiply-add.  Only the first and the last group of four codes of a
// row pay per-code range checks.
#pragma once

#include "common.cuh"

namespace qmoe {

__device__ __forceinline__ uint32_t entry_len(uint32_t e) { return e & 15u; }
__device__ __forceinline__ uint32_t entry_nz_pos(uint32_t e, int k) {  // 0..27, or >= 0x80 if absent
  return __byte_perm(e, 0u, 0x4441u + (uint32_t)k);
}

// Table lookups.  GlobalLookup reads the 256 KB sparse table through L1/L2.  HotLookup keeps the
// codes [0, kHotLow) and [kHotHigh, 65536) -- 40 960 entries, 160 KB, about 90 % of the codes the
// greedy encoder emits at 90 % sparsity -- in shared memory and falls back to global memory for the
// rest.  The high range is stored right after the low one, so both are read with the code itself as
// index and a per-range base.
constexpr uint32_t kHotLow = 24576;
constexpr uint32_t kHotHigh = 49152;
constexpr uint32_t kHotSlots = kHotLow + (65536 - kHotHigh);

struct GlobalLookup {
  const uint32_t *__restrict__ tab;
  __device__ __forceinline__ uint32_t operator()(uint32_t code) const { return __ldg(tab + code); }
};

struct HotLookup {
  uint32_t hot_addr;                 // shared-space byte address of the kHotSlots entries
  const uint32_t *__restrict__ tab;  // global memory, all 65 536 entries
  // Exactly one of three predicated loads executes per lane; no branch, no divergence.
  __device__ __forceinline__ uint32_t operator()(uint32_t code) const {
    uint32_t e;
    const uint32_t saddr = hot_addr + code * 4u;
    const uint32_t *gaddr = tab + code;
    asm("{\n\t"
        ".reg .pred plo, phi, pmid;\n\t"
        "setp.lt.u32 plo, %1, 24576;\n\t"
        "setp.ge.u32 phi, %1, 49152;\n\t"
        "setp.ge.and.u32 pmid, %1, 24576, !phi;\n\t"
        "@plo ld.shared.b32 %0, [%2];\n\t"
        "@phi ld.shared.b32 %0, [%2 + -98304];\n\t"
        "@pmid ld.global.nc.b32 %0, [%3];\n\t"
        "}"
        : "=r"(e)
        : "r"(code), "r"(saddr), "l"(gaddr));
    return e;
  }
};
// The same for a store whose code values were renumbered by decreasing frequency: the first n_hot
// entries live in shared memory, the rest in global memory.
struct HotLookupLow {
  uint32_t hot_addr;
  const uint32_t *__restrict__ tab;
  uint32_t n_hot;
  __device__ __forceinline__ uint32_t operator()(uint32_t code) const {
    uint32_t e;
    const uint32_t saddr = hot_addr + code * 4u;
    const uint32_t *gaddr = tab + code;
    asm("{\n\t"
        ".reg .pred p;\n\t"
        "setp.lt.u32 p, %1, %4;\n\t"
        "@p ld.shared.b32 %0, [%2];\n\t"
        "@!p ld.global.nc.b32 %0, [%3];\n\t"
        "}"
        : "=r"(e)
        : "r"(code), "r"(saddr), "l"(gaddr), "r"(n_hot));
    return e;
  }
};
static_assert(kHotLow == 24576 && kHotHigh == 49152 && (kHotHigh - kHotLow) * 4 == 98304,
              "HotLookup's inline PTX hard-codes the hot ranges");

// Digit-by-digit decode of one code from the reference table (sub1_cuda_kernel.cu:153-154,
// 188-189): position t lives in word t / 14 at bit 4 + 2 * (t % 14).  Used only for entries that
// do not fit the sparse form.  Returns the number of weights the code covers.
template <class Sink>
__device__ __noinline__ int dense_code(const int32_t *__restrict__ dec, uint32_t code, int pos, Sink &sink) {
  const uint32_t w0 = (uint32_t)__ldg(dec + 2 * code);
  const uint32_t w1 = (uint32_t)__ldg(dec + 2 * code + 1);
  int len = (int)(w0 & 15u);
  len = len > 14 ? 14 : len;
  for (int t = 0; t < 2 * len; t++) {
    const uint32_t w = t < 14 ? w0 : w1;
    const int tt = t < 14 ? t : t - 14;
    const uint32_t digit = (w >> (4 + 2 * tt)) & 3u;
    if (digit == 1u || digit == 2u) sink.dense(pos + t, digit);
  }
  return 2 * len;
}

__device__ __forceinline__ uint32_t chunk_code(const uint4 &q, int j) {
  const uint32_t w = j < 2 ? q.x : j < 4 ? q.y : j < 6 ? q.z : q.w;
  return (j & 1) ? (w >> 16) : (w & 0xffffu);
}

// A code advances the position by at most 28 weights and the position is clamped once per four
// codes, so x must be followed by this many zero entries.
constexpr int kWalkPad = 4 * 28 + 32;

// Where the eight codes of a chunk come from.  StreamFetch: the reference's stream (rows back to
// back), read through a 16-byte aligned pointer.  LaneFetch: the lane-interleaved layout, in which
// the 32 rows of a row block alternate chunk by chunk (chunk k of row l at uint4 index k * 32 + l),
// so that the 32 loads of a warp cover 512 contiguous bytes.
struct StreamFetch {
  const uint16_t *__restrict__ codes_al;
  __device__ __forceinline__ uint4 operator()(int c) const {
    return __ldg(reinterpret_cast<const uint4 *>(codes_al + c));
  }
};
struct LaneFetch {
  const uint4 *__restrict__ p;  // chunk 0 of this lane's row
  __device__ __forceinline__ uint4 operator()(int c) const { return __ldg(p + (c >> 3) * 32); }
};

// Walks codes [b_al, e_al) (indices as fetch() takes them; fetch(c) returns codes c .. c + 7 for c a
// multiple of eight) and feeds every entry to the sink.  Positions are kept scaled by the sink's element size
// (pos << Sink::kShift) so that they are shared-memory byte offsets; `pos_limit` (in weights)
// clamps the running position after every four codes so that a corrupt stream can never index past the
// kWalkPad zero entries that follow x in shared memory.  Returns the final position in weights
// (== padded width for a well-formed row).
//
// Software pipeline in half chunks: while the four entries of one half are consumed, the table
// lookups of the next half are in flight, and the code load runs a whole chunk ahead, so neither the
// shared-memory lookups nor the (rarer, slower) global ones are waited for -- with the same number
// of live registers as a loop that looks up eight entries and consumes them at once.
template <bool GENERAL, class Fetch, class Lookup, class Sink>
__device__ __forceinline__ int walk_row(const Fetch &fetch, int b_al, int e_al, const Lookup &lookup,
                                        const int32_t *__restrict__ dec, int pos_limit, Sink &sink) {
  constexpr int S = Sink::kShift;
  uint32_t posb = 0;
  const uint32_t limit_b = (uint32_t)pos_limit << S;
  int c = b_al & ~7;
  if (c >= e_al) return 0;
  uint4 q_cur = fetch(c);
  uint4 q_next = q_cur;
  if (c + 8 < e_al) q_next = fetch(c + 8);
  uint32_t ea[4], eb[4];
  // Every 16-bit value is a valid table index, so the lookups are unconditional; slots outside
  // the row (first and last chunk only) are then replaced by the null entry.
#pragma unroll
  for (int j = 0; j < 4; j++) ea[j] = lookup(chunk_code(q_cur, j));

  auto consume = [&](uint32_t (&e)[4], const uint4 &q, int first) {
    if (first < b_al || first + 4 > e_al) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int idx = first + j;
        e[j] = (idx >= b_al && idx < e_al) ? e[j] : kEntryNull;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (GENERAL) {
        if ((e[j] & 0xffu) == 0x80u) {
          const int pos = (int)(posb >> S);
          posb = ((uint32_t)(pos + dense_code(dec, chunk_code(q, (first & 4) + j), pos, sink))) << S;
          continue;
        }
      }
      sink.entry(e[j], posb);
      posb += entry_len(e[j]) << (S + 1);
    }
    posb = min(posb, limit_b);
  };

  for (; c < e_al; c += 8) {
#pragma unroll
    for (int j = 0; j < 4; j++) eb[j] = lookup(chunk_code(q_cur, 4 + j));
    consume(ea, q_cur, c);
    const uint4 q_now = q_cur;
    q_cur = q_next;
    if (c + 16 < e_al) q_next = fetch(c + 16);
    if (c + 8 < e_al) {
#pragma unroll
      for (int j = 0; j < 4; j++) ea[j] = lookup(chunk_code(q_cur, j));
    }
    consume(eb, q_now, c + 4);
  }
  return (int)(posb >> S);
}

}  // namespace qmoe
