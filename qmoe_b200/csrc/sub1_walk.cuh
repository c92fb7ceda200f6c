// Row walker shared by the decode, matvec and grouped kernels.
//
// One thread owns one row of a compressed matrix.  Rows are encoded independently and their codes
// cover the row exactly (sub1_cuda_kernel.cu:211-239), so a thread needs only its row's span
// [row_off[r], row_off[r+1]) of the code stream: it streams the span with aligned 128-bit loads
// (8 codes), looks every code up in the sparse table and keeps a running column position.  There
// is no cross-lane dependency, no shuffle and no barrier inside a row.
#pragma once

#include "common.cuh"

namespace qmoe {

// Field accessors of a sparse-table entry (layout in common.cuh).
__device__ __forceinline__ int entry_weights(uint32_t e) { return (int)(e & 31u); }

// Digit-by-digit decode of one code from the reference table (sub1_cuda_kernel.cu:153-154,
// 188-189): position t lives in word t / 14 at bit 4 + 2 * (t % 14).  Used only for entries that
// do not fit the sparse form.
template <class Sink>
__device__ __forceinline__ int dense_code(const int32_t *__restrict__ dec, uint32_t code, int pos,
                                          Sink &sink) {
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

// Walks codes [b_al, e_al) (indices relative to the 16-byte aligned pointer codes_al) and feeds
// every entry to the sink.  `pos_limit` clamps the running position so that a corrupt stream can
// never index past the zero padding that follows x in shared memory.  Returns the final position
// (== padded width for a well-formed row).
template <bool GENERAL, class Sink>
__device__ __forceinline__ int walk_row(const uint16_t *__restrict__ codes_al, int b_al, int e_al,
                                        const uint32_t *__restrict__ tab,
                                        const int32_t *__restrict__ dec, int pos_limit, Sink &sink) {
  int pos = 0;
  for (int c = b_al & ~7; c < e_al; c += 8) {
    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(codes_al + c));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int idx = c + j;
      const bool valid = idx >= b_al && idx < e_al;
      const uint32_t code = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu);
      uint32_t e = 0;
      if (valid) e = __ldg(tab + code);
      if (GENERAL) {
        if (valid && entry_weights(e) == 0) {
          pos = min(pos + dense_code(dec, code, pos, sink), pos_limit);
          continue;
        }
      }
      sink.entry(e, pos);
      pos = min(pos + entry_weights(e), pos_limit);
    }
  }
  return pos;
}

}  // namespace qmoe
