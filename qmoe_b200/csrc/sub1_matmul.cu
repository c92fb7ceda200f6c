// Fused dictionary decode + matvec / small-batch matmul for sm_100a, and the decode-to-symbols
// kernel.  Replaces Sub1MatVec (sub1_cuda_kernel.cu:129-202) and the per-token launch loop of
// Sub1Linear.forward (sub1.py:132-143).
//
// Design (differs from the reference on purpose):
//  * one THREAD per row instead of one warp per row: codes are streamed with aligned 128-bit
//    loads, the running column position is a private register, nothing is shuffled or synchronised
//    inside a row, and all 32 lanes do useful work;
//  * a derived 4-byte sparse dictionary (common.cuh) turns a code into at most three gathers from
//    the activation vector, each followed by one multiply-add with min_r or max_r, instead of 28
//    multiply-adds;
//  * the activations of up to four tokens are interleaved in shared memory so that one decode
//    serves all of them (one 4- or 8-byte shared load per non-zero: fp32 for one token, bf16 pairs
//    or quads for more);
//  * a work list of (matrix, row block, token group) items lets one launch cover every active
//    expert of a MoE layer;
//  * for such launches the code streams are read from a lane-interleaved copy (32 rows alternate
//    chunk by chunk, so a warp's loads are contiguous) whose code values are renumbered by
//    frequency, and the most frequent 45-53 thousand dictionary entries sit in shared memory.
#include "common.cuh"
#include "sub1_walk.cuh"

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <type_traits>
#include <vector>

namespace qmoe {

constexpr int kRowsPerItem = 256;     // single-matrix kernel: threads per CTA == rows per work item
constexpr int kGroupedThreads = 1024; // grouped kernel: one persistent CTA per SM, rows per work item
constexpr int kMaxGroup = 4;          // tokens decoded together
constexpr int kPad = kWalkPad;        // zero entries after x (see walk_row)

static inline int rows_per_chunk(int height, int rows_per_item) {
  const int chunks = (height + rows_per_item - 1) / rows_per_item;
  int rpc = (height + chunks - 1) / chunks;
  rpc = (rpc + 31) / 32 * 32;
  return rpc;
}
__device__ __forceinline__ int rows_per_chunk_dev(int height, int rows_per_item) {
  const int chunks = (height + rows_per_item - 1) / rows_per_item;
  const int rpc = (height + chunks - 1) / chunks;
  return (rpc + 31) / 32 * 32;
}
static inline int chunk_count(int height, int rows_per_item) {
  const int rpc = rows_per_chunk(height, rows_per_item);
  return (height + rpc - 1) / rpc;
}

// ---- sinks ------------------------------------------------------------------------------------
// Shared loads that execute only where the non-zero exists; absent lanes keep zeros (and cost no
// shared-memory bandwidth), so the adds that follow need no presence test.
__device__ __forceinline__ void lds_pred_b16(uint32_t &v, uint32_t addr, uint32_t pos_byte) {
  asm("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %2, 128;\n\tmov.b32 %0, 0;\n\t"
      "@p ld.shared.u16 %0, [%1];\n\t}" : "=r"(v) : "r"(addr), "r"(pos_byte));
}
__device__ __forceinline__ void lds_pred_b32(uint32_t &v, uint32_t addr, uint32_t pos_byte) {
  asm("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %2, 128;\n\tmov.b32 %0, 0;\n\t"
      "@p ld.shared.b32 %0, [%1];\n\t}" : "=r"(v) : "r"(addr), "r"(pos_byte));
}
__device__ __forceinline__ void lds_pred_b64(uint32_t &v0, uint32_t &v1, uint32_t addr, uint32_t pos_byte) {
  asm("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %3, 128;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\t"
      "@p ld.shared.v2.b32 {%0, %1}, [%2];\n\t}" : "=r"(v0), "=r"(v1) : "r"(addr), "r"(pos_byte));
}
__device__ __forceinline__ void lds_pred_b128(uint32_t (&v)[4], uint32_t addr, uint32_t pos_byte) {
  asm("{\n\t.reg .pred p;\n\tsetp.lt.u32 p, %5, 128;\n\tmov.b32 %0, 0;\n\tmov.b32 %1, 0;\n\t"
      "mov.b32 %2, 0;\n\tmov.b32 %3, 0;\n\t@p ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr), "r"(pos_byte));
}

constexpr int ilog2(int v) { return v <= 1 ? 0 : 1 + ilog2(v / 2); }

// acc2 += c * v2 on a pair of floats with one packed instruction (fma.rn.f32x2).
__device__ __forceinline__ void fma_pair(float &a0, float &a1, float c, float v0, float v1) {
  asm("{\n\t.reg .b64 ra, rc, rv;\n\t"
      "mov.b64 ra, {%0, %1};\n\tmov.b64 rc, {%2, %2};\n\tmov.b64 rv, {%3, %4};\n\t"
      "fma.rn.f32x2 ra, rc, rv, ra;\n\t"
      "mov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(c), "f"(v0), "f"(v1));
}

// Accumulates, for T tokens, acc[t] = sum over the non-zeros of a row of w * x[t][c] in fp32, with
// w = min_r for digit 1 and max_r for digit 2 (the reference's fp32 multiply-add per weight,
// sub1_cuda_kernel.cu:188-192).  x lives in shared memory as [position][T], fp32 (F32) or bf16.
template <int T, bool F32>
struct MatSink {
  using elem = typename std::conditional<F32, float, __nv_bfloat16>::type;
  static constexpr int kShift = ilog2(T * (F32 ? 4 : 2));  // log2(bytes per position)
  static __device__ __forceinline__ elem stage(__nv_bfloat16 v) {
    if constexpr (F32) return __bfloat162float(v);
    else return v;
  }
  uint32_t xs_addr;  // shared-space byte address of x
  float mn, mx;      // the row's two weight values
  float acc[T];

  __device__ __forceinline__ void reset(float row_min, float row_max, uint32_t addr) {
    xs_addr = addr;
    mn = row_min;
    mx = row_max;
#pragma unroll
    for (int t = 0; t < T; t++) acc[t] = 0.f;
  }
  __device__ __forceinline__ void load(float (&vf)[T], uint32_t addr, uint32_t pos_byte) {
    if constexpr (F32) {
      uint32_t v[4] = {0u, 0u, 0u, 0u};
      if constexpr (T == 1) lds_pred_b32(v[0], addr, pos_byte);
      else if constexpr (T == 2) lds_pred_b64(v[0], v[1], addr, pos_byte);
      else lds_pred_b128(v, addr, pos_byte);
#pragma unroll
      for (int t = 0; t < T; t++) vf[t] = __uint_as_float(v[t]);
    } else {
      uint32_t v0 = 0u, v1 = 0u;
      if constexpr (T == 1) lds_pred_b16(v0, addr, pos_byte);
      else if constexpr (T == 2) lds_pred_b32(v0, addr, pos_byte);
      else lds_pred_b64(v0, v1, addr, pos_byte);
      vf[0] = __uint_as_float(v0 << 16);
      if constexpr (T >= 2) vf[1] = __uint_as_float(v0 & 0xffff0000u);
      if constexpr (T >= 4) {
        vf[2] = __uint_as_float(v1 << 16);
        vf[3] = __uint_as_float(v1 & 0xffff0000u);
      }
    }
  }
  __device__ __forceinline__ void add(float c, const float (&vf)[T]) {
    if constexpr (T == 1) {
      acc[0] = fmaf(c, vf[0], acc[0]);
    } else {
#pragma unroll
      for (int t = 0; t < T; t += 2) fma_pair(acc[t], acc[t + 1], c, vf[t], vf[t + 1]);
    }
  }
  __device__ __forceinline__ void entry(uint32_t e, uint32_t posb) {
    const uint32_t base = xs_addr + posb;
#pragma unroll
    for (int k = 0; k < 3; k++) {
      const uint32_t o = entry_nz_pos(e, k);
      float vf[T];
      load(vf, base + (o << kShift), o);  // zeros where the non-zero is absent
      add((e & (0x10u << k)) ? mx : mn, vf);
    }
  }
  __device__ __forceinline__ void dense(int p, uint32_t digit) {
    float vf[T];
    load(vf, xs_addr + ((uint32_t)p << kShift), 0u);
    add(digit == 1u ? mn : mx, vf);
  }
};

struct SymbolSink {
  static constexpr int kShift = 0;
  uint8_t *row;  // width bytes, pre-zeroed
  int width;
  __device__ __forceinline__ void put(int p, uint8_t d) {
    if (p < width) row[p] = d;
  }
  __device__ __forceinline__ void entry(uint32_t e, uint32_t pos) {
#pragma unroll
    for (int k = 0; k < 3; k++) {
      const uint32_t o = entry_nz_pos(e, k);
      if (o < 0x80u) put((int)(pos + o), (e & (0x10u << k)) ? 2 : 1);
    }
  }
  __device__ __forceinline__ void dense(int p, uint32_t digit) { put(p, (uint8_t)digit); }
};

// ---- kernel arguments ---------------------------------------------------------------------------
struct MatmulArgs {
  const uint32_t *tab;
  const int32_t *dec;
  const uint16_t *codes;
  const int32_t *row_off;
  const __nv_bfloat162 *minmax;
  const qmoe_matrix_desc *descs;  // grouped mode
  const uint4 *il;                // grouped mode, lane-interleaved streams (or null)
  const long long *blk_base;      // first uint4 of every 32-row block of `il`, plus the end
  const int32_t *il_rows;         // optional: row of its matrix that position p of the interleaved store holds
  const uint32_t *il_tab;         // sparse table in the order of the interleaved store's code values
  const int32_t *il_dec;          // reference table words in that order
  int n_hot;                      // entries of il_tab kept in shared memory
  qmoe_matrix_desc single;        // uniform mode
  const __nv_bfloat16 *x;
  __nv_bfloat16 *y;
  long long x_stride, y_stride;
  const int32_t *x_rows, *y_rows;  // grouped mode: token t reads row x_rows[t] / writes row y_rows[t] (null: t)
  const unsigned long long *y_ptrs;  // grouped mode, optional: address of token t's output row (then y, y_stride
                                     // and y_rows are not used); the row may lie in another GPU's memory
  const int4 *items;  // grouped mode: {matrix, first row, first token, rows | tokens << 16}
  int *header;        // grouped mode: header[0] = item count, header[1] = fetch counter
  // Fused launch of both linears of the expert FFN (grouped mode, `fused` != 0): the items of the
  // second linear follow those of the first in one fetch order; `second` says where they read and
  // write; items2 / header2 are their list and count; done[pair] counts the finished items of the
  // first linear per (expert, token group), which an item of the second waits for.
  struct SecondIO {
    const __nv_bfloat16 *x;
    __nv_bfloat16 *y;
    long long x_stride, y_stride;
    const int32_t *y_rows;
    const unsigned long long *y_ptrs;
    int flags;
  } second;
  const int4 *items2;
  const int *header2;
  int *done;
  int *wait_status;
  int fused;
  unsigned x_half_bytes;  // grouped mode: bytes of the activations of a one- or two-token item (half the area)
  int chunks, rpc, tokens;  // uniform mode
  int flags;
};

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// `second`: an item of the second linear of a fused launch (reads and writes through a.second).
template <int T, class SinkT>
__device__ __forceinline__ void store_row(const MatmulArgs &a, const SinkT &sink, int row, int tok0, int ntok,
                                          bool second = false) {
  const unsigned long long *y_ptrs = second ? a.second.y_ptrs : a.y_ptrs;
  const int32_t *y_rows = second ? a.second.y_rows : a.y_rows;
  const int flags = second ? a.second.flags : a.flags;
#pragma unroll
  for (int t = 0; t < T; t++) {
    if (t < ntok) {
      // fp32 accumulate, round to bf16, then add in bf16 (sub1_cuda_kernel.cu:197-200).
      float v = bf16_round(sink.acc[t]);
      __nv_bfloat16 *yp;
      if (y_ptrs != nullptr) {
        yp = reinterpret_cast<__nv_bfloat16 *>(y_ptrs[tok0 + t]) + row;
      } else {
        const long long out_row = y_rows != nullptr ? y_rows[tok0 + t] : tok0 + t;
        yp = (second ? a.second.y : a.y) + out_row * (second ? a.second.y_stride : a.y_stride) + row;
      }
      if (flags & QMOE_FLAG_ACCUMULATE) v = bf16_round(__bfloat162float(*yp) + v);
      if (flags & QMOE_FLAG_RELU) v = fmaxf(v, 0.f);
      *yp = __float2bfloat16_rn(v);
    }
  }
}

template <int T, class SinkT>
__device__ __forceinline__ void stage_tokens(const MatmulArgs &a, int W, int wlim, int tok0, int ntok,
                                             typename SinkT::elem *xs, bool second = false) {
  // xs[c][t] = x[row of token tok0 + t][c], zero beyond the width / token count.
  const __nv_bfloat16 *xp[T];
#pragma unroll
  for (int t = 0; t < T; t++) {
    const int tok = tok0 + (t < ntok ? t : 0);
    if (second) xp[t] = a.second.x + (long long)tok * a.second.x_stride;  // indexed by slot
    else xp[t] = a.x + (a.x_rows != nullptr ? (long long)a.x_rows[tok] : (long long)tok) * a.x_stride;
  }
  for (int c = threadIdx.x; c < wlim + kPad; c += blockDim.x) {
#pragma unroll
    for (int t = 0; t < T; t++) {
      __nv_bfloat16 v = __float2bfloat16_rn(0.f);
      if (c < W && t < ntok) {
        // rows written by other CTAs of the same launch are read from L2, never from this SM's L1
        if (second) v = __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short *>(xp[t] + c)));
        else v = xp[t][c];
      }
      xs[c * T + t] = SinkT::stage(v);
    }
  }
}

template <int T, bool GENERAL, class SinkT, int G = 2, class Lookup>
__device__ __forceinline__ void warp_rows_staged(const MatmulArgs &a, const qmoe_matrix_desc &d, int row0,
                                                 int nrows, int tok0, int ntok, typename SinkT::elem *xs,
                                                 const Lookup &lookup, bool second = false);

// Rows [row0, row0 + nrows) one per thread; with an interleaved store, `tail_rows` further rows
// (what a height like 2080 leaves after blocks of 1024) one per warp, against the same staged x.
template <int T, bool GENERAL, class SinkT, bool IL = false, class Lookup>
__device__ __forceinline__ void process_item(const MatmulArgs &a, const qmoe_matrix_desc &d, int row0,
                                             int nrows, int tok0, int ntok, typename SinkT::elem *xs,
                                             const Lookup &lookup, int tail_rows = 0, bool second = false,
                                             bool staged = false) {
  const int tid = threadIdx.x;
  const int W = d.width;
  const int wlim = (W + 1) & ~1;

  // What a thread needs to know about its row is loaded BEFORE the activations are staged, so that
  // these dependent global loads (row list -> offsets, block base) and the first lines of the row's
  // code stream travel while the CTA stages x, not after the barrier.
  // With an interleaved store whose rows were re-ordered (rows of similar length side by side), thread
  // tid walks the stream at POSITION row0 + tid, which belongs to row il_rows[...] of the matrix.
  const bool active = tid < nrows;
  const int pos = row0 + tid;
  int row = pos;
  long long b = 0, e = 0, first = 0, n = 0;
  __nv_bfloat162 mm = __floats2bfloat162_rn(0.f, 0.f);
  if (active) {
    if constexpr (IL) {
      if (a.il_rows != nullptr) {
        row = a.il_rows[d.minmax_base + pos];
        row = row < 0 ? 0 : (row >= d.height ? d.height - 1 : row);
      }
    }
    const int32_t *ro = a.row_off + d.rowoff_base;
    b = ro[row];
    e = ro[row + 1];
    b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
    e = e < b ? b : (e > d.n_codes ? d.n_codes : e);
    mm = a.minmax[d.minmax_base + row];
    if constexpr (IL) {
      // Row blocks of 32 rows start at multiples of 32 in every matrix and in the store.
      const long long gblk = (d.minmax_base + pos) >> 5;
      first = a.blk_base[gblk];
      const long long room = (a.blk_base[gblk + 1] - first) >> 5 << 3;  // codes per row of this block
      n = e - b < room ? e - b : room;
      const uint4 *src = a.il + first + (pos & 31);
      asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
      if (n > 8) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + 32));
    }
  }

  if (!staged) {  // else xs was filled during the CTA's previous item, whose last barrier ordered it
    stage_tokens<T, SinkT>(a, W, wlim, tok0, ntok, xs, second);
    __syncthreads();
  }

  if (active) {
    SinkT sink;
    sink.reset(__bfloat162float(mm.x), __bfloat162float(mm.y), (uint32_t)__cvta_generic_to_shared(xs));
    if constexpr (IL) {
      walk_row<GENERAL>(LaneFetch{a.il + first + (pos & 31)}, 0, (int)n, lookup, a.il_dec, wlim, sink);
    } else {
      const uint16_t *codes_m = a.codes + d.code_base;
      const int mis = (int)((reinterpret_cast<uintptr_t>(codes_m) & 15u) >> 1);
      walk_row<GENERAL>(StreamFetch{codes_m - mis}, (int)b + mis, (int)e + mis, lookup, a.dec, wlim, sink);
    }

    store_row<T>(a, sink, row, tok0, ntok, second);
  }
  if constexpr (IL) {
    if (tail_rows > 0)
      warp_rows_staged<T, GENERAL, SinkT>(a, d, row0 + nrows, tail_rows, tok0, ntok, xs, lookup, second);
  }
}

// One CTA per (row block, token group) of a single matrix; the sparse table is read through L1/L2.
template <bool GENERAL>
__global__ void __launch_bounds__(kRowsPerItem) k_matmul_uniform(const MatmulArgs a) {
  extern __shared__ __align__(16) float xs_f32[];
  const int chunk = blockIdx.x % a.chunks;
  const int group = blockIdx.x / a.chunks;
  const int row0 = chunk * a.rpc;
  const int nrows = min(a.rpc, a.single.height - row0);
  const int tok0 = group * kMaxGroup;
  const int ntok = min(kMaxGroup, a.tokens - tok0);
  const GlobalLookup lookup{a.tab};
  if (ntok <= 1) process_item<1, GENERAL, MatSink<1, true>>(a, a.single, row0, nrows, tok0, ntok, xs_f32, lookup);
  else if (ntok == 2) process_item<2, GENERAL, MatSink<2, true>>(a, a.single, row0, nrows, tok0, ntok, xs_f32, lookup);
  else process_item<4, GENERAL, MatSink<4, true>>(a, a.single, row0, nrows, tok0, ntok, xs_f32, lookup);
}

// ---- single matrix, one WARP per row --------------------------------------------------------------
// A lone 0.2-1.1 MB matrix is a latency problem, not a bandwidth one: with one thread per row a
// 768 x 3072 matrix offers 768 threads that each walk 132 codes in sequence.  Here a warp shares a
// row: lane i takes code base + i, the lanes' column positions come from a warp prefix sum of the
// code lengths, and the two partial sums are reduced with shuffles at the end of the row.  The
// serial depth of a row drops from its number of codes to that number / 32.
constexpr int kWarpRowThreads = 256;

// One row by a whole warp: code_at(i) returns code i of the row (0 <= i < n), `tab` / `dec` are the
// tables for those code values.  Leaves the row's sums, reduced over the lanes, in sink.acc.
template <bool GENERAL, class SinkT, class CodeAt, class Lookup>
__device__ __forceinline__ void warp_row_sum(const CodeAt &code_at, int n, const Lookup &lookup,
                                             const int32_t *__restrict__ dec, uint32_t limit, SinkT &sink,
                                             int lane) {
  constexpr int S = SinkT::kShift;
  uint32_t row_pos = 0;
  // Two groups of 32 codes per iteration (both dictionary lookups in flight together), and the
  // codes of the next iteration are requested before this one is processed.
  uint32_t code0 = 0, code1 = 0;
  if (lane < n) code0 = code_at(lane);
  if (32 + lane < n) code1 = code_at(32 + lane);
  for (int base = 0; base < n; base += 64) {
    const bool v0 = base + lane < n, v1 = base + 32 + lane < n;
    const uint32_t c0 = code0, c1 = code1;
    uint32_t e0 = kEntryNull, e1 = kEntryNull;
    if (v0) e0 = lookup(c0);
    if (v1) e1 = lookup(c1);
    if (base + 64 + lane < n) code0 = code_at(base + 64 + lane);
    if (base + 96 + lane < n) code1 = code_at(base + 96 + lane);
    uint32_t len0 = 2u * entry_len(e0), len1 = 2u * entry_len(e1);
    bool d0 = false, d1 = false;
    if (GENERAL) {
      d0 = (e0 & 0xffu) == 0x80u;
      d1 = (e1 & 0xffu) == 0x80u;
      if (d0) len0 = 2u * min((uint32_t)__ldg(dec + 2 * c0) & 15u, 14u);
      if (d1) len1 = 2u * min((uint32_t)__ldg(dec + 2 * c1) & 15u, 14u);
    }
    uint32_t i0 = len0, i1 = len1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t u0 = __shfl_up_sync(0xffffffffu, i0, o);
      const uint32_t u1 = __shfl_up_sync(0xffffffffu, i1, o);
      if (lane >= o) {
        i0 += u0;
        i1 += u1;
      }
    }
    const uint32_t total0 = __shfl_sync(0xffffffffu, i0, 31), total1 = __shfl_sync(0xffffffffu, i1, 31);
    const uint32_t p0 = min(row_pos + i0 - len0, limit);
    const uint32_t p1 = min(row_pos + total0 + i1 - len1, limit);
    if (GENERAL && d0) dense_code(dec, c0, (int)p0, sink);
    else sink.entry(e0, p0 << S);
    if (GENERAL && d1) dense_code(dec, c1, (int)p1, sink);
    else sink.entry(e1, p1 << S);
    row_pos = min(row_pos + total0 + total1, limit);
  }
#pragma unroll
  for (int t = 0; t < (int)(sizeof(sink.acc) / sizeof(float)); t++) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sink.acc[t] += __shfl_xor_sync(0xffffffffu, sink.acc[t], o);
  }
}

// The same with G groups of 32 codes per iteration (fewer dependent rounds for long rows).
template <bool GENERAL, int G, class SinkT, class CodeAt, class Lookup>
__device__ __forceinline__ void warp_row_sum_groups(const CodeAt &code_at, int n, const Lookup &lookup,
                                             const int32_t *__restrict__ dec, uint32_t limit, SinkT &sink,
                                             int lane) {
  constexpr int S = SinkT::kShift;
  uint32_t row_pos = 0;
  // G groups of 32 codes per iteration (their dictionary lookups in flight together), and the
  // codes of the next iteration are requested before this one is processed.
  uint32_t code[G];
#pragma unroll
  for (int g = 0; g < G; g++) code[g] = 32 * g + lane < n ? code_at(32 * g + lane) : 0u;
  for (int base = 0; base < n; base += 32 * G) {
    uint32_t c[G], e[G], len[G];
    bool dense[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      c[g] = code[g];
      e[g] = base + 32 * g + lane < n ? lookup(c[g]) : kEntryNull;
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      const int next = base + 32 * (G + g) + lane;
      if (next < n) code[g] = code_at(next);
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      len[g] = 2u * entry_len(e[g]);
      dense[g] = false;
      if (GENERAL) {
        dense[g] = (e[g] & 0xffu) == 0x80u;
        if (dense[g]) len[g] = 2u * min((uint32_t)__ldg(dec + 2 * c[g]) & 15u, 14u);
      }
    }
    uint32_t incl[G];
#pragma unroll
    for (int g = 0; g < G; g++) incl[g] = len[g];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
      for (int g = 0; g < G; g++) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, incl[g], o);
        if (lane >= o) incl[g] += u;
      }
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      const uint32_t total = __shfl_sync(0xffffffffu, incl[g], 31);
      const uint32_t p = min(row_pos + incl[g] - len[g], limit);
      if (GENERAL && dense[g]) dense_code(dec, c[g], (int)p, sink);
      else sink.entry(e[g], p << S);
      row_pos = min(row_pos + total, limit);
    }
  }
#pragma unroll
  for (int t = 0; t < (int)(sizeof(sink.acc) / sizeof(float)); t++) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sink.acc[t] += __shfl_xor_sync(0xffffffffu, sink.acc[t], o);
  }
}

template <int T, bool GENERAL>
__device__ __forceinline__ void warp_rows(const MatmulArgs &a, int row0, int nrows, int tok0, int ntok, float *xs) {
  using SinkT = MatSink<T, true>;
  const qmoe_matrix_desc &d = a.single;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int wlim = (d.width + 1) & ~1;
  stage_tokens<T, SinkT>(a, d.width, wlim, tok0, ntok, xs);
  __syncthreads();
  for (int r = warp; r < nrows; r += nwarps) {
    const int row = row0 + r;
    long long b = a.row_off[row], e = a.row_off[row + 1];
    b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
    e = e < b ? b : (e > d.n_codes ? d.n_codes : e);
    const __nv_bfloat162 mm = a.minmax[row];
    SinkT sink;
    sink.reset(__bfloat162float(mm.x), __bfloat162float(mm.y), (uint32_t)__cvta_generic_to_shared(xs));
    const uint16_t *src = a.codes + b;
    warp_row_sum<GENERAL>([&](int i) { return (uint32_t)src[i]; }, (int)(e - b), GlobalLookup{a.tab}, a.dec,
                          (uint32_t)wlim, sink, lane);
    if (lane == 0) store_row<T>(a, sink, row, tok0, ntok);
  }
}

// The same for a work item of an interleaved store: code i of row l of a block is element i % 8
// of the 16-byte entry (i / 8) * 32 + l.
template <int T, bool GENERAL, class SinkT, int G, class Lookup>
__device__ __forceinline__ void warp_rows_staged(const MatmulArgs &a, const qmoe_matrix_desc &d, int row0,
                                                 int nrows, int tok0, int ntok, typename SinkT::elem *xs,
                                                 const Lookup &lookup, bool second) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int wlim = (d.width + 1) & ~1;
  const int32_t *ro = a.row_off + d.rowoff_base;
  for (int r = warp; r < nrows; r += nwarps) {
    const int pos = row0 + r;  // position in the store; its row of the matrix may differ (il_rows)
    int row = pos;
    if (a.il_rows != nullptr) {
      row = a.il_rows[d.minmax_base + pos];
      row = row < 0 ? 0 : (row >= d.height ? d.height - 1 : row);
    }
    long long b = ro[row], e = ro[row + 1];
    b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
    e = e < b ? b : (e > d.n_codes ? d.n_codes : e);
    const long long gblk = (d.minmax_base + pos) >> 5;
    const long long first = a.blk_base[gblk];
    const long long room = (a.blk_base[gblk + 1] - first) >> 5 << 3;
    const int n = (int)(e - b < room ? e - b : room);
    const uint16_t *src = reinterpret_cast<const uint16_t *>(a.il + first + (pos & 31));
    const __nv_bfloat162 mm = a.minmax[d.minmax_base + row];
    SinkT sink;
    sink.reset(__bfloat162float(mm.x), __bfloat162float(mm.y), (uint32_t)__cvta_generic_to_shared(xs));
    const auto code_at = [&](int i) { return (uint32_t)__ldg(src + (i >> 3) * 256 + (i & 7)); };
    if constexpr (G == 2) warp_row_sum<GENERAL>(code_at, n, lookup, a.il_dec, (uint32_t)wlim, sink, lane);
    else warp_row_sum_groups<GENERAL, G>(code_at, n, lookup, a.il_dec, (uint32_t)wlim, sink, lane);
    if (lane == 0) store_row<T>(a, sink, row, tok0, ntok, second);
  }
}

template <int T, bool GENERAL, class SinkT, int G>
__device__ __forceinline__ void warp_rows_item(const MatmulArgs &a, const qmoe_matrix_desc &d, int row0, int nrows,
                                               int tok0, int ntok, typename SinkT::elem *xs) {
  stage_tokens<T, SinkT>(a, d.width, (d.width + 1) & ~1, tok0, ntok, xs);
  __syncthreads();
  warp_rows_staged<T, GENERAL, SinkT, G>(a, d, row0, nrows, tok0, ntok, xs, GlobalLookup{a.il_tab});
}

// grid.x = row blocks of a.rpc rows, grid.y = token groups of kMaxGroup tokens.
template <bool GENERAL>
__global__ void __launch_bounds__(kWarpRowThreads) k_matmul_warp_rows(const MatmulArgs a) {
  extern __shared__ __align__(16) float xs_f32[];
  const int row0 = blockIdx.x * a.rpc;
  const int nrows = min(a.rpc, a.single.height - row0);
  const int tok0 = blockIdx.y * kMaxGroup;
  const int ntok = min(kMaxGroup, a.tokens - tok0);
  if (ntok <= 1) warp_rows<1, GENERAL>(a, row0, nrows, tok0, ntok, xs_f32);
  else if (ntok == 2) warp_rows<2, GENERAL>(a, row0, nrows, tok0, ntok, xs_f32);
  else warp_rows<4, GENERAL>(a, row0, nrows, tok0, ntok, xs_f32);
}

constexpr unsigned long long kFusedWaitNs = 2000000000ull;  // an item of the second linear waits this long at most

// Persistent CTAs (one per SM) pulling items of a device-built work list.  Shared memory holds the
// hot part of the sparse table (loaded once per CTA) followed by the bf16 activations of the
// current item.
// AHEAD2: the CTA claims its items two ahead instead of one, which lets it stage the next item's
// activations early (below).  Claiming ahead fixes who gets the launch's last items by launch order
// instead of by who is free first: with a few items per SM that costs more than the staging saves
// (160 pairs of c-2048, wo: 260 us against 226 us), with twenty and more it does not show.  The
// host takes AHEAD2 for the large steps that run one launch per linear.
template <bool GENERAL, bool IL, bool AHEAD2 = false>
__global__ void __launch_bounds__(kGroupedThreads, 1) k_matmul_grouped(const MatmulArgs a) {
  extern __shared__ __align__(16) uint32_t smem_u32[];
  constexpr int kAhead = AHEAD2 ? 2 : 1, kSlots = kAhead + 1;
  __shared__ int s_item[kSlots];
  __shared__ int4 s_it[kSlots];
  __shared__ qmoe_matrix_desc s_desc[kSlots];
  uint32_t *hot = smem_u32;
  const uint32_t n_hot = IL ? (uint32_t)a.n_hot : kHotSlots;
  char *xs_base = reinterpret_cast<char *>(smem_u32 + n_hot);
  const int n_first = a.header[0];
  const int n_items = n_first + (a.fused ? a.header2[0] : 0);
  if (n_items <= 0) return;
  // items per (expert, token group) of either linear, written by k_build_work behind the counts
  const int per_pair_first = a.fused ? a.header[14] : 0, per_pair_second = a.fused ? a.header[15] : 1;
  using Lookup = typename std::conditional<IL, HotLookupLow, HotLookup>::type;
  Lookup lookup;
  if constexpr (IL) {
    // n_hot is a multiple of 1024 and both tables are 16-byte aligned
    for (uint32_t i = threadIdx.x; i < n_hot / 4; i += blockDim.x)
      reinterpret_cast<uint4 *>(hot)[i] = __ldg(reinterpret_cast<const uint4 *>(a.il_tab) + i);
    lookup = HotLookupLow{(uint32_t)__cvta_generic_to_shared(hot), a.il_tab, n_hot};
  } else {
    for (uint32_t i = threadIdx.x; i < kHotSlots; i += blockDim.x)
      hot[i] = __ldg(a.tab + (i < kHotLow ? i : i + (kHotHigh - kHotLow)));
    lookup = HotLookup{(uint32_t)__cvta_generic_to_shared(hot), a.tab};
  }
  // The CTA knows its next TWO items: their index, list entry and matrix descriptor sit in a ring of
  // three shared-memory slots.  They are fetched while the current item is worked on, by the CTA's
  // last thread (with rows sorted longest first it has the shortest row, or none): it issues the
  // fetch-counter atomic at the start of an item and completes the dependent loads after its own
  // row, so nobody waits for an atomic and two dependent global loads per item.
  // Knowing the next item also lets the threads that are done with their row stage its activations:
  // the activations of an item of one or two tokens take half of the area that four tokens need, so
  // two such items in a row (most of a step: items are ordered by token count) use the two halves in
  // turn, and the second one starts without loads, conversions or a barrier.
  auto fetch_index = [&]() { return atomicAdd(a.header + 1, 1); };
  auto publish = [&](int slot, int i) {
    s_item[slot] = i;
    if (i < n_items) {
      const bool sec = i >= n_first;
      const int4 it = sec ? a.items2[i - n_first] : a.items[i];
      s_it[slot] = it;
      s_desc[slot] = a.descs[it.x];
    }
  };
  const bool duty = threadIdx.x == blockDim.x - 1;
  if (duty) {
    publish(0, fetch_index());
    if (AHEAD2) publish(1, fetch_index());
  }
  __syncthreads();  // also orders the table fill before the first lookups
  bool staged = false;  // this item's activations were staged during the previous item
  int half = 0;         // which half of the area they are in (items of one or two tokens)
  for (int slot = 0;; slot = slot == kSlots - 1 ? 0 : slot + 1) {
    const int i = s_item[slot];
    if (i >= n_items) break;
    const int slot1 = slot == kSlots - 1 ? 0 : slot + 1;            // the next item (known at once only with AHEAD2)
    const int slot_new = AHEAD2 ? (slot1 == kSlots - 1 ? 0 : slot1 + 1) : slot1;  // where the item claimed now goes
    int later_index = 0;
    if (duty) later_index = fetch_index();
    const bool second = i >= n_first;
    const int j = second ? i - n_first : i;
    const int4 it = s_it[slot];
    const qmoe_matrix_desc d = s_desc[slot];
    const int nrows = it.w & 0x7fff, ntok = it.w >> 16;
    const int tail = (it.w & 0x8000) ? d.height - (it.y + nrows) : 0;
    const bool small = AHEAD2 && IL && ntok <= 2;
    if (!staged) half = 0;
    void *xs = xs_base + (small ? (size_t)half * a.x_half_bytes : 0);
    if (second && per_pair_first > 0) {
      // The hidden activations of this (expert, token group) come from the items of the first linear,
      // all of which were fetched before this one (one fetch order) by CTAs that are running: wait
      // until they have stored their rows.  The wait is bounded in time all the same; when it runs out
      // the status word is raised and the item goes ahead on whatever is there.
      if (threadIdx.x == 0) {
        const int *flag = a.done + j / per_pair_second;
        unsigned long long t0 = 0;
        for (unsigned spins = 0;; spins++) {
          int v;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
          if (v >= per_pair_first) break;
          unsigned long long t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
          if (spins == 0) t0 = t;
          if (t - t0 > kFusedWaitNs) {
            atomicAdd(a.wait_status, 1);
            break;
          }
          __nanosleep(100);
        }
      }
      __syncthreads();
    }
    // one token: fp32 activations (no conversion per gather); two and four: bf16, so that a gather
    // is one 4- or 8-byte shared load (two 4-byte words per lane cost twice the bank cycles)
    if (ntok <= 1)
      process_item<1, GENERAL, MatSink<1, true>, IL>(a, d, it.y, nrows, it.z, ntok, reinterpret_cast<float *>(xs), lookup,
                                                     tail, second, staged);
    else if (ntok == 2)
      process_item<2, GENERAL, MatSink<2, false>, IL>(a, d, it.y, nrows, it.z, ntok,
                                                      reinterpret_cast<__nv_bfloat16 *>(xs), lookup, tail, second, staged);
    else
      process_item<4, GENERAL, MatSink<4, false>, IL>(a, d, it.y, nrows, it.z, ntok,
                                                      reinterpret_cast<__nv_bfloat16 *>(xs), lookup, tail, second, staged);
    // This thread's rows are stored.  If this item and the CTA's next one both take half of the area,
    // help stage the next one's activations into the other half (its last reader was the item before
    // this one, which ended with a barrier).  Items of the second linear of a fused launch have to
    // wait for their input first and are staged when they start.
    bool next_staged = false;
    if (small) {
      const int i1 = s_item[slot1];
      if (i1 < n_first) {  // a valid item of the (first) linear
        const int4 nx = s_it[slot1];
        const int nt1 = nx.w >> 16;
        if (nt1 <= 2) {
          next_staged = true;
          const int w1 = s_desc[slot1].width, wl1 = (w1 + 1) & ~1;
          void *xn = xs_base + (size_t)(half ^ 1) * a.x_half_bytes;
          if (nt1 <= 1) stage_tokens<1, MatSink<1, true>>(a, w1, wl1, nx.z, nt1, reinterpret_cast<float *>(xn));
          else stage_tokens<2, MatSink<2, false>>(a, w1, wl1, nx.z, nt1, reinterpret_cast<__nv_bfloat16 *>(xn));
        }
      }
    }
    if (duty) publish(slot_new, later_index);
    __syncthreads();  // every row of the item is stored; the next item's activations and the newly claimed entry are in place
    if (a.fused && !second && threadIdx.x == 0) {
      __threadfence();  // the rows stored by the whole CTA (ordered by the barrier) before the count
      atomicAdd(a.done + j / per_pair_first, 1);
    }
    if (next_staged) half ^= 1;
    staged = next_staged;
  }
}

// Work items of an interleaved store whose rows are shared out one per WARP: the rows that are left
// when a matrix's height is not a multiple of the 1024 rows a CTA of k_matmul_grouped takes, and
// whole layers when so few experts are active (one token per step while generating) that rows per
// thread could not fill the GPU.  Several CTAs per SM; the table is read through L1/L2.
// G: groups of 32 codes per round of a row.  A row of w weights has about w / 23 codes; the host
// picks nine groups for wide matrices, so that a 6144-wide row (about 265 codes) is one round of
// dictionary lookups instead of three, and four otherwise (fewer registers, more CTAs per SM).
template <bool GENERAL, int G>
__global__ void __launch_bounds__(kWarpRowThreads) k_matmul_grouped_warp(const MatmulArgs a) {
  extern __shared__ __align__(16) uint32_t smem_u32[];
  const int n_items = a.header[0];
  // items are few and equal (eight rows each): a fixed assignment saves the fetch counter's latency
  for (int i = blockIdx.x; i < n_items; i += gridDim.x) {
    const int4 it = a.items[i];
    const qmoe_matrix_desc d = a.descs[it.x];
    const int nrows = it.w & 0xffff, ntok = it.w >> 16;
    if (ntok <= 1)
      warp_rows_item<1, GENERAL, MatSink<1, true>, G>(a, d, it.y, nrows, it.z, ntok, reinterpret_cast<float *>(smem_u32));
    else if (ntok == 2)
      warp_rows_item<2, GENERAL, MatSink<2, false>, G>(a, d, it.y, nrows, it.z, ntok,
                                                       reinterpret_cast<__nv_bfloat16 *>(smem_u32));
    else
      warp_rows_item<4, GENERAL, MatSink<4, false>, G>(a, d, it.y, nrows, it.z, ntok,
                                                       reinterpret_cast<__nv_bfloat16 *>(smem_u32));
    __syncthreads();  // xs is rewritten by the next round
  }
}

// Decode to ternary symbols, one thread per row.
template <bool GENERAL>
__global__ void k_decode(const uint32_t *__restrict__ tab, const int32_t *__restrict__ dec,
                         const uint16_t *__restrict__ codes, const int32_t *__restrict__ row_off,
                         uint8_t *__restrict__ sym, int32_t *status, int height, int width,
                         long long n_codes) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= height) return;
  const int mis = (int)((reinterpret_cast<uintptr_t>(codes) & 15u) >> 1);
  long long b = row_off[row], e = row_off[row + 1];
  const bool span_ok = b >= 0 && e >= b && e <= n_codes;
  b = b < 0 ? 0 : (b > n_codes ? n_codes : b);
  e = e < b ? b : (e > n_codes ? n_codes : e);
  SymbolSink sink{sym + (size_t)row * width, width};
  const int wlim = (width + 1) & ~1;
  const int pos = walk_row<GENERAL>(StreamFetch{codes - mis}, (int)b + mis, (int)e + mis, GlobalLookup{tab}, dec, wlim + 2, sink);
  if (status != nullptr && (pos != wlim || !span_ok)) atomicAdd(status, 1);
}

// ---- sparse table construction ------------------------------------------------------------------
__global__ void k_build_table(const int32_t *__restrict__ dec, uint32_t *__restrict__ tab,
                              int *nonconforming) {
  const int code = blockIdx.x * blockDim.x + threadIdx.x;
  if (code >= QMOE_DICT_COUNT) return;
  const uint32_t w0 = (uint32_t)dec[2 * code], w1 = (uint32_t)dec[2 * code + 1];
  const int len = (int)(w0 & 15u);
  bool ok = len >= 1 && len <= 14 && (int)(w1 & 15u) == len;
  uint32_t e = kEntryNull | (uint32_t)len;
  int nz = 0;
  for (int t = 0; t < 28; t++) {
    const uint32_t w = t < 14 ? w0 : w1;
    const uint32_t digit = (w >> (4 + 2 * (t % 14))) & 3u;
    if (digit == 0u) continue;
    if (t >= 2 * len || digit == 3u || nz == 3) { ok = false; break; }
    e &= ~(0xffu << (8 + 8 * nz));
    e |= (uint32_t)t << (8 + 8 * nz);
    if (digit == 2u) e |= 0x10u << nz;
    nz++;
  }
  if (!ok) {
    e = kEntryDense;  // decoded digit by digit from `dec`
    atomicAdd(nonconforming, 1);
  }
  tab[code] = e;
}

// ---- launchers ----------------------------------------------------------------------------------
static size_t smem_bytes(int width, int group) {
  const int wlim = (width + 1) & ~1;
  return (size_t)(wlim + kPad) * group * sizeof(float);
}
static size_t grouped_x_bytes(int width, int group) {
  const int wlim = (width + 1) & ~1;
  return (size_t)(wlim + kPad) * group * sizeof(__nv_bfloat16);
}
static size_t grouped_smem_bytes(int width, int group) {
  return sizeof(uint32_t) * kHotSlots + grouped_x_bytes(width, group);
}
// Interleaved stores: whatever the activations leave of the 227 KB goes to the table.
constexpr size_t kSmemPerCta = 232448 - 1024;  // opt-in limit minus static shared memory and slack
static int hot_entries_for(int width) {
  const size_t left = kSmemPerCta - grouped_x_bytes(width, kMaxGroup);
  size_t n = left / sizeof(uint32_t) / 1024 * 1024;
  return (int)(n > QMOE_DICT_COUNT ? QMOE_DICT_COUNT : n);
}

template <bool GENERAL>
static int set_smem_limits() {
  QMOE_CUDA(cudaFuncSetAttribute(k_matmul_uniform<GENERAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(QMOE_MAX_WIDTH, kMaxGroup)));
  QMOE_CUDA(cudaFuncSetAttribute(k_matmul_warp_rows<GENERAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_bytes(QMOE_MAX_WIDTH, kMaxGroup)));
  QMOE_CUDA(cudaFuncSetAttribute(k_matmul_grouped<GENERAL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)grouped_smem_bytes(QMOE_MAX_WIDTH, kMaxGroup)));
  QMOE_CUDA(cudaFuncSetAttribute(k_matmul_grouped<GENERAL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemPerCta));
  if constexpr (!GENERAL)
    QMOE_CUDA(cudaFuncSetAttribute((k_matmul_grouped<false, true, true>), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)kSmemPerCta));
  QMOE_CUDA(cudaFuncSetAttribute((k_matmul_grouped_warp<GENERAL, 4>), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)grouped_x_bytes(QMOE_MAX_WIDTH, kMaxGroup)));
  QMOE_CUDA(cudaFuncSetAttribute((k_matmul_grouped_warp<GENERAL, 9>), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)grouped_x_bytes(QMOE_MAX_WIDTH, kMaxGroup)));
  return QMOE_OK;
}

static int ensure_smem_limits(int device) {
  static bool done[64] = {false};
  if (device < 0 || device >= 64) {
    set_error("device index %d out of range", device);
    return QMOE_ERR_INVALID_ARG;
  }
  std::lock_guard<std::mutex> lock(setup_mutex());
  if (!done[device]) {
    int rc = set_smem_limits<false>();
    if (rc) return rc;
    rc = set_smem_limits<true>();
    if (rc) return rc;
    done[device] = true;
  }
  return QMOE_OK;
}

int launch_matmul_uniform(const SparseTable &tab, const int32_t *dec, const uint16_t *codes,
                          const int32_t *row_off, const void *minmax, const void *x, void *y, int height,
                          int width, int64_t n_codes, int tokens, int64_t x_stride, int64_t y_stride,
                          int flags, int device, cudaStream_t stream) {
  int rc = ensure_smem_limits(device);
  if (rc) return rc;
  MatmulArgs a{};
  a.tab = tab.entries;
  a.dec = dec;
  a.codes = codes;
  a.row_off = row_off;
  a.minmax = reinterpret_cast<const __nv_bfloat162 *>(minmax);
  a.single.code_base = 0;
  a.single.n_codes = n_codes;
  a.single.rowoff_base = 0;
  a.single.minmax_base = 0;
  a.single.height = height;
  a.single.width = width;
  a.x = reinterpret_cast<const __nv_bfloat16 *>(x);
  a.y = reinterpret_cast<__nv_bfloat16 *>(y);
  a.x_stride = x_stride;
  a.y_stride = y_stride;
  a.tokens = tokens;
  a.flags = flags;
  const int groups = (tokens + kMaxGroup - 1) / kMaxGroup;
  const int group = tokens >= 3 ? 4 : tokens;
  const size_t smem = smem_bytes(width, group);
  // rows per CTA: a multiple of the CTA's eight warps, aiming at up to eight CTAs per SM
  const int warps = kWarpRowThreads / 32;
  const int target = 8 * sm_count(device);
  int rpc = (height + target - 1) / target;
  rpc = (rpc + warps - 1) / warps * warps;
  a.rpc = rpc;
  a.chunks = (height + rpc - 1) / rpc;
  const dim3 grid((unsigned)a.chunks, (unsigned)groups);
  if (tab.conforming)
    QMOE_LAUNCH(k_matmul_warp_rows<false>, grid, kWarpRowThreads, smem, stream, a);
  else
    QMOE_LAUNCH(k_matmul_warp_rows<true>, grid, kWarpRowThreads, smem, stream, a);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_decode(const SparseTable &tab, const int32_t *dec, const uint16_t *codes, const int32_t *row_off,
                  uint8_t *sym, int32_t *status, int height, int width, int64_t n_codes,
                  cudaStream_t stream) {
  QMOE_CUDA(cudaMemsetAsync(sym, 0, (size_t)height * width, stream));
  if (status != nullptr) QMOE_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  const int threads = 128;
  const int blocks = (height + threads - 1) / threads;
  if (tab.conforming)
    QMOE_LAUNCH(k_decode<false>, blocks, threads, 0, stream, tab.entries, dec, codes, row_off, sym, status, height, width, n_codes);
  else
    QMOE_LAUNCH(k_decode<true>, blocks, threads, 0, stream, tab.entries, dec, codes, row_off, sym, status, height, width, n_codes);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_build_table(const int32_t *dec, uint32_t *tab, int *nonconforming, cudaStream_t stream) {
  QMOE_CUDA(cudaMemsetAsync(nonconforming, 0, sizeof(int), stream));
  QMOE_LAUNCH(k_build_table, QMOE_DICT_COUNT / 256, 256, 0, stream, dec, tab, nonconforming);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

// ---- renumbering of code values --------------------------------------------------------------------
__global__ void k_code_histogram(const uint16_t *__restrict__ codes, long long n,
                                 unsigned long long *__restrict__ hist) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    atomicAdd(hist + codes[i], 1ull);
}

// dec_out[2 * remap[c] + i] = dec[2 * c + i]: the reference table in the order of the new code values.
__global__ void k_permute_dec(const int32_t *__restrict__ dec, const uint32_t *__restrict__ remap,
                              int32_t *__restrict__ dec_out, int *bad) {
  const int code = blockIdx.x * blockDim.x + threadIdx.x;
  if (code >= QMOE_DICT_COUNT) return;
  const uint32_t to = remap != nullptr ? remap[code] : (uint32_t)code;
  if (to >= (uint32_t)QMOE_DICT_COUNT) {
    atomicAdd(bad, 1);
    return;
  }
  dec_out[2 * to] = dec[2 * code];
  dec_out[2 * to + 1] = dec[2 * code + 1];
}

int launch_code_histogram(const uint16_t *codes, int64_t n, uint64_t *hist, cudaStream_t stream) {
  QMOE_LAUNCH(k_code_histogram, 148 * 8, 256, 0, stream, codes, (long long)n,
              reinterpret_cast<unsigned long long *>(hist));
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

// Entries of dec_out that no code was mapped to (remap is not a permutation) keep length 0.
__global__ void k_count_unset(const int32_t *__restrict__ dec_out, const int32_t *__restrict__ dec, int *bad) {
  const int code = blockIdx.x * blockDim.x + threadIdx.x;
  if (code >= QMOE_DICT_COUNT) return;
  if (dec_out[2 * code] == 0 && dec_out[2 * code + 1] == 0) atomicAdd(bad, 1);
  if (dec[2 * code] == 0 && dec[2 * code + 1] == 0) atomicSub(bad, 1);  // all-zero words of the source itself
}

// scratch2[0] := number of out-of-range or colliding targets, scratch2[1] := non-conforming entries.
int launch_remap_tables(const int32_t *dec, const uint32_t *remap, uint32_t *tab_out, int32_t *dec_out,
                        int *scratch2, cudaStream_t stream) {
  QMOE_CUDA(cudaMemsetAsync(scratch2, 0, 2 * sizeof(int), stream));
  QMOE_CUDA(cudaMemsetAsync(dec_out, 0, sizeof(int32_t) * 2 * QMOE_DICT_COUNT, stream));
  QMOE_LAUNCH(k_permute_dec, QMOE_DICT_COUNT / 256, 256, 0, stream, dec, remap, dec_out, scratch2);
  QMOE_CUDA(cudaGetLastError());
  QMOE_LAUNCH(k_count_unset, QMOE_DICT_COUNT / 256, 256, 0, stream, dec_out, dec, scratch2);
  QMOE_CUDA(cudaGetLastError());
  QMOE_LAUNCH(k_build_table, QMOE_DICT_COUNT / 256, 256, 0, stream, dec_out, tab_out, scratch2 + 1);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

// ---- lane-interleaved code streams ----------------------------------------------------------------
// One-time re-layout of a store's code streams for the grouped kernel.  Rows are taken in blocks of
// 32 (one warp); inside a block, chunk k (codes 8k .. 8k+7) of row l is the uint4 at index
// k * 32 + l, so the 32 lanes of a warp read 512 contiguous bytes per step instead of 32 separate
// cache lines.  Every row of a block is padded with zero codes to the block's longest row, rounded
// up to a whole chunk; the row lengths still come from row_off.  Heights must be multiples of 32.
// `rows` (optional): the row of its matrix that every position of the store holds (a permutation of
// the rows inside each matrix); blocks are then made of the rows at 32 consecutive positions.
__device__ __forceinline__ int row_at(const int32_t *__restrict__ rows, const qmoe_matrix_desc &d, int pos) {
  if (rows == nullptr) return pos;
  const int r = rows[d.minmax_base + pos];
  return r < 0 ? 0 : (r >= d.height ? d.height - 1 : r);
}

__global__ void k_interleave_count(const int32_t *__restrict__ row_off, const qmoe_matrix_desc *__restrict__ descs,
                                   const int32_t *__restrict__ rows, int32_t *__restrict__ blk_units) {
  const qmoe_matrix_desc d = descs[blockIdx.x];
  const int32_t *ro = row_off + d.rowoff_base;
  for (int blk = threadIdx.x; blk < d.height / 32; blk += blockDim.x) {
    int longest = 0;
    for (int l = 0; l < 32; l++) {
      const int r = row_at(rows, d, blk * 32 + l);
      const int n = ro[r + 1] - ro[r];
      longest = n > longest ? n : longest;
    }
    blk_units[d.minmax_base / 32 + blk] = (longest + 7) / 8 * 32;  // uint4 entries of this block
  }
}

__global__ void k_interleave_emit(const uint16_t *__restrict__ codes, const int32_t *__restrict__ row_off,
                                  const qmoe_matrix_desc *__restrict__ descs,
                                  const int32_t *__restrict__ rows, const long long *__restrict__ blk_base,
                                  const uint32_t *__restrict__ remap, uint4 *__restrict__ il) {
  const qmoe_matrix_desc d = descs[blockIdx.y];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int32_t *ro = row_off + d.rowoff_base;
  const uint16_t *src = codes + d.code_base;
  for (int blk = blockIdx.x * nwarps + warp; blk < d.height / 32; blk += gridDim.x * nwarps) {
    const long long gblk = d.minmax_base / 32 + blk;
    const long long first = blk_base[gblk];
    const int chunks = (int)((blk_base[gblk + 1] - first) >> 5);
    const int r = row_at(rows, d, blk * 32 + lane);
    long long b = ro[r], e = ro[r + 1];
    b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
    e = e < b ? b : (e > d.n_codes ? d.n_codes : e);
    for (int k = 0; k < chunks; k++) {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const long long idx = b + 8 * k + j;
        uint32_t code = idx < e ? src[idx] : 0u;
        if (remap != nullptr) code = __ldg(remap + code) & 0xffffu;
        w[j >> 1] |= code << (16 * (j & 1));
      }
      il[first + (long long)k * 32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

int launch_interleave_count(const int32_t *row_off, const qmoe_matrix_desc *descs, int n_matrices,
                            const int32_t *rows, int32_t *blk_units, cudaStream_t stream) {
  QMOE_LAUNCH(k_interleave_count, (unsigned)n_matrices, 256, 0, stream, row_off, descs, rows, blk_units);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

int launch_interleave_emit(const uint16_t *codes, const int32_t *row_off, const qmoe_matrix_desc *descs,
                           int n_matrices, const int32_t *rows, const int64_t *blk_base, const uint32_t *remap,
                           void *il, cudaStream_t stream) {
  const int per_pass = 32768;  // grid.y limit is 65535
  for (int m0 = 0; m0 < n_matrices; m0 += per_pass) {
    const int n = n_matrices - m0 < per_pass ? n_matrices - m0 : per_pass;
    QMOE_LAUNCH(k_interleave_emit, dim3(8, (unsigned)n), 256, 0, stream, codes, row_off, descs + m0, rows,
                reinterpret_cast<const long long *>(blk_base), remap, reinterpret_cast<uint4 *>(il));
    QMOE_CUDA(cudaGetLastError());
  }
  return QMOE_OK;
}

// ---- grouped expert FFN -------------------------------------------------------------------------
// Work buffer layout: int header[16] | int4 items_wi[cap] | int4 items_wo[cap] | tile items of wi |
// tile items of wo | warp items of wi | warp items of wo | int done[max_slots] (finished wi items per
// (expert, token group), for the launch that runs both linears).
// header[0] = number of wi items, [1] = wi fetch counter (the only one of a fused launch), [2] = number
// of wo items, [3] = wo counter, [4] / [5] = tile items of wi / wo, [6] / [7] = rows per item of wi /
// wo, [9] = tokens decoded together, [10] .. [13] = counts and fetch counters of the warp items of wi
// and wo, [14] / [15] = per-thread items per (expert, token group) of wi / wo.
//
// Who takes which rows is decided here, on the device, from the number of (expert, token group)
// pairs.  A full layer (hundreds of pairs) is cut into items of up to 1024 rows for
// k_matmul_grouped, one row per thread of its persistent CTAs.  With an interleaved store, rows that
// do not fill such an item (heights like 2080 = 2 x 1024 + 32) are done one per warp by the CTA that
// takes the matrix's last item, and when so few pairs exist (one token per step while generating)
// that rows per thread could not fill the SMs, everything goes to k_matmul_grouped_warp in items of
// 32 rows.  In between, the items are made finer than 1024 rows
// until there are about two per SM.  Without an interleaved store there is no warp kernel.
constexpr int kExtraItems = 8192;
// Fixed cost of a work item in rows of work.  A thread walks its row at the latency of the dependent
// lookups and gathers, so an item of 128 rows takes more than half the time of one of 1024 (measured
// on 160 pairs of c-2048: 43 us against 74 us for wo, 18 us against 31 us for wi): finer items only
// pay when they save a whole round of the SMs.
constexpr int kItemOverheadRows = 1024;
constexpr int kWarpItemRows = 8;             // one row per warp of a k_matmul_grouped_warp CTA
constexpr int kWarpRemainderMax = 256;      // most rows of a matrix that are left to the warp kernel
constexpr int kSmallRows = 148 * 8 * 32;    // fewer rows in total (less than eight warps of rows per SM):
                                            // the warp kernel takes all of them

struct WorkPhase {
  int4 *items;
  int capacity;  // entries available in `items`
  int4 *warp_items;
  int warp_capacity;
  int height;    // rows of the phase's matrices (d_ff for wi, d_model for wo)
  int which;     // 0 = wi (matrix 2e), 1 = wo (matrix 2e + 1)
};

__global__ void __launch_bounds__(1024) k_build_work(const int32_t *__restrict__ offsets, int n_experts,
                                                     int max_slots, int tile_min, int sms,
                                                     int use_warp, int *header, WorkPhase p0, WorkPhase p1,
                                                     int forced_wi, int forced_wo, int *done) {
  __shared__ int s_warp[32];
  __shared__ int s_base;
  __shared__ int s_total;
  __shared__ unsigned long long s_best;
  __shared__ int s_cls[kMaxGroup];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  auto group_count = [&](int e, int &first, int &count) {
    first = 0;
    count = 0;
    if (e < n_experts) {
      first = offsets[e];
      count = offsets[e + 1] - first;
      count = count < 0 ? 0 : count;
      if (tile_min > 0 && count >= tile_min) count = 0;  // handled by the tensor-core tile path
    }
    return (count + kMaxGroup - 1) / kMaxGroup;
  };
  // pass 1: total number of (expert, token group) pairs, and how many of them have 1, 2, 3, 4 tokens
  if (tid == 0) s_total = 0;
  if (tid < kMaxGroup) s_cls[tid] = 0;
  __syncthreads();
  {
    int mine = 0, first, count, per_cls[kMaxGroup] = {};
    for (int e = tid; e < n_experts; e += blockDim.x) {
      mine += group_count(e, first, count);
      per_cls[kMaxGroup - 1] += count / kMaxGroup;
      if (count % kMaxGroup) per_cls[count % kMaxGroup - 1] += 1;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0 && mine) atomicAdd(&s_total, mine);
#pragma unroll
    for (int c = 0; c < kMaxGroup; c++) {
      int v = per_cls[c];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && v) atomicAdd(&s_cls[c], v);
    }
  }
  __syncthreads();
  const int total = min(s_total, max_slots);
  for (int g = tid; g < total; g += blockDim.x) done[g] = 0;  // finished first-linear items per pair

  // ---- how either linear is cut ----------------------------------------------------------------
  int rpc_of[2], main_of[2], chunks_of[2], wchunks_of[2], tail_of[2];
  for (int phase = 0; phase < 2; phase++) {
    const WorkPhase &p = phase == 0 ? p0 : p1;
    const int H = p.height;
    // rows [0, main_rows) in items of rpc rows for the per-thread kernel, the rest in warp items
    int rpc = rows_per_chunk_dev(H, kGroupedThreads), main_rows = H;
    if (use_warp && (long long)total * H <= kSmallRows) {
      main_rows = 0;
    } else if (total > 0) {
      const int rest = H % kGroupedThreads;
      if (use_warp && H >= kGroupedThreads && rest != 0 && rest <= kWarpRemainderMax) main_rows = H - rest;
      // c equal items per pair: the c whose whole rounds of the SMs cost least.  Candidate c0 + tid is
      // priced by thread tid; the cheapest (the smallest c among equals) wins.
      const int c0 = (main_rows + kGroupedThreads - 1) / kGroupedThreads;
      if (tid == 0) s_best = ~0ull;
      __syncthreads();
      if (tid <= 64) {
        const int c = c0 + tid;
        if (c * 32 <= main_rows || tid == 0) {
          const int rows = ((main_rows + c - 1) / c + 31) / 32 * 32;
          const int per_pair = (main_rows + rows - 1) / rows;
          if (tid == 0 || (long long)total * per_pair <= p.capacity) {
            const unsigned long long rounds = ((unsigned long long)total * per_pair + sms - 1) / sms;
            const unsigned long long cost = rounds * (unsigned long long)(rows + kItemOverheadRows);
            atomicMin(&s_best, (cost << 24) | ((unsigned long long)tid << 16) | (unsigned long long)rows);
          }
        }
      }
      __syncthreads();
      int best_rows = (int)(s_best & 0xffffull);
      const int forced = phase == 0 ? forced_wi : forced_wo;  // measurements: a given number of items per matrix
      if (forced > 0 && forced * 32 <= main_rows && (long long)total * forced <= p.capacity)
        best_rows = ((main_rows + forced - 1) / forced + 31) / 32 * 32;
      rpc = best_rows;
      __syncthreads();  // s_best is reset for the other linear
    }
    rpc_of[phase] = rpc;
    main_of[phase] = main_rows;
    chunks_of[phase] = (main_rows + rpc - 1) / rpc;
    // what is left after the per-thread items: with none of those, items for the warp kernel;
    // otherwise the CTA that takes the last per-thread item does them, one row per warp (bit 15)
    wchunks_of[phase] = main_rows == 0 ? (H + kWarpItemRows - 1) / kWarpItemRows : 0;
    tail_of[phase] = main_rows > 0 && main_rows < H ? 0x8000 : 0;
  }

  // ---- the items ---------------------------------------------------------------------------------
  // Longest items first: the groups of four tokens of all experts, then those of three, two and one
  // (an item's time grows with its tokens, and with a handful of items per SM the order in which the
  // CTAs fetch them decides how uneven the last round is).  The pairs get the same index in both
  // linears.
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int cls = kMaxGroup; cls >= 1; cls--) {
    if (s_cls[cls - 1] == 0) continue;  // no group of this size in the step (one token: three of four passes)
    for (int e0 = 0; e0 < n_experts; e0 += blockDim.x) {
      const int e = e0 + tid;
      int first, count;
      group_count(e, first, count);
      const int full = count / kMaxGroup, rem = count % kMaxGroup;
      const int groups = cls == kMaxGroup ? full : (rem == cls ? 1 : 0);
      const int first_tok = cls == kMaxGroup ? first : first + full * kMaxGroup;
      // exclusive scan of `groups` over the block
      int incl = groups;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (lane == 31) s_warp[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        int w = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, w, o);
          if (lane >= o) w += v;
        }
        s_warp[lane] = w;
      }
      __syncthreads();
      const int base = s_base + (warp ? s_warp[warp - 1] : 0) + incl - groups;
      for (int phase = 0; phase < 2; phase++) {
        const WorkPhase &p = phase == 0 ? p0 : p1;
        const int H = p.height, rpc = rpc_of[phase], main_rows = main_of[phase], chunks = chunks_of[phase];
        const int wchunks = wchunks_of[phase], tail_flag = tail_of[phase];
        // Items for the per-thread kernel (a few per group): every lane writes those of its expert.
        for (int g = 0; g < groups && chunks > 0; g++) {
          const int gi = base + g;
          if (gi >= max_slots || (long long)(gi + 1) * chunks > p.capacity) break;  // cannot happen for valid offsets
          const int tok0 = first_tok + g * kMaxGroup;
          for (int k = 0; k < chunks; k++) {
            const int row0 = k * rpc;
            p.items[(size_t)gi * chunks + k] =
                make_int4(2 * e + p.which, row0, tok0,
                          min(rpc, main_rows - row0) | (k == chunks - 1 ? tail_flag : 0) | (cls << 16));
          }
        }
        // Items for the warp kernel (hundreds per group, but only in steps with a handful of groups):
        // the whole warp writes those of each lane's expert in turn.
        unsigned busy = __ballot_sync(0xffffffffu, groups > 0 && wchunks > 0);
        while (busy) {
          const int src = __ffs(busy) - 1;
          busy &= busy - 1;
          const int o_e = __shfl_sync(0xffffffffu, e, src), o_first = __shfl_sync(0xffffffffu, first_tok, src);
          const int o_groups = __shfl_sync(0xffffffffu, groups, src);
          const int o_base = __shfl_sync(0xffffffffu, base, src);
          for (int g = 0; g < o_groups; g++) {
            const int gi = o_base + g;
            if (gi >= max_slots || (long long)(gi + 1) * wchunks > p.warp_capacity) break;
            const int tok0 = o_first + g * kMaxGroup;
            for (int k = lane; k < wchunks; k += 32) {
              const int row0 = k * kWarpItemRows;
              p.warp_items[(size_t)gi * wchunks + k] =
                  make_int4(2 * o_e + p.which, row0, tok0, min(kWarpItemRows, H - row0) | (cls << 16));
            }
          }
        }
      }
      __syncthreads();
      if (tid == 0) s_base += s_warp[31];
      __syncthreads();
    }
  }
  if (tid == 0) {
    const int groups_done = min(s_base, max_slots);
    for (int phase = 0; phase < 2; phase++) {
      header[2 * phase] = groups_done * chunks_of[phase];
      header[2 * phase + 1] = 0;
      header[10 + 2 * phase] = groups_done * wchunks_of[phase];
      header[11 + 2 * phase] = 0;
      header[6 + phase] = rpc_of[phase];      // rows per item of this phase (reports)
      header[14 + phase] = chunks_of[phase];  // per-thread items per (expert, token group) of this phase
    }
    header[9] = kMaxGroup;
  }
}

// Tensor-core tile path (sub1_tile.cu).
int64_t tile_work_bytes(int max_slots, int d_model, int d_ff);
int tile_cap_blocks(int max_slots);
int launch_build_tile_work(const int32_t *offsets, int n_experts, int tile_min, int d_model, int d_ff,
                           int max_slots, int *header, int4 *items_wi, int4 *items_wo, cudaStream_t stream);
int launch_tile_phase(const uint32_t *tab, const uint16_t *codes, const int32_t *row_off, const void *minmax,
                      const qmoe_matrix_desc *descs, const void *x, void *y, long long x_stride, long long y_stride,
                      const int32_t *x_rows, const int32_t *y_rows, const unsigned long long *y_ptrs, const int4 *items,
                      const int *n_items, int flags, int max_items, int device, cudaStream_t stream);

// Experts with at least this many tokens take the tile path (0 disables it).  The default is the
// measured break-even on a switch-large-128 layer with a skewed router (eight hot experts share half
// of the tokens): at about 140 tokens per hot expert the per-row kernel (36 passes of four tokens) is
// still faster, 0.67 ms against 0.79 ms per layer; at about 560 tokens the tile path wins, 2.16 ms
// against 2.41 ms; at about 2200 tokens, 5.05 ms against 6.96 ms.  The environment variable exists
// for such measurements.
static std::atomic<int> g_tile_min{-1};  // -1: not yet initialised from the environment
static int clamp_tile_min(int t) { return t <= 0 ? 0 : (t < 8 ? 8 : t); }
static int tile_min_tokens() {
  int v = g_tile_min.load(std::memory_order_relaxed);
  if (v < 0) {
    const char *s = getenv("QMOE_TILE_MIN_TOKENS");
    v = clamp_tile_min(s ? atoi(s) : 448);
    g_tile_min.store(v, std::memory_order_relaxed);
  }
  return v;
}
// Both linears' per-thread items in one launch (qmoe_moe_set_fused_phases; default on).
static std::atomic<int> g_fused_phases{1};
int set_fused_phases(int on) { return g_fused_phases.exchange(on != 0 ? 1 : 0, std::memory_order_relaxed); }

// Items per matrix forced by qmoe_moe_set_items_per_matrix (0: chosen on the device).
static std::atomic<int> g_forced_items[2] = {{0}, {0}};
void set_items_per_matrix(int wi, int wo) {
  g_forced_items[0].store(wi > 0 ? wi : 0, std::memory_order_relaxed);
  g_forced_items[1].store(wo > 0 ? wo : 0, std::memory_order_relaxed);
}

int set_tile_min_tokens(int tokens) {
  const int before = tile_min_tokens();
  g_tile_min.store(clamp_tile_min(tokens), std::memory_order_relaxed);
  return before;
}

static int64_t item_capacity(int max_slots, int height) {
  return (int64_t)max_slots * chunk_count(height, kGroupedThreads) + kExtraItems;
}

static int64_t warp_item_capacity(int max_slots) {
  (void)max_slots;  // only steps with at most kSmallRows rows use warp items
  return kSmallRows / kWarpItemRows + kExtraItems;
}

int64_t moe_work_bytes(int max_slots, int d_model, int d_ff) {
  return 64 + (item_capacity(max_slots, d_ff) + item_capacity(max_slots, d_model) +
               2 * warp_item_capacity(max_slots)) * (int64_t)sizeof(int4) +
         tile_work_bytes(max_slots, d_model, d_ff) + ((int64_t)max_slots * 4 + 15) / 16 * 16;
}

// What the last qmoe_moe_grouped_ffn call with this work buffer planned (a host read-back for tests
// and reports): out[0] / out[1] = per-thread items of wi / wo, out[2] / out[3] = row-per-warp items
// of wi / wo, out[4] / out[5] = rows per per-thread item of wi / wo, out[6] / out[7] = tile items of
// wi / wo, out[8] = tokens decoded together, out[9] = wo items whose CTA also does the matrix's
// remainder rows one per warp.
int work_summary(const void *work, int max_slots, int d_ff, int32_t *out, cudaStream_t stream) {
  int header[16];
  QMOE_CUDA(cudaMemcpyAsync(header, work, sizeof(header), cudaMemcpyDeviceToHost, stream));
  QMOE_CUDA(cudaStreamSynchronize(stream));
  const int64_t cap_wi = item_capacity(max_slots, d_ff);
  int n_wo = header[2];
  n_wo = n_wo < 0 ? 0 : n_wo;
  std::vector<int4> items((size_t)n_wo);
  if (n_wo > 0) {
    const char *base = reinterpret_cast<const char *>(work) + 64 + cap_wi * sizeof(int4);
    QMOE_CUDA(cudaMemcpyAsync(items.data(), base, sizeof(int4) * (size_t)n_wo, cudaMemcpyDeviceToHost, stream));
    QMOE_CUDA(cudaStreamSynchronize(stream));
  }
  int flagged = 0;
  for (const int4 &it : items) flagged += (it.w & 0x8000) ? 1 : 0;
  out[0] = header[0];
  out[1] = header[2];
  out[2] = header[10];
  out[3] = header[12];
  out[4] = header[6];
  out[5] = header[7];
  out[6] = header[4];
  out[7] = header[5];
  out[8] = header[9];
  out[9] = flagged;
  return QMOE_OK;
}

int launch_grouped_ffn(const SparseTable &tab, const int32_t *dec, const uint16_t *codes,
                       const int32_t *row_off, const void *minmax, const qmoe_matrix_desc *descs,
                       const qmoe_interleaved_store *ils, const int32_t *offsets, const void *xs,
                       int64_t xs_stride, const int32_t *x_rows, void *hs, void *ys, int64_t ys_stride,
                       const int32_t *y_rows, const unsigned long long *y_ptrs, void *work, int n_experts,
                       int max_slots, int d_model, int d_ff, int device, cudaStream_t stream) {
  int rc = ensure_smem_limits(device);
  if (rc) return rc;
  const int sms = sm_count(device);
  int *header = reinterpret_cast<int *>(work);
  WorkPhase ph[2];
  ph[0].items = reinterpret_cast<int4 *>(reinterpret_cast<char *>(work) + 64);
  ph[0].capacity = (int)item_capacity(max_slots, d_ff);
  ph[0].height = d_ff;
  ph[0].which = 0;
  ph[1].items = ph[0].items + ph[0].capacity;
  ph[1].capacity = (int)item_capacity(max_slots, d_model);
  ph[1].height = d_model;
  ph[1].which = 1;
  int4 *tile_wi = ph[1].items + ph[1].capacity;
  int4 *tile_wo = tile_wi + (size_t)tile_cap_blocks(max_slots) * ((d_ff + 127) / 128);
  ph[0].warp_items = tile_wo + (size_t)tile_cap_blocks(max_slots) * ((d_model + 127) / 128);
  ph[0].warp_capacity = ph[1].warp_capacity = (int)warp_item_capacity(max_slots);
  ph[1].warp_items = ph[0].warp_items + ph[0].warp_capacity;
  int *done = reinterpret_cast<int *>(ph[1].warp_items + ph[1].warp_capacity);  // int[max_slots]
  const bool il = ils != nullptr;
  // The tile path decodes the row-by-row streams; a store that kept only its interleaved copy
  // (codes == nullptr) sends every expert through the per-row kernel.
  // max_slots bounds the tokens of the step, so launches that cannot get work are left out: the
  // tile path when no expert can reach its threshold, the per-thread kernel when the step is small
  // enough for the warp kernel whatever the routing (see k_build_work).
  int tile_min = tab.conforming && codes != nullptr ? tile_min_tokens() : 0;
  if (tile_min > max_slots) tile_min = 0;
  QMOE_LAUNCH(k_build_work, 1, 1024, 0, stream, offsets, n_experts, max_slots, tile_min, sms, il ? 1 : 0,
              header, ph[0], ph[1], g_forced_items[0].load(std::memory_order_relaxed),
              g_forced_items[1].load(std::memory_order_relaxed), done);
  QMOE_CUDA(cudaGetLastError());
  if (tile_min > 0) {
    rc = launch_build_tile_work(offsets, n_experts, tile_min, d_model, d_ff, max_slots, header, tile_wi, tile_wo, stream);
    if (rc) return rc;
  }

  MatmulArgs a{};
  a.tab = tab.entries;
  a.dec = dec;
  a.codes = codes;
  a.row_off = row_off;
  a.minmax = reinterpret_cast<const __nv_bfloat162 *>(minmax);
  a.descs = descs;
  if (il) {
    a.il = reinterpret_cast<const uint4 *>(ils->codes);
    a.blk_base = reinterpret_cast<const long long *>(ils->blk_base);
    a.il_tab = ils->table;
    a.il_dec = ils->dec;
    a.il_rows = ils->rows;
  }
  cudaEvent_t *events = nullptr;
  const bool timed = profile_begin(device, &events);

  // what either linear reads, writes and works through
  MatmulArgs pa[2];
  size_t smem_of[2];
  for (int phase = 0; phase < 2; phase++) {
    const int width = phase == 0 ? d_model : d_ff;
    MatmulArgs &p = pa[phase];
    p = a;
    p.x = reinterpret_cast<const __nv_bfloat16 *>(phase == 0 ? xs : hs);
    p.y = reinterpret_cast<__nv_bfloat16 *>(phase == 0 ? hs : ys);
    p.x_stride = phase == 0 ? xs_stride : width;
    p.y_stride = phase == 0 ? d_ff : ys_stride;
    p.x_rows = phase == 0 ? x_rows : nullptr;   // the hidden activation in between is indexed by slot
    p.y_rows = phase == 0 ? nullptr : y_rows;
    p.y_ptrs = phase == 0 ? nullptr : y_ptrs;
    p.items = ph[phase].items;
    p.header = header + 2 * phase;
    p.flags = phase == 0 ? QMOE_FLAG_RELU : 0;
    p.x_half_bytes = (unsigned)(grouped_x_bytes(width, kMaxGroup) / 2);
    p.n_hot = hot_entries_for(width);
    smem_of[phase] = il ? sizeof(uint32_t) * p.n_hot + grouped_x_bytes(width, kMaxGroup)
                        : grouped_smem_bytes(width, kMaxGroup);
  }
  const unsigned grid = (unsigned)sms;  // the table in shared memory allows one CTA per SM
  auto launch_tiles = [&](int phase) -> int {
    if (tile_min <= 0) return QMOE_OK;
    const MatmulArgs &p = pa[phase];
    const int rows_blocks = ((phase == 0 ? d_ff : d_model) + 127) / 128;
    return launch_tile_phase(tab.entries, codes, row_off, minmax, descs, p.x, p.y, p.x_stride, p.y_stride, p.x_rows,
                             p.y_rows, p.y_ptrs, phase == 0 ? tile_wi : tile_wo, header + 4 + phase, p.flags,
                             tile_cap_blocks(max_slots) * rows_blocks, device, stream);
  };
  auto launch_threads = [&](const MatmulArgs &p, size_t smem, bool ahead2) -> int {
    if (tab.conforming && il && ahead2)
      QMOE_LAUNCH((k_matmul_grouped<false, true, true>), grid, kGroupedThreads, smem, stream, p);
    else if (tab.conforming && il)
      QMOE_LAUNCH((k_matmul_grouped<false, true>), grid, kGroupedThreads, smem, stream, p);
    else if (tab.conforming)
      QMOE_LAUNCH((k_matmul_grouped<false, false>), grid, kGroupedThreads, smem, stream, p);
    else if (il)
      QMOE_LAUNCH((k_matmul_grouped<true, true>), grid, kGroupedThreads, smem, stream, p);
    else
      QMOE_LAUNCH((k_matmul_grouped<true, false>), grid, kGroupedThreads, smem, stream, p);
    QMOE_CUDA(cudaGetLastError());
    return QMOE_OK;
  };
  auto launch_warps = [&](int phase) -> int {
    if (!il) return QMOE_OK;
    const int width = phase == 0 ? d_model : d_ff;
    MatmulArgs w = pa[phase];
    w.items = ph[phase].warp_items;
    w.header = header + 10 + 2 * phase;
    const size_t wsmem = grouped_x_bytes(width, kMaxGroup);
    int per_sm = (int)(kSmemPerCta / (wsmem + 1024));  // CTAs of 256 threads that fit one SM
    per_sm = per_sm > 8 ? 8 : (per_sm < 1 ? 1 : per_sm);
    const unsigned wgrid = (unsigned)(per_sm * sms);
    const bool long_rows = width > 3072;
    if (tab.conforming && long_rows)
      QMOE_LAUNCH((k_matmul_grouped_warp<false, 9>), wgrid, kWarpRowThreads, wsmem, stream, w);
    else if (tab.conforming)
      QMOE_LAUNCH((k_matmul_grouped_warp<false, 4>), wgrid, kWarpRowThreads, wsmem, stream, w);
    else if (long_rows)
      QMOE_LAUNCH((k_matmul_grouped_warp<true, 9>), wgrid, kWarpRowThreads, wsmem, stream, w);
    else
      QMOE_LAUNCH((k_matmul_grouped_warp<true, 4>), wgrid, kWarpRowThreads, wsmem, stream, w);
    QMOE_CUDA(cudaGetLastError());
    return QMOE_OK;
  };
  // every step this small goes to the warp kernel whatever the routing
  auto all_small = [&](int phase) { return il && (long long)max_slots * (phase == 0 ? d_ff : d_model) <= kSmallRows; };

  // The fused launch keeps the smaller of the two hot tables for both linears, which costs wi about
  // 1 % on a full layer (3.04 against 3.01 ms for 2048 tokens on 2048 experts) and saves 3 % when a
  // step has only a few items per SM (one rank of eight: 456 against 469 us): taken for steps of at
  // most eight token slots per SM.
  if (il && g_fused_phases.load(std::memory_order_relaxed) != 0 && max_slots <= 8 * sms) {
    // One launch for the per-thread items of both linears: the CTAs go from the last items of wi
    // straight to the first of wo instead of idling until the slowest has finished (with a few
    // hundred items on 148 SMs, as on one rank of eight, that idle part is a fifth of the time).
    // Tile and warp items keep their own launches: wi's before, wo's after.
    if ((rc = launch_tiles(0)) != QMOE_OK || (rc = launch_tiles(1)) != QMOE_OK) return rc;
    if (timed) QMOE_CUDA(cudaEventRecord(events[0], stream));
    if ((rc = launch_warps(0)) != QMOE_OK) return rc;
    if (!(all_small(0) && all_small(1))) {
      const int wide = d_model > d_ff ? d_model : d_ff;
      MatmulArgs f = pa[0];
      f.second.x = pa[1].x;
      f.second.y = pa[1].y;
      f.second.x_stride = pa[1].x_stride;
      f.second.y_stride = pa[1].y_stride;
      f.second.y_rows = pa[1].y_rows;
      f.second.y_ptrs = pa[1].y_ptrs;
      f.second.flags = pa[1].flags;
      f.items2 = pa[1].items;
      f.header2 = pa[1].header;
      f.done = done;
      f.wait_status = tile_status_word(device);
      if (f.wait_status == nullptr) return cuda_fail(cudaGetLastError(), "status word");
      f.fused = 1;
      f.x_half_bytes = (unsigned)(grouped_x_bytes(wide, kMaxGroup) / 2);
      f.n_hot = hot_entries_for(wide);
      if ((rc = launch_threads(f, sizeof(uint32_t) * f.n_hot + grouped_x_bytes(wide, kMaxGroup), false)) != QMOE_OK)
        return rc;
    }
    if ((rc = launch_warps(1)) != QMOE_OK) return rc;
    if (timed) {
      // one duration for both linears: reported as the first, the second reads as zero
      QMOE_CUDA(cudaEventRecord(events[1], stream));
      QMOE_CUDA(cudaEventRecord(events[2], stream));
      QMOE_CUDA(cudaEventRecord(events[3], stream));
    }
    return QMOE_OK;
  }

  for (int phase = 0; phase < 2; phase++) {
    if ((rc = launch_tiles(phase)) != QMOE_OK) return rc;
    if (timed) QMOE_CUDA(cudaEventRecord(events[2 * phase], stream));
    // steps of more than eight token slots per SM come here: claim two items ahead and stage early
    if (!all_small(phase) && (rc = launch_threads(pa[phase], smem_of[phase], max_slots > 8 * sms)) != QMOE_OK) return rc;
    if ((rc = launch_warps(phase)) != QMOE_OK) return rc;
    if (timed) QMOE_CUDA(cudaEventRecord(events[2 * phase + 1], stream));
  }
  return QMOE_OK;
}


// ---- matvec for callers that must not allocate --------------------------------------------------
// qmoe_sub1_matvec normally keeps its derived 4-byte dictionary in memory that the library obtains
// with cudaMalloc the first time it sees a `dec` pointer.  Some callers cannot tolerate that: code
// running under a framework that owns all device memory and forbids side allocations, a process
// whose memory budget is fully handed to a pool, or a host thread that must never block inside the
// driver's allocator.  For them the scratch lives in this fixed array, which is part of the
// library's device image: every GPU that loads the library carries these ~256 KB until the process
// exits, whether or not the entry point is ever used.
//
// The array is shared by every call on a device and keeps whatever the previous call left in it.
// Each call therefore rebuilds the dictionary from the `dec` it was given and clears the one word
// that has to start at zero (the malformed-entry counter), all on the caller's stream.  Two calls
// that are in flight on the same GPU at the same time (different streams or threads) write the
// array concurrently and race; callers serialise them.
constexpr size_t kNoAllocEntries = QMOE_DICT_COUNT;      // the derived dictionary, 4 bytes per code
constexpr size_t kNoAllocWords = kNoAllocEntries + 64;   // + the counter word (padded to 256 bytes)
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocWords];

// In host code the name g_noalloc_scratch is only a handle for the symbol, not a device address;
// the address each device gave the array is looked up once per device, with that device current.
static uint32_t *noalloc_scratch_address(int device, cudaError_t *err) {
  static uint32_t *address[64] = {nullptr};
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  *err = cudaSuccess;
  if (address[device] == nullptr) {
    void *p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (*err != cudaSuccess) return nullptr;
    address[device] = reinterpret_cast<uint32_t *>(p);
  }
  return address[device];
}

}  // namespace qmoe

extern "C" int qmoe_sub1_matvec_noalloc(const int32_t *dec_dev, const uint16_t *w_comp_dev,
                                        const int32_t *row_off_dev, const void *ter_minmax_dev,
                                        const void *x_dev, void *y_dev, int height, int width,
                                        int64_t n_codes, int device, void *stream_) {
  using namespace qmoe;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  QMOE_REQUIRE(dec_dev && row_off_dev && ter_minmax_dev && x_dev && y_dev && (w_comp_dev || n_codes == 0),
               "null device pointer");
  QMOE_REQUIRE(height >= 1 && width >= 1 && n_codes >= 0, "bad shape");
  QMOE_REQUIRE(device >= 0 && device < 64, "device index out of range");
  if (width > QMOE_MAX_WIDTH) {
    set_error("qmoe_sub1_matvec_noalloc: width %d is beyond the maximum of %d columns", width, QMOE_MAX_WIDTH);
    return QMOE_ERR_UNSUPPORTED;
  }
  if (n_codes >= (int64_t)1 << 31) {
    set_error("qmoe_sub1_matvec_noalloc: %lld codes are beyond the maximum of 2^31-1 per matrix",
              (long long)n_codes);
    return QMOE_ERR_UNSUPPORTED;
  }
  QMOE_REQUIRE((reinterpret_cast<uintptr_t>(w_comp_dev) & 1u) == 0 &&
                   (reinterpret_cast<uintptr_t>(row_off_dev) & 3u) == 0 &&
                   (reinterpret_cast<uintptr_t>(ter_minmax_dev) & 3u) == 0 &&
                   ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev)) & 1u) == 0,
               "misaligned pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  // First call on a device: resolves the scratch address and raises the kernels' shared-memory
  // limit.  Neither allocates, but both are set-up calls: make this first call outside any stream
  // capture.
  cudaError_t err;
  uint32_t *scratch = noalloc_scratch_address(device, &err);
  if (scratch == nullptr) return cuda_fail(err, "cudaGetSymbolAddress(g_noalloc_scratch)");
  int rc = ensure_smem_limits(device);
  if (rc) return rc;

  int *counter = reinterpret_cast<int *>(scratch + kNoAllocEntries);
  QMOE_CUDA(cudaMemsetAsync(counter, 0, sizeof(int), stream));
  QMOE_LAUNCH(k_build_table, QMOE_DICT_COUNT / 256, 256, 0, stream, dec_dev, scratch, counter);
  QMOE_CUDA(cudaGetLastError());

  MatmulArgs a{};
  a.tab = scratch;
  a.dec = dec_dev;
  a.codes = w_comp_dev;
  a.row_off = row_off_dev;
  a.minmax = reinterpret_cast<const __nv_bfloat162 *>(ter_minmax_dev);
  a.single.n_codes = n_codes;
  a.single.height = height;
  a.single.width = width;
  a.x = reinterpret_cast<const __nv_bfloat16 *>(x_dev);
  a.y = reinterpret_cast<__nv_bfloat16 *>(y_dev);
  a.x_stride = width;
  a.y_stride = height;
  a.chunks = chunk_count(height, kRowsPerItem);
  a.rpc = rows_per_chunk(height, kRowsPerItem);
  a.tokens = 1;
  a.flags = QMOE_FLAG_ACCUMULATE;
  // The kernel variant that can also decode malformed entries digit by digit: which entries are
  // malformed is known only on the device, and reading the counter back would need a synchronise.
  QMOE_LAUNCH(k_matmul_uniform<true>, (unsigned)a.chunks, kRowsPerItem, smem_bytes(width, 1), stream, a);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

namespace qmoe {
}  // namespace qmoe
