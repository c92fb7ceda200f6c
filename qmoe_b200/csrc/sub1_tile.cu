// Tensor-core tile path for experts that received many tokens (the skewed-router case): the rows of
// a compressed matrix are decoded ONCE into a dense bf16 tile in shared memory and multiplied with
// up to 64 tokens by tcgen05.mma, instead of being re-decoded for every group of four tokens.
//
//   D[128 rows, 64 tokens] (fp32, tensor memory)  +=  A[128 rows, 128 cols] * B[64 tokens, 128 cols]^T
//
// A holds the decoded weights {0, min_r, max_r} as bf16 (the reference's decode-then-bf16-matmul
// semantics, test.py:176), B the tokens' activations; both are written by ordinary shared stores in
// the K-major no-swizzle core-matrix layout (8 rows x 16 bytes per core matrix), so no tensor map
// and no bulk copy is involved.  One CTA owns 128 rows: thread r of its first warpgroup decodes row r
// (the same one-thread-per-row walk as the other kernels, restricted to a window of 128 columns per
// step) and later reads row r of the accumulator from tensor memory; a second warpgroup clears and
// fills the tiles one window ahead.
//
// Every wait on the MMA-completion mbarrier is bounded; on a timeout the CTA records an error,
// releases its tensor memory and returns.
#include "common.cuh"
#include "sub1_walk.cuh"

#include <atomic>

namespace qmoe {

constexpr int kTileM = 128;        // rows per CTA (== threads)
constexpr int kTileN = 64;         // token columns per item (zero padded)
constexpr int kTileK = 128;        // matrix columns decoded per step
constexpr int kTileChunks = kTileK / 8;
constexpr uint32_t kTmemCols = 64; // fp32 accumulator columns (power of two >= 32)
constexpr uint32_t kWaitLimit = 1u << 24;

// Bound of the waits that DECIDE whether a CTA gives up (tests lower it to 1, "do not poll at all",
// to make a wait run out without anything hanging; 0 = kWaitLimit).  The clean-up waits before tensor memory is
// released always get the full limit.
static std::atomic<uint32_t> g_wait_limit{0};
int set_tile_wait_limit(uint32_t spins) {
  g_wait_limit.store(spins, std::memory_order_relaxed);
  return QMOE_OK;
}

struct TileArgs {
  const uint32_t *tab;
  const uint16_t *codes;
  const int32_t *row_off;
  const __nv_bfloat162 *minmax;
  const qmoe_matrix_desc *descs;
  const __nv_bfloat16 *x;
  __nv_bfloat16 *y;
  long long x_stride, y_stride;
  const int32_t *x_rows, *y_rows;  // token t reads row x_rows[t] / writes row y_rows[t] (null: t)
  const unsigned long long *y_ptrs;  // optional: address of token t's output row (replaces y, y_stride, y_rows)
  const int4 *items;   // {matrix, first row, first token, tokens}
  const int *n_items;  // device scalar
  int *status;         // device word: incremented when a bounded wait gives up (sticky)
  int flags;
  uint32_t wait_limit; // spins of the waits that decide to give up
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor: K-major, no swizzle.  In 16-byte units: start address, leading
// byte offset = distance between the two 8-column halves of one K=16 step, stride byte offset =
// distance between groups of 8 rows; bits 46-47 = 1 (descriptor version of this architecture).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// Instruction descriptor of kind::f16: fp32 accumulate, bf16 x bf16, both K-major, M x N.
__device__ __forceinline__ uint32_t make_instr_desc(int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                    // accumulator format: F32
  d |= 1u << 7;                    // A format: BF16
  d |= 1u << 10;                   // B format: BF16
  d |= (uint32_t)(n >> 3) << 17;   // N / 8
  d |= (uint32_t)(m >> 4) << 24;   // M / 16
  return d;
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_addr, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t mbar_addr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_addr) : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t mbar_addr, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_addr), "r"(count) : "memory");
}
// Bounded wait for the phase with the given parity: at most limit - 1 polls (each of which may itself
// block for a short, hardware-defined time); false if they ran out.  A limit of 1 gives up at once.
__device__ __forceinline__ bool mbar_wait(uint32_t mbar_addr, uint32_t parity, uint32_t limit = kWaitLimit) {
  for (uint32_t i = 1; i < limit; i++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(mbar_addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 16 consecutive fp32 accumulator columns of this thread's row (lane) of tensor memory.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- kernel ---------------------------------------------------------------------------------------
constexpr int kTileThreads = 2 * kTileM;  // warps 0-3 decode rows, warps 4-7 stage the tiles

__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Two warpgroups and two shared-memory stages.  For window w (128 columns) and stage s = w & 1:
//   stagers  (threads 128..255): wait until the MMAs that read stage s two windows ago are complete,
//            zero the A tile, copy the tokens' activations into the B tile, signal "stage s filled";
//   decoders (threads 0..127):   wait for "stage s filled", scatter the non-zeros of their row into
//            the A tile, synchronise among themselves, and one thread issues the eight K=16 MMAs and
//            commits them to the stage's mbarrier.
// The stagers run up to one window ahead of the decoders, and the tensor core runs behind both.
__device__ __forceinline__ __nv_bfloat16 *out_row_ptr(const TileArgs &a, int tok) {
  if (a.y_ptrs != nullptr) return reinterpret_cast<__nv_bfloat16 *>(a.y_ptrs[tok]);
  const long long out_row = a.y_rows != nullptr ? a.y_rows[tok] : tok;
  return a.y + out_row * a.y_stride;
}

__global__ void __launch_bounds__(kTileThreads, 1) k_tile_matmul(const TileArgs a) {
  constexpr int kABytes = kTileChunks * kTileM * 16;  // [column chunk][row][8 bf16]
  constexpr int kBBytes = kTileChunks * kTileN * 16;  // [column chunk][token][8 bf16]
  constexpr int kBUnits = kTileChunks * kTileN / kTileM;
  extern __shared__ __align__(128) uint8_t tile_smem[];  // A stage 0 | A stage 1 | B stage 0 | B stage 1
  __shared__ __align__(8) uint64_t s_mbar[2];
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_fail;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool decoder = tid < kTileM;
  const int t = decoder ? tid : tid - kTileM;  // index inside the warpgroup
  const uint32_t mbar0 = smem_u32(&s_mbar[0]), mbar1 = smem_u32(&s_mbar[1]);
  if (*a.n_items <= 0) return;  // nothing routed to the tile path this step (uniform over the grid)

  if (tid == 0) {
    mbar_init(mbar0, 1);
    mbar_init(mbar1, 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  const uint32_t idesc = make_instr_desc(kTileM, kTileN);
  const int n_items = *a.n_items;
  uint32_t uses0 = 0u, uses1 = 0u;  // MMA batches committed per stage; batch n completes phase (n - 1) & 1

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int4 it = a.items[item];
    const qmoe_matrix_desc d = a.descs[it.x];
    const int tok0 = it.z, ntok = it.w;
    const int W = d.width;
    const int n_windows = (W + kTileK - 1) / kTileK;

    if (!decoder) {
      // ---- stagers --------------------------------------------------------------------------------
      const __nv_bfloat16 *src[kBUnits];
      bool live[kBUnits];
#pragma unroll
      for (int i = 0; i < kBUnits; i++) {
        const int u = t + i * kTileM;
        const int n = u & (kTileN - 1), c = u >> 6;
        live[i] = n < ntok;
        const int tok = tok0 + (live[i] ? n : 0);
        src[i] = a.x + (a.x_rows != nullptr ? (long long)a.x_rows[tok] : (long long)tok) * a.x_stride + 8 * c;
      }
      for (int w = 0; w < n_windows; w++) {
        const int st = w & 1, k0 = w * kTileK;
        uint8_t *A = tile_smem + st * kABytes, *B = tile_smem + 2 * kABytes + st * kBBytes;
        uint4 v[kBUnits];
#pragma unroll
        for (int i = 0; i < kBUnits; i++) {  // issue the loads first: they overlap the wait below
          const int k = k0 + 8 * ((t + i * kTileM) >> 6);
          const __nv_bfloat16 *p = src[i] + k0;
          v[i] = make_uint4(0u, 0u, 0u, 0u);
          if (live[i] && k < W) {
            if (k + 8 <= W && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
              v[i] = __ldg(reinterpret_cast<const uint4 *>(p));
            } else {
              uint16_t h[8];
#pragma unroll
              for (int j = 0; j < 8; j++) h[j] = (k + j < W) ? __bfloat16_as_ushort(p[j]) : (uint16_t)0;
              v[i].x = h[0] | ((uint32_t)h[1] << 16);
              v[i].y = h[2] | ((uint32_t)h[3] << 16);
              v[i].z = h[4] | ((uint32_t)h[5] << 16);
              v[i].w = h[6] | ((uint32_t)h[7] << 16);
            }
          }
        }
        const uint32_t used = st ? uses1 : uses0;
        if (used > 0 && !s_fail && !mbar_wait(st ? mbar1 : mbar0, (used - 1u) & 1u, a.wait_limit)) s_fail = 1;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < kTileChunks; c++)
          *reinterpret_cast<uint4 *>(A + c * (kTileM * 16) + t * 16) = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < kBUnits; i++) {
          const int u = t + i * kTileM;
          *reinterpret_cast<uint4 *>(B + (u >> 6) * (kTileN * 16) + (u & (kTileN - 1)) * 16) = v[i];
        }
        fence_async_proxy();
        named_arrive(1 + st, kTileThreads);
        if (st) uses1++;
        else uses0++;
      }
    } else {
      // ---- decoders -------------------------------------------------------------------------------
      const int row = it.y + t;
      const bool valid_row = row < d.height;
      const uint16_t *codes = a.codes + d.code_base;
      int ci = 0, ce = 0;
      uint32_t mn = 0, mx = 0;
      if (valid_row) {
        const int32_t *ro = a.row_off + d.rowoff_base;
        long long b = ro[row], e2 = ro[row + 1];
        b = b < 0 ? 0 : (b > d.n_codes ? d.n_codes : b);
        e2 = e2 < b ? b : (e2 > d.n_codes ? d.n_codes : e2);
        ci = (int)b;
        ce = (int)e2;
        const __nv_bfloat162 mm = a.minmax[d.minmax_base + row];
        mn = __bfloat16_as_ushort(mm.x);
        mx = __bfloat16_as_ushort(mm.y);
      }
      // Codes are fetched eight at a time (one aligned 128-bit load) and their table entries are
      // looked up together; both run ahead of their use: while the entries of chunk c are consumed,
      // the entries of chunk c + 1 and the codes of chunk c + 2 are already in flight.
      const int mis = (int)((reinterpret_cast<uintptr_t>(codes) & 15u) >> 1);
      const uint16_t *codes_al = codes - mis;
      const int end_al = ce + mis;
      uint32_t ebuf[8], enext[8];
      int chunk = (ci + mis) >> 3;  // chunk whose entries are in ebuf
      auto load_codes = [&](int c) -> uint4 {
        return (valid_row && c * 8 < end_al) ? __ldg(reinterpret_cast<const uint4 *>(codes_al + (long long)c * 8))
                                             : make_uint4(0u, 0u, 0u, 0u);
      };
      auto lookup8 = [&](const uint4 &q, uint32_t (&dst)[8]) {
#pragma unroll
        for (int j = 0; j < 8; j++) dst[j] = __ldg(a.tab + chunk_code(q, j));
      };
      uint4 q2;
      {
        const uint4 q0 = load_codes(chunk), q1 = load_codes(chunk + 1);
        q2 = load_codes(chunk + 2);
        lookup8(q0, ebuf);
        lookup8(q1, enext);
      }
      int pos = 0, len = 0;
      uint32_t e = kEntryNull;
      bool have = false;

      for (int w = 0; w < n_windows; w++) {
        const int st = w & 1, k0 = w * kTileK, k1 = k0 + kTileK;
        uint8_t *A = tile_smem + st * kABytes;
        named_sync(1 + st, kTileThreads);  // the stage is zeroed and holds the activations
        if (valid_row) {
          for (;;) {
            if (!have) {
              if (ci >= ce || pos >= k1) break;
              const int ia = ci + mis;
              if ((ia >> 3) != chunk) {  // codes are consumed in order: this is chunk + 1
                chunk = ia >> 3;
#pragma unroll
                for (int j = 0; j < 8; j++) ebuf[j] = enext[j];
                lookup8(q2, enext);
                q2 = load_codes(chunk + 2);
              }
              e = ebuf[ia & 7];
              len = 2 * (int)entry_len(e);
              have = true;
            }
#pragma unroll
            for (int k = 0; k < 3; k++) {
              const uint32_t o = entry_nz_pos(e, k);
              const int kk = pos + (int)o - k0;
              if (o < 0x80u && (unsigned)kk < (unsigned)kTileK)
                *reinterpret_cast<uint16_t *>(A + (kk >> 3) * (kTileM * 16) + t * 16 + (kk & 7) * 2) =
                    (uint16_t)((e & (0x10u << k)) ? mx : mn);
            }
            if (pos + len > k1) break;  // straddles the window: applied again in the next one
            pos += len;
            ci++;
            have = false;
          }
        }
        fence_async_proxy();
        named_sync(3, kTileM);
        if (tid == 0) {
          tc_fence_after();
          const uint32_t a_addr = smem_u32(A), b_addr = smem_u32(tile_smem + 2 * kABytes + st * kBBytes);
#pragma unroll
          for (int s = 0; s < kTileK / 16; s++) {
            const uint64_t da = make_smem_desc(a_addr + s * 2 * (kTileM * 16), kTileM * 16, 128);
            const uint64_t db = make_smem_desc(b_addr + s * 2 * (kTileN * 16), kTileN * 16, 128);
            mma_bf16(tmem, da, db, idesc, (w > 0 || s > 0) ? 1u : 0u);
          }
          mma_commit(st ? mbar1 : mbar0);
        }
        if (st) uses1++;
        else uses0++;
      }
      // all MMAs of the item are complete when the last commit has arrived
      const int last = (n_windows - 1) & 1;
      const uint32_t used = last ? uses1 : uses0;
      if (!s_fail && !mbar_wait(last ? mbar1 : mbar0, (used - 1u) & 1u, a.wait_limit)) s_fail = 1;
      tc_fence_after();
    }
    __syncthreads();
    if (s_fail) {  // uniform: read after the barrier
      // This CTA gives up.  The rows of this and of its remaining items are written as zeros so that
      // what later stages read is defined; the sticky status word tells the host.
      for (int rest = item; rest < n_items; rest += gridDim.x) {
        const int4 ri = a.items[rest];
        const qmoe_matrix_desc rd = a.descs[ri.x];
        for (int i = tid; i < kTileM * ri.w; i += kTileThreads) {
          const int r = ri.y + (i % kTileM), n = i / kTileM;
          if (r < rd.height) out_row_ptr(a, ri.z + n)[r] = __float2bfloat16_rn(0.f);
        }
      }
      break;
    }

    if (decoder) {  // epilogue: row t of the accumulator -> y[token][row]
      const int row = it.y + t;
      const bool valid_row = row < d.height;
      const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
      for (int j = 0; j < kTileN / 16; j++) {
        uint32_t v[16];
        tmem_ld16(taddr + j * 16, v);
#pragma unroll
        for (int i = 0; i < 16; i++) {
          const int n = j * 16 + i;
          if (valid_row && n < ntok) {
            float r = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i])));
            if (a.flags & QMOE_FLAG_RELU) r = fmaxf(r, 0.f);
            out_row_ptr(a, tok0 + n)[row] = __float2bfloat16_rn(r);
          }
        }
      }
    }
    tc_fence_before();
    __syncthreads();  // the accumulator is overwritten by the next item's first MMA
    tc_fence_after();
  }

  if (s_fail) {
    if (tid == 0 && a.status != nullptr) atomicAdd(a.status, 1);
    // one more bounded wait per stage for MMAs that may still be in flight
    if (tid == 0) {
      if (uses0 > 0) mbar_wait(mbar0, (uses0 - 1u) & 1u);
      if (uses1 > 0) mbar_wait(mbar1, (uses1 - 1u) & 1u);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// ---- work list of the tile path ---------------------------------------------------------------------
// Experts with at least `tile_min` tokens are cut into blocks of up to 64 tokens; every block becomes
// ceil(height / 128) items per linear.  header[4] / header[5] receive the item counts of wi / wo,
// (timeouts are counted in the library's sticky per-device status word, not here).
__global__ void __launch_bounds__(1024) k_build_tile_work(const int32_t *__restrict__ offsets, int n_experts,
                                                          int tile_min, int d_model, int d_ff, int cap_blocks,
                                                          int *header, int4 *items_wi, int4 *items_wo) {
  __shared__ int s_blocks;
  if (threadIdx.x == 0) s_blocks = 0;
  __syncthreads();
  const int rb_wi = (d_ff + kTileM - 1) / kTileM, rb_wo = (d_model + kTileM - 1) / kTileM;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int first = offsets[e];
    const int count = offsets[e + 1] - first;
    if (count < tile_min) continue;
    const int nb = (count + kTileN - 1) / kTileN;
    const int base = atomicAdd(&s_blocks, nb);
    for (int b = 0; b < nb; b++) {
      const int blk = base + b;
      if (blk >= cap_blocks) break;
      const int tok0 = first + b * kTileN;
      const int nt = min(kTileN, count - b * kTileN);
      for (int r = 0; r < rb_wi; r++) items_wi[(size_t)blk * rb_wi + r] = make_int4(2 * e, r * kTileM, tok0, nt);
      for (int r = 0; r < rb_wo; r++) items_wo[(size_t)blk * rb_wo + r] = make_int4(2 * e + 1, r * kTileM, tok0, nt);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int blocks = min(s_blocks, cap_blocks);
    header[4] = blocks * rb_wi;
    header[5] = blocks * rb_wo;
  }
}

int tile_cap_blocks(int max_slots) { return max_slots / 8 + 1; }

int64_t tile_work_bytes(int max_slots, int d_model, int d_ff) {
  const int64_t rb = (d_ff + kTileM - 1) / kTileM + (d_model + kTileM - 1) / kTileM;
  return (int64_t)tile_cap_blocks(max_slots) * rb * (int64_t)sizeof(int4);
}

int launch_build_tile_work(const int32_t *offsets, int n_experts, int tile_min, int d_model, int d_ff,
                           int max_slots, int *header, int4 *items_wi, int4 *items_wo, cudaStream_t stream) {
  QMOE_LAUNCH(k_build_tile_work, 1, 1024, 0, stream, offsets, n_experts, tile_min, d_model, d_ff,
              tile_cap_blocks(max_slots), header, items_wi, items_wo);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

// One linear (wi or wo) of every expert on the tile path.
int launch_tile_phase(const uint32_t *tab, const uint16_t *codes, const int32_t *row_off, const void *minmax,
                      const qmoe_matrix_desc *descs, const void *x, void *y, long long x_stride, long long y_stride,
                      const int32_t *x_rows, const int32_t *y_rows, const unsigned long long *y_ptrs, const int4 *items,
                      const int *n_items, int flags, int max_items, int device, cudaStream_t stream) {
  TileArgs a{};
  a.tab = tab;
  a.codes = codes;
  a.row_off = row_off;
  a.minmax = reinterpret_cast<const __nv_bfloat162 *>(minmax);
  a.descs = descs;
  a.x = reinterpret_cast<const __nv_bfloat16 *>(x);
  a.y = reinterpret_cast<__nv_bfloat16 *>(y);
  a.x_stride = x_stride;
  a.y_stride = y_stride;
  a.x_rows = x_rows;
  a.y_rows = y_rows;
  a.y_ptrs = y_ptrs;
  a.items = items;
  a.n_items = n_items;
  a.status = tile_status_word(device);
  a.flags = flags;
  const uint32_t limit = g_wait_limit.load(std::memory_order_relaxed);
  a.wait_limit = limit ? limit : kWaitLimit;
  int grid = 4 * sm_count(device);
  grid = grid > max_items ? max_items : grid;
  grid = grid < 1 ? 1 : grid;
  constexpr int kSmem = 2 * (kTileChunks * kTileM * 16) + 2 * (kTileChunks * kTileN * 16);
  static bool configured[64] = {false};
  if (device >= 0 && device < 64) {
    std::lock_guard<std::mutex> lock(setup_mutex());
    if (!configured[device]) {
      QMOE_CUDA(cudaFuncSetAttribute(k_tile_matmul, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
      configured[device] = true;
    }
  }
  QMOE_LAUNCH(k_tile_matmul, grid, kTileThreads, kSmem, stream, a);
  QMOE_CUDA(cudaGetLastError());
  return QMOE_OK;
}

}  // namespace qmoe
