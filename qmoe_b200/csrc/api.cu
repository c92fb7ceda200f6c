// C ABI (include/qmoe_sub1.h): argument checks, per-device caches and the host-side dictionary
// construction.  Kernels live in sub1_matmul.cu, sub1_pack.cu and moe_route.cu.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <queue>
#include <utility>
#include <vector>

namespace qmoe {

// ---- error plumbing -------------------------------------------------------------------------
static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return QMOE_ERR_CUDA;
}

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// ---- optional event timing of the grouped launches ----------------------------------------------
static std::mutex g_profile_mutex;
static bool g_profile_on = false;
struct ProfileCall {
  cudaEvent_t ev[4];
  int device;
};
static std::vector<ProfileCall> g_profile_calls;
constexpr size_t kMaxProfileCalls = 256;

bool profile_begin(int device, cudaEvent_t **events) {
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  if (!g_profile_on || g_profile_calls.size() >= kMaxProfileCalls) return false;
  ProfileCall c{};
  c.device = device;
  for (int i = 0; i < 4; i++) {
    if (cudaEventCreate(&c.ev[i]) != cudaSuccess) {
      for (int j = 0; j < i; j++) cudaEventDestroy(c.ev[j]);
      return false;
    }
  }
  g_profile_calls.push_back(c);
  *events = g_profile_calls.back().ev;
  return true;
}

std::mutex &setup_mutex() {
  static std::mutex m;
  return m;
}

int *tile_status_word(int device) {
  static int *word[64] = {nullptr};
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(setup_mutex());
  if (word[device] == nullptr) {
    int *p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    if (cudaMemset(p, 0, sizeof(int)) != cudaSuccess) {
      cudaFree(p);
      return nullptr;
    }
    word[device] = p;
  }
  return word[device];
}

int sm_count(int device) {
  static int cached[64] = {0};
  if (device < 0 || device >= 64) return 148;
  std::lock_guard<std::mutex> lock(setup_mutex());
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device] = n;
  }
  return cached[device];
}

// ---- launchers defined in the kernel files ------------------------------------------------------
int launch_build_table(const int32_t *dec, uint32_t *tab, int *nonconforming, cudaStream_t stream);
int launch_matmul_uniform(const SparseTable &tab, const int32_t *dec, const uint16_t *codes,
                          const int32_t *row_off, const void *minmax, const void *x, void *y, int height,
                          int width, int64_t n_codes, int tokens, int64_t x_stride, int64_t y_stride,
                          int flags, int device, cudaStream_t stream);
int launch_decode(const SparseTable &tab, const int32_t *dec, const uint16_t *codes, const int32_t *row_off,
                  uint8_t *sym, int32_t *status, int height, int width, int64_t n_codes, cudaStream_t stream);
int64_t moe_work_bytes(int max_slots, int d_model, int d_ff);
int set_tile_min_tokens(int tokens);
void set_items_per_matrix(int wi, int wo);
int set_fused_phases(int on);
int set_tile_wait_limit(uint32_t spins);
int work_summary(const void *work, int max_slots, int d_ff, int32_t *out, cudaStream_t stream);
int launch_grouped_ffn(const SparseTable &tab, const int32_t *dec, const uint16_t *codes,
                       const int32_t *row_off, const void *minmax, const qmoe_matrix_desc *descs,
                       const qmoe_interleaved_store *ils, const int32_t *offsets, const void *xs,
                       int64_t xs_stride, const int32_t *x_rows, void *hs, void *ys, int64_t ys_stride,
                       const int32_t *y_rows, const unsigned long long *y_ptrs, void *work, int n_experts,
                       int max_slots, int d_model, int d_ff, int device, cudaStream_t stream);
int launch_keep(const int32_t *choice, int32_t *expert, int n_tokens, int n_experts, int seq_len, int capacity,
                cudaStream_t stream);
int launch_ep_dispatch(const int32_t *choice, const void *hidden, int64_t hidden_stride, int32_t *expert,
                       int32_t *dest, int32_t *slot, void *send, void *const *blocks, int *overflow, int n_tokens,
                       int n_experts, int local_experts, int seq_len, int capacity, int n_ranks, int cap, int d_model,
                       cudaStream_t stream);
int launch_ep_plan(const void *rows, int64_t row_stride, int d_model, const int32_t *meta, int n_rows, int n_buckets,
                   int32_t *offsets, int32_t *slot_of_row, int32_t *row_of_slot, const uint64_t *out_blocks,
                   int rows_per_block, int64_t out_row_bytes, uint64_t *out_ptr_of_slot, cudaStream_t stream);
int launch_peer_barrier(int32_t *const *flag_blocks, int rank, int n_ranks, int channel, uint64_t limit_ns,
                        int *status, cudaStream_t stream);
int launch_combine_add(const void *ys, const void *hidden, const int32_t *slot, const void *prob,
                       const void *residual, void *out, int n_tokens, int d_model, cudaStream_t stream);
int launch_route_small(const float *logits, const void *hidden, int n_tokens, int n_experts, int d_model,
                       int capacity, void *prob, int32_t *offsets, int32_t *slot, void *xs, cudaStream_t stream);
int launch_gemv(const void *x, const void *ln_w, const void *w, const void *residual, void *y, void *normed_out,
                int n, int k, float eps, int f32_out, cudaStream_t stream);
int launch_rms_norm(const void *x, const void *w, void *out, int rows, int d, float eps, cudaStream_t stream);
int launch_decode_attention(const void *qkv, void *k_cache, void *v_cache, const int64_t *pos, void *out,
                            int heads, int hd, int max_len, float scale, const float *bias, int *status,
                            cudaStream_t stream);
int launch_code_histogram(const uint16_t *codes, int64_t n, uint64_t *hist, cudaStream_t stream);
int launch_remap_tables(const int32_t *dec, const uint32_t *remap, uint32_t *tab_out, int32_t *dec_out,
                        int *scratch2, cudaStream_t stream);
int launch_interleave_count(const int32_t *row_off, const qmoe_matrix_desc *descs, int n_matrices, const int32_t *rows,
                            int32_t *blk_units, cudaStream_t stream);
int launch_interleave_emit(const uint16_t *codes, const int32_t *row_off, const qmoe_matrix_desc *descs,
                           int n_matrices, const int32_t *rows, const int64_t *blk_base, const uint32_t *remap,
                           void *il, cudaStream_t stream);
int launch_pack_prepare(const int32_t *trie, int32_t *w_tern, int32_t *row_off, int height, int width,
                        cudaStream_t stream);
int launch_pack_emit(const int32_t *w_tern, const int32_t *row_off, uint16_t *w_comp, int height, int width,
                     cudaStream_t stream);
int launch_pack_u8_count(const int32_t *trie, const uint8_t *sym, uint16_t *codes_tmp, int32_t *row_len,
                         int n_mat, int height, int width, cudaStream_t stream);
int launch_pack_u8_gather(const uint16_t *codes_tmp, const int32_t *row_off, const int64_t *mat_base,
                          uint16_t *out, int n_mat, int height, int width, cudaStream_t stream);
int launch_synth_ternary(uint8_t *sym, int64_t count, uint64_t seed, uint64_t first_index, float p_zero,
                         cudaStream_t stream);
int launch_route(const float *logits, int32_t *choice, void *prob, int n_tokens, int n_experts,
                 cudaStream_t stream);
int launch_rank(const int32_t *choice, int32_t *bucket, int32_t *rank, int32_t *counts, int n_tokens,
                int n_buckets, int seq_len, int capacity, cudaStream_t stream);
int launch_scan(const int32_t *counts, int32_t *offsets, int n, cudaStream_t stream);
int launch_permute(const int32_t *bucket, const int32_t *rank, const int32_t *offsets, int32_t *slot,
                   const void *hidden, void *xs, int n_tokens, int d_model, int64_t hidden_stride,
                   int64_t xs_stride, cudaStream_t stream);
int launch_unpermute(const void *ys, const int32_t *slot, void *out, int n_tokens, int d_model,
                     int64_t ys_stride, int64_t out_stride, cudaStream_t stream);
int launch_combine(const void *ys, const void *hidden, const int32_t *slot, const void *prob, void *out,
                   int n_tokens, int d_model, cudaStream_t stream);

// ---- sparse table cache ---------------------------------------------------------------------------
struct CachedTable {
  uint32_t *entries;
  bool conforming;
};
static std::mutex g_mutex;
static std::map<std::pair<int, const void *>, CachedTable> g_tables;

int get_sparse_table(const int32_t *dec_dev, int device, cudaStream_t stream, SparseTable *out) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const auto key = std::make_pair(device, (const void *)dec_dev);
  auto it = g_tables.find(key);
  if (it == g_tables.end()) {
    // First use of this table on this device: build the sparse form and learn whether any entry
    // needs the digit-by-digit path.  This synchronises the stream once.
    uint32_t *entries = nullptr;
    int *flag = nullptr;
    QMOE_CUDA(cudaMalloc(&entries, sizeof(uint32_t) * QMOE_DICT_COUNT));
    cudaError_t e = cudaMalloc(&flag, sizeof(int));
    if (e != cudaSuccess) {
      cudaFree(entries);
      return cuda_fail(e, "cudaMalloc(flag)");
    }
    int rc = launch_build_table(dec_dev, entries, flag, stream);
    int host_flag = 0;
    if (rc == QMOE_OK) {
      e = cudaMemcpyAsync(&host_flag, flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) rc = cuda_fail(e, "sparse table build");
    }
    cudaFree(flag);
    if (rc != QMOE_OK) {
      cudaFree(entries);
      return rc;
    }
    it = g_tables.emplace(key, CachedTable{entries, host_flag == 0}).first;
  }
  out->entries = it->second.entries;
  out->conforming = it->second.conforming;
  return QMOE_OK;
}

// dec == nullptr: every table of the device.
static int release_tables(int device, const void *dec = nullptr) {
  std::lock_guard<std::mutex> lock(g_mutex);
  for (auto it = g_tables.begin(); it != g_tables.end();) {
    if (it->first.first == device && (dec == nullptr || it->first.second == dec)) {
      cudaFree(it->second.entries);
      it = g_tables.erase(it);
    } else {
      ++it;
    }
  }
  return QMOE_OK;
}

// ---- dictionary construction (host) ---------------------------------------------------------------
// Best-first enumeration of the 65 536 most probable sequences of 1..14 ternary pairs under
// P(0) = 0.885, exactly as setup() orders them (sub1.py:29-57): priority = running float64 product
// that starts at -1.0 and is multiplied by the pair probability at every extension; ties are broken
// by comparing the pair lists lexicographically, a prefix sorting before its extensions.
struct Candidate {
  double prio;
  int32_t parent;  // dictionary index of the sequence without its last pair (65536 = empty)
  uint8_t len;
  uint8_t seq[14];
};
struct CandidateAfter {
  bool operator()(const Candidate &a, const Candidate &b) const {  // true if a pops after b
    if (a.prio != b.prio) return a.prio > b.prio;
    const int n = a.len < b.len ? a.len : b.len;
    const int c = memcmp(a.seq, b.seq, n);
    if (c != 0) return c > 0;
    return a.len > b.len;
  }
};

static int build_dictionary(int32_t *dec, int32_t *trie) {
  const double zeros = .885;
  const double q[3] = {zeros, (1 - zeros) / 2, (1 - zeros) / 2};
  double pair_prob[9];
  for (int hi = 0; hi < 3; hi++)
    for (int lo = 0; lo < 3; lo++) pair_prob[3 * hi + lo] = (1. * q[hi]) * q[lo];

  std::priority_queue<Candidate, std::vector<Candidate>, CandidateAfter> pq;
  Candidate root{};
  root.prio = -1.;
  root.parent = -1;
  root.len = 0;
  pq.push(root);
  for (int i = 0; i < (QMOE_DICT_COUNT + 1) * 9; i++) trie[i] = -1;
  int count = 0;
  while (count < QMOE_DICT_COUNT) {
    if (pq.empty()) return QMOE_ERR_UNSUPPORTED;
    const Candidate top = pq.top();
    pq.pop();
    int idx = QMOE_TRIE_ROOT;
    if (top.len > 0) {
      idx = count++;
      // Table words (sub1.py:60-72): low nibble = length in pairs; pair j of each half at bits
      // 4+4j..7+4j, first weight (p % 3) in the low two bits, second (p / 3) in the high two.
      uint32_t words[2] = {0u, 0u};
      for (int j = 0; j < top.len; j++) {
        const uint32_t p = top.seq[j];
        const uint32_t nib = (p % 3) | ((p / 3) << 2);
        words[j / 7] |= nib << (4 + 4 * (j % 7));
      }
      dec[2 * idx + 0] = (int32_t)(words[0] | top.len);
      dec[2 * idx + 1] = (int32_t)(words[1] | top.len);
      trie[9 * top.parent + top.seq[top.len - 1]] = idx;  // sub1.py:86-97
    }
    if (top.len == 14) continue;
    for (int p = 0; p < 9; p++) {
      Candidate c = top;
      c.prio = top.prio * pair_prob[p];
      c.seq[c.len++] = (uint8_t)p;
      c.parent = idx;
      pq.push(c);
    }
  }
  return QMOE_OK;
}

static cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

}  // namespace qmoe

using namespace qmoe;

extern "C" {

const char *qmoe_last_error(void) { return g_error; }
int qmoe_version(void) { return 100; }

int qmoe_sub1_build_dictionary(int32_t *dec_host, int32_t *trie_host) {
  QMOE_REQUIRE(dec_host != nullptr && trie_host != nullptr, "null output pointer");
  return build_dictionary(dec_host, trie_host);
}

static int check_matrix_args(const char *fn, const void *dec, const void *w_comp, const void *row_off,
                             const void *minmax, int height, int width, int64_t n_codes) {
  if (dec == nullptr || row_off == nullptr || minmax == nullptr || (w_comp == nullptr && n_codes > 0)) {
    set_error("%s: null device pointer", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (height < 1 || width < 1 || n_codes < 0) {
    set_error("%s: bad shape height=%d width=%d n_codes=%lld", fn, height, width, (long long)n_codes);
    return QMOE_ERR_INVALID_ARG;
  }
  if (width > QMOE_MAX_WIDTH) {
    set_error("%s: width %d exceeds QMOE_MAX_WIDTH (%d)", fn, width, QMOE_MAX_WIDTH);
    return QMOE_ERR_UNSUPPORTED;
  }
  if (n_codes >= (int64_t)1 << 31) {
    set_error("%s: a single matrix is limited to 2^31-1 codes", fn);
    return QMOE_ERR_UNSUPPORTED;
  }
  if ((reinterpret_cast<uintptr_t>(w_comp) & 1u) || (reinterpret_cast<uintptr_t>(row_off) & 3u) ||
      (reinterpret_cast<uintptr_t>(minmax) & 3u)) {
    set_error("%s: misaligned pointer (w_comp 2, row_off 4, ter_minmax 4 bytes)", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  return QMOE_OK;
}

int qmoe_sub1_matmul(const int32_t *dec_dev, const uint16_t *w_comp_dev, const int32_t *row_off_dev,
                     const void *ter_minmax_dev, const void *x_dev, void *y_dev, int height, int width,
                     int64_t n_codes, int tokens, int64_t x_stride, int64_t y_stride, int flags, int device,
                     void *stream) {
  int rc = check_matrix_args(__func__, dec_dev, w_comp_dev, row_off_dev, ter_minmax_dev, height, width, n_codes);
  if (rc) return rc;
  QMOE_REQUIRE(tokens >= 0, "negative token count");
  if (tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(x_dev != nullptr && y_dev != nullptr, "null activation pointer");
  QMOE_REQUIRE(x_stride >= width && y_stride >= height, "row stride smaller than the row");
  QMOE_REQUIRE(((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev)) & 1u) == 0,
               "misaligned bf16 pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  SparseTable tab;
  rc = get_sparse_table(dec_dev, device, as_stream(stream), &tab);
  if (rc) return rc;
  return launch_matmul_uniform(tab, dec_dev, w_comp_dev, row_off_dev, ter_minmax_dev, x_dev, y_dev, height,
                               width, n_codes, tokens, x_stride, y_stride, flags, device, as_stream(stream));
}

int qmoe_sub1_matvec(const int32_t *dec_dev, const uint16_t *w_comp_dev, const int32_t *row_off_dev,
                     const void *ter_minmax_dev, const void *x_dev, void *y_dev, int height, int width,
                     int64_t n_codes, int device, void *stream) {
  return qmoe_sub1_matmul(dec_dev, w_comp_dev, row_off_dev, ter_minmax_dev, x_dev, y_dev, height, width,
                          n_codes, 1, width, height, QMOE_FLAG_ACCUMULATE, device, stream);
}

int qmoe_sub1_decode(const int32_t *dec_dev, const uint16_t *w_comp_dev, const int32_t *row_off_dev,
                     uint8_t *sym_dev, int32_t *status_dev, int height, int width, int64_t n_codes, int device,
                     void *stream) {
  int rc = check_matrix_args(__func__, dec_dev, w_comp_dev, row_off_dev, dec_dev, height, width, n_codes);
  if (rc) return rc;
  QMOE_REQUIRE(sym_dev != nullptr, "null output pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  SparseTable tab;
  rc = get_sparse_table(dec_dev, device, as_stream(stream), &tab);
  if (rc) return rc;
  return launch_decode(tab, dec_dev, w_comp_dev, row_off_dev, sym_dev, status_dev, height, width, n_codes,
                       as_stream(stream));
}

int qmoe_sub1_pack_prepare(const int32_t *trie_dev, int32_t *w_tern_dev, int32_t *row_off_dev, int height,
                           int width, int device, void *stream) {
  QMOE_REQUIRE(trie_dev != nullptr && w_tern_dev != nullptr && row_off_dev != nullptr, "null device pointer");
  QMOE_REQUIRE(height >= 1 && width >= 1, "bad shape");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_pack_prepare(trie_dev, w_tern_dev, row_off_dev, height, width, as_stream(stream));
}

int qmoe_sub1_pack_emit(const int32_t *w_tern_dev, const int32_t *row_off_dev, uint16_t *w_comp_dev,
                        int height, int width, int device, void *stream) {
  QMOE_REQUIRE(w_tern_dev != nullptr && row_off_dev != nullptr && w_comp_dev != nullptr, "null device pointer");
  QMOE_REQUIRE(height >= 1 && width >= 1, "bad shape");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_pack_emit(w_tern_dev, row_off_dev, w_comp_dev, height, width, as_stream(stream));
}

int qmoe_sub1_pack_u8_count(const int32_t *trie_dev, const uint8_t *sym_dev, uint16_t *codes_tmp_dev,
                            int32_t *row_len_dev, int n_mat, int height, int width, int device, void *stream) {
  QMOE_REQUIRE(trie_dev && sym_dev && codes_tmp_dev && row_len_dev, "null device pointer");
  QMOE_REQUIRE(n_mat >= 1 && height >= 1 && width >= 2 && (width & 1) == 0, "bad shape (width must be even)");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_pack_u8_count(trie_dev, sym_dev, codes_tmp_dev, row_len_dev, n_mat, height, width,
                              as_stream(stream));
}

int qmoe_sub1_pack_u8_gather(const uint16_t *codes_tmp_dev, const int32_t *row_off_dev,
                             const int64_t *mat_base_dev, uint16_t *out_dev, int n_mat, int height, int width,
                             int device, void *stream) {
  QMOE_REQUIRE(codes_tmp_dev && row_off_dev && mat_base_dev && out_dev, "null device pointer");
  QMOE_REQUIRE(n_mat >= 1 && height >= 1 && width >= 2 && (width & 1) == 0, "bad shape (width must be even)");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_pack_u8_gather(codes_tmp_dev, row_off_dev, mat_base_dev, out_dev, n_mat, height, width,
                               as_stream(stream));
}

int qmoe_synth_ternary(uint8_t *sym_dev, int64_t count, uint64_t seed, uint64_t first_index, float p_zero,
                       int device, void *stream) {
  QMOE_REQUIRE(sym_dev != nullptr && count >= 0, "bad arguments");
  QMOE_REQUIRE(p_zero >= 0.f && p_zero <= 1.f, "p_zero outside [0, 1]");
  if (count == 0) return QMOE_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_synth_ternary(sym_dev, count, seed, first_index, p_zero, as_stream(stream));
}

int qmoe_moe_route(const float *logits_dev, int32_t *choice_dev, void *prob_dev, int n_tokens, int n_experts,
                   int device, void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && n_experts >= 1, "bad shape");
  if (n_tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(logits_dev && choice_dev && prob_dev, "null device pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_route(logits_dev, choice_dev, prob_dev, n_tokens, n_experts, as_stream(stream));
}

int qmoe_moe_rank(const int32_t *choice_dev, int32_t *bucket_dev, int32_t *rank_dev, int32_t *counts_dev,
                  int n_tokens, int n_buckets, int seq_len, int capacity, int device, void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && n_buckets >= 1, "bad shape");
  QMOE_REQUIRE(counts_dev != nullptr, "null counts pointer");
  QMOE_REQUIRE((choice_dev && bucket_dev && rank_dev) || n_tokens == 0, "null device pointer");
  QMOE_REQUIRE(choice_dev != bucket_dev || n_tokens == 0, "bucket_dev must not alias choice_dev");
  QMOE_REQUIRE(seq_len >= 1 && n_tokens % seq_len == 0, "n_tokens must be a multiple of seq_len");
  QMOE_REQUIRE(capacity >= 0, "negative capacity");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_rank(choice_dev, bucket_dev, rank_dev, counts_dev, n_tokens, n_buckets, seq_len, capacity,
                     as_stream(stream));
}

int qmoe_moe_keep(const int32_t *choice_dev, int32_t *expert_dev, int n_tokens, int n_experts, int seq_len,
                  int capacity, int device, void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && n_experts >= 1, "bad shape");
  if (n_tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(choice_dev && expert_dev && choice_dev != expert_dev, "null or aliased device pointer");
  QMOE_REQUIRE(seq_len >= 1 && n_tokens % seq_len == 0, "n_tokens must be a multiple of seq_len");
  QMOE_REQUIRE(capacity >= 0, "negative capacity");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_keep(choice_dev, expert_dev, n_tokens, n_experts, seq_len, capacity, as_stream(stream));
}

int qmoe_moe_scan(const int32_t *counts_dev, int32_t *offsets_dev, int n, int device, void *stream) {
  QMOE_REQUIRE(counts_dev && offsets_dev && n >= 1, "bad arguments");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_scan(counts_dev, offsets_dev, n, as_stream(stream));
}

int qmoe_moe_permute(const int32_t *bucket_dev, const int32_t *rank_dev, const int32_t *offsets_dev,
                     int32_t *slot_dev, const void *hidden_dev, void *xs_dev, int n_tokens, int d_model,
                     int64_t hidden_stride, int64_t xs_stride, int device, void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && d_model >= 1, "bad shape");
  if (n_tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(bucket_dev && rank_dev && offsets_dev && slot_dev && hidden_dev && xs_dev, "null device pointer");
  QMOE_REQUIRE(hidden_stride >= d_model && xs_stride >= d_model, "row stride smaller than the row");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_permute(bucket_dev, rank_dev, offsets_dev, slot_dev, hidden_dev, xs_dev, n_tokens, d_model,
                        hidden_stride, xs_stride, as_stream(stream));
}

int qmoe_moe_unpermute(const void *ys_dev, const int32_t *slot_dev, void *out_dev, int n_tokens, int d_model,
                       int64_t ys_stride, int64_t out_stride, int device, void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && d_model >= 1, "bad shape");
  if (n_tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(ys_dev && slot_dev && out_dev, "null device pointer");
  QMOE_REQUIRE(ys_stride >= d_model && out_stride >= d_model, "row stride smaller than the row");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_unpermute(ys_dev, slot_dev, out_dev, n_tokens, d_model, ys_stride, out_stride, as_stream(stream));
}

int qmoe_moe_set_tile_min_tokens(int tokens) { return set_tile_min_tokens(tokens); }

int qmoe_moe_set_fused_phases(int on) { return set_fused_phases(on); }

int qmoe_moe_set_items_per_matrix(int wi, int wo) {
  set_items_per_matrix(wi, wo);
  return QMOE_OK;
}

int64_t qmoe_moe_work_bytes(int n_experts, int max_slots, int d_model, int d_ff) {
  (void)n_experts;
  if (max_slots < 0 || d_model < 1 || d_ff < 1) return QMOE_ERR_INVALID_ARG;
  return moe_work_bytes(max_slots, d_model, d_ff);
}

int qmoe_moe_work_summary(const void *work_dev, int max_slots, int d_ff, int32_t *out_host, int device,
                          void *stream) {
  QMOE_REQUIRE(work_dev != nullptr && out_host != nullptr, "null pointer");
  QMOE_REQUIRE(max_slots >= 1 && d_ff >= 1, "bad shape");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return work_summary(work_dev, max_slots, d_ff, out_host, as_stream(stream));
}

static int grouped_ffn_entry(const char *fn, const int32_t *dec_dev, const uint16_t *codes_dev,
                             const int32_t *row_off_dev, const void *minmax_dev, const qmoe_matrix_desc *descs_dev,
                             const qmoe_interleaved_store *ils, const int32_t *offsets_dev,
                             const void *xs_dev, int64_t xs_stride, const int32_t *x_rows_dev, void *hs_dev,
                             void *ys_dev, int64_t ys_stride, const int32_t *y_rows_dev, const uint64_t *y_ptrs_dev,
                             void *work_dev, int n_experts, int max_slots, int d_model, int d_ff, int device,
                             void *stream) {
  if (!(dec_dev && (codes_dev || ils) && row_off_dev && minmax_dev && descs_dev && offsets_dev && work_dev)) {
    set_error("%s: null device pointer", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (!(n_experts >= 1 && max_slots >= 0 && d_model >= 1 && d_ff >= 1)) {
    set_error("%s: bad shape", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (d_model > QMOE_MAX_WIDTH || d_ff > QMOE_MAX_WIDTH) {
    set_error("%s: d_model/d_ff exceed QMOE_MAX_WIDTH (%d)", fn, QMOE_MAX_WIDTH);
    return QMOE_ERR_UNSUPPORTED;
  }
  if (ils && !(ils->codes && ils->blk_base && ils->table && ils->dec)) {
    set_error("%s: null pointer in the interleaved store", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (ils && (d_model % 32 != 0 || d_ff % 32 != 0)) {
    set_error("%s: lane-interleaved streams need d_model and d_ff to be multiples of 32", fn);
    return QMOE_ERR_UNSUPPORTED;
  }
  if (max_slots == 0) return QMOE_OK;
  if (!(xs_dev && hs_dev && (ys_dev || y_ptrs_dev))) {
    set_error("%s: null activation pointer", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (xs_stride < d_model || (!y_ptrs_dev && ys_stride < d_model)) {
    set_error("%s: row stride smaller than d_model", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(codes_dev) & 15u) != 0 ||
      (ils && ((reinterpret_cast<uintptr_t>(ils->codes) | reinterpret_cast<uintptr_t>(ils->table)) & 15u) != 0)) {
    set_error("%s: code stores must be 16-byte aligned", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  SparseTable tab;
  int rc = get_sparse_table(dec_dev, device, as_stream(stream), &tab);
  if (rc) return rc;
  return launch_grouped_ffn(tab, dec_dev, codes_dev, row_off_dev, minmax_dev, descs_dev, ils,
                            offsets_dev, xs_dev, xs_stride, x_rows_dev, hs_dev, ys_dev, ys_stride, y_rows_dev,
                            reinterpret_cast<const unsigned long long *>(y_ptrs_dev), work_dev, n_experts, max_slots,
                            d_model, d_ff, device, as_stream(stream));
}

int qmoe_moe_grouped_ffn(const int32_t *dec_dev, const uint16_t *codes_dev, const int32_t *row_off_dev,
                         const void *minmax_dev, const qmoe_matrix_desc *descs_dev, const int32_t *offsets_dev,
                         const void *xs_dev, void *hs_dev, void *ys_dev, void *work_dev, int n_experts,
                         int max_slots, int d_model, int d_ff, int device, void *stream) {
  return grouped_ffn_entry(__func__, dec_dev, codes_dev, row_off_dev, minmax_dev, descs_dev, nullptr,
                           offsets_dev, xs_dev, d_model, nullptr, hs_dev, ys_dev, d_model, nullptr, nullptr, work_dev,
                           n_experts, max_slots, d_model, d_ff, device, stream);
}

int qmoe_moe_grouped_ffn_interleaved(const int32_t *dec_dev, const uint16_t *codes_dev,
                                     const int32_t *row_off_dev, const void *minmax_dev,
                                     const qmoe_matrix_desc *descs_dev, const qmoe_interleaved_store *store,
                                     const int32_t *offsets_dev, const void *xs_dev, void *hs_dev, void *ys_dev,
                                     void *work_dev, int n_experts, int max_slots, int d_model, int d_ff,
                                     int device, void *stream) {
  QMOE_REQUIRE(store != nullptr, "null interleaved store");
  return grouped_ffn_entry(__func__, dec_dev, codes_dev, row_off_dev, minmax_dev, descs_dev, store, offsets_dev,
                           xs_dev, d_model, nullptr, hs_dev, ys_dev, d_model, nullptr, nullptr, work_dev, n_experts,
                           max_slots, d_model, d_ff, device, stream);
}

int qmoe_moe_grouped_ffn_rows(const int32_t *dec_dev, const uint16_t *codes_dev, const int32_t *row_off_dev,
                              const void *minmax_dev, const qmoe_matrix_desc *descs_dev,
                              const qmoe_interleaved_store *store, const int32_t *offsets_dev, const void *xs_dev,
                              int64_t xs_stride, const int32_t *x_rows_dev, void *hs_dev, void *ys_dev,
                              int64_t ys_stride, const int32_t *y_rows_dev, void *work_dev, int n_experts,
                              int max_slots, int d_model, int d_ff, int device, void *stream) {
  return grouped_ffn_entry(__func__, dec_dev, codes_dev, row_off_dev, minmax_dev, descs_dev, store, offsets_dev,
                           xs_dev, xs_stride, x_rows_dev, hs_dev, ys_dev, ys_stride, y_rows_dev, nullptr, work_dev,
                           n_experts, max_slots, d_model, d_ff, device, stream);
}

int qmoe_moe_grouped_ffn_scatter(const int32_t *dec_dev, const uint16_t *codes_dev, const int32_t *row_off_dev,
                                 const void *minmax_dev, const qmoe_matrix_desc *descs_dev,
                                 const qmoe_interleaved_store *store, const int32_t *offsets_dev, const void *xs_dev,
                                 int64_t xs_stride, const int32_t *x_rows_dev, void *hs_dev,
                                 const uint64_t *y_row_ptrs_dev, void *work_dev, int n_experts, int max_slots,
                                 int d_model, int d_ff, int device, void *stream) {
  QMOE_REQUIRE(y_row_ptrs_dev != nullptr || max_slots == 0, "null pointer list");
  return grouped_ffn_entry(__func__, dec_dev, codes_dev, row_off_dev, minmax_dev, descs_dev, store, offsets_dev,
                           xs_dev, xs_stride, x_rows_dev, hs_dev, nullptr, 0, nullptr, y_row_ptrs_dev, work_dev,
                           n_experts, max_slots, d_model, d_ff, device, stream);
}

static int ep_dispatch_entry(const char *fn, const int32_t *choice_dev, const void *hidden_dev, int64_t hidden_stride,
                             int32_t *expert_dev, int32_t *dest_dev, int32_t *slot_dev, void *send_dev,
                             void *const *blocks_dev, int32_t *overflow_dev, int n_tokens, int n_experts, int n_ranks,
                             int seq_len, int expert_capacity, int pair_capacity, int d_model, int device,
                             void *stream) {
  const bool ok_shape = n_tokens >= 0 && n_experts >= 1 && n_ranks >= 1 && d_model >= 2 && d_model % 2 == 0 &&
                        pair_capacity >= 0 && n_experts % n_ranks == 0 && seq_len >= 1 && n_tokens % seq_len == 0 &&
                        expert_capacity >= 0;
  if (!ok_shape) {
    set_error("%s: bad shape (even d_model, experts a multiple of the ranks, tokens a multiple of seq_len)", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (n_tokens == 0 && pair_capacity == 0) return QMOE_OK;
  if (!((send_dev || blocks_dev) && overflow_dev &&
        (n_tokens == 0 || (choice_dev && hidden_dev && expert_dev && dest_dev && slot_dev)))) {
    set_error("%s: null device pointer", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (hidden_stride < d_model || (reinterpret_cast<uintptr_t>(send_dev) & 3u) != 0) {
    set_error("%s: row stride smaller than the row, or a send buffer that is not 4-byte aligned", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_ep_dispatch(choice_dev, hidden_dev, hidden_stride, expert_dev, dest_dev, slot_dev, send_dev, blocks_dev,
                            overflow_dev, n_tokens, n_experts, n_experts / n_ranks, seq_len, expert_capacity,
                            n_ranks, pair_capacity, d_model, as_stream(stream));
}

int qmoe_moe_ep_dispatch(const int32_t *choice_dev, const void *hidden_dev, int64_t hidden_stride,
                         int32_t *expert_dev, int32_t *dest_dev, int32_t *slot_dev, void *send_dev,
                         int32_t *overflow_dev, int n_tokens, int n_experts, int n_ranks, int seq_len,
                         int expert_capacity, int pair_capacity, int d_model, int device, void *stream) {
  QMOE_REQUIRE(send_dev != nullptr || (n_tokens == 0 && pair_capacity == 0), "null send buffer");
  return ep_dispatch_entry(__func__, choice_dev, hidden_dev, hidden_stride, expert_dev, dest_dev, slot_dev, send_dev,
                           nullptr, overflow_dev, n_tokens, n_experts, n_ranks, seq_len, expert_capacity,
                           pair_capacity, d_model, device, stream);
}

int qmoe_moe_ep_dispatch_peer(const int32_t *choice_dev, const void *hidden_dev, int64_t hidden_stride,
                              int32_t *expert_dev, int32_t *dest_dev, int32_t *slot_dev, void *const *dest_blocks_dev,
                              int32_t *overflow_dev, int n_tokens, int n_experts, int n_ranks, int seq_len,
                              int expert_capacity, int pair_capacity, int d_model, int device, void *stream) {
  QMOE_REQUIRE(dest_blocks_dev != nullptr, "null block list");
  return ep_dispatch_entry(__func__, choice_dev, hidden_dev, hidden_stride, expert_dev, dest_dev, slot_dev, nullptr,
                           dest_blocks_dev, overflow_dev, n_tokens, n_experts, n_ranks, seq_len, expert_capacity,
                           pair_capacity, d_model, device, stream);
}

static int plan_entry(const char *fn, const void *rows_dev, int64_t row_stride, int d_model, const int32_t *bucket_dev,
                      int n_rows, int n_buckets, int32_t *offsets_dev, int32_t *slot_of_row_dev,
                      int32_t *row_of_slot_dev, const uint64_t *out_blocks_dev, int rows_per_block,
                      int64_t out_row_bytes, uint64_t *out_ptr_of_slot_dev, int device, void *stream) {
  if (!(n_rows >= 0 && n_buckets >= 1)) {
    set_error("%s: bad shape", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (n_buckets > 4096) {
    set_error("%s: at most 4096 buckets (their sizes and first slots are kept in shared memory)", fn);
    return QMOE_ERR_UNSUPPORTED;
  }
  if (!(offsets_dev && (n_rows == 0 || ((rows_dev || bucket_dev) && slot_of_row_dev && row_of_slot_dev)))) {
    set_error("%s: null device pointer", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (rows_dev && !(d_model >= 2 && d_model % 2 == 0 && row_stride >= d_model + 2 &&
                    (reinterpret_cast<uintptr_t>(rows_dev) & 3u) == 0 && row_stride % 2 == 0)) {
    set_error("%s: rows with a trailer need an even d_model, a stride that holds the trailer and 4-byte alignment", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_ep_plan(rows_dev, row_stride, d_model, bucket_dev, n_rows, n_buckets, offsets_dev, slot_of_row_dev,
                        row_of_slot_dev, out_blocks_dev, rows_per_block, out_row_bytes, out_ptr_of_slot_dev,
                        as_stream(stream));
}

int qmoe_moe_plan(const void *rows_dev, int64_t row_stride, int d_model, const int32_t *bucket_dev, int n_rows,
                  int n_buckets, int32_t *offsets_dev, int32_t *slot_of_row_dev, int32_t *row_of_slot_dev,
                  int device, void *stream) {
  return plan_entry(__func__, rows_dev, row_stride, d_model, bucket_dev, n_rows, n_buckets, offsets_dev,
                    slot_of_row_dev, row_of_slot_dev, nullptr, 0, 0, nullptr, device, stream);
}

int qmoe_moe_plan_peer(const void *rows_dev, int64_t row_stride, int d_model, int n_rows, int n_buckets,
                       int32_t *offsets_dev, int32_t *slot_of_row_dev, int32_t *row_of_slot_dev,
                       const uint64_t *out_blocks_dev, int rows_per_block, int64_t out_row_bytes,
                       uint64_t *out_ptr_of_slot_dev, int device, void *stream) {
  QMOE_REQUIRE(rows_dev != nullptr || n_rows == 0, "null rows pointer");
  QMOE_REQUIRE(out_blocks_dev && out_ptr_of_slot_dev && rows_per_block >= 1 && out_row_bytes >= 2 &&
                   out_row_bytes % 2 == 0,
               "bad output block list");
  return plan_entry(__func__, rows_dev, row_stride, d_model, nullptr, n_rows, n_buckets, offsets_dev, slot_of_row_dev,
                    row_of_slot_dev, out_blocks_dev, rows_per_block, out_row_bytes, out_ptr_of_slot_dev, device, stream);
}

int qmoe_moe_peer_barrier(int32_t *const *flag_blocks_dev, int rank, int n_ranks, int channel, int64_t limit_ms,
                          int32_t *status_dev, int device, void *stream) {
  QMOE_REQUIRE(flag_blocks_dev && status_dev, "null device pointer");
  QMOE_REQUIRE(n_ranks >= 1 && n_ranks <= 1024 && rank >= 0 && rank < n_ranks && channel >= 0, "bad rank or channel");
  QMOE_REQUIRE(limit_ms >= 1, "the wait needs a limit of at least a millisecond");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_peer_barrier(flag_blocks_dev, rank, n_ranks, channel, (uint64_t)limit_ms * 1000000ull, status_dev,
                             as_stream(stream));
}

int qmoe_sub1_code_histogram(const uint16_t *codes_dev, int64_t n_codes, uint64_t *hist_dev, int device,
                             void *stream) {
  QMOE_REQUIRE(codes_dev && hist_dev, "null device pointer");
  QMOE_REQUIRE(n_codes >= 0, "bad count");
  if (n_codes == 0) return QMOE_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_code_histogram(codes_dev, n_codes, hist_dev, as_stream(stream));
}

int qmoe_sub1_remap_tables(const int32_t *dec_dev, const uint32_t *remap_dev, uint32_t *table_out_dev,
                           int32_t *dec_out_dev, int device, void *stream) {
  QMOE_REQUIRE(dec_dev && table_out_dev && dec_out_dev, "null device pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  int *scratch = nullptr;
  QMOE_CUDA(cudaMalloc(&scratch, 2 * sizeof(int)));
  int rc = launch_remap_tables(dec_dev, remap_dev, table_out_dev, dec_out_dev, scratch, as_stream(stream));
  int host[2] = {0, 0};
  if (rc == QMOE_OK) {
    cudaError_t e = cudaMemcpyAsync(host, scratch, sizeof(host), cudaMemcpyDeviceToHost, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) rc = cuda_fail(e, "remap tables");
  }
  cudaFree(scratch);
  if (rc) return rc;
  if (host[0] != 0) {
    set_error("%s: remap is not a permutation of 0..65535", __func__);
    return QMOE_ERR_INVALID_ARG;
  }
  return QMOE_OK;
}

static int interleave_count_entry(const char *fn, const int32_t *row_off_dev, const qmoe_matrix_desc *descs_dev,
                                  const qmoe_matrix_desc *descs_host, int n_matrices, const int32_t *rows_dev,
                                  int32_t *blk_units_dev, int device, void *stream) {
  if (!(row_off_dev && descs_dev && descs_host && blk_units_dev) || n_matrices < 1) {
    set_error("%s: null pointer or bad matrix count", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  int64_t rows = 0;
  for (int m = 0; m < n_matrices; m++) {
    if (descs_host[m].height % 32 != 0 || descs_host[m].minmax_base != rows) {
      set_error("%s: matrix %d: heights must be multiples of 32 and rows must be stored back to back", fn, m);
      return QMOE_ERR_UNSUPPORTED;
    }
    rows += descs_host[m].height;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_interleave_count(row_off_dev, descs_dev, n_matrices, rows_dev, blk_units_dev, as_stream(stream));
}

int qmoe_moe_interleave_count(const int32_t *row_off_dev, const qmoe_matrix_desc *descs_dev,
                              const qmoe_matrix_desc *descs_host, int n_matrices, int32_t *blk_units_dev,
                              int device, void *stream) {
  return interleave_count_entry(__func__, row_off_dev, descs_dev, descs_host, n_matrices, nullptr, blk_units_dev,
                                device, stream);
}

int qmoe_moe_interleave_count_rows(const int32_t *row_off_dev, const qmoe_matrix_desc *descs_dev,
                                   const qmoe_matrix_desc *descs_host, int n_matrices, const int32_t *rows_dev,
                                   int32_t *blk_units_dev, int device, void *stream) {
  QMOE_REQUIRE(rows_dev != nullptr, "null row list");
  return interleave_count_entry(__func__, row_off_dev, descs_dev, descs_host, n_matrices, rows_dev, blk_units_dev,
                                device, stream);
}

static int interleave_emit_entry(const char *fn, const uint16_t *codes_dev, const int32_t *row_off_dev,
                                 const qmoe_matrix_desc *descs_dev, int n_matrices, const int32_t *rows_dev,
                                 const int64_t *blk_base_dev, const uint32_t *remap_dev, void *il_codes_dev,
                                 int device, void *stream) {
  if (!(codes_dev && row_off_dev && descs_dev && blk_base_dev && il_codes_dev) || n_matrices < 1) {
    set_error("%s: null pointer or bad matrix count", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(il_codes_dev) & 15u) != 0) {
    set_error("%s: interleaved store must be 16-byte aligned", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_interleave_emit(codes_dev, row_off_dev, descs_dev, n_matrices, rows_dev, blk_base_dev, remap_dev,
                                il_codes_dev, as_stream(stream));
}

int qmoe_moe_interleave_emit(const uint16_t *codes_dev, const int32_t *row_off_dev,
                             const qmoe_matrix_desc *descs_dev, int n_matrices, const int64_t *blk_base_dev,
                             const uint32_t *remap_dev, void *il_codes_dev, int device, void *stream) {
  return interleave_emit_entry(__func__, codes_dev, row_off_dev, descs_dev, n_matrices, nullptr, blk_base_dev,
                               remap_dev, il_codes_dev, device, stream);
}

int qmoe_moe_interleave_emit_rows(const uint16_t *codes_dev, const int32_t *row_off_dev,
                                  const qmoe_matrix_desc *descs_dev, int n_matrices, const int32_t *rows_dev,
                                  const int64_t *blk_base_dev, const uint32_t *remap_dev, void *il_codes_dev,
                                  int device, void *stream) {
  QMOE_REQUIRE(rows_dev != nullptr, "null row list");
  return interleave_emit_entry(__func__, codes_dev, row_off_dev, descs_dev, n_matrices, rows_dev, blk_base_dev,
                               remap_dev, il_codes_dev, device, stream);
}

int qmoe_moe_combine(const void *ys_dev, const void *hidden_dev, const int32_t *slot_dev, const void *prob_dev,
                     void *out_dev, int n_tokens, int d_model, int device, void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && d_model >= 1, "bad shape");
  if (n_tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(hidden_dev && slot_dev && prob_dev && out_dev, "null device pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_combine(ys_dev, hidden_dev, slot_dev, prob_dev, out_dev, n_tokens, d_model, as_stream(stream));
}

int qmoe_moe_combine_add(const void *ys_dev, const void *hidden_dev, const int32_t *slot_dev, const void *prob_dev,
                         const void *residual_dev, void *out_dev, int n_tokens, int d_model, int device,
                         void *stream) {
  QMOE_REQUIRE(n_tokens >= 0 && d_model >= 1, "bad shape");
  if (n_tokens == 0) return QMOE_OK;
  QMOE_REQUIRE(hidden_dev && slot_dev && prob_dev && residual_dev && out_dev, "null device pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_combine_add(ys_dev, hidden_dev, slot_dev, prob_dev, residual_dev, out_dev, n_tokens, d_model,
                            as_stream(stream));
}

int qmoe_moe_route_small(const float *logits_dev, const void *hidden_dev, int n_tokens, int n_experts, int d_model,
                         int capacity, void *prob_dev, int32_t *offsets_dev, int32_t *slot_dev, void *xs_dev,
                         int device, void *stream) {
  QMOE_REQUIRE(logits_dev && hidden_dev && prob_dev && offsets_dev && slot_dev && xs_dev, "null device pointer");
  QMOE_REQUIRE(n_tokens >= 1 && n_experts >= 1 && d_model >= 1 && capacity >= 0, "bad shape");
  if (n_tokens > 32) {
    set_error("%s: at most 32 tokens (use qmoe_moe_route / _rank / _scan / _permute)", __func__);
    return QMOE_ERR_UNSUPPORTED;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_route_small(logits_dev, hidden_dev, n_tokens, n_experts, d_model, capacity, prob_dev, offsets_dev,
                            slot_dev, xs_dev, as_stream(stream));
}

int qmoe_rms_norm(const void *x_dev, const void *weight_dev, void *out_dev, int rows, int d, float eps,
                  int device, void *stream) {
  QMOE_REQUIRE(rows >= 0 && d >= 1, "bad shape");
  if (rows == 0) return QMOE_OK;
  QMOE_REQUIRE(x_dev && weight_dev && out_dev, "null device pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_rms_norm(x_dev, weight_dev, out_dev, rows, d, eps, as_stream(stream));
}

int qmoe_gemv(const void *x_dev, const void *ln_weight_dev, const void *w_dev, const void *residual_dev, void *y_dev,
              void *normed_out_dev, int n, int k, float eps, int f32_out, int device, void *stream) {
  QMOE_REQUIRE(x_dev && w_dev && y_dev, "null device pointer");
  QMOE_REQUIRE(n >= 1 && k >= 8 && k % 8 == 0, "bad shape (k must be a multiple of 8)");
  QMOE_REQUIRE((reinterpret_cast<uintptr_t>(w_dev) & 15u) == 0, "matrix must be 16-byte aligned");
  QMOE_REQUIRE(!(ln_weight_dev && residual_dev), "norm and residual cannot be combined");
  QMOE_REQUIRE(!(residual_dev && f32_out), "residual output is bf16");
  if (k > 8192) {
    set_error("%s: k <= 8192 is supported", __func__);
    return QMOE_ERR_UNSUPPORTED;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_gemv(x_dev, ln_weight_dev, w_dev, residual_dev, y_dev, normed_out_dev, n, k, eps, f32_out,
                     as_stream(stream));
}

static int decode_attention_entry(const char *fn, const void *qkv_dev, void *k_cache_dev, void *v_cache_dev,
                                  const int64_t *pos_dev, void *out_dev, int heads, int head_dim, int max_len,
                                  float scale, const float *bias_dev, int32_t *status_dev, int device, void *stream) {
  if (!(qkv_dev && k_cache_dev && v_cache_dev && pos_dev && out_dev) || heads < 1 || head_dim < 1 || max_len < 1) {
    set_error("%s: null device pointer or bad shape", fn);
    return QMOE_ERR_INVALID_ARG;
  }
  if (head_dim > 256) {
    set_error("%s: head_dim <= 256 is supported", fn);
    return QMOE_ERR_UNSUPPORTED;
  }
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return launch_decode_attention(qkv_dev, k_cache_dev, v_cache_dev, pos_dev, out_dev, heads, head_dim, max_len, scale,
                                 bias_dev, status_dev, as_stream(stream));
}

int qmoe_decode_attention(const void *qkv_dev, void *k_cache_dev, void *v_cache_dev, const int64_t *pos_dev,
                          void *out_dev, int heads, int head_dim, int max_len, int device, void *stream) {
  return decode_attention_entry(__func__, qkv_dev, k_cache_dev, v_cache_dev, pos_dev, out_dev, heads, head_dim,
                                max_len, 0.f, nullptr, nullptr, device, stream);
}

int qmoe_decode_attention_ex(const void *qkv_dev, void *k_cache_dev, void *v_cache_dev, const int64_t *pos_dev,
                             void *out_dev, int heads, int head_dim, int max_len, float scale, const float *bias_dev,
                             int32_t *status_dev, int device, void *stream) {
  return decode_attention_entry(__func__, qkv_dev, k_cache_dev, v_cache_dev, pos_dev, out_dev, heads, head_dim,
                                max_len, scale, bias_dev, status_dev, device, stream);
}

int64_t qmoe_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int qmoe_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  g_profile_on = on != 0;
  if (g_profile_on) g_profile_calls.reserve(kMaxProfileCalls);  // event pointers handed out stay valid
  return QMOE_OK;
}

int qmoe_profile_read(float *wi_ms, float *wo_ms, int *n_calls) {
  QMOE_REQUIRE(wi_ms && wo_ms && n_calls, "null output pointer");
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  float wi = 0.f, wo = 0.f;
  int n = 0;
  int rc = QMOE_OK;
  for (auto &c : g_profile_calls) {
    float a = 0.f, b = 0.f;
    cudaError_t e = cudaEventSynchronize(c.ev[3]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&a, c.ev[0], c.ev[1]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&b, c.ev[2], c.ev[3]);
    if (e == cudaSuccess) {
      wi += a;
      wo += b;
      n++;
    } else {
      rc = cuda_fail(e, "profile events");
    }
    for (int i = 0; i < 4; i++) cudaEventDestroy(c.ev[i]);
  }
  g_profile_calls.clear();
  *wi_ms = wi;
  *wo_ms = wo;
  *n_calls = n;
  return rc;
}

int qmoe_sub1_release(int device) {
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return release_tables(device);
}

int qmoe_sub1_forget(const int32_t *dec_dev, int device) {
  QMOE_REQUIRE(dec_dev != nullptr, "null device pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  return release_tables(device, dec_dev);
}

int qmoe_moe_set_tile_wait_limit(uint32_t spins) { return set_tile_wait_limit(spins); }

int qmoe_moe_tile_timeouts(int device, int reset, int *count_out) {
  QMOE_REQUIRE(count_out != nullptr, "null output pointer");
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
  int *word = tile_status_word(device);
  if (word == nullptr) return cuda_fail(cudaGetLastError(), "tile status word");
  QMOE_CUDA(cudaDeviceSynchronize());
  QMOE_CUDA(cudaMemcpy(count_out, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (reset) QMOE_CUDA(cudaMemset(word, 0, sizeof(int)));
  return QMOE_OK;
}

}  // extern "C"
