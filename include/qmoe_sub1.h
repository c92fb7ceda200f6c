/*
 * qmoe_sub1.h -- C ABI of the B200 (sm_100a) implementation of QMoE's compressed-expert
 * inference path: fused dictionary decode + matvec / small-batch matmul, the encoder, and the
 * grouped expert FFN of a top-1 MoE layer.
 *
 * Every entry point takes plain pointers and sizes.  Pointers named *_dev are device pointers on
 * `device`; all work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 * default stream, which is what the reference launches on, sub1_cuda_kernel.cu:29).  Functions
 * return QMOE_OK (0) or a negative status; qmoe_last_error() gives a message for the calling
 * thread.  There is no CPU fallback: without a usable CUDA device the compute entry points fail.
 *
 * Reference citations are into IST-DASLab/qmoe.
 */
#ifndef QMOE_SUB1_H_
#define QMOE_SUB1_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMOE_OK 0
#define QMOE_ERR_INVALID_ARG (-1)   /* null pointer, negative size, odd width, ... */
#define QMOE_ERR_CUDA (-2)          /* a CUDA runtime call or a launch failed */
#define QMOE_ERR_UNSUPPORTED (-3)   /* shape or table outside what the kernels handle */
#define QMOE_ERR_STREAM (-4)        /* a code stream failed validation (rows not tiled exactly) */
#define QMOE_ERR_TIMEOUT (-5)       /* a bounded device-side wait gave up */

#define QMOE_DICT_COUNT 65536       /* sub1.py:30 */
#define QMOE_TRIE_ROOT 65536        /* sub1_cuda_kernel.cu:209 */

/* Flags of qmoe_sub1_matmul / grouped calls. */
#define QMOE_FLAG_ACCUMULATE 1      /* y += bf16(Wx) (sub1_cuda_kernel.cu:199-200); else y = bf16(Wx) */
#define QMOE_FLAG_RELU 2            /* y = max(bf16(Wx), 0); the ReLU between wi and wo (sub1.py:317) */

const char *qmoe_last_error(void);
int qmoe_version(void);

/* Host-side construction of the fixed dictionary: dec int32[2*65536] and trie int32[65537*9],
 * bit-identical to setup() in sub1.py:29-102.  Both are host pointers. */
int qmoe_sub1_build_dictionary(int32_t *dec_host, int32_t *trie_host);

/* Replaces sub1matvec (sub1_cuda.cpp:35-45 -> sub1matvec_cuda, sub1_cuda_kernel.cu:70-88 ->
 * Sub1MatVec, :129-202): y[r] += bf16(sum_c W[r,c] x[c]) for one compressed matrix and one bf16
 * vector.  Any height >= 1 and any width >= 1 (odd widths included, width <= QMOE_MAX_WIDTH) is
 * accepted, not only the reference's six hard-coded shapes.
 *
 * The library derives a 4-byte form of `dec` the first time it sees a (device, dec_dev) pair and
 * keeps it, keyed by that ADDRESS.  The cache does not look at the contents again: after
 * overwriting a dec tensor in place, or after freeing it (an allocator may hand the same address
 * to a different table later), call qmoe_sub1_forget (or qmoe_sub1_release) before the address is
 * used again.  The Python shim does this when a dec tensor is garbage collected.
 *   dec_dev        int32[131072]   decoder table (sub1.py:60-72)
 *   w_comp_dev     uint16[n_codes] code stream, rows concatenated
 *   row_off_dev    int32[height+1] exclusive prefix sums of codes per row
 *   ter_minmax_dev bf16[2*height]  interleaved (min_r, max_r)
 *   x_dev          bf16[width], y_dev bf16[height] (read-modify-write) */
int qmoe_sub1_matvec(const int32_t *dec_dev, const uint16_t *w_comp_dev, const int32_t *row_off_dev,
                     const void *ter_minmax_dev, const void *x_dev, void *y_dev, int height,
                     int width, int64_t n_codes, int device, void *stream);

/* No counterpart in the reference: qmoe_sub1_matvec for callers that must not allocate device
 * memory -- code hosted by a framework that owns all GPU memory and forbids side allocations, a
 * process whose memory budget is entirely given to a pool, a thread that may never block in the
 * driver's allocator.  Same arguments and result as qmoe_sub1_matvec, but the derived dictionary
 * lives in a fixed array inside the library's device image (about 256 KB, held by every GPU that
 * loads the library until the process exits) and nothing is allocated, by this call or by any
 * routine it uses.  Limits: width <= QMOE_MAX_WIDTH, fewer than 2^31 codes; larger input is
 * rejected with QMOE_ERR_UNSUPPORTED.  The array is shared by all calls and rebuilt from `dec_dev`
 * by each of them on `stream`, so calls that overlap on one GPU (other streams or threads) race and
 * must be serialised by the caller.  The first call on a device also looks up the array's address
 * and raises a kernel attribute; make that first call before any stream capture. */
int qmoe_sub1_matvec_noalloc(const int32_t *dec_dev, const uint16_t *w_comp_dev,
                             const int32_t *row_off_dev, const void *ter_minmax_dev, const void *x_dev,
                             void *y_dev, int height, int width, int64_t n_codes, int device,
                             void *stream);

/* Replaces the per-token loop of Sub1Linear.forward (sub1.py:132-143): x[tokens, width] ->
 * y[tokens, height] with the codes decoded once per group of tokens.  x rows are `x_stride`
 * elements apart, y rows `y_stride`.  flags: QMOE_FLAG_*. */
int qmoe_sub1_matmul(const int32_t *dec_dev, const uint16_t *w_comp_dev, const int32_t *row_off_dev,
                     const void *ter_minmax_dev, const void *x_dev, void *y_dev, int height,
                     int width, int64_t n_codes, int tokens, int64_t x_stride, int64_t y_stride,
                     int flags, int device, void *stream);

/* Decodes a compressed matrix to ternary symbols uint8[height, width] (0, 1 = row min, 2 = row
 * max) with the same table walk the matvec kernels use; the GPU twin of decompress()
 * (test.py:103-115).  status_dev (int32[1], may be NULL) receives the number of rows whose codes
 * do not cover exactly `width` weights. */
int qmoe_sub1_decode(const int32_t *dec_dev, const uint16_t *w_comp_dev, const int32_t *row_off_dev,
                     uint8_t *sym_dev, int32_t *status_dev, int height, int width, int64_t n_codes,
                     int device, void *stream);

/* Replaces sub1pack (sub1_cuda.cpp:47-54 -> sub1pack_cuda, sub1_cuda_kernel.cu:92-126), split in
 * two so that the caller owns the allocation of the output between the phases.
 * prepare = row_off.zero_() + Sub1PreparePack (:211-239) + cumsum: greedy longest-match walk of
 * every row; the row's codes overwrite the head of the row in w_tern (int32[height, width], values
 * 0/1/2, clobbered exactly like the reference) and row_off (int32[height+1]) ends as exclusive
 * prefix sums.  Any height >= 1 (the reference needs height % 32 == 0).
 * emit = Sub1Pack (:241-250): compaction into w_comp_dev uint16[row_off[height]]. */
int qmoe_sub1_pack_prepare(const int32_t *trie_dev, int32_t *w_tern_dev, int32_t *row_off_dev,
                           int height, int width, int device, void *stream);
int qmoe_sub1_pack_emit(const int32_t *w_tern_dev, const int32_t *row_off_dev, uint16_t *w_comp_dev,
                        int height, int width, int device, void *stream);

/* Batched encoder on uint8 symbols for `n_mat` matrices of one shape (sym_dev uint8[n_mat,
 * height, width]); no host synchronisation.  count: codes_tmp_dev uint16[n_mat, height, width/2]
 * receives each row's codes, row_len_dev int32[n_mat*height] the per-row counts.  The caller then
 * prefix-sums row_len into per-matrix row_off and a per-matrix base (in codes), and calls gather:
 * out_dev[mat_base[m] + row_off[m][r] + i] = codes of row r.  Same greedy rule as
 * sub1_cuda_kernel.cu:211-239. */
int qmoe_sub1_pack_u8_count(const int32_t *trie_dev, const uint8_t *sym_dev, uint16_t *codes_tmp_dev,
                            int32_t *row_len_dev, int n_mat, int height, int width, int device,
                            void *stream);
int qmoe_sub1_pack_u8_gather(const uint16_t *codes_tmp_dev, const int32_t *row_off_dev,
                             const int64_t *mat_base_dev, uint16_t *out_dev, int n_mat, int height,
                             int width, int device, void *stream);

/* Seeded synthetic ternary symbols for benchmarks: sym[i] = 0 with probability p_zero, else 1 or 2
 * with equal probability, from a counter-based hash of (seed, first_index + i). */
int qmoe_synth_ternary(uint8_t *sym_dev, int64_t count, uint64_t seed, uint64_t first_index,
                       float p_zero, int device, void *stream);

/* ---- Grouped expert FFN of one top-1 MoE layer (FasterMLP.forward, sub1.py:306-321) --------- */

/* One compressed matrix inside an expert store.  All offsets are in elements of the store's
 * arrays; code_base must be a multiple of 8 (16-byte aligned streams). */
typedef struct {
  int64_t code_base;    /* first code of the matrix in the store's uint16 code array */
  int64_t n_codes;
  int64_t rowoff_base;  /* first of the matrix's height+1 row offsets (relative to code_base) */
  int64_t minmax_base;  /* first (min,max) pair of the matrix, in bf16x2 units */
  int32_t height;
  int32_t width;
} qmoe_matrix_desc;

/* Top-1 choice of the Switch router the reference calls at sub1.py:310 (transformers 4.28
 * SwitchTransformersTop1Router): probabilities = softmax(logits) in fp32 rounded to bf16,
 * choice = first index holding the largest bf16 probability, prob = that probability.
 *   logits_dev float[n_tokens, n_experts]; choice_dev int32[n_tokens]; prob_dev bf16[n_tokens] */
int qmoe_moe_route(const float *logits_dev, int32_t *choice_dev, void *prob_dev, int n_tokens,
                   int n_experts, int device, void *stream);

/* Capacity rule + stable ranking.  A token is kept when fewer than `capacity` earlier tokens of
 * its own sequence (seq_len consecutive tokens; n_tokens % seq_len == 0) made the same choice --
 * the router's cumsum(one_hot) <= expert_capacity mask.  Tokens whose choice is negative count as
 * dropped already.
 *   bucket_dev int32[n_tokens]  choice if kept, else -1 (must not alias choice_dev)
 *   rank_dev   int32[n_tokens]  number of earlier kept tokens (whole batch) in the same bucket
 *   counts_dev int32[n_buckets] kept tokens per bucket (overwritten)
 * Deterministic: ranks follow token order. */
int qmoe_moe_rank(const int32_t *choice_dev, int32_t *bucket_dev, int32_t *rank_dev, int32_t *counts_dev,
                  int n_tokens, int n_buckets, int seq_len, int capacity, int device, void *stream);

/* The capacity rule alone, one launch: expert_dev[t] = choice_dev[t] if kept, else -1 (must not
 * alias choice_dev). */
int qmoe_moe_keep(const int32_t *choice_dev, int32_t *expert_dev, int n_tokens, int n_experts, int seq_len,
                  int capacity, int device, void *stream);

/* offsets[0..n] = exclusive prefix sums of counts[0..n) (offsets has n+1 entries). */
int qmoe_moe_scan(const int32_t *counts_dev, int32_t *offsets_dev, int n, int device, void *stream);

/* slot[token] = offsets[bucket] + rank (or -1 when bucket < 0) and xs[slot] = hidden[token]: the
 * gather of kept tokens into bucket order.  hidden/xs are bf16 rows of d_model elements; hidden
 * rows are hidden_stride elements apart, xs rows xs_stride. */
int qmoe_moe_permute(const int32_t *bucket_dev, const int32_t *rank_dev, const int32_t *offsets_dev,
                     int32_t *slot_dev, const void *hidden_dev, void *xs_dev, int n_tokens, int d_model,
                     int64_t hidden_stride, int64_t xs_stride, int device, void *stream);

/* out[i] = ys[slot[i]] for slot[i] >= 0; rows with slot < 0 are zero-filled. */
int qmoe_moe_unpermute(const void *ys_dev, const int32_t *slot_dev, void *out_dev, int n_tokens, int d_model,
                       int64_t ys_stride, int64_t out_stride, int device, void *stream);

/* Grouped wo(ReLU(wi(x))) over every expert that received tokens: tokens are sorted by expert,
 * expert e owns rows offsets[e]..offsets[e+1] of xs / hs / ys.  descs_dev[2e] is wi (height d_ff,
 * width d_model), descs_dev[2e+1] is wo.  Everything is decided on the device from offsets_dev;
 * no host synchronisation.  work_dev is caller-provided scratch of qmoe_moe_work_bytes() bytes.
 *   xs_dev bf16[n_slots, d_model], hs_dev bf16[n_slots, d_ff], ys_dev bf16[n_slots, d_model] */
int64_t qmoe_moe_work_bytes(int n_experts, int max_slots, int d_model, int d_ff);

/* Inside qmoe_moe_grouped_ffn, experts with at least `tokens` tokens are multiplied on the tensor
 * cores (tcgen05): their rows are decoded once into bf16 tiles in shared memory and multiplied with
 * blocks of 64 tokens, instead of being re-decoded for every group of four tokens.  0 disables that
 * path; values below 8 are raised to 8.  Default 448 (or the environment variable
 * QMOE_TILE_MIN_TOKENS), the measured break-even.  Returns the previous value.  No counterpart in
 * the reference, which runs one matvec per token (sub1.py:139-142). */
int qmoe_moe_set_tile_min_tokens(int tokens);

/* For measurements: the per-row kernel of qmoe_moe_grouped_ffn normally cuts every matrix into the
 * number of equal work items that fills whole rounds of the SMs best (decided on the device from
 * the step's routing).  A value > 0 forces that many items per wi / wo matrix instead (ignored
 * where it would not fit the work buffer or give items of fewer than 32 rows); 0 restores the
 * choice.  Process-wide. */
int qmoe_moe_set_items_per_matrix(int wi, int wo);

/* With lane-interleaved streams, qmoe_moe_grouped_ffn runs the per-thread work items of wi and of wo
 * in ONE persistent launch: an item of wo starts as soon as the items of wi for the same (expert,
 * token group) have stored their rows (a completion count per pair, waited for at most two seconds;
 * a wait that runs out is counted in the word qmoe_moe_tile_timeouts reads), so no SM idles
 * between the two linears.  Taken for steps of at most eight token slots per SM (max_slots <= 8 *
 * SMs), where a step has only a handful of items per SM; larger steps keep one launch per linear,
 * whose hot dictionary part is sized for each width.  on = 0 always uses one launch per linear
 * (measurements); returns the previous setting.  Process-wide, default 1. */
int qmoe_moe_set_fused_phases(int on);

/* Host read-back (synchronises `stream`) of what the last qmoe_moe_grouped_ffn call that used
 * work_dev planned, for tests and reports; max_slots / d_ff as in that call.  out_host int32[10]:
 * [0] / [1] row-per-thread work items of wi / wo, [2] / [3] row-per-warp work items of wi / wo,
 * [4] / [5] rows per row-per-thread item of wi / wo, [6] / [7] tensor-core tile items of wi / wo,
 * [8] tokens decoded together, [9] wo items whose CTA also does the remainder rows of its matrix
 * (a height that is not a multiple of 1024) one row per warp.  No counterpart in the reference
 * (one launch per token and matrix, sub1.py:139-142). */
int qmoe_moe_work_summary(const void *work_dev, int max_slots, int d_ff, int32_t *out_host, int device,
                          void *stream);
int qmoe_moe_grouped_ffn(const int32_t *dec_dev, const uint16_t *codes_dev, const int32_t *row_off_dev,
                         const void *minmax_dev, const qmoe_matrix_desc *descs_dev,
                         const int32_t *offsets_dev, const void *xs_dev, void *hs_dev, void *ys_dev,
                         void *work_dev, int n_experts, int max_slots, int d_model, int d_ff,
                         int device, void *stream);

/* Lane-interleaved copy of a store's code streams, the layout the grouped kernel reads fastest.
 * No counterpart in the reference, whose kernel (sub1_cuda_kernel.cu:129-202) reads w_comp row by
 * row; the copy holds the same codes (optionally renumbered) and decodes to the same weights.
 * Rows are taken in blocks of 32; chunk k (codes 8k..8k+7) of row l of a block is the 16-byte entry
 * k * 32 + l of the block, and every row of a block is zero-padded to the block's longest row
 * rounded up to 8 codes.  Heights must be multiples of 32 and the matrices' rows consecutive
 * (minmax_base = rows before).
 *
 * Renumbering: the kernel keeps the first entries of the table in shared memory (as many as the
 * activations leave room for, 45 000 - 53 000 of the 65 536), so the copy may store remap[code]
 * instead of code, with remap a permutation that gives frequent codes small numbers
 * (qmoe_sub1_code_histogram counts them); qmoe_sub1_remap_tables writes the sparse table and the
 * reference table words in the new order (remap_dev NULL = identity).
 *   1. qmoe_moe_interleave_count: blk_units_dev int32[total_rows / 32] := 16-byte entries per block
 *      (descs_host: the same descriptors in host memory, for validation);
 *   2. the caller forms blk_base int64[total_rows / 32 + 1], the exclusive prefix sum, and allocates
 *      16 * blk_base[last] bytes;
 *   3. qmoe_moe_interleave_emit fills them;
 *   4. qmoe_moe_grouped_ffn_interleaved is qmoe_moe_grouped_ffn reading the copy.  Experts on the
 *      tensor-core tile path still read codes_dev with dec_dev; codes_dev may be NULL (a store that
 *      freed its row-by-row streams), which turns that path off. */
typedef struct qmoe_interleaved_store {
  const void *codes;       /* 16-byte entries, device */
  const int64_t *blk_base; /* [total_rows / 32 + 1], device */
  const uint32_t *table;   /* uint32[65536] from qmoe_sub1_remap_tables, device */
  const int32_t *dec;      /* int32[131072] from qmoe_sub1_remap_tables, device */
  const int32_t *rows;     /* NULL, or int32[total_rows], device: the row of its matrix whose stream sits at
                              position p of the store (a permutation inside every matrix, the one given to
                              qmoe_moe_interleave_count_rows / _emit_rows).  Blocks are made of 32 consecutive
                              POSITIONS; putting rows of similar length side by side (sorted by code count
                              inside every 1024 positions) lets the 32 lanes of a warp finish together and
                              shrinks the padding.  Results do not depend on it. */
} qmoe_interleaved_store;

int qmoe_sub1_code_histogram(const uint16_t *codes_dev, int64_t n_codes, uint64_t *hist_dev /* [65536], added to */,
                             int device, void *stream);
int qmoe_sub1_remap_tables(const int32_t *dec_dev, const uint32_t *remap_dev /* [65536] or NULL */,
                           uint32_t *table_out_dev, int32_t *dec_out_dev, int device, void *stream);
int qmoe_moe_interleave_count(const int32_t *row_off_dev, const qmoe_matrix_desc *descs_dev,
                              const qmoe_matrix_desc *descs_host, int n_matrices, int32_t *blk_units_dev,
                              int device, void *stream);
int qmoe_moe_interleave_emit(const uint16_t *codes_dev, const int32_t *row_off_dev,
                             const qmoe_matrix_desc *descs_dev, int n_matrices, const int64_t *blk_base_dev,
                             const uint32_t *remap_dev /* [65536] or NULL */, void *il_codes_dev, int device,
                             void *stream);
int qmoe_moe_interleave_count_rows(const int32_t *row_off_dev, const qmoe_matrix_desc *descs_dev,
                                   const qmoe_matrix_desc *descs_host, int n_matrices, const int32_t *rows_dev,
                                   int32_t *blk_units_dev, int device, void *stream);
int qmoe_moe_interleave_emit_rows(const uint16_t *codes_dev, const int32_t *row_off_dev,
                                  const qmoe_matrix_desc *descs_dev, int n_matrices, const int32_t *rows_dev,
                                  const int64_t *blk_base_dev, const uint32_t *remap_dev /* [65536] or NULL */,
                                  void *il_codes_dev, int device, void *stream);
int qmoe_moe_grouped_ffn_interleaved(const int32_t *dec_dev, const uint16_t *codes_dev,
                                     const int32_t *row_off_dev, const void *minmax_dev,
                                     const qmoe_matrix_desc *descs_dev, const qmoe_interleaved_store *store,
                                     const int32_t *offsets_dev, const void *xs_dev, void *hs_dev, void *ys_dev,
                                     void *work_dev, int n_experts, int max_slots, int d_model, int d_ff,
                                     int device, void *stream);

/* qmoe_moe_grouped_ffn(_interleaved) with row lists instead of sorted copies: token (slot) s reads
 * its input from row x_rows_dev[s] of xs_dev (rows xs_stride elements apart) and its result goes to
 * row y_rows_dev[s] of ys_dev (rows ys_stride apart); NULL lists mean s itself.  hs_dev stays
 * bf16[max_slots, d_ff] indexed by slot.  store may be NULL (row-by-row streams).  With this the
 * layer needs no permute / un-permute pass over its activations. */
int qmoe_moe_grouped_ffn_rows(const int32_t *dec_dev, const uint16_t *codes_dev, const int32_t *row_off_dev,
                              const void *minmax_dev, const qmoe_matrix_desc *descs_dev,
                              const qmoe_interleaved_store *store, const int32_t *offsets_dev, const void *xs_dev,
                              int64_t xs_stride, const int32_t *x_rows_dev, void *hs_dev, void *ys_dev,
                              int64_t ys_stride, const int32_t *y_rows_dev, void *work_dev, int n_experts,
                              int max_slots, int d_model, int d_ff, int device, void *stream);

/* Dispatch metadata of the expert-parallel layer (qmoe_b200/ep.py); the reference only moves whole
 * activations between GPUs (sub1.py:307-309,320) and loops over experts on the host (:315-317).
 *
 * qmoe_moe_ep_dispatch, two launches: (1) the router's capacity rule on the global expert choice
 * (as qmoe_moe_rank: expert_dev[t] = choice or -1), the owning rank dest_dev[t] = expert /
 * (n_experts / n_ranks), and the trailers of all n_ranks * pair_capacity exchange slots reset to -1;
 * (2) per token: its stable rank among the kept tokens with the same destination, its slot
 * dest * pair_capacity + rank (slot_dev[t]), the copy of its row into send_dev[slot] (rows of
 * d_model + 8 bf16: the row, then a 16-byte trailer whose first int32 is the expert's index on its
 * rank).  A token whose rank does not fit pair_capacity is not sent: slot -1 -- it passes through
 * the layer scaled by its router probability, like a token dropped by the capacity rule -- and
 * *overflow_dev is incremented (the caller zeroes it once and reads it at its own sync points).
 *
 * qmoe_moe_plan, one launch: buckets rows into n_buckets groups, stable in row order.  The bucket
 * of row i is the int32 at element d_model of row i of rows_dev (rows row_stride elements apart:
 * the trailer above) or, with rows_dev NULL, bucket_dev[i]; values outside [0, n_buckets) mean
 * "no row".  offsets_dev int32[n_buckets + 1]: exclusive prefix sums of the bucket sizes;
 * slot_of_row_dev[i] = offsets[bucket] + rank (or -1); row_of_slot_dev[slot] = i (entries at and
 * beyond offsets[n_buckets] are left untouched).  At most 4096 buckets. */
int qmoe_moe_ep_dispatch(const int32_t *choice_dev, const void *hidden_dev, int64_t hidden_stride,
                         int32_t *expert_dev, int32_t *dest_dev, int32_t *slot_dev, void *send_dev,
                         int32_t *overflow_dev, int n_tokens, int n_experts, int n_ranks, int seq_len,
                         int expert_capacity, int pair_capacity, int d_model, int device, void *stream);
int qmoe_moe_plan(const void *rows_dev, int64_t row_stride, int d_model, const int32_t *bucket_dev, int n_rows,
                  int n_buckets, int32_t *offsets_dev, int32_t *slot_of_row_dev, int32_t *row_of_slot_dev,
                  int device, void *stream);

/* The same exchange over peer memory (NVLink / NVSwitch), without a collective library in the data
 * path.  The reference has nothing to compare: its GPUs only ever pass whole activations on
 * (sub1.py:307-309,320).  Every rank owns a receive buffer of n_ranks * pair_capacity rows of
 * d_model + 8 bf16 and a return buffer of n_ranks * pair_capacity rows of d_model bf16 that its peers
 * have mapped (CUDA IPC, the driver's virtual memory API, or torch's symmetric memory); block r of
 * either belongs to rank r.  All pointers below are addresses valid on THIS GPU.
 *
 * qmoe_moe_ep_dispatch_peer: qmoe_moe_ep_dispatch that stores every kept row straight into its
 * destination's receive buffer.  dest_blocks_dev[d] (device array of n_ranks pointers) = first row
 * of this rank's block in rank d's receive buffer.  slot_dev as above (dest * pair_capacity + rank).
 *
 * qmoe_moe_plan_peer: qmoe_moe_plan over the trailers of the received rows that also emits, for
 * every slot s, the address of its result row: out_ptr_of_slot_dev[s] = out_blocks_dev[i /
 * rows_per_block] + (i % rows_per_block) * out_row_bytes for the received row i = row_of_slot[s];
 * out_blocks_dev[q] (device array of n_ranks addresses) = first row of this rank's block in rank
 * q's return buffer, rows_per_block = pair_capacity.
 *
 * qmoe_moe_grouped_ffn_scatter: qmoe_moe_grouped_ffn_rows whose result rows are stored to the
 * addresses y_row_ptrs_dev[s] (2-byte aligned, d_model bf16 each; may lie in a peer's memory).
 *
 * qmoe_moe_peer_barrier, one launch of one CTA: makes this GPU's earlier stores visible to its
 * peers, raises flag [channel][rank] in every peer's flag block and waits for flag [channel][p] of
 * every peer p in its own (flag_blocks_dev: device array of n_ranks pointers to the ranks' blocks of
 * at least (channel + 1) * n_ranks int32, zeroed before first use; a flag is cleared by the rank that
 * waited for it, so the blocks need no reset between steps).  Ranks must launch matching barriers in
 * the same order, each on its own GPU (never two ranks on one GPU: they would wait for each other's
 * kernels).  The waits end after limit_ms milliseconds; *status_dev is then incremented and the
 * kernel returns: from then on the buffers' contents are undefined and the flag blocks must be
 * zeroed again by all ranks before reuse.  Use one channel per barrier of a step. */
int qmoe_moe_ep_dispatch_peer(const int32_t *choice_dev, const void *hidden_dev, int64_t hidden_stride,
                              int32_t *expert_dev, int32_t *dest_dev, int32_t *slot_dev, void *const *dest_blocks_dev,
                              int32_t *overflow_dev, int n_tokens, int n_experts, int n_ranks, int seq_len,
                              int expert_capacity, int pair_capacity, int d_model, int device, void *stream);
int qmoe_moe_plan_peer(const void *rows_dev, int64_t row_stride, int d_model, int n_rows, int n_buckets,
                       int32_t *offsets_dev, int32_t *slot_of_row_dev, int32_t *row_of_slot_dev,
                       const uint64_t *out_blocks_dev, int rows_per_block, int64_t out_row_bytes,
                       uint64_t *out_ptr_of_slot_dev, int device, void *stream);
int qmoe_moe_grouped_ffn_scatter(const int32_t *dec_dev, const uint16_t *codes_dev, const int32_t *row_off_dev,
                                 const void *minmax_dev, const qmoe_matrix_desc *descs_dev,
                                 const qmoe_interleaved_store *store, const int32_t *offsets_dev, const void *xs_dev,
                                 int64_t xs_stride, const int32_t *x_rows_dev, void *hs_dev,
                                 const uint64_t *y_row_ptrs_dev, void *work_dev, int n_experts, int max_slots,
                                 int d_model, int d_ff, int device, void *stream);
int qmoe_moe_peer_barrier(int32_t *const *flag_blocks_dev, int rank, int n_ranks, int channel, int64_t limit_ms,
                          int32_t *status_dev, int device, void *stream);

/* out[token] = bf16(prob[token] * (slot >= 0 ? ys[slot] : hidden[token])): the scatter back to
 * token order, the pass-through of dropped tokens and the router-probability scaling of
 * sub1.py:312,318. */
int qmoe_moe_combine(const void *ys_dev, const void *hidden_dev, const int32_t *slot_dev,
                     const void *prob_dev, void *out_dev, int n_tokens, int d_model, int device,
                     void *stream);

/* Fused helpers of the batch-1 decode step of the generation harness (qmoe_b200/decoder.py).  No
 * counterpart in the reference, which leaves these parts to HuggingFace's Switch Transformers
 * modules behind model.generate (sub1.py:373-379).
 *   qmoe_moe_combine_add: out = bf16(residual + qmoe_moe_combine(...)), one launch.
 *   qmoe_moe_route_small: qmoe_moe_route + _rank + _scan + _permute for at most 32 tokens of one
 *     sequence in one launch: prob bf16[n], offsets int32[n_experts + 1], slot int32[n] (-1 =
 *     dropped by the capacity rule), xs[slot] = hidden[token].
 *   qmoe_rms_norm: out[r] = bf16(bf16(x[r] * rsqrt(mean(x[r]^2) + eps)) * weight), bf16 [rows, d].
 *   qmoe_gemv: y = W x for one token, W bf16 [n][k] row-major (k a multiple of 8, k <= 8192,
 *     16-byte aligned), fp32 accumulation.  ln_weight_dev != NULL: x is first RMS-normalised as in
 *     qmoe_rms_norm (and stored to normed_out_dev if that is not NULL).  residual_dev != NULL:
 *     y = bf16(residual + bf16(W x)).  f32_out: y is fp32[n], else bf16[n].
 *   qmoe_decode_attention: one new token of causal self-attention.  qkv_dev bf16 [3][heads][head_dim]
 *     of the token; caches bf16 [heads][max_len][head_dim]; *pos_dev (device int64) is the token's
 *     position: its key and value are written there, then
 *     out[head] = softmax(q . K[0..pos] / sqrt(head_dim)) V[0..pos] (fp32 arithmetic, bf16 result).
 *     head_dim <= 256.  A position outside [0, max_len) is clamped (the last slot is overwritten).
 *   qmoe_decode_attention_ex: the same with the score scale given (scale <= 0: 1 / sqrt(head_dim);
 *     T5 / Switch attention uses 1), an optional additive bias bias_dev fp32 [heads][max_len] (the
 *     relative-position bias of the query's row, per key position) and, when status_dev is not NULL,
 *     a position outside [0, max_len) refused: *status_dev is incremented and nothing is written. */
int qmoe_moe_combine_add(const void *ys_dev, const void *hidden_dev, const int32_t *slot_dev,
                         const void *prob_dev, const void *residual_dev, void *out_dev, int n_tokens,
                         int d_model, int device, void *stream);
int qmoe_moe_route_small(const float *logits_dev, const void *hidden_dev, int n_tokens, int n_experts,
                         int d_model, int capacity, void *prob_dev, int32_t *offsets_dev, int32_t *slot_dev,
                         void *xs_dev, int device, void *stream);
int qmoe_rms_norm(const void *x_dev, const void *weight_dev, void *out_dev, int rows, int d, float eps,
                  int device, void *stream);
int qmoe_gemv(const void *x_dev, const void *ln_weight_dev, const void *w_dev, const void *residual_dev,
              void *y_dev, void *normed_out_dev, int n, int k, float eps, int f32_out, int device, void *stream);
int qmoe_decode_attention(const void *qkv_dev, void *k_cache_dev, void *v_cache_dev, const int64_t *pos_dev,
                          void *out_dev, int heads, int head_dim, int max_len, int device, void *stream);
int qmoe_decode_attention_ex(const void *qkv_dev, void *k_cache_dev, void *v_cache_dev, const int64_t *pos_dev,
                             void *out_dev, int heads, int head_dim, int max_len, float scale, const float *bias_dev,
                             int32_t *status_dev, int device, void *stream);

/* Number of kernels this library has launched in the calling process (all devices, all entry points). */
int64_t qmoe_launch_count(void);

/* Optional timing of the two grouped launches inside qmoe_moe_grouped_ffn, for roofline reports.
 * qmoe_profile_enable(1) makes every later qmoe_moe_grouped_ffn call record CUDA events around its
 * wi launch and its wo launch on the call's stream (at most 256 calls are kept; later ones are not
 * recorded).  qmoe_profile_read synchronises on the recorded events, returns the summed durations in
 * milliseconds and the number of recorded calls, and clears the record. */
int qmoe_profile_enable(int on);
int qmoe_profile_read(float *wi_ms, float *wo_ms, int *n_calls);

/* Frees every per-device cache the library holds (derived decoder tables keyed by the dec pointer).
 * Call it after overwriting a dec tensor in place, and before unloading. */
int qmoe_sub1_release(int device);

/* Frees the cached derived table of one (device, dec_dev) pair, if any: to be called when that dec
 * tensor is freed or overwritten, so that a later table at the same address is derived afresh.  No
 * counterpart in the reference, which reads `dec` directly in its kernel (sub1_cuda_kernel.cu:188). */
int qmoe_sub1_forget(const int32_t *dec_dev, int device);

/* Status of the tensor-core tile kernels inside qmoe_moe_grouped_ffn.  Each of their waits on an
 * MMA-completion barrier is bounded; a CTA whose wait runs out stops, writes zeros for the output
 * rows it did not finish and adds one to a per-device word that no later call clears.
 * qmoe_moe_tile_timeouts synchronises the device, stores that word in *count_out and clears it when
 * `reset` is non-zero: callers check it at their own synchronisation points, non-zero means that
 * outputs since the last reset are incomplete.  qmoe_moe_set_tile_wait_limit(spins) lowers the
 * bound of such a wait to spins - 1 polls (1: give up without polling; 0 restores the default of
 * 2^24); it exists so that a test can make a wait run out without anything hanging.  No counterpart in the reference. */
int qmoe_moe_tile_timeouts(int device, int reset, int *count_out);
int qmoe_moe_set_tile_wait_limit(uint32_t spins);

#define QMOE_MAX_WIDTH 8192

#ifdef __cplusplus
}
#endif
#endif /* QMOE_SUB1_H_ */
