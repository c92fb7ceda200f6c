/*
 * CPU oracle for the QMoE sub-1-bit compressed-expert path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithms of the reference implementation
 * (IST-DASLab/qmoe) that define the compressed format and its arithmetic.  It is used by the
 * test-suite, by the smoke check and by the CPU-baseline leg of the benchmark as the checker /
 * the timed CPU baseline.  Nothing in the shipped GPU path calls into it.
 *
 * Parity status: PINNED.  The dictionary and trie it builds hash to the SHA-256 values obtained by
 * running the reference's own setup() (sub1.py:29-102), and the encoder/decoder agree with the
 * reference's CPU twins greedy()/decompress() (test.py:86-115) on the committed golden vectors
 * (tests/golden/).
 *
 * Each function cites the reference file:line it follows.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define DICT_COUNT 65536   /* sub1.py:30  COUNT = 2 ** 16 */
#define MAX_PAIRS 14       /* sub1.py:54  sequences are at most 14 pairs long */
#define TRIE_ROOT 65536    /* sub1_cuda_kernel.cu:209 */

/* ------------------------------------------------------------------------------------------ */
/* bf16 helpers: torch / CUDA round-to-nearest-even conversion                                  */
/* ------------------------------------------------------------------------------------------ */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN stays NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16(f); }
float oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/* ------------------------------------------------------------------------------------------ */
/* Dictionary + trie construction: sub1.py:29-102 (duplicated at test.py:29-78)                 */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
  double prio;               /* negative probability, as in the reference's heap tuples */
  int32_t parent;            /* dictionary index of the sequence minus its last pair */
  uint8_t len;
  uint8_t seq[MAX_PAIRS];
} node_t;

/* Python tuple order (float, list): floats first, then lists lexicographically with a proper
 * prefix sorting before its extensions (sub1.py:49-57 relies on it for ties). */
static int node_less(const node_t *a, const node_t *b) {
  if (a->prio < b->prio) return 1;
  if (a->prio > b->prio) return 0;
  int n = a->len < b->len ? a->len : b->len;
  for (int i = 0; i < n; i++) {
    if (a->seq[i] != b->seq[i]) return a->seq[i] < b->seq[i];
  }
  return a->len < b->len;
}

typedef struct { node_t *v; size_t n, cap; } heap_t;

static int heap_push(heap_t *h, const node_t *x) {
  if (h->n == h->cap) {
    size_t nc = h->cap ? 2 * h->cap : 1024;
    node_t *nv = (node_t *)realloc(h->v, nc * sizeof(node_t));
    if (!nv) return -1;
    h->v = nv; h->cap = nc;
  }
  size_t i = h->n++;
  while (i > 0) {
    size_t p = (i - 1) / 2;
    if (!node_less(x, &h->v[p])) break;
    h->v[i] = h->v[p];
    i = p;
  }
  h->v[i] = *x;
  return 0;
}

static node_t heap_pop(heap_t *h) {
  node_t top = h->v[0];
  node_t last = h->v[--h->n];
  size_t i = 0;
  for (;;) {
    size_t c = 2 * i + 1;
    if (c >= h->n) break;
    if (c + 1 < h->n && node_less(&h->v[c + 1], &h->v[c])) c++;
    if (!node_less(&h->v[c], &last)) break;
    h->v[i] = h->v[c];
    i = c;
  }
  if (h->n) h->v[i] = last;
  return top;
}

/* Builds dec int32[2*65536] and trie int32[65537*9].  Returns 0 on success.
 * sub1.py:29-102. */
int oracle_build_dictionary(int32_t *dec, int32_t *trie) {
  /* sub1.py:31-44: symbol probabilities, then the 9 pair probabilities in the order the nested
   * gen() produces them: pair p = 3*a + b has probability (1.0 * q[a]) * q[b]. */
  const double zeros = .885;
  double q[3] = { zeros, (1 - zeros) / 2, (1 - zeros) / 2 };
  double pp[9];
  for (int a = 0; a < 3; a++)
    for (int b = 0; b < 3; b++)
      pp[3 * a + b] = (1. * q[a]) * q[b];

  heap_t h = { 0, 0, 0 };
  node_t root;
  memset(&root, 0, sizeof(root));
  root.prio = -1.;
  root.parent = -1;
  if (heap_push(&h, &root)) return -1;

  uint32_t *udec = (uint32_t *)dec;
  memset(udec, 0, sizeof(uint32_t) * 2 * DICT_COUNT);
  for (int i = 0; i < (DICT_COUNT + 1) * 9; i++) trie[i] = -1;

  int count = 0;
  while (count < DICT_COUNT) {            /* sub1.py:50 */
    if (h.n == 0) { free(h.v); return -2; }
    node_t top = heap_pop(&h);
    int idx = TRIE_ROOT;
    if (top.prio != -1.) {                /* sub1.py:52-53: the empty sequence is not an entry */
      idx = count++;
      /* sub1.py:60-72: pack pairs 0-6 into word 0 and 7-13 into word 1; the low nibble of each
       * word is the length in pairs; pair j sits at bits 4+4j..7+4j with the first weight
       * (p % 3) in the low two bits. */
      uint32_t w0 = 0, w1 = 0;
      for (int j = 0; j < top.len && j < 7; j++) {
        uint32_t r = top.seq[j];
        w0 |= (r % 3) << (4 * j + 0);
        w0 |= (r / 3) << (4 * j + 2);
      }
      for (int j = 7; j < top.len; j++) {
        uint32_t r = top.seq[j];
        w1 |= (r % 3) << (4 * (j - 7) + 0);
        w1 |= (r / 3) << (4 * (j - 7) + 2);
      }
      udec[2 * idx + 0] = (w0 << 4) | top.len;
      udec[2 * idx + 1] = (w1 << 4) | top.len;
      /* sub1.py:74-97: trie array row = parent sequence (root row 65536), column = last pair. */
      trie[9 * top.parent + top.seq[top.len - 1]] = idx;
    }
    if (top.len == MAX_PAIRS) continue;   /* sub1.py:54-55 */
    for (int i = 0; i < 9; i++) {         /* sub1.py:56-57 */
      node_t c = top;
      c.prio = top.prio * pp[i];
      c.seq[c.len++] = (uint8_t)i;
      c.parent = idx;
      if (heap_push(&h, &c)) { free(h.v); return -1; }
    }
  }
  free(h.v);
  return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* Encoder: greedy longest match.  test.py:86-100 (greedy) == sub1_cuda_kernel.cu:211-239        */
/* ------------------------------------------------------------------------------------------ */
/* sym: `width` ternary symbols (0,1,2) of one row.  out must hold (width+1)/2 codes.
 * Returns the number of codes written. */
int oracle_encode_row(const int32_t *trie, const uint8_t *sym, int width, uint16_t *out) {
  int node = TRIE_ROOT;
  int n = 0;
  for (int i = 0; i < width; i += 2) {
    /* sub1_cuda_kernel.cu:223-228: pair = 3*s[i+1] + s[i]; an odd trailing weight stands alone */
    int num = sym[i];
    if (i + 1 < width) num += 3 * sym[i + 1];
    if (trie[9 * node + num] == -1) {     /* sub1_cuda_kernel.cu:230-233, test.py:92-94 */
      out[n++] = (uint16_t)node;
      node = TRIE_ROOT;
    }
    node = trie[9 * node + num];
  }
  if (width > 0) out[n++] = (uint16_t)node; /* sub1_cuda_kernel.cu:236, test.py:97-98 */
  return n;
}

/* Encodes a whole matrix row by row (test.py:146-151).  codes must hold height*((width+1)/2)
 * entries in the worst case; row_off gets height+1 exclusive prefix sums.  Returns total codes. */
int64_t oracle_encode_matrix(const int32_t *trie, const uint8_t *sym, int height, int width,
                             uint16_t *codes, int32_t *row_off) {
  int64_t total = 0;
  row_off[0] = 0;
  for (int r = 0; r < height; r++) {
    total += oracle_encode_row(trie, sym + (size_t)r * width, width, codes + total);
    row_off[r + 1] = (int32_t)total;
  }
  return total;
}

/* ------------------------------------------------------------------------------------------ */
/* Decoder.  test.py:103-115 (decompress) and the table-word decode of                           */
/* sub1_cuda_kernel.cu:153-154,188-189                                                           */
/* ------------------------------------------------------------------------------------------ */
/* Decodes one row's codes into ternary symbols; returns the number of weights produced, or -1 if
 * the codes do not cover exactly `width` weights (odd widths: the last pair is cut, as
 * decompress() breaks at the row end). */
int oracle_decode_row(const int32_t *dec, const uint16_t *codes, int n_codes, int width,
                      uint8_t *sym) {
  int pos = 0;
  for (int k = 0; k < n_codes; k++) {
    uint32_t w[2];
    w[0] = (uint32_t)dec[2 * codes[k] + 0];
    w[1] = (uint32_t)dec[2 * codes[k] + 1];
    int len = (int)(w[0] & 0xf);
    for (int t = 0; t < 2 * len; t++) {
      /* decoded position t lives in word t/14 at bit 4 + 2*(t%14) */
      int s = (int)((w[t / 14] >> (4 + 2 * (t % 14))) & 3u);
      if (pos >= width) {
        if ((width & 1) && t == 2 * len - 1 && k == n_codes - 1 && pos == width) break;
        return -1;
      }
      sym[pos++] = (uint8_t)s;
    }
  }
  return pos == width ? pos : -1;
}

int oracle_decode_matrix(const int32_t *dec, const uint16_t *codes, const int32_t *row_off,
                         int height, int width, uint8_t *sym) {
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(|:bad)
  for (int r = 0; r < height; r++) {
    int got = oracle_decode_row(dec, codes + row_off[r], row_off[r + 1] - row_off[r], width,
                                sym + (size_t)r * width);
    if (got != width) bad |= 1;
  }
  return bad ? -1 : 0;
}

/* ------------------------------------------------------------------------------------------ */
/* Decode-then-matmul.  Semantics of test.py:176,180 (dense bf16 matmul on the decompressed       */
/* matrix) with the kernel's output rule sub1_cuda_kernel.cu:197-200:                            */
/*   y[r] = bf16( float(y[r]) + float( bf16( sum_c W[r,c]*x[c] ) ) ),  fp32 accumulation,        */
/*   W[r,c] in {0, min_r, max_r} (sub1_cuda_kernel.cu:157,170-171,189-190).                      */
/* ------------------------------------------------------------------------------------------ */
/* minmax: bf16 bits, interleaved (min_r, max_r) (sub1.py:149).  x: [tokens, width] bf16 bits,
 * y: [tokens, height] bf16 bits, updated in place (+=). */
int oracle_matvec(const int32_t *dec, const uint16_t *codes, const int32_t *row_off,
                  const uint16_t *minmax, const uint16_t *x, uint16_t *y, int height, int width,
                  int tokens) {
  int bad = 0;
#pragma omp parallel
  {
    uint8_t *sym = (uint8_t *)malloc((size_t)width + 2);
    float *xf = (float *)malloc(sizeof(float) * (size_t)width * (tokens > 0 ? tokens : 1));
    for (int t = 0; t < tokens; t++)
      for (int c = 0; c < width; c++) xf[(size_t)t * width + c] = bf16_to_f32(x[(size_t)t * width + c]);
#pragma omp for schedule(static) reduction(|:bad)
    for (int r = 0; r < height; r++) {
      int got = oracle_decode_row(dec, codes + row_off[r], row_off[r + 1] - row_off[r], width, sym);
      if (got != width) { bad |= 1; continue; }
      float deq[3];
      deq[0] = 0.f;
      deq[1] = bf16_to_f32(minmax[2 * r + 0]);
      deq[2] = bf16_to_f32(minmax[2 * r + 1]);
      for (int t = 0; t < tokens; t++) {
        const float *xt = xf + (size_t)t * width;
        float acc = 0.f;
        for (int c = 0; c < width; c++) {
          if (sym[c]) acc += deq[sym[c]] * xt[c];
        }
        uint16_t *yy = &y[(size_t)t * height + r];
        *yy = f32_to_bf16(bf16_to_f32(*yy) + bf16_to_f32(f32_to_bf16(acc)));
      }
    }
    free(sym);
    free(xf);
  }
  return bad ? -1 : 0;
}

/* Expert FFN wo(ReLU(wi(x))) with a bf16 hidden activation (HF DenseActDense as called at
 * sub1.py:317; both linears are Sub1Linear.forward, sub1.py:132-143, which zero y first).
 * hidden: scratch [tokens, d_ff] bf16 bits; y: [tokens, d_model] bf16 bits (overwritten). */
int oracle_expert_ffn(const int32_t *dec,
                      const uint16_t *wi_codes, const int32_t *wi_row_off, const uint16_t *wi_minmax,
                      const uint16_t *wo_codes, const int32_t *wo_row_off, const uint16_t *wo_minmax,
                      const uint16_t *x, uint16_t *hidden, uint16_t *y,
                      int d_model, int d_ff, int tokens) {
  memset(hidden, 0, sizeof(uint16_t) * (size_t)tokens * d_ff);
  memset(y, 0, sizeof(uint16_t) * (size_t)tokens * d_model);
  if (oracle_matvec(dec, wi_codes, wi_row_off, wi_minmax, x, hidden, d_ff, d_model, tokens)) return -1;
  for (size_t i = 0; i < (size_t)tokens * d_ff; i++)
    if (hidden[i] & 0x8000u) hidden[i] = 0; /* ReLU on bf16 bits: negative (and -0) -> +0 */
  if (oracle_matvec(dec, wo_codes, wo_row_off, wo_minmax, hidden, y, d_model, d_ff, tokens)) return -1;
  return 0;
}

/* CPU twin of the benchmark's seeded symbol generator (splitmix64 of (seed, index / 4) gives four
 * 16-bit uniforms; u < t0 -> 0, the rest split evenly between 1 and 2).  Not part of the reference:
 * it only lets the CPU baseline build the same synthetic experts without a GPU. */
static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

void oracle_synth_ternary(uint8_t *sym, int64_t count, uint64_t seed, uint64_t first_index, float p_zero) {
  const uint32_t t0 = (uint32_t)((double)p_zero * 65536.0 + 0.5);
  const uint32_t t1 = t0 + (65536u - (t0 > 65536u ? 65536u : t0)) / 2u;
  const uint64_t base = seed * 0xD1342543DE82EF95ull;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; i++) {
    const uint64_t idx = first_index + (uint64_t)i;
    const uint64_t h = splitmix64(base + (idx >> 2));
    const uint32_t u = (uint32_t)(h >> (16 * (idx & 3))) & 0xffffu;
    sym[i] = u < t0 ? 0 : (u < t1 ? 1 : 2);
  }
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers that start one process per GPU export OMP_NUM_THREADS=1; the CPU baseline is meant to use
 * the host's cores, so the benchmark sets the count explicitly. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
