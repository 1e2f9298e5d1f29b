/*
 * EntroPack-Lossy (E8 lattice + coset-conditioned rANS) CPU oracle -- TEST INFRASTRUCTURE ONLY
 * (see oracle_common.h).
 *
 * Restates entropack/schemes/lattice_rans/eager.py (nearest_e8 :18-39, point_to_fields :42-51,
 * stream statistics :61-86, byte model :94-107, stream tables :269-305, reconstruction :355-396),
 * entropack/schemes/lattice_rans/rans.py (normalisation :12-53, encode :133-186, decode :189-221,
 * size model :224-258) and the buffer schema of entropack/schemes/lattice_rans/format.py:91-98.
 *
 * Two reductions cannot follow the reference bit for bit because the reference leaves their order
 * to torch: the row RMS and the least-squares row-scale refit. Both are defined here with a fixed
 * order modelled on the reference's own CUDA refit kernel (lattice_rans.cu:262-309): 256 fp32
 * partial sums (partial t takes the 8-element vectors t, t+256, ... of the row, elements in
 * order), then a halving tree. The CUDA product uses the same order, so product and oracle agree
 * bit for bit; against the reference they agree to the last few ulps of `scales`.
 */
#include "oracle_common.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define N_TABLES 17
#define REDUCE_WIDTH 256

/* ---- normalisation, lattice_rans/rans.py:12-53 (sorted multi-pass form) ------------------- */
typedef struct { double key; int index; } keyed_t;

static int keyed_cmp(const void* a, const void* b) {
  const keyed_t* x = (const keyed_t*)a;
  const keyed_t* y = (const keyed_t*)b;
  if (x->key < y->key) return -1;
  if (x->key > y->key) return 1;
  return x->index - y->index;
}

int orc_lattice_normalize(const int64_t* counts, int n, int table_size, uint16_t* freq_out) {
  if (n <= 0) return ORC_ERR_NORMALIZE;
  if (n > table_size) return ORC_ERR_ALPHABET;
  int64_t total = 0;
  int present = 0;
  for (int s = 0; s < n; ++s) { total += counts[s]; present += counts[s] != 0; }
  if (total == 0) return ORC_ERR_NORMALIZE;
  double* target = (double*)malloc(sizeof(double) * (size_t)n);
  int64_t* freq = (int64_t*)malloc(sizeof(int64_t) * (size_t)n);
  keyed_t* order = (keyed_t*)malloc(sizeof(keyed_t) * (size_t)n);
  if (!target || !freq || !order) { free(target); free(freq); free(order); return ORC_ERR_ALLOC; }
  const double ratio = (double)table_size / (double)total;
  int64_t sum = 0;
  for (int s = 0; s < n; ++s) {
    target[s] = (double)counts[s] * ratio;
    freq[s] = (int64_t)floor(target[s]);
    if (counts[s] != 0 && freq[s] < 1) freq[s] = 1;
    sum += freq[s];
  }
  int status = ORC_OK;
  int64_t difference = (int64_t)table_size - sum;
  if (difference > 0) {
    int m = 0;
    for (int s = 0; s < n; ++s) if (counts[s] != 0) { order[m].key = -(target[s] - (double)freq[s]); order[m].index = s; ++m; }
    qsort(order, (size_t)m, sizeof(keyed_t), keyed_cmp);
    int64_t need = difference;
    while (need > 0) {
      const int64_t take = need < m ? need : m;
      for (int64_t i = 0; i < take; ++i) freq[order[i].index] += 1;
      need -= take;
    }
  } else if (difference < 0) {
    int m = 0;
    for (int s = 0; s < n; ++s) if (counts[s] != 0 && freq[s] > 1) { order[m].key = target[s] - (double)freq[s]; order[m].index = s; ++m; }
    if (m == 0) status = ORC_ERR_NORMALIZE;
    qsort(order, (size_t)m, sizeof(keyed_t), keyed_cmp);
    int64_t need = -difference;
    while (status == ORC_OK && need > 0) {
      int64_t taken = 0;
      /* one pass over the symbols that were still above 1 when the pass began */
      int live = 0;
      for (int i = 0; i < m; ++i) live += freq[order[i].index] > 1;
      if (live == 0) { status = ORC_ERR_NORMALIZE; break; }
      const int64_t quota = need < live ? need : live;
      for (int i = 0; i < m && taken < quota; ++i) {
        if (freq[order[i].index] > 1) { freq[order[i].index] -= 1; ++taken; }
      }
      need -= taken;
    }
  }
  if (status == ORC_OK) for (int s = 0; s < n; ++s) freq_out[s] = (uint16_t)freq[s];
  free(target); free(freq); free(order);
  return status;
}

/* ---- nearest E8 point and field split ------------------------------------------------------ */
/* nearest point of D8 (integer vectors with even sum): lattice_rans/eager.py:18-27 */
static void nearest_dn(const float* y, int* out) {
  float f[8], r[8];
  int parity = 0;
  for (int j = 0; j < 8; ++j) {
    f[j] = rintf(y[j]);
    r[j] = y[j] - f[j];
    parity += (int)f[j];
  }
  int idx = 0;
  float best = -1.0f;
  for (int j = 0; j < 8; ++j) {
    const float a = fabsf(r[j]);
    if (a > best) { best = a; idx = j; }
  }
  for (int j = 0; j < 8; ++j) out[j] = (int)f[j];
  if (parity & 1) out[idx] += (r[idx] < 0.0f) ? -1 : 1;
}

/* fp64 squared distance, summed in the order torch's sum(dim=1) uses for 8 elements
 * (lattice_rans/eager.py:30-39; the order is spelled out at lattice_rans.cu:89-101) */
static double dist2(const float* y, const int* z, float offset) {
  double s[8];
  for (int j = 0; j < 8; ++j) {
    const double c = (double)z[j] + (double)offset;
    const double r = (double)y[j] - c;
    s[j] = r * r;
  }
  return ((s[0] + s[4]) + (s[2] + s[6])) + ((s[1] + s[5]) + (s[3] + s[7]));
}

/* Quantise rows [rows, cols] of fp32 values: y = (x / rms_row) / s, nearest E8 point, fields
 * (z0..z6, m) and coset c. lattice_rans/eager.py:30-51,88-96; lattice_rans.cu:149-241. */
int orc_e8_quantize(const float* x, const float* rms, float s, int64_t rows, int64_t cols, int32_t* fields, int32_t* cosets) {
  if (cols % 8 != 0 || rows <= 0 || cols <= 0) return ORC_ERR_ARG;
  const int64_t vecs_per_row = cols / 8;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    const float rmsv = rms[row];
    for (int64_t v = 0; v < vecs_per_row; ++v) {
      const float* w = x + row * cols + v * 8;
      float y[8], ym[8];
      for (int j = 0; j < 8; ++j) {
        const float t = w[j] / rmsv;
        y[j] = t / s;
        ym[j] = y[j] - 0.5f;
      }
      int z0[8], z1[8];
      nearest_dn(y, z0);
      nearest_dn(ym, z1);
      const double d0 = dist2(y, z0, 0.0f);
      const double d1 = dist2(y, z1, 0.5f);
      const int c = d0 <= d1 ? 0 : 1;
      const int* z = c ? z1 : z0;
      int par = 0;
      int32_t* out = fields + (row * vecs_per_row + v) * 8;
      for (int j = 0; j < 7; ++j) { out[j] = z[j]; par += z[j]; }
      par &= 1;
      out[7] = (z[7] - par) >> 1;
      cosets[row * vecs_per_row + v] = c;
    }
  }
  return ORC_OK;
}

/* fixed-order fp32 reduction shared by the RMS and the refit (see the file header) */
static float tree_reduce(float* partial) {
  for (int offset = REDUCE_WIDTH / 2; offset > 0; offset >>= 1) {
    for (int t = 0; t < offset; ++t) partial[t] = partial[t] + partial[t + offset];
  }
  return partial[0];
}

/* rms_row = max(sqrt(mean(x^2)), 1e-12), lattice_rans/eager.py:88-91 */
void orc_row_rms(const float* x, int64_t rows, int64_t cols, float* rms) {
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    float partial[REDUCE_WIDTH];
    for (int t = 0; t < REDUCE_WIDTH; ++t) {
      float acc = 0.0f;
      for (int64_t vec = t; vec < cols / 8; vec += REDUCE_WIDTH) {
        for (int j = 0; j < 8; ++j) {
          const float v = x[row * cols + vec * 8 + j];
          acc = acc + v * v;
        }
      }
      partial[t] = acc;
    }
    const float mean = tree_reduce(partial) / (float)cols;
    const float r = sqrtf(mean);
    rms[row] = r > 1.0e-12f ? r : 1.0e-12f;
  }
}

/* scale_r = sum(x p) / sum(p^2), lattice_rans/eager.py:209-224; fallback rule lattice_rans.cu:299-304 */
void orc_refit_scales(const float* x, const int32_t* fields, const int32_t* cosets, const float* rms, float s,
                      int64_t rows, int64_t cols, float* scales) {
  const int64_t vecs_per_row = cols / 8;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    float num[REDUCE_WIDTH], den[REDUCE_WIDTH];
    for (int t = 0; t < REDUCE_WIDTH; ++t) {
      float n_acc = 0.0f, d_acc = 0.0f;
      for (int64_t vec = t; vec < vecs_per_row; vec += REDUCE_WIDTH) {
        const int64_t vector = row * vecs_per_row + vec;
        const int32_t* f = fields + vector * 8;
        const float half = cosets[vector] ? 0.5f : 0.0f;
        int parity = 0;
        for (int j = 0; j < 7; ++j) parity += f[j];
        for (int j = 0; j < 8; ++j) {
          const int z = j < 7 ? f[j] : 2 * f[7] + (parity & 1);
          const float point = (float)z + half;
          const float value = x[row * cols + vec * 8 + j];
          const float xp = value * point;
          const float pp = point * point;
          n_acc = n_acc + xp;
          d_acc = d_acc + pp;
        }
      }
      num[t] = n_acc;
      den[t] = d_acc;
    }
    const float numerator = tree_reduce(num);
    const float denominator = tree_reduce(den);
    const float fallback = s * rms[row];
    float fitted = denominator > 0.0f ? numerator / denominator : fallback;
    if (!(isfinite(fitted) && fitted > 0.0f)) fitted = fallback;
    scales[row] = fitted;
  }
}

/* Per-stream min/max: minmax[2*st], minmax[2*st+1] for the 16 (field, coset) streams, minmax[32] =
 * max coset. lattice_rans/eager.py:61-74. Untouched streams keep INT32_MAX / INT32_MIN. */
void orc_lattice_minmax(const int32_t* fields, const int32_t* cosets, int64_t vectors, int32_t* minmax) {
  for (int t = 0; t < 33; ++t) minmax[t] = ((t & 1) == 0 && t != 32) ? INT32_MAX : INT32_MIN;
  for (int64_t v = 0; v < vectors; ++v) {
    const int c = cosets[v];
    if (c > minmax[32]) minmax[32] = c;
    for (int j = 0; j < 8; ++j) {
      const int st = j * 2 + c;
      const int32_t value = fields[v * 8 + j];
      if (value < minmax[st * 2]) minmax[st * 2] = value;
      if (value > minmax[st * 2 + 1]) minmax[st * 2 + 1] = value;
    }
  }
}

/* Histogram of every stream into bins laid out table after table; returns stream_meta-style rows
 * (n_symbols, sym_min, freq_offset, alphabet) in meta[17][4] (freq_offset counts non-empty
 * alphabets only) and the per-table bin offsets. lattice_rans/eager.py:61-86. */
int64_t orc_lattice_histogram(const int32_t* fields, const int32_t* cosets, int64_t vectors, const int32_t* minmax,
                              int64_t* meta, int64_t* bins, int64_t bins_capacity) {
  int64_t alphabet[N_TABLES], sym_min[N_TABLES], offset[N_TABLES];
  alphabet[0] = (int64_t)minmax[32] + 1;
  sym_min[0] = 0;
  for (int st = 0; st < 16; ++st) {
    const int live = minmax[st * 2] != INT32_MAX;
    alphabet[1 + st] = live ? (int64_t)minmax[st * 2 + 1] - minmax[st * 2] + 1 : 0;
    sym_min[1 + st] = live ? minmax[st * 2] : 0;
  }
  int64_t cursor = 0;
  for (int t = 0; t < N_TABLES; ++t) { offset[t] = cursor; cursor += alphabet[t]; }
  if (cursor > bins_capacity) return -cursor;
  memset(bins, 0, sizeof(int64_t) * (size_t)cursor);
  for (int64_t v = 0; v < vectors; ++v) {
    const int c = cosets[v];
    bins[offset[0] + c] += 1;
    for (int j = 0; j < 8; ++j) {
      const int t = 1 + j * 2 + c;
      bins[offset[t] + (fields[v * 8 + j] - sym_min[t])] += 1;
    }
  }
  int64_t n0 = bins[offset[0]];
  int64_t n1 = alphabet[0] > 1 ? bins[offset[0] + 1] : 0;
  int64_t freq_cursor = 0;
  for (int t = 0; t < N_TABLES; ++t) {
    const int64_t n_symbols = t == 0 ? vectors : (((t - 1) & 1) == 0 ? n0 : n1);
    meta[t * 4 + 0] = n_symbols;
    meta[t * 4 + 1] = sym_min[t];
    meta[t * 4 + 2] = freq_cursor;
    meta[t * 4 + 3] = n_symbols ? alphabet[t] : 0;
    freq_cursor += meta[t * 4 + 3];
  }
  return cursor;
}

/* Container-size model of the rate search. rans.coded_bytes + vector_stream_analytic_bytes
 * (lattice_rans/rans.py:224-258); the caller adds the scale-independent terms of
 * lattice_rans/eager.py:102-107. bins are laid out as orc_lattice_histogram wrote them (table t at
 * the running sum of the alphabets computed from minmax). */
double orc_lattice_coded_bytes(const int64_t* meta, const int64_t* bins, int prob_bits, int64_t tile_elements, int* status) {
  const int table_size = 1 << prob_bits;
  double bits = 0.0, overflow_bits = 0.0;
  int64_t frequency_bytes = 0;
  int64_t offset = 0;
  *status = ORC_OK;
  for (int t = 0; t < N_TABLES; ++t) {
    const int64_t n_symbols = meta[t * 4 + 0];
    const int64_t alphabet = meta[t * 4 + 3];
    if (n_symbols && alphabet <= table_size) {
      uint16_t* freq = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)alphabet);
      const int rc = orc_lattice_normalize(bins + offset, (int)alphabet, table_size, freq);
      if (rc != ORC_OK) { free(freq); *status = rc; return 0.0; }
      bits += orc_quantized_cross_entropy(bins + offset, freq, (int)alphabet, prob_bits);
      frequency_bytes += alphabet * 2;
      free(freq);
    } else {
      overflow_bits += (double)n_symbols * (double)prob_bits;
    }
    offset += alphabet;
  }
  int64_t tile_vectors = tile_elements / 9;
  if (tile_vectors < 32) tile_vectors = 32;
  const int64_t num_vectors = meta[0];
  int64_t tiles = (num_vectors + tile_vectors - 1) / tile_vectors;
  if (tiles < 1) tiles = 1;
  const double residual_bits = (double)(tiles * ORC_NUM_STATES * 16);
  double excess = bits - residual_bits;
  if (excess < 0.0) excess = 0.0;
  const int64_t payload_words = (int64_t)ceil(excess / 16.0);
  const double total = (double)(payload_words * 2 + tiles * ORC_NUM_STATES * 4 + (tiles + 1) * 4 + frequency_bytes);
  return total + overflow_bits / 8.0;
}

/* Normalised frequency tables for the final encode, concatenated over non-empty tables.
 * lattice_rans/eager.py:269-296. Returns the number of u16 entries written. */
int64_t orc_lattice_freq_tables(const int64_t* meta, const int64_t* bins, int prob_bits, uint16_t* freq_tables) {
  const int table_size = 1 << prob_bits;
  int64_t offset = 0, written = 0;
  for (int t = 0; t < N_TABLES; ++t) {
    const int64_t alphabet = meta[t * 4 + 3];
    if (alphabet) {
      const int rc = orc_lattice_normalize(bins + offset, (int)alphabet, table_size, freq_tables + written);
      if (rc != ORC_OK) return rc;
      written += alphabet;
    }
    offset += meta[t * 4 + 0] ? alphabet : 0;
  }
  return written;
}

/* ---- rANS over the 17 conditional tables -------------------------------------------------- */
static inline void encode_step(uint32_t* state, uint32_t f, uint32_t cdf, int prob_bits, uint16_t* words, int64_t* n_words) {
  uint32_t x = *state;
  if ((uint64_t)x >= ((uint64_t)f << (31 - prob_bits))) {
    words[(*n_words)++] = (uint16_t)(x & 0xFFFFu);
    x >>= 16;
  }
  *state = (x / f) * (1u << prob_bits) + (x % f) + cdf;
}

/* rans.encode_vector_stream, lattice_rans/rans.py:133-186. Field values are absolute; sym_min comes
 * from meta. payload_out needs tiles * tile_vectors * 9 words. Returns payload words or < 0. */
int64_t orc_lattice_encode(const int32_t* fields, const int32_t* cosets, int64_t vectors, const int64_t* meta,
                           const uint16_t* freq_tables, int prob_bits, int64_t tile_elements, uint16_t* payload_out,
                           uint32_t* offsets_out, uint32_t* states_out) {
  int64_t tile_vectors = tile_elements / 9;
  if (tile_vectors < 32) tile_vectors = 32;
  int64_t tiles = (vectors + tile_vectors - 1) / tile_vectors;
  if (tiles < 1) tiles = 1;
  /* exclusive cdfs per table */
  int64_t total_alpha = 0;
  for (int t = 0; t < N_TABLES; ++t) total_alpha += meta[t * 4 + 3];
  uint32_t* cdf = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(total_alpha + 1));
  uint16_t* scratch = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)tiles * (size_t)tile_vectors * 9);
  int64_t* sizes = (int64_t*)malloc(sizeof(int64_t) * (size_t)tiles);
  if (!cdf || !scratch || !sizes) { free(cdf); free(scratch); free(sizes); return ORC_ERR_ALLOC; }
  for (int t = 0; t < N_TABLES; ++t) {
    uint32_t running = 0;
    const int64_t off = meta[t * 4 + 2];
    for (int64_t s = 0; s < meta[t * 4 + 3]; ++s) { cdf[off + s] = running; running += freq_tables[off + s]; }
  }
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t tile = 0; tile < tiles; ++tile) {
    const int64_t begin = tile * tile_vectors;
    const int64_t end = (begin + tile_vectors < vectors) ? begin + tile_vectors : vectors;
    uint32_t st[ORC_NUM_STATES];
    for (int l = 0; l < ORC_NUM_STATES; ++l) st[l] = ORC_STATE_MIN;
    uint16_t* words = scratch + tile * tile_vectors * 9;
    int64_t n_words = 0;
    for (int64_t base = begin; base < end; base += ORC_NUM_STATES) {
      const int limit = (int)((end - base < ORC_NUM_STATES) ? (end - base) : ORC_NUM_STATES);
      for (int field = 7; field >= 0; --field) {
        for (int lane = 0; lane < limit; ++lane) {
          const int64_t v = base + lane;
          const int t = 1 + 2 * field + cosets[v];
          const int64_t symbol = (int64_t)fields[v * 8 + field] - meta[t * 4 + 1];
          const int64_t off = meta[t * 4 + 2];
          encode_step(&st[lane], freq_tables[off + symbol], cdf[off + symbol], prob_bits, words, &n_words);
        }
      }
      for (int lane = 0; lane < limit; ++lane) {
        const int symbol = cosets[base + lane];
        encode_step(&st[lane], freq_tables[symbol], cdf[symbol], prob_bits, words, &n_words);
      }
    }
    memcpy(states_out + tile * ORC_NUM_STATES, st, sizeof(st));
    sizes[tile] = n_words;
  }
  int64_t total = 0;
  offsets_out[0] = 0;
  for (int64_t tile = 0; tile < tiles; ++tile) {
    memcpy(payload_out + total, scratch + tile * tile_vectors * 9, sizeof(uint16_t) * (size_t)sizes[tile]);
    total += sizes[tile];
    offsets_out[tile + 1] = (uint32_t)total;
  }
  free(cdf); free(scratch); free(sizes);
  return total;
}

typedef struct {
  const uint16_t* slot_symbol; /* [17][table_size] slot -> symbol */
  const uint16_t* freq;        /* stored frequencies, concatenated over tables */
  const uint32_t* cdf;         /* exclusive cdf per symbol, same layout */
  const int32_t* meta;         /* stream_meta [17][4] */
  int prob_bits;
} lattice_tables_t;

/* One 32-vector group: coset first, then fields 0..7 conditioned on it, each followed by the
 * shared renormalisation read (lattice_rans/rans.py:98-130). Returns the new word pointer or -1. */
static int64_t decode_vector_group(const lattice_tables_t* tb, uint32_t* st, const uint16_t* words, int64_t pointer,
                                   int valid, int* coset, int (*value)[8]) {
  const uint32_t mask = (1u << tb->prob_bits) - 1u;
  const int table_size = 1 << tb->prob_bits;
  for (int step = 0; step < 9; ++step) {
    int reads[ORC_NUM_STATES];
    int n_reads = 0;
    for (int lane = 0; lane < valid; ++lane) {
      const int t = step == 0 ? 0 : 1 + 2 * (step - 1) + coset[lane];
      const int64_t off = tb->meta[t * 4 + 2];
      const uint32_t x = st[lane];
      const uint32_t slot = x & mask;
      const uint32_t symbol = tb->slot_symbol[(size_t)t * table_size + slot];
      st[lane] = (uint32_t)tb->freq[off + symbol] * (x >> tb->prob_bits) + (slot - tb->cdf[off + symbol]);
      if (step == 0) coset[lane] = (int)symbol;
      else value[lane][step - 1] = (int)symbol + tb->meta[t * 4 + 1];
      if (st[lane] < ORC_STATE_MIN) reads[n_reads++] = lane;
    }
    const int64_t first_word = pointer - n_reads;
    if (first_word < 0) return -1;
    for (int i = 0; i < n_reads; ++i) st[reads[i]] = (st[reads[i]] << 16) | words[first_word + i];
    pointer = first_word;
  }
  return pointer;
}

/* Decode + reconstruct: rans.decode_vector_stream (lattice_rans/rans.py:189-221) then
 * _restore_field_minima/_reconstruct (lattice_rans/eager.py:336-352): out = fl32(fl32(z + c/2) * scale_row).
 * Output is fp32 [rows, cols]; the container cast (format.py:153-168) is applied by the caller.
 * If fields_out/cosets_out are non-NULL the decoded symbols are returned too. */
int orc_lattice_decode(const uint16_t* payload, const uint32_t* offsets, const uint32_t* states, const int32_t* stream_meta,
                       const uint16_t* freq_tables, const float* scales, int64_t rows, int64_t cols, int prob_bits,
                       int64_t tile_elements, float* output, int32_t* fields_out, int32_t* cosets_out) {
  if (cols <= 0 || cols % 8 != 0 || rows <= 0 || prob_bits < 9 || prob_bits > 15) return ORC_ERR_ARG;
  const int table_size = 1 << prob_bits;
  const int64_t vecs_per_row = cols / 8;
  const int64_t vectors = rows * vecs_per_row;
  int64_t tile_vectors = tile_elements / 9;
  if (tile_vectors < 32) tile_vectors = 32;
  int64_t tiles = (vectors + tile_vectors - 1) / tile_vectors;
  if (tiles < 1) tiles = 1;
  int64_t total_alpha = 0;
  for (int t = 0; t < N_TABLES; ++t) total_alpha += stream_meta[t * 4 + 3];
  uint16_t* slot_symbol = (uint16_t*)calloc((size_t)N_TABLES * (size_t)table_size, sizeof(uint16_t));
  uint32_t* cdf = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(total_alpha + 1));
  if (!slot_symbol || !cdf) { free(slot_symbol); free(cdf); return ORC_ERR_ALLOC; }
  for (int t = 0; t < N_TABLES; ++t) {
    const int64_t off = stream_meta[t * 4 + 2];
    const int64_t alphabet = stream_meta[t * 4 + 3];
    uint32_t running = 0;
    for (int64_t s = 0; s < alphabet; ++s) {
      cdf[off + s] = running;
      const uint32_t f = freq_tables[off + s];
      if (running + f > (uint32_t)table_size) { free(slot_symbol); free(cdf); return ORC_ERR_ARG; }
      for (uint32_t k = 0; k < f; ++k) slot_symbol[(size_t)t * table_size + running + k] = (uint16_t)s;
      running += f;
    }
  }
  const lattice_tables_t tb = {slot_symbol, freq_tables, cdf, stream_meta, prob_bits};
  int status = ORC_OK;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t tile = 0; tile < tiles; ++tile) {
    const int64_t begin = tile * tile_vectors;
    const int64_t count = (vectors - begin < tile_vectors) ? vectors - begin : tile_vectors;
    const uint16_t* words = payload + offsets[tile];
    int64_t pointer = (int64_t)offsets[tile + 1] - (int64_t)offsets[tile];
    uint32_t st[ORC_NUM_STATES];
    memcpy(st, states + tile * ORC_NUM_STATES, sizeof(st));
    /* groups run back to front; the partial group at the end of the tile comes first */
    int64_t group_begin = count - (count % ORC_NUM_STATES);
    int valid = (int)(count % ORC_NUM_STATES);
    if (valid == 0) { group_begin -= ORC_NUM_STATES; valid = ORC_NUM_STATES; }
    while (group_begin >= 0 && pointer >= 0) {
      int coset[ORC_NUM_STATES];
      int value[ORC_NUM_STATES][8];
      pointer = decode_vector_group(&tb, st, words, pointer, valid, coset, value);
      if (pointer < 0) break;
      for (int lane = 0; lane < valid; ++lane) {
        const int64_t vector = begin + group_begin + lane;
        int parity = 0;
        for (int j = 0; j < 7; ++j) parity += value[lane][j];
        if (fields_out) {
          for (int j = 0; j < 8; ++j) fields_out[vector * 8 + j] = value[lane][j];
          cosets_out[vector] = coset[lane];
        }
        value[lane][7] = 2 * value[lane][7] + (parity & 1);
        const float half = coset[lane] ? 0.5f : 0.0f;
        const float scale = scales[vector / vecs_per_row];
        float* out = output + vector * 8;
        for (int j = 0; j < 8; ++j) {
          const float p = (float)value[lane][j] + half;
          out[j] = p * scale;
        }
      }
      group_begin -= ORC_NUM_STATES;
      valid = ORC_NUM_STATES;
    }
    const int local = pointer < 0 ? ORC_ERR_TRUNCATED : (pointer != 0 ? ORC_ERR_UNREAD : ORC_OK);
    if (local != ORC_OK) {
#pragma omp critical
      status = local;
    }
  }
  free(slot_symbol); free(cdf);
  return status;
}

/* fp32 -> bf16 round-to-nearest-even after the clamp of format.py:167-168 (finite inputs only) */
void orc_f32_to_bf16(const float* in, int64_t n, uint16_t* out) {
  const float limit = 3.3895313892515355e38f;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float v = in[i];
    if (v > limit) v = limit;
    if (v < -limit) v = -limit;
    uint32_t bits;
    memcpy(&bits, &v, 4);
    bits += 0x7FFFu + ((bits >> 16) & 1u);
    out[i] = (uint16_t)(bits >> 16);
  }
}
