/*
 * Tile-ANS CPU oracle -- TEST INFRASTRUCTURE ONLY (see oracle_common.h).
 *
 * Restates entropack/schemes/tile_ans/eager.py (encode :176-230, decode :259-307, table
 * construction :16-145) and the buffer schema of entropack/schemes/tile_ans/format.py:58-64.
 */
#include "oracle_common.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------------------------------------
 * Frequency normalisation, tile_ans/eager.py:16-48. The reference drives a binary heap keyed by
 * (-residual, symbol) / (residual, symbol); popping the heap minimum is a selection of the
 * smallest key with ties to the smaller symbol, which is what the loops below do directly.
 * ------------------------------------------------------------------------------------------- */
int orc_normalize_counts(const int64_t* counts, int n, int table_size, uint16_t* freq_out) {
  int64_t total = 0;
  int present = 0;
  for (int s = 0; s < n; ++s) {
    if (counts[s] < 0) return ORC_ERR_ARG;
    total += counts[s];
    present += counts[s] != 0;
  }
  if (present == 0) return ORC_ERR_NORMALIZE;

  double* target = (double*)malloc(sizeof(double) * (size_t)n);
  double* key = (double*)malloc(sizeof(double) * (size_t)n);
  int64_t* freq = (int64_t*)malloc(sizeof(int64_t) * (size_t)n);
  char* live = (char*)malloc((size_t)n);
  if (!target || !key || !freq || !live) {
    free(target); free(key); free(freq); free(live);
    return ORC_ERR_ALLOC;
  }
  const double ratio = (double)table_size / (double)total;
  int64_t sum = 0;
  for (int s = 0; s < n; ++s) {
    target[s] = (double)counts[s] * ratio;
    freq[s] = (int64_t)floor(target[s]);
    if (counts[s] != 0 && freq[s] < 1) freq[s] = 1;
    sum += freq[s];
  }
  int64_t difference = (int64_t)table_size - sum;
  int status = ORC_OK;
  if (difference > 0) {
    for (int s = 0; s < n; ++s) {
      live[s] = counts[s] != 0;
      key[s] = -(target[s] - (double)freq[s]);
    }
    for (int64_t step = 0; step < difference; ++step) {
      int best = -1;
      for (int s = 0; s < n; ++s) {
        if (live[s] && (best < 0 || key[s] < key[best])) best = s;
      }
      freq[best] += 1;
      key[best] += 1.0;
    }
  } else if (difference < 0) {
    int queued = 0;
    for (int s = 0; s < n; ++s) {
      live[s] = counts[s] != 0 && freq[s] > 1;
      queued += live[s];
      key[s] = target[s] - (double)freq[s];
    }
    if (queued == 0) status = ORC_ERR_NORMALIZE;
    for (int64_t step = 0; status == ORC_OK && step < -difference; ++step) {
      int best = -1;
      for (int s = 0; s < n; ++s) {
        if (live[s] && (best < 0 || key[s] < key[best])) best = s;
      }
      if (best < 0) { status = ORC_ERR_NORMALIZE; break; }
      freq[best] -= 1;
      if (freq[best] > 1) {
        key[best] += 1.0;
      } else {
        live[best] = 0;
      }
    }
  }
  if (status == ORC_OK) {
    for (int s = 0; s < n; ++s) freq_out[s] = (uint16_t)freq[s];
  }
  free(target); free(key); free(freq); free(live);
  return status;
}

double orc_quantized_cross_entropy(const int64_t* counts, const uint16_t* freq, int n, int prob_bits) {
  double bits = 0.0;
  for (int s = 0; s < n; ++s) {
    if (counts[s] > 0) bits += (double)counts[s] * ((double)prob_bits - log2((double)freq[s]));
  }
  return bits;
}

/* tile_ans/eager.py:88-106 */
static void lane_modes_from_counts(const int64_t* counts, int num_lanes, double raw_lane_threshold,
                                   int64_t tile_elements, const uint16_t* freqs, int prob_bits,
                                   uint8_t* modes) {
  double effective = 8.0 - (double)(ORC_NUM_STATES * 32) / (double)tile_elements;
  if (raw_lane_threshold < effective) effective = raw_lane_threshold;
  for (int lane = 0; lane < num_lanes; ++lane) {
    const int64_t* c = counts + lane * 256;
    int64_t total = 0;
    for (int s = 0; s < 256; ++s) total += c[s];
    double bits_per_symbol;
    if (freqs == NULL) {
      double h = 0.0;
      for (int s = 0; s < 256; ++s) {
        if (c[s] > 0) {
          const double p = (double)c[s] / (double)total;
          h += p * log2(p);
        }
      }
      bits_per_symbol = -h;
    } else {
      bits_per_symbol = orc_quantized_cross_entropy(c, freqs + lane * 256, 256, prob_bits) / (double)total;
    }
    modes[lane] = bits_per_symbol >= effective ? 1 : 0;
  }
}

/* Table choice: explicit probability_bits -> tile_ans/eager.py:189-193; automatic (0) ->
 * select_coding_options, tile_ans/eager.py:109-145. Outputs freqs[num_lanes][256], modes[num_lanes]. */
int orc_tile_ans_plan(const int64_t* counts, int num_lanes, int64_t tile_elements, double raw_lane_threshold,
                      int prob_bits_in, int* prob_bits_out, uint16_t* freqs, uint8_t* modes) {
  if (num_lanes <= 0 || num_lanes > 8 || tile_elements <= 0) return ORC_ERR_ARG;
  if (prob_bits_in != 0) {
    if (prob_bits_in < 9 || prob_bits_in > 12) return ORC_ERR_ARG;
    for (int lane = 0; lane < num_lanes; ++lane) {
      const int rc = orc_normalize_counts(counts + lane * 256, 256, 1 << prob_bits_in, freqs + lane * 256);
      if (rc != ORC_OK) return rc;
    }
    lane_modes_from_counts(counts, num_lanes, raw_lane_threshold, tile_elements, NULL, 0, modes);
    *prob_bits_out = prob_bits_in;
    return ORC_OK;
  }

  int64_t num_elements = 0;
  for (int s = 0; s < 256; ++s) num_elements += counts[s];
  const int64_t tiles = (num_elements + tile_elements - 1) / tile_elements;
  const int64_t full_tiles = num_elements / tile_elements;
  const int64_t tail = num_elements % tile_elements;
  const int64_t raw_words = full_tiles * ((tile_elements + 1) / 2) + (tail + 1) / 2;
  const double original_bytes = (double)num_elements * (double)num_lanes;

  uint8_t plain[8];
  lane_modes_from_counts(counts, num_lanes, raw_lane_threshold, tile_elements, NULL, 0, plain);
  int all_raw = 1;
  for (int lane = 0; lane < num_lanes; ++lane) all_raw &= plain[lane] == 1;
  const int variants = all_raw ? 1 : 4;

  uint16_t cand_freqs[4][8 * 256];
  uint8_t cand_modes[4][8];
  double cand_bytes[4];
  for (int v = 0; v < variants; ++v) {
    const int pb = 9 + v;
    const int table_size = 1 << pb;
    for (int lane = 0; lane < num_lanes; ++lane) {
      const int rc = orc_normalize_counts(counts + lane * 256, 256, table_size, cand_freqs[v] + lane * 256);
      if (rc != ORC_OK) return rc;
    }
    lane_modes_from_counts(counts, num_lanes, raw_lane_threshold, tile_elements, cand_freqs[v], pb, cand_modes[v]);
    double estimated = (double)((tiles * num_lanes + 1) * 4 + (int64_t)num_lanes * table_size * 4 + num_lanes + 5 * 8);
    for (int lane = 0; lane < num_lanes; ++lane) {
      if (cand_modes[v][lane] == 1) {
        estimated += (double)(raw_words * 2);
      } else {
        estimated += orc_quantized_cross_entropy(counts + lane * 256, cand_freqs[v] + lane * 256, 256, pb) / 8.0;
        estimated += (double)(tiles * ORC_NUM_STATES * 4);
      }
    }
    cand_bytes[v] = estimated;
  }
  double best = cand_bytes[0];
  for (int v = 1; v < variants; ++v) if (cand_bytes[v] < best) best = cand_bytes[v];
  const double tolerance = original_bytes * 0.0015;
  int chosen = -1;
  for (int v = 0; v < variants; ++v) {
    if (cand_bytes[v] <= best + tolerance) { chosen = v; break; }
  }
  *prob_bits_out = 9 + chosen;
  memcpy(freqs, cand_freqs[chosen], sizeof(uint16_t) * 256 * (size_t)num_lanes);
  memcpy(modes, cand_modes[chosen], (size_t)num_lanes);
  return ORC_OK;
}

/* decode_tables[lane][slot] = cdf << 20 | (f & 0xFFF) << 8 | symbol, f == 4096 stored as 0;
 * tile_ans/eager.py:51-72. Also emits the exclusive cdfs the encoder needs. */
void orc_tile_ans_tables(const uint16_t* freqs, int num_lanes, int prob_bits, uint16_t* cdfs, uint32_t* decode_tables) {
  const int table_size = 1 << prob_bits;
  for (int lane = 0; lane < num_lanes; ++lane) {
    uint32_t running = 0;
    for (int symbol = 0; symbol < 256; ++symbol) {
      cdfs[lane * 256 + symbol] = (uint16_t)running;
      const uint32_t value = freqs[lane * 256 + symbol];
      if (value) {
        const uint32_t packed_frequency = value == 4096 ? 0u : value;
        const uint32_t entry = (running << 20) | (packed_frequency << 8) | (uint32_t)symbol;
        for (uint32_t slot = running; slot < running + value; ++slot) decode_tables[(size_t)lane * table_size + slot] = entry;
        running += value;
      }
    }
  }
}

/* One ANS stream: tile_ans/eager.py:156-173. `words` has room for `count` entries. */
static int64_t encode_stream(const uint8_t* input, int64_t stride, int64_t count, const uint16_t* freq,
                             const uint16_t* cdf, int prob_bits, uint32_t* states_out, uint16_t* words) {
  uint32_t states[ORC_NUM_STATES];
  for (int l = 0; l < ORC_NUM_STATES; ++l) states[l] = ORC_STATE_MIN;
  const uint32_t table_size = 1u << prob_bits;
  const int shift = 31 - prob_bits;
  int64_t n_words = 0;
  for (int64_t base = 0; base < count; base += ORC_NUM_STATES) {
    const int limit = (int)((count - base < ORC_NUM_STATES) ? (count - base) : ORC_NUM_STATES);
    for (int lane = 0; lane < limit; ++lane) {
      const uint32_t symbol = input[(base + lane) * stride];
      const uint32_t f = freq[symbol];
      uint32_t x = states[lane];
      if ((uint64_t)x >= ((uint64_t)f << shift)) {
        words[n_words++] = (uint16_t)(x & 0xFFFFu);
        x >>= 16;
      }
      states[lane] = (x / f) * table_size + (x % f) + cdf[symbol];
    }
  }
  memcpy(states_out, states, sizeof(states));
  return n_words;
}

/* Whole-tensor encode, tile_ans/eager.py:176-230. `input` is the element bytes (little endian),
 * payload_out must hold num_lanes * tiles * tile_elements words (worst case one word per symbol).
 * Returns the payload length in words, or a negative error. Tiles are encoded in parallel. */
int64_t orc_tile_ans_encode(const uint8_t* input, int64_t num_elements, int num_lanes, int64_t tile_elements,
                            int prob_bits, const uint16_t* freqs, const uint8_t* modes, uint16_t* payload_out,
                            uint32_t* offsets_out, uint32_t* states_out) {
  if (num_elements <= 0 || num_lanes <= 0 || tile_elements <= 0) return ORC_ERR_ARG;
  const int64_t tiles = (num_elements + tile_elements - 1) / tile_elements;
  const int64_t streams = tiles * num_lanes;
  uint16_t cdfs[8 * 256];
  for (int lane = 0; lane < num_lanes; ++lane) {
    uint32_t running = 0;
    for (int s = 0; s < 256; ++s) {
      cdfs[lane * 256 + s] = (uint16_t)running;
      running += freqs[lane * 256 + s];
    }
  }
  int ans_rank[8];
  int rank = 0;
  for (int lane = 0; lane < num_lanes; ++lane) {
    ans_rank[lane] = rank;
    rank += modes[lane] == 0;
  }
  uint16_t* scratch = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)streams * (size_t)tile_elements);
  int64_t* sizes = (int64_t*)malloc(sizeof(int64_t) * (size_t)streams);
  if (!scratch || !sizes) { free(scratch); free(sizes); return ORC_ERR_ALLOC; }

#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t stream = 0; stream < streams; ++stream) {
    const int lane = (int)(stream / tiles);
    const int64_t tile = stream % tiles;
    const int64_t begin = tile * tile_elements;
    const int64_t count = (num_elements - begin < tile_elements) ? (num_elements - begin) : tile_elements;
    const uint8_t* src = input + begin * num_lanes + lane;
    uint16_t* words = scratch + stream * tile_elements;
    if (modes[lane] == 1) {
      /* raw stream, tile_ans/eager.py:148-153: two bytes per word, even element in the low byte */
      const int64_t n_words = (count + 1) / 2;
      for (int64_t w = 0; w < n_words; ++w) {
        const uint32_t low = src[(2 * w) * num_lanes];
        const uint32_t high = (2 * w + 1 < count) ? src[(2 * w + 1) * num_lanes] : 0u;
        words[w] = (uint16_t)(low | (high << 8));
      }
      sizes[stream] = n_words;
    } else {
      sizes[stream] = encode_stream(src, num_lanes, count, freqs + lane * 256, cdfs + lane * 256, prob_bits,
                                    states_out + ((int64_t)ans_rank[lane] * tiles + tile) * ORC_NUM_STATES, words);
    }
  }
  int64_t total = 0;
  offsets_out[0] = 0;
  for (int64_t stream = 0; stream < streams; ++stream) {
    memcpy(payload_out + total, scratch + stream * tile_elements, sizeof(uint16_t) * (size_t)sizes[stream]);
    total += sizes[stream];
    if (total >= ((int64_t)1 << 32)) { free(scratch); free(sizes); return ORC_ERR_ARG; }
    offsets_out[stream + 1] = (uint32_t)total;
  }
  free(scratch);
  free(sizes);
  return total;
}

/* One reverse group of the decoder, tile_ans/eager.py:233-256. Returns the new word pointer or -1. */
static int64_t decode_group(uint32_t* states, const uint32_t* table, const uint16_t* words, int64_t pointer,
                            uint8_t* output, int64_t stride, int valid_lanes, int prob_bits) {
  const uint32_t table_size = 1u << prob_bits;
  int reads[ORC_NUM_STATES];
  int n_reads = 0;
  for (int lane = 0; lane < valid_lanes; ++lane) {
    uint32_t x = states[lane];
    const uint32_t slot = x & (table_size - 1);
    const uint32_t entry = table[slot];
    uint32_t f = (entry >> 8) & 0xFFFu;
    if (f == 0) f = table_size;
    const uint32_t cdf = entry >> 20;
    output[lane * stride] = (uint8_t)(entry & 0xFFu);
    x = f * (x >> prob_bits) + (slot - cdf);
    states[lane] = x;
    if (x < ORC_STATE_MIN) reads[n_reads++] = lane;
  }
  const int64_t first_word = pointer - n_reads;
  if (first_word < 0) return -1;
  for (int i = 0; i < n_reads; ++i) {
    const int lane = reads[i];
    states[lane] = (states[lane] << 16) | words[first_word + i];
  }
  return first_word;
}

/* Whole-tensor decode, tile_ans/eager.py:259-307. Writes num_elements * num_lanes bytes. */
int orc_tile_ans_decode(const uint16_t* payload, const uint32_t* offsets, const uint32_t* states,
                        const uint32_t* decode_tables, const uint8_t* modes, int64_t tile_elements,
                        int prob_bits, int num_lanes, int64_t num_elements, uint8_t* output) {
  if (num_elements <= 0 || num_lanes <= 0 || tile_elements <= 0 || prob_bits < 9 || prob_bits > 12) return ORC_ERR_ARG;
  const int64_t tiles = (num_elements + tile_elements - 1) / tile_elements;
  const int64_t streams = tiles * num_lanes;
  const int table_size = 1 << prob_bits;
  int ans_rank[8];
  int rank = 0;
  for (int lane = 0; lane < num_lanes; ++lane) {
    ans_rank[lane] = rank;
    rank += modes[lane] == 0;
  }
  int status = ORC_OK;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t stream = 0; stream < streams; ++stream) {
    const int lane = (int)(stream / tiles);
    const int64_t tile = stream % tiles;
    const int64_t tile_begin = tile * tile_elements;
    const int64_t count = (num_elements - tile_begin < tile_elements) ? (num_elements - tile_begin) : tile_elements;
    const int64_t begin = offsets[stream];
    int64_t pointer = (int64_t)offsets[stream + 1] - begin;
    const uint16_t* words = payload + begin;
    uint8_t* out = output + tile_begin * num_lanes + lane;
    int local = ORC_OK;
    if (modes[lane] == 1) {
      if (pointer != (count + 1) / 2) {
        local = ORC_ERR_RAW_LENGTH;
      } else {
        for (int64_t e = 0; e < count; ++e) out[e * num_lanes] = (uint8_t)(words[e >> 1] >> ((e & 1) * 8));
      }
    } else {
      uint32_t st[ORC_NUM_STATES];
      memcpy(st, states + ((int64_t)ans_rank[lane] * tiles + tile) * ORC_NUM_STATES, sizeof(st));
      const uint32_t* table = decode_tables + (size_t)lane * table_size;
      const int remainder = (int)(count % ORC_NUM_STATES);
      int64_t offset = count - remainder;
      if (remainder) {
        pointer = decode_group(st, table, words, pointer, out + offset * num_lanes, num_lanes, remainder, prob_bits);
      }
      while (pointer >= 0 && offset > 0) {
        offset -= ORC_NUM_STATES;
        pointer = decode_group(st, table, words, pointer, out + offset * num_lanes, num_lanes, ORC_NUM_STATES, prob_bits);
      }
      if (pointer < 0) local = ORC_ERR_TRUNCATED;
      else if (pointer != 0) local = ORC_ERR_UNREAD;
    }
    if (local != ORC_OK) {
#pragma omp critical
      status = local;
    }
  }
  return status;
}
