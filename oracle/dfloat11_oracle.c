/*
 * DFloat11 (Huffman-coded bf16 exponents) CPU oracle -- TEST INFRASTRUCTURE ONLY (see
 * oracle_common.h).
 *
 * Restates entropack/schemes/dfloat11/eager.py (LUT construction :72-116, bitstream and region
 * metadata :119-198, decode :200-243) and the schema of entropack/schemes/dfloat11/format.py:32-63.
 *
 * Codeword assignment: the reference obtains its prefix code from the third-party package
 * `dahuffman` (>= 0.4, pyproject.toml:18), which is neither vendored nor installed. This file builds
 * its own optimal prefix code (Huffman lengths, canonical assignment, one reserved end-of-stream
 * codeword of weight 1 as the reference's codec has). Codeword values are therefore "parity
 * unpinned"; everything downstream of the code table (LUT bytes, bitstream, thread_meta,
 * output_positions) is pinned by running the reference's own functions on the same table.
 */
#include "oracle_common.h"

#include <stdlib.h>
#include <string.h>

#define DF_SYMBOLS 257 /* 256 exponent values + end-of-stream */
#define DF_EOF 256
#define DF_MAX_LEVELS 64

/* Huffman code lengths by repeated merging of the two lightest nodes; ties go to the node created
 * first (leaves in symbol order, then internal nodes in creation order). */
static int huffman_lengths(const int64_t* weight, int* length) {
  int64_t w[2 * DF_SYMBOLS];
  int parent[2 * DF_SYMBOLS];
  char alive[2 * DF_SYMBOLS];
  int nodes = 0, live = 0;
  int leaf_of[DF_SYMBOLS];
  for (int s = 0; s < DF_SYMBOLS; ++s) {
    leaf_of[s] = -1;
    length[s] = 0;
    if (weight[s] > 0) {
      w[nodes] = weight[s];
      parent[nodes] = -1;
      alive[nodes] = 1;
      leaf_of[s] = nodes++;
      ++live;
    }
  }
  if (live == 1) {
    for (int s = 0; s < DF_SYMBOLS; ++s) if (leaf_of[s] >= 0) length[s] = 1;
    return 1;
  }
  while (live > 1) {
    int a = -1, b = -1;
    for (int i = 0; i < nodes; ++i) {
      if (!alive[i]) continue;
      if (a < 0 || w[i] < w[a]) { b = a; a = i; }
      else if (b < 0 || w[i] < w[b]) { b = i; }
    }
    w[nodes] = w[a] + w[b];
    parent[nodes] = -1;
    alive[nodes] = 1;
    alive[a] = alive[b] = 0;
    parent[a] = parent[b] = nodes;
    ++nodes;
    --live;
  }
  int longest = 0;
  for (int s = 0; s < DF_SYMBOLS; ++s) {
    if (leaf_of[s] < 0) continue;
    int depth = 0;
    for (int i = leaf_of[s]; parent[i] >= 0; i = parent[i]) ++depth;
    length[s] = depth;
    if (depth > longest) longest = depth;
  }
  return longest;
}

/* Code table for a 256-bin exponent histogram: lengths (0 = absent) and right-aligned code values
 * for the 256 symbols plus end-of-stream at index 256. Codes longer than 32 bits are avoided the way
 * dfloat11/eager.py:53-67 does: the k rarest symbols are re-counted as 1, k = 2, 3, ... */
int orc_dfloat11_build_code(const int64_t* counts, int32_t* code_len, uint32_t* code_val) {
  int64_t weight[DF_SYMBOLS];
  int present = 0;
  for (int s = 0; s < 256; ++s) { weight[s] = counts[s]; present += counts[s] > 0; }
  weight[DF_EOF] = 1;
  if (present == 0) return ORC_ERR_ARG;
  int length[DF_SYMBOLS];
  int longest = huffman_lengths(weight, length);
  for (int k = 2; longest > 32 && k <= present; ++k) {
    for (int s = 0; s < 256; ++s) weight[s] = counts[s];
    char flattened[256] = {0};
    for (int pick = 0; pick < k; ++pick) {
      int best = -1;
      for (int s = 0; s < 256; ++s) {
        if (counts[s] > 0 && !flattened[s] && (best < 0 || counts[s] < counts[best])) best = s;
      }
      flattened[best] = 1;
      weight[best] = 1;
    }
    longest = huffman_lengths(weight, length);
  }
  if (longest > 32) return ORC_ERR_ARG;
  /* canonical assignment: ascending (length, symbol) */
  uint64_t code = 0;
  int previous = 0;
  for (int len = 1; len <= 32; ++len) {
    for (int s = 0; s < DF_SYMBOLS; ++s) {
      if (length[s] != len) continue;
      code <<= (len - previous);
      previous = len;
      code_len[s] = len;
      code_val[s] = (uint32_t)code;
      code += 1;
    }
  }
  for (int s = 0; s < DF_SYMBOLS; ++s) if (length[s] == 0) { code_len[s] = 0; code_val[s] = 0; }
  return ORC_OK;
}

/* Multi-level byte LUTs, dfloat11/eager.py:72-116. Level k serves one byte-aligned proper prefix of
 * the codewords (levels ordered by prefix length, then prefix value); an entry is either a symbol or
 * 256 - child_level; the extra last row is the code length per symbol. Returns the number of rows
 * written (levels + 1) or a negative error. luts_out must hold (DF_MAX_LEVELS + 1) * 256 bytes. */
int orc_dfloat11_build_luts(const int32_t* code_len, const uint32_t* code_val, uint8_t* luts_out) {
  uint32_t prefix_val[DF_MAX_LEVELS];
  int prefix_len[DF_MAX_LEVELS];
  int levels = 1;
  prefix_val[0] = 0;
  prefix_len[0] = 0;
  for (int plen = 8; plen <= 24; plen += 8) {
    /* distinct prefixes of this length, ascending */
    uint32_t found[DF_SYMBOLS];
    int n_found = 0;
    for (int s = 0; s < 256; ++s) {
      const int bits = code_len[s];
      if (bits == 0 || (bits - 1) / 8 * 8 != plen) continue;
      const uint32_t p = code_val[s] >> (bits - plen);
      int seen = 0;
      for (int i = 0; i < n_found; ++i) seen |= found[i] == p;
      if (!seen) found[n_found++] = p;
    }
    for (int i = 0; i < n_found; ++i) {
      for (int j = i + 1; j < n_found; ++j) if (found[j] < found[i]) { const uint32_t t = found[i]; found[i] = found[j]; found[j] = t; }
    }
    for (int i = 0; i < n_found; ++i) {
      if (levels >= DF_MAX_LEVELS) return ORC_ERR_ARG;
      prefix_val[levels] = found[i];
      prefix_len[levels] = plen;
      ++levels;
    }
  }
  memset(luts_out, 0, (size_t)(levels + 1) * 256);
  for (int level = 0; level < levels; ++level) {
    int assigned[256];
    for (int i = 0; i < 256; ++i) assigned[i] = -1;
    const int plen = prefix_len[level];
    for (int s = 0; s < 256; ++s) {
      const int bits = code_len[s];
      if (bits == 0 || bits <= plen) continue;
      if (plen && (code_val[s] >> (bits - plen)) != prefix_val[level]) continue;
      const uint32_t rest_bits = (uint32_t)(bits - plen);
      const uint32_t rest = code_val[s] & (rest_bits >= 32 ? 0xFFFFFFFFu : ((1u << rest_bits) - 1u));
      int key, value;
      if ((bits - 1) / 8 * 8 == plen) {
        key = (int)(rest << (8 - rest_bits));      /* remaining bits left-justified in the byte */
        value = s;
      } else {
        key = (int)(rest >> (rest_bits - 8));       /* next whole byte selects a child level */
        const uint32_t child_prefix = code_val[s] >> (bits - plen - 8);
        int child = -1;
        for (int i = 0; i < levels; ++i) if (prefix_len[i] == plen + 8 && prefix_val[i] == child_prefix) child = i;
        if (child < 0) return ORC_ERR_ARG;
        value = 256 - child;
      }
      if (assigned[key] >= 0 && assigned[key] != value) return ORC_ERR_ARG;
      assigned[key] = value;
    }
    int current = 0;
    for (int i = 0; i < 256; ++i) {
      if (assigned[i] >= 0) current = assigned[i];
      luts_out[level * 256 + i] = (uint8_t)current;
    }
  }
  for (int s = 0; s < 256; ++s) luts_out[levels * 256 + s] = (uint8_t)code_len[s];
  return levels + 1;
}

/* Total payload bits of a bf16 tensor under a code table. */
int64_t orc_dfloat11_total_bits(const uint16_t* bf16_bits, int64_t n, const int32_t* code_len) {
  int64_t total = 0;
  for (int64_t i = 0; i < n; ++i) total += code_len[(bf16_bits[i] >> 7) & 0xFF];
  return total;
}

/* Bitstream + metadata, dfloat11/eager.py:119-198 and encode_weights :173-188.
 * encoded_out: ceil(total_bits / 8) bytes; thread_meta_out: blocks * threads_per_block entries;
 * output_positions_out: blocks + 1 entries, with blocks = ceil(n_bytes / (bpt * tpb)).
 * Returns max(diff(output_positions)) (the third layout field) or a negative error. */
int64_t orc_dfloat11_encode(const uint16_t* bf16_bits, int64_t n, const int32_t* code_len, const uint32_t* code_val,
                            int bytes_per_thread, int threads_per_block, uint8_t* encoded_out, uint8_t* sign_mantissa_out,
                            uint16_t* thread_meta_out, uint32_t* output_positions_out) {
  if (n <= 0 || bytes_per_thread <= 0 || threads_per_block <= 0) return ORC_ERR_ARG;
  const int64_t region_bits = 8 * (int64_t)bytes_per_thread;
  const int64_t block_bits = region_bits * threads_per_block;
  const int64_t total_bits = orc_dfloat11_total_bits(bf16_bits, n, code_len);
  const int64_t n_bytes = (total_bits + 7) / 8;
  const int64_t blocks = (n_bytes + (int64_t)bytes_per_thread * threads_per_block - 1) / ((int64_t)bytes_per_thread * threads_per_block);
  const int64_t n_regions = blocks * threads_per_block;
  memset(encoded_out, 0, (size_t)n_bytes);
  memset(thread_meta_out, 0, sizeof(uint16_t) * (size_t)n_regions);

  int64_t regions_seen = 0, blocks_seen = 0;
  int64_t bit = 0;
  int64_t current_count = 0, current_gap = 0;
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t bits16 = bf16_bits[i];
    const uint32_t exponent = (bits16 >> 7) & 0xFFu;
    sign_mantissa_out[i] = (uint8_t)(((bits16 >> 8) & 0x80u) | (bits16 & 0x7Fu));
    if (bit / region_bits + 1 > regions_seen) {
      if (regions_seen > 0) {
        if (current_gap > 31 || current_count > 2047) return ORC_ERR_ARG;
        thread_meta_out[regions_seen - 1] = (uint16_t)((current_gap << 11) | current_count);
      }
      current_gap = bit - bit / region_bits * region_bits;
      current_count = 0;
      ++regions_seen;
    }
    if (bit / block_bits + 1 > blocks_seen) output_positions_out[blocks_seen++] = (uint32_t)i;
    ++current_count;
    const int len = code_len[exponent];
    if (len <= 0) return ORC_ERR_ARG;
    const uint32_t val = code_val[exponent];
    for (int k = len - 1; k >= 0; --k, ++bit) {
      if ((val >> k) & 1u) encoded_out[bit >> 3] |= (uint8_t)(0x80u >> (bit & 7));
    }
  }
  if (regions_seen > 0) {
    if (current_gap > 31 || current_count > 2047) return ORC_ERR_ARG;
    thread_meta_out[regions_seen - 1] = (uint16_t)((current_gap << 11) | current_count);
  }
  if (total_bits & 7) {
    /* the final partial byte is completed with the leading bits of the end-of-stream codeword */
    if (total_bits / region_bits + 1 > regions_seen) ++regions_seen; /* (gap 0, count 0): already zero */
    if (total_bits / block_bits + 1 > blocks_seen) output_positions_out[blocks_seen++] = (uint32_t)n;
    const int len = code_len[DF_EOF];
    const uint32_t val = code_val[DF_EOF];
    int64_t b = total_bits;
    for (int k = len - 1; k >= 0 && (b >> 3) < n_bytes; --k, ++b) {
      if ((val >> k) & 1u) encoded_out[b >> 3] |= (uint8_t)(0x80u >> (b & 7));
    }
  }
  if (blocks_seen != blocks) return ORC_ERR_ARG;
  output_positions_out[blocks] = (uint32_t)n;
  int64_t widest = 0;
  for (int64_t blk = 0; blk < blocks; ++blk) {
    const int64_t d = (int64_t)output_positions_out[blk + 1] - (int64_t)output_positions_out[blk];
    if (d > widest) widest = d;
  }
  return widest;
}

static inline uint32_t peek_byte(const uint8_t* data, int64_t n_bytes, int64_t bit) {
  const int64_t byte = bit >> 3;
  const uint32_t shift = (uint32_t)(bit & 7);
  const uint32_t hi = byte < n_bytes ? data[byte] : 0u;
  const uint32_t lo = byte + 1 < n_bytes ? data[byte + 1] : 0u;
  return ((hi << shift) | (lo >> (8 - shift))) & 0xFFu;
}

static inline uint32_t walk_luts(const uint8_t* luts, int num_levels, const uint8_t* encoded, int64_t n_bytes, int64_t* cursor) {
  const uint32_t ptr_min = num_levels > 1 ? (uint32_t)(256 - (num_levels - 1)) : 256u;
  int level = 0, hop = 0;
  for (;;) {
    const uint32_t entry = luts[level * 256 + peek_byte(encoded, n_bytes, *cursor + hop * 8)];
    if (num_levels > 1 && entry >= ptr_min) {
      level = 256 - (int)entry;
      ++hop;
    } else {
      *cursor += luts[num_levels * 256 + entry];
      return entry;
    }
  }
}

/* Sequential decode exactly as the eager lane does it (dfloat11/eager.py:200-243): one cursor over
 * the whole bitstream, region metadata ignored. */
void orc_dfloat11_decode_sequential(const uint8_t* luts, int num_luts, const uint8_t* encoded, int64_t n_bytes,
                                    const uint8_t* sign_mantissa, int64_t n, uint16_t* out_bits) {
  int64_t cursor = 0;
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t exponent = walk_luts(luts, num_luts - 1, encoded, n_bytes, &cursor);
    const uint32_t sm = sign_mantissa[i];
    out_bits[i] = (uint16_t)(((sm & 0x80u) << 8) | (exponent << 7) | (sm & 0x7Fu));
  }
}

/* Region-parallel decode through thread_meta / output_positions, the access pattern of the
 * reference's CUDA lane (dfloat11.cu:314-522); checks that the metadata describe the stream. */
int orc_dfloat11_decode_regions(const uint8_t* luts, int num_luts, const uint8_t* encoded, int64_t n_bytes,
                                const uint8_t* sign_mantissa, int64_t n, const uint32_t* output_positions,
                                const uint16_t* thread_meta, int bytes_per_thread, int threads_per_block, uint16_t* out_bits) {
  const int64_t bytes_per_block = (int64_t)bytes_per_thread * threads_per_block;
  const int64_t blocks = (n_bytes + bytes_per_block - 1) / bytes_per_block;
  int status = ORC_OK;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t blk = 0; blk < blocks; ++blk) {
    int64_t index = output_positions[blk];
    for (int t = 0; t < threads_per_block; ++t) {
      const int64_t region = blk * threads_per_block + t;
      const uint32_t meta = thread_meta[region];
      int64_t cursor = region * bytes_per_thread * 8 + (meta >> 11);
      const int count = (int)(meta & 2047u);
      for (int k = 0; k < count; ++k, ++index) {
        if (index >= n) { status = ORC_ERR_TRUNCATED; break; }
        const uint32_t exponent = walk_luts(luts, num_luts - 1, encoded, n_bytes, &cursor);
        const uint32_t sm = sign_mantissa[index];
        out_bits[index] = (uint16_t)(((sm & 0x80u) << 8) | (exponent << 7) | (sm & 0x7Fu));
      }
    }
    if (index != (int64_t)output_positions[blk + 1]) status = ORC_ERR_UNREAD;
  }
  return status;
}
