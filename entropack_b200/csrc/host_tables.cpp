// Host-side pieces of the C ABI: status strings, CUDA error capture, and the Tile-ANS table planner
// (histogram -> probability_bits, lane modes, frequencies, cdfs, decode tables).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <queue>
#include <string>
#include <utility>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/entropack_b200.h"

namespace ep {

static thread_local std::string g_last_cuda_error;

int record_cuda_error(cudaError_t error, const char* where) {
  g_last_cuda_error = std::string(where ? where : "?") + ": " + cudaGetErrorName(error) + " (" + cudaGetErrorString(error) + ")";
  return EP_ERR_CUDA;
}

namespace {

constexpr int kStatesPerTile = 32;

// Largest-remainder allocation of `table_size` slots to the symbols of a histogram: every present
// symbol gets at least one slot, leftovers go to the largest fractional parts, ties to the smaller
// symbol; an overshoot (from the clamp to one) is taken back from the smallest fractional parts among
// symbols still above one. Same results as normalize_counts, entropack/schemes/tile_ans/eager.py:16-48.
int normalize(const uint64_t* counts, int symbols, int table_size, uint16_t* frequencies) {
  uint64_t total = 0;
  for (int s = 0; s < symbols; ++s) total += counts[s];
  if (total == 0) return EP_ERR_NORMALIZE;
  std::vector<double> target(symbols);
  std::vector<int64_t> freq(symbols);
  const double ratio = static_cast<double>(table_size) / static_cast<double>(total);
  int64_t sum = 0;
  for (int s = 0; s < symbols; ++s) {
    target[s] = static_cast<double>(counts[s]) * ratio;
    freq[s] = static_cast<int64_t>(std::floor(target[s]));
    if (counts[s] != 0 && freq[s] < 1) freq[s] = 1;
    sum += freq[s];
  }
  int64_t difference = table_size - sum;
  using Item = std::pair<double, int>;
  std::priority_queue<Item, std::vector<Item>, std::greater<Item>> queue;
  if (difference > 0) {
    for (int s = 0; s < symbols; ++s) if (counts[s] != 0) queue.emplace(-(target[s] - static_cast<double>(freq[s])), s);
    for (; difference > 0; --difference) {
      Item item = queue.top();
      queue.pop();
      freq[item.second] += 1;
      queue.emplace(item.first + 1.0, item.second);
    }
  } else if (difference < 0) {
    for (int s = 0; s < symbols; ++s) {
      if (counts[s] != 0 && freq[s] > 1) queue.emplace(target[s] - static_cast<double>(freq[s]), s);
    }
    for (; difference < 0; ++difference) {
      if (queue.empty()) return EP_ERR_NORMALIZE;
      Item item = queue.top();
      queue.pop();
      freq[item.second] -= 1;
      if (freq[item.second] > 1) queue.emplace(item.first + 1.0, item.second);
    }
  }
  for (int s = 0; s < symbols; ++s) frequencies[s] = static_cast<uint16_t>(freq[s]);
  return EP_OK;
}

double coded_bits(const uint64_t* counts, const uint16_t* frequencies, int prob_bits) {
  double bits = 0.0;
  for (int s = 0; s < 256; ++s) {
    if (counts[s]) bits += static_cast<double>(counts[s]) * (prob_bits - std::log2(static_cast<double>(frequencies[s])));
  }
  return bits;
}

// A lane is stored raw when coding it would not pay: estimated bits per symbol at or above
// min(threshold, 8 - 32*32/tile_elements) (the per-tile state overhead). With `frequencies` the
// estimate is the cross entropy under the quantised table, otherwise the plain entropy.
void choose_modes(const uint64_t* histograms, int lanes, double threshold, int64_t tile_elements, const uint16_t* frequencies,
                  int prob_bits, uint8_t* modes) {
  const double effective = std::min(threshold, 8.0 - static_cast<double>(kStatesPerTile * 32) / static_cast<double>(tile_elements));
  for (int lane = 0; lane < lanes; ++lane) {
    const uint64_t* counts = histograms + lane * 256;
    uint64_t total = 0;
    for (int s = 0; s < 256; ++s) total += counts[s];
    double bits_per_symbol;
    if (frequencies == nullptr) {
      double h = 0.0;
      for (int s = 0; s < 256; ++s) {
        if (counts[s]) {
          const double p = static_cast<double>(counts[s]) / static_cast<double>(total);
          h += p * std::log2(p);
        }
      }
      bits_per_symbol = -h;
    } else {
      bits_per_symbol = coded_bits(counts, frequencies + lane * 256, prob_bits) / static_cast<double>(total);
    }
    modes[lane] = bits_per_symbol >= effective ? 1 : 0;
  }
}

}  // namespace
}  // namespace ep

namespace ep {
namespace {

constexpr int kLatticeTables = 17;

// Largest-remainder allocation for the lossy codec's tables (alphabets up to 2^15): one stable sort
// by fractional part instead of a heap; same results as normalize() above for every histogram.
// Mirrors _normalize_counts, entropack/schemes/lattice_rans/rans.py:12-53.
int normalize_sorted(const int64_t* counts, int symbols, int table_size, uint16_t* frequencies) {
  if (symbols <= 0) return EP_ERR_NORMALIZE;
  if (symbols > table_size) return EP_ERR_ALPHABET;
  int64_t total = 0;
  for (int s = 0; s < symbols; ++s) total += counts[s];
  if (total == 0) return EP_ERR_NORMALIZE;
  std::vector<double> residual(symbols);
  std::vector<int64_t> freq(symbols);
  const double ratio = static_cast<double>(table_size) / static_cast<double>(total);
  int64_t sum = 0;
  for (int s = 0; s < symbols; ++s) {
    const double target = static_cast<double>(counts[s]) * ratio;
    freq[s] = static_cast<int64_t>(std::floor(target));
    if (counts[s] != 0 && freq[s] < 1) freq[s] = 1;
    residual[s] = target - static_cast<double>(freq[s]);
    sum += freq[s];
  }
  int64_t difference = table_size - sum;
  std::vector<int> order;
  order.reserve(symbols);
  if (difference > 0) {
    for (int s = 0; s < symbols; ++s) if (counts[s] != 0) order.push_back(s);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return residual[a] > residual[b]; });
    while (difference > 0) {
      const int64_t take = std::min<int64_t>(difference, static_cast<int64_t>(order.size()));
      for (int64_t i = 0; i < take; ++i) freq[order[i]] += 1;
      difference -= take;
    }
  } else if (difference < 0) {
    for (int s = 0; s < symbols; ++s) if (counts[s] != 0 && freq[s] > 1) order.push_back(s);
    if (order.empty()) return EP_ERR_NORMALIZE;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return residual[a] < residual[b]; });
    int64_t need = -difference;
    while (need > 0) {
      int64_t live = 0;
      for (int s : order) live += freq[s] > 1;
      if (live == 0) return EP_ERR_NORMALIZE;
      int64_t quota = std::min(need, live);
      need -= quota;
      for (int s : order) {
        if (quota == 0) break;
        if (freq[s] > 1) {
          freq[s] -= 1;
          --quota;
        }
      }
    }
  }
  for (int s = 0; s < symbols; ++s) frequencies[s] = static_cast<uint16_t>(freq[s]);
  return EP_OK;
}

// Tables of one quantisation pass, from the device's min/max record and compact bins.
struct LatticeStats {
  int64_t n_symbols[kLatticeTables];
  int64_t sym_min[kLatticeTables];
  int64_t alphabet[kLatticeTables];
  std::vector<int64_t> counts[kLatticeTables];
};

int gather_stats(const int32_t* minmax, const int32_t* bins, int64_t vectors, LatticeStats* stats) {
  constexpr int32_t kUnset = 0x7FFFFFFF;
  if (minmax[33] != 0) return EP_ERR_ALPHABET;  // a field left the int16 range
  int64_t cursor = 2;
  stats->alphabet[0] = static_cast<int64_t>(minmax[32]) + 1;
  stats->sym_min[0] = 0;
  stats->n_symbols[0] = vectors;
  stats->counts[0].assign(bins, bins + stats->alphabet[0]);
  const int64_t by_coset[2] = {bins[0], bins[1]};
  if (by_coset[0] + by_coset[1] != vectors) return EP_ERR_INVALID_ARGUMENT;
  for (int st = 0; st < 16; ++st) {
    const int t = 1 + st;
    const bool live = minmax[st * 2] != kUnset;
    stats->alphabet[t] = live ? static_cast<int64_t>(minmax[st * 2 + 1]) - minmax[st * 2] + 1 : 0;
    stats->sym_min[t] = live ? minmax[st * 2] : 0;
    stats->n_symbols[t] = by_coset[st & 1];
    stats->counts[t].assign(bins + cursor, bins + cursor + stats->alphabet[t]);
    cursor += stats->alphabet[t];
  }
  return EP_OK;
}

}  // namespace
}  // namespace ep

extern "C" int64_t ep_lattice_bins_needed(const int32_t* minmax_host) {
  if (!minmax_host) return EP_ERR_INVALID_ARGUMENT;
  int64_t cursor = 2;
  for (int st = 0; st < 16; ++st) {
    if (minmax_host[st * 2] != 0x7FFFFFFF) cursor += static_cast<int64_t>(minmax_host[st * 2 + 1]) - minmax_host[st * 2] + 1;
  }
  return cursor;
}

extern "C" int ep_lattice_max_alphabet(const int32_t* minmax_host) {
  if (!minmax_host) return EP_ERR_INVALID_ARGUMENT;
  int64_t widest = static_cast<int64_t>(minmax_host[32]) + 1;
  for (int st = 0; st < 16; ++st) {
    if (minmax_host[st * 2] != 0x7FFFFFFF) widest = std::max(widest, static_cast<int64_t>(minmax_host[st * 2 + 1]) - minmax_host[st * 2] + 1);
  }
  return widest > 0x7FFFFFFF ? 0x7FFFFFFF : static_cast<int>(widest);
}

extern "C" int ep_lattice_coded_bytes(const int32_t* minmax_host, const int32_t* bins_host, int64_t vectors, int prob_bits,
                                      int64_t tile_elements, double* bytes_out) {
  using namespace ep;
  if (!minmax_host || !bins_host || !bytes_out || vectors <= 0 || prob_bits < 9 || prob_bits > 15 || tile_elements <= 0) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  LatticeStats stats;
  const int rc = gather_stats(minmax_host, bins_host, vectors, &stats);
  if (rc != EP_OK) return rc;
  const int table_size = 1 << prob_bits;
  double bits = 0.0, overflow_bits = 0.0;
  int64_t frequency_bytes = 0;
  std::vector<uint16_t> freq;
  for (int t = 0; t < kLatticeTables; ++t) {
    if (stats.n_symbols[t] && stats.alphabet[t] <= table_size) {
      freq.resize(stats.alphabet[t]);
      const int status = normalize_sorted(stats.counts[t].data(), static_cast<int>(stats.alphabet[t]), table_size, freq.data());
      if (status != EP_OK) return status;
      for (int64_t s = 0; s < stats.alphabet[t]; ++s) {
        if (stats.counts[t][s] > 0) bits += static_cast<double>(stats.counts[t][s]) * (prob_bits - std::log2(static_cast<double>(freq[s])));
      }
      frequency_bytes += stats.alphabet[t] * 2;
    } else {
      overflow_bits += static_cast<double>(stats.n_symbols[t]) * prob_bits;
    }
  }
  const int64_t tile_vectors = std::max<int64_t>(32, tile_elements / 9);
  const int64_t tiles = std::max<int64_t>(1, (vectors + tile_vectors - 1) / tile_vectors);
  const double excess = std::max(0.0, bits - static_cast<double>(tiles * 32 * 16));
  const int64_t payload_words = static_cast<int64_t>(std::ceil(excess / 16.0));
  *bytes_out = static_cast<double>(payload_words * 2 + tiles * 32 * 4 + (tiles + 1) * 4 + frequency_bytes) + overflow_bits / 8.0;
  return EP_OK;
}

extern "C" int ep_lattice_tables(const int32_t* minmax_host, const int32_t* bins_host, int64_t vectors, int prob_bits,
                                 int32_t* stream_meta_host, uint16_t* freq_tables_host, int64_t freq_capacity,
                                 int64_t* freq_entries_out) {
  using namespace ep;
  if (!minmax_host || !bins_host || !stream_meta_host || !freq_tables_host || !freq_entries_out || vectors <= 0 ||
      prob_bits < 9 || prob_bits > 15) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  LatticeStats stats;
  const int rc = gather_stats(minmax_host, bins_host, vectors, &stats);
  if (rc != EP_OK) return rc;
  const int table_size = 1 << prob_bits;
  int64_t cursor = 0;
  for (int t = 0; t < kLatticeTables; ++t) {
    const int64_t alphabet = stats.n_symbols[t] ? stats.alphabet[t] : 0;
    if (alphabet > table_size) return EP_ERR_ALPHABET;
    if (cursor + alphabet > freq_capacity) return EP_ERR_INVALID_ARGUMENT;
    if (alphabet) {
      const int status = normalize_sorted(stats.counts[t].data(), static_cast<int>(alphabet), table_size, freq_tables_host + cursor);
      if (status != EP_OK) return status;
    }
    stream_meta_host[t * 4 + 0] = static_cast<int32_t>(stats.n_symbols[t]);
    stream_meta_host[t * 4 + 1] = static_cast<int32_t>(stats.sym_min[t]);
    stream_meta_host[t * 4 + 2] = static_cast<int32_t>(cursor);
    stream_meta_host[t * 4 + 3] = static_cast<int32_t>(alphabet);
    cursor += alphabet;
  }
  *freq_entries_out = cursor;
  return EP_OK;
}

extern "C" const char* ep_status_string(int status) {
  switch (status) {
    case EP_OK: return "ok";
    case EP_ERR_INVALID_ARGUMENT: return "invalid argument";
    case EP_ERR_UNSUPPORTED: return "unsupported configuration";
    case EP_ERR_CUDA: return "CUDA runtime error";
    case EP_ERR_NORMALIZE: return "unable to normalize rANS frequencies";
    case EP_ERR_ALPHABET: return "alphabet exceeds the rANS table";
    case EP_ERR_TOO_LARGE: return "tensor too large for this entry point";
    default: return "unknown status";
  }
}

namespace ep {
namespace {
constexpr int kAllSms = 148;          // B200 (ep_common.cuh's kSmCount; this file is plain C++)
thread_local int g_decode_sms = 0;    // 0: no limit
thread_local int g_product_sms = 0;
}  // namespace
int decode_sm_limit() { return g_decode_sms > 0 && g_decode_sms < kAllSms ? g_decode_sms : kAllSms; }
int product_sm_limit() { return g_product_sms > 0 && g_product_sms < kAllSms ? g_product_sms : kAllSms; }
}  // namespace ep

extern "C" int ep_set_sm_limits(int decode_sms, int product_sms) {
  if (decode_sms < 0 || product_sms < 0) return EP_ERR_INVALID_ARGUMENT;
  ep::g_decode_sms = decode_sms;
  ep::g_product_sms = product_sms;
  return EP_OK;
}

extern "C" int ep_abi_version(void) { return 3; }

extern "C" const char* ep_last_cuda_error(void) { return ep::g_last_cuda_error.c_str(); }

extern "C" int ep_tile_ans_plan(const uint64_t* histograms_host, int num_lanes, int64_t tile_elements,
                                double raw_lane_threshold, int prob_bits_in, int* prob_bits_out, uint16_t* frequencies_host,
                                uint16_t* cdfs_host, uint32_t* decode_tables_host, uint8_t* lane_modes_host) {
  using namespace ep;
  if (!histograms_host || !prob_bits_out || !frequencies_host || !cdfs_host || !decode_tables_host || !lane_modes_host) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (num_lanes < 1 || num_lanes > 8 || tile_elements <= 0 || raw_lane_threshold < 0.0 || raw_lane_threshold > 8.0) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (prob_bits_in != 0 && (prob_bits_in < 9 || prob_bits_in > 12)) return EP_ERR_INVALID_ARGUMENT;
  uint64_t num_elements = 0;
  for (int s = 0; s < 256; ++s) num_elements += histograms_host[s];
  if (num_elements == 0) return EP_ERR_INVALID_ARGUMENT;

  int prob_bits = prob_bits_in;
  if (prob_bits_in != 0) {
    for (int lane = 0; lane < num_lanes; ++lane) {
      const int rc = normalize(histograms_host + lane * 256, 256, 1 << prob_bits, frequencies_host + lane * 256);
      if (rc != EP_OK) return rc;
    }
    choose_modes(histograms_host, num_lanes, raw_lane_threshold, tile_elements, nullptr, 0, lane_modes_host);
  } else {
    // Price every table size; take the smallest one within 0.15 % of the original size of the cheapest.
    const int64_t n = static_cast<int64_t>(num_elements);
    const int64_t tiles = (n + tile_elements - 1) / tile_elements;
    const int64_t raw_words = (n / tile_elements) * ((tile_elements + 1) / 2) + ((n % tile_elements) + 1) / 2;
    uint8_t plain[8];
    choose_modes(histograms_host, num_lanes, raw_lane_threshold, tile_elements, nullptr, 0, plain);
    const bool all_raw = std::all_of(plain, plain + num_lanes, [](uint8_t m) { return m == 1; });
    const int variants = all_raw ? 1 : 4;
    std::vector<uint16_t> freq(static_cast<size_t>(4) * num_lanes * 256);
    uint8_t modes[4][8];
    double bytes[4];
    for (int v = 0; v < variants; ++v) {
      const int pb = 9 + v;
      uint16_t* f = freq.data() + static_cast<size_t>(v) * num_lanes * 256;
      for (int lane = 0; lane < num_lanes; ++lane) {
        const int rc = normalize(histograms_host + lane * 256, 256, 1 << pb, f + lane * 256);
        if (rc != EP_OK) return rc;
      }
      choose_modes(histograms_host, num_lanes, raw_lane_threshold, tile_elements, f, pb, modes[v]);
      double estimate = static_cast<double>((tiles * num_lanes + 1) * 4 + static_cast<int64_t>(num_lanes) * (4 << pb) + num_lanes + 40);
      for (int lane = 0; lane < num_lanes; ++lane) {
        if (modes[v][lane] == 1) {
          estimate += static_cast<double>(raw_words * 2);
        } else {
          estimate += coded_bits(histograms_host + lane * 256, f + lane * 256, pb) / 8.0;
          estimate += static_cast<double>(tiles * kStatesPerTile * 4);
        }
      }
      bytes[v] = estimate;
    }
    const double best = *std::min_element(bytes, bytes + variants);
    const double tolerance = static_cast<double>(n) * num_lanes * 0.0015;
    int chosen = 0;
    while (bytes[chosen] > best + tolerance) ++chosen;
    prob_bits = 9 + chosen;
    std::memcpy(frequencies_host, freq.data() + static_cast<size_t>(chosen) * num_lanes * 256, sizeof(uint16_t) * num_lanes * 256);
    std::memcpy(lane_modes_host, modes[chosen], num_lanes);
  }
  *prob_bits_out = prob_bits;
  const uint32_t table_size = 1u << prob_bits;
  for (int lane = 0; lane < num_lanes; ++lane) {
    uint32_t running = 0;
    for (uint32_t symbol = 0; symbol < 256; ++symbol) {
      const uint32_t f = frequencies_host[lane * 256 + symbol];
      cdfs_host[lane * 256 + symbol] = static_cast<uint16_t>(running);
      if (running + f > table_size) return EP_ERR_NORMALIZE;
      const uint32_t entry = (running << 20) | ((f & 0xFFFu) << 8) | symbol;
      std::fill(decode_tables_host + static_cast<size_t>(lane) * table_size + running,
                decode_tables_host + static_cast<size_t>(lane) * table_size + running + f, entry);
      running += f;
    }
    if (running != table_size) return EP_ERR_NORMALIZE;
  }
  return EP_OK;
}

// ------------------------------------------------------------------------------------------------
// DFloat11: prefix code over the 256 bf16 exponent values plus one end-of-stream codeword, and the
// multi-level byte look-up tables the bitstream carries.
// ------------------------------------------------------------------------------------------------
namespace ep {
namespace {

constexpr int kDfSymbols = 257;  // 256 exponents + end of stream (index 256, weight 1)

// Huffman code lengths: merge the two lightest nodes until one is left; among equal weights the node
// created first (leaves in symbol order, then internal nodes in creation order) is taken first.
int huffman_lengths(const uint64_t* weight, int* length) {
  struct Node { uint64_t weight; int order; };
  auto heavier = [](const Node& a, const Node& b) { return a.weight != b.weight ? a.weight > b.weight : a.order > b.order; };
  std::priority_queue<Node, std::vector<Node>, decltype(heavier)> queue(heavier);
  std::vector<int> parent;
  int leaf[kDfSymbols];
  for (int s = 0; s < kDfSymbols; ++s) {
    leaf[s] = -1;
    length[s] = 0;
    if (weight[s]) {
      leaf[s] = static_cast<int>(parent.size());
      queue.push({weight[s], leaf[s]});
      parent.push_back(-1);
    }
  }
  if (queue.size() == 1) {
    for (int s = 0; s < kDfSymbols; ++s) if (leaf[s] >= 0) length[s] = 1;
    return 1;
  }
  while (queue.size() > 1) {
    const Node a = queue.top(); queue.pop();
    const Node b = queue.top(); queue.pop();
    const int merged = static_cast<int>(parent.size());
    parent.push_back(-1);
    parent[a.order] = parent[b.order] = merged;
    queue.push({a.weight + b.weight, merged});
  }
  int longest = 0;
  for (int s = 0; s < kDfSymbols; ++s) {
    if (leaf[s] < 0) continue;
    int depth = 0;
    for (int node = leaf[s]; parent[node] >= 0; node = parent[node]) ++depth;
    length[s] = depth;
    longest = std::max(longest, depth);
  }
  return longest;
}

}  // namespace
}  // namespace ep

extern "C" int ep_dfloat11_build_code(const uint64_t* histogram_host, int32_t* code_len_host, uint32_t* code_val_host) {
  using namespace ep;
  if (!histogram_host || !code_len_host || !code_val_host) return EP_ERR_INVALID_ARGUMENT;
  uint64_t weight[kDfSymbols];
  int present = 0;
  for (int s = 0; s < 256; ++s) present += histogram_host[s] != 0;
  if (present == 0) return EP_ERR_INVALID_ARGUMENT;
  int length[kDfSymbols];
  std::copy(histogram_host, histogram_host + 256, weight);
  weight[256] = 1;
  int longest = huffman_lengths(weight, length);
  // Codes must fit 32 bits: if they do not, count the k rarest symbols as 1 and rebuild, k = 2, 3, ...
  // (the reference's rule, entropack/schemes/dfloat11/eager.py:53-67).
  for (int k = 2; longest > 32 && k <= present; ++k) {
    std::copy(histogram_host, histogram_host + 256, weight);
    std::vector<int> order;
    for (int s = 0; s < 256; ++s) if (histogram_host[s]) order.push_back(s);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return histogram_host[a] < histogram_host[b]; });
    for (int i = 0; i < k; ++i) weight[order[i]] = 1;
    longest = huffman_lengths(weight, length);
  }
  if (longest > 32) return EP_ERR_UNSUPPORTED;
  uint64_t code = 0;
  int previous = 0;
  for (int bits = 1; bits <= 32; ++bits) {  // canonical: ascending (length, symbol)
    for (int s = 0; s < kDfSymbols; ++s) {
      if (length[s] != bits) continue;
      code <<= (bits - previous);
      previous = bits;
      code_len_host[s] = bits;
      code_val_host[s] = static_cast<uint32_t>(code++);
    }
  }
  for (int s = 0; s < kDfSymbols; ++s) if (length[s] == 0) code_len_host[s] = 0, code_val_host[s] = 0;
  return EP_OK;
}

extern "C" int ep_dfloat11_build_luts(const int32_t* code_len_host, const uint32_t* code_val_host, uint8_t* luts_host,
                                      int max_rows, int* rows_out) {
  // Level k serves one byte-aligned proper prefix of the codewords (level 0: the empty prefix; the others
  // ordered by prefix length, then value). A level's entry for a byte is the symbol whose code ends inside
  // that byte, or 256 - child level when the code continues; gaps repeat the entry before them. The last
  // row is the code length per symbol. Layout of get_luts, entropack/schemes/dfloat11/eager.py:72-116.
  if (!code_len_host || !code_val_host || !luts_host || !rows_out || max_rows < 2) return EP_ERR_INVALID_ARGUMENT;
  struct Prefix { int bits; uint32_t value; };
  std::vector<Prefix> levels{{0, 0u}};
  for (int bits = 8; bits <= 24; bits += 8) {
    std::vector<uint32_t> found;
    for (int s = 0; s < 256; ++s) {
      const int len = code_len_host[s];
      if (len && (len - 1) / 8 * 8 == bits) found.push_back(code_val_host[s] >> (len - bits));
    }
    std::sort(found.begin(), found.end());
    found.erase(std::unique(found.begin(), found.end()), found.end());
    for (uint32_t value : found) levels.push_back({bits, value});
  }
  const int count = static_cast<int>(levels.size());
  if (count + 1 > max_rows) return EP_ERR_UNSUPPORTED;
  std::memset(luts_host, 0, static_cast<size_t>(count + 1) * 256);
  for (int level = 0; level < count; ++level) {
    int slot[256];
    std::fill(slot, slot + 256, -1);
    const int skip = levels[level].bits;
    for (int s = 0; s < 256; ++s) {
      const int len = code_len_host[s];
      if (len == 0 || len <= skip) continue;
      if (skip && (code_val_host[s] >> (len - skip)) != levels[level].value) continue;
      const int rest = len - skip;
      const uint32_t tail = rest >= 32 ? code_val_host[s] : (code_val_host[s] & ((1u << rest) - 1u));
      int key, value;
      if (rest <= 8) {
        key = static_cast<int>(tail << (8 - rest));
        value = s;
      } else {
        key = static_cast<int>(tail >> (rest - 8));
        const uint32_t child_prefix = code_val_host[s] >> (rest - 8);
        int child = -1;
        for (int i = 0; i < count; ++i) if (levels[i].bits == skip + 8 && levels[i].value == child_prefix) child = i;
        if (child < 0) return EP_ERR_UNSUPPORTED;
        value = 256 - child;
      }
      if (slot[key] >= 0 && slot[key] != value) return EP_ERR_UNSUPPORTED;
      slot[key] = value;
    }
    int current = 0;
    for (int byte = 0; byte < 256; ++byte) {
      if (slot[byte] >= 0) current = slot[byte];
      luts_host[level * 256 + byte] = static_cast<uint8_t>(current);
    }
  }
  for (int s = 0; s < 256; ++s) luts_host[count * 256 + s] = static_cast<uint8_t>(code_len_host[s]);
  *rows_out = count + 1;
  return EP_OK;
}
