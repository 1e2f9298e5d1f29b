// EntroPack-Lossy decode for sm_100a: coset-conditioned rANS over 17 tables, E8 reconstruction and the
// container cast, fused into one kernel.
//
// Format (entropack/schemes/lattice_rans/format.py:91-98, rans.py:133-221): vectors of 8 values in
// row-major order are cut into tiles of `tile_vectors`; a tile is a 32-way interleaved rANS stream
// read back to front. Per group of 32 vectors the decoder reads the coset (table 0) and then fields
// 0..7 (table 1 + 2*field + coset). Field 7 is m with z7 = 2m + (sum(z0..z6) & 1). A value is
// fl32(fl32(z + coset/2) * scale[row]) cast to the container dtype.
//
// One warp decodes one tile at a time; a persistent block walks the tile list. The slot tables are
// rebuilt from the stored frequencies inside the kernel -- no host-side plan, no cached side tables:
//   * shared path (prob_bits <= 11, every alphabet <= 512): each block builds all 17 tables as packed
//     32-bit entries (symbol | (slot - cdf) << 9 | freq << 20) in its own shared memory;
//   * global path (anything else): a small kernel first writes 64-bit entries
//     (symbol | freq << 16 | (slot - cdf) << 32) into caller-provided scratch, read through L1.
// Payload words reach the chain through the per-warp cp.async ring of rans_ring.cuh.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <mutex>
#include <type_traits>

#include "ep_common.cuh"
#include "rans_ring.cuh"

namespace ep {
namespace {

constexpr int kTables = 17;
constexpr int kDecodeWarps = 24;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kSharedMaxProbBits = 11;
constexpr int kSharedMaxAlphabet = 512;     // 32-bit entries hold 9 bits of symbol
constexpr int kWideMaxAlphabet = 2048;      // wide shared tables: a byte per slot carries the symbol's high bits
// Where the 17 slot tables live.
constexpr int kTablesGlobal = 0;       // 64-bit entries in caller scratch (prob_bits above 11)
constexpr int kTablesShared = 1;       // packed 32-bit entries in shared memory: symbol | delta << 9 | freq << 20
constexpr int kTablesSharedWide = 2;   // shared memory, alphabets up to 2048: symbol low 10 bits | (freq - 1) << 10 | delta << 21,
                                       // plus the symbol's bits above 10 in a byte table behind the 17 word tables

struct LatticeDecodeParams {
  const uint16_t* payload;
  int64_t payload_words;
  const uint32_t* offsets;
  const uint32_t* states;
  const int32_t* stream_meta;   // [17][4]: n_symbols, sym_min, freq_offset, alphabet
  const uint16_t* freq_tables;
  int64_t freq_entries;         // length of freq_tables: no table record can make a read go past it
  const float* scales;
  void* output;
  const uint64_t* global_tables;  // [17][1 << prob_bits], global path only
  const uint32_t* slot_tables;    // shared paths: the tables as an earlier launch exported them (null: build them here)
  uint32_t* export_tables;        // kModeExport: where the freshly built tables go
  int64_t vectors;
  int64_t tiles;
  int tile_vectors;
  int vecs_per_row;
  int prob_bits;
  int store_kind;
  int* error;
  // fused product (kModeProduct): activations bf16 [tokens][8 * vecs_per_row], accumulators fp32 [tokens][rows]
  const __nv_bfloat16* activations;
  float* products;           // [tokens][rows] accumulators, then one word counting the blocks that are done
  const __nv_bfloat16* bias;  // [rows] or null
  __nv_bfloat16* product_out; // [tokens][rows]
  int tokens;
  int rows;
};

// What the decode kernel does with a reconstructed vector.
constexpr int kModeStore = 0;       // any container dtype (store_kind)
constexpr int kModeStoreBf16 = 1;   // bf16, one 16-byte store
constexpr int kModeProduct = 2;     // nothing is stored: the vector is multiplied into up to kMaxTokens dot products
constexpr int kModeStoreCodes = 4;  // e4m3 or int8 codes (the 8-bit layers' weights), one 8-byte store
constexpr int kModeExport = 3;      // no decoding: the block builds the slot tables and writes them to global memory
constexpr int kMaxTokens = 4;    // instantiated for 1, 2 and 4 tokens: every token costs its instructions whether used or not

// ---- container cast (entropack/schemes/lattice_rans/format.py:153-168) ---------------------------
template <typename T>
__device__ __forceinline__ T snap_integer(float value, float low, float high_exclusive) {
  const float high = nextafterf(high_exclusive, 0.0f);
  return static_cast<T>(fminf(fmaxf(rintf(value), low), high));
}

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  const float limit = 3.3895313892515355e38f;  // largest finite bf16
  const __nv_bfloat16 h = __float2bfloat16_rn(fminf(fmaxf(v, -limit), limit));
  return static_cast<uint32_t>(__bfloat16_as_ushort(h));
}

// Two values as a pair of bf16, the first in the low half: round to nearest even, anything beyond the largest finite
// bf16 (infinities included) becomes that value with its sign.
__device__ __forceinline__ uint32_t bf16x2_saturating(float low, float high) {
  uint32_t pair;
  asm("cvt.rn.satfinite.bf16x2.f32 %0, %1, %2;" : "=r"(pair) : "f"(high), "f"(low));
  return pair;
}

// Writes the eight reconstructed values of vector `vector` as `kind` elements.
__device__ __forceinline__ void store_vector(void* output, int64_t vector, const float* v, int kind) {
  char* const base = static_cast<char*>(output);
  switch (kind) {
    case EP_STORE_BF16: {
      uint4 packed;
      packed.x = bf16_bits(v[0]) | (bf16_bits(v[1]) << 16);
      packed.y = bf16_bits(v[2]) | (bf16_bits(v[3]) << 16);
      packed.z = bf16_bits(v[4]) | (bf16_bits(v[5]) << 16);
      packed.w = bf16_bits(v[6]) | (bf16_bits(v[7]) << 16);
      *reinterpret_cast<uint4*>(base + vector * 16) = packed;
      break;
    }
    case EP_STORE_F16: {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t lo = __half_as_ushort(__float2half_rn(fminf(fmaxf(v[2 * j], -65504.0f), 65504.0f)));
        const uint32_t hi = __half_as_ushort(__float2half_rn(fminf(fmaxf(v[2 * j + 1], -65504.0f), 65504.0f)));
        w[j] = lo | (hi << 16);
      }
      *reinterpret_cast<uint4*>(base + vector * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      break;
    }
    case EP_STORE_F32: {
      float4* out = reinterpret_cast<float4*>(base + vector * 32);
      out[0] = make_float4(v[0], v[1], v[2], v[3]);
      out[1] = make_float4(v[4], v[5], v[6], v[7]);
      break;
    }
    case EP_STORE_F8_E4M3:
    case EP_STORE_F8_E5M2: {
      const float limit = kind == EP_STORE_F8_E4M3 ? 448.0f : 57344.0f;
      const __nv_fp8_interpretation_t interpretation = kind == EP_STORE_F8_E4M3 ? __NV_E4M3 : __NV_E5M2;
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t bits = __nv_cvt_float_to_fp8(fminf(fmaxf(v[j], -limit), limit), __NV_SATFINITE, interpretation);
        w[j >> 2] |= bits << (8 * (j & 3));
      }
      *reinterpret_cast<uint2*>(base + vector * 8) = make_uint2(w[0], w[1]);
      break;
    }
    case EP_STORE_I8:
    case EP_STORE_U8:
    case EP_STORE_BOOL: {
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t bits;
        if (kind == EP_STORE_I8) bits = static_cast<uint8_t>(snap_integer<int8_t>(v[j], -128.0f, 128.0f));
        else if (kind == EP_STORE_U8) bits = snap_integer<uint8_t>(v[j], 0.0f, 256.0f);
        else bits = rintf(v[j]) != 0.0f ? 1u : 0u;
        w[j >> 2] |= bits << (8 * (j & 3));
      }
      *reinterpret_cast<uint2*>(base + vector * 8) = make_uint2(w[0], w[1]);
      break;
    }
    case EP_STORE_I16:
    case EP_STORE_U16: {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t bits = kind == EP_STORE_I16 ? static_cast<uint16_t>(snap_integer<int16_t>(v[j], -32768.0f, 32768.0f))
                                                   : snap_integer<uint16_t>(v[j], 0.0f, 65536.0f);
        w[j >> 1] |= bits << (16 * (j & 1));
      }
      *reinterpret_cast<uint4*>(base + vector * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      break;
    }
    case EP_STORE_I32:
    case EP_STORE_U32: {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        w[j] = kind == EP_STORE_I32 ? static_cast<uint32_t>(snap_integer<int32_t>(v[j], -2147483648.0f, 2147483648.0f))
                                    : snap_integer<uint32_t>(v[j], 0.0f, 4294967296.0f);
      }
      uint4* out = reinterpret_cast<uint4*>(base + vector * 32);
      out[0] = make_uint4(w[0], w[1], w[2], w[3]);
      out[1] = make_uint4(w[4], w[5], w[6], w[7]);
      break;
    }
    default: {  // EP_STORE_I64 / EP_STORE_U64
      unsigned long long* out = reinterpret_cast<unsigned long long*>(base + vector * 64);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        out[j] = kind == EP_STORE_I64
            ? static_cast<unsigned long long>(snap_integer<long long>(v[j], -9223372036854775808.0f, 9223372036854775808.0f))
            : snap_integer<unsigned long long>(v[j], 0.0f, 18446744073709551616.0f);
      }
      break;
    }
  }
}

// ---- slot tables -----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_entry32(uint32_t symbol, uint32_t freq, uint32_t delta) {
  return symbol | (delta << 9) | (freq << 20);
}
__device__ __forceinline__ uint64_t pack_entry64(uint32_t symbol, uint32_t freq, uint32_t delta) {
  return static_cast<uint64_t>(symbol) | (static_cast<uint64_t>(freq) << 16) | (static_cast<uint64_t>(delta) << 32);
}

// One warp fills table `t`: symbols in order, the 32 threads sharing each symbol's run of slots. Slots
// the stored frequencies do not cover (a corrupt table) keep entry 0, which decodes to symbol 0; a table
// record that points outside the `freq_entries` stored frequencies, or claims more symbols than slots, is
// cut to what exists.
template <typename Entry, typename Pack>
__device__ __forceinline__ void fill_table(Entry* table, const int32_t* stream_meta, const uint16_t* freq_tables,
                                           int64_t freq_entries, int t, uint32_t table_size, uint32_t lane, Pack pack) {
  const int64_t offset = stream_meta[t * 4 + 2];
  int alphabet = min(stream_meta[t * 4 + 3], static_cast<int>(table_size));
  if (offset < 0 || offset >= freq_entries) alphabet = 0;
  else alphabet = static_cast<int>(min(static_cast<int64_t>(alphabet), freq_entries - offset));
  for (uint32_t slot = lane; slot < table_size; slot += 32) table[slot] = Entry(0);
  __syncwarp();
  uint32_t running = 0;
  for (int base = 0; base < alphabet; base += 32) {
    const uint32_t mine = base + static_cast<int>(lane) < alphabet ? freq_tables[offset + base + lane] : 0u;
    const int batch = min(32, alphabet - base);
    for (int k = 0; k < batch; ++k) {
      const uint32_t freq = __shfl_sync(0xFFFFFFFFu, mine, k);
      const uint32_t end = min(running + freq, table_size);
      for (uint32_t slot = running + lane; slot < end; slot += 32) table[slot] = pack(static_cast<uint32_t>(base + k), freq, slot - running);
      running = end;
    }
  }
}

__global__ void __launch_bounds__(32) lattice_build_tables_kernel(uint64_t* tables, const int32_t* stream_meta,
                                                                  const uint16_t* freq_tables, int64_t freq_entries, int prob_bits) {
  const uint32_t table_size = 1u << prob_bits;
  fill_table<uint64_t>(tables + static_cast<size_t>(blockIdx.x) * table_size, stream_meta, freq_tables, freq_entries, blockIdx.x,
                       table_size, lane_id(), pack_entry64);
}

// ---- decode ----------------------------------------------------------------------------------------
// TABLES: where the slot tables live. MODE: what happens to a reconstructed vector. TOKENS: kModeProduct only.
// PB: the container's prob_bits when it is the usual 11 (shifts, masks and table offsets become literals), 0 = read
// it from the parameters.
template <int TABLES, int MODE, int TOKENS = 0, int PB = 0>
__global__ void __launch_bounds__(kDecodeThreads, 1) lattice_decode_kernel(const LatticeDecodeParams p) {
  // 256-word ring chunks (upkeep twice per group of nine steps) wherever shared memory has the room: everywhere but
  // beside the wide tables
  using Ring = WordRing<TABLES == kTablesSharedWide ? 7 : 8>;
  extern __shared__ __align__(16) uint32_t shared_tables[];  // [17][table_size] on the shared paths (then [17][table_size] bytes when wide)
  // smallest value of every field for either coset: field_min[c][f] = sym_min of table 1 + 2 f + c
  __shared__ __align__(16) int field_min[2][8];
  const uint32_t lane = lane_id();
  const int warp = threadIdx.x >> 5;
  const int prob_bits = PB ? PB : p.prob_bits;
  const uint32_t table_size = 1u << prob_bits;
  const uint32_t slot_mask = table_size - 1u;
  const uint32_t mask_ge = lanemask_ge();
  const uint32_t shared_base = static_cast<uint32_t>(__cvta_generic_to_shared(shared_tables));

  if (threadIdx.x < 16) field_min[threadIdx.x & 1][threadIdx.x >> 1] = p.stream_meta[(1 + threadIdx.x) * 4 + 1];
  if (TABLES != kTablesGlobal && p.slot_tables != nullptr) {
    // The tables were built once for this container (kModeExport) and come in as they are: 16-byte asynchronous
    // copies, all in flight at once.
    const uint32_t words = kTables * table_size + (TABLES == kTablesSharedWide ? kTables * table_size / 4 : 0u);
    for (uint32_t at = threadIdx.x * 4u; at < words; at += kDecodeThreads * 4u) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(shared_base + at * 4u), "l"(p.slot_tables + at) : "memory");
    }
    ring_commit();     // waited for below, together with the first tile's ring chunks
  } else if (TABLES != kTablesGlobal) {
    // The 17 slot tables are built by the whole block, one work item per (table, run of 32 symbols): first the
    // frequency total of every run, then, from the totals before it, each run's first slot; inside a run every thread
    // fills the slots of its own symbol when that symbol is rare and the warp shares the slots of a frequent one. (One
    // warp per table, symbol after symbol, costs a table of a few hundred mostly rare symbols thousands of cycles while
    // the rest of the block waits.)
    constexpr bool kWide = TABLES == kTablesSharedWide;
    constexpr int kAlphabetLimit = kWide ? kWideMaxAlphabet : kSharedMaxAlphabet;
    constexpr int kRuns = kAlphabetLimit / 32;
    constexpr int kMaxEntries = kTables * kAlphabetLimit;
    uint8_t* const high_bits = reinterpret_cast<uint8_t*>(shared_tables + kTables * table_size);   // wide tables only
    const auto pack = [](uint32_t symbol, uint32_t freq, uint32_t delta) {
      return kWide ? ((symbol & 0x3FFu) | ((freq - 1u) << 10) | (delta << 21)) : pack_entry32(symbol, freq, delta);
    };
    __shared__ uint32_t run_total[kTables][kRuns];
    __shared__ uint32_t run_start[kTables][kRuns];
    __shared__ int meta[kTables * 4];
    // The stream records and the stored frequencies come to shared memory first, in two passes of the whole block (the
    // rings' space is free until decoding starts), so the table build below never waits on global memory.
    if (threadIdx.x < kTables * 4) meta[threadIdx.x] = p.stream_meta[threadIdx.x];
    for (uint32_t slot = threadIdx.x; slot < kTables * table_size; slot += kDecodeThreads) shared_tables[slot] = 0u;
    if (kWide) {
      for (uint32_t slot = threadIdx.x; slot < kTables * table_size / 4; slot += kDecodeThreads) {
        reinterpret_cast<uint32_t*>(high_bits)[slot] = 0u;
      }
    }
    __syncthreads();
    // landing area for the frequencies: the rings' space, behind the tables; a container with more entries than fit
    // there (only possible with wide tables) has them read from global memory instead
    uint16_t* const staged_freq = reinterpret_cast<uint16_t*>(shared_tables + kTables * table_size) + (kWide ? kTables * table_size / 2 : 0);
    const int entries = static_cast<int>(max(int64_t(0), min(static_cast<int64_t>(min(meta[(kTables - 1) * 4 + 2] + meta[(kTables - 1) * 4 + 3], kMaxEntries)),
                                                             p.freq_entries)));
    const bool staged = entries * 2 <= kDecodeWarps * static_cast<int>(Ring::kBytes);
    if (staged) {
      for (int i = threadIdx.x; i < entries; i += kDecodeThreads) staged_freq[i] = p.freq_tables[i];
    }
    __syncthreads();
    auto frequency = [&](int t, int symbol) -> uint32_t {
      const int alphabet = min(meta[t * 4 + 3], kAlphabetLimit);
      const int at = meta[t * 4 + 2] + symbol;
      if (!(symbol < alphabet && at >= 0 && at < entries)) return 0u;
      return staged ? staged_freq[at] : __ldg(p.freq_tables + at);
    };
    // live work items, table after table: first_item[t] .. first_item[t + 1] are table t's runs of 32 symbols
    __shared__ int first_item[kTables + 1];
    if (threadIdx.x == 0) {
      int total = 0;
      for (int t = 0; t < kTables; ++t) {
        first_item[t] = total;
        total += (max(0, min(meta[t * 4 + 3], kAlphabetLimit)) + 31) / 32;
      }
      first_item[kTables] = total;
    }
    __syncthreads();
    const int items = first_item[kTables];
    auto locate = [&](int item, int& t, int& run) {
      t = 0;
      while (t + 1 < kTables && first_item[t + 1] <= item) ++t;
      run = item - first_item[t];
    };
    for (int item = warp; item < items; item += kDecodeWarps) {
      int t, run;
      locate(item, t, run);
      const uint32_t freq = frequency(t, run * 32 + static_cast<int>(lane));
      const uint32_t total = __reduce_add_sync(0xFFFFFFFFu, freq);
      if (lane == 0) run_total[t][run] = total;
    }
    __syncthreads();
    // each run's first slot: the totals of the runs before it in its table
    for (int index = threadIdx.x; index < kTables * kRuns; index += kDecodeThreads) {
      const int t = index / kRuns, run = index % kRuns;
      if (run < first_item[t + 1] - first_item[t]) {
        uint32_t before = 0;
        for (int r = 0; r < run; ++r) before += run_total[t][r];
        run_start[t][run] = before;
      }
    }
    __syncthreads();
    for (int item = warp; item < items; item += kDecodeWarps) {
      int t, run;
      locate(item, t, run);
      uint32_t* table = shared_tables + static_cast<size_t>(t) * table_size;
      const int symbol = run * 32 + static_cast<int>(lane);
      const uint32_t freq = frequency(t, symbol);
      uint32_t inclusive = freq;
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, inclusive, step);
        if (lane >= static_cast<uint32_t>(step)) inclusive += below;
      }
      const uint32_t first = run_start[t][run] + inclusive - freq;    // this symbol's first slot
      // rare symbols: every thread fills its own
      const bool rare = freq < 32u;
      const uint32_t longest = __reduce_max_sync(0xFFFFFFFFu, rare ? freq : 0u);
      for (uint32_t j = 0; j < longest; ++j) {
        if (rare && j < freq && first + j < table_size) {
          table[first + j] = pack(static_cast<uint32_t>(symbol), freq, j);
          if (kWide) high_bits[static_cast<size_t>(t) * table_size + first + j] = static_cast<uint8_t>(symbol >> 10);
        }
      }
      // frequent symbols: the warp shares each one's slots
      uint32_t frequent = __ballot_sync(0xFFFFFFFFu, !rare);
      while (frequent) {
        const int k = __ffs(frequent) - 1;
        frequent &= frequent - 1u;
        const uint32_t f = __shfl_sync(0xFFFFFFFFu, freq, k);
        const uint32_t at = __shfl_sync(0xFFFFFFFFu, first, k);
        for (uint32_t j = lane; j < f && at + j < table_size; j += 32) {
          table[at + j] = pack(static_cast<uint32_t>(run * 32 + k), f, j);
          if (kWide) high_bits[static_cast<size_t>(t) * table_size + at + j] = static_cast<uint8_t>((run * 32 + k) >> 10);
        }
      }
    }
  }
  // tables built here: the build read its frequencies from the rings' space, which the first ring fetch below overwrites
  if (MODE == kModeExport || (TABLES != kTablesGlobal && p.slot_tables == nullptr)) __syncthreads();
  if (MODE == kModeExport) {
    const uint32_t words = kTables * table_size + (TABLES == kTablesSharedWide ? kTables * table_size / 4 : 0u);
    for (uint32_t at = threadIdx.x; at < words; at += kDecodeThreads) p.export_tables[at] = shared_tables[at];
    return;
  }

  const uint32_t table_bytes = TABLES == kTablesGlobal ? 0u : kTables * table_size * (TABLES == kTablesSharedWide ? 5u : 4u);
  const uint32_t ring = ((shared_base + table_bytes + Ring::kBytes - 1u) & ~(Ring::kBytes - 1u)) + static_cast<uint32_t>(warp) * Ring::kBytes;
  // a row holds at least a group's 32 vectors: stepping back one group crosses at most one row boundary
  const bool long_rows = p.vecs_per_row >= 32;

  // State of the tile a warp is decoding, set by open_tile.
  int64_t tile_begin = 0;
  int count = 0;
  uint32_t x = 0;
  int origin = 0, cursor = 0, chunk = -1, refill_at = 0;
  // Reads a tile's stream bounds and states and asks for the three ring chunks at the stream's end; false for a tile
  // whose offsets are out of range (reported, skipped). `drain`: the previous tile's last prefetch may still be in
  // flight and every thread must be past its reads of the old ring contents before the ring is refilled.
  auto open_tile = [&](int64_t tile, bool drain) -> bool {
    tile_begin = tile * p.tile_vectors;
    count = static_cast<int>(min(static_cast<int64_t>(p.tile_vectors), p.vectors - tile_begin));
    // through a warp reduction, so that the cursor arithmetic and its tests are known to be warp-uniform
    const uint32_t begin = __reduce_min_sync(0xFFFFFFFFu, p.offsets[tile]);
    const uint32_t end = __reduce_min_sync(0xFFFFFFFFu, p.offsets[tile + 1]);
    if (end < begin || static_cast<int64_t>(end) > p.payload_words) {
      if (lane == 0) report(p.error, EP_STREAM_BAD_OFFSETS);
      return false;
    }
    x = p.states[tile * kNumStates + lane];
    origin = 2 * static_cast<int>(begin & (Ring::kWords - 1));
    cursor = origin + 2 * static_cast<int>(end - begin);
    chunk = end > begin ? static_cast<int>((end - 1u) >> Ring::kLog) : -1;
    refill_at = origin + 2 * static_cast<int>((static_cast<int64_t>(chunk) << Ring::kLog) - static_cast<int64_t>(begin));
    if (drain) {
      ring_wait_all();
      __syncwarp();
    }
    Ring::fetch_clipped(p.payload, p.payload_words, ring, chunk, lane);
    Ring::fetch_clipped(p.payload, p.payload_words, ring, chunk - 1, lane);
    Ring::fetch_clipped(p.payload, p.payload_words, ring, chunk - 2, lane);
    ring_commit();
    return true;
  };

  // tile t goes to block t mod grid: every SM gets its share even when there are fewer tiles than warp slots. A warp's
  // first tile is opened before the block meets at the barrier behind the tables: its bounds, states and ring chunks
  // travel while the tables are still being copied in (or were being built).
  int64_t tile = static_cast<int64_t>(warp) * gridDim.x + blockIdx.x;
  bool first_pass = true;
  const bool first_open = tile < p.tiles && open_tile(tile, false);
  ring_wait_all();
  __syncthreads();
  for (; tile < p.tiles; tile += static_cast<int64_t>(gridDim.x) * kDecodeWarps, first_pass = false) {
    if (first_pass) {
      if (!first_open) continue;
    } else {
      if (!open_tile(tile, true)) continue;
      ring_wait_all();
      __syncwarp();
    }
    Ring::fetch_interior(p.payload, ring, chunk - 3, lane);
    ring_commit();

    // One symbol from the table that starts `table_first` entries into the table array, `coset_at` entries further for
    // the tables of coset 1 (a multiple of the table size, so it can be or-ed into the slot). Same chain as the Tile-ANS
    // decoder; `valid` is a literal in the main loop, so its tests fold away there.
    auto step = [&](uint32_t table_first, uint32_t coset_at, auto valid) -> uint32_t {
      constexpr bool kWholeGroup = std::is_same<decltype(valid), std::true_type>::value;
      uint32_t symbol = 0;
      if (valid) {
        const uint32_t slot = (x & slot_mask) | coset_at;
        if (TABLES == kTablesShared) {
          // entry = symbol | delta << 9 | freq << 20, so entry >> 9 = freq * 2048 + delta and
          // freq * (x >> prob_bits) + delta = freq * ((x >> prob_bits) - 2048) + (entry >> 9): one shift between the
          // table read and the multiply-add
          const uint32_t entry = shared_tables[table_first + slot];
          symbol = entry & 0x1FFu;
          x = (entry >> 20) * ((x >> prob_bits) - 2048u) + (entry >> 9);
        } else if (TABLES == kTablesSharedWide) {
          const uint32_t entry = shared_tables[table_first + slot];
          const uint32_t high = reinterpret_cast<const uint8_t*>(shared_tables + kTables * table_size)[table_first + slot];
          symbol = (entry & 0x3FFu) | (high << 10);
          x = (((entry >> 10) & 0x7FFu) + 1u) * (x >> prob_bits) + (entry >> 21);
        } else {
          const uint64_t entry = __ldg(p.global_tables + table_first + slot);
          symbol = static_cast<uint32_t>(entry) & 0xFFFFu;
          x = ((static_cast<uint32_t>(entry) >> 16) & 0xFFFFu) * (x >> prob_bits) + static_cast<uint32_t>(entry >> 32);
        }
      }
      if constexpr (kWholeGroup) {
        renormalize_from_ring<Ring::kBytes>(x, cursor, ring, mask_ge);
      } else {
        const bool need = valid && x < kStateMin;
        const uint32_t vote = __ballot_sync(0xFFFFFFFFu, need);
        const int below = cursor - 2 * static_cast<int>(__popc(vote & mask_ge));
        const uint32_t merged = __byte_perm(load_shared_u16((static_cast<uint32_t>(below) & (Ring::kBytes - 2u)) | ring), x, 0x5410);
        x = need ? merged : x;
        cursor = __shfl_sync(0xFFFFFFFFu, below, 0);   // thread 0 counted every reader
      }
      return symbol;
    };
    auto upkeep = [&]() {
      // needed at most once where the stream is intact (a corrupt one reads stale ring words, inside the ring, and is
      // reported at the tile's end); the test is the same in every thread, and the vote tells the compiler so
      if (__any_sync(0xFFFFFFFFu, cursor <= refill_at)) {
        refill_at -= 2 * Ring::kChunk;
        chunk -= 1;
        ring_wait_all();
        __syncwarp();
        Ring::fetch_interior(p.payload, ring, chunk - 3, lane);
        ring_commit();
      }
    };

    // groups of 32 vectors, back to front; a partial group at the tile's end comes first
    int offset = count - (count & 31);
    if ((count & 31) == 0) offset -= 32;
    // row and column (in vectors) of this thread's vector in the current group, stepped back 32 per group
    int row = static_cast<int>(static_cast<uint32_t>(tile_begin + offset + lane) / static_cast<uint32_t>(p.vecs_per_row));
    int col = static_cast<int>(static_cast<uint32_t>(tile_begin + offset + lane) - static_cast<uint32_t>(row) * p.vecs_per_row);
    uint32_t seen_cosets = 0;     // every coset symbol or-ed together: anything above 1 is a corrupt table
    // kModeProduct: this thread's running dot products for the weight row it is in, flushed with one atomic add per
    // token whenever its vectors move on to another row, and at the end of the tile
    constexpr int kTokens = TOKENS > 0 ? TOKENS : 1;
    float running[kTokens];
    int running_row = -1;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) running[t] = 0.0f;
    auto flush_products = [&]() {
      if (running_row >= 0) {
#pragma unroll
        for (int t = 0; t < kTokens; ++t) {
          if (t < p.tokens) atomicAdd(p.products + static_cast<int64_t>(t) * p.rows + running_row, running[t]);
          running[t] = 0.0f;
        }
      }
    };
    auto decode_group = [&](auto valid) {
      // the row's scale, and in kModeProduct the activations this vector will meet, are requested before the vector's
      // nine chain steps, so that their latency (an L2 round trip once the payload stream has pushed them out of L1)
      // hides behind the chain
      const float scale = valid ? __ldg(p.scales + row) : 0.0f;
      uint4 early[kTokens];
      if (MODE == kModeProduct && valid) {
#pragma unroll
        for (int t = 0; t < kTokens; ++t) {
          if (t < p.tokens) early[t] = __ldg(reinterpret_cast<const uint4*>(p.activations + (static_cast<int64_t>(t) * p.vecs_per_row + col) * 8));
        }
      }
      uint32_t coset = step(0u, 0u, valid);
      seen_cosets |= coset;
      coset = min(coset, 1u);      // a corrupt coset table must not steer the look-ups past the 17 tables
      const uint32_t coset_at = coset << prob_bits;
      // each value is reconstructed right behind the step that decoded it, in the shadow of the next step's chain
      // (table read, vote, ring read), instead of all eight after the last step
      const int4 low = *reinterpret_cast<const int4*>(&field_min[coset][0]);
      const int4 high = *reinterpret_cast<const int4*>(&field_min[coset][4]);
      const int lows[8] = {low.x, low.y, low.z, low.w, high.x, high.y, high.z, high.w};
      const float half = coset ? 0.5f : 0.0f;
      int value[8];
      float v[8];
#pragma unroll
      for (int field = 0; field < 8; ++field) {
        value[field] = static_cast<int>(step((1 + 2 * field) * table_size, coset_at, valid)) + lows[field];
        if (field < 7) v[field] = __fmul_rn(__fadd_rn(static_cast<float>(value[field]), half), scale);
        // upkeep every kStepsPerUpkeep steps at most: after fields 3 and 7 (five and four steps), or 1, 4 and 7
        if (Ring::kStepsPerUpkeep >= 8 ? (field == 3 || field == 7) : (field == 1 || field == 4 || field == 7)) upkeep();
      }
      if (valid) {
        // z7 = 2 m + (z0 + ... + z6 mod 2); the parity of a sum is the exclusive-or of the low bits
        const int parity = (value[0] ^ value[1] ^ value[2]) ^ (value[3] ^ value[4] ^ value[5]) ^ value[6];
        value[7] = 2 * value[7] + (parity & 1);
        const int64_t vector = tile_begin + offset + lane;
        v[7] = __fmul_rn(__fadd_rn(static_cast<float>(value[7]), half), scale);
        if (MODE == kModeProduct) {
          if (row != running_row) {
            flush_products();
            running_row = row;
          }
          // the weight as the dense layer sees it: rounded to bf16 first
          float w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
#pragma unroll
          for (int t = 0; t < kTokens; ++t) {
            if (t < p.tokens) {
              const uint32_t words[4] = {early[t].x, early[t].y, early[t].z, early[t].w};
              float sum = running[t];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                sum = fmaf(w[2 * j], __uint_as_float(words[j] << 16), sum);
                sum = fmaf(w[2 * j + 1], __uint_as_float(words[j] & 0xFFFF0000u), sum);
              }
              running[t] = sum;
            }
          }
        } else if (MODE == kModeStoreBf16) {
          // the container cast clamps to the largest finite bf16 before it rounds; the saturating conversion does both
          // (and keeps a NaN a NaN, as the reference's clamp does), so no value needs a second look
          uint4 packed;
          packed.x = bf16x2_saturating(v[0], v[1]);
          packed.y = bf16x2_saturating(v[2], v[3]);
          packed.z = bf16x2_saturating(v[4], v[5]);
          packed.w = bf16x2_saturating(v[6], v[7]);
          *reinterpret_cast<uint4*>(static_cast<char*>(p.output) + vector * 16) = packed;
        } else if (MODE == kModeStoreCodes) {
          // the saturating conversions give what clamping first and converting then gives
          {
            uint2 packed;
            if (p.store_kind == EP_STORE_F8_E4M3) {
              const uint32_t a = __nv_cvt_float2_to_fp8x2(make_float2(v[0], v[1]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t b = __nv_cvt_float2_to_fp8x2(make_float2(v[2], v[3]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t c = __nv_cvt_float2_to_fp8x2(make_float2(v[4], v[5]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t d = __nv_cvt_float2_to_fp8x2(make_float2(v[6], v[7]), __NV_SATFINITE, __NV_E4M3);
              packed = make_uint2(a | (b << 16), c | (d << 16));
            } else {
              // round to nearest even and saturate to [-128, 127] in one conversion each, low bytes gathered pairwise
              uint32_t code[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(code[j]) : "f"(v[j]));
              packed.x = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
              packed.y = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
            }
            *reinterpret_cast<uint2*>(static_cast<char*>(p.output) + vector * 8) = packed;
          }
        } else {
          store_vector(p.output, vector, v, p.store_kind);
        }
      }
      offset -= 32;
      col -= 32;
      if (long_rows) {
        const bool wrapped = col < 0;
        col += wrapped ? p.vecs_per_row : 0;
        row -= wrapped ? 1 : 0;
      } else {
        while (col < 0) {
          col += p.vecs_per_row;
          row -= 1;
        }
      }
    };
    if (count & 31) decode_group(lane < static_cast<uint32_t>(count & 31));
    while (offset >= 0) decode_group(std::true_type{});
    if (MODE == kModeProduct) {
      flush_products();
      running_row = -1;
    }
    const bool dirty = __any_sync(0xFFFFFFFFu, x != kStateMin);
    const bool bad_coset = __any_sync(0xFFFFFFFFu, seen_cosets > 1u);
    const int left = (cursor - origin) / 2;
    if (lane == 0) {
      if (bad_coset) report(p.error, EP_STREAM_BAD_SYMBOL);
      else if (left < 0) report(p.error, EP_STREAM_UNDERRUN);
      else if (left != 0 || dirty) report(p.error, EP_STREAM_NOT_CONSUMED);
    }
  }
  if (MODE == kModeProduct) {
    // The block that finishes last turns the accumulators into the layer's output: y = bf16(sum + bias).
    __shared__ bool last_block;
    __threadfence();
    __syncthreads();
    const int64_t total = static_cast<int64_t>(p.tokens) * p.rows;
    if (threadIdx.x == 0) {
      const unsigned int done = atomicAdd(reinterpret_cast<unsigned int*>(p.products + total), 1u);
      last_block = done == gridDim.x - 1;
    }
    __syncthreads();
    if (last_block) {
      __threadfence();
      for (int64_t i = threadIdx.x; i < total; i += kDecodeThreads) {
        const float sum = __ldcg(p.products + i);   // from L2, where the other blocks' atomic adds landed
        p.product_out[i] = __float2bfloat16_rn(sum + (p.bias ? __bfloat162float(p.bias[i % p.rows]) : 0.0f));
      }
    }
  }
}

}  // namespace
}  // namespace ep

using namespace ep;

extern "C" int64_t ep_lattice_decode_scratch_bytes(int prob_bits, int max_alphabet) {
  if (prob_bits < 9 || prob_bits > 15) return EP_ERR_INVALID_ARGUMENT;
  if (prob_bits <= kSharedMaxProbBits) return 0;   // both shared-memory layouts together cover every alphabet up to 2^11
  return static_cast<int64_t>(kTables) * sizeof(uint64_t) << prob_bits;
}

extern "C" int64_t ep_lattice_slot_tables_bytes(int prob_bits, int max_alphabet) {
  if (prob_bits < 9 || prob_bits > 15 || max_alphabet < 0 || max_alphabet > (1 << prob_bits)) return EP_ERR_INVALID_ARGUMENT;
  const int64_t slots = static_cast<int64_t>(kTables) << prob_bits;
  if (prob_bits > kSharedMaxProbBits) return slots * 8;
  return max_alphabet <= kSharedMaxAlphabet ? slots * 4 : slots * 5;
}

extern "C" int ep_lattice_build_slot_tables(const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev, int64_t freq_entries,
                                            int prob_bits, int max_alphabet, void* slot_tables_dev, int64_t slot_tables_bytes,
                                            ep_stream_t stream) {
  const int64_t needed = ep_lattice_slot_tables_bytes(prob_bits, max_alphabet);
  if (needed < 0) return static_cast<int>(needed);
  if (!stream_meta_dev || !freq_tables_dev || freq_entries < 0 || !slot_tables_dev || slot_tables_bytes < needed ||
      (reinterpret_cast<uintptr_t>(slot_tables_dev) & 15u)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (prob_bits > kSharedMaxProbBits) {
    lattice_build_tables_kernel<<<kTables, 32, 0, s>>>(static_cast<uint64_t*>(slot_tables_dev), stream_meta_dev, freq_tables_dev,
                                                       freq_entries, prob_bits);
    return check_launch("lattice_build_tables_kernel");
  }
  // one block of the decode kernel in its export mode: it builds the tables exactly as a decode would and writes them out
  LatticeDecodeParams p = {};
  p.stream_meta = stream_meta_dev;
  p.freq_tables = freq_tables_dev;
  p.freq_entries = freq_entries;
  p.prob_bits = prob_bits;
  p.export_tables = static_cast<uint32_t*>(slot_tables_dev);
  const bool wide = max_alphabet > kSharedMaxAlphabet;
  const size_t shared = static_cast<size_t>(needed) + static_cast<size_t>(kDecodeWarps + 1) * (wide ? WordRing<7>::kBytes : WordRing<8>::kBytes);
  if (wide) {
    EP_CUDA_CHECK(cudaFuncSetAttribute(lattice_decode_kernel<kTablesSharedWide, kModeExport, 0, 0>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
    lattice_decode_kernel<kTablesSharedWide, kModeExport, 0, 0><<<1, kDecodeThreads, shared, s>>>(p);
  } else {
    EP_CUDA_CHECK(cudaFuncSetAttribute(lattice_decode_kernel<kTablesShared, kModeExport, 0, 0>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
    lattice_decode_kernel<kTablesShared, kModeExport, 0, 0><<<1, kDecodeThreads, shared, s>>>(p);
  }
  return check_launch("lattice_decode_kernel (table export)");
}

namespace ep {
namespace {

// Size of a container's slot tables as the decode kernel wants them: 32-bit entries (plus a byte per slot behind them
// for alphabets beyond 512) when they go to shared memory, 64-bit entries when they stay in global memory.
int64_t slot_table_bytes(int prob_bits, int max_alphabet) {
  const int64_t slots = static_cast<int64_t>(kTables) << prob_bits;
  if (prob_bits > kSharedMaxProbBits) return slots * 8;
  return max_alphabet <= kSharedMaxAlphabet ? slots * 4 : slots * 5;
}

// The kernel for one table layout and prob_bits specialisation, picked by what is done with a vector.
template <int TABLES, int PB, typename Launch>
int launch_for_mode(Launch&& launch, size_t shared, bool product, int tokens, int store_kind) {
  if (product) {
    return tokens == 1 ? launch(lattice_decode_kernel<TABLES, kModeProduct, 1, PB>, shared)
         : tokens == 2 ? launch(lattice_decode_kernel<TABLES, kModeProduct, 2, PB>, shared)
                       : launch(lattice_decode_kernel<TABLES, kModeProduct, 4, PB>, shared);
  }
  if (store_kind == EP_STORE_BF16) return launch(lattice_decode_kernel<TABLES, kModeStoreBf16, 0, PB>, shared);
  if (store_kind == EP_STORE_F8_E4M3 || store_kind == EP_STORE_I8) return launch(lattice_decode_kernel<TABLES, kModeStoreCodes, 0, PB>, shared);
  return launch(lattice_decode_kernel<TABLES, kModeStore, 0, PB>, shared);
}

// Validates the arguments, fills the parameter block and launches the decode (plus the table-build
// kernel on the global path). `tables` must hold 17 * 2^prob_bits 64-bit entries when the container
// needs the global path; it is ignored otherwise.
int launch_lattice_decode(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                          const uint32_t* states_dev, const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev,
                          int64_t freq_entries, const float* scales_dev, void* output_dev, int store_kind, int64_t rows,
                          int64_t cols, int prob_bits, int64_t tile_elements, int max_alphabet, uint64_t* tables,
                          int64_t table_bytes, bool tables_ready, int* error_dev, cudaStream_t s,
                          const __nv_bfloat16* activations = nullptr,
                          float* products = nullptr, int tokens = 0, const __nv_bfloat16* bias = nullptr,
                          __nv_bfloat16* product_out = nullptr) {
  if (rows <= 0 || cols <= 0 || (cols & 7) != 0 || prob_bits < 9 || prob_bits > 15 || tile_elements <= 0 ||
      store_kind < 0 || store_kind > EP_STORE_BOOL || max_alphabet < 0 || max_alphabet > (1 << prob_bits) ||
      payload_words < 0 || freq_entries < 0 || !offsets_dev || !states_dev || !stream_meta_dev || !freq_tables_dev ||
      !scales_dev || (!output_dev && !products)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (payload_words > 0 && !payload_dev) return EP_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(payload_dev) & 15u) || (reinterpret_cast<uintptr_t>(output_dev) & 15u)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  const int64_t vectors = rows * (cols / 8);
  if (vectors >= (int64_t(1) << 31)) return EP_ERR_TOO_LARGE;
  LatticeDecodeParams p;
  p.payload = payload_dev;
  p.payload_words = payload_words;
  p.offsets = offsets_dev;
  p.states = states_dev;
  p.stream_meta = stream_meta_dev;
  p.freq_tables = freq_tables_dev;
  p.freq_entries = freq_entries;
  p.scales = scales_dev;
  p.output = output_dev;
  p.global_tables = nullptr;
  p.slot_tables = nullptr;
  p.export_tables = nullptr;
  p.vectors = vectors;
  const int64_t tile_vectors = tile_elements / 9 < 32 ? 32 : tile_elements / 9;
  if (tile_vectors > 0x7FFFFFFF) return EP_ERR_TOO_LARGE;
  p.tile_vectors = static_cast<int>(tile_vectors);
  p.tiles = (vectors + tile_vectors - 1) / tile_vectors;
  p.vecs_per_row = static_cast<int>(cols / 8);
  p.prob_bits = prob_bits;
  p.store_kind = store_kind;
  p.error = error_dev;
  p.activations = activations;
  p.products = products;
  p.bias = bias;
  p.product_out = product_out;
  p.tokens = tokens;
  p.rows = static_cast<int>(rows);
  // one persistent block per SM (of the SMs this thread's launches may fill); with fewer tiles than that, one block per tile
  const int sms = decode_sm_limit();
  const unsigned blocks = static_cast<unsigned>(p.tiles < sms ? p.tiles : sms);
  // one ring per warp, plus one ring's worth of slack for aligning the first to its size
  const size_t ring_bytes = static_cast<size_t>(kDecodeWarps + 1) * WordRing<8>::kBytes;
  const size_t narrow_ring_bytes = static_cast<size_t>(kDecodeWarps + 1) * WordRing<7>::kBytes;
  const auto launch = [&](auto kernel, size_t shared) -> int {
    EP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
    kernel<<<blocks, kDecodeThreads, shared, s>>>(p);
    return EP_OK;
  };
  const bool product = products != nullptr;
  int launched = EP_OK;
  if (tables_ready) {
    // tables built for this container by ep_lattice_build_slot_tables: the shared paths copy them in, the global path reads them
    if (!tables || table_bytes < slot_table_bytes(prob_bits, max_alphabet) || (reinterpret_cast<uintptr_t>(tables) & 15u)) {
      return EP_ERR_INVALID_ARGUMENT;
    }
    p.slot_tables = reinterpret_cast<const uint32_t*>(tables);
  }
  if (prob_bits <= kSharedMaxProbBits && max_alphabet <= kSharedMaxAlphabet) {
    const size_t shared = (static_cast<size_t>(kTables) * sizeof(uint32_t) << prob_bits) + ring_bytes;
    launched = prob_bits == 11 ? launch_for_mode<kTablesShared, 11>(launch, shared, product, tokens, store_kind)
                               : launch_for_mode<kTablesShared, 0>(launch, shared, product, tokens, store_kind);
  } else if (prob_bits <= kSharedMaxProbBits) {
    // alphabets beyond 512 (fine scales, heavy-tailed rows): word tables plus a byte table of high symbol bits
    const size_t shared = (static_cast<size_t>(kTables) * 5 << prob_bits) + narrow_ring_bytes;
    launched = prob_bits == 11 ? launch_for_mode<kTablesSharedWide, 11>(launch, shared, product, tokens, store_kind)
                               : launch_for_mode<kTablesSharedWide, 0>(launch, shared, product, tokens, store_kind);
  } else {
    const int64_t needed = static_cast<int64_t>(kTables) * sizeof(uint64_t) << prob_bits;
    if (!tables || table_bytes < needed || (reinterpret_cast<uintptr_t>(tables) & 7u)) return EP_ERR_INVALID_ARGUMENT;
    if (!tables_ready) lattice_build_tables_kernel<<<kTables, 32, 0, s>>>(tables, stream_meta_dev, freq_tables_dev, freq_entries, prob_bits);
    p.global_tables = tables;
    p.slot_tables = nullptr;
    launched = launch_for_mode<kTablesGlobal, 0>(launch, ring_bytes, product, tokens, store_kind);
  }
  if (launched != EP_OK) return launched;
  return check_launch("lattice_decode_kernel");
}

}  // namespace
}  // namespace ep

extern "C" int ep_lattice_linear_forward(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                                         const uint32_t* states_dev, const int32_t* stream_meta_dev,
                                         const uint16_t* freq_tables_dev, int64_t freq_entries, const float* scales_dev,
                                         int64_t rows, int64_t cols,
                                         int prob_bits, int64_t tile_elements, int max_alphabet, void* table_scratch_dev,
                                         int64_t table_scratch_bytes, int tables_ready, const void* x_dev, const void* bias_dev,
                                         int tokens,
                                         float* products_dev, void* y_dev, int* error_dev, ep_stream_t stream) {
  if (!x_dev || !products_dev || !y_dev || tokens < 1 || tokens > ep::kMaxTokens || rows <= 0 || rows > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (reinterpret_cast<uintptr_t>(x_dev) & 15u) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = static_cast<int64_t>(tokens) * rows;
  EP_CUDA_CHECK(cudaMemsetAsync(products_dev, 0, sizeof(float) * (total + 1), s));   // accumulators and the block counter
  return ep::launch_lattice_decode(payload_dev, payload_words, offsets_dev, states_dev, stream_meta_dev, freq_tables_dev,
                                   freq_entries, scales_dev, nullptr, EP_STORE_BF16, rows, cols, prob_bits, tile_elements, max_alphabet,
                                   static_cast<uint64_t*>(table_scratch_dev), table_scratch_bytes, tables_ready != 0, error_dev, s,
                                   static_cast<const __nv_bfloat16*>(x_dev), products_dev, tokens,
                                   static_cast<const __nv_bfloat16*>(bias_dev), static_cast<__nv_bfloat16*>(y_dev));
}

extern "C" int ep_lattice_decode(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                                 const uint32_t* states_dev, const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev,
                                 int64_t freq_entries, const float* scales_dev, void* output_dev, int store_kind, int64_t rows, int64_t cols,
                                 int prob_bits, int64_t tile_elements, int max_alphabet, void* table_scratch_dev,
                                 int64_t table_scratch_bytes, int tables_ready, int* error_dev, ep_stream_t stream) {
  return launch_lattice_decode(payload_dev, payload_words, offsets_dev, states_dev, stream_meta_dev, freq_tables_dev, freq_entries,
                               scales_dev, output_dev, store_kind, rows, cols, prob_bits, tile_elements, max_alphabet,
                               static_cast<uint64_t*>(table_scratch_dev), table_scratch_bytes, tables_ready != 0, error_dev,
                               static_cast<cudaStream_t>(stream));
}

// ---- decode without any allocation --------------------------------------------------------------------
// Some hosts of this library may not allocate device memory at the moment they need a decode: an
// inference server that has handed all of HBM to its own pool, or a thread running between a
// framework's allocator callbacks where a cudaMalloc would deadlock or synchronise the device. For
// them the 64-bit slot tables of the global-table path live in this fixed array instead of in
// caller-provided scratch. It costs 17 * 2^13 * 8 bytes (1.06 MB) on every GPU that loads the library,
// until the process exits, and caps the containers this entry point accepts on that path at
// prob_bits 13. Containers that take the shared-memory path never touch it.
constexpr int kStaticMaxProbBits = 13;
constexpr size_t kStaticTableBytes = (static_cast<size_t>(ep::kTables) * sizeof(uint64_t)) << kStaticMaxProbBits;
static __device__ __align__(256) unsigned char g_static_slot_tables[kStaticTableBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
uint64_t* g_static_address[kMaxDevices] = {};

// The array's name is only a host-side handle; kernels need its device address, which differs per GPU.
// Looked up once per device, with that device current (the caller's current device).
int static_tables_for_current_device(uint64_t** tables) {
  int device = -1;
  EP_CUDA_CHECK(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return EP_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> guard(g_static_mutex);
  if (g_static_address[device] == nullptr) {
    void* address = nullptr;
    EP_CUDA_CHECK(cudaGetSymbolAddress(&address, g_static_slot_tables));
    g_static_address[device] = static_cast<uint64_t*>(address);
  }
  *tables = g_static_address[device];
  return EP_OK;
}
}  // namespace

extern "C" int ep_lattice_decode_static_max_prob_bits(void) { return kStaticMaxProbBits; }

extern "C" int ep_lattice_decode_static(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                                        const uint32_t* states_dev, const int32_t* stream_meta_dev,
                                        const uint16_t* freq_tables_dev, int64_t freq_entries, const float* scales_dev,
                                        void* output_dev, int store_kind, int64_t rows, int64_t cols, int prob_bits, int64_t tile_elements,
                                        int max_alphabet, int* error_dev, ep_stream_t stream) {
  const bool shared_path = prob_bits <= kSharedMaxProbBits;
  if (!shared_path && prob_bits > kStaticMaxProbBits && prob_bits <= 15) return EP_ERR_TOO_LARGE;
  uint64_t* tables = nullptr;
  const int rc = static_tables_for_current_device(&tables);
  if (rc != EP_OK) return rc;
  return launch_lattice_decode(payload_dev, payload_words, offsets_dev, states_dev, stream_meta_dev, freq_tables_dev, freq_entries,
                               scales_dev, output_dev, store_kind, rows, cols, prob_bits, tile_elements, max_alphabet, tables,
                               static_cast<int64_t>(kStaticTableBytes), false, error_dev, static_cast<cudaStream_t>(stream));
}
