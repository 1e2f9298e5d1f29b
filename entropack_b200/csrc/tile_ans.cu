// Tile-ANS (lossless byte-lane rANS) kernels for sm_100a and their C entry points.
//
// Format (entropack/schemes/tile_ans/format.py:58-64, eager.py:176-307): the tensor's elements are
// split into byte lanes; each lane is cut into tiles of `tile_elements` symbols; a (lane, tile)
// stream is either raw bytes or a 32-way interleaved rANS stream of 16-bit words that the decoder
// consumes back to front. Stream index = lane * tiles + tile.
//
// Decode: one warp owns one tile across ALL byte lanes, so every element is rebuilt in registers and
// leaves with a single whole-element store (32 consecutive elements per warp store), whatever the
// lane pattern. Coded lanes keep one rANS state per thread and look symbols up in a shared-memory
// table that is re-packed at staging time to hold `slot - cdf` directly.
//
// Encode: one warp owns one tile across all byte lanes as well, so the input is read once as whole
// elements. Division by the symbol frequency uses a per-symbol 32-bit reciprocal with one correction.
#include <type_traits>

#include "ep_common.cuh"
#include "rans_ring.cuh"

namespace ep {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxLanes = 8;

struct LaneSetup {
  uint32_t raw_mask;            // bit b set: byte lane b is stored raw
  uint8_t ans_rank[kMaxLanes];  // rank of byte lane b among the coded lanes
  int ans_lanes;
};

struct DecodeParams {
  const uint16_t* payload;
  int64_t payload_words;
  const uint32_t* offsets;
  const uint32_t* states;
  const uint32_t* tables;
  void* output;
  int64_t num_elements;
  int64_t tile_elements;
  int64_t tiles;
  int64_t first_tile;  // this launch decodes tiles [first_tile, tile_end)
  int64_t tile_end;
  int prob_bits;
  LaneSetup lanes;
  int* error;
};

template <int BYTES> struct Element;
template <> struct Element<1> { using type = uint8_t; };
template <> struct Element<2> { using type = uint16_t; };
template <> struct Element<4> { using type = uint32_t; };
template <> struct Element<8> { using type = uint64_t; };

// Shared table entry: symbol | (slot - cdf) << 8 | frequency << 20, so that entry >> 8 is
// frequency * 4096 + (slot - cdf) and the state update frequency * (x >> prob_bits) + (slot - cdf) becomes
// (entry >> 20) * ((x >> prob_bits) - 4096) + (entry >> 8): one shift between the table read and the
// multiply-add. A frequency field of 0 can only mean "the whole table" (one symbol, 4096 slots): such a
// lane decodes to a constant and never reads.
template <int NLANES>
__device__ __forceinline__ void stage_decode_tables(const DecodeParams& p, uint32_t* shared_tables, int* constant_symbol) {
  const uint32_t table_size = 1u << p.prob_bits;
  if (threadIdx.x < kMaxLanes) constant_symbol[threadIdx.x] = -1;
  __syncthreads();
#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    if ((p.lanes.raw_mask >> b) & 1u) continue;
    const uint32_t* source = p.tables + static_cast<size_t>(b) * table_size;
    uint32_t* staged = shared_tables + static_cast<size_t>(p.lanes.ans_rank[b]) * table_size;
    const auto repack = [](uint32_t entry, uint32_t slot) {
      return (entry & 0xFFu) | (((slot - (entry >> 20)) & 0xFFFu) << 8) | ((entry >> 8) << 20);
    };
    if (threadIdx.x == 0) {
      const uint32_t entry = source[0];
      if (((entry >> 8) & 0xFFFu) == 0u) constant_symbol[b] = static_cast<int>(entry & 0xFFu);
    }
    if ((reinterpret_cast<uintptr_t>(source) & 15u) == 0) {
      // four entries per load and store (the table has at least 512 entries)
      const uint4* source4 = reinterpret_cast<const uint4*>(source);
      uint4* staged4 = reinterpret_cast<uint4*>(staged);
      for (uint32_t quad = threadIdx.x; quad < table_size / 4; quad += blockDim.x) {
        const uint4 e = __ldg(source4 + quad);
        const uint32_t slot = quad * 4;
        staged4[quad] = make_uint4(repack(e.x, slot), repack(e.y, slot + 1), repack(e.z, slot + 2), repack(e.w, slot + 3));
      }
    } else {
      for (uint32_t slot = threadIdx.x; slot < table_size; slot += blockDim.x) staged[slot] = repack(source[slot], slot);
    }
  }
  __syncthreads();
}

// General-purpose decoder: one element per thread per step, words read straight from global memory.
// Used when the tile size is odd or the buffers are not 16-byte aligned, i.e. when the staged decoder
// below cannot use vector stores and 16-byte copies.
template <int NLANES>
__global__ void __launch_bounds__(kThreads) tile_ans_decode_simple_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint32_t shared_tables[];
  __shared__ int constant_symbol[kMaxLanes];
  using element_t = typename Element<NLANES>::type;
  const uint32_t table_size = 1u << p.prob_bits;
  stage_decode_tables<NLANES>(p, shared_tables, constant_symbol);

  const int64_t tile = p.first_tile + static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (tile >= p.tile_end) return;
  const uint32_t lane = lane_id();
  const uint32_t mask_ge = lanemask_ge();
  const uint32_t slot_mask = table_size - 1u;
  const int64_t tile_begin = tile * p.tile_elements;
  const int count = static_cast<int>(min(p.tile_elements, p.num_elements - tile_begin));

  const uint8_t* raw_bytes[NLANES];
  const uint16_t* words[NLANES];
  const uint32_t* table[NLANES];
  int position[NLANES];
  uint32_t state[NLANES];
  int constant[NLANES];
  int failure = 0;
#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    const int64_t stream = static_cast<int64_t>(b) * p.tiles + tile;
    const uint32_t begin = p.offsets[stream];
    const uint32_t end = p.offsets[stream + 1];
    if (end < begin || static_cast<int64_t>(end) > p.payload_words) failure = EP_STREAM_BAD_OFFSETS;
    raw_bytes[b] = reinterpret_cast<const uint8_t*>(p.payload + begin);
    words[b] = p.payload + begin;
    position[b] = static_cast<int>(end - begin);
    table[b] = shared_tables;
    state[b] = kStateMin;
    constant[b] = constant_symbol[b];
    if ((p.lanes.raw_mask >> b) & 1u) {
      if (!failure && end - begin != static_cast<uint32_t>((count + 1) >> 1)) failure = EP_STREAM_BAD_RAW_LENGTH;
    } else {
      const int rank = p.lanes.ans_rank[b];
      table[b] = shared_tables + static_cast<size_t>(rank) * table_size;
      state[b] = p.states[(static_cast<int64_t>(rank) * p.tiles + tile) * kNumStates + lane];
    }
  }
  if (failure) {
    if (lane == 0) report(p.error, failure);
    return;
  }

  element_t* out = static_cast<element_t*>(p.output) + tile_begin;
  // Groups of 32 symbols run back to front; a partial group at the tile's end comes first.
  int offset = count - (count & 31);
  bool valid = lane < static_cast<uint32_t>(count & 31);
  if ((count & 31) == 0) {
    offset -= 32;
    valid = true;
  }
  for (; offset >= 0; offset -= 32, valid = true) {
    element_t value = 0;
#pragma unroll
    for (int b = 0; b < NLANES; ++b) {
      uint32_t byte = 0;
      if ((p.lanes.raw_mask >> b) & 1u) {
        if (valid) byte = raw_bytes[b][offset + lane];
      } else if (constant[b] >= 0) {
        byte = static_cast<uint32_t>(constant[b]);
      } else {
        if (valid) {
          const uint32_t x = state[b];
          const uint32_t slot = x & slot_mask;
          const uint32_t entry = table[b][slot];
          byte = entry & 0xFFu;
          state[b] = (entry >> 20) * ((x >> p.prob_bits) - 4096u) + (entry >> 8);
        }
        renormalize(valid, state[b], words[b], position[b], mask_ge);
      }
      value |= static_cast<element_t>(static_cast<element_t>(byte) << (8 * b));
    }
    if (valid) out[offset + lane] = value;
  }

#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    if (((p.lanes.raw_mask >> b) & 1u) || constant[b] >= 0) continue;
    const bool dirty = __any_sync(0xFFFFFFFFu, state[b] != kStateMin);
    if (position[b] < 0) failure = EP_STREAM_UNDERRUN;
    else if (position[b] != 0 || dirty) failure = EP_STREAM_NOT_CONSUMED;
  }
  if (failure && lane == 0) report(p.error, failure);
}

// ------------------------------------------------------------------------------------------------
// Staged decoder (the fast path).
//
// The rANS chain is serial per thread, so every memory access inside it has to be on chip and cheap
// to address:
//   * the stream's 16-bit words are pulled into a per-warp shared-memory ring by 16-byte cp.async
//     copies issued a chunk (128 words) ahead of the chunks being consumed; ring reads are masked
//     into the ring, so even a corrupt stream cannot read out of bounds;
//   * decoded symbols go to a per-warp shared staging block of 512 elements; the 16 groups of a full
//     block are unrolled so every staging store has an immediate offset;
//   * after each block the warp merges staged symbols with the raw lanes' bytes (plain coalesced
//     loads, independent of the chain, many in flight) and writes whole elements with vector stores
//     (two elements per thread; sixteen for one-byte elements).
// All shared-memory state is addressed by 32-bit offsets from the one dynamic shared array, so the
// compiler emits plain LDS/STS with scaled addressing.
// ------------------------------------------------------------------------------------------------
constexpr int kBlockElems = 512;   // elements staged per warp between merges (16 groups of 32)
constexpr int kDecodeBlocksPerSm = 7;   // 56 warps of 32 registers: a tensor of 8192 tiles is resident all at once
// The other block shape: 14 warps, four blocks to an SM (the same 56 resident warps). Four table copies instead of
// seven leave room for the 256-word ring chunks at every probability width, and a block's table is staged for 14 tiles.
constexpr int kByteWarps = 14;
constexpr int kByteBlocksPerSm = 4;
// State of one coded byte lane of the tile a warp is decoding.
struct CodedLane {
  uint32_t state;       // this thread's rANS state
  uint32_t table;       // index (in u32) of the lane's table inside the shared array
  uint32_t ring;        // shared address of the warp's word ring (aligned to the ring size, 1 KB)
  uint32_t stage;       // index (in bytes) of this thread's byte in the warp's staging block (block base + lane)
  int cursor;           // 2 * ((stream begin mod ring size) + words not yet consumed): byte offset just past the next word
  int refill_at;        // cursor value at or below which the chunk boundary has been crossed
  int chunk;            // payload chunk holding the next word to be read
};

// RAW_MASK >= 0 fixes the lane pattern at compile time (dead per-lane state disappears from the register file);
// RAW_MASK < 0 reads it from the parameters. CHUNK_LOG picks the ring: 256-word chunks (upkeep every eight steps)
// where shared memory has the room, 128-word chunks otherwise. WARPS: eight warps to a block and seven blocks to an SM,
// or fourteen and four (the same 56 resident warps with four table copies instead of seven).
template <int NLANES, int RAW_MASK, int CHUNK_LOG, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, (NLANES <= 2 || (NLANES == 4 && RAW_MASK == 7)) ? 56 / WARPS : (NLANES == 4 && WARPS == 8 ? 3 : 1))
tile_ans_decode_kernel(const DecodeParams p) {
  using Ring = WordRing<CHUNK_LOG>;
  constexpr int kWarps = WARPS;     // shadows the file-wide block shape of the other kernels
  extern __shared__ __align__(16) uint32_t shared_tables[];
  __shared__ int constant_symbol[kMaxLanes];
  __shared__ uint32_t raw_begins[kWarps][kMaxLanes];
  using element_t = typename Element<NLANES>::type;
  uint16_t* const shared_words = reinterpret_cast<uint16_t*>(shared_tables);
  uint8_t* const shared_bytes = reinterpret_cast<uint8_t*>(shared_tables);
  const uint32_t table_size = 1u << p.prob_bits;
  const uint32_t raw_mask = RAW_MASK >= 0 ? static_cast<uint32_t>(RAW_MASK) : p.lanes.raw_mask;
  stage_decode_tables<NLANES>(p, shared_tables, constant_symbol);

  const int warp = threadIdx.x >> 5;
  const int64_t tile = p.first_tile + static_cast<int64_t>(blockIdx.x) * kWarps + warp;
  if (tile >= p.tile_end) return;
  const uint32_t lane = lane_id();
  const uint32_t mask_ge = lanemask_ge();
  const uint32_t slot_mask = table_size - 1u;
  const int prob_bits = p.prob_bits;
  const int64_t tile_begin = tile * p.tile_elements;
  const int count = static_cast<int>(min(p.tile_elements, p.num_elements - tile_begin));
  const int ans_lanes = p.lanes.ans_lanes;
  const uint32_t shared_base = static_cast<uint32_t>(__cvta_generic_to_shared(shared_tables));

  // dynamic shared memory: tables | pad to the ring size | rings[warp][rank] | staging[warp][rank]
  constexpr uint32_t kRingBytes = Ring::kBytes;
  const uint32_t rings_address = (shared_base + static_cast<uint32_t>(ans_lanes) * table_size * 4u + kRingBytes - 1u) & ~(kRingBytes - 1u);
  const uint32_t staging_at = (rings_address - shared_base) + static_cast<uint32_t>(kWarps * ans_lanes) * kRingBytes;  // in bytes

  // raw lanes: index of the stream's first 16-bit word in the payload, kept in shared memory (read once per merge)
  uint32_t* const raw_begin = raw_begins[warp];
  CodedLane coded[NLANES];
  int failure = 0;
  bool raw_near_end = false;    // a raw stream ends within 8 bytes of the payload's end: no over-reading loads there
#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    const int64_t stream = static_cast<int64_t>(b) * p.tiles + tile;
    // The bounds of a coded stream pass through a warp-wide reduction: it tells the compiler that they, and the
    // cursor arithmetic built on them, are the same in all 32 threads, so tests on them become uniform branches.
    const bool is_raw = (raw_mask >> b) & 1u;
    const uint32_t begin = is_raw ? p.offsets[stream] : __reduce_min_sync(0xFFFFFFFFu, p.offsets[stream]);
    const uint32_t end = is_raw ? p.offsets[stream + 1] : __reduce_min_sync(0xFFFFFFFFu, p.offsets[stream + 1]);
    if (end < begin || static_cast<int64_t>(end) > p.payload_words) failure = EP_STREAM_BAD_OFFSETS;
    if (lane == 0) raw_begin[b] = begin;
    const uint32_t rank = RAW_MASK >= 0 ? static_cast<uint32_t>(__builtin_popcount(~static_cast<uint32_t>(RAW_MASK) & ((1u << b) - 1u)))
                                        : p.lanes.ans_rank[b];
    CodedLane& c = coded[b];
    c.table = rank * table_size;
    c.ring = rings_address + (static_cast<uint32_t>(warp * ans_lanes) + rank) * kRingBytes;
    c.stage = staging_at + (static_cast<uint32_t>(warp * ans_lanes) + rank) * kBlockElems + lane;
    const int origin = 2 * static_cast<int>(begin & (Ring::kWords - 1));
    c.cursor = origin + 2 * static_cast<int>(end - begin);
    c.chunk = end > begin ? static_cast<int>((end - 1u) >> Ring::kLog) : -1;
    c.refill_at = origin + 2 * static_cast<int>((static_cast<int64_t>(c.chunk) << Ring::kLog) - static_cast<int64_t>(begin));
    c.state = kStateMin;
    if ((raw_mask >> b) & 1u) {
      if (!failure && end - begin != static_cast<uint32_t>((count + 1) >> 1)) failure = EP_STREAM_BAD_RAW_LENGTH;
      raw_near_end = raw_near_end || static_cast<int64_t>(end) + 4 > p.payload_words;
    } else {
      c.state = p.states[(static_cast<int64_t>(rank) * p.tiles + tile) * kNumStates + lane];
    }
  }
  if (failure) {
    if (lane == 0) report(p.error, failure);
    return;
  }
  // Three chunks resident, the fourth on its way.
#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    if ((raw_mask >> b) & 1u) continue;
    const uint32_t ring_address = coded[b].ring;
    Ring::fetch_clipped(p.payload, p.payload_words, ring_address, coded[b].chunk, lane);
    Ring::fetch_clipped(p.payload, p.payload_words, ring_address, coded[b].chunk - 1, lane);
    Ring::fetch_clipped(p.payload, p.payload_words, ring_address, coded[b].chunk - 2, lane);
  }
  ring_commit();
  ring_wait_all();
  __syncwarp();
#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    if ((raw_mask >> b) & 1u) continue;
    Ring::fetch_interior(p.payload, coded[b].ring, coded[b].chunk - 3, lane);
  }
  ring_commit();

  element_t* out = static_cast<element_t*>(p.output) + tile_begin;
  // One decode step of every coded lane for the group at `in_block` (offset inside the staging block).
  // Branch-free: every thread loads a ring word and only the threads that need it merge it in. A
  // single-symbol lane (frequency field 0) runs through the same code: its table yields the right
  // symbol for every slot, its state and cursor become meaningless, all ring reads stay inside the
  // ring, and its final consistency check is skipped.
  auto chain_step = [&](int in_block, auto valid) {
    constexpr bool kWholeGroup = std::is_same<decltype(valid), std::true_type>::value;
#pragma unroll
    for (int b = 0; b < NLANES; ++b) {
      if ((raw_mask >> b) & 1u) continue;
      CodedLane& c = coded[b];
      uint32_t x = c.state;
      if (valid) {
        const uint32_t entry = shared_tables[c.table + (x & slot_mask)];
        shared_bytes[c.stage + in_block] = static_cast<uint8_t>(entry);
        x = (entry >> 20) * ((x >> prob_bits) - 4096u) + (entry >> 8);
      }
      if constexpr (kWholeGroup) {
        renormalize_from_ring<kRingBytes>(x, c.cursor, c.ring, mask_ge);
        c.state = x;
      } else {
        const bool need = valid && x < kStateMin;
        const uint32_t vote = __ballot_sync(0xFFFFFFFFu, need);
        // this thread's word sits 2 * (readers at or above this lane) bytes below the cursor; thread 0 counts every
        // reader, so its position is the cursor for the next step
        const int below = c.cursor - 2 * static_cast<int>(__popc(vote & mask_ge));
        const uint32_t merged = __byte_perm(load_shared_u16((static_cast<uint32_t>(below) & (kRingBytes - 2u)) | c.ring), x, 0x5410);
        c.state = need ? merged : x;
        c.cursor = __shfl_sync(0xFFFFFFFFu, below, 0);
      }
    }
  };
  // Ring upkeep, run once every Ring::kStepsPerUpkeep steps. Three chunks at and below the cursor's chunk are
  // resident and a fourth is in flight; that many steps consume at most one chunk, so at most one chunk
  // boundary is crossed between two calls and every read in between stays inside resident chunks.
  // On a crossing, the chunk requested one crossing ago is made visible to the warp and the next one
  // down is requested into the ring slot that has just been vacated.
  auto ring_upkeep = [&]() {
#pragma unroll
    for (int b = 0; b < NLANES; ++b) {
      if ((raw_mask >> b) & 1u) continue;
      CodedLane& c = coded[b];
      if (c.cursor <= c.refill_at) {
        c.refill_at -= 2 * Ring::kChunk;
        c.chunk -= 1;
        ring_wait_all();
        __syncwarp();
        Ring::fetch_interior(p.payload, c.ring, c.chunk - 3, lane);
        ring_commit();
      }
    }
  };
  // `steps` consecutive full groups ending at offset `first` (the highest group first), then one upkeep
  auto chain_run = [&](int first) {
#pragma unroll
    for (int k = Ring::kStepsPerUpkeep - 1; k >= 0; --k) chain_step(first + 32 * k, std::true_type{});
    ring_upkeep();
  };

  const uint8_t* payload_bytes = reinterpret_cast<const uint8_t*>(p.payload);
  // kGroup elements = 16 bytes of output per thread; needs every tile to start on a 16-byte boundary
  constexpr int kGroup = 16 / NLANES;
  const bool wide = (p.tile_elements % kGroup) == 0;
  for (int block_lo = ((count - 1) / kBlockElems) * kBlockElems; block_lo >= 0; block_lo -= kBlockElems) {
    const int block_hi = min(block_lo + kBlockElems, count);
    const bool full = block_hi - block_lo == kBlockElems;
    // The merge phase below reads this block's raw bytes (512 per raw lane) right after the chain phase; asking L2 for
    // them now takes the DRAM part of that latency off the warp's serial path. Four threads per raw lane, one 128-byte
    // line each (plus one for a stream that straddles a fifth line).
    if (NLANES > 1 && raw_mask != 0u && !(NLANES == 2 && RAW_MASK == 1)) {
#pragma unroll
      for (int b = 0; b < NLANES; ++b) {
        if (((raw_mask >> b) & 1u) && lane < 5u) {
          const uint8_t* line = payload_bytes + 2 * static_cast<int64_t>(raw_begin[b]) + block_lo + static_cast<int>(lane) * 128;
          if (line < payload_bytes + 2 * p.payload_words) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
        }
      }
    }
    // fp16 / bf16 (low byte raw, high byte coded): the block's raw words are asked for here, into registers, and are
    // there when the chain phase is over; no prefetch, no wait in the merge phase.
    constexpr bool kRawAhead = NLANES == 2 && RAW_MASK == 1;
    const bool lean = full && wide && !(raw_near_end && block_hi == count);
    uint32_t ahead[2][3] = {{0u, 0u, 0u}, {0u, 0u, 0u}};
    bool odd_start = false;   // the raw stream starts on an odd 16-bit word: eight bytes then straddle three payload words
    if (kRawAhead && lean) {
      const uint32_t first = raw_begin[0];
      odd_start = first & 1u;
      const uint32_t* const source =
          reinterpret_cast<const uint32_t*>(p.payload) + ((first >> 1) + (static_cast<uint32_t>(block_lo) >> 2) + lane * 2u);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        ahead[half][0] = __ldg(source + 64 * half);
        ahead[half][1] = __ldg(source + 64 * half + 1);
        if (odd_start) ahead[half][2] = __ldg(source + 64 * half + 2);
      }
    }
    // ---- chain phase: groups of 32 symbols, back to front; only the tile's last group can be partial
    if (full) {
      static_assert(kBlockElems % (32 * Ring::kStepsPerUpkeep) == 0, "a staging block is a whole number of runs");
#pragma unroll
      for (int first = kBlockElems - 32 * Ring::kStepsPerUpkeep; first >= 0; first -= 32 * Ring::kStepsPerUpkeep) chain_run(first);
    } else {
      const int tail = (block_hi - block_lo) & 31;
      for (int offset = block_hi - (tail ? tail : 32); offset >= block_lo; offset -= 32) {
        chain_step(offset - block_lo, offset + static_cast<int>(lane) < block_hi);
        ring_upkeep();
      }
    }
    __syncwarp();
    // ---- merge phase: raw bytes + staged symbols -> whole elements
    if (kRawAhead && lean) {
      // a thread makes 8 elements from two of the words it asked for (funnelled out of three where the raw stream starts
      // on an odd 16-bit word) and 8 staged symbols, twice per block
      const uint32_t staged = (coded[NLANES - 1].stage - lane) + lane * 8u;
      uint4* const target = reinterpret_cast<uint4*>(out + block_lo) + lane;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t low = odd_start ? __funnelshift_r(ahead[half][0], ahead[half][1], 16) : ahead[half][0];
        const uint32_t high = odd_start ? __funnelshift_r(ahead[half][1], ahead[half][2], 16) : ahead[half][1];
        const uint2 symbols = *reinterpret_cast<const uint2*>(shared_bytes + staged + 256 * half);
        target[32 * half] = make_uint4(__byte_perm(low, symbols.x, 0x5140), __byte_perm(low, symbols.x, 0x7362),
                                       __byte_perm(high, symbols.y, 0x5140), __byte_perm(high, symbols.y, 0x7362));
      }
    } else if (lean && NLANES == 4 && RAW_MASK == 7) {
      // fp32 with three raw bytes and the top byte coded, written out for the least arithmetic: a thread makes 4 elements
      // from two payload words per raw lane (funnelled by 16 bits where that lane's stream starts on an odd 16-bit word)
      // and 4 staged symbols, four times per block, the loads of two rounds in flight together; every address is one
      // 32-bit index plus literal offsets.
      const uint32_t word = (static_cast<uint32_t>(block_lo) >> 2) + lane;
      const uint32_t* const payload32 = reinterpret_cast<const uint32_t*>(p.payload);
      const uint32_t staged = ((coded[NLANES - 1].stage - lane) >> 2) + lane;   // in 32-bit words
      uint4* const target = reinterpret_cast<uint4*>(out + block_lo) + lane;
#pragma unroll
      for (int pair = 0; pair < 2; ++pair) {
        uint32_t raw[2][3];
#pragma unroll
        for (int b = 0; b < 3; ++b) {
          const uint32_t first = raw_begin[b];
          const uint32_t* const source = payload32 + ((first >> 1) + word + 64u * pair);
          if (first & 1u) {
            const uint32_t a = __ldg(source), a1 = __ldg(source + 1), c = __ldg(source + 32), c1 = __ldg(source + 33);
            raw[0][b] = __funnelshift_r(a, a1, 16);
            raw[1][b] = __funnelshift_r(c, c1, 16);
          } else {
            raw[0][b] = __ldg(source);
            raw[1][b] = __ldg(source + 32);
          }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t symbols = shared_tables[staged + 32 * (2 * pair + k)];
          const uint32_t ab_low = __byte_perm(raw[k][0], raw[k][1], 0x5140);
          const uint32_t ab_high = __byte_perm(raw[k][0], raw[k][1], 0x7362);
          const uint32_t cd_low = __byte_perm(raw[k][2], symbols, 0x5140);
          const uint32_t cd_high = __byte_perm(raw[k][2], symbols, 0x7362);
          target[32 * (2 * pair + k)] = make_uint4(__byte_perm(ab_low, cd_low, 0x5410), __byte_perm(ab_low, cd_low, 0x7632),
                                                   __byte_perm(ab_high, cd_high, 0x5410), __byte_perm(ab_high, cd_high, 0x7632));
        }
      }
    } else if (lean) {
      // Every thread gathers kGroup consecutive bytes of each lane (one vector read of the staging block, or
      // aligned 32-bit loads of the raw stream, shifted by 16 bits where the stream starts on an odd word),
      // transposes them into kGroup whole elements and stores 16 bytes.
      constexpr int kWords = kGroup / 4 > 0 ? kGroup / 4 : 1;   // 32-bit words per lane and thread
#pragma unroll 2
      for (int in_block = static_cast<int>(lane) * kGroup; in_block < kBlockElems; in_block += 32 * kGroup) {
        uint32_t bytes[NLANES][kWords];
#pragma unroll
        for (int b = 0; b < NLANES; ++b) {
          if ((raw_mask >> b) & 1u) {
            const uint32_t first_word = raw_begin[b] + (static_cast<uint32_t>(block_lo + in_block) >> 1);   // 16-bit units
            if (kGroup >= 4) {
              // block_lo + in_block is a multiple of 4, so the stream's first word alone decides the shift
              const uint32_t* aligned = reinterpret_cast<const uint32_t*>(p.payload) + (raw_begin[b] >> 1) +
                                        (static_cast<uint32_t>(block_lo + in_block) >> 2);
              const uint32_t shift = (raw_begin[b] & 1u) << 4;
              uint32_t loaded[kWords + 1];
#pragma unroll
              for (int w = 0; w < kWords; ++w) loaded[w] = __ldg(aligned + w);
              loaded[kWords] = shift ? __ldg(aligned + kWords) : 0u;
#pragma unroll
              for (int w = 0; w < kWords; ++w) bytes[b][w] = __funnelshift_r(loaded[w], loaded[w + 1], shift);
            } else {
              bytes[b][0] = __ldg(p.payload + first_word);
            }
          } else {
            const uint32_t at = (coded[b].stage - lane) + static_cast<uint32_t>(in_block);
            if (kGroup == 16) {
              const uint4 v = *reinterpret_cast<const uint4*>(shared_bytes + at);
              bytes[b][0] = v.x; bytes[b][kWords > 1 ? 1 : 0] = v.y; bytes[b][kWords > 2 ? 2 : 0] = v.z; bytes[b][kWords > 3 ? 3 : 0] = v.w;
            } else if (kGroup == 8) {
              const uint2 v = *reinterpret_cast<const uint2*>(shared_bytes + at);
              bytes[b][0] = v.x; bytes[b][kWords > 1 ? 1 : 0] = v.y;
            } else if (kGroup == 4) {
              bytes[b][0] = shared_tables[at >> 2];
            } else {
              bytes[b][0] = shared_words[at >> 1];
            }
          }
        }
        uint4 packed;
        if (NLANES == 1) {
          packed = make_uint4(bytes[0][0], bytes[0][kWords > 1 ? 1 : 0], bytes[0][kWords > 2 ? 2 : 0], bytes[0][kWords > 3 ? 3 : 0]);
        } else if (NLANES == 2) {
          const uint32_t* a = bytes[0];
          const uint32_t* c = bytes[NLANES > 1 ? 1 : 0];
          packed = make_uint4(__byte_perm(a[0], c[0], 0x5140), __byte_perm(a[0], c[0], 0x7362),
                              __byte_perm(a[kWords > 1 ? 1 : 0], c[kWords > 1 ? 1 : 0], 0x5140),
                              __byte_perm(a[kWords > 1 ? 1 : 0], c[kWords > 1 ? 1 : 0], 0x7362));
        } else if (NLANES == 4) {
          const uint32_t ab_low = __byte_perm(bytes[0][0], bytes[NLANES > 1 ? 1 : 0][0], 0x5140);
          const uint32_t ab_high = __byte_perm(bytes[0][0], bytes[NLANES > 1 ? 1 : 0][0], 0x7362);
          const uint32_t cd_low = __byte_perm(bytes[NLANES > 2 ? 2 : 0][0], bytes[NLANES > 3 ? 3 : 0][0], 0x5140);
          const uint32_t cd_high = __byte_perm(bytes[NLANES > 2 ? 2 : 0][0], bytes[NLANES > 3 ? 3 : 0][0], 0x7362);
          packed = make_uint4(__byte_perm(ab_low, cd_low, 0x5410), __byte_perm(ab_low, cd_low, 0x7632),
                              __byte_perm(ab_high, cd_high, 0x5410), __byte_perm(ab_high, cd_high, 0x7632));
        } else {
          // two 8-byte elements: byte b of element k is byte k of lane b's pair
          uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
          for (int b = 0; b < NLANES; ++b) {
            words[b >> 2] |= (bytes[b][0] & 0xFFu) << (8 * (b & 3));
            words[2 + (b >> 2)] |= ((bytes[b][0] >> 8) & 0xFFu) << (8 * (b & 3));
          }
          packed = make_uint4(words[0], words[1], words[2], words[3]);
        }
        *reinterpret_cast<uint4*>(out + block_lo + in_block) = packed;
      }
    } else {
      // ragged block, tile size that breaks the 16-byte alignment, or end of the payload: one element per thread
      for (int k = static_cast<int>(lane); k < block_hi - block_lo; k += 32) {
        element_t value = 0;
#pragma unroll
        for (int b = 0; b < NLANES; ++b) {
          uint32_t byte;
          if ((raw_mask >> b) & 1u) {
            byte = __ldg(payload_bytes + 2 * static_cast<int64_t>(raw_begin[b]) + block_lo + k);
          } else {
            byte = shared_bytes[(coded[b].stage - lane) + static_cast<uint32_t>(k)];
          }
          value |= static_cast<element_t>(static_cast<element_t>(byte) << (8 * b));
        }
        out[block_lo + k] = value;
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    if (((raw_mask >> b) & 1u) || constant_symbol[b] >= 0) continue;
    const bool dirty = __any_sync(0xFFFFFFFFu, coded[b].state != kStateMin);
    // words left = (cursor - 2 * (stream begin mod ring size)) / 2; the begin is read again rather than kept in a register
    const uint32_t begin = __reduce_min_sync(0xFFFFFFFFu, p.offsets[static_cast<int64_t>(b) * p.tiles + tile]);
    const int left = (coded[b].cursor - 2 * static_cast<int>(begin & (Ring::kWords - 1))) / 2;
    if (left < 0) failure = EP_STREAM_UNDERRUN;
    else if (left != 0 || dirty) failure = EP_STREAM_NOT_CONSUMED;
  }
  if (failure && lane == 0) report(p.error, failure);
}

// ------------------------------------------------------------------------------------------------
// One-byte elements with their single lane coded (fp8, int8, uint8): there is nothing to merge, so
// each step stores its 32 symbols straight to the output (32 consecutive bytes per warp: one full
// sector) and the step shrinks to its chain -- table read, store, multiply-add, renormalisation.
// Runs of Ring::kStepsPerUpkeep steps are written out with the stores at literal offsets from one
// base pointer per run. Needs tiles of whole 32-byte groups (tile_elements a multiple of 32).
// ------------------------------------------------------------------------------------------------
template <int OFFSET>
__device__ __forceinline__ void store_low_byte(uint8_t* base, uint32_t value) {
  asm volatile("st.global.u8 [%0 + %1], %2;" ::"l"(base), "n"(OFFSET), "r"(value) : "memory");
}

template <int CHUNK_LOG>
__global__ void __launch_bounds__(kByteWarps * 32, kByteBlocksPerSm) tile_ans_decode_bytes_kernel(const DecodeParams p) {
  using Ring = WordRing<CHUNK_LOG>;
  static_assert(Ring::kStepsPerUpkeep == 4 || Ring::kStepsPerUpkeep == 8, "runs are written out for four or eight steps");
  extern __shared__ __align__(16) uint32_t shared_tables[];
  __shared__ int constant_symbol[kMaxLanes];
  const uint32_t table_size = 1u << p.prob_bits;
  stage_decode_tables<1>(p, shared_tables, constant_symbol);

  const int warp = threadIdx.x >> 5;
  const int64_t tile = p.first_tile + static_cast<int64_t>(blockIdx.x) * kByteWarps + warp;
  if (tile >= p.tile_end) return;
  const uint32_t lane = lane_id();
  const uint32_t mask_ge = lanemask_ge();
  const uint32_t slot_mask = table_size - 1u;
  const int prob_bits = p.prob_bits;
  const int64_t tile_begin = tile * p.tile_elements;
  const int count = static_cast<int>(min(p.tile_elements, p.num_elements - tile_begin));
  const uint32_t shared_base = static_cast<uint32_t>(__cvta_generic_to_shared(shared_tables));
  const uint32_t ring = ((shared_base + table_size * 4u + Ring::kBytes - 1u) & ~(Ring::kBytes - 1u)) + static_cast<uint32_t>(warp) * Ring::kBytes;

  // through a warp reduction: the compiler then knows the bounds, and the cursor arithmetic built on them, to be
  // the same in all 32 threads
  const uint32_t begin = __reduce_min_sync(0xFFFFFFFFu, p.offsets[tile]);
  const uint32_t end = __reduce_min_sync(0xFFFFFFFFu, p.offsets[tile + 1]);
  if (end < begin || static_cast<int64_t>(end) > p.payload_words) {
    if (lane == 0) report(p.error, EP_STREAM_BAD_OFFSETS);
    return;
  }
  uint32_t x = p.states[tile * kNumStates + lane];
  const int origin = 2 * static_cast<int>(begin & (Ring::kWords - 1));
  int cursor = origin + 2 * static_cast<int>(end - begin);
  int chunk = end > begin ? static_cast<int>((end - 1u) >> Ring::kLog) : -1;
  int refill_at = origin + 2 * static_cast<int>((static_cast<int64_t>(chunk) << Ring::kLog) - static_cast<int64_t>(begin));
  // three chunks resident, the fourth on its way
  Ring::fetch_clipped(p.payload, p.payload_words, ring, chunk, lane);
  Ring::fetch_clipped(p.payload, p.payload_words, ring, chunk - 1, lane);
  Ring::fetch_clipped(p.payload, p.payload_words, ring, chunk - 2, lane);
  ring_commit();
  ring_wait_all();
  __syncwarp();
  Ring::fetch_interior(p.payload, ring, chunk - 3, lane);
  ring_commit();

  const auto upkeep = [&]() {
    if (__any_sync(0xFFFFFFFFu, cursor <= refill_at)) {   // the same in every thread; the vote tells the compiler so
      refill_at -= 2 * Ring::kChunk;
      chunk -= 1;
      ring_wait_all();
      __syncwarp();
      Ring::fetch_interior(p.payload, ring, chunk - 3, lane);
      ring_commit();
    }
  };
  uint8_t* const out = static_cast<uint8_t*>(p.output) + tile_begin + lane;
  // a single group, possibly partial (the tensor's last tile), with its own upkeep
  const auto single_step = [&](int offset, bool valid) {
    if (valid) {
      const uint32_t entry = shared_tables[x & slot_mask];
      out[offset] = static_cast<uint8_t>(entry);
      x = (entry >> 20) * ((x >> prob_bits) - 4096u) + (entry >> 8);
    }
    const bool need = valid && x < kStateMin;
    const uint32_t vote = __ballot_sync(0xFFFFFFFFu, need);
    const int below = cursor - 2 * static_cast<int>(__popc(vote & mask_ge));
    const uint32_t merged = __byte_perm(load_shared_u16((static_cast<uint32_t>(below) & (Ring::kBytes - 2u)) | ring), x, 0x5410);
    x = need ? merged : x;
    cursor = __shfl_sync(0xFFFFFFFFu, below, 0);
    upkeep();
  };
  int offset = count;
  if (count & 31) {
    offset -= count & 31;
    single_step(offset, lane < static_cast<uint32_t>(count & 31));
  }
  constexpr int kRun = 32 * Ring::kStepsPerUpkeep;
  while (offset % kRun) {
    offset -= 32;
    single_step(offset, true);
  }
#define EP_BYTE_STEP(K)                                                        \
  {                                                                            \
    const uint32_t entry = shared_tables[x & slot_mask];                       \
    store_low_byte<(K) * 32>(run, entry);                                      \
    x = (entry >> 20) * ((x >> prob_bits) - 4096u) + (entry >> 8);             \
    renormalize_from_ring<Ring::kBytes>(x, cursor, ring, mask_ge);             \
  }
  uint8_t* run = out + offset;
  while (offset > 0) {
    offset -= kRun;
    run -= kRun;
    if (Ring::kStepsPerUpkeep == 8) {
      EP_BYTE_STEP(7) EP_BYTE_STEP(6) EP_BYTE_STEP(5) EP_BYTE_STEP(4)
    }
    EP_BYTE_STEP(3) EP_BYTE_STEP(2) EP_BYTE_STEP(1) EP_BYTE_STEP(0)
    upkeep();
  }
#undef EP_BYTE_STEP

  if (constant_symbol[0] < 0) {
    const bool dirty = __any_sync(0xFFFFFFFFu, x != kStateMin);
    const int left = (cursor - origin) / 2;
    int failure = 0;
    if (left < 0) failure = EP_STREAM_UNDERRUN;
    else if (left != 0 || dirty) failure = EP_STREAM_NOT_CONSUMED;
    if (failure && lane == 0) report(p.error, failure);
  }
}

// ------------------------------------------------------------------------------------------------
// Histogram: one private 256-bin table per (warp, byte lane) in shared memory, folded per block.
// ------------------------------------------------------------------------------------------------
template <int NLANES>
__global__ void __launch_bounds__(kThreads) tile_ans_histogram_kernel(const uint8_t* __restrict__ input, int64_t num_elements,
                                                                      unsigned long long* __restrict__ histograms) {
  using element_t = typename Element<NLANES>::type;
  // 8 lanes x 8 copies would pass the 48 KB static limit, so wide elements share a copy per warp pair
  constexpr int kCopies = NLANES == 8 ? kWarps / 2 : kWarps;
  __shared__ uint32_t bins[kCopies][NLANES][256];
  uint32_t* flat = &bins[0][0][0];
  for (int i = threadIdx.x; i < kCopies * NLANES * 256; i += kThreads) flat[i] = 0;
  __syncthreads();
  const int warp = (threadIdx.x >> 5) % kCopies;
  const element_t* elements = reinterpret_cast<const element_t*>(input);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; e < num_elements; e += stride) {
    const element_t value = elements[e];
#pragma unroll
    for (int b = 0; b < NLANES; ++b) atomicAdd(&bins[warp][b][(value >> (8 * b)) & 0xFF], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < NLANES * 256; i += kThreads) {
    uint32_t sum = 0;
#pragma unroll
    for (int w = 0; w < kCopies; ++w) sum += flat[w * NLANES * 256 + i];
    if (sum) atomicAdd(histograms + i, static_cast<unsigned long long>(sum));
  }
}

// ------------------------------------------------------------------------------------------------
// Encode
// ------------------------------------------------------------------------------------------------
struct EncodeParams {
  const void* input;
  int64_t num_elements;
  int64_t tile_elements;
  int64_t tiles;
  int prob_bits;
  const uint16_t* frequencies;  // [lanes][256]
  const uint16_t* cdfs;         // [lanes][256]
  LaneSetup lanes;
  uint16_t* scratch;            // [lanes * tiles][tile_elements]
  uint32_t* word_counts;        // [lanes * tiles]
  uint32_t* states;             // [ans_lanes * tiles][32]
};

// Per coded lane and symbol: .x = frequency | cdf << 16, .y = floor(2^32 / frequency) (frequency 1
// is stored as 0xFFFFFFFF; the correction step below absorbs the off-by-one either way).
template <int NLANES>
__global__ void __launch_bounds__(kThreads) tile_ans_encode_kernel(const EncodeParams p) {
  using element_t = typename Element<NLANES>::type;
  __shared__ uint2 symbol_table[NLANES][256];
  for (int i = threadIdx.x; i < NLANES * 256; i += kThreads) {
    const uint32_t f = p.frequencies[i];
    const uint32_t c = p.cdfs[i];
    const uint32_t reciprocal = f > 1u ? static_cast<uint32_t>(0x100000000ull / f) : 0xFFFFFFFFu;
    (&symbol_table[0][0])[i] = make_uint2(f | (c << 16), reciprocal);
  }
  __syncthreads();

  const int64_t tile = static_cast<int64_t>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (tile >= p.tiles) return;
  const uint32_t lane = lane_id();
  const uint32_t mask_lt = lanemask_lt();
  const int64_t tile_begin = tile * p.tile_elements;
  const int count = static_cast<int>(min(p.tile_elements, p.num_elements - tile_begin));
  const element_t* in = static_cast<const element_t*>(p.input) + tile_begin;
  const uint32_t emit_shift = 31 - p.prob_bits;

  uint16_t* slot[NLANES];
  uint32_t state[NLANES];
  uint32_t emitted[NLANES];
#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    slot[b] = p.scratch + (static_cast<int64_t>(b) * p.tiles + tile) * p.tile_elements;
    state[b] = kStateMin;
    emitted[b] = 0;
  }

  for (int base = 0; base < count; base += 32) {
    const bool valid = base + static_cast<int>(lane) < count;
    const element_t value = valid ? in[base + lane] : element_t(0);
#pragma unroll
    for (int b = 0; b < NLANES; ++b) {
      const uint32_t symbol = static_cast<uint32_t>(value >> (8 * b)) & 0xFFu;
      if ((p.lanes.raw_mask >> b) & 1u) {
        // a raw stream is the lane's bytes in element order (two per little-endian word)
        if (valid) reinterpret_cast<uint8_t*>(slot[b])[base + lane] = static_cast<uint8_t>(symbol);
        continue;
      }
      const uint2 info = symbol_table[b][symbol];
      const uint32_t f = info.x & 0xFFFFu;
      uint32_t x = state[b];
      const bool emit = valid && x >= (f << emit_shift);
      const uint32_t vote = __ballot_sync(0xFFFFFFFFu, emit);
      if (emit) {
        slot[b][emitted[b] + __popc(vote & mask_lt)] = static_cast<uint16_t>(x);
        x >>= 16;
      }
      emitted[b] += __popc(vote);
      if (valid) {
        uint32_t q = __umulhi(x, info.y);
        uint32_t r = x - q * f;
        if (r >= f) {
          r -= f;
          q += 1;
        }
        state[b] = (q << p.prob_bits) + r + (info.x >> 16);
      }
    }
  }

#pragma unroll
  for (int b = 0; b < NLANES; ++b) {
    const int64_t stream = static_cast<int64_t>(b) * p.tiles + tile;
    if ((p.lanes.raw_mask >> b) & 1u) {
      if (lane == 0) {
        if (count & 1) reinterpret_cast<uint8_t*>(slot[b])[count] = 0;
        p.word_counts[stream] = static_cast<uint32_t>((count + 1) >> 1);
      }
    } else {
      p.states[(static_cast<int64_t>(p.lanes.ans_rank[b]) * p.tiles + tile) * kNumStates + lane] = state[b];
      if (lane == 0) p.word_counts[stream] = emitted[b];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Exclusive scan of u32 counts (single block, sequential over 1024-wide chunks) and stream gather.
// ------------------------------------------------------------------------------------------------
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads) exclusive_scan_u32_kernel(const uint32_t* __restrict__ counts, int64_t count,
                                                                          uint32_t* __restrict__ offsets,
                                                                          unsigned long long* __restrict__ total) {
  __shared__ unsigned long long warp_sums[32];
  __shared__ unsigned long long carry_shared;
  const uint32_t lane = lane_id();
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_shared = 0;
  __syncthreads();
  for (int64_t base = 0; base < count; base += kScanThreads) {
    const int64_t index = base + threadIdx.x;
    const unsigned long long own = index < count ? counts[index] : 0ull;
    unsigned long long inclusive = own;
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
      const unsigned long long below = __shfl_up_sync(0xFFFFFFFFu, inclusive, step);
      if (lane >= static_cast<uint32_t>(step)) inclusive += below;
    }
    if (lane == 31) warp_sums[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
      unsigned long long sum = warp_sums[lane];
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const unsigned long long below = __shfl_up_sync(0xFFFFFFFFu, sum, step);
        if (lane >= static_cast<uint32_t>(step)) sum += below;
      }
      warp_sums[lane] = sum;
    }
    __syncthreads();
    const unsigned long long carry = carry_shared;
    const unsigned long long before = carry + (warp > 0 ? warp_sums[warp - 1] : 0ull) + inclusive - own;
    if (index < count) offsets[index] = static_cast<uint32_t>(before);
    __syncthreads();
    if (threadIdx.x == kScanThreads - 1) carry_shared = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    offsets[count] = static_cast<uint32_t>(carry_shared);
    total[0] = carry_shared;
  }
}

__global__ void __launch_bounds__(kThreads) compact_streams_kernel(const uint16_t* __restrict__ scratch,
                                                                   const uint32_t* __restrict__ offsets,
                                                                   uint16_t* __restrict__ payload, int64_t slot_words,
                                                                   int64_t streams) {
  for (int64_t stream = blockIdx.x; stream < streams; stream += gridDim.x) {
    const uint32_t begin = offsets[stream];
    const uint32_t words = offsets[stream + 1] - begin;
    const uint16_t* source = scratch + stream * slot_words;
    uint16_t* target = payload + begin;
    // 32-bit body between 4-byte-aligned ends; the slot base is 4-byte aligned when slot_words is even
    const uint32_t head = (begin & 1u) && words ? 1u : 0u;
    if (head && threadIdx.x == 0) target[0] = source[0];
    if ((slot_words & 1) == 0 && head == 0) {
      const uint32_t pairs = words >> 1;
      const uint32_t* source32 = reinterpret_cast<const uint32_t*>(source);
      uint32_t* target32 = reinterpret_cast<uint32_t*>(target);
      for (uint32_t i = threadIdx.x; i < pairs; i += kThreads) target32[i] = source32[i];
      if ((words & 1u) && threadIdx.x == 0) target[words - 1] = source[words - 1];
    } else {
      for (uint32_t i = head + threadIdx.x; i < words; i += kThreads) target[i] = source[i];
    }
  }
}

int make_lane_setup(const uint8_t* lane_modes_host, int num_lanes, LaneSetup* setup) {
  if (lane_modes_host == nullptr) return EP_ERR_INVALID_ARGUMENT;
  if (num_lanes != 1 && num_lanes != 2 && num_lanes != 4 && num_lanes != 8) return EP_ERR_UNSUPPORTED;
  setup->raw_mask = 0;
  setup->ans_lanes = 0;
  for (int b = 0; b < kMaxLanes; ++b) setup->ans_rank[b] = 0;
  for (int b = 0; b < num_lanes; ++b) {
    if (lane_modes_host[b] > 1) return EP_ERR_INVALID_ARGUMENT;
    if (lane_modes_host[b] == 1) {
      setup->raw_mask |= 1u << b;
    } else {
      setup->ans_rank[b] = static_cast<uint8_t>(setup->ans_lanes++);
    }
  }
  return EP_OK;
}

template <typename Kernel>
int allow_shared(Kernel kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    EP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  }
  return EP_OK;
}

// Shared memory of one block of the staged decoder.
template <int CHUNK_LOG>
size_t staged_shared_bytes(size_t table_bytes, int ans_lanes, int warps) {
  const size_t per_warp_lane = WordRing<CHUNK_LOG>::kBytes + kBlockElems;
  // one ring's worth of padding lets the kernel align the rings to their own size
  return table_bytes + WordRing<CHUNK_LOG>::kBytes + static_cast<size_t>(warps) * ans_lanes * per_warp_lane;
}

template <int NLANES, int RAW_MASK, int CHUNK_LOG, int WARPS>
int launch_staged(const DecodeParams& p, size_t shared, cudaStream_t stream) {
  const int rc = allow_shared(tile_ans_decode_kernel<NLANES, RAW_MASK, CHUNK_LOG, WARPS>, shared);
  if (rc != EP_OK) return rc;
  const int64_t tiles = p.tile_end - p.first_tile;
  const dim3 grid(static_cast<unsigned>((tiles + WARPS - 1) / WARPS));
  tile_ans_decode_kernel<NLANES, RAW_MASK, CHUNK_LOG, WARPS><<<grid, WARPS * 32, shared, stream>>>(p);
  return EP_OK;
}

// `blocks` blocks of `bytes` shared memory each fit one SM (227 KB, 1 KB of it reserved per block, plus the kernels'
// static words)
inline bool fits_sm(size_t bytes, int blocks) { return (bytes + 1024 + 512) * blocks <= 227 * 1024; }

// Block shape and ring of the staged decoder for one lane pattern: fourteen warps and 256-word chunks where four such
// blocks fit an SM, else eight warps with 256-word chunks where seven fit, else eight warps and 128-word chunks.
// Four-byte elements measured no better with the wider chunks and keep eight warps and 128 words.
template <int NLANES, int RAW_MASK>
int launch_staged_shape(const DecodeParams& p, size_t table_bytes, cudaStream_t stream) {
  const int lanes = p.lanes.ans_lanes;
  if (NLANES <= 2) {
    const size_t big = staged_shared_bytes<8>(table_bytes, lanes, kByteWarps);
    if (fits_sm(big, kByteBlocksPerSm)) return launch_staged<NLANES, RAW_MASK, 8, kByteWarps>(p, big, stream);
    const size_t wide = staged_shared_bytes<8>(table_bytes, lanes, kWarps);
    if (fits_sm(wide, kDecodeBlocksPerSm)) return launch_staged<NLANES, RAW_MASK, 8, kWarps>(p, wide, stream);
  }
  if (NLANES == 4 && RAW_MASK == 7) {
    // fp32 with its top byte coded: 14-warp blocks as well (a table staged for 14 tiles, four copies an SM), 128-word chunks
    const size_t tall = staged_shared_bytes<7>(table_bytes, lanes, kByteWarps);
    if (fits_sm(tall, kByteBlocksPerSm)) return launch_staged<NLANES, RAW_MASK, 7, kByteWarps>(p, tall, stream);
  }
  return launch_staged<NLANES, RAW_MASK, 7, kWarps>(p, staged_shared_bytes<7>(table_bytes, lanes, kWarps), stream);
}

template <int NLANES>
int launch_decode(const DecodeParams& p, dim3 grid, size_t table_bytes, bool staged, cudaStream_t stream) {
  if (staged && NLANES == 1 && p.lanes.raw_mask == 0u && p.tile_elements % 32 == 0) {
    // one coded byte lane in tiles of whole 32-byte groups: the dedicated kernel (rings only, no staging block), 14
    // tiles to a block; 16 KB of table and 30 KB of rings at most, four blocks to an SM
    const size_t shared = table_bytes + WordRing<8>::kBytes * (kByteWarps + 1);
    const int64_t tiles = p.tile_end - p.first_tile;
    const dim3 byte_grid(static_cast<unsigned>((tiles + kByteWarps - 1) / kByteWarps));
    const int rc = allow_shared(tile_ans_decode_bytes_kernel<8>, shared);
    if (rc != EP_OK) return rc;
    tile_ans_decode_bytes_kernel<8><<<byte_grid, kByteWarps * 32, shared, stream>>>(p);
    return EP_OK;
  }
  if (staged) {
    // common patterns get their own instantiation: everything coded, or only the top byte coded
    constexpr int top_only = (1 << (NLANES - 1)) - 1;
    if (p.lanes.raw_mask == 0u && NLANES <= 2) return launch_staged_shape<NLANES, 0>(p, table_bytes, stream);
    if (NLANES > 1 && p.lanes.raw_mask == static_cast<uint32_t>(top_only)) return launch_staged_shape<NLANES, top_only>(p, table_bytes, stream);
    return launch_staged_shape<NLANES, -1>(p, table_bytes, stream);
  } else {
    const int rc = allow_shared(tile_ans_decode_simple_kernel<NLANES>, table_bytes);
    if (rc != EP_OK) return rc;
    tile_ans_decode_simple_kernel<NLANES><<<grid, kThreads, table_bytes, stream>>>(p);
  }
  return EP_OK;
}

}  // namespace
}  // namespace ep

using namespace ep;

extern "C" int ep_tile_ans_decode_tiles(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                                        const uint32_t* states_dev, const uint32_t* decode_tables_dev,
                                        const uint8_t* lane_modes_host, void* output_dev, int64_t num_elements,
                                        int64_t tile_elements, int prob_bits, int num_lanes, int64_t first_tile,
                                        int64_t tile_count, int* error_dev, ep_stream_t stream) {
  if (num_elements <= 0 || tile_elements <= 0 || tile_elements > 0x7FFFFFFF || prob_bits < 9 || prob_bits > 12 ||
      payload_words < 0 || offsets_dev == nullptr || output_dev == nullptr) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  DecodeParams p;
  const int status = make_lane_setup(lane_modes_host, num_lanes, &p.lanes);
  if (status != EP_OK) return status;
  if (p.lanes.ans_lanes > 0 && (states_dev == nullptr || decode_tables_dev == nullptr)) return EP_ERR_INVALID_ARGUMENT;
  if (payload_words > 0 && payload_dev == nullptr) return EP_ERR_INVALID_ARGUMENT;
  p.payload = payload_dev;
  p.payload_words = payload_words;
  p.offsets = offsets_dev;
  p.states = states_dev;
  p.tables = decode_tables_dev;
  p.output = output_dev;
  p.num_elements = num_elements;
  p.tile_elements = tile_elements;
  p.tiles = (num_elements + tile_elements - 1) / tile_elements;
  if (first_tile < 0 || tile_count < 0 || first_tile > p.tiles || tile_count > p.tiles - first_tile) return EP_ERR_INVALID_ARGUMENT;
  if (tile_count == 0) return EP_OK;
  p.first_tile = first_tile;
  p.tile_end = first_tile + tile_count;
  p.prob_bits = prob_bits;
  p.error = error_dev;
  const int64_t blocks = (tile_count + kWarps - 1) / kWarps;
  if (blocks > 0x7FFFFFFF) return EP_ERR_TOO_LARGE;
  const size_t table_bytes = static_cast<size_t>(p.lanes.ans_lanes) * sizeof(uint32_t) << prob_bits;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(blocks));
  // The staged decoder needs 16-byte aligned payload and output and an even tile size; anything else
  // takes the general kernel.
  const bool staged = (tile_elements & 1) == 0 && (reinterpret_cast<uintptr_t>(payload_dev) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(output_dev) & 15u) == 0;
  int rc = EP_OK;
  switch (num_lanes) {
    case 1: rc = launch_decode<1>(p, grid, table_bytes, staged, s); break;
    case 2: rc = launch_decode<2>(p, grid, table_bytes, staged, s); break;
    case 4: rc = launch_decode<4>(p, grid, table_bytes, staged, s); break;
    default: rc = launch_decode<8>(p, grid, table_bytes, staged, s); break;
  }
  if (rc != EP_OK) return rc;
  return check_launch("tile_ans_decode_kernel");
}

extern "C" int ep_tile_ans_decode(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                                  const uint32_t* states_dev, const uint32_t* decode_tables_dev,
                                  const uint8_t* lane_modes_host, void* output_dev, int64_t num_elements,
                                  int64_t tile_elements, int prob_bits, int num_lanes, int* error_dev, ep_stream_t stream) {
  if (num_elements <= 0 || tile_elements <= 0) return EP_ERR_INVALID_ARGUMENT;
  const int64_t tiles = (num_elements + tile_elements - 1) / tile_elements;
  return ep_tile_ans_decode_tiles(payload_dev, payload_words, offsets_dev, states_dev, decode_tables_dev, lane_modes_host,
                                  output_dev, num_elements, tile_elements, prob_bits, num_lanes, 0, tiles, error_dev, stream);
}

extern "C" int ep_tile_ans_histogram(const void* input_dev, int64_t num_elements, int num_lanes, uint64_t* histograms_dev,
                                     ep_stream_t stream) {
  if (input_dev == nullptr || histograms_dev == nullptr || num_elements <= 0) return EP_ERR_INVALID_ARGUMENT;
  if (num_lanes != 1 && num_lanes != 2 && num_lanes != 4 && num_lanes != 8) return EP_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EP_CUDA_CHECK(cudaMemsetAsync(histograms_dev, 0, sizeof(uint64_t) * 256 * num_lanes, s));
  const int64_t wanted = (num_elements + kThreads - 1) / kThreads;
  const int per_sm = num_lanes >= 8 ? 3 : (num_lanes == 4 ? 6 : 8);
  const unsigned blocks = static_cast<unsigned>(wanted < kSmCount * per_sm ? wanted : kSmCount * per_sm);
  auto* out = reinterpret_cast<unsigned long long*>(histograms_dev);
  const auto* in = static_cast<const uint8_t*>(input_dev);
  switch (num_lanes) {
    case 1: tile_ans_histogram_kernel<1><<<blocks, kThreads, 0, s>>>(in, num_elements, out); break;
    case 2: tile_ans_histogram_kernel<2><<<blocks, kThreads, 0, s>>>(in, num_elements, out); break;
    case 4: tile_ans_histogram_kernel<4><<<blocks, kThreads, 0, s>>>(in, num_elements, out); break;
    default: tile_ans_histogram_kernel<8><<<blocks, kThreads, 0, s>>>(in, num_elements, out); break;
  }
  return check_launch("tile_ans_histogram_kernel");
}

extern "C" int ep_tile_ans_encode(const void* input_dev, int64_t num_elements, int num_lanes, int64_t tile_elements,
                                  int prob_bits, const uint16_t* frequencies_dev, const uint16_t* cdfs_dev,
                                  const uint8_t* lane_modes_host, uint16_t* scratch_dev, uint32_t* word_counts_dev,
                                  uint32_t* states_dev, ep_stream_t stream) {
  if (input_dev == nullptr || num_elements <= 0 || tile_elements <= 0 || tile_elements > 0x7FFFFFFF || prob_bits < 9 ||
      prob_bits > 12 || frequencies_dev == nullptr || cdfs_dev == nullptr || scratch_dev == nullptr ||
      word_counts_dev == nullptr) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  EncodeParams p;
  const int status = make_lane_setup(lane_modes_host, num_lanes, &p.lanes);
  if (status != EP_OK) return status;
  if (p.lanes.ans_lanes > 0 && states_dev == nullptr) return EP_ERR_INVALID_ARGUMENT;
  p.input = input_dev;
  p.num_elements = num_elements;
  p.tile_elements = tile_elements;
  p.tiles = (num_elements + tile_elements - 1) / tile_elements;
  p.prob_bits = prob_bits;
  p.frequencies = frequencies_dev;
  p.cdfs = cdfs_dev;
  p.scratch = scratch_dev;
  p.word_counts = word_counts_dev;
  p.states = states_dev;
  const int64_t blocks = (p.tiles + kWarps - 1) / kWarps;
  if (blocks > 0x7FFFFFFF) return EP_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(blocks));
  switch (num_lanes) {
    case 1: tile_ans_encode_kernel<1><<<grid, kThreads, 0, s>>>(p); break;
    case 2: tile_ans_encode_kernel<2><<<grid, kThreads, 0, s>>>(p); break;
    case 4: tile_ans_encode_kernel<4><<<grid, kThreads, 0, s>>>(p); break;
    default: tile_ans_encode_kernel<8><<<grid, kThreads, 0, s>>>(p); break;
  }
  return check_launch("tile_ans_encode_kernel");
}

extern "C" int ep_exclusive_scan_u32(const uint32_t* counts_dev, int64_t count, uint32_t* offsets_dev, uint64_t* total_dev,
                                     ep_stream_t stream) {
  if (counts_dev == nullptr || offsets_dev == nullptr || total_dev == nullptr || count < 0) return EP_ERR_INVALID_ARGUMENT;
  exclusive_scan_u32_kernel<<<1, kScanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      counts_dev, count, offsets_dev, reinterpret_cast<unsigned long long*>(total_dev));
  return check_launch("exclusive_scan_u32_kernel");
}

extern "C" int ep_compact_streams(const uint16_t* scratch_dev, const uint32_t* offsets_dev, uint16_t* payload_dev,
                                  int64_t slot_words, int64_t streams, ep_stream_t stream) {
  if (scratch_dev == nullptr || offsets_dev == nullptr || slot_words <= 0 || streams <= 0) return EP_ERR_INVALID_ARGUMENT;
  if (payload_dev == nullptr) return EP_ERR_INVALID_ARGUMENT;
  const int64_t wanted = streams < kSmCount * 8 ? streams : kSmCount * 8;
  compact_streams_kernel<<<static_cast<unsigned>(wanted), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      scratch_dev, offsets_dev, payload_dev, slot_words, streams);
  return check_launch("compact_streams_kernel");
}
