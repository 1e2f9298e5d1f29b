// DFloat11 (Huffman-coded bf16 exponents + raw sign/mantissa byte) for sm_100a.
//
// Format (entropack/schemes/dfloat11/format.py:32-63, eager.py:72-198): the exponent byte of every bf16
// value is Huffman coded MSB-first into `encoded_exponent`; the other eight bits travel raw in
// `sign_mantissa`. The stream is cut into regions of `bytes_per_thread` bytes, `threads_per_block`
// regions to a block; thread_meta[r] = gap << 11 | count gives, for region r, the bit offset of the first
// codeword that starts there and how many start there; output_positions[b] is the first element of
// block b. luts[k] are 256-entry byte tables (entry = symbol, or 256 - child level), the last row is the
// code length per symbol.
//
// Decode, two kernels, one thread per region in both. Block kernel (a container's first decode, and layouts the other
// one does not take): a CUDA block serves up to four blocks of the format; their bytes are staged once into shared
// memory as big-endian words, the LUT levels are fused with the length row into 16-bit entries (one shared load per
// level), each thread walks its codewords with a two-word register window, symbols go to a shared staging array and
// leave as coalesced 16-byte bf16 stores merged with sign_mantissa. Warp kernel (later decodes, with the tables an
// earlier call built and kept): the unit of work is a run of 32 regions, a warp to each, persistent blocks, inputs by
// bulk copies asked for ahead of their use; described in front of it below.
//
// Encode: two passes over the input. Pass 1 sums code lengths per chunk of 1024 elements; a scan gives
// every chunk its bit offset; pass 2 re-reads the chunk, places every codeword with at most three
// atomicOr on 32-bit words (big-endian bit order), splits off sign_mantissa, and derives the region and
// block metadata from the same bit positions.
#include "ep_common.cuh"

#include <algorithm>

namespace ep {
namespace {

constexpr int kMaxLevels = 64;
constexpr uint32_t kPointerFlag = 0x8000u;
// Multi-symbol table: indexed by the next MULTI_BITS bits of the stream, a 64-bit entry holds up to four whole codewords
// that fit in those bits: .x = their symbols, one per byte; .y = the bits consumed after none (zero), one, two, three
// and four of them in five 4-bit fields, and their number in bits 24-26 (0: the first codeword is longer than the
// window or than a level-0 look-up, take the one-symbol path). A thread with fewer symbols left than the entry holds
// takes only those and advances by the field of that number, so neither the end of a region nor a finished thread
// needs a path of its own. Exponent codes average under three
// bits, so most look-ups deliver three or four symbols. The table is built inside the kernel with a 10-bit window, or
// once per container with an 11-bit window (ep_dfloat11_build_decode_tables) and copied in by every later decode.
constexpr int kBuiltMultiBits = 10;
constexpr int kKeptMultiBits = 11;
constexpr int kMaxFormatBlocks = 4;   // blocks of the format served by one CUDA block, at most
// The warp-per-unit kernel: two blocks of up to 20 warps to an SM, the most that 48 registers a thread allow. What a
// warp does is a chain of dependent steps, so throughput comes from the number of warps in flight.
constexpr int kWarpKernelBlocksPerSm = 2;
constexpr int kWarpKernelMaxWarps = 20;

__device__ __forceinline__ uint32_t byte_swap(uint32_t x) { return __byte_perm(x, 0, 0x0123); }

__device__ __forceinline__ uint64_t pack_bf16x4(uint32_t exponents, uint32_t sign_mantissa) {
  // per byte: bits = (sm & 0x80) << 8 | exp << 7 | (sm & 0x7F)
  const uint32_t low = ((exponents & 0x01010101u) << 7) | (sign_mantissa & 0x7F7F7F7Fu);   // low bytes of the 4 values
  const uint32_t high = (sign_mantissa & 0x80808080u) | ((exponents >> 1) & 0x7F7F7F7Fu);  // high bytes
  return static_cast<uint64_t>(__byte_perm(low, high, 0x5140)) | (static_cast<uint64_t>(__byte_perm(low, high, 0x7362)) << 32);
}

struct DecodeParams {
  const uint8_t* luts;
  const uint8_t* encoded;
  const uint8_t* sign_mantissa;
  const uint32_t* output_positions;
  const uint16_t* thread_meta;
  uint16_t* out;
  int64_t n_bytes;
  int64_t n_elements;
  int num_luts;
  int bytes_per_thread;
  int threads_per_block;
  int stage_elems;
  int64_t blocks;   // blocks of the format (threads_per_block regions each)
  int groups;       // how many of them one CUDA block serves
  int* error;
  const uint32_t* kept_tables;   // fused level tables + multi-symbol table as an earlier launch exported them, or null
  int64_t units;                 // warp kernel: runs of 32 regions in the whole stream
  int units_per_block;           // warp kernel: runs per block of the format
  int stage_alloc;               // warp kernel: elements a warp's shared slices hold
  uint32_t* export_tables;       // EXPORT: where the freshly built tables go
};

// Words of the fused level tables (u16[levels][256], padded to 16 bytes) in front of the multi-symbol table.
__host__ __device__ inline uint32_t level_table_words(int levels) { return (static_cast<uint32_t>(levels) * 128u + 3u) & ~3u; }

template <int MULTI_BITS, bool EXPORT>
__global__ void __launch_bounds__(1024) dfloat11_decode_kernel(const DecodeParams p) {
  constexpr int kMultiBits = MULTI_BITS;
  constexpr int kMultiEntries = 1 << MULTI_BITS;
  extern __shared__ __align__(16) uint32_t shared[];
  // A CUDA block serves `p.groups` consecutive blocks of the format side by side, one per group of `group_threads`
  // threads, so that the code tables are staged and the multi-symbol table built once for all of them.
  // layout: fused tables u16[levels][256] | multi-symbol table u32[1024] | scan u32[kMaxFormatBlocks][32] |
  //         per group: stream words u32[block_words] | exponents u8[stage_bytes]
  const int levels = p.num_luts - 1;
  uint16_t* const tables = reinterpret_cast<uint16_t*>(shared);
  uint2* const multi = reinterpret_cast<uint2*>(shared + level_table_words(levels));
  uint32_t* const scan_base = reinterpret_cast<uint32_t*>(multi + kMultiEntries);
  const int block_bytes = p.bytes_per_thread * p.threads_per_block;
  const int block_words = ((block_bytes + 3) / 4 + 3) & ~1;  // two look-ahead words, even count keeps what follows 8-byte aligned
  const int stage_bytes = (p.stage_elems + 16 + 15) & ~15;
  const int group_threads = blockDim.x / p.groups;           // a multiple of 32
  const int group = threadIdx.x / group_threads;
  const int member = threadIdx.x - group * group_threads;     // this thread's index inside its format block
  const int64_t format_block = static_cast<int64_t>(blockIdx.x) * p.groups + group;
  const bool present = format_block < p.blocks;               // the last CUDA block may have idle groups
  uint32_t* const scan = scan_base + group * 32;
  uint32_t* const words = scan_base + kMaxFormatBlocks * 32 + group * (block_words + stage_bytes / 4);
  uint8_t* const exponents_base = reinterpret_cast<uint8_t*>(words + block_words);
  const uint32_t lane = lane_id();
  const int warp = member >> 5;
  const int warps = group_threads >> 5;

  const bool kept = !EXPORT && p.kept_tables != nullptr;
  if (kept) {
    // both tables as they were exported: 16-byte asynchronous copies, waited for together with nothing else
    const uint32_t words = level_table_words(levels) + 2u * kMultiEntries;
    const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(shared));
    for (uint32_t at = threadIdx.x * 4u; at < words; at += blockDim.x * 4u) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + at * 4u), "l"(p.kept_tables + at) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const uint32_t pointer_min = levels > 1 ? 256u - (levels - 1) : 256u;
  const uint8_t* lengths = p.luts + levels * 256;
  for (int i = threadIdx.x; i < levels * 256 && !kept; i += blockDim.x) {
    const uint32_t entry = p.luts[i];
    // a pointer names a child level; clamp it into the staged tables so a corrupt row cannot index outside them
    tables[i] = entry >= pointer_min ? static_cast<uint16_t>(kPointerFlag | min(256u - entry, static_cast<uint32_t>(levels - 1)))
                                     : static_cast<uint16_t>(entry | (static_cast<uint32_t>(lengths[entry]) << 8));
  }
  const int64_t block_base = format_block * block_bytes;
  for (int w = member; w < block_words && present && !EXPORT; w += group_threads) {
    const int64_t byte = block_base + static_cast<int64_t>(w) * 4;
    uint32_t value = 0;
    if (byte + 4 <= p.n_bytes && ((reinterpret_cast<uintptr_t>(p.encoded) + byte) & 3u) == 0) {
      value = byte_swap(*reinterpret_cast<const uint32_t*>(p.encoded + byte));
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) value = (value << 8) | (byte + k < p.n_bytes ? p.encoded[byte + k] : 0u);
    }
    words[w] = value;
  }

  if (kept) asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();   // level-0 entries are in place
  for (int v = threadIdx.x; v < kMultiEntries && !kept; v += blockDim.x) {
    uint32_t packed = 0, lengths = 0, used = 0, found = 0;
    while (found < 4u) {
      const uint32_t rest = (static_cast<uint32_t>(v) << used) & (kMultiEntries - 1);      // bits not yet consumed, left-aligned
      uint32_t entry = tables[rest >> (kMultiBits - 8)];
      if (entry & kPointerFlag) {
        // a codeword of nine bits or more: what the window holds beyond the first byte, zero-extended, picks in the child
        // level; if the codeword fits the window (checked below) the padding took no part in the choice
        const uint32_t second = (rest & ((1u << (kMultiBits - 8)) - 1u)) << (16 - kMultiBits);
        entry = tables[(entry & 0xFFu) * 256u + second];
      }
      const uint32_t length = (entry >> 8) & 0x3Fu;
      if ((entry & kPointerFlag) || length == 0u || used + length > static_cast<uint32_t>(kMultiBits)) break;
      packed |= (entry & 0xFFu) << (8 * found);
      used += length;
      ++found;
      lengths |= used << (4 * found);
    }
    multi[v] = make_uint2(packed, lengths | (found << 24));
  }
  if (EXPORT) {
    __syncthreads();
    const uint32_t words = level_table_words(levels) + 2u * kMultiEntries;
    for (uint32_t at = threadIdx.x; at < words; at += blockDim.x) p.export_tables[at] = shared[at];
    return;
  }
  const bool active = present && member < p.threads_per_block;
  const int64_t region = format_block * p.threads_per_block + member;
  const uint32_t meta = active ? p.thread_meta[region] : 0u;
  int count = static_cast<int>(meta & 2047u);

  // exclusive scan of the counts over the format block
  uint32_t inclusive = static_cast<uint32_t>(count);
#pragma unroll
  for (int step = 1; step < 32; step <<= 1) {
    const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, inclusive, step);
    if (lane >= static_cast<uint32_t>(step)) inclusive += below;
  }
  if (lane == 31) scan[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    uint32_t total = lane < static_cast<uint32_t>(warps) ? scan[lane] : 0u;
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
      const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, total, step);
      if (lane >= static_cast<uint32_t>(step)) total += below;
    }
    scan[lane] = total;
  }
  __syncthreads();
  int local_base = static_cast<int>((warp > 0 ? scan[warp - 1] : 0u) + inclusive) - count;

  int64_t out_base = present ? p.output_positions[format_block] : 0;
  int64_t block_elems = present ? static_cast<int64_t>(p.output_positions[format_block + 1]) - out_base : 0;
  if (out_base > p.n_elements || block_elems < 0 || block_elems > p.stage_elems || out_base + block_elems > p.n_elements) {
    // inconsistent positions (corrupt container): write nothing for this block
    if (member == 0) report(p.error, EP_STREAM_BAD_OFFSETS);
    out_base = 0;
    block_elems = 0;
    count = 0;
  }
  // The write-back after the walk reads this block's sign/mantissa bytes; asking L2 for them now takes the DRAM part of
  // that latency out of the block's serial path (one 128-byte line per thread).
  for (int64_t line = static_cast<int64_t>(member) * 128; line < block_elems; line += static_cast<int64_t>(group_threads) * 128) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p.sign_mantissa + out_base + line));
  }
  uint8_t* const exponents = exponents_base + (out_base & 7);  // keeps 8-element output groups aligned in shared memory too
  if (local_base + count > p.stage_elems) {  // only a corrupt container gets here
    count = local_base < p.stage_elems ? p.stage_elems - local_base : 0;
    if (active) report(p.error, EP_STREAM_NOT_CONSUMED);
  }

  // Walk this region's codewords. Every thread of the warp runs the same instruction stream, without branches that could
  // split it: a thread that is done (or idle) takes zero symbols, the four staging stores are predicated on how many
  // symbols the look-up delivered, the window's second word is re-read every round (the first one moves up when the
  // cursor crossed into it), and the one-symbol path for codewords longer than the window is entered by the whole
  // warp, and only in rounds where some thread needs it.
  uint32_t bit = static_cast<uint32_t>(member) * p.bytes_per_thread * 8u + (meta >> 11);
  uint32_t word_index = bit >> 5;
  const uint32_t last_word = static_cast<uint32_t>(block_words - 1);
  uint32_t current = words[min(word_index, last_word - 1u)];
  uint32_t next = words[min(word_index + 1u, last_word)];
  int i = 0;
  while (__any_sync(0xFFFFFFFFu, i < count)) {
    const bool active = i < count;
    const uint32_t window = __funnelshift_l(next, current, bit & 31u);
    const uint2 fast = multi[window >> (32 - kMultiBits)];
    const uint32_t held = fast.y >> 24;                       // whole codewords in the window's first bits
    uint32_t found = active ? min(held, static_cast<uint32_t>(count - i)) : 0u;
    uint32_t advance = (fast.y >> (4u * found)) & 0xFu;
    uint32_t symbols = fast.x;
    if (__any_sync(0xFFFFFFFFu, active && held == 0u)) {
      if (active && held == 0u) {
        uint32_t entry = tables[window >> 24];
        uint32_t peek = window;
#pragma unroll 1
        for (int hop = 0; hop < 3 && (entry & kPointerFlag); ++hop) {  // code longer than this level: the next byte picks in the child level
          peek <<= 8;
          entry = tables[(entry & 0xFFu) * 256u + (peek >> 24)];
        }
        symbols = entry & 0xFFu;
        found = 1u;
        advance = (entry >> 8) & 0x3Fu;
      }
    }
    uint8_t* const target = exponents + local_base + i;
    if (found > 0u) target[0] = static_cast<uint8_t>(symbols);
    if (found > 1u) target[1] = static_cast<uint8_t>(symbols >> 8);
    if (found > 2u) target[2] = static_cast<uint8_t>(symbols >> 16);
    if (found > 3u) target[3] = static_cast<uint8_t>(symbols >> 24);
    i += static_cast<int>(found);
    bit += advance;
    const uint32_t now = bit >> 5;
    current = now != word_index ? next : current;      // at most one word further: a codeword has 32 bits at most
    word_index = now;
    next = words[min(now + 1u, last_word)];
  }
  __syncthreads();

  // write back: 8 elements (16 bytes of bf16) per thread per iteration, aligned on 8-element groups
  const int64_t head = min(block_elems, (8 - (out_base & 7)) & 7);
  for (int64_t j = member; j < head; j += group_threads) {
    const int64_t g = out_base + j;
    const uint32_t sm = p.sign_mantissa[g];
    p.out[g] = static_cast<uint16_t>(((sm & 0x80u) << 8) | (static_cast<uint32_t>(exponents[j]) << 7) | (sm & 0x7Fu));
  }
  const int64_t groups = (block_elems - head) >> 3;
  const bool wide = (reinterpret_cast<uintptr_t>(p.sign_mantissa) & 7u) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
  for (int64_t c = member; c < groups; c += group_threads) {
    const int64_t j = head + (c << 3);
    const int64_t g = out_base + j;
    if (wide) {
      const uint2 e = *reinterpret_cast<const uint2*>(exponents + j);
      const uint2 s = __ldg(reinterpret_cast<const uint2*>(p.sign_mantissa + g));
      const uint64_t lo = pack_bf16x4(e.x, s.x);
      const uint64_t hi = pack_bf16x4(e.y, s.y);
      *reinterpret_cast<uint4*>(p.out + g) = make_uint4(static_cast<uint32_t>(lo), static_cast<uint32_t>(lo >> 32),
                                                        static_cast<uint32_t>(hi), static_cast<uint32_t>(hi >> 32));
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t sm = p.sign_mantissa[g + k];
        p.out[g + k] = static_cast<uint16_t>(((sm & 0x80u) << 8) | (static_cast<uint32_t>(exponents[j + k]) << 7) | (sm & 0x7Fu));
      }
    }
  }
  for (int64_t j = head + (groups << 3) + member; j < block_elems; j += group_threads) {
    const int64_t g = out_base + j;
    const uint32_t sm = p.sign_mantissa[g];
    p.out[g] = static_cast<uint16_t>(((sm & 0x80u) << 8) | (static_cast<uint32_t>(exponents[j]) << 7) | (sm & 0x7Fu));
  }
}

// ---- decode, one warp per run of 32 regions ----------------------------------------------------------
// Used when the container's kept tables are at hand and the stream is laid out in whole words. The unit of work is a run
// of 32 consecutive regions of one block of the format: a warp walks them (one region per thread), stages the exponents
// in its own slice of shared memory and writes the bf16 values out, with no barrier between warps. A block of the
// format no longer maps to a CUDA block: where a unit's output starts follows from output_positions plus the counts of
// the block's earlier regions, which the warp adds up itself. Two CUDA blocks per SM run until the units are used up
// (unit = warp's number in the grid, then + warps in the grid), so the 17 KB of tables are copied in twice per SM, and
// what a unit reads from global memory is asked for ahead of its use:
//   * region records and positions of the unit after this one: loaded into registers before this unit's walk;
//   * this unit's stream bytes: a bulk copy into the warp's stream slice, issued while the previous unit is written out;
//   * this unit's sign/mantissa bytes: a bulk copy into the warp's byte slice, issued when its walk starts.
// The bulk copies (cp.async.bulk, completion on an mbarrier per warp and kind) are issued by one thread and carried out
// by the copy engine: a warp that asks for its bytes goes straight on, however many copies are queued already, which
// per-thread cp.async copies did not allow once every warp of the GPU asked at the same moment.
// A unit that decodes to more elements than the slice holds (the host sizes it from the mean, regions of all-equal
// exponents exceed it) is walked without staging, each thread storing its own values.
// What bounds it: the walk's shared-memory traffic (four one-byte stores per round to addresses that share banks at
// random, the look-up) and the integer pipe, about equally; global memory is far from it.
// Offsets into the stream, the records and the output are 32-bit here: the host sends larger containers to the block kernel.
struct UnitHead {
  uint32_t region;     // the unit's first region
  uint32_t meta;       // this thread's region record (0: no region)
  uint32_t before;     // this thread's share of the counts of the block's earlier regions, beyond the first three runs
  uint32_t earlier0, earlier1, earlier2;   // this thread's records in the block's first three runs (zero where the unit is
                                           // one of them): kept as loaded, so that asking for them does not wait for them
  uint32_t first;      // output_positions[block]
  uint32_t last;       // output_positions[block + 1]
};

struct Unit {
  uint32_t start;      // first element of the unit in the output
  uint32_t gap;
  int count;           // codewords that start in this thread's region
  int local;           // elements of the unit in front of this thread's
  int total;           // elements of the unit
};

// Which unit a warp is at: its number, and the same split into block of the format and run inside the block, stepped
// without a division.
struct UnitCursor {
  uint32_t index;
  uint32_t block;
  uint32_t run;
};

__device__ __forceinline__ void step(UnitCursor& at, uint32_t stride, uint32_t stride_blocks, uint32_t stride_runs, uint32_t runs_per_block) {
  at.index += stride;
  at.block += stride_blocks;
  at.run += stride_runs;
  if (at.run >= runs_per_block) {
    at.run -= runs_per_block;
    ++at.block;
  }
}

__device__ __forceinline__ UnitHead load_unit_head(const DecodeParams& p, const UnitCursor& at, uint32_t lane) {
  UnitHead head = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  if (at.index < static_cast<uint32_t>(p.units)) {
    const uint32_t block_region = at.block * static_cast<uint32_t>(p.threads_per_block);
    const uint16_t* const records = p.thread_meta + (block_region + lane);
    head.region = block_region + at.run * 32u;
    if (at.run * 32u + lane < static_cast<uint32_t>(p.threads_per_block)) head.meta = records[at.run * 32u];
    if (at.run > 0u) head.earlier0 = records[0];
    if (at.run > 1u) head.earlier1 = records[32];
    if (at.run > 2u) head.earlier2 = records[64];
    for (uint32_t k = 3u; k < at.run; ++k) head.before += records[k * 32u] & 2047u;   // blocks of more than 128 regions
    head.first = p.output_positions[at.block];
    head.last = p.output_positions[at.block + 1u];
  }
  return head;
}

__device__ __forceinline__ Unit open_unit(const DecodeParams& p, const UnitHead& head, uint32_t lane) {
  Unit unit;
  unit.gap = head.meta >> 11;
  unit.count = static_cast<int>(head.meta & 2047u);
  uint32_t inclusive = static_cast<uint32_t>(unit.count);
#pragma unroll
  for (int step = 1; step < 32; step <<= 1) {
    const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, inclusive, step);
    if (lane >= static_cast<uint32_t>(step)) inclusive += below;
  }
  unit.local = static_cast<int>(inclusive) - unit.count;
  unit.total = static_cast<int>(__shfl_sync(0xFFFFFFFFu, inclusive, 31));   // at most 32 * 2047
  const uint32_t before = __reduce_add_sync(0xFFFFFFFFu, head.before + (head.earlier0 & 2047u) + (head.earlier1 & 2047u) +
                                                             (head.earlier2 & 2047u));   // at most 1024 * 2047
  unit.start = head.first + before;
  // a codeword has one bit at least: more of them than a region has bits is a corrupt record
  const bool counts_bad = __any_sync(0xFFFFFFFFu, unit.count > 8 * p.bytes_per_thread);
  const bool positions_bad = counts_bad || head.first > head.last || head.last > static_cast<uint32_t>(p.n_elements);
  const bool overrun = before + static_cast<uint32_t>(unit.total) > head.last - head.first;
  if (positions_bad || overrun) {   // only a corrupt container gets here: write nothing for this unit
    if (lane == 0) report(p.error, positions_bad ? EP_STREAM_BAD_OFFSETS : EP_STREAM_NOT_CONSUMED);
    unit.count = 0;
    unit.total = 0;
    unit.start = 0;
  }
  return unit;
}

// Bounded wait on a phase of an mbarrier; false when the limit ran out (a copy that never completes).
constexpr uint32_t kCopyWaitLimit = 1u << 22;
__device__ __forceinline__ bool copy_wait(uint32_t barrier_at, uint32_t parity) {
  for (uint32_t spin = 0; spin < kCopyWaitLimit; ++spin) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done)
                 : "r"(barrier_at), "r"(parity)
                 : "memory");
    if (done) return true;
  }
  return false;
}

// One bulk copy (issued by the calling thread, carried out by the copy engine while the warp goes on) of the 16-byte
// pieces that cover [from, from + bytes) of `source`, whose base is 16-byte aligned, into a shared slice at the same
// offset modulo 16; its completion flips the phase of the mbarrier. Pieces must lie inside the source: the caller clips.
__device__ __forceinline__ void bulk_copy_in(const uint8_t* source, uint32_t first_piece_byte, uint32_t size, uint32_t slice,
                                             uint32_t barrier_at) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barrier_at), "r"(size) : "memory");
  if (size) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(slice),
                 "l"(source + first_piece_byte), "r"(size), "r"(barrier_at)
                 : "memory");
  }
}

// The warp's copy of a span: thread 0 issues the bulk copy of the whole 16-byte pieces inside the source; where the
// span's last piece crosses the source's end (the last unit of a container), the threads bring the bytes short of the
// end in with plain loads, and what lies beyond stays as it was: a valid stream never looks at it.
__device__ __forceinline__ void copy_in_span(const uint8_t* __restrict__ source, uint32_t limit, uint32_t from, uint32_t bytes,
                                             uint32_t slice, uint8_t* slice_generic, uint32_t barrier_at, uint32_t lane) {
  const uint32_t aligned = from & ~15u;
  uint32_t size = ((from & 15u) + bytes + 15u) & ~15u;
  if (size > limit - min(aligned, limit)) {
    const uint32_t whole = (limit & ~15u) - min(aligned, limit & ~15u);
    const uint32_t rest_from = aligned + whole;
    if (rest_from + lane < limit && lane < 16u) slice_generic[whole + lane] = source[rest_from + lane];
    size = whole;
  }
  if (lane == 0) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the slice was last touched through ordinary loads and stores
    bulk_copy_in(source, aligned, size, slice, barrier_at);
  }
}

__device__ __forceinline__ uint16_t bf16_bits(uint32_t exponent, uint32_t sign_mantissa) {
  return static_cast<uint16_t>(((sign_mantissa & 0x80u) << 8) | (exponent << 7) | (sign_mantissa & 0x7Fu));
}

// Four bf16 values from four exponents and four sign/mantissa bytes: per value the high byte is sign | exponent >> 1
// and the low byte exponent << 7 | mantissa, each a bitwise select under 0x80 per byte (one lop3), then interleaved.
__device__ __forceinline__ uint2 merge_bf16x4(uint32_t exponents, uint32_t sign_mantissa) {
  uint32_t low, high;
  asm("lop3.b32 %0, %1, %2, 0x80808080, 0xE4;" : "=r"(low) : "r"(exponents << 7), "r"(sign_mantissa));
  asm("lop3.b32 %0, %1, %2, 0x80808080, 0xE4;" : "=r"(high) : "r"(sign_mantissa), "r"(exponents >> 1));
  return make_uint2(__byte_perm(low, high, 0x5140), __byte_perm(low, high, 0x7362));
}

// Walks this thread's region: `left` codewords from bit `bit` of the warp's stream slice on. STAGED: exponents go to the
// warp's shared slice from `target` on (a shared address). Otherwise values go straight to the output from `element` on.
// Every thread of the warp runs the same instructions: a finished thread takes zero symbols, the four byte stores are
// predicated on the number of symbols delivered, and the one-symbol path for codewords longer than the window is
// entered by the whole warp in rounds where some thread needs it. The stream word two ahead is read at the top of a
// round, before the advance is known, so that the look-up is the only shared-memory read on the path from one round to
// the next. The two halves of a round are written out in PTX to keep them at the instructions they need: the
// compiler's version of the same statements came to twice as many.
// The walk ends when the codewords are used up, wherever the cursor then is: `left` is at most the number of bits in a
// region (checked when the unit is opened) and a codeword at most 32 bits, so a corrupt stream reads at most
// 32 x bytes_per_thread bytes past its region, which the block's shared memory is padded for. Returns the final cursor.
// HELD: regions of 16 bytes. A thread then reads its four stream words once (one 16-byte load, no bank conflicts), takes
// the look-ahead word from its neighbour, and feeds the window from registers: the walk reads shared memory for the
// look-ups only, and a corrupt stream cannot take it past what it holds.
template <bool STAGED, bool HELD>
__device__ __forceinline__ uint32_t walk_region(const DecodeParams& p, const uint16_t* tables, uint32_t multi_at, uint32_t words_at,
                                                uint32_t bit, uint32_t left, uint32_t target, uint32_t element) {
  uint32_t word_at = words_at + ((bit >> 5) << 2);   // shared address of the word the cursor is in
  uint32_t current, next, third = 0u, fourth = 0u, fifth = 0u;
  if (HELD) {
    // bit < 32 + the region's first bit: the cursor starts in the region's first word
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(current), "=r"(next), "=r"(third), "=r"(fourth) : "r"(word_at));
    uint32_t beyond;   // the warp's last region looks ahead into the word behind the unit's stream bytes
    asm volatile("ld.shared.u32 %0, [%1+16];" : "=r"(beyond) : "r"(word_at));
    fifth = __shfl_down_sync(0xFFFFFFFFu, current, 1);
    if (lane_id() == 31u) fifth = beyond;
    third = byte_swap(third);
    fourth = byte_swap(fourth);
    fifth = byte_swap(fifth);
  } else {
    asm volatile("ld.shared.u32 %0, [%2];\n\tld.shared.u32 %1, [%2+4];" : "=r"(current), "=r"(next) : "r"(word_at));
  }
  current = byte_swap(current);
  next = byte_swap(next);
  while (__any_sync(0xFFFFFFFFu, left != 0u)) {
    uint32_t window, symbols, found, advance, after = 0u, slow;
    if (!HELD) {
      asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(after) : "r"(word_at));
      after = byte_swap(after);
    }
    asm volatile(
        "{\n\t"
        ".reg .pred act, none;\n\t"
        ".reg .b32 idx, fy, held, sh;\n\t"
        "shf.l.wrap.b32 %0, %6, %7, %5;\n\t"           // the 32 bits under the cursor (the shift wraps at 32)
        "shr.u32 idx, %0, 21;\n\t"
        "mad.lo.u32 idx, idx, 8, %9;\n\t"
        "ld.shared.v2.u32 {%1, fy}, [idx];\n\t"         // up to four codewords of the next 11 bits
        "shr.u32 held, fy, 24;\n\t"
        "min.u32 %2, held, %8;\n\t"                    // a finished thread (none left) takes none
        "shl.b32 sh, %2, 2;\n\t"
        "shr.u32 %3, fy, sh;\n\t"
        "and.b32 %3, %3, 15;\n\t"                        // bits consumed by `found` codewords (field 0 is zero)
        "setp.ne.u32 act, %8, 0;\n\t"
        "setp.eq.and.u32 none, held, 0, act;\n\t"
        "selp.u32 %4, 1, 0, none;\n\t"
        "}\n"
        : "=&r"(window), "=&r"(symbols), "=&r"(found), "=&r"(advance), "=&r"(slow)
        : "r"(bit), "r"(next), "r"(current), "r"(left), "r"(multi_at));
    if (__any_sync(0xFFFFFFFFu, slow)) {
      if (slow) {
        uint32_t entry = tables[window >> 24];
        uint32_t peek = window;
#pragma unroll 1
        for (int hop = 0; hop < 3 && (entry & kPointerFlag); ++hop) {  // code longer than this level: the next byte picks in the child level
          peek <<= 8;
          entry = tables[(entry & 0xFFu) * 256u + (peek >> 24)];
        }
        symbols = entry & 0xFFu;
        found = 1u;
        advance = (entry >> 8) & 0x3Fu;
      }
    }
    if (STAGED) {
      asm volatile(
          "{\n\t"
          ".reg .pred q;\n\t"
          ".reg .b32 b;\n\t"
          "setp.gt.u32 q, %1, 0;\n\t"
          "@q st.shared.u8 [%0], %2;\n\t"
          "setp.gt.u32 q, %1, 1;\n\t"
          "shr.u32 b, %2, 8;\n\t"
          "@q st.shared.u8 [%0+1], b;\n\t"
          "setp.gt.u32 q, %1, 2;\n\t"
          "shr.u32 b, %2, 16;\n\t"
          "@q st.shared.u8 [%0+2], b;\n\t"
          "setp.gt.u32 q, %1, 3;\n\t"
          "shr.u32 b, %2, 24;\n\t"
          "@q st.shared.u8 [%0+3], b;\n\t"
          "}\n" ::"r"(target),
          "r"(found), "r"(symbols)
          : "memory");
      target += found;
    } else {
      for (uint32_t k = 0; k < found; ++k) p.out[element + k] = bf16_bits((symbols >> (8u * k)) & 0xFFu, p.sign_mantissa[element + k]);
      element += found;
    }
    if (HELD) {
      asm volatile(
          "{\n\t"
          ".reg .pred cross;\n\t"
          ".reg .b32 moved, changed;\n\t"
          "sub.u32 %0, %0, %6;\n\t"
          "add.u32 moved, %1, %7;\n\t"
          "xor.b32 changed, moved, %1;\n\t"
          "setp.gt.u32 cross, changed, 31;\n\t"          // into the next word (at most one: a codeword has 32 bits at most)
          "mov.b32 %1, moved;\n\t"
          "@cross mov.b32 %2, %3;\n\t"
          "@cross mov.b32 %3, %4;\n\t"                   // the words still to come move up
          "@cross mov.b32 %4, %5;\n\t"
          "@cross mov.b32 %5, %8;\n\t"
          "}\n"
          : "+r"(left), "+r"(bit), "+r"(current), "+r"(next), "+r"(third), "+r"(fourth)
          : "r"(found), "r"(advance), "r"(fifth));
    } else {
      asm volatile(
          "{\n\t"
          ".reg .pred cross;\n\t"
          ".reg .b32 moved, changed;\n\t"
          "sub.u32 %0, %0, %5;\n\t"
          "add.u32 moved, %1, %6;\n\t"
          "xor.b32 changed, moved, %1;\n\t"
          "setp.gt.u32 cross, changed, 31;\n\t"
          "mov.b32 %1, moved;\n\t"
          "@cross mov.b32 %2, %3;\n\t"
          "@cross mov.b32 %3, %7;\n\t"
          "@cross add.u32 %4, %4, 4;\n\t"               // the cursor's word in shared memory
          "}\n"
          : "+r"(left), "+r"(bit), "+r"(current), "+r"(next), "+r"(word_at)
          : "r"(found), "r"(advance), "r"(after));
    }
  }
  return bit;
}

template <bool HELD>
__global__ void __launch_bounds__(kWarpKernelMaxWarps * 32, kWarpKernelBlocksPerSm) dfloat11_decode_warps_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) uint32_t shared[];
  // layout: fused tables u16[levels][256] | multi-symbol table uint2[2048] | mbarriers: tables, then two per warp |
  //         per warp: stream bytes [32 * bytes_per_thread + 48] | exponents [stage_alloc + 32] | sign/mantissa [stage_alloc + 32] |
  //         32 * bytes_per_thread + 64 bytes that only a walk over a corrupt stream reads
  const int levels = p.num_luts - 1;
  const uint32_t table_words = level_table_words(levels) + 2u * (1u << kKeptMultiBits);
  const uint32_t shared_base = static_cast<uint32_t>(__cvta_generic_to_shared(shared));
  const uint16_t* const tables = reinterpret_cast<const uint16_t*>(shared);
  const uint32_t multi_at = shared_base + level_table_words(levels) * 4u;

  const uint32_t lane = lane_id();
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t warps = blockDim.x >> 5;
  const uint32_t region_bytes = static_cast<uint32_t>(p.bytes_per_thread);
  const uint32_t stream_slice = 32u * region_bytes + 48u;
  const uint32_t byte_slice = static_cast<uint32_t>(p.stage_alloc) + 32u;
  const uint32_t barrier_bytes = (8u + 16u * warps + 15u) & ~15u;
  const uint32_t tables_barrier = shared_base + table_words * 4u;
  const uint32_t stream_barrier = tables_barrier + 8u + 16u * warp;   // flips when the warp's stream bytes are in
  const uint32_t rest_barrier = stream_barrier + 8u;                    // flips when its sign/mantissa bytes are in
  const uint32_t slices_offset = table_words * 4u + barrier_bytes + warp * (stream_slice + 2u * byte_slice);
  uint8_t* const slice = reinterpret_cast<uint8_t*>(shared) + slices_offset;
  uint8_t* const exponents = slice + stream_slice;
  uint8_t* const sign_mantissa = slice + stream_slice + byte_slice;
  const uint32_t words_at = shared_base + slices_offset;
  const uint32_t exponents_at = words_at + stream_slice;
  const uint32_t sign_mantissa_at = exponents_at + byte_slice;

  // unit = warp's number in the grid (neighbouring units to neighbouring SMs), then + warps in the grid
  const uint32_t units = static_cast<uint32_t>(p.units);
  const uint32_t stride = gridDim.x * warps;
  const uint32_t runs_per_block = static_cast<uint32_t>(p.units_per_block);
  const uint32_t stride_blocks = stride / runs_per_block;
  const uint32_t stride_runs = stride - stride_blocks * runs_per_block;
  const uint32_t stream_bytes = static_cast<uint32_t>(p.n_bytes);
  const uint32_t elements = static_cast<uint32_t>(p.n_elements);
  const uint32_t stage_alloc = static_cast<uint32_t>(p.stage_alloc);
  UnitCursor next_at;
  next_at.index = blockIdx.x + warp * gridDim.x;
  next_at.block = next_at.index / runs_per_block;
  next_at.run = next_at.index - next_at.block * runs_per_block;
  uint32_t index = next_at.index;
  // Order of the requests: the first unit's region records (a warp waits for them first), its stream bytes (the copy
  // needs no record), then the tables; the records of the unit after it once the first ones are in. Sign/mantissa bytes
  // are asked for when a unit's walk starts: they are not needed before it ends. Stream bytes, sign/mantissa bytes and
  // tables come in by bulk copies that one thread issues and the copy engine carries out, so that asking for them
  // holds no warp up, however much is in flight already.
  const UnitHead opening = load_unit_head(p, next_at, lane);
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(stream_barrier));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(rest_barrier));
    if (warp == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tables_barrier));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  uint32_t first_byte = opening.region * region_bytes;
  // the stream bytes of the unit plus four bytes of look-ahead for the last region
  if (index < units) copy_in_span(p.encoded, stream_bytes, first_byte, 32u * region_bytes + 4u, words_at, slice, stream_barrier, lane);
  if (threadIdx.x == 0) bulk_copy_in(reinterpret_cast<const uint8_t*>(p.kept_tables), 0u, table_words * 4u, shared_base, tables_barrier);
  Unit unit = open_unit(p, opening, lane);
  bool staged = static_cast<uint32_t>(unit.total) <= stage_alloc;
  step(next_at, stride, stride_blocks, stride_runs, runs_per_block);
  UnitHead ahead = load_unit_head(p, next_at, lane);
  __syncthreads();   // the tables' barrier is initialised for every thread to wait on; from here on the warps go their own ways
  bool copies_arrive = copy_wait(tables_barrier, 0u);
  uint32_t parity = 0u;   // of the phase the warp's two barriers are in (each flips once per unit)
  bool stream_ahead = false, rest_asked = false;   // copies in flight beyond the phase `parity` of the stream barrier / on the other one
  while (index < units && copies_arrive) {
    stream_ahead = false;
    const uint32_t shift = unit.start & 15u;                                      // of the unit's first element in the byte slices
    const bool rest_staged = staged && unit.total > 0;
    if (rest_staged) {
      copy_in_span(p.sign_mantissa, elements, unit.start, static_cast<uint32_t>(unit.total), sign_mantissa_at, sign_mantissa, rest_barrier, lane);
    } else if (lane == 0) {
      bulk_copy_in(p.sign_mantissa, 0u, 0u, sign_mantissa_at, rest_barrier);   // nothing to bring in: the phase still flips
    }
    rest_asked = true;
    copies_arrive = copy_wait(stream_barrier, parity);   // this unit's stream bytes
    __syncwarp();
    if (!copies_arrive) break;
    const uint32_t first_bit = ((first_byte & 15u) + lane * region_bytes) * 8u;   // of this thread's region in the slice
    uint32_t cursor;
    if (staged) {
      cursor = walk_region<true, HELD>(p, tables, multi_at, words_at, first_bit + unit.gap, static_cast<uint32_t>(unit.count),
                                 exponents_at + shift + static_cast<uint32_t>(unit.local), 0u);
    } else {
      cursor = walk_region<false, HELD>(p, tables, multi_at, words_at, first_bit + unit.gap, static_cast<uint32_t>(unit.count), 0u,
                                  unit.start + static_cast<uint32_t>(unit.local));
    }
    // a region's last codeword starts inside it and has 32 bits at most
    if (cursor >= first_bit + region_bytes * 8u + 32u) report(p.error, EP_STREAM_NOT_CONSUMED);
    __syncwarp();
    // the slice of stream bytes is free: the next unit's can come in while this one is written out
    first_byte = ahead.region * region_bytes;
    if (next_at.index < units) {
      copy_in_span(p.encoded, stream_bytes, first_byte, 32u * region_bytes + 4u, words_at, slice, stream_barrier, lane);
      stream_ahead = true;
    }
    const Unit following = open_unit(p, ahead, lane);
    const bool following_staged = static_cast<uint32_t>(following.total) <= stage_alloc;
    copies_arrive = copy_wait(rest_barrier, parity);   // this unit's sign/mantissa bytes
    __syncwarp();
    if (!copies_arrive) break;
    rest_asked = false;
    if (staged) {
      // 8 elements (16 bytes of bf16) per thread per round, on 8-element boundaries of the output
      const uint32_t total = static_cast<uint32_t>(unit.total);
      const uint32_t head = min(total, (8u - (unit.start & 7u)) & 7u);
      const uint32_t groups = (total - head) >> 3;
      uint16_t* const out = p.out + unit.start;
      const uint8_t* const staged_exponents = exponents + shift;
      const uint8_t* const staged_rest = sign_mantissa + shift;
      if (lane < head) out[lane] = bf16_bits(staged_exponents[lane], staged_rest[lane]);
      for (uint32_t j = head + lane * 8u; j < head + groups * 8u; j += 256u) {
        const uint2 e = *reinterpret_cast<const uint2*>(staged_exponents + j);
        const uint2 r = *reinterpret_cast<const uint2*>(staged_rest + j);
        const uint2 lower = merge_bf16x4(e.x, r.x);
        const uint2 upper = merge_bf16x4(e.y, r.y);
        *reinterpret_cast<uint4*>(out + j) = make_uint4(lower.x, lower.y, upper.x, upper.y);
      }
      const uint32_t j = head + groups * 8u + lane;
      if (j < total) out[j] = bf16_bits(staged_exponents[j], staged_rest[j]);
    }
    parity ^= 1u;
    index = next_at.index;
    step(next_at, stride, stride_blocks, stride_runs, runs_per_block);
    ahead = load_unit_head(p, next_at, lane);
    unit = following;
    staged = following_staged;
    __syncwarp();   // every thread is done with this unit's slices
  }
  if (!copies_arrive) {
    // A copy did not complete within the limit: say so and take no further unit. What this warp still has in flight
    // gets one more bounded wait each, so that the block does not retire under a copy into its shared memory.
    if (lane == 0) report(p.error, EP_KERNEL_TIMEOUT);
    copy_wait(tables_barrier, 0u);
    copy_wait(stream_barrier, parity);
    if (stream_ahead) copy_wait(stream_barrier, parity ^ 1u);
    if (rest_asked) copy_wait(rest_barrier, parity);
  }
}

// ---- encode ----------------------------------------------------------------------------------------
constexpr int kHistThreads = 256;

__global__ void __launch_bounds__(kHistThreads) exponent_histogram_kernel(const uint16_t* __restrict__ bits, int64_t n,
                                                                          unsigned long long* __restrict__ histogram) {
  __shared__ uint32_t bins[8][256];
  for (int i = threadIdx.x; i < 8 * 256; i += kHistThreads) (&bins[0][0])[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kHistThreads * 2;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * kHistThreads + threadIdx.x) * 2; i < n; i += stride) {
    if (i + 1 < n) {
      const uint32_t pair = *reinterpret_cast<const uint32_t*>(bits + i);
      atomicAdd(&bins[warp][(pair >> 7) & 0xFF], 1u);
      atomicAdd(&bins[warp][(pair >> 23) & 0xFF], 1u);
    } else {
      atomicAdd(&bins[warp][(bits[i] >> 7) & 0xFF], 1u);
    }
  }
  __syncthreads();
  if (threadIdx.x < 256) {
    uint32_t sum = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += bins[w][threadIdx.x];
    if (sum) atomicAdd(histogram + threadIdx.x, static_cast<unsigned long long>(sum));
  }
}

constexpr int kChunkThreads = 128;   // one chunk = 128 threads x 8 elements
constexpr int kPerThread = 8;
constexpr int kChunkElems = kChunkThreads * kPerThread;

struct CodeTable {
  uint32_t value[256];
  uint8_t length[256];
};

__global__ void __launch_bounds__(kChunkThreads) chunk_bits_kernel(const uint16_t* __restrict__ bits, int64_t n,
                                                                   const int32_t* __restrict__ code_len, uint32_t* __restrict__ chunk_bits) {
  __shared__ uint8_t length[256];
  __shared__ uint32_t warp_sum[kChunkThreads / 32];
  for (int i = threadIdx.x; i < 256; i += kChunkThreads) length[i] = static_cast<uint8_t>(code_len[i]);
  __syncthreads();
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kChunkElems + static_cast<int64_t>(threadIdx.x) * kPerThread;
  uint32_t total = 0;
  if (first + kPerThread <= n) {
    const uint4 raw = *reinterpret_cast<const uint4*>(bits + first);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) total += length[(w[k] >> 7) & 0xFF] + length[(w[k] >> 23) & 0xFF];
  } else {
    for (int64_t i = first; i < n; ++i) total += length[(bits[i] >> 7) & 0xFF];
  }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) total += __shfl_xor_sync(0xFFFFFFFFu, total, step);
  if (lane_id() == 0) warp_sum[threadIdx.x >> 5] = total;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t sum = 0;
#pragma unroll
    for (int w = 0; w < kChunkThreads / 32; ++w) sum += warp_sum[w];
    chunk_bits[blockIdx.x] = sum;
  }
}

struct PackParams {
  const uint16_t* bits;
  int64_t n;
  const int32_t* code_len;
  const int32_t* code_val;
  const uint32_t* chunk_offsets;   // bit offset of every chunk (exclusive scan of chunk_bits)
  uint32_t* encoded_words;         // zeroed; big-endian bit order inside each byte-swapped 32-bit word
  uint8_t* sign_mantissa;
  uint32_t* region_count;          // [regions] zeroed
  uint32_t* region_gap;            // [regions] zeroed
  uint32_t* output_positions;      // [blocks + 1] pre-set to n
  uint32_t region_bits;
  uint32_t block_bits;
  int64_t regions;
};

// ORs `length` bits of `value` into the stream at bit position `at` (MSB-first bit order). Words are kept
// byte-swapped in memory so that the final byte order is the stream's.
__device__ __forceinline__ void put_bits(uint32_t* words, uint64_t at, uint32_t value, uint32_t length) {
  const uint64_t word = at >> 5;
  const uint32_t offset = static_cast<uint32_t>(at & 31u);
  const uint64_t aligned = static_cast<uint64_t>(value) << (64u - length - offset);  // length <= 32, offset <= 31
  const uint32_t hi = static_cast<uint32_t>(aligned >> 32);
  const uint32_t lo = static_cast<uint32_t>(aligned);
  if (hi) atomicOr(words + word, byte_swap(hi));
  if (lo) atomicOr(words + word + 1, byte_swap(lo));
}

__global__ void __launch_bounds__(kChunkThreads) pack_kernel(const PackParams p) {
  __shared__ uint32_t value[256];
  __shared__ uint8_t length[256];
  __shared__ uint32_t warp_sum[kChunkThreads / 32];
  for (int i = threadIdx.x; i < 256; i += kChunkThreads) {
    value[i] = static_cast<uint32_t>(p.code_val[i]);
    length[i] = static_cast<uint8_t>(p.code_len[i]);
  }
  __syncthreads();
  const uint32_t lane = lane_id();
  const int warp = threadIdx.x >> 5;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kChunkElems + static_cast<int64_t>(threadIdx.x) * kPerThread;
  const int mine = static_cast<int>(max(int64_t(0), min(static_cast<int64_t>(kPerThread), p.n - first)));
  uint32_t exponent[kPerThread];
  uint32_t own_bits = 0;
  uint32_t sm[2] = {0u, 0u};
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    exponent[k] = 0;
    if (k < mine) {
      const uint32_t v = p.bits[first + k];
      exponent[k] = (v >> 7) & 0xFFu;
      sm[k >> 2] |= (((v >> 8) & 0x80u) | (v & 0x7Fu)) << (8 * (k & 3));
      own_bits += length[exponent[k]];
    }
  }
  if (mine == kPerThread) {
    *reinterpret_cast<uint2*>(p.sign_mantissa + first) = make_uint2(sm[0], sm[1]);
  } else {
    for (int k = 0; k < mine; ++k) p.sign_mantissa[first + k] = static_cast<uint8_t>(sm[k >> 2] >> (8 * (k & 3)));
  }
  // exclusive scan of own_bits over the chunk
  uint32_t inclusive = own_bits;
#pragma unroll
  for (int step = 1; step < 32; step <<= 1) {
    const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, inclusive, step);
    if (lane >= static_cast<uint32_t>(step)) inclusive += below;
  }
  if (lane == 31) warp_sum[warp] = inclusive;
  __syncthreads();
  uint32_t before = 0;
  for (int w = 0; w < warp; ++w) before += warp_sum[w];
  uint64_t at = static_cast<uint64_t>(p.chunk_offsets[blockIdx.x]) + before + inclusive - own_bits;

  // Previous element's region/block, to detect where a new one starts. The element before this thread's
  // first one ends where ours begins, so its start is `at - its length`; only its region matters and a
  // codeword is at most 32 bits <= one region, so "starts in an earlier region" == "at - 1 is earlier or
  // the element starts exactly at a region boundary" is not enough -- fetch the true previous start.
  uint32_t previous_length = 0;
  if (first > 0 && mine > 0) previous_length = length[(p.bits[first - 1] >> 7) & 0xFFu];
  uint64_t previous_start = at - previous_length;
  bool has_previous = first > 0;
  uint32_t run_region = 0xFFFFFFFFu, run_count = 0;
#pragma unroll
  for (int k = 0; k < kPerThread; ++k) {
    if (k >= mine) break;
    const uint32_t len = length[exponent[k]];
    put_bits(p.encoded_words, at, value[exponent[k]], len);
    const uint32_t region = static_cast<uint32_t>(at / p.region_bits);
    const bool new_region = !has_previous || static_cast<uint32_t>(previous_start / p.region_bits) != region;
    if (new_region) p.region_gap[region] = static_cast<uint32_t>(at - static_cast<uint64_t>(region) * p.region_bits);
    if (!has_previous || previous_start / p.block_bits != at / p.block_bits) {
      p.output_positions[at / p.block_bits] = static_cast<uint32_t>(first + k);
    }
    if (region != run_region) {
      if (run_count) atomicAdd(p.region_count + run_region, run_count);
      run_region = region;
      run_count = 0;
    }
    run_count += 1;
    previous_start = at;
    has_previous = true;
    at += len;
  }
  if (run_count) atomicAdd(p.region_count + run_region, run_count);
}

__global__ void finish_stream_kernel(uint32_t* encoded_words, uint64_t total_bits, uint32_t eof_value, uint32_t eof_length,
                                     const uint32_t* region_count, const uint32_t* region_gap, uint16_t* thread_meta, int64_t regions) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r == 0 && (total_bits & 7u)) {
    // complete the last byte with the leading bits of the end-of-stream codeword
    const uint32_t room = 8u - static_cast<uint32_t>(total_bits & 7u);
    const uint32_t lead = eof_length >= room ? eof_value >> (eof_length - room) : eof_value << (room - eof_length);
    put_bits(encoded_words, total_bits, lead & ((1u << room) - 1u), room);
  }
  if (r < regions) thread_meta[r] = static_cast<uint16_t>((region_gap[r] << 11) | (region_count[r] & 2047u));
}

__global__ void fill_u32_kernel(uint32_t* target, int64_t count, uint32_t value) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) target[i] = value;
}

}  // namespace
}  // namespace ep

using namespace ep;

extern "C" int64_t ep_dfloat11_decode_tables_bytes(int num_luts) {
  if (num_luts < 2 || num_luts > kMaxLevels + 1) return EP_ERR_INVALID_ARGUMENT;
  return static_cast<int64_t>(level_table_words(num_luts - 1) + 2u * (1u << kKeptMultiBits)) * 4;
}

extern "C" int ep_dfloat11_build_decode_tables(const uint8_t* luts_dev, int num_luts, void* tables_dev, int64_t tables_bytes,
                                               ep_stream_t stream) {
  const int64_t needed = ep_dfloat11_decode_tables_bytes(num_luts);
  if (needed < 0) return static_cast<int>(needed);
  if (!luts_dev || !tables_dev || tables_bytes < needed || (reinterpret_cast<uintptr_t>(tables_dev) & 15u)) return EP_ERR_INVALID_ARGUMENT;
  DecodeParams p = {};
  p.luts = luts_dev;
  p.num_luts = num_luts;
  p.bytes_per_thread = 16;
  p.threads_per_block = 128;
  p.groups = 1;
  p.export_tables = static_cast<uint32_t*>(tables_dev);
  if (needed > 48 * 1024) {
    EP_CUDA_CHECK(cudaFuncSetAttribute(dfloat11_decode_kernel<kKeptMultiBits, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(needed)));
  }
  dfloat11_decode_kernel<kKeptMultiBits, true><<<1, 512, static_cast<size_t>(needed), static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("dfloat11_decode_kernel (table export)");
}

// The warp-per-unit kernel, for streams laid out in whole words behind 16-byte aligned bases. EP_ERR_UNSUPPORTED: not
// such a stream (or slices too large for shared memory); nothing was launched.
static int launch_decode_warps(DecodeParams p, ep_stream_t stream) {
  const uintptr_t bases = reinterpret_cast<uintptr_t>(p.encoded) | reinterpret_cast<uintptr_t>(p.sign_mantissa) |
                          reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.kept_tables);
  if ((bases & 15u) || (p.bytes_per_thread & 3) || p.bytes_per_thread > 1024) return EP_ERR_UNSUPPORTED;
  p.units_per_block = (p.threads_per_block + 31) / 32;
  p.units = p.blocks * p.units_per_block;
  // the kernel keeps offsets into the stream, the records and the output in 32 bits
  const int64_t covered = p.blocks * static_cast<int64_t>(p.threads_per_block) * p.bytes_per_thread;
  if (p.units > 0x3FFFFFFF || covered + 64 > 0xFFFFFFFFll || p.n_elements > 0xFFFFFFFFll) return EP_ERR_UNSUPPORTED;
  // A warp's byte slices hold an eighth more than the mean unit; a unit above that is decoded without staging.
  const int64_t mean = (p.n_elements + p.units - 1) / p.units;
  const int64_t widest = 32 * 8 * static_cast<int64_t>(p.bytes_per_thread);   // a codeword has one bit at least
  p.stage_alloc = static_cast<int>((std::min(mean + mean / 8 + 48, widest) + 15) & ~int64_t(15));
  const size_t tables = static_cast<size_t>(level_table_words(p.num_luts - 1) + 2u * (1u << kKeptMultiBits)) * 4;
  const size_t per_warp = 32u * static_cast<size_t>(p.bytes_per_thread) + 48u + 2u * (static_cast<size_t>(p.stage_alloc) + 32u);
  const size_t block_room = (227 * 1024) / kWarpKernelBlocksPerSm - 1024;   // the SM's shared memory, less what each block reserves
  const size_t overrun_pad = 32u * static_cast<size_t>(p.bytes_per_thread) + 64u;   // what a walk over a corrupt stream may read past its slice
  const auto barriers = [](int warps) { return (static_cast<size_t>(8 + 16 * warps) + 15) & ~size_t(15); };   // mbarriers: tables, two per warp
  const size_t fixed = tables + overrun_pad + barriers(kWarpKernelMaxWarps);
  if (fixed + 2 * per_warp > block_room) return EP_ERR_UNSUPPORTED;
  int warps = static_cast<int>(std::min<size_t>(kWarpKernelMaxWarps, (block_room - fixed) / per_warp));
  const int64_t slots = static_cast<int64_t>(kSmCount) * kWarpKernelBlocksPerSm;   // blocks in flight
  if (p.units > warps * slots) {
    // every warp takes ceil(units / warps in the grid) units one after another: of the block sizes from half the
    // largest up, take the one that leaves the fewest of those turns empty (the larger one unless the gain is clear)
    int best = warps;
    double best_fill = 0.0;
    for (int w = warps; w >= std::max(2, warps / 2); --w) {
      const int64_t in_grid = w * slots;
      const int64_t turns = (p.units + in_grid - 1) / in_grid;
      const double fill = static_cast<double>(p.units) / static_cast<double>(turns * in_grid);
      if (fill > best_fill + 0.02) { best_fill = fill; best = w; }
    }
    warps = best;
  }
  // few units: fewer warps to a block, so that the blocks still spread over the SMs
  warps = static_cast<int>(std::min<int64_t>(warps, std::max<int64_t>(2, (p.units + slots - 1) / slots)));
  const size_t shared = tables + barriers(warps) + warps * per_warp + overrun_pad;
  const int64_t grid = std::min<int64_t>(slots, (p.units + warps - 1) / warps);
  const auto kernel = p.bytes_per_thread == 16 ? dfloat11_decode_warps_kernel<true> : dfloat11_decode_warps_kernel<false>;
  if (shared > 48 * 1024) EP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
  kernel<<<static_cast<unsigned>(grid), warps * 32, shared, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("dfloat11_decode_warps_kernel");
}

extern "C" int ep_dfloat11_decode(const uint8_t* luts_dev, int num_luts, const uint8_t* encoded_dev, int64_t n_bytes,
                                  const uint8_t* sign_mantissa_dev, const uint32_t* output_positions_dev,
                                  const uint16_t* thread_meta_dev, void* output_dev, int64_t n_elements, int bytes_per_thread,
                                  int threads_per_block, int max_block_elems, const void* decode_tables_dev,
                                  int64_t decode_tables_bytes, int* error_dev, ep_stream_t stream) {
  if (!luts_dev || !sign_mantissa_dev || !output_positions_dev || !thread_meta_dev || !output_dev || n_elements <= 0 ||
      n_bytes < 0 || num_luts < 2 || num_luts > kMaxLevels + 1 || bytes_per_thread <= 0 || threads_per_block <= 0 ||
      max_block_elems < 0) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (n_bytes > 0 && !encoded_dev) return EP_ERR_INVALID_ARGUMENT;
  if (threads_per_block > 1024) return EP_ERR_UNSUPPORTED;
  const bool kept = decode_tables_dev != nullptr;
  if (kept && (decode_tables_bytes < ep_dfloat11_decode_tables_bytes(num_luts) || (reinterpret_cast<uintptr_t>(decode_tables_dev) & 15u))) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  const int64_t block_bytes = static_cast<int64_t>(bytes_per_thread) * threads_per_block;
  const int64_t blocks = (n_bytes + block_bytes - 1) / block_bytes;
  if (blocks == 0) return EP_OK;
  if (blocks > 0x7FFFFFFF) return EP_ERR_TOO_LARGE;
  DecodeParams p = {};
  p.luts = luts_dev;
  p.encoded = encoded_dev;
  p.sign_mantissa = sign_mantissa_dev;
  p.output_positions = output_positions_dev;
  p.thread_meta = thread_meta_dev;
  p.out = static_cast<uint16_t*>(output_dev);
  p.n_bytes = n_bytes;
  p.n_elements = n_elements;
  p.num_luts = num_luts;
  p.bytes_per_thread = bytes_per_thread;
  p.threads_per_block = threads_per_block;
  p.stage_elems = max_block_elems;
  p.error = error_dev;
  p.kept_tables = static_cast<const uint32_t*>(decode_tables_dev);
  p.blocks = blocks;
  if (kept) {
    const int rc = launch_decode_warps(p, stream);
    if (rc != EP_ERR_UNSUPPORTED) return rc;   // else: a layout the warp kernel does not take, the block kernel does
  }
  const int threads = (threads_per_block + 31) / 32 * 32;
  const size_t block_words = ((block_bytes + 3) / 4 + 3) & ~size_t(1);
  const size_t stage_bytes = (static_cast<size_t>(max_block_elems) + 16 + 15) & ~size_t(15);
  const size_t multi_bytes = static_cast<size_t>(8) << (kept ? kKeptMultiBits : kBuiltMultiBits);
  const size_t fixed = static_cast<size_t>(level_table_words(num_luts - 1)) * 4 + multi_bytes + kMaxFormatBlocks * 32 * 4;
  const size_t per_group = block_words * 4 + stage_bytes;
  // four blocks of the format to a CUDA block while four such CUDA blocks still fit an SM's shared memory
  int groups = kMaxFormatBlocks;
  while (groups > 1 && (threads * groups > 1024 || fixed + groups * per_group > 55 * 1024 || blocks < groups)) groups >>= 1;
  const size_t shared = fixed + groups * per_group;
  if (shared > 227 * 1024) return EP_ERR_UNSUPPORTED;
  p.blocks = blocks;
  p.groups = groups;
  const int64_t grid = (blocks + groups - 1) / groups;
  const auto launch = [&](auto kernel) -> int {
    if (shared > 48 * 1024) EP_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
    kernel<<<static_cast<unsigned>(grid), threads * groups, shared, static_cast<cudaStream_t>(stream)>>>(p);
    return EP_OK;
  };
  const int rc = kept ? launch(dfloat11_decode_kernel<kKeptMultiBits, false>) : launch(dfloat11_decode_kernel<kBuiltMultiBits, false>);
  if (rc != EP_OK) return rc;
  return check_launch("dfloat11_decode_kernel");
}

extern "C" int ep_dfloat11_histogram(const void* bf16_dev, int64_t n_elements, uint64_t* histogram_dev, ep_stream_t stream) {
  if (!bf16_dev || !histogram_dev || n_elements <= 0 || (reinterpret_cast<uintptr_t>(bf16_dev) & 3u)) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EP_CUDA_CHECK(cudaMemsetAsync(histogram_dev, 0, 256 * sizeof(uint64_t), s));
  const int64_t wanted = (n_elements / 2 + kHistThreads) / kHistThreads;
  const unsigned blocks = static_cast<unsigned>(wanted < kSmCount * 8 ? wanted : kSmCount * 8);
  exponent_histogram_kernel<<<blocks, kHistThreads, 0, s>>>(static_cast<const uint16_t*>(bf16_dev), n_elements,
                                                            reinterpret_cast<unsigned long long*>(histogram_dev));
  return check_launch("exponent_histogram_kernel");
}

extern "C" int64_t ep_dfloat11_chunks(int64_t n_elements) { return n_elements <= 0 ? 0 : (n_elements + kChunkElems - 1) / kChunkElems; }

extern "C" int ep_dfloat11_chunk_bits(const void* bf16_dev, int64_t n_elements, const int32_t* code_len_dev, uint32_t* chunk_bits_dev,
                                      ep_stream_t stream) {
  if (!bf16_dev || !code_len_dev || !chunk_bits_dev || n_elements <= 0 || (reinterpret_cast<uintptr_t>(bf16_dev) & 15u)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  const int64_t chunks = ep_dfloat11_chunks(n_elements);
  if (chunks > 0x7FFFFFFF) return EP_ERR_TOO_LARGE;
  chunk_bits_kernel<<<static_cast<unsigned>(chunks), kChunkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(bf16_dev), n_elements, code_len_dev, chunk_bits_dev);
  return check_launch("chunk_bits_kernel");
}

extern "C" int ep_dfloat11_pack(const void* bf16_dev, int64_t n_elements, const int32_t* code_len_dev, const int32_t* code_val_dev,
                                const uint32_t* chunk_offsets_dev, uint64_t total_bits, int bytes_per_thread, int threads_per_block,
                                int eof_length, uint32_t eof_value, uint8_t* encoded_dev, uint8_t* sign_mantissa_dev,
                                uint16_t* thread_meta_dev, uint32_t* output_positions_dev, uint32_t* region_scratch_dev,
                                ep_stream_t stream) {
  if (!bf16_dev || !code_len_dev || !code_val_dev || !chunk_offsets_dev || !encoded_dev || !sign_mantissa_dev || !thread_meta_dev ||
      !output_positions_dev || !region_scratch_dev || n_elements <= 0 || n_elements >= (int64_t(1) << 32) ||
      total_bits == 0 || total_bits >= (uint64_t(1) << 32) || bytes_per_thread < 5 || bytes_per_thread > 255 ||
      threads_per_block <= 0 || eof_length <= 0 || eof_length > 32) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(encoded_dev) & 3u) || (reinterpret_cast<uintptr_t>(sign_mantissa_dev) & 7u)) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n_bytes = static_cast<int64_t>((total_bits + 7) / 8);
  const int64_t block_bytes = static_cast<int64_t>(bytes_per_thread) * threads_per_block;
  const int64_t blocks = (n_bytes + block_bytes - 1) / block_bytes;
  const int64_t regions = blocks * threads_per_block;
  // the caller sizes encoded_dev to a multiple of 4 bytes plus 4 (put_bits may touch the word after the last)
  EP_CUDA_CHECK(cudaMemsetAsync(encoded_dev, 0, static_cast<size_t>((n_bytes + 3) / 4 * 4 + 4), s));
  EP_CUDA_CHECK(cudaMemsetAsync(region_scratch_dev, 0, sizeof(uint32_t) * 2 * regions, s));
  fill_u32_kernel<<<static_cast<unsigned>((blocks + 1 + 255) / 256), 256, 0, s>>>(output_positions_dev, blocks + 1,
                                                                                   static_cast<uint32_t>(n_elements));
  PackParams p;
  p.bits = static_cast<const uint16_t*>(bf16_dev);
  p.n = n_elements;
  p.code_len = code_len_dev;
  p.code_val = code_val_dev;
  p.chunk_offsets = chunk_offsets_dev;
  p.encoded_words = reinterpret_cast<uint32_t*>(encoded_dev);
  p.sign_mantissa = sign_mantissa_dev;
  p.region_count = region_scratch_dev;
  p.region_gap = region_scratch_dev + regions;
  p.output_positions = output_positions_dev;
  p.region_bits = static_cast<uint32_t>(bytes_per_thread) * 8u;
  p.block_bits = p.region_bits * static_cast<uint32_t>(threads_per_block);
  p.regions = regions;
  const int64_t chunks = ep_dfloat11_chunks(n_elements);
  pack_kernel<<<static_cast<unsigned>(chunks), kChunkThreads, 0, s>>>(p);
  finish_stream_kernel<<<static_cast<unsigned>((regions + 255) / 256), 256, 0, s>>>(
      p.encoded_words, total_bits, eof_value, static_cast<uint32_t>(eof_length), p.region_count, p.region_gap, thread_meta_dev, regions);
  return check_launch("dfloat11 pack");
}
