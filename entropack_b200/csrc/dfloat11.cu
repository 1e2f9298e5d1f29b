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
// Decode: one CUDA block per format block, one thread per region. The block's bytes are staged once into
// shared memory as big-endian words, the LUT levels are fused with the length row into 16-bit entries
// (one shared load per level), each thread walks its codewords with a two-word register window, symbols
// go to a shared staging array and leave as coalesced 16-byte bf16 stores merged with sign_mantissa.
//
// Encode: two passes over the input. Pass 1 sums code lengths per chunk of 1024 elements; a scan gives
// every chunk its bit offset; pass 2 re-reads the chunk, places every codeword with at most three
// atomicOr on 32-bit words (big-endian bit order), splits off sign_mantissa, and derives the region and
// block metadata from the same bit positions.
#include "ep_common.cuh"

namespace ep {
namespace {

constexpr int kMaxLevels = 64;
constexpr uint32_t kPointerFlag = 0x8000u;
// Multi-symbol table: indexed by the next MULTI_BITS bits of the stream, a 64-bit entry holds up to four whole codewords
// that fit in those bits: .x = their symbols, one per byte; .y = the bits consumed after one, two, three and four of
// them in four 4-bit fields, and their number in bits 16-18 (0: the first codeword is longer than the window or than a
// level-0 look-up, take the one-symbol path). A thread with fewer symbols left than the entry holds takes only those
// and advances by their length, so the end of a region needs no path of its own. Exponent codes average under three
// bits, so most look-ups deliver three or four symbols. The table is built inside the kernel with a 10-bit window, or
// once per container with an 11-bit window (ep_dfloat11_build_decode_tables) and copied in by every later decode.
constexpr int kBuiltMultiBits = 10;
constexpr int kKeptMultiBits = 11;
constexpr int kMaxFormatBlocks = 4;   // blocks of the format served by one CUDA block, at most

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
      const uint32_t entry = tables[rest >> (kMultiBits - 8)];
      const uint32_t length = (entry >> 8) & 0x3Fu;
      if ((entry & kPointerFlag) || length == 0u || used + length > static_cast<uint32_t>(kMultiBits)) break;
      packed |= (entry & 0xFFu) << (8 * found);
      used += length;
      lengths |= used << (4 * found);
      ++found;
    }
    multi[v] = make_uint2(packed, lengths | (found << 16));
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
    const uint32_t held = fast.y >> 16;                       // whole codewords in the window's first bits
    uint32_t found = active ? min(held, static_cast<uint32_t>(count - i)) : 0u;
    uint32_t advance = found ? (fast.y >> (4u * found - 4u)) & 0xFu : 0u;
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
