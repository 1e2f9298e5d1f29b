// Per-warp shared-memory ring of rANS payload words, filled by cp.async copies.
//
// A decoder warp consumes its stream back to front, at most 32 words per step. The ring holds four
// chunks of 128 or 256 words and is indexed by (payload word index mod ring size), so a word's ring slot
// never depends on where the stream starts. The warp keeps the chunk under its cursor and the two below
// it resident and a fourth in flight; upkeep at least every chunk / 32 steps preserves that.
// Ring reads are masked into the ring: a corrupt stream reads stale words, never out of bounds.
#pragma once

#include "ep_common.cuh"

namespace ep {

// A ring of four chunks of 2^CHUNK_LOG words (128 or 256): three resident and one in flight.
// A decoder that consumes at most 32 words per step has to run its upkeep at least every kChunk / 32
// steps: four steps with 128-word chunks, eight with 256-word chunks (half the upkeep, twice the shared memory).
template <int CHUNK_LOG>
struct WordRing {
  static_assert(CHUNK_LOG == 7 || CHUNK_LOG == 8, "a thread copies 8 or 16 bytes of a chunk");
  static constexpr int kLog = CHUNK_LOG;
  static constexpr int kChunk = 1 << CHUNK_LOG;          // words per chunk
  static constexpr int kWords = 4 * kChunk;              // words in the ring
  static constexpr uint32_t kBytes = kWords * 2u;
  static constexpr int kStepsPerUpkeep = kChunk / 32;

  // Chunk `chunk` of the payload into its ring slot, 16 bytes per thread; the first chunks of a stream may
  // straddle the end of the payload, so the copy length is clipped there.
  static __device__ __forceinline__ void fetch_clipped(const uint16_t* __restrict__ payload, int64_t payload_words,
                                                       uint32_t ring_address, int chunk, uint32_t lane) {
    if (chunk < 0 || lane >= kChunk / 8) return;
    const int64_t word = static_cast<int64_t>(chunk) * kChunk + lane * 8;
    const int64_t remaining = payload_words - word;
    if (remaining <= 0) return;
    const int bytes = remaining >= 8 ? 16 : static_cast<int>(remaining) * 2;
    const uint32_t target = ring_address + static_cast<uint32_t>(((chunk & 3) * kChunk + lane * 8) * 2);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(target), "l"(payload + word), "r"(bytes) : "memory");
  }

  // A chunk known to lie wholly inside the payload (any chunk below one already fetched): all 32 threads
  // copy an equal share. `chunk` is the same in every thread, so the test does not split the warp.
  static __device__ __forceinline__ void fetch_interior(const uint16_t* __restrict__ payload, uint32_t ring_address, int chunk,
                                                        uint32_t lane) {
    if (chunk >= 0) {
      constexpr int kPiece = kChunk / 32;     // words per thread: 4 or 8
      const uint32_t target = ring_address + static_cast<uint32_t>(((chunk & 3) * kChunk + lane * kPiece) * 2);
      const uint16_t* source = payload + (static_cast<int64_t>(chunk) * kChunk + lane * kPiece);
      if (kPiece == 4) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(target), "l"(source) : "memory");
      } else {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target), "l"(source) : "memory");
      }
    }
  }
};

__device__ __forceinline__ uint32_t load_shared_u16(uint32_t address) {
  uint16_t value;
  // volatile: ordered against the (volatile) copies that refill the ring, never merged with another read
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(value) : "r"(address));
  return value;
}

// The renormalisation half of a decode step, written out so that it stays branch-free and keeps its nine
// instructions: every thread whose state fell below 2^15 takes one word from the tail of the stream (the
// highest such thread the last word), all threads read the ring (masked into it) and only the needy merge.
// `cursor` is the byte offset just past the next unread word, relative to the ring's origin, and comes back
// lowered by two bytes per reader (thread 0 sees every reader, so the warp minimum is the new cursor).
template <uint32_t RING_BYTES>
__device__ __forceinline__ void renormalize_from_ring(uint32_t& state, int& cursor, uint32_t ring_address, uint32_t mask_ge) {
  asm volatile(
      "{\n\t"
      ".reg .pred need;\n\t"
      ".reg .b32 readers, at, word;\n\t"
      "setp.lt.u32 need, %0, 32768;\n\t"
      "vote.sync.ballot.b32 readers, need, 0xffffffff;\n\t"
      "and.b32 readers, readers, %3;\n\t"
      "popc.b32 readers, readers;\n\t"
      "mad.lo.s32 at, readers, -2, %1;\n\t"
      "redux.sync.min.s32 %1, at, 0xffffffff;\n\t"
      "lop3.b32 at, at, %4, %2, 0xEA;\n\t"          // (at & (RING_BYTES - 2)) | ring_address
      "ld.shared.u16 word, [at];\n\t"
      "@need prmt.b32 %0, word, %0, 0x5410;\n\t"     // state = state << 16 | word
      "}\n"
      : "+r"(state), "+r"(cursor)
      : "r"(ring_address), "r"(mask_ge), "n"(RING_BYTES - 2u)
      : "memory");
}

__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ring_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }


}  // namespace ep
