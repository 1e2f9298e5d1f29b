// Per-warp shared-memory ring of rANS payload words, filled by cp.async copies.
//
// A decoder warp consumes its stream back to front, at most 32 words per step. The ring holds four
// chunks of 128 words and is indexed by (payload word index mod 512), so a word's ring slot never
// depends on where the stream starts. The warp keeps the chunk under its cursor and the two below it
// resident and a fourth in flight; upkeep at least every four steps (<= 128 words) preserves that.
// Ring reads are masked into the ring: a corrupt stream reads stale words, never out of bounds.
#pragma once

#include "ep_common.cuh"

namespace ep {

constexpr int kChunkLog = 7;       // ring chunk: 128 words = 256 bytes = sixteen 16-byte copies
constexpr int kChunkWords = 1 << kChunkLog;
constexpr int kRingWords = 4 * kChunkWords;

// Copies chunk `chunk` of the payload into its ring slot (threads 0..15, 16 bytes each). The first
// chunks of a stream may straddle the end of the payload, so the copy length is clipped there.
__device__ __forceinline__ void ring_fetch_clipped(const uint16_t* __restrict__ payload, int64_t payload_words,
                                                   uint32_t ring_address, int chunk, uint32_t lane) {
  if (chunk < 0 || lane >= kChunkWords / 8) return;
  const int64_t word = static_cast<int64_t>(chunk) * kChunkWords + lane * 8;
  const int64_t remaining = payload_words - word;
  if (remaining <= 0) return;
  const int bytes = remaining >= 8 ? 16 : static_cast<int>(remaining) * 2;
  const uint32_t target = ring_address + static_cast<uint32_t>(((chunk & 3) * kChunkWords + lane * 8) * 2);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(target), "l"(payload + word), "r"(bytes) : "memory");
}

// Same for a chunk known to lie wholly inside the payload (any chunk below one already fetched): all
// 32 threads copy 8 bytes each. `chunk` is the same in every thread, so the test does not split the warp.
__device__ __forceinline__ void ring_fetch_interior(const uint16_t* __restrict__ payload, uint32_t ring_address, int chunk,
                                                    uint32_t lane) {
  if (chunk >= 0) {
    const uint32_t target = ring_address + static_cast<uint32_t>(((chunk & 3) * kChunkWords + lane * 4) * 2);
    const uint16_t* source = payload + (static_cast<int64_t>(chunk) * kChunkWords + lane * 4);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(target), "l"(source) : "memory");
  }
}

__device__ __forceinline__ uint32_t load_shared_u16(uint32_t address) {
  uint16_t value;
  // volatile: ordered against the (volatile) copies that refill the ring, never merged with another read
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(value) : "r"(address));
  return value;
}

__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ring_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }


}  // namespace ep
