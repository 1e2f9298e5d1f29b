// Shared device helpers and host-side launch plumbing for the entropack_b200 kernels (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/entropack_b200.h"

namespace ep {

constexpr int kNumStates = 32;            // interleaved rANS states per tile == one warp
constexpr uint32_t kStateMin = 1u << 15;  // renormalisation threshold, 16-bit words
constexpr int kSmCount = 148;             // B200

// How many SMs the calling thread's next launches of the lossy decode / the tensor-core product may fill
// (ep_set_sm_limits); kSmCount when no limit is set.
int decode_sm_limit();
int product_sm_limit();

// Records the first CUDA failure text for ep_last_cuda_error() and maps it to EP_ERR_CUDA.
int record_cuda_error(cudaError_t error, const char* where);

#define EP_CUDA_CHECK(expr)                                              \
  do {                                                                   \
    const cudaError_t ep_cuda_status_ = (expr);                          \
    if (ep_cuda_status_ != cudaSuccess) {                                \
      return ::ep::record_cuda_error(ep_cuda_status_, #expr);            \
    }                                                                    \
  } while (0)

inline int check_launch(const char* where) {
  const cudaError_t error = cudaGetLastError();
  return error == cudaSuccess ? EP_OK : record_cuda_error(error, where);
}

// The special-register reads are volatile so the compiler keeps the value in a register instead of
// re-reading the (slow) special register wherever it is used.
__device__ __forceinline__ uint32_t lane_id() {
  uint32_t lane;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(lane));
  return lane;
}

__device__ __forceinline__ uint32_t lanemask_ge() {
  uint32_t mask;
  asm volatile("mov.u32 %0, %%lanemask_ge;" : "=r"(mask));
  return mask;
}

__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t mask;
  asm volatile("mov.u32 %0, %%lanemask_lt;" : "=r"(mask));
  return mask;
}

__device__ __forceinline__ void report(int* error, int code) {
  if (error != nullptr) atomicCAS(error, 0, code);
}

// Warp-wide renormalisation read of the reverse (decoder) direction. Every lane whose state fell
// below 2^15 takes one 16-bit word from the tail of the stream; among the readers the highest lane
// takes the last word. `position` is the warp-uniform count of words still unread, relative to
// `words`. A read that would fall before the stream start returns 0 instead of touching memory, so a
// corrupt stream yields wrong symbols, never a fault; `position` going negative is the underrun
// signal the caller checks at the end of the tile.
__device__ __forceinline__ void renormalize(bool valid, uint32_t& state, const uint16_t* __restrict__ words, int& position,
                                            uint32_t mask_ge) {
  const bool need = valid && state < kStateMin;
  const uint32_t vote = __ballot_sync(0xFFFFFFFFu, need);
  if (need) {
    const int index = position - static_cast<int>(__popc(vote & mask_ge));
    const uint32_t word = index >= 0 ? static_cast<uint32_t>(__ldg(words + index)) : 0u;
    state = (state << 16) | word;
  }
  position -= __popc(vote);
}

}  // namespace ep
