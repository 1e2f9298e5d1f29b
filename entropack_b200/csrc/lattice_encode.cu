// EntroPack-Lossy encode kernels for sm_100a: row RMS, nearest-E8 quantisation with per-stream
// min/max, per-stream histograms, least-squares row-scale refit and the 17-table rANS encoder.
//
// Arithmetic contract (bit-exact with the CPU restatement used by the tests, and with the reference's
// quantiser, entropack/schemes/lattice_rans/eager.py:18-51 / lattice_rans.cu:59-241):
//   y = fl32(fl32(x / rms_row) / s); nearest point of D8 and of D8 + 1/2 by round-half-even plus a
//   parity fix on the largest-residual coordinate (first index on ties, +1 when the residual is 0);
//   squared distances in fp64, summed ((s0+s4)+(s2+s6))+((s1+s5)+(s3+s7)); ties go to the integer coset.
// The two row reductions (RMS, refit) use one fixed order everywhere: 256 fp32 partial sums, partial t
// taking the row's 8-element vectors t, t+256, ... in order, then a halving tree. No fused multiply-add.
#include <cuda_bf16.h>

#include <cmath>
#include <vector>

#include "ep_common.cuh"

namespace ep {
namespace {

constexpr int kThreads = 256;
constexpr int kTables = 17;
constexpr int kMinMaxLen = 34;  // 16 streams x (min, max), max coset, int16-overflow flag
constexpr int kIntMax = 0x7FFFFFFF;
constexpr int kIntMin = -0x7FFFFFFF - 1;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* x) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x[2 * j] = __uint_as_float(w[j] << 16);
    x[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load8(const float* p, float* x) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// fixed-order block reduction: 256 partials, halving tree; result valid in thread 0
__device__ __forceinline__ float tree_reduce(float* partial, float mine) {
  partial[threadIdx.x] = mine;
  __syncthreads();
  for (int width = kThreads / 2; width > 0; width >>= 1) {
    if (threadIdx.x < width) partial[threadIdx.x] = __fadd_rn(partial[threadIdx.x], partial[threadIdx.x + width]);
    __syncthreads();
  }
  const float total = partial[0];
  __syncthreads();
  return total;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) row_rms_kernel(const T* __restrict__ weight, int64_t cols, float* __restrict__ rms) {
  __shared__ float partial[kThreads];
  const int64_t row = blockIdx.x;
  const int vecs_per_row = static_cast<int>(cols >> 3);
  float acc = 0.0f;
  for (int v = threadIdx.x; v < vecs_per_row; v += kThreads) {
    float x[8];
    load8(weight + row * cols + static_cast<int64_t>(v) * 8, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = __fadd_rn(acc, __fmul_rn(x[j], x[j]));
  }
  const float total = tree_reduce(partial, acc);
  if (threadIdx.x == 0) {
    const float r = __fsqrt_rn(__fdiv_rn(total, static_cast<float>(cols)));
    rms[row] = r > 1.0e-12f ? r : 1.0e-12f;
  }
}

__device__ __forceinline__ void nearest_d8(const float* y, int* z) {
  float residual[8];
  int parity = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float f = rintf(y[j]);
    residual[j] = __fsub_rn(y[j], f);
    z[j] = static_cast<int>(f);
    parity += z[j];
  }
  if (parity & 1) {
    int at = 0;
    float largest = -1.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = fabsf(residual[j]);
      if (a > largest) {
        largest = a;
        at = j;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j == at) z[j] += residual[j] < 0.0f ? -1 : 1;
    }
  }
}

__device__ __forceinline__ double distance2(const float* y, const int* z, double offset) {
  double s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const double r = __dsub_rn(static_cast<double>(y[j]), __dadd_rn(static_cast<double>(z[j]), offset));
    s[j] = __dmul_rn(r, r);
  }
  return __dadd_rn(__dadd_rn(__dadd_rn(s[0], s[4]), __dadd_rn(s[2], s[6])), __dadd_rn(__dadd_rn(s[1], s[5]), __dadd_rn(s[3], s[7])));
}

// One thread per vector (grid-stride). fields[v] = z0..z6, m as int16; cosets[v] = 0 / 1.
// minmax (pre-set to INT_MAX / INT_MIN / 0 by the host wrapper) collects per-stream bounds.
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_kernel(const T* __restrict__ weight, const float* __restrict__ rms, float s,
                                                            int64_t vectors, int vecs_per_row, int16_t* __restrict__ fields,
                                                            uint8_t* __restrict__ cosets, int* __restrict__ minmax) {
  __shared__ int block_minmax[kMinMaxLen];
  for (int t = threadIdx.x; t < kMinMaxLen; t += kThreads) block_minmax[t] = (t < 32 && !(t & 1)) ? kIntMax : (t < 32 ? kIntMin : 0);
  __syncthreads();
  int low[2][8], high[2][8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    low[0][j] = low[1][j] = kIntMax;
    high[0][j] = high[1][j] = kIntMin;
  }
  int any_coset = 0, overflow = 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; v < vectors; v += stride) {
    const uint32_t row = static_cast<uint32_t>(v) / static_cast<uint32_t>(vecs_per_row);
    float x[8], y[8], shifted[8];
    load8(weight + v * 8, x);
    const float row_rms = rms[row];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      y[j] = __fdiv_rn(__fdiv_rn(x[j], row_rms), s);
      shifted[j] = __fsub_rn(y[j], 0.5f);
    }
    int z0[8], z1[8];
    nearest_d8(y, z0);
    nearest_d8(shifted, z1);
    const bool integer_coset = distance2(y, z0, 0.0) <= distance2(y, z1, 0.5);
    int z[8];
    int parity = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      z[j] = integer_coset ? z0[j] : z1[j];
      if (j < 7) parity += z[j];
    }
    z[7] = (z[7] - (parity & 1)) >> 1;
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int clamped = max(-32768, min(32767, z[j]));
      overflow |= clamped != z[j];
      if (integer_coset) {
        low[0][j] = min(low[0][j], z[j]);
        high[0][j] = max(high[0][j], z[j]);
      } else {
        low[1][j] = min(low[1][j], z[j]);
        high[1][j] = max(high[1][j], z[j]);
      }
      if (j & 1) packed[j >> 1] |= static_cast<uint32_t>(clamped & 0xFFFF) << 16;
      else packed[j >> 1] = static_cast<uint32_t>(clamped & 0xFFFF);
    }
    *reinterpret_cast<uint4*>(fields + v * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    cosets[v] = integer_coset ? 0 : 1;
    any_coset |= integer_coset ? 0 : 1;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int stream = j * 2 + c;
      if (low[c][j] != kIntMax) {
        atomicMin(&block_minmax[stream * 2], low[c][j]);
        atomicMax(&block_minmax[stream * 2 + 1], high[c][j]);
      }
    }
  }
  if (any_coset) atomicMax(&block_minmax[32], 1);
  if (overflow) atomicMax(&block_minmax[33], 1);
  __syncthreads();
  for (int t = threadIdx.x; t < kMinMaxLen; t += kThreads) {
    const int value = block_minmax[t];
    if (t < 32 && !(t & 1)) {
      if (value != kIntMax) atomicMin(&minmax[t], value);
    } else if (value != (t < 32 ? kIntMin : 0)) {
      atomicMax(&minmax[t], value);
    }
  }
}

// Bin layout: table 0 (coset) has 2 bins, table 1 + st has max - min + 1 bins (0 when the stream is
// empty), tables back to back. bins_used[0] receives the total; when it exceeds the capacity nothing is
// counted and the caller must fall back.
__device__ __forceinline__ void bin_layout(const int* minmax, int* offset, int* sym_min) {
  int cursor = 2;
  offset[0] = 0;
  sym_min[0] = 0;
  for (int st = 0; st < 16; ++st) {
    const bool live = minmax[st * 2] != kIntMax;
    offset[1 + st] = cursor;
    sym_min[1 + st] = live ? minmax[st * 2] : 0;
    cursor += live ? minmax[st * 2 + 1] - minmax[st * 2] + 1 : 0;
  }
  offset[kTables] = cursor;
}

// Counts go to shared-memory bins first and are folded into the global ones at the end. Where all the tables' bins fit
// the shared array they are all there; where they do not (alphabets of a thousand symbols and more: fine scales on
// heavy-tailed rows), every field table keeps a window of `shared_capacity / 16` bins around the value 0, where
// nearly all of its symbols fall, and only what lies outside takes a global atomic.
__global__ void __launch_bounds__(kThreads) histogram_kernel(const int16_t* __restrict__ fields, const uint8_t* __restrict__ cosets,
                                                             int64_t vectors, const int* __restrict__ minmax, int* __restrict__ bins,
                                                             int bins_capacity, int shared_capacity, int* __restrict__ bins_used) {
  extern __shared__ int shared_bins[];
  __shared__ int offset[kTables + 1];
  __shared__ int sym_min[kTables];
  __shared__ int window_min[kTables];    // windowed mode: the value of a table's first shared bin
  if (threadIdx.x == 0) bin_layout(minmax, offset, sym_min);
  __syncthreads();
  const int total = offset[kTables];
  if (blockIdx.x == 0 && threadIdx.x == 0) bins_used[0] = total;
  if (total > bins_capacity) return;
  const bool staged = total <= shared_capacity;
  const int window = (shared_capacity - 2) / 16;   // bins per field table in windowed mode (the coset's two come first)
  if (!staged && threadIdx.x < kTables) {
    const int t = threadIdx.x;
    // centred on 0, moved inside the table's own range where that starts above or ends below
    const int bins_here = offset[t + 1] - offset[t];
    const int first = max(sym_min[t], min(-window / 2, sym_min[t] + bins_here - window));
    window_min[t] = t == 0 ? 0 : first;
  }
  const int staged_bins = staged ? total : 2 + 16 * window;
  for (int t = threadIdx.x; t < staged_bins; t += kThreads) shared_bins[t] = 0;
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; v < vectors; v += stride) {
    const int c = cosets[v];
    const uint4 raw = *reinterpret_cast<const uint4*>(fields + v * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    atomicAdd(&shared_bins[c], 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int value = static_cast<int16_t>((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
      const int table = 1 + j * 2 + c;
      if (staged) {
        atomicAdd(&shared_bins[offset[table] + (value - sym_min[table])], 1);
      } else {
        const int in_window = value - window_min[table];
        if (static_cast<unsigned>(in_window) < static_cast<unsigned>(window)) {
          atomicAdd(&shared_bins[2 + (table - 1) * window + in_window], 1);
        } else {
          atomicAdd(&bins[offset[table] + (value - sym_min[table])], 1);
        }
      }
    }
  }
  __syncthreads();
  if (staged) {
    for (int t = threadIdx.x; t < total; t += kThreads) {
      if (shared_bins[t]) atomicAdd(&bins[t], shared_bins[t]);
    }
  } else {
    for (int t = threadIdx.x; t < staged_bins; t += kThreads) {
      const int count = shared_bins[t];
      if (!count) continue;
      if (t < 2) {
        atomicAdd(&bins[t], count);
      } else {
        const int table = 1 + (t - 2) / window;
        const int value = window_min[table] + (t - 2) % window;
        const int bin = value - sym_min[table];
        // a window may reach past a narrow table's range: nothing was counted there
        if (bin >= 0 && bin < offset[table + 1] - offset[table]) atomicAdd(&bins[offset[table] + bin], count);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) refit_kernel(const T* __restrict__ weight, const int16_t* __restrict__ fields,
                                                         const uint8_t* __restrict__ cosets, const float* __restrict__ rms, float s,
                                                         int64_t cols, float* __restrict__ scales, float* __restrict__ row_sse) {
  __shared__ float partial[kThreads];
  const int64_t row = blockIdx.x;
  const int vecs_per_row = static_cast<int>(cols >> 3);
  float numerator = 0.0f, denominator = 0.0f, energy = 0.0f;
  for (int v = threadIdx.x; v < vecs_per_row; v += kThreads) {
    const int64_t vector = row * vecs_per_row + v;
    float x[8];
    load8(weight + vector * 8, x);
    const uint4 raw = *reinterpret_cast<const uint4*>(fields + vector * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    const float half = cosets[vector] ? 0.5f : 0.0f;
    int z[8];
    int parity = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      z[j] = static_cast<int16_t>((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
      if (j < 7) parity += z[j];
    }
    z[7] = 2 * z[7] + (parity & 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float point = __fadd_rn(static_cast<float>(z[j]), half);
      numerator = __fadd_rn(numerator, __fmul_rn(x[j], point));
      denominator = __fadd_rn(denominator, __fmul_rn(point, point));
      energy = __fadd_rn(energy, __fmul_rn(x[j], x[j]));
    }
  }
  const float num = tree_reduce(partial, numerator);
  const float den = tree_reduce(partial, denominator);
  const float total_energy = row_sse ? tree_reduce(partial, energy) : 0.0f;   // same for the whole block
  if (threadIdx.x == 0) {
    const float fallback = __fmul_rn(s, rms[row]);
    float fitted = den > 0.0f ? __fdiv_rn(num, den) : fallback;
    if (!(isfinite(fitted) && fitted > 0.0f)) fitted = fallback;
    scales[row] = fitted;
    // squared error of the row at its least-squares scale: |x|^2 - (x.p)^2 / |p|^2, never below zero
    if (row_sse) row_sse[row] = den > 0.0f ? fmaxf(__fsub_rn(total_energy, __fdiv_rn(__fmul_rn(num, num), den)), 0.0f) : total_energy;
  }
}

// ---- per-row rate-distortion refinement --------------------------------------------------------------
// Per-stream bounds of symbols that are already quantised (a mixture of rows taken from several candidate
// quantisations has no quantiser pass of its own to collect them).
__global__ void __launch_bounds__(kThreads) minmax_kernel(const int16_t* __restrict__ fields, const uint8_t* __restrict__ cosets,
                                                          int64_t vectors, int* __restrict__ minmax) {
  __shared__ int block_minmax[kMinMaxLen];
  for (int t = threadIdx.x; t < kMinMaxLen; t += kThreads) block_minmax[t] = (t < 32 && !(t & 1)) ? kIntMax : (t < 32 ? kIntMin : 0);
  __syncthreads();
  int low[2][8], high[2][8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    low[0][j] = low[1][j] = kIntMax;
    high[0][j] = high[1][j] = kIntMin;
  }
  int any_coset = 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; v < vectors; v += stride) {
    const int c = cosets[v] ? 1 : 0;
    any_coset |= c;
    const uint4 raw = *reinterpret_cast<const uint4*>(fields + v * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int value = static_cast<int16_t>((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
      if (c) {
        low[1][j] = min(low[1][j], value);
        high[1][j] = max(high[1][j], value);
      } else {
        low[0][j] = min(low[0][j], value);
        high[0][j] = max(high[0][j], value);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      if (low[c][j] != kIntMax) {
        atomicMin(&block_minmax[(j * 2 + c) * 2], low[c][j]);
        atomicMax(&block_minmax[(j * 2 + c) * 2 + 1], high[c][j]);
      }
    }
  }
  if (any_coset) atomicMax(&block_minmax[32], 1);
  __syncthreads();
  for (int t = threadIdx.x; t < kMinMaxLen; t += kThreads) {
    const int value = block_minmax[t];
    if (t < 32 && !(t & 1)) {
      if (value != kIntMax) atomicMin(&minmax[t], value);
    } else if (value != (t < 32 ? kIntMin : 0)) {
      atomicMax(&minmax[t], value);
    }
  }
}

// rates[row] = sum over the row's vectors of the modelled bits of its nine symbols: the coset from table 0,
// field f given coset c from table 1 + 2 f + c (rdo.row_rates, entropack/schemes/lattice_rans/rdo.py:70-84).
// `values` holds the 17 tables back to back, table t at offsets[t] with its first entry standing for symbol
// minima[t]. A vector's nine terms are added in stream order, as in the reference; vectors are then summed in
// the fixed order of the other row reductions.
__global__ void __launch_bounds__(kThreads) row_rates_kernel(const int16_t* __restrict__ fields, const uint8_t* __restrict__ cosets,
                                                             int vecs_per_row, const float* __restrict__ values,
                                                             const int* __restrict__ offsets, const int* __restrict__ minima,
                                                             float* __restrict__ rates) {
  __shared__ float partial[kThreads];
  __shared__ int offset[kTables + 1];
  __shared__ int minimum[kTables];
  if (threadIdx.x <= kTables) offset[threadIdx.x] = offsets[threadIdx.x];
  if (threadIdx.x < kTables) minimum[threadIdx.x] = minima[threadIdx.x];
  __syncthreads();
  const int64_t row = blockIdx.x;
  float acc = 0.0f;
  for (int v = threadIdx.x; v < vecs_per_row; v += kThreads) {
    const int64_t vector = row * vecs_per_row + v;
    const int c = cosets[vector] ? 1 : 0;
    const uint4 raw = *reinterpret_cast<const uint4*>(fields + vector * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float rate = __ldg(values + offset[0] + min(c, offset[1] - offset[0] - 1));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int value = static_cast<int16_t>((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu);
      const int table = 1 + 2 * j + c;
      const int width = offset[table + 1] - offset[table];
      const int index = max(0, min(value - minimum[table], width - 1));   // the tables span every candidate's range
      rate = __fadd_rn(rate, width > 0 ? __ldg(values + offset[table] + index) : 0.0f);
    }
    acc = __fadd_rn(acc, rate);
  }
  const float total = tree_reduce(partial, acc);
  if (threadIdx.x == 0) rates[row] = total;
}

// Row r of the output is row r of candidate choice[r] (rdo.select_candidate_rows, rdo.py:103-120).
__global__ void __launch_bounds__(kThreads) select_rows_kernel(const int16_t* const* __restrict__ candidate_fields,
                                                               const uint8_t* const* __restrict__ candidate_cosets, int candidates,
                                                               const int* __restrict__ choice, int64_t vectors, int vecs_per_row,
                                                               int16_t* __restrict__ fields, uint8_t* __restrict__ cosets) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; v < vectors; v += stride) {
    const uint32_t row = static_cast<uint32_t>(v) / static_cast<uint32_t>(vecs_per_row);
    const int k = max(0, min(choice[row], candidates - 1));
    *reinterpret_cast<uint4*>(fields + v * 8) = *reinterpret_cast<const uint4*>(candidate_fields[k] + v * 8);
    cosets[v] = candidate_cosets[k][v];
  }
}

// ---- rANS encode -----------------------------------------------------------------------------------
struct EncodeParams {
  const int16_t* fields;
  const uint8_t* cosets;
  const int32_t* stream_meta;
  const uint16_t* freq_tables;
  int freq_entries;
  int64_t vectors;
  int64_t tiles;
  int tile_vectors;
  int prob_bits;
  uint16_t* scratch;      // [tiles][tile_vectors * 9]
  uint32_t* word_counts;  // [tiles]
  uint32_t* states;       // [tiles][32]
};

constexpr int kEncodeWarps = 8;
constexpr int kStagedSymbols = 6000;  // symbol records staged in shared memory (47 KB); larger alphabets read global

// Per symbol of every table (laid out like freq_tables): .x = freq | cdf << 16, .y = floor(2^32 / freq)
// (0xFFFFFFFF for freq 1); the correction step after the multiply absorbs the truncation.
__global__ void __launch_bounds__(32) symbol_tables_kernel(const int32_t* __restrict__ stream_meta,
                                                           const uint16_t* __restrict__ freq_tables, uint2* __restrict__ symbols) {
  const uint32_t lane = lane_id();
  const int t = blockIdx.x;
  const int offset = stream_meta[t * 4 + 2];
  const int alphabet = stream_meta[t * 4 + 3];
  uint32_t running = 0;
  for (int base = 0; base < alphabet; base += 32) {
    const bool live = base + static_cast<int>(lane) < alphabet;
    const uint32_t f = live ? freq_tables[offset + base + lane] : 0u;
    uint32_t inclusive = f;
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
      const uint32_t below = __shfl_up_sync(0xFFFFFFFFu, inclusive, step);
      if (lane >= static_cast<uint32_t>(step)) inclusive += below;
    }
    if (live) {
      const uint32_t cdf = running + inclusive - f;
      const uint32_t reciprocal = f > 1u ? static_cast<uint32_t>(0x100000000ull / f) : 0xFFFFFFFFu;
      symbols[offset + base + lane] = make_uint2(f | (cdf << 16), reciprocal);
    }
    running += __shfl_sync(0xFFFFFFFFu, inclusive, 31);
  }
}

// One warp per tile, forward over groups of 32 vectors; per group fields 7..0 and then the coset are
// pushed, each step emitting the low 16 bits of every state that would overflow (lower lanes first).
template <bool STAGED>
__global__ void __launch_bounds__(kEncodeWarps * 32) lattice_encode_kernel(const EncodeParams p, const uint2* __restrict__ symbols) {
  __shared__ uint2 staged_symbols[STAGED ? kStagedSymbols : 1];
  __shared__ int sym_min[kTables];
  __shared__ int freq_offset[kTables];
  if (threadIdx.x < kTables) {
    sym_min[threadIdx.x] = p.stream_meta[threadIdx.x * 4 + 1];
    freq_offset[threadIdx.x] = p.stream_meta[threadIdx.x * 4 + 2];
  }
  if (STAGED) {
    for (int i = threadIdx.x; i < p.freq_entries; i += kEncodeWarps * 32) staged_symbols[i] = symbols[i];
  }
  __syncthreads();
  const uint32_t lane = lane_id();
  const uint32_t mask_lt = lanemask_lt();
  const int64_t tile = static_cast<int64_t>(blockIdx.x) * kEncodeWarps + (threadIdx.x >> 5);
  if (tile >= p.tiles) return;
  const int64_t tile_begin = tile * p.tile_vectors;
  const int count = static_cast<int>(min(static_cast<int64_t>(p.tile_vectors), p.vectors - tile_begin));
  uint16_t* const slot = p.scratch + tile * p.tile_vectors * 9;
  const uint32_t emit_shift = 31 - p.prob_bits;
  const int prob_bits = p.prob_bits;
  uint32_t x = kStateMin;
  uint32_t emitted = 0;

  auto push = [&](bool valid, int record) {
    const uint2 info = valid ? (STAGED ? staged_symbols[record] : __ldg(symbols + record)) : make_uint2(1u, 0xFFFFFFFFu);
    const uint32_t f = info.x & 0xFFFFu;
    const bool emit = valid && x >= (f << emit_shift);
    const uint32_t vote = __ballot_sync(0xFFFFFFFFu, emit);
    if (emit) {
      slot[emitted + __popc(vote & mask_lt)] = static_cast<uint16_t>(x);
      x >>= 16;
    }
    emitted += __popc(vote);
    if (valid) {
      uint32_t q = __umulhi(x, info.y);
      uint32_t r = x - q * f;
      if (r >= f) {
        r -= f;
        q += 1;
      }
      x = (q << prob_bits) + r + (info.x >> 16);
    }
  };

  for (int base = 0; base < count; base += 32) {
    const bool valid = base + static_cast<int>(lane) < count;
    const int64_t vector = tile_begin + base + lane;
    uint4 raw = make_uint4(0, 0, 0, 0);
    int c = 0;
    if (valid) {
      raw = *reinterpret_cast<const uint4*>(p.fields + vector * 8);
      c = p.cosets[vector];
    }
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int field = 7; field >= 0; --field) {
      const int value = static_cast<int16_t>((w[field >> 1] >> (16 * (field & 1))) & 0xFFFFu);
      const int table = 1 + 2 * field + c;
      push(valid, freq_offset[table] + (value - sym_min[table]));
    }
    push(valid, freq_offset[0] + c);
  }
  p.states[tile * kNumStates + lane] = x;
  if (lane == 0) p.word_counts[tile] = emitted;
}

template <typename T>
int launch_rows(const T* weight, int64_t rows, int64_t cols, float* rms, cudaStream_t s) {
  row_rms_kernel<T><<<static_cast<unsigned>(rows), kThreads, 0, s>>>(weight, cols, rms);
  return check_launch("row_rms_kernel");
}

int check_matrix(const void* weight, int64_t rows, int64_t cols) {
  if (!weight || rows <= 0 || cols <= 0 || (cols & 7) != 0) return EP_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(weight) & 15u) return EP_ERR_INVALID_ARGUMENT;
  if (rows > 0x7FFFFFFF || rows * (cols / 8) >= (int64_t(1) << 31)) return EP_ERR_TOO_LARGE;
  return EP_OK;
}

}  // namespace
}  // namespace ep

using namespace ep;

extern "C" int ep_lattice_row_rms(const void* weight_dev, int is_bf16, int64_t rows, int64_t cols, float* rms_dev,
                                  ep_stream_t stream) {
  const int rc = check_matrix(weight_dev, rows, cols);
  if (rc != EP_OK || !rms_dev) return rc != EP_OK ? rc : EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return is_bf16 ? launch_rows(static_cast<const __nv_bfloat16*>(weight_dev), rows, cols, rms_dev, s)
                 : launch_rows(static_cast<const float*>(weight_dev), rows, cols, rms_dev, s);
}

extern "C" int ep_lattice_quantize(const void* weight_dev, int is_bf16, const float* rms_dev, int64_t rows, int64_t cols,
                                   float scale, int16_t* fields_dev, uint8_t* cosets_dev, int32_t* minmax_dev,
                                   ep_stream_t stream) {
  const int rc = check_matrix(weight_dev, rows, cols);
  if (rc != EP_OK) return rc;
  if (!rms_dev || !fields_dev || !cosets_dev || !minmax_dev || !(scale > 0.0f)) return EP_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(fields_dev) & 15u) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int initial[kMinMaxLen];
  for (int t = 0; t < kMinMaxLen; ++t) initial[t] = (t < 32 && !(t & 1)) ? kIntMax : (t < 32 ? kIntMin : 0);
  EP_CUDA_CHECK(cudaMemcpyAsync(minmax_dev, initial, sizeof(initial), cudaMemcpyHostToDevice, s));
  const int64_t vectors = rows * (cols / 8);
  const int64_t wanted = (vectors + kThreads - 1) / kThreads;
  const unsigned blocks = static_cast<unsigned>(wanted < kSmCount * 8 ? wanted : kSmCount * 8);
  const int vecs_per_row = static_cast<int>(cols / 8);
  if (is_bf16) {
    quantize_kernel<<<blocks, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(weight_dev), rms_dev, scale, vectors, vecs_per_row,
                                                fields_dev, cosets_dev, minmax_dev);
  } else {
    quantize_kernel<<<blocks, kThreads, 0, s>>>(static_cast<const float*>(weight_dev), rms_dev, scale, vectors, vecs_per_row,
                                                fields_dev, cosets_dev, minmax_dev);
  }
  return check_launch("quantize_kernel");
}

extern "C" int ep_lattice_histogram(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t vectors,
                                    const int32_t* minmax_dev, int32_t* bins_dev, int64_t bins_capacity, int32_t* bins_used_dev,
                                    ep_stream_t stream) {
  if (!fields_dev || !cosets_dev || !minmax_dev || !bins_dev || !bins_used_dev || vectors <= 0 || bins_capacity <= 0 ||
      bins_capacity > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EP_CUDA_CHECK(cudaMemsetAsync(bins_dev, 0, sizeof(int32_t) * bins_capacity, s));
  constexpr int kSharedBins = 10240;  // 40 KB of dynamic shared memory
  const int64_t wanted = (vectors + kThreads - 1) / kThreads;
  const unsigned blocks = static_cast<unsigned>(wanted < kSmCount * 4 ? wanted : kSmCount * 4);
  histogram_kernel<<<blocks, kThreads, kSharedBins * sizeof(int), s>>>(fields_dev, cosets_dev, vectors, minmax_dev, bins_dev,
                                                                       static_cast<int>(bins_capacity), kSharedBins, bins_used_dev);
  return check_launch("histogram_kernel");
}

// Layout of the statistics buffer the search and the encoder share: the min/max record, the count of bins it
// implies, one pad word (keeps the bins 16-byte aligned), then the bins.
constexpr int kStatsUsedAt = kMinMaxLen;
constexpr int kStatsHeaderWords = kMinMaxLen + 2;

extern "C" int ep_lattice_search_scale(const void* weight_dev, int is_bf16, const float* rms_dev, int64_t rows, int64_t cols,
                                       int16_t* fields_dev, uint8_t* cosets_dev, int32_t* stats_dev, int64_t bins_capacity,
                                       double target_bpp, int prob_bits, int64_t tile_elements, int iterations, double low,
                                       double high, double fixed_bytes, double* scale_host, int64_t* bins_needed_host,
                                       ep_stream_t stream) {
  const int rc = check_matrix(weight_dev, rows, cols);
  if (rc != EP_OK) return rc;
  if (!stats_dev || !scale_host || !bins_needed_host || bins_capacity <= 0 || iterations < 0 || !(low > 0.0) || !(high >= low)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t vectors = rows * (cols / 8);
  const double elements = static_cast<double>(rows) * static_cast<double>(cols);
  // Most searches use a few thousand bins: the header and that many come back in one copy, the rest only when needed.
  const int64_t first_bins = bins_capacity < 4096 ? bins_capacity : 4096;
  std::vector<int32_t> host(static_cast<size_t>(kStatsHeaderWords + bins_capacity));
  *bins_needed_host = 0;
  for (int step = 0; step < iterations; ++step) {
    const double middle = std::sqrt(low * high);
    int status = ep_lattice_quantize(weight_dev, is_bf16, rms_dev, rows, cols, static_cast<float>(middle), fields_dev, cosets_dev,
                                     stats_dev, stream);
    if (status != EP_OK) return status;
    status = ep_lattice_histogram(fields_dev, cosets_dev, vectors, stats_dev, stats_dev + kStatsHeaderWords, bins_capacity,
                                  stats_dev + kStatsUsedAt, stream);
    if (status != EP_OK) return status;
    EP_CUDA_CHECK(cudaMemcpyAsync(host.data(), stats_dev, sizeof(int32_t) * (kStatsHeaderWords + first_bins), cudaMemcpyDeviceToHost, s));
    EP_CUDA_CHECK(cudaStreamSynchronize(s));
    const int64_t used = host[kStatsUsedAt];
    if (used > bins_capacity) {
      *bins_needed_host = used;
      return EP_MORE_BINS;
    }
    if (used > first_bins) {
      EP_CUDA_CHECK(cudaMemcpyAsync(host.data() + kStatsHeaderWords + first_bins, stats_dev + kStatsHeaderWords + first_bins,
                                    sizeof(int32_t) * (used - first_bins), cudaMemcpyDeviceToHost, s));
      EP_CUDA_CHECK(cudaStreamSynchronize(s));
    }
    double total = HUGE_VAL;   // a field that left the int16 range: far too fine a scale for any table
    if (host[kMinMaxLen - 1] == 0) {
      status = ep_lattice_coded_bytes(host.data(), host.data() + kStatsHeaderWords, vectors, prob_bits, tile_elements, &total);
      if (status != EP_OK) return status;
    }
    total += static_cast<double>(rows) * 4.0 + fixed_bytes;
    if (8.0 * total / elements > target_bpp) {
      low = middle;
    } else {
      high = middle;
    }
  }
  *scale_host = std::sqrt(low * high);
  return EP_OK;
}

extern "C" int ep_lattice_refit_scales(const void* weight_dev, int is_bf16, const int16_t* fields_dev, const uint8_t* cosets_dev,
                                       const float* rms_dev, float scale, int64_t rows, int64_t cols, float* scales_dev,
                                       ep_stream_t stream) {
  const int rc = check_matrix(weight_dev, rows, cols);
  if (rc != EP_OK) return rc;
  if (!fields_dev || !cosets_dev || !rms_dev || !scales_dev) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16) {
    refit_kernel<<<static_cast<unsigned>(rows), kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(weight_dev), fields_dev, cosets_dev,
                                                                  rms_dev, scale, cols, scales_dev, nullptr);
  } else {
    refit_kernel<<<static_cast<unsigned>(rows), kThreads, 0, s>>>(static_cast<const float*>(weight_dev), fields_dev, cosets_dev, rms_dev,
                                                                  scale, cols, scales_dev, nullptr);
  }
  return check_launch("refit_kernel");
}

extern "C" int ep_lattice_refit_rows(const void* weight_dev, int is_bf16, const int16_t* fields_dev, const uint8_t* cosets_dev,
                                     const float* rms_dev, float scale, int64_t rows, int64_t cols, float* scales_dev,
                                     float* row_sse_dev, ep_stream_t stream) {
  const int rc = check_matrix(weight_dev, rows, cols);
  if (rc != EP_OK) return rc;
  if (!fields_dev || !cosets_dev || !rms_dev || !scales_dev || !row_sse_dev) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16) {
    refit_kernel<<<static_cast<unsigned>(rows), kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(weight_dev), fields_dev, cosets_dev,
                                                                  rms_dev, scale, cols, scales_dev, row_sse_dev);
  } else {
    refit_kernel<<<static_cast<unsigned>(rows), kThreads, 0, s>>>(static_cast<const float*>(weight_dev), fields_dev, cosets_dev, rms_dev,
                                                                  scale, cols, scales_dev, row_sse_dev);
  }
  return check_launch("refit_kernel");
}

extern "C" int ep_lattice_minmax(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t vectors, int32_t* minmax_dev,
                                 ep_stream_t stream) {
  if (!fields_dev || !cosets_dev || !minmax_dev || vectors <= 0) return EP_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(fields_dev) & 15u) return EP_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int initial[kMinMaxLen];
  for (int t = 0; t < kMinMaxLen; ++t) initial[t] = (t < 32 && !(t & 1)) ? kIntMax : (t < 32 ? kIntMin : 0);
  EP_CUDA_CHECK(cudaMemcpyAsync(minmax_dev, initial, sizeof(initial), cudaMemcpyHostToDevice, s));
  const int64_t wanted = (vectors + kThreads - 1) / kThreads;
  const unsigned blocks = static_cast<unsigned>(wanted < kSmCount * 8 ? wanted : kSmCount * 8);
  minmax_kernel<<<blocks, kThreads, 0, s>>>(fields_dev, cosets_dev, vectors, minmax_dev);
  return check_launch("minmax_kernel");
}

extern "C" int ep_lattice_row_rates(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t rows, int64_t cols,
                                    const float* rate_values_dev, const int32_t* rate_offsets_dev, const int32_t* rate_minima_dev,
                                    float* rates_dev, ep_stream_t stream) {
  if (!fields_dev || !cosets_dev || !rate_values_dev || !rate_offsets_dev || !rate_minima_dev || !rates_dev || rows <= 0 ||
      cols <= 0 || (cols & 7) != 0 || rows > 0x7FFFFFFF || cols / 8 > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (reinterpret_cast<uintptr_t>(fields_dev) & 15u) return EP_ERR_INVALID_ARGUMENT;
  row_rates_kernel<<<static_cast<unsigned>(rows), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      fields_dev, cosets_dev, static_cast<int>(cols / 8), rate_values_dev, rate_offsets_dev, rate_minima_dev, rates_dev);
  return check_launch("row_rates_kernel");
}

extern "C" int ep_lattice_select_rows(const int16_t* const* candidate_fields_dev, const uint8_t* const* candidate_cosets_dev,
                                      int candidates, const int32_t* choice_dev, int64_t rows, int64_t cols, int16_t* fields_dev,
                                      uint8_t* cosets_dev, ep_stream_t stream) {
  if (!candidate_fields_dev || !candidate_cosets_dev || candidates <= 0 || !choice_dev || !fields_dev || !cosets_dev || rows <= 0 ||
      cols <= 0 || (cols & 7) != 0 || cols / 8 > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  const int64_t vectors = rows * (cols / 8);
  if (vectors >= (int64_t(1) << 32)) return EP_ERR_TOO_LARGE;
  const int64_t wanted = (vectors + kThreads - 1) / kThreads;
  const unsigned blocks = static_cast<unsigned>(wanted < kSmCount * 8 ? wanted : kSmCount * 8);
  select_rows_kernel<<<blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      candidate_fields_dev, candidate_cosets_dev, candidates, choice_dev, vectors, static_cast<int>(cols / 8), fields_dev, cosets_dev);
  return check_launch("select_rows_kernel");
}

extern "C" int64_t ep_lattice_encode_scratch_words(int64_t vectors, int64_t tile_elements) {
  if (vectors <= 0 || tile_elements <= 0) return EP_ERR_INVALID_ARGUMENT;
  const int64_t tile_vectors = tile_elements / 9 < 32 ? 32 : tile_elements / 9;
  const int64_t tiles = (vectors + tile_vectors - 1) / tile_vectors;
  return tiles * tile_vectors * 9;
}

extern "C" int ep_lattice_encode(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t vectors,
                                 const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev, int64_t freq_entries,
                                 int prob_bits, int64_t tile_elements, void* symbol_scratch_dev, uint16_t* scratch_dev,
                                 uint32_t* word_counts_dev, uint32_t* states_dev, ep_stream_t stream) {
  if (!fields_dev || !cosets_dev || !stream_meta_dev || !freq_tables_dev || !symbol_scratch_dev || !scratch_dev ||
      !word_counts_dev || !states_dev || vectors <= 0 || vectors >= (int64_t(1) << 31) || freq_entries <= 0 ||
      freq_entries > 17 * 32768 || prob_bits < 9 || prob_bits > 15 || tile_elements <= 0) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (reinterpret_cast<uintptr_t>(symbol_scratch_dev) & 7u) return EP_ERR_INVALID_ARGUMENT;
  EncodeParams p;
  p.fields = fields_dev;
  p.cosets = cosets_dev;
  p.stream_meta = stream_meta_dev;
  p.freq_tables = freq_tables_dev;
  p.freq_entries = static_cast<int>(freq_entries);
  p.vectors = vectors;
  const int64_t tile_vectors = tile_elements / 9 < 32 ? 32 : tile_elements / 9;
  if (tile_vectors > 0x7FFFFFFF / 9) return EP_ERR_TOO_LARGE;
  p.tile_vectors = static_cast<int>(tile_vectors);
  p.tiles = (vectors + tile_vectors - 1) / tile_vectors;
  p.prob_bits = prob_bits;
  p.scratch = scratch_dev;
  p.word_counts = word_counts_dev;
  p.states = states_dev;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint2* symbols = static_cast<uint2*>(symbol_scratch_dev);
  symbol_tables_kernel<<<kTables, 32, 0, s>>>(stream_meta_dev, freq_tables_dev, symbols);
  const unsigned blocks = static_cast<unsigned>((p.tiles + kEncodeWarps - 1) / kEncodeWarps);
  if (freq_entries <= kStagedSymbols) {
    lattice_encode_kernel<true><<<blocks, kEncodeWarps * 32, 0, s>>>(p, symbols);
  } else {
    lattice_encode_kernel<false><<<blocks, kEncodeWarps * 32, 0, s>>>(p, symbols);
  }
  return check_launch("lattice_encode_kernel");
}
