// y[M,N] = x[M,K] . W[N,K]^T (+ bias) in bf16 with fp32 accumulation: the GEMM behind CompressedLinear.forward.
//
// W is the weight the fused decode kernel has just written (K-contiguous rows, exactly the K-major B
// operand); for the layer shapes in question it is still resident in the 126 MB L2 when this runs.
//
//   * M <= 16: `linear_stream_kernel` -- a bandwidth kernel: the weight goes from global memory straight
//     into m16n8k16 fragments, eight features per block, K split over the block's eight warps.
//   * M > 16: `linear_tcgen05_kernel` -- persistent blocks, 128 x TILE_N output tiles on the 5th-generation
//     tensor cores. TMA (cp.async.bulk.tensor, 128-byte swizzle) fills a shared-memory ring of A and B
//     tiles; one elected thread issues tcgen05.mma (M128 x TILE_N x K16, fp32 accumulators in TMEM) straight
//     from shared memory; four warps read an accumulator back with tcgen05.ld, add the bias, round to bf16
//     and store, while the MMA thread already fills the second accumulator buffer with the block's next
//     tile. TILE_N (32..256) is chosen per call. Every mbarrier wait is bounded: on a timeout the block
//     raises the error word, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>

#include "ep_common.cuh"

namespace ep {
namespace {

// ------------------------------------------------------------------------------------------------
// few rows of activations: the weight is streamed once, straight into MMA fragments
// ------------------------------------------------------------------------------------------------
// With M <= 64 the product is a pass over the weight at memory speed, and the 128-row tcgen05 tile is the
// wrong tool: its shortest instruction still reads 128 rows of A from shared memory, so a narrow tile is
// bound by instruction issue, not by bytes. Here a block of eight warps owns eight output features. Each
// warp takes every eighth 32-element slice of K: a thread loads 16 bytes (8 consecutive k) of its feature's
// weight row -- the block's loads cover whole 64-byte runs of eight rows -- and the matching 16 bytes of
// each activation row it needs (a few hundred KB in all, so they come from L1/L2), and feeds them to two
// m16n8k16 tensor-core instructions. The instruction's k index is only a summation index, so "thread t
// holds k = 8t .. 8t+7" is as good as the canonical fragment order as long as A and B agree. The eight
// partial tiles meet in shared memory at the end. Nothing is staged, every load of a thread is independent
// of the others, and the loop is unrolled so that half a dozen 16-byte loads per thread are in flight.
constexpr int kStreamThreads = 256;
constexpr int kStreamWarps = kStreamThreads / 32;
constexpr int kStreamMaxM = 16;
// Four blocks to an SM hold a 3840-feature layer's 480 blocks in one wave and leave the compiler 64 registers: told so, it
// keeps more loads in flight than with the 40 it takes unprompted (16.4 -> 14.3 us at 3840 x 3840); eight-fold
// unrolling at 80 or more registers runs in two waves and takes 22 us or more.
constexpr int kStreamBlocksPerSm = 4;

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// GROUPS sets of eight output features per block: a warp multiplies the activation fragments it has loaded with
// GROUPS weight fragments, so a wide layer (10240 features: 1280 sets) still runs as one wave of blocks -- 427 blocks of
// three sets instead of 1280 of one, which would take more than two -- and reads the activations a third as often.
template <int GROUPS>
__global__ void __launch_bounds__(kStreamThreads, GROUPS == 1 ? kStreamBlocksPerSm : kStreamBlocksPerSm - 1)
linear_stream_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                     __nv_bfloat16* __restrict__ y, int m, int n, int k) {
  __shared__ float partial[kStreamWarps][GROUPS][4][32];
  const uint32_t lane = lane_id();
  const int warp = threadIdx.x >> 5;
  const int group = lane >> 2;      // feature within a set of eight / activation row
  const int quad = lane & 3;        // which 8 of the slice's 32 k
  const int first = blockIdx.x * 8 * GROUPS;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const uint4* w_row[GROUPS];
  bool real[GROUPS];
  float acc[GROUPS][4];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    const int feature = first + 8 * g + group;
    real[g] = feature < n;
    w_row[g] = reinterpret_cast<const uint4*>(w + static_cast<int64_t>(min(feature, n - 1)) * k);
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.0f;
  }
  const int upper = group, lower = group + 8;

  const int slices = (k + 31) / 32;
#pragma unroll 2
  for (int slice = warp; slice < slices; slice += kStreamWarps) {
    const int at = slice * 32 + quad * 8;                 // first k of this thread's 16 bytes
    const bool inside = at < k;                           // k is a multiple of 8: a 16-byte piece is in or out as a whole
    uint4 b[GROUPS];
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) b[g] = inside && real[g] ? __ldg(w_row[g] + (at >> 3)) : zero;
    const uint4 au = inside && upper < m ? __ldg(reinterpret_cast<const uint4*>(x + static_cast<int64_t>(upper) * k + at)) : zero;
    const uint4 al = inside && lower < m ? __ldg(reinterpret_cast<const uint4*>(x + static_cast<int64_t>(lower) * k + at)) : zero;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      mma_m16n8k16(acc[g], au.x, al.x, au.y, al.y, b[g].x, b[g].y);
      mma_m16n8k16(acc[g], au.z, al.z, au.w, al.w, b[g].z, b[g].w);
    }
  }
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
#pragma unroll
    for (int j = 0; j < 4; ++j) partial[warp][g][j][lane] = acc[g][j];
  }
  __syncthreads();
  // accumulator fragment: c0, c1 = (row group, columns 2 quad, 2 quad + 1), c2, c3 = the same columns of row group + 8
  for (int item = threadIdx.x; item < GROUPS * 4 * 32; item += kStreamThreads) {
    const int g = item / 128, j = (item >> 5) & 3, holder = item & 31;
    float total = 0.0f;
#pragma unroll
    for (int v = 0; v < kStreamWarps; ++v) total += partial[v][g][j][holder];
    const int row = (holder >> 2) + (j >= 2 ? 8 : 0);
    const int column = first + 8 * g + (holder & 3) * 2 + (j & 1);
    if (row < m && column < n) {
      const float bias_value = bias ? __bfloat162float(bias[column]) : 0.0f;
      y[static_cast<int64_t>(row) * n + column] = __float2bfloat16_rn(total + bias_value);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// per-row 8-bit quantisation of activations (QuantizedLinear._quantize_rows, entropack/linear/linear.py:286-293)
// ------------------------------------------------------------------------------------------------
// scale = max(absmax / 448, eps); code = e4m3(clamp(fl32(x / scale), -448, 448)), round to nearest even.
__device__ __forceinline__ float as_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float as_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float as_float(float v) { return v; }

// INT8: scale = max(absmax / 127, eps), code = clamp(rint(x / scale), -127, 127) (round half to even, like torch.round).
template <bool INT8> __device__ __forceinline__ uint8_t quantize_value(float value, float scale) {
  if (INT8) {
    const float scaled = fminf(fmaxf(rintf(__fdiv_rn(value, scale)), -127.0f), 127.0f);
    return static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(scaled)));
  }
  const float scaled = fminf(fmaxf(__fdiv_rn(value, scale), -448.0f), 448.0f);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3));
}

// One block per row. `VECTOR`: the row is read 16 bytes at a time (8 bf16 / fp16 or 4 fp32 values) and its codes are
// written 8 or 4 at a time; the host picks it when every row starts on a 16-byte boundary. The second pass over the
// row (a few KB) comes out of L1.
template <typename T, bool INT8, bool VECTOR>
__global__ void __launch_bounds__(256) quantize_rows_8bit_kernel(const T* __restrict__ x, int64_t cols, uint8_t* __restrict__ codes,
                                                                 float* __restrict__ scales) {
  constexpr int kVector = 16 / sizeof(T);
  __shared__ float partial[8];
  __shared__ float row_scale;
  const T* row = x + static_cast<int64_t>(blockIdx.x) * cols;
  float largest = 0.0f;
  if (VECTOR) {
    for (int64_t c = static_cast<int64_t>(threadIdx.x) * kVector; c < cols; c += 256 * kVector) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
      const T* values = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < kVector; ++i) largest = fmaxf(largest, fabsf(as_float(values[i])));
    }
  } else {
    for (int64_t c = threadIdx.x; c < cols; c += 256) largest = fmaxf(largest, fabsf(as_float(row[c])));
  }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xFFFFFFFFu, largest, step));
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = largest;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = partial[0];
    for (int w = 1; w < 8; ++w) total = fmaxf(total, partial[w]);
    // absmax / 448 the way torch evaluates a division by a host scalar on a GPU: times the fp32 reciprocal;
    // clamped at the float32 epsilon like the reference
    row_scale = fmaxf(__fmul_rn(total, __fdiv_rn(1.0f, INT8 ? 127.0f : 448.0f)), 1.1920928955078125e-07f);
    scales[blockIdx.x] = row_scale;
  }
  __syncthreads();
  const float scale = row_scale;
  uint8_t* out = codes + static_cast<int64_t>(blockIdx.x) * cols;
  if (VECTOR) {
    for (int64_t c = static_cast<int64_t>(threadIdx.x) * kVector; c < cols; c += 256 * kVector) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
      const T* values = reinterpret_cast<const T*>(&raw);
      uint32_t packed[kVector / 4];
#pragma unroll
      for (int i = 0; i < kVector; i += 4) {
        packed[i / 4] = static_cast<uint32_t>(quantize_value<INT8>(as_float(values[i]), scale)) |
                        static_cast<uint32_t>(quantize_value<INT8>(as_float(values[i + 1]), scale)) << 8 |
                        static_cast<uint32_t>(quantize_value<INT8>(as_float(values[i + 2]), scale)) << 16 |
                        static_cast<uint32_t>(quantize_value<INT8>(as_float(values[i + 3]), scale)) << 24;
      }
      if (kVector == 8) {
        *reinterpret_cast<uint2*>(out + c) = make_uint2(packed[0], packed[kVector / 4 - 1]);
      } else {
        *reinterpret_cast<uint32_t*>(out + c) = packed[0];
      }
    }
  } else {
    for (int64_t c = threadIdx.x; c < cols; c += 256) out[c] = quantize_value<INT8>(as_float(row[c]), scale);
  }
}

// The same, for rows of at most 256 * HELD 16-byte pieces (4096 bf16 values at HELD = 2): a thread keeps its pieces in
// registers between the maximum and the conversion, so the row is read once, and every thread derives the scale from
// the eight warp maxima itself, so the block meets at one barrier. FP8 codes are converted two at a time.
template <typename T, bool INT8, int HELD>
__global__ void __launch_bounds__(256) quantize_rows_held_kernel(const T* __restrict__ x, int64_t cols, uint8_t* __restrict__ codes,
                                                                 float* __restrict__ scales) {
  constexpr int kVector = 16 / sizeof(T);
  __shared__ float partial[8];
  const T* row = x + static_cast<int64_t>(blockIdx.x) * cols;
  uint4 held[HELD];
  float largest = 0.0f;
#pragma unroll
  for (int h = 0; h < HELD; ++h) {
    const int64_t c = static_cast<int64_t>(h * 256 + static_cast<int>(threadIdx.x)) * kVector;
    held[h] = c < cols ? __ldcs(reinterpret_cast<const uint4*>(row + c)) : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int h = 0; h < HELD; ++h) {
    const T* values = reinterpret_cast<const T*>(&held[h]);
#pragma unroll
    for (int i = 0; i < kVector; ++i) largest = fmaxf(largest, fabsf(as_float(values[i])));
  }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xFFFFFFFFu, largest, step));
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = largest;
  __syncthreads();
  float total = partial[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) total = fmaxf(total, partial[w]);
  const float scale = fmaxf(__fmul_rn(total, __fdiv_rn(1.0f, INT8 ? 127.0f : 448.0f)), 1.1920928955078125e-07f);
  if (threadIdx.x == 0) scales[blockIdx.x] = scale;
  uint8_t* out = codes + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
  for (int h = 0; h < HELD; ++h) {
    const int64_t c = static_cast<int64_t>(h * 256 + static_cast<int>(threadIdx.x)) * kVector;
    if (c >= cols) continue;
    const T* values = reinterpret_cast<const T*>(&held[h]);
    uint32_t packed[kVector / 4];
#pragma unroll
    for (int i = 0; i < kVector; i += 4) {
      if (INT8) {
        packed[i / 4] = static_cast<uint32_t>(quantize_value<true>(as_float(values[i]), scale)) |
                        static_cast<uint32_t>(quantize_value<true>(as_float(values[i + 1]), scale)) << 8 |
                        static_cast<uint32_t>(quantize_value<true>(as_float(values[i + 2]), scale)) << 16 |
                        static_cast<uint32_t>(quantize_value<true>(as_float(values[i + 3]), scale)) << 24;
      } else {
        float scaled[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) scaled[j] = fminf(fmaxf(__fdiv_rn(as_float(values[i + j]), scale), -448.0f), 448.0f);
        const uint32_t low = __nv_cvt_float2_to_fp8x2(make_float2(scaled[0], scaled[1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t high = __nv_cvt_float2_to_fp8x2(make_float2(scaled[2], scaled[3]), __NV_SATFINITE, __NV_E4M3);
        packed[i / 4] = low | high << 16;
      }
    }
    if (kVector == 8) {
      *reinterpret_cast<uint2*>(out + c) = make_uint2(packed[0], packed[kVector / 4 - 1]);
    } else {
      *reinterpret_cast<uint32_t*>(out + c) = packed[0];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// ConvRot: y = x . R per group of `group` consecutive features (entropack/linear/convrot.py:35-61)
// ------------------------------------------------------------------------------------------------
// R is the Kronecker power of the 4 x 4 matrix ((1,1,1,-1),(1,1,-1,1),(1,-1,1,1),(-1,1,1,1)) divided by sqrt(group):
// symmetric and its own inverse, so the same pass rotates activations, rotates weight rows and undoes either. A
// Kronecker power factors into one radix-4 butterfly pass per base-4 digit of the index, so a row costs
// log4(group) passes over fp32 values in shared memory instead of a group x group product.
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }

template <typename T>
__global__ void __launch_bounds__(256) convrot_rows_kernel(const T* __restrict__ x, int64_t cols, int group, T* __restrict__ y) {
  extern __shared__ float row_values[];
  const T* source = x + static_cast<int64_t>(blockIdx.x) * cols;
  for (int64_t c = threadIdx.x; c < cols; c += 256) row_values[c] = as_float(source[c]);
  __syncthreads();
  const int64_t quads = cols / 4;
  for (int stride = 1; stride < group; stride *= 4) {
    for (int64_t q = threadIdx.x; q < quads; q += 256) {
      // the q-th index whose base-4 digit at this stride is zero
      const int64_t base = (q / stride) * stride * 4 + q % stride;
      const float a = row_values[base], b = row_values[base + stride], c = row_values[base + 2 * stride], d = row_values[base + 3 * stride];
      row_values[base] = (a + b) + (c - d);
      row_values[base + stride] = (a + b) - (c - d);
      row_values[base + 2 * stride] = (a - b) + (c + d);
      row_values[base + 3 * stride] = (c + d) - (a - b);
    }
    __syncthreads();
  }
  const float scale = rsqrtf(static_cast<float>(group));
  T* target = y + static_cast<int64_t>(blockIdx.x) * cols;
  for (int64_t c = threadIdx.x; c < cols; c += 256) target[c] = from_float<T>(row_values[c] * scale);
}

// ------------------------------------------------------------------------------------------------
// tcgen05 GEMM
// ------------------------------------------------------------------------------------------------
constexpr int kTileM = 128;
constexpr int kTileK = 64;               // 64 bf16 = one 128-byte swizzle row
constexpr int kTileBytesA = kTileM * kTileK * 2;        // 16 KB
constexpr int kEpilogueWarps = 8;        // two per TMEM lane quadrant, each draining half of the tile's columns
constexpr int kGemmThreads = 64 + 32 * kEpilogueWarps;   // warp 0: TMA, warp 1: MMA + TMEM owner, the rest: epilogue
constexpr uint32_t kWaitLimit = 1u << 24;
constexpr int kGemmTimeout = 9;          // value written to the error word when a wait runs out

// The output tile is 128 rows by TILE_N columns, of which the first A_ROWS rows are real.
//   * TILE_N = 256 is for large M: a 128 x 128 tile would need 8 KB of operands per 64-cycle MMA, all the
//     shared-memory bandwidth there is, and twice the L2 traffic per flop.
//   * Narrow tiles (32, 64) are for few rows of activations, where the weight is streamed once: the grid has
//     to cover the SMs, and what counts is weight bytes in flight. There the TMA box of the activations is
//     cut down to A_ROWS rows (16, 32 or 64) -- boxes that hang over the end of the tensor are slow to fill --
//     which makes a stage small enough for a deep ring and three blocks per SM. The MMA still reads 128
//     rows: the rest of its A operand is whatever follows in shared memory (the next A tiles, then the B
//     tiles), and the accumulator rows that come out of it are never stored.
template <int TILE_N, int A_ROWS> struct TileShape {
  static_assert(TILE_N == 32 || TILE_N == 64 || TILE_N == 128 || TILE_N == 256, "accumulator columns: a power of two from 32 to 256");
  static_assert(A_ROWS == 16 || A_ROWS == 32 || A_ROWS == 64 || A_ROWS == 128, "activation rows per box");
  static constexpr int kBytesA = A_ROWS * kTileK * 2;
  static constexpr int kBytesB = TILE_N * kTileK * 2;
  static constexpr int kStageBytes = kBytesA + kBytesB;
  static constexpr int kBlocksPerSm = A_ROWS < 128 ? 3 : 1;
  static constexpr int kBudget = A_ROWS < 128 ? 72 * 1024 : 192 * 1024;
  static constexpr int kStages = kBudget / kStageBytes < 16 ? kBudget / kStageBytes : 16;
  static constexpr int kSharedBytes = kStages * kStageBytes + 1024;
  static_assert(kStages >= 3, "the ring needs a few stages");
  static_assert(kStages * kBytesB >= kTileBytesA - kBytesA, "the MMA's 128-row read of the last A tile must stay inside the B tiles");
  static constexpr uint32_t kTmemColumns = TILE_N;
  // Instruction descriptors: fp32 accumulate (bit 4), both operands K-major, N and M encoded /8 and /16.
  // kind::f16 with bf16 A and B (format 1 in bits 7-9 and 10-12); kind::f8f6f4 with e4m3 A and B (format 0).
  static constexpr uint32_t kShapeBits = (static_cast<uint32_t>(TILE_N >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
  static constexpr uint32_t kInstructionBf16 = (1u << 4) | (1u << 7) | (1u << 10) | kShapeBits;
  static constexpr uint32_t kInstructionFp8 = (1u << 4) | kShapeBits;
  // kind::i8: signed 8-bit A and B (format 1), 32-bit integer accumulators (format 2 in bits 4-5)
  static constexpr uint32_t kInstructionInt8 = (2u << 4) | (1u << 7) | (1u << 10) | kShapeBits;
};

// Operand kinds of the tensor-core kernel. A shared-memory row is 128 bytes either way: 64 bf16 or 128 fp8
// elements, consumed by four MMAs of 32 bytes of K each.
constexpr int kOperandBf16 = 0;
constexpr int kOperandFp8 = 1;
constexpr int kOperandInt8 = 2;

__device__ __forceinline__ uint32_t shared_address(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void barrier_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(bar)), "r"(count));
}
__device__ __forceinline__ void barrier_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(bar)), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity; false when the limit ran out.
__device__ __forceinline__ bool barrier_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t address = shared_address(bar);
  for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(address), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* target, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(shared_address(target)), "l"(map), "r"(shared_address(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored in 128-byte-swizzled rows: start address
// (16-byte units), stride between 8-row groups = 1024 bytes, descriptor version 1, swizzle mode 128 B.
__device__ __forceinline__ uint64_t matrix_descriptor(uint32_t tile_address) {
  uint64_t d = (tile_address & 0x3FFFFu) >> 4;
  d |= static_cast<uint64_t>(1) << 16;            // leading-dimension offset: unused for swizzled K-major
  d |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride-dimension offset
  d |= static_cast<uint64_t>(1) << 46;            // descriptor version
  d |= static_cast<uint64_t>(2) << 61;            // 128-byte swizzle
  return d;
}
constexpr int kMaxOutputCopies = 7;   // peers of an eight-GPU node

struct GemmParams {
  const __nv_bfloat16* bias;     // bf16 operands: optional bias in bf16
  __nv_bfloat16* y;
  int m, n, k;                   // k in elements
  int* error;
  // fp8 operands: y = acc * row_scale[row] * column_scale[col] + bias_f32[col], written as bf16 (y) or fp32 (y_f32)
  const float* row_scale;
  const float* column_scale;
  const float* bias_f32;
  float* y_f32;
  int pair_tile_n;               // two-block kernel: columns per tile (a multiple of 32, 64..256)
  // Column-sharded output (bf16 results only): this product is columns y_col0 .. y_col0 + n of rows that are y_ld
  // elements apart (0: the rows are n elements apart), and every tile is stored to y and to y_copy[0 .. y_copies) --
  // the same rows in the other GPUs' output buffers, written with ordinary stores through peer mappings.
  int64_t y_ld;
  int y_col0;
  int y_copies;
  __nv_bfloat16* y_copy[kMaxOutputCopies];
};

// Loads 32 consecutive accumulator columns of this thread's TMEM lane and waits for them.
__device__ __forceinline__ void load_accumulator_chunk(uint32_t (&v)[32], uint32_t address) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(address) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Epilogue arithmetic and stores of one thread's 32 accumulator values: row `row`, columns col .. col + 31 (the
// caller has checked row < m and col < n). bf16 operands: + bias; 8-bit operands: accumulator * row scale *
// column scale + bias. `staged_scale` / `staged_bias` point at the 32 columns' factors in shared memory (zero
// outside the matrix), or are null, in which case the factors come from global memory.
// `scatter_stage` (per warp, 32 rows of kScatterRowPieces 16-byte pieces; may be null) is used for the copies into the
// other GPUs' buffers: a thread holds 64 bytes of one row, and stored as they are, each store instruction would carry
// 32 separate 16-byte pieces across NVLink. Staged through shared memory, four threads share a row and an instruction
// carries eight contiguous 64-byte runs.
constexpr int kScatterRowPieces = 5;   // four pieces of data, one of padding against bank conflicts

template <int OPERAND, bool SCATTER = false>
__device__ __forceinline__ void finish_chunk(uint32_t (&v)[32], const GemmParams& p, int row, int col, float row_scale,
                                             const float* staged_scale, const float* staged_bias, uint4* scatter_stage = nullptr) {
  constexpr bool kScaled = OPERAND != kOperandBf16;
  // the plain product (SCATTER false) knows nothing of row pitches, column offsets and copies
  const int64_t ld = SCATTER && p.y_ld ? p.y_ld : p.n;
  const int col0 = SCATTER ? p.y_col0 : 0;
  const int copies = SCATTER ? p.y_copies : 0;
  const bool whole = col + 32 <= p.n && ((ld | col0) & 7) == 0;
  const int64_t at = static_cast<int64_t>(row) * ld + col0 + col;
  if (staged_bias != nullptr) {
    const float4* scales = reinterpret_cast<const float4*>(staged_scale);
    const float4* biases = reinterpret_cast<const float4*>(staged_bias);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const float4 b = biases[g];
      const float bias[4] = {b.x, b.y, b.z, b.w};
      if (kScaled) {
        const float4 cs = scales[g];
        const float scale[4] = {row_scale * cs.x, row_scale * cs.y, row_scale * cs.z, row_scale * cs.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t raw = v[g * 4 + j];
          const float accumulated = OPERAND == kOperandInt8 ? static_cast<float>(static_cast<int>(raw)) : __uint_as_float(raw);
          v[g * 4 + j] = __float_as_uint(fmaf(accumulated, scale[j], bias[j]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[g * 4 + j] = __float_as_uint(__uint_as_float(v[g * 4 + j]) + bias[j]);
      }
    }
  } else if (kScaled) {
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const bool inside = whole || col + c < p.n;
      const float scale = inside ? row_scale * p.column_scale[col + c] : 0.0f;
      const float b = inside && p.bias_f32 ? p.bias_f32[col + c] : 0.0f;
      const float accumulated = OPERAND == kOperandInt8 ? static_cast<float>(static_cast<int>(v[c])) : __uint_as_float(v[c]);
      v[c] = __float_as_uint(fmaf(accumulated, scale, b));
    }
  } else if (p.bias) {
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      if (whole || col + c < p.n) v[c] = __float_as_uint(__uint_as_float(v[c]) + __bfloat162float(p.bias[col + c]));
    }
  }
  if (kScaled && p.y_f32) {
    if (whole) {
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        *reinterpret_cast<uint4*>(p.y_f32 + at + g * 4) = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
      }
    } else {
      for (int c = 0; c < 32 && col + c < p.n; ++c) p.y_f32[at + c] = __uint_as_float(v[c]);
    }
  } else if (whole) {
    uint32_t packed[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(v[j * 2]), __uint_as_float(v[j * 2 + 1]));
      packed[j] = *reinterpret_cast<const uint32_t*>(&pair);
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      *reinterpret_cast<uint4*>(p.y + at + g * 8) = make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
    }
    if (copies > 0 && scatter_stage == nullptr) {
      for (int copy = 0; copy < copies; ++copy) {
        __nv_bfloat16* const target = p.y_copy[copy] + at;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          *reinterpret_cast<uint4*>(target + g * 8) = make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
        }
      }
    } else if (copies > 0) {
      const uint32_t lane = lane_id();
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        scatter_stage[lane * kScatterRowPieces + g] = make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
      }
    }
  } else {
    for (int c = 0; c < 32 && col + c < p.n; ++c) {
      const __nv_bfloat16 value = __float2bfloat16_rn(__uint_as_float(v[c]));
      p.y[at + c] = value;
      for (int copy = 0; copy < copies; ++copy) p.y_copy[copy][at + c] = value;
    }
  }
}

// Second half of the staged scatter, run by the whole warp: the 32 rows x 32 columns that finish_chunk left in
// `scatter_stage` go to every copy, four threads to a row, rows past the matrix skipped.
__device__ __forceinline__ void scatter_rows(const GemmParams& p, const uint4* scatter_stage, int first_row, int col, uint32_t lane) {
  const int64_t ld = p.y_ld ? p.y_ld : p.n;
  const int piece = static_cast<int>(lane & 3u);
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int in_tile = pass * 8 + static_cast<int>(lane >> 2);
    const int row = first_row + in_tile;
    if (row < p.m) {
      const uint4 value = scatter_stage[in_tile * kScatterRowPieces + piece];
      const int64_t at = static_cast<int64_t>(row) * ld + p.y_col0 + col + piece * 8;
      for (int copy = 0; copy < p.y_copies; ++copy) *reinterpret_cast<uint4*>(p.y_copy[copy] + at) = value;
    }
  }
}

// Per-warp staging of the column factors of `columns` consecutive columns starting at `first_col`.
template <int OPERAND>
__device__ __forceinline__ void stage_column_factors(const GemmParams& p, float* scales, float* biases, int first_col, int columns,
                                                     uint32_t lane) {
  constexpr bool kScaled = OPERAND != kOperandBf16;
  __syncwarp();   // the previous tile's reads of the factors are over
  for (int c = static_cast<int>(lane); c < columns; c += 32) {
    const int col = first_col + c;
    float scale = 0.0f, bias = 0.0f;
    if (col < p.n) {
      if (kScaled) {
        scale = p.column_scale[col];
        if (p.bias_f32) bias = p.bias_f32[col];
      } else if (p.bias) {
        bias = __bfloat162float(p.bias[col]);
      }
    }
    scales[c] = scale;
    biases[c] = bias;
  }
  __syncwarp();
}

template <int TILE_N, int A_ROWS, int OPERAND>
__global__ void __launch_bounds__(kGemmThreads, TileShape<TILE_N, A_ROWS>::kBlocksPerSm)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
  using Shape = TileShape<TILE_N, A_ROWS>;
  constexpr int kStages = Shape::kStages;
  constexpr int kBytesA = Shape::kBytesA;
  constexpr int kBytesB = Shape::kBytesB;
  constexpr uint32_t kTmemColumns = Shape::kTmemColumns;
  constexpr uint32_t kInstruction = OPERAND == kOperandFp8 ? Shape::kInstructionFp8
                                    : (OPERAND == kOperandInt8 ? Shape::kInstructionInt8 : Shape::kInstructionBf16);
  constexpr bool kScaled = OPERAND != kOperandBf16;                     // 8-bit operands: scaled epilogue
  constexpr int kElementsPerStep = kScaled ? 128 : 64;                  // one 128-byte row of K
  extern __shared__ uint8_t raw_shared[];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ __align__(8) uint64_t empty[kStages];
  __shared__ __align__(8) uint64_t accumulator_ready[2];   // MMA -> epilogue, one per accumulator buffer
  __shared__ __align__(8) uint64_t accumulator_free[2];    // epilogue -> MMA
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int failed;   // polled by the other warps' loops: volatile, so the reads are not hoisted out of them
  // Per epilogue warp, the column factors of its share of the tile (half the columns; all 32 of the narrowest tile)
  // as fp32: [0] weight scale (8-bit operands), [1] bias; zero outside the matrix. Every thread of a warp needs all of them for its row, so they are read from global memory once per
  // warp and tile and then come from shared memory as broadcast 16-byte reads. (Wide tiles only: the narrow ones
  // run three blocks per SM with no shared memory to spare, and store a handful of rows.)
  constexpr bool kStageColumns = A_ROWS == kTileM;
  __shared__ __align__(16) float column_factors[kStageColumns ? kEpilogueWarps : 1][2][kStageColumns ? (TILE_N >= 64 ? TILE_N / 2 : 32) : 4];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern; all A tiles come first, then all B tiles
  uint8_t* tiles_a = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_shared) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* tiles_b = tiles_a + kStages * kBytesA;
  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const int k_steps = (p.k + kElementsPerStep - 1) / kElementsPerStep;
  // The block is persistent: it takes output tiles blockIdx.x, blockIdx.x + gridDim.x, ... in an order that
  // runs along N first, so the blocks at work at any moment share their rows of activations in L2.
  const int n_tiles = (p.n + TILE_N - 1) / TILE_N;
  const int total_tiles = n_tiles * ((p.m + kTileM - 1) / kTileM);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      barrier_init(&full[s], 1);
      barrier_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(&accumulator_ready[b], 1);
      barrier_init(&accumulator_free[b], kEpilogueWarps);   // one arrival per epilogue warp
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(shared_address(&tmem_base_holder)),
                 "r"(2u * kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_holder;

  if (warp == 0 && lane == 0) {
    // ---- producer: one thread feeds the ring, straight through tile boundaries
    int step = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
      const int m0 = (tile / n_tiles) * kTileM;
      const int n0 = (tile % n_tiles) * TILE_N;
      for (int ks = 0; ks < k_steps; ++ks, ++step) {
        const int s = step % kStages;
        if (step >= kStages && !barrier_wait(&empty[s], ((step / kStages) - 1) & 1)) {
          failed = 1;
          break;
        }
        barrier_expect(&full[s], kBytesA + kBytesB);
        tma_load_2d(tiles_a + s * kBytesA, &map_x, &full[s], ks * kElementsPerStep, m0);
        tma_load_2d(tiles_b + s * kBytesB, &map_w, &full[s], ks * kElementsPerStep, n0);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: four K16 instructions per stage into the tile's accumulator buffer, stage handed back after
    int step = 0;
    int local = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local) {
      const int buffer = local & 1;
      // the epilogue must have drained this buffer (two tiles ago); a fresh barrier passes the first two waits
      if (!barrier_wait(&accumulator_free[buffer], ((local >> 1) & 1) ^ 1)) {
        failed = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t accumulator = tmem_base + static_cast<uint32_t>(buffer) * kTmemColumns;
      bool ok = true;
      for (int ks = 0; ks < k_steps; ++ks, ++step) {
        const int s = step % kStages;
        ok = barrier_wait(&full[s], (step / kStages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a = matrix_descriptor(shared_address(tiles_a + s * kBytesA));
        const uint64_t b = matrix_descriptor(shared_address(tiles_b + s * kBytesB));
#pragma unroll
        for (int kk = 0; kk < kTileK / 16; ++kk) {
          const uint32_t accumulate = (ks | kk) ? 1u : 0u;
          if (OPERAND == kOperandFp8) {
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
                ::"r"(accumulator), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(kInstruction), "r"(accumulate) : "memory");
          } else if (OPERAND == kOperandInt8) {
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                ::"r"(accumulator), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(kInstruction), "r"(accumulate) : "memory");
          } else {
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                ::"r"(accumulator), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(kInstruction), "r"(accumulate) : "memory");
          }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(shared_address(&empty[s])) : "memory");
      }
      if (!ok) failed = 1;
      // arrives once every MMA issued so far has completed (also on the failure path, so the epilogue wakes)
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                   ::"r"(shared_address(&accumulator_ready[buffer])) : "memory");
      if (!ok) break;
    }
  } else if (warp >= 2) {
    // ---- epilogue: a warp reaches the 32 TMEM lanes of its quadrant (warp index mod 4); two warps share a quadrant,
    // one per half of the tile's columns; they drain one buffer while the MMA issuer fills the other
    const int quadrant = warp & 3;
    const int member = warp - 2;                        // 0..7: which epilogue warp
    constexpr int kChunks = TILE_N / 32;                // 32 columns at a time
    constexpr int kChunksPerWarp = kChunks >= 2 ? kChunks / 2 : 1;
    const int first_chunk = kChunks >= 2 ? (member >> 2) * kChunksPerWarp : 0;
    const bool has_columns = kChunks >= 2 || member < 4;
    int local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buffer = local & 1;
      const int m0 = (tile / n_tiles) * kTileM;
      const int n0 = (tile % n_tiles) * TILE_N;
      if (kStageColumns && (kScaled || p.bias)) {
        stage_column_factors<OPERAND>(p, column_factors[member][0], column_factors[member][1], n0 + first_chunk * 32, kChunksPerWarp * 32, lane);
      }
      const bool ready = barrier_wait(&accumulator_ready[buffer], (local >> 1) & 1);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!ready || failed) {
        if (lane == 0) failed = 1;
        break;
      }
      const int row = m0 + quadrant * 32 + static_cast<int>(lane);
      if (!has_columns) {   // a 32-column tile has one chunk: the quadrant's second warp only hands the buffer back
        if (lane == 0) {
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(shared_address(&accumulator_free[buffer])) : "memory");
        }
        continue;
      }
      const float row_scale = kScaled && row < p.m ? p.row_scale[row] : 1.0f;
#pragma unroll 1
      for (int chunk = first_chunk; chunk < first_chunk + kChunksPerWarp; ++chunk) {
        uint32_t v[32];
        const uint32_t address = tmem_base + static_cast<uint32_t>(buffer) * kTmemColumns +
                                 (static_cast<uint32_t>(quadrant * 32) << 16) + static_cast<uint32_t>(chunk * 32);
        load_accumulator_chunk(v, address);
        if (chunk == first_chunk + kChunksPerWarp - 1) {
          // this warp's share of the buffer is in registers: hand it back before the stores
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(shared_address(&accumulator_free[buffer])) : "memory");
          }
        }
        const int col = n0 + chunk * 32;
        if (row < p.m && col < p.n) {
          const bool staged = kStageColumns && (kScaled || p.bias);
          finish_chunk<OPERAND>(v, p, row, col, row_scale, staged ? &column_factors[member][0][(chunk - first_chunk) * 32] : nullptr,
                                staged ? &column_factors[member][1][(chunk - first_chunk) * 32] : nullptr);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * kTmemColumns) : "memory");
  }
  if (threadIdx.x == 0 && failed) report(p.error, kGemmTimeout);
}


// ---------------------------------------------------------------------------------------------------------------
// Two-block tiles (tcgen05 cta_group::2). A pair of blocks on neighbouring SMs, launched as a cluster of two,
// computes a 256 x 256 output tile: each block stages its own 128 rows of activations and its own 128 weight rows
// (half of the tile's columns) per K step, and one MMA instruction issued by the pair's first block multiplies all
// 256 rows by all 256 columns, reading both blocks' shared memory and writing each block's 128 rows of fp32
// accumulators into that block's TMEM. Per block and K step that is 32 KB of operands for a 128 x 256 slice of the
// tile, against 48 KB when a block works alone: the single-block kernel is bound by what one SM can pull through
// its shared memory (TMA writes plus the MMA's reads), and this one by the tensor cores.
//   * Both blocks run a producer thread; the loads of both land on the first block's `full` barrier
//     (cp.async.bulk.tensor with cta_group::2 may signal the partner's barrier), which expects the bytes of both.
//   * tcgen05.commit with a two-block multicast mask hands a stage back to both producers and tells both
//     blocks' epilogue warps that an accumulator buffer is complete.
//   * The epilogue warps of both blocks arrive on the first block's `accumulator_free` barrier.
//   * The cluster barrier brackets the kernel: no block signals a partner whose barriers are not initialised yet,
//     and none leaves while its partner may still read its shared memory or write its barriers.
// Every mbarrier wait is bounded as in the single-block kernel; a block that gives up stops signalling, its
// partner's waits run out in turn, and both report the timeout.
// The tile is 256 rows by `pair_tile_n` columns, 256 at most. Narrower tiles (224, 192) are for products whose
// count of 256-wide tiles leaves most pairs idle in the last round: 4096 x 3840 is 240 such tiles for 74 pairs,
// 3.24 rounds that take 4, and 288 tiles of 224 columns, 3.9 rounds that take 4 x 224/256 = 3.5.
constexpr int kPairTileM = 2 * kTileM;
constexpr int kPairTileN = 256;                               // widest tile: sizes shared memory and TMEM
constexpr int kPairBytesA = kTileM * kTileK * 2;              // this block's 128 activation rows: 16 KB
constexpr int kPairBytesB = (kPairTileN / 2) * kTileK * 2;    // this block's weight rows (half the tile's columns): up to 16 KB
constexpr int kPairStages = 6;
constexpr int kPairSharedBytes = kPairStages * (kPairBytesA + kPairBytesB) + 1024;
constexpr uint32_t kPairShapeBits = static_cast<uint32_t>(kPairTileM >> 4) << 24;   // the column count is added per launch

// Order of the pairs' tiles. The tiles at work at any moment are consecutive in this order, and what they read
// together is what has to stay in L2: with rows of tiles taken one after the other, 74 tiles of a wide layer span
// every weight row and the whole weight streams through L2 once per round. Here the order runs down bands of
// kPairBandRows tile rows, column by column, so 74 consecutive tiles cover about 8 x 9 tiles: a ninth of the
// weight and an eighth of the activations.
constexpr int kPairBandRows = 8;
__device__ __forceinline__ void pair_tile_position(int tile, int n_tiles, int m_tiles, int* m_index, int* n_index) {
  const int band_tiles = kPairBandRows * n_tiles;
  const int band = tile / band_tiles;
  const int first_row = band * kPairBandRows;
  const int rows = min(kPairBandRows, m_tiles - first_row);
  const int within = tile - band * band_tiles;
  *m_index = first_row + within % rows;
  *n_index = within / rows;
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
// Address, in the cluster's shared window, of the first block's copy of a shared variable of this block.
__device__ __forceinline__ uint32_t first_block_address(uint32_t local) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
  return remote;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One box into this block's shared memory; the bytes are counted on a barrier that may belong to the partner.
__device__ __forceinline__ void tma_load_2d_pair(void* target, const CUtensorMap* map, uint32_t barrier_address, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(shared_address(target)), "l"(map), "r"(barrier_address), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void commit_to_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(shared_address(bar)), "h"(both) : "memory");
}

template <int OPERAND, bool SCATTER = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
linear_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
  constexpr uint32_t kInstruction = OPERAND == kOperandFp8 ? ((1u << 4) | kPairShapeBits)
                                    : (OPERAND == kOperandInt8 ? ((2u << 4) | (1u << 7) | (1u << 10) | kPairShapeBits)
                                                               : ((1u << 4) | (1u << 7) | (1u << 10) | kPairShapeBits));
  constexpr bool kScaled = OPERAND != kOperandBf16;
  constexpr int kElementsPerStep = kScaled ? 128 : 64;
  constexpr uint32_t kColumns = kPairTileN;              // TMEM columns per accumulator buffer
  extern __shared__ uint8_t raw_shared[];
  __shared__ __align__(8) uint64_t full[kPairStages];        // used in the first block: operands of both blocks have landed
  __shared__ __align__(8) uint64_t empty[kPairStages];       // in each block: the MMAs that read the stage are done
  __shared__ __align__(8) uint64_t accumulator_ready[2];     // in each block: this block's rows of the buffer are complete
  __shared__ __align__(8) uint64_t accumulator_free[2];      // used in the first block: both blocks have drained the buffer
  __shared__ uint32_t tmem_base_holder;
  __shared__ volatile int failed;   // polled by the other warps' loops: volatile, so the reads are not hoisted out of them
  __shared__ __align__(16) float column_factors[kEpilogueWarps][2][kPairTileN / 2];
  __shared__ __align__(16) uint4 scatter_stage[SCATTER ? kEpilogueWarps : 1][SCATTER ? 32 * kScatterRowPieces : 1];   // column-sharded output only
  uint8_t* tiles_a = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_shared) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* tiles_b = tiles_a + kPairStages * kPairBytesA;
  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;
  const int k_steps = (p.k + kElementsPerStep - 1) / kElementsPerStep;
  const int tile_n = p.pair_tile_n;
  const int n_tiles = (p.n + tile_n - 1) / tile_n;
  const int m_tiles = (p.m + kPairTileM - 1) / kPairTileM;
  const int total_tiles = n_tiles * m_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      barrier_init(&full[s], 1);
      barrier_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(&accumulator_ready[b], 1);
      barrier_init(&accumulator_free[b], 2 * kEpilogueWarps);   // one arrival per epilogue warp of either block
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // the same warp of both blocks allocates (and later frees) the pair's accumulator columns
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(shared_address(&tmem_base_holder)),
                 "r"(2u * kColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_holder;

  if (warp == 0 && lane == 0) {
    // ---- producer (both blocks): this block's rows of the activations and of the weight, counted on the first
    // block's barrier
    const uint32_t full_first = first_block_address(shared_address(&full[0]));
    int step = 0;
    for (int tile = pair; tile < total_tiles && !failed; tile += pairs) {
      int m_index, n_index;
      pair_tile_position(tile, n_tiles, m_tiles, &m_index, &n_index);
      const int m0 = m_index * kPairTileM + static_cast<int>(rank) * kTileM;
      const int n0 = n_index * tile_n + static_cast<int>(rank) * (tile_n / 2);
      for (int ks = 0; ks < k_steps; ++ks, ++step) {
        const int s = step % kPairStages;
        if (step >= kPairStages && !barrier_wait(&empty[s], ((step / kPairStages) - 1) & 1)) {
          failed = 1;
          break;
        }
        if (rank == 0) barrier_expect(&full[s], 2 * (kPairBytesA + (tile_n / 2) * kTileK * 2));
        tma_load_2d_pair(tiles_a + s * kPairBytesA, &map_x, full_first + 8u * s, ks * kElementsPerStep, m0);
        tma_load_2d_pair(tiles_b + s * kPairBytesB, &map_w, full_first + 8u * s, ks * kElementsPerStep, n0);
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer (first block only): four K-slices per stage, 256 rows x tile_n columns each
    const uint32_t instruction = kInstruction | (static_cast<uint32_t>(tile_n >> 3) << 17);
    int step = 0;
    int local = 0;
    for (int tile = pair; tile < total_tiles && !failed; tile += pairs, ++local) {
      const int buffer = local & 1;
      if (!barrier_wait(&accumulator_free[buffer], ((local >> 1) & 1) ^ 1)) {
        failed = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t accumulator = tmem_base + static_cast<uint32_t>(buffer) * kColumns;
      bool ok = true;
      for (int ks = 0; ks < k_steps; ++ks, ++step) {
        const int s = step % kPairStages;
        ok = barrier_wait(&full[s], (step / kPairStages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a = matrix_descriptor(shared_address(tiles_a + s * kPairBytesA));
        const uint64_t b = matrix_descriptor(shared_address(tiles_b + s * kPairBytesB));
#pragma unroll
        for (int kk = 0; kk < kTileK / 16; ++kk) {
          const uint32_t accumulate = (ks | kk) ? 1u : 0u;
          if (OPERAND == kOperandFp8) {
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
                ::"r"(accumulator), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(instruction), "r"(accumulate) : "memory");
          } else if (OPERAND == kOperandInt8) {
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}"
                ::"r"(accumulator), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(instruction), "r"(accumulate) : "memory");
          } else {
            asm volatile(
                "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                ::"r"(accumulator), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(instruction), "r"(accumulate) : "memory");
          }
        }
        commit_to_pair(&empty[s]);
      }
      if (!ok) failed = 1;
      commit_to_pair(&accumulator_ready[buffer]);   // also on the failure path, so that the epilogue warps wake
      if (!ok) break;
    }
  } else if (warp >= 2) {
    // ---- epilogue (both blocks): as in the single-block kernel, on this block's 128 rows of the tile
    const int quadrant = warp & 3;
    const int member = warp - 2;
    // the quadrant's first warp takes the larger half of the tile's 32-column chunks (2 to 8 of them)
    const int chunks = tile_n / 32;
    const int first_chunk = (member >> 2) * ((chunks + 1) / 2);
    const int chunks_here = (member >> 2) ? chunks / 2 : (chunks + 1) / 2;
    const uint32_t free_first = first_block_address(shared_address(&accumulator_free[0]));
    int local = 0;
    for (int tile = pair; tile < total_tiles; tile += pairs, ++local) {
      const int buffer = local & 1;
      int m_index, n_index;
      pair_tile_position(tile, n_tiles, m_tiles, &m_index, &n_index);
      const int m0 = m_index * kPairTileM + static_cast<int>(rank) * kTileM;
      const int n0 = n_index * tile_n;
      const bool staged = kScaled || p.bias;
      if (staged) {
        stage_column_factors<OPERAND>(p, column_factors[member][0], column_factors[member][1], n0 + first_chunk * 32, chunks_here * 32, lane);
      }
      const bool ready = barrier_wait(&accumulator_ready[buffer], (local >> 1) & 1);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!ready || failed) {
        if (lane == 0) failed = 1;
        break;
      }
      const int row = m0 + quadrant * 32 + static_cast<int>(lane);
      const float row_scale = kScaled && row < p.m ? p.row_scale[row] : 1.0f;
#pragma unroll 1
      for (int chunk = first_chunk; chunk < first_chunk + chunks_here; ++chunk) {
        uint32_t v[32];
        load_accumulator_chunk(v, tmem_base + static_cast<uint32_t>(buffer) * kColumns + (static_cast<uint32_t>(quadrant * 32) << 16) +
                                      static_cast<uint32_t>(chunk * 32));
        if (chunk == first_chunk + chunks_here - 1) {
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(free_first + 8u * buffer) : "memory");
          }
        }
        const int col = n0 + chunk * 32;
        // the copies of a whole, 16-byte aligned chunk leave through the warp's staging area (the same test as in finish_chunk)
        const bool through_stage = SCATTER && p.y_copies > 0 && col + 32 <= p.n && (((p.y_ld ? p.y_ld : p.n) | p.y_col0) & 7) == 0;
        if (row < p.m && col < p.n) {
          finish_chunk<OPERAND, SCATTER>(v, p, row, col, row_scale, staged ? &column_factors[member][0][(chunk - first_chunk) * 32] : nullptr,
                                         staged ? &column_factors[member][1][(chunk - first_chunk) * 32] : nullptr,
                                         through_stage ? scatter_stage[SCATTER ? member : 0] : nullptr);
        }
        if (through_stage) {
          __syncwarp();
          scatter_rows(p, scatter_stage[SCATTER ? member : 0], m0 + quadrant * 32, col, lane);
          __syncwarp();
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * kColumns) : "memory");
  }
  if (threadIdx.x == 0 && failed) report(p.error, kGemmTimeout);
}

}  // namespace
}  // namespace ep

namespace ep {
namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so the library does not link libcuda.
EncodeTiled tensor_map_encoder() {
  static std::once_flag once;
  static EncodeTiled encoder = nullptr;
  std::call_once(once, [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess) {
      encoder = reinterpret_cast<EncodeTiled>(entry);
    }
  });
  return encoder;
}

// rows x k row-major matrix of bf16 or one-byte elements; boxes of box_rows rows x 128 bytes, 128-byte swizzle, zero
// fill outside the tensor
bool make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows, int operand) {
  EncodeTiled encode = tensor_map_encoder();
  if (!encode) return false;
  const int element_bytes = operand == kOperandBf16 ? 2 : 1;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * element_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / element_bytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, operand == kOperandBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                const_cast<void*>(base), dims, strides, box, element_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Sets of eight features per block: as few as keep the whole layer in one wave of resident blocks (four blocks an SM
// with one set, three with more), four at most.
int launch_stream(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* bias, __nv_bfloat16* y, int m, int n, int k,
                  cudaStream_t s) {
  const int sets = (n + 7) / 8;
  const auto blocks = [sets](int per_block) { return static_cast<unsigned>((sets + per_block - 1) / per_block); };
  if (sets <= kStreamBlocksPerSm * kSmCount) {
    linear_stream_kernel<1><<<blocks(1), kStreamThreads, 0, s>>>(x, w, bias, y, m, n, k);
  } else if (blocks(2) <= static_cast<unsigned>((kStreamBlocksPerSm - 1) * kSmCount)) {
    linear_stream_kernel<2><<<blocks(2), kStreamThreads, 0, s>>>(x, w, bias, y, m, n, k);
  } else if (blocks(3) <= static_cast<unsigned>((kStreamBlocksPerSm - 1) * kSmCount)) {
    linear_stream_kernel<3><<<blocks(3), kStreamThreads, 0, s>>>(x, w, bias, y, m, n, k);
  } else {
    linear_stream_kernel<4><<<blocks(4), kStreamThreads, 0, s>>>(x, w, bias, y, m, n, k);
  }
  return check_launch("linear_stream_kernel");
}

template <int TILE_N, int A_ROWS, int OPERAND>
int launch_tcgen05(const void* x_dev, const void* weight_dev, const GemmParams& p, cudaStream_t s) {
  using Shape = TileShape<TILE_N, A_ROWS>;
  CUtensorMap map_x, map_w;
  if (!make_tile_map(&map_x, x_dev, p.m, p.k, A_ROWS, OPERAND) || !make_tile_map(&map_w, weight_dev, p.n, p.k, TILE_N, OPERAND)) {
    return EP_ERR_UNSUPPORTED;
  }
  EP_CUDA_CHECK(cudaFuncSetAttribute(linear_tcgen05_kernel<TILE_N, A_ROWS, OPERAND>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Shape::kSharedBytes));
  const int64_t tiles = static_cast<int64_t>((p.n + TILE_N - 1) / TILE_N) * ((p.m + kTileM - 1) / kTileM);
  const int64_t resident = static_cast<int64_t>(product_sm_limit()) * Shape::kBlocksPerSm;
  const unsigned grid = static_cast<unsigned>(tiles < resident ? tiles : resident);
  linear_tcgen05_kernel<TILE_N, A_ROWS, OPERAND><<<grid, kGemmThreads, Shape::kSharedBytes, s>>>(map_x, map_w, p);
  return EP_OK;
}

template <int TILE_N, int OPERAND>
int launch_narrow(const void* x_dev, const void* weight_dev, const GemmParams& p, cudaStream_t s) {
  if (p.m <= 16) return launch_tcgen05<TILE_N, 16, OPERAND>(x_dev, weight_dev, p, s);
  if (p.m <= 32) return launch_tcgen05<TILE_N, 32, OPERAND>(x_dev, weight_dev, p, s);
  if (p.m <= 64) return launch_tcgen05<TILE_N, 64, OPERAND>(x_dev, weight_dev, p, s);
  return launch_tcgen05<TILE_N, 128, OPERAND>(x_dev, weight_dev, p, s);
}

// Pairs of blocks that can be resident at once (0 when clusters of two cannot be launched here); asked once per
// operand type.
template <int OPERAND>
int resident_pairs() {
  static std::once_flag once;
  static int pairs = 0;
  std::call_once(once, [] {
    if (cudaFuncSetAttribute(linear_tcgen05_pair_kernel<OPERAND>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSharedBytes) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * kSmCount);
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = kPairSharedBytes;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, linear_tcgen05_pair_kernel<OPERAND>, &config) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    pairs = clusters;
  });
  return pairs;
}

template <int OPERAND, bool SCATTER = false>
int launch_pair(const void* x_dev, const void* weight_dev, const GemmParams& problem, int tile_n, int pairs, cudaStream_t s) {
  GemmParams p = problem;
  p.pair_tile_n = tile_n;
  CUtensorMap map_x, map_w;
  if (!make_tile_map(&map_x, x_dev, p.m, p.k, kTileM, OPERAND) || !make_tile_map(&map_w, weight_dev, p.n, p.k, tile_n / 2, OPERAND)) {
    return EP_ERR_UNSUPPORTED;
  }
  const int64_t tiles = static_cast<int64_t>((p.n + tile_n - 1) / tile_n) * ((p.m + kPairTileM - 1) / kPairTileM);
  // per device, so on every launch (the occupancy query above ran on whichever device came first)
  EP_CUDA_CHECK(cudaFuncSetAttribute(linear_tcgen05_pair_kernel<OPERAND, SCATTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSharedBytes));
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 2;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2u * static_cast<unsigned>(tiles < pairs ? tiles : pairs));
  config.blockDim = dim3(kGemmThreads);
  config.dynamicSmemBytes = kPairSharedBytes;
  config.stream = s;
  config.attrs = &attribute;
  config.numAttrs = 1;
  EP_CUDA_CHECK(cudaLaunchKernelEx(&config, linear_tcgen05_pair_kernel<OPERAND, SCATTER>, map_x, map_w, p));
  return EP_OK;
}

// Tile shape. What a K step costs an SM, in clocks: the tensor cores need 2 x columns (four MMAs of 128 rows), and
// the shared memory, which takes the TMA's writes and feeds the MMA's reads at 128 bytes per clock, needs
// 2 x (rows staged for A + rows staged for B). A single block stages 128 (or fewer) + columns rows; a block of a pair
// stages 128 + columns / 2 for the same 128 x columns slice of the output. Tiles beyond what is resident at once run
// in further rounds: take the shape with the least rounds x clocks, the two-block tiles first among equals.
template <int OPERAND>
int launch_best_tile(const void* x_dev, const void* weight_dev, const GemmParams& p, cudaStream_t s) {
  const int64_t row_tiles = (p.m + kTileM - 1) / kTileM;
  const int a_rows = p.m <= 16 ? 16 : (p.m <= 32 ? 32 : (p.m <= 64 ? 64 : 128));
  int tile_n = 32;
  bool two_blocks = false;
  int64_t best = -1;
  const int sms = product_sm_limit();
  const int pairs = p.m > kTileM ? std::min(resident_pairs<OPERAND>(), sms / 2) : 0;
  if (pairs >= 32) {
    const int64_t row_pairs = (p.m + kPairTileM - 1) / kPairTileM;
    for (int candidate = kPairTileN; candidate >= 64; candidate -= 32) {
      const int64_t tiles = static_cast<int64_t>((p.n + candidate - 1) / candidate) * row_pairs;
      const int64_t clocks = 2 * candidate > 256 + candidate ? 2 * candidate : 256 + candidate;
      const int64_t cost = ((tiles + pairs - 1) / pairs) * clocks;
      if (best < 0 || cost < best) {
        best = cost;
        tile_n = candidate;
        two_blocks = true;
      }
    }
  }
  for (int candidate = 256; candidate >= 32; candidate >>= 1) {
    const bool narrow = candidate <= 64;
    const int box_a = narrow ? a_rows : 128;
    const int64_t blocks = row_tiles * ((p.n + candidate - 1) / candidate);
    const int64_t resident = static_cast<int64_t>(sms) * (box_a < 128 ? 3 : 1);
    const int64_t cost = ((blocks + resident - 1) / resident) * 2 * (box_a + candidate);
    if (best < 0 || cost < best) {
      best = cost;
      tile_n = candidate;
      two_blocks = false;
    }
  }
  if (two_blocks) {
    const int rc = launch_pair<OPERAND>(x_dev, weight_dev, p, tile_n, pairs, s);
    if (rc != EP_OK) return rc;
    return check_launch("linear_tcgen05_pair_kernel");
  }
  int rc = EP_ERR_UNSUPPORTED;
  switch (tile_n) {
    case 256: rc = launch_tcgen05<256, 128, OPERAND>(x_dev, weight_dev, p, s); break;
    case 128: rc = launch_tcgen05<128, 128, OPERAND>(x_dev, weight_dev, p, s); break;
    case 64: rc = launch_narrow<64, OPERAND>(x_dev, weight_dev, p, s); break;
    default: rc = launch_narrow<32, OPERAND>(x_dev, weight_dev, p, s); break;
  }
  if (rc != EP_OK) return rc;
  return check_launch("linear_tcgen05_kernel");
}

// The column-sharded product: two-block tiles only (more than 128 rows of activations), tile width by the same cost.
int launch_scatter(const void* x_dev, const void* weight_dev, const GemmParams& p, cudaStream_t s) {
  const int pairs = p.m > kTileM ? resident_pairs<kOperandBf16>() : 0;
  if (pairs < 1) return EP_ERR_UNSUPPORTED;
  const int64_t row_pairs = (p.m + kPairTileM - 1) / kPairTileM;
  int tile_n = kPairTileN;
  int64_t best = -1;
  for (int candidate = kPairTileN; candidate >= 64; candidate -= 32) {
    const int64_t tiles = static_cast<int64_t>((p.n + candidate - 1) / candidate) * row_pairs;
    const int64_t clocks = 2 * candidate > 256 + candidate ? 2 * candidate : 256 + candidate;
    const int64_t cost = ((tiles + pairs - 1) / pairs) * clocks;
    if (best < 0 || cost < best) {
      best = cost;
      tile_n = candidate;
    }
  }
  const int rc = launch_pair<kOperandBf16, true>(x_dev, weight_dev, p, tile_n, pairs, s);
  if (rc != EP_OK) return rc;
  return check_launch("linear_tcgen05_pair_kernel (column-sharded)");
}

}  // namespace
}  // namespace ep

using namespace ep;

extern "C" int ep_linear_forward(const void* x_dev, const void* weight_dev, const void* bias_dev, void* y_dev, int64_t m, int64_t n,
                                 int64_t k, int* error_dev, ep_stream_t stream) {
  if (!x_dev || !weight_dev || !y_dev || m <= 0 || n <= 0 || k <= 0 || (k & 7) != 0 || m > 0x7FFFFFFF || n > 0x7FFFFFFF ||
      k > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(x_dev) & 15u) || (reinterpret_cast<uintptr_t>(weight_dev) & 15u) ||
      (reinterpret_cast<uintptr_t>(y_dev) & 15u)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* x = static_cast<const __nv_bfloat16*>(x_dev);
  const auto* w = static_cast<const __nv_bfloat16*>(weight_dev);
  const auto* bias = static_cast<const __nv_bfloat16*>(bias_dev);
  auto* y = static_cast<__nv_bfloat16*>(y_dev);
  const int mi = static_cast<int>(m), ni = static_cast<int>(n), ki = static_cast<int>(k);
  if (m <= kStreamMaxM) return launch_stream(x, w, bias, y, mi, ni, ki, s);
  GemmParams p = {};
  p.bias = bias;
  p.y = y;
  p.m = mi;
  p.n = ni;
  p.k = ki;
  p.error = error_dev;
  return launch_best_tile<kOperandBf16>(x_dev, weight_dev, p, s);
}

extern "C" int ep_linear_forward_scatter(const void* x_dev, const void* weight_dev, const void* bias_dev, void* y_dev,
                                         void* const* y_peers_host, int peers, int64_t y_ld, int64_t y_col0, int64_t m, int64_t n,
                                         int64_t k, int* error_dev, ep_stream_t stream) {
  if (!x_dev || !weight_dev || !y_dev || m <= 0 || n <= 0 || k <= 0 || (k & 7) != 0 || m > 0x7FFFFFFF || n > 0x7FFFFFFF ||
      k > 0x7FFFFFFF || peers < 0 || peers > kMaxOutputCopies || (peers > 0 && !y_peers_host) || y_col0 < 0 || y_ld < y_col0 + n ||
      y_ld > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if (m <= kTileM) return EP_ERR_UNSUPPORTED;   // the two-block tensor-core kernel only: a few tokens' outputs are cheaper to gather
  if ((reinterpret_cast<uintptr_t>(x_dev) & 15u) || (reinterpret_cast<uintptr_t>(weight_dev) & 15u) ||
      (reinterpret_cast<uintptr_t>(y_dev) & 15u)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  GemmParams p = {};
  p.bias = static_cast<const __nv_bfloat16*>(bias_dev);
  p.y = static_cast<__nv_bfloat16*>(y_dev);
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.error = error_dev;
  p.y_ld = y_ld;
  p.y_col0 = static_cast<int>(y_col0);
  p.y_copies = peers;
  for (int copy = 0; copy < peers; ++copy) {
    if (!y_peers_host[copy] || (reinterpret_cast<uintptr_t>(y_peers_host[copy]) & 15u)) return EP_ERR_INVALID_ARGUMENT;
    p.y_copy[copy] = static_cast<__nv_bfloat16*>(y_peers_host[copy]);
  }
  return launch_scatter(x_dev, weight_dev, p, static_cast<cudaStream_t>(stream));
}

// ---- barrier between the GPUs of a column-sharded layer ---------------------------------------------------------
// Each rank owns a row of `world` 32-bit flags that its peers can write (a peer mapping of the same allocation on every
// rank). Thread r of the one block tells peer r "rank `rank` has arrived at `epoch`" with a system-scope release store
// into the peer's row and then polls its own row's slot r until that peer's arrival shows, for at most `timeout_ns`:
// a peer that never arrives costs that long and an error word, never a hang.
namespace ep {
namespace {
struct PeerBarrierParams {
  uint32_t* flags[kMaxOutputCopies + 1];   // flags[r]: rank r's row, as mapped on this GPU
  int rank;
  int world;
  uint32_t epoch;
  unsigned long long timeout_ns;
  int* error;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerBarrierParams p) {
  const int peer = threadIdx.x;
  if (peer >= p.world || peer == p.rank) return;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[peer] + p.rank), "r"(p.epoch) : "memory");
  const uint32_t* mine = p.flags[p.rank] + peer;
  unsigned long long begin, now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(begin));
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int32_t>(seen - p.epoch) >= 0) return;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - begin > p.timeout_ns) {
      report(p.error, EP_KERNEL_TIMEOUT);
      return;
    }
    __nanosleep(200);
  }
}
}  // namespace
}  // namespace ep

extern "C" int ep_peer_barrier(void* const* flag_rows_host, int rank, int world, uint32_t epoch, int64_t timeout_us, int* error_dev,
                               ep_stream_t stream) {
  if (!flag_rows_host || world < 1 || world > kMaxOutputCopies + 1 || rank < 0 || rank >= world || timeout_us <= 0 ||
      timeout_us > 60 * 1000 * 1000) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  PeerBarrierParams p = {};
  for (int r = 0; r < world; ++r) {
    if (!flag_rows_host[r] || (reinterpret_cast<uintptr_t>(flag_rows_host[r]) & 3u)) return EP_ERR_INVALID_ARGUMENT;
    p.flags[r] = static_cast<uint32_t*>(flag_rows_host[r]);
  }
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.timeout_ns = static_cast<unsigned long long>(timeout_us) * 1000ull;
  p.error = error_dev;
  if (world == 1) return EP_OK;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_launch("peer_barrier_kernel");
}

namespace {
template <int OPERAND>
int scaled_forward(const void* x_codes_dev, const void* weight_codes_dev, const float* x_scale_dev, const float* weight_scale_dev,
                   const float* bias_dev, void* y_dev, int y_is_f32, int64_t m, int64_t n, int64_t k, int* error_dev,
                   ep_stream_t stream) {
  if (!x_codes_dev || !weight_codes_dev || !x_scale_dev || !weight_scale_dev || !y_dev || m <= 0 || n <= 0 || k <= 0 ||
      (k & 15) != 0 || m > 0x7FFFFFFF || n > 0x7FFFFFFF || k > 0x7FFFFFFF) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(x_codes_dev) & 15u) || (reinterpret_cast<uintptr_t>(weight_codes_dev) & 15u) ||
      (reinterpret_cast<uintptr_t>(y_dev) & 15u)) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  GemmParams p = {};
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.error = error_dev;
  p.row_scale = x_scale_dev;
  p.column_scale = weight_scale_dev;
  p.bias_f32 = bias_dev;
  if (y_is_f32) p.y_f32 = static_cast<float*>(y_dev);
  else p.y = static_cast<__nv_bfloat16*>(y_dev);
  return launch_best_tile<OPERAND>(x_codes_dev, weight_codes_dev, p, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int ep_linear_forward_fp8(const void* x_codes_dev, const void* weight_codes_dev, const float* x_scale_dev,
                                     const float* weight_scale_dev, const float* bias_dev, void* y_dev, int y_is_f32, int64_t m,
                                     int64_t n, int64_t k, int* error_dev, ep_stream_t stream) {
  return scaled_forward<kOperandFp8>(x_codes_dev, weight_codes_dev, x_scale_dev, weight_scale_dev, bias_dev, y_dev, y_is_f32, m, n, k,
                                     error_dev, stream);
}

extern "C" int ep_linear_forward_int8(const void* x_codes_dev, const void* weight_codes_dev, const float* x_scale_dev,
                                      const float* weight_scale_dev, const float* bias_dev, void* y_dev, int y_is_f32, int64_t m,
                                      int64_t n, int64_t k, int* error_dev, ep_stream_t stream) {
  return scaled_forward<kOperandInt8>(x_codes_dev, weight_codes_dev, x_scale_dev, weight_scale_dev, bias_dev, y_dev, y_is_f32, m, n, k,
                                      error_dev, stream);
}

namespace {
template <bool INT8>
int quantize_rows(const void* x_dev, int x_kind, int64_t rows, int64_t cols, void* codes_dev, float* scales_dev, ep_stream_t stream) {
  if (!x_dev || !codes_dev || !scales_dev || rows <= 0 || cols <= 0 || rows > 0x7FFFFFFF || x_kind < 0 || x_kind > 2) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>(rows);
  auto* codes = static_cast<uint8_t*>(codes_dev);
  // 16 bytes of a row at a time when every row (and its codes) starts on such a boundary
  const int64_t element_bytes = x_kind == 2 ? 4 : 2;
  const int64_t per_vector = 16 / element_bytes;
  const bool vector = cols % per_vector == 0 && (reinterpret_cast<uintptr_t>(x_dev) & 15u) == 0 && (reinterpret_cast<uintptr_t>(codes_dev) & 7u) == 0;
  const int64_t pieces = vector ? cols / per_vector : 0;     // 16-byte pieces of a row; up to 1024 stay in registers
#define EP_LAUNCH_QUANTIZE(TYPE)                                                                                                   \
  if (vector && pieces <= 256) {                                                                                                   \
    quantize_rows_held_kernel<TYPE, INT8, 1><<<blocks, 256, 0, s>>>(static_cast<const TYPE*>(x_dev), cols, codes, scales_dev);     \
  } else if (vector && pieces <= 512) {                                                                                            \
    quantize_rows_held_kernel<TYPE, INT8, 2><<<blocks, 256, 0, s>>>(static_cast<const TYPE*>(x_dev), cols, codes, scales_dev);     \
  } else if (vector && pieces <= 1024) {                                                                                           \
    quantize_rows_held_kernel<TYPE, INT8, 4><<<blocks, 256, 0, s>>>(static_cast<const TYPE*>(x_dev), cols, codes, scales_dev);     \
  } else if (vector) {                                                                                                             \
    quantize_rows_8bit_kernel<TYPE, INT8, true><<<blocks, 256, 0, s>>>(static_cast<const TYPE*>(x_dev), cols, codes, scales_dev);  \
  } else {                                                                                                                         \
    quantize_rows_8bit_kernel<TYPE, INT8, false><<<blocks, 256, 0, s>>>(static_cast<const TYPE*>(x_dev), cols, codes, scales_dev); \
  }
  switch (x_kind) {
    case 0: EP_LAUNCH_QUANTIZE(__nv_bfloat16) break;
    case 1: EP_LAUNCH_QUANTIZE(__half) break;
    default: EP_LAUNCH_QUANTIZE(float) break;
  }
#undef EP_LAUNCH_QUANTIZE
  return check_launch("quantize_rows kernel");
}
}  // namespace

extern "C" int ep_quantize_rows_fp8(const void* x_dev, int x_kind, int64_t rows, int64_t cols, void* codes_dev, float* scales_dev,
                                    ep_stream_t stream) {
  return quantize_rows<false>(x_dev, x_kind, rows, cols, codes_dev, scales_dev, stream);
}

extern "C" int ep_quantize_rows_int8(const void* x_dev, int x_kind, int64_t rows, int64_t cols, void* codes_dev, float* scales_dev,
                                     ep_stream_t stream) {
  return quantize_rows<true>(x_dev, x_kind, rows, cols, codes_dev, scales_dev, stream);
}

extern "C" int ep_convrot_rows(const void* x_dev, int x_kind, int64_t rows, int64_t cols, int group, void* y_dev, ep_stream_t stream) {
  const bool power_of_four = group >= 4 && (group & (group - 1)) == 0 && (__builtin_ctz(static_cast<unsigned>(group)) % 2) == 0;
  if (!x_dev || !y_dev || rows <= 0 || cols <= 0 || rows > 0x7FFFFFFF || x_kind < 0 || x_kind > 2 || !power_of_four ||
      cols % group != 0) {
    return EP_ERR_INVALID_ARGUMENT;
  }
  const size_t shared = static_cast<size_t>(cols) * sizeof(float);
  if (shared > 200 * 1024) return EP_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>(rows);
  switch (x_kind) {
    case 0:
      EP_CUDA_CHECK(cudaFuncSetAttribute(convrot_rows_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
      convrot_rows_kernel<<<blocks, 256, shared, s>>>(static_cast<const __nv_bfloat16*>(x_dev), cols, group, static_cast<__nv_bfloat16*>(y_dev));
      break;
    case 1:
      EP_CUDA_CHECK(cudaFuncSetAttribute(convrot_rows_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
      convrot_rows_kernel<<<blocks, 256, shared, s>>>(static_cast<const __half*>(x_dev), cols, group, static_cast<__half*>(y_dev));
      break;
    default:
      EP_CUDA_CHECK(cudaFuncSetAttribute(convrot_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
      convrot_rows_kernel<<<blocks, 256, shared, s>>>(static_cast<const float*>(x_dev), cols, group, static_cast<float*>(y_dev));
      break;
  }
  return check_launch("convrot_rows_kernel");
}
