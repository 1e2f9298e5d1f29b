// y[M,N] = x[M,K] . W[N,K]^T (+ bias) in bf16 with fp32 accumulation: the GEMM behind CompressedLinear.forward.
//
// W is the weight the fused decode kernel has just written (K-contiguous rows, exactly the K-major B
// operand); for the layer shapes in question it is still resident in the 126 MB L2 when this runs.
//
//   * M <= 16: `linear_small_m_kernel` -- a bandwidth kernel on CUDA cores. One warp per output feature
//     streams that weight row once with 16-byte loads and keeps up to 16 dot products going against the
//     activations staged in shared memory; a 5-step shuffle reduction finishes each.
//   * M > 16: `linear_tcgen05_kernel` -- 128 x 128 output tile per block on the 5th-generation tensor cores.
//     TMA (cp.async.bulk.tensor, 128-byte swizzle) fills a 4-stage shared-memory ring of 128 x 64 A and B
//     tiles; one elected thread issues tcgen05.mma (M128 N128 K16, fp32 accumulators in TMEM) straight from
//     shared memory; four warps read the accumulator back with tcgen05.ld, add the bias, round to bf16 and
//     store. Every mbarrier wait is bounded: on a timeout the block raises the error word, frees its TMEM
//     and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "ep_common.cuh"

namespace ep {
namespace {

// ------------------------------------------------------------------------------------------------
// small M
// ------------------------------------------------------------------------------------------------
constexpr int kSmallThreads = 256;
constexpr int kSmallMaxM = 16;

template <int MROWS>
__global__ void __launch_bounds__(kSmallThreads) linear_small_m_kernel(const __nv_bfloat16* __restrict__ x,
                                                                       const __nv_bfloat16* __restrict__ w,
                                                                       const __nv_bfloat16* __restrict__ bias,
                                                                       __nv_bfloat16* __restrict__ y, int m, int n, int k) {
  extern __shared__ __align__(16) __nv_bfloat16 staged_x[];  // [MROWS][k], rows beyond m are zero
  for (int i = threadIdx.x * 8; i < MROWS * k; i += kSmallThreads * 8) {
    const int row = i / k;
    uint4 value = make_uint4(0, 0, 0, 0);
    if (row < m) value = *reinterpret_cast<const uint4*>(x + i);
    *reinterpret_cast<uint4*>(staged_x + i) = value;
  }
  __syncthreads();
  const uint32_t lane = lane_id();
  const int warps = kSmallThreads / 32;
  for (int feature = blockIdx.x * warps + (threadIdx.x >> 5); feature < n; feature += gridDim.x * warps) {
    float acc[MROWS];
#pragma unroll
    for (int r = 0; r < MROWS; ++r) acc[r] = 0.0f;
    const __nv_bfloat16* row = w + static_cast<int64_t>(feature) * k;
    for (int c = lane * 8; c < k; c += 32 * 8) {
      const uint4 packed = __ldg(reinterpret_cast<const uint4*>(row + c));
      const __nv_bfloat162* wv = reinterpret_cast<const __nv_bfloat162*>(&packed);
      float wf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 pair = __bfloat1622float2(wv[j]);
        wf[2 * j] = pair.x;
        wf[2 * j + 1] = pair.y;
      }
#pragma unroll
      for (int r = 0; r < MROWS; ++r) {
        const uint4 xp = *reinterpret_cast<const uint4*>(staged_x + r * k + c);
        const __nv_bfloat162* xv = reinterpret_cast<const __nv_bfloat162*>(&xp);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 pair = __bfloat1622float2(xv[j]);
          acc[r] = fmaf(wf[2 * j], pair.x, acc[r]);
          acc[r] = fmaf(wf[2 * j + 1], pair.y, acc[r]);
        }
      }
    }
    const float b = bias ? __bfloat162float(bias[feature]) : 0.0f;
#pragma unroll
    for (int r = 0; r < MROWS; ++r) {
      float total = acc[r];
#pragma unroll
      for (int step = 16; step > 0; step >>= 1) total += __shfl_xor_sync(0xFFFFFFFFu, total, step);
      if (lane == 0 && r < m) y[static_cast<int64_t>(r) * n + feature] = __float2bfloat16_rn(total + b);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// tcgen05 GEMM
// ------------------------------------------------------------------------------------------------
constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kTileK = 64;               // 64 bf16 = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kTileBytes = kTileM * kTileK * 2;         // 16 KB, A and B tiles alike
constexpr int kGemmThreads = 192;        // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr uint32_t kTmemColumns = 128;   // fp32 accumulator: 128 lanes x 128 columns
constexpr uint32_t kWaitLimit = 1u << 24;
constexpr int kGemmTimeout = 9;          // value written to the error word when a wait runs out

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
// Instruction descriptor, kind::f16: fp32 accumulate, bf16 A and B, both K-major, N and M encoded /8 and /16.
constexpr uint32_t kInstruction = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
                                  (static_cast<uint32_t>(kTileM >> 4) << 24);

struct GemmParams {
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  int m, n, k;
  int* error;
};

__global__ void __launch_bounds__(kGemmThreads, 1) linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                         const __grid_constant__ CUtensorMap map_w, const GemmParams p) {
  extern __shared__ uint8_t raw_shared[];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ __align__(8) uint64_t empty[kStages];
  __shared__ __align__(8) uint64_t accumulator_ready;
  __shared__ uint32_t tmem_base_holder;
  __shared__ int failed;
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_shared) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const int m0 = blockIdx.y * kTileM;
  const int n0 = blockIdx.x * kTileN;
  const int k_steps = (p.k + kTileK - 1) / kTileK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      barrier_init(&full[s], 1);
      barrier_init(&empty[s], 1);
    }
    barrier_init(&accumulator_ready, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(shared_address(&tmem_base_holder)),
                 "r"(kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_holder;

  if (warp == 0 && lane == 0) {
    // ---- producer: one thread feeds the ring
    for (int step = 0; step < k_steps; ++step) {
      const int s = step % kStages;
      if (step >= kStages && !barrier_wait(&empty[s], ((step / kStages) - 1) & 1)) {
        failed = 1;
        break;
      }
      barrier_expect(&full[s], 2 * kTileBytes);
      tma_load_2d(tiles + s * 2 * kTileBytes, &map_x, &full[s], step * kTileK, m0);
      tma_load_2d(tiles + s * 2 * kTileBytes + kTileBytes, &map_w, &full[s], step * kTileK, n0);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: four K16 instructions per stage, then hand the stage back
    bool ok = true;
    for (int step = 0; step < k_steps && ok; ++step) {
      const int s = step % kStages;
      ok = barrier_wait(&full[s], (step / kStages) & 1);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t a = matrix_descriptor(shared_address(tiles + s * 2 * kTileBytes));
      const uint64_t b = matrix_descriptor(shared_address(tiles + s * 2 * kTileBytes + kTileBytes));
#pragma unroll
      for (int kk = 0; kk < kTileK / 16; ++kk) {
        const uint32_t accumulate = (step | kk) ? 1u : 0u;
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
            ::"r"(tmem_base), "l"(a + 2u * kk), "l"(b + 2u * kk), "r"(kInstruction), "r"(accumulate) : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(shared_address(&empty[s])) : "memory");
    }
    if (!ok) failed = 1;
    // arrives once every MMA issued so far has completed (also on the failure path, so the epilogue wakes)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(shared_address(&accumulator_ready)) : "memory");
  } else if (warp >= 2) {
    // ---- epilogue: each warp owns the 32 TMEM lanes of its quadrant (warp index mod 4)
    const int quadrant = warp & 3;
    const bool ready = barrier_wait(&accumulator_ready, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = m0 + quadrant * 32 + static_cast<int>(lane);
    if (ready && !failed) {
#pragma unroll 1
      for (int chunk = 0; chunk < kTileN / 32; ++chunk) {
        uint32_t v[32];
        const uint32_t address = tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + static_cast<uint32_t>(chunk * 32);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
              "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
              "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
              "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(address) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col = n0 + chunk * 32;
        if (row < p.m && col < p.n) {
          __nv_bfloat16* out = p.y + static_cast<int64_t>(row) * p.n + col;
          if (col + 32 <= p.n && (p.n & 7) == 0) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t packed[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int c = g * 8 + j * 2;
                const float b0 = p.bias ? __bfloat162float(p.bias[col + c]) : 0.0f;
                const float b1 = p.bias ? __bfloat162float(p.bias[col + c + 1]) : 0.0f;
                const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(v[c]) + b0, __uint_as_float(v[c + 1]) + b1);
                packed[j] = *reinterpret_cast<const uint32_t*>(&pair);
              }
              *reinterpret_cast<uint4*>(out + g * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          } else {
            for (int c = 0; c < 32 && col + c < p.n; ++c) {
              const float b = p.bias ? __bfloat162float(p.bias[col + c]) : 0.0f;
              out[c] = __float2bfloat16_rn(__uint_as_float(v[c]) + b);
            }
          }
        }
      }
    } else if (lane == 0) {
      failed = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
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

// rows x k bf16, row-major; boxes of 128 rows x 64 columns, 128-byte swizzle, zero fill outside the tensor
bool make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k) {
  EncodeTiled encode = tensor_map_encoder();
  if (!encode) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {kTileK, kTileM};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MROWS>
int launch_small(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* bias, __nv_bfloat16* y, int m, int n, int k,
                 cudaStream_t s) {
  const size_t shared = static_cast<size_t>(MROWS) * k * sizeof(__nv_bfloat16);
  if (shared > 200 * 1024) return EP_ERR_UNSUPPORTED;
  if (shared > 48 * 1024) {
    EP_CUDA_CHECK(cudaFuncSetAttribute(linear_small_m_kernel<MROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
  }
  const int warps = kSmallThreads / 32;
  const int wanted = (n + warps - 1) / warps;
  const int blocks = wanted < kSmCount * 2 ? wanted : kSmCount * 2;
  linear_small_m_kernel<MROWS><<<blocks, kSmallThreads, shared, s>>>(x, w, bias, y, m, n, k);
  return check_launch("linear_small_m_kernel");
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
  if (m <= kSmallMaxM) {
    int rc = EP_ERR_UNSUPPORTED;
    if (m == 1) rc = launch_small<1>(x, w, bias, y, mi, ni, ki, s);
    else if (m <= 4) rc = launch_small<4>(x, w, bias, y, mi, ni, ki, s);
    else if (m <= 8) rc = launch_small<8>(x, w, bias, y, mi, ni, ki, s);
    else rc = launch_small<16>(x, w, bias, y, mi, ni, ki, s);
    if (rc != EP_ERR_UNSUPPORTED) return rc;   // very wide K does not fit shared memory: use the tensor-core kernel
  }
  CUtensorMap map_x, map_w;
  if (!make_tile_map(&map_x, x_dev, m, k) || !make_tile_map(&map_w, weight_dev, n, k)) return EP_ERR_UNSUPPORTED;
  GemmParams p;
  p.bias = bias;
  p.y = y;
  p.m = mi;
  p.n = ni;
  p.k = ki;
  p.error = error_dev;
  const size_t shared = static_cast<size_t>(kStages) * 2 * kTileBytes + 1024;
  EP_CUDA_CHECK(cudaFuncSetAttribute(linear_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)));
  const dim3 grid(static_cast<unsigned>((n + kTileN - 1) / kTileN), static_cast<unsigned>((m + kTileM - 1) / kTileM));
  linear_tcgen05_kernel<<<grid, kGemmThreads, shared, s>>>(map_x, map_w, p);
  return check_launch("linear_tcgen05_kernel");
}
