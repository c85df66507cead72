// Device helpers shared by the tensor-core (tcgen05) kernels: swizzled operand addressing, per-warp barrier arrivals,
// bounded waits that unwind the whole CTA, the fast stablemax transform, and the host-side tensor-map encoder.
#pragma once
#include <cuda.h>

#include "flare_common.cuh"
#include "sm100_ptx.cuh"

namespace flare {
namespace tc {

using namespace sm100;

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a [rows][64 x bf16] operand block with 128-byte swizzle
__device__ __forceinline__ uint32_t swz_chunk_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// One arrival per warp: 32 lanes arriving one by one are 32 serialised shared-memory atomics.  __syncwarp orders the
// lanes' earlier writes before lane 0's releasing arrive.
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// Bounded wait that also gives up as soon as another role of the CTA has given up (`abort_flag` set).  The wait
// suspends in hardware in slices of at most kWaitSliceNs and wakes on completion.  The bound is a count of slices (kWaitSlices x kWaitSliceNs = 2 s when every slice runs its
// full length) rather than a wall-clock reading: reading %globaltimer on this path cost about a microsecond per wait.
constexpr uint32_t kWaitSliceNs = 20000u;
constexpr uint32_t kWaitSlices = 100000u;
// `polls`: how many cheap test-and-branch rounds come before the first suspension.  Every round is a handful of
// instructions issued on the waiting warp's scheduler, where they compete with the working warps: use a few dozen only
// where the partner is known to be at most a few hundred cycles behind, 1-2 where the wait is expected to be long.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int polls) {
#pragma unroll 1
  for (int spin = 0; spin < polls; ++spin)
    if (mbar_test_wait(bar, parity)) return true;
#pragma unroll 1
  for (uint32_t slice = 0; slice < kWaitSlices; ++slice) {
    if (mbar_try_wait(bar, parity, kWaitSliceNs)) return true;  // sleeps in hardware, wakes on completion
    if (*abort_flag != 0) return false;
  }
  return false;
}

// the same for a barrier that threads of the partner CTA of a cluster arrive on
__device__ __forceinline__ bool wait_or_abort_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
  for (uint32_t slice = 0; slice < kWaitSlices; ++slice) {
    if (mbar_try_wait_cluster(bar, parity, kWaitSliceNs)) return true;
    if (*abort_flag != 0) return false;
  }
  return false;
}

// stablemax encoder weight with approximate reciprocal; powers 1..4 by multiplication
__device__ __forceinline__ float sigma_fast(float x, float p) {
  const float base = 1.0f + fabsf(x);
  float r;
  if (p == 1.0f) r = base;
  else if (p == 2.0f) r = base * base;
  else if (p == 3.0f) r = base * base * base;
  else if (p == 4.0f) { const float b2 = base * base; r = b2 * b2; }
  else r = exp2f(p * __log2f(base));
  return x >= 0.0f ? r : rcp_approx(r);
}

__device__ __forceinline__ float bf16_lo(uint32_t pk) { return __uint_as_float(pk << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pk) { return __uint_as_float(pk & 0xffff0000u); }

// K-major operand in a [blocks][128 rows][64] buffer: k-step j covers 16 elements of the contraction
__device__ __forceinline__ uint64_t kmaj_step(uint64_t desc, int j) {
  return desc + (uint64_t)(((j >> 2) * 16384 + (j & 3) * 32) >> 4);
}
// MN-major operand (contraction along the rows): k-step j covers 16 rows
__device__ __forceinline__ uint64_t mnmaj_step(uint64_t desc, int j) { return desc + (uint64_t)((j * 2048) >> 4); }

// ---------------------------------------------------------------------------------------------
// host: bf16 tensor map with 128-byte swizzle.  dims innermost first, strides in elements for dims 1..rank-1.
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

// (any 16-bit element type: the copies do no arithmetic)
inline bool make_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const int64_t* strides_elems,
                          const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[5], gstride[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstride[i] = (cuuint64_t)strides_elems[i] * 2;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bx, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace flare
