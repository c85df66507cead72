// Shared device/host helpers for the FLARE B200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/flare_b200.h"

namespace flare {

constexpr float kNegInf = -INFINITY;

// ---------------------------------------------------------------------------------------------
// host-side error plumbing
// ---------------------------------------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* where);

#define FLARE_CUDA_CHECK(expr)                         \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) {                           \
      ::flare::set_cuda_error(_e, #expr);              \
      return FLARE_ERR_CUDA;                           \
    }                                                  \
  } while (0)

int sm_count();

// Per-kernel timing for callers that ask for a profile (the reference's profile=True returns one entry per kernel
// launch, causal_flare/autoregressive/training.py:4-50).  While switched on (flare_profile_enable) every launch site
// brackets its kernel with a pair of CUDA events on the launch stream; flare_profile_entry reads them back.
struct LaunchTimer {
  LaunchTimer(const char* name, cudaStream_t stream);
  ~LaunchTimer();
  int slot;
  cudaStream_t stream;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline int dtype_size(int dtype) { return dtype == FLARE_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------------------------
// runtime-typed element access (dtype is uniform per launch, so these branches never diverge)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// Load 8 consecutive elements starting at element index `off` (off % 8 == 0, base 16-byte aligned).
__device__ __forceinline__ void load8(const void* base, int dtype, int64_t off, float (&out)[8]) {
  if (dtype == FLARE_F32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    float4 a = __ldg(p), b = __ldg(p + 1);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + off));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    if (dtype == FLARE_BF16) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[2 * i] = bf16_bits_to_float(w[i] & 0xffffu);
        out[2 * i + 1] = bf16_bits_to_float(w[i] >> 16);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        const float2 f = __half22float2(h);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
      }
    }
  }
}

__device__ __forceinline__ float load1(const void* base, int dtype, int64_t off) {
  if (dtype == FLARE_F32) return reinterpret_cast<const float*>(base)[off];
  if (dtype == FLARE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
  return __half2float(reinterpret_cast<const __half*>(base)[off]);
}

__device__ __forceinline__ void store1(void* base, int dtype, int64_t off, float x) {
  if (dtype == FLARE_F32) reinterpret_cast<float*>(base)[off] = x;
  else if (dtype == FLARE_BF16) reinterpret_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(x);
  else reinterpret_cast<__half*>(base)[off] = __float2half_rn(x);
}

// Store 4 consecutive elements (off % 4 == 0, base 16-byte aligned).
__device__ __forceinline__ void store4(void* base, int dtype, int64_t off, float a, float b, float c, float d) {
  if (dtype == FLARE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off) = make_float4(a, b, c, d);
  } else if (dtype == FLARE_BF16) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&lo);
    r.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + off) = r;
  } else {
    __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&lo);
    r.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + off) = r;
  }
}

// ---------------------------------------------------------------------------------------------
// score transforms
// ---------------------------------------------------------------------------------------------
// sigma(x) = (1+x)^p for x >= 0, (1-x)^-p for x < 0.
__device__ __forceinline__ float stablemax_sigma(float x, float p) {
  const float base = 1.0f + fabsf(x);
  float r;
  if (p == 1.0f) r = base;
  else if (p == 2.0f) r = base * base;
  else if (p == 3.0f) r = base * base * base;
  else if (p == 4.0f) { const float b2 = base * base; r = b2 * b2; }
  else r = exp2f(p * log2f(base));
  return x >= 0.0f ? r : 1.0f / r;
}

// sigma'(x) / sigma(x) = p / (1 + |x|) on both branches.
__device__ __forceinline__ float stablemax_slope_ratio(float x, float p) { return p / (1.0f + fabsf(x)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace flare
