// Shared pieces of the row-wise (bandwidth-bound) kernels: a row of H bf16 elements is held in the
// registers of TPR threads as NV vectors of 8 elements each; 256-thread CTAs process 256/TPR rows
// at a time. Row statistics are reduced with warp shuffles (and one shared-memory hop when a row
// spans several warps).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

constexpr int kRowThreads = 256;

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// Streaming variants: data touched once should not displace what later kernels reuse from L2.
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Sum over the TPR threads that own one row. `sred` is a shared float[8] (one slot per warp).
// Must be called by every thread of the CTA when TPR > 32 (it contains __syncthreads).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* sred) {
#pragma unroll
  for (int o = (TPR < 32 ? TPR : 32) / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (TPR > 32) {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) sred[warp] = v;
    __syncthreads();
    constexpr int W = TPR / 32;
    const int w0 = (warp / W) * W;
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < W; ++i) t += sred[w0 + i];
    __syncthreads();
    v = t;
  }
  return v;
}

// Dispatch on the row width: picks (TPR, NV) with TPR * NV * 8 >= H.
#define LB_ROW_DISPATCH(H, ...)                                    \
  do {                                                             \
    if ((H) <= 128) {                                              \
      constexpr int TPR = 16, NV = 1;                              \
      __VA_ARGS__;                                                      \
    } else if ((H) <= 256) {                                       \
      constexpr int TPR = 32, NV = 1;                              \
      __VA_ARGS__;                                                      \
    } else if ((H) <= 512) {                                       \
      constexpr int TPR = 32, NV = 2;                              \
      __VA_ARGS__;                                                      \
    } else if ((H) <= 1024) {                                      \
      constexpr int TPR = 32, NV = 4;                              \
      __VA_ARGS__;                                                      \
    } else if ((H) <= 2048) {                                      \
      constexpr int TPR = 64, NV = 4;                              \
      __VA_ARGS__;                                                      \
    } else if ((H) <= 4096) {                                      \
      constexpr int TPR = 128, NV = 4;                             \
      __VA_ARGS__;                                                      \
    } else if ((H) <= 8192) {                                      \
      constexpr int TPR = 256, NV = 4;                             \
      __VA_ARGS__;                                                      \
    } else {                                                       \
      return -3;                                                   \
    }                                                              \
  } while (0)

// Narrow variant for kernels with long-lived per-column accumulators (backward passes): twice the
// threads per row, half the vectors per thread, so that more CTAs fit per SM.
#define LB_ROW_DISPATCH_NARROW(H, ...)                              \
  do {                                                             \
    if ((H) <= 128) {                                              \
      constexpr int TPR = 16, NV = 1;                              \
      __VA_ARGS__;                                                 \
    } else if ((H) <= 256) {                                       \
      constexpr int TPR = 32, NV = 1;                              \
      __VA_ARGS__;                                                 \
    } else if ((H) <= 512) {                                       \
      constexpr int TPR = 64, NV = 1;                              \
      __VA_ARGS__;                                                 \
    } else if ((H) <= 1024) {                                      \
      constexpr int TPR = 64, NV = 2;                              \
      __VA_ARGS__;                                                 \
    } else if ((H) <= 2048) {                                      \
      constexpr int TPR = 128, NV = 2;                             \
      __VA_ARGS__;                                                 \
    } else if ((H) <= 4096) {                                      \
      constexpr int TPR = 256, NV = 2;                             \
      __VA_ARGS__;                                                 \
    } else if ((H) <= 8192) {                                      \
      constexpr int TPR = 256, NV = 4;                             \
      __VA_ARGS__;                                                 \
    } else {                                                       \
      return -3;                                                   \
    }                                                              \
  } while (0)

inline int row_num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

inline int launch_rc() { return cudaGetLastError() == cudaSuccess ? 0 : -11; }

}  // namespace lb
