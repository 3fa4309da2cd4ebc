// Shared definitions of the varlen attention kernels.
//
// Tiling. Queries of the G = Hq / Hk heads that share one KV head are stacked along the M
// dimension of the MMA: a 128-row tile holds G heads x QT tokens (QT = 128 / G), so short
// sequences still fill the tensor-core tile and K/V tiles are loaded once per group. Row r of a
// tile is head g = r / QT, token tok0 + r % QT.
//
// Plan. Sequence lengths live on the device; a one-block planning kernel turns cu_seqlens into a
// list of (sequence, tile) pairs that every layer's forward and backward launch reuses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

constexpr int kAttnKvBlock = 64;   // KV rows per inner step of the forward and dQ kernels
constexpr int kLog2e = 0;          // (placeholder to keep the namespace non-empty for constexprs)
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

// plan[0] = number of tiles; then (sequence index, tile index within the sequence) pairs.
struct AttnPlanView {
  const int* data;
  __device__ __forceinline__ int count() const { return data[0]; }
  __device__ __forceinline__ int seq(int i) const { return data[1 + 2 * i]; }
  __device__ __forceinline__ int tile(int i) const { return data[2 + 2 * i]; }
};

}  // namespace lb
