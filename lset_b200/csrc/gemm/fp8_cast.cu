// Dynamic-scaling casts from bf16 to 8-bit floats (e4m3 / e5m2) for the kind::f8f6f4 GEMM.
//
// Two kernels:
//   fp8_amax_kernel  max |x| per tensor, per row or per column (bit pattern of a non-negative
//                    float, reduced with integer atomicMax)
//   fp8_cast_kernel  q = sat(x * fmax / amax) as 8-bit floats, written row-major and / or transposed
//                    (the GEMM wants both operands K-major, so the products of the backward pass read
//                    transposed copies), plus the dequantisation factors amax / fmax.
//
// Takes the place of torchao's float8 cast kernels behind the reference's FP8 training switch
// (lset/train/quantization/fp8.py:11-45).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {
namespace {

constexpr float kAmaxFloor = 1e-12f;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// MODE 0: one value for the tensor; 1: one per row; 2: one per column.
// Block: 256 threads over a 32-row x 256-column tile; lane = 8 consecutive columns.
template <int MODE>
__global__ void __launch_bounds__(256) fp8_amax_kernel(const __nv_bfloat16* __restrict__ x, int R,
                                                       int C, long long ldx,
                                                       unsigned* __restrict__ out) {
  __shared__ unsigned s_col[256];
  __shared__ unsigned s_warp[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * 32 + warp * 4;
  if (MODE == 2) s_col[threadIdx.x] = 0u;
  if (MODE == 2) __syncthreads();
  float cm[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float tmax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + i;
    float rm = 0.f;
    if (r < R && c0 < C) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)r * ldx + c0);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = fabsf(bf16_lo(w[j])), b = fabsf(bf16_hi(w[j]));
        cm[2 * j] = fmaxf(cm[2 * j], a);
        cm[2 * j + 1] = fmaxf(cm[2 * j + 1], b);
        rm = fmaxf(rm, fmaxf(a, b));
      }
    }
    if (MODE == 1) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, o));
      if (lane == 0 && r < R && rm > 0.f) atomicMax(out + r, __float_as_uint(rm));
    }
    tmax = fmaxf(tmax, rm);
  }
  if (MODE == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    if (lane == 0) s_warp[warp] = __float_as_uint(tmax);
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned m = 0u;
      for (int i = 0; i < 8; ++i) m = max(m, s_warp[i]);
      if (m > 0u) atomicMax(out, m);
    }
  }
  if (MODE == 2) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (cm[j] > 0.f) atomicMax(&s_col[lane * 8 + j], __float_as_uint(cm[j]));
    __syncthreads();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < C && s_col[threadIdx.x] > 0u) atomicMax(out + c, s_col[threadIdx.x]);
  }
}

template <int E5M2>
__device__ __forceinline__ uint32_t cvt4(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t kind = E5M2 ? __NV_E5M2 : __NV_E4M3;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
  return lo | (hi << 16);
}

// Block: 256 threads over a 64 x 64 tile. Scale of element (r, c): fmax / max(amax, floor) with
// amax per tensor (MODE 0), per row (1) or per column (2).
template <int MODE, int E5M2>
__global__ void __launch_bounds__(256)
    fp8_cast_kernel(const __nv_bfloat16* __restrict__ x, int R, int C, long long ldx,
                    const unsigned* __restrict__ amax, uint8_t* __restrict__ out, long long ldo,
                    uint8_t* __restrict__ out_t, long long ldt, float* __restrict__ inv_scale) {
  constexpr float kFmax = E5M2 ? 57344.f : 448.f;
  constexpr int kStride = 68;  // bytes per tile row in shared memory
  __shared__ __align__(16) uint8_t tile[64 * kStride];
  __shared__ float s_scale[64];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  if (threadIdx.x < 64) {
    float am;
    if (MODE == 0) {
      am = __uint_as_float(amax[0]);
    } else if (MODE == 1) {
      am = (r0 + threadIdx.x < R) ? __uint_as_float(amax[r0 + threadIdx.x]) : 1.f;
    } else {
      am = (c0 + threadIdx.x < C) ? __uint_as_float(amax[c0 + threadIdx.x]) : 1.f;
    }
    am = fmaxf(am, kAmaxFloor);
    s_scale[threadIdx.x] = kFmax / am;
    if (inv_scale != nullptr) {
      if (MODE == 0) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) inv_scale[0] = am / kFmax;
      } else if (MODE == 1) {
        if (blockIdx.x == 0 && r0 + threadIdx.x < R) inv_scale[r0 + threadIdx.x] = am / kFmax;
      } else {
        if (blockIdx.y == 0 && c0 + threadIdx.x < C) inv_scale[c0 + threadIdx.x] = am / kFmax;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int item = threadIdx.x + u * 256;  // 64 rows x 8 groups of 8 columns
    const int lr = item >> 3, lc = (item & 7) * 8;
    const int r = r0 + lr, c = c0 + lc;
    uint32_t q0 = 0u, q1 = 0u;
    if (r < R && c < C) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)r * ldx + c);
      float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                    bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
      if (MODE == 2) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= s_scale[lc + j];
      } else {
        const float s = s_scale[MODE == 1 ? lr : 0];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= s;
      }
      q0 = cvt4<E5M2>(f[0], f[1], f[2], f[3]);
      q1 = cvt4<E5M2>(f[4], f[5], f[6], f[7]);
      if (out != nullptr) *reinterpret_cast<uint2*>(out + (long long)r * ldo + c) = make_uint2(q0, q1);
    }
    if (out_t != nullptr) {
      *reinterpret_cast<uint32_t*>(tile + lr * kStride + lc) = q0;
      *reinterpret_cast<uint32_t*>(tile + lr * kStride + lc + 4) = q1;
    }
  }
  if (out_t == nullptr) return;
  __syncthreads();
  // transposed write: row c of out_t holds column c of x; 16 source rows per thread
  const int tc = threadIdx.x >> 2, tr = (threadIdx.x & 3) * 16;
  if (c0 + tc < C && r0 + tr < ldt) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t acc = 0u;
#pragma unroll
      for (int b = 0; b < 4; ++b)
        acc |= uint32_t(tile[(tr + 4 * j + b) * kStride + tc]) << (8 * b);
      w[j] = acc;
    }
    *reinterpret_cast<uint4*>(out_t + (long long)(c0 + tc) * ldt + r0 + tr) =
        make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace
}  // namespace lb

// max |x| of a bf16 matrix [R, C] (row stride ldx elements; C and ldx multiples of 8).
// mode 0: out[0]; 1: out[R]; 2: out[C]. `out` receives the bit patterns (zero where all zero).
extern "C" int lb_fp8_amax(const void* x, int R, int C, long long ldx, int mode, unsigned* out,
                           void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (R <= 0 || C <= 0) return 0;
  if ((C & 7) || (ldx & 7) || mode < 0 || mode > 2) return -3;
  const size_t n = mode == 0 ? 1 : (mode == 1 ? size_t(R) : size_t(C));
  if (cudaMemsetAsync(out, 0, n * sizeof(unsigned), stream) != cudaSuccess) return -11;
  dim3 grid((C + 255) / 256, (R + 31) / 32);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  if (mode == 0)
    fp8_amax_kernel<0><<<grid, 256, 0, stream>>>(xp, R, C, ldx, out);
  else if (mode == 1)
    fp8_amax_kernel<1><<<grid, 256, 0, stream>>>(xp, R, C, ldx, out);
  else
    fp8_amax_kernel<2><<<grid, 256, 0, stream>>>(xp, R, C, ldx, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Quantise x [R, C] with the maxima from lb_fp8_amax (same mode). out: [R, ldo] bytes (nullable),
// out_t: [C, ldt] bytes (nullable; ldt >= R and a multiple of 16, bytes past R are written as
// zero up to ldt), inv_scale: dequantisation factors (1, R or C floats; nullable).
extern "C" int lb_fp8_cast(const void* x, int R, int C, long long ldx, int mode,
                           const unsigned* amax, int e5m2, void* out, long long ldo, void* out_t,
                           long long ldt, float* inv_scale, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (R <= 0 || C <= 0) return 0;
  if ((C & 7) || (ldx & 7) || mode < 0 || mode > 2) return -3;
  if (out != nullptr && ((ldo & 7) || ldo < C)) return -3;
  if (out_t != nullptr && ((ldt & 15) || ldt < R)) return -3;
  dim3 grid((C + 63) / 64, (R + 63) / 64);
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  uint8_t* o = reinterpret_cast<uint8_t*>(out);
  uint8_t* ot = reinterpret_cast<uint8_t*>(out_t);
#define LB_CAST(MODE, E)                                                                    \
  fp8_cast_kernel<MODE, E><<<grid, 256, 0, stream>>>(xp, R, C, ldx, amax, o, ldo, ot, ldt, \
                                                     inv_scale)
  if (e5m2) {
    if (mode == 0) LB_CAST(0, 1);
    else if (mode == 1) LB_CAST(1, 1);
    else LB_CAST(2, 1);
  } else {
    if (mode == 0) LB_CAST(0, 0);
    else if (mode == 1) LB_CAST(1, 0);
    else LB_CAST(2, 0);
  }
#undef LB_CAST
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
