// Gated activations and GELU, forward and backward, as flat 16-byte-vector kernels.
//
//   swiglu: out = silu(gate) * up          geglu: out = gelu_tanh(gate) * up       gelu: exact (erf)
// gate and up may be the two halves of one fused gate_up projection output (explicit row strides),
// and the backward writes d_gate and d_up side by side so a fused projection gets one dgrad GEMM.
// Counterparts: lset/kernels/swiglu.py:21-74, lset/kernels/geglu.py:22-86, aten GELU in
// lset/models/encoder/bert/model.py:107.
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

enum { kSwiglu = 0, kGeglu = 1 };

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ float gelu_tanh_(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad_(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

template <int KIND>
__global__ void __launch_bounds__(256)
    glu_fwd_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up, long long ld_in,
                   bf16* __restrict__ out, long long ld_out, long long T, int I) {
  const int vec_per_row = I / 8;
  const long long total = T * vec_per_row;
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += 1LL * gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = int(i % vec_per_row) * 8;
    float g[8], u[8], o[8];
    unpack8(ld16(gate + r * ld_in + c), g);
    unpack8(ld16(up + r * ld_in + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = KIND == kSwiglu ? g[j] * sigmoidf_(g[j]) : gelu_tanh_(g[j]);
      o[j] = a * u[j];
    }
    st16(out + r * ld_out + c, pack8(o));
  }
}

template <int KIND>
__global__ void __launch_bounds__(256)
    glu_bwd_kernel(const bf16* __restrict__ dout, long long ld_dout, const bf16* __restrict__ gate,
                   const bf16* __restrict__ up, long long ld_in, bf16* __restrict__ dgate,
                   bf16* __restrict__ dup, long long ld_d, long long T, int I) {
  const int vec_per_row = I / 8;
  const long long total = T * vec_per_row;
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += 1LL * gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = int(i % vec_per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld16(gate + r * ld_in + c), g);
    unpack8(ld16(up + r * ld_in + c), u);
    unpack8(ld16(dout + r * ld_dout + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float act, dact;
      if (KIND == kSwiglu) {
        const float s = sigmoidf_(g[j]);
        act = g[j] * s;
        dact = s * (1.f + g[j] * (1.f - s));
      } else {
        act = gelu_tanh_(g[j]);
        dact = gelu_tanh_grad_(g[j]);
      }
      du[j] = d[j] * act;
      dg[j] = d[j] * u[j] * dact;
    }
    st16(dgate + r * ld_d + c, pack8(dg));
    st16(dup + r * ld_d + c, pack8(du));
  }
}

__global__ void __launch_bounds__(256)
    gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n8) {
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += 1LL * gridDim.x * blockDim.x) {
    float v[8];
    unpack8(ld16(x + i * 8), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.5f * v[j] * (1.f + erff(v[j] * 0.7071067811865476f));
    st16(y + i * 8, pack8(v));
  }
}

__global__ void __launch_bounds__(256)
    gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx,
                    long long n8) {
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += 1LL * gridDim.x * blockDim.x) {
    float v[8], g[8];
    unpack8(ld16(x + i * 8), v);
    unpack8(ld16(dy + i * 8), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cdf = 0.5f * (1.f + erff(v[j] * 0.7071067811865476f));
      const float pdf = 0.3989422804014327f * __expf(-0.5f * v[j] * v[j]);
      g[j] *= cdf + v[j] * pdf;
    }
    st16(dx + i * 8, pack8(g));
  }
}

int flat_grid(long long work_items) {
  long long g = (work_items + 255) / 256;
  const long long cap = 1LL * row_num_sms() * 16;
  if (g > cap) g = cap;
  return int(g > 0 ? g : 1);
}

}  // namespace
}  // namespace lb

using namespace lb;

// kind: 0 = SwiGLU, 1 = GeGLU (tanh). gate/up rows are ld_in apart; I must be a multiple of 8.
extern "C" int lb_glu_fwd(int kind, const void* gate, const void* up, long long ld_in, void* out,
                          long long ld_out, long long T, int I, void* stream) {
  if (T <= 0 || I <= 0) return 0;
  if ((I & 7) || (ld_in & 7) || (ld_out & 7)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = flat_grid(T * (I / 8));
  if (kind == kSwiglu)
    glu_fwd_kernel<kSwiglu><<<grid, 256, 0, st>>>((const bf16*)gate, (const bf16*)up, ld_in,
                                                  (bf16*)out, ld_out, T, I);
  else
    glu_fwd_kernel<kGeglu><<<grid, 256, 0, st>>>((const bf16*)gate, (const bf16*)up, ld_in,
                                                 (bf16*)out, ld_out, T, I);
  return launch_rc();
}

extern "C" int lb_glu_bwd(int kind, const void* dout, long long ld_dout, const void* gate,
                          const void* up, long long ld_in, void* dgate, void* dup, long long ld_d,
                          long long T, int I, void* stream) {
  if (T <= 0 || I <= 0) return 0;
  if ((I & 7) || (ld_in & 7) || (ld_dout & 7) || (ld_d & 7)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = flat_grid(T * (I / 8));
  if (kind == kSwiglu)
    glu_bwd_kernel<kSwiglu><<<grid, 256, 0, st>>>((const bf16*)dout, ld_dout, (const bf16*)gate,
                                                  (const bf16*)up, ld_in, (bf16*)dgate, (bf16*)dup,
                                                  ld_d, T, I);
  else
    glu_bwd_kernel<kGeglu><<<grid, 256, 0, st>>>((const bf16*)dout, ld_dout, (const bf16*)gate,
                                                 (const bf16*)up, ld_in, (bf16*)dgate, (bf16*)dup,
                                                 ld_d, T, I);
  return launch_rc();
}

extern "C" int lb_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n & 7) return -3;
  gelu_fwd_kernel<<<flat_grid(n / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)x, (bf16*)y, n / 8);
  return launch_rc();
}

extern "C" int lb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n & 7) return -3;
  gelu_bwd_kernel<<<flat_grid(n / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)dy, (const bf16*)x, (bf16*)dx, n / 8);
  return launch_rc();
}
