// Optimiser kernels over flat fp32 buffers: sum of squares (for the global gradient norm), the clip
// coefficient, and a fused AdamW step that also writes the bf16 compute copy of the parameters and
// clears the gradient. The clip coefficient stays on the device, so a step needs no host sync.
// Replaces torch.optim.AdamW(fused=True) and clip_grad_norm_ (lset/train/engine.py:258-264,399-406).
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

__global__ void __launch_bounds__(256)
    sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float sred[8];
  float s = 0.f;
  const long long n4 = n / 4;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += 1LL * gridDim.x * blockDim.x) {
    const float4 v = x4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  }
  s = row_sum<256>(s, sred);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void __launch_bounds__(256)
    sumsq_final_kernel(const float* __restrict__ partial, int P, float* __restrict__ out,
                       int accumulate) {
  __shared__ float sred[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = row_sum<256>(s, sred);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

// coef_out[0] = min(1, max_norm / (norm + 1e-6)); coef_out[1] = norm. max_norm <= 0 disables.
// coef_out[2] = 1 when this step must not be applied: `fault` (nullable device float, e.g. the
// status words of all ranks summed) is non-zero, i.e. some kernel of the step gave up a bounded
// wait and the gradients cannot be trusted. The AdamW kernels return at once when they see it,
// so a faulted step leaves parameters and moments untouched without the host having to look.
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm,
                                 float* __restrict__ coef_out, const float* __restrict__ fault) {
  const float norm = sqrtf(sumsq[0]);
  coef_out[1] = norm;
  coef_out[0] = (max_norm > 0.f) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  coef_out[2] = (fault != nullptr && fault[0] != 0.f) ? 1.f : 0.f;
}

struct AdamArgs {
  float* p;          // fp32 master weights
  float* g;          // fp32 gradients
  float* m;
  float* v;
  bf16* p_bf16;      // nullable: bf16 compute copy written after the update
  long long n;
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, grad_scale;
  const float* coef;  // nullable: [0] clip coefficient, [2] non-zero = skip this step
  int zero_grad;
};

__global__ void __launch_bounds__(256) adamw_kernel(AdamArgs a) {
  if (a.coef != nullptr && a.coef[2] != 0.f) return;
  const float gs = a.grad_scale * (a.coef != nullptr ? a.coef[0] : 1.f);
  const float step = a.lr / a.bc1;
  const float decay = 1.f - a.lr * a.wd;
  const long long n4 = a.n / 4;
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += 1LL * gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(a.p)[i];
    float4 g = reinterpret_cast<float4*>(a.g)[i];
    float4 m = reinterpret_cast<float4*>(a.m)[i];
    float4 v = reinterpret_cast<float4*>(a.v)[i];
    float* pp = &p.x;
    float* gp = &g.x;
    float* mp = &m.x;
    float* vp = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gp[j] * gs;
      mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gj;
      vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
      const float denom = sqrtf(vp[j]) / a.bc2_sqrt + a.eps;
      pp[j] = pp[j] * decay - step * mp[j] / denom;
    }
    reinterpret_cast<float4*>(a.p)[i] = p;
    reinterpret_cast<float4*>(a.m)[i] = m;
    reinterpret_cast<float4*>(a.v)[i] = v;
    if (a.zero_grad) reinterpret_cast<float4*>(a.g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.p_bf16 != nullptr) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(a.p_bf16)[i] = o;
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < a.n; i += blockDim.x) {
      const float gj = a.g[i] * gs;
      const float mj = a.beta1 * a.m[i] + (1.f - a.beta1) * gj;
      const float vj = a.beta2 * a.v[i] + (1.f - a.beta2) * gj * gj;
      const float denom = sqrtf(vj) / a.bc2_sqrt + a.eps;
      const float pj = a.p[i] * decay - step * mj / denom;
      a.p[i] = pj;
      a.m[i] = mj;
      a.v[i] = vj;
      if (a.zero_grad) a.g[i] = 0.f;
      if (a.p_bf16 != nullptr) a.p_bf16[i] = __float2bfloat16_rn(pj);
    }
  }
}

}  // namespace
}  // namespace lb

using namespace lb;

extern "C" int lb_sumsq_partial_rows() { return row_num_sms() * 4; }

// out[0] (+)= sum(x^2). scratch: lb_sumsq_partial_rows() floats.
extern "C" int lb_sumsq_f32(const float* x, long long n, float* scratch, float* out, int accumulate,
                            void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return -3;
  long long g = (n / 4 + 255) / 256;
  const long long cap = lb_sumsq_partial_rows();
  const int grid = int(g < 1 ? 1 : (g > cap ? cap : g));
  sumsq_partial_kernel<<<grid, 256, 0, st>>>(x, n, scratch);
  sumsq_final_kernel<<<1, 256, 0, st>>>(scratch, grid, out, accumulate);
  return launch_rc();
}

// coef_out: 3 floats (see clip_coef_kernel); fault: nullable device float.
extern "C" int lb_clip_coef(const float* sumsq, float max_norm, float* coef_out, const float* fault,
                            void* stream) {
  clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, coef_out,
                                                                        fault);
  return launch_rc();
}

extern "C" int lb_adamw_f32(float* p, float* g, float* m, float* v, void* p_bf16, long long n,
                            float lr, float beta1, float beta2, float eps, float wd, float bc1,
                            float bc2_sqrt, float grad_scale, const float* coef, int zero_grad,
                            void* stream) {
  if (n <= 0) return 0;
  if (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
        reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) != 0)
    return -3;
  if (p_bf16 != nullptr && (reinterpret_cast<uintptr_t>(p_bf16) & 7u) != 0) return -3;
  AdamArgs a{p, g, m, v, (bf16*)p_bf16, n, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, grad_scale,
             coef, zero_grad};
  long long grid = (n / 4 + 255) / 256;
  const long long cap = 1LL * row_num_sms() * 16;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  adamw_kernel<<<int(grid), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return launch_rc();
}
