// RMSNorm and LayerNorm, forward and backward, each with an optional fused residual add.
//
//   rms  : nr = bf16(r + a) (when a residual is given);  rstd = rsqrt(mean(nr^2) + eps);
//          y = bf16(nr * rstd) * (w + w_off)          (w_off = 1 for Gemma's "(1 + w)" weights)
//   ln   : same with mean subtraction and a bias.
// The normalised value is rounded to bf16 before the weight multiply, and the weight gradient
// accumulates dy * bf16(xhat) in fp32: the rounding points of the reference kernels
// (lset/kernels/rmsnorm.py:68-73,99-114; lset/kernels/residual_rmsnorm.py:58-77;
// lset/kernels/layernorm.py:73-77; lset/kernels/residual_layernorm.py:46-139).
//
// Backward runs on a persistent grid; every CTA writes one fp32 partial row of dW (and dB) to a
// caller-provided scratch buffer, and a second small kernel sums the partials.
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads)
    rms_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res_in,
                   const bf16* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ res_out,
                   float* __restrict__ rstd_out, int N, int H, float eps, float w_off) {
  __shared__ float sred[8];
  extern __shared__ float sw[];  // weights (+ offset) as fp32, shared by all rows of the CTA
  constexpr int ROWS = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  for (int i = threadIdx.x; i < H; i += kRowThreads) sw[i] = __bfloat162float(w[i]) + w_off;
  __syncthreads();
  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    float xv[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        unpack8(ld16(x + row * H + idx), xv[v]);
        if (res_in != nullptr) {
          float rv[8];
          unpack8(ld16(res_in + row * H + idx), rv);
#pragma unroll
          for (int i = 0; i < 8; ++i) xv[v][i] = bf16_round(xv[v][i] + rv[i]);
          st16(res_out + row * H + idx, pack8(xv[v]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += xv[v][i] * xv[v][i];
      }
    }
    ss = row_sum<TPR>(ss, sred);
    const float rstd = rsqrtf(ss / float(H) + eps);
    if (valid && t == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float o[8];
        const float4 w0 = *reinterpret_cast<const float4*>(sw + idx);
        const float4 w1 = *reinterpret_cast<const float4*>(sw + idx + 4);
        const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = bf16_round(xv[v][i] * rstd) * wl[i];
        st16(y + row * H + idx, pack8(o));
      }
    }
  }
}

// Gemma's post-norm pair in one pass: z = bf16(bf16(a·rstd1)·w1); nr = bf16(residual + z);
// y = bf16(nr·rstd2)·w2. The row stays in registers between the two norms; a, rstd1, nr and rstd2
// are what the two backward launches need.
template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads)
    rms_double_fwd_kernel(const bf16* __restrict__ a, const bf16* __restrict__ res_in,
                          const bf16* __restrict__ w1, const bf16* __restrict__ w2,
                          bf16* __restrict__ y, bf16* __restrict__ res_out,
                          float* __restrict__ rstd1_out, float* __restrict__ rstd2_out, int N, int H,
                          float eps, float w_off) {
  __shared__ float sred[8];
  extern __shared__ float sw[];  // [H] first weights, [H] second weights (+ offset)
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  constexpr int ROWS = kRowThreads / TPR;
  for (int i = threadIdx.x; i < H; i += kRowThreads) {
    sw[i] = __bfloat162float(w1[i]) + w_off;
    sw[H + i] = __bfloat162float(w2[i]) + w_off;
  }
  __syncthreads();
  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    float xv[NV][8];
    uint4 rq[NV];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        unpack8(ld16(a + row * H + idx), xv[v]);
        rq[v] = ld16(res_in + row * H + idx);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += xv[v][i] * xv[v][i];
      }
    }
    ss = row_sum<TPR>(ss, sred);
    const float rstd1 = rsqrtf(ss / float(H) + eps);
    float ss2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float rv[8];
        unpack8(rq[v], rv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float z = bf16_round(bf16_round(xv[v][i] * rstd1) * sw[idx + i]);
          xv[v][i] = bf16_round(rv[i] + z);
          ss2 += xv[v][i] * xv[v][i];
        }
        st16(res_out + row * H + idx, pack8(xv[v]));
      }
    }
    ss2 = row_sum<TPR>(ss2, sred);
    const float rstd2 = rsqrtf(ss2 / float(H) + eps);
    if (valid && t == 0) {
      rstd1_out[row] = rstd1;
      rstd2_out[row] = rstd2;
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = bf16_round(xv[v][i] * rstd2) * sw[H + idx + i];
        st16(y + row * H + idx, pack8(o));
      }
    }
  }
}

// Backward keeps x and dy as packed bf16 in registers (unpacked twice) and the weights in shared
// memory, so that only the fp32 dW accumulators are long-lived: two CTAs fit per SM.
template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads, 3)
    rms_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ dres,
                   const bf16* __restrict__ xin, const bf16* __restrict__ w,
                   const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                   float* __restrict__ dw_partial, int N, int H, float w_off) {
  __shared__ float sred[8];
  extern __shared__ float sdw[];  // [H] dW accumulator of the CTA, then [H] weights
  float* sw = sdw + H;
  constexpr int ROWS = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  float dwacc[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[v][i] = 0.f;
  for (int i = threadIdx.x; i < H; i += kRowThreads) {
    sdw[i] = 0.f;
    sw[i] = __bfloat162float(w[i]) + w_off;
  }
  __syncthreads();

  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    const float rstd = valid ? rstd_in[row] : 0.f;
    uint4 xq[NV], gq[NV], rq[NV];
    float dot = 0.f;
    // every load of the row is requested before the first use
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        xq[v] = ld16(xin + row * H + idx);
        gq[v] = ld16(dy + row * H + idx);
        if (dres != nullptr) rq[v] = ld16(dres + row * H + idx);
      }
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float xh[8], g[8];
        unpack8(xq[v], xh);
        unpack8(gq[v], g);
        const float4 w0 = *reinterpret_cast<const float4*>(sw + idx);
        const float4 w1 = *reinterpret_cast<const float4*>(sw + idx + 4);
        const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[i] *= rstd;
          dot += g[i] * wl[i] * xh[i];
          dwacc[v][i] += g[i] * bf16_round(xh[i]);
        }
      }
    }
    dot = row_sum<TPR>(dot, sred) / float(H);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float xh[8], g[8], o[8];
        unpack8(xq[v], xh);
        unpack8(gq[v], g);
        const float4 w0 = *reinterpret_cast<const float4*>(sw + idx);
        const float4 w1 = *reinterpret_cast<const float4*>(sw + idx + 4);
        const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (g[i] * wl[i] - xh[i] * rstd * dot);
        if (dres != nullptr) {
          float dr[8];
          unpack8(rq[v], dr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += dr[i];
        }
        st16(dx + row * H + idx, pack8(o));
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int idx = (v * TPR + t) * 8;
    if (idx < H) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&sdw[idx + i], dwacc[v][i]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += kRowThreads) dw_partial[1LL * blockIdx.x * H + i] = sdw[i];
}

template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads)
    ln_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res_in,
                  const bf16* __restrict__ w, const bf16* __restrict__ b, bf16* __restrict__ y,
                  bf16* __restrict__ res_out, float* __restrict__ mean_out,
                  float* __restrict__ rstd_out, int N, int H, float eps) {
  __shared__ float sred[8];
  constexpr int ROWS = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  float wv[NV][8], bv[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int idx = (v * TPR + t) * 8;
    if (idx < H) {
      unpack8(ld16(w + idx), wv[v]);
      if (b != nullptr) {
        unpack8(ld16(b + idx), bv[v]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) bv[v][i] = 0.f;
      }
    }
  }
  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    float xv[NV][8];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        unpack8(ld16(x + row * H + idx), xv[v]);
        if (res_in != nullptr) {
          float rv[8];
          unpack8(ld16(res_in + row * H + idx), rv);
#pragma unroll
          for (int i = 0; i < 8; ++i) xv[v][i] = bf16_round(xv[v][i] + rv[i]);
          st16(res_out + row * H + idx, pack8(xv[v]));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) s += xv[v][i];
      }
    }
    const float mean = row_sum<TPR>(s, sred) / float(H);
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = xv[v][i] - mean;
          ss += d * d;
        }
      }
    }
    const float rstd = rsqrtf(row_sum<TPR>(ss, sred) / float(H) + eps);
    if (valid && t == 0) {
      if (mean_out != nullptr) mean_out[row] = mean;
      if (rstd_out != nullptr) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = bf16_round((xv[v][i] - mean) * rstd) * wv[v][i] + bv[v][i];
        st16(y + row * H + idx, pack8(o));
      }
    }
  }
}

template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads)
    ln_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ dres,
                  const bf16* __restrict__ xin, const bf16* __restrict__ w,
                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                  bf16* __restrict__ dx, float* __restrict__ dwb_partial, int N, int H) {
  __shared__ float sred[8];
  extern __shared__ float sdw[];  // [2, H]: dW then dB
  constexpr int ROWS = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  float wv[NV][8], dwacc[NV][8], dbacc[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int idx = (v * TPR + t) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[v][i] = dbacc[v][i] = 0.f;
    if (idx < H) unpack8(ld16(w + idx), wv[v]);
  }
  for (int i = threadIdx.x; i < 2 * H; i += kRowThreads) sdw[i] = 0.f;

  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    const float rstd = valid ? rstd_in[row] : 0.f;
    const float mean = valid ? mean_in[row] : 0.f;
    float xh[NV][8], m[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float g[8];
        unpack8(ld16(xin + row * H + idx), xh[v]);
        unpack8(ld16(dy + row * H + idx), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[v][i] = (xh[v][i] - mean) * rstd;
          m[v][i] = g[i] * wv[v][i];
          s1 += m[v][i];
          s2 += m[v][i] * xh[v][i];
          dwacc[v][i] += g[i] * bf16_round(xh[v][i]);
          dbacc[v][i] += g[i];
        }
      }
    }
    s1 = row_sum<TPR>(s1, sred) / float(H);
    s2 = row_sum<TPR>(s2, sred) / float(H);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int idx = (v * TPR + t) * 8;
      if (valid && idx < H) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (m[v][i] - s1 - xh[v][i] * s2);
        if (dres != nullptr) {
          float dr[8];
          unpack8(ld16(dres + row * H + idx), dr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += dr[i];
        }
        st16(dx + row * H + idx, pack8(o));
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int idx = (v * TPR + t) * 8;
    if (idx < H) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        atomicAdd(&sdw[idx + i], dwacc[v][i]);
        atomicAdd(&sdw[H + idx + i], dbacc[v][i]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * H; i += kRowThreads)
    dwb_partial[1LL * blockIdx.x * 2 * H + i] = sdw[i];
}

// out[c] (+)= sum_p partial[p, c]. A CTA owns 32 columns; its 32 warps each sum a slice of the
// partial rows (coalesced 128-byte reads), then the slices are combined in shared memory.
__global__ void __launch_bounds__(1024)
    colsum_kernel(const float* __restrict__ partial, int P, int C, void* out, int out_fp32,
                  int accumulate) {
  __shared__ float sm[32][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < C)
    for (int p = grp; p < P; p += 32) s += partial[1LL * p * C + c];
  sm[grp][lane] = s;
  __syncthreads();
  if (grp == 0 && c < C) {
    float tot = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < 32; ++g2) tot += sm[g2][lane];
    if (out_fp32) {
      float* o = reinterpret_cast<float*>(out);
      o[c] = accumulate ? o[c] + tot : tot;
    } else {
      bf16* o = reinterpret_cast<bf16*>(out);
      o[c] = __float2bfloat16_rn(accumulate ? __bfloat162float(o[c]) + tot : tot);
    }
  }
}

int bwd_grid(int N, int rows_per_cta) {
  const int need = (N + rows_per_cta - 1) / rows_per_cta;
  const int cap = row_num_sms() * 6;  // two waves at three CTAs per SM
  return need < cap ? (need > 0 ? need : 1) : cap;
}

}  // namespace
}  // namespace lb

using namespace lb;

// Number of fp32 partial rows that the backward kernels may write (scratch = rows * H floats for
// RMSNorm, rows * 2H for LayerNorm).
extern "C" int lb_norm_bwd_partial_rows() { return row_num_sms() * 8; }

extern "C" int lb_rms_norm_fwd(const void* x, const void* res_in, const void* w, void* y,
                               void* res_out, float* rstd, int N, int H, float eps, float w_off,
                               void* stream) {
  if (N <= 0) return 0;
  if (H & 7) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  LB_ROW_DISPATCH(H, {
    constexpr int ROWS = kRowThreads / TPR;
    const int grid = (N + ROWS - 1) / ROWS;
    rms_fwd_kernel<TPR, NV><<<grid, kRowThreads, H * sizeof(float), st>>>(
        (const bf16*)x, (const bf16*)res_in, (const bf16*)w, (bf16*)y, (bf16*)res_out, rstd, N, H,
        eps, w_off);
  });
  return launch_rc();
}

// Fused forward of rmsnorm(a)·w1 → + residual → rmsnorm(·)·w2. Outputs y, res_out (the new
// residual stream), rstd1 (of a) and rstd2 (of res_out).
extern "C" int lb_rms_norm_double_fwd(const void* a, const void* res_in, const void* w1,
                                      const void* w2, void* y, void* res_out, float* rstd1,
                                      float* rstd2, int N, int H, float eps, float w_off,
                                      void* stream) {
  if (N <= 0) return 0;
  if ((H & 7) || 2 * H * sizeof(float) > 48 * 1024) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  LB_ROW_DISPATCH(H, {
    constexpr int ROWS = kRowThreads / TPR;
    const int grid = (N + ROWS - 1) / ROWS;
    rms_double_fwd_kernel<TPR, NV><<<grid, kRowThreads, 2 * H * sizeof(float), st>>>(
        (const bf16*)a, (const bf16*)res_in, (const bf16*)w1, (const bf16*)w2, (bf16*)y,
        (bf16*)res_out, rstd1, rstd2, N, H, eps, w_off);
  });
  return launch_rc();
}

// dw_out: [H] fp32 or bf16; scratch: lb_norm_bwd_partial_rows() * H floats.
extern "C" int lb_rms_norm_bwd(const void* dy, const void* dres, const void* xin, const void* w,
                               const float* rstd, void* dx, float* scratch, void* dw_out,
                               int dw_fp32, int dw_accumulate, int N, int H, float w_off,
                               void* stream) {
  if (N <= 0) return 0;
  if (H & 7) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = 1;
  LB_ROW_DISPATCH_NARROW(H, {
    constexpr int ROWS = kRowThreads / TPR;
    grid = bwd_grid(N, ROWS);
    if (2 * H * sizeof(float) > 48 * 1024)  // wide rows: opt in above the 48 KB default
      cudaFuncSetAttribute(rms_bwd_kernel<TPR, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           2 * H * (int)sizeof(float));
    rms_bwd_kernel<TPR, NV><<<grid, kRowThreads, 2 * H * sizeof(float), st>>>(
        (const bf16*)dy, (const bf16*)dres, (const bf16*)xin, (const bf16*)w, rstd, (bf16*)dx,
        scratch, N, H, w_off);
  });
  if (dw_out != nullptr)
    colsum_kernel<<<(H + 31) / 32, 1024, 0, st>>>(scratch, grid, H, dw_out, dw_fp32, dw_accumulate);
  return launch_rc();
}

extern "C" int lb_layer_norm_fwd(const void* x, const void* res_in, const void* w, const void* b,
                                 void* y, void* res_out, float* mean, float* rstd, int N, int H,
                                 float eps, void* stream) {
  if (N <= 0) return 0;
  if (H & 7) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  LB_ROW_DISPATCH(H, {
    constexpr int ROWS = kRowThreads / TPR;
    const int grid = (N + ROWS - 1) / ROWS;
    ln_fwd_kernel<TPR, NV><<<grid, kRowThreads, 0, st>>>(
        (const bf16*)x, (const bf16*)res_in, (const bf16*)w, (const bf16*)b, (bf16*)y,
        (bf16*)res_out, mean, rstd, N, H, eps);
  });
  return launch_rc();
}

// dwb_out: [2, H] (dW then dB), fp32 or bf16; scratch: lb_norm_bwd_partial_rows() * 2H floats.
extern "C" int lb_layer_norm_bwd(const void* dy, const void* dres, const void* xin, const void* w,
                                 const float* mean, const float* rstd, void* dx, float* scratch,
                                 void* dwb_out, int dw_fp32, int dw_accumulate, int N, int H,
                                 void* stream) {
  if (N <= 0) return 0;
  if (H & 7) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = 1;
  LB_ROW_DISPATCH_NARROW(H, {
    constexpr int ROWS = kRowThreads / TPR;
    grid = bwd_grid(N, ROWS);
    if (2 * H * sizeof(float) > 48 * 1024)
      cudaFuncSetAttribute(ln_bwd_kernel<TPR, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           2 * H * (int)sizeof(float));
    ln_bwd_kernel<TPR, NV><<<grid, kRowThreads, 2 * H * sizeof(float), st>>>(
        (const bf16*)dy, (const bf16*)dres, (const bf16*)xin, (const bf16*)w, mean, rstd, (bf16*)dx,
        scratch, N, H);
  });
  if (dwb_out != nullptr)
    colsum_kernel<<<(2 * H + 31) / 32, 1024, 0, st>>>(scratch, grid, 2 * H, dwb_out, dw_fp32,
                                                       dw_accumulate);
  return launch_rc();
}

extern "C" int lb_colsum(const float* partial, int P, int C, void* out, int out_fp32,
                         int accumulate, void* stream) {
  if (C <= 0) return 0;
  colsum_kernel<<<(C + 31) / 32, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      partial, P, C, out, out_fp32, accumulate);
  return launch_rc();
}

// ------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (see norm_noalloc.h): same kernels as lb_rms_norm_bwd, with the
// per-CTA partials in a fixed array that is part of the library image.
// ------------------------------------------------------------------------------------------------
#include <mutex>

#include "norm_noalloc.h"

namespace {

// One copy per device that loads the library. In host code this name is only a handle for
// cudaGetSymbolAddress; the kernels receive the looked-up device address.
static __device__ __align__(256) float g_noalloc_partials[LB_NOALLOC_MAX_PARTIAL_ROWS * LB_NOALLOC_MAX_H];

constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_ptr[kNoAllocMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the array on the current device; looked up once per device.
int noalloc_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices)
    return LB_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials) != cudaSuccess ||
        p == nullptr) {
      cudaGetLastError();  // clear the sticky-free error state for the caller
      return LB_NOALLOC_ERR_SYMBOL;
    }
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace

extern "C" const char* lb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case LB_NOALLOC_ERR_TOO_LARGE:
      return "row width H exceeds LB_NOALLOC_MAX_H (4096): the built-in scratch array is too small";
    case LB_NOALLOC_ERR_SYMBOL:
      return "cudaGetSymbolAddress failed for the built-in scratch array on the current device";
    case LB_NOALLOC_ERR_DEVICE: return "current device index is outside the library's device table";
    case -3: return "bad shape: H must be a positive multiple of 8";
    case -11: return "kernel launch failed";
    default: return "unknown error";
  }
}

extern "C" int lb_rms_norm_bwd_noalloc(const void* dy, const void* dres, const void* xin,
                                       const void* w, const float* rstd, void* dx, void* dw_out,
                                       int dw_fp32, int dw_accumulate, int N, int H, float w_off,
                                       void* stream) {
  if (N <= 0) return 0;
  if (H <= 0 || (H & 7)) return -3;
  if (H > LB_NOALLOC_MAX_H) return LB_NOALLOC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int grid = 1;
  LB_ROW_DISPATCH_NARROW(H, {
    constexpr int ROWS = kRowThreads / TPR;
    grid = bwd_grid(N, ROWS);
    if (grid > LB_NOALLOC_MAX_PARTIAL_ROWS) grid = LB_NOALLOC_MAX_PARTIAL_ROWS;
    if (2 * H * sizeof(float) > 48 * 1024)  // wide rows: opt in above the 48 KB default
      cudaFuncSetAttribute(rms_bwd_kernel<TPR, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           2 * H * (int)sizeof(float));
    rms_bwd_kernel<TPR, NV><<<grid, kRowThreads, 2 * H * sizeof(float), st>>>(
        (const bf16*)dy, (const bf16*)dres, (const bf16*)xin, (const bf16*)w, rstd, (bf16*)dx,
        scratch, N, H, w_off);
  });
  if (dw_out != nullptr)
    colsum_kernel<<<(H + 31) / 32, 1024, 0, st>>>(scratch, grid, H, dw_out, dw_fp32, dw_accumulate);
  return launch_rc();
}
