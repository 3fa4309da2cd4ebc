// Pooling and L2 normalisation kernels.
//
//   l2norm          y = x / max(||x||, eps), rows may be a prefix slice of a wider matrix
//   gather_l2norm   out[m] = l2norm(x[idx[m]])  — last-token / CLS pooling on a packed stream
//   segment_mean    out[m] = mean(x[cu[m] : cu[m+1]])  — mean pooling on a packed stream; the
//                   tokens of one segment are spread over the threads of a CTA, not walked serially
// Counterparts: lset/kernels/normalize.py:31-128, lset/kernels/pool_normalize.py:14-114,
// lset/kernels/segment_pool.py:14-147.
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

// x rows gathered through idx (nullptr = identity). Backward scatters through the same idx.
template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads)
    l2norm_fwd_kernel(const bf16* __restrict__ x, long long ldx, const long long* __restrict__ idx,
                      bf16* __restrict__ y, long long ldy, float* __restrict__ norm_out, int N,
                      int D, float eps, int normalize) {
  __shared__ float sred[8];
  constexpr int ROWS = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    const long long src = valid ? (idx != nullptr ? idx[row] : row) : 0;
    float xv[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * TPR + t) * 8;
      if (valid && c < D) {
        unpack8(ld16(x + src * ldx + c), xv[v]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += xv[v][i] * xv[v][i];
      }
    }
    ss = row_sum<TPR>(ss, sred);
    const float nrm = fmaxf(sqrtf(ss), eps);
    const float inv = normalize ? 1.f / nrm : 1.f;
    if (valid && t == 0 && norm_out != nullptr) norm_out[row] = nrm;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * TPR + t) * 8;
      if (valid && c < D) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = xv[v][i] * inv;
        st16(y + row * ldy + c, pack8(o));
      }
    }
  }
}

// gx = (gy - y <y, gy>) / norm, written to dx[idx[row]] (rows not named by idx stay untouched).
template <int TPR, int NV>
__global__ void __launch_bounds__(kRowThreads)
    l2norm_bwd_kernel(const bf16* __restrict__ gy, long long ldgy, const bf16* __restrict__ y,
                      long long ldy, const float* __restrict__ norm_in,
                      const long long* __restrict__ idx, bf16* __restrict__ dx, long long lddx,
                      int N, int D, int normalize) {
  __shared__ float sred[8];
  constexpr int ROWS = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  for (long long row0 = 1LL * blockIdx.x * ROWS; row0 < N; row0 += 1LL * gridDim.x * ROWS) {
    const long long row = row0 + r;
    const bool valid = row < N;
    const long long dst = valid ? (idx != nullptr ? idx[row] : row) : 0;
    float gv[NV][8], yv[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * TPR + t) * 8;
      if (valid && c < D) {
        unpack8(ld16(gy + row * ldgy + c), gv[v]);
        if (normalize) {
          unpack8(ld16(y + row * ldy + c), yv[v]);
#pragma unroll
          for (int i = 0; i < 8; ++i) dot += gv[v][i] * yv[v][i];
        }
      }
    }
    if (normalize) dot = row_sum<TPR>(dot, sred);
    const float inv = (valid && normalize) ? 1.f / norm_in[row] : 1.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c = (v * TPR + t) * 8;
      if (valid && c < D) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = normalize ? (gv[v][i] - yv[v][i] * dot) * inv : gv[v][i];
        st16(dx + dst * lddx + c, pack8(o));
      }
    }
  }
}

// One CTA per segment. Threads are (column-vector, token-subset) pairs; subsets are combined in
// shared memory. weighted = 1 weights token j (1-based inside its segment) by j / sum(j).
__global__ void __launch_bounds__(kRowThreads)
    segment_mean_fwd_kernel(const bf16* __restrict__ x, const int* __restrict__ cu,
                            bf16* __restrict__ out, int H, int weighted) {
  extern __shared__ float sacc[];  // [S, H]
  const int seg = blockIdx.x;
  const int t0 = cu[seg], t1 = cu[seg + 1];
  const int len = t1 - t0;
  const int CV = min(H / 8, kRowThreads);
  const int S = kRowThreads / CV;
  const int cvi = threadIdx.x % CV;
  const int sub = threadIdx.x / CV;
  const bool active = sub < S;
  const float wden = weighted ? 0.5f * float(len) * float(len + 1) : float(len);
  for (int c = cvi * 8; c < H; c += CV * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (active) {
      for (int tok = t0 + sub; tok < t1; tok += S) {
        float v[8];
        unpack8(ld16(x + 1LL * tok * H + c), v);
        const float wt = weighted ? float(tok - t0 + 1) : 1.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += wt * v[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sacc[sub * H + c + i] = acc[i];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += kRowThreads) {
    float s = 0.f;
    for (int k = 0; k < S; ++k) s += sacc[k * H + c];
    out[1LL * seg * H + c] = __float2bfloat16_rn(len > 0 ? s / wden : 0.f);
  }
}

// dx[tok] = g[seg] * weight(tok) for every token of the segment.
__global__ void __launch_bounds__(kRowThreads)
    segment_mean_bwd_kernel(const bf16* __restrict__ g, const int* __restrict__ cu,
                            bf16* __restrict__ dx, int H, int weighted) {
  const int seg = blockIdx.x;
  const int t0 = cu[seg], t1 = cu[seg + 1];
  const int len = t1 - t0;
  if (len <= 0) return;
  const float wden = weighted ? 0.5f * float(len) * float(len + 1) : float(len);
  const int vec_per_row = H / 8;
  const long long total = 1LL * len * vec_per_row;
  for (long long i = threadIdx.x; i < total; i += kRowThreads) {
    const int tok = t0 + int(i / vec_per_row);
    const int c = int(i % vec_per_row) * 8;
    float v[8];
    unpack8(ld16(g + 1LL * seg * H + c), v);
    const float wt = (weighted ? float(tok - t0 + 1) : 1.f) / wden;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= wt;
    st16(dx + 1LL * tok * H + c, pack8(v));
  }
}

}  // namespace
}  // namespace lb

using namespace lb;

// idx: optional int64 row indices into x (gather). normalize = 0 turns this into a pure gather.
extern "C" int lb_l2norm_fwd(const void* x, long long ldx, const long long* idx, void* y,
                             long long ldy, float* norm, int N, int D, float eps, int normalize,
                             void* stream) {
  if (N <= 0) return 0;
  if ((D & 7) || (ldx & 7) || (ldy & 7)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  LB_ROW_DISPATCH(D, {
    constexpr int ROWS = kRowThreads / TPR;
    const int grid = (N + ROWS - 1) / ROWS;
    l2norm_fwd_kernel<TPR, NV><<<grid, kRowThreads, 0, st>>>((const bf16*)x, ldx, idx, (bf16*)y,
                                                             ldy, norm, N, D, eps, normalize);
  });
  return launch_rc();
}

extern "C" int lb_l2norm_bwd(const void* gy, long long ldgy, const void* y, long long ldy,
                             const float* norm, const long long* idx, void* dx, long long lddx,
                             int N, int D, int normalize, void* stream) {
  if (N <= 0) return 0;
  if ((D & 7) || (ldgy & 7) || (ldy & 7) || (lddx & 7)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  LB_ROW_DISPATCH(D, {
    constexpr int ROWS = kRowThreads / TPR;
    const int grid = (N + ROWS - 1) / ROWS;
    l2norm_bwd_kernel<TPR, NV><<<grid, kRowThreads, 0, st>>>(
        (const bf16*)gy, ldgy, (const bf16*)y, ldy, norm, idx, (bf16*)dx, lddx, N, D, normalize);
  });
  return launch_rc();
}

extern "C" int lb_segment_mean_fwd(const void* x, const int* cu_seqlens, void* out, int M, int H,
                                   int weighted, void* stream) {
  if (M <= 0) return 0;
  if (H & 7) return -3;
  const int CV = (H / 8) < kRowThreads ? (H / 8) : kRowThreads;
  const int S = kRowThreads / CV;
  const size_t smem = size_t(S) * H * sizeof(float);
  if (smem > 48 * 1024) return -3;
  segment_mean_fwd_kernel<<<M, kRowThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)x, cu_seqlens, (bf16*)out, H, weighted);
  return launch_rc();
}

extern "C" int lb_segment_mean_bwd(const void* g, const int* cu_seqlens, void* dx, int M, int H,
                                   int weighted, void* stream) {
  if (M <= 0) return 0;
  if (H & 7) return -3;
  segment_mean_bwd_kernel<<<M, kRowThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)g, cu_seqlens, (bf16*)dx, H, weighted);
  return launch_rc();
}
