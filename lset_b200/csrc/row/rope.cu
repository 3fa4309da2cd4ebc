// Per-head RMSNorm fused with rotary position embedding for Q and K, forward and backward, plus
// the rope-only variant (do_norm = 0). One launch handles every (token, head) of both Q and K; the
// cos/sin rows are gathered by position id inside the kernel.
//
//   xn = bf16(x * rstd) * w            (per head, statistics over head_dim, when do_norm)
//   y[:h/2] = xn[:h/2] * cos - xn[h/2:] * sin ;  y[h/2:] = xn[h/2:] * cos + xn[:h/2] * sin
//
// Counterpart of the reference's Triton kernels (lset/kernels/qk_norm_rope.py:79-134,191-287 and
// lset/kernels/rope.py:12-75). Inputs may be slices of a fused QKV projection output (row strides
// are explicit), so no split/copy of the QKV tensor is needed.
#include "../common/api.h"
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

struct RopeArgs {
  const bf16* q_in;
  const bf16* k_in;
  long long ldq_in, ldk_in;
  const bf16* qw;
  const bf16* kw;
  const float* cos;  // [P, hd/2]
  const float* sin;
  const void* pos;   // int32 or int64 [T]; nullptr -> token index modulo pos_mod
  int pos_i64;
  int pos_mod;
  bf16* q_out;
  bf16* k_out;
  long long ldq_out, ldk_out;
  float* q_rstd;  // [T, Hq]
  float* k_rstd;  // [T, Hk]
  int T, Hq, Hk;
  float eps, w_off;
  int do_norm;
};

__device__ __forceinline__ int token_pos(const RopeArgs& a, long long tok) {
  if (a.pos == nullptr) return int(tok % a.pos_mod);
  return a.pos_i64 ? int(reinterpret_cast<const long long*>(a.pos)[tok])
                   : reinterpret_cast<const int*>(a.pos)[tok];
}

template <int HD>
__global__ void __launch_bounds__(kRowThreads) qk_rope_fwd_kernel(RopeArgs a) {
  constexpr int LPH = HD / 8;  // lanes per head
  constexpr int UPB = kRowThreads / LPH;
  const int l = threadIdx.x % LPH;
  const int u_in_block = threadIdx.x / LPH;
  const int heads = a.Hq + a.Hk;
  const long long units = 1LL * a.T * heads;
  const int e0 = l * 8;
  const int c0 = e0 % (HD / 2);
  const bool first_half = l < LPH / 2;
  float wq[8], wk[8];
  if (a.do_norm) {
    unpack8(ld16(a.qw + e0), wq);
    unpack8(ld16(a.kw + e0), wk);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      wq[i] += a.w_off;
      wk[i] += a.w_off;
    }
  }
  for (long long u0 = 1LL * blockIdx.x * UPB; u0 < units; u0 += 1LL * gridDim.x * UPB) {
    const long long u = u0 + u_in_block;
    const bool valid = u < units;
    // 32-bit index math: 64-bit division is many times slower and units fit in 32 bits
    const unsigned u32 = unsigned(u);
    const long long tok = valid ? u32 / unsigned(heads) : 0;
    const int h = valid ? int(u32 % unsigned(heads)) : 0;
    const bool is_q = h < a.Hq;
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = 0.f;
    if (valid) {
      const bf16* src = is_q ? a.q_in + tok * a.ldq_in + h * HD + e0
                             : a.k_in + tok * a.ldk_in + (h - a.Hq) * HD + e0;
      unpack8(ld16(src), x);
    }
    if (a.do_norm) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / float(HD) + a.eps);
      if (valid && l == 0) {
        if (is_q) a.q_rstd[tok * a.Hq + h] = rstd;
        else a.k_rstd[tok * a.Hk + (h - a.Hq)] = rstd;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = bf16_round(x[i] * rstd) * (is_q ? wq[i] : wk[i]);
    }
    float p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = __shfl_xor_sync(0xffffffffu, x[i], LPH / 2);
    if (valid) {
      const int pos = token_pos(a, tok);
      const float4* cp = reinterpret_cast<const float4*>(a.cos + 1LL * pos * (HD / 2) + c0);
      const float4* sp = reinterpret_cast<const float4*>(a.sin + 1LL * pos * (HD / 2) + c0);
      float c[8], s[8];
      *reinterpret_cast<float4*>(c) = cp[0];
      *reinterpret_cast<float4*>(c + 4) = cp[1];
      *reinterpret_cast<float4*>(s) = sp[0];
      *reinterpret_cast<float4*>(s + 4) = sp[1];
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = first_half ? x[i] * c[i] - p[i] * s[i] : x[i] * c[i] + p[i] * s[i];
      bf16* dst = is_q ? a.q_out + tok * a.ldq_out + h * HD + e0
                       : a.k_out + tok * a.ldk_out + (h - a.Hq) * HD + e0;
      st16(dst, pack8(y));
    }
  }
}

struct RopeBwdArgs {
  const bf16* dq;   // grads of rotated outputs
  const bf16* dk;
  long long lddq, lddk;
  const bf16* q_in;  // forward inputs (pre-norm)
  const bf16* k_in;
  long long ldq_in, ldk_in;
  const bf16* qw;
  const bf16* kw;
  const float* cos;
  const float* sin;
  const void* pos;
  int pos_i64;
  int pos_mod;
  const float* q_rstd;
  const float* k_rstd;
  bf16* dq_in;  // grads of the forward inputs
  bf16* dk_in;
  long long lddq_in, lddk_in;
  float* dw_partial;  // [grid, 2, HD]
  int T, Hq, Hk;
  float w_off;
  int do_norm;
};

template <int HD>
__global__ void __launch_bounds__(kRowThreads) qk_rope_bwd_kernel(RopeBwdArgs a) {
  constexpr int LPH = HD / 8;
  constexpr int UPB = kRowThreads / LPH;
  __shared__ float sdw[2 * HD];
  const int l = threadIdx.x % LPH;
  const int u_in_block = threadIdx.x / LPH;
  const int heads = a.Hq + a.Hk;
  const long long units = 1LL * a.T * heads;
  const int e0 = l * 8;
  const int c0 = e0 % (HD / 2);
  const bool first_half = l < LPH / 2;
  float wq[8], wk[8], dwq[8], dwk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) dwq[i] = dwk[i] = 0.f;
  if (a.do_norm) {
    unpack8(ld16(a.qw + e0), wq);
    unpack8(ld16(a.kw + e0), wk);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      wq[i] += a.w_off;
      wk[i] += a.w_off;
    }
  }
  for (int i = threadIdx.x; i < 2 * HD; i += kRowThreads) sdw[i] = 0.f;
  RopeArgs pa;  // only the position fields are used by token_pos
  pa.pos = a.pos;
  pa.pos_i64 = a.pos_i64;
  pa.pos_mod = a.pos_mod;

  for (long long u0 = 1LL * blockIdx.x * UPB; u0 < units; u0 += 1LL * gridDim.x * UPB) {
    const long long u = u0 + u_in_block;
    const bool valid = u < units;
    // 32-bit index math: 64-bit division is many times slower and units fit in 32 bits
    const unsigned u32 = unsigned(u);
    const long long tok = valid ? u32 / unsigned(heads) : 0;
    const int h = valid ? int(u32 % unsigned(heads)) : 0;
    const bool is_q = h < a.Hq;
    float g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = 0.f;
    if (valid) {
      const bf16* src = is_q ? a.dq + tok * a.lddq + h * HD + e0
                             : a.dk + tok * a.lddk + (h - a.Hq) * HD + e0;
      unpack8(ld16(src), g);
    }
    float p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = __shfl_xor_sync(0xffffffffu, g[i], LPH / 2);
    float gn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) gn[i] = 0.f;
    if (valid) {
      const int pos = token_pos(pa, tok);
      const float4* cp = reinterpret_cast<const float4*>(a.cos + 1LL * pos * (HD / 2) + c0);
      const float4* sp = reinterpret_cast<const float4*>(a.sin + 1LL * pos * (HD / 2) + c0);
      float c[8], s[8];
      *reinterpret_cast<float4*>(c) = cp[0];
      *reinterpret_cast<float4*>(c + 4) = cp[1];
      *reinterpret_cast<float4*>(s) = sp[0];
      *reinterpret_cast<float4*>(s + 4) = sp[1];
#pragma unroll
      for (int i = 0; i < 8; ++i) gn[i] = first_half ? g[i] * c[i] + p[i] * s[i] : g[i] * c[i] - p[i] * s[i];
    }
    float o[8];
    if (a.do_norm) {
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
      float rstd = 0.f;
      if (valid) {
        const bf16* src = is_q ? a.q_in + tok * a.ldq_in + h * HD + e0
                               : a.k_in + tok * a.ldk_in + (h - a.Hq) * HD + e0;
        unpack8(ld16(src), x);
        rstd = is_q ? a.q_rstd[tok * a.Hq + h] : a.k_rstd[tok * a.Hk + (h - a.Hq)];
      }
      float m[8];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] *= rstd;  // xhat
        m[i] = gn[i] * (is_q ? wq[i] : wk[i]);
        dot += m[i] * x[i];
        const float dwv = gn[i] * bf16_round(x[i]);
        if (is_q) dwq[i] += dwv;
        else dwk[i] += dwv;
      }
#pragma unroll
      for (int s = LPH / 2; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
      dot /= float(HD);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rstd * (m[i] - x[i] * dot);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = gn[i];
    }
    if (valid) {
      bf16* dst = is_q ? a.dq_in + tok * a.lddq_in + h * HD + e0
                       : a.dk_in + tok * a.lddk_in + (h - a.Hq) * HD + e0;
      st16(dst, pack8(o));
    }
  }
  if (a.do_norm && a.dw_partial != nullptr) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      atomicAdd(&sdw[e0 + i], dwq[i]);
      atomicAdd(&sdw[HD + e0 + i], dwk[i]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * HD; i += kRowThreads)
      a.dw_partial[1LL * blockIdx.x * 2 * HD + i] = sdw[i];
  }
}

}  // namespace
}  // namespace lb

using namespace lb;

extern "C" int lb_rope_bwd_partial_rows() { return row_num_sms() * 8; }

extern "C" int lb_qk_norm_rope_fwd(const void* q_in, long long ldq_in, const void* k_in,
                                   long long ldk_in, const void* qw, const void* kw,
                                   const float* cos, const float* sin, const void* pos, int pos_i64,
                                   int pos_mod, void* q_out, long long ldq_out, void* k_out,
                                   long long ldk_out, float* q_rstd, float* k_rstd, int T, int Hq,
                                   int Hk, int hd, float eps, float w_off, int do_norm,
                                   void* stream) {
  if (T <= 0) return 0;
  if ((ldq_in | ldk_in | ldq_out | ldk_out) & 7) return -3;
  if (1LL * T * (Hq + Hk) >= (1LL << 32)) return -3;
  RopeArgs a{(const bf16*)q_in, (const bf16*)k_in, ldq_in, ldk_in, (const bf16*)qw, (const bf16*)kw,
             cos, sin, pos, pos_i64, pos_mod > 0 ? pos_mod : 1, (bf16*)q_out, (bf16*)k_out, ldq_out,
             ldk_out, q_rstd, k_rstd, T, Hq, Hk, eps, w_off, do_norm};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long units = 1LL * T * (Hq + Hk);
  auto grid_for = [&](int lph) {
    const long long upb = kRowThreads / lph;
    long long g = (units + upb - 1) / upb;
    const long long cap = 1LL * row_num_sms() * 16;
    return int(g < cap ? g : cap);
  };
  if (hd == 128) qk_rope_fwd_kernel<128><<<grid_for(16), kRowThreads, 0, st>>>(a);
  else if (hd == 64) qk_rope_fwd_kernel<64><<<grid_for(8), kRowThreads, 0, st>>>(a);
  else if (hd == 256) qk_rope_fwd_kernel<256><<<grid_for(32), kRowThreads, 0, st>>>(a);
  else return -3;
  return launch_rc();
}

// dw_out: [2, hd] (q weight grad then k weight grad); scratch: lb_rope_bwd_partial_rows()*2*hd floats.
extern "C" int lb_qk_norm_rope_bwd(const void* dq, long long lddq, const void* dk, long long lddk,
                                   const void* q_in, long long ldq_in, const void* k_in,
                                   long long ldk_in, const void* qw, const void* kw,
                                   const float* cos, const float* sin, const void* pos, int pos_i64,
                                   int pos_mod, const float* q_rstd, const float* k_rstd,
                                   void* dq_in, long long lddq_in, void* dk_in, long long lddk_in,
                                   float* scratch, void* dw_out, int dw_fp32, int dw_accumulate,
                                   int T, int Hq, int Hk, int hd, float w_off, int do_norm,
                                   void* stream) {
  if (T <= 0) return 0;
  if ((lddq | lddk | ldq_in | ldk_in | lddq_in | lddk_in) & 7) return -3;
  if (1LL * T * (Hq + Hk) >= (1LL << 32)) return -3;
  RopeBwdArgs a{(const bf16*)dq, (const bf16*)dk, lddq, lddk, (const bf16*)q_in, (const bf16*)k_in,
                ldq_in, ldk_in, (const bf16*)qw, (const bf16*)kw, cos, sin, pos, pos_i64,
                pos_mod > 0 ? pos_mod : 1, q_rstd, k_rstd, (bf16*)dq_in, (bf16*)dk_in, lddq_in,
                lddk_in, scratch, T, Hq, Hk, w_off, do_norm};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long units = 1LL * T * (Hq + Hk);
  auto grid_for = [&](int lph) {
    const long long upb = kRowThreads / lph;
    long long g = (units + upb - 1) / upb;
    const long long cap = 1LL * row_num_sms() * 8;
    return int(g < cap ? (g > 0 ? g : 1) : cap);
  };
  int grid;
  if (hd == 128) { grid = grid_for(16); qk_rope_bwd_kernel<128><<<grid, kRowThreads, 0, st>>>(a); }
  else if (hd == 64) { grid = grid_for(8); qk_rope_bwd_kernel<64><<<grid, kRowThreads, 0, st>>>(a); }
  else if (hd == 256) { grid = grid_for(32); qk_rope_bwd_kernel<256><<<grid, kRowThreads, 0, st>>>(a); }
  else return -3;
  if (do_norm && dw_out != nullptr && scratch != nullptr) {
    return lb_colsum(scratch, grid, 2 * hd, dw_out, dw_fp32, dw_accumulate, stream);
  }
  return launch_rc();
}
