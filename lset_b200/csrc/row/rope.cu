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

// A group of HD/8 lanes owns one token at a time and walks over its heads UB at a time: the cos/sin
// row and the position are fetched once per token, and the 16-byte loads of the next UB heads are
// already in flight while the current UB heads are normalised, rotated and stored (the kernel is
// bound by memory latency otherwise).
template <int HD>
__global__ void __launch_bounds__(kRowThreads, 3) qk_rope_fwd_kernel(RopeArgs a) {
  constexpr int LPH = HD / 8;  // lanes per head
  constexpr int TPB = kRowThreads / LPH;
  constexpr int UB = 4;
  __shared__ float swt[2 * HD];  // q then k norm weights (+ offset)
  const int l = threadIdx.x % LPH;
  const int g = threadIdx.x / LPH;
  const int heads = a.Hq + a.Hk;
  const int e0 = l * 8;
  const int c0 = e0 % (HD / 2);
  const bool first_half = l < LPH / 2;
  for (int i = threadIdx.x; i < 2 * HD; i += kRowThreads)
    swt[i] = a.do_norm ? __bfloat162float(i < HD ? a.qw[i] : a.kw[i - HD]) + a.w_off : 1.f;
  __syncthreads();
  for (int tok0 = blockIdx.x * TPB; tok0 < a.T; tok0 += gridDim.x * TPB) {
    const long long tok = tok0 + g;
    const bool valid = tok < a.T;
    const bf16* qrow = a.q_in + tok * a.ldq_in + e0;
    const bf16* krow = a.k_in + tok * a.ldk_in + e0;
    bf16* qdst = a.q_out + tok * a.ldq_out + e0;
    bf16* kdst = a.k_out + tok * a.ldk_out + e0;
    auto load_batch = [&](int h0, uint4 (&raw)[UB]) {
#pragma unroll
      for (int j = 0; j < UB; ++j) {
        const int h = h0 + j;
        raw[j] = make_uint4(0u, 0u, 0u, 0u);
        if (valid && h < heads) raw[j] = ld16(h < a.Hq ? qrow + h * HD : krow + (h - a.Hq) * HD);
      }
    };
    uint4 cur[UB], nxt[UB];
    load_batch(0, cur);
    float c[8], s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = s[i] = 0.f;
    if (valid) {
      const int pos = token_pos(a, tok);
      const float4* cp = reinterpret_cast<const float4*>(a.cos + 1LL * pos * (HD / 2) + c0);
      const float4* sp = reinterpret_cast<const float4*>(a.sin + 1LL * pos * (HD / 2) + c0);
      *reinterpret_cast<float4*>(c) = cp[0];
      *reinterpret_cast<float4*>(c + 4) = cp[1];
      *reinterpret_cast<float4*>(s) = sp[0];
      *reinterpret_cast<float4*>(s + 4) = sp[1];
    }
    if (!first_half) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] = -s[i];  // y = x*c - partner*s (first half), + (second)
    }
    for (int h0 = 0; h0 < heads; h0 += UB) {
      if (h0 + UB < heads) load_batch(h0 + UB, nxt);
#pragma unroll
      for (int j = 0; j < UB; ++j) {
        const int h = h0 + j;
        if (h >= heads) break;  // uniform over the CTA
        const bool is_q = h < a.Hq;
        float x[8];
        unpack8(cur[j], x);
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
          const float* wt = swt + (is_q ? 0 : HD) + e0;
          const float4 w0 = *reinterpret_cast<const float4*>(wt);
          const float4 w1 = *reinterpret_cast<const float4*>(wt + 4);
          const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = bf16_round(x[i] * rstd) * wl[i];
        }
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float p = __shfl_xor_sync(0xffffffffu, x[i], LPH / 2);
          y[i] = x[i] * c[i] - p * s[i];
        }
        if (valid) st16(is_q ? qdst + h * HD : kdst + (h - a.Hq) * HD, pack8(y));
      }
#pragma unroll
      for (int j = 0; j < UB; ++j) cur[j] = nxt[j];
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

// Same token-per-lane-group walk as the forward kernel, UB heads at a time: the gradient rows, the
// forward inputs and the saved rstd of UB heads are requested before any of them is used.
template <int HD>
__global__ void __launch_bounds__(kRowThreads, 2) qk_rope_bwd_kernel(RopeBwdArgs a) {
  constexpr int LPH = HD / 8;
  constexpr int TPB = kRowThreads / LPH;
  constexpr int UB = 4;
  __shared__ float sdw[2 * HD];
  __shared__ float swt[2 * HD];  // q then k norm weights (+ offset)
  const int l = threadIdx.x % LPH;
  const int g = threadIdx.x / LPH;
  const int heads = a.Hq + a.Hk;
  const int e0 = l * 8;
  const int c0 = e0 % (HD / 2);
  const bool first_half = l < LPH / 2;
  float dwq[8], dwk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) dwq[i] = dwk[i] = 0.f;
  for (int i = threadIdx.x; i < 2 * HD; i += kRowThreads) {
    sdw[i] = 0.f;
    swt[i] = a.do_norm ? __bfloat162float(i < HD ? a.qw[i] : a.kw[i - HD]) + a.w_off : 1.f;
  }
  __syncthreads();
  RopeArgs pa;  // only the position fields are used by token_pos
  pa.pos = a.pos;
  pa.pos_i64 = a.pos_i64;
  pa.pos_mod = a.pos_mod;

  for (int tok0 = blockIdx.x * TPB; tok0 < a.T; tok0 += gridDim.x * TPB) {
    const long long tok = tok0 + g;
    const bool valid = tok < a.T;
    float c[8], s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = s[i] = 0.f;
    if (valid) {
      const int pos = token_pos(pa, tok);
      const float4* cp = reinterpret_cast<const float4*>(a.cos + 1LL * pos * (HD / 2) + c0);
      const float4* sp = reinterpret_cast<const float4*>(a.sin + 1LL * pos * (HD / 2) + c0);
      *reinterpret_cast<float4*>(c) = cp[0];
      *reinterpret_cast<float4*>(c + 4) = cp[1];
      *reinterpret_cast<float4*>(s) = sp[0];
      *reinterpret_cast<float4*>(s + 4) = sp[1];
    }
    if (!first_half) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] = -s[i];  // gn = g*c + partner*s (first half), - (second)
    }
    const bf16* gq = a.dq + tok * a.lddq + e0;
    const bf16* gk = a.dk + tok * a.lddk + e0;
    const bf16* xq = a.q_in + tok * a.ldq_in + e0;
    const bf16* xk = a.k_in + tok * a.ldk_in + e0;
    bf16* oq = a.dq_in + tok * a.lddq_in + e0;
    bf16* ok = a.dk_in + tok * a.lddk_in + e0;
    for (int h0 = 0; h0 < heads; h0 += UB) {
      uint4 graw[UB], xraw[UB];
      float rs[UB];
#pragma unroll
      for (int j = 0; j < UB; ++j) {
        const int h = h0 + j;
        graw[j] = xraw[j] = make_uint4(0u, 0u, 0u, 0u);
        rs[j] = 0.f;
        if (valid && h < heads) {
          const bool is_q = h < a.Hq;
          graw[j] = ld16(is_q ? gq + h * HD : gk + (h - a.Hq) * HD);
          if (a.do_norm) {
            xraw[j] = ld16(is_q ? xq + h * HD : xk + (h - a.Hq) * HD);
            rs[j] = is_q ? a.q_rstd[tok * a.Hq + h] : a.k_rstd[tok * a.Hk + (h - a.Hq)];
          }
        }
      }
#pragma unroll
      for (int j = 0; j < UB; ++j) {
        const int h = h0 + j;
        if (h >= heads) break;  // uniform over the CTA
        const bool is_q = h < a.Hq;
        float gv[8], gn[8], o[8];
        unpack8(graw[j], gv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float p = __shfl_xor_sync(0xffffffffu, gv[i], LPH / 2);
          gn[i] = gv[i] * c[i] + p * s[i];
        }
        if (a.do_norm) {
          float x[8], m[8];
          unpack8(xraw[j], x);
          const float rstd = rs[j];
          const float* wt = swt + (is_q ? 0 : HD) + e0;
          const float4 w0 = *reinterpret_cast<const float4*>(wt);
          const float4 w1 = *reinterpret_cast<const float4*>(wt + 4);
          const float wl[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          float dot = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            x[i] *= rstd;  // xhat
            m[i] = gn[i] * wl[i];
            dot += m[i] * x[i];
            const float dwv = gn[i] * bf16_round(x[i]);
            if (is_q) dwq[i] += dwv;
            else dwk[i] += dwv;
          }
#pragma unroll
          for (int sh = LPH / 2; sh > 0; sh >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sh);
          dot /= float(HD);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = rstd * (m[i] - x[i] * dot);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = gn[i];
        }
        if (valid) st16(is_q ? oq + h * HD : ok + (h - a.Hq) * HD, pack8(o));
      }
    }
  }
  if (a.do_norm && a.dw_partial != nullptr) {
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
  auto grid_for = [&](int lph) {
    const long long tpb = kRowThreads / lph;
    long long g = (T + tpb - 1) / tpb;
    const long long cap = 1LL * row_num_sms() * 6;  // two waves at three CTAs per SM
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
  auto grid_for = [&](int lph) {
    const long long tpb = kRowThreads / lph;
    long long g = (T + tpb - 1) / tpb;
    const long long cap = 1LL * row_num_sms() * 4;
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
