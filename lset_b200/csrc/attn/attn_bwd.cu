// Varlen flash attention backward on tcgen05, without atomics: three launches.
//
//   delta     delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]
//   dQ        one 256-thread CTA per (sequence, query tile, KV head), two CTAs per SM, walking KV
//             blocks of 64:
//               S = Q·Kᵀ, dP = dO·Vᵀ (TMEM) -> dS = P∘(dP − delta)·scale (bf16, written over the V
//               block in smem) -> dQ += dS·K
//   dK/dV     one 256-thread CTA per (sequence, 128-row KV tile, KV head), walking (query block,
//             head) pairs through a 3-deep TMA ring, with Sᵀ/dPᵀ double-buffered in TMEM so the
//             score products of step i+1 run while step i is in the softmax-gradient math:
//               Sᵀ = K·Qᵀ, dPᵀ = V·dOᵀ (TMEM) -> Pᵀ, dSᵀ (bf16, smem) -> dV += Pᵀ·dO, dK += dSᵀ·Q
// Thread t owns accumulator row t % 128 and a half (dQ kernel, 256 threads) or a quarter (dK/dV
// kernel, 512 threads) of the 64 columns of a score block.
// The Q / dO / K / V tiles are loaded once by TMA and serve both as K-major operands (contraction
// over head_dim) and as MN-major operands (contraction over tokens); nothing is transposed in
// memory. Probabilities are recomputed from the forward's LSE.
//
// Counterpart of the flash_attn / varlen_attn backward used by the reference through autograd
// (lset/models/decoder/qwen3/attention.py:203-234).
#include "../common/api.h"
#include "../common/ptx.cuh"
#include "../common/row.cuh"
#include "../common/tma_desc.h"
#include "attn_common.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

// ------------------------------------------------------------------------------------ delta
template <int HD>
__global__ void __launch_bounds__(256)
    attn_delta_kernel(const bf16* __restrict__ dO, long long lddo, const bf16* __restrict__ O,
                      long long ldo, float* __restrict__ delta, int T, int Hq) {
  constexpr int LPH = HD / 8;
  constexpr int UPB = 256 / LPH;
  const int l = threadIdx.x % LPH;
  const long long units = 1LL * T * Hq;
  for (long long u0 = 1LL * blockIdx.x * UPB; u0 < units; u0 += 1LL * gridDim.x * UPB) {
    const long long u = u0 + threadIdx.x / LPH;
    float s = 0.f;
    long long tok = 0;
    int h = 0;
    if (u < units) {
      tok = u / Hq;
      h = int(u % Hq);
      float a[8], b[8];
      unpack8(ld16(dO + tok * lddo + h * HD + l * 8), a);
      unpack8(ld16(O + tok * ldo + h * HD + l * 8), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += a[i] * b[i];
    }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (u < units && l == 0) delta[1LL * h * T + tok] = s;
  }
}

struct AttnBwdArgs {
  const int* seq_start;  // first token of each sequence
  const int* seq_end;    // one past its last token
  const int* plan;
  const float* lse;    // [Hq, T]
  const float* delta;  // [Hq, T]
  bf16* dQ;
  long long lddq;
  bf16* dK;
  long long lddk;
  bf16* dV;
  long long lddv;
  int T, Hq, Hk;
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  int causal;
  int* status;
};

__device__ __forceinline__ void ld_row32(uint32_t taddr, float (&s)[32]) {
  uint32_t t0[32];
  tmem_ld_32x32b_x32(taddr, t0);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 32; ++c) s[c] = __uint_as_float(t0[c]);
}

// Write 32 values of one row into columns [32*half, 32*half+32) of a 128-row x 64-column bf16 tile
// stored K-major with the 128-byte swizzle.
__device__ __forceinline__ void st_half_row_bf16_swz(uint8_t* tile, int row, int half,
                                                     const float (&v)[32]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = pack_bf16x2(v[c * 8 + 0], v[c * 8 + 1]);
    q.y = pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
    q.z = pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
    q.w = pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + swz128_offset(row, half * 4 + c)) = q;
  }
}

// 16-column variants for kernels whose threads own a quarter of a 64-column block.
__device__ __forceinline__ void ld_row16(uint32_t taddr, float (&s)[16]) {
  uint32_t t0[16];
  tmem_ld_32x32b_x16(taddr, t0);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 16; ++c) s[c] = __uint_as_float(t0[c]);
}

// Write 16 values of one row into columns [16*quarter, 16*quarter+16) of a 128-row x 64-column
// bf16 tile stored K-major with the 128-byte swizzle.
__device__ __forceinline__ void st_quarter_row_bf16_swz(uint8_t* tile, int row, int quarter,
                                                        const float (&v)[16]) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint4 q;
    q.x = pack_bf16x2(v[c * 8 + 0], v[c * 8 + 1]);
    q.y = pack_bf16x2(v[c * 8 + 2], v[c * 8 + 3]);
    q.z = pack_bf16x2(v[c * 8 + 4], v[c * 8 + 5]);
    q.w = pack_bf16x2(v[c * 8 + 6], v[c * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + swz128_offset(row, quarter * 2 + c)) = q;
  }
}

// Store NCOLS (a multiple of 16) accumulator columns of one row as bf16 to dst when `pred`.
template <int NCOLS>
__device__ __forceinline__ void store_acc_cols16(uint32_t taddr, bf16* dst, bool pred) {
#pragma unroll 1
  for (int c = 0; c < NCOLS / 16; ++c) {
    uint32_t o[16];
    tmem_ld_32x32b_x16(taddr + c * 16, o);
    tmem_ld_wait();
    if (pred) {
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        uint4 q;
        q.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1]));
        q.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3]));
        q.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5]));
        q.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7]));
        *reinterpret_cast<uint4*>(dst + c * 16 + v * 8) = q;
      }
    }
  }
}

// Store NCOLS accumulator columns (fp32, starting at taddr) of one row as bf16 to dst when `pred`.
template <int NCOLS>
__device__ __forceinline__ void store_acc_cols(uint32_t taddr, bf16* dst, bool pred) {
#pragma unroll 1
  for (int c = 0; c < NCOLS / 32; ++c) {
    uint32_t o[32];
    tmem_ld_32x32b_x32(taddr + c * 32, o);
    tmem_ld_wait();
    if (pred) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 q;
        q.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1]));
        q.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3]));
        q.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5]));
        q.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7]));
        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = q;
      }
    }
  }
}

// Store one accumulator row (HD fp32 columns starting at taddr) as bf16 to dst when `pred`.
template <int HD>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, bf16* dst, bool pred) {
#pragma unroll 1
  for (int c = 0; c < HD / 32; ++c) {
    uint32_t o[32];
    tmem_ld_32x32b_x32(taddr + c * 32, o);
    tmem_ld_wait();
    if (pred) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        uint4 q;
        q.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]), __uint_as_float(o[8 * v + 1]));
        q.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3]));
        q.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5]));
        q.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7]));
        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = q;
      }
    }
  }
}

// ------------------------------------------------------------------------------------ dQ
constexpr int kBwdThreads = 256;

template <int HD>
struct DqCfg {
  static constexpr int PANELS = HD / 64;
  static constexpr int Q_BYTES = 128 * HD * 2;
  static constexpr int KV_BYTES = kAttnKvBlock * HD * 2;
  static constexpr int DS_BYTES = 128 * kAttnKvBlock * 2;
  // dS is written over the V block (V is dead once dP = dO·Vᵀ has completed) when it fits.
  static constexpr bool DS_IN_V = KV_BYTES >= DS_BYTES;
  static constexpr int SMEM_BYTES = 2 * Q_BYTES + 2 * KV_BYTES + (DS_IN_V ? 0 : DS_BYTES) + 1024 + 128;
  static constexpr int DQ_COL = 128;
  static constexpr int TMEM_COLS = (128 + HD) <= 256 ? 256 : 512;
};

template <int HD>
__global__ void __launch_bounds__(kBwdThreads)
    attn_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   AttnBwdArgs a) {
  using C = DqCfg<HD>;
  AttnPlanView plan{a.plan};
  if (int(blockIdx.x) >= plan.count()) return;
  const int b = plan.seq(blockIdx.x);
  const int qt = plan.tile(blockIdx.x);
  const int hk = blockIdx.y;
  const int G = a.Hq / a.Hk;
  const int QT = 128 / G;
  const int seq0 = a.seq_start[b];
  const int len = a.seq_end[b] - seq0;
  const int q0 = qt * QT;
  const int kv_end = a.causal ? min(len, q0 + QT) : len;
  const int nblk = (kv_end + kAttnKvBlock - 1) / kAttnKvBlock;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::Q_BYTES;
  uint8_t* sK = sdO + C::Q_BYTES;
  uint8_t* sV = sK + C::KV_BYTES;
  uint8_t* sdS = C::DS_IN_V ? sV : (sV + C::KV_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + C::KV_BYTES + (C::DS_IN_V ? 0 : C::DS_BYTES));
  uint64_t* bar_q = bars;
  uint64_t* bar_kv = bars + 1;
  uint64_t* bar_s = bars + 2;
  uint64_t* bar_dq = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int half = warp >> 2;  // which 32 of the 64 KV columns this thread handles
  auto load_kv = [&](int j) {
    mbar_expect_tx(bar_kv, 2 * C::KV_BYTES);
#pragma unroll
    for (int p = 0; p < C::PANELS; ++p) {
      tma_load_2d(sK + p * (kAttnKvBlock * 128), &tmK, bar_kv, hk * HD + p * 64,
                  seq0 + j * kAttnKvBlock);
      tma_load_2d(sV + p * (kAttnKvBlock * 128), &tmV, bar_kv, hk * HD + p * 64,
                  seq0 + j * kAttnKvBlock);
    }
  };
  // first loads before the TMEM allocation and the CTA barrier: their latency runs under the set-up
  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_dq, 1);
    mbar_fence_init();
    mbar_expect_tx(bar_q, 2 * C::Q_BYTES);
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int p = 0; p < C::PANELS; ++p) {
        tma_load_2d(sQ + p * (128 * 128) + g * QT * 128, &tmQ, bar_q, (hk * G + g) * HD + p * 64,
                    seq0 + q0);
        tma_load_2d(sdO + p * (128 * 128) + g * QT * 128, &tmdO, bar_q, (hk * G + g) * HD + p * 64,
                    seq0 + q0);
      }
    load_kv(0);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (uint32_t((warp & 3) * 32) << 16);

  const int r = tid & 127;
  const int g = r / QT;
  const int qpos = q0 + r % QT;
  const bool row_valid = qpos < len;
  const long long tok = 1LL * seq0 + qpos;
  const int head = hk * G + g;
  const float lse2 = row_valid ? a.lse[1LL * head * a.T + tok] * kLog2eF : 0.f;
  const float dlt = row_valid ? a.delta[1LL * head * a.T + tok] : 0.f;
  constexpr uint32_t idesc_s = umma_idesc_bf16(128, kAttnKvBlock, 0, 0);
  constexpr uint32_t idesc_dq = umma_idesc_bf16(128, HD, 0, 1);
  bool failed = false;
  {
    const bool ok = mbar_wait(bar_q, 0);
    if (__syncthreads_or(!ok)) {
      report_status(a.status, kStatusTimeoutProducer);
      failed = true;
    }
  }
  // One CTA-wide barrier per KV block (before the dQ product is issued). Thread 0 alone waits for
  // the loads and for the dQ product that frees the K / V slot; every thread waits for the score
  // products itself; whether a wait ran out anywhere is agreed on at the barrier.
  for (int j = 0; j < nblk && !failed; ++j) {
    bool ok = true;
    if (tid == 0) {
      ok = mbar_wait(bar_kv, j & 1);
      if (ok) {
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), da = smem_u32(sdO);
        const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t aoff = (ks / 4) * (128 * 128) + (ks % 4) * 32;
          const uint32_t boff = (ks / 4) * (kAttnKvBlock * 128) + (ks % 4) * 32;
          umma_bf16(tmem_base, umma_smem_desc(qa + aoff, 16, 1024),
                    umma_smem_desc(ka + boff, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t aoff = (ks / 4) * (128 * 128) + (ks % 4) * 32;
          const uint32_t boff = (ks / 4) * (kAttnKvBlock * 128) + (ks % 4) * 32;
          umma_bf16(tmem_base + 64, umma_smem_desc(da + aoff, 16, 1024),
                    umma_smem_desc(va + boff, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_s);
      }
    }
    ok = ok && mbar_wait(bar_s, j & 1);
    tc_fence_after();
    float ds[32];
    {
      float s[32];
      ld_row32(tmem_row + half * 32, s);
      ld_row32(tmem_row + 64 + half * 32, ds);
      const int kv0 = j * kAttnKvBlock + half * 32;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int kvpos = kv0 + c;
        const bool valid = row_valid && kvpos < len && (!a.causal || kvpos <= qpos);
        const float p = valid ? exp2f(s[c] * a.scale_log2 - lse2) : 0.f;
        ds[c] = p * (ds[c] - dlt) * a.scale;
      }
    }
    // S and dP are complete (bar_s), so the V block may be overwritten by dS
    st_half_row_bf16_swz(sdS, r, half, ds);
    fence_proxy_async_smem();
    tc_fence_before();
    if (__syncthreads_or(!ok)) {
      report_status(a.status, kStatusTimeoutMma);
      failed = true;
      break;
    }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t sa = smem_u32(sdS);
      const uint32_t ka = smem_u32(sK);
#pragma unroll
      for (int ks = 0; ks < kAttnKvBlock / 16; ++ks)
        umma_bf16(tmem_base + C::DQ_COL, umma_smem_desc(sa + ks * 32, 16, 1024),
                  umma_smem_desc(ka + ks * 2048, kAttnKvBlock * 128, 1024), idesc_dq,
                  (j > 0 || ks > 0) ? 1u : 0u);
      umma_commit(bar_dq);
      // the K block and the dS / V slot are in use until this block's dQ product is done; a wait
      // that runs out here leaves the next block unloaded, and its wait then fails for everybody
      if (j + 1 < nblk) {
        if (mbar_wait(bar_dq, j & 1))
          load_kv(j + 1);
        else
          report_status(a.status, kStatusTimeoutMma);
      }
    }
  }
  if (!failed) {
    const bool ok = mbar_wait(bar_dq, (nblk - 1) & 1);
    if (__syncthreads_or(!ok)) {
      report_status(a.status, kStatusTimeoutMma);
      failed = true;
    }
  }
  if (!failed) {
    tc_fence_after();
    store_acc_cols<HD / 2>(tmem_row + C::DQ_COL + half * (HD / 2),
                           a.dQ + tok * a.lddq + head * HD + half * (HD / 2), row_valid);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ------------------------------------------------------------------------------------ dK / dV
template <int HD>
struct DkvCfg {
  static constexpr int PANELS = HD / 64;
  static constexpr int KV_BYTES = 128 * HD * 2;  // resident K tile and V tile
  static constexpr int QB_BYTES = 64 * HD * 2;   // one query block of Q or dO
  static constexpr int QBUFS = 3;                // TMA ring depth for (Q, dO) blocks
  static constexpr int PT_BYTES = 128 * 64 * 2;
  static constexpr int SMEM_BYTES =
      2 * KV_BYTES + 2 * QBUFS * QB_BYTES + 2 * PT_BYTES + 1024 /*stats*/ + 1024 /*align*/ + 128;
  // TMEM: two (Sᵀ, dPᵀ) buffers of 64 + 64 columns, then the dV and dK accumulators.
  static constexpr int DV_COL = 256;
  static constexpr int DK_COL = 256 + HD;
  static constexpr int TMEM_COLS = 512;
  static_assert(256 + 2 * HD <= 512, "head_dim too large for the dK/dV accumulators");
};

// 512 threads: thread t owns accumulator row t % 128 and a quarter (t / 128) of the 64 columns of
// a score block. With 256 threads (two warps per scheduler) the softmax-gradient math of a step
// was bound by instruction latency, not by the tensor pipe.
constexpr int kDkvThreads = 512;

template <int HD>
__global__ void __launch_bounds__(kDkvThreads)
    attn_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    AttnBwdArgs a) {
  using C = DkvCfg<HD>;
  AttnPlanView plan{a.plan};
  if (int(blockIdx.x) >= plan.count()) return;
  const int b = plan.seq(blockIdx.x);
  const int kt = plan.tile(blockIdx.x);
  const int hk = blockIdx.y;
  const int G = a.Hq / a.Hk;
  const int seq0 = a.seq_start[b];
  const int len = a.seq_end[b] - seq0;
  const int kv0 = kt * 128;
  const int nqb = (len + 63) / 64;
  const int qb_start = a.causal ? (kv0 / 64) : 0;
  const int n_inner = (nqb - qb_start) * G;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::KV_BYTES;
  uint8_t* sQ = sV + C::KV_BYTES;               // [QBUFS]
  uint8_t* sdO = sQ + C::QBUFS * C::QB_BYTES;   // [QBUFS]
  uint8_t* sPT = sdO + C::QBUFS * C::QB_BYTES;
  uint8_t* sdST = sPT + C::PT_BYTES;
  float* sStat = reinterpret_cast<float*>(sdST + C::PT_BYTES);  // [2 bufs][2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 256);
  uint64_t* bar_kv = bars;
  uint64_t* bar_q = bars + 1;    // [QBUFS]
  uint64_t* bar_s = bars + 4;    // [2]
  uint64_t* bar_acc = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int quarter = warp >> 2;  // which 16 of the 64 score columns this thread handles
  constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
  constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, 0, 1);

  auto load_q = [&](int i) {
    const int buf = i % C::QBUFS;
    const int qb = qb_start + i / G;
    const int head = hk * G + i % G;
    mbar_expect_tx(&bar_q[buf], 2 * C::QB_BYTES);
#pragma unroll
    for (int p = 0; p < C::PANELS; ++p) {
      tma_load_2d(sQ + buf * C::QB_BYTES + p * (64 * 128), &tmQ, &bar_q[buf], head * HD + p * 64,
                  seq0 + qb * 64);
      tma_load_2d(sdO + buf * C::QB_BYTES + p * (64 * 128), &tmdO, &bar_q[buf], head * HD + p * 64,
                  seq0 + qb * 64);
    }
  };
  // Barriers, then the K / V tile and the first two (Q, dO) blocks are requested before the TMEM
  // allocation and the CTA barrier, so the load latency runs under that set-up.
  if (tid == 0) {
    mbar_init(bar_kv, 1);
    for (int i = 0; i < C::QBUFS; ++i) mbar_init(&bar_q[i], 1);
    mbar_init(&bar_s[0], 1);
    mbar_init(&bar_s[1], 1);
    mbar_init(bar_acc, 1);
    mbar_fence_init();
    mbar_expect_tx(bar_kv, 2 * C::KV_BYTES);
#pragma unroll
    for (int p = 0; p < C::PANELS; ++p) {
      tma_load_2d(sK + p * (128 * 128), &tmK, bar_kv, hk * HD + p * 64, seq0 + kv0);
      tma_load_2d(sV + p * (128 * 128), &tmV, bar_kv, hk * HD + p * 64, seq0 + kv0);
    }
    if (n_inner > 0) load_q(0);
    if (n_inner > 1) load_q(1);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (uint32_t((warp & 3) * 32) << 16);

  // Sᵀ = K·Qᵀ and dPᵀ = V·dOᵀ of inner step i into TMEM buffer i & 1 (issued by thread 0).
  auto issue_scores = [&](int i) -> bool {
    const int buf = i % C::QBUFS;
    if (!mbar_wait(&bar_q[buf], (i / C::QBUFS) & 1)) {
      report_status(a.status, kStatusTimeoutProducer);
      return false;
    }
    tc_fence_after();
    const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
    const uint32_t qa = smem_u32(sQ + buf * C::QB_BYTES);
    const uint32_t da = smem_u32(sdO + buf * C::QB_BYTES);
    const uint32_t dcol = tmem_base + (i & 1) * 128;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const uint32_t aoff = (ks / 4) * (128 * 128) + (ks % 4) * 32;
      const uint32_t boff = (ks / 4) * (64 * 128) + (ks % 4) * 32;
      umma_bf16(dcol, umma_smem_desc(ka + aoff, 16, 1024), umma_smem_desc(qa + boff, 16, 1024),
                idesc_s, ks > 0 ? 1u : 0u);
    }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const uint32_t aoff = (ks / 4) * (128 * 128) + (ks % 4) * 32;
      const uint32_t boff = (ks / 4) * (64 * 128) + (ks % 4) * 32;
      umma_bf16(dcol + 64, umma_smem_desc(va + aoff, 16, 1024), umma_smem_desc(da + boff, 16, 1024),
                idesc_s, ks > 0 ? 1u : 0u);
    }
    umma_commit(&bar_s[i & 1]);
    return true;
  };

  const int r = tid & 127;
  const int kvpos = kv0 + r;
  const bool row_valid = kvpos < len;
  bool failed = false;
  // lse / delta of a block's 64 queries (read by every row), staged one step ahead
  auto stage_stats = [&](int i) {
    if (tid < 64) {
      const int qp = (qb_start + i / G) * 64 + tid;
      const int head = hk * G + i % G;
      const bool v = qp < len;
      sStat[(i & 1) * 128 + tid] = v ? a.lse[1LL * head * a.T + seq0 + qp] * kLog2eF : 0.f;
      sStat[(i & 1) * 128 + 64 + tid] = v ? a.delta[1LL * head * a.T + seq0 + qp] : 0.f;
    }
  };
  if (n_inner > 0) stage_stats(0);
  {
    const bool ok = mbar_wait(bar_kv, 0);
    if (__syncthreads_or(!ok)) {
      report_status(a.status, kStatusTimeoutProducer);
      failed = true;
    }
  }
  if (!failed && tid == 0 && n_inner > 0) issue_scores(0);

  // One CTA-wide barrier per step (before the accumulation products are issued). Every thread
  // waits on the mbarriers itself; whether a wait ran out anywhere is agreed on at that barrier.
  for (int i = 0; i < n_inner && !failed; ++i) {
    const int sb = i & 1;
    const int qbuf = i % C::QBUFS;
    const int qb = qb_start + i / G;
    bool ok = mbar_wait(&bar_s[sb], (i >> 1) & 1);
    tc_fence_after();
    // The score products of the next step go to the tensor pipe now: their TMEM buffer was last
    // read by step i - 1 (complete in every thread before that step's barrier), and they then run
    // under this step's softmax-gradient math instead of behind this step's accumulation products.
    if (tid == 0 && ok && i + 1 < n_inner) ok = issue_scores(i + 1);
    if (i + 1 < n_inner) stage_stats(i + 1);
    float pt[16], dst[16];
    ld_row16(tmem_row + sb * 128 + quarter * 16, pt);
    ld_row16(tmem_row + sb * 128 + 64 + quarter * 16, dst);
    {
      const float* lse2 = sStat + sb * 128 + quarter * 16;
      const float* dl = lse2 + 64;
      const int qbase = qb * 64 + quarter * 16;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const int qp = qbase + c;
        const bool valid = row_valid && qp < len && (!a.causal || kvpos <= qp);
        const float p = valid ? exp2f(pt[c] * a.scale_log2 - lse2[c]) : 0.f;
        pt[c] = p;
        dst[c] = p * (dst[c] - dl[c]) * a.scale;
      }
    }
    if (i > 0) {
      // previous dV/dK products done: the Pᵀ/dSᵀ tiles and ring slot (i-1) % 3 are free
      ok = mbar_wait(bar_acc, (i - 1) & 1) && ok;
      tc_fence_after();
    }
    if (tid == 0 && ok && i + 2 < n_inner) load_q(i + 2);
    st_quarter_row_bf16_swz(sPT, r, quarter, pt);
    st_quarter_row_bf16_swz(sdST, r, quarter, dst);
    fence_proxy_async_smem();
    tc_fence_before();
    if (__syncthreads_or(!ok)) {
      report_status(a.status, kStatusTimeoutMma);
      failed = true;
      break;
    }
    if (tid == 0) {
      tc_fence_after();
      const uint32_t pa = smem_u32(sPT), sa = smem_u32(sdST);
      const uint32_t qa = smem_u32(sQ + qbuf * C::QB_BYTES);
      const uint32_t da = smem_u32(sdO + qbuf * C::QB_BYTES);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(tmem_base + C::DV_COL, umma_smem_desc(pa + ks * 32, 16, 1024),
                  umma_smem_desc(da + ks * 2048, 64 * 128, 1024), idesc_acc,
                  (i > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_bf16(tmem_base + C::DK_COL, umma_smem_desc(sa + ks * 32, 16, 1024),
                  umma_smem_desc(qa + ks * 2048, 64 * 128, 1024), idesc_acc,
                  (i > 0 || ks > 0) ? 1u : 0u);
      umma_commit(bar_acc);
    }
  }
  if (!failed && n_inner > 0) {
    const bool ok = mbar_wait(bar_acc, (n_inner - 1) & 1);
    if (__syncthreads_or(!ok)) {
      report_status(a.status, kStatusTimeoutMma);
      failed = true;
    }
  }
  if (!failed && n_inner > 0) {
    tc_fence_after();
    const long long tok = 1LL * seq0 + kvpos;
    store_acc_cols16<HD / 4>(tmem_row + C::DV_COL + quarter * (HD / 4),
                             a.dV + tok * a.lddv + hk * HD + quarter * (HD / 4), row_valid);
    store_acc_cols16<HD / 4>(tmem_row + C::DK_COL + quarter * (HD / 4),
                             a.dK + tok * a.lddk + hk * HD + quarter * (HD / 4), row_valid);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int HD>
int launch_bwd(const void* dO, long long lddo, const void* q, long long ldq, const void* k,
               long long ldk, const void* v, long long ldv, const void* o, long long ldo,
               float* delta, const int* plan_q, int cap_q, const int* plan_kv, int cap_kv,
               AttnBwdArgs a, cudaStream_t st) {
  const int G = a.Hq / a.Hk;
  const int QT = 128 / G;
  {
    constexpr int UPB = 256 / (HD / 8);
    long long grid = (1LL * a.T * a.Hq + UPB - 1) / UPB;
    const long long cap = 1LL * row_num_sms() * 16;
    if (grid > cap) grid = cap;
    attn_delta_kernel<HD><<<int(grid), 256, 0, st>>>((const bf16*)dO, lddo, (const bf16*)o, ldo,
                                                     delta, a.T, a.Hq);
  }
  CUtensorMap tmQ, tmdO, tmK, tmV;
  int rc;
  // dQ kernel: Q / dO tiles of QT tokens per head, K / V blocks of 64.
  if ((rc = make_tmap_2d(&tmQ, q, 2, (uint64_t)a.Hq * HD, a.T, (uint64_t)ldq * 2, 64, QT, true))) return rc;
  if ((rc = make_tmap_2d(&tmdO, dO, 2, (uint64_t)a.Hq * HD, a.T, (uint64_t)lddo * 2, 64, QT, true))) return rc;
  if ((rc = make_tmap_2d(&tmK, k, 2, (uint64_t)a.Hk * HD, a.T, (uint64_t)ldk * 2, 64, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmV, v, 2, (uint64_t)a.Hk * HD, a.T, (uint64_t)ldv * 2, 64, 64, true))) return rc;
  {
    using C = DqCfg<HD>;
    auto kern = attn_dq_kernel<HD>;
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
          cudaSuccess)
        return -10;
      configured = true;
    }
    a.plan = plan_q;
    kern<<<dim3(cap_q, a.Hk), kBwdThreads, C::SMEM_BYTES, st>>>(tmQ, tmdO, tmK, tmV, a);
  }
  // dK/dV kernel: resident K / V tiles of 128 rows, Q / dO blocks of 64 tokens.
  if ((rc = make_tmap_2d(&tmQ, q, 2, (uint64_t)a.Hq * HD, a.T, (uint64_t)ldq * 2, 64, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdO, dO, 2, (uint64_t)a.Hq * HD, a.T, (uint64_t)lddo * 2, 64, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmK, k, 2, (uint64_t)a.Hk * HD, a.T, (uint64_t)ldk * 2, 64, 128, true))) return rc;
  if ((rc = make_tmap_2d(&tmV, v, 2, (uint64_t)a.Hk * HD, a.T, (uint64_t)ldv * 2, 64, 128, true))) return rc;
  {
    using C = DkvCfg<HD>;
    auto kern = attn_dkv_kernel<HD>;
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
          cudaSuccess)
        return -10;
      configured = true;
    }
    a.plan = plan_kv;
    kern<<<dim3(cap_kv, a.Hk), kDkvThreads, C::SMEM_BYTES, st>>>(tmQ, tmdO, tmK, tmV, a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace
}  // namespace lb

using namespace lb;

// plan_q: tiles of 128 / (Hq/Hk) tokens; plan_kv: tiles of 128 tokens. delta: [Hq, T] scratch.
extern "C" int lb_attn_bwd(const void* dO, long long lddo, const void* q, long long ldq,
                           const void* k, long long ldk, const void* v, long long ldv,
                           const void* o, long long ldo, const float* lse, float* delta,
                           const int* seq_start, const int* seq_end, const int* plan_q, int cap_q,
                           const int* plan_kv,
                           int cap_kv, void* dq, long long lddq, void* dk, long long lddk, void* dv,
                           long long lddv, int T, int Hq, int Hk, int hd, float softmax_scale,
                           int causal, int* status, void* stream) {
  if (T <= 0) return 0;
  if (Hk <= 0 || Hq % Hk != 0) return -3;
  const int G = Hq / Hk;
  if (G != 1 && G != 2 && G != 4 && G != 8) return -3;
  if ((lddo | ldq | ldk | ldv | ldo | lddq | lddk | lddv) & 7) return -3;
  AttnBwdArgs a{seq_start, seq_end, nullptr, lse, delta, (bf16*)dq, lddq, (bf16*)dk, lddk, (bf16*)dv, lddv,
                T, Hq, Hk, softmax_scale, softmax_scale * kLog2eF, causal, status};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (hd != 128 && hd != 64) return -3;
  // gradient rows of tokens behind the last sequence are written by no kernel below
  if (int rc = lb_attn_zero_tail(plan_q, cap_q, T, dq, lddq, Hq * hd, dk, lddk, Hk * hd, dv, lddv,
                                 Hk * hd, stream))
    return rc;
  if (hd == 128)
    return launch_bwd<128>(dO, lddo, q, ldq, k, ldk, v, ldv, o, ldo, delta, plan_q, cap_q, plan_kv,
                           cap_kv, a, st);
  if (hd == 64)
    return launch_bwd<64>(dO, lddo, q, ldq, k, ldk, v, ldv, o, ldo, delta, plan_q, cap_q, plan_kv,
                          cap_kv, a, st);
  return -3;
}
