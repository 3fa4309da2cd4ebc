// Varlen (packed) flash attention forward on tcgen05: causal or bidirectional, grouped-query heads.
//
// Persistent 128-thread CTAs (two per SM) walk over the (KV head, sequence, query tile) work items;
// TMEM and the barriers are set up once per CTA and the next item's Q and first K/V block are
// requested during the last block of the current one. Per KV block of 64:
//   S = Q·Kᵀ          tcgen05.mma, A = Q tile (128 x hd), B = K block (64 x hd), S in TMEM
//   online softmax     thread r owns row r: tcgen05.ld, mask, running max / sum in registers;
//                      the O accumulator in TMEM is rescaled only when the max moved by > 2^8
//   O += P·V          P (bf16) is written into the shared-memory slot of the K block it came from,
//                      V is consumed in place as an MN-major operand (no transpose)
// Q/K/V are read with TMA straight out of the (possibly fused) projection output through explicit
// row strides. Writes O and the natural-log LSE per (head, token) for the backward.
//
// Replaces flash_attn_varlen_func / varlen_attn / SDPA in the reference
// (lset/models/decoder/qwen3/attention.py:169-272, lset/models/encoder/bert/model.py:264-319).
#include "../common/ptx.cuh"
#include "../common/tma_desc.h"
#include "attn_common.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

struct AttnFwdArgs {
  const int* seq_start;  // first token of each sequence
  const int* seq_end;    // one past its last token
  const int* plan;
  unsigned* work_counter;  // zeroed by the launcher: hands out work items past the first wave
  bf16* O;
  long long ldo;   // elements between consecutive tokens of O
  float* lse;      // [Hq, T]
  int T, Hq, Hk;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int* status;
};

template <int HD>
struct FwdCfg {
  static constexpr int PANELS = HD / 64;
  static constexpr int Q_BYTES = 128 * HD * 2;
  static constexpr int KV_BYTES = kAttnKvBlock * HD * 2;
  static constexpr int P_BYTES = 128 * kAttnKvBlock * 2;
  static constexpr bool P_IN_K = KV_BYTES >= P_BYTES;
  static constexpr int SMEM_BYTES =
      Q_BYTES + 4 * KV_BYTES + (P_IN_K ? 0 : P_BYTES) + 1024 + 128;
  static constexpr int TMEM_COLS = (64 + HD) <= 128 ? 128 : ((64 + HD) <= 256 ? 256 : 512);
  static constexpr int O_COL = 64;
};

// Work item w of the persistent grid: KV head w / tiles, query tile w % tiles of the plan.
struct FwdTile {
  int seq0, len, q0, nblk, hk;
};

template <int HD>
__global__ void __launch_bounds__(128)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, AttnFwdArgs a) {
  using C = FwdCfg<HD>;
  AttnPlanView plan{a.plan};
  const int tiles = plan.count();
  const int total = tiles * a.Hk;
  if (int(blockIdx.x) >= total) return;
  const int G = a.Hq / a.Hk;
  const int QT = 128 / G;
  auto decode = [&](int w) {
    FwdTile t;
    t.hk = w / tiles;
    const int i = w - t.hk * tiles;
    const int b = plan.seq(i);
    t.seq0 = a.seq_start[b];
    t.len = a.seq_end[b] - t.seq0;
    t.q0 = plan.tile(i) * QT;
    const int kv_end = a.causal ? min(t.len, t.q0 + QT) : t.len;
    t.nblk = (kv_end + kAttnKvBlock - 1) / kAttnKvBlock;
    return t;
  };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;          // two buffers
  uint8_t* sV = sK + 2 * C::KV_BYTES;     // two buffers
  uint8_t* sPx = sV + 2 * C::KV_BYTES;    // separate P buffer (only when !P_IN_K)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sPx + (C::P_IN_K ? 0 : C::P_BYTES));
  uint64_t* bar_q = bars;
  uint64_t* bar_kv = bars + 1;  // [2]
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  __shared__ int s_next[2];  // next work item of this CTA, published by thread 0 one tile ahead

  // KV block n of this CTA's whole run (all tiles) lives in slot n & 1; its barrier phase is
  // (n >> 1) & 1. The score and P·V barriers complete once per block: phase n & 1.
  auto load_kv = [&](const FwdTile& t, int j, int n) {
    const int buf = n & 1;
    mbar_expect_tx(&bar_kv[buf], 2 * C::KV_BYTES);
#pragma unroll
    for (int p = 0; p < C::PANELS; ++p) {
      tma_load_2d(sK + buf * C::KV_BYTES + p * (kAttnKvBlock * 128), &tmK, &bar_kv[buf],
                  t.hk * HD + p * 64, t.seq0 + j * kAttnKvBlock);
      tma_load_2d(sV + buf * C::KV_BYTES + p * (kAttnKvBlock * 128), &tmV, &bar_kv[buf],
                  t.hk * HD + p * 64, t.seq0 + j * kAttnKvBlock);
    }
  };
  auto load_q = [&](const FwdTile& t) {
    mbar_expect_tx(bar_q, C::Q_BYTES);
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int p = 0; p < C::PANELS; ++p)
        tma_load_2d(sQ + p * (128 * 128) + g * QT * 128, &tmQ, bar_q,
                    (t.hk * G + g) * HD + p * 64, t.seq0 + t.q0);
  };

  FwdTile cur = decode(blockIdx.x);
  // The first loads are issued before the TMEM allocation and the CTA-wide barrier, so their
  // latency runs under that set-up instead of after it.
  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(&bar_kv[0], 1);
    mbar_init(&bar_kv[1], 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_fence_init();
    load_q(cur);
    load_kv(cur, 0, 0);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (uint32_t(warp * 32) << 16);
  constexpr uint32_t idesc_s = umma_idesc_bf16(128, kAttnKvBlock, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);

  const int r = tid;
  const int g = r / QT;
  bool failed = false;
  int n = 0;  // KV blocks processed so far by this CTA (over all its tiles)

  // Persistent loop: TMEM and the barriers are set up once; the Q tile and the first K/V block of
  // the next work item are requested while the current one is still in its last block.
  // Work items past the first wave are handed out by an atomic counter (tiles differ in length:
  // causal tiles late in a sequence see more KV blocks), fetched one tile ahead so that the next
  // item's loads can be requested early.
  for (int w = blockIdx.x, it = 0; w < total && !failed; ++it) {
    if (tid == 0) s_next[it & 1] = int(atomicAdd(a.work_counter, 1u)) + int(gridDim.x);
    __syncthreads();
    const int w_next = s_next[it & 1];
    const bool has_next = w_next < total;
    const FwdTile nxt = has_next ? decode(w_next) : cur;
    const int qpos = cur.q0 + r % QT;
    const bool row_valid = qpos < cur.len;
    const int len = cur.len;
    const int nblk = cur.nblk;
    float m_ref = -INFINITY;
    float l_sum = 0.f;

    {
      const bool ok = mbar_wait(bar_q, it & 1);
      if (__syncthreads_or(!ok)) {
        report_status(a.status, kStatusTimeoutProducer);
        failed = true;
        break;
      }
    }

    for (int j = 0; j < nblk; ++j, ++n) {
      const int buf = n & 1;
      const bool last = j + 1 == nblk;
      // 1. K/V block landed -> S = Q K^T
      {
        const bool ok = mbar_wait(&bar_kv[buf], (n >> 1) & 1);
        if (__syncthreads_or(!ok)) {
          report_status(a.status, kStatusTimeoutProducer);
          failed = true;
          break;
        }
      }
      if (tid == 0) {
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ);
        const uint32_t ka = smem_u32(sK + buf * C::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t ad = umma_smem_desc(qa + (ks / 4) * (128 * 128) + (ks % 4) * 32, 16, 1024);
          const uint64_t bd =
              umma_smem_desc(ka + (ks / 4) * (kAttnKvBlock * 128) + (ks % 4) * 32, 16, 1024);
          umma_bf16(tmem_base, ad, bd, idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(bar_s);
      }
      // 2. softmax statistics of this block
      {
        const bool ok = mbar_wait(bar_s, n & 1);
        if (__syncthreads_or(!ok)) {
          report_status(a.status, kStatusTimeoutMma);
          failed = true;
          break;
        }
      }
      tc_fence_after();
      // the last score product of this tile has read Q: the next tile's Q may land now
      if (tid == 0 && last && has_next) load_q(nxt);
      float s[kAttnKvBlock];
      {
        uint32_t t0[32], t1[32];
        tmem_ld_32x32b_x32(tmem_row, t0);
        tmem_ld_32x32b_x32(tmem_row + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          s[c] = __uint_as_float(t0[c]);
          s[32 + c] = __uint_as_float(t1[c]);
        }
      }
      float mx = -INFINITY;
      const int kv0 = j * kAttnKvBlock;
#pragma unroll
      for (int c = 0; c < kAttnKvBlock; ++c) {
        const int kvpos = kv0 + c;
        const bool valid = row_valid && kvpos < len && (!a.causal || kvpos <= qpos);
        s[c] = valid ? s[c] * a.scale_log2 : -INFINITY;
        mx = fmaxf(mx, s[c]);
      }
      // 3. previous P·V finished: its K/V/P slots are free and O may be touched (for the first
      //    block of a tile the previous tile's epilogue has already waited for it)
      if (j > 0) {
        const bool ok = mbar_wait(bar_o, (n - 1) & 1);
        if (__syncthreads_or(!ok)) {
          report_status(a.status, kStatusTimeoutMma);
          failed = true;
          break;
        }
        tc_fence_after();
      }
      if (tid == 0) {
        if (!last) load_kv(cur, j + 1, n + 1);
        else if (has_next) load_kv(nxt, 0, n + 1);  // first block of the next work item
      }
      // 4. lazy rescale, P -> shared memory
      const float m_new = fmaxf(m_ref, mx);
      const bool need = m_new > m_ref + 8.f;
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = (m_new == -INFINITY) ? 1.f
                            : (m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_new));
        l_sum *= alpha;
        m_ref = m_new;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_row + C::O_COL + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tmem_row + C::O_COL + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      uint8_t* sP = C::P_IN_K ? (sK + buf * C::KV_BYTES) : sPx;
#pragma unroll
      for (int c8 = 0; c8 < kAttnKvBlock / 8; ++c8) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p[i] = exp2f(s[c8 * 8 + i] - m_use);
          l_sum += p[i];
        }
        uint4 q;
        q.x = pack_bf16x2(p[0], p[1]);
        q.y = pack_bf16x2(p[2], p[3]);
        q.z = pack_bf16x2(p[4], p[5]);
        q.w = pack_bf16x2(p[6], p[7]);
        *reinterpret_cast<uint4*>(sP + swz128_offset(r, c8)) = q;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();
      // 5. O += P V
      if (tid == 0) {
        tc_fence_after();
        const uint32_t pa = smem_u32(sP);
        const uint32_t va = smem_u32(sV + buf * C::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < kAttnKvBlock / 16; ++ks) {
          const uint64_t ad = umma_smem_desc(pa + ks * 32, 16, 1024);
          const uint64_t bd = umma_smem_desc(va + ks * 2048, kAttnKvBlock * 128, 1024);
          umma_bf16(tmem_base + C::O_COL, ad, bd, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar_o);
      }
    }
    if (failed) break;

    {
      const bool ok = mbar_wait(bar_o, (n - 1) & 1);
      if (__syncthreads_or(!ok)) {
        report_status(a.status, kStatusTimeoutMma);
        failed = true;
        break;
      }
    }
    tc_fence_after();
    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
    const long long tok = 1LL * cur.seq0 + qpos;
    bf16* orow = a.O + tok * a.ldo + (cur.hk * G + g) * HD;
#pragma unroll 1
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t o[32];
      tmem_ld_32x32b_x32(tmem_row + C::O_COL + c * 32, o);
      tmem_ld_wait();
      if (row_valid) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 q;
          q.x = pack_bf16x2(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
          q.y = pack_bf16x2(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
          q.z = pack_bf16x2(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
          q.w = pack_bf16x2(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = q;
        }
      }
    }
    if (row_valid && a.lse != nullptr)
      a.lse[1LL * (cur.hk * G + g) * a.T + tok] =
          (l_sum > 0.f) ? (m_ref * kLn2F + logf(l_sum)) : -INFINITY;
    // the accumulator reads above are ordered before the next tile's MMAs (issued by thread 0
    // after the CTA barrier at the top of the next tile)
    tc_fence_before();
    cur = nxt;
    w = w_next;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// One block: prefix over sequences -> (sequence, tile) list. plan[0] = tile count.
__global__ void attn_plan_kernel(const int* __restrict__ seq_start,
                                 const int* __restrict__ seq_end, int B, int tile_tokens,
                                 int* __restrict__ plan, int capacity) {
  __shared__ int s_base;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  for (int b0 = 0; b0 < B; b0 += blockDim.x) {
    const int b = b0 + threadIdx.x;
    int nt = 0;
    if (b < B) nt = max(0, (seq_end[b] - seq_start[b] + tile_tokens - 1) / tile_tokens);
    // inclusive scan over the block (simple Hillis-Steele in shared memory)
    __shared__ int scan[256];
    scan[threadIdx.x] = nt;
    __syncthreads();
    for (int o = 1; o < blockDim.x; o <<= 1) {
      int v = threadIdx.x >= o ? scan[threadIdx.x - o] : 0;
      __syncthreads();
      scan[threadIdx.x] += v;
      __syncthreads();
    }
    const int start = s_base + scan[threadIdx.x] - nt;
    for (int t = 0; t < nt; ++t) {
      if (start + t < capacity) {
        plan[1 + 2 * (start + t)] = b;
        plan[2 + 2 * (start + t)] = t;
      }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) s_base += scan[threadIdx.x];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    plan[0] = s_base < capacity ? s_base : capacity;
    // second spare word (the first is the forward kernel's work counter): one past the last token
    // that belongs to a sequence. Tokens behind it (a stream padded to a fixed budget) are
    // written by no attention kernel; the launchers clear those rows.
    plan[1 + 2 * capacity + 1] = seq_end[B - 1];
  }
}

// Rows [*end, T) of up to three [T, w] bf16 matrices := 0 (nothing to do when *end >= T).
__global__ void __launch_bounds__(256)
    attn_zero_tail_kernel(const int* __restrict__ end_ptr, int T, bf16* p0, long long ld0, int w0,
                          bf16* p1, long long ld1, int w1, bf16* p2, long long ld2, int w2) {
  const int end = *end_ptr;
  if (end >= T || end < 0) return;
  bf16* ps[3] = {p0, p1, p2};
  const long long lds[3] = {ld0, ld1, ld2};
  const int ws[3] = {w0, w1, w2};
  for (int m = 0; m < 3; ++m) {
    if (ps[m] == nullptr) continue;
    const int vec = ws[m] / 8;
    const long long total = 1LL * (T - end) * vec;
    for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += 1LL * gridDim.x * blockDim.x) {
      const long long r = end + i / vec, c = (i % vec) * 8;
      *reinterpret_cast<uint4*>(ps[m] + r * lds[m] + c) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

template <int HD>
int launch_fwd(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
               const AttnFwdArgs& a, int max_tiles, cudaStream_t st) {
  using C = FwdCfg<HD>;
  auto kern = attn_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured = true;
  }
  // persistent: as many CTAs as fit at once (shared memory allows two per SM at head_dim <= 128),
  // never more than the upper bound of the work items; a CTA beyond the real count exits at once
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long upper = 1LL * max_tiles * a.Hk;
  const long long resident = 1LL * sms * (C::SMEM_BYTES <= 113 * 1024 ? 2 : 1);
  const int grid = static_cast<int>(upper < resident ? upper : resident);
  kern<<<grid, 128, C::SMEM_BYTES, st>>>(tmQ, tmK, tmV, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace
}  // namespace lb

using namespace lb;

// plan: int32 [1 + 2 * capacity + 1] (the last word is scratch for the attention kernels);
// capacity >= ceil(T / tile_tokens) + B always suffices.
// Clears the rows behind the last sequence of a stream (see attn_plan_kernel). plan / capacity as
// passed to lb_attn_plan; widths in elements, multiples of 8; unused matrices null.
extern "C" int lb_attn_zero_tail(const int* plan, int capacity, int T, void* p0, long long ld0,
                                 int w0, void* p1, long long ld1, int w1, void* p2, long long ld2,
                                 int w2, void* stream) {
  if (T <= 0) return 0;
  if ((w0 | w1 | w2) & 7) return -3;
  attn_zero_tail_kernel<<<64, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      plan + 1 + 2 * capacity + 1, T, (bf16*)p0, ld0, w0, (bf16*)p1, ld1, w1, (bf16*)p2, ld2, w2);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int lb_attn_plan(const int* seq_start, const int* seq_end, int B, int tile_tokens,
                            int* plan, int capacity, void* stream) {
  if (B <= 0) return -3;
  attn_plan_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(seq_start, seq_end, B,
                                                                         tile_tokens, plan, capacity);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Sequence b owns tokens [seq_start[b], seq_end[b]) of the stream (for a packed batch these are
// cu_seqlens and cu_seqlens + 1; for a padded batch they skip the padding).
// q: [T, Hq, hd] with token stride ldq (elements); k, v: [T, Hk, hd] with strides ldk, ldv.
// plan was built with tile_tokens = 128 / (Hq / Hk). o: [T, Hq, hd] stride ldo; lse: [Hq, T] fp32.
extern "C" int lb_attn_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                           long long ldv, const int* seq_start, const int* seq_end, const int* plan,
                           int max_tiles,
                           void* o, long long ldo, float* lse, int T, int Hq, int Hk, int hd,
                           float softmax_scale, int causal, int* status, void* stream) {
  if (T <= 0 || max_tiles <= 0) return 0;
  if (Hk <= 0 || Hq % Hk != 0) return -3;
  const int G = Hq / Hk;
  if (G != 1 && G != 2 && G != 4 && G != 8) return -3;
  if ((ldq | ldk | ldv | ldo) & 7) return -3;
  const int QT = 128 / G;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_2d(&tmQ, q, 2, (uint64_t)Hq * hd, (uint64_t)T, (uint64_t)ldq * 2, 64, QT, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, 2, (uint64_t)Hk * hd, (uint64_t)T, (uint64_t)ldk * 2, 64, kAttnKvBlock,
                    true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, 2, (uint64_t)Hk * hd, (uint64_t)T, (uint64_t)ldv * 2, 64, kAttnKvBlock,
                    true);
  if (rc) return rc;
  // the plan buffer carries two spare words behind its 1 + 2 * max_tiles entries: this kernel's
  // work counter and the end of the stream's last sequence
  unsigned* counter = reinterpret_cast<unsigned*>(const_cast<int*>(plan)) + 1 + 2 * max_tiles;
  AttnFwdArgs a{seq_start, seq_end, plan, counter, (bf16*)o, ldo, lse, T, Hq, Hk,
                softmax_scale * kLog2eF, causal, status};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), st) != cudaSuccess) return -12;
  if (hd != 128 && hd != 64 && hd != 256) return -3;
  rc = lb_attn_zero_tail(plan, max_tiles, T, o, ldo, Hq * hd, nullptr, 0, 0, nullptr, 0, 0, stream);
  if (rc) return rc;
  if (hd == 128) return launch_fwd<128>(tmQ, tmK, tmV, a, max_tiles, st);
  if (hd == 64) return launch_fwd<64>(tmQ, tmK, tmV, a, max_tiles, st);
  if (hd == 256) return launch_fwd<256>(tmQ, tmK, tmV, a, max_tiles, st);
  return -3;
}
