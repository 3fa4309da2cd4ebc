// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] (+)= A · B^T      A: M x K,  B: N x K,  fp32 accumulation in tensor memory.
//
// Either operand may be stored "K-major" (rows = M/N index, K contiguous; the layout of an
// nn.Linear input or weight) or "MN-major" (rows = K index, M/N contiguous). That covers all three
// products of a linear layer without any transposition pass:
//   fprop  Y = X · W^T        A = X  (K-major),  B = W  (K-major)
//   dgrad  dX = dY · W        A = dY (K-major),  B = W  (MN-major: rows are the contracted N)
//   wgrad  dW = dY^T · X      A = dY (MN-major), B = X  (MN-major), contraction over tokens
//
// Structure (one CTA per SM, 192 threads):
//   warp 0    TMA producer: cp.async.bulk.tensor tiles of A and B into a 128B-swizzled smem ring
//   warp 1    one thread issues tcgen05.mma (128 x BN x 16) into one of two TMEM accumulators
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator, add bias / convert / store / reduce,
//             while warp 1 already fills the other accumulator with the next tile.
// Tiles are walked with a static stride over a persistent grid; an optional split along K makes
// enough tiles for the long-K weight-gradient products and reduces with red.global.add.f32.
//
// Replaces cuBLAS behind nn.Linear in the reference (lset/models/decoder/qwen3/attention.py:102-104,
// lset/models/decoder/qwen3/mlp.py:28).
#include <cuda_bf16.h>
#include <stdlib.h>

#include "../common/ptx.cuh"
#include "../common/tma_desc.h"

namespace lb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGatherThreads = 256;  // + 2 pull warps

// Number of epilogue warps. The plain store / reduce epilogue of the bf16 kernel runs on eight
// (two per tensor-memory lane quarter, each taking half of the tile's columns): at K = 1024 the
// main loop of a 128 x 256 tile lasts about as long as four warps need to drain it, and the drain
// then bounds the kernel. The loss / GLU epilogues, the 8-bit kernel and the peer-gather variants
// (which already carry two pull warps) keep four.
template <int EPI, int GATHER, int F8>
constexpr int epi_warps() {
  return (EPI == 0 /*EPI_STORE*/ && GATHER == 0 && F8 == 0) ? 8 : 4;
}
template <int EPI, int GATHER, int F8>
constexpr int gemm_threads() {
  return GATHER ? kGatherThreads : 64 + 32 * epi_warps<EPI, GATHER, F8>();
}

struct GemmArgs {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;  // nullable, length N
  int accumulate;             // fp32 output only: C += result (red.global.add)
  int splits;                 // >= 1, split of the K range
  int kb_per_split;
  int raster_m_fast;          // tile order: consecutive tiles walk M first (B tile shared in L2)
  int kb_ext;                 // extra k-blocks read through the second tensor-map pair (A2, B2):
                              // C = A·Bᵀ + A2·B2ᵀ in one accumulator pass (LoRA: A2 = x·A_loraᵀ)
  // contrastive-loss epilogues (EPI_LSE / EPI_PGRAD): scores s = acc * scale
  float scale;                // 1 / temperature
  const float* lse;           // [M] natural-log LSE (EPI_PGRAD input)
  float* part;                // [tiles_n, M, 2] running (max, sum) in log2 domain (EPI_LSE output)
  float* pos;                 // [M] score of the target column (EPI_LSE output)
  const float* coef;          // device scalar multiplied into the probabilities' gradient
  long long target_offset;    // target column of row r is r + target_offset
  // label-matrix losses (labels != nullptr): int8 labels [M, ld_labels] (1 positive, 0 negative,
  // < 0 ignored; ld_labels a multiple of 32 and >= N, padding = ignored), optional target weights
  // tw [M, ld_tw] fp32 (soft labels; zero where ignored), row_scale [M] (1 / number of positives,
  // or 1 / sum of the target weights) and row_w [M] (weight of the row in the mean; 0 = skipped).
  const signed char* labels;
  long long ld_labels;
  const float* tw;
  long long ld_tw;
  const float* row_scale;
  const float* row_w;
  // 0: LSE over label >= 0, target t = tw or max(label, 0) (weighted cross-entropy family);
  // 1: multi-positive NCE: LSE over label == 0 only; the gradient of a positive is
  //    sigmoid(s - lse) - 1, of a negative exp(s - lse) * row_scale (row_scale = sum over the
  //    row's positives of sigmoid(lse - s_p)).
  int loss_mode;
  // EPI_GLU: B = fused [gate; up] weight [2 * glu_I, K]; N = glu_I features. A 128 x 256 tile holds
  // gate and up of the same 128 features side by side; the epilogue stores both halves into
  // C = gate_up [M, 2 * glu_I] (for the backward) and act(gate) * up into glu_h [M, glu_I].
  int glu_I;
  void* glu_h;
  long long ld_h;
  int glu_kind;  // 0 = SwiGLU, 1 = tanh-GeGLU
  // ---- peer gather (GATHER 1: rows of B, GATHER 2: rows of A): the rows live in `world` ranks'
  // buffers, n_local rows each; two extra warps pull them into b_local ([world * n_local, K], the
  // base of that operand's tensor map) and publish one flag per (rank, row tile); tiles are
  // visited in pull order, own rank first (its rows are placed by the host, no pull).
  const void* b_peers[8];
  void* b_local;
  long long ldb_peer;         // row stride (elements) of every rank's buffer and of b_local
  int n_local, world, rank;
  unsigned* flags;            // [world * tiles_per_peer], value == epoch when the tile is local
  unsigned* chunk_counter;    // work-stealing counter of the pull warps (reset by the host)
  unsigned epoch;
  // The first copy_ctas CTAs of a gather launch compute no tiles: all of their warps pull. Two
  // pull warps per computing CTA keep too few bytes in flight to fill NVLink at eight ranks; a
  // copy CTA keeps 8 warps x 8 KB on the wire.
  int copy_ctas;
  // ---- peer scatter of C (fp32 accumulate only): row r belongs to rank r / c_rows_per_peer and
  // is reduced into that rank's buffer with red.global.add over NVLink.
  void* c_peers[8];
  int c_rows_per_peer;        // 0 = C is a single local matrix
  int c_store;                // bf16 scatter: plain stores (every source rank owns a slot of the
                              // destination, summed by the owner afterwards) instead of reductions
  // ---- 8-bit float operands (F8 kernels): the accumulator of element (r, c) is multiplied by
  // f8_sa[r * f8_sa_stride] * f8_sb[c * f8_sb_stride] (the operands' dequantisation factors; a
  // stride of 0 is one factor for the whole tensor). Operand formats: 0 = e4m3, 1 = e5m2.
  const float* f8_sa;
  const float* f8_sb;
  int f8_sa_stride, f8_sb_stride;
  int f8_a_e5m2, f8_b_e5m2;
  int* status;
};

enum { EPI_STORE = 0, EPI_LSE = 1, EPI_PGRAD = 2, EPI_GLU = 3 };
constexpr float kLog2e = 1.4426950408889634f;

template <int BN, int EW = 4, int F8 = 0>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  // per epilogue warp: a staging block that turns "one row per lane" (the TMEM load layout) into
  // "one 128-byte row segment per 8 lanes" for global memory: 32 x 32 fp32 (row stride 33 words)
  // for the fp32 reductions, 32 rows x 64 bf16 columns (row stride 144 bytes) for bf16 stores;
  // both strides are conflict-free for the lane-per-row writes and the 8-lanes-per-row reads
  // With eight epilogue warps the bf16 staging block is 32 rows x 32 columns (row stride 80
  // bytes, also conflict-free) and is flushed after every chunk, so that the blocks of all warps
  // still fit beside the four operand stages.
  static constexpr int EPI_STAGE_WORDS = EW == 8 ? 32 * 33 : 32 * 36;
  static constexpr int EPI_STAGE_BYTES = EW * EPI_STAGE_WORDS * 4;
  // per epilogue warp: the BN per-column dequantisation factors of the current tile (8-bit GEMM)
  static constexpr int EPI_SCALE_BYTES = F8 ? 4 * 256 * 4 : 0;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ +
                                    EPI_STAGE_BYTES + EPI_SCALE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
};

__device__ __forceinline__ void red_add4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// 8 bf16 values added into memory in one 16-byte reduction (packed bf16x2 lanes)
__device__ __forceinline__ void red_add8_bf16(void* dst, const uint4& v) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

template <int A_MN, int B_MN, int BN, typename OutT, int EPI, int GATHER = 0, int F8 = 0>
__global__ void __launch_bounds__(gemm_threads<EPI, GATHER, F8>(), 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmA2,
                     const __grid_constant__ CUtensorMap tmB2, GemmArgs g) {
  constexpr int EW = epi_warps<EPI, GATHER, F8>();
  using C = Cfg<BN, EW, F8>;
  // 8-bit operands: K-major only; a k-block is still 128 bytes of every row, i.e. 128 elements,
  // and the shared-memory tiles, swizzle and descriptors are byte-for-byte those of the bf16 form.
  static_assert(!F8 || (!A_MN && !B_MN && GATHER == 0 && EPI == EPI_STORE), "fp8: plain TN GEMM");
  constexpr int BKE = F8 ? 2 * BK : BK;  // elements per k-block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tfull = empty + C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  [[maybe_unused]] float* epi_stage =
      reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 32 * EW);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (g.kb_ext > 0) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // CTAs that compute tiles are numbered 0 .. ncta-1 (a gather launch puts its copy CTAs first)
  [[maybe_unused]] const int n_copy = GATHER ? g.copy_ctas : 0;
  const int cta = int(blockIdx.x) - n_copy;
  const int ncta = int(gridDim.x) - n_copy;
  // GATHER 1: rows of B come from the peers; GATHER 2: rows of A do. n_local = rows per rank.
  constexpr int kGatherRows = GATHER == 2 ? BM : BN;
  constexpr int kPullRows = 16;  // rows per pull item (one warp); divides BM and BN
  // (1 without a gather, so that the index arithmetic below stays defined)
  [[maybe_unused]] const int tiles_per_peer = GATHER ? (g.n_local + kGatherRows - 1) / kGatherRows : 1;
  const int tiles_m = GATHER == 2 ? g.world * tiles_per_peer : (g.M + BM - 1) / BM;
  constexpr int kTileN = EPI == EPI_GLU ? 128 : BN;  // output features (columns) per tile
  const int tiles_n = GATHER == 1 ? g.world * tiles_per_peer : (g.N + kTileN - 1) / kTileN;
  const int kb_main = (g.K + BKE - 1) / BKE;
  const int kb_total = kb_main + g.kb_ext;
  const int total = tiles_m * tiles_n * g.splits;
  // (m0, n0, flag index) of the `mn`-th output tile
  auto decode = [&](int mn, int& m0, int& n0, int& chunk) {
    if constexpr (GATHER == 1) {
      m0 = (mn % tiles_m) * BM;
      const int ni = mn / tiles_m;
      const int peer = (g.rank + ni / tiles_per_peer) % g.world;
      chunk = peer * tiles_per_peer + ni % tiles_per_peer;
      n0 = peer * g.n_local + (ni % tiles_per_peer) * BN;
    } else if constexpr (GATHER == 2) {
      n0 = (mn % tiles_n) * BN;
      const int mi = mn / tiles_n;
      const int peer = (g.rank + mi / tiles_per_peer) % g.world;
      chunk = peer * tiles_per_peer + mi % tiles_per_peer;
      m0 = peer * g.n_local + (mi % tiles_per_peer) * BM;
    } else {
      m0 = (g.raster_m_fast ? mn % tiles_m : mn / tiles_n) * BM;
      n0 = (g.raster_m_fast ? mn / tiles_m : mn % tiles_n) * kTileN;
      chunk = 0;
    }
  };

  // The rows of a chunk (one row tile of one rank) are pulled as items of kPullRows rows by
  // different warps; flags[chunk] counts completed items and only ever grows: after the call with
  // epoch e it holds e * items_of_chunk(chunk).
  [[maybe_unused]] auto items_of_chunk = [&](int chunk) {
    const int t = chunk % tiles_per_peer;
    const int rows = min(kGatherRows, g.n_local - t * kGatherRows);
    return (rows + kPullRows - 1) / kPullRows;
  };

  if (warp == 0 && cta >= 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < total && ok; tile += ncta) {
        const int split = tile / (tiles_m * tiles_n);
        const int mn = tile - split * (tiles_m * tiles_n);
        int m0, n0, chunk;
        decode(mn, m0, n0, chunk);
        if constexpr (GATHER) {
          // the rows of this tile must have been pulled into local memory
          bool landed = false;
          const unsigned long long t0 = globaltimer_ns();
          for (unsigned it2 = 0;; ++it2) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(g.flags + chunk) : "memory");
            if (v >= g.epoch * unsigned(items_of_chunk(chunk))) {
              landed = true;
              break;
            }
            if ((it2 & 63u) == 63u && globaltimer_ns() - t0 > kWaitLimitNs) break;
          }
          if (!landed) {
            report_status(g.status, kStatusTimeoutPeer);
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(kb0 + g.kb_per_split, kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u)) {
            report_status(g.status, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], C::STAGE_BYTES);
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          // k-blocks past the main contraction come from the second operand pair
          const bool ext = kb >= kb_main;
          const CUtensorMap* ta = ext ? &tmA2 : &tmA;
          const CUtensorMap* tb = ext ? &tmB2 : &tmB;
          const int kc = (ext ? kb - kb_main : kb) * BKE;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (BK * 128), ta, &full[stage], m0 + 64 * c, kc);
          } else {
            tma_load_2d(sa, ta, &full[stage], kc, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (BK * 128), tb, &full[stage], n0 + 64 * c, kc);
          } else if constexpr (EPI == EPI_GLU) {
            // gate rows and up rows of the same 128 features, side by side in the B tile
            tma_load_2d(sb, tb, &full[stage], kc, n0);
            tma_load_2d(sb + 128 * 128, tb, &full[stage], kc, g.glu_I + n0);
          } else {
            tma_load_2d(sb, tb, &full[stage], kc, n0);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Let copies that were already issued land before the CTA gives its shared memory back.
        for (int s = 0; s < C::STAGES; ++s) mbar_wait(&full[s], 0, 2000000ull);
      }
    }
    __syncwarp();
  } else if (warp == 1 && cta >= 0) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = F8 ? umma_idesc_f8(BM, BN, g.f8_a_e5m2, g.f8_b_e5m2)
                                : umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = cta; tile < total && ok; tile += ncta, ++it) {
        const int split = tile / (tiles_m * tiles_n);
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(kb0 + g.kb_per_split, kb_total);
        const int acc = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aphase ^ 1u)) {
          report_status(g.status, kStatusTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase)) {
            report_status(g.status, kStatusTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc(sa + k * 2048, BK * 128, 1024)
                                        : umma_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(sb + k * 2048, BK * 128, 1024)
                                        : umma_smem_desc(sb + k * 32, 16, 1024);
            if constexpr (F8)
              umma_f8(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else
              umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
    __syncwarp();
  } else if (GATHER && (warp >= 6 || cta < 0)) {
    // ------------------------------------------------------------------ pull warps (6, 7; every
    // warp of a copy CTA)
    if constexpr (GATHER) {
      constexpr int kItemsPerTile = kGatherRows / kPullRows;
      const int items_total = g.world * tiles_per_peer * kItemsPerTile;
      const long long vec_per_row = (2LL * g.K) / 16;
      for (;;) {
        unsigned c = 0;
        if (lane == 0) c = atomicAdd(g.chunk_counter, 1u);
        c = __shfl_sync(0xffffffffu, c, 0);
        if (c >= unsigned(items_total)) break;
        const int tile_i = int(c) / kItemsPerTile;      // tiles in consumption order
        const int sub = int(c) % kItemsPerTile;
        const int peer = (g.rank + tile_i / tiles_per_peer) % g.world;
        const int t = tile_i % tiles_per_peer;
        const int r0 = t * kGatherRows + sub * kPullRows;
        const int tile_end = min((t + 1) * kGatherRows, g.n_local);
        if (r0 >= tile_end) continue;                   // short last tile: no such item
        const int r1 = min(r0 + kPullRows, tile_end);
        if (peer != g.rank) {                           // own rows are in place already
          const char* src = static_cast<const char*>(g.b_peers[peer]);
          char* dst = static_cast<char*>(g.b_local) + 2LL * peer * g.n_local * g.ldb_peer;
          const long long total_vec = vec_per_row * (r1 - r0);
          // 16 x 16 bytes per lane in flight: a warp keeps 8 KB on the wire, which is what the
          // NVLink round trip needs for two pull warps per SM to reach the link rate
          constexpr int kPullDepth = 16;
          for (long long i0 = 0; i0 < total_vec; i0 += 32 * kPullDepth) {
            uint4 buf[kPullDepth];
#pragma unroll
            for (int u = 0; u < kPullDepth; ++u) {
              const long long i = i0 + u * 32 + lane;
              if (i < total_vec) {
                const long long rr = r0 + i / vec_per_row, cc = i % vec_per_row;
                buf[u] = *reinterpret_cast<const uint4*>(src + 2LL * rr * g.ldb_peer + cc * 16);
              }
            }
#pragma unroll
            for (int u = 0; u < kPullDepth; ++u) {
              const long long i = i0 + u * 32 + lane;
              if (i < total_vec) {
                const long long rr = r0 + i / vec_per_row, cc = i % vec_per_row;
                *reinterpret_cast<uint4*>(dst + 2LL * rr * g.ldb_peer + cc * 16) = buf[u];
              }
            }
          }
          __threadfence();
        }
        __syncwarp();
        if (lane == 0) {
          unsigned* fp = g.flags + (peer * tiles_per_peer + t);
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(fp) : "memory");
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, or 2..9)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    // eight warps: warps 2..5 take the first half of the tile's 32-column chunks, 6..9 the second
    [[maybe_unused]] const int half = (warp - 2) >> 2;
    constexpr int kChunks = BN / 32 / (EW / 4);
    OutT* Cout = reinterpret_cast<OutT*>(g.C);
    int it = 0;
    for (int tile = cta; tile < total; tile += ncta, ++it) {
      const int split = tile / (tiles_m * tiles_n);
      const int mn = tile - split * (tiles_m * tiles_n);
      int m0, n0, chunk;
      decode(mn, m0, n0, chunk);
      const int n_limit = GATHER == 1 ? min(g.N, (n0 / g.n_local + 1) * g.n_local) : g.N;
      const int m_limit = GATHER == 2 ? min(g.M, (m0 / g.n_local + 1) * g.n_local) : g.M;
      const int acc = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aphase)) {
        report_status(g.status, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      if constexpr (EPI == EPI_GLU) {
        // gate chunk c and up chunk c of the tile -> gate_up (both halves) and h = act(gate) * up.
        // Values are rounded to bf16 before the activation, as the stand-alone GLU kernel sees them.
        uint8_t* sblk = reinterpret_cast<uint8_t*>(epi_stage + (warp - 2) * C::EPI_STAGE_WORDS);
        __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(g.C);
        __nv_bfloat16* hout = reinterpret_cast<__nv_bfloat16*>(g.glu_h);
        const int I = g.glu_I;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + c * 32, rg);
          tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + 128 + c * 32, ru);
          tmem_ld_wait();
          const int f = n0 + c * 32;
          if (f >= I) continue;  // uniform over the warp
          uint32_t pg[16], pu[16], ph[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pg[j] = pack_bf16x2(__uint_as_float(rg[2 * j]), __uint_as_float(rg[2 * j + 1]));
            pu[j] = pack_bf16x2(__uint_as_float(ru[2 * j]), __uint_as_float(ru[2 * j + 1]));
            const float2 gv = unpack_bf16x2(pg[j]), uv = unpack_bf16x2(pu[j]);
            float a0, a1;
            if (g.glu_kind == 0) {
              a0 = gv.x * (1.f / (1.f + __expf(-gv.x)));
              a1 = gv.y * (1.f / (1.f + __expf(-gv.y)));
            } else {
              const float k0 = 0.7978845608028654f, k1 = 0.044715f;
              a0 = 0.5f * gv.x * (1.f + tanhf(k0 * (gv.x + k1 * gv.x * gv.x * gv.x)));
              a1 = 0.5f * gv.y * (1.f + tanhf(k0 * (gv.y + k1 * gv.y * gv.y * gv.y)));
            }
            ph[j] = pack_bf16x2(a0 * uv.x, a1 * uv.y);
          }
          uint8_t* srow = sblk + lane * 144;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<uint4*>(srow + 16 * j) =
                make_uint4(pg[4 * j], pg[4 * j + 1], pg[4 * j + 2], pg[4 * j + 3]);
            *reinterpret_cast<uint4*>(srow + 64 + 16 * j) =
                make_uint4(pu[4 * j], pu[4 * j + 1], pu[4 * j + 2], pu[4 * j + 3]);
          }
          __syncwarp();
          {
            const int rr = lane >> 3, cc = lane & 7;
            const int fcol = f + (cc & 3) * 8;
            const long long col = (cc < 4 ? 0 : I) + fcol;
            if (fcol < I) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int lr = i * 4 + rr;
                const int grow = m0 + q * 32 + lr;
                if (grow < g.M)
                  *reinterpret_cast<uint4*>(gu + static_cast<long long>(grow) * g.ldc + col) =
                      *reinterpret_cast<const uint4*>(sblk + lr * 144 + cc * 16);
              }
            }
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(srow + 16 * j) =
                make_uint4(ph[4 * j], ph[4 * j + 1], ph[4 * j + 2], ph[4 * j + 3]);
          __syncwarp();
          {
            const int rr = lane >> 2, cc = lane & 3;
            const int fcol = f + cc * 8;
            if (fcol < I) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int lr = i * 8 + rr;
                const int grow = m0 + q * 32 + lr;
                if (grow < g.M)
                  *reinterpret_cast<uint4*>(hout + static_cast<long long>(grow) * g.ld_h + fcol) =
                      *reinterpret_cast<const uint4*>(sblk + lr * 144 + cc * 16);
              }
            }
          }
          __syncwarp();
        }
        tc_fence_before();
        mbar_arrive(&tempty[acc]);
        continue;
      }
      const int row = m0 + q * 32 + lane;
      const bool add_bias = (g.bias != nullptr) && (split == 0);
      [[maybe_unused]] float m_run = -INFINITY, l_run = 0.f, pos_val = 0.f;
      [[maybe_unused]] bool pos_here = false;
      [[maybe_unused]] const long long target = row + g.target_offset;
      [[maybe_unused]] const float s2 = g.scale * kLog2e;
      [[maybe_unused]] float lse2 = 0.f, cf = 0.f;
      [[maybe_unused]] const bool lbl = g.labels != nullptr;
      [[maybe_unused]] float rscale = 0.f;
      [[maybe_unused]] float f8_row = 1.f;
      [[maybe_unused]] float* f8_cols = reinterpret_cast<float*>(
          smem + C::STAGES * C::STAGE_BYTES + 256 + C::EPI_STAGE_BYTES) + (warp - 2) * 256;
      if constexpr (F8) {
        f8_row = (row < m_limit) ? g.f8_sa[(long long)row * g.f8_sa_stride] : 0.f;
        if (g.f8_sb_stride == 0) {
          f8_row *= g.f8_sb[0];  // one factor for all of B: folded into the row factor
        } else {
          __syncwarp();
#pragma unroll
          for (int i = 0; i < BN / 32; ++i) {
            const int cj = n0 + i * 32 + lane;
            f8_cols[i * 32 + lane] = cj < g.N ? g.f8_sb[cj] : 0.f;
          }
          __syncwarp();
        }
      }
      if constexpr (EPI == EPI_PGRAD) {
        lse2 = (row < m_limit) ? g.lse[row] * kLog2e : 0.f;
        cf = g.coef != nullptr ? g.coef[0] : 1.f;
        if (lbl && row < m_limit) {
          cf *= g.row_w[row];
          rscale = g.row_scale[row];
        }
      }
#pragma unroll 1
      for (int c = (EW == 8 ? half * kChunks : 0); c < (EW == 8 ? (half + 1) * kChunks : BN / 32);
           ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if constexpr (F8) {
          // dequantise in place: row factor of A times column factor of B
          if (g.f8_sb_stride == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f8_row);
          } else {
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 sb = *reinterpret_cast<const float4*>(f8_cols + c * 32 + 4 * j4);
              r[4 * j4] = __float_as_uint(__uint_as_float(r[4 * j4]) * f8_row * sb.x);
              r[4 * j4 + 1] = __float_as_uint(__uint_as_float(r[4 * j4 + 1]) * f8_row * sb.y);
              r[4 * j4 + 2] = __float_as_uint(__uint_as_float(r[4 * j4 + 2]) * f8_row * sb.z);
              r[4 * j4 + 3] = __float_as_uint(__uint_as_float(r[4 * j4 + 3]) * f8_row * sb.w);
            }
          }
        }
        if (row < m_limit && col0 < g.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          [[maybe_unused]] uint32_t lab[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
          if constexpr (EPI != EPI_STORE) {
            if (lbl) {
              const uint4* lp = reinterpret_cast<const uint4*>(
                  g.labels + static_cast<long long>(row) * g.ld_labels + col0);
              const uint4 l0 = lp[0], l1 = lp[1];
              lab[0] = l0.x; lab[1] = l0.y; lab[2] = l0.z; lab[3] = l0.w;
              lab[4] = l1.x; lab[5] = l1.y; lab[6] = l1.z; lab[7] = l1.w;
            }
          }
          // label of column j of this chunk, sign-extended
          [[maybe_unused]] auto label_at = [&](int j) {
            return static_cast<int>(static_cast<signed char>((lab[j >> 2] >> ((j & 3) * 8)) & 0xffu));
          };
          if constexpr (EPI == EPI_LSE) {
            float cm = -INFINITY;
            if (lbl) {
              const float* twp =
                  g.tw != nullptr ? g.tw + static_cast<long long>(row) * g.ld_tw + col0 : nullptr;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int l = label_at(j);
                const bool in = (col0 + j < n_limit) && (g.loss_mode == 1 ? l == 0 : l >= 0);
                if (in) {
                  if (twp != nullptr) pos_val += twp[j] * v[j] * g.scale;
                  else if (l > 0) pos_val += float(l) * v[j] * g.scale;
                }
                v[j] = in ? v[j] * s2 : -INFINITY;
                cm = fmaxf(cm, v[j]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const bool in = col0 + j < n_limit;
                if (in && col0 + j == target) {
                  pos_val = v[j] * g.scale;
                  pos_here = true;
                }
                v[j] = in ? v[j] * s2 : -INFINITY;
                cm = fmaxf(cm, v[j]);
              }
            }
            const float m_new = fmaxf(m_run, cm);
            if (m_new > -INFINITY) {  // a chunk of ignored columns leaves the running pair alone
              float sum = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) sum += exp2f(v[j] - m_new);
              l_run = l_run * exp2f(m_run - m_new) + sum;
              m_run = m_new;
            }
          } else {
            if constexpr (EPI == EPI_PGRAD) {
              if (lbl) {
                const float* twp =
                    g.tw != nullptr ? g.tw + static_cast<long long>(row) * g.ld_tw + col0 : nullptr;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const int l = label_at(j);
                  const bool in = (col0 + j < g.N) && l >= 0;
                  const float e = in ? exp2f(v[j] * s2 - lse2) : 0.f;  // exp(s - lse)
                  if (g.loss_mode == 1) {
                    // positives: sigmoid(s - lse) - 1 = -1 / (1 + e); negatives: e * row_scale
                    v[j] = (!in || cf == 0.f) ? 0.f : (l > 0 ? -cf / (1.f + e) : e * rscale * cf);
                  } else {
                    const float t =
                        !in ? 0.f : (twp != nullptr ? twp[j] * rscale : (l > 0 ? float(l) * rscale : 0.f));
                    v[j] = cf == 0.f ? 0.f : (e - t) * cf;  // skipped rows: no inf * 0
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float p = exp2f(v[j] * s2 - lse2);
                  v[j] = (p - ((col0 + j == target) ? 1.f : 0.f)) * cf;
                }
              }
            }
            if (add_bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < g.N) v[j] += __bfloat162float(g.bias[col0 + j]);
            }
            OutT* dst = Cout + static_cast<long long>(row) * g.ldc + col0;
            if constexpr (sizeof(OutT) == 4) {
              if (g.c_rows_per_peer > 0)
                dst = reinterpret_cast<OutT*>(g.c_peers[row / g.c_rows_per_peer]) +
                      static_cast<long long>(row % g.c_rows_per_peer) * g.ldc + col0;
            }
            if constexpr (sizeof(OutT) == 2) {
              // this lane's 32 columns go to its row of the staging block (flushed below)
              uint8_t* srow = reinterpret_cast<uint8_t*>(epi_stage + (warp - 2) * C::EPI_STAGE_WORDS) +
                              (EW == 8 ? lane * 80 : lane * 144 + (c & 1) * 64);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 pk;
                pk.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
                pk.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                pk.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                pk.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                *reinterpret_cast<uint4*>(srow + 16 * j) = pk;
              }
              (void)dst;
            } else {
              float* fd = reinterpret_cast<float*>(dst);
              if (g.accumulate) {
                // handled below by the whole warp (row-coalesced reductions)
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (col0 + 4 * j < g.N)
                    *reinterpret_cast<float4*>(fd + 4 * j) =
                        make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
            }
          }
        }
        if constexpr (sizeof(OutT) == 2 && EPI != EPI_LSE && EW == 8) {
          // The warp writes its 32 x 32 block out after every chunk: 4 lanes cover one 64-byte row
          // segment, a store instruction fills eight of them.
          __syncwarp();
          const uint8_t* sblk =
              reinterpret_cast<const uint8_t*>(epi_stage + (warp - 2) * C::EPI_STAGE_WORDS);
          const int rr = lane >> 2, cc = lane & 3;
          const int colb = n0 + c * 32 + cc * 8;
          if (colb < g.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int lr = i * 8 + rr;
              const int grow = m0 + q * 32 + lr;
              if (grow < m_limit) {
                const uint4 pk = *reinterpret_cast<const uint4*>(sblk + lr * 80 + cc * 16);
                if (g.c_rows_per_peer > 0) {
                  // reduce-scatter in bf16: the row's owner accumulates over NVLink
                  OutT* base = reinterpret_cast<OutT*>(g.c_peers[grow / g.c_rows_per_peer]) +
                               static_cast<long long>(grow % g.c_rows_per_peer) * g.ldc;
                  if (g.c_store)
                    *reinterpret_cast<uint4*>(base + colb) = pk;
                  else
                    red_add8_bf16(base + colb, pk);
                } else {
                  *reinterpret_cast<uint4*>(Cout + static_cast<long long>(grow) * g.ldc + colb) = pk;
                }
              }
            }
          }
          __syncwarp();
        }
        if constexpr (sizeof(OutT) == 2 && EPI != EPI_LSE && EW != 8) {
          // After every second 32-column chunk the warp writes its 32 x 64 block out: 8 lanes cover
          // one 128-byte row segment, so each store instruction fills four whole lines.
          if (c & 1) {
            __syncwarp();
            const uint8_t* sblk =
                reinterpret_cast<const uint8_t*>(epi_stage + (warp - 2) * C::EPI_STAGE_WORDS);
            const int rr = lane >> 3, cc = lane & 7;
            const int colb = n0 + (c - 1) * 32 + cc * 8;
            if (colb < g.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int lr = i * 4 + rr;
                const int grow = m0 + q * 32 + lr;
                if (grow < m_limit) {
                  const uint4 pk = *reinterpret_cast<const uint4*>(sblk + lr * 144 + cc * 16);
                  if (g.c_rows_per_peer > 0) {
                    // reduce-scatter in bf16: the row's owner accumulates over NVLink
                    OutT* base = reinterpret_cast<OutT*>(g.c_peers[grow / g.c_rows_per_peer]) +
                                 static_cast<long long>(grow % g.c_rows_per_peer) * g.ldc;
                    if (g.c_store)
                      *reinterpret_cast<uint4*>(base + colb) = pk;
                    else
                      red_add8_bf16(base + colb, pk);
                  } else {
                    *reinterpret_cast<uint4*>(Cout + static_cast<long long>(grow) * g.ldc + colb) = pk;
                  }
                }
              }
            }
            __syncwarp();
          }
        }
        if constexpr (sizeof(OutT) == 4 && EPI == EPI_STORE) {
          if (g.accumulate && col0 < g.N) {
            // Transpose through shared memory: lane = row on the way in, 8 lanes = one 128-byte
            // row segment on the way out, so every reduction instruction covers 4 full lines
            // (local L2 atomics and, for peer-owned rows, NVLink reductions both want whole lines).
            float* st = epi_stage + (warp - 2) * C::EPI_STAGE_WORDS;
            const bool add_b = add_bias;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = __uint_as_float(r[j]);
              if (add_b && col0 + j < g.N) x += __bfloat162float(g.bias[col0 + j]);
              st[lane * 33 + j] = x;
            }
            __syncwarp();
            const int rr = lane >> 3, cc = (lane & 7) * 4;
            if (col0 + cc < g.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int lr = i * 4 + rr;
                const int grow = m0 + q * 32 + lr;
                if (grow < m_limit) {
                  const float* sp = st + lr * 33 + cc;
                  float* base;
                  if (g.c_rows_per_peer > 0)
                    base = reinterpret_cast<float*>(g.c_peers[grow / g.c_rows_per_peer]) +
                           static_cast<long long>(grow % g.c_rows_per_peer) * g.ldc;
                  else
                    base = reinterpret_cast<float*>(g.C) + static_cast<long long>(grow) * g.ldc;
                  red_add4(base + col0 + cc, sp[0], sp[1], sp[2], sp[3]);
                }
              }
            }
            __syncwarp();
          }
        }
      }
      if constexpr (EPI == EPI_LSE) {
        if (row < m_limit) {
          const int part_idx = GATHER == 1 ? chunk : n0 / BN;
          float* pp = g.part + (static_cast<long long>(part_idx) * g.M + row) * 2;
          pp[0] = m_run;
          pp[1] = l_run;
          if (lbl) {
            if (pos_val != 0.f) atomicAdd(&g.pos[row], pos_val);  // several column tiles add up
          } else if (pos_here) {
            g.pos[row] = pos_val;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

int g_num_sms = 0;

int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int A_MN, int B_MN, int BN, typename OutT, int EPI = EPI_STORE, int GATHER = 0,
          int F8 = 0>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& g, int grid,
           cudaStream_t stream, const CUtensorMap* tmA2 = nullptr,
           const CUtensorMap* tmB2 = nullptr) {
  using C = Cfg<BN, epi_warps<EPI, GATHER, F8>(), F8>;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, BN, OutT, EPI, GATHER, F8>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured = true;
  }
  kern<<<grid, gemm_threads<EPI, GATHER, F8>(), C::SMEM_BYTES, stream>>>(
      tmA, tmB, tmA2 != nullptr ? *tmA2 : tmA, tmB2 != nullptr ? *tmB2 : tmB, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Split of the contraction for a product whose output tiles alone do not fill the SMs evenly
// (the weight gradients: few tiles, a contraction over all tokens). Cost model in units of one
// k-block of tensor-core work: every wave of `sms` items takes max(kb_per, kEpi), where kEpi is
// the fp32 reduction epilogue of an item, hidden behind the next item's main loop only when that
// is at least as long. More splits mean more reduction traffic, so a candidate must win by 2 %.
int auto_splits(long long tiles, int kb_total, int sms) {
  constexpr int kEpi = 32, kMinKb = 32;
  if (kb_total < 2 * kMinKb) return 1;
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 32; ++s) {
    const int kb_per = (kb_total + s - 1) / s;
    if (s > 1 && kb_per < kMinKb) break;
    const int se = (kb_total + kb_per - 1) / kb_per;
    const long long items = tiles * se;
    const long long waves = (items + sms - 1) / sms;
    const double cost = double(waves) * (kb_per > kEpi ? kb_per : kEpi) + kEpi;
    if (cost < best_cost * 0.98) {
      best = se;
      best_cost = cost;
    }
  }
  return best;
}

template <int A_MN, int B_MN, int BN>
int launch_out(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& g, int grid,
               bool out_fp32, cudaStream_t stream) {
  return out_fp32 ? launch<A_MN, B_MN, BN, float>(tmA, tmB, g, grid, stream)
                  : launch<A_MN, B_MN, BN, __nv_bfloat16>(tmA, tmB, g, grid, stream);
}

}  // namespace
}  // namespace lb

// C = A · B^T with bf16 operands.
//   a_mn = 0: A is [M, K] row-major with row stride lda; a_mn = 1: A is stored [K, M], stride lda.
//   b_mn = 0: B is [N, K] row-major with row stride ldb; b_mn = 1: B is stored [K, N], stride ldb.
//   out_fp32: C is float (else bf16), row stride ldc. accumulate (fp32 only): C += product.
//   splits: split of K (fp32 accumulate only; >1 forces accumulate; 0 = chosen here, see
//   auto_splits: the caller must then pass accumulate = 1 and an initialised C).
//   bn: 0 = auto, 128 or 256.
// All leading dimensions and N must be multiples of 8 elements; base pointers 16-byte aligned.
// Returns 0 or a negative code; device-side timeouts are reported through *status (device int).
extern "C" int lb_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                                 int out_fp32, int accumulate, int splits, int* status,
                                 void* stream_);
extern "C" int lb_gemm_bf16_2cta_ext(const void* A, const void* B, const void* A2, const void* B2,
                                     void* C, int M, int N, int K, int K2, long long lda,
                                     long long ldb, long long lda2, long long ldb2, long long ldc,
                                     int b_mn, int* status, void* stream_);
extern "C" int lb_gemm_bf16_2cta_push(const void* A, const void* B, const void* const* c_peers,
                                      int world, int rows_per_peer, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int a_mn,
                                      int b_mn, int* status, void* stream_);
extern "C" int lb_gemm_bf16_2cta_ag(const void* const* a_peers, void* a_all, const void* B, void* C,
                                    int rows_local, int world, int rank, int N, int K,
                                    long long lda, long long ldb, long long ldc, int b_mn,
                                    unsigned* flags, unsigned* counter, unsigned epoch,
                                    int* status, void* stream_);
extern "C" int lb_gemm_2cta_pairs();

// The plain products (no bias, no scatter to other GPUs, at least one 256 x 256 tile), those with
// a second operand pair appended to the contraction and the bf16 accumulation into a local buffer
// run on the CTA-pair kernel of gemm_2cta.cu: the same speed per kernel within a few percent, at less shared-memory
// traffic per FLOP, which under the power cap is worth about 3 % of a training step.
// LSET_B200_GEMM_2CTA=0 (or lb_gemm_use_2cta(0)) keeps everything on the one-CTA kernel.
static int g_use_2cta = -1;
static int use_2cta() {
  if (g_use_2cta < 0) {
    const char* e = getenv("LSET_B200_GEMM_2CTA");
    g_use_2cta = e != nullptr ? (atoi(e) != 0) : 1;
  }
  return g_use_2cta;
}
// v = 0 / 1 switches the CTA-pair kernel off / on for this process; v < 0 only queries.
extern "C" int lb_gemm_use_2cta(int v) {
  if (v >= 0) g_use_2cta = v != 0;
  return use_2cta();
}

static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K,
                          long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                          int out_fp32, int accumulate, const void* bias, int splits, int bn,
                          int* status, void* stream_, const void* const* c_peers, int c_world,
                          int c_rows_per_peer, int c_store = 0) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -4;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3)) return -3;
  if (!out_fp32 && (ldc & 7)) return -3;
  const bool scatter = c_peers != nullptr && c_rows_per_peer > 0;
  if (!out_fp32 && !scatter && (accumulate || splits > 1)) return -5;
  if (!out_fp32 && scatter) splits = 1;  // bf16 reduce-scatter: one pass over the contraction

  const int tiles_m = (M + BM - 1) / BM;
  const int sms = num_sms();
  if (use_2cta() && bias == nullptr && scatter && c_world == 1 && !c_store && !out_fp32 &&
      bn == 0 &&
      M >= 256 && N >= 256)  // "scatter" to this GPU only: C += A · op(B) in bf16
    return lb_gemm_bf16_2cta(A, B, const_cast<void*>(c_peers[0]), M, N, K, lda, ldb, ldc, a_mn,
                             b_mn, 0, 1, 1, status, stream_);
  if (use_2cta() && bias == nullptr && scatter && c_store && !out_fp32 && bn == 0 && M >= 256 &&
      N >= 256 && c_world <= 8)  // reduce-scatter by slots: rows stored into the owners' areas
    return lb_gemm_bf16_2cta_push(A, B, c_peers, c_world, c_rows_per_peer, M, N, K, lda, ldb, ldc,
                                  a_mn, b_mn, status, stream_);
  if (use_2cta() && bias == nullptr && !scatter && bn == 0 && M >= 256 && N >= 256) {
    int s2 = splits;
    if (s2 == 0) {
      const long long t2 = 1LL * ((M + 255) / 256) * ((N + 255) / 256);
      s2 = (out_fp32 && accumulate)
               ? auto_splits(t2, (K + BK - 1) / BK, lb_gemm_2cta_pairs()) : 1;
    }
    return lb_gemm_bf16_2cta(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, s2,
                             status, stream_);
  }
  if (bn != 128 && bn != 256) {
    auto eff = [&](int b) {
      const long long t = 1LL * tiles_m * ((N + b - 1) / b);
      const long long waves = (t + sms - 1) / sms;
      return double(t) * b / double(waves * sms);  // useful columns per SM-slot
    };
    bn = (N > 128 && eff(256) >= eff(128)) ? 256 : 128;
  }
  const int tiles_n = (N + bn - 1) / bn;
  const int kb_total = (K + BK - 1) / BK;
  if (splits == 0)
    splits = (out_fp32 && accumulate) ? auto_splits(1LL * tiles_m * tiles_n, kb_total, sms) : 1;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  int kb_per = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per - 1) / kb_per;
  if (splits > 1) accumulate = 1;

  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn)
    rc = make_tmap_2d(&tmA, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, true);
  else
    rc = make_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true);
  else
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, bn, true);
  if (rc) return rc;

  GemmArgs g{};
  g.raster_m_fast = tiles_n > tiles_m ? 1 : 0;
  g.M = M;
  g.N = N;
  g.K = K;
  g.C = C;
  g.ldc = ldc;
  g.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  g.accumulate = accumulate;
  g.splits = splits;
  g.kb_per_split = kb_per;
  g.status = status;
  if (c_peers != nullptr && c_rows_per_peer > 0) {
    if (c_world > 8) return -3;
    for (int i = 0; i < c_world; ++i) g.c_peers[i] = const_cast<void*>(c_peers[i]);
    g.c_rows_per_peer = c_rows_per_peer;
    g.c_store = c_store;
    g.accumulate = 1;
  }
  const long long total = 1LL * tiles_m * tiles_n * splits;
  const int grid = (int)(total < sms ? total : sms);
  const bool f32 = out_fp32 != 0;

#define LB_DISPATCH(AM, BMJ)                                                        \
  (bn == 256 ? launch_out<AM, BMJ, 256>(tmA, tmB, g, grid, f32, stream)             \
             : launch_out<AM, BMJ, 128>(tmA, tmB, g, grid, f32, stream))
  if (!a_mn && !b_mn) return LB_DISPATCH(0, 0);
  if (!a_mn && b_mn) return LB_DISPATCH(0, 1);
  if (a_mn && b_mn) return LB_DISPATCH(1, 1);
  return LB_DISPATCH(1, 0);
#undef LB_DISPATCH
}

extern "C" int lb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                            int out_fp32, int accumulate, const void* bias, int splits, int bn,
                            int* status, void* stream_) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, bias,
                        splits, bn, status, stream_, nullptr, 0, 0);
}

// C = (A · B^T) ∘ (sa ⊗ sb) with 8-bit float operands (tcgen05 kind::f8f6f4, fp32 accumulation).
//   A: [M, K] row-major bytes, row stride lda; B: [N, K] row-major bytes, row stride ldb (both
//   K-major; lda, ldb multiples of 16). a_e5m2 / b_e5m2: 0 = e4m3, 1 = e5m2.
//   sa / sb: dequantisation factors (device fp32), one per row of A / row of B when the stride is 1,
//   one for the whole tensor when it is 0.
//   out_fp32, accumulate, splits, bias, bn: as in lb_gemm_bf16.
extern "C" int lb_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K,
                           long long lda, long long ldb, long long ldc, int a_e5m2, int b_e5m2,
                           const float* sa, int sa_stride, const float* sb, int sb_stride,
                           int out_fp32, int accumulate, const void* bias, int splits, int bn,
                           int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -4;
  if ((N & 7) || (lda & 15) || (ldb & 15) || (ldc & 3)) return -3;
  if (!out_fp32 && (ldc & 7)) return -3;
  if (sa == nullptr || sb == nullptr) return -3;
  if (!out_fp32 && (accumulate || splits > 1)) return -5;
  constexpr int BKE = 2 * BK;
  const int tiles_m = (M + BM - 1) / BM;
  const int sms = num_sms();
  if (bn != 128 && bn != 256) {
    auto eff = [&](int b) {
      const long long t = 1LL * tiles_m * ((N + b - 1) / b);
      const long long waves = (t + sms - 1) / sms;
      return double(t) * b / double(waves * sms);
    };
    bn = (N > 128 && eff(256) >= eff(128)) ? 256 : 128;
  }
  const int tiles_n = (N + bn - 1) / bn;
  const int kb_total = (K + BKE - 1) / BKE;
  if (splits == 0)
    splits = (out_fp32 && accumulate) ? auto_splits(1LL * tiles_m * tiles_n, kb_total, sms) : 1;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  const int kb_per = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per - 1) / kb_per;
  if (splits > 1) accumulate = 1;

  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, 1, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BKE, BM, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BKE, bn, true);
  if (rc) return rc;

  GemmArgs g{};
  g.raster_m_fast = tiles_n > tiles_m ? 1 : 0;
  g.M = M;
  g.N = N;
  g.K = K;
  g.C = C;
  g.ldc = ldc;
  g.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  g.accumulate = accumulate;
  g.splits = splits;
  g.kb_per_split = kb_per;
  g.status = status;
  g.f8_sa = sa;
  g.f8_sb = sb;
  g.f8_sa_stride = sa_stride ? 1 : 0;
  g.f8_sb_stride = sb_stride ? 1 : 0;
  g.f8_a_e5m2 = a_e5m2 ? 1 : 0;
  g.f8_b_e5m2 = b_e5m2 ? 1 : 0;
  const long long total = 1LL * tiles_m * tiles_n * splits;
  const int grid = (int)(total < sms ? total : sms);
  if (bn == 256)
    return out_fp32 ? launch<0, 0, 256, float, EPI_STORE, 0, 1>(tmA, tmB, g, grid, stream)
                    : launch<0, 0, 256, __nv_bfloat16, EPI_STORE, 0, 1>(tmA, tmB, g, grid, stream);
  return out_fp32 ? launch<0, 0, 128, float, EPI_STORE, 0, 1>(tmA, tmB, g, grid, stream)
                  : launch<0, 0, 128, __nv_bfloat16, EPI_STORE, 0, 1>(tmA, tmB, g, grid, stream);
}

// GEMM fused with a reduce-scatter: C has M = world * rows_per_peer rows; row r is added (fp32
// red.global.add over NVLink) into rank r / rows_per_peer's buffer c_peers[...] at local row
// r % rows_per_peer. The buffers must be zeroed (or hold the value to accumulate onto) beforehand.
extern "C" int lb_gemm_bf16_scatter(const void* A, const void* B, const void* const* c_peers,
                                    int world, int rows_per_peer, int M, int N, int K,
                                    long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                                    int splits, int bn, int* status, void* stream_) {
  if (M != world * rows_per_peer) return -3;
  return gemm_bf16_impl(A, B, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, 1, 1, nullptr, splits, bn,
                        status, stream_, c_peers, world, rows_per_peer);
}


// ------------------------------------------------------------------------------------------------
// Contrastive loss on the GEMM: scores s = (Q · Kᵀ) / temperature never leave tensor memory.
//   forward   every 128 x BN tile folds its scores into a per-row running (max, sum) pair and picks
//             out the target column; a small kernel merges the pairs into the row LSE and the loss.
//   backward  the same product is recomputed and the epilogue writes W = (softmax − onehot) · coef
//             in bf16; dQ = W · K and dK = Wᵀ · Q are two more calls of the plain GEMM above.
// Replaces the reference's Triton / CUDA fused loss kernels for the diagonal-target case
// (lset/kernels/loss.py:186-289,402-495; lset/kernels/experimental/csrc/loss_sm100.cu:340-643)
// without an int8 label matrix.
// ------------------------------------------------------------------------------------------------
namespace lb {
namespace {

// lse[r] = ln(sum_j exp(s_rj)); loss_sum += sum_r (lse[r] − pos[r]) (one atomicAdd per block).
__global__ void __launch_bounds__(256)
    lse_merge_kernel(const float* __restrict__ part, int tiles_n, int M, const float* __restrict__ pos,
                     float* __restrict__ lse, float* __restrict__ loss_sum) {
  __shared__ float sred[8];
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  float contrib = 0.f;
  if (r < M) {
    float m = -INFINITY, l = 0.f;
    for (int t = 0; t < tiles_n; ++t) {
      const float mt = part[(1LL * t * M + r) * 2], lt = part[(1LL * t * M + r) * 2 + 1];
      const float mn = fmaxf(m, mt);
      if (mn > -INFINITY) l = l * exp2f(m - mn) + lt * exp2f(mt - mn);
      m = mn;
    }
    const float v = (m + log2f(l)) * 0.6931471805599453f;
    lse[r] = v;
    contrib = v - pos[r];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = contrib;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sred[i];
    atomicAdd(loss_sum, s);
  }
}

// Label-matrix variant: per_q = lse − row_scale · pos; loss_sum += sum_r row_w[r] · per_q. Rows
// without a valid column get lse = 0 (their row_w is 0).
__global__ void __launch_bounds__(256)
    lse_merge_label_kernel(const float* __restrict__ part, int tiles_n, int M,
                           const float* __restrict__ pos, const float* __restrict__ row_scale,
                           const float* __restrict__ row_w, float* __restrict__ lse,
                           float* __restrict__ loss_sum) {
  __shared__ float sred[8];
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  float contrib = 0.f;
  if (r < M) {
    float m = -INFINITY, l = 0.f;
    for (int t = 0; t < tiles_n; ++t) {
      const float mt = part[(1LL * t * M + r) * 2], lt = part[(1LL * t * M + r) * 2 + 1];
      const float mn = fmaxf(m, mt);
      if (mn > -INFINITY) l = l * exp2f(m - mn) + lt * exp2f(mt - mn);
      m = mn;
    }
    const float v = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : 0.f;
    lse[r] = v;
    const float w = row_w[r];
    if (w != 0.f) contrib = w * (v - row_scale[r] * pos[r]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
  if ((threadIdx.x & 31) == 0) sred[threadIdx.x >> 5] = contrib;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sred[i];
    atomicAdd(loss_sum, s);
  }
}

int loss_tile_bn(int M, int N) {
  (void)M;
  return N > 128 ? 256 : 128;
}

int prep_loss(const void* Q, const void* Kd, int M, int N, int D, long long ldq, long long ldk,
              int bn, CUtensorMap* tmA, CUtensorMap* tmB, GemmArgs* g, int* grid) {
  if (M <= 0 || N <= 0 || D <= 0) return -4;
  if ((ldq & 7) || (ldk & 7)) return -3;
  int rc = make_tmap_2d(tmA, Q, 2, (uint64_t)D, (uint64_t)M, (uint64_t)ldq * 2, BK, BM, true);
  if (rc) return rc;
  rc = make_tmap_2d(tmB, Kd, 2, (uint64_t)D, (uint64_t)N, (uint64_t)ldk * 2, BK, bn, true);
  if (rc) return rc;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
  *g = GemmArgs{};
  g->M = M;
  g->N = N;
  g->K = D;
  g->splits = 1;
  g->kb_per_split = (D + BK - 1) / BK;
  g->raster_m_fast = tiles_n > tiles_m ? 1 : 0;
  const long long total = 1LL * tiles_m * tiles_n;
  const int sms = num_sms();
  *grid = (int)(total < sms ? total : sms);
  return 0;
}

}  // namespace
}  // namespace lb

// Number of floats of scratch that lb_infonce_fwd needs for M queries against N passages.
// Same with bf16 accumulators in the owners' buffers (red.global.add on packed bf16x2): half the
// NVLink bytes of the fp32 form, for activations whose reduce-scatter would be bf16 anyway.
extern "C" int lb_gemm_bf16_scatter16(const void* A, const void* B, const void* const* c_peers,
                                      int world, int rows_per_peer, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int a_mn,
                                      int b_mn, int bn, int* status, void* stream_) {
  if (M != world * rows_per_peer) return -3;
  return gemm_bf16_impl(A, B, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, 0, 1, nullptr, 1, bn,
                        status, stream_, c_peers, world, rows_per_peer);
}

// Reduce-scatter without reductions on the wire: as lb_gemm_bf16_scatter16, but every output row
// is *stored* (plain 16-byte stores) at local row r % rows_per_peer of c_peers[r / rows_per_peer].
// The caller passes, for every destination rank, the address of the slot that belongs to this
// (source) rank inside that rank's buffer of `world` slots; the owner sums its slots afterwards
// (lb_take_sum). Stores pack into larger NVLink packets than reductions do, nothing has to be
// cleared, and the sum has a fixed order.
extern "C" int lb_gemm_bf16_push16(const void* A, const void* B, const void* const* c_peers,
                                   int world, int rows_per_peer, int M, int N, int K, long long lda,
                                   long long ldb, long long ldc, int a_mn, int b_mn, int bn,
                                   int* status, void* stream_) {
  if (M != world * rows_per_peer) return -3;
  return gemm_bf16_impl(A, B, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, 0, 1, nullptr, 1, bn,
                        status, stream_, c_peers, world, rows_per_peer, 1);
}

// Gated-MLP input projection with the activation in the epilogue: gate_up [M, 2I] = A · Wᵀ for the
// fused weight W = [gate; up] ([2I, K]) and h [M, I] = act(gate) * up, act = SiLU (kind 0) or
// tanh-GELU (kind 1). gate_up is written too: the backward of the activation needs it.
extern "C" int lb_gemm_glu(const void* A, const void* W, void* gate_up, void* h, int M, int I, int K,
                           long long lda, long long ldw, long long ld_gu, long long ld_h, int kind,
                           int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || I <= 0) return 0;
  if (K <= 0) return -4;
  if ((I & 7) || (lda & 7) || (ldw & 7) || (ld_gu & 7) || (ld_h & 7)) return -3;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, W, 2, (uint64_t)K, (uint64_t)2 * I, (uint64_t)ldw * 2, BK, 128, true);
  if (rc) return rc;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (I + 127) / 128;
  GemmArgs g{};
  g.raster_m_fast = tiles_n > tiles_m ? 1 : 0;
  g.M = M;
  g.N = I;
  g.K = K;
  g.C = gate_up;
  g.ldc = ld_gu;
  g.splits = 1;
  g.kb_per_split = (K + BK - 1) / BK;
  g.glu_I = I;
  g.glu_h = h;
  g.ld_h = ld_h;
  g.glu_kind = kind;
  g.status = status;
  const long long total = 1LL * tiles_m * tiles_n;
  const int sms = num_sms();
  const int grid = (int)(total < sms ? total : sms);
  return launch<0, 0, 256, __nv_bfloat16, EPI_GLU>(tmA, tmB, g, grid, stream);
}

// C[M, N] (bf16) = A · op(B) + A2 · op(B2) (+ bias) in one pass over the accumulator: the k-blocks
// of the second pair are appended to the contraction. A [M, K] and A2 [M, K2] are K-major;
// op(B) = Bᵀ for B [N, K], B2 [N, K2] (b_mn = 0) or B for B [K, N], B2 [K2, N] (b_mn = 1).
// K2 is a multiple of 8 (a LoRA rank); its k-block is zero-filled by TMA up to 64.
extern "C" int lb_gemm_bf16_ext(const void* A, const void* B, const void* A2, const void* B2,
                                void* C, int M, int N, int K, int K2, long long lda,
                                long long ldb, long long lda2, long long ldb2, long long ldc,
                                int b_mn, const void* bias, int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K2 <= 0) return -4;
  if ((N & 7) || (K2 & 7) || (lda & 7) || (ldb & 7) || (lda2 & 7) || (ldb2 & 7) || (ldc & 7))
    return -3;
  if (use_2cta() && bias == nullptr && M >= 256 && N >= 256)
    return lb_gemm_bf16_2cta_ext(A, B, A2, B2, C, M, N, K, K2, lda, ldb, lda2, ldb2, ldc, b_mn,
                                 status, stream_);
  const int tiles_m = (M + BM - 1) / BM;
  const int bn = N > 128 ? 256 : 128;
  const int tiles_n = (N + bn - 1) / bn;
  CUtensorMap tmA, tmB, tmA2, tmB2;
  int rc = make_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmA2, A2, 2, (uint64_t)K2, (uint64_t)M, (uint64_t)lda2 * 2, BK, BM, true);
  if (rc) return rc;
  if (b_mn) {
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB2, B2, 2, (uint64_t)N, (uint64_t)K2, (uint64_t)ldb2 * 2, 64, BK, true);
  } else {
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, bn, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB2, B2, 2, (uint64_t)K2, (uint64_t)N, (uint64_t)ldb2 * 2, BK, bn, true);
  }
  if (rc) return rc;
  GemmArgs g{};
  g.raster_m_fast = tiles_n > tiles_m ? 1 : 0;
  g.M = M;
  g.N = N;
  g.K = K;
  g.C = C;
  g.ldc = ldc;
  g.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  g.splits = 1;
  g.kb_ext = (K2 + BK - 1) / BK;
  g.kb_per_split = (K + BK - 1) / BK + g.kb_ext;
  g.status = status;
  const long long total = 1LL * tiles_m * tiles_n;
  const int sms = num_sms();
  const int grid = (int)(total < sms ? total : sms);
  if (b_mn)
    return bn == 256
               ? launch<0, 1, 256, __nv_bfloat16>(tmA, tmB, g, grid, stream, &tmA2, &tmB2)
               : launch<0, 1, 128, __nv_bfloat16>(tmA, tmB, g, grid, stream, &tmA2, &tmB2);
  return bn == 256 ? launch<0, 0, 256, __nv_bfloat16>(tmA, tmB, g, grid, stream, &tmA2, &tmB2)
                   : launch<0, 0, 128, __nv_bfloat16>(tmA, tmB, g, grid, stream, &tmA2, &tmB2);
}

extern "C" long long lb_infonce_scratch_floats(int M, int N) {
  const int bn = lb::loss_tile_bn(M, N);
  return 2LL * ((N + bn - 1) / bn) * M + M;
}

// q: [M, D] bf16 (row stride ldq), k: [N, D] bf16 (row stride ldk). The positive of query r is
// passage r + target_offset. Outputs: lse [M] fp32, loss_sum (device scalar, += sum_r (lse − pos)).
// scratch: lb_infonce_scratch_floats(M, N) floats.
extern "C" int lb_infonce_fwd(const void* q, long long ldq, const void* k, long long ldk, int M,
                              int N, int D, float inv_temperature, long long target_offset,
                              float* scratch, float* lse, float* loss_sum, int* status,
                              void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int bn = loss_tile_bn(M, N);
  CUtensorMap tmA, tmB;
  GemmArgs g;
  int grid;
  if (int rc = prep_loss(q, k, M, N, D, ldq, ldk, bn, &tmA, &tmB, &g, &grid)) return rc;
  const int tiles_n = (N + bn - 1) / bn;
  g.scale = inv_temperature;
  g.part = scratch;
  g.pos = scratch + 2LL * tiles_n * M;
  g.target_offset = target_offset;
  g.status = status;
  int rc = bn == 256 ? launch<0, 0, 256, __nv_bfloat16, EPI_LSE>(tmA, tmB, g, grid, stream)
                     : launch<0, 0, 128, __nv_bfloat16, EPI_LSE>(tmA, tmB, g, grid, stream);
  if (rc) return rc;
  lse_merge_kernel<<<(M + 255) / 256, 256, 0, stream>>>(g.part, tiles_n, M, g.pos, lse, loss_sum);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// W[r, c] = (exp(s_rc − lse[r]) − [c == r + target_offset]) * coef[0], bf16, row stride ldw
// (multiple of 8, >= N). coef: device scalar (upstream gradient / (temperature * denominator)).
extern "C" int lb_infonce_pgrad(const void* q, long long ldq, const void* k, long long ldk, int M,
                                int N, int D, float inv_temperature, long long target_offset,
                                const float* lse, const float* coef, void* W, long long ldw,
                                int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if ((N & 7) || (ldw & 7)) return -3;
  const int bn = loss_tile_bn(M, N);
  CUtensorMap tmA, tmB;
  GemmArgs g;
  int grid;
  if (int rc = prep_loss(q, k, M, N, D, ldq, ldk, bn, &tmA, &tmB, &g, &grid)) return rc;
  g.scale = inv_temperature;
  g.lse = lse;
  g.coef = coef;
  g.C = W;
  g.ldc = ldw;
  g.target_offset = target_offset;
  g.status = status;
  return bn == 256 ? launch<0, 0, 256, __nv_bfloat16, EPI_PGRAD>(tmA, tmB, g, grid, stream)
                   : launch<0, 0, 128, __nv_bfloat16, EPI_PGRAD>(tmA, tmB, g, grid, stream);
}

// Label-matrix contrastive loss (multi-positive NCE and soft-label cross-entropy) on the same
// streaming kernels: loss_sum += sum_r row_w[r] · (LSE_{valid c} s_rc − row_scale[r] · sum_c t_rc s_rc)
// with t = max(label, 0) (tw == nullptr) or t = tw. labels: int8 [M, ld_labels], ld_labels % 32 == 0,
// >= N, padded with a negative value; tw: fp32 [M, ld_tw] or nullptr, same padding rule (zeros).
// loss_mode 1 (multi-positive NCE): lse[r] is the LSE over the negatives (label == 0) only and
// loss_sum is not meaningful; the caller forms the loss from lse and the positives' scores.
// scratch: lb_infonce_scratch_floats(M, N) floats.
extern "C" int lb_label_loss_fwd(const void* q, long long ldq, const void* k, long long ldk, int M,
                                 int N, int D, float inv_temperature, const void* labels,
                                 long long ld_labels, const float* tw, long long ld_tw,
                                 const float* row_scale, const float* row_w, int loss_mode,
                                 float* scratch, float* lse, float* loss_sum, int* status,
                                 void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (labels == nullptr || (ld_labels & 31) || ld_labels < N) return -3;
  if (tw != nullptr && ((ld_tw & 31) || ld_tw < N)) return -3;
  const int bn = loss_tile_bn(M, N);
  CUtensorMap tmA, tmB;
  GemmArgs g;
  int grid;
  if (int rc = prep_loss(q, k, M, N, D, ldq, ldk, bn, &tmA, &tmB, &g, &grid)) return rc;
  const int tiles_n = (N + bn - 1) / bn;
  g.scale = inv_temperature;
  g.part = scratch;
  g.pos = scratch + 2LL * tiles_n * M;
  g.labels = static_cast<const signed char*>(labels);
  g.ld_labels = ld_labels;
  g.tw = tw;
  g.ld_tw = ld_tw;
  g.row_scale = row_scale;
  g.row_w = row_w;
  g.loss_mode = loss_mode;
  g.status = status;
  if (cudaMemsetAsync(g.pos, 0, sizeof(float) * M, stream) != cudaSuccess) return -12;
  int rc = bn == 256 ? launch<0, 0, 256, __nv_bfloat16, EPI_LSE>(tmA, tmB, g, grid, stream)
                     : launch<0, 0, 128, __nv_bfloat16, EPI_LSE>(tmA, tmB, g, grid, stream);
  if (rc) return rc;
  lse_merge_label_kernel<<<(M + 255) / 256, 256, 0, stream>>>(g.part, tiles_n, M, g.pos, row_scale,
                                                             row_w, lse, loss_sum);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// W[r, c] = ([label_rc >= 0] · exp(s_rc − lse[r]) − row_scale[r] · t_rc) · row_w[r] · coef[0], bf16
// (loss_mode 0); loss_mode 1: positives (sigmoid(s − lse) − 1) · row_w · coef, negatives
// exp(s − lse) · row_scale · row_w · coef.
extern "C" int lb_label_loss_pgrad(const void* q, long long ldq, const void* k, long long ldk, int M,
                                   int N, int D, float inv_temperature, const void* labels,
                                   long long ld_labels, const float* tw, long long ld_tw,
                                   const float* row_scale, const float* row_w, int loss_mode,
                                   const float* lse, const float* coef, void* W, long long ldw,
                                   int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if ((N & 7) || (ldw & 7)) return -3;
  if (labels == nullptr || (ld_labels & 31) || ld_labels < N) return -3;
  if (tw != nullptr && ((ld_tw & 31) || ld_tw < N)) return -3;
  const int bn = loss_tile_bn(M, N);
  CUtensorMap tmA, tmB;
  GemmArgs g;
  int grid;
  if (int rc = prep_loss(q, k, M, N, D, ldq, ldk, bn, &tmA, &tmB, &g, &grid)) return rc;
  g.scale = inv_temperature;
  g.lse = lse;
  g.coef = coef;
  g.C = W;
  g.ldc = ldw;
  g.labels = static_cast<const signed char*>(labels);
  g.ld_labels = ld_labels;
  g.tw = tw;
  g.ld_tw = ld_tw;
  g.row_scale = row_scale;
  g.row_w = row_w;
  g.loss_mode = loss_mode;
  g.status = status;
  return bn == 256 ? launch<0, 0, 256, __nv_bfloat16, EPI_PGRAD>(tmA, tmB, g, grid, stream)
                   : launch<0, 0, 128, __nv_bfloat16, EPI_PGRAD>(tmA, tmB, g, grid, stream);
}

// Cross-rank InfoNCE forward: the passages of all `world` ranks (n_local rows each, in symmetric
// buffers k_peers[r]) are pulled into k_all ([world * n_local, D], local) by two extra warps per
// CTA while the tensor-core tiles consume them in pull order, own rank first. The caller orders
// the launch after every rank has written its passages and keeps k_all for the backward.
// flags: [world * ceil(n_local / 256)] zero-initialised once; counter: one u32; epoch: 1, 2, 3, …
// on successive calls that use these flags (a flag counts the 16-row items pulled so far).
// part/lse layout as in lb_infonce_fwd with tiles = world * ceil(n_local / 256).
namespace lb {
namespace {
// Grid of a gather launch: the CTAs that compute tiles plus the copy CTAs in front of them (16 of
// the SMs, more when the product has fewer tiles than SMs). Copy CTAs are only worth their SMs
// when the transfer is a sizeable part of the kernel: pulling `pull_bytes` at ~700 GB/s must take
// more than half of what the product's `flops` take at ~1.4 PFLOP/s. Otherwise (and on a single
// rank) the two pull warps of every computing CTA keep up.
int gather_grid(long long total, int sms, int world, double pull_bytes, double flops,
                int* copy_ctas) {
  const bool comm_heavy = pull_bytes / 700e9 > 0.5 * flops / 1.4e15;
  if (world <= 1 || !comm_heavy) {
    *copy_ctas = 0;
    return (int)(total < sms ? total : sms);
  }
  const int compute = (int)(total < sms - 16 ? total : sms - 16);
  int copy = sms - compute;
  if (copy > 48) copy = 48;
  *copy_ctas = copy;
  return compute + copy;
}
}  // namespace
}  // namespace lb

extern "C" long long lb_infonce_xrank_scratch_floats(int M, int n_local, int world) {
  return 2LL * world * ((n_local + 255) / 256) * M + M;
}

extern "C" int lb_infonce_fwd_xrank(const void* q, long long ldq, const void* const* k_peers,
                                    void* k_all, long long ldk, int M, int n_local, int world,
                                    int rank, int D, float inv_temperature, long long target_offset,
                                    float* scratch, float* lse, float* loss_sum, unsigned* flags,
                                    unsigned* counter, unsigned epoch, int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 1 || world > 8 || (n_local & 7) || (D & 7)) return -3;
  const int N = world * n_local;
  CUtensorMap tmA, tmB;
  GemmArgs g;
  int grid;
  if (int rc = prep_loss(q, k_all, M, N, D, ldq, ldk, 256, &tmA, &tmB, &g, &grid)) return rc;
  const int tiles_per_peer = (n_local + 255) / 256;
  const int chunks = world * tiles_per_peer;
  const long long total = 1LL * ((M + BM - 1) / BM) * chunks;
  const int sms = num_sms();
  grid = gather_grid(total, sms, world, 2.0 * (world - 1) * n_local * D, 2.0 * M * N * D,
                     &g.copy_ctas);
  g.scale = inv_temperature;
  g.part = scratch;
  g.pos = scratch + 2LL * chunks * M;
  g.target_offset = target_offset;
  for (int i = 0; i < world; ++i) g.b_peers[i] = k_peers[i];
  g.b_local = k_all;
  g.ldb_peer = ldk;
  g.n_local = n_local;
  g.world = world;
  g.rank = rank;
  g.flags = flags;
  g.chunk_counter = counter;
  g.epoch = epoch;
  g.status = status;
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), stream) != cudaSuccess) return -12;
  int rc = launch<0, 0, 256, __nv_bfloat16, EPI_LSE, 1>(tmA, tmB, g, grid, stream);
  if (rc) return rc;
  lse_merge_kernel<<<(M + 255) / 256, 256, 0, stream>>>(g.part, chunks, M, g.pos, lse, loss_sum);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// All-gather fused into a GEMM (tensor-parallel column layers and the input-gradient of row
// layers): C[world * rows_local, N] = A_all · Bᵀ where A_all's rows are spread over `world` ranks
// (a_peers[r]: rank r's [rows_local, K] bf16 slice in symmetric memory). Two extra warps per CTA
// pull the peers' rows into a_all (local, [world * rows_local, K]; the caller has already copied
// its own slice there) while the tensor-core tiles consume them in pull order, own rank first.
// a_all is complete when the kernel ends, so the backward can reuse it. b_mn as in lb_gemm_bf16.
// flags: [world * ceil(rows_local / 128)] u32, zero-initialised once; epoch: 1, 2, 3, … on
// successive calls that use these flags (a flag counts the 16-row items pulled so far).
extern "C" int lb_gemm_bf16_ag(const void* const* a_peers, void* a_all, const void* B, void* C,
                               int rows_local, int world, int rank, int N, int K, long long lda,
                               long long ldb, long long ldc, int b_mn, const void* bias,
                               unsigned* flags, unsigned* counter, unsigned epoch, int* status,
                               void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 1 || world > 8 || rows_local <= 0 || N <= 0 || K <= 0) return -3;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -3;
  const int M = world * rows_local;
  // Compute-heavy products run on the CTA-pair kernel; where the transfer dominates (many ranks,
  // few output columns) the one-CTA kernel with its copy CTAs stays.
  if (use_2cta() && bias == nullptr && N >= 256 && rows_local >= 256 &&
      !(2.0 * (world - 1) * rows_local * K / 700e9 > 0.5 * 2.0 * M * N * K / 1.4e15))
    return lb_gemm_bf16_2cta_ag(a_peers, a_all, B, C, rows_local, world, rank, N, K, lda, ldb, ldc,
                                b_mn, flags, counter, epoch, status, stream_);
  const int bn = N > 128 ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, a_all, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true);
  else
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, bn, true);
  if (rc) return rc;
  GemmArgs g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.C = C;
  g.ldc = ldc;
  g.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  g.splits = 1;
  g.kb_per_split = (K + BK - 1) / BK;
  for (int i = 0; i < world; ++i) g.b_peers[i] = a_peers[i];
  g.b_local = a_all;
  g.ldb_peer = lda;
  g.n_local = rows_local;
  g.world = world;
  g.rank = rank;
  g.flags = flags;
  g.chunk_counter = counter;
  g.epoch = epoch;
  g.status = status;
  const int tiles_per_peer = (rows_local + BM - 1) / BM;
  const long long total = 1LL * world * tiles_per_peer * ((N + bn - 1) / bn);
  const int sms = num_sms();
  const int grid = gather_grid(total, sms, world, 2.0 * (world - 1) * rows_local * K,
                               2.0 * M * N * K, &g.copy_ctas);
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), stream) != cudaSuccess) return -12;
  if (b_mn)
    return bn == 256 ? launch<0, 1, 256, __nv_bfloat16, EPI_STORE, 2>(tmA, tmB, g, grid, stream)
                     : launch<0, 1, 128, __nv_bfloat16, EPI_STORE, 2>(tmA, tmB, g, grid, stream);
  return bn == 256 ? launch<0, 0, 256, __nv_bfloat16, EPI_STORE, 2>(tmA, tmB, g, grid, stream)
                   : launch<0, 0, 128, __nv_bfloat16, EPI_STORE, 2>(tmA, tmB, g, grid, stream);
}
