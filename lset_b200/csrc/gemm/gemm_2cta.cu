// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): C[M,N] (+)= A · Bᵀ, one 256 x 256 tile per pair.
//
// Two CTAs of a 2-CTA cluster (one SM each) work on one tile. CTA r of the pair stages its own
// 128 rows of A and its own 128 of the tile's 256 rows of B; one thread of the leader CTA (rank 0)
// issues tcgen05.mma.cta_group::2 with M = 256, N = 256, which reads A from both CTAs' shared
// memory (rows 0..127 from the leader, 128..255 from the peer) and both halves of B, and leaves
// rows 128 r .. 128 r + 127 of the fp32 accumulator in CTA r's tensor memory. Against the
// one-CTA kernel (gemm_bf16.cu, 128 x 256 tiles) every CTA stages and reads 32 KB instead of 48 KB
// of operands per 64 elements of contraction depth for the same tensor-core work, which is what the kernel spends
// its power on when the clock is power-limited.
//
//   warp 0      TMA producer (own A rows, own half of B, into this CTA's shared memory; the loads
//               of both CTAs complete on the leader's barrier)
//   warp 1      leader: MMA issuer
//   warps 2-9   epilogue: drain this CTA's 128 x 256 accumulator (two accumulators in TMEM, so the
//               next tile's main loop runs meanwhile)
//
// Barriers. full[s] (leader): armed by the leader's producer with the bytes of both CTAs' loads of
// stage s; the peer's loads name it as their completion barrier (the cta_group::2 form of the TMA
// load allows a barrier in the partner CTA). empty[s] and tfull[a], in both CTAs: one
// tcgen05.commit per CTA after the MMAs of the stage / tile (the peer's barrier through its
// cluster address). tempty[a] (leader): one arrival per
// epilogue warp of both CTAs. Every wait is bounded; a CTA that gives up reports through the
// status word and still meets its partner at the final cluster barrier, so nothing is left
// waiting.
//
// Operand layouts, split-K and the output forms are those of lb_gemm_bf16 (see gemm_bf16.cu).
#include <cuda_bf16.h>
#include <stdlib.h>

#include "../common/ptx.cuh"
#include "../common/tma_desc.h"

namespace lb {
namespace {

constexpr int BMc = 128;      // rows of A / C per CTA
constexpr int BNp = 256;      // columns of C per pair
constexpr int BNh = 128;      // rows of B staged per CTA
// A stage is 128 deep: per stage the producer, the MMA issuer and the barriers go through one
// hand-over (wait, expect, commit) for eight MMAs. With 64-deep stages (six of them, the same
// bytes in flight) the same kernel was 7-10 % slower: the hand-overs per k-block, not operand
// delivery, were what kept the tensor pipe waiting.
constexpr int BK = 128;       // contraction depth of one pipeline stage
constexpr int kStages = 3;
constexpr int BKT = 64;       // contraction depth of one TMA box of a K-major operand (one
                              // 128-byte swizzle row); a stage holds BK / BKT such boxes
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int A_BYTES = BMc * BK * 2;
constexpr int B_BYTES = BNh * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WORDS = 32 * 33;
constexpr int SMEM_BYTES = kStages * STAGE_BYTES + 1024 + 512 + kEpiWarps * EPI_WORDS * 4;
constexpr int TMEM_COLS = 2 * BNp;

struct Args2 {
  int M, N, K;
  int K2;           // contraction length of the second operand pair (0: none); its k-blocks follow
                    // those of the first pair (rank-r adapter terms appended to the base product)
  void* C;
  long long ldc;
  int accumulate;   // C += result (red.global.add: fp32 scalars or packed bf16 pairs)
  // bf16 output rows stored to other GPUs (reduce-scatter by slots): row r goes to local row
  // r % c_rows_per_peer of c_peers[r / c_rows_per_peer]; 0 rows per peer = plain local C
  void* c_peers[8];
  int c_rows_per_peer;
  // gather of A rows (GATHER kernels): the rows live in `world` ranks' buffers a_peers[r]
  // ([n_local, K], row stride lda_peer elements); two extra warps per CTA pull the peers' rows
  // into a_local ([world * n_local, K], what tmA maps) as items of 16 rows, and flags[c] counts
  // the items of 128-row chunk c that have landed (it only grows: epoch * items after call epoch).
  const void* a_peers[8];
  void* a_local;
  long long lda_peer;
  int n_local, world, rank;
  unsigned* flags;
  unsigned* chunk_counter;
  unsigned epoch;
  int splits, kb_per_split;
  int raster_m_fast;
  int* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `p` (own shared memory) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
// Arrival on a barrier of the partner CTA. No data written by this thread is handed over with it
// (the barriers of this kernel order TMA writes, tensor-core reads and TMEM reads, all of which
// complete before the arrival is issued), so the default semantics are enough; cluster-scope
// acquire / release on the per-stage path costs a fence per k-block in the issuing threads.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load into this CTA's shared memory whose completion bytes are counted on `bar_cluster`,
// a barrier of either CTA of the pair (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tm,
                                                 uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster), "r"(x),
        "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// D (both CTAs' tensor memory) (+)= A (both CTAs' smem) * B (both CTAs' smem); leader thread only.
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once the tcgen05
// operations issued so far have completed: one commit per CTA, the peer's barrier through its
// address in the cluster's shared-memory window.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar, uint32_t peer_rank) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   map_to_cta(bar, peer_rank))
               : "memory");
}

__device__ __forceinline__ void red_add8_bf16(void* dst, const uint4& v) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void red_add4(float* dst, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

constexpr int kPullWarps = 2;

template <int A_MN, int B_MN, typename OutT, int GATHER = 0>
__global__ void __launch_bounds__(kThreads + (GATHER ? 32 * kPullWarps : 0), 1)
    gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmA2,
                     const __grid_constant__ CUtensorMap tmB2, Args2 g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * STAGE_BYTES);
  uint64_t* empty = full + kStages;
  uint64_t* tfull = empty + kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  float* epi_stage = reinterpret_cast<float*>(smem + kStages * STAGE_BYTES + 512);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 2 * kEpiWarps);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (g.K2 > 0) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything arrives on them from afar
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // gather: tiles are laid out rank by rank (a tile never spans two ranks' rows) and visited own
  // rank first, then the peers in the order their rows are pulled
  [[maybe_unused]] const int tiles_per_peer = GATHER ? (g.n_local + 2 * BMc - 1) / (2 * BMc) : 1;
  [[maybe_unused]] const int chunks_per_peer = GATHER ? (g.n_local + BMc - 1) / BMc : 1;
  const int tiles_m = GATHER ? g.world * tiles_per_peer : (g.M + 2 * BMc - 1) / (2 * BMc);
  const int tiles_n = (g.N + BNp - 1) / BNp;
  const int kb_first = (g.K + BK - 1) / BK;                    // k-blocks of the first operand pair
  const int kb_total = kb_first + (g.K2 + BK - 1) / BK;
  const int total = tiles_m * tiles_n * g.splits;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  // m0: first row of this CTA's half of the tile; m_limit: rows from there on that belong to the
  // tile's rank (gather) or exist at all; chunk: flag index of this CTA's rows (gather; -1: none)
  auto decode = [&](int mn, int& m0, int& n0, int& m_limit, int& chunk) {
    if constexpr (GATHER) {
      n0 = (mn % tiles_n) * BNp;
      const int mi = mn / tiles_n;
      const int peer = (g.rank + mi / tiles_per_peer) % g.world;
      const int row_in_peer = (mi % tiles_per_peer) * (2 * BMc) + int(rank) * BMc;
      m0 = peer * g.n_local + row_in_peer;
      m_limit = min(g.M, (peer + 1) * g.n_local);
      chunk = row_in_peer < g.n_local ? peer * chunks_per_peer + row_in_peer / BMc : -1;
    } else {
      m0 = (g.raster_m_fast ? mn % tiles_m : mn / tiles_n) * (2 * BMc) + int(rank) * BMc;
      n0 = (g.raster_m_fast ? mn / tiles_m : mn % tiles_n) * BNp;
      m_limit = g.M;
      chunk = -1;
    }
  };
  constexpr int kPullRows = 16;  // rows per pull item (one warp)
  [[maybe_unused]] auto items_of_chunk = [&](int chunk) {
    const int t = chunk % chunks_per_peer;
    const int rows = min(BMc, g.n_local - t * BMc);
    return (rows + kPullRows - 1) / kPullRows;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < total && ok; tile += npairs) {
        const int split = tile / (tiles_m * tiles_n);
        int m0, n0, m_limit, chunk;
        decode(tile - split * (tiles_m * tiles_n), m0, n0, m_limit, chunk);
        if constexpr (GATHER) {
          if (chunk >= 0) {
            // this CTA's rows of the tile must have been pulled into local memory
            bool landed = false;
            const unsigned want = g.epoch * unsigned(items_of_chunk(chunk));
            const unsigned long long t0 = globaltimer_ns();
            for (unsigned it2 = 0;; ++it2) {
              unsigned v;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];"
                           : "=r"(v)
                           : "l"(g.flags + chunk)
                           : "memory");
              if (v >= want) {
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
        }
        const int nb = n0 + int(rank) * BNh;          // this CTA's half of the B tile
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(kb0 + g.kb_per_split, kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u)) {
            report_status(g.status, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar = map_to_cta(&full[stage], 0);
          const bool second = kb >= kb_first;   // past the first pair: rows beyond K2 read as zero
          const CUtensorMap* ta = second ? &tmA2 : &tmA;
          const CUtensorMap* tb = second ? &tmB2 : &tmB;
          const int kc = (second ? kb - kb_first : kb) * BK;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BMc / 64; ++c)
              tma_load_2d_pair(sa + c * (BK * 128), ta, bar, m0 + 64 * c, kc);
          } else {
#pragma unroll
            for (int h = 0; h < BK / BKT; ++h)
              tma_load_2d_pair(sa + h * (BMc * 128), ta, bar, kc + BKT * h, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BNh / 64; ++c)
              tma_load_2d_pair(sb + c * (BK * 128), tb, bar, nb + 64 * c, kc);
          } else {
#pragma unroll
            for (int h = 0; h < BK / BKT; ++h)
              tma_load_2d_pair(sb + h * (BNh * 128), tb, bar, kc + BKT * h, nb);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // copies already issued into this CTA's shared memory land within microseconds: give them
        // a bounded grace period before the CTA heads for the exit
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------------------------------------------------------- MMA issuer (leader)
      const uint32_t idesc = umma_idesc_bf16(2 * BMc, BNp, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < total && ok; tile += npairs, ++it) {
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
        const uint32_t d_tmem = tmem_base + acc * BNp;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase)) {
            report_status(g.status, kStatusTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc =
                A_MN ? umma_smem_desc(sa + k * 2048, BK * 128, 1024)
                     : umma_smem_desc(sa + (k / 4) * (BMc * 128) + (k % 4) * 32, 16, 1024);
            const uint64_t bdesc =
                B_MN ? umma_smem_desc(sb + k * 2048, BK * 128, 1024)
                     : umma_smem_desc(sb + (k / 4) * (BNh * 128) + (k % 4) * 32, 16, 1024);
            umma2_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty[stage], 1u);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma2_commit_both(&tfull[acc], 1u);
      }
    }
    __syncwarp();
  } else if (GATHER && warp >= 2 + kEpiWarps) {
    // ------------------------------------------------------------------ pull warps (10, 11)
    if constexpr (GATHER) {
      constexpr int kItemsPerChunk = BMc / kPullRows;
      const int items_total = g.world * chunks_per_peer * kItemsPerChunk;
      const long long vec_per_row = (2LL * g.K) / 16;
      for (;;) {
        unsigned c = 0;
        if (lane == 0) c = atomicAdd(g.chunk_counter, 1u);
        c = __shfl_sync(0xffffffffu, c, 0);
        if (c >= unsigned(items_total)) break;
        const int chunk_i = int(c) / kItemsPerChunk;    // chunks in consumption order
        const int sub = int(c) % kItemsPerChunk;
        const int peer = (g.rank + chunk_i / chunks_per_peer) % g.world;
        const int t = chunk_i % chunks_per_peer;
        const int r0 = t * BMc + sub * kPullRows;
        const int chunk_end = min((t + 1) * BMc, g.n_local);
        if (r0 >= chunk_end) continue;                  // short last chunk: no such item
        const int r1 = min(r0 + kPullRows, chunk_end);
        if (peer != g.rank) {                           // own rows are in place already
          const char* src = static_cast<const char*>(g.a_peers[peer]);
          char* dst = static_cast<char*>(g.a_local) + 2LL * peer * g.n_local * g.lda_peer;
          const long long total_vec = vec_per_row * (r1 - r0);
          constexpr int kPullDepth = 16;  // 16 x 16 bytes per lane in flight
          for (long long i0 = 0; i0 < total_vec; i0 += 32 * kPullDepth) {
            uint4 buf[kPullDepth];
#pragma unroll
            for (int u = 0; u < kPullDepth; ++u) {
              const long long i = i0 + u * 32 + lane;
              if (i < total_vec) {
                const long long rr = r0 + i / vec_per_row, cc = i % vec_per_row;
                buf[u] = *reinterpret_cast<const uint4*>(src + 2LL * rr * g.lda_peer + cc * 16);
              }
            }
#pragma unroll
            for (int u = 0; u < kPullDepth; ++u) {
              const long long i = i0 + u * 32 + lane;
              if (i < total_vec) {
                const long long rr = r0 + i / vec_per_row, cc = i % vec_per_row;
                *reinterpret_cast<uint4*>(dst + 2LL * rr * g.lda_peer + cc * 16) = buf[u];
              }
            }
          }
          __threadfence();
        }
        __syncwarp();
        if (lane == 0) {
          unsigned* fp = g.flags + (peer * chunks_per_peer + t);
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(fp) : "memory");
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kChunks = BNp / 32 / 2;
    OutT* Cout = reinterpret_cast<OutT*>(g.C);
    const uint32_t tempty_leader0 = map_to_cta(&tempty[0], 0);
    const uint32_t tempty_leader1 = map_to_cta(&tempty[1], 0);
    int it = 0;
    for (int tile = pair; tile < total; tile += npairs, ++it) {
      const int split = tile / (tiles_m * tiles_n);
      int m0, n0, m_limit, chunk;
      decode(tile - split * (tiles_m * tiles_n), m0, n0, m_limit, chunk);
      const int acc = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aphase)) {
        report_status(g.status, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c = half * kChunks; c < (half + 1) * kChunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BNp + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if constexpr (sizeof(OutT) == 2) {
          uint8_t* sblk = reinterpret_cast<uint8_t*>(epi_stage + (warp - 2) * EPI_WORDS);
          uint8_t* srow = sblk + lane * 80;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
            pk.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            pk.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            pk.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(srow + 16 * j) = pk;
          }
          __syncwarp();
          const int rr = lane >> 2, cc = lane & 3;
          const int colb = col0 + cc * 8;
          if (colb < g.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int lr = i * 8 + rr;
              const int grow = m0 + q * 32 + lr;
              if (grow < m_limit) {
                OutT* dst =
                    (g.c_rows_per_peer > 0
                         ? reinterpret_cast<OutT*>(g.c_peers[grow / g.c_rows_per_peer]) +
                               static_cast<long long>(grow % g.c_rows_per_peer) * g.ldc
                         : Cout + static_cast<long long>(grow) * g.ldc) +
                    colb;
                const uint4 pk = *reinterpret_cast<const uint4*>(sblk + lr * 80 + cc * 16);
                if (g.accumulate)
                  red_add8_bf16(dst, pk);
                else
                  *reinterpret_cast<uint4*>(dst) = pk;
              }
            }
          }
          __syncwarp();
        } else {
          if (g.accumulate) {
            float* st = epi_stage + (warp - 2) * EPI_WORDS;
#pragma unroll
            for (int j = 0; j < 32; ++j) st[lane * 33 + j] = __uint_as_float(r[j]);
            __syncwarp();
            const int rr = lane >> 3, cc = (lane & 7) * 4;
            if (col0 + cc < g.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int lr = i * 4 + rr;
                const int grow = m0 + q * 32 + lr;
                if (grow < m_limit) {
                  const float* sp = st + lr * 33 + cc;
                  red_add4(reinterpret_cast<float*>(g.C) + static_cast<long long>(grow) * g.ldc +
                               col0 + cc,
                           sp[0], sp[1], sp[2], sp[3]);
                }
              }
            }
            __syncwarp();
          } else if (row < m_limit && col0 < g.N) {
            float* fd = reinterpret_cast<float*>(g.C) + static_cast<long long>(row) * g.ldc + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col0 + 4 * j < g.N)
                *reinterpret_cast<float4*>(fd + 4 * j) =
                    make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          }
        }
      }
      // this warp is done reading the accumulator: one arrival at the leader's barrier
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc ? tempty_leader1 : tempty_leader0);
    }
  }

  // Nobody leaves while the partner may still read this CTA's shared memory, arrive on its
  // barriers or (the leader's MMAs) write its tensor memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc2(tmem_base, TMEM_COLS);
}

// Number of CTA pairs that can be resident at once. Not every SM has a partner it can form a
// 2-CTA cluster with (parts ship with single SMs of a pair fused off), so this can be below
// SMs / 2; a persistent grid larger than it would run in two waves.
int g_max_pairs = 0;

template <int A_MN, int B_MN, typename OutT, int GATHER = 0>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2,
            const CUtensorMap& tmB2, const Args2& g, long long total, cudaStream_t stream) {
  auto kern = gemm_2cta_kernel<A_MN, B_MN, OutT, GATHER>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads + (GATHER ? 32 * kPullWarps : 0), 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (g_max_pairs == 0) {
    int dev = 0, sms = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms > 1 ? sms / 2 * 2 : 2, 1, 1);
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sms / 2 > 0 ? sms / 2 : 1;
    }
    g_max_pairs = n;
  }
  const int pairs = (int)(total < g_max_pairs ? total : g_max_pairs);
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmA2, tmB2, g) == cudaSuccess ? 0 : -11;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace
}  // namespace lb

namespace lb {
namespace {

// C[M, N] = or += A · op(B) (+ A2 · op(B2) when K2 > 0; A2 is K-major like A, B2 laid out like B).
int run2(const void* A, const void* B, const void* A2, const void* B2, void* C, int M, int N, int K,
         int K2, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc,
         int a_mn, int b_mn, int out_fp32, int accumulate, int splits, int* status,
         cudaStream_t stream, const void* const* c_peers = nullptr, int c_world = 0,
         int c_rows_per_peer = 0) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -4;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 3)) return -3;
  if (!out_fp32 && ((ldc & 7) || splits > 1)) return -5;
  if (K2 > 0 && (a_mn || splits > 1 || (K2 & 7) || (lda2 & 7) || (ldb2 & 7))) return -5;
  const int kb_total = (K + BK - 1) / BK + (K2 > 0 ? (K2 + BK - 1) / BK : 0);
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  const int kb_per = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per - 1) / kb_per;
  if (splits > 1) accumulate = 1;
  CUtensorMap tmA, tmB, tmA2, tmB2;
  int rc;
  if (a_mn)
    rc = make_tmap_2d(&tmA, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, true);
  else
    rc = make_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BKT, BMc, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true);
  else
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BKT, BNh, true);
  if (rc) return rc;
  if (K2 > 0) {
    rc = make_tmap_2d(&tmA2, A2, 2, (uint64_t)K2, (uint64_t)M, (uint64_t)lda2 * 2, BKT, BMc, true);
    if (rc) return rc;
    if (b_mn)
      rc = make_tmap_2d(&tmB2, B2, 2, (uint64_t)N, (uint64_t)K2, (uint64_t)ldb2 * 2, 64, BK, true);
    else
      rc = make_tmap_2d(&tmB2, B2, 2, (uint64_t)K2, (uint64_t)N, (uint64_t)ldb2 * 2, BKT, BNh, true);
    if (rc) return rc;
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  const int tiles_m = (M + 2 * BMc - 1) / (2 * BMc);
  const int tiles_n = (N + BNp - 1) / BNp;
  Args2 g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.K2 = K2 > 0 ? K2 : 0;
  g.C = C;
  g.ldc = ldc;
  g.accumulate = accumulate;
  g.splits = splits;
  g.kb_per_split = kb_per;
  g.raster_m_fast = tiles_n > tiles_m ? 1 : 0;
  g.status = status;
  if (c_peers != nullptr && c_rows_per_peer > 0) {
    if (c_world < 1 || c_world > 8 || out_fp32 || accumulate || splits > 1) return -5;
    for (int i = 0; i < c_world; ++i) g.c_peers[i] = const_cast<void*>(c_peers[i]);
    g.c_rows_per_peer = c_rows_per_peer;
  }
  const long long total = 1LL * tiles_m * tiles_n * splits;
#define LB2(AM, BMJ)                                                                    \
  (out_fp32 ? launch2<AM, BMJ, float>(tmA, tmB, tmA2, tmB2, g, total, stream)          \
            : launch2<AM, BMJ, __nv_bfloat16>(tmA, tmB, tmA2, tmB2, g, total, stream))
  if (!a_mn && !b_mn) return LB2(0, 0);
  if (!a_mn && b_mn) return LB2(0, 1);
  if (a_mn && b_mn) return LB2(1, 1);
  return LB2(1, 0);
#undef LB2
}

}  // namespace
}  // namespace lb

// Same contract as lb_gemm_bf16 without bias and with splits given explicitly (>= 1); a bf16
// output may be accumulated into (packed red.global.add, unsplit only). Returns -5 / -6 for forms
// this kernel does not take (the caller then uses the one-CTA kernel).
extern "C" int lb_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                                 int out_fp32, int accumulate, int splits, int* status,
                                 void* stream_) {
  return lb::run2(A, B, nullptr, nullptr, C, M, N, K, 0, lda, ldb, 0, 0, ldc, a_mn, b_mn, out_fp32,
                  accumulate, splits, status, reinterpret_cast<cudaStream_t>(stream_));
}

// Same contract as lb_gemm_bf16_ext without bias: bf16 C = A · op(B) + A2 · op(B2).
extern "C" int lb_gemm_bf16_2cta_ext(const void* A, const void* B, const void* A2, const void* B2,
                                     void* C, int M, int N, int K, int K2, long long lda,
                                     long long ldb, long long lda2, long long ldb2, long long ldc,
                                     int b_mn, int* status, void* stream_) {
  if (K2 <= 0) return -4;
  return lb::run2(A, B, A2, B2, C, M, N, K, K2, lda, ldb, lda2, ldb2, ldc, 0, b_mn, 0, 0, 1, status,
                  reinterpret_cast<cudaStream_t>(stream_));
}

// CTA pairs resident at once (the slots of the caller's split heuristic); SMs / 2 until the first
// launch has asked the driver.
extern "C" int lb_gemm_2cta_pairs() {
  return lb::g_max_pairs > 0 ? lb::g_max_pairs : lb::sm_count() / 2;
}

// bf16 C rows stored into per-rank buffers (see lb_gemm_bf16_push16 in gemm_bf16.cu): row r of the
// product goes to local row r % rows_per_peer of c_peers[r / rows_per_peer].
extern "C" int lb_gemm_bf16_2cta_push(const void* A, const void* B, const void* const* c_peers,
                                      int world, int rows_per_peer, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int a_mn,
                                      int b_mn, int* status, void* stream_) {
  if (M != world * rows_per_peer) return -3;
  return lb::run2(A, B, nullptr, nullptr, nullptr, M, N, K, 0, lda, ldb, 0, 0, ldc, a_mn, b_mn, 0, 0,
                  1, status, reinterpret_cast<cudaStream_t>(stream_), c_peers, world,
                  rows_per_peer);
}

// All-gather fused into the product (see lb_gemm_bf16_ag in gemm_bf16.cu, whose contract this
// shares, without bias): C[world * rows_local, N] = A_all · op(B), the peers' rows of A_all pulled
// by two extra warps per CTA while the tiles consume them in pull order. The caller has copied
// its own rows into a_all and zeroed nothing: `counter` is reset here.
extern "C" int lb_gemm_bf16_2cta_ag(const void* const* a_peers, void* a_all, const void* B, void* C,
                                    int rows_local, int world, int rank, int N, int K,
                                    long long lda, long long ldb, long long ldc, int b_mn,
                                    unsigned* flags, unsigned* counter, unsigned epoch,
                                    int* status, void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 1 || world > 8 || rank < 0 || rank >= world || rows_local <= 0 || N <= 0 || K <= 0)
    return -3;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -3;
  const int M = world * rows_local;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, a_all, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BKT, BMc, true);
  if (rc) return rc;
  if (b_mn)
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, true);
  else
    rc = make_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BKT, BNh, true);
  if (rc) return rc;
  Args2 g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.C = C;
  g.ldc = ldc;
  g.splits = 1;
  g.kb_per_split = (K + BK - 1) / BK;
  g.status = status;
  for (int i = 0; i < world; ++i) g.a_peers[i] = a_peers[i];
  g.a_local = a_all;
  g.lda_peer = lda;
  g.n_local = rows_local;
  g.world = world;
  g.rank = rank;
  g.flags = flags;
  g.chunk_counter = counter;
  g.epoch = epoch;
  const long long total =
      1LL * world * ((rows_local + 2 * BMc - 1) / (2 * BMc)) * ((N + BNp - 1) / BNp);
  if (cudaMemsetAsync(counter, 0, sizeof(unsigned), stream) != cudaSuccess) return -12;
  return b_mn ? launch2<0, 1, __nv_bfloat16, 1>(tmA, tmB, tmA, tmB, g, total, stream)
              : launch2<0, 0, __nv_bfloat16, 1>(tmA, tmB, tmA, tmB, g, total, stream);
}
