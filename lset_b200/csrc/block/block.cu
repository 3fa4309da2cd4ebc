// Decoder-block runner: see block.h. Host code only, except for one small scaling kernel; every
// heavy launch goes through the library's own launchers (declared in common/api.h).
#include "block.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"

namespace {

constexpr size_t kAlign = 256;

inline size_t up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

inline int tp_tokens(const LbTpCtx* tp) { return tp->world * tp->rows; }

// Carves 256-byte aligned slices out of one arena. With a null base it only measures.
struct Arena {
  char* base;
  size_t off = 0;
  explicit Arena(void* b) : base(static_cast<char*>(b)) {}
  void* take(size_t bytes) {
    void* p = base ? base + off : nullptr;
    off += up(bytes);
    return p;
  }
  __nv_bfloat16* bf(size_t n) { return static_cast<__nv_bfloat16*>(take(n * 2)); }
  float* f32(size_t n) { return static_cast<float*>(take(n * 4)); }
};

__global__ void scale_bf16_kernel(__nv_bfloat16* x, long long n, float s) {
  long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x;
  const long long step = 1LL * gridDim.x * blockDim.x;
  for (; i < n; i += step) x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * s);
}

int scale_bf16(__nv_bfloat16* x, long long n, float s, cudaStream_t st) {
  if (n <= 0) return 0;
  long long g = (n + 255) / 256;
  if (g > 1184) g = 1184;
  scale_bf16_kernel<<<int(g), 256, 0, st>>>(x, n, s);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

struct Saved {
  __nv_bfloat16 *x1, *res1, *qkv, *qr, *kr, *o, *x2, *gu, *h;
  float *rstd1, *rstd2, *q_rstd, *k_rstd, *lse;
  __nv_bfloat16* ts[8];  // LoRA: s · x · Aᵀ per linear (qkv parts 0-2, o 3, gate_up parts 4-5, down 6)
};

const LbLinear* linear_at(const LbBlockDesc* d, int i) {
  switch (i) {
    case 0: case 1: case 2: return i < d->qkv.n ? &d->qkv.part[i] : nullptr;
    case 3: return &d->o_proj;
    case 4: case 5: return i - 4 < d->gate_up.n ? &d->gate_up.part[i - 4] : nullptr;
    case 6: return &d->down;
    default: return nullptr;
  }
}

// `T` rows for everything the projections and the attention see; `R` rows for what lives on the
// token-sharded stream (R == T when the stream is not sharded).
Saved carve_saved(const LbBlockDesc* d, int T, int R, int has_residual, Arena& a) {
  Saved s{};
  const size_t t = (size_t)T, r = (size_t)R;
  s.x1 = a.bf(t * d->H);
  s.res1 = has_residual ? a.bf(r * d->H) : nullptr;
  s.rstd1 = a.f32(r);
  s.qkv = a.bf(t * d->qkv.width);
  s.qr = a.bf(t * d->Hq * d->hd);
  s.kr = a.bf(t * d->Hk * d->hd);
  s.q_rstd = d->qk_norm ? a.f32(t * d->Hq) : nullptr;
  s.k_rstd = d->qk_norm ? a.f32(t * d->Hk) : nullptr;
  s.o = a.bf(t * d->Hq * d->hd);
  s.lse = a.f32(t * d->Hq);
  s.rstd2 = a.f32(r);
  s.x2 = a.bf(t * d->H);
  s.gu = a.bf(t * d->gate_up.width);
  s.h = a.bf(t * d->I);
  for (int i = 0; i < 7; ++i) {
    const LbLinear* l = linear_at(d, i);
    s.ts[i] = (l != nullptr && l->lora_r > 0) ? a.bf(t * l->lora_r) : nullptr;
  }
  return s;
}

struct Work {
  __nv_bfloat16 *dres2, *dh, *dgu, *dx2, *dO, *dqr, *dkr, *dqkv, *dx1, *us;
  __nv_bfloat16 *dy_all, *dres_all;  // token-sharded stream: gathered output gradients
  float* delta;
};

Work carve_work(const LbBlockDesc* d, int T, int R, bool sharded, Arena& a) {
  Work w{};
  const size_t t = (size_t)T, r = (size_t)R;
  w.dres2 = sharded ? nullptr : a.bf(r * d->H);  // sharded: lives in the publication area
  int rmax = 0;
  for (int i = 0; i < 7; ++i) {
    const LbLinear* l = linear_at(d, i);
    if (l != nullptr && l->lora_r > rmax) rmax = l->lora_r;
  }
  w.us = rmax > 0 ? a.bf(t * rmax) : nullptr;
  // The MLP half of the backward is finished before the attention half starts: both overlay
  // the same region.
  const size_t mark = a.off;
  w.dy_all = sharded ? a.bf(t * d->H) : nullptr;
  w.dh = a.bf(t * d->I);
  w.dgu = a.bf(t * d->gate_up.width);
  w.dx2 = a.bf(r * d->H);
  const size_t end_mlp = a.off;
  a.off = mark;
  w.dres_all = sharded ? a.bf(t * d->H) : nullptr;
  w.dO = a.bf(t * d->Hq * d->hd);
  w.dqr = a.bf(t * d->Hq * d->hd);
  w.dkr = a.bf(t * d->Hk * d->hd);
  w.dqkv = a.bf(t * d->qkv.width);
  w.dx1 = a.bf(r * d->H);
  w.delta = a.f32(t * d->Hq);
  if (a.off < end_mlp) a.off = end_mlp;
  return w;
}

#define LB_TRY(expr)          \
  do {                        \
    const int rc_ = (expr);   \
    if (rc_ != 0) return rc_; \
  } while (0)

// y[:, :n_out] (row stride ldy) = x · Wᵀ (+ LoRA). `ts` receives s · x · Aᵀ when the linear has adapters.
int lin_fwd(const LbLinear& l, const __nv_bfloat16* x, long long ldx, __nv_bfloat16* y,
            long long ldy, int T, __nv_bfloat16* ts, const LbStreamCtx* c) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  if (l.lora_r > 0) {
    LB_TRY(lb_gemm_bf16(x, l.lora_a, ts, T, l.lora_r, l.k_in, ldx, l.k_in, l.lora_r, 0, 0, 0, 0,
                        nullptr, 1, 0, c->status, c->stream));
    LB_TRY(scale_bf16(ts, 1LL * T * l.lora_r, l.lora_scale, st));
    return lb_gemm_bf16_ext(x, l.w, ts, l.lora_b, y, T, l.n_out, l.k_in, l.lora_r, ldx, l.ldw,
                            l.lora_r, l.lora_r, ldy, 0, nullptr, c->status, c->stream);
  }
  return lb_gemm_bf16(x, l.w, y, T, l.n_out, l.k_in, ldx, l.ldw, ldy, 0, 0, 0, 0, nullptr, 1, 0,
                      c->status, c->stream);
}

// dx[T, k_in] (contiguous) = or += dy · W (+ s · (dy · B) · A). `us` is scratch for s · dy · B and is
// left filled for the weight-gradient step that follows.
int lin_dgrad(const LbLinear& l, const __nv_bfloat16* dy, long long lddy, __nv_bfloat16* dx, int T,
              bool accumulate, __nv_bfloat16* us, const LbStreamCtx* c) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  const void* peers[1] = {dx};
  if (l.lora_r > 0) {
    LB_TRY(lb_gemm_bf16(dy, l.lora_b, us, T, l.lora_r, l.n_out, lddy, l.lora_r, l.lora_r, 0, 1, 0, 0,
                        nullptr, 1, 0, c->status, c->stream));
    LB_TRY(scale_bf16(us, 1LL * T * l.lora_r, l.lora_scale, st));
    if (!accumulate)
      return lb_gemm_bf16_ext(dy, l.w, us, l.lora_a, dx, T, l.k_in, l.n_out, l.lora_r, lddy, l.ldw,
                              l.lora_r, l.k_in, l.k_in, 1, nullptr, c->status, c->stream);
    LB_TRY(lb_gemm_bf16_scatter16(dy, l.w, peers, 1, T, T, l.k_in, l.n_out, lddy, l.ldw, l.k_in, 0,
                                  1, 0, c->status, c->stream));
    return lb_gemm_bf16_scatter16(us, l.lora_a, peers, 1, T, T, l.k_in, l.lora_r, l.lora_r, l.k_in,
                                  l.k_in, 0, 1, 0, c->status, c->stream);
  }
  if (!accumulate)
    return lb_gemm_bf16(dy, l.w, dx, T, l.k_in, l.n_out, lddy, l.ldw, l.k_in, 0, 1, 0, 0, nullptr, 1,
                        0, c->status, c->stream);
  return lb_gemm_bf16_scatter16(dy, l.w, peers, 1, T, T, l.k_in, l.n_out, lddy, l.ldw, l.k_in, 0, 1,
                                0, c->status, c->stream);
}

// dW += dyᵀ · x; adapters: dA += usᵀ · x, dB += dyᵀ · ts. Frozen tensors (null accumulators) are skipped.
int lin_wgrad(const LbLinear& l, const __nv_bfloat16* dy, long long lddy, const __nv_bfloat16* x,
              long long ldx, int T, const __nv_bfloat16* ts, const __nv_bfloat16* us,
              const LbStreamCtx* c) {
  if (l.wgrad != nullptr)
    LB_TRY(lb_gemm_bf16(dy, x, l.wgrad, l.n_out, l.k_in, T, lddy, ldx, l.k_in, 1, 1, 1, 1, nullptr,
                        0 /*auto*/, 0, c->status, c->stream));
  if (l.lora_r > 0) {
    if (l.lora_a_grad != nullptr)
      LB_TRY(lb_gemm_bf16(us, x, l.lora_a_grad, l.lora_r, l.k_in, T, l.lora_r, ldx, l.k_in, 1, 1, 1,
                          1, nullptr, 0, 0, c->status, c->stream));
    if (l.lora_b_grad != nullptr)
      LB_TRY(lb_gemm_bf16(dy, ts, l.lora_b_grad, l.n_out, l.lora_r, T, lddy, l.lora_r, l.lora_r, 1,
                          1, 1, 1, nullptr, 0, 0, c->status,
                          c->stream));
  }
  return 0;
}

int lin_fwd_launches(const LbLinear& l) { return l.lora_r > 0 ? 3 : 1; }

int lin_bwd_launches(const LbLinear& l, bool accumulate) {
  int n = l.wgrad != nullptr ? 1 : 0;
  if (l.lora_r > 0)
    n += 3 + (accumulate ? 1 : 0) + (l.lora_a_grad != nullptr) + (l.lora_b_grad != nullptr);
  else
    n += 1;
  return n;
}

// ---- token-sharded stream (tensor parallelism with sequence parallelism) ------------------------
// Running counters of one call. The double-buffering rule of the symmetric areas: use e touches
// half e & 1 and contains exactly one barrier; a half is rewritten two uses later, after the
// barrier of the use in between, which every peer joins only after its GEMM of use e is complete
// in stream order. A reduce-scatter half is read (its slots summed) right after the barrier of
// its use and rewritten two uses later under the same rule.
struct TpRun {
  const LbTpCtx* t;
  unsigned ag_epoch, ag_calls, rs_epoch, bar_epoch;
  explicit TpRun(const LbTpCtx* tp)
      : t(tp), ag_epoch(tp->ag_epoch), ag_calls(tp->ag_calls), rs_epoch(tp->rs_epoch),
        bar_epoch(tp->bar_epoch) {}
  // half of the publication area the next gathered GEMM uses: the producer of the shard may
  // write straight into it
  __nv_bfloat16* next_slot() const {
    return static_cast<__nv_bfloat16*>(t->ag_local[(ag_epoch + 1) & 1]);
  }
};

int tp_barrier(TpRun& r, const LbStreamCtx* c) {
  ++r.bar_epoch;
  return lb_device_barrier(r.t->pads, r.t->world, r.t->rank, r.bar_epoch, r.t->bar_limit_ns,
                           c->status, c->stream);
}

// y[Tp, N] (row stride ldy) = all_gather(shard)[Tp, K] · op(w); `x_all` [Tp, K] receives the
// gathered rows (own rows by a local copy, the peers' rows by the pull warps of the GEMM).
// op(w) = wᵀ for w [N, K] (b_mn 0) or w for w [K, N] (b_mn 1).
int tp_ag_gemm(TpRun& r, const __nv_bfloat16* shard, __nv_bfloat16* x_all, const LbLinear& l,
               int b_mn, __nv_bfloat16* y, long long ldy, int N, int K, const LbStreamCtx* c) {
  const LbTpCtx* t = r.t;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  ++r.ag_epoch;
  ++r.ag_calls;
  const int half = r.ag_epoch & 1;
  __nv_bfloat16* slot = static_cast<__nv_bfloat16*>(t->ag_local[half]);
  const size_t bytes = (size_t)t->rows * K * 2;
  if (shard != slot &&
      cudaMemcpyAsync(slot, shard, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
    return -11;
  if (cudaMemcpyAsync(x_all + (size_t)t->rank * t->rows * K, shard, bytes,
                      cudaMemcpyDeviceToDevice, st) != cudaSuccess)
    return -11;
  LB_TRY(tp_barrier(r, c));  // every shard is published
  return lb_gemm_bf16_ag(t->ag_peers[half], x_all, l.w, y, t->rows, t->world, t->rank, N, K, K,
                         l.ldw, ldy, b_mn, nullptr, t->ag_flags, t->ag_counter, r.ag_calls,
                         c->status, c->stream);
}

// out[rows, N] = reduce_scatter(a[Tp, K] · op(w)): every rank stores its partial rows into its
// own slot of the owner's area from the GEMM epilogue; the owner sums its slots after the barrier.
int tp_gemm_rs(TpRun& r, const __nv_bfloat16* a, long long lda, const LbLinear& l, int b_mn,
               __nv_bfloat16* out, int N, int K, const LbStreamCtx* c) {
  const LbTpCtx* t = r.t;
  ++r.rs_epoch;
  const int half = r.rs_epoch & 1;
  LB_TRY(lb_gemm_bf16_push16(a, l.w, t->rs_peers[half], t->world, t->rows, tp_tokens(t), N, K, lda,
                             l.ldw, N, 0, b_mn, 0, c->status, c->stream));
  LB_TRY(tp_barrier(r, c));  // every contribution has landed
  return lb_take_sum(t->rs_local[half], out, (long long)t->rows * N, t->world, c->stream);
}

bool tp_shape_ok(const LbBlockDesc* d, const LbStreamCtx* c, const LbTpCtx* t) {
  if (t->world < 2 || t->world > 8 || t->rank < 0 || t->rank >= t->world || t->rows <= 0)
    return false;
  if (c->T > tp_tokens(t) || !c->packed) return false;
  if (d->qkv.n != 1 || d->gate_up.n != 1) return false;
  for (int i = 0; i < 7; ++i) {
    const LbLinear* l = linear_at(d, i);
    if (l != nullptr && l->lora_r > 0) return false;
  }
  return true;
}

int block_fwd_tp(const LbBlockDesc* d, const LbStreamCtx* c, const LbBlockIO* io) {
  const LbTpCtx* t = io->tp;
  if (!tp_shape_ok(d, c, t)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  const int T = c->T, R = t->rows, Tp = tp_tokens(t);
  Arena arena(io->saved);
  const Saved s = carve_saved(d, Tp, R, io->residual != nullptr, arena);
  const int H = d->H, hd = d->hd, Nq = d->Hq * hd, Nk = d->Hk * hd, W = d->qkv.width, I = d->I;
  const __nv_bfloat16* branch = static_cast<const __nv_bfloat16*>(io->branch);
  const __nv_bfloat16* stream_in = io->residual != nullptr ? s.res1 : branch;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(io->out);
  TpRun r(t);

  __nv_bfloat16* x1s = r.next_slot();
  LB_TRY(lb_rms_norm_fwd(branch, io->residual, d->ln1_w, x1s, s.res1, s.rstd1, R, H, d->eps,
                         d->w_off, c->stream));
  LB_TRY(tp_ag_gemm(r, x1s, s.x1, d->qkv.part[0], 0, s.qkv, W, W, H, c));
  LB_TRY(lb_qk_norm_rope_fwd(s.qkv, W, s.qkv + Nq, W, d->qk_norm ? d->qn_w : nullptr,
                             d->qk_norm ? d->kn_w : nullptr, c->cos, c->sin, c->pos, c->pos_i64, 1,
                             s.qr, Nq, s.kr, Nk, s.q_rstd, s.k_rstd, T, d->Hq, d->Hk, hd, d->eps,
                             d->w_off, d->qk_norm, c->stream));
  if (Tp > T &&  // rows that pad the stream to a multiple of the group size
      cudaMemsetAsync(s.o + (size_t)T * Nq, 0, (size_t)(Tp - T) * Nq * 2, st) != cudaSuccess)
    return -11;
  LB_TRY(lb_attn_fwd(s.qr, Nq, s.kr, Nk, s.qkv + Nq + Nk, W, c->seq_start, c->seq_end, c->plan_q,
                     c->cap_q, s.o, Nq, s.lse, T, d->Hq, d->Hk, hd, d->softmax_scale, d->causal,
                     c->status, c->stream));
  LB_TRY(tp_gemm_rs(r, s.o, Nq, d->o_proj, 0, out, H, Nq, c));
  __nv_bfloat16* x2s = r.next_slot();
  LB_TRY(lb_rms_norm_fwd(out, stream_in, d->ln2_w, x2s, io->res_out, s.rstd2, R, H, d->eps,
                         d->w_off, c->stream));
  LB_TRY(tp_ag_gemm(r, x2s, s.x2, d->gate_up.part[0], 0, s.gu, 2 * I, 2 * I, H, c));
  LB_TRY(lb_glu_fwd(d->act_kind, s.gu, s.gu + I, 2 * I, s.h, I, Tp, I, c->stream));
  return tp_gemm_rs(r, s.h, I, d->down, 0, out, H, I, c);
}

int block_bwd_tp(const LbBlockDesc* d, const LbStreamCtx* c, const LbBlockIO* io) {
  const LbTpCtx* t = io->tp;
  if (!tp_shape_ok(d, c, t)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  const int T = c->T, R = t->rows, Tp = tp_tokens(t);
  const bool has_res = io->residual != nullptr;
  Arena sa(io->saved);
  const Saved s = carve_saved(d, Tp, R, has_res, sa);
  Arena wa(io->work);
  const Work w = carve_work(d, Tp, R, true, wa);
  const int H = d->H, hd = d->hd, Nq = d->Hq * hd, Nk = d->Hk * hd, W = d->qkv.width, I = d->I;
  const __nv_bfloat16* d_out = static_cast<const __nv_bfloat16*>(io->d_out);
  const __nv_bfloat16* stream_in =
      has_res ? s.res1 : static_cast<const __nv_bfloat16*>(io->branch);
  TpRun r(t);

  // ---- MLP: down is row-parallel (its output gradient is gathered), gate-up column-parallel
  // (its input gradient is reduced and scattered)
  LB_TRY(tp_ag_gemm(r, d_out, w.dy_all, d->down, 1, w.dh, I, I, H, c));
  LB_TRY(lin_wgrad(d->down, w.dy_all, H, s.h, I, Tp, nullptr, nullptr, c));
  LB_TRY(lb_glu_bwd(d->act_kind, w.dh, I, s.gu, s.gu + I, 2 * I, w.dgu, w.dgu + I, 2 * I, Tp, I,
                    c->stream));
  LB_TRY(tp_gemm_rs(r, w.dgu, 2 * I, d->gate_up.part[0], 1, w.dx2, H, 2 * I, c));
  LB_TRY(lin_wgrad(d->gate_up.part[0], w.dgu, 2 * I, s.x2, H, Tp, nullptr, nullptr, c));
  // the gradient of the stream after the attention branch: written where the next gathered GEMM
  // publishes from, and read again by the first norm's backward at the end of this call
  __nv_bfloat16* dres2 = r.next_slot();
  LB_TRY(lb_rms_norm_bwd(w.dx2, io->d_res_out, io->res_out, d->ln2_w, s.rstd2, dres2,
                         c->norm_scratch, d->ln2_wgrad, 1, 1, R, H, d->w_off, c->stream));
  // ---- attention
  LB_TRY(tp_ag_gemm(r, dres2, w.dres_all, d->o_proj, 1, w.dO, Nq, Nq, H, c));
  LB_TRY(lin_wgrad(d->o_proj, w.dres_all, H, s.o, Nq, Tp, nullptr, nullptr, c));
  if (Tp > T &&
      cudaMemsetAsync(w.dqkv + (size_t)T * W, 0, (size_t)(Tp - T) * W * 2, st) != cudaSuccess)
    return -11;
  LB_TRY(lb_attn_bwd(w.dO, Nq, s.qr, Nq, s.kr, Nk, s.qkv + Nq + Nk, W, s.o, Nq, s.lse, w.delta,
                     c->seq_start, c->seq_end, c->plan_q, c->cap_q, c->plan_kv, c->cap_kv, w.dqr, Nq,
                     w.dkr, Nk, w.dqkv + Nq + Nk, W, T, d->Hq, d->Hk, hd, d->softmax_scale,
                     d->causal, c->status, c->stream));
  {
    const bool want_dw = d->qk_norm && d->qn_wgrad != nullptr && d->kn_wgrad != nullptr;
    const bool direct = want_dw && d->kn_wgrad == d->qn_wgrad + hd;
    void* dw_out = !want_dw ? nullptr : (direct ? (void*)d->qn_wgrad : (void*)c->wg_tmp);
    LB_TRY(lb_qk_norm_rope_bwd(w.dqr, Nq, w.dkr, Nk, s.qkv, W, s.qkv + Nq, W,
                               d->qk_norm ? d->qn_w : nullptr, d->qk_norm ? d->kn_w : nullptr,
                               c->cos, c->sin, c->pos, c->pos_i64, 1, s.q_rstd, s.k_rstd, w.dqkv, W,
                               w.dqkv + Nq, W, d->qk_norm ? c->rope_scratch : nullptr, dw_out, 1,
                               direct ? 1 : 0, T, d->Hq, d->Hk, hd, d->w_off, d->qk_norm,
                               c->stream));
    if (want_dw && !direct) {
      LB_TRY(lb_colsum(c->wg_tmp, 1, hd, d->qn_wgrad, 1, 1, c->stream));
      LB_TRY(lb_colsum(c->wg_tmp + hd, 1, hd, d->kn_wgrad, 1, 1, c->stream));
    }
  }
  LB_TRY(tp_gemm_rs(r, w.dqkv, W, d->qkv.part[0], 1, w.dx1, H, W, c));
  LB_TRY(lin_wgrad(d->qkv.part[0], w.dqkv, W, s.x1, H, Tp, nullptr, nullptr, c));
  return lb_rms_norm_bwd(w.dx1, dres2, stream_in, d->ln1_w, s.rstd1, io->dx, c->norm_scratch,
                         d->ln1_wgrad, 1, 1, R, H, d->w_off, c->stream);
}

}  // namespace

extern "C" size_t lb_block_saved_bytes(const LbBlockDesc* d, int T, int has_residual,
                                       const LbTpCtx* tp) {
  Arena a(nullptr);
  if (tp != nullptr)
    carve_saved(d, tp_tokens(tp), tp->rows, has_residual, a);
  else
    carve_saved(d, T, T, has_residual, a);
  return a.off;
}

extern "C" size_t lb_block_work_bytes(const LbBlockDesc* d, int T, const LbTpCtx* tp) {
  Arena a(nullptr);
  if (tp != nullptr)
    carve_work(d, tp_tokens(tp), tp->rows, true, a);
  else
    carve_work(d, T, T, false, a);
  return a.off;
}

extern "C" int lb_block_fwd_launches(const LbBlockDesc* d, const LbStreamCtx* c, int has_residual,
                                     const LbTpCtx* tp) {
  (void)has_residual;
  if (tp != nullptr)  // two norms, rope, attention (2), glu; 2 gathered GEMMs (own-row copy, barrier,
    return 6 + 2 * 3 + 2 * 3;  // GEMM) and 2 reduced GEMMs (GEMM, barrier, take-and-clear)
  int n = 6;  // two norms, rope, attention (tail clear + kernel), glu
  for (int i = 0; i < 7; ++i) {
    const LbLinear* l = linear_at(d, i);
    if (l != nullptr) n += lin_fwd_launches(*l);
  }
  return n + (c->packed ? 0 : 1);
}

extern "C" int lb_block_bwd_launches(const LbBlockDesc* d, const LbStreamCtx* c,
                                     const LbTpCtx* tp) {
  int n = 1 + 4 + 1;  // glu, attention (tail clear, delta, dq, dkv), rope
  n += d->ln1_wgrad != nullptr ? 2 : 1;
  n += d->ln2_wgrad != nullptr ? 2 : 1;
  if (d->qk_norm && d->qn_wgrad != nullptr) n += d->kn_wgrad == d->qn_wgrad + d->hd ? 1 : 3;
  if (tp != nullptr) {
    n += 2 * 3 + 1 + 2 * 3;  // as in the forward, plus the copy of d_out into the publication area
    for (int i = 0; i < 7; ++i) {
      const LbLinear* l = linear_at(d, i);
      if (l != nullptr && l->wgrad != nullptr) n += 1;
    }
    return n;
  }
  for (int i = 0; i < 7; ++i) {
    const LbLinear* l = linear_at(d, i);
    if (l != nullptr) n += lin_bwd_launches(*l, (i == 1 || i == 2 || i == 5));
  }
  return n + (c->packed ? 0 : 3);
}

extern "C" int lb_block_fwd(const LbBlockDesc* d, const LbStreamCtx* c, const LbBlockIO* io) {
  const int T = c->T;
  if (T <= 0) return 0;
  if (io->tp != nullptr) return block_fwd_tp(d, c, io);
  if (d->qkv.n < 1 || d->qkv.n > 3 || d->gate_up.n < 1 || d->gate_up.n > 2) return -3;
  if (d->qkv.width != (d->Hq + 2 * d->Hk) * d->hd || d->gate_up.width != 2 * d->I) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  Arena arena(io->saved);
  const Saved s = carve_saved(d, T, T, io->residual != nullptr, arena);
  const int H = d->H, hd = d->hd, Nq = d->Hq * hd, Nk = d->Hk * hd, W = d->qkv.width;
  const __nv_bfloat16* branch = static_cast<const __nv_bfloat16*>(io->branch);
  const __nv_bfloat16* stream_in = io->residual != nullptr ? s.res1 : branch;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(io->out);

  LB_TRY(lb_rms_norm_fwd(branch, io->residual, d->ln1_w, s.x1, s.res1, s.rstd1, T, H, d->eps,
                         d->w_off, c->stream));
  for (int p = 0, col = 0; p < d->qkv.n; ++p) {
    LB_TRY(lin_fwd(d->qkv.part[p], s.x1, H, s.qkv + col, W, T, s.ts[p], c));
    col += d->qkv.part[p].n_out;
  }
  LB_TRY(lb_qk_norm_rope_fwd(s.qkv, W, s.qkv + Nq, W, d->qk_norm ? d->qn_w : nullptr,
                             d->qk_norm ? d->kn_w : nullptr, c->cos, c->sin, c->pos, c->pos_i64, 1,
                             s.qr, Nq, s.kr, Nk, s.q_rstd, s.k_rstd, T, d->Hq, d->Hk, hd, d->eps,
                             d->w_off, d->qk_norm, c->stream));
  if (!c->packed) {  // rows of padding are never written by the attention kernel
    if (cudaMemsetAsync(s.o, 0, (size_t)T * Nq * 2, st) != cudaSuccess) return -11;
  }
  LB_TRY(lb_attn_fwd(s.qr, Nq, s.kr, Nk, s.qkv + Nq + Nk, W, c->seq_start, c->seq_end, c->plan_q,
                     c->cap_q, s.o, Nq, s.lse, T, d->Hq, d->Hk, hd, d->softmax_scale, d->causal,
                     c->status, c->stream));
  // attention branch output: staged in `out`, consumed by the second norm before the MLP writes there
  LB_TRY(lin_fwd(d->o_proj, s.o, Nq, out, H, T, s.ts[3], c));
  LB_TRY(lb_rms_norm_fwd(out, stream_in, d->ln2_w, s.x2, io->res_out, s.rstd2, T, H, d->eps,
                         d->w_off, c->stream));
  for (int p = 0, col = 0; p < d->gate_up.n; ++p) {
    LB_TRY(lin_fwd(d->gate_up.part[p], s.x2, H, s.gu + col, 2 * d->I, T, s.ts[4 + p], c));
    col += d->gate_up.part[p].n_out;
  }
  LB_TRY(lb_glu_fwd(d->act_kind, s.gu, s.gu + d->I, 2 * d->I, s.h, d->I, T, d->I, c->stream));
  return lin_fwd(d->down, s.h, d->I, out, H, T, s.ts[6], c);
}

extern "C" int lb_block_bwd(const LbBlockDesc* d, const LbStreamCtx* c, const LbBlockIO* io) {
  const int T = c->T;
  if (T <= 0) return 0;
  if (io->tp != nullptr) return block_bwd_tp(d, c, io);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(c->stream);
  const bool has_res = io->residual != nullptr;
  Arena sa(io->saved);
  const Saved s = carve_saved(d, T, T, has_res, sa);
  Arena wa(io->work);
  const Work w = carve_work(d, T, T, false, wa);
  const int H = d->H, hd = d->hd, Nq = d->Hq * hd, Nk = d->Hk * hd, W = d->qkv.width, I = d->I;
  const __nv_bfloat16* d_out = static_cast<const __nv_bfloat16*>(io->d_out);
  const __nv_bfloat16* stream_in =
      has_res ? s.res1 : static_cast<const __nv_bfloat16*>(io->branch);

  // ---- MLP
  LB_TRY(lin_dgrad(d->down, d_out, H, w.dh, T, false, w.us, c));
  LB_TRY(lin_wgrad(d->down, d_out, H, s.h, I, T, s.ts[6], w.us, c));
  LB_TRY(lb_glu_bwd(d->act_kind, w.dh, I, s.gu, s.gu + I, 2 * I, w.dgu, w.dgu + I, 2 * I, T, I,
                    c->stream));
  for (int p = 0, col = 0; p < d->gate_up.n; ++p) {
    const LbLinear& l = d->gate_up.part[p];
    LB_TRY(lin_dgrad(l, w.dgu + col, 2 * I, w.dx2, T, p > 0, w.us, c));
    LB_TRY(lin_wgrad(l, w.dgu + col, 2 * I, s.x2, H, T, s.ts[4 + p], w.us, c));
    col += l.n_out;
  }
  // second norm: the gradient of its input is both the attention branch's and the stream's
  LB_TRY(lb_rms_norm_bwd(w.dx2, io->d_res_out, io->res_out, d->ln2_w, s.rstd2, w.dres2,
                         c->norm_scratch, d->ln2_wgrad, 1, 1, T, H, d->w_off, c->stream));
  // ---- attention
  LB_TRY(lin_dgrad(d->o_proj, w.dres2, H, w.dO, T, false, w.us, c));
  LB_TRY(lin_wgrad(d->o_proj, w.dres2, H, s.o, Nq, T, s.ts[3], w.us, c));
  if (!c->packed) {
    if (cudaMemsetAsync(w.dqr, 0, (size_t)T * Nq * 2, st) != cudaSuccess ||
        cudaMemsetAsync(w.dkr, 0, (size_t)T * Nk * 2, st) != cudaSuccess ||
        cudaMemsetAsync(w.dqkv, 0, (size_t)T * W * 2, st) != cudaSuccess)
      return -11;
  }
  LB_TRY(lb_attn_bwd(w.dO, Nq, s.qr, Nq, s.kr, Nk, s.qkv + Nq + Nk, W, s.o, Nq, s.lse, w.delta,
                     c->seq_start, c->seq_end, c->plan_q, c->cap_q, c->plan_kv, c->cap_kv, w.dqr, Nq,
                     w.dkr, Nk, w.dqkv + Nq + Nk, W, T, d->Hq, d->Hk, hd, d->softmax_scale,
                     d->causal, c->status, c->stream));
  {
    const bool want_dw = d->qk_norm && d->qn_wgrad != nullptr && d->kn_wgrad != nullptr;
    const bool direct = want_dw && d->kn_wgrad == d->qn_wgrad + hd;
    void* dw_out = !want_dw ? nullptr : (direct ? (void*)d->qn_wgrad : (void*)c->wg_tmp);
    LB_TRY(lb_qk_norm_rope_bwd(w.dqr, Nq, w.dkr, Nk, s.qkv, W, s.qkv + Nq, W,
                               d->qk_norm ? d->qn_w : nullptr, d->qk_norm ? d->kn_w : nullptr,
                               c->cos, c->sin, c->pos, c->pos_i64, 1, s.q_rstd, s.k_rstd, w.dqkv, W,
                               w.dqkv + Nq, W, d->qk_norm ? c->rope_scratch : nullptr, dw_out, 1,
                               direct ? 1 : 0, T, d->Hq, d->Hk, hd, d->w_off, d->qk_norm,
                               c->stream));
    if (want_dw && !direct) {
      LB_TRY(lb_colsum(c->wg_tmp, 1, hd, d->qn_wgrad, 1, 1, c->stream));
      LB_TRY(lb_colsum(c->wg_tmp + hd, 1, hd, d->kn_wgrad, 1, 1, c->stream));
    }
  }
  for (int p = 0, col = 0; p < d->qkv.n; ++p) {
    const LbLinear& l = d->qkv.part[p];
    LB_TRY(lin_dgrad(l, w.dqkv + col, W, w.dx1, T, p > 0, w.us, c));
    LB_TRY(lin_wgrad(l, w.dqkv + col, W, s.x1, H, T, s.ts[p], w.us, c));
    col += l.n_out;
  }
  return lb_rms_norm_bwd(w.dx1, w.dres2, stream_in, d->ln1_w, s.rstd1, io->dx, c->norm_scratch,
                         d->ln1_wgrad, 1, 1, T, H, d->w_off, c->stream);
}
