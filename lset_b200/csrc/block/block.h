// One decoder block per call: the launch sequence of a pre-norm transformer block (RMSNorm, QKV
// projection, per-head QK-norm + RoPE, varlen attention, output projection, RMSNorm, gated MLP)
// issued from C++ in one entry point for the forward and one for the backward, so that the host
// cost per block is two foreign calls instead of several dozen.
//
// The structs below are mirrored field by field by ctypes structures in lset_b200/ops/block.py.
// Every pointer is a device pointer; bf16 tensors are row-major with the stated widths.
// Counterpart of the Python-level block of the reference (lset/models/decoder/qwen3/block.py:23-68,
// attention.py:97-167, mlp.py:22-28), which issues the same sequence through torch ops.
#pragma once

#include <stddef.h>

extern "C" {

// y = x · Wᵀ (+ s · (x · Aᵀ) · Bᵀ when lora_r > 0). `wgrad` is the fp32 accumulator that receives
// dW (+=); null means the weight is frozen. Same for the adapter matrices.
struct LbLinear {
  const void* w;        // [n_out, k_in] bf16, row stride ldw
  float* wgrad;         // [n_out, k_in] fp32 contiguous, or null
  const void* lora_a;   // [r, k_in] bf16 contiguous, or null
  const void* lora_b;   // [n_out, r] bf16 contiguous
  float* lora_a_grad;   // [r, k_in] fp32 or null
  float* lora_b_grad;   // [n_out, r] fp32 or null
  long long ldw;
  int n_out;
  int k_in;
  int lora_r;
  float lora_scale;
};

// A projection whose output columns are the concatenation of `n` linears (1 = fused weight).
struct LbProjection {
  LbLinear part[3];
  int n;
  int width;  // total output columns
};

struct LbBlockDesc {
  int H, Hq, Hk, hd, I;
  int causal;
  int act_kind;   // 0 = SwiGLU, 1 = GeGLU(tanh)
  int qk_norm;    // per-head RMSNorm of q and k before RoPE
  float eps, w_off, softmax_scale;
  const void* ln1_w;
  float* ln1_wgrad;
  const void* ln2_w;
  float* ln2_wgrad;
  const void* qn_w;
  float* qn_wgrad;
  const void* kn_w;
  float* kn_wgrad;
  LbProjection qkv;      // columns: q heads, k heads, v heads
  LbProjection gate_up;  // columns: gate, up
  LbLinear o_proj;
  LbLinear down;
};

// Per-forward context of the packed token stream (shared by all blocks of one model forward).
struct LbStreamCtx {
  int T;
  int packed;            // 0: padded batch flattened; rows outside every sequence must stay zero
  const float* cos;
  const float* sin;
  const void* pos;
  int pos_i64;
  const int* seq_start;
  const int* seq_end;
  const int* plan_q;     // tile list for 128 / (Hq / Hk) tokens per tile
  int cap_q;
  const int* plan_kv;    // tile list for 128 tokens per tile (backward)
  int cap_kv;
  int* status;           // device status word for bounded waits
  float* norm_scratch;   // lb_norm_bwd_partial_rows() * H floats
  float* rope_scratch;   // lb_rope_bwd_partial_rows() * 2 * hd floats
  float* wg_tmp;         // 2 * hd floats (QK-norm weight gradient staging)
  void* stream;
};

// Tensor parallelism with a token-sharded residual stream (sequence parallelism): the block's
// input and output hold `rows` tokens of this rank, the column-parallel projections (QKV, gate-up)
// gather the shards of all ranks inside their GEMM and the row-parallel ones (o_proj, down) reduce
// and scatter their output from the GEMM epilogue. The descriptor then carries this rank's head
// and FFN-column counts. Buffers live in symmetric memory owned by the caller: a publication area
// of width H (two halves used alternately, one use per gathered GEMM) and bf16 reduce-scatter
// areas of width H with one slot per source rank (two halves, one use per reduced GEMM). Each of the forward and the backward call makes
// exactly two uses of either and four device barriers; the caller advances its counters by those
// amounts after the call.
struct LbTpCtx {
  int world, rank;
  int rows;                        // token rows of this rank; projections see world * rows tokens
  int reserved;
  const void* const* ag_peers[2];  // per half: host array of `world` device pointers
  void* ag_local[2];               // this rank's half
  unsigned* ag_flags;              // arrival flags of the pulled row tiles (for this row count)
  unsigned* ag_counter;            // work counter of the gather GEMM
  const void* const* rs_peers[2];  // per half: per destination rank, this rank's slot in its area
  void* rs_local[2];               // this rank's area: world slots of rows * H elements
  const void* const* pads;         // device-barrier flag pads of every rank
  unsigned long long bar_limit_ns;
  unsigned ag_epoch;               // uses of the publication area before this call
  unsigned ag_calls;               // uses of these flag words before this call
  unsigned rs_epoch;               // uses of the accumulators before this call
  unsigned bar_epoch;              // barriers passed before this call
};

struct LbBlockIO {
  // forward
  const void* branch;    // [T, H] un-added output of the previous block (or the embeddings)
  const void* residual;  // [T, H] or null (first block: the stream starts at `branch`)
  void* out;             // [T, H] MLP output (un-added)
  void* res_out;         // [T, H] residual stream after the attention branch was added
  void* saved;           // activation arena, lb_block_saved_bytes() bytes, 256-byte aligned
  // backward
  const void* d_out;     // [T, H] gradient of `out`
  const void* d_res_out; // [T, H] gradient of `res_out`, or null
  void* dx;              // [T, H] gradient of `branch` (and of `residual`: they are equal)
  void* work;            // lb_block_work_bytes() bytes, 256-byte aligned
  const LbTpCtx* tp;     // null: the stream is not token-sharded
};

// Bytes of the activation arena the forward fills and the backward reads (`tp` may be null; with it
// T is ignored and the sizes follow world * rows gathered tokens and `rows` local ones).
size_t lb_block_saved_bytes(const LbBlockDesc* d, int T, int has_residual, const LbTpCtx* tp);
// Bytes of temporary storage the backward needs.
size_t lb_block_work_bytes(const LbBlockDesc* d, int T, const LbTpCtx* tp);
// Number of kernel launches the two calls issue (for benchmark reporting).
int lb_block_fwd_launches(const LbBlockDesc* d, const LbStreamCtx* c, int has_residual,
                          const LbTpCtx* tp);
int lb_block_bwd_launches(const LbBlockDesc* d, const LbStreamCtx* c, const LbTpCtx* tp);

// Returns 0, or the negative code of the first launcher that failed.
int lb_block_fwd(const LbBlockDesc* d, const LbStreamCtx* c, const LbBlockIO* io);
int lb_block_bwd(const LbBlockDesc* d, const LbStreamCtx* c, const LbBlockIO* io);

}  // extern "C"
