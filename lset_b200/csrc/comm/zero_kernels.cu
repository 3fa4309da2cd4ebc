// Sharded-optimizer collectives fused with their compute, over NVLink peer memory.
//
// Every rank keeps, per parameter group, a full fp32 gradient buffer and a full bf16 parameter
// buffer in symmetric memory (same size on all ranks, all peers mapped). Rank r owns the slice
// [lo, lo + n) of each.
//
//   reduce_shard   g[i] = scale * sum_p grad_p[lo + i]   (p over all ranks, plain peer loads, fp32
//                  accumulation in a rank-rotated order)  + per-CTA sum of squares for the norm.
//                  = reduce-scatter fused with the averaging and the gradient-norm reduction.
//   adamw_push     AdamW on the owned slice (fp32 master + moments), then the new bf16 values are
//                  stored into EVERY rank's parameter buffer = optimizer step fused with the
//                  parameter all-gather (a push: each byte crosses NVLink once per peer).
//
// Neither kernel waits on another GPU itself. Ordering between ranks (gradients complete before
// they are read, pushes complete before the next forward) comes from a launch placed in front of
// them on the same stream: by default the device barrier of comm/probe.cu, a kernel that spins,
// with an iteration limit, on flags in symmetric memory and reports a peer that never arrives
// through the status word; with LSET_B200_DEVICE_BARRIER=0 a one-element NCCL all-reduce instead.
// The AdamW kernel honours the skip flag that the clip-coefficient kernel derives from the status
// words of all ranks, so a step whose barrier timed out changes no parameter.
//
// Replaces, for the sharded runtime, the NCCL reduce-scatter / all-gather that FSDP2 issues for the
// reference (lset/distributed/parallel.py:129-160) plus clip_grad_norm_ and AdamW(fused=True)
// (lset/train/engine.py:258-264,399-406).
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;
constexpr int kMaxPeers = 16;

struct PeerPtrs {
  void* p[kMaxPeers];
};

__global__ void __launch_bounds__(256)
    reduce_shard_kernel(PeerPtrs grads, int world, int rank, long long lo, long long n, float scale,
                        float* __restrict__ out, float* __restrict__ sumsq_partial, int accumulate) {
  __shared__ float sred[8];
  float ss = 0.f;
  const long long n4 = n / 4;
  // Four independent 16-byte loads per thread and peer are issued before any is consumed: with
  // one load in flight per thread the NVLink round trip, not the link, sets the rate.
  constexpr int U = 4;
  const long long stride = 1LL * gridDim.x * blockDim.x;
  for (long long i0 = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += U * stride) {
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < world; ++k) {
      const int p = (rank + k) % world;  // start with the local copy, then walk the peers
      const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[p]) + lo);
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        v[u] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[u].x += v[u].x;
        acc[u].y += v[u].y;
        acc[u].z += v[u].z;
        acc[u].w += v[u].w;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) break;
      float4 a = acc[u];
      a.x *= scale;
      a.y *= scale;
      a.z *= scale;
      a.w *= scale;
      if (accumulate) {  // micro-steps of gradient accumulation add up in the shard
        const float4 o = reinterpret_cast<const float4*>(out)[i];
        a.x += o.x;
        a.y += o.y;
        a.z += o.z;
        a.w += o.w;
      }
      reinterpret_cast<float4*>(out)[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) {
      float a = 0.f;
      for (int k = 0; k < world; ++k)
        a += static_cast<const float*>(grads.p[(rank + k) % world])[lo + i];
      a *= scale;
      if (accumulate) a += out[i];
      out[i] = a;
      ss += a * a;
    }
  }
  ss = row_sum<256>(ss, sred);
  if (threadIdx.x == 0) sumsq_partial[blockIdx.x] = ss;
}

__global__ void __launch_bounds__(256)
    sumsq_fold_kernel(const float* __restrict__ partial, int P, float* __restrict__ out) {
  __shared__ float sred[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) s += partial[i];
  s = row_sum<256>(s, sred);
  if (threadIdx.x == 0) out[0] += s;
}

struct AdamPushArgs {
  float* p;
  const float* g;
  float* m;
  float* v;
  PeerPtrs params;  // bf16 parameter buffers of all ranks
  int world, rank;
  long long lo, n;
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt;
  const float* coef;
};

__global__ void __launch_bounds__(256) adamw_push_kernel(AdamPushArgs a) {
  if (a.coef != nullptr && a.coef[2] != 0.f) return;   // the step was marked faulted: apply nothing
  const float gs = a.coef != nullptr ? a.coef[0] : 1.f;
  const float step = a.lr / a.bc1;
  const float decay = 1.f - a.lr * a.wd;
  const long long n4 = a.n / 4;
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += 1LL * gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(a.p)[i];
    const float4 g = reinterpret_cast<const float4*>(a.g)[i];
    float4 m = reinterpret_cast<float4*>(a.m)[i];
    float4 v = reinterpret_cast<float4*>(a.v)[i];
    float* pp = &p.x;
    const float* gp = &g.x;
    float* mp = &m.x;
    float* vp = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gp[j] * gs;
      mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gj;
      vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
      pp[j] = pp[j] * decay - step * mp[j] / (sqrtf(vp[j]) / a.bc2_sqrt + a.eps);
    }
    reinterpret_cast<float4*>(a.p)[i] = p;
    reinterpret_cast<float4*>(a.m)[i] = m;
    reinterpret_cast<float4*>(a.v)[i] = v;
    __nv_bfloat162 lo2 = __floats2bfloat162_rn(p.x, p.y);
    __nv_bfloat162 hi2 = __floats2bfloat162_rn(p.z, p.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo2);
    o.y = *reinterpret_cast<uint32_t*>(&hi2);
    for (int k = 0; k < a.world; ++k) {
      bf16* dst = static_cast<bf16*>(a.params.p[(a.rank + k) % a.world]) + a.lo;
      reinterpret_cast<uint2*>(dst)[i] = o;
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < a.n; i += blockDim.x) {
      const float gj = a.g[i] * gs;
      const float mj = a.beta1 * a.m[i] + (1.f - a.beta1) * gj;
      const float vj = a.beta2 * a.v[i] + (1.f - a.beta2) * gj * gj;
      const float pj = a.p[i] * decay - step * mj / (sqrtf(vj) / a.bc2_sqrt + a.eps);
      a.p[i] = pj;
      a.m[i] = mj;
      a.v[i] = vj;
      for (int k = 0; k < a.world; ++k)
        (static_cast<bf16*>(a.params.p[(a.rank + k) % a.world]) + a.lo)[i] = __float2bfloat16_rn(pj);
    }
  }
}

// dst[r * n16 + i] = shard of rank r (16-byte vectors), own shard first, then the peers in
// rank-rotated order so that the ranks do not all read the same peer at the same time.
__global__ void __launch_bounds__(256)
    gather_shards_kernel(PeerPtrs shards, int world, int rank, long long n16, uint4* __restrict__ dst) {
  for (int k = 0; k < world; ++k) {
    const int p = (rank + k) % world;
    const uint4* src = static_cast<const uint4*>(shards.p[p]);
    uint4* out = dst + 1LL * p * n16;
    constexpr int U = 4;   // loads in flight per thread (NVLink round trips overlap)
    const long long stride = 1LL * gridDim.x * blockDim.x;
    for (long long i0 = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i0 < n16; i0 += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < n16) v[u] = src[i0 + u * stride];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * stride < n16) out[i0 + u * stride] = v[u];
    }
  }
}

int comm_grid(long long n4) {
  long long g = (n4 + 255) / 256;
  const long long cap = 1LL * row_num_sms() * 4;
  if (g > cap) g = cap;
  return int(g < 1 ? 1 : g);
}

}  // namespace
}  // namespace lb

using namespace lb;

extern "C" int lb_reduce_shard_partial_rows() { return row_num_sms() * 4; }

// grad_ptrs: host array of `world` device pointers (fp32 full gradient buffers, own included).
// out: fp32 [n]; sumsq: device scalar that receives += sum(out^2); scratch: partial_rows floats.
// lo must be a multiple of 4 elements. accumulate: out += result (the sum of squares is then that of
// the accumulated values).
extern "C" int lb_reduce_shard_f32(const void* const* grad_ptrs, int world, int rank, long long lo,
                                   long long n, float scale, float* out, float* scratch,
                                   float* sumsq, int accumulate, void* stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > kMaxPeers || (lo & 3)) return -3;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = const_cast<void*>(grad_ptrs[i]);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = comm_grid(n / 4);
  reduce_shard_kernel<<<grid, 256, 0, st>>>(pp, world, rank, lo, n, scale, out, scratch, accumulate);
  if (sumsq != nullptr) sumsq_fold_kernel<<<1, 256, 0, st>>>(scratch, grid, sumsq);
  return launch_rc();
}

// Parameter all-gather over peer memory (sharded-parameter mode): every rank holds one shard of
// `bytes` bytes (a multiple of 16) in symmetric memory; dst receives all of them in rank order.
// Plain peer loads; the caller orders "shards final on every rank" before this launch.
extern "C" int lb_gather_shards(const void* const* shard_ptrs, int world, int rank, long long bytes,
                                void* dst, void* stream) {
  if (bytes <= 0) return 0;
  if (world < 1 || world > kMaxPeers || (bytes & 15)) return -3;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = const_cast<void*>(shard_ptrs[i]);
  gather_shards_kernel<<<comm_grid(bytes / 16), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      pp, world, rank, bytes / 16, static_cast<uint4*>(dst));
  return launch_rc();
}

// param_ptrs: host array of `world` device pointers to the bf16 parameter buffers of all ranks.
extern "C" int lb_adamw_push(float* p, const float* g, float* m, float* v,
                             const void* const* param_ptrs, int world, int rank, long long lo,
                             long long n, float lr, float beta1, float beta2, float eps, float wd,
                             float bc1, float bc2_sqrt, const float* coef, void* stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > kMaxPeers || (lo & 3)) return -3;
  AdamPushArgs a;
  a.p = p;
  a.g = g;
  a.m = m;
  a.v = v;
  for (int i = 0; i < world; ++i) a.params.p[i] = const_cast<void*>(param_ptrs[i]);
  a.world = world;
  a.rank = rank;
  a.lo = lo;
  a.n = n;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.wd = wd;
  a.bc1 = bc1;
  a.bc2_sqrt = bc2_sqrt;
  a.coef = coef;
  adamw_push_kernel<<<comm_grid(n / 4), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return launch_rc();
}

// ------------------------------------------------------------------------------------------------
// take_clear: out (bf16) = acc, acc = 0 in one pass. The reduce-scatter accumulators of the fused
// tensor-parallel GEMMs are read once and must be zero again before their next use.
namespace lb {
namespace {

template <bool ACC_FP32>
__global__ void __launch_bounds__(256)
    take_clear_kernel(void* __restrict__ acc, bf16* __restrict__ out, long long n8) {
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += 1LL * gridDim.x * blockDim.x) {
    if constexpr (ACC_FP32) {
      float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
      const float4 x = a[0], y = a[1];
      const float v[8] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w};
      st16(out + 8 * i, pack8(v));
      a[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      uint4* a = reinterpret_cast<uint4*>(acc) + i;
      st16(out + 8 * i, *a);
      *a = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// out[i] = sum over w of slots[w * n + i] (bf16 slots, fp32 sum in slot order, bf16 result).
template <int W>
__global__ void __launch_bounds__(256)
    take_sum_kernel(const bf16* __restrict__ slots, bf16* __restrict__ out, long long n8) {
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += 1LL * gridDim.x * blockDim.x) {
    uint4 part[W];
#pragma unroll
    for (int w = 0; w < W; ++w) part[w] = *reinterpret_cast<const uint4*>(slots + (w * n8 + i) * 8);
    float v[8];
    unpack8(part[0], v);
#pragma unroll
    for (int w = 1; w < W; ++w) {
      float u[8];
      unpack8(part[w], u);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += u[j];
    }
    st16(out + 8 * i, pack8(v));
  }
}

}  // namespace
}  // namespace lb

// slots: world x n bf16 (slot w holds rank w's partial result), out: n bf16; n a multiple of 8.
extern "C" int lb_take_sum(const void* slots, void* out, long long n, int world, void* stream) {
  using namespace lb;
  if (n <= 0) return 0;
  if ((n & 7) || world < 1 || world > 8) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = comm_grid(n / 8);
  const bf16* s = reinterpret_cast<const bf16*>(slots);
  bf16* o = reinterpret_cast<bf16*>(out);
  switch (world) {
    case 1: take_sum_kernel<1><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    case 2: take_sum_kernel<2><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    case 3: take_sum_kernel<3><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    case 4: take_sum_kernel<4><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    case 5: take_sum_kernel<5><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    case 6: take_sum_kernel<6><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    case 7: take_sum_kernel<7><<<grid, 256, 0, st>>>(s, o, n / 8); break;
    default: take_sum_kernel<8><<<grid, 256, 0, st>>>(s, o, n / 8); break;
  }
  return launch_rc();
}

// acc: n elements (fp32 when acc_fp32, else bf16), out: n bf16; n a multiple of 8, both 16-byte
// aligned.
extern "C" int lb_take_clear(void* acc, void* out, long long n, int acc_fp32, void* stream) {
  if (n <= 0) return 0;
  if (n & 7) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = comm_grid(n / 8);
  if (acc_fp32)
    take_clear_kernel<true><<<grid, 256, 0, st>>>(acc, reinterpret_cast<bf16*>(out), n / 8);
  else
    take_clear_kernel<false><<<grid, 256, 0, st>>>(acc, reinterpret_cast<bf16*>(out), n / 8);
  return launch_rc();
}
