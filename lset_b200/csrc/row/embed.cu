// Embedding lookup (up to three tables summed, for BERT's word + position + token-type) and its
// backward, which scatters token gradients into fp32 table gradients with vector reductions.
// Replaces the aten embedding ops used at lset/models/decoder/qwen3/model.py:63,109 and
// lset/models/encoder/bert/model.py:14-44.
#include "../common/row.cuh"

namespace lb {
namespace {

using bf16 = __nv_bfloat16;

__global__ void __launch_bounds__(256)
    embed_fwd_kernel(const long long* __restrict__ ids0, const bf16* __restrict__ tab0,
                     const long long* __restrict__ ids1, const bf16* __restrict__ tab1,
                     const long long* __restrict__ ids2, const bf16* __restrict__ tab2,
                     bf16* __restrict__ out, long long T, int H, float scale) {
  const int vec_per_row = H / 8;
  const long long total = T * vec_per_row;
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += 1LL * gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = int(i % vec_per_row) * 8;
    float a[8];
    unpack8(ld16(tab0 + ids0[t] * H + c), a);
    if (tab1 != nullptr) {
      float b[8];
      unpack8(ld16(tab1 + ids1[t] * H + c), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    if (tab2 != nullptr) {
      float b[8];
      unpack8(ld16(tab2 + ids2[t] * H + c), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
    }
    if (scale != 1.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] *= scale;
    }
    st16(out + t * H + c, pack8(a));
  }
}

__global__ void __launch_bounds__(256)
    embed_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dy,
                     float* __restrict__ dtab, long long T, int H, float scale) {
  const int vec_per_row = H / 8;
  const long long total = T * vec_per_row;
  for (long long i = 1LL * blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += 1LL * gridDim.x * blockDim.x) {
    const long long t = i / vec_per_row;
    const int c = int(i % vec_per_row) * 8;
    float g[8];
    unpack8(ld16(dy + t * H + c), g);
    float* dst = dtab + ids[t] * H + c;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(g[0] * scale),
                 "f"(g[1] * scale), "f"(g[2] * scale), "f"(g[3] * scale)
                 : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(g[4] * scale),
                 "f"(g[5] * scale), "f"(g[6] * scale), "f"(g[7] * scale)
                 : "memory");
  }
}

int flat_grid(long long work_items) {
  long long g = (work_items + 255) / 256;
  const long long cap = 1LL * row_num_sms() * 16;
  if (g > cap) g = cap;
  return int(g > 0 ? g : 1);
}

}  // namespace
}  // namespace lb

using namespace lb;

// out[t] = scale * (tab0[ids0[t]] + tab1[ids1[t]] + tab2[ids2[t]]); tab1/tab2 may be null.
extern "C" int lb_embedding_fwd(const long long* ids0, const void* tab0, const long long* ids1,
                                const void* tab1, const long long* ids2, const void* tab2,
                                void* out, long long T, int H, float scale, void* stream) {
  if (T <= 0) return 0;
  if (H & 7) return -3;
  embed_fwd_kernel<<<flat_grid(T * (H / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids0, (const bf16*)tab0, ids1, (const bf16*)tab1, ids2, (const bf16*)tab2, (bf16*)out, T, H,
      scale);
  return launch_rc();
}

// dtab[ids[t]] += scale * dy[t]   (fp32 table gradient, must be initialised by the caller)
extern "C" int lb_embedding_bwd(const long long* ids, const void* dy, float* dtab, long long T,
                                int H, float scale, void* stream) {
  if (T <= 0) return 0;
  if (H & 7) return -3;
  embed_bwd_kernel<<<flat_grid(T * (H / 8)), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ids, (const bf16*)dy, dtab, T, H, scale);
  return launch_rc();
}
