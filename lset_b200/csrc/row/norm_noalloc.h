// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this
// library whose code runs where an allocation is not possible: inside a region that another
// framework's allocator already owns in full, in a real-time serving loop that forbids
// cudaMalloc's implicit device synchronisation, or in a host process that has handed every byte
// of the GPU to a memory pool it cannot grow. Such a caller can still provide the inputs and the
// outputs, but not the scratch buffer that the regular lb_rms_norm_bwd needs for its per-CTA
// weight-gradient partials.
//
// lb_rms_norm_bwd_noalloc computes exactly what lb_rms_norm_bwd computes (same kernels), but the
// partials live in one fixed array inside the library image (5 MiB of device memory per GPU that
// loads the library, held until the process exits). It calls no cudaMalloc / cudaFree and no
// allocating library routine.
//
// Limits and rules:
//   * H (row width) must be a multiple of 8 and at most LB_NOALLOC_MAX_H; larger rows are rejected
//     with LB_NOALLOC_ERR_TOO_LARGE (nothing is launched). N (rows) is unlimited.
//   * The first call on each device looks the array's device address up once (with that device
//     current). Make that first call outside any CUDA stream capture.
//   * All calls share the one array per device and it keeps whatever the last call left in it.
//     Nothing in it has to start at zero: every partial row that the reduction reads is rewritten
//     by the same call first. Two calls that overlap on the GPU (different streams, or two host
//     threads) race on the array: serialise them on one stream or with events.
#pragma once

#define LB_NOALLOC_MAX_H 4096
#define LB_NOALLOC_MAX_PARTIAL_ROWS 320
#define LB_NOALLOC_ERR_TOO_LARGE (-20)  // H > LB_NOALLOC_MAX_H
#define LB_NOALLOC_ERR_SYMBOL (-21)     // cudaGetSymbolAddress failed for the current device
#define LB_NOALLOC_ERR_DEVICE (-22)     // device index outside the table kept by the library

#ifdef __cplusplus
extern "C" {
#endif

// dy, dres (nullable), xin, w: bf16 inputs as for lb_rms_norm_bwd; rstd: fp32 [N];
// dx: bf16 [N, H] output; dw_out: [H] output, fp32 (dw_fp32 = 1) or bf16, overwritten or, with
// dw_accumulate = 1, added to. Returns 0, a negative LB_NOALLOC_ERR_* code, or the launch error
// codes of the library (-3 bad shape, -11 launch failure).
int lb_rms_norm_bwd_noalloc(const void* dy, const void* dres, const void* xin, const void* w,
                            const float* rstd, void* dx, void* dw_out, int dw_fp32,
                            int dw_accumulate, int N, int H, float w_off, void* stream);

// Human-readable text for a return code of the function above.
const char* lb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
