// Host-side construction of TMA tensor maps. The driver entry point is resolved through the CUDA
// runtime so that the library has no link-time dependency on libcuda (it can be built and loaded
// on a machine without a GPU driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {

// Returns 0 on success, otherwise a negative code (-1: entry point unavailable, -(2000 + CUresult): encode failed,
// -3: arguments break a TMA rule that the driver does not check).
//
// 2-D bf16 tensor: `inner` contiguous elements per row, `outer` rows, `row_stride_bytes` between
// rows (multiple of 16). Box = box_inner x box_outer elements; box_inner * 2 must be 128 when
// swizzle128 is set (the only mode the UMMA kernels here consume).
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128);

}  // namespace lb
