// tma_host.h -- host-side construction of TMA tensor maps.  The driver entry point is looked up
// through the runtime (cudaGetDriverEntryPoint), so the library does not link libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ppml_b200 {

enum class TmaType { F32, TF32, F16, BF16, U8 };

// 3-D row-major tensor [d2][d1][d0] (d0 innermost, contiguous).  stride1/stride2 are byte strides
// of d1 and d2 and must be multiples of 16; base must be 16-byte aligned.  The box is
// box0 x box1 x 1.  swizzle: 0 none, 1 the 128-byte swizzle (16-byte chunks; box0 * element size == 128),
// 2 the 128-byte swizzle with 32-byte chunks (the only layout the tensor core reads 32-bit operands from
// when their row index, not K, is contiguous), 3 the 64-byte swizzle (box0 * element size == 64), 4 the 32-byte swizzle
// (box0 * element size == 32).
// Out-of-range elements read as zero.  Returns false when the driver rejects the arguments.
bool make_tmap_3d(CUtensorMap* out, TmaType type, const void* base,
                  uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
                  uint32_t box0, uint32_t box1, int swizzle);

// The same for a 4-D tensor [d3][d2][d1][d0] with arbitrary (16-byte multiple) strides of d1, d2 and d3; box0 x box1 x 1 x 1.
// The strides need not be ordered: d1 may be the dimension with the largest stride.
bool make_tmap_4d(CUtensorMap* out, TmaType type, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                  uint64_t stride1_bytes, uint64_t stride2_bytes, uint64_t stride3_bytes, uint32_t box0, uint32_t box1, int swizzle);

inline int tma_elem_size(TmaType t) {
    switch (t) { case TmaType::F32: case TmaType::TF32: return 4; case TmaType::F16: case TmaType::BF16: return 2; default: return 1; }
}

}  // namespace ppml_b200
