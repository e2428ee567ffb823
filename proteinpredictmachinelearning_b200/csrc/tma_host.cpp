#include "tma_host.h"

#include <mutex>

namespace ppml_b200 {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

}  // namespace

bool make_tmap_3d(CUtensorMap* out, TmaType type, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                  uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, int swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    CUtensorMapDataType dt;
    switch (type) {
        case TmaType::F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
        case TmaType::TF32: dt = CU_TENSOR_MAP_DATA_TYPE_TFLOAT32; break;
        case TmaType::F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
        case TmaType::BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (stride1_bytes & 15u) || (stride2_bytes & 15u)) return false;
    if (d0 == 0 || d1 == 0 || d2 == 0) return false;
    // a degenerate outer extent still needs a legal stride
    if (stride2_bytes == 0) stride2_bytes = stride1_bytes * d1;
    cuuint64_t gdim[3] = {d0, d1, d2};
    cuuint64_t gstride[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle == 4 ? CU_TENSOR_MAP_SWIZZLE_32B : swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_64B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                            : (swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_tmap_4d(CUtensorMap* out, TmaType type, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                  uint64_t stride1_bytes, uint64_t stride2_bytes, uint64_t stride3_bytes, uint32_t box0, uint32_t box1, int swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    CUtensorMapDataType dt;
    switch (type) {
        case TmaType::F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
        case TmaType::TF32: dt = CU_TENSOR_MAP_DATA_TYPE_TFLOAT32; break;
        case TmaType::F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
        case TmaType::BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (stride1_bytes & 15u) || (stride2_bytes & 15u) || (stride3_bytes & 15u)) return false;
    if (d0 == 0 || d1 == 0 || d2 == 0 || d3 == 0 || stride1_bytes == 0 || stride2_bytes == 0) return false;
    if (stride3_bytes == 0) stride3_bytes = stride2_bytes * d2;      // a degenerate outer extent still needs a legal stride
    cuuint64_t gdim[4] = {d0, d1, d2, d3};
    cuuint64_t gstride[3] = {stride1_bytes, stride2_bytes, stride3_bytes};
    cuuint32_t box[4] = {box0, box1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, dt, 4, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle == 4 ? CU_TENSOR_MAP_SWIZZLE_32B : swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_64B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                            : (swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace ppml_b200
