#include "tensor_map.h"

#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <mutex>

namespace kfa {
namespace {

PFN_cuTensorMapEncodeTiled encoder() {
    static PFN_cuTensorMapEncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(ptr);
    });
    return fn;
}

}  // namespace

bool tma_compatible(const void* ptr, const int64_t* strides, int64_t B, int64_t H, int64_t S) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || strides[3] != 1) return false;
    const int64_t extent[3] = {B, H, S};
    for (int i = 0; i < 3; ++i) {
        if (extent[i] == 1) continue;
        if (strides[i] <= 0 || strides[i] % 8 != 0 || strides[i] >= (int64_t(1) << 38)) return false;
    }
    return true;
}

bool encode_bhsd_map(CUtensorMap* map, const void* ptr, CUtensorMapDataType dtype, int64_t D, int64_t S, int64_t H,
                     int64_t B, const int64_t* strides, int box_channels, int box_rows) {
    PFN_cuTensorMapEncodeTiled fn = encoder();
    if (!fn) return false;
    // A stride of an extent-1 axis is never used for addressing; give it a legal value.
    const int64_t row_bytes = ((D * 2 + 15) / 16) * 16;
    auto bytes = [&](int64_t extent, int64_t stride) -> cuuint64_t {
        return extent == 1 ? (cuuint64_t)row_bytes : (cuuint64_t)(stride * 2);
    };
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t gstrides[3] = {bytes(S, strides[2]), bytes(H, strides[1]), bytes(B, strides[0])};
    cuuint32_t box[4] = {(cuuint32_t)box_channels, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = fn(map, dtype, 4, const_cast<void*>(ptr), dims, gstrides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace kfa
