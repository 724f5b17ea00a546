// Row-wise load/store helpers shared by the general and neighbourhood kernels.
// VEC = rows are channel-contiguous, 16-byte aligned, D a multiple of 8.
#pragma once
#include "kfa_common.cuh"

namespace kfa {

template <typename T, bool VEC>
__device__ __forceinline__ void load8(const T* row, int64_t stride, int d, int D, float (&x)[8]) {
    if constexpr (VEC) {
        uint4 raw = *reinterpret_cast<const uint4*>(row + d);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = to_float<T>(e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (d + i < D) ? to_float<T>(row[(int64_t)(d + i) * stride]) : 0.f;
    }
}

template <typename T, bool VEC>
__device__ __forceinline__ float2 load2(const T* row, int64_t stride, int d, int D) {
    if constexpr (VEC) {
        uint32_t raw = *reinterpret_cast<const uint32_t*>(row + d);
        const T* e = reinterpret_cast<const T*>(&raw);
        return make_float2(to_float<T>(e[0]), to_float<T>(e[1]));
    } else {
        float a = d < D ? to_float<T>(row[(int64_t)d * stride]) : 0.f;
        float b = d + 1 < D ? to_float<T>(row[(int64_t)(d + 1) * stride]) : 0.f;
        return make_float2(a, b);
    }
}

template <typename T, bool VEC>
__device__ __forceinline__ void store2(T* row, int64_t stride, int d, int D, float a, float b) {
    if constexpr (VEC) {
        T pair[2] = {from_float<T>(a), from_float<T>(b)};
        *reinterpret_cast<uint32_t*>(row + d) = *reinterpret_cast<uint32_t*>(pair);
    } else {
        if (d < D) row[(int64_t)d * stride] = from_float<T>(a);
        if (d + 1 < D) row[(int64_t)(d + 1) * stride] = from_float<T>(b);
    }
}

// Copies R rows (or zero rows past `limit`) into shared memory as FP32, padded to a multiple of 8.
template <typename T, int R>
__device__ __forceinline__ void stage_rows(float* dst, int Dp, const T* base, int64_t row_stride, int64_t d_stride,
                                           int row0, int limit, int D, int lane) {
    for (int r = 0; r < R; ++r)
        for (int d = lane; d < Dp; d += 32)
            dst[r * Dp + d] = (row0 + r < limit && d < D)
                                  ? to_float<T>(base[(int64_t)(row0 + r) * row_stride + (int64_t)d * d_stride])
                                  : 0.f;
}

}  // namespace kfa
