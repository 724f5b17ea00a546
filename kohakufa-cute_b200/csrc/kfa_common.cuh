// Shared parameter blocks and small device helpers for all attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <math.h>

// Grids below this many CTAs are ordered tile row by tile row over all heads (see the pipeline kernels).
#ifndef KFA_ROW_MAJOR_LIMIT
#define KFA_ROW_MAJOR_LIMIT (4 * 148)
#endif

namespace kfa {

constexpr float kLog2e = 1.4426950408889634f;

// Operands of one attention call.  Strides are in elements; index order is
// (batch, head, sequence, channel).  Unused pointers are null.
struct AttnParams {
    const void* q;
    const void* k;
    const void* v;
    const uint8_t* mask;  // bool, expanded to [B,Hq,Sq,Sk] with stride 0 on broadcast axes
    void* out;            // forward output (written) or saved output (read by backward)
    float* maximum;       // [B,Hq,Sq]
    float* logsum;        // [B,Hq,Sq]
    const void* dout;
    float* delta;         // [B,Hq,Sq] scratch: sum_d O * dO
    float* aux;           // [B,Hq,Sq] scratch: neighbourhood correction t
    void* dq;
    void* dk;
    void* dv;
    int32_t* blocks;      // 64x64 mask tile states
    int64_t qs[4], ks[4], vs[4], os[4], ms[4], gs[4], dqs[4], dks[4], dvs[4];
    int64_t bs[4];        // strides of `blocks` (0 on collapsed axes)
    int B, Hq, Hkv, Sq, Sk, D, group;
    float scale;
    int causal;
    int has_mask;
    // neighbourhood geometry (nd = 0 for ordinary attention); axis order slowest..fastest,
    // 2-D grids use ext[0] = 1, win[0] = 1.
    int nd;
    int ext[3];
    int win[3];
    int two_term;
    // Block-wise calls (one block of a longer key sequence, or one of its gradient contributions):
    // running != 0: the forward folds its block into a running FP32 state instead of writing a normalised output:
    //   `out` is the unnormalised FP32 accumulator [B,Hq,Sq,D] (strides `os`), `maximum` the running unscaled row
    //   maximum and `run_sum` the running sum of probabilities relative to it (both [B,Hq,Sq], unit row stride,
    //   batch and head strides `ss`).
    // grad_f32 bit 0: dq/dk/dv are FP32 tensors; bit 1: add to dq instead of overwriting it; bit 2: same for dk, dv.
    float* run_sum;
    int64_t ss[2];
    // Wide-head backward in passes over key ranges (sequences whose stored score matrices exceed the workspace
    // limit): the pass sees keys [k0, k0 + Sk) of the call, so a key is visible under a causal mask iff
    // col <= row + causal_shift (causal_shift = -k0), and dQ accumulates over the passes in FP32:
    // dq_pass 0 = single pass (write the 16-bit gradient), 1 = first (write dq_acc), 2 = middle (add to dq_acc),
    // 3 = last (add dq_acc, write the 16-bit gradient).  dq_acc is [B,Hq,Sq,D] of the pass, contiguous.
    int causal_shift;
    int dq_pass;
    float* dq_acc;
    int running;
    int grad_f32;
    int* status;      // device-visible status word (mapped host memory)
    int* abort_flag;  // device memory: set by the first CTA whose bounded wait gives up; later CTAs skip their work
};

// (batch, head, position) of row `row_id` of a [B, H, S] row space.  32-bit divisions when the index fits: a 64-bit
// division costs more instructions than the loads of a row in the row-wise kernels.
__device__ __forceinline__ void split_row(int64_t row_id, int S, int H, int& s, int& h, int& b) {
    if (row_id <= 0xffffffffll) {
        const uint32_t head = (uint32_t)row_id / (uint32_t)S;
        s = (int)((uint32_t)row_id - head * (uint32_t)S);
        b = (int)(head / (uint32_t)H);
        h = (int)(head - (uint32_t)b * (uint32_t)H);
    } else {
        s = (int)(row_id % S);
        h = (int)((row_id / S) % H);
        b = (int)(row_id / ((int64_t)S * H));
    }
}

template <typename T>
__device__ __forceinline__ float to_float(T x);
template <>
__device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// One round trip through the 16-bit type.
template <typename T>
__device__ __forceinline__ float round_low(float x) { return to_float<T>(from_float<T>(x)); }

__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Window start of a neighbourhood query on one axis: clamp(p - w/2, 0, e - w).
__host__ __device__ __forceinline__ int na_start(int p, int e, int w) {
    int s = p - w / 2;
    s = s < 0 ? 0 : s;
    return s > e - w ? e - w : s;
}
// Inclusive range of query coordinates whose window holds key coordinate `c`.
__host__ __device__ __forceinline__ void na_inverse(int c, int e, int w, int& lo, int& hi) {
    lo = (c - w + 1 <= 0) ? 0 : c - w + 1 + w / 2;
    hi = (c >= e - w) ? e - 1 : c + w / 2;
}

}  // namespace kfa
