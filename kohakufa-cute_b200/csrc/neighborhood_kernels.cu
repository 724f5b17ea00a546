// Neighbourhood (shifted-window) attention, head dim 64, 2-D and 3-D grids.
//
// Every query sees exactly prod(window) keys: on each axis the window starts at
// clamp(q - w/2, 0, extent - w).  The kernels enumerate exactly those keys (and,
// for the key/value gradients, exactly the queries whose window holds the key),
// so no score outside the window is ever computed.  One warp owns one row of
// its output; a lane takes one neighbour per step.
//
// Arithmetic (reference: docs/precision.md:46-80 and
// src/kohakufa_cute/neighborhood_kernels.py:193-212, 348-365 of the reference
// project):
//   forward     as ordinary attention; 3-D grids add the rounding residual of the
//               weight as a second product term (hi = round(p), lo = round(p - hi)).
//   backward    P32 = ex2((s' - m)|scale|log2e - logsum) stays FP32 when forming dS.
//     query     dS_q = round(P32 (dP - delta));
//               dQ = (sum dS_q K - (sum dS_q / sum round(P32)) sum round(P32) K) * scale;
//               publishes t = sum P32 (dP - delta) / sum P32.
//     key       dS_k = round(P32 ((dP - delta) - t)); dK = (sum dS_k Q) * scale.
//     value     dV = sum round(P32) dO.
#include "kfa_common.cuh"
#include "row_access.cuh"
#include "launchers.h"

namespace kfa {
namespace {

constexpr int kD = 64;

struct Coord {
    int z, y, x;
};
__device__ __forceinline__ Coord unflatten(const AttnParams& p, int token) {
    Coord c;
    c.x = token % p.ext[2];
    const int t = token / p.ext[2];
    c.y = t % p.ext[1];
    c.z = t / p.ext[1];
    return c;
}

template <typename T, bool VEC>
__device__ __forceinline__ float dot64(const float* a, const T* row, int64_t stride) {
    float s = 0.f;
#pragma unroll
    for (int d = 0; d < kD; d += 8) {
        float x[8];
        load8<T, VEC>(row, stride, d, kD, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += a[d + i] * x[i];
    }
    return s;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(128) na_forward(AttnParams p) {
    __shared__ float sq[4][kD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row_id = (int64_t)blockIdx.x * 4 + warp;
    if (row_id >= (int64_t)p.B * p.Hq * p.Sq) return;
    int row, h, b;
    split_row(row_id, p.Sq, p.Hq, row, h, b);
    const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)h * p.qs[1] + (int64_t)row * p.qs[2];
    const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)h * p.ks[1];
    const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)h * p.vs[1];
    for (int d = lane; d < kD; d += 32) sq[warp][d] = to_float<T>(qrow[(int64_t)d * p.qs[3]]);
    __syncwarp();
    const Coord qc = unflatten(p, row);
    const int z0 = na_start(qc.z, p.ext[0], p.win[0]), y0 = na_start(qc.y, p.ext[1], p.win[1]),
              x0 = na_start(qc.x, p.ext[2], p.win[2]);
    const int W = p.win[0] * p.win[1] * p.win[2], wyx = p.win[1] * p.win[2];
    const float sign = p.scale >= 0.f ? 1.f : -1.f;
    const float c2 = fabsf(p.scale) * kLog2e;
    float m = -INFINITY, l = 0.f, a0 = 0.f, a1 = 0.f;
    for (int t0 = 0; t0 < W; t0 += 32) {
        const int idx = t0 + lane;
        const bool valid = idx < W;
        int key = 0;
        float sp = -INFINITY;
        if (valid) {
            const int dz = idx / wyx, rem = idx % wyx;
            key = ((z0 + dz) * p.ext[1] + (y0 + rem / p.win[2])) * p.ext[2] + x0 + rem % p.win[2];
            sp = dot64<T, VEC>(sq[warp], kb + (int64_t)key * p.ks[2], p.ks[3]) * sign;
        }
        const float m_new = fmaxf(m, warp_max(sp));
        const float alpha = (m == -INFINITY) ? 0.f : fast_ex2((m - m_new) * c2);
        const float pr = valid ? fast_ex2((sp - m_new) * c2) : 0.f;
        l = l * alpha + warp_sum(pr);
        a0 *= alpha;
        a1 *= alpha;
        m = m_new;
        const float hi = round_low<T>(pr);
        const float lo = p.two_term ? round_low<T>(pr - hi) : 0.f;
        const int jn = min(32, W - t0);
        for (int j = 0; j < jn; ++j) {
            const float hj = __shfl_sync(0xffffffffu, hi, j), lj = __shfl_sync(0xffffffffu, lo, j);
            const int kj = __shfl_sync(0xffffffffu, key, j);
            const float2 x = load2<T, VEC>(vb + (int64_t)kj * p.vs[2], p.vs[3], 2 * lane, kD);
            a0 += hj * x.x;
            a1 += hj * x.y;
            if (p.two_term) {
                a0 += lj * x.x;
                a1 += lj * x.y;
            }
        }
    }
    const float den = l > 0.f ? l : 1.f;
    T* orow = reinterpret_cast<T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] + (int64_t)row * p.os[2];
    store2<T, VEC>(orow, p.os[3], 2 * lane, kD, a0 / den, a1 / den);
    if (lane == 0) {
        p.maximum[row_id] = m;
        p.logsum[row_id] = log2f(den);
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(128) na_backward_q(AttnParams p) {
    __shared__ float sq[4][kD], sg[4][kD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row_id = (int64_t)blockIdx.x * 4 + warp;
    if (row_id >= (int64_t)p.B * p.Hq * p.Sq) return;
    int row, h, b;
    split_row(row_id, p.Sq, p.Hq, row, h, b);
    const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)h * p.qs[1] + (int64_t)row * p.qs[2];
    const T* grow = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1] + (int64_t)row * p.gs[2];
    const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)h * p.ks[1];
    const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)h * p.vs[1];
    for (int d = lane; d < kD; d += 32) {
        sq[warp][d] = to_float<T>(qrow[(int64_t)d * p.qs[3]]);
        sg[warp][d] = to_float<T>(grow[(int64_t)d * p.gs[3]]);
    }
    __syncwarp();
    const Coord qc = unflatten(p, row);
    const int z0 = na_start(qc.z, p.ext[0], p.win[0]), y0 = na_start(qc.y, p.ext[1], p.win[1]),
              x0 = na_start(qc.x, p.ext[2], p.win[2]);
    const int W = p.win[0] * p.win[1] * p.win[2], wyx = p.win[1] * p.win[2];
    const float sign = p.scale >= 0.f ? 1.f : -1.f;
    const float c2 = fabsf(p.scale) * kLog2e;
    const float mx = p.maximum[row_id], ls = p.logsum[row_id], dl = p.delta[row_id];
    float sum_ds = 0.f, mass = 0.f, t_num = 0.f, t_den = 0.f;
    float a0 = 0.f, a1 = 0.f, w0 = 0.f, w1 = 0.f;
    for (int t0 = 0; t0 < W; t0 += 32) {
        const int idx = t0 + lane;
        const bool valid = idx < W;
        int key = 0;
        float p32 = 0.f, res = 0.f;
        if (valid) {
            const int dz = idx / wyx, rem = idx % wyx;
            key = ((z0 + dz) * p.ext[1] + (y0 + rem / p.win[2])) * p.ext[2] + x0 + rem % p.win[2];
            const float sp = dot64<T, VEC>(sq[warp], kb + (int64_t)key * p.ks[2], p.ks[3]) * sign;
            const float dp = dot64<T, VEC>(sg[warp], vb + (int64_t)key * p.vs[2], p.vs[3]);
            p32 = fast_ex2((sp - mx) * c2 - ls);
            res = dp - dl;
        }
        const float ds = round_low<T>(p32 * res);
        const float pl = round_low<T>(p32);
        sum_ds += ds;
        mass += pl;
        t_num += p32 * res;
        t_den += p32;
        const int jn = min(32, W - t0);
        for (int j = 0; j < jn; ++j) {
            const float dj = __shfl_sync(0xffffffffu, ds, j), pj = __shfl_sync(0xffffffffu, pl, j);
            const int kj = __shfl_sync(0xffffffffu, key, j);
            const float2 x = load2<T, VEC>(kb + (int64_t)kj * p.ks[2], p.ks[3], 2 * lane, kD);
            a0 += dj * x.x;
            a1 += dj * x.y;
            w0 += pj * x.x;
            w1 += pj * x.y;
        }
    }
    sum_ds = warp_sum(sum_ds);
    mass = warp_sum(mass);
    t_num = warp_sum(t_num);
    t_den = warp_sum(t_den);
    const float ratio = mass != 0.f ? sum_ds / mass : 0.f;
    T* orow = reinterpret_cast<T*>(p.dq) + (int64_t)b * p.dqs[0] + (int64_t)h * p.dqs[1] + (int64_t)row * p.dqs[2];
    store2<T, VEC>(orow, p.dqs[3], 2 * lane, kD, (a0 - ratio * w0) * p.scale, (a1 - ratio * w1) * p.scale);
    if (lane == 0) p.aux[row_id] = t_den != 0.f ? t_num / t_den : 0.f;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(128) na_backward_kv(AttnParams p) {
    __shared__ float sk[4][kD], sv[4][kD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t key_id = (int64_t)blockIdx.x * 4 + warp;
    if (key_id >= (int64_t)p.B * p.Hq * p.Sk) return;
    int key, h, b;
    split_row(key_id, p.Sk, p.Hq, key, h, b);
    const T* krow = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)h * p.ks[1] + (int64_t)key * p.ks[2];
    const T* vrow = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)h * p.vs[1] + (int64_t)key * p.vs[2];
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)h * p.qs[1];
    const T* gb = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1];
    for (int d = lane; d < kD; d += 32) {
        sk[warp][d] = to_float<T>(krow[(int64_t)d * p.ks[3]]);
        sv[warp][d] = to_float<T>(vrow[(int64_t)d * p.vs[3]]);
    }
    __syncwarp();
    const Coord kc = unflatten(p, key);
    int zl, zh, yl, yh, xl, xh;
    na_inverse(kc.z, p.ext[0], p.win[0], zl, zh);
    na_inverse(kc.y, p.ext[1], p.win[1], yl, yh);
    na_inverse(kc.x, p.ext[2], p.win[2], xl, xh);
    const int nx = xh - xl + 1, ny = yh - yl + 1, nz = zh - zl + 1;
    const int W = nx * ny * nz, nyx = ny * nx;
    const float sign = p.scale >= 0.f ? 1.f : -1.f;
    const float c2 = fabsf(p.scale) * kLog2e;
    const int64_t sbase = ((int64_t)b * p.Hq + h) * p.Sq;
    float k0 = 0.f, k1 = 0.f, v0 = 0.f, v1 = 0.f;
    for (int t0 = 0; t0 < W; t0 += 32) {
        const int idx = t0 + lane;
        const bool valid = idx < W;
        int row = 0;
        float pl = 0.f, ds = 0.f;
        if (valid) {
            const int dz = idx / nyx, rem = idx % nyx;
            row = ((zl + dz) * p.ext[1] + (yl + rem / nx)) * p.ext[2] + xl + rem % nx;
            const float sp = dot64<T, VEC>(sk[warp], qb + (int64_t)row * p.qs[2], p.qs[3]) * sign;
            const float dp = dot64<T, VEC>(sv[warp], gb + (int64_t)row * p.gs[2], p.gs[3]);
            const float p32 = fast_ex2((sp - p.maximum[sbase + row]) * c2 - p.logsum[sbase + row]);
            const float res = dp - p.delta[sbase + row];
            pl = round_low<T>(p32);
            ds = round_low<T>(p32 * (res - p.aux[sbase + row]));
        }
        const int jn = min(32, W - t0);
        for (int j = 0; j < jn; ++j) {
            const float dj = __shfl_sync(0xffffffffu, ds, j), pj = __shfl_sync(0xffffffffu, pl, j);
            const int rj = __shfl_sync(0xffffffffu, row, j);
            const float2 qx = load2<T, VEC>(qb + (int64_t)rj * p.qs[2], p.qs[3], 2 * lane, kD);
            const float2 gx = load2<T, VEC>(gb + (int64_t)rj * p.gs[2], p.gs[3], 2 * lane, kD);
            k0 += dj * qx.x;
            k1 += dj * qx.y;
            v0 += pj * gx.x;
            v1 += pj * gx.y;
        }
    }
    T* dkrow = reinterpret_cast<T*>(p.dk) + (int64_t)b * p.dks[0] + (int64_t)h * p.dks[1] + (int64_t)key * p.dks[2];
    T* dvrow = reinterpret_cast<T*>(p.dv) + (int64_t)b * p.dvs[0] + (int64_t)h * p.dvs[1] + (int64_t)key * p.dvs[2];
    store2<T, VEC>(dkrow, p.dks[3], 2 * lane, kD, k0 * p.scale, k1 * p.scale);
    store2<T, VEC>(dvrow, p.dvs[3], 2 * lane, kD, v0, v1);
}

template <typename T>
cudaError_t forward_t(const AttnParams& p, cudaStream_t st) {
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    const unsigned grid = (unsigned)((rows + 3) / 4);
    if (general_vector_path(p, false)) na_forward<T, true><<<grid, 128, 0, st>>>(p);
    else na_forward<T, false><<<grid, 128, 0, st>>>(p);
    return cudaGetLastError();
}
template <typename T>
cudaError_t backward_t(const AttnParams& p, int which, cudaStream_t st) {
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    const unsigned grid = (unsigned)((rows + 3) / 4);
    const bool vec = general_vector_path(p, true);
    if (which == 0) {
        if (vec) na_backward_q<T, true><<<grid, 128, 0, st>>>(p);
        else na_backward_q<T, false><<<grid, 128, 0, st>>>(p);
    } else {
        if (vec) na_backward_kv<T, true><<<grid, 128, 0, st>>>(p);
        else na_backward_kv<T, false><<<grid, 128, 0, st>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_neighborhood_forward(const AttnParams& p, bool bf16, cudaStream_t st) {
    return bf16 ? forward_t<__nv_bfloat16>(p, st) : forward_t<__half>(p, st);
}
cudaError_t launch_neighborhood_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st) {
    return bf16 ? backward_t<__nv_bfloat16>(p, which, st) : backward_t<__half>(p, which, st);
}

}  // namespace kfa
