// General attention kernels: any head dim 1..512, any strides, full boolean
// masks, causal, grouped-query heads.  They are the catch-all family behind
// the tensor-memory pipeline kernels and follow the same arithmetic contract:
//
//   forward   s' = (q.k) * sign(scale); running maximum on s' (unscaled);
//             p = ex2((s' - m) * |scale| * log2e); l sums unrounded p;
//             acc += round(p) * v;  out = round(acc / l); saves m and log2(l).
//   backward  P = ex2((s' - m) * |scale| * log2e - logsum), P_low = round(P),
//             dS_low = round(P_low * (dP - delta)), FP32 accumulation, the
//             signed scale multiplies dQ/dK after accumulation.
//
// (Reference behaviour: src/kohakufa_cute/kernels.py:1286-1333, 1960-2056,
// 866-906 of the reference project.)
//
// Work layout: one warp owns R rows of its output; the 32 lanes each take one
// row of the opposite operand per step (a 32-wide column block), so score
// products are lane-private dot products and the P.V style products broadcast
// one lane's weight while the lanes sweep the channel axis in pairs.
#include "kfa_common.cuh"
#include "row_access.cuh"
#include "launchers.h"

namespace kfa {

namespace {

constexpr int kWarps = 4;

__device__ __forceinline__ bool mask_bit(const AttnParams& p, int b, int h, int r, int c) {
    return p.mask[(int64_t)b * p.ms[0] + (int64_t)h * p.ms[1] + (int64_t)r * p.ms[2] + (int64_t)c * p.ms[3]] != 0;
}

// 64x64 tile state from the table: 0 hidden, 1 mixed, 2 fully visible.
__device__ __forceinline__ int tile_state(const AttnParams& p, int b, int h, int tq, int tk) {
    return p.blocks[(int64_t)b * p.bs[0] + (int64_t)h * p.bs[1] + (int64_t)tq * p.bs[2] + (int64_t)tk * p.bs[3]];
}

// ------------------------------------------------------------------ forward
template <typename T, int R, int DI2, bool VEC>
__global__ void __launch_bounds__(kWarps * 32) general_forward(AttnParams p) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D, Dp = (D + 7) & ~7;
    const int64_t tiles = (p.Sq + kWarps * R - 1) / (kWarps * R);
    const int tile = (int)(blockIdx.x % tiles);
    const int64_t bh = blockIdx.x / tiles;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int row0 = tile * kWarps * R + warp * R;
    if (row0 >= p.Sq) return;
    const int kvh = h / p.group;
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)h * p.qs[1];
    const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)kvh * p.ks[1];
    const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)kvh * p.vs[1];
    float* myq = smem + warp * R * Dp;
    stage_rows<T, R>(myq, Dp, qb, p.qs[2], p.qs[3], row0, p.Sq, D, lane);
    __syncwarp();

    const float sign = p.scale >= 0.f ? 1.f : -1.f;
    const float c2 = fabsf(p.scale) * kLog2e;
    float m[R], l[R], acc[R][DI2][2];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < DI2; ++i) acc[r][i][0] = acc[r][i][1] = 0.f;
    }
    const int last_row = min(row0 + R, p.Sq) - 1;
    const int kend = p.causal ? min(p.Sk, last_row + 1) : p.Sk;
    for (int k0 = 0; k0 < kend; k0 += 32) {
        if (p.has_mask && (k0 & 63) == 0) {
            // skip a 64-key block that the tile table marks hidden for every row of this warp
            int tq0 = row0 >> 6, tq1 = last_row >> 6;
            bool any = tile_state(p, b, h, tq0, k0 >> 6) != 0 || tile_state(p, b, h, tq1, k0 >> 6) != 0;
            if (!any) { k0 += 32; continue; }
        }
        const int c = k0 + lane;
        const bool in_range = c < kend;
        float s[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] = 0.f;
        if (in_range) {
            const T* krow = kb + (int64_t)c * p.ks[2];
            for (int d = 0; d < Dp; d += 8) {
                float kx[8];
                load8<T, VEC>(krow, p.ks[3], d, D, kx);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float4 a = *reinterpret_cast<const float4*>(myq + r * Dp + d);
                    const float4 e = *reinterpret_cast<const float4*>(myq + r * Dp + d + 4);
                    s[r] += a.x * kx[0] + a.y * kx[1] + a.z * kx[2] + a.w * kx[3] + e.x * kx[4] + e.y * kx[5] +
                            e.z * kx[6] + e.w * kx[7];
                }
            }
        }
        float plow[R];
        bool any_weight = false;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = row0 + r;
            bool vis = in_range && row < p.Sq && (!p.causal || c <= row);
            if (vis && p.has_mask) vis = mask_bit(p, b, h, row, c);
            const float sp = vis ? s[r] * sign : -INFINITY;
            const float m_new = fmaxf(m[r], warp_max(sp));
            float alpha = 1.f, pr = 0.f;
            if (m_new != -INFINITY) {
                alpha = (m[r] == -INFINITY) ? 0.f : fast_ex2((m[r] - m_new) * c2);
                pr = vis ? fast_ex2((sp - m_new) * c2) : 0.f;
            }
            l[r] = l[r] * alpha + warp_sum(pr);
#pragma unroll
            for (int i = 0; i < DI2; ++i) {
                acc[r][i][0] *= alpha;
                acc[r][i][1] *= alpha;
            }
            plow[r] = round_low<T>(pr);
            m[r] = m_new;
            any_weight |= __any_sync(0xffffffffu, plow[r] != 0.f);
        }
        if (!any_weight) continue;
        const int jn = min(32, kend - k0);
        for (int j = 0; j < jn; ++j) {
            float pj[R];
            bool live = false;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                pj[r] = __shfl_sync(0xffffffffu, plow[r], j);
                live |= pj[r] != 0.f;
            }
            if (!live) continue;
            const T* vrow = vb + (int64_t)(k0 + j) * p.vs[2];
#pragma unroll
            for (int i = 0; i < DI2; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < D) {
                    const float2 x = load2<T, VEC>(vrow, p.vs[3], d, D);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        acc[r][i][0] += pj[r] * x.x;
                        acc[r][i][1] += pj[r] * x.y;
                    }
                }
            }
        }
    }
    T* ob = reinterpret_cast<T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = row0 + r;
        if (row >= p.Sq) break;
        const float den = l[r] > 0.f ? l[r] : 1.f;
        T* orow = ob + (int64_t)row * p.os[2];
#pragma unroll
        for (int i = 0; i < DI2; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < D) store2<T, VEC>(orow, p.os[3], d, D, acc[r][i][0] / den, acc[r][i][1] / den);
        }
        if (lane == 0 && p.maximum) {
            const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + row;
            p.maximum[si] = m[r];
            p.logsum[si] = log2f(den);
        }
    }
}

// -------------------------------------------------------------------- delta
// delta[b,h,r] = sum_d f32(O) * f32(dO); one thread per row, channels in ascending order with
// fused multiply-adds.  The backward kernels below form dP = dO . V with the same chain, so for
// a row whose output equals a value row (a single visible key) dP - delta is exactly zero.
template <typename T>
__global__ void __launch_bounds__(128) output_delta(AttnParams p) {
    const int64_t row_id = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    if (row_id >= rows) return;
    int r, h, b;
    split_row(row_id, p.Sq, p.Hq, r, h, b);
    const T* o = reinterpret_cast<const T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] + (int64_t)r * p.os[2];
    const T* g = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1] + (int64_t)r * p.gs[2];
    float sum = 0.f;
    for (int d = 0; d < p.D; ++d)
        sum = fmaf(to_float<T>(g[(int64_t)d * p.gs[3]]), to_float<T>(o[(int64_t)d * p.os[3]]), sum);
    p.delta[row_id] = sum;
}

// ------------------------------------------------------------ backward: dQ
template <typename T, int R, int DI2, bool VEC>
__global__ void __launch_bounds__(kWarps * 32) general_backward_q(AttnParams p) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D, Dp = (D + 7) & ~7;
    const int64_t tiles = (p.Sq + kWarps * R - 1) / (kWarps * R);
    const int tile = (int)(blockIdx.x % tiles);
    const int64_t bh = blockIdx.x / tiles;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int row0 = tile * kWarps * R + warp * R;
    if (row0 >= p.Sq) return;
    const int kvh = h / p.group;
    const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)h * p.qs[1];
    const T* gb = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1];
    const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)kvh * p.ks[1];
    const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)kvh * p.vs[1];
    float* myq = smem + warp * 2 * R * Dp;
    float* myg = myq + R * Dp;
    stage_rows<T, R>(myq, Dp, qb, p.qs[2], p.qs[3], row0, p.Sq, D, lane);
    stage_rows<T, R>(myg, Dp, gb, p.gs[2], p.gs[3], row0, p.Sq, D, lane);
    __syncwarp();
    const float sign = p.scale >= 0.f ? 1.f : -1.f;
    const float c2 = fabsf(p.scale) * kLog2e;
    float mx[R], ls[R], dl[R], acc[R][DI2][2];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = min(row0 + r, p.Sq - 1);
        const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + row;
        mx[r] = p.maximum[si];
        ls[r] = p.logsum[si];
        dl[r] = p.delta[si];
#pragma unroll
        for (int i = 0; i < DI2; ++i) acc[r][i][0] = acc[r][i][1] = 0.f;
    }
    const int last_row = min(row0 + R, p.Sq) - 1;
    const int kend = p.causal ? min(p.Sk, last_row + 1) : p.Sk;
    for (int k0 = 0; k0 < kend; k0 += 32) {
        if (p.has_mask && (k0 & 63) == 0) {
            int tq0 = row0 >> 6, tq1 = last_row >> 6;
            bool any = tile_state(p, b, h, tq0, k0 >> 6) != 0 || tile_state(p, b, h, tq1, k0 >> 6) != 0;
            if (!any) { k0 += 32; continue; }
        }
        const int c = k0 + lane;
        const bool in_range = c < kend;
        float s[R], dp[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] = dp[r] = 0.f;
        if (in_range) {
            const T* krow = kb + (int64_t)c * p.ks[2];
            const T* vrow = vb + (int64_t)c * p.vs[2];
            for (int d = 0; d < Dp; d += 8) {
                float kx[8], vx[8];
                load8<T, VEC>(krow, p.ks[3], d, D, kx);
                load8<T, VEC>(vrow, p.vs[3], d, D, vx);
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        s[r] += myq[r * Dp + d + i] * kx[i];
                        dp[r] = fmaf(myg[r * Dp + d + i], vx[i], dp[r]);
                    }
                }
            }
        }
        float ds[R];
        bool any_weight = false;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = row0 + r;
            bool vis = in_range && row < p.Sq && (!p.causal || c <= row);
            if (vis && p.has_mask) vis = mask_bit(p, b, h, row, c);
            const float pr = vis ? fast_ex2((s[r] * sign - mx[r]) * c2 - ls[r]) : 0.f;
            ds[r] = round_low<T>(round_low<T>(pr) * (dp[r] - dl[r]));
            any_weight |= __any_sync(0xffffffffu, ds[r] != 0.f);
        }
        if (!any_weight) continue;
        const int jn = min(32, kend - k0);
        for (int j = 0; j < jn; ++j) {
            float dj[R];
            bool live = false;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                dj[r] = __shfl_sync(0xffffffffu, ds[r], j);
                live |= dj[r] != 0.f;
            }
            if (!live) continue;
            const T* krow = kb + (int64_t)(k0 + j) * p.ks[2];
#pragma unroll
            for (int i = 0; i < DI2; ++i) {
                const int d = 2 * (lane + 32 * i);
                if (d < D) {
                    const float2 x = load2<T, VEC>(krow, p.ks[3], d, D);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        acc[r][i][0] += dj[r] * x.x;
                        acc[r][i][1] += dj[r] * x.y;
                    }
                }
            }
        }
    }
    T* ob = reinterpret_cast<T*>(p.dq) + (int64_t)b * p.dqs[0] + (int64_t)h * p.dqs[1];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = row0 + r;
        if (row >= p.Sq) break;
        T* orow = ob + (int64_t)row * p.dqs[2];
#pragma unroll
        for (int i = 0; i < DI2; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < D) store2<T, VEC>(orow, p.dqs[3], d, D, acc[r][i][0] * p.scale, acc[r][i][1] * p.scale);
        }
    }
}

// -------------------------------------------------------- backward: dK, dV
template <typename T, int R, int DI2, bool VEC>
__global__ void __launch_bounds__(kWarps * 32) general_backward_kv(AttnParams p) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D, Dp = (D + 7) & ~7;
    const int64_t tiles = (p.Sk + kWarps * R - 1) / (kWarps * R);
    const int tile = (int)(blockIdx.x % tiles);
    const int64_t bh = blockIdx.x / tiles;
    const int kvh = (int)(bh % p.Hkv), b = (int)(bh / p.Hkv);
    const int key0 = tile * kWarps * R + warp * R;
    if (key0 >= p.Sk) return;
    const T* kb = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)kvh * p.ks[1];
    const T* vb = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)kvh * p.vs[1];
    float* myk = smem + warp * 2 * R * Dp;
    float* myv = myk + R * Dp;
    stage_rows<T, R>(myk, Dp, kb, p.ks[2], p.ks[3], key0, p.Sk, D, lane);
    stage_rows<T, R>(myv, Dp, vb, p.vs[2], p.vs[3], key0, p.Sk, D, lane);
    __syncwarp();
    const float sign = p.scale >= 0.f ? 1.f : -1.f;
    const float c2 = fabsf(p.scale) * kLog2e;
    float ak[R][DI2][2], av[R][DI2][2];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < DI2; ++i) ak[r][i][0] = ak[r][i][1] = av[r][i][0] = av[r][i][1] = 0.f;
    const int q_begin = p.causal ? (key0 & ~31) : 0;  // causal: only queries r >= key see the key
    for (int g = 0; g < p.group; ++g) {
        const int h = kvh * p.group + g;
        const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)h * p.qs[1];
        const T* gb = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1];
        const int64_t sbase = ((int64_t)b * p.Hq + h) * p.Sq;
        for (int q0 = q_begin; q0 < p.Sq; q0 += 32) {
            if (p.has_mask && (q0 & 63) == 0) {
                int tk0 = key0 >> 6, tk1 = (min(key0 + R, p.Sk) - 1) >> 6;
                bool any = tile_state(p, b, h, q0 >> 6, tk0) != 0 || tile_state(p, b, h, q0 >> 6, tk1) != 0;
                if (!any) { q0 += 32; continue; }
            }
            const int row = q0 + lane;
            const bool in_range = row < p.Sq;
            float s[R], dp[R];
#pragma unroll
            for (int r = 0; r < R; ++r) s[r] = dp[r] = 0.f;
            float mx = 0.f, ls = 0.f, dl = 0.f;
            if (in_range) {
                mx = p.maximum[sbase + row];
                ls = p.logsum[sbase + row];
                dl = p.delta[sbase + row];
                const T* qrow = qb + (int64_t)row * p.qs[2];
                const T* grow = gb + (int64_t)row * p.gs[2];
                for (int d = 0; d < Dp; d += 8) {
                    float qx[8], gx[8];
                    load8<T, VEC>(qrow, p.qs[3], d, D, qx);
                    load8<T, VEC>(grow, p.gs[3], d, D, gx);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            s[r] += myk[r * Dp + d + i] * qx[i];
                            dp[r] = fmaf(gx[i], myv[r * Dp + d + i], dp[r]);
                        }
                    }
                }
            }
            float pl[R], ds[R];
            bool any_weight = false;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int c = key0 + r;
                bool vis = in_range && c < p.Sk && (!p.causal || c <= row);
                if (vis && p.has_mask) vis = mask_bit(p, b, h, row, c);
                const float pr = vis ? fast_ex2((s[r] * sign - mx) * c2 - ls) : 0.f;
                pl[r] = round_low<T>(pr);
                ds[r] = round_low<T>(pl[r] * (dp[r] - dl));
                any_weight |= __any_sync(0xffffffffu, pl[r] != 0.f || ds[r] != 0.f);
            }
            if (!any_weight) continue;
            const int jn = min(32, p.Sq - q0);
            for (int j = 0; j < jn; ++j) {
                float pj[R], dj[R];
                bool live = false;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    pj[r] = __shfl_sync(0xffffffffu, pl[r], j);
                    dj[r] = __shfl_sync(0xffffffffu, ds[r], j);
                    live |= pj[r] != 0.f || dj[r] != 0.f;
                }
                if (!live) continue;
                const T* qrow = qb + (int64_t)(q0 + j) * p.qs[2];
                const T* grow = gb + (int64_t)(q0 + j) * p.gs[2];
#pragma unroll
                for (int i = 0; i < DI2; ++i) {
                    const int d = 2 * (lane + 32 * i);
                    if (d < D) {
                        const float2 qx = load2<T, VEC>(qrow, p.qs[3], d, D);
                        const float2 gx = load2<T, VEC>(grow, p.gs[3], d, D);
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            ak[r][i][0] += dj[r] * qx.x;
                            ak[r][i][1] += dj[r] * qx.y;
                            av[r][i][0] += pj[r] * gx.x;
                            av[r][i][1] += pj[r] * gx.y;
                        }
                    }
                }
            }
        }
    }
    T* dkb = reinterpret_cast<T*>(p.dk) + (int64_t)b * p.dks[0] + (int64_t)kvh * p.dks[1];
    T* dvb = reinterpret_cast<T*>(p.dv) + (int64_t)b * p.dvs[0] + (int64_t)kvh * p.dvs[1];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int c = key0 + r;
        if (c >= p.Sk) break;
#pragma unroll
        for (int i = 0; i < DI2; ++i) {
            const int d = 2 * (lane + 32 * i);
            if (d < D) {
                store2<T, VEC>(dkb + (int64_t)c * p.dks[2], p.dks[3], d, D, ak[r][i][0] * p.scale, ak[r][i][1] * p.scale);
                store2<T, VEC>(dvb + (int64_t)c * p.dvs[2], p.dvs[3], d, D, av[r][i][0], av[r][i][1]);
            }
        }
    }
}

// ---------------------------------------------------------------- pack mask
// One warp classifies one 64x64 tile of the expanded mask: 0 no visible element,
// 2 every in-bounds element visible, 1 otherwise.  Axes on which the mask has
// stride 0 are collapsed to extent 1 in the table.
__global__ void __launch_bounds__(128) pack_mask(AttnParams p, int nb, int nh, int nq, int nk) {
    const int lane = threadIdx.x & 31;
    const int64_t tile_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t total = (int64_t)nb * nh * nq * nk;
    if (tile_id >= total) return;
    const int tk = (int)(tile_id % nk);
    const int tq = (int)((tile_id / nk) % nq);
    const int h = (int)((tile_id / ((int64_t)nk * nq)) % nh);
    const int b = (int)(tile_id / ((int64_t)nk * nq * nh));
    const int rows = p.ms[2] == 0 ? 1 : min(64, p.Sq - tq * 64);
    const int cols = p.ms[3] == 0 ? 1 : min(64, p.Sk - tk * 64);
    int seen = 0;
    for (int e = lane; e < rows * cols; e += 32) {
        const int r = tq * 64 + e / cols, c = tk * 64 + e % cols;
        seen += mask_bit(p, b, h, r, c) ? 1 : 0;
    }
    seen = __reduce_add_sync(0xffffffffu, seen);
    if (lane == 0) p.blocks[tile_id] = seen == 0 ? 0 : (seen == rows * cols ? 2 : 1);
}

// --------------------------------------------------------------- centre keys
// mean[b,h,d] over the sequence axis in FP32 (fixed summation order: rows strided by 8 inside a
// block, then the sequence splits in ascending order), then out = round(f32(k) - mean).
constexpr int kMeanSplits = 32;
bool vector_ok(const void* ptr, const int64_t* s, int D);

template <typename T>
__global__ void __launch_bounds__(256) column_partial(const T* k, float* partial, int H, int S, int D, int splits,
                                                      int64_t s0, int64_t s1, int64_t s2, int64_t s3) {
    __shared__ float part[8][33];
    // batch*head on grid.x (no 65535 limit there), channel block on grid.y, sequence split on grid.z
    const int bh = blockIdx.x, b = bh / H, h = bh % H, split = blockIdx.z;
    const int d = blockIdx.y * 32 + (threadIdx.x & 31);
    const int lane_s = threadIdx.x >> 5;
    const int rows_per = (S + splits - 1) / splits;
    const int r0 = split * rows_per, r1 = min(S, r0 + rows_per);
    const T* base = k + (int64_t)b * s0 + (int64_t)h * s1;
    float sum = 0.f;
    if (d < D)
        for (int s = r0 + lane_s; s < r1; s += 8) sum += to_float<T>(base[(int64_t)s * s2 + (int64_t)d * s3]);
    part[lane_s][threadIdx.x & 31] = sum;
    __syncthreads();
    if (lane_s == 0 && d < D) {
        float total = 0.f;
        for (int i = 0; i < 8; ++i) total += part[i][threadIdx.x];
        partial[((int64_t)bh * splits + split) * D + d] = total;
    }
}
__global__ void __launch_bounds__(128) finish_mean(const float* partial, float* mean, int S, int D, int splits) {
    const int bh = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += 128) {
        float total = 0.f;
        for (int i = 0; i < splits; ++i) total += partial[((int64_t)bh * splits + i) * D + d];
        mean[(int64_t)bh * D + d] = total / (float)S;
    }
}
// One thread per 8 consecutive channels (VEC) or per element.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) subtract_mean(const T* k, const float* mean, T* out, int H, int S, int D,
                                                     int64_t s0, int64_t s1, int64_t s2, int64_t s3, int64_t o0,
                                                     int64_t o1, int64_t o2, int64_t o3) {
    // one-dimensional grid: `per_head` blocks per (batch, head)
    const int64_t items = VEC ? (int64_t)S * (D / 8) : (int64_t)S * D;
    const int64_t per_head = (items + 255) / 256;
    const int bh = (int)(blockIdx.x / per_head), b = bh / H, h = bh % H;
    const int64_t idx = (int64_t)(blockIdx.x % per_head) * 256 + threadIdx.x;
    if (VEC) {
        const int per_row = D / 8;
        if (idx >= (int64_t)S * per_row) return;
        const int s = (int)(idx / per_row), d = (int)(idx % per_row) * 8;
        const uint4 raw = *reinterpret_cast<const uint4*>(k + (int64_t)b * s0 + (int64_t)h * s1 + (int64_t)s * s2 + d);
        const float4 m0 = *reinterpret_cast<const float4*>(mean + (int64_t)bh * D + d);
        const float4 m1 = *reinterpret_cast<const float4*>(mean + (int64_t)bh * D + d + 4);
        const float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        const T* e = reinterpret_cast<const T*>(&raw);
        uint4 res;
        T* r = reinterpret_cast<T*>(&res);
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = from_float<T>(to_float<T>(e[i]) - mv[i]);
        *reinterpret_cast<uint4*>(out + (int64_t)b * o0 + (int64_t)h * o1 + (int64_t)s * o2 + d) = res;
    } else {
        if (idx >= (int64_t)S * D) return;
        const int s = (int)(idx / D), d = (int)(idx % D);
        const float x = to_float<T>(k[(int64_t)b * s0 + (int64_t)h * s1 + (int64_t)s * s2 + (int64_t)d * s3]);
        out[(int64_t)b * o0 + (int64_t)h * o1 + (int64_t)s * o2 + (int64_t)d * o3] =
            from_float<T>(x - mean[(int64_t)bh * D + d]);
    }
}

// -------------------------------------------------------------- ring merge
// Folds one partial attention result into the running FP32 result.  Each side is
// a normalised output with its (maximum, logsum) pair; the merged weight of a side
// is ex2((m_side - m) * |scale| * log2e + logsum_side).
template <typename T>
__global__ void __launch_bounds__(128) merge_partial(float* acc, float* am, float* al, const T* part, const float* pm,
                                                     const float* pl, int64_t rows, int D, float c2, int64_t a_row,
                                                     int64_t p_b, int64_t p_h, int64_t p_s, int64_t p_d, int H, int S) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int s, h, b;
    split_row(row, S, H, s, h, b);
    const float m0 = am[row], l0 = al[row], m1 = pm[row], l1 = pl[row];
    const float m = fmaxf(m0, m1);
    float w0 = 0.f, w1 = 0.f;
    if (m != -INFINITY) {
        w0 = (m0 == -INFINITY) ? 0.f : fast_ex2((m0 - m) * c2 + l0);
        w1 = (m1 == -INFINITY) ? 0.f : fast_ex2((m1 - m) * c2 + l1);
    }
    const float total = w0 + w1;
    const float inv = total > 0.f ? 1.f / total : 0.f;
    const T* prow = part + (int64_t)b * p_b + (int64_t)h * p_h + (int64_t)s * p_s;
    float* arow = acc + row * a_row;
    for (int d = lane; d < D; d += 32)
        arow[d] = (arow[d] * w0 + to_float<T>(prow[(int64_t)d * p_d]) * w1) * inv;
    if (lane == 0) {
        am[row] = m;
        al[row] = total > 0.f ? log2f(total) : 0.f;
    }
}

// Closes a running forward state (block-wise calls over a longer key sequence): one division per row, the output
// rounded once to the 16-bit type, and the statistics of the operator's contract (unscaled maximum, log2 of the sum).
template <typename T>
__global__ void __launch_bounds__(128) finish_running(T* out, float* maximum, float* logsum, const float* acc,
                                                      const float* run_max, const float* run_sum, int64_t rows, int D,
                                                      int64_t a_b, int64_t a_h, int64_t a_s, int64_t o_b, int64_t o_h,
                                                      int64_t o_s, int64_t o_d, int H, int S) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int s, h, b;
    split_row(row, S, H, s, h, b);
    const float l = run_sum[row];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float* arow = acc + (int64_t)b * a_b + (int64_t)h * a_h + (int64_t)s * a_s;
    T* orow = out + (int64_t)b * o_b + (int64_t)h * o_h + (int64_t)s * o_s;
    for (int d = lane; d < D; d += 32) orow[(int64_t)d * o_d] = from_float<T>(arow[d] * inv);
    if (lane == 0) {
        maximum[row] = l > 0.f ? run_max[row] : -INFINITY;
        logsum[row] = l > 0.f ? log2f(l) : 0.f;
    }
}

// Merges the partial results of a forward pass split over the key axis: `splits` normalised outputs with their
// (maximum, logsum) pairs -> one output row, rounded once, and the statistics of the whole key range.
// part is [splits, rows, D] (16-bit, contiguous), pm / pl are [splits, rows].
template <typename T>
__global__ void __launch_bounds__(128) merge_splits(T* out, float* maximum, float* logsum, const T* part, const float* pm,
                                                    const float* pl, int splits, int64_t rows, int D, float c2,
                                                    int64_t o_b, int64_t o_h, int64_t o_s, int64_t o_d, int H, int S) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int s, h, b;
    split_row(row, S, H, s, h, b);
    float m = -INFINITY;
    for (int i = 0; i < splits; ++i) m = fmaxf(m, pm[(int64_t)i * rows + row]);
    float total = 0.f;
    for (int i = 0; i < splits; ++i) {
        const float mi = pm[(int64_t)i * rows + row];
        if (mi != -INFINITY) total += fast_ex2((mi - m) * c2 + pl[(int64_t)i * rows + row]);
    }
    const float inv = total > 0.f ? 1.f / total : 0.f;
    T* orow = out + (int64_t)b * o_b + (int64_t)h * o_h + (int64_t)s * o_s;
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int i = 0; i < splits; ++i) {
            const float mi = pm[(int64_t)i * rows + row];
            if (mi == -INFINITY) continue;
            const float w = fast_ex2((mi - m) * c2 + pl[(int64_t)i * rows + row]);
            acc += w * to_float<T>(part[((int64_t)i * rows + row) * D + d]);
        }
        orow[(int64_t)d * o_d] = from_float<T>(acc * inv);
    }
    if (lane == 0 && maximum) {
        maximum[row] = m;
        logsum[row] = total > 0.f ? log2f(total) : 0.f;
    }
}

inline int64_t blocks_for(int64_t items, int per_block) { return (items + per_block - 1) / per_block; }

template <typename T, bool VEC>
cudaError_t launch_forward_t(const AttnParams& p, cudaStream_t st) {
    constexpr int R = 4;
    const int Dp = (p.D + 7) & ~7;
    const size_t smem = (size_t)kWarps * R * Dp * sizeof(float);
    const int64_t grid = blocks_for(p.Sq, kWarps * R) * p.B * p.Hq;
    if (p.D <= 64) general_forward<T, R, 1, VEC><<<(unsigned)grid, kWarps * 32, smem, st>>>(p);
    else if (p.D <= 128) general_forward<T, R, 2, VEC><<<(unsigned)grid, kWarps * 32, smem, st>>>(p);
    else if (p.D <= 256) general_forward<T, R, 4, VEC><<<(unsigned)grid, kWarps * 32, smem, st>>>(p);
    else general_forward<T, R, 8, VEC><<<(unsigned)grid, kWarps * 32, smem, st>>>(p);
    return cudaGetLastError();
}

template <typename T, bool VEC>
cudaError_t launch_backward_t(const AttnParams& p, int which, cudaStream_t st) {
    constexpr int R = 2;
    const int Dp = (p.D + 7) & ~7;
    const size_t smem = (size_t)kWarps * 2 * R * Dp * sizeof(float);
    const int64_t gq = blocks_for(p.Sq, kWarps * R) * p.B * p.Hq;
    const int64_t gk = blocks_for(p.Sk, kWarps * R) * p.B * p.Hkv;
#define KFA_BWD(DI2)                                                                                     \
    if (which == 0) general_backward_q<T, R, DI2, VEC><<<(unsigned)gq, kWarps * 32, smem, st>>>(p);      \
    else general_backward_kv<T, R, DI2, VEC><<<(unsigned)gk, kWarps * 32, smem, st>>>(p);
    if (p.D <= 64) { KFA_BWD(1) }
    else if (p.D <= 128) { KFA_BWD(2) }
    else if (p.D <= 256) { KFA_BWD(4) }
    else { KFA_BWD(8) }
#undef KFA_BWD
    return cudaGetLastError();
}

bool vector_ok(const void* ptr, const int64_t* s, int D) {
    if (s[3] != 1 || D % 8 != 0) return false;
    if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return false;
    return s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0;
}

}  // namespace

bool general_vector_path(const AttnParams& p, bool backward) {
    bool ok = vector_ok(p.q, p.qs, p.D) && vector_ok(p.k, p.ks, p.D) && vector_ok(p.v, p.vs, p.D);
    if (!backward) return ok && vector_ok(p.out, p.os, p.D);
    return ok && vector_ok(p.dout, p.gs, p.D) && vector_ok(p.dq, p.dqs, p.D) && vector_ok(p.dk, p.dks, p.D) &&
           vector_ok(p.dv, p.dvs, p.D);
}

cudaError_t launch_pack_mask(const AttnParams& p, int nb, int nh, int nq, int nk, cudaStream_t st) {
    const int64_t total = (int64_t)nb * nh * nq * nk;
    pack_mask<<<(unsigned)blocks_for(total, 4), 128, 0, st>>>(p, nb, nh, nq, nk);
    return cudaGetLastError();
}

cudaError_t launch_general_forward(const AttnParams& p, bool bf16, cudaStream_t st) {
    const bool vec = general_vector_path(p, false);
    if (bf16) return vec ? launch_forward_t<__nv_bfloat16, true>(p, st) : launch_forward_t<__nv_bfloat16, false>(p, st);
    return vec ? launch_forward_t<__half, true>(p, st) : launch_forward_t<__half, false>(p, st);
}

cudaError_t launch_output_delta(const AttnParams& p, bool bf16, cudaStream_t st) {
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    if (bf16) output_delta<__nv_bfloat16><<<(unsigned)blocks_for(rows, 128), 128, 0, st>>>(p);
    else output_delta<__half><<<(unsigned)blocks_for(rows, 128), 128, 0, st>>>(p);
    return cudaGetLastError();
}

// which: 0 = query-gradient kernel, 1 = key/value-gradient kernel
cudaError_t launch_general_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st) {
    const bool vec = general_vector_path(p, true);
    if (bf16)
        return vec ? launch_backward_t<__nv_bfloat16, true>(p, which, st)
                   : launch_backward_t<__nv_bfloat16, false>(p, which, st);
    return vec ? launch_backward_t<__half, true>(p, which, st) : launch_backward_t<__half, false>(p, which, st);
}

// workspace: kMeanSplits * B*H*D partial sums followed by B*H*D means
cudaError_t launch_center_keys(const void* k, void* out, float* workspace, bool bf16, int B, int H, int S, int D,
                               const int64_t* ks, const int64_t* os, cudaStream_t st, int* launches) {
    // one launch over thread-block clusters when a head's slab fits in shared memory and the device can
    // co-schedule the cluster; a failed cluster launch (a partition that cannot) falls through as well
    if (center_keys_cluster_supported(k, out, B, H, S, D, ks, os) && center_keys_cluster_schedulable(bf16, S, D)) {
        if (launch_center_keys_cluster(k, out, bf16, B, H, S, D, ks, os, st) == cudaSuccess) {
            if (launches) *launches = 1;
            return cudaSuccess;
        }
        cudaGetLastError();
    }
    if (launches) *launches = 3;
    const int splits = max(1, min(kMeanSplits, S / 128));
    float* partial = workspace;
    float* mean = workspace + (int64_t)kMeanSplits * B * H * D;
    const bool vec = vector_ok(k, ks, D) && vector_ok(out, os, D);
    const int64_t items = vec ? (int64_t)S * (D / 8) : (int64_t)S * D;
    const int64_t sub_blocks = blocks_for(items, 256) * B * H;
    if (sub_blocks > INT32_MAX) return cudaErrorInvalidConfiguration;
    dim3 g1(B * H, (D + 31) / 32, splits);
    const unsigned g3 = (unsigned)sub_blocks;
    if (bf16) {
        using T = __nv_bfloat16;
        column_partial<T><<<g1, 256, 0, st>>>((const T*)k, partial, H, S, D, splits, ks[0], ks[1], ks[2], ks[3]);
        finish_mean<<<B * H, 128, 0, st>>>(partial, mean, S, D, splits);
        if (vec) subtract_mean<T, true><<<g3, 256, 0, st>>>((const T*)k, mean, (T*)out, H, S, D, ks[0], ks[1], ks[2], ks[3], os[0], os[1], os[2], os[3]);
        else subtract_mean<T, false><<<g3, 256, 0, st>>>((const T*)k, mean, (T*)out, H, S, D, ks[0], ks[1], ks[2], ks[3], os[0], os[1], os[2], os[3]);
    } else {
        using T = __half;
        column_partial<T><<<g1, 256, 0, st>>>((const T*)k, partial, H, S, D, splits, ks[0], ks[1], ks[2], ks[3]);
        finish_mean<<<B * H, 128, 0, st>>>(partial, mean, S, D, splits);
        if (vec) subtract_mean<T, true><<<g3, 256, 0, st>>>((const T*)k, mean, (T*)out, H, S, D, ks[0], ks[1], ks[2], ks[3], os[0], os[1], os[2], os[3]);
        else subtract_mean<T, false><<<g3, 256, 0, st>>>((const T*)k, mean, (T*)out, H, S, D, ks[0], ks[1], ks[2], ks[3], os[0], os[1], os[2], os[3]);
    }
    return cudaGetLastError();
}

cudaError_t launch_merge_splits(void* out, float* maximum, float* logsum, const void* part, const float* pm,
                                const float* pl, bool bf16, int splits, int B, int H, int S, int D, const int64_t* os,
                                float scale, cudaStream_t st) {
    const int64_t rows = (int64_t)B * H * S;
    const float c2 = fabsf(scale) * kLog2e;
    const unsigned grid = (unsigned)blocks_for(rows, 4);
    if (bf16)
        merge_splits<__nv_bfloat16><<<grid, 128, 0, st>>>((__nv_bfloat16*)out, maximum, logsum, (const __nv_bfloat16*)part,
                                                          pm, pl, splits, rows, D, c2, os[0], os[1], os[2], os[3], H, S);
    else
        merge_splits<__half><<<grid, 128, 0, st>>>((__half*)out, maximum, logsum, (const __half*)part, pm, pl, splits, rows,
                                                   D, c2, os[0], os[1], os[2], os[3], H, S);
    return cudaGetLastError();
}

cudaError_t launch_merge_partial(float* acc, float* am, float* al, const void* part, const float* pm, const float* pl,
                                 bool bf16, int B, int H, int S, int D, const int64_t* ps, float scale,
                                 cudaStream_t st) {
    const int64_t rows = (int64_t)B * H * S;
    const float c2 = fabsf(scale) * kLog2e;
    if (bf16)
        merge_partial<__nv_bfloat16><<<(unsigned)blocks_for(rows, 4), 128, 0, st>>>(
            acc, am, al, (const __nv_bfloat16*)part, pm, pl, rows, D, c2, D, ps[0], ps[1], ps[2], ps[3], H, S);
    else
        merge_partial<__half><<<(unsigned)blocks_for(rows, 4), 128, 0, st>>>(acc, am, al, (const __half*)part, pm, pl,
                                                                            rows, D, c2, D, ps[0], ps[1], ps[2],
                                                                            ps[3], H, S);
    return cudaGetLastError();
}

cudaError_t launch_finish_running(void* out, float* maximum, float* logsum, const float* acc, const float* run_max,
                                  const float* run_sum, bool bf16, int B, int H, int S, int D, const int64_t* as,
                                  const int64_t* os, cudaStream_t st) {
    const int64_t rows = (int64_t)B * H * S;
    if (bf16)
        finish_running<__nv_bfloat16><<<(unsigned)blocks_for(rows, 4), 128, 0, st>>>(
            (__nv_bfloat16*)out, maximum, logsum, acc, run_max, run_sum, rows, D, as[0], as[1], as[2], os[0], os[1],
            os[2], os[3], H, S);
    else
        finish_running<__half><<<(unsigned)blocks_for(rows, 4), 128, 0, st>>>((__half*)out, maximum, logsum, acc,
                                                                              run_max, run_sum, rows, D, as[0], as[1],
                                                                              as[2], os[0], os[1], os[2], os[3], H, S);
    return cudaGetLastError();
}

}  // namespace kfa
