// Consumer warpgroups of the backward pipeline: scores -> P -> dS, and the gradient epilogue.
//
// A consumer thread owns one owner row (tensor-memory lane) and 64 / kGroups of the 64 columns of
// every sub-tile (warpgroup g takes columns [g*kCols, (g+1)*kCols)).  Per element, in FP32:
//   P      = ex2((s' - m) * |scale| * log2e - logsum)      s' arrives already sign-adjusted
//   P_low  = round(P)                                       one rounding to the input type
//   dS_low = round(P_low * (dP - delta))
// m, logsum and delta belong to the query: the row for query owners (registers), the column for
// key owners (staged in shared memory).  Hidden entries get P = 0.
#pragma once
#include "pipeline_backward_roles.cuh"

namespace kfa {
namespace bwd {

template <int D, bool BF16, bool KV>
__device__ __forceinline__ void consumer_role(const AttnParams& p, const Work<KV>& w, Shared& sh, uint32_t tmem,
                                              const float* s_stats, int wg, int warp, int lane) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    volatile int* abort_word = &sh.abort_word;
    const int r = (warp & 3) * 32 + lane;  // owner row inside the tile == tensor-memory lane
    const int owner_row = w.owner0 + r;
    const int owner_len = KV ? p.Sk : p.Sq;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float c2 = fabsf(p.scale) * kLog2e;
    const uint64_t c2_pair = f2_pack(c2, c2);

    // per-row quantities
    float row_m = INFINITY, row_ls = 0.f, row_dl = 0.f;
    bool row_ok = owner_row < owner_len;
    // The mask element of (query head hq, query r, key c) is mask_b[hq*ms[1] + r*ms[2] + c*ms[3]].
    const uint8_t* mask_b = p.has_mask ? p.mask + (int64_t)w.b * p.ms[0] : nullptr;
    const bool key_padding = p.has_mask && p.ms[1] == 0 && p.ms[2] == 0;  // one line for all heads and queries
    if (KV) {
        if (row_ok && key_padding) row_ok = mask_b[(int64_t)owner_row * p.ms[3]] != 0;
    } else if (row_ok) {
        const int64_t si = ((int64_t)w.b * p.Hq + w.head) * p.Sq + owner_row;
        row_m = p.maximum[si];
        row_ls = p.logsum[si];
        row_dl = p.delta[si];
        if (row_m == -INFINITY) row_m = INFINITY;  // nothing visible: every P is zero
    }

    // Every consumer warpgroup works on every sub-tile: this one takes columns [wg*kCols, (wg+1)*kCols).
    int g, i;
    w.begin(p, g, i);
    int unit = 0;
    bool ok = true;
    while (w.valid(g) && ok) {
        if (KV) ok = mbar_wait(&sh.stats_full[unit & 1], (unit >> 1) & 1, abort_word, 140);
        // key owners under key padding need no per-element test: a hidden key is a hidden owner row
        const int state = (KV && (key_padding || !p.has_mask)) ? 2 : w.state(p, g, i);
        // this thread's line of mask elements and the step between its columns
        const uint8_t* mline = nullptr;
        int64_t mstep = 0;
        if (state == 1) {
            const int64_t hq = w.query_head(g);
            if (KV) {
                mline = mask_b + hq * p.ms[1] + (int64_t)min(owner_row, p.Sk - 1) * p.ms[3];
                mstep = p.ms[2];  // columns are queries
            } else {
                mline = mask_b + hq * p.ms[1] + (int64_t)min(owner_row, p.Sq - 1) * p.ms[2];
                mstep = p.ms[3];  // columns are keys
            }
        }
        const int col_last = (KV ? p.Sq : p.Sk) - 1;
        for (int sub = 0; sub < 2 && ok; ++sub) {
            KFA_TRACE_POINT(1, 1);
            ok = mbar_wait(&sh.sdp_ready[sub], unit & 1, abort_word, 141 + sub);
            if (!ok) break;
            KFA_TRACE_POINT(1, 2);
            tc_fence_after();
            const uint32_t s_addr = lane_base + sub * 128 + wg * kCols, dp_addr = s_addr + 64;
            uint32_t s[kCols], dp[kCols];
            tmem_ld(s_addr, s);
            tmem_ld(dp_addr, dp);
            tmem_wait_ld();
            KFA_TRACE_POINT(1, 3);

            // columns [lo, hi) of this thread's 32 are visible
            const int col0 = i * kTile + sub * kSub + wg * kCols;  // first streamed row (key or query)
            int lo = 0, hi = kCols;
            if (KV) {
                if (p.causal) lo = owner_row - col0;  // query index must be >= key index
                if (!row_ok) lo = kCols;
            } else {
                hi = p.Sk - col0;
                if (p.causal) hi = min(hi, owner_row - col0 + 1);
            }
            const bool clip = __any_sync(0xffffffffu, lo > 0 || hi < kCols);
            const float* st = s_stats + (unit & 1) * 3 * kTile + sub * kSub + wg * kCols;

            uint32_t pw[kCols / 2], dw[kCols / 2];
            const bool masked = clip || state == 1;
            // One pair of columns: probabilities, their rounding, and the rounded score gradient.
            auto pair = [&](int c, bool apply_mask) {
                float m0, m1, l0, l1, d0, d1;
                if (KV) {
                    const float2 mm = *reinterpret_cast<const float2*>(st + c);
                    const float2 ll = *reinterpret_cast<const float2*>(st + kTile + c);
                    const float2 dd = *reinterpret_cast<const float2*>(st + 2 * kTile + c);
                    m0 = mm.x, m1 = mm.y, l0 = ll.x, l1 = ll.y, d0 = dd.x, d1 = dd.y;
                } else {
                    m0 = m1 = row_m, l0 = l1 = row_ls, d0 = d1 = row_dl;
                }
#ifdef KFA_SCALAR_MATH
                float pa = ex2((__uint_as_float(s[c]) - m0) * c2 - l0);
                float pb = ex2((__uint_as_float(s[c + 1]) - m1) * c2 - l1);
#else
                float ea, eb;
                f2_unpack(f2_sub(f2_mul(f2_sub(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])),
                                               f2_pack(m0, m1)), c2_pair), f2_pack(l0, l1)), ea, eb);
                float pa = ex2(ea), pb = ex2(eb);
#endif
                if (apply_mask) {
                    pa = (c >= lo && c < hi) ? pa : 0.f;
                    pb = (c + 1 >= lo && c + 1 < hi) ? pb : 0.f;
                    if (state == 1) {
                        pa = mline[(int64_t)min(col0 + c, col_last) * mstep] != 0 ? pa : 0.f;
                        pb = mline[(int64_t)min(col0 + c + 1, col_last) * mstep] != 0 ? pb : 0.f;
                    }
                }
                const uint32_t packed = pack2<BF16>(pa, pb);
                pw[c / 2] = packed;
                const float2 pl = unpack2<BF16>(packed);
#ifdef KFA_SCALAR_MATH
                const float da = pl.x * (__uint_as_float(dp[c]) - d0), db = pl.y * (__uint_as_float(dp[c + 1]) - d1);
#else
                float da, db;
                f2_unpack(f2_mul(f2_pack(pl.x, pl.y),
                                 f2_sub(f2_pack(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), f2_pack(d0, d1))),
                          da, db);
#endif
                dw[c / 2] = pack2<BF16>(da, db);
            };
            if (masked) {
#pragma unroll
                for (int c = 0; c < kCols; c += 2) pair(c, true);
            } else {
#pragma unroll
                for (int c = 0; c < kCols; c += 2) pair(c, false);
            }
            // P_low over the head of this thread's S columns (key owners only), dS_low over its dP columns
            KFA_TRACE_POINT(1, 4);
            if (KV) tmem_st(s_addr, pw);
            tmem_st(dp_addr, dw);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sh.done[sub]);
            KFA_TRACE_POINT(1, 5);
        }
        if (KV && ok) mbar_arrive(&sh.stats_empty[unit & 1]);
        w.next(p, g, i);
        ++unit;
    }

    // ---------------------------------------------------------------- epilogue
    // Each warpgroup stores D / kGroups channels of every gradient row.
    constexpr int kHalf = D / kGroups;
    const int ch0 = wg * kHalf;
    T* out1 = nullptr;  // dQ or dK (scaled)
    T* out2 = nullptr;  // dV
    if (owner_row < owner_len) {
        if (KV) {
            out1 = reinterpret_cast<T*>(p.dk) + (int64_t)w.b * p.dks[0] + (int64_t)w.head * p.dks[1] +
                   (int64_t)owner_row * p.dks[2] + ch0;
            out2 = reinterpret_cast<T*>(p.dv) + (int64_t)w.b * p.dvs[0] + (int64_t)w.head * p.dvs[1] +
                   (int64_t)owner_row * p.dvs[2] + ch0;
        } else {
            out1 = reinterpret_cast<T*>(p.dq) + (int64_t)w.b * p.dqs[0] + (int64_t)w.head * p.dqs[1] +
                   (int64_t)owner_row * p.dqs[2] + ch0;
        }
    }
    if (unit == 0) {
        // no visible work for this owner tile: the gradients are exactly zero
        if (ok && out1)
            for (int d = 0; d < kHalf; d += 8) *reinterpret_cast<uint4*>(out1 + d) = make_uint4(0, 0, 0, 0);
        if (ok && out2)
            for (int d = 0; d < kHalf; d += 8) *reinterpret_cast<uint4*>(out2 + d) = make_uint4(0, 0, 0, 0);
        return;
    }
    if (ok) ok = mbar_wait(&sh.final_done, 0, abort_word, 150);
    if (!ok) return;
    tc_fence_after();
#pragma unroll
    for (int which = 0; which < (KV ? 2 : 1); ++which) {
        const uint32_t acc = lane_base + (which == 0 ? 384 : 256) + ch0;
        T* out = which == 0 ? out1 : out2;
        const float mul = which == 0 ? p.scale : 1.f;
        constexpr int kStep = kHalf < 32 ? 16 : 32;
#pragma unroll
        for (int c = 0; c < kHalf; c += kStep) {
            uint32_t v[kStep];
            tmem_ld(acc + c, v);
            tmem_wait_ld();
            if (out) {
#pragma unroll
                for (int e = 0; e < kStep; e += 8) {
                    uint4 o;
                    o.x = pack2<BF16>(__uint_as_float(v[e]) * mul, __uint_as_float(v[e + 1]) * mul);
                    o.y = pack2<BF16>(__uint_as_float(v[e + 2]) * mul, __uint_as_float(v[e + 3]) * mul);
                    o.z = pack2<BF16>(__uint_as_float(v[e + 4]) * mul, __uint_as_float(v[e + 5]) * mul);
                    o.w = pack2<BF16>(__uint_as_float(v[e + 6]) * mul, __uint_as_float(v[e + 7]) * mul);
                    *reinterpret_cast<uint4*>(out + c + e) = o;
                }
            }
        }
    }
}

}  // namespace bwd
}  // namespace kfa
