// Consumer warpgroups of the key/value-gradient kernel: shifted scores -> P -> dS, and the gradient epilogue.
//
// A consumer thread owns one key row (tensor-memory lane) and 64 of the 128 query columns of every
// unit (warpgroup g takes columns [g*64, (g+1)*64)).  The tensor core delivers
//   s~ = s' - m - logsum / c      and      dP~ = dP - delta
// (s' already sign-adjusted; the per-query statistics are subtracted by one more step of the score
// products, see pipeline_backward_kv_roles.cuh), so that per element, in FP32:
//   P      = ex2(s~ * c)          c = |scale| * log2(e)
//   P_low  = round(P)             one rounding to the input type
//   dS_low = round(P_low * dP~)
// Hidden entries get P = 0.  The work of a unit runs in two phases so that the tensor core never waits
// for all of it: P_low needs only the score tile and goes back at once (dV and the next score tile run
// under the second phase), dS_low needs the dP tile and the P_low values kept in registers.
#pragma once
#include "pipeline_backward_kv_roles.cuh"

namespace kfa {
namespace bwd {
namespace kv {

template <int D, bool BF16>
__device__ __forceinline__ void consumer_role(const Maps& maps, const AttnParams& p, const Work<true>& w, Shared& sh,
                                              uint32_t tmem, uint8_t* s_owner, int wg, int warp, int lane) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    volatile int* abort_word = &sh.abort_word;
    const int r = (warp & 3) * 32 + lane;  // key row inside the tile == tensor-memory lane
    const int owner_row = w.owner0 + r;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float c2 = fabsf(p.scale) * kLog2e;
    const uint64_t c2_pair = f2_pack(c2, c2);

    bool row_ok = owner_row < p.Sk;
    // The mask element of (query head hq, query r, key c) is mask_b[hq*ms[1] + r*ms[2] + c*ms[3]].
    const uint8_t* mask_b = p.has_mask ? p.mask + (int64_t)w.b * p.ms[0] : nullptr;
    const bool key_padding = p.has_mask && p.ms[1] == 0 && p.ms[2] == 0;  // one line for all heads and queries
    if (row_ok && key_padding) row_ok = mask_b[(int64_t)owner_row * p.ms[3]] != 0;

    const uint32_t s_addr = lane_base + kColS + wg * kCols, dp_addr = lane_base + kColDp + wg * kCols;
    int g, i;
    w.begin(p, g, i);
    int unit = 0;
    bool ok = true;
    PH_DECL;
    while (w.valid(g) && ok) {
        PH(5);
        // under key padding (or without a mask) no per-element test is needed: a hidden key is a hidden owner row
        const int state = (key_padding || !p.has_mask) ? 2 : w.state(p, g, i);
        // this thread's line of mask elements (its columns are queries)
        const uint8_t* mline = nullptr;
        if (state == 1)
            mline = mask_b + (int64_t)w.query_head(g) * p.ms[1] + (int64_t)min(owner_row, p.Sk - 1) * p.ms[3];
        // columns [lo, 64) of this thread's 64 are visible: the query index must be >= the key index
        const int col0 = i * kTile + wg * kCols;  // first query of this thread's columns
        int lo = p.causal ? owner_row - col0 : 0;
        if (!row_ok) lo = kCols;
        const bool masked = __any_sync(0xffffffffu, lo > 0) || state == 1;

        // ------------------------------------------------------------ P_low
        PH(4);
        ok = mbar_wait(&sh.s_ready, unit & 1, abort_word, 141);
        if (!ok) break;
        PH(0);
        tc_fence_after();
        uint32_t pw[kCols / 2];
        {
            uint32_t s[kCols];
            tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
            tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
            tmem_wait_ld();
            PH(1);
            auto prob = [&](int c, bool apply_mask) {
                float ea, eb;
                f2_unpack(f2_mul(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), c2_pair), ea, eb);
                float pa = ex2(ea), pb = ex2(eb);
                if (apply_mask) {
                    pa = c >= lo ? pa : 0.f;
                    pb = c + 1 >= lo ? pb : 0.f;
                    if (state == 1) {
                        pa = mline[(int64_t)min(col0 + c, p.Sq - 1) * p.ms[2]] != 0 ? pa : 0.f;
                        pb = mline[(int64_t)min(col0 + c + 1, p.Sq - 1) * p.ms[2]] != 0 ? pb : 0.f;
                    }
                }
                pw[c / 2] = pack2<BF16>(pa, pb);
            };
            // Both consumer warpgroups form probabilities at the same time, and together they ask the
            // special-function unit for one result per score: where no score is hidden (no mask, every streamed
            // query inside the sequence), every fourth pair is evaluated on the FMA and integer pipes instead.
            auto prob_poly = [&](int c) {
                float pa, pb;
                ex2_poly_pair(f2_mul(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), c2_pair), pa, pb);
                pw[c / 2] = pack2<BF16>(pa, pb);
            };
            if (masked) {
#pragma unroll
                for (int c = 0; c < kCols; c += 2) prob(c, true);
            } else if (!p.has_mask && col0 + kCols <= p.Sq) {
#pragma unroll
                for (int c = 0; c < kCols; c += 2) {
                    if ((c & 6) == 6) prob_poly(c);
                    else prob(c, false);
                }
            } else {
#pragma unroll
                for (int c = 0; c < kCols; c += 2) prob(c, false);
            }
        }
        PH(2);
        tmem_st(s_addr, pw);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sh.p_done);
        PH(3);

        // ----------------------------------------------------------- dS_low
        ok = mbar_wait(&sh.dp_ready, unit & 1, abort_word, 142);
        if (!ok) break;
        PH(6);
        tc_fence_after();
        uint32_t dw[kCols / 2];
        {
            uint32_t dp[kCols];
            tmem_ld32(dp_addr, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
            tmem_ld32(dp_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
            tmem_wait_ld();
            PH(1);
#pragma unroll
            for (int c = 0; c < kCols; c += 2) {
                const float2 pl = unpack2<BF16>(pw[c / 2]);
                float da, db;
                f2_unpack(f2_mul(f2_pack(pl.x, pl.y), f2_pack(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1]))),
                          da, db);
                dw[c / 2] = pack2<BF16>(da, db);
            }
        }
        PH(7);
        tmem_st(dp_addr, dw);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sh.ds_done);
        PH(3);
        w.next(p, g, i);
        ++unit;
    }

    PH(5);
    if ((threadIdx.x & 127) == 0) PH_FLUSH(8 + wg);
    // ---------------------------------------------------------------- epilogue
    // Each warpgroup stores D / kGroups channels of every gradient row.
    constexpr int kHalf = D / kGroups;
    const int ch0 = wg * kHalf;
    T* out1 = nullptr;  // dK (scaled)
    T* out2 = nullptr;  // dV
    if (owner_row < p.Sk) {
        out1 = reinterpret_cast<T*>(p.dk) + (int64_t)w.b * p.dks[0] + (int64_t)w.head * p.dks[1] +
               (int64_t)owner_row * p.dks[2] + ch0;
        out2 = reinterpret_cast<T*>(p.dv) + (int64_t)w.b * p.dvs[0] + (int64_t)w.head * p.dvs[1] +
               (int64_t)owner_row * p.dvs[2] + ch0;
    }
    if (p.grad_f32) {
        // FP32 partial gradients of a block-wise call: plain vector stores (or read-add-write) per row
        const bool add = (p.grad_f32 & 4) != 0;
        if (!ok) return;
        const bool live = owner_row < p.Sk;  // (the tensor-memory loads below are warp-wide: every lane runs them)
        float* f1 = reinterpret_cast<float*>(p.dk) + (int64_t)w.b * p.dks[0] + (int64_t)w.head * p.dks[1] +
                    (int64_t)owner_row * p.dks[2] + ch0;
        float* f2 = reinterpret_cast<float*>(p.dv) + (int64_t)w.b * p.dvs[0] + (int64_t)w.head * p.dvs[1] +
                    (int64_t)owner_row * p.dvs[2] + ch0;
        if (unit == 0) {
            if (!add && live)
                for (int d = 0; d < kHalf && ch0 + d < p.D; d += 4) {
                    *reinterpret_cast<float4*>(f1 + d) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4*>(f2 + d) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            return;
        }
        if (!mbar_wait(&sh.final_done, 0, abort_word, 150)) return;
        tc_fence_after();
        constexpr int kStepF = kHalf < 32 ? 16 : 32;
#pragma unroll
        for (int c = 0; c < kHalf; c += kStepF) {
            uint32_t v[kStepF];
            tmem_ld(lane_base + kColDk + ch0 + c, v);
            tmem_wait_ld();
            put_f32(f1 + c, v, live ? p.D - ch0 - c : 0, p.scale, add);
            tmem_ld(lane_base + kColDv + ch0 + c, v);
            tmem_wait_ld();
            put_f32(f2 + c, v, live ? p.D - ch0 - c : 0, 1.f, add);
        }
        return;
    }
    if (unit == 0) {
        // no visible work for this key tile: the gradients are exactly zero
        if (ok && out1)
            for (int d = 0; d < kHalf && ch0 + d < p.D; d += 8) {
                *reinterpret_cast<uint4*>(out1 + d) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(out2 + d) = make_uint4(0, 0, 0, 0);
            }
        return;
    }
    if (ok) ok = mbar_wait(&sh.final_done, 0, abort_word, 150);
    if (!ok) return;
    tc_fence_after();
    // The tiles go through the (now dead) K and V buffers in the swizzled box layout and leave as tiled
    // stores: whole 128-byte lines instead of 16 bytes per row and instruction.  Rows beyond the sequence
    // end are not written by the stores.
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        const uint32_t acc = lane_base + (which == 0 ? kColDk : kColDv) + ch0;
        uint8_t* stage = s_owner + which * Cfg<D>::kTileBytes;
        const float mul = which == 0 ? p.scale : 1.f;
        constexpr int kStep = kHalf < 32 ? 16 : 32;
#pragma unroll
        for (int c = 0; c < kHalf; c += kStep) {
            uint32_t v[kStep];
            tmem_ld(acc + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < kStep; e += 8) {
                uint4 o;
                o.x = pack2<BF16>(__uint_as_float(v[e]) * mul, __uint_as_float(v[e + 1]) * mul);
                o.y = pack2<BF16>(__uint_as_float(v[e + 2]) * mul, __uint_as_float(v[e + 3]) * mul);
                o.z = pack2<BF16>(__uint_as_float(v[e + 4]) * mul, __uint_as_float(v[e + 5]) * mul);
                o.w = pack2<BF16>(__uint_as_float(v[e + 6]) * mul, __uint_as_float(v[e + 7]) * mul);
                const int chunk = (ch0 + c + e) >> 3;
                *reinterpret_cast<uint4*>(stage + (chunk >> 3) * (kTile * 128) + sw128_chunk(r, chunk & 7)) = o;
            }
        }
    }
    fence_async_smem();
    mbar_arrive(&sh.out_staged);
    if (threadIdx.x == 0 && mbar_wait(&sh.out_staged, 0, abort_word, 151)) {
        for (int c = 0; c < Cfg<D>::kChunks; ++c) {
            tma_store_4d(&maps.dk, s_owner + c * (kTile * 128), c * 64, w.owner0, w.head, w.b);
            tma_store_4d(&maps.dv, s_owner + Cfg<D>::kTileBytes + c * (kTile * 128), c * 64, w.owner0, w.head, w.b);
        }
        tma_store_commit();
        tma_store_wait_read();
    }
}

}  // namespace kv
}  // namespace bwd
}  // namespace kfa
