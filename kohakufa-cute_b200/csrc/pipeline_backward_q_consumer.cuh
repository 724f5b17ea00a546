// Consumer warpgroups of the query-gradient kernel: scores -> P -> dS, and the dQ epilogue.
//
// A consumer thread owns one query row (tensor-memory lane) and 64 of the 128 key columns of every
// unit (warpgroup g takes columns [g*64, (g+1)*64)).  Per element, in FP32:
//   P      = ex2((s' - m) * |scale| * log2e - logsum)      s' arrives already sign-adjusted
//   P_low  = round(P)                                       one rounding to the input type
//   dS_low = round(P_low * (dP - delta))
// m, logsum and delta belong to the query row and live in registers.  Hidden entries get P = 0.
// P_low of a unit is formed as soon as its score tile is there (the tensor core is still busy with
// the previous unit's dQ and this unit's dP); the dP values are then pulled into registers, the dP
// buffer is handed back, and dS_low is packed over the thread's own (dead) score columns.
#pragma once
#include "pipeline_backward_q_roles.cuh"

namespace kfa {
namespace bwd {
namespace q {

template <int D, bool BF16>
__device__ __forceinline__ void consumer_role(const Maps& maps, const AttnParams& p, const Work<false>& w, Shared& sh,
                                              uint32_t tmem, uint8_t* s_owner, int wg, int warp, int lane) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    volatile int* abort_word = &sh.abort_word;
    const int r = (warp & 3) * 32 + lane;  // query row inside the tile == tensor-memory lane
    const int owner_row = w.owner0 + r;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float c2 = fabsf(p.scale) * kLog2e;
    const uint64_t c2_pair = f2_pack(c2, c2);

    float row_m = INFINITY, row_ls = 0.f, row_dl = 0.f;
    if (owner_row < p.Sq) {
        const int64_t si = ((int64_t)w.b * p.Hq + w.head) * p.Sq + owner_row;
        row_m = p.maximum[si];
        row_ls = p.logsum[si];
        row_dl = p.delta[si];
        if (row_m == -INFINITY) row_m = INFINITY;  // nothing visible: every P is zero
    }
    const uint64_t m_pair = f2_pack(row_m, row_m), ls_pair = f2_pack(row_ls, row_ls), dl_pair = f2_pack(row_dl, row_dl);
    // The mask element of (query head h, query r, key c) is mask_b[h*ms[1] + r*ms[2] + c*ms[3]].
    const uint8_t* mline_head = p.has_mask ? p.mask + (int64_t)w.b * p.ms[0] + (int64_t)w.head * p.ms[1] +
                                                 (int64_t)min(owner_row, p.Sq - 1) * p.ms[2]
                                           : nullptr;

    // every row of this warp has visible keys (no mask, no row beyond the sequence end): statistics are finite
    const bool rows_real = !p.has_mask && __all_sync(0xffffffffu, owner_row < p.Sq && row_m != INFINITY);
    int g, i;
    w.begin(p, g, i);
    int unit = 0;
    bool ok = true;
    PH_DECL;
    while (w.valid(g) && ok) {
        PH(5);
        const int state = w.state(p, g, i);
        const int x = unit & 1;  // score buffer of this unit
        const uint32_t s_addr = lane_base + kColS + x * 128 + wg * kCols;
        const uint32_t dp_addr = lane_base + kColDp + wg * kCols;
        // leading columns of this thread's 64 that pass the sequence end and the causal bound
        const int col0 = i * kTile + wg * kCols;
        int hi = p.Sk - col0;
        if (p.causal) hi = min(hi, owner_row - col0 + 1);
        const bool masked = __any_sync(0xffffffffu, hi < kCols) || state == 1;

        // ------------------------------------------------------------ P_low
        PH(4);
        ok = mbar_wait(&sh.s_ready[x], (unit >> 1) & 1, abort_word, 141);
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
                f2_unpack(f2_sub(f2_mul(f2_sub(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), m_pair),
                                        c2_pair), ls_pair), ea, eb);
                float pa = ex2(ea), pb = ex2(eb);
                if (apply_mask) {
                    pa = c < hi ? pa : 0.f;
                    pb = c + 1 < hi ? pb : 0.f;
                    if (state == 1) {
                        pa = mline_head[(int64_t)min(col0 + c, p.Sk - 1) * p.ms[3]] != 0 ? pa : 0.f;
                        pb = mline_head[(int64_t)min(col0 + c + 1, p.Sk - 1) * p.ms[3]] != 0 ? pb : 0.f;
                    }
                }
                pw[c / 2] = pack2<BF16>(pa, pb);
            };
            // Both consumer warpgroups form probabilities at the same time, and together they ask the
            // special-function unit for one result per score: where no score is hidden, every fourth pair is
            // evaluated on the FMA and integer pipes instead.
            auto prob_poly = [&](int c) {
                float pa, pb;
                ex2_poly_pair(f2_sub(f2_mul(f2_sub(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), m_pair),
                                            c2_pair), ls_pair), pa, pb);
                pw[c / 2] = pack2<BF16>(pa, pb);
            };
            if (masked) {
#pragma unroll
                for (int c = 0; c < kCols; c += 2) prob(c, true);
            } else if (rows_real) {
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
            // the dP buffer may be refilled: the next dP product runs under the arithmetic below
            tc_fence_before();
            mbar_arrive(&sh.dp_free);
            PH(1);
#pragma unroll
            for (int c = 0; c < kCols; c += 2) {
                const float2 pl = unpack2<BF16>(pw[c / 2]);
                float da, db;
                f2_unpack(f2_mul(f2_pack(pl.x, pl.y),
                                 f2_sub(f2_pack(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), dl_pair)),
                          da, db);
                dw[c / 2] = pack2<BF16>(da, db);
            }
        }
        PH(7);
        tmem_st(s_addr, dw);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sh.ds_done);
        PH(3);
        w.next(p, g, i);
        ++unit;
    }

    PH(5);
    if ((threadIdx.x & 127) == 0) PH_FLUSH(wg);
    // ---------------------------------------------------------------- epilogue
    // Each warpgroup stores D / kGroups channels of every dQ row.
    constexpr int kHalf = D / kGroups;
    const int ch0 = wg * kHalf;
    T* out = nullptr;
    if (owner_row < p.Sq)
        out = reinterpret_cast<T*>(p.dq) + (int64_t)w.b * p.dqs[0] + (int64_t)w.head * p.dqs[1] +
              (int64_t)owner_row * p.dqs[2] + ch0;
    if (p.grad_f32) {
        // FP32 partial gradient of a block-wise call: plain vector stores (or read-add-write) per row
        const bool add = (p.grad_f32 & 2) != 0;
        if (!ok) return;
        const bool live = owner_row < p.Sq;  // (the tensor-memory loads below are warp-wide: every lane runs them)
        float* f = reinterpret_cast<float*>(p.dq) + (int64_t)w.b * p.dqs[0] + (int64_t)w.head * p.dqs[1] +
                   (int64_t)owner_row * p.dqs[2] + ch0;
        if (unit == 0) {
            if (!add && live)
                for (int d = 0; d < kHalf && ch0 + d < p.D; d += 4)
                    *reinterpret_cast<float4*>(f + d) = make_float4(0.f, 0.f, 0.f, 0.f);
            return;
        }
        if (!mbar_wait(&sh.final_done, 0, abort_word, 150)) return;
        tc_fence_after();
        constexpr int kStepF = kHalf < 32 ? 16 : 32;
#pragma unroll
        for (int c = 0; c < kHalf; c += kStepF) {
            uint32_t v[kStepF];
            tmem_ld(lane_base + kColGrad + ch0 + c, v);
            tmem_wait_ld();
            put_f32(f + c, v, live ? p.D - ch0 - c : 0, p.scale, add);
        }
        return;
    }
    if (unit == 0) {
        // no visible work for this query tile: the gradient is exactly zero
        if (ok && out)
            for (int d = 0; d < kHalf && ch0 + d < p.D; d += 8) *reinterpret_cast<uint4*>(out + d) = make_uint4(0, 0, 0, 0);
        return;
    }
    if (ok) ok = mbar_wait(&sh.final_done, 0, abort_word, 150);
    if (!ok) return;
    tc_fence_after();
    // The scaled tile goes through the (now dead) Q buffer in the swizzled box layout and leaves as tiled
    // stores: whole 128-byte lines instead of 16 bytes per row and instruction.  Rows beyond the sequence
    // end are not written by the store.
    const uint32_t acc = lane_base + kColGrad + ch0;
    const float mul = p.scale;
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
            *reinterpret_cast<uint4*>(s_owner + (chunk >> 3) * (kTile * 128) + sw128_chunk(r, chunk & 7)) = o;
        }
    }
    fence_async_smem();
    mbar_arrive(&sh.out_staged);
    if (threadIdx.x == 0 && mbar_wait(&sh.out_staged, 0, abort_word, 151)) {
        for (int c = 0; c < Cfg<D>::kChunks; ++c)
            tma_store_4d(&maps.dq, s_owner + c * (kTile * 128), c * 64, w.owner0, w.head, w.b);
        tma_store_commit();
        tma_store_wait_read();
    }
}

}  // namespace q
}  // namespace bwd
}  // namespace kfa
