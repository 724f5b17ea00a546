// Key/value-gradient kernel of the backward pass on the tensor-memory pipeline: shared context and the
// loader / MMA-issuer / statistics roles.  The consumer role is in pipeline_backward_kv_consumer.cuh.
//
// A CTA owns 128 key rows of one (batch, K/V head), keeps K and V resident and streams the (Q, dO)
// tiles of every query head in the group that can see its keys; it produces dK = (sum dS_low^T Q) * scale
// and dV = sum P_low^T dO.  One owner per output row, so no atomics are needed.
// Per streamed 128-query tile ("unit") the tensor core runs full 128 x 128 products, which execute at
// the math rate (a 64-column score product is limited by shared-memory operand reads):
//   S  = K x Q^T - 1 x (m + logsum / c)^T        dP = V x dO^T - 1 x delta^T
//   dV += P_low x dO          dK += dS_low x Q    (A operand read from tensor memory)
// and the consumers work in two phases per unit: P_low from S (handed back at once, so that dV and the
// next S run while the consumers continue), then dS_low from dP and the P_low kept in registers.
// The subtraction of the per-query statistics is one more K = 16 step of the score products: the
// statistics warp splits each FP32 statistic exactly into three BF16 pieces and lays them out as a
// 16-channel operand tile, and the other operand is a constant tile of -1 entries.  The consumers thus
// receive shifted scores and shifted dP and need no per-column values of their own: a consumer thread
// owns a key (row), its columns are queries, and fetching three statistics per column from shared
// memory cost more than all of its arithmetic (the shared-memory return path delivers 128 bytes per
// cycle per SM however the loads are shaped).  S - m is formed in the FP32 accumulator with both terms
// at full precision, as the shifted-score contract wants; c = |scale| * log2(e) is applied afterwards.
// Tensor memory (512 columns): S | dP | dV | dK, 128 columns each.  The 16-bit P_low / dS_low of a
// consumer warpgroup overwrite the first 32 of its 64 own S / dP columns.  One thread issues every
// product, in the order that keeps the consumers fed: dV(u), S(u+1), dK(u), dP(u+1).
// (Reference behaviour: src/kohakufa_cute/blackwell_pipeline.py:610-662, 1279-1306 of the
// reference project; arithmetic contract docs/precision.md:13-23.)
#pragma once
#include "pipeline_backward_common.cuh"

namespace kfa {
namespace bwd {
namespace kv {

constexpr int kCols = kTile / kGroups;  // columns of a unit per consumer thread
constexpr int kMaxPairs = 4;
constexpr int kStatTileBytes = kTile * 32;  // 128 rows x 16 BF16 channels, plain (unswizzled) K-major layout
constexpr float kHiddenRow = 3.0e38f;       // "maximum" of a query that saw nothing: every probability becomes zero

template <int D>
struct Cfg {
    static constexpr int kChunks = D / 64;
    static constexpr int kTileBytes = kTile * D * 2;
    static constexpr int kPairs = D == 128 ? 2 : 4;  // ring slots, each holds both streamed operands
    static constexpr int kStatsBytes = 4 * kStatTileBytes;  // two constant tiles, two statistics buffers
    static constexpr int kSmemBytes = 2 * kTileBytes + kPairs * 2 * kTileBytes + kStatsBytes + 1024 + 256;
};

struct Shared {
    uint64_t owner_full;
    uint64_t pair_full[kMaxPairs];
    uint64_t pair_empty[kMaxPairs];
    uint64_t s_ready;      // score tile filled
    uint64_t dp_ready;     // dP tile filled
    uint64_t p_done;       // every consumer stored its P_low
    uint64_t ds_done;      // every consumer stored its dS_low
    uint64_t stats_full[2];
    uint64_t stats_empty[2];
    uint64_t final_done;
    uint64_t out_staged;   // every consumer has put its part of the gradient tiles into shared memory
    uint32_t tmem_base;
    int abort_word;
};

constexpr uint32_t kColS = 0, kColDp = 128, kColDv = 256, kColDk = 384;

// Byte offset of the 16-byte chunk (row n, channels 8*half .. 8*half+7) in a statistics tile: 8-row groups of
// 256 bytes, each holding the two 128-byte core matrices of its channel halves.
__device__ __forceinline__ uint32_t stat_chunk(int n, int half) { return (n >> 3) * 256 + half * 128 + (n & 7) * 16; }

// Shared-memory matrix descriptor of such a tile (no swizzle): 128 bytes between the two channel halves,
// 256 bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 16;  // leading-dimension offset: between the channel halves
    d |= static_cast<uint64_t>(256 >> 4) << 32;  // stride offset: between 8-row groups
    d |= 1ull << 46;  // descriptor version for sm_100
    return d;
}

template <int D>
__device__ __forceinline__ void loader_role(const Maps& maps, const AttnParams& p, const Work<true>& w, Shared& sh,
                                            uint8_t* s_owner, uint8_t* s_ring) {
    using C = Cfg<D>;
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.g);
    mbar_expect_tx(&sh.owner_full, 2 * C::kTileBytes);
    for (int c = 0; c < C::kChunks; ++c) {
        tma_load_4d(s_owner + c * (kTile * 128), &maps.k, &sh.owner_full, c * 64, w.owner0, w.head, w.b);
        tma_load_4d(s_owner + C::kTileBytes + c * (kTile * 128), &maps.v, &sh.owner_full, c * 64, w.owner0, w.head,
                    w.b);
    }
    int unit = 0;
    bool ok = true;
    while (w.valid(g) && ok) {
        const int slot = unit % C::kPairs, round = unit / C::kPairs;
        if (round > 0) ok = mbar_wait(&sh.pair_empty[slot], (round - 1) & 1, abort_word, 110);
        if (!ok) break;
        const int head = w.query_head(g);
        uint8_t* dst = s_ring + slot * 2 * C::kTileBytes;
        mbar_expect_tx(&sh.pair_full[slot], 2 * C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c) {
            tma_load_4d(dst + c * (kTile * 128), &maps.q, &sh.pair_full[slot], c * 64, i * kTile, head, w.b);
            tma_load_4d(dst + C::kTileBytes + c * (kTile * 128), &maps.g, &sh.pair_full[slot], c * 64, i * kTile,
                        head, w.b);
        }
        w.next(p, g, i);
        ++unit;
    }
}

// One thread issues all tensor-core work.  Per unit u, once P_low(u) is back: dV += P_low(u) x dO(u), then
// S(u+1) into the score columns that product has just read; once dS_low(u) is back: dK += dS_low(u) x Q(u),
// then dP(u+1) into the dP columns.  The consumers form dS_low(u) while dV(u) and S(u+1) run, and P_low(u+1)
// while dK(u) and dP(u+1) run.
template <int D, bool BF16>
__device__ __forceinline__ void mma_role(const AttnParams& p, const Work<true>& w, Shared& sh, uint32_t tmem,
                                         uint8_t* s_owner, uint8_t* s_ring, uint8_t* s_stat) {
    using C = Cfg<D>;
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    // A negative scale takes maxima over -S: the forward saved statistics of -S, so negate operand A.
    const uint32_t idesc_s = umma_idesc(kTile, kTile, BF16 ? 1 : 0, false, false);
    const uint32_t idesc_neg = idesc_s | (p.scale < 0.f ? kUmmaNegateA : 0u);
    constexpr uint32_t idesc_x = umma_idesc(kTile, kTile, 1, false, false);  // the statistics step: BF16 tiles, never negated
    constexpr uint32_t idesc_g = umma_idesc(kTile, D, BF16 ? 1 : 0, false, true);
    const uint32_t own = smem_u32(s_owner), ring = smem_u32(s_ring);
    // Descriptors are built once; per instruction only the start-address field advances.
    const uint64_t own_desc = umma_desc_sw128(own, 16, 1024);
    const uint64_t ring_k_desc = umma_desc_sw128(ring, 16, 1024);            // K-major view (score products)
    const uint64_t ring_mn_desc = umma_desc_sw128(ring, kTile * 128, 1024);  // MN-major view (gradient products)
    const uint64_t ones_desc = umma_desc_plain(smem_u32(s_stat));
    const uint64_t stat_desc = umma_desc_plain(smem_u32(s_stat) + 2 * kStatTileBytes);

    // which: 0 = S (K with Q), 1 = dP (V with dO)
    auto issue_scores = [&](int slot, int which, int stat_buf) {
        const uint32_t st = slot * 2 * C::kTileBytes + which * C::kTileBytes;
        const uint32_t col = tmem + (which == 0 ? kColS : kColDp);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
            umma_ss(col, umma_desc_advance(own_desc, which * C::kTileBytes + off),
                    umma_desc_advance(ring_k_desc, st + off), which == 0 ? idesc_neg : idesc_s, kk > 0);
        }
        // minus the statistics of the unit's 128 queries
        umma_ss(col, umma_desc_advance(ones_desc, which * kStatTileBytes),
                umma_desc_advance(stat_desc, stat_buf * kStatTileBytes), idesc_x, 1);
    };
    // which: 0 = dV (P_low in the S columns, with dO), 1 = dK (dS_low in the dP columns, with Q)
    auto issue_grads = [&](int slot, int which, bool accumulate) {
        const uint32_t st = slot * 2 * C::kTileBytes + (1 - which) * C::kTileBytes;
        const uint32_t a_col = tmem + (which == 0 ? kColS : kColDp);
        const uint32_t d_col = tmem + (which == 0 ? kColDv : kColDk);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
            // consumer warpgroup g keeps its 64 columns as 32 packed columns at the head of its own range
            const uint32_t a_off = (kk / 4) * kCols + (kk % 4) * 8;
            umma_ts(d_col, a_col + a_off, umma_desc_advance(ring_mn_desc, st + kk * 2048), idesc_g,
                    accumulate || kk > 0);
        }
    };

    bool ok = mbar_wait(&sh.owner_full, 0, abort_word, 120);
    if (ok) ok = mbar_wait(&sh.pair_full[0], 0, abort_word, 121);
    if (ok) ok = mbar_wait(&sh.stats_full[0], 0, abort_word, 125);
    if (!ok) return;
    tc_fence_after();
    issue_scores(0, 0, 0);
    umma_commit(&sh.s_ready);
    issue_scores(0, 1, 0);
    umma_commit(&sh.dp_ready);
    umma_commit(&sh.stats_empty[0]);
    int unit = 0;
    PH_DECL;
    while (w.valid(g) && ok) {
        int gn = g, in = i;
        w.next(p, gn, in);
        const bool more = w.valid(gn);
        const int slot = unit % C::kPairs, nslot = (unit + 1) % C::kPairs, nbuf = (unit + 1) & 1;
        PH(4);
        ok = mbar_wait(&sh.p_done, unit & 1, abort_word, 122);
        if (!ok) break;
        PH(0);
        tc_fence_after();
        issue_grads(slot, 0, unit > 0);
        PH(1);
        if (more) {
            ok = mbar_wait(&sh.pair_full[nslot], ((unit + 1) / C::kPairs) & 1, abort_word, 124);
            if (ok) ok = mbar_wait(&sh.stats_full[nbuf], ((unit + 1) >> 1) & 1, abort_word, 125);
            if (!ok) break;
            PH(2);
            tc_fence_after();
            issue_scores(nslot, 0, nbuf);
            umma_commit(&sh.s_ready);
            PH(3);
        }
        ok = mbar_wait(&sh.ds_done, unit & 1, abort_word, 123);
        if (!ok) break;
        PH(5);
        tc_fence_after();
        issue_grads(slot, 1, unit > 0);
        umma_commit(&sh.pair_empty[slot]);
        PH(1);
        if (more) {
            issue_scores(nslot, 1, nbuf);
            umma_commit(&sh.dp_ready);
            umma_commit(&sh.stats_empty[nbuf]);
            PH(3);
        }
        g = gn;
        i = in;
        ++unit;
    }
    if (ok) umma_commit(&sh.final_done);
    PH_FLUSH(8 + 2);
}

// Splits an FP32 value into three BF16 pieces whose sum is the value (each piece takes the leading eight
// significant bits of what is left).
__device__ __forceinline__ void split3(float x, uint32_t& h1, uint32_t& h2, uint32_t& h3) {
    const __nv_bfloat16 a = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(a);
    const __nv_bfloat16 b = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(b);
    const __nv_bfloat16 c = __float2bfloat16_rn(r2);
    h1 = __bfloat16_as_ushort(a);
    h2 = __bfloat16_as_ushort(b);
    h3 = __bfloat16_as_ushort(c);
}

// One warp prepares the operand tiles of the statistics step.  Once: two constant tiles with -1 in the
// channels that carry (m, logsum / c) and delta respectively.  Per unit: for each of the 128 streamed
// queries the row [m1 m2 m3 l1 l2 l3 0 0 | d1 d2 d3 0 0 0 0 0] of BF16 pieces.  A query beyond the
// sequence end, or one that saw no key in the forward pass (maximum = -inf), gets a huge maximum so
// that its probabilities evaluate to exactly zero.
__device__ __forceinline__ void stats_role(const AttnParams& p, const Work<true>& w, Shared& sh, uint8_t* s_stat,
                                           int lane) {
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    const float inv_c2 = 1.f / (fabsf(p.scale) * kLog2e);
    constexpr uint32_t kMinusOne = 0xBF80u;  // BF16 -1
    for (int n = lane; n < kTile; n += 32) {
        const uint4 six = make_uint4(kMinusOne | (kMinusOne << 16), kMinusOne | (kMinusOne << 16),
                                     kMinusOne | (kMinusOne << 16), 0u);
        const uint4 three = make_uint4(kMinusOne | (kMinusOne << 16), kMinusOne, 0u, 0u);
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(s_stat + stat_chunk(n, 0)) = six;                      // S: channels 0..5
        *reinterpret_cast<uint4*>(s_stat + stat_chunk(n, 1)) = zero;
        *reinterpret_cast<uint4*>(s_stat + kStatTileBytes + stat_chunk(n, 0)) = zero;    // dP: channels 8..10
        *reinterpret_cast<uint4*>(s_stat + kStatTileBytes + stat_chunk(n, 1)) = three;
    }
    int unit = 0;
    bool ok = true;
    while (w.valid(g) && ok) {
        const int buf = unit & 1;
        if (unit >= 2) ok = mbar_wait(&sh.stats_empty[buf], ((unit >> 1) - 1) & 1, abort_word, 130);
        if (!ok) break;
        const int64_t base = ((int64_t)w.b * p.Hq + w.query_head(g)) * p.Sq;
        uint8_t* dst = s_stat + (2 + buf) * kStatTileBytes;
        // all twelve loads first: they are independent, and one memory latency per unit is what this warp can afford
        float m[kTile / 32], ls[kTile / 32], dl[kTile / 32];
#pragma unroll
        for (int j = 0; j < kTile / 32; ++j) {
            const int row = i * kTile + j * 32 + lane;
            m[j] = kHiddenRow, ls[j] = 0.f, dl[j] = 0.f;
            if (row < p.Sq) {
                m[j] = p.maximum[base + row];
                ls[j] = p.logsum[base + row];
                dl[j] = p.delta[base + row];
            }
        }
#pragma unroll
        for (int j = 0; j < kTile / 32; ++j) {
            const int c = j * 32 + lane;
            if (m[j] == -INFINITY) m[j] = kHiddenRow, ls[j] = 0.f;
            uint32_t m1, m2, m3, l1, l2, l3, d1, d2, d3;
            split3(m[j], m1, m2, m3);
            split3(ls[j] * inv_c2, l1, l2, l3);
            split3(dl[j], d1, d2, d3);
            *reinterpret_cast<uint4*>(dst + stat_chunk(c, 0)) = make_uint4(m1 | (m2 << 16), m3 | (l1 << 16), l2 | (l3 << 16), 0u);
            *reinterpret_cast<uint4*>(dst + stat_chunk(c, 1)) = make_uint4(d1 | (d2 << 16), d3, 0u, 0u);
        }
        fence_async_smem();  // the tensor core reads these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.stats_full[buf]);
        w.next(p, g, i);
        ++unit;
    }
}

}  // namespace kv
}  // namespace bwd
}  // namespace kfa
