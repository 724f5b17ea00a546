// Backward pass on the tensor-memory pipeline: shared context, work iteration, and the
// loader / MMA-issuer / statistics roles.  The consumer role is in
// pipeline_backward_consumer.cuh and the kernel itself in pipeline_backward.cu.
//
// One kernel template serves both gradient owners:
//   KV = false  a CTA owns 128 query rows of one (batch, query head) and streams key tiles;
//               it produces dQ = (sum dS_low K) * scale.
//   KV = true   a CTA owns 128 key rows of one (batch, K/V head) and streams the query tiles of
//               every query head in the group; it produces dK = (sum dS_low^T Q) * scale and
//               dV = sum P_low^T dO.  One owner per output row, so no atomics are needed.
// Each streamed 128-row tile is processed as two 64-wide sub-tiles in two tensor-memory buffers:
// while the consumer warpgroups turn one sub-tile's scores into P and dS (64 / kGroups columns each),
// the tensor core works on the other sub-tile.  Per sub-tile the tensor core runs
//   S  = A1 x B1^T   (A1 = owner operand 1: Q or K;  B1 = streamed operand 1: K or Q)
//   dP = A2 x B2^T   (A2 = owner operand 2: dO or V; B2 = streamed operand 2: V or dO)
//   grad1 += dS_low x B1      (dQ, or dK)          A operand read from tensor memory
//   grad2 += P_low  x B2      (dV; KV only)        A operand read from tensor memory
// Tensor memory (512 columns): [S_0 | dP_0 | S_1 | dP_1] 64 columns each, grad2 at 256, grad1 at
// 384.  The 16-bit P and dS overwrite the first 32 columns of their own S / dP buffer.
// (Reference behaviour: src/kohakufa_cute/blackwell_pipeline.py:610-662, 1279-1306 of the
// reference project; arithmetic contract docs/precision.md:13-23.)
#pragma once
#include "kfa_common.cuh"
#include "sm100_ptx.cuh"

namespace kfa {
namespace bwd {

constexpr int kTile = 128;     // owner rows, and rows of a streamed tile
constexpr int kSub = 64;       // columns of one sub-tile
#ifndef KFA_BWD_CONSUMER_GROUPS
#define KFA_BWD_CONSUMER_GROUPS 2
#endif
constexpr int kGroups = KFA_BWD_CONSUMER_GROUPS;  // consumer warpgroups; each takes 64 / kGroups columns of a sub-tile
constexpr int kCols = kSub / kGroups;
constexpr int kConsumers = 128 * kGroups;
constexpr int kRoleWarp = 4 * kGroups;            // first warp of the role warpgroup: MMA 0, MMA 1, loader, statistics
constexpr int kThreads = kConsumers + 128;
constexpr int kMaxPairs = 4;

template <int D>
struct Cfg {
    static constexpr int kChunks = D / 64;
    static constexpr int kTileBytes = kTile * D * 2;
    static constexpr int kPairs = D == 128 ? 2 : 4;  // ring slots, each holds both streamed operands
    static constexpr int kStatsBytes = 2 * 3 * kTile * 4;
    static constexpr int kSmemBytes = 2 * kTileBytes + kPairs * 2 * kTileBytes + kStatsBytes + 1024 + 256;
};

struct Maps {
    CUtensorMap q, k, v, g;  // g = dO
};

struct Shared {
    uint64_t owner_full;
    uint64_t pair_full[kMaxPairs];
    uint64_t pair_empty[kMaxPairs];
    uint64_t sdp_ready[2];
    uint64_t done[2];
    uint64_t stats_full[2];
    uint64_t stats_empty[2];
    uint64_t final_done;
    uint32_t tmem_base;
    int abort_word;
};

// Combined state of the 128 queries [q_lo, q_lo + 128) x 128 keys of tile j for query head h, from
// the 64x64 table entries: 0 hidden, 2 visible, 1 mixed.  Collapsed (broadcast) axes of the table have
// stride 0, so a mask broadcast over queries reads one row of entries.
__device__ __forceinline__ int tile_state(const AttnParams& p, int b, int h, int q_lo, int j) {
    if (!p.has_mask) return 2;
    const int nk64 = (p.Sk + 63) >> 6;
    const int32_t* base = p.blocks + (int64_t)b * p.bs[0] + (int64_t)h * p.bs[1];
    // two row blocks x two key blocks; the four loads are independent (one memory latency, not four)
    const int64_t r0 = (int64_t)(q_lo >> 6) * p.bs[2];
    const int64_t r1 = (int64_t)((min(q_lo + kTile, p.Sq) - 1) >> 6) * p.bs[2];
    const int64_t c0 = (int64_t)(2 * j) * p.bs[3], c1 = (int64_t)min(2 * j + 1, nk64 - 1) * p.bs[3];
    const int s00 = base[r0 + c0], s01 = base[r0 + c1], s10 = base[r1 + c0], s11 = base[r1 + c1];
    if ((s00 | s01 | s10 | s11) == 0) return 0;
    return (s00 & s01 & s10 & s11) == 2 ? 2 : 1;
}

// The CTA's place in the problem and its stream of work units.
template <bool KV>
struct Work {
    int b, head, owner0;  // batch, owner head (query head or K/V head), first owner row
    int first, end;       // streamed tile range [first, end)
    int groups;           // query heads per owner (KV) or 1
    int fixed;            // state shared by every unit of this CTA (2 without a mask), or -1: look each unit up

    __device__ __forceinline__ void init(const AttnParams& p) {
        const int owner_len = KV ? p.Sk : p.Sq;
        const int heads = KV ? p.Hkv : p.Hq;
        const int nblk = (owner_len + kTile - 1) / kTile;
        // Heavy tiles first (late query tiles, early key tiles under a causal mask).  Large grids go head by
        // head; grids of a few waves go tile row by tile row over all heads, so that no head's heavy tiles
        // start in the last wave.
        const int64_t nbh = (int64_t)p.B * heads;
        const bool by_row = (int64_t)gridDim.x < KFA_ROW_MAJOR_LIMIT;
        int blk = (int)(by_row ? blockIdx.x / nbh : blockIdx.x % nblk);
        if (!KV) blk = nblk - 1 - blk;
        const int64_t bh = by_row ? blockIdx.x % nbh : blockIdx.x / nblk;
        head = (int)(bh % heads);
        b = (int)(bh / heads);
        owner0 = blk * kTile;
        fixed = p.has_mask ? -1 : 2;
        if (KV) {
            groups = p.group;
            first = p.causal ? owner0 / kTile : 0;  // only queries r >= key see the key
            end = (p.Sq + kTile - 1) / kTile;
            // key padding (one line of mask for all queries and heads): a hidden key tile has no work at all
            if (p.has_mask && p.bs[1] == 0 && p.bs[2] == 0) {
                fixed = tile_state(p, b, 0, 0, blk);
                if (fixed == 0) end = first;
            }
        } else {
            groups = 1;
            first = 0;
            const int row_hi = min(p.Sq, owner0 + kTile);
            const int k_hi = p.causal ? min(p.Sk, row_hi) : p.Sk;
            end = (k_hi + kTile - 1) / kTile;
        }
    }
    // Unit cursor: (g, i) = (query head of the group, streamed tile).  Units whose 128 x 128 block the mask
    // table marks hidden are skipped; every role walks the same sequence.
    __device__ __forceinline__ int state(const AttnParams& p, int g, int i) const {
        if (fixed >= 0) return fixed;
        return KV ? tile_state(p, b, head * groups + g, i * kTile, owner0 / kTile)
                  : tile_state(p, b, head, owner0, i);
    }
    __device__ __forceinline__ void settle(const AttnParams& p, int& g, int& i) const {
        while (g < groups) {
            while (i < end && state(p, g, i) == 0) ++i;
            if (i < end) return;
            ++g;
            i = first;
        }
    }
    __device__ __forceinline__ void begin(const AttnParams& p, int& g, int& i) const {
        g = first < end ? 0 : groups;
        i = first;
        settle(p, g, i);
    }
    __device__ __forceinline__ void next(const AttnParams& p, int& g, int& i) const {
        ++i;
        settle(p, g, i);
    }
    __device__ __forceinline__ bool valid(int g) const { return g < groups; }
    __device__ __forceinline__ int query_head(int g) const { return KV ? head * groups + g : head; }
};

template <int D, bool KV>
__device__ __forceinline__ void loader_role(const Maps& maps, const AttnParams& p, const Work<KV>& w, Shared& sh,
                                            uint8_t* s_owner, uint8_t* s_ring) {
    using C = Cfg<D>;
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    const int kvh = KV ? w.head : w.head / p.group;
    // owner operands: (K, V) for key owners, (Q, dO) for query owners
    const CUtensorMap* own1 = KV ? &maps.k : &maps.q;
    const CUtensorMap* own2 = KV ? &maps.v : &maps.g;
    tma_prefetch_desc(own1);
    tma_prefetch_desc(own2);
    mbar_expect_tx(&sh.owner_full, 2 * C::kTileBytes);
    for (int c = 0; c < C::kChunks; ++c) {
        tma_load_4d(s_owner + c * (kTile * 128), own1, &sh.owner_full, c * 64, w.owner0, w.head, w.b);
        tma_load_4d(s_owner + C::kTileBytes + c * (kTile * 128), own2, &sh.owner_full, c * 64, w.owner0, w.head, w.b);
    }
    const CUtensorMap* st1 = KV ? &maps.q : &maps.k;
    const CUtensorMap* st2 = KV ? &maps.g : &maps.v;
    int unit = 0;
    bool ok = true;
    while (w.valid(g) && ok) {
        const int slot = unit % C::kPairs, round = unit / C::kPairs;
        if (round > 0) ok = mbar_wait(&sh.pair_empty[slot], (round - 1) & 1, abort_word, 110);
        if (!ok) break;
        const int head = KV ? w.query_head(g) : kvh;
        uint8_t* dst = s_ring + slot * 2 * C::kTileBytes;
        mbar_expect_tx(&sh.pair_full[slot], 2 * C::kTileBytes);
        for (int c = 0; c < C::kChunks; ++c) {
            tma_load_4d(dst + c * (kTile * 128), st1, &sh.pair_full[slot], c * 64, i * kTile, head, w.b);
            tma_load_4d(dst + C::kTileBytes + c * (kTile * 128), st2, &sh.pair_full[slot], c * 64, i * kTile, head,
                        w.b);
        }
        w.next(p, g, i);
        ++unit;
    }
}

// Two threads issue the tensor-core work, each its own in-order chain per sub-tile buffer b:
//   chain 0:  grad2 += P_low x B2 (key owners) ... then S_b of the sub-tile after next
//   chain 1:  grad1 += dS_low x B1            ... then dP_b of the sub-tile after next
// A tcgen05.mma occupies its issuing thread for about a hundred cycles, so two issuers keep the
// tensor core much busier than one.  The split follows the buffers: everything that reads or
// overwrites S_b (and the P_low packed into it) is in chain 0, everything that touches dP_b
// (and dS_low) in chain 1, so no ordering between the two threads is needed.
template <int D, bool BF16, bool KV>
__device__ __forceinline__ void mma_role(const AttnParams& p, const Work<KV>& w, Shared& sh, uint32_t tmem,
                                         uint8_t* s_owner, uint8_t* s_ring, int chain) {
    using C = Cfg<D>;
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    // A negative scale takes maxima over -S: the forward saved statistics of -S, so negate operand A.
    const uint32_t idesc_s = umma_idesc(kTile, kSub, BF16 ? 1 : 0, false, false) |
                             (chain == 0 && p.scale < 0.f ? kUmmaNegateA : 0u);
    constexpr uint32_t idesc_g = umma_idesc(kTile, D, BF16 ? 1 : 0, false, true);
    // chain 0 works with owner/streamed operand 1 for scores and streamed operand 2 for its gradient;
    // chain 1 the other way round.
    const uint32_t own = smem_u32(s_owner) + chain * C::kTileBytes, ring = smem_u32(s_ring);
    const uint32_t score_src = chain * C::kTileBytes;        // streamed operand feeding S (0) / dP (1)
    const uint32_t grad_src = (1 - chain) * C::kTileBytes;   // streamed operand feeding grad2 (0) / grad1 (1)
    const uint32_t grad_col = tmem + (chain == 0 ? 256 : 384);
    const bool has_grad = KV || chain == 1;
    // Descriptors are built once; per instruction only the start-address field advances.
    const uint64_t own_desc = umma_desc_sw128(own, 16, 1024);
    const uint64_t ring_k_desc = umma_desc_sw128(ring, 16, 1024);            // K-major view (score products)
    const uint64_t ring_mn_desc = umma_desc_sw128(ring, kTile * 128, 1024);  // MN-major view (gradient products)

    auto issue_scores = [&](int slot, int sub) {
        const uint32_t st = slot * 2 * C::kTileBytes + score_src + sub * 8192;
        const uint32_t col = tmem + sub * 128 + chain * 64;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
            umma_ss(col, umma_desc_advance(own_desc, off), umma_desc_advance(ring_k_desc, st + off), idesc_s, kk > 0);
        }
        umma_commit(&sh.sdp_ready[sub]);
    };
    auto issue_grads = [&](int slot, int sub, bool accumulate) {
        const uint32_t st = slot * 2 * C::kTileBytes + grad_src;
        const uint32_t a_col = tmem + sub * 128 + chain * 64;
#pragma unroll
        for (int kk = 0; kk < kSub / 16; ++kk) {
            const uint32_t rows = (sub * 4 + kk) * 2048;  // 16 streamed rows per step, 128 bytes each
            // each consumer warpgroup packs its kCols columns into the first kCols/2 columns of its own range
            const uint32_t a_off = ((kk * 16) / kCols) * kCols + ((kk * 16) % kCols) / 2;
            umma_ts(grad_col, a_col + a_off, umma_desc_advance(ring_mn_desc, st + rows), idesc_g,
                    accumulate || kk > 0);
        }
    };

    bool ok = mbar_wait(&sh.owner_full, 0, abort_word, 120);
    if (ok) ok = mbar_wait(&sh.pair_full[0], 0, abort_word, 121);
    if (!ok) return;
    tc_fence_after();
    issue_scores(0, 0);
    issue_scores(0, 1);
    int unit = 0;
    while (w.valid(g) && ok) {
        int gn = g, in = i;
        w.next(p, gn, in);
        const bool more = w.valid(gn);
        const int slot = unit % C::kPairs, nslot = (unit + 1) % C::kPairs;
        for (int sub = 0; sub < 2 && ok; ++sub) {
            KFA_TRACE_POINT(chain * 2, 1);
            ok = mbar_wait(&sh.done[sub], unit & 1, abort_word, 122 + sub);
            if (!ok) break;
            KFA_TRACE_POINT(chain * 2, 2);
            tc_fence_after();
            if (has_grad) issue_grads(slot, sub, unit > 0 || sub > 0);
            KFA_TRACE_POINT(chain * 2, 3);
            if (sub == 1) umma_commit(&sh.pair_empty[slot]);
            if (more) {
                if (sub == 0) {
                    ok = mbar_wait(&sh.pair_full[nslot], ((unit + 1) / C::kPairs) & 1, abort_word, 124);
                    if (!ok) break;
                    tc_fence_after();
                }
                issue_scores(nslot, sub);
                KFA_TRACE_POINT(chain * 2, 4);
            }
        }
        g = gn;
        i = in;
        ++unit;
    }
    if (ok) umma_commit(&sh.final_done);
}

// Key owners need the three row statistics of every streamed query: one warp stages them.
// A query beyond the sequence end, or one that saw no key in the forward pass (maximum = -inf),
// gets maximum = +inf so that its probabilities evaluate to exactly zero.
template <bool KV>
__device__ __forceinline__ void stats_role(const AttnParams& p, const Work<KV>& w, Shared& sh, float* s_stats,
                                           int lane) {
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    int unit = 0;
    bool ok = true;
    while (w.valid(g) && ok) {
        const int buf = unit & 1;
        if (unit >= 2) ok = mbar_wait(&sh.stats_empty[buf], ((unit >> 1) - 1) & 1, abort_word, 130);
        if (!ok) break;
        const int64_t base = ((int64_t)w.b * p.Hq + w.query_head(g)) * p.Sq;
        float* dst = s_stats + buf * 3 * kTile;
        for (int c = lane; c < kTile; c += 32) {
            const int row = i * kTile + c;
            float m = INFINITY, ls = 0.f, dl = 0.f;
            if (row < p.Sq) {
                m = p.maximum[base + row];
                ls = p.logsum[base + row];
                dl = p.delta[base + row];
                if (m == -INFINITY) m = INFINITY;
            }
            dst[c] = m;
            dst[kTile + c] = ls;
            dst[2 * kTile + c] = dl;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.stats_full[buf]);
        w.next(p, g, i);
        ++unit;
    }
}

}  // namespace bwd
}  // namespace kfa
