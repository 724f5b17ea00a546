// Query-gradient kernel of the backward pass on the tensor-memory pipeline: shared context and the
// loader / MMA-issuer roles.  The consumer role is in pipeline_backward_q_consumer.cuh.
//
// A CTA owns 128 query rows of one (batch, query head), keeps Q and dO resident and streams the
// 128-key tiles ("units") its rows can see.  Per unit the tensor core runs full 128 x 128 products,
// which execute at the math rate (a 64-column score product is limited by shared-memory reads):
//   S   = Q  x K^T            dP = dO x V^T            dQ += dS_low x K   (A operand from tensor memory)
// Tensor memory (512 columns): S_a | S_b | dP | dQ.  The score tile is double buffered; dS_low is packed
// into the (dead) score buffer of its unit, and the dP buffer is handed back as soon as the consumers hold
// its values, so the next dP product runs under the dS arithmetic and the S product of the unit after next
// under everything else.  K and V travel in separate rings: a V tile is dead after its dP product, a K tile
// only after the dQ product, so K gets three slots and V two (224 KB of shared memory with Q and dO).
// (Reference behaviour: src/kohakufa_cute/blackwell_pipeline.py:610-662, 1279-1306 of the
// reference project; arithmetic contract docs/precision.md:13-23.)
#pragma once
#include "pipeline_backward_common.cuh"

namespace kfa {
namespace bwd {
namespace q {

constexpr int kCols = kTile / kGroups;  // columns of a unit per consumer thread
constexpr int kMaxSlots = 4;

template <int D>
struct Cfg {
    static constexpr int kChunks = D / 64;
    static constexpr int kTileBytes = kTile * D * 2;
    static constexpr int kKeySlots = D == 128 ? 3 : 4;
    static constexpr int kValueSlots = D == 128 ? 2 : 4;
    static constexpr int kSmemBytes = (2 + kKeySlots + kValueSlots) * kTileBytes + 1024 + 512;
};

struct Shared {
    uint64_t owner_full;
    uint64_t k_full[kMaxSlots], k_empty[kMaxSlots];  // a K slot is released by both issuers (S and dQ products)
    uint64_t v_full[kMaxSlots], v_empty[kMaxSlots];
    uint64_t s_ready[2];   // score buffer x filled
    uint64_t s_free[2];    // the dQ product has read dS_low out of score buffer x
    uint64_t dp_ready;     // dP buffer filled
    uint64_t dp_free;      // every consumer holds its dP values
    uint64_t ds_done;      // every consumer stored its dS_low
    uint64_t final_done;
    uint64_t out_staged;   // every consumer has put its part of the gradient tile into shared memory
    uint32_t tmem_base;
    int abort_word;
};

constexpr uint32_t kColS = 0, kColDp = 256, kColGrad = 384;

template <int D>
__device__ __forceinline__ void loader_role(const Maps& maps, const AttnParams& p, const Work<false>& w, Shared& sh,
                                            uint8_t* s_owner, uint8_t* s_keys, uint8_t* s_values) {
    using C = Cfg<D>;
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    const int kvh = w.head / p.group;
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.g);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    mbar_expect_tx(&sh.owner_full, 2 * C::kTileBytes);
    for (int c = 0; c < C::kChunks; ++c) {
        tma_load_4d(s_owner + c * (kTile * 128), &maps.q, &sh.owner_full, c * 64, w.owner0, w.head, w.b);
        tma_load_4d(s_owner + C::kTileBytes + c * (kTile * 128), &maps.g, &sh.owner_full, c * 64, w.owner0, w.head,
                    w.b);
    }
    int unit = 0;
    bool ok = true;
    while (w.valid(g) && ok) {
        // K first while the rings fill (the S product needs it first); afterwards a V slot frees earlier
        // than a K slot, so V goes first and the loader never waits on K with a V copy still to issue
        for (int step = 0; step < 2 && ok; ++step) {
            const bool key = (step == 0) == (unit < C::kKeySlots);
            const int slots = key ? C::kKeySlots : C::kValueSlots;
            const int slot = unit % slots, round = unit / slots;
            uint64_t* full = key ? &sh.k_full[slot] : &sh.v_full[slot];
            if (round > 0)
                ok = mbar_wait(key ? &sh.k_empty[slot] : &sh.v_empty[slot], (round - 1) & 1, abort_word, 110);
            if (!ok) break;
            uint8_t* dst = (key ? s_keys : s_values) + slot * C::kTileBytes;
            mbar_expect_tx(full, C::kTileBytes);
            for (int c = 0; c < C::kChunks; ++c)
                tma_load_4d(dst + c * (kTile * 128), key ? &maps.k : &maps.v, full, c * 64, i * kTile, kvh, w.b);
        }
        w.next(p, g, i);
        ++unit;
    }
}

// Two threads issue the tensor-core work, each its own in-order chain:
//   chain 0:  S of every unit, into the two score buffers in turn
//   chain 1:  dP of the coming unit as soon as the consumers hold the current one, then dQ += dS_low x K
// s_free orders the two chains on a score buffer (chain 1 reads dS_low out of it, chain 0 refills it).
template <int D, bool BF16>
__device__ __forceinline__ void mma_role(const AttnParams& p, const Work<false>& w, Shared& sh, uint32_t tmem,
                                         uint8_t* s_owner, uint8_t* s_keys, uint8_t* s_values, int chain) {
    using C = Cfg<D>;
    volatile int* abort_word = &sh.abort_word;
    int g, i;
    w.begin(p, g, i);
    if (!w.valid(g)) return;
    // A negative scale takes maxima over -S: the forward saved statistics of -S, so negate operand A.
    const uint32_t idesc_s = umma_idesc(kTile, kTile, BF16 ? 1 : 0, false, false) |
                             (chain == 0 && p.scale < 0.f ? kUmmaNegateA : 0u);
    constexpr uint32_t idesc_g = umma_idesc(kTile, D, BF16 ? 1 : 0, false, true);
    // Descriptors are built once; per instruction only the start-address field advances.
    const uint64_t own_desc = umma_desc_sw128(smem_u32(s_owner) + chain * C::kTileBytes, 16, 1024);
    const uint64_t score_desc = umma_desc_sw128(smem_u32(chain == 0 ? s_keys : s_values), 16, 1024);  // K-major view
    const uint64_t grad_desc = umma_desc_sw128(smem_u32(s_keys), kTile * 128, 1024);                   // MN-major view

    auto issue_scores = [&](int slot, uint32_t col) {
        const uint32_t st = slot * C::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * (kTile * 128) + (kk % 4) * 32;
            umma_ss(col, umma_desc_advance(own_desc, off), umma_desc_advance(score_desc, st + off), idesc_s, kk > 0);
        }
    };
    // A = dS_low packed into tensor memory at a_col: consumer warpgroup g keeps its 64 columns as 32 packed
    // columns at the head of its own range [g * 64, g * 64 + 32)
    auto issue_grad = [&](int slot, uint32_t a_col, bool accumulate) {
        const uint32_t st = slot * C::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
            const uint32_t a_off = (kk / 4) * kCols + (kk % 4) * 8;
            umma_ts(tmem + kColGrad, a_col + a_off, umma_desc_advance(grad_desc, st + kk * 2048), idesc_g,
                    accumulate || kk > 0);
        }
    };

    bool ok = mbar_wait(&sh.owner_full, 0, abort_word, 120);
    if (!ok) return;
    PH_DECL;
    if (chain == 0) {
        int unit = 0;
        while (w.valid(g) && ok) {
            const int x = unit & 1, slot = unit % C::kKeySlots;
            PH(4);
            if (unit >= 2) ok = mbar_wait(&sh.s_free[x], ((unit >> 1) - 1) & 1, abort_word, 125);
            if (!ok) break;
            PH(0);
            ok = mbar_wait(&sh.k_full[slot], (unit / C::kKeySlots) & 1, abort_word, 121);
            if (!ok) break;
            PH(2);
            tc_fence_after();
            issue_scores(slot, tmem + kColS + x * 128);
            umma_commit(&sh.s_ready[x]);
            umma_commit(&sh.k_empty[slot]);
            PH(3);
            w.next(p, g, i);
            ++unit;
        }
    } else {
        ok = mbar_wait(&sh.v_full[0], 0, abort_word, 121);
        if (!ok) return;
        tc_fence_after();
        issue_scores(0, tmem + kColDp);
        umma_commit(&sh.dp_ready);
        umma_commit(&sh.v_empty[0]);
        int unit = 0;
        while (w.valid(g) && ok) {
            int gn = g, in = i;
            w.next(p, gn, in);
            const bool more = w.valid(gn);
            const int x = unit & 1, kslot = unit % C::kKeySlots, vslot = (unit + 1) % C::kValueSlots;
            PH(4);
            if (more) {
                ok = mbar_wait(&sh.dp_free, unit & 1, abort_word, 126);
                PH(5);
                if (ok) ok = mbar_wait(&sh.v_full[vslot], ((unit + 1) / C::kValueSlots) & 1, abort_word, 124);
                if (!ok) break;
                PH(2);
                tc_fence_after();
                issue_scores(vslot, tmem + kColDp);
                umma_commit(&sh.dp_ready);
                umma_commit(&sh.v_empty[vslot]);
                PH(3);
            }
            ok = mbar_wait(&sh.ds_done, unit & 1, abort_word, 123);
            // the K tile was waited for by the other issuer; this wait makes its arrival visible here too
            if (ok) ok = mbar_wait(&sh.k_full[kslot], (unit / C::kKeySlots) & 1, abort_word, 127);
            if (!ok) break;
            PH(0);
            tc_fence_after();
            issue_grad(kslot, tmem + kColS + x * 128, unit > 0);
            umma_commit(&sh.s_free[x]);
            umma_commit(&sh.k_empty[kslot]);
            PH(1);
            g = gn;
            i = in;
            ++unit;
        }
    }
    if (ok) umma_commit(&sh.final_done);
    PH_FLUSH(2 + chain);
}

}  // namespace q
}  // namespace bwd
}  // namespace kfa
