// Attention forward on the Blackwell tensor-memory pipeline (tcgen05 + TMEM + TMA),
// head dims that are multiples of 8 up to 128 (run as 64 or 128 channels: the tiled loads fill the channels
// beyond the head with zeros, which add nothing to either product, and the tiled store drops them again),
// FP16/BF16, causal and/or boolean masks, grouped-query heads.
//
// One CTA owns 256 query rows of one (batch, query head) as two 128-row tiles and walks
// the 128-key tiles they can see.  Warp roles (384 threads):
//   warps 0-3  softmax of query tile 0   (thread i <-> TMEM lane i <-> query row i)
//   warps 4-7  softmax of query tile 1
//   warp  8    issues every tcgen05.mma (one elected lane), owns the TMEM allocation
//   warp  9    TMA loader (one elected lane); warps 10-11 idle (they complete the warpgroup so
//              that registers can be moved from it to the softmax warpgroups)
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 columns each.  The 16-bit
// probabilities overwrite the first 64 columns of their score tile and feed the second
// product straight from tensor memory; they are handed over in two halves of 64 keys, so
// the first half of P*V runs while the second half of the exponentials is formed.  While
// one tile's softmax runs, the tensor core works on the other tile, and K/V tiles are
// shared by both.  Block-wise callers (one block of a longer key sequence per call) get
// the tile folded into a running FP32 state instead of a normalised output.
//
// Arithmetic (reference behaviour: src/kohakufa_cute/blackwell_pipeline.py:141-209,
// 423-439 and kernels.py:1286-1333 of the reference project): scores are used unscaled,
// the row maximum is subtracted before the multiplication by |scale|*log2e, the
// normaliser sums unrounded probabilities while the product uses probabilities rounded
// once to the input type, and the saved statistics are the exact unscaled row maximum
// and log2 of the normaliser relative to it.  The accumulator is re-based only when
// the running maximum has grown by more than 2^8 in probability terms; the statistics
// are corrected for the difference at the end, so they do not depend on that choice.
#include "kfa_common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

#include <atomic>
#include <type_traits>

namespace kfa {
namespace {


constexpr int kTileQ = 128;
constexpr int kTileK = 128;
constexpr int kThreads = 384;  // three warpgroups: softmax 0, softmax 1, (MMA, loader, 2 idle warps)
// The accumulator is re-based when the row maximum has grown by more than 2^kRebase in probability terms.  Until then
// probabilities are formed against the stale maximum and may reach 2^kRebase: 2^14 stays inside FP16, and BF16 has
// FP32's range (row sums stay below 2^32 * keys, far inside FP32).  Re-basing costs a round trip of the output
// accumulator through registers on the softmax's critical path, so it should be rare also for large logits.
template <bool BF16>
__host__ __device__ constexpr float rebase_limit() { return BF16 ? 32.0f : 14.0f; }
constexpr int kMaxKeyTiles = 4096;  // masked calls keep one state byte per key tile in shared memory

template <int D>
struct FwdCfg {
    static constexpr int kChunks = D / 64;                 // 64-channel TMA boxes per tile
    static constexpr int kTileBytes = kTileK * D * 2;      // one Q, K or V tile
    static constexpr int kStages = D == 128 ? 4 : 6;       // K/V ring slots
    static constexpr int kSmemBytes =
        2 * kTileBytes + kStages * kTileBytes + 1024 /*align*/ + 256 /*barriers*/ + kMaxKeyTiles;
};

struct FwdMaps {
    CUtensorMap q, k, v, o;
};

struct Shared {
    uint64_t q_full;
    uint64_t kv_full[6];
    uint64_t kv_empty[6];
    uint64_t s_ready[2];
    uint64_t p_half[2][2];  // [tile][half of the keys]: those probabilities of the tile are in tensor memory
    uint64_t o_staged[2];  // every softmax thread of the tile has put its output row into shared memory
    uint32_t tmem_base;
    int abort_word;
    uint8_t tile_state[kMaxKeyTiles];  // per key tile of this CTA: 0 hidden, 1 mixed, 2 visible (masked calls)
};

// Combined state of key tile j (128 keys) for the CTA's query rows [q0, q0 + 256), from the 64x64
// table entries: 0 hidden, 2 visible, 1 mixed.  Masks broadcast over queries have one row of entries.
__device__ __forceinline__ int key_tile_state(const AttnParams& p, int b, int h, int q0, int j) {
    if (!p.has_mask) return 2;
    const int nk64 = (p.Sk + 63) >> 6;
    const int32_t* base = p.blocks + (int64_t)b * p.bs[0] + (int64_t)h * p.bs[1];
    int r0 = 0, r1 = 0;
    if (p.bs[2] != 0) {
        r0 = q0 >> 6;
        r1 = (min(q0 + 2 * kTileQ, p.Sq) - 1) >> 6;
    }
    const int c1 = min(2 * j + 1, nk64 - 1);
    bool any = false, all = true;
    for (int r = r0; r <= r1; ++r)
        for (int c = 2 * j; c <= c1; ++c) {
            const int s = base[(int64_t)r * p.bs[2] + (int64_t)c * p.bs[3]];
            any = any || s != 0;
            all = all && s == 2;
        }
    return all ? 2 : (any ? 1 : 0);
}

// MASKED = false is the instantiation for calls without a mask (the flag is cleared at compile time).
template <int D, bool BF16, bool MASKED>
__global__ void __launch_bounds__(kThreads, 1) pipeline_forward(const __grid_constant__ FwdMaps maps, AttnParams p) {
    if (!MASKED) p.has_mask = 0;
    using Cfg = FwdCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                          // two query tiles
    uint8_t* sKV = smem + 2 * Cfg::kTileBytes;   // ring of K/V tiles
    Shared& sh = *reinterpret_cast<Shared*>(sKV + Cfg::kStages * Cfg::kTileBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = (p.Sq + 2 * kTileQ - 1) / (2 * kTileQ);
    // Heavy (late) causal blocks first.  Large grids go head by head (a head's CTAs share K/V in L2 and the
    // last wave is made of light blocks); grids of a few waves go block-row by block-row over all heads, so
    // that no head's heavy blocks start in the last wave.
    const int64_t nbh = (int64_t)p.B * p.Hq;
    // (row by row also when all K/V of the call fit in half of L2: measured 4.6 % faster on 2048 CTAs)
    const bool by_row = (int64_t)gridDim.x < KFA_ROW_MAJOR_LIMIT ||
                        (int64_t)p.B * p.Hkv * p.Sk * D * 4 <= (int64_t(64) << 20);
    const int qblk = nblk - 1 - (int)(by_row ? blockIdx.x / nbh : blockIdx.x % nblk);
    const int64_t bh = by_row ? blockIdx.x % nbh : blockIdx.x / nblk;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int kvh = h / p.group;
    const int q0 = qblk * 2 * kTileQ;

    // key tiles each query tile may see
    int n_t[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int row_lo = q0 + t * kTileQ;
        if (row_lo >= p.Sq) {
            n_t[t] = 0;
        } else {
            const int row_hi = min(p.Sq, row_lo + kTileQ);
            const int k_hi = p.causal ? min(p.Sk, row_hi) : p.Sk;
            n_t[t] = (k_hi + kTileK - 1) / kTileK;
        }
    }
    const int n_max = max(n_t[0], n_t[1]);

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.q_full, 1);
        for (int i = 0; i < Cfg::kStages; ++i) {
            mbar_init(&sh.kv_full[i], 1);
            mbar_init(&sh.kv_empty[i], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&sh.s_ready[t], 1);
            mbar_init(&sh.p_half[t][0], kTileQ);
            mbar_init(&sh.p_half[t][1], kTileQ);
            mbar_init(&sh.o_staged[t], kTileQ);
        }
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(&sh.tmem_base, 512);
        tmem_relinquish();
    }
    if (p.has_mask)
        for (int j = threadIdx.x; j < n_max; j += kThreads) sh.tile_state[j] = (uint8_t)key_tile_state(p, b, h, q0, j);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    const uint8_t* states = sh.tile_state;
    const bool masked_call = p.has_mask != 0;
    auto state_of = [&](int j) -> int { return masked_call ? states[j] : 2; };
    volatile int* abort_word = &sh.abort_word;

    const bool dead = sh.abort_word != 0;  // set before the barrier above: skip straight to the tear-down
    if (dead) {
    } else if (warp >= 8) {
      reg_dealloc<88>();
      if (warp == 9) {
        // ------------------------------------------------------------ loader
        if (elect_one()) {
            tma_prefetch_desc(&maps.q);
            tma_prefetch_desc(&maps.k);
            tma_prefetch_desc(&maps.v);
            const int active = (n_t[0] > 0 ? 1 : 0) + (n_t[1] > 0 ? 1 : 0);
            mbar_expect_tx(&sh.q_full, active * Cfg::kTileBytes);
            for (int t = 0; t < 2; ++t)
                if (n_t[t] > 0)
                    for (int c = 0; c < Cfg::kChunks; ++c)
                        tma_load_4d(sQ + t * Cfg::kTileBytes + c * (kTileQ * 128), &maps.q, &sh.q_full, c * 64,
                                    q0 + t * kTileQ, h, b);
            int slot_use = 0;
            bool ok = true;
            for (int j = 0; j < n_max && ok; ++j) {
                if (state_of(j) == 0) continue;
                for (int which = 0; which < 2 && ok; ++which) {  // K tile, then V tile
                    const int slot = slot_use % Cfg::kStages, round = slot_use / Cfg::kStages;
                    if (round > 0) ok = mbar_wait(&sh.kv_empty[slot], (round - 1) & 1, abort_word, 10);
                    if (!ok) break;
                    mbar_expect_tx(&sh.kv_full[slot], Cfg::kTileBytes);
                    const CUtensorMap* map = which == 0 ? &maps.k : &maps.v;
                    for (int c = 0; c < Cfg::kChunks; ++c)
                        tma_load_4d(sKV + slot * Cfg::kTileBytes + c * (kTileK * 128), map, &sh.kv_full[slot], c * 64,
                                    j * kTileK, kvh, b);
                    ++slot_use;
                }
            }
        }
      } else if (warp == 8) {
        // ------------------------------------------------------- MMA issuer
        if (elect_one()) {
            // a negative scale takes the maximum over -S: negate the A operand of the score product
            const uint32_t idesc_s =
                umma_idesc(kTileQ, kTileK, BF16 ? 1 : 0, false, false) | (p.scale < 0.f ? kUmmaNegateA : 0u);
            constexpr uint32_t idesc_o = umma_idesc(kTileQ, D, BF16 ? 1 : 0, false, true);
            const uint32_t q_addr = smem_u32(sQ), kv_addr = smem_u32(sKV);
            // Descriptors are built once; per instruction only the start-address field advances.
            const uint64_t q_desc = umma_desc_sw128(q_addr, 16, 1024), k_desc = umma_desc_sw128(kv_addr, 16, 1024);
            const uint64_t v_desc = umma_desc_sw128(kv_addr, kTileK * 128, 1024);
            auto issue_s = [&](int t, int slot) {
                const uint32_t a0 = t * Cfg::kTileBytes, b0 = slot * Cfg::kTileBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * (kTileQ * 128) + (kk % 4) * 32;
                    umma_ss(tmem + t * 128, umma_desc_advance(q_desc, a0 + off), umma_desc_advance(k_desc, b0 + off),
                            idesc_s, kk > 0);
                }
            };
            // P*V over one half of the tile's keys (the half whose probabilities have been handed over: the first
            // half of the product runs while the softmax still forms the second half of the probabilities)
            auto issue_o = [&](int t, int slot, int half, bool accumulate) {
                const uint32_t b0 = slot * Cfg::kTileBytes;
#pragma unroll
                for (int kk = half * (kTileK / 32); kk < (half + 1) * (kTileK / 32); ++kk)
                    umma_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, umma_desc_advance(v_desc, b0 + kk * 2048),
                            idesc_o, accumulate || kk > 0);
            };
            bool ok = mbar_wait(&sh.q_full, 0, abort_word, 20);
            int slot_use = 0, iter[2] = {0, 0};
            PH_DECL;
            // first visible key tile
            int j = 0;
            while (j < n_max && state_of(j) == 0) ++j;
            if (ok && j < n_max) {
                const int slot = slot_use % Cfg::kStages;
                ok = mbar_wait(&sh.kv_full[slot], (slot_use / Cfg::kStages) & 1, abort_word, 21);
                if (ok) {
                    tc_fence_after();
                    for (int t = 0; t < 2; ++t)
                        if (j < n_t[t]) {
                            issue_s(t, slot);
                            umma_commit(&sh.s_ready[t]);
                        }
                    umma_commit(&sh.kv_empty[slot]);
                    ++slot_use;
                }
            }
            while (ok && j < n_max) {
                int jn = j + 1;
                while (jn < n_max && state_of(jn) == 0) ++jn;
                const int v_slot = slot_use % Cfg::kStages, v_par = (slot_use / Cfg::kStages) & 1;
                ++slot_use;
                int k_slot = -1, k_par = 0;
                if (jn < n_max) {
                    k_slot = slot_use % Cfg::kStages;
                    k_par = (slot_use / Cfg::kStages) & 1;
                    ++slot_use;
                }
                PH(5);
                ok = mbar_wait(&sh.kv_full[v_slot], v_par, abort_word, 22);
                PH(0);
                bool k_waited = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (j >= n_t[t]) continue;
                    ok = mbar_wait(&sh.p_half[t][0], iter[t] & 1, abort_word, 23 + t);
                    if (!ok) break;
                    PH(1);
                    tc_fence_after();
                    issue_o(t, v_slot, 0, iter[t] > 0);
                    PH(2);
                    ok = mbar_wait(&sh.p_half[t][1], iter[t] & 1, abort_word, 26 + t);
                    if (!ok) break;
                    PH(1);
                    tc_fence_after();
                    issue_o(t, v_slot, 1, true);
                    PH(2);
                    if (jn < n_t[t]) {
                        if (!k_waited) {
                            ok = mbar_wait(&sh.kv_full[k_slot], k_par, abort_word, 25);
                            if (!ok) break;
                            tc_fence_after();
                            k_waited = true;
                        }
                        PH(3);
                        issue_s(t, k_slot);
                    }
                    umma_commit(&sh.s_ready[t]);
                    PH(4);
                    ++iter[t];
                }
                if (!ok) break;
                umma_commit(&sh.kv_empty[v_slot]);
                if (k_slot >= 0) umma_commit(&sh.kv_empty[k_slot]);
                j = jn;
            }
            PH_FLUSH(2);
        }
      }
    } else {
        reg_alloc<208>();
        // ---------------------------------------------------------- softmax
        const int t = warp >> 2;
        const int row_in_tile = (warp & 3) * 32 + lane;
        const int row = q0 + t * kTileQ + row_in_tile;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + t * 128, o_addr = lane_base + 256 + t * 128;
        const float c2 = fabsf(p.scale) * kLog2e;
        const uint64_t c2_pair = f2_pack(c2, c2);
        // this row's line of the mask (every row shares one line when the mask is broadcast over queries)
        const uint8_t* kmask = p.has_mask ? p.mask + (int64_t)b * p.ms[0] + (int64_t)h * p.ms[1] +
                                                (int64_t)min(row, p.Sq - 1) * p.ms[2]
                                          : nullptr;
        float m_used = -INFINITY, m_true = -INFINITY, l = 0.f;
        int iter = 0;
        bool ok = true;
        PH_DECL;
        for (int j = 0; j < n_t[t] && ok; ++j) {
            const int state = state_of(j);
            if (state == 0) continue;
            PH(5);
            ok = mbar_wait(&sh.s_ready[t], iter & 1, abort_word, 30 + t);
            if (!ok) break;
            PH(0);
            tc_fence_after();
            // scores arrive already multiplied by sign(scale) (negated A operand for negative scales)
            float s[kTileK];
#pragma unroll
            for (int c = 0; c < kTileK; c += 32) {
                uint32_t r[32];
                tmem_ld32(s_addr + c, r);
#pragma unroll
                for (int i = 0; i < 32; ++i) s[c + i] = __uint_as_float(r[i]);
            }
            tmem_wait_ld();
            tmem_loaded(s);
            PH(1);
            const int key0 = j * kTileK;
            // leading columns of this tile that pass the sequence-end and causal bounds for this row
            int lim = p.Sk - key0;
            if (p.causal) lim = min(lim, row - key0 + 1);
            if (lim < kTileK) {
#pragma unroll
                for (int c = 0; c < kTileK; ++c) s[c] = c < lim ? s[c] : -INFINITY;
            }
            if (state == 1) {
#pragma unroll
                for (int c = 0; c < kTileK; ++c) {
                    const int key = min(key0 + c, p.Sk - 1);
                    s[c] = kmask[(int64_t)key * p.ms[3]] != 0 ? s[c] : -INFINITY;
                }
            }
            // four independent chains of three-input maxima
            float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
            float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
            for (int c = 12; c < kTileK - 4; c += 8) {
                mx0 = max3(mx0, s[c], s[c + 1]);
                mx1 = max3(mx1, s[c + 2], s[c + 3]);
                mx2 = max3(mx2, s[c + 4], s[c + 5]);
                mx3 = max3(mx3, s[c + 6], s[c + 7]);
            }
            mx0 = max3(mx0, s[kTileK - 4], s[kTileK - 3]);
            mx1 = max3(mx1, s[kTileK - 2], s[kTileK - 1]);
            const float mx = fmaxf(max3(mx0, mx1, mx2), mx3);
            m_true = fmaxf(m_true, mx);
            const bool rebase = mx > m_used && (m_used == -INFINITY || (mx - m_used) * c2 > rebase_limit<BF16>());
            float alpha = 1.f;
            if (rebase) {
                alpha = (m_used == -INFINITY) ? 0.f : ex2((m_used - mx) * c2);
                l *= alpha;
                m_used = mx;
            }
            if (iter > 0 && __any_sync(0xffffffffu, rebase)) {
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(o_addr + c, r);
                }
            }
            PH(2);
            const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
            const uint64_t m_pair = f2_pack(m_safe, m_safe);
            uint64_t sum_a = f2_pack(0.f, 0.f), sum_b = sum_a;
#pragma unroll
            for (int c = 0; c < kTileK; c += 32) {
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    // (s - m) first, then the multiplication by |scale|*log2e, two lanes per instruction
                    float pa, pb, pc, pd;
                    f2_unpack(f2_mul(f2_sub(f2_pack(s[c + 2 * i], s[c + 2 * i + 1]), m_pair), c2_pair), pa, pb);
                    f2_unpack(f2_mul(f2_sub(f2_pack(s[c + 2 * i + 2], s[c + 2 * i + 3]), m_pair), c2_pair), pc, pd);
                    pa = ex2(pa);
                    pb = ex2(pb);
                    pc = ex2(pc);
                    pd = ex2(pd);
                    sum_a = f2_add(sum_a, f2_pack(pa, pb));
                    sum_b = f2_add(sum_b, f2_pack(pc, pd));
                    w[i] = pack2<BF16>(pa, pb);
                    w[i + 1] = pack2<BF16>(pc, pd);
                }
                tmem_st16(s_addr + c / 2, w);
                if (c == kTileK / 2 - 32) {  // the first half of the keys is done: hand it over
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&sh.p_half[t][0]);
                }
            }
            {
                float x0, x1, x2, x3;
                f2_unpack(sum_a, x0, x1);
                f2_unpack(sum_b, x2, x3);
                l += (x0 + x1) + (x2 + x3);
            }
            PH(3);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sh.p_half[t][1]);
            PH(4);
            ++iter;
        }
        if ((threadIdx.x & 127) == 0) PH_FLUSH(t);
        // epilogue: wait for the last product, normalise, store
        if (ok && iter == 0 && row < p.Sq && n_t[t] > 0 && !p.running) {
            // every key tile of this row is hidden: zero output, empty statistics
            using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
            T* orow = reinterpret_cast<T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] + (int64_t)row * p.os[2];
            const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + row;
            for (int d = 0; d < p.D; d += 8) *reinterpret_cast<uint4*>(orow + d) = make_uint4(0, 0, 0, 0);
            if (p.maximum) {  // no statistics are kept for a forward pass without gradients
                p.maximum[si] = -INFINITY;
                p.logsum[si] = 0.f;
            }
        }
        if (iter > 0 && p.running) {
            // Block of a longer key sequence: fold (accumulator, maximum, sum) into the caller's running FP32 state
            // with the (maximum, sum) merge of the reference's split forward (split_forward.py:219-245); nothing is
            // rounded to the 16-bit type and nothing is divided here.
            if (ok) ok = mbar_wait(&sh.s_ready[t], iter & 1, abort_word, 32 + t);
            if (ok) {
                // (every lane runs the tensor-memory loads, which are warp-wide; rows beyond the sequence end
                // only skip the global accesses)
                tc_fence_after();
                const bool live = row < p.Sq;
                const int64_t si = (int64_t)b * p.ss[0] + (int64_t)h * p.ss[1] + (live ? row : 0);
                const float m_old = live ? p.maximum[si] : -INFINITY, l_old = live ? p.run_sum[si] : 0.f;
                const float m_new = fmaxf(m_old, m_true);
                const float w_old = m_old == -INFINITY ? 0.f : ex2((m_old - m_new) * c2);
                const float w_blk = m_used == -INFINITY ? 0.f : ex2((m_used - m_new) * c2);
                float* arow = reinterpret_cast<float*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] +
                              (int64_t)row * p.os[2];
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        if (live && c + i < p.D) {
                            float4 a = *reinterpret_cast<float4*>(arow + c + i);
                            a.x = a.x * w_old + __uint_as_float(r[i]) * w_blk;
                            a.y = a.y * w_old + __uint_as_float(r[i + 1]) * w_blk;
                            a.z = a.z * w_old + __uint_as_float(r[i + 2]) * w_blk;
                            a.w = a.w * w_old + __uint_as_float(r[i + 3]) * w_blk;
                            *reinterpret_cast<float4*>(arow + c + i) = a;
                        }
                    }
                }
                if (live) {
                    p.maximum[si] = m_new;
                    p.run_sum[si] = l_old * w_old + l * w_blk;
                }
            }
        } else if (iter > 0) {
            if (ok) ok = mbar_wait(&sh.s_ready[t], iter & 1, abort_word, 32 + t);
            if (ok) {
                tc_fence_after();
                const float den = l > 0.f ? l : 1.f;
                const float inv_den = 1.f / den;  // one division per row; the elements are multiplied
                // The normalised tile goes through this tile's (now dead) Q buffer in the swizzled box layout and
                // leaves as tiled stores: whole 128-byte lines instead of 16 bytes per row and instruction.
                uint8_t* stage = sQ + t * Cfg::kTileBytes;
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack2<BF16>(__uint_as_float(r[i]) * inv_den, __uint_as_float(r[i + 1]) * inv_den);
                        w.y = pack2<BF16>(__uint_as_float(r[i + 2]) * inv_den, __uint_as_float(r[i + 3]) * inv_den);
                        w.z = pack2<BF16>(__uint_as_float(r[i + 4]) * inv_den, __uint_as_float(r[i + 5]) * inv_den);
                        w.w = pack2<BF16>(__uint_as_float(r[i + 6]) * inv_den, __uint_as_float(r[i + 7]) * inv_den);
                        const int chunk = (c + i) >> 3;  // 16-byte chunk of the row: box chunk / 8, position chunk % 8
                        *reinterpret_cast<uint4*>(stage + (chunk >> 3) * (kTileQ * 128) + sw128_chunk(row_in_tile, chunk & 7)) = w;
                    }
                }
                fence_async_smem();
                mbar_arrive(&sh.o_staged[t]);
                if (row_in_tile == 0 && mbar_wait(&sh.o_staged[t], 0, abort_word, 34 + t)) {
                    for (int c = 0; c < Cfg::kChunks; ++c)
                        tma_store_4d(&maps.o, stage + c * (kTileQ * 128), c * 64, q0 + t * kTileQ, h, b);
                    tma_store_commit();
                    tma_store_wait_read();
                }
                if (row < p.Sq && p.maximum) {
                    const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + row;
                    p.maximum[si] = m_true;
                    p.logsum[si] = l > 0.f ? log2f(l) + (m_used - m_true) * c2 : 0.f;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 1000 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == 8) tmem_dealloc(tmem, 512);
}

std::atomic<int> g_configured{0};

template <int D, bool BF16>
cudaError_t launch_t(const AttnParams& p, cudaStream_t st) {
    using Cfg = FwdCfg<D>;
    // The shared-memory opt-in is per device; it is cheap, so it is simply repeated per call.
    auto kernel = p.has_mask ? pipeline_forward<D, BF16, true> : pipeline_forward<D, BF16, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    constexpr int variant = (D == 128 ? 0 : 2) + (BF16 ? 0 : 1);  // D = channels the kernel runs with (p.D rounded up)
    const int bit = 1 << variant;
    if (!(g_configured.load() & bit)) g_configured |= bit;
    FwdMaps maps;
    const CUtensorMapDataType dt = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!encode_bhsd_map(&maps.q, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTileQ)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.k, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTileK)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.v, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTileK)) return cudaErrorInvalidValue;
    if (p.running)
        maps.o = maps.q;  // not used: the running state is written with plain stores
    else if (!encode_bhsd_map(&maps.o, p.out, dt, p.D, p.Sq, p.Hq, p.B, p.os, 64, kTileQ))
        return cudaErrorInvalidValue;
    const int64_t grid = (int64_t)((p.Sq + 2 * kTileQ - 1) / (2 * kTileQ)) * p.B * p.Hq;
    kernel<<<(unsigned)grid, kThreads, Cfg::kSmemBytes, st>>>(maps, p);
    return cudaGetLastError();
}

}  // namespace

bool pipeline_forward_supported(const AttnParams& p, bool bf16) {
    (void)bf16;
    if (p.D < 8 || p.D > 128 || p.D % 8 != 0) return false;  // rows of whole 16-byte pieces
    if (p.nd != 0) return false;
    if (p.scale == 0.f || p.Sk < 2) return false;  // hidden scores are -inf; -inf * 0 is not representable in the fast path
    if (p.has_mask && (p.Sk + kTileK - 1) / kTileK > kMaxKeyTiles) return false;
    if (!tma_compatible(p.q, p.qs, p.B, p.Hq, p.Sq) || !tma_compatible(p.k, p.ks, p.B, p.Hkv, p.Sk) ||
        !tma_compatible(p.v, p.vs, p.B, p.Hkv, p.Sk))
        return false;
    if (p.running) {  // FP32 rows read and written as 16-byte vectors
        if (p.os[3] != 1 || reinterpret_cast<uintptr_t>(p.out) % 16 != 0 || p.os[0] % 4 || p.os[1] % 4 || p.os[2] % 4)
            return false;
    } else if (!tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq)) {
        return false;  // 16-byte vector stores per row
    }
    return true;
}

cudaError_t launch_pipeline_forward(const AttnParams& p, bool bf16, cudaStream_t st) {
    if (p.D > 64) return bf16 ? launch_t<128, true>(p, st) : launch_t<128, false>(p, st);
    return bf16 ? launch_t<64, true>(p, st) : launch_t<64, false>(p, st);
}

KFA_PHASE_EXPORT(kfa_debug_phases_fwd)

int pipeline_forward_variants() { return __builtin_popcount(g_configured.load()); }
void pipeline_forward_forget() { g_configured = 0; }

}  // namespace kfa
