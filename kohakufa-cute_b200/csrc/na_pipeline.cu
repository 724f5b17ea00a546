// Neighbourhood attention (head dim 64, 2-D and 3-D grids) on the Blackwell tensor-memory pipeline.
//
// A CTA owns 128 consecutive tokens of one (batch, head) and walks only the dense tiles of partner
// tokens that its rows can see (na_tiles.cuh); inside a tile every row applies its own bit mask, so
// exactly the window contributes.  The kernels are small enough (<= 256 tensor-memory columns,
// < 100 KB shared memory, 192 threads) for two CTAs per SM, which overlaps one CTA's softmax with
// the other's tensor-core work.
//
// Arithmetic (reference behaviour: docs/precision.md:46-80 and
// src/kohakufa_cute/neighborhood_kernels.py:193-212, 348-365 of the reference project):
//   forward   shifted-score online softmax as for ordinary attention; on 3-D grids the rounding
//             residual of each weight enters a second product term (hi = rd(p), lo = rd(p - hi)).
//   backward  P32 = ex2((s' - m)|scale|log2e - logsum) stays FP32 when forming dS.
//     query   dS_q = rd(P32 (dP - delta));
//             dQ = (sum dS_q K - (sum dS_q / sum rd(P32)) sum rd(P32) K) * scale;
//             publishes t = sum P32 (dP - delta) / sum P32.
//     key     dS_k = rd(P32 ((dP - delta) - t)); dK = (sum dS_k Q) * scale;  dV = sum rd(P32) dO.
#include "kfa_common.cuh"
#include "launchers.h"
#include "na_tiles.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

#include <type_traits>

namespace kfa {
namespace {

using namespace na;

constexpr int kTile = 128;
constexpr int kChunkBytes = kTile * 128;  // 128 rows x 64 channels, 16-bit
constexpr int kRing = 5;
// The accumulator is re-based when the row maximum has grown by more than this power of two in probability terms:
// probabilities against the stale maximum stay inside FP16 (2^14) or BF16's FP32 range (2^32), and the round trip of
// the accumulator through registers stays rare also for large logits.
template <bool BF16>
__host__ __device__ constexpr float rebase_limit() { return BF16 ? 32.0f : 14.0f; }

struct NaMaps {
    CUtensorMap q, k, v, g;
};

// ------------------------------------------------------------------------------------------ forward
struct FwdShared {
    uint64_t q_full;
    uint64_t full[kRing];
    uint64_t empty[kRing];
    uint64_t s_ready;
    uint64_t p_ready;
    uint32_t tmem_base;
    int abort_word;
    uint32_t bitmap[kMapWords];
};

// 192 threads: warps 0-3 softmax (thread <-> query row), warp 4 MMA issuer, warp 5 loader.
// Tensor memory (256 columns): S at 0 (rd(p) overwrites its first 64 columns), O at 128, the
// residual weights at 192.
template <bool BF16, bool TWO>
__global__ void __launch_bounds__(192, 2) na_tc_forward(const __grid_constant__ NaMaps maps, AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sRing = smem + kChunkBytes;
    FwdShared& sh = *reinterpret_cast<FwdShared*>(sRing + kRing * kChunkBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = (p.Sq + kTile - 1) / kTile;
    const int qblk = (int)(blockIdx.x % nblk);
    const int64_t bh = blockIdx.x / nblk;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int q0 = qblk * kTile;
    PH_DECL;

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.q_full, 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.empty[i], 1);
        }
        mbar_init(&sh.s_ready, 1);
        mbar_init(&sh.p_ready, kTile);
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < kMapWords; i += blockDim.x) sh.bitmap[i] = 0;
    if (warp == 4) {
        tmem_alloc(&sh.tmem_base, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const int row = q0 + warp * 32 + lane;
    const bool row_ok = warp < 4 && row < p.Sq;
    Box box = {0, -1, 0, -1, 0, -1};
    if (row_ok) box = query_box(p, row);
    if (warp < 4) mark_tiles_warp(p, box, row_ok, kTile, sh.bitmap);
    __syncthreads();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_word = &sh.abort_word;

    if (sh.abort_word != 0) {
        // an earlier CTA gave up: skip straight to the tear-down
    } else if (warp == 5) {
        if (elect_one()) {
            tma_prefetch_desc(&maps.q);
            tma_prefetch_desc(&maps.k);
            tma_prefetch_desc(&maps.v);
            mbar_expect_tx(&sh.q_full, kChunkBytes);
            tma_load_4d(sQ, &maps.q, &sh.q_full, 0, q0, h, b);
            int pos = 0;
            bool ok = true;
            for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1))
                for (int which = 0; which < 2 && ok; ++which, ++pos) {
                    const int slot = pos % kRing, round = pos / kRing;
                    if (round > 0) ok = mbar_wait(&sh.empty[slot], (round - 1) & 1, abort_word, 10);
                    if (!ok) break;
                    mbar_expect_tx(&sh.full[slot], kChunkBytes);
                    tma_load_4d(sRing + slot * kChunkBytes, which == 0 ? &maps.k : &maps.v, &sh.full[slot], 0,
                                j * kTile, h, b);
                }
        }
    } else if (warp == 4) {
        if (elect_one()) {
            const uint32_t idesc_s =
                umma_idesc(kTile, kTile, BF16 ? 1 : 0, false, false) | (p.scale < 0.f ? kUmmaNegateA : 0u);
            constexpr uint32_t idesc_o = umma_idesc(kTile, 64, BF16 ? 1 : 0, false, true);
            const uint64_t q_desc = umma_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t k_desc = umma_desc_sw128(smem_u32(sRing), 16, 1024);
            const uint64_t v_desc = umma_desc_sw128(smem_u32(sRing), kChunkBytes, 1024);
            bool ok = mbar_wait(&sh.q_full, 0, abort_word, 20);
            int pos = 0, iter = 0;
            for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1)) {
                const int ks = pos % kRing;
                ok = mbar_wait(&sh.full[ks], (pos / kRing) & 1, abort_word, 21);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_ss(tmem, umma_desc_advance(q_desc, kk * 32), umma_desc_advance(k_desc, ks * kChunkBytes + kk * 32),
                            idesc_s, kk > 0);
                umma_commit(&sh.empty[ks]);
                umma_commit(&sh.s_ready);
                ++pos;
                const int vs = pos % kRing;
                ok = mbar_wait(&sh.full[vs], (pos / kRing) & 1, abort_word, 22);
                if (ok) ok = mbar_wait(&sh.p_ready, iter & 1, abort_word, 23);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)
                    umma_ts(tmem + 128, tmem + kk * 8, umma_desc_advance(v_desc, vs * kChunkBytes + kk * 2048), idesc_o,
                            iter > 0 || kk > 0);
                if (TWO) {
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        umma_ts(tmem + 128, tmem + 192 + kk * 8, umma_desc_advance(v_desc, vs * kChunkBytes + kk * 2048),
                                idesc_o, 1);
                }
                umma_commit(&sh.empty[vs]);
                ++pos;
                ++iter;
            }
            if (ok) umma_commit(&sh.s_ready);
        }
    } else {
        using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        const uint32_t s_addr = lane_base, o_addr = lane_base + 128, lo_addr = lane_base + 192;
        const float c2 = fabsf(p.scale) * kLog2e;
        float m_used = -INFINITY, m_true = -INFINITY, l = 0.f;
        int iter = 0;
        bool ok = true;
        PH(6);
        BoxCursor cursor = box_cursor(p, box);
        for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1)) {
            uint32_t vis[4] = {0, 0, 0, 0};
            if (row_ok) box_mask_walk<4>(p, box, cursor, j * kTile, vis);
            PH(5);
            ok = mbar_wait(&sh.s_ready, iter & 1, abort_word, 30);
            if (!ok) break;
            PH(0);
            tc_fence_after();
            // pass 1: hide what the row does not see (written back as -inf), maximum of the rest
            // 32-column chunks that no row of this warp can see are skipped (their weights are zero)
            uint32_t live = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) live |= (__any_sync(0xffffffffu, vis[c] != 0) ? 1u : 0u) << c;
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (!((live >> c) & 1u)) continue;
                uint32_t r[32];
                tmem_ld32(s_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    r[i] = hide(r[i], vis[c], i);
                    r[i + 1] = hide(r[i + 1], vis[c], i + 1);
                    mx0 = fmaxf(mx0, __uint_as_float(r[i]));
                    mx1 = fmaxf(mx1, __uint_as_float(r[i + 1]));
                }
                tmem_st32(s_addr + c * 32, r);
            }
            const float mx = fmaxf(mx0, mx1);
            tmem_wait_st();
            PH(1);
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
                for (int c = 0; c < 64; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(o_addr + c, r);
                }
            }
            PH(2);
            // pass 2: weights (hidden scores give exact zeros), their rounding and its residual, the normaliser
            const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
            const uint64_t m_pair = f2_pack(m_safe, m_safe), c2_pair = f2_pack(c2, c2);
            uint64_t sum = f2_pack(0.f, 0.f);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32], hi[16], lo[16];
                if (!((live >> c) & 1u)) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) hi[i] = 0;
                    tmem_st16(s_addr + c * 16, hi);
                    if (TWO) tmem_st16(lo_addr + c * 16, hi);
                    continue;
                }
                tmem_ld32(s_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float pa, pb;
                    f2_unpack(f2_mul(f2_sub(f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), m_pair), c2_pair),
                              pa, pb);
                    pa = ex2(pa);
                    pb = ex2(pb);
                    const uint64_t pp = f2_pack(pa, pb);
                    sum = f2_add(sum, pp);
                    const uint32_t w = pack2<BF16>(pa, pb);
                    hi[i / 2] = w;
                    if (TWO) {
                        const float2 back = unpack2<BF16>(w);
                        float ra, rb;
                        f2_unpack(f2_sub(pp, f2_pack(back.x, back.y)), ra, rb);
                        lo[i / 2] = pack2<BF16>(ra, rb);
                    }
                }
                tmem_st16(s_addr + c * 16, hi);
                if (TWO) tmem_st16(lo_addr + c * 16, lo);
            }
            float sum0, sum1;
            f2_unpack(sum, sum0, sum1);
            l += sum0 + sum1;
            PH(3);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sh.p_ready);
            PH(4);
            ++iter;
        }
        if (iter > 0 && ok) ok = mbar_wait(&sh.s_ready, iter & 1, abort_word, 31);
        PH(0);
        if (ok) {
            // tensor-memory loads are warp-collective: every lane takes part, only the stores are per row
            T* orow = reinterpret_cast<T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] +
                      (int64_t)(row_ok ? row : 0) * p.os[2];
            const float den = l > 0.f ? l : 1.f;
            const float inv_den = 1.f / den;  // one division per row; the elements are multiplied
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 64; c += 32) {
                uint32_t r[32];
                if (iter > 0) {
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0;
                }
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack2<BF16>(__uint_as_float(r[i]) * inv_den, __uint_as_float(r[i + 1]) * inv_den);
                        w.y = pack2<BF16>(__uint_as_float(r[i + 2]) * inv_den, __uint_as_float(r[i + 3]) * inv_den);
                        w.z = pack2<BF16>(__uint_as_float(r[i + 4]) * inv_den, __uint_as_float(r[i + 5]) * inv_den);
                        w.w = pack2<BF16>(__uint_as_float(r[i + 6]) * inv_den, __uint_as_float(r[i + 7]) * inv_den);
                        *reinterpret_cast<uint4*>(orow + c + i) = w;
                    }
                }
            }
            if (row_ok) {
                const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + row;
                p.maximum[si] = m_true;
                p.logsum[si] = l > 0.f ? log2f(l) + (m_used - m_true) * c2 : 0.f;
            }
        }
        PH(7);
        if (threadIdx.x == 0) PH_FLUSH(0);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 4000 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == 4) tmem_dealloc(tmem, 256);
}

// ----------------------------------------------------------------------------------------- backward
constexpr int kSub = 64;                      // partner tokens per streamed tile
constexpr int kSubBytes = kSub * 128;         // 64 rows x 64 channels
constexpr int kStages = 4;                    // ring stages, each holds both streamed operands

struct BwdShared {
    uint64_t own_full;
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t sdp_ready;
    uint64_t ops_ready;
    uint64_t done;
    uint32_t tmem_base;
    int abort_word;
    uint32_t bitmap[kMapWords];
    alignas(16) float stats[2][4][kSub];  // per streamed query: maximum, logsum, delta + t (key owners only; the fourth row is unused)
};

struct BwdMaps {
    CUtensorMap own0, own1, st0, st1;
};

// KV = false: the CTA owns 128 queries (own0 = Q, own1 = dO) and streams (K, V) tiles of 64 keys.
// KV = true:  the CTA owns 128 keys (own0 = K, own1 = V) and streams (Q, dO) tiles of 64 queries.
// Per streamed tile the tensor core forms S and dP (owner rows x 64), the consumer warps turn them
// into two 16-bit operands in place, and two accumulators collect
//   KV = false:  acc0 += dS_q K,       acc1 += rd(P32) K
//   KV = true:   acc0 += rd(P32)^T dO,  acc1 += dS_k^T Q
// Tensor memory (256 columns): S at 0, dP at 64, acc0 at 128, acc1 at 192.
template <bool KV, bool BF16>
__global__ void __launch_bounds__(192, 2) na_tc_backward(const __grid_constant__ BwdMaps maps, AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sOwn = smem;                         // two owner operands, 16 KB each
    uint8_t* sRing = smem + 2 * kChunkBytes;      // stages of (streamed 0, streamed 1), 8 KB each
    BwdShared& sh = *reinterpret_cast<BwdShared*>(sRing + kStages * 2 * kSubBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int owner_len = KV ? p.Sk : p.Sq;
    const int nblk = (owner_len + kTile - 1) / kTile;
    const int blk = (int)(blockIdx.x % nblk);
    const int64_t bh = blockIdx.x / nblk;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int owner0 = blk * kTile;

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.own_full, 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.empty[i], 1);
        }
        mbar_init(&sh.sdp_ready, 1);
        mbar_init(&sh.ops_ready, kTile);
        mbar_init(&sh.done, 1);
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < kMapWords; i += blockDim.x) sh.bitmap[i] = 0;
    if (warp == 4) {
        tmem_alloc(&sh.tmem_base, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const int row = owner0 + warp * 32 + lane;
    const bool row_ok = warp < 4 && row < owner_len;
    Box box = {0, -1, 0, -1, 0, -1};
    if (row_ok) box = KV ? key_box(p, row) : query_box(p, row);
    if (warp < 4) mark_tiles_warp(p, box, row_ok, kSub, sh.bitmap);
    __syncthreads();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_word = &sh.abort_word;

    if (sh.abort_word != 0) {
        // an earlier CTA gave up: skip straight to the tear-down
    } else if (warp == 5) {
        if (elect_one()) {
            tma_prefetch_desc(&maps.own0);
            tma_prefetch_desc(&maps.own1);
            tma_prefetch_desc(&maps.st0);
            tma_prefetch_desc(&maps.st1);
            mbar_expect_tx(&sh.own_full, 2 * kChunkBytes);
            tma_load_4d(sOwn, &maps.own0, &sh.own_full, 0, owner0, h, b);
            tma_load_4d(sOwn + kChunkBytes, &maps.own1, &sh.own_full, 0, owner0, h, b);
            int n = 0;
            bool ok = true;
            for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1), ++n) {
                const int st = n % kStages, round = n / kStages;
                if (round > 0) ok = mbar_wait(&sh.empty[st], (round - 1) & 1, abort_word, 60);
                if (!ok) break;
                mbar_expect_tx(&sh.full[st], 2 * kSubBytes);
                tma_load_4d(sRing + st * 2 * kSubBytes, &maps.st0, &sh.full[st], 0, j * kSub, h, b);
                tma_load_4d(sRing + st * 2 * kSubBytes + kSubBytes, &maps.st1, &sh.full[st], 0, j * kSub, h, b);
            }
        }
    } else if (warp == 4) {
        if (elect_one()) {
            const uint32_t idesc_s = umma_idesc(kTile, kSub, BF16 ? 1 : 0, false, false);
            const uint32_t idesc_neg = idesc_s | (p.scale < 0.f ? kUmmaNegateA : 0u);
            constexpr uint32_t idesc_g = umma_idesc(kTile, 64, BF16 ? 1 : 0, false, true);
            const uint64_t own_desc = umma_desc_sw128(smem_u32(sOwn), 16, 1024);
            const uint64_t ring_k = umma_desc_sw128(smem_u32(sRing), 16, 1024);          // K-major view (scores)
            const uint64_t ring_mn = umma_desc_sw128(smem_u32(sRing), kSubBytes, 1024);  // MN-major view (gradients)
            bool ok = mbar_wait(&sh.own_full, 0, abort_word, 61);
            int n = 0;
            for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1), ++n) {
                const int st = n % kStages;
                const uint32_t base = st * 2 * kSubBytes;
                ok = mbar_wait(&sh.full[st], (n / kStages) & 1, abort_word, 62);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_ss(tmem, umma_desc_advance(own_desc, kk * 32), umma_desc_advance(ring_k, base + kk * 32),
                            idesc_neg, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_ss(tmem + 64, umma_desc_advance(own_desc, kChunkBytes + kk * 32),
                            umma_desc_advance(ring_k, base + kSubBytes + kk * 32), idesc_s, kk > 0);
                umma_commit(&sh.sdp_ready);
                ok = mbar_wait(&sh.ops_ready, n & 1, abort_word, 63);
                if (!ok) break;
                tc_fence_after();
                // acc0: operand over S with streamed K (query owners) / dO (key owners)
                const uint32_t b0 = base + (KV ? kSubBytes : 0);
#pragma unroll
                for (int kk = 0; kk < kSub / 16; ++kk)
                    umma_ts(tmem + 128, tmem + kk * 8, umma_desc_advance(ring_mn, b0 + kk * 2048), idesc_g,
                            n > 0 || kk > 0);
                // acc1: operand over dP with streamed K (query owners) / Q (key owners)
#pragma unroll
                for (int kk = 0; kk < kSub / 16; ++kk)
                    umma_ts(tmem + 192, tmem + 64 + kk * 8, umma_desc_advance(ring_mn, base + kk * 2048), idesc_g,
                            n > 0 || kk > 0);
                umma_commit(&sh.empty[st]);
            }
            if (ok) umma_commit(&sh.done);
        }
    } else {
        using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        const float c2 = fabsf(p.scale) * kLog2e;
        const int64_t stat0 = ((int64_t)b * p.Hq + h) * p.Sq;
        float row_m = INFINITY, row_ls = 0.f, row_dl = 0.f;
        if (!KV && row_ok) {
            row_m = p.maximum[stat0 + row];
            row_ls = p.logsum[stat0 + row];
            row_dl = p.delta[stat0 + row];
            if (row_m == -INFINITY) row_m = INFINITY;
        }
        uint64_t acc_ds = f2_pack(0.f, 0.f), acc_mass = acc_ds, acc_num = acc_ds, acc_den = acc_ds;
        const int tid = warp * 32 + lane;
        int n = 0;
        bool ok = true;
        BoxCursor cursor = box_cursor(p, box);
        for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1), ++n) {
            const int part0 = j * kSub;
            if (KV) {
                // stage the statistics of the 64 streamed queries (two threads per query)
                float* stat = &sh.stats[n & 1][0][0];
                if (tid < kSub) {
                    const int qi = part0 + tid;
                    const bool in = qi < p.Sq;
                    float m = in ? p.maximum[stat0 + qi] : INFINITY;
                    if (m == -INFINITY) m = INFINITY;
                    stat[tid] = m;
                    stat[kSub + tid] = in ? p.logsum[stat0 + qi] : 0.f;
                } else {
                    const int qi = part0 + tid - kSub;
                    const bool in = qi < p.Sq;
                    // (dP - delta) - t is formed as dP - (delta + t): the sum is staged once per query
                    stat[2 * kSub + tid - kSub] = in ? p.delta[stat0 + qi] + p.aux[stat0 + qi] : 0.f;
                }
                bar_sync(1, kTile);
            }
            uint32_t vis[2] = {0, 0};
            if (row_ok) box_mask_walk<2>(p, box, cursor, part0, vis);
            ok = mbar_wait(&sh.sdp_ready, n & 1, abort_word, 64);
            if (!ok) break;
            tc_fence_after();
            const float* stat = &sh.stats[n & 1][0][0];
            const uint64_t c2_pair = f2_pack(c2, c2);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t s[32], dp[32], w0[16], w1[16];
                if (!__any_sync(0xffffffffu, vis[half] != 0)) {
                    // no row of this warp sees these 32 partners: both operands are zero
#pragma unroll
                    for (int i = 0; i < 16; ++i) w0[i] = 0;
                    tmem_st16(lane_base + half * 16, w0);
                    tmem_st16(lane_base + 64 + half * 16, w0);
                    continue;
                }
                tmem_ld32(lane_base + half * 32, s);
                tmem_ld32(lane_base + 64 + half * 32, dp);
                tmem_wait_ld();
                float4 mm4, ll4, dd4;  // key owners: the statistics of four streamed queries per 16-byte load
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    uint64_t m2, ls2, dl2;
                    if (KV) {
                        if ((c & 2) == 0) {
                            mm4 = *reinterpret_cast<const float4*>(stat + half * 32 + c);
                            ll4 = *reinterpret_cast<const float4*>(stat + kSub + half * 32 + c);
                            dd4 = *reinterpret_cast<const float4*>(stat + 2 * kSub + half * 32 + c);
                        }
                        m2 = (c & 2) == 0 ? f2_pack(mm4.x, mm4.y) : f2_pack(mm4.z, mm4.w);
                        ls2 = (c & 2) == 0 ? f2_pack(ll4.x, ll4.y) : f2_pack(ll4.z, ll4.w);
                        dl2 = (c & 2) == 0 ? f2_pack(dd4.x, dd4.y) : f2_pack(dd4.z, dd4.w);  // delta + t of the query
                    } else {
                        m2 = f2_pack(row_m, row_m);
                        ls2 = f2_pack(row_ls, row_ls);
                        dl2 = f2_pack(row_dl, row_dl);
                    }
                    // hidden entries: score -inf, so P32 is an exact zero and so is everything built from it
                    const uint64_t sc = f2_pack(__uint_as_float(hide(s[c], vis[half], c)),
                                                __uint_as_float(hide(s[c + 1], vis[half], c + 1)));
                    float ea, eb;
                    f2_unpack(f2_sub(f2_mul(f2_sub(sc, m2), c2_pair), ls2), ea, eb);
                    const uint64_t p32 = f2_pack(ex2(ea), ex2(eb));
                    const uint64_t prod =
                        f2_mul(p32, f2_sub(f2_pack(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), dl2));
                    float pa, pb, da, db;
                    f2_unpack(p32, pa, pb);
                    f2_unpack(prod, da, db);
                    const uint32_t pl = pack2<BF16>(pa, pb), ds = pack2<BF16>(da, db);
                    if (!KV) {
                        const float2 plf = unpack2<BF16>(pl), dsf = unpack2<BF16>(ds);
                        acc_ds = f2_add(acc_ds, f2_pack(dsf.x, dsf.y));
                        acc_mass = f2_add(acc_mass, f2_pack(plf.x, plf.y));
                        acc_num = f2_add(acc_num, prod);
                        acc_den = f2_add(acc_den, p32);
                    }
                    // 16-bit operands: over S goes dS_q (query owners) / rd(P32) (key owners); over dP the other
                    w0[c / 2] = KV ? pl : ds;
                    w1[c / 2] = KV ? ds : pl;
                }
                tmem_st16(lane_base + half * 16, w0);
                tmem_st16(lane_base + 64 + half * 16, w1);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sh.ops_ready);
        }
        if (n > 0 && ok) ok = mbar_wait(&sh.done, 0, abort_word, 65);
        if (ok) {
            tc_fence_after();
            T* out0 = nullptr;
            T* out1 = nullptr;
            const int r = row_ok ? row : 0;
            if (KV) {
                out0 = reinterpret_cast<T*>(p.dv) + (int64_t)b * p.dvs[0] + (int64_t)h * p.dvs[1] + (int64_t)r * p.dvs[2];
                out1 = reinterpret_cast<T*>(p.dk) + (int64_t)b * p.dks[0] + (int64_t)h * p.dks[1] + (int64_t)r * p.dks[2];
            } else {
                out0 = reinterpret_cast<T*>(p.dq) + (int64_t)b * p.dqs[0] + (int64_t)h * p.dqs[1] + (int64_t)r * p.dqs[2];
            }
            float u0, u1;
            f2_unpack(acc_ds, u0, u1);
            const float sum_ds = u0 + u1;
            f2_unpack(acc_mass, u0, u1);
            const float mass = u0 + u1;
            f2_unpack(acc_num, u0, u1);
            const float t_num = u0 + u1;
            f2_unpack(acc_den, u0, u1);
            const float t_den = u0 + u1;
            const float ratio = mass != 0.f ? sum_ds / mass : 0.f;
#pragma unroll
            for (int c = 0; c < 64; c += 32) {
                uint32_t a0[32], a1[32];
                if (n > 0) {
                    tmem_ld32(lane_base + 128 + c, a0);
                    tmem_ld32(lane_base + 192 + c, a1);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) a0[i] = a1[i] = 0;
                }
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float x[8], y[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float u = __uint_as_float(a0[i + e]), v = __uint_as_float(a1[i + e]);
                            x[e] = KV ? u : (u - ratio * v) * p.scale;
                            y[e] = v * p.scale;
                        }
                        *reinterpret_cast<uint4*>(out0 + c + i) =
                            make_uint4(pack2<BF16>(x[0], x[1]), pack2<BF16>(x[2], x[3]), pack2<BF16>(x[4], x[5]),
                                       pack2<BF16>(x[6], x[7]));
                        if (KV)
                            *reinterpret_cast<uint4*>(out1 + c + i) =
                                make_uint4(pack2<BF16>(y[0], y[1]), pack2<BF16>(y[2], y[3]), pack2<BF16>(y[4], y[5]),
                                           pack2<BF16>(y[6], y[7]));
                    }
                }
            }
            if (!KV && row_ok) p.aux[stat0 + row] = t_den != 0.f ? t_num / t_den : 0.f;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 4100 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == 4) tmem_dealloc(tmem, 256);
}

constexpr int kBwdSmem = 2 * kChunkBytes + kStages * 2 * kSubBytes + 4096 + 1024;

constexpr int kFwdSmem = (1 + kRing) * kChunkBytes + 1024 + 1024;

bool encode_all(NaMaps* maps, const AttnParams& p, bool bf16, bool backward, int box_rows_partner) {
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    (void)box_rows_partner;
    if (!encode_bhsd_map(&maps->q, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTile)) return false;
    if (!encode_bhsd_map(&maps->k, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTile)) return false;
    if (!encode_bhsd_map(&maps->v, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTile)) return false;
    if (backward) {
        if (!encode_bhsd_map(&maps->g, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, kTile)) return false;
    } else {
        maps->g = maps->q;
    }
    return true;
}

template <bool BF16>
cudaError_t forward_t(const AttnParams& p, cudaStream_t st) {
    auto kernel = p.two_term ? na_tc_forward<BF16, true> : na_tc_forward<BF16, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (e != cudaSuccess) return e;
    // two CTAs per SM need the largest shared-memory carve-out
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    NaMaps maps;
    if (!encode_all(&maps, p, BF16, false, kTile)) return cudaErrorInvalidValue;
    const int64_t grid = (int64_t)((p.Sq + kTile - 1) / kTile) * p.B * p.Hq;
    kernel<<<(unsigned)grid, 192, kFwdSmem, st>>>(maps, p);
    return cudaGetLastError();
}

template <bool KV, bool BF16>
cudaError_t backward_t(const AttnParams& p, cudaStream_t st) {
    cudaError_t e =
        cudaFuncSetAttribute(na_tc_backward<KV, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(na_tc_backward<KV, BF16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    const CUtensorMapDataType dt = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    BwdMaps maps;
    bool ok;
    if (KV) {
        ok = encode_bhsd_map(&maps.own0, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTile) &&
             encode_bhsd_map(&maps.own1, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTile) &&
             encode_bhsd_map(&maps.st0, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kSub) &&
             encode_bhsd_map(&maps.st1, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, kSub);
    } else {
        ok = encode_bhsd_map(&maps.own0, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTile) &&
             encode_bhsd_map(&maps.own1, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, kTile) &&
             encode_bhsd_map(&maps.st0, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kSub) &&
             encode_bhsd_map(&maps.st1, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kSub);
    }
    if (!ok) return cudaErrorInvalidValue;
    const int owner_len = KV ? p.Sk : p.Sq;
    const int64_t grid = (int64_t)((owner_len + kTile - 1) / kTile) * p.B * p.Hq;
    na_tc_backward<KV, BF16><<<(unsigned)grid, 192, kBwdSmem, st>>>(maps, p);
    return cudaGetLastError();
}

bool common_supported(const AttnParams& p) {
    if (p.nd != 2 && p.nd != 3) return false;
    if (p.D != 64 || p.Hq != p.Hkv || p.Sq != p.Sk) return false;
    if (p.scale == 0.f || p.Sk < 2) return false;
    if ((int64_t)p.Sk > (int64_t)kMapWords * 32 * 64) return false;  // bitmap capacity at 64-token tiles
    return tma_compatible(p.q, p.qs, p.B, p.Hq, p.Sq) && tma_compatible(p.k, p.ks, p.B, p.Hkv, p.Sk) &&
           tma_compatible(p.v, p.vs, p.B, p.Hkv, p.Sk);
}

}  // namespace

bool na_pipeline_forward_supported(const AttnParams& p) {
    return common_supported(p) && tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq);
}

cudaError_t launch_na_pipeline_forward(const AttnParams& p, bool bf16, cudaStream_t st) {
    return bf16 ? forward_t<true>(p, st) : forward_t<false>(p, st);
}

bool na_pipeline_backward_supported(const AttnParams& p) {
    return common_supported(p) && tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq) &&
           tma_compatible(p.dout, p.gs, p.B, p.Hq, p.Sq) && tma_compatible(p.dq, p.dqs, p.B, p.Hq, p.Sq) &&
           tma_compatible(p.dk, p.dks, p.B, p.Hkv, p.Sk) && tma_compatible(p.dv, p.dvs, p.B, p.Hkv, p.Sk);
}

// which 0: dQ and the per-query correction t (must run first); 1: dK and dV.
cudaError_t launch_na_pipeline_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st) {
    if (which == 0) return bf16 ? backward_t<false, true>(p, st) : backward_t<false, false>(p, st);
    return bf16 ? backward_t<true, true>(p, st) : backward_t<true, false>(p, st);
}


KFA_PHASE_EXPORT(kfa_debug_phases_na)

}  // namespace kfa
