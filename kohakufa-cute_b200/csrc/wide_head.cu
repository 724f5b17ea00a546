// Wide heads (256, 384 or 512 channels) on the Blackwell tensor-memory pipeline.
//
// A 128-row accumulator with 512 FP32 channels fills the whole tensor memory of an SM, and two
// 128 x 512 operands do not fit its shared memory, so the narrow-head kernels do not scale up.
// This family splits the work differently:
//
//   wide_forward   a CTA owns 128 query rows and ONE HALF of the output channels.  It forms the
//                  full score tile S = Q K^T (Q resident, K streamed as 64-channel chunks), runs
//                  the shifted-score online softmax, and accumulates O[:, half] = P V[:, half].
//                  The sibling CTA repeats the scores for the other half (1.5x the algorithmic
//                  tensor work, no exchange between CTAs).
//   wide_scores    backward, step 1 and 2: P_low = rd(ex2((s'-m)c - logsum)) and
//                  dS_low = rd(P_low (dP - delta)) are written ONCE as 16-bit matrices
//                  [B, Hq, Sq, Sk] into the caller's workspace (Q resident / K streamed for P,
//                  dO resident / V streamed for dS).  Hidden entries are exact zeros.
//   wide_grad      backward, step 3: dQ = dS_low K, dK = dS_low^T Q, dV = P_low^T dO as plain
//                  tensor-core products over the stored matrices; a CTA owns 128 output rows and
//                  one half of the channels, so no score is recomputed and no atomics are needed.
//
// The arithmetic is the operator's contract (reference behaviour:
// src/kohakufa_cute/blackwell_pipeline.py:141-209, 610-662 and docs/precision.md:13-23 of the
// reference project): P_low and dS_low are rounded once - exactly the values that are stored -
// every product accumulates in FP32, and the signed scale is applied after accumulation.
#include "kfa_common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

#include <type_traits>

namespace kfa {
namespace {

constexpr int kTile = 128;
constexpr int kChunkBytes = kTile * 128;  // 128 rows x 64 channels of a 16-bit type (one TMA box)
constexpr int kRing = 6;                  // 16 KB slots for streamed chunks
// The accumulator is re-based when the row maximum has grown by more than this power of two in probability terms:
// probabilities against the stale maximum stay inside FP16 (2^14) or BF16's FP32 range (2^32), and the round trip of
// the accumulator through registers stays rare also for large logits.
template <bool BF16>
__host__ __device__ constexpr float rebase_limit() { return BF16 ? 32.0f : 14.0f; }

// Combined state of key tile j (128 keys) for the query rows [q0, q0 + 128), from the 64x64 table entries:
// 0 hidden, 2 visible, 1 mixed.  Masks broadcast over queries have one row of entries.
__device__ __forceinline__ int key_tile_state(const AttnParams& p, int b, int h, int q0, int j) {
    if (!p.has_mask) return 2;
    const int nk64 = (p.Sk + 63) >> 6;
    const int32_t* base = p.blocks + (int64_t)b * p.bs[0] + (int64_t)h * p.bs[1];
    int r0 = 0, r1 = 0;
    if (p.bs[2] != 0) {
        r0 = q0 >> 6;
        r1 = (min(q0 + kTile, p.Sq) - 1) >> 6;
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

// Key tiles a 128-row query tile starting at q0 may see.
__device__ __forceinline__ int key_tiles_of(const AttnParams& p, int q0) {
    const int row_hi = min(p.Sq, q0 + kTile);
    const int k_hi = p.causal ? max(0, min(p.Sk, row_hi + p.causal_shift)) : p.Sk;
    return (k_hi + kTile - 1) / kTile;
}

struct WideMaps {
    CUtensorMap a, b, c;
};

// ------------------------------------------------------------------------------------------ forward
struct FwdShared {
    uint64_t q_full;
    uint64_t full[kRing];
    uint64_t empty[kRing];
    uint64_t s_ready;
    uint64_t p_ready;
    uint64_t pvb_done;
    uint32_t tmem_base;
    int abort_word;
};

// maps.a = Q, maps.b = K, maps.c = V.  256 threads: warps 0-3 softmax (thread <-> query row),
// warps 4 and 6 MMA issuers, warps 5 and 7 loaders.  A tcgen05.mma holds its issuing thread for about a
// hundred cycles whatever its size, and a 512-channel score tile needs 32 of them, so the scores are
// formed by TWO issuers into two partial accumulators: issuer 0 contracts the even 64-channel chunks
// into S_a (column 0), issuer 1 the odd ones into S_b (column 128); the softmax adds the two.  Each
// issuer then forms its share of the output channels of O[:, half] (column 256) from P_low, which
// overwrites the first 64 columns of S_a.
template <bool BF16>
__global__ void __launch_bounds__(256, 1) wide_forward(const __grid_constant__ WideMaps maps, AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int chunks = p.D >> 6, hc = chunks >> 1;
    uint8_t* sQ = smem;
    uint8_t* sRing = smem + chunks * kChunkBytes;
    FwdShared& sh = *reinterpret_cast<FwdShared*>(sRing + kRing * kChunkBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = blockIdx.x & 1;
    const int64_t rest = blockIdx.x >> 1;
    // Tile-major block order: under a causal mask the late (heavy) query tiles of EVERY head are
    // dispatched before any light one, which keeps the last wave short.
    const int nblk = (p.Sq + kTile - 1) / kTile;
    const int64_t nbh = (int64_t)p.B * p.Hq;
    const int qblk = nblk - 1 - (int)(rest / nbh);
    const int64_t bh = rest % nbh;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int kvh = h / p.group;
    const int q0 = qblk * kTile;
    const int n_tiles = key_tiles_of(p, q0);

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.q_full, 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.empty[i], 1);
        }
        mbar_init(&sh.s_ready, 2);  // both issuers
        mbar_init(&sh.p_ready, kTile);
        mbar_init(&sh.pvb_done, 1);
        mbar_fence_init();
    }
    if (warp == 4) {
        tmem_alloc(&sh.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_word = &sh.abort_word;

    if (sh.abort_word != 0) {
        // an earlier CTA gave up: skip straight to the tear-down
    } else if (warp == 5 || warp == 7) {
        // --------------------------------------------------------------- loaders
        // Two loading threads take alternate ring positions: one thread's stream of 16 KB boxes does not
        // keep the ring full.
        if (elect_one()) {
            const int me = warp == 5 ? 0 : 1;
            tma_prefetch_desc(&maps.a);
            tma_prefetch_desc(&maps.b);
            tma_prefetch_desc(&maps.c);
            if (me == 0) {
                mbar_expect_tx(&sh.q_full, chunks * kChunkBytes);
                for (int c = 0; c < chunks; ++c)
                    tma_load_4d(sQ + c * kChunkBytes, &maps.a, &sh.q_full, c * 64, q0, h, b);
            }
            int pos = 0;
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (key_tile_state(p, b, h, q0, j) == 0) continue;
                // the K chunks of the tile, then the V chunks of this CTA's channel half
                for (int i = 0; i < chunks + hc && ok; ++i, ++pos) {
                    if ((pos & 1) != me) continue;
                    const int slot = pos % kRing, round = pos / kRing;
                    if (round > 0) ok = mbar_wait(&sh.empty[slot], (round - 1) & 1, abort_word, 10);
                    if (!ok) break;
                    mbar_expect_tx(&sh.full[slot], kChunkBytes);
                    if (i < chunks)
                        tma_load_4d(sRing + slot * kChunkBytes, &maps.b, &sh.full[slot], i * 64, j * kTile, kvh, b);
                    else
                        tma_load_4d(sRing + slot * kChunkBytes, &maps.c, &sh.full[slot],
                                    (half * hc + i - chunks) * 64, j * kTile, kvh, b);
                }
            }
        }
    } else if (warp == 4 || warp == 6) {
        // ----------------------------------------------------------- MMA issuers
        if (elect_one()) {
            const int who = warp == 4 ? 0 : 1;
            const uint32_t idesc_s =
                umma_idesc(kTile, kTile, BF16 ? 1 : 0, false, false) | (p.scale < 0.f ? kUmmaNegateA : 0u);
            // output channels of this CTA are split between the issuers by V chunk
            const int ha = (hc + 1) / 2;
            const int v_first = who == 0 ? 0 : ha, v_count = who == 0 ? ha : hc - ha;
            const uint32_t idesc_o = umma_idesc(kTile, 64 * v_count, BF16 ? 1 : 0, false, true);
            const uint64_t q_desc = umma_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t k_desc = umma_desc_sw128(smem_u32(sRing), 16, 1024);
            // the V chunks of one tile sit in consecutive slots: one instruction spans an issuer's share
            const uint64_t v_desc = umma_desc_sw128(smem_u32(sRing), kChunkBytes, 1024);
            bool ok = mbar_wait(&sh.q_full, 0, abort_word, 20);
            int pos = 0, iter = 0;
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (key_tile_state(p, b, h, q0, j) == 0) continue;
                // S_a also holds P_low of the previous tile, which issuer 1's product is still reading
                if (who == 0 && iter > 0) ok = mbar_wait(&sh.pvb_done, (iter - 1) & 1, abort_word, 24);
                for (int c = 0; c < chunks && ok; ++c, ++pos) {
                    if ((c & 1) != who) continue;
                    const int slot = pos % kRing;
                    ok = mbar_wait(&sh.full[slot], (pos / kRing) & 1, abort_word, 21);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_ss(tmem + who * 128, umma_desc_advance(q_desc, c * kChunkBytes + kk * 32),
                                umma_desc_advance(k_desc, slot * kChunkBytes + kk * 32), idesc_s, c > who || kk > 0);
                    umma_commit(&sh.empty[slot]);
                }
                if (!ok) break;
                umma_commit(&sh.s_ready);
                const int s0 = (pos + v_first) % kRing;
                for (int i = 0; i < v_count && ok; ++i)
                    ok = mbar_wait(&sh.full[(pos + v_first + i) % kRing], ((pos + v_first + i) / kRing) & 1, abort_word,
                                   22);
                if (ok) ok = mbar_wait(&sh.p_ready, iter & 1, abort_word, 23);
                if (!ok) break;
                tc_fence_after();
                if (v_count > 0) {
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        umma_ts(tmem + 256 + v_first * 64, tmem + kk * 8,
                                umma_desc_advance(v_desc, s0 * kChunkBytes + kk * 2048), idesc_o, iter > 0 || kk > 0);
                }
                for (int i = 0; i < v_count; ++i) umma_commit(&sh.empty[(pos + v_first + i) % kRing]);
                if (who == 1) umma_commit(&sh.pvb_done);
                pos += hc;
                ++iter;
            }
            if (ok) umma_commit(&sh.s_ready);  // completion of the last product
        }
    } else if (warp < 4) {
        // --------------------------------------------------------------- softmax
        using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const int row = q0 + warp * 32 + lane;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        const uint32_t s_addr = lane_base, o_addr = lane_base + 256;
        const int width = 64 * hc;  // output channels of this CTA
        const float c2 = fabsf(p.scale) * kLog2e;
        const uint64_t c2_pair = f2_pack(c2, c2);
        // this row's line of the mask (every row shares one line when the mask is broadcast over queries)
        const uint8_t* kmask = p.has_mask ? p.mask + (int64_t)b * p.ms[0] + (int64_t)h * p.ms[1] +
                                                (int64_t)min(row, p.Sq - 1) * p.ms[2]
                                          : nullptr;
        float m_used = -INFINITY, m_true = -INFINITY, l = 0.f;
        int iter = 0;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int state = key_tile_state(p, b, h, q0, j);
            if (state == 0) continue;
            ok = mbar_wait(&sh.s_ready, iter & 1, abort_word, 30);
            if (!ok) break;
            tc_fence_after();
            float s[kTile];
#pragma unroll
            for (int c = 0; c < kTile; c += 32) {
                uint32_t ra[32], rb[32];
                tmem_ld32(s_addr + c, ra);
                tmem_ld32(s_addr + 128 + c, rb);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) s[c + i] = __uint_as_float(ra[i]) + __uint_as_float(rb[i]);
            }
            const int key0 = j * kTile;
            int lim = p.Sk - key0;
            if (p.causal) lim = min(lim, row + p.causal_shift - key0 + 1);
            if (lim < kTile) {
#pragma unroll
                for (int c = 0; c < kTile; ++c) s[c] = c < lim ? s[c] : -INFINITY;
            }
            if (state == 1) {
#pragma unroll
                for (int c = 0; c < kTile; ++c) {
                    const int key = min(key0 + c, p.Sk - 1);
                    s[c] = kmask[(int64_t)key * p.ms[3]] != 0 ? s[c] : -INFINITY;
                }
            }
            float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
#pragma unroll
            for (int c = 6; c < kTile - 2; c += 4) {
                mx0 = max3(mx0, s[c], s[c + 1]);
                mx1 = max3(mx1, s[c + 2], s[c + 3]);
            }
            const float mx = max3(mx0, mx1, fmaxf(s[kTile - 2], s[kTile - 1]));
            m_true = fmaxf(m_true, mx);
            const bool rebase = mx > m_used && (m_used == -INFINITY || (mx - m_used) * c2 > rebase_limit<BF16>());
            float alpha = 1.f;
            if (rebase) {
                alpha = (m_used == -INFINITY) ? 0.f : ex2((m_used - mx) * c2);
                l *= alpha;
                m_used = mx;
            }
            // s_ready of this tile was committed after the previous product, so O is quiescent here
            if (iter > 0 && __any_sync(0xffffffffu, rebase)) {
                for (int c = 0; c < width; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(o_addr + c, r);
                }
            }
            const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
            const uint64_t m_pair = f2_pack(m_safe, m_safe);
            uint64_t sum_a = f2_pack(0.f, 0.f), sum_b = sum_a;
#pragma unroll
            for (int c = 0; c < kTile; c += 32) {
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
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
            }
            {
                float x0, x1, x2, x3;
                f2_unpack(sum_a, x0, x1);
                f2_unpack(sum_b, x2, x3);
                l += (x0 + x1) + (x2 + x3);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sh.p_ready);
            ++iter;
        }
        T* orow = reinterpret_cast<T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] + (int64_t)row * p.os[2] +
                  half * width;
        const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + row;
        if (ok && iter == 0 && row < p.Sq) {
            // every key tile of this row is hidden: zero output, empty statistics
            for (int d = 0; d < width; d += 8) *reinterpret_cast<uint4*>(orow + d) = make_uint4(0, 0, 0, 0);
            if (half == 0 && p.maximum) {
                p.maximum[si] = -INFINITY;
                p.logsum[si] = 0.f;
            }
        }
        if (iter > 0) {
            if (ok) ok = mbar_wait(&sh.s_ready, iter & 1, abort_word, 31);
            if (ok) {
                tc_fence_after();
                const float den = l > 0.f ? l : 1.f;
                const float inv_den = 1.f / den;  // one division per row; the elements are multiplied
                for (int c = 0; c < width; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c, r);
                    tmem_wait_ld();
                    if (row < p.Sq) {
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
                if (row < p.Sq && half == 0 && p.maximum) {
                    p.maximum[si] = m_true;
                    p.logsum[si] = l > 0.f ? log2f(l) + (m_used - m_true) * c2 : 0.f;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 3000 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == 4) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------- backward: P and dS matrices
// The stored matrices: 16-bit [B, Hq, Sq, pitch] with pitch = Sk rounded up to 128.
struct Stored {
    void* p_low;
    void* ds_low;
    int64_t pitch;
    int parts;  // CTAs that share one query tile's key tiles (tile j goes to part j % parts)
};

struct ScoreShared {
    uint64_t own_full;
    uint64_t full[kRing];
    uint64_t empty[kRing];
    uint64_t s_ready[2];
    uint64_t s_free[2];
    uint32_t tmem_base;
    int abort_word;
};

// MODE 0: maps.a = Q (resident), maps.b = K (streamed); writes P_low.
// MODE 1: maps.a = dO (resident), maps.b = V (streamed); reads P_low, writes dS_low.
// 256 threads: warps 0-3 consumers (thread <-> query row), warps 4 and 6 MMA issuers, warp 5 loader.
// Two score buffers in tensor memory (columns 0 and 256, each a pair of partial accumulators) let the
// tensor core run one tile ahead.
template <int MODE, bool BF16>
__global__ void __launch_bounds__(256, 1) wide_scores(const __grid_constant__ WideMaps maps, AttnParams p, Stored st) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int chunks = p.D >> 6;
    uint8_t* sOwn = smem;
    uint8_t* sRing = smem + chunks * kChunkBytes;
    ScoreShared& sh = *reinterpret_cast<ScoreShared*>(sRing + kRing * kChunkBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = (p.Sq + kTile - 1) / kTile;
    const int64_t nbh = (int64_t)p.B * p.Hq;
    const int part = (int)(blockIdx.x % st.parts);
    const int64_t rest = blockIdx.x / st.parts;
    const int qblk = nblk - 1 - (int)(rest / nbh);  // tile-major order, heavy causal tiles first
    const int64_t bh = rest % nbh;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    const int kvh = h / p.group;
    const int q0 = qblk * kTile;
    const int n_tiles = key_tiles_of(p, q0);

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.own_full, 1);
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh.s_ready[i], 2);  // both issuers
            mbar_init(&sh.s_free[i], kTile);
        }
        mbar_fence_init();
    }
    if (warp == 4) {
        tmem_alloc(&sh.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_word = &sh.abort_word;

    if (sh.abort_word != 0) {
        // an earlier CTA gave up: skip straight to the tear-down
    } else if (warp == 5) {
        if (elect_one()) {
            tma_prefetch_desc(&maps.a);
            tma_prefetch_desc(&maps.b);
            mbar_expect_tx(&sh.own_full, chunks * kChunkBytes);
            for (int c = 0; c < chunks; ++c)
                tma_load_4d(sOwn + c * kChunkBytes, &maps.a, &sh.own_full, c * 64, q0, h, b);
            int pos = 0;
            bool ok = true;
            for (int j = part; j < n_tiles && ok; j += st.parts)
                for (int c = 0; c < chunks && ok; ++c, ++pos) {
                    const int slot = pos % kRing, round = pos / kRing;
                    if (round > 0) ok = mbar_wait(&sh.empty[slot], (round - 1) & 1, abort_word, 40);
                    if (!ok) break;
                    mbar_expect_tx(&sh.full[slot], kChunkBytes);
                    tma_load_4d(sRing + slot * kChunkBytes, &maps.b, &sh.full[slot], c * 64, j * kTile, kvh, b);
                }
        }
    } else if (warp == 4 || warp == 6) {
        // Two issuers share the contraction: issuer 0 the even 64-channel chunks, issuer 1 the odd ones,
        // each into its own partial accumulator (columns +0 and +128 of the score buffer).
        if (elect_one()) {
            const int who = warp == 4 ? 0 : 1;
            const uint32_t idesc = umma_idesc(kTile, kTile, BF16 ? 1 : 0, false, false) |
                                   (MODE == 0 && p.scale < 0.f ? kUmmaNegateA : 0u);
            const uint64_t a_desc = umma_desc_sw128(smem_u32(sOwn), 16, 1024);
            const uint64_t b_desc = umma_desc_sw128(smem_u32(sRing), 16, 1024);
            bool ok = mbar_wait(&sh.own_full, 0, abort_word, 41);
            int pos = 0;
            for (int n = 0; part + n * st.parts < n_tiles && ok; ++n) {
                const int buf = n & 1;
                if (n >= 2) ok = mbar_wait(&sh.s_free[buf], ((n >> 1) - 1) & 1, abort_word, 42);
                if (!ok) break;
                tc_fence_after();
                for (int c = 0; c < chunks && ok; ++c, ++pos) {
                    if ((c & 1) != who) continue;
                    const int slot = pos % kRing;
                    ok = mbar_wait(&sh.full[slot], (pos / kRing) & 1, abort_word, 43);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_ss(tmem + buf * 256 + who * 128, umma_desc_advance(a_desc, c * kChunkBytes + kk * 32),
                                umma_desc_advance(b_desc, slot * kChunkBytes + kk * 32), idesc, c > who || kk > 0);
                    umma_commit(&sh.empty[slot]);
                }
                if (ok) umma_commit(&sh.s_ready[buf]);
            }
        }
    } else if (warp < 4) {
        const int row = q0 + warp * 32 + lane;
        const bool row_ok = row < p.Sq;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        const float c2 = fabsf(p.scale) * kLog2e;
        const uint64_t c2_pair = f2_pack(c2, c2);
        const int64_t si = ((int64_t)b * p.Hq + h) * p.Sq + (row_ok ? row : 0);
        float row_m = INFINITY, row_ls = 0.f, row_dl = 0.f;
        if (row_ok) {
            if (MODE == 0) {
                row_m = p.maximum[si];
                row_ls = p.logsum[si];
                if (row_m == -INFINITY) row_m = INFINITY;  // nothing visible: every P is zero
            } else {
                row_dl = p.delta[si];
            }
        }
        const uint8_t* kmask = p.has_mask ? p.mask + (int64_t)b * p.ms[0] + (int64_t)h * p.ms[1] +
                                                (int64_t)min(row, p.Sq - 1) * p.ms[2]
                                          : nullptr;
        const int64_t row_off = (((int64_t)b * p.Hq + h) * p.Sq + (row_ok ? row : 0)) * st.pitch;
        uint16_t* p_row = reinterpret_cast<uint16_t*>(st.p_low) + row_off;
        uint16_t* ds_row = reinterpret_cast<uint16_t*>(st.ds_low) + row_off;
        bool ok = true;
        for (int n = 0; part + n * st.parts < n_tiles && ok; ++n) {
            const int j = part + n * st.parts;
            const int buf = n & 1, key0 = j * kTile;
            uint4 pl[16];
            if (MODE == 1 && row_ok) {
#pragma unroll
                for (int i = 0; i < 16; ++i) pl[i] = *reinterpret_cast<const uint4*>(p_row + key0 + i * 8);
            }
            ok = mbar_wait(&sh.s_ready[buf], (n >> 1) & 1, abort_word, 44);
            if (!ok) break;
            tc_fence_after();
            float s[kTile];
#pragma unroll
            for (int c = 0; c < kTile; c += 32) {
                uint32_t ra[32], rb[32];
                tmem_ld32(lane_base + buf * 256 + c, ra);
                tmem_ld32(lane_base + buf * 256 + 128 + c, rb);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) s[c + i] = __uint_as_float(ra[i]) + __uint_as_float(rb[i]);
            }
            tc_fence_before();
            mbar_arrive(&sh.s_free[buf]);
            if (!row_ok) continue;
            if (MODE == 0) {
                int lim = p.Sk - key0;
                if (p.causal) lim = min(lim, row + p.causal_shift - key0 + 1);
                const int state = key_tile_state(p, b, h, q0, j);
                const uint64_t m_pair = f2_pack(row_m, row_m), l_pair = f2_pack(row_ls, row_ls);
#pragma unroll
                for (int c = 0; c < kTile; c += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        float pa, pb;
                        f2_unpack(f2_sub(f2_mul(f2_sub(f2_pack(s[c + i], s[c + i + 1]), m_pair), c2_pair), l_pair), pa,
                                  pb);
                        pa = ex2(pa);
                        pb = ex2(pb);
                        pa = c + i < lim ? pa : 0.f;
                        pb = c + i + 1 < lim ? pb : 0.f;
                        if (state != 2) {
                            pa = kmask[(int64_t)min(key0 + c + i, p.Sk - 1) * p.ms[3]] != 0 ? pa : 0.f;
                            pb = kmask[(int64_t)min(key0 + c + i + 1, p.Sk - 1) * p.ms[3]] != 0 ? pb : 0.f;
                        }
                        w[i / 2] = pack2<BF16>(pa, pb);
                    }
                    *reinterpret_cast<uint4*>(p_row + key0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
                const uint64_t d_pair = f2_pack(row_dl, row_dl);
#pragma unroll
                for (int c = 0; c < kTile; c += 8) {
                    const uint32_t in[4] = {pl[c / 8].x, pl[c / 8].y, pl[c / 8].z, pl[c / 8].w};
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const float2 pv = unpack2<BF16>(in[i / 2]);
                        float da, db;
                        f2_unpack(f2_mul(f2_pack(pv.x, pv.y), f2_sub(f2_pack(s[c + i], s[c + i + 1]), d_pair)), da, db);
                        // a hidden entry has P_low = 0; keep its gradient an exact zero whatever dP holds
                        da = pv.x == 0.f ? 0.f : da;
                        db = pv.y == 0.f ? 0.f : db;
                        w[i / 2] = pack2<BF16>(da, db);
                    }
                    *reinterpret_cast<uint4*>(ds_row + key0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 3100 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == 4) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------- backward: gradient products
constexpr int kGradStages = 2;  // two CTAs share an SM: one's start-up and epilogue run under the other's loads and products
constexpr int kHalfChunkBytes = 64 * 128;  // 64 rows x 64 elements of a 16-bit type

struct GradShared {
    uint64_t full[kGradStages];
    uint64_t empty[kGradStages];
    uint64_t done;
    uint32_t tmem_base;
    int abort_word;
};

struct GradMaps {
    CUtensorMap ds;              // dS_low, boxes of 64 keys x 128 queries (dQ: the matrix is the K-major A operand)
    CUtensorMap ds64, p64;       // the two stored matrices, boxes of 64 keys x 64 queries (dK, dV: MN-major A)
    CUtensorMap k64, q64, g64;   // K, Q and dO, boxes of 64 channels x 64 rows
};

// One launch forms all three gradients; the block index selects the product:
//   0: dQ[q tile] = scale * sum_kt dS_low[q tile, kt] K[kt]        (A K-major,  rows = queries)
//   1: dK[k tile] = scale * sum_{g,i} dS_low[i, k tile]^T Q_g[i]   (A MN-major, rows = keys)
//   2: dV[k tile] =         sum_{g,i} P_low[i, k tile]^T dO_g[i]
// (first `n_dq` blocks dQ, then `n_kv` blocks dK, then `n_kv` blocks dV; inside a product heavy causal
// tiles of all heads come first, so the launch ends on light dV tiles.)  A CTA owns 128 output rows and
// one half of the channels.  192 threads: warps 0-3 epilogue (thread <-> output row), warp 4 MMA issuer, warp 5
// loader.  A stage holds HALF of a unit's contraction range: 64 keys (dQ) or 64 queries (dK, dV) of the matrix
// block (16 KB) and the same 64 rows x D/2 channels of the other operand; four such stages keep three loads in
// flight while the fourth is consumed (with whole units per stage only one 96 KB load was in flight, and the
// launch ran at a third of the rate at which shared memory can be filled).
template <bool BF16>
__global__ void __launch_bounds__(192, 2) wide_grad(const __grid_constant__ GradMaps maps, AttnParams p, unsigned n_dq,
                                                    unsigned n_kv) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int which = blockIdx.x < n_dq ? 0 : (blockIdx.x < n_dq + n_kv ? 1 : 2);
    const unsigned local = blockIdx.x - (which == 0 ? 0u : (which == 1 ? n_dq : n_dq + n_kv));
    const bool KV = which != 0;
    const CUtensorMap* map_a = which == 0 ? &maps.ds : (which == 1 ? &maps.ds64 : &maps.p64);
    const CUtensorMap* map_b = which == 0 ? &maps.k64 : (which == 1 ? &maps.q64 : &maps.g64);
    const int hc = p.D >> 7;
    const int stage_bytes = kChunkBytes + hc * kHalfChunkBytes;
    GradShared& sh = *reinterpret_cast<GradShared*>(smem + kGradStages * stage_bytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = local & 1;
    const int64_t rest = local >> 1;
    const int owner_len = KV ? p.Sk : p.Sq, heads = KV ? p.Hkv : p.Hq;
    const int nblk = (owner_len + kTile - 1) / kTile;
    const int64_t nbh = (int64_t)p.B * heads;
    int blk = (int)(rest / nbh);    // tile-major order over all heads
    if (!KV) blk = nblk - 1 - blk;  // causal: late query tiles and early key tiles carry the most work
    const int64_t bh = rest % nbh;
    const int head = (int)(bh % heads), b = (int)(bh / heads);
    const int owner0 = blk * kTile;
    // streamed tile range and the number of passes over it (query heads of the group)
    int first = 0, end, passes = 1;
    if (KV) {
        first = p.causal ? max(0, (owner0 - p.causal_shift) / kTile) : 0;  // first query tile that sees these keys
        end = (p.Sq + kTile - 1) / kTile;
        passes = p.group;
    } else {
        end = key_tiles_of(p, owner0);
    }
    const int per_pass = max(end - first, 0);
    const int units = per_pass * passes;

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        for (int i = 0; i < kGradStages; ++i) {
            mbar_init(&sh.full[i], 1);
            mbar_init(&sh.empty[i], 1);
        }
        mbar_init(&sh.done, 1);
        mbar_fence_init();
    }
    if (warp == 4) {
        tmem_alloc(&sh.tmem_base, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_word = &sh.abort_word;

    if (sh.abort_word != 0) {
        // an earlier CTA gave up: skip straight to the tear-down
    } else if (warp == 5) {
        if (units > 0 && elect_one()) {
            tma_prefetch_desc(map_a);
            tma_prefetch_desc(map_b);
            bool ok = true;
            for (int v = 0; v < 2 * units && ok; ++v) {
                const int u = v >> 1, sub = v & 1;  // unit and half of its contraction range
                const int g = u / per_pass, i = first + u % per_pass;
                const int s = v % kGradStages, round = v / kGradStages;
                if (round > 0) ok = mbar_wait(&sh.empty[s], (round - 1) & 1, abort_word, 50);
                if (!ok) break;
                uint8_t* dst = smem + s * stage_bytes;
                mbar_expect_tx(&sh.full[s], stage_bytes);
                const int hq = KV ? head * p.group + g : head;
                if (KV) {
                    // 64 queries of the streamed tile x the owner's 128 keys, as two boxes of 64 keys
                    for (int c = 0; c < 2; ++c)
                        tma_load_4d(dst + c * kHalfChunkBytes, map_a, &sh.full[s], owner0 + c * 64, i * kTile + sub * 64,
                                    hq, b);
                } else {
                    // the owner's 128 queries x 64 keys of the streamed tile
                    tma_load_4d(dst, map_a, &sh.full[s], i * kTile + sub * 64, owner0, hq, b);
                }
                // the other operand: the same 64 rows of K (dQ) or of Q / dO (dK / dV), this CTA's channels
                const int b_row = i * kTile + sub * 64, b_head = KV ? hq : head / p.group;
                for (int c = 0; c < hc; ++c)
                    tma_load_4d(dst + kChunkBytes + c * kHalfChunkBytes, map_b, &sh.full[s], (half * hc + c) * 64, b_row,
                                b_head, b);
            }
        }
    } else if (warp == 4) {
        if (units > 0 && elect_one()) {
            const uint32_t idesc = umma_idesc(kTile, 64 * hc, BF16 ? 1 : 0, KV, true);
            const uint32_t base = smem_u32(smem);
            const uint64_t a_desc = KV ? umma_desc_sw128(base, kHalfChunkBytes, 1024) : umma_desc_sw128(base, 16, 1024);
            const uint64_t b_desc = umma_desc_sw128(base + kChunkBytes, kHalfChunkBytes, 1024);
            bool ok = true;
            for (int v = 0; v < 2 * units && ok; ++v) {
                const int s = v % kGradStages;
                ok = mbar_wait(&sh.full[s], (v / kGradStages) & 1, abort_word, 51);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {  // 64 contraction rows per stage
                    const uint32_t a_off = KV ? kk * 2048 : kk * 32;
                    umma_ss(tmem, umma_desc_advance(a_desc, s * stage_bytes + a_off),
                            umma_desc_advance(b_desc, s * stage_bytes + kk * 2048), idesc, v > 0 || kk > 0);
                }
                umma_commit(&sh.empty[s]);
            }
            if (ok) umma_commit(&sh.done);
        }
    } else {
        using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
        const int row = owner0 + warp * 32 + lane;
        const int width = 64 * hc;
        void* base = which == 0 ? p.dq : which == 1 ? p.dk : p.dv;
        const int64_t* os = which == 0 ? p.dqs : which == 1 ? p.dks : p.dvs;
        T* out = reinterpret_cast<T*>(base) + (int64_t)b * os[0] + (int64_t)head * os[1] + (int64_t)row * os[2] +
                 half * width;
        const float mul = which == 2 ? 1.f : p.scale;
        // dQ of a call that runs in passes over key ranges: FP32 partial sums between the passes
        const int pass = which == 0 ? p.dq_pass : 0;
        float* part = pass ? p.dq_acc + (((int64_t)b * p.Hq + head) * p.Sq + min(row, p.Sq - 1)) * p.D + half * width
                           : nullptr;
        if (units == 0) {
            if (row < owner_len) {
                if (pass == 0) {
                    for (int d = 0; d < width; d += 8) *reinterpret_cast<uint4*>(out + d) = make_uint4(0, 0, 0, 0);
                } else if (pass == 1) {
                    for (int d = 0; d < width; d += 4) *reinterpret_cast<float4*>(part + d) = make_float4(0.f, 0.f, 0.f, 0.f);
                } else if (pass == 3) {
                    for (int d = 0; d < width; d += 2)
                        *reinterpret_cast<uint32_t*>(out + d) = pack2<BF16>(part[d], part[d + 1]);
                }
            }
        } else if (mbar_wait(&sh.done, 0, abort_word, 52)) {
            tc_fence_after();
            const uint32_t acc = tmem + (static_cast<uint32_t>(warp * 32) << 16);
            for (int c = 0; c < width; c += 32) {
                uint32_t v[32];
                tmem_ld32(acc + c, v);
                tmem_wait_ld();
                if (pass != 0 && row < owner_len) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        float x = __uint_as_float(v[e]) * mul;
                        if (pass != 1) x += part[c + e];
                        v[e] = __float_as_uint(x);
                    }
                    if (pass != 3) {
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            *reinterpret_cast<float4*>(part + c + e) =
                                make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                                            __uint_as_float(v[e + 3]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint4 o;
                            o.x = pack2<BF16>(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
                            o.y = pack2<BF16>(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                            o.z = pack2<BF16>(__uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
                            o.w = pack2<BF16>(__uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
                            *reinterpret_cast<uint4*>(out + c + e) = o;
                        }
                    }
                } else if (row < owner_len) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
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
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 3200 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == 4) tmem_dealloc(tmem, 256);
}

// delta[row] = sum_d f32(O) f32(dO): one warp per row, 16-byte loads.
template <typename T>
__global__ void __launch_bounds__(256) wide_delta(AttnParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t row_id = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    if (row_id >= rows) return;
    int r, h, b;
    split_row(row_id, p.Sq, p.Hq, r, h, b);
    const T* o = reinterpret_cast<const T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] + (int64_t)r * p.os[2];
    const T* g = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1] + (int64_t)r * p.gs[2];
    float sum = 0.f;
    for (int d = lane * 8; d < p.D; d += 256) {
        const uint4 ov = *reinterpret_cast<const uint4*>(o + d), gv = *reinterpret_cast<const uint4*>(g + d);
        const T* oe = reinterpret_cast<const T*>(&ov);
        const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum = fmaf(to_float<T>(oe[e]), to_float<T>(ge[e]), sum);
    }
    sum = warp_sum(sum);
    if (lane == 0) p.delta[row_id] = sum;
}

// ------------------------------------------------------------------------------------ host side
int smem_scores(int D) { return (D / 64 + kRing) * kChunkBytes + 1024 + 256; }
int smem_grad(int D) { return kGradStages * (kChunkBytes + (D / 128) * kHalfChunkBytes) + 1024 + 256; }

bool wide_common(const AttnParams& p) {
    if (p.D != 256 && p.D != 384 && p.D != 512) return false;
    if (p.nd != 0) return false;
    if (p.scale == 0.f || p.Sk < 2) return false;  // exact-zero guarantees of those cases live in the general kernels
    return tma_compatible(p.q, p.qs, p.B, p.Hq, p.Sq) && tma_compatible(p.k, p.ks, p.B, p.Hkv, p.Sk) &&
           tma_compatible(p.v, p.vs, p.B, p.Hkv, p.Sk);
}

CUtensorMapDataType map_type(bool bf16) {
    return bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

bool encode_stored(CUtensorMap* map, const void* ptr, bool bf16, const AttnParams& p, int64_t pitch, int box_rows = kTile) {
    const int64_t strides[4] = {(int64_t)p.Hq * p.Sq * pitch, (int64_t)p.Sq * pitch, pitch, 1};
    return encode_bhsd_map(map, ptr, map_type(bf16), p.Sk, p.Sq, p.Hq, p.B, strides, 64, box_rows);
}

template <typename K>
cudaError_t opt_in(K kernel, int bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

template <bool BF16>
cudaError_t forward_t(const AttnParams& p, cudaStream_t st) {
    const int bytes = smem_scores(p.D);
    cudaError_t e = opt_in(wide_forward<BF16>, bytes);
    if (e != cudaSuccess) return e;
    WideMaps maps;
    const CUtensorMapDataType dt = map_type(BF16);
    if (!encode_bhsd_map(&maps.a, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTile) ||
        !encode_bhsd_map(&maps.b, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTile) ||
        !encode_bhsd_map(&maps.c, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTile))
        return cudaErrorInvalidValue;
    const int64_t grid = (int64_t)((p.Sq + kTile - 1) / kTile) * p.B * p.Hq * 2;
    wide_forward<BF16><<<(unsigned)grid, 256, bytes, st>>>(maps, p);
    return cudaGetLastError();
}

template <int MODE, bool BF16>
cudaError_t scores_t(const AttnParams& p, const Stored& stored, cudaStream_t st) {
    const int bytes = smem_scores(p.D);
    cudaError_t e = opt_in(wide_scores<MODE, BF16>, bytes);
    if (e != cudaSuccess) return e;
    WideMaps maps;
    const CUtensorMapDataType dt = map_type(BF16);
    const bool ok = MODE == 0 ? encode_bhsd_map(&maps.a, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTile) &&
                                    encode_bhsd_map(&maps.b, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTile)
                              : encode_bhsd_map(&maps.a, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, kTile) &&
                                    encode_bhsd_map(&maps.b, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTile);
    if (!ok) return cudaErrorInvalidValue;
    maps.c = maps.a;
    const int64_t grid = (int64_t)((p.Sq + kTile - 1) / kTile) * p.B * p.Hq * stored.parts;
    wide_scores<MODE, BF16><<<(unsigned)grid, 256, bytes, st>>>(maps, p, stored);
    return cudaGetLastError();
}

template <bool BF16>
cudaError_t grad_t(const AttnParams& p, const Stored& stored, cudaStream_t st) {
    const int bytes = smem_grad(p.D);
    cudaError_t e = opt_in(wide_grad<BF16>, bytes);
    if (e != cudaSuccess) return e;
    GradMaps maps;
    const CUtensorMapDataType dt = map_type(BF16);
    const bool ok = encode_stored(&maps.ds, stored.ds_low, BF16, p, stored.pitch) &&
                    encode_stored(&maps.ds64, stored.ds_low, BF16, p, stored.pitch, 64) &&
                    encode_stored(&maps.p64, stored.p_low, BF16, p, stored.pitch, 64) &&
                    encode_bhsd_map(&maps.k64, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, 64) &&
                    encode_bhsd_map(&maps.q64, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, 64) &&
                    encode_bhsd_map(&maps.g64, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, 64);
    if (!ok) return cudaErrorInvalidValue;
    const int64_t n_dq = (int64_t)((p.Sq + kTile - 1) / kTile) * p.B * p.Hq * 2;
    const int64_t n_kv = (int64_t)((p.Sk + kTile - 1) / kTile) * p.B * p.Hkv * 2;
    wide_grad<BF16><<<(unsigned)(n_dq + 2 * n_kv), 192, bytes, st>>>(maps, p, (unsigned)n_dq, (unsigned)n_kv);
    return cudaGetLastError();
}

}  // namespace

bool wide_forward_supported(const AttnParams& p) {
    return wide_common(p) && tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq);
}

cudaError_t launch_wide_forward(const AttnParams& p, bool bf16, cudaStream_t st) {
    return bf16 ? forward_t<true>(p, st) : forward_t<false>(p, st);
}

size_t wide_stored_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk) {
    const int64_t pitch = (Sk + kTile - 1) / kTile * kTile;
    return (size_t)((B * Hq * Sq * pitch * 2 + 255) / 256 * 256);
}

bool wide_backward_supported(const AttnParams& p) {
    return wide_common(p) && tma_compatible(p.dout, p.gs, p.B, p.Hq, p.Sq) &&
           tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq) &&
           tma_compatible(p.dq, p.dqs, p.B, p.Hq, p.Sq) && tma_compatible(p.dk, p.dks, p.B, p.Hkv, p.Sk) &&
           tma_compatible(p.dv, p.dvs, p.B, p.Hkv, p.Sk);
}

cudaError_t launch_wide_delta(const AttnParams& p, bool bf16, cudaStream_t st) {
    const unsigned grid = (unsigned)(((int64_t)p.B * p.Hq * p.Sq + 7) / 8);
    if (bf16) wide_delta<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
    else wide_delta<__half><<<grid, 256, 0, st>>>(p);
    return cudaGetLastError();
}

// step 0: P_low, 1: dS_low, 2: dQ, dK and dV in one launch.  `stored` holds the two matrices back to back.
cudaError_t launch_wide_backward(const AttnParams& p, bool bf16, int step, void* stored, cudaStream_t st) {
    Stored s;
    s.pitch = (p.Sk + kTile - 1) / kTile * kTile;
    // few query tiles: two CTAs share each tile's key range so that the grid covers the GPU
    s.parts = (int64_t)((p.Sq + kTile - 1) / kTile) * p.B * p.Hq < 600 && p.Sk > kTile ? 2 : 1;
    s.p_low = stored;
    s.ds_low = static_cast<char*>(stored) + wide_stored_bytes(p.B, p.Hq, p.Sq, p.Sk);
    switch (step) {
        case 0: return bf16 ? scores_t<0, true>(p, s, st) : scores_t<0, false>(p, s, st);
        case 1: return bf16 ? scores_t<1, true>(p, s, st) : scores_t<1, false>(p, s, st);
        default: return bf16 ? grad_t<true>(p, s, st) : grad_t<false>(p, s, st);
    }
}


}  // namespace kfa
