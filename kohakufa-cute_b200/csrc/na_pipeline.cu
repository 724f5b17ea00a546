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
constexpr float kRebase = 8.0f;

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
template <bool BF16>
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

    if (threadIdx.x == 0) {
        sh.abort_word = 0;
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
    if (row_ok) {
        box = query_box(p, row);
        mark_tiles(p, box, kTile, sh.bitmap);
    }
    __syncthreads();
    const uint32_t tmem = sh.tmem_base;
    volatile int* abort_word = &sh.abort_word;

    if (warp == 5) {
        if (lane == 0) {
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
        if (lane == 0) {
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
                if (p.two_term) {
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
        for (int j = next_tile(sh.bitmap, 0); j >= 0 && ok; j = next_tile(sh.bitmap, j + 1)) {
            uint32_t vis[4] = {0, 0, 0, 0};
            if (row_ok) box_mask<4>(p, box, j * kTile, p.Sk, vis);
            ok = mbar_wait(&sh.s_ready, iter & 1, abort_word, 30);
            if (!ok) break;
            tc_fence_after();
            // pass 1: maximum over the visible scores of this tile
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(s_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (vis[c] >> i) & 1u ? __uint_as_float(r[i]) : -INFINITY);
            }
            m_true = fmaxf(m_true, mx);
            const bool rebase = mx > m_used && (m_used == -INFINITY || (mx - m_used) * c2 > kRebase);
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
            // pass 2: weights, their rounding (and its residual), the normaliser
            const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32], hi[16], lo[16];
                tmem_ld32(s_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float pa = ex2((__uint_as_float(r[i]) - m_safe) * c2);
                    float pb = ex2((__uint_as_float(r[i + 1]) - m_safe) * c2);
                    pa = (vis[c] >> i) & 1u ? pa : 0.f;
                    pb = (vis[c] >> (i + 1)) & 1u ? pb : 0.f;
                    sum0 += pa;
                    sum1 += pb;
                    const uint32_t w = pack2<BF16>(pa, pb);
                    hi[i / 2] = w;
                    const float2 back = unpack2<BF16>(w);
                    lo[i / 2] = pack2<BF16>(pa - back.x, pb - back.y);
                }
                tmem_st16(s_addr + c * 16, hi);
                if (p.two_term) tmem_st16(lo_addr + c * 16, lo);
            }
            l += sum0 + sum1;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sh.p_ready);
            ++iter;
        }
        if (iter > 0 && ok) ok = mbar_wait(&sh.s_ready, iter & 1, abort_word, 31);
        if (ok) {
            // tensor-memory loads are warp-collective: every lane takes part, only the stores are per row
            T* orow = reinterpret_cast<T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] +
                      (int64_t)(row_ok ? row : 0) * p.os[2];
            const float den = l > 0.f ? l : 1.f;
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
                        w.x = pack2<BF16>(__uint_as_float(r[i]) / den, __uint_as_float(r[i + 1]) / den);
                        w.y = pack2<BF16>(__uint_as_float(r[i + 2]) / den, __uint_as_float(r[i + 3]) / den);
                        w.z = pack2<BF16>(__uint_as_float(r[i + 4]) / den, __uint_as_float(r[i + 5]) / den);
                        w.w = pack2<BF16>(__uint_as_float(r[i + 6]) / den, __uint_as_float(r[i + 7]) / den);
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
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0) *p.status = 4000 + sh.abort_word;
    if (warp == 4) tmem_dealloc(tmem, 256);
}

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
    cudaError_t e = cudaFuncSetAttribute(na_tc_forward<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    if (e != cudaSuccess) return e;
    NaMaps maps;
    if (!encode_all(&maps, p, BF16, false, kTile)) return cudaErrorInvalidValue;
    const int64_t grid = (int64_t)((p.Sq + kTile - 1) / kTile) * p.B * p.Hq;
    na_tc_forward<BF16><<<(unsigned)grid, 192, kFwdSmem, st>>>(maps, p);
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

}  // namespace kfa
