// Shared pieces of the two backward kernels: tensor maps, mask-table lookup and the work iterator.
#pragma once
#include "kfa_common.cuh"
#include "sm100_ptx.cuh"

namespace kfa {
namespace bwd {

constexpr int kTile = 128;     // owner rows, and rows of a streamed tile
constexpr int kGroups = 2;     // consumer warpgroups
constexpr int kConsumers = 128 * kGroups;
constexpr int kRoleWarp = 4 * kGroups;            // first warp of the role warpgroup: MMA 0, MMA 1, loader, statistics
constexpr int kThreads = kConsumers + 128;

struct Maps {
    CUtensorMap q, k, v, g;  // g = dO
    CUtensorMap dq, dk, dv;  // outputs, stored as whole tiles from shared memory
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
        // Heavy tiles first (late query tiles, early key tiles under a causal mask), tile row by tile row over a
        // chunk of heads: the grid then ends with the light tiles of its last chunk, whereas a head-by-head order
        // starts heavy tiles of the last heads in the final wave.  A chunk holds as many heads as keep the streamed
        // operands (K, V of the chunk's K/V heads, or Q, dO of its query heads) within half of the L2 cache.
        const int64_t nbh = (int64_t)p.B * heads;
        const int64_t streamed = KV ? (int64_t)p.group * p.Sq * p.D * 4 : ((int64_t)p.Sk * p.D * 4 + p.group - 1) / p.group;
        int64_t chunk = (int64_t(64) << 20) / (streamed > 0 ? streamed : 1);
        chunk = chunk < 1 ? 1 : (chunk > nbh ? nbh : chunk);
        if ((int64_t)gridDim.x < KFA_ROW_MAJOR_LIMIT) chunk = nbh;
        const int64_t per_chunk = chunk * nblk, full = nbh / chunk;
        int64_t c = blockIdx.x / per_chunk, within, size;
        if (c < full) {
            within = blockIdx.x - c * per_chunk;
            size = chunk;
        } else {
            c = full;
            within = blockIdx.x - full * per_chunk;
            size = nbh - full * chunk;
        }
        int blk = (int)(within / size);
        if (!KV) blk = nblk - 1 - blk;
        const int64_t bh = c * chunk + within % size;
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

// FP32 gradient rows for block-wise callers (one block of a longer sequence per call): `n` accumulator values
// times `mul` are written to, or added to, `row[0..n)` as 16-byte vectors; channels at or beyond `valid` are skipped.
template <int N>
__device__ __forceinline__ void put_f32(float* row, const uint32_t (&v)[N], int valid, float mul, bool add) {
#pragma unroll
    for (int e = 0; e < N; e += 4) {
        if (e < valid) {
            float4 a = add ? *reinterpret_cast<const float4*>(row + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            a.x += __uint_as_float(v[e]) * mul;
            a.y += __uint_as_float(v[e + 1]) * mul;
            a.z += __uint_as_float(v[e + 2]) * mul;
            a.w += __uint_as_float(v[e + 3]) * mul;
            *reinterpret_cast<float4*>(row + e) = a;
        }
    }
}

}  // namespace bwd
}  // namespace kfa
