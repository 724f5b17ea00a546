// Neighbourhood attention on dense tensor-core tiles: window geometry as tile lists and bit masks.
//
// Tokens are numbered z-major, x fastest.  A query sees the box of keys
// [z0, z0+wz) x [y0, y0+wy) x [x0, x0+wx) with starts clamp(q - w/2, 0, extent - w); a key is seen
// by the box of queries given by the inverse ranges (reference behaviour:
// src/kohakufa_cute/neighborhood_kernels.py:193-212 of the reference project).  Either way the
// visible partners of one token are a box, and inside one (z, y) row of the grid a box is a
// contiguous run of tokens.  The kernels therefore
//   * mark, per CTA, the dense tiles of partner tokens that any of their 128 owner rows can see
//     (a bitmap in shared memory, built once), and walk only those tiles;
//   * give every owner row a bit mask per tile (one bit per partner token) that is applied to the
//     dense score tile, so that exactly the window contributes.
#pragma once
#include "kfa_common.cuh"

namespace kfa {
namespace na {

constexpr int kMapWords = 128;  // up to 4096 tiles per partner sequence

struct Box {
    int zlo, zhi, ylo, yhi, xlo, xhi;  // inclusive coordinate ranges
};

// Keys visible to query `token`.
__host__ __device__ __forceinline__ Box query_box(const AttnParams& p, int token) {
    const int x = token % p.ext[2], t = token / p.ext[2], y = t % p.ext[1], z = t / p.ext[1];
    Box b;
    b.zlo = na_start(z, p.ext[0], p.win[0]);
    b.zhi = b.zlo + p.win[0] - 1;
    b.ylo = na_start(y, p.ext[1], p.win[1]);
    b.yhi = b.ylo + p.win[1] - 1;
    b.xlo = na_start(x, p.ext[2], p.win[2]);
    b.xhi = b.xlo + p.win[2] - 1;
    return b;
}

// Queries that see key `token`.
__host__ __device__ __forceinline__ Box key_box(const AttnParams& p, int token) {
    const int x = token % p.ext[2], t = token / p.ext[2], y = t % p.ext[1], z = t / p.ext[1];
    Box b;
    na_inverse(z, p.ext[0], p.win[0], b.zlo, b.zhi);
    na_inverse(y, p.ext[1], p.win[1], b.ylo, b.yhi);
    na_inverse(x, p.ext[2], p.win[2], b.xlo, b.xhi);
    return b;
}

// Sets, in the shared bitmap, every tile of `width` partner tokens that the box touches.
__device__ __forceinline__ void mark_tiles(const AttnParams& p, const Box& b, int width, uint32_t* bitmap) {
    for (int z = b.zlo; z <= b.zhi; ++z)
        for (int y = b.ylo; y <= b.yhi; ++y) {
            const int row0 = (z * p.ext[1] + y) * p.ext[2];
            const int first = (row0 + b.xlo) / width, last = (row0 + b.xhi) / width;
            for (int t = first; t <= last; ++t) atomicOr(&bitmap[t >> 5], 1u << (t & 31));
        }
}

// The same for a whole warp (every lane calls it; `valid` says whether the lane has a box).  The lanes of a warp are
// consecutive tokens, so their boxes nearly always share the z and y ranges: the warp then marks the tiles of the
// hull of its x ranges once, one (z, y) row per lane, instead of every lane marking every row (32 conflicting
// shared-memory atomics per row).  The hull may mark a tile no lane sees: such a tile contributes nothing.
__device__ __forceinline__ void mark_tiles_warp(const AttnParams& p, const Box& b, bool valid, int width,
                                                uint32_t* bitmap) {
    const unsigned full = 0xffffffffu;
    const unsigned have = __ballot_sync(full, valid);
    if (have == 0) return;
    const int leader = __ffs(have) - 1, lane = threadIdx.x & 31;
    const int zlo = __shfl_sync(full, b.zlo, leader), zhi = __shfl_sync(full, b.zhi, leader);
    const int ylo = __shfl_sync(full, b.ylo, leader), yhi = __shfl_sync(full, b.yhi, leader);
    const bool same = !valid || (b.zlo == zlo && b.zhi == zhi && b.ylo == ylo && b.yhi == yhi);
    if (__all_sync(full, same)) {
        const int xlo = __reduce_min_sync(full, valid ? b.xlo : 0x7fffffff);
        const int xhi = __reduce_max_sync(full, valid ? b.xhi : -1);
        const int ny = yhi - ylo + 1, rows = (zhi - zlo + 1) * ny;
        for (int i = lane; i < rows; i += 32) {
            const int z = zlo + i / ny, y = ylo + i % ny;
            const int row0 = (z * p.ext[1] + y) * p.ext[2];
            const int first = (row0 + xlo) / width, last = (row0 + xhi) / width;
            for (int t = first; t <= last; ++t) atomicOr(&bitmap[t >> 5], 1u << (t & 31));
        }
    } else if (valid) {
        mark_tiles(p, b, width, bitmap);
    }
}

// First marked tile with index >= j, or -1.
__device__ __forceinline__ int next_tile(const uint32_t* bitmap, int j) {
    int w = j >> 5;
    if (w >= kMapWords) return -1;
    uint32_t cur = bitmap[w] & (0xffffffffu << (j & 31));
    while (cur == 0) {
        if (++w >= kMapWords) return -1;
        cur = bitmap[w];
    }
    return (w << 5) + __ffs(cur) - 1;
}

// Bit c of the result (word c / 32) is set when partner token tok0 + c lies in the box.
// `limit` is the length of the partner sequence.  The tile is walked grid row by grid row (two integer
// divisions per call, none per row).
template <int WORDS>
__host__ __device__ __forceinline__ void box_mask(const AttnParams& p, const Box& b, int tok0, int limit, uint32_t (&m)[WORDS]) {
#pragma unroll
    for (int w = 0; w < WORDS; ++w) m[w] = 0;
    const int ex = p.ext[2], ey = p.ext[1];
    const int last = min(tok0 + 32 * WORDS, limit) - 1 - tok0;  // last bit that is a real token
    const int r = tok0 / ex;
    int z = r / ey, y = r - z * ey;
    for (int base = r * ex - tok0; base <= last; base += ex) {  // bit index of the row's x = 0
        if (z >= b.zlo && z <= b.zhi && y >= b.ylo && y <= b.yhi) {
            const int lo = max(base + b.xlo, 0), hi = min(base + b.xhi, 32 * WORDS - 1);
            if (lo <= hi) {
#pragma unroll
                for (int w = 0; w < WORDS; ++w) {
                    const int a = max(lo - 32 * w, 0), e = min(hi - 32 * w, 31);
                    if (a <= e) m[w] |= (0xffffffffu >> (31 - (e - a))) << a;
                }
            }
        }
        if (++y == ey) {
            y = 0;
            ++z;
        }
    }
}

// The same masks for a walk over tiles in increasing order (any tiles may be left out): the cursor stands on the first
// grid row of the box that is not yet wholly behind the walk, so a call touches only the rows of the box that reach
// into its tile (box_mask tests every grid row of the tile and divides twice per call).
struct BoxCursor {
    int next;  // token of (z, y, xlo), the start of the row's run; kDone when the box is used up
    int z, y;
};
constexpr int kDone = 0x3fffffff;

__host__ __device__ __forceinline__ BoxCursor box_cursor(const AttnParams& p, const Box& b) {
    BoxCursor c;
    c.z = b.zlo;
    c.y = b.ylo;
    const bool empty = b.zhi < b.zlo || b.yhi < b.ylo || b.xhi < b.xlo;
    c.next = empty ? kDone : (b.zlo * p.ext[1] + b.ylo) * p.ext[2] + b.xlo;
    return c;
}

__host__ __device__ __forceinline__ void box_cursor_advance(const AttnParams& p, const Box& b, BoxCursor& c) {
    if (c.y < b.yhi) {
        ++c.y;
        c.next += p.ext[2];
    } else if (c.z < b.zhi) {
        ++c.z;
        c.y = b.ylo;
        c.next = (c.z * p.ext[1] + b.ylo) * p.ext[2] + b.xlo;
    } else {
        c.next = kDone;
    }
}

// Bit c of the result (word c / 32) is set when partner token tok0 + c lies in the box.  tok0 must not decrease
// from one call to the next with the same cursor.
template <int WORDS>
__host__ __device__ __forceinline__ void box_mask_walk(const AttnParams& p, const Box& b, BoxCursor& c, int tok0,
                                                       uint32_t (&m)[WORDS]) {
    static_assert(WORDS == 2 || WORDS == 4, "tiles of 64 or 128 partner tokens");
#pragma unroll
    for (int w = 0; w < WORDS; ++w) m[w] = 0;
    const int len = b.xhi - b.xlo;  // run length - 1
    const int end = tok0 + 32 * WORDS;
    while (c.next + len < tok0) box_cursor_advance(p, b, c);
    while (c.next < end) {
        const int lo = (c.next > tok0 ? c.next : tok0) - tok0;
        const int hi = (c.next + len < end ? c.next + len : end - 1) - tok0;
#pragma unroll
        for (int q = 0; q < WORDS / 2; ++q) {  // 64 bits at a time
            const int a = lo - 64 * q > 0 ? lo - 64 * q : 0, e = hi - 64 * q < 63 ? hi - 64 * q : 63;
            if (a <= e) {
                const unsigned long long bits = (~0ull >> (63 - (e - a))) << a;
                m[2 * q] |= static_cast<uint32_t>(bits);
                m[2 * q + 1] |= static_cast<uint32_t>(bits >> 32);
            }
        }
        if (c.next + len >= end) break;  // the run goes on in the next tile: the cursor stays on it
        box_cursor_advance(p, b, c);
    }
}

// -inf where bit `i` of `vis` is clear, the score itself where it is set.
__device__ __forceinline__ uint32_t hide(uint32_t score_bits, uint32_t vis, int i) {
    return (vis & (1u << i)) != 0 ? score_bits : 0xff800000u;
}

}  // namespace na
}  // namespace kfa
