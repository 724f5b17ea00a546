// Host program: the cursor-based window masks (box_mask_walk) against box_mask and against the definition
// (a partner token is visible when its coordinates lie in the box), for query boxes and key boxes, tiles of
// 64 and 128 tokens, walks over all tiles and over subsets of them.  Prints "ok <cases>" and returns 0, or
// prints the first mismatch and returns 1.  Built and run by tests/test_na_mask_walk_host.py.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "na_tiles.cuh"

using namespace kfa;
using namespace kfa::na;

static bool in_box(const AttnParams& p, const Box& b, int token) {
    const int x = token % p.ext[2], t = token / p.ext[2], y = t % p.ext[1], z = t / p.ext[1];
    return z >= b.zlo && z <= b.zhi && y >= b.ylo && y <= b.yhi && x >= b.xlo && x <= b.xhi;
}

template <int WORDS>
static long check(const AttnParams& p, const Box& b, int total, int stride, int phase) {
    long cases = 0;
    BoxCursor c = box_cursor(p, b);
    int n = 0;
    for (int tok0 = 0; tok0 < total; tok0 += 32 * WORDS, ++n) {
        if (stride > 1 && (n + phase) % stride == 0) continue;  // a tile the walk leaves out
        uint32_t walk[WORDS], direct[WORDS];
        box_mask_walk<WORDS>(p, b, c, tok0, walk);
        box_mask<WORDS>(p, b, tok0, total, direct);
        for (int bit = 0; bit < 32 * WORDS; ++bit) {
            const int token = tok0 + bit;
            const bool want = token < total && in_box(p, b, token);
            const bool got = (walk[bit >> 5] >> (bit & 31)) & 1u;
            const bool old = (direct[bit >> 5] >> (bit & 31)) & 1u;
            if (got != want || old != want) {
                std::printf("mismatch: ext %d %d %d win %d %d %d box z %d..%d y %d..%d x %d..%d tile %d bit %d want %d walk %d direct %d\n",
                            p.ext[0], p.ext[1], p.ext[2], p.win[0], p.win[1], p.win[2], b.zlo, b.zhi, b.ylo, b.yhi,
                            b.xlo, b.xhi, tok0, bit, (int)want, (int)got, (int)old);
                return -1;
            }
        }
        ++cases;
    }
    return cases;
}

int main() {
    const int grids[][6] = {{16, 32, 32, 3, 7, 7}, {1, 64, 64, 1, 7, 7}, {5, 7, 9, 3, 3, 5},   {3, 10, 33, 3, 7, 7},
                            {2, 5, 130, 1, 3, 33}, {4, 4, 4, 4, 4, 4},   {1, 1, 300, 1, 1, 11}, {1, 9, 31, 1, 9, 31},
                            {7, 3, 65, 5, 1, 9},   {1, 20, 64, 1, 5, 13}};
    long cases = 0;
    for (const auto& g : grids) {
        AttnParams p;
        std::memset(&p, 0, sizeof(p));
        p.nd = g[0] == 1 ? 2 : 3;
        for (int i = 0; i < 3; ++i) {
            p.ext[i] = g[i];
            p.win[i] = g[3 + i];
        }
        const int total = g[0] * g[1] * g[2];
        const int step = total > 5000 ? 7 : 1;  // large grids: every seventh token (all residues of x, y, z occur)
        for (int token = 0; token < total; token += step)
            for (int kind = 0; kind < 2; ++kind) {
                const Box b = kind == 0 ? query_box(p, token) : key_box(p, token);
                for (int stride = 1; stride <= 3; ++stride)
                    for (int phase = 0; phase < stride; ++phase) {
                        const long a = check<2>(p, b, total, stride, phase);
                        const long c = check<4>(p, b, total, stride, phase);
                        if (a < 0 || c < 0) return 1;
                        cases += a + c;
                    }
            }
    }
    // an empty box never sets a bit
    {
        AttnParams p;
        std::memset(&p, 0, sizeof(p));
        p.ext[0] = 2, p.ext[1] = 8, p.ext[2] = 40;
        p.win[0] = 1, p.win[1] = 3, p.win[2] = 5;
        const Box b = {0, -1, 0, -1, 0, -1};
        BoxCursor c = box_cursor(p, b);
        for (int tok0 = 0; tok0 < 640; tok0 += 128) {
            uint32_t m[4];
            box_mask_walk<4>(p, b, c, tok0, m);
            if (m[0] | m[1] | m[2] | m[3]) {
                std::printf("mismatch: empty box set a bit in tile %d\n", tok0);
                return 1;
            }
            ++cases;
        }
    }
    std::printf("ok %ld\n", cases);
    return 0;
}
