// Forward for a handful of query rows against a long key sequence (token-by-token decoding with a key/value
// cache): at most eight query rows per K/V head (query positions x grouped-query heads), no mask, not causal.
//
// Such a call reads every key and value once and does almost no arithmetic, so its floor is the HBM time of K and
// V; a 128-row tensor-core tile would spend 127 rows on nothing and put one CTA per head on the GPU.  Here the keys
// of one (batch, K/V head) are split over CTAs (`splits` key ranges) and over the eight warps of a CTA (blocks of
// eight keys, round robin); a warp's lanes split the channels, so a key or value row is one coalesced load of the
// warp, and the eight loads of a block are issued before anything is added up.  Every warp keeps a running
// (maximum, sum, accumulator) per query row, the warps of a CTA and then the CTAs of a head are merged with the
// (maximum, sum) arithmetic of the reference's split forward (src/kohakufa_cute/split_forward.py:219-245 of the
// reference project).  The arithmetic contract is the operator's: unscaled scores, the maximum subtracted before
// the multiplication by |scale| log2e, the sum over unrounded probabilities, the product with probabilities
// rounded once to the 16-bit type, one division and one rounding at the end.
#include "kfa_common.cuh"
#include "launchers.h"

namespace kfa {
namespace {

constexpr int kWarps = 8;       // warps per CTA
constexpr int kBlockKeys = 8;   // keys a warp loads before it adds anything up

struct DecodeParams {
    const void* q;
    const void* k;
    const void* v;
    int64_t qs[4], ks[4], vs[4];
    int B, Hq, Hkv, Sq, Sk, group, rows;  // rows = Sq * group: query rows per K/V head
    int splits, keys_per_split;
    float c2, sign;
    float* part_out;  // [splits, B * Hkv * rows, D] unnormalised accumulators relative to part_max
    float* part_max;  // [splits, B * Hkv * rows]
    float* part_sum;  // [splits, B * Hkv * rows]
};

// Element `c` of a row piece held as packed 16-bit pairs (register arithmetic only: no detour through memory).
template <typename T>
__device__ __forceinline__ float element(const uint32_t* words, int c);
template <>
__device__ __forceinline__ float element<__nv_bfloat16>(const uint32_t* words, int c) {
    const uint32_t w = words[c >> 1];
    return __uint_as_float((c & 1) ? (w & 0xffff0000u) : (w << 16));
}
template <>
__device__ __forceinline__ float element<__half>(const uint32_t* words, int c) {
    const uint32_t w = words[c >> 1];
    return __half2float(__ushort_as_half(static_cast<unsigned short>((c & 1) ? (w >> 16) : (w & 0xffffu))));
}

// This lane's piece of a key or value row: kVec channels as kVec / 2 words.
template <int kVec>
__device__ __forceinline__ void load_piece(const void* src, uint32_t (&words)[kVec / 2]) {
    if (kVec == 4) {
        const uint2 t = *reinterpret_cast<const uint2*>(src);
        words[0] = t.x;
        words[kVec / 2 - 1] = t.y;
    } else {
        words[0] = *reinterpret_cast<const uint32_t*>(src);
    }
}

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One (batch, K/V head, key range) per CTA.  D = 64 or 128 channels, R = query rows rounded up to a power of two.
template <typename T, int D, int R>
__global__ void __launch_bounds__(kWarps * 32) decode_partial(DecodeParams p) {
    constexpr int kVec = D / 32;  // channels per lane
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x % p.splits;
    const int64_t unit = blockIdx.x / p.splits;  // (batch, K/V head)
    const int kvh = (int)(unit % p.Hkv), b = (int)(unit / p.Hkv);

    float qreg[R][kVec];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int g = r / p.Sq, sq = r - g * p.Sq;
        const T* qrow = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.qs[0] + (int64_t)(kvh * p.group + g) * p.qs[1] +
                        (int64_t)sq * p.qs[2] + lane * kVec;
#pragma unroll
        for (int c = 0; c < kVec; ++c) qreg[r][c] = r < p.rows ? to_float<T>(qrow[c]) * p.sign : 0.f;
    }
    const T* kbase = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.ks[0] + (int64_t)kvh * p.ks[1] + lane * kVec;
    const T* vbase = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.vs[0] + (int64_t)kvh * p.vs[1] + lane * kVec;
    const int key_begin = split * p.keys_per_split, key_end = min(p.Sk, key_begin + p.keys_per_split);

    // Scores of a block: N = R x 8 partial dot products per lane (index row * 8 + key).  They are summed over the
    // lanes by a transposing reduction (each step a lane keeps one half of its values and adds the partner's copy
    // of that half: N - 1 shuffles instead of 5 N), after which score `idx` is owned by lane idx / CF (N >= 32) or
    // by the REP lanes idx * REP ... (N < 32).  The lanes that own the scores of one query row are an aligned group
    // of G = 32 / R lanes; the softmax of the block is done once, by the owners, and the rounded probabilities and
    // the rows' rescale factors are then broadcast to all lanes for the product with V.
    constexpr int N = R * kBlockKeys;
    constexpr int CF = N >= 32 ? N / 32 : 1;
    constexpr int REP = N >= 32 ? 1 : 32 / N;
    constexpr int G = 32 / R;
    const int my_row = lane / G;
    float m_run = -INFINITY, l_run = 0.f;  // running maximum and sum of this lane's row (equal within its group)
    float o[R][kVec];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < kVec; ++c) o[r][c] = 0.f;
    for (int base = key_begin + warp * kBlockKeys; base < key_end; base += kWarps * kBlockKeys) {
        uint32_t kv[kBlockKeys][kVec / 2], vv[kBlockKeys][kVec / 2];
#pragma unroll
        for (int j = 0; j < kBlockKeys; ++j) {
            const int key = min(base + j, key_end - 1);  // rows beyond the range repeat the last one and are hidden below
            load_piece<kVec>(kbase + (int64_t)key * p.ks[2], kv[j]);
            load_piece<kVec>(vbase + (int64_t)key * p.vs[2], vv[j]);
        }
        float s[N];
#pragma unroll
        for (int j = 0; j < kBlockKeys; ++j) {
            float kf[kVec];
#pragma unroll
            for (int c = 0; c < kVec; ++c) kf[c] = element<T>(kv[j], c);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float sum = 0.f;
#pragma unroll
                for (int c = 0; c < kVec; ++c) sum = fmaf(qreg[r][c], kf[c], sum);
                s[r * kBlockKeys + j] = sum;
            }
        }
#pragma unroll
        for (int step = 0; step < 5; ++step) {
            const int off = 16 >> step;
            constexpr int kFull = N;
            const int count = (kFull >> step) > 1 ? (kFull >> step) : 1;  // values held before this step
            if (count > 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < N / 2; ++i) {
                    if (i < count / 2) {
                        const float send = upper ? s[i] : s[i + count / 2];
                        const float keep = upper ? s[i + count / 2] : s[i];
                        s[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                }
            } else {
                s[0] += __shfl_xor_sync(0xffffffffu, s[0], off);
            }
        }
        // the owners' softmax of the block
        float mine[CF], mx = -INFINITY;
#pragma unroll
        for (int t = 0; t < CF; ++t) {
            const int idx = N >= 32 ? lane * CF + t : lane / REP;
            mine[t] = base + (idx % kBlockKeys) < key_end ? s[t] : -INFINITY;
            mx = fmaxf(mx, mine[t]);
        }
#pragma unroll
        for (int off = G / 2; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float mn = fmaxf(m_run, mx);  // finite: the first key of a block is always inside the range
        const float alpha = m_run == -INFINITY ? 0.f : ex2f((m_run - mn) * p.c2);
        float low[CF], sum = 0.f;
#pragma unroll
        for (int t = 0; t < CF; ++t) {
            const float pj = ex2f((mine[t] - mn) * p.c2);
            sum += pj;
            low[t] = round_low<T>(pj);
        }
        if (REP > 1 && lane % REP != 0) sum = 0.f;  // a score owned by several lanes is counted once
#pragma unroll
        for (int off = G / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        m_run = mn;
        l_run = l_run * alpha + sum;
        // every lane: its channels of O for every row
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float a = __shfl_sync(0xffffffffu, alpha, r * G);
#pragma unroll
            for (int c = 0; c < kVec; ++c) o[r][c] *= a;
        }
#pragma unroll
        for (int j = 0; j < kBlockKeys; ++j) {
            float vf[kVec];
#pragma unroll
            for (int c = 0; c < kVec; ++c) vf[c] = element<T>(vv[j], c);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int idx = r * kBlockKeys + j;
                const float pl = __shfl_sync(0xffffffffu, low[idx % CF], N >= 32 ? idx / CF : idx * REP);
#pragma unroll
                for (int c = 0; c < kVec; ++c) o[r][c] = fmaf(pl, vf[c], o[r][c]);
            }
        }
    }

    // the warps of the CTA, merged in a fixed order
    __shared__ float sm_m[kWarps][R], sm_l[kWarps][R];
    __shared__ float sm_o[kWarps][R][D];
    if (lane % G == 0) {
        sm_m[warp][my_row] = m_run;
        sm_l[warp][my_row] = l_run;
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < kVec; ++c) sm_o[warp][r][lane * kVec + c] = o[r][c];
    __syncthreads();
    const int64_t all_rows = (int64_t)p.B * p.Hkv * p.rows;
    for (int idx = threadIdx.x; idx < p.rows * D; idx += kWarps * 32) {
        const int r = idx / D, d = idx - r * D;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, sm_m[w][r]);
        float sum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float weight = sm_m[w][r] == -INFINITY ? 0.f : ex2f((sm_m[w][r] - mx) * p.c2);
            sum += sm_l[w][r] * weight;
            acc += sm_o[w][r][d] * weight;
        }
        const int64_t row = unit * p.rows + r;
        p.part_out[((int64_t)split * all_rows + row) * D + d] = acc;
        if (d == 0) {
            p.part_max[(int64_t)split * all_rows + row] = mx;
            p.part_sum[(int64_t)split * all_rows + row] = sum;
        }
    }
}

// One CTA per query row, one thread per channel: the key ranges merged, one division, one rounding, the operator's
// statistics.  The weights of the ranges are formed once (first warp) and shared; a thread's loads over the ranges
// are independent, so the call costs one memory latency, not one per range.
constexpr int kMaxSplits = 64;

template <typename T>
__global__ void __launch_bounds__(128) decode_merge(DecodeParams p, int D, T* out, int64_t o_b, int64_t o_h, int64_t o_s,
                                                    float* maximum, float* logsum) {
    __shared__ float weight[kMaxSplits];
    __shared__ float total_shared, max_shared;
    const int64_t all_rows = (int64_t)p.B * p.Hkv * p.rows;
    const int64_t row = blockIdx.x;
    const int r = (int)(row % p.rows);
    const int64_t unit = row / p.rows;
    const int kvh = (int)(unit % p.Hkv), b = (int)(unit / p.Hkv);
    const int g = r / p.Sq, sq = r - g * p.Sq, hq = kvh * p.group + g;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float m0 = lane < p.splits ? p.part_max[(int64_t)lane * all_rows + row] : -INFINITY;
        float m1 = lane + 32 < p.splits ? p.part_max[(int64_t)(lane + 32) * all_rows + row] : -INFINITY;
        const float mx = warp_max(fmaxf(m0, m1));
        const float w0 = m0 == -INFINITY ? 0.f : ex2f((m0 - mx) * p.c2);
        const float w1 = m1 == -INFINITY ? 0.f : ex2f((m1 - mx) * p.c2);
        float sum = 0.f;
        if (lane < p.splits) sum += p.part_sum[(int64_t)lane * all_rows + row] * w0;
        if (lane + 32 < p.splits) sum += p.part_sum[(int64_t)(lane + 32) * all_rows + row] * w1;
        sum = warp_sum(sum);
        weight[lane] = w0;
        weight[lane + 32] = w1;
        if (lane == 0) {
            total_shared = sum;
            max_shared = mx;
        }
    }
    __syncthreads();
    const float total = total_shared;
    const float inv = total > 0.f ? 1.f / total : 0.f;
    const int d = threadIdx.x;
    if (d < D) {
        float part[kMaxSplits], acc = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxSplits; ++i)  // every load is issued before the first is used
            part[i] = i < p.splits ? p.part_out[((int64_t)i * all_rows + row) * D + d] : 0.f;
#pragma unroll
        for (int i = 0; i < kMaxSplits; ++i) acc = fmaf(part[i], i < p.splits ? weight[i] : 0.f, acc);
        out[(int64_t)b * o_b + (int64_t)hq * o_h + (int64_t)sq * o_s + d] = from_float<T>(acc * inv);
    }
    if (threadIdx.x == 0 && maximum) {
        const int64_t si = ((int64_t)b * p.Hq + hq) * p.Sq + sq;
        maximum[si] = total > 0.f ? max_shared : -INFINITY;
        logsum[si] = total > 0.f ? log2f(total) : 0.f;
    }
}

// Key ranges per (batch, K/V head): about four CTAs per SM over the whole call, at least 256 keys each (several
// short CTAs per slot balance better than one wave of long ones: measured).
int splits_for(int64_t units, int64_t Sk) {
    int64_t want = (4 * 148 + units - 1) / units;
    const int64_t most = Sk / 256 > 0 ? Sk / 256 : 1;
    want = want < 1 ? 1 : (want > most ? most : want);
    return (int)(want > kMaxSplits ? kMaxSplits : want);
}

template <typename T, int D>
cudaError_t launch_partial(const DecodeParams& p, cudaStream_t st) {
    const unsigned grid = (unsigned)((int64_t)p.B * p.Hkv * p.splits);
    if (p.rows <= 1) decode_partial<T, D, 1><<<grid, kWarps * 32, 0, st>>>(p);
    else if (p.rows <= 2) decode_partial<T, D, 2><<<grid, kWarps * 32, 0, st>>>(p);
    else if (p.rows <= 4) decode_partial<T, D, 4><<<grid, kWarps * 32, 0, st>>>(p);
    else decode_partial<T, D, 8><<<grid, kWarps * 32, 0, st>>>(p);
    return cudaGetLastError();
}

}  // namespace

bool decode_forward_supported(const AttnParams& p) {
    if (p.D != 64 && p.D != 128) return false;
    if (p.nd != 0 || p.has_mask || p.causal || p.scale == 0.f) return false;
    if ((int64_t)p.Sq * p.group > 8 || p.Sk < 512) return false;
    auto rows_ok = [](const void* ptr, const int64_t* st) {
        return st[3] == 1 && reinterpret_cast<uintptr_t>(ptr) % 8 == 0 && st[0] % 4 == 0 && st[1] % 4 == 0 && st[2] % 4 == 0;
    };
    return rows_ok(p.q, p.qs) && rows_ok(p.k, p.ks) && rows_ok(p.v, p.vs) && p.os[3] == 1;
}

size_t decode_forward_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Sk, int64_t D) {
    if (Hkv <= 0) return 0;
    const int64_t rows = B * Hq * Sq;
    const int splits = splits_for(B * Hkv, Sk);
    return (size_t)(splits * rows * (D + 2)) * sizeof(float);
}

cudaError_t launch_decode_forward(const AttnParams& p, bool bf16, void* workspace, int* launches, cudaStream_t st) {
    DecodeParams d;
    d.q = p.q;
    d.k = p.k;
    d.v = p.v;
    for (int i = 0; i < 4; ++i) {
        d.qs[i] = p.qs[i];
        d.ks[i] = p.ks[i];
        d.vs[i] = p.vs[i];
    }
    d.B = p.B;
    d.Hq = p.Hq;
    d.Hkv = p.Hkv;
    d.Sq = p.Sq;
    d.Sk = p.Sk;
    d.group = p.group;
    d.rows = p.Sq * p.group;
    d.splits = splits_for((int64_t)p.B * p.Hkv, p.Sk);
    d.keys_per_split = ((p.Sk + d.splits - 1) / d.splits + 63) / 64 * 64;
    d.c2 = fabsf(p.scale) * kLog2e;
    d.sign = p.scale < 0.f ? -1.f : 1.f;
    const int64_t all_rows = (int64_t)p.B * p.Hkv * d.rows;
    d.part_out = static_cast<float*>(workspace);
    d.part_max = d.part_out + (int64_t)d.splits * all_rows * p.D;
    d.part_sum = d.part_max + (int64_t)d.splits * all_rows;
    cudaError_t e;
    if (p.D == 128) e = bf16 ? launch_partial<__nv_bfloat16, 128>(d, st) : launch_partial<__half, 128>(d, st);
    else e = bf16 ? launch_partial<__nv_bfloat16, 64>(d, st) : launch_partial<__half, 64>(d, st);
    if (e != cudaSuccess) return e;
    const unsigned grid = (unsigned)all_rows;
    if (bf16)
        decode_merge<__nv_bfloat16><<<grid, 128, 0, st>>>(d, p.D, static_cast<__nv_bfloat16*>(p.out), p.os[0], p.os[1],
                                                          p.os[2], p.maximum, p.logsum);
    else
        decode_merge<__half><<<grid, 128, 0, st>>>(d, p.D, static_cast<__half*>(p.out), p.os[0], p.os[1], p.os[2],
                                                   p.maximum, p.logsum);
    if (launches) *launches = 2;
    return cudaGetLastError();
}

}  // namespace kfa
