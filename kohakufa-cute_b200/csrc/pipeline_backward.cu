// Attention backward on the tensor-memory pipeline: the two gradient kernels, support predicate and launchers.
// The roles are described in pipeline_backward_{kv,q}_roles.cuh / pipeline_backward_{kv,q}_consumer.cuh.
#include <type_traits>

#include "kfa_common.cuh"
#include "launchers.h"
#include "pipeline_backward_kv_consumer.cuh"
#include "pipeline_backward_q_consumer.cuh"
#include "tensor_map.h"

#include <atomic>

namespace kfa {

int pipeline_forward_variants();
void pipeline_forward_forget();

namespace {


using namespace bwd;

// Key/value-gradient kernel.  MASKED = false is the instantiation for calls without a mask: the flag is
// cleared at compile time, so none of the mask-table or mask-element code survives in it.
template <int D, bool BF16, bool MASKED>
__global__ void __launch_bounds__(kThreads, 1) pipeline_backward_kv(const __grid_constant__ Maps maps, AttnParams p) {
    if (!MASKED) p.has_mask = 0;
    using C = kv::Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_owner = smem;                           // K and V of the owner tile
    uint8_t* s_ring = smem + 2 * C::kTileBytes;        // ring of streamed (Q, dO) pairs
    uint8_t* s_stat = s_ring + C::kPairs * 2 * C::kTileBytes;   // operand tiles of the statistics step
    kv::Shared& sh = *reinterpret_cast<kv::Shared*>(s_stat + C::kStatsBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    Work<true> w;
    w.init(p);

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.owner_full, 1);
        for (int s = 0; s < C::kPairs; ++s) {
            mbar_init(&sh.pair_full[s], 1);
            mbar_init(&sh.pair_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sh.stats_full[s], 1);
            mbar_init(&sh.stats_empty[s], 1);
        }
        mbar_init(&sh.s_ready, 1);
        mbar_init(&sh.dp_ready, 1);
        mbar_init(&sh.p_done, kConsumers);
        mbar_init(&sh.ds_done, kConsumers);
        mbar_init(&sh.final_done, 1);
        mbar_init(&sh.out_staged, kConsumers);
        mbar_fence_init();
    }
    if (warp == kRoleWarp) {
        tmem_alloc(&sh.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    const bool dead = sh.abort_word != 0;  // set before the barrier above: skip straight to the tear-down

    // Registers move from the role warpgroup to the two consumer warpgroups.
    if (dead) {
    } else if (warp >= kRoleWarp) {
        reg_dealloc<96>();
        if (warp == kRoleWarp) {
            if (elect_one()) kv::mma_role<D, BF16>(p, w, sh, tmem, s_owner, s_ring, s_stat);
        } else if (warp == kRoleWarp + 1) {
        } else if (warp == kRoleWarp + 2) {
            if (elect_one()) kv::loader_role<D>(maps, p, w, sh, s_owner, s_ring);
        } else {
            kv::stats_role(p, w, sh, s_stat, lane);
        }
    } else {
        reg_alloc<200>();
        kv::consumer_role<D, BF16>(maps, p, w, sh, tmem, s_owner, warp >> 2, warp, lane);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 2000 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == kRoleWarp) tmem_dealloc(tmem, 512);
}

// Query-gradient kernel.
template <int D, bool BF16, bool MASKED>
__global__ void __launch_bounds__(kThreads, 1) pipeline_backward_q(const __grid_constant__ Maps maps, AttnParams p) {
    if (!MASKED) p.has_mask = 0;
    using C = q::Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_owner = smem;                                       // Q and dO of the owner tile
    uint8_t* s_keys = smem + 2 * C::kTileBytes;                    // ring of K tiles
    uint8_t* s_values = s_keys + C::kKeySlots * C::kTileBytes;     // ring of V tiles
    q::Shared& sh = *reinterpret_cast<q::Shared*>(s_values + C::kValueSlots * C::kTileBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    Work<false> w;
    w.init(p);

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.owner_full, 1);
        for (int s = 0; s < q::kMaxSlots; ++s) {
            mbar_init(&sh.k_full[s], 1);
            mbar_init(&sh.k_empty[s], 2);  // the S product and the dQ product both read a K tile
            mbar_init(&sh.v_full[s], 1);
            mbar_init(&sh.v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sh.s_ready[s], 1);
            mbar_init(&sh.s_free[s], 1);
        }
        mbar_init(&sh.dp_ready, 1);
        mbar_init(&sh.dp_free, kConsumers);
        mbar_init(&sh.ds_done, kConsumers);
        mbar_init(&sh.final_done, 2);
        mbar_init(&sh.out_staged, kConsumers);
        mbar_fence_init();
    }
    if (warp == kRoleWarp) {
        tmem_alloc(&sh.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;
    const bool dead = sh.abort_word != 0;

    if (dead) {
    } else if (warp >= kRoleWarp) {
        reg_dealloc<96>();
        if (warp <= kRoleWarp + 1) {
            if (elect_one()) q::mma_role<D, BF16>(p, w, sh, tmem, s_owner, s_keys, s_values, warp - kRoleWarp);
        } else if (warp == kRoleWarp + 2) {
            if (elect_one()) q::loader_role<D>(maps, p, w, sh, s_owner, s_keys, s_values);
        }
    } else {
        reg_alloc<200>();
        q::consumer_role<D, BF16>(maps, p, w, sh, tmem, s_owner, warp >> 2, warp, lane);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {
        *p.status = 2000 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;
    }
    if (warp == kRoleWarp) tmem_dealloc(tmem, 512);
}

// delta[row] = sum_d O * dO with coalesced 16-byte loads: D/8 threads per row (D = 64 or 128 covers the
// head's p.D channels; the threads beyond them add zero), kDeltaBatch rows per thread so that each thread has
// 2 x kDeltaBatch independent loads in flight before the first use.
constexpr int kDeltaBatch = 2;

template <typename T, int D>
__global__ void __launch_bounds__(256) output_delta_rows(AttnParams p) {
    constexpr int kLanes = D / 8, kRows = 256 / kLanes;
    const int sub = threadIdx.x % kLanes;
    const int64_t first = (int64_t)blockIdx.x * (kRows * kDeltaBatch) + threadIdx.x / kLanes;
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    const bool channels = sub * 8 < p.D;
    uint4 ov[kDeltaBatch], gv[kDeltaBatch];
#pragma unroll
    for (int j = 0; j < kDeltaBatch; ++j) {
        const int64_t row_id = first + j * kRows;
        ov[j] = gv[j] = make_uint4(0, 0, 0, 0);
        if (row_id < rows && channels) {
            int r, h, b;
            split_row(row_id, p.Sq, p.Hq, r, h, b);
            const T* o = reinterpret_cast<const T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] +
                         (int64_t)r * p.os[2] + sub * 8;
            const T* g = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1] +
                         (int64_t)r * p.gs[2] + sub * 8;
            ov[j] = *reinterpret_cast<const uint4*>(o);
            gv[j] = *reinterpret_cast<const uint4*>(g);
        }
    }
#pragma unroll
    for (int j = 0; j < kDeltaBatch; ++j) {
        const T* oe = reinterpret_cast<const T*>(&ov[j]);
        const T* ge = reinterpret_cast<const T*>(&gv[j]);
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) sum = fmaf(to_float<T>(oe[e]), to_float<T>(ge[e]), sum);
#pragma unroll
        for (int o = kLanes / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const int64_t row_id = first + j * kRows;
        if (sub == 0 && row_id < rows) p.delta[row_id] = sum;
    }
}

std::atomic<int> g_configured{0};

template <int D, bool BF16, bool KV>
cudaError_t launch_t(const AttnParams& p, cudaStream_t st) {
    constexpr int kSmem = KV ? kv::Cfg<D>::kSmemBytes : q::Cfg<D>::kSmemBytes;
    using Kernel = void (*)(const Maps, AttnParams);
    Kernel kernel;
    if (KV) kernel = p.has_mask ? pipeline_backward_kv<D, BF16, true> : pipeline_backward_kv<D, BF16, false>;
    else kernel = p.has_mask ? pipeline_backward_q<D, BF16, true> : pipeline_backward_q<D, BF16, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return e;
    constexpr int variant = (D == 128 ? 0 : 4) + (BF16 ? 0 : 2) + (KV ? 1 : 0);
    if (!(g_configured.load() & (1 << variant))) g_configured |= 1 << variant;
    Maps maps;
    const CUtensorMapDataType dt = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!encode_bhsd_map(&maps.q, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTile)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.k, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTile)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.v, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTile)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.g, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, kTile)) return cudaErrorInvalidValue;
    if (p.grad_f32) {
        maps.dq = maps.dk = maps.dv = maps.q;  // not used: FP32 gradients are written with plain stores
    } else if (KV) {
        if (!encode_bhsd_map(&maps.dk, p.dk, dt, p.D, p.Sk, p.Hkv, p.B, p.dks, 64, kTile)) return cudaErrorInvalidValue;
        if (!encode_bhsd_map(&maps.dv, p.dv, dt, p.D, p.Sk, p.Hkv, p.B, p.dvs, 64, kTile)) return cudaErrorInvalidValue;
        maps.dq = maps.dk;
    } else {
        if (!encode_bhsd_map(&maps.dq, p.dq, dt, p.D, p.Sq, p.Hq, p.B, p.dqs, 64, kTile)) return cudaErrorInvalidValue;
        maps.dk = maps.dv = maps.dq;
    }
    const int64_t tiles = KV ? (p.Sk + kTile - 1) / kTile : (p.Sq + kTile - 1) / kTile;
    const int64_t grid = tiles * p.B * (KV ? p.Hkv : p.Hq);
    kernel<<<(unsigned)grid, kThreads, kSmem, st>>>(maps, p);
    return cudaGetLastError();
}

}  // namespace

bool pipeline_backward_supported(const AttnParams& p, bool bf16) {
    (void)bf16;
    if (p.D < 8 || p.D > 128 || p.D % 8 != 0) return false;  // run as 64 or 128 channels, zero-filled by the loads
    if (p.nd != 0 || p.scale == 0.f) return false;
    if (p.Sk < 2) return false;  // a single key has P = 1: the general kernels keep dS exactly zero there
    if (!tma_compatible(p.q, p.qs, p.B, p.Hq, p.Sq) || !tma_compatible(p.k, p.ks, p.B, p.Hkv, p.Sk) ||
        !tma_compatible(p.v, p.vs, p.B, p.Hkv, p.Sk) || !tma_compatible(p.dout, p.gs, p.B, p.Hq, p.Sq))
        return false;
    if (!tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq)) return false;  // 16-byte vector loads per row (delta)
    if (p.grad_f32) {  // FP32 rows read and written as 16-byte vectors
        auto rows_ok = [](const void* ptr, const int64_t* st) {
            return st[3] == 1 && reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && st[0] % 4 == 0 && st[1] % 4 == 0 &&
                   st[2] % 4 == 0;
        };
        return rows_ok(p.dq, p.dqs) && rows_ok(p.dk, p.dks) && rows_ok(p.dv, p.dvs);
    }
    return tma_compatible(p.dq, p.dqs, p.B, p.Hq, p.Sq) && tma_compatible(p.dk, p.dks, p.B, p.Hkv, p.Sk) &&
           tma_compatible(p.dv, p.dvs, p.B, p.Hkv, p.Sk);
}

// which: 0 = query-gradient kernel, 1 = key/value-gradient kernel
cudaError_t launch_pipeline_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st) {
    if (p.D > 64) {
        if (which == 0) return bf16 ? launch_t<128, true, false>(p, st) : launch_t<128, false, false>(p, st);
        return bf16 ? launch_t<128, true, true>(p, st) : launch_t<128, false, true>(p, st);
    }
    if (which == 0) return bf16 ? launch_t<64, true, false>(p, st) : launch_t<64, false, false>(p, st);
    return bf16 ? launch_t<64, true, true>(p, st) : launch_t<64, false, true>(p, st);
}

// delta for the pipeline family (rows are 16-byte aligned and channel-contiguous there)
cudaError_t launch_pipeline_delta(const AttnParams& p, bool bf16, cudaStream_t st) {
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    if (p.D > 64) {
        const unsigned grid = (unsigned)((rows + 16 * kDeltaBatch - 1) / (16 * kDeltaBatch));
        if (bf16) output_delta_rows<__nv_bfloat16, 128><<<grid, 256, 0, st>>>(p);
        else output_delta_rows<__half, 128><<<grid, 256, 0, st>>>(p);
    } else {
        const unsigned grid = (unsigned)((rows + 32 * kDeltaBatch - 1) / (32 * kDeltaBatch));
        if (bf16) output_delta_rows<__nv_bfloat16, 64><<<grid, 256, 0, st>>>(p);
        else output_delta_rows<__half, 64><<<grid, 256, 0, st>>>(p);
    }
    return cudaGetLastError();
}

KFA_PHASE_EXPORT(kfa_debug_phases_bwd)

int pipeline_configured_variants() { return pipeline_forward_variants() + __builtin_popcount(g_configured.load()); }
void pipeline_forget_variants() {
    pipeline_forward_forget();
    g_configured = 0;
}

}  // namespace kfa
