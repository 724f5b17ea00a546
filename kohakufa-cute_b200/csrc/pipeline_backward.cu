// Attention backward on the tensor-memory pipeline: kernel, support predicate and launchers.
// The roles are described in pipeline_backward_roles.cuh / pipeline_backward_consumer.cuh.
#include <type_traits>

#include "kfa_common.cuh"
#include "launchers.h"
#include "pipeline_backward_consumer.cuh"
#include "tensor_map.h"

#include <atomic>

namespace kfa {

int pipeline_forward_variants();
void pipeline_forward_forget();

namespace {

using namespace bwd;

// MASKED = false is the instantiation for calls without a mask: the flag is cleared at compile time, so
// none of the mask-table or mask-element code survives in it.
template <int D, bool BF16, bool KV, bool MASKED>
__global__ void __launch_bounds__(kThreads, 1) pipeline_backward(const __grid_constant__ Maps maps, AttnParams p) {
    if (!MASKED) p.has_mask = 0;
    using C = Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_owner = smem;                           // owner operands 1 and 2
    uint8_t* s_ring = smem + 2 * C::kTileBytes;        // ring of streamed operand pairs
    float* s_stats = reinterpret_cast<float*>(s_ring + C::kPairs * 2 * C::kTileBytes);
    Shared& sh = *reinterpret_cast<Shared*>(reinterpret_cast<uint8_t*>(s_stats) + C::kStatsBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    Work<KV> w;
    w.init(p);

    if (threadIdx.x == 0) {
        sh.abort_word = *reinterpret_cast<volatile int*>(p.abort_flag) != 0 ? 90 : 0;  // 90: an earlier CTA gave up
        mbar_init(&sh.owner_full, 1);
        for (int s = 0; s < C::kPairs; ++s) {
            mbar_init(&sh.pair_full[s], 1);
            mbar_init(&sh.pair_empty[s], 2);  // both MMA issuers release a slot
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sh.sdp_ready[s], 2);   // S from issuer 0, dP from issuer 1
            mbar_init(&sh.done[s], kConsumers);
            mbar_init(&sh.stats_full[s], 1);
            mbar_init(&sh.stats_empty[s], kConsumers);
        }
        mbar_init(&sh.final_done, 2);
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

    // With two consumer warpgroups (384 threads, 168 registers at launch) registers move from the role
    // warpgroup to the consumers; with four (640 threads, 96 registers) every role fits as launched.
    if (dead) {
    } else if (warp >= kRoleWarp) {
        if (kGroups == 2) reg_dealloc<96>();
        if (warp <= kRoleWarp + 1) {
            if (lane == 0) mma_role<D, BF16, KV>(p, w, sh, tmem, s_owner, s_ring, warp - kRoleWarp);
        } else if (warp == kRoleWarp + 2) {
            if (lane == 0) loader_role<D, KV>(maps, p, w, sh, s_owner, s_ring);
        } else {
            if (KV) stats_role<KV>(p, w, sh, s_stats, lane);
        }
    } else {
        if (kGroups == 2) reg_alloc<200>();
        consumer_role<D, BF16, KV>(p, w, sh, tmem, s_stats, warp >> 2, warp, lane);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sh.abort_word != 0 && sh.abort_word != 90) {  // 90 = skipped: already reported
        *p.status = 2000 + sh.abort_word;
        *reinterpret_cast<volatile int*>(p.abort_flag) = 1;  // the remaining CTAs of this and later launches skip their work
    }
    if (warp == kRoleWarp) tmem_dealloc(tmem, 512);
}

// delta[row] = sum_d O * dO with coalesced 16-byte loads: D/8 threads per row.
template <typename T, int D>
__global__ void __launch_bounds__(256) output_delta_rows(AttnParams p) {
    constexpr int kLanes = D / 8, kRows = 256 / kLanes;
    const int sub = threadIdx.x % kLanes;
    const int64_t row_id = (int64_t)blockIdx.x * kRows + threadIdx.x / kLanes;
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    float sum = 0.f;
    if (row_id < rows) {
        const int r = (int)(row_id % p.Sq);
        const int h = (int)((row_id / p.Sq) % p.Hq);
        const int b = (int)(row_id / ((int64_t)p.Sq * p.Hq));
        const T* o = reinterpret_cast<const T*>(p.out) + (int64_t)b * p.os[0] + (int64_t)h * p.os[1] +
                     (int64_t)r * p.os[2] + sub * 8;
        const T* g = reinterpret_cast<const T*>(p.dout) + (int64_t)b * p.gs[0] + (int64_t)h * p.gs[1] +
                     (int64_t)r * p.gs[2] + sub * 8;
        const uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
        const T* oe = reinterpret_cast<const T*>(&ov);
        const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum = fmaf(to_float<T>(oe[e]), to_float<T>(ge[e]), sum);
    }
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (sub == 0 && row_id < rows) p.delta[row_id] = sum;
}

std::atomic<int> g_configured{0};

template <int D, bool BF16, bool KV>
cudaError_t launch_t(const AttnParams& p, cudaStream_t st) {
    using C = Cfg<D>;
    auto kernel = p.has_mask ? pipeline_backward<D, BF16, KV, true> : pipeline_backward<D, BF16, KV, false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    constexpr int variant = (D == 128 ? 0 : 4) + (BF16 ? 0 : 2) + (KV ? 1 : 0);
    if (!(g_configured.load() & (1 << variant))) g_configured |= 1 << variant;
    Maps maps;
    const CUtensorMapDataType dt = BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (!encode_bhsd_map(&maps.q, p.q, dt, p.D, p.Sq, p.Hq, p.B, p.qs, 64, kTile)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.k, p.k, dt, p.D, p.Sk, p.Hkv, p.B, p.ks, 64, kTile)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.v, p.v, dt, p.D, p.Sk, p.Hkv, p.B, p.vs, 64, kTile)) return cudaErrorInvalidValue;
    if (!encode_bhsd_map(&maps.g, p.dout, dt, p.D, p.Sq, p.Hq, p.B, p.gs, 64, kTile)) return cudaErrorInvalidValue;
    const int64_t tiles = KV ? (p.Sk + kTile - 1) / kTile : (p.Sq + kTile - 1) / kTile;
    const int64_t grid = tiles * p.B * (KV ? p.Hkv : p.Hq);
    kernel<<<(unsigned)grid, kThreads, C::kSmemBytes, st>>>(maps, p);
    return cudaGetLastError();
}

}  // namespace

bool pipeline_backward_supported(const AttnParams& p, bool bf16) {
    (void)bf16;
    if (p.D != 64 && p.D != 128) return false;
    if (p.nd != 0 || p.scale == 0.f) return false;
    if (p.Sk < 2) return false;  // a single key has P = 1: the general kernels keep dS exactly zero there
    if (!tma_compatible(p.q, p.qs, p.B, p.Hq, p.Sq) || !tma_compatible(p.k, p.ks, p.B, p.Hkv, p.Sk) ||
        !tma_compatible(p.v, p.vs, p.B, p.Hkv, p.Sk) || !tma_compatible(p.dout, p.gs, p.B, p.Hq, p.Sq))
        return false;
    // 16-byte vector stores / loads per row
    return tma_compatible(p.dq, p.dqs, p.B, p.Hq, p.Sq) && tma_compatible(p.dk, p.dks, p.B, p.Hkv, p.Sk) &&
           tma_compatible(p.dv, p.dvs, p.B, p.Hkv, p.Sk) && tma_compatible(p.out, p.os, p.B, p.Hq, p.Sq);
}

// which: 0 = query-gradient kernel, 1 = key/value-gradient kernel
cudaError_t launch_pipeline_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st) {
    if (p.D == 128) {
        if (which == 0) return bf16 ? launch_t<128, true, false>(p, st) : launch_t<128, false, false>(p, st);
        return bf16 ? launch_t<128, true, true>(p, st) : launch_t<128, false, true>(p, st);
    }
    if (which == 0) return bf16 ? launch_t<64, true, false>(p, st) : launch_t<64, false, false>(p, st);
    return bf16 ? launch_t<64, true, true>(p, st) : launch_t<64, false, true>(p, st);
}

// delta for the pipeline family (rows are 16-byte aligned and channel-contiguous there)
cudaError_t launch_pipeline_delta(const AttnParams& p, bool bf16, cudaStream_t st) {
    const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
    if (p.D == 128) {
        const unsigned grid = (unsigned)((rows + 15) / 16);
        if (bf16) output_delta_rows<__nv_bfloat16, 128><<<grid, 256, 0, st>>>(p);
        else output_delta_rows<__half, 128><<<grid, 256, 0, st>>>(p);
    } else {
        const unsigned grid = (unsigned)((rows + 31) / 32);
        if (bf16) output_delta_rows<__nv_bfloat16, 64><<<grid, 256, 0, st>>>(p);
        else output_delta_rows<__half, 64><<<grid, 256, 0, st>>>(p);
    }
    return cudaGetLastError();
}

#ifdef KFA_TRACE
extern "C" __attribute__((visibility("default"))) int kfa_debug_trace(long long* out, int* counts) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_kfa_trace, sizeof(long long) * 4 * 1024);
    cudaMemcpyFromSymbol(counts, g_kfa_trace_n, sizeof(int) * 4);
    int zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_kfa_trace_n, zero, sizeof(zero));
    return 0;
}
#endif

int pipeline_configured_variants() { return pipeline_forward_variants() + __builtin_popcount(g_configured.load()); }
void pipeline_forget_variants() {
    pipeline_forward_forget();
    g_configured = 0;
}

}  // namespace kfa
