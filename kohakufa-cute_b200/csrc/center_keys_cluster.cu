// Key centering in one launch: k_c = round(f32(k) - mean_S f32(k)) per (batch, K/V head, channel).
//
// A thread-block cluster of 8 CTAs owns one (batch, head); every CTA keeps its slab of S/8 rows in
// shared memory while the column sums are combined across the cluster through distributed shared
// memory, then subtracts the mean from the resident slab and writes it out.  The keys are read from
// HBM once and written once, with no partial-sum buffers and a single launch (the three-kernel path
// reads them twice and launches three times).  All sums run in a fixed order, so results are
// bitwise reproducible.  (Reference behaviour: src/kohakufa_cute/api.py:100-103 of the reference project.)
#include <cooperative_groups.h>

#include <atomic>

#include "kfa_common.cuh"
#include "launchers.h"

namespace kfa {
namespace {

namespace cg = cooperative_groups;
constexpr int kCluster = 8;
constexpr int kThreads = 1024;  // one CTA per SM: enough 16-byte loads in flight to cover the memory latency

template <typename T>
__global__ void __launch_bounds__(kThreads) center_keys_cluster(const T* k, T* out, int H, int S, int D, int rows_per_cta,
                                                           int64_t k0, int64_t k1, int64_t k2, int64_t o0, int64_t o1,
                                                           int64_t o2) {
    extern __shared__ __align__(16) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int bh = blockIdx.x / kCluster, b = bh / H, h = bh % H;
    const int pieces = D / 8;            // 16-byte pieces per row
    const int lanes = kThreads / pieces;  // rows in flight per pass
    const int piece = threadIdx.x % pieces, lane = threadIdx.x / pieces;
    uint4* slab = reinterpret_cast<uint4*>(smem);
    float* part = reinterpret_cast<float*>(smem + (size_t)rows_per_cta * D * 2);  // [lanes][D]
    float* total = part + lanes * D;                                              // this CTA's column sums
    float* mean = total + D;

    const int row0 = rank * rows_per_cta;
    const int rows = max(0, min(S - row0, rows_per_cta));
    const T* src = k + (int64_t)b * k0 + (int64_t)h * k1 + (int64_t)row0 * k2 + piece * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // eight independent 16-byte loads in flight per thread (the pass is bound by memory latency otherwise)
    constexpr int kBatch = 8;
    for (int r0 = lane; r0 < rows; r0 += lanes * kBatch) {
        uint4 x[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int r = r0 + j * lanes;
            x[j] = r < rows ? *reinterpret_cast<const uint4*>(src + (int64_t)r * k2) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int r = r0 + j * lanes;
            if (r < rows) {
                slab[r * pieces + piece] = x[j];
                const T* e = reinterpret_cast<const T*>(&x[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += to_float<T>(e[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) part[lane * D + piece * 8 + i] = acc[i];
    __syncthreads();
    // fold the row lanes pairwise (fixed order: bitwise reproducible), then the eight CTAs of the cluster
    for (int width = lanes / 2; width >= 1; width /= 2) {
        for (int i = threadIdx.x; i < width * D; i += kThreads) part[i] += part[i + width * D];
        __syncthreads();
    }
    for (int d = threadIdx.x; d < D; d += kThreads) total[d] = part[d];
    cluster.sync();
    for (int d = threadIdx.x; d < D; d += kThreads) {
        float v[kCluster];
#pragma unroll
        for (int c = 0; c < kCluster; ++c) v[c] = cluster.map_shared_rank(total, c)[d];  // eight loads in flight
        mean[d] = (((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]))) / (float)S;
    }
    cluster.sync();  // every remote read is done before a CTA may exit; the means are visible to the block
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = mean[piece * 8 + i];
    T* dst = out + (int64_t)b * o0 + (int64_t)h * o1 + (int64_t)row0 * o2 + piece * 8;
    for (int r = lane; r < rows; r += lanes) {
        const uint4 x = slab[r * pieces + piece];
        const T* e = reinterpret_cast<const T*>(&x);
        uint4 y;
        T* w = reinterpret_cast<T*>(&y);
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = from_float<T>(to_float<T>(e[i]) - m[i]);
        *reinterpret_cast<uint4*>(dst + (int64_t)r * o2) = y;
    }
}

template <typename T>
cudaError_t launch_t(const void* k, void* out, int B, int H, int S, int D, const int64_t* ks, const int64_t* os,
                     cudaStream_t st) {
    const int rows_per_cta = (S + kCluster - 1) / kCluster;
    const int lanes = kThreads / (D / 8);
    const size_t bytes = (size_t)rows_per_cta * D * 2 + (size_t)(lanes * D + 2 * D) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(center_keys_cluster<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(B * H * kCluster));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = bytes;
    config.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, center_keys_cluster<T>, static_cast<const T*>(k), static_cast<T*>(out), H, S, D,
                              rows_per_cta, ks[0], ks[1], ks[2], os[0], os[1], os[2]);
}

}  // namespace

// Shapes the one-launch path serves: 16-byte addressable rows on both sides, 64/128/256/512 channels,
// and a slab of S/8 rows that fits beside the reduction scratch in shared memory.
bool center_keys_cluster_supported(const void* k, const void* out, int S, int D, const int64_t* ks, const int64_t* os) {
    if (D != 64 && D != 128 && D != 256 && D != 512) return false;
    if (S < 64) return false;
    if (ks[3] != 1 || os[3] != 1 || ks[2] % 8 != 0 || os[2] % 8 != 0 || ks[1] % 8 != 0 || os[1] % 8 != 0 ||
        ks[0] % 8 != 0 || os[0] % 8 != 0)
        return false;
    if (reinterpret_cast<uintptr_t>(k) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0) return false;
    const size_t rows_per_cta = ((size_t)S + kCluster - 1) / kCluster;
    const size_t bytes = rows_per_cta * D * 2 + (size_t)((kThreads / (D / 8)) * D + 2 * D) * sizeof(float);
    return bytes <= 200 * 1024;
}

// Whether a cluster of 8 CTAs with this much shared memory each can be resident on the current device at all
// (a partitioned or smaller device may not manage).  Asked once per (device, type, shared-memory size class).
bool center_keys_cluster_schedulable(bool bf16, int S, int D) {
    static std::atomic<int> cache[64][2][2];  // 0 unknown, 1 yes, 2 no; [device][type][small/large shared memory]
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    const size_t rows_per_cta = ((size_t)S + kCluster - 1) / kCluster;
    const size_t bytes = rows_per_cta * D * 2 + (size_t)((kThreads / (D / 8)) * D + 2 * D) * sizeof(float);
    const int cls = bytes > 100 * 1024 ? 1 : 0;
    const int seen = cache[dev][bf16 ? 1 : 0][cls].load();
    if (seen) return seen == 1;
    // ask for the larger size of the class, so that one answer covers every size in it
    const size_t ask = cls ? 200 * 1024 : 100 * 1024;
    const void* fn = bf16 ? (const void*)center_keys_cluster<__nv_bfloat16> : (const void*)center_keys_cluster<__half>;
    int clusters = 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(kCluster);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = ask;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    bool ok = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ask) == cudaSuccess &&
              cudaOccupancyMaxActiveClusters(&clusters, fn, &config) == cudaSuccess && clusters > 0;
    if (!ok) cudaGetLastError();
    cache[dev][bf16 ? 1 : 0][cls] = ok ? 1 : 2;
    return ok;
}

cudaError_t launch_center_keys_cluster(const void* k, void* out, bool bf16, int B, int H, int S, int D,
                                       const int64_t* ks, const int64_t* os, cudaStream_t st) {
    return bf16 ? launch_t<__nv_bfloat16>(k, out, B, H, S, D, ks, os, st)
                : launch_t<__half>(k, out, B, H, S, D, ks, os, st);
}

}  // namespace kfa
