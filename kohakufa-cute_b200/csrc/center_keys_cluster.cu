// Key centering in one launch: k_c = round(f32(k) - mean_S f32(k)) per (batch, K/V head, channel).
//
// A thread-block cluster of 8 CTAs owns one (batch, head).  Every CTA sums the columns of its S/8 rows, the
// column sums are combined across the cluster through distributed shared memory, and the CTA then subtracts the
// mean from its rows and writes them out.  Between the two steps the rows stay in shared memory (large tensors:
// read from HBM once, written once) or, when the whole tensor fits L2 with room to spare, are read a second time
// from L2 by a lighter kernel of which two CTAs fit an SM.  No partial-sum buffers and a single launch (the
// three-kernel path reads the keys twice and launches three times).  All sums run in a fixed order, so results are
// bitwise reproducible.  (Reference behaviour: src/kohakufa_cute/api.py:100-103 of the reference project.)
#include <cooperative_groups.h>

#include <atomic>

#include "kfa_common.cuh"
#include "launchers.h"

namespace kfa {
namespace {

namespace cg = cooperative_groups;
constexpr int kCluster = 8;
// With the slab in shared memory: 1024 threads, one CTA per SM (enough 16-byte loads in flight to cover the memory
// latency).  Without it (the slab read a second time, from L2): 512 threads, two CTAs per SM.
__host__ __device__ constexpr int threads_of(bool slab) { return slab ? 1024 : 512; }

template <typename T, bool kSlab>
__global__ void __launch_bounds__(threads_of(kSlab), kSlab ? 1 : 2) center_keys_cluster(const T* k, T* out, int H, int S, int D, int rows_per_cta,
                                                           int64_t k0, int64_t k1, int64_t k2, int64_t o0, int64_t o1,
                                                           int64_t o2) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kThreads = threads_of(kSlab);
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int bh = blockIdx.x / kCluster, b = bh / H, h = bh % H;
    const int pieces = D / 8;            // 16-byte pieces per row
    const int lanes = kThreads / pieces;  // rows in flight per pass
    const int piece = threadIdx.x % pieces, lane = threadIdx.x / pieces;
    uint4* slab = reinterpret_cast<uint4*>(smem);
    float* part = reinterpret_cast<float*>(smem + (kSlab ? (size_t)rows_per_cta * D * 2 : 0));  // [lanes][D]
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
                if (kSlab) slab[r * pieces + piece] = x[j];
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
    if (kSlab) {
        for (int r = lane; r < rows; r += lanes) {
            const uint4 x = slab[r * pieces + piece];
            const T* e = reinterpret_cast<const T*>(&x);
            uint4 y;
            T* w = reinterpret_cast<T*>(&y);
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = from_float<T>(to_float<T>(e[i]) - m[i]);
            *reinterpret_cast<uint4*>(dst + (int64_t)r * o2) = y;
        }
    } else {
        // second reading of the slab: from L2, where the first one left it
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
                    const T* e = reinterpret_cast<const T*>(&x[j]);
                    uint4 y;
                    T* w = reinterpret_cast<T*>(&y);
#pragma unroll
                    for (int i = 0; i < 8; ++i) w[i] = from_float<T>(to_float<T>(e[i]) - m[i]);
                    *reinterpret_cast<uint4*>(dst + (int64_t)r * o2) = y;
                }
            }
        }
    }
}

size_t shared_bytes(bool slab, int S, int D) {
    const size_t rows_per_cta = ((size_t)S + kCluster - 1) / kCluster;
    const size_t scratch = (size_t)((threads_of(slab) / (D / 8)) * D + 2 * D) * sizeof(float);
    return (slab ? rows_per_cta * D * 2 : 0) + scratch;
}

// The slab is read a second time from L2 instead of being kept in shared memory when the whole tensor and its
// centred copy fit L2 with room to spare: the CTAs are then light (two per SM, any sequence length), whereas the
// shared-memory slabs of a large call fill every SM and run as successive waves of clusters, each wave loading,
// reducing and storing in turn (measured at B4 H8 S4096 D128: 23 against 35 us per call).
bool reread_slab(int B, int H, int S, int D) { return (int64_t)B * H * S * D * 2 <= (40ll << 20); }

template <typename T, bool kSlab>
cudaError_t launch_t(const void* k, void* out, int B, int H, int S, int D, const int64_t* ks, const int64_t* os,
                     cudaStream_t st) {
    const int rows_per_cta = (S + kCluster - 1) / kCluster;
    const size_t bytes = shared_bytes(kSlab, S, D);
    cudaError_t e =
        cudaFuncSetAttribute(center_keys_cluster<T, kSlab>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(B * H * kCluster));
    config.blockDim = dim3(threads_of(kSlab));
    config.dynamicSmemBytes = bytes;
    config.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, center_keys_cluster<T, kSlab>, static_cast<const T*>(k), static_cast<T*>(out), H,
                              S, D, rows_per_cta, ks[0], ks[1], ks[2], os[0], os[1], os[2]);
}

}  // namespace

// Shapes the one-launch path serves: 16-byte addressable rows on both sides, 64/128/256/512 channels, and either a
// tensor small enough for the second reading from L2 or a slab of S/8 rows that fits beside the reduction scratch in
// shared memory.
bool center_keys_cluster_supported(const void* k, const void* out, int B, int H, int S, int D, const int64_t* ks,
                                   const int64_t* os) {
    if (D != 64 && D != 128 && D != 256 && D != 512) return false;
    if (S < 64) return false;
    if (ks[3] != 1 || os[3] != 1 || ks[2] % 8 != 0 || os[2] % 8 != 0 || ks[1] % 8 != 0 || os[1] % 8 != 0 ||
        ks[0] % 8 != 0 || os[0] % 8 != 0)
        return false;
    if (reinterpret_cast<uintptr_t>(k) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0) return false;
    return reread_slab(B, H, S, D) || shared_bytes(true, S, D) <= 200 * 1024;
}

// Whether a cluster of 8 CTAs with this much shared memory each can be resident on the current device at all
// (a partitioned or smaller device may not manage).  Asked once per (device, type, shared-memory size class); the
// answer for the slab kernel covers the lighter kernel without a slab.
bool center_keys_cluster_schedulable(bool bf16, int S, int D) {
    static std::atomic<int> cache[64][2][2];  // 0 unknown, 1 yes, 2 no; [device][type][small/large shared memory]
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    const size_t bytes = shared_bytes(true, S, D);
    const int cls = bytes > 100 * 1024 ? 1 : 0;
    const int seen = cache[dev][bf16 ? 1 : 0][cls].load();
    if (seen) return seen == 1;
    // ask for the larger size of the class, so that one answer covers every size in it
    const size_t ask = cls ? 200 * 1024 : 100 * 1024;
    const void* fn = bf16 ? (const void*)center_keys_cluster<__nv_bfloat16, true>
                          : (const void*)center_keys_cluster<__half, true>;
    int clusters = 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(kCluster);
    config.blockDim = dim3(threads_of(true));
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
    if (reread_slab(B, H, S, D))
        return bf16 ? launch_t<__nv_bfloat16, false>(k, out, B, H, S, D, ks, os, st)
                    : launch_t<__half, false>(k, out, B, H, S, D, ks, os, st);
    return bf16 ? launch_t<__nv_bfloat16, true>(k, out, B, H, S, D, ks, os, st)
                : launch_t<__half, true>(k, out, B, H, S, D, ks, os, st);
}

}  // namespace kfa
