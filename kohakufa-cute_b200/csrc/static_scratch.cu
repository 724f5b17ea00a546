// Key centring without any allocation: kfa_center_keys_static.
//
// Some hosts of this library may not allocate device memory once they are running: a serving
// process that sized its memory arena at start-up and treats every later cudaMalloc as a bug
// (it synchronises the whole device and can fail under a full arena), or a plain C plugin host
// that owns nothing but the q/k/v buffers it passes in and has no allocator to ask for scratch.
// For them this entry point keeps the scratch of the key-centring kernels (the per-split column
// sums and the means) in a fixed array that is part of the loaded library image, so each GPU
// that loads the library holds kStaticFloats * 4 bytes (about 2.1 MB) until the process exits.
//
// Rules that follow from sharing one array:
//   * sizes whose scratch does not fit (batch * heads * channels > kfa_center_keys_static_limit())
//     are rejected with KFA_TOO_LARGE; nothing is launched;
//   * the array keeps whatever the previous call left in it.  The kernels overwrite every element
//     they later read, so nothing has to be cleared between calls;
//   * shapes the one-launch thread-block-cluster kernel serves (64/128/256/512 channels, at least 64 rows,
//     16-byte addressable rows, a sequence slab that fits in shared memory) need no scratch and do not
//     touch the array; every other shape runs the three-kernel path through it;
//   * two calls of the second kind that overlap in time on the same GPU (different streams or threads)
//     race on the array: serialise them, or use kfa_center_keys with caller-owned scratch;
//   * the first call on each device looks up the array's device address (with that device
//     current).  Make that first call before starting any stream capture on the device.
#include "../../include/kfa.h"
#include "kfa_common.cuh"
#include "launchers.h"

#include <cstdio>
#include <mutex>

namespace kfa {
void note_failure(int code, const char* message);  // records the thread's last error (kfa_api.cu)
void count_launches(const char* name, int n);
cudaError_t timed_launch(const char* name, cudaStream_t st, cudaError_t (*launch)(void*), void* context);
}  // namespace kfa

namespace {

constexpr int kSplits = 32;                        // sequence splits of the column-sum kernel
constexpr size_t kMaxUnits = 16384;                // largest batch * heads * channels served
constexpr size_t kStaticFloats = kMaxUnits * (kSplits + 1);

// In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) float g_center_scratch[kStaticFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the array on the current device, looked up once per device.
float* scratch_address(int* error) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        kfa::note_failure(KFA_CUDA_ERROR, "cudaGetDevice failed while locating the static scratch");
        *error = KFA_CUDA_ERROR;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_address[device]) {
        float* address = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_center_scratch);
        if (e != cudaSuccess || !address) {
            char text[160];
            std::snprintf(text, sizeof(text), "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
            kfa::note_failure(KFA_CUDA_ERROR, text);
            *error = KFA_CUDA_ERROR;
            return nullptr;
        }
        g_scratch_address[device] = address;
    }
    return g_scratch_address[device];
}

}  // namespace

extern "C" {

size_t kfa_center_keys_static_limit(void) { return kMaxUnits; }

int kfa_center_keys_static(const kfa_tensor* k, kfa_tensor* centered, void* stream) {
    if (!k || !k->data || k->ndim != 4 || (k->dtype != KFA_F16 && k->dtype != KFA_BF16)) {
        kfa::note_failure(KFA_INVALID_ARGUMENT, "center_keys requires a 4D FP16/BF16 tensor");
        return KFA_INVALID_ARGUMENT;
    }
    if (!centered || !centered->data || centered->dtype != k->dtype || centered->ndim != 4) {
        kfa::note_failure(KFA_INVALID_ARGUMENT, "centered must match the shape and dtype of its source tensor");
        return KFA_INVALID_ARGUMENT;
    }
    for (int i = 0; i < 4; ++i) {
        if (k->sizes[i] <= 0 || k->sizes[i] > INT32_MAX || centered->sizes[i] != k->sizes[i]) {
            kfa::note_failure(KFA_INVALID_ARGUMENT, "center_keys: bad or mismatching extent");
            return KFA_INVALID_ARGUMENT;
        }
    }
    const size_t units = (size_t)k->sizes[0] * k->sizes[1] * k->sizes[3];
    if (units > kMaxUnits) {
        char text[200];
        std::snprintf(text, sizeof(text),
                      "kfa_center_keys_static: batch*heads*channels = %zu exceeds the fixed scratch capacity %zu "
                      "(use kfa_center_keys with caller-owned scratch)",
                      units, kMaxUnits);
        kfa::note_failure(KFA_TOO_LARGE, text);
        return KFA_TOO_LARGE;
    }
    int error = 0;
    float* scratch = scratch_address(&error);
    if (!scratch) return error;
    struct Call {
        const kfa_tensor* k;
        kfa_tensor* centered;
        float* scratch;
        cudaStream_t stream;
        int launches;
    } call = {k, centered, scratch, static_cast<cudaStream_t>(stream), 0};
    // through the library's timing wrapper, so that per-kernel profiles and launch statistics show this entry point
    cudaError_t ce = kfa::timed_launch(
        "center_keys_static", call.stream,
        [](void* context) {
            Call& c = *static_cast<Call*>(context);
            return kfa::launch_center_keys(c.k->data, c.centered->data, c.scratch, c.k->dtype == KFA_BF16,
                                           (int)c.k->sizes[0], (int)c.k->sizes[1], (int)c.k->sizes[2],
                                           (int)c.k->sizes[3], c.k->strides, c.centered->strides, c.stream, &c.launches);
        },
        &call);
    if (ce != cudaSuccess) {
        kfa::note_failure(KFA_CUDA_ERROR, cudaGetErrorString(ce));
        return KFA_CUDA_ERROR;
    }
    // one kernel when the shape suits the thread-block-cluster kernel (which needs no scratch at all), three when
    // the partial sums and means go through the static array; the wrapper has counted the first
    if (call.launches > 1) kfa::count_launches("center_keys_static", call.launches - 1);
    return 0;
}

}  // extern "C"
