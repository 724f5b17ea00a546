// C ABI of libkfa.so: argument validation, kernel-family selection and launches.
// Declarations and the reference interfaces they replace are in include/kfa.h.
#include "../../include/kfa.h"
#include "kfa_common.cuh"
#include "launchers.h"

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    return fail(KFA_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
}

// Optional per-kernel timing with CUDA events on the launching stream.
struct Sample {
    const char* name;
    cudaEvent_t begin, end;
};
std::mutex g_profile_mutex;
std::atomic<bool> g_profile_on{false};
std::vector<Sample> g_samples;
struct Total {
    const char* name;
    double ms;
    uint64_t launches;
};
std::vector<Total> g_totals;

// Launches per kernel name since load (observability: kfa_launch_stats).
constexpr int kMaxStatNames = 48;
struct LaunchStat {
    std::atomic<const char*> name{nullptr};
    std::atomic<uint64_t> launches{0};
};
LaunchStat g_launch_stats[kMaxStatNames];

void count_kernel(const char* name, uint64_t n) {
    g_launches += n;
    for (int i = 0; i < kMaxStatNames; ++i) {
        const char* seen = g_launch_stats[i].name.load(std::memory_order_acquire);
        if (seen == nullptr) {
            const char* expected = nullptr;
            if (g_launch_stats[i].name.compare_exchange_strong(expected, name, std::memory_order_acq_rel)) seen = name;
            else seen = expected;
        }
        if (seen == name || std::strcmp(seen, name) == 0) {
            g_launch_stats[i].launches += n;
            return;
        }
    }
}

#ifdef KFA_NVTX
// Ranges around every launch for timeline tools (compile with -DKFA_NVTX; needs the toolkit's nvtx3 headers).
}  // namespace
#include <nvtx3/nvToolsExt.h>
namespace {
struct Range {
    explicit Range(const char* name) { nvtxRangePushA(name); }
    ~Range() { nvtxRangePop(); }
};
#else
struct Range {
    explicit Range(const char*) {}
};
#endif

// Runs one launch; when profiling is on, brackets it with events.
template <typename F>
cudaError_t timed(const char* name, cudaStream_t st, F&& launch) {
    count_kernel(name, 1);
    Range range(name);
    if (!g_profile_on.load(std::memory_order_relaxed)) return launch();
    Sample s{name, nullptr, nullptr};
    cudaEventCreate(&s.begin);
    cudaEventCreate(&s.end);
    cudaEventRecord(s.begin, st);
    cudaError_t e = launch();
    cudaEventRecord(s.end, st);
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    g_samples.push_back(s);
    return e;
}

// A side stream with its fork/join events per (host thread, device, caller stream), created on first use and
// kept for the thread's lifetime.  Per thread, because two host threads that record the same event pair
// (even on the same caller stream) would race on the records.
struct Side {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
thread_local std::vector<std::pair<std::pair<int, cudaStream_t>, Side*>> g_sides;

Side* side_stream_for(cudaStream_t user) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    for (auto& entry : g_sides)
        if (entry.first.first == dev && entry.first.second == user) return entry.second;
    // creating a stream is not allowed while the caller's stream is being captured: stay on one stream then
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(user, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return nullptr;
    }
    Side* side = new Side;
    if (cudaStreamCreateWithFlags(&side->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&side->fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&side->join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        delete side;
        return nullptr;
    }
    g_sides.push_back({{dev, user}, side});
    return side;
}

// Per-device status word in mapped host memory: kernels write it only when a
// bounded wait gives up; the host reads it without synchronising.
constexpr int kMaxDevices = 64;
int* g_status_host[kMaxDevices] = {};
int* g_status_dev[kMaxDevices] = {};
int* g_abort_dev[kMaxDevices] = {};  // device memory: launch-wide abort flag (see AttnParams::abort_flag)
std::mutex g_status_mutex;

// `st` is the stream the caller is about to launch on: the first call on a device allocates the status word
// and the abort flag, which is not allowed while that stream is being captured.
int* status_word(int* err, cudaStream_t st = nullptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        *err = cuda_fail(e, "cudaGetDevice");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_dev[dev]) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess) cudaGetLastError();
        if (capturing != cudaStreamCaptureStatusNone) {
            *err = fail(KFA_CUDA_ERROR,
                        "the first call on a device sets up per-device state and cannot run under stream capture: "
                        "call kfa_init() (or run one call) on this device before capturing");
            return nullptr;
        }
        int* host = nullptr;
        e = cudaHostAlloc(reinterpret_cast<void**>(&host), 64, cudaHostAllocMapped | cudaHostAllocPortable);
        if (e != cudaSuccess) {
            *err = cuda_fail(e, "cudaHostAlloc(status)");
            return nullptr;
        }
        std::memset(host, 0, 64);
        int* devp = nullptr;
        e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&devp), host, 0);
        if (e != cudaSuccess) {
            *err = cuda_fail(e, "cudaHostGetDevicePointer(status)");
            return nullptr;
        }
        int* flag = nullptr;
        e = cudaMalloc(reinterpret_cast<void**>(&flag), 256);
        if (e == cudaSuccess) e = cudaMemset(flag, 0, 256);
        if (e != cudaSuccess) {
            *err = cuda_fail(e, "cudaMalloc(abort flag)");
            return nullptr;
        }
        g_status_host[dev] = host;
        g_status_dev[dev] = devp;
        g_abort_dev[dev] = flag;
    }
    return g_status_dev[dev];
}

int* abort_flag_of_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    return g_abort_dev[dev];
}

// A bounded device-side wait that ran out leaves its code in the status word and keeps every later
// tensor-memory launch idle; entry points refuse to launch (and to hand back unwritten outputs) until the
// report is acknowledged with kfa_device_status(1).  Reading the mapped word is a plain host load.
int check_device_ok() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    int* host = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_status_mutex);
        host = g_status_host[dev];
    }
    if (!host) return 0;
    const int code = *reinterpret_cast<volatile int*>(host);
    if (code == 0) return 0;
    return fail(KFA_DEVICE_TIMEOUT,
                "a device-side wait of an earlier launch ran out (status %d); results since then are invalid. "
                "Acknowledge with kfa_device_status(1) before launching again", code);
}

bool is_half_type(const kfa_tensor* t) { return t->dtype == KFA_F16 || t->dtype == KFA_BF16; }

void copy4(int64_t* dst, const int64_t* src) {
    for (int i = 0; i < 4; ++i) dst[i] = src[i];
}

bool contiguous3(const kfa_tensor* t, int64_t b, int64_t h, int64_t s) {
    return t && t->data && t->dtype == KFA_F32 && t->ndim == 3 && t->sizes[0] == b && t->sizes[1] == h &&
           t->sizes[2] == s && t->strides[2] == 1 && t->strides[1] == s && t->strides[0] == h * s;
}

bool same_shape(const kfa_tensor* a, const kfa_tensor* b) {
    if (a->ndim != b->ndim) return false;
    for (int i = 0; i < a->ndim; ++i)
        if (a->sizes[i] != b->sizes[i]) return false;
    return true;
}

// Shared checks for q/k/v (messages mirror the reference's validation wording: api.py:76-97).
int check_qkv(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v) {
    if (!q || !k || !v || !q->data || !k->data || !v->data) return fail(KFA_INVALID_ARGUMENT, "null Q/K/V");
    if (q->ndim != 4 || k->ndim != 4 || v->ndim != 4)
        return fail(KFA_INVALID_ARGUMENT, "attention requires 4D [batch, heads, sequence, dim] Q/K/V");
    if (!is_half_type(q) || k->dtype != q->dtype || v->dtype != q->dtype)
        return fail(KFA_INVALID_ARGUMENT, "attention requires matching FP16/BF16 Q/K/V; FP32 attention is unsupported");
    for (int i = 0; i < 4; ++i)
        if (q->sizes[i] <= 0 || k->sizes[i] <= 0)
            return fail(KFA_INVALID_ARGUMENT, "attention requires nonempty Q/K/V");
    if (!same_shape(k, v) || q->sizes[0] != k->sizes[0] || q->sizes[3] != k->sizes[3])
        return fail(KFA_INVALID_ARGUMENT, "attention requires matching batch/head dimensions and equal K/V shapes");
    if (q->sizes[1] % k->sizes[1] != 0 || q->sizes[3] > 512)
        return fail(KFA_INVALID_ARGUMENT, "attention requires head dimensions 1..512 and query heads divisible by K/V heads");
    if (q->sizes[2] > INT32_MAX || k->sizes[2] > INT32_MAX || q->sizes[0] * q->sizes[1] > INT32_MAX)
        return fail(KFA_TOO_LARGE, "sequence length or batch*heads exceeds 2^31-1");
    return 0;
}

int fill_common(kfa::AttnParams& p, const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v,
                const kfa_tensor* mask, float scale, int causal, cudaStream_t st = nullptr) {
    std::memset(&p, 0, sizeof(p));
    p.q = q->data;
    p.k = k->data;
    p.v = v->data;
    copy4(p.qs, q->strides);
    copy4(p.ks, k->strides);
    copy4(p.vs, v->strides);
    p.B = (int)q->sizes[0];
    p.Hq = (int)q->sizes[1];
    p.Hkv = (int)k->sizes[1];
    p.Sq = (int)q->sizes[2];
    p.Sk = (int)k->sizes[2];
    p.D = (int)q->sizes[3];
    p.group = p.Hq / p.Hkv;
    p.scale = scale;
    p.causal = causal ? 1 : 0;
    if (mask) {
        if (mask->dtype != KFA_BOOL || mask->ndim != 4 || !mask->data)
            return fail(KFA_INVALID_ARGUMENT, "attention requires a boolean mask expanded to [B,Hq,Sq,Sk]");
        if (mask->sizes[0] != q->sizes[0] || mask->sizes[1] != q->sizes[1] || mask->sizes[2] != q->sizes[2] ||
            mask->sizes[3] != k->sizes[2])
            return fail(KFA_INVALID_ARGUMENT, "mask shape does not match [B,Hq,Sq,Sk]");
        p.mask = static_cast<const uint8_t*>(mask->data);
        copy4(p.ms, mask->strides);
        p.has_mask = 1;
    }
    int err = 0;
    p.status = status_word(&err, st);
    p.abort_flag = abort_flag_of_current_device();
    return err;
}

// Extents of the tile table for this mask (extent 1 on stride-0 axes).
void block_extents(const kfa::AttnParams& p, int64_t (&n)[4]) {
    n[0] = p.ms[0] == 0 ? 1 : p.B;
    n[1] = p.ms[1] == 0 ? 1 : p.Hq;
    n[2] = p.ms[2] == 0 ? 1 : (p.Sq + 63) / 64;
    n[3] = p.ms[3] == 0 ? 1 : (p.Sk + 63) / 64;
}

int bind_blocks(kfa::AttnParams& p, const kfa_tensor* blocks) {
    if (!p.has_mask) return 0;
    int64_t n[4];
    block_extents(p, n);
    if (!blocks || !blocks->data || blocks->dtype != KFA_I32 || blocks->ndim != 4)
        return fail(KFA_INVALID_ARGUMENT, "masked attention requires an int32 4-D tile table");
    for (int i = 0; i < 4; ++i)
        if (blocks->sizes[i] != n[i])
            return fail(KFA_INVALID_ARGUMENT, "tile table extent %d is %lld, expected %lld", i,
                        (long long)blocks->sizes[i], (long long)n[i]);
    // The table is dense over its own extents; collapsed axes get stride 0 for lookups.
    if (blocks->strides[3] != 1 || blocks->strides[2] != n[3] || blocks->strides[1] != n[2] * n[3] ||
        blocks->strides[0] != n[1] * n[2] * n[3])
        return fail(KFA_INVALID_ARGUMENT, "tile table must be contiguous");
    p.blocks = static_cast<int32_t*>(blocks->data);
    p.bs[0] = n[0] == 1 ? 0 : blocks->strides[0];
    p.bs[1] = n[1] == 1 ? 0 : blocks->strides[1];
    p.bs[2] = n[2] == 1 ? 0 : blocks->strides[2];
    p.bs[3] = n[3] == 1 ? 0 : blocks->strides[3];
    return 0;
}

int check_like(const kfa_tensor* t, const kfa_tensor* like, const char* name) {
    if (!t || !t->data || t->dtype != like->dtype || !same_shape(t, like))
        return fail(KFA_INVALID_ARGUMENT, "%s must match the shape and dtype of its source tensor", name);
    return 0;
}

int geometry(kfa::AttnParams& p, const int64_t* spatial, int nd, const int64_t* window) {
    if ((nd != 2 && nd != 3) || !spatial || !window)
        return fail(KFA_INVALID_ARGUMENT, "spatial_shape must contain two or three positive integers");
    int64_t tokens = 1;
    for (int i = 0; i < 3; ++i) {
        const int src = i - (3 - nd);
        const int64_t e = src < 0 ? 1 : spatial[src], w = src < 0 ? 1 : window[src];
        if (e <= 0 || e > INT32_MAX) return fail(KFA_INVALID_ARGUMENT, "spatial_shape must contain positive integers");
        if (w <= 0 || w > e)
            return fail(KFA_INVALID_ARGUMENT, "window_size must contain positive integers no larger than spatial_shape");
        p.ext[i] = (int)e;
        p.win[i] = (int)w;
        tokens *= e;
    }
    if (tokens != p.Sq || p.Sq != p.Sk || p.D != 64 || p.Hq != p.Hkv)
        return fail(KFA_INVALID_ARGUMENT,
                    "neighborhood attention requires matching [B, heads, prod(spatial_shape), 64] Q/K/V");
    p.nd = nd;
    return 0;
}

}  // namespace

namespace kfa {
void note_failure(int code, const char* message) { fail(code, "%s", message); }
void count_launches(const char* name, int n) { count_kernel(name, (uint64_t)n); }
// One launch sequence under the per-kernel event timing and launch statistics of this file (for entry points that
// live in other translation units).
cudaError_t timed_launch(const char* name, cudaStream_t st, cudaError_t (*launch)(void*), void* context) {
    return timed(name, st, [&] { return launch(context); });
}
}  // namespace kfa

extern "C" {

int kfa_version(void) { return (0 << 16) | 1; }

const char* kfa_last_error(void) { return g_error; }

uint64_t kfa_launch_count(void) { return g_launches.load(); }

int kfa_launch_stats(int index, char* name, size_t name_bytes, uint64_t* launches) {
    if (index < 0 || index >= kMaxStatNames || !name || name_bytes == 0)
        return fail(KFA_INVALID_ARGUMENT, "launch statistics entry %d does not exist", index);
    const char* seen = g_launch_stats[index].name.load(std::memory_order_acquire);
    if (!seen) return fail(KFA_INVALID_ARGUMENT, "launch statistics entry %d does not exist", index);
    std::snprintf(name, name_bytes, "%s", seen);
    if (launches) *launches = g_launch_stats[index].launches.load();
    return 0;
}

int kfa_init(void) {
    int err = 0;
    return status_word(&err) ? 0 : err;
}

int kfa_cache_size(void) { return kfa::pipeline_configured_variants(); }

void kfa_clear_cache(void) { kfa::pipeline_forget_variants(); }

int kfa_device_status(int reset) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_host[dev]) return 0;
    const int value = *reinterpret_cast<volatile int*>(g_status_host[dev]);
    if (reset) {
        *reinterpret_cast<volatile int*>(g_status_host[dev]) = 0;
        // after a reported failure the abort flag keeps every later CTA idle until it is cleared here
        if (value != 0 && g_abort_dev[dev]) cudaMemset(g_abort_dev[dev], 0, 256);
    }
    return value;
}

int kfa_self_test_wait(long long limit_cycles, int ctas, int* skipped_out, void* stream) {
    if (limit_cycles <= 0 || limit_cycles > 2000000000LL || ctas <= 0 || ctas > 65535)
        return fail(KFA_INVALID_ARGUMENT, "self test: limit must be 1..2e9 cycles and ctas 1..65535");
    int err = 0;
    int* status = status_word(&err);
    if (!status) return err;
    int* flag = abort_flag_of_current_device();
    int* counter = nullptr;
    cudaError_t ce = cudaMalloc(reinterpret_cast<void**>(&counter), sizeof(int));
    if (ce != cudaSuccess) return cuda_fail(ce, "self test allocation");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaMemsetAsync(counter, 0, sizeof(int), st);
    ce = kfa::launch_wait_probe(status, flag, limit_cycles, ctas, counter, st);
    int skipped = 0;
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(&skipped, counter, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
    cudaFree(counter);
    if (ce != cudaSuccess) return cuda_fail(ce, "self test launch");
    if (skipped_out) *skipped_out = skipped;
    return 0;
}

void kfa_profile_enable(int on) {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    g_profile_on = on != 0;
}

int kfa_profile_collect(void) {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    for (Sample& s : g_samples) {
        float ms = 0.f;
        if (cudaEventSynchronize(s.end) == cudaSuccess && cudaEventElapsedTime(&ms, s.begin, s.end) == cudaSuccess) {
            bool found = false;
            for (Total& t : g_totals)
                if (std::strcmp(t.name, s.name) == 0) {
                    t.ms += ms;
                    t.launches += 1;
                    found = true;
                }
            if (!found) g_totals.push_back(Total{s.name, ms, 1});
        }
        cudaEventDestroy(s.begin);
        cudaEventDestroy(s.end);
    }
    g_samples.clear();
    return (int)g_totals.size();
}

int kfa_profile_entry(int index, char* name, size_t name_bytes, double* total_ms, uint64_t* launches) {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    if (index < 0 || index >= (int)g_totals.size() || !name || name_bytes == 0)
        return fail(KFA_INVALID_ARGUMENT, "profile entry %d does not exist", index);
    std::snprintf(name, name_bytes, "%s", g_totals[index].name);
    if (total_ms) *total_ms = g_totals[index].ms;
    if (launches) *launches = g_totals[index].launches;
    return 0;
}

void kfa_profile_reset(void) {
    std::lock_guard<std::mutex> lock(g_profile_mutex);
    g_totals.clear();
}

}  // extern "C"

namespace {

size_t delta_bytes(const kfa_tensor* q) {
    const size_t rows = (size_t)q->sizes[0] * q->sizes[1] * q->sizes[2];
    return ((rows * sizeof(float) + 255) / 256) * 256;
}

// Scratch of the wide-head backward behind the delta rows: the P_low and dS_low matrices of one pass.
// A pass covers as many K/V heads (with their query heads) of one batch element as fit 2 GiB per matrix,
// or the whole call when everything fits.  When a single K/V head's group alone exceeds the limit the
// passes also run over key ranges of that group: the matrices then hold [group, Sq, keys_per_pass] and dQ
// is accumulated over the key ranges in an FP32 buffer behind them.  Zero when the head is not wide.
// KFA_WIDE_MATRIX_BYTES overrides the limit (a smaller value trades workspace for more passes).
size_t wide_matrix_limit() {
    if (const char* text = std::getenv("KFA_WIDE_MATRIX_BYTES")) {
        const long long value = std::atoll(text);
        if (value > 0) return (size_t)value;
    }
    return size_t(2) << 30;
}

struct WidePlan {
    int heads_per_pass = 0;   // K/V heads per pass; 0 = not a wide-head call
    bool single = false;      // one pass over the whole call (all batches)
    int keys_per_pass = 0;    // > 0: passes over key ranges of one K/V head group (a multiple of 128)
    size_t matrix_bytes = 0;  // one stored matrix of a pass
    size_t dq_bytes = 0;      // FP32 dQ partial sums of one head group (key-range passes only)
};

WidePlan wide_plan(const kfa_tensor* q, const kfa_tensor* k) {
    WidePlan plan;
    if (!q || !k || q->ndim != 4 || k->ndim != 4) return plan;
    const int64_t D = q->sizes[3];
    if (D != 256 && D != 384 && D != 512) return plan;
    const int64_t B = q->sizes[0], Hq = q->sizes[1], Hkv = k->sizes[1], Sq = q->sizes[2], Sk = k->sizes[2];
    if (Hkv <= 0 || Hq % Hkv != 0) return plan;
    const size_t kWideMatrixLimit = wide_matrix_limit();
    const size_t all = kfa::wide_stored_bytes(B, Hq, Sq, Sk);
    if (all <= kWideMatrixLimit) {
        plan.heads_per_pass = (int)Hkv;
        plan.single = true;
        plan.matrix_bytes = all;
        return plan;
    }
    const int64_t group = Hq / Hkv;
    const size_t one_group = kfa::wide_stored_bytes(1, group, Sq, Sk);
    if (one_group > kWideMatrixLimit) {
        // key ranges of one head group: as many 128-key tiles as the limit holds, at least one
        const int64_t tile_bytes = group * Sq * 128 * 2;
        const int64_t tiles = std::max<int64_t>(1, (int64_t)(kWideMatrixLimit / (size_t)tile_bytes));
        plan.heads_per_pass = 1;
        plan.keys_per_pass = (int)std::min<int64_t>(tiles * 128, (Sk + 127) / 128 * 128);
        plan.matrix_bytes = kfa::wide_stored_bytes(1, group, Sq, plan.keys_per_pass);
        plan.dq_bytes = ((size_t)(group * Sq * D) * sizeof(float) + 255) / 256 * 256;
        return plan;
    }
    plan.heads_per_pass = (int)std::min<int64_t>(Hkv, (int64_t)(kWideMatrixLimit / one_group));
    plan.matrix_bytes = kfa::wide_stored_bytes(1, group * plan.heads_per_pass, Sq, Sk);
    return plan;
}

size_t wide_extra_bytes(const kfa_tensor* q, const kfa_tensor* k) {
    const WidePlan plan = wide_plan(q, k);
    return 2 * plan.matrix_bytes + plan.dq_bytes;
}

// The same call restricted to batch element b and K/V heads [h0, h0 + n).
kfa::AttnParams wide_slice(const kfa::AttnParams& p, int b, int h0, int n) {
    kfa::AttnParams s = p;
    const int g = p.group, q0 = h0 * g;
    auto shift = [](const void* base, int64_t elements) {
        return static_cast<const void*>(static_cast<const char*>(base) + elements * 2);
    };
    s.q = shift(p.q, b * p.qs[0] + q0 * p.qs[1]);
    s.k = shift(p.k, b * p.ks[0] + h0 * p.ks[1]);
    s.v = shift(p.v, b * p.vs[0] + h0 * p.vs[1]);
    s.out = const_cast<void*>(shift(p.out, b * p.os[0] + q0 * p.os[1]));
    s.dout = shift(p.dout, b * p.gs[0] + q0 * p.gs[1]);
    s.dq = const_cast<void*>(shift(p.dq, b * p.dqs[0] + q0 * p.dqs[1]));
    s.dk = const_cast<void*>(shift(p.dk, b * p.dks[0] + h0 * p.dks[1]));
    s.dv = const_cast<void*>(shift(p.dv, b * p.dvs[0] + h0 * p.dvs[1]));
    const int64_t stat = ((int64_t)b * p.Hq + q0) * p.Sq;
    s.maximum = p.maximum + stat;
    s.logsum = p.logsum + stat;
    s.delta = p.delta + stat;
    if (p.has_mask) {
        s.mask = p.mask + b * p.ms[0] + q0 * p.ms[1];
        s.blocks = p.blocks + b * p.bs[0] + q0 * p.bs[1];
    }
    s.B = 1;
    s.Hq = n * g;
    s.Hkv = n;
    return s;
}

// A pass restricted further to keys [k0, k0 + n) of its head group; `position` is 1 first, 2 middle, 3 last.
kfa::AttnParams wide_key_range(const kfa::AttnParams& p, int k0, int n, int position, float* dq_acc) {
    kfa::AttnParams s = p;
    auto shift = [](const void* base, int64_t elements) {
        return static_cast<const void*>(static_cast<const char*>(base) + elements * 2);
    };
    s.k = shift(p.k, (int64_t)k0 * p.ks[2]);
    s.v = shift(p.v, (int64_t)k0 * p.vs[2]);
    s.dk = const_cast<void*>(shift(p.dk, (int64_t)k0 * p.dks[2]));
    s.dv = const_cast<void*>(shift(p.dv, (int64_t)k0 * p.dvs[2]));
    if (p.has_mask) {
        s.mask = p.mask + (int64_t)k0 * p.ms[3];
        s.blocks = p.blocks + (int64_t)(k0 / 64) * p.bs[3];
    }
    s.Sk = n;
    s.causal_shift = -k0;
    s.dq_pass = position;
    s.dq_acc = dq_acc;
    return s;
}

}  // namespace

extern "C" {

int kfa_selected_family(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                        int causal, int backward) {
    if (check_qkv(q, k, v)) return -1;
    kfa::AttnParams p;
    if (fill_common(p, q, k, v, mask, 1.f, causal)) return -1;
    // Output strides follow the inputs (the caller allocates them like q/k/v).
    p.out = const_cast<void*>(q->data);
    copy4(p.os, q->strides);
    p.dout = q->data;
    copy4(p.gs, q->strides);
    p.dq = const_cast<void*>(q->data);
    copy4(p.dqs, q->strides);
    p.dk = const_cast<void*>(k->data);
    copy4(p.dks, k->strides);
    p.dv = const_cast<void*>(v->data);
    copy4(p.dvs, v->strides);
    const bool bf16 = q->dtype == KFA_BF16;
    if (backward) {
        if (kfa::pipeline_backward_supported(p, bf16)) return 1;
        return kfa::wide_backward_supported(p) && wide_extra_bytes(q, k) > 0 ? 2 : 0;
    }
    if (kfa::pipeline_forward_supported(p, bf16)) return 1;
    return kfa::wide_forward_supported(p) ? 2 : 0;
}

int kfa_forward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                kfa_tensor* out, kfa_tensor* maximum, kfa_tensor* logsum, kfa_tensor* blocks, float scale,
                int causal, void* stream) {
    if (int e = check_device_ok()) return e;
    if (int e = check_qkv(q, k, v)) return e;
    kfa::AttnParams p;
    if (int e = fill_common(p, q, k, v, mask, scale, causal, static_cast<cudaStream_t>(stream))) return e;
    if (int e = check_like(out, q, "out")) return e;
    // both statistics, or neither (a forward pass nobody will differentiate keeps none)
    const bool keep_statistics = maximum != nullptr || logsum != nullptr;
    if (keep_statistics && (!contiguous3(maximum, p.B, p.Hq, p.Sq) || !contiguous3(logsum, p.B, p.Hq, p.Sq)))
        return fail(KFA_INVALID_ARGUMENT, "maximum/logsum must be contiguous float32 [B,Hq,Sq] (or both NULL)");
    if (int e = bind_blocks(p, blocks)) return e;
    p.out = out->data;
    copy4(p.os, out->strides);
    p.maximum = keep_statistics ? static_cast<float*>(maximum->data) : nullptr;
    p.logsum = keep_statistics ? static_cast<float*>(logsum->data) : nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf16 = q->dtype == KFA_BF16;
    cudaError_t ce;
    if (p.has_mask) {
        int64_t n[4];
        block_extents(p, n);
        ce = timed("pack_mask", st, [&] { return kfa::launch_pack_mask(p, (int)n[0], (int)n[1], (int)n[2], (int)n[3], st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "pack_mask launch");
    }
    if (kfa::pipeline_forward_supported(p, bf16)) {
        ce = timed("pipeline_forward", st, [&] { return kfa::launch_pipeline_forward(p, bf16, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "pipeline forward launch");
    } else if (kfa::wide_forward_supported(p)) {
        ce = timed("wide_forward", st, [&] { return kfa::launch_wide_forward(p, bf16, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "wide-head forward launch");
    } else {
        ce = timed("general_forward", st, [&] { return kfa::launch_general_forward(p, bf16, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "general forward launch");
    }
    return 0;
}

size_t kfa_forward_decode_workspace_bytes(const kfa_tensor* q, const kfa_tensor* k) {
    if (!q || !k || q->ndim != 4 || k->ndim != 4) return 0;
    return kfa::decode_forward_workspace_bytes(q->sizes[0], q->sizes[1], k->sizes[1], q->sizes[2], k->sizes[2], q->sizes[3]);
}

int kfa_forward_decode(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, kfa_tensor* out,
                       kfa_tensor* maximum, kfa_tensor* logsum, void* workspace, size_t workspace_bytes, float scale,
                       void* stream) {
    if (int e = check_device_ok()) return e;
    if (int e = check_qkv(q, k, v)) return e;
    kfa::AttnParams p;
    if (int e = fill_common(p, q, k, v, nullptr, scale, 0, static_cast<cudaStream_t>(stream))) return e;
    if (int e = check_like(out, q, "out")) return e;
    const bool keep_statistics = maximum != nullptr || logsum != nullptr;
    if (keep_statistics && (!contiguous3(maximum, p.B, p.Hq, p.Sq) || !contiguous3(logsum, p.B, p.Hq, p.Sq)))
        return fail(KFA_INVALID_ARGUMENT, "maximum/logsum must be contiguous float32 [B,Hq,Sq] (or both NULL)");
    p.out = out->data;
    copy4(p.os, out->strides);
    p.maximum = keep_statistics ? static_cast<float*>(maximum->data) : nullptr;
    p.logsum = keep_statistics ? static_cast<float*>(logsum->data) : nullptr;
    if (!kfa::decode_forward_supported(p))
        return fail(KFA_INVALID_ARGUMENT,
                    "decode forward serves at most 8 query rows per K/V head (positions x grouped heads), 64 or 128 "
                    "channels, at least 512 keys, no mask, not causal, a non-zero scale, 8-byte addressable rows");
    if (!workspace || workspace_bytes < kfa_forward_decode_workspace_bytes(q, k) ||
        reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
        return fail(KFA_INVALID_ARGUMENT, "decode forward workspace too small or not 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int launches = 0;
    cudaError_t ce = timed("decode_forward", st, [&] {
        return kfa::launch_decode_forward(p, q->dtype == KFA_BF16, workspace, &launches, st);
    });
    if (ce != cudaSuccess) return cuda_fail(ce, "decode forward launch");
    if (launches > 1) count_kernel("decode_forward", (uint64_t)(launches - 1));
    return 0;
}

int kfa_pack_mask(const kfa_tensor* mask, kfa_tensor* blocks, void* stream) {
    if (!mask || !mask->data || mask->dtype != KFA_BOOL || mask->ndim != 4)
        return fail(KFA_INVALID_ARGUMENT, "pack_mask requires a boolean mask expanded to [B,Hq,Sq,Sk]");
    for (int i = 0; i < 4; ++i)
        if (mask->sizes[i] <= 0 || mask->sizes[i] > INT32_MAX) return fail(KFA_INVALID_ARGUMENT, "pack_mask: bad extent");
    kfa::AttnParams p;
    std::memset(&p, 0, sizeof(p));
    p.B = (int)mask->sizes[0];
    p.Hq = (int)mask->sizes[1];
    p.Sq = (int)mask->sizes[2];
    p.Sk = (int)mask->sizes[3];
    p.mask = static_cast<const uint8_t*>(mask->data);
    copy4(p.ms, mask->strides);
    p.has_mask = 1;
    if (int e = bind_blocks(p, blocks)) return e;
    int64_t n[4];
    block_extents(p, n);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t ce =
        timed("pack_mask", st, [&] { return kfa::launch_pack_mask(p, (int)n[0], (int)n[1], (int)n[2], (int)n[3], st); });
    if (ce != cudaSuccess) return cuda_fail(ce, "pack_mask launch");
    return 0;
}

size_t kfa_backward_workspace_bytes(const kfa_tensor* q, const kfa_tensor* k) {
    if (!q || q->ndim != 4) return 0;
    return delta_bytes(q) + wide_extra_bytes(q, k);
}

}  // extern "C"

namespace {

// FP32 gradient tensor of a block-wise call: the shape of `like`, float32, channel-contiguous.
int check_f32_like(const kfa_tensor* t, const kfa_tensor* like, const char* name) {
    if (!t || !t->data || t->dtype != KFA_F32 || !same_shape(t, like) || t->strides[3] != 1)
        return fail(KFA_INVALID_ARGUMENT, "%s must be a float32 tensor with the shape of its source and unit channel stride", name);
    return 0;
}

// grad_f32 = 0: the operator's backward.  Otherwise the block-wise form: FP32 gradients (bit 0), added to dq
// (bit 1) and to dk, dv (bit 2) instead of overwriting them.
int backward_impl(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                  const kfa_tensor* out, const kfa_tensor* maximum, const kfa_tensor* logsum, const kfa_tensor* dout,
                  const kfa_tensor* blocks, kfa_tensor* dq, kfa_tensor* dk, kfa_tensor* dv, void* workspace,
                  size_t workspace_bytes, float scale, int causal, int grad_f32, void* stream) {
    if (int e = check_device_ok()) return e;
    if (int e = check_qkv(q, k, v)) return e;
    kfa::AttnParams p;
    if (int e = fill_common(p, q, k, v, mask, scale, causal, static_cast<cudaStream_t>(stream))) return e;
    if (int e = check_like(out, q, "out")) return e;
    if (int e = check_like(dout, q, "dout")) return e;
    if (grad_f32) {
        if (int e = check_f32_like(dq, q, "dq")) return e;
        if (int e = check_f32_like(dk, k, "dk")) return e;
        if (int e = check_f32_like(dv, v, "dv")) return e;
    } else {
        if (int e = check_like(dq, q, "dq")) return e;
        if (int e = check_like(dk, k, "dk")) return e;
        if (int e = check_like(dv, v, "dv")) return e;
    }
    p.grad_f32 = grad_f32;
    if (!contiguous3(maximum, p.B, p.Hq, p.Sq) || !contiguous3(logsum, p.B, p.Hq, p.Sq))
        return fail(KFA_INVALID_ARGUMENT, "maximum/logsum must be contiguous float32 [B,Hq,Sq]");
    if (int e = bind_blocks(p, blocks)) return e;
    if (!workspace || workspace_bytes < kfa_backward_workspace_bytes(q, k) ||
        reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return fail(KFA_INVALID_ARGUMENT, "backward workspace too small or not 256-byte aligned");
    p.out = const_cast<void*>(out->data);
    copy4(p.os, out->strides);
    p.maximum = static_cast<float*>(maximum->data);
    p.logsum = static_cast<float*>(logsum->data);
    p.dout = dout->data;
    copy4(p.gs, dout->strides);
    p.delta = static_cast<float*>(workspace);
    p.dq = dq->data;
    copy4(p.dqs, dq->strides);
    p.dk = dk->data;
    copy4(p.dks, dk->strides);
    p.dv = dv->data;
    copy4(p.dvs, dv->strides);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf16 = q->dtype == KFA_BF16;
    const bool pipeline = kfa::pipeline_backward_supported(p, bf16);
    if (grad_f32 && !pipeline)
        return fail(KFA_INVALID_ARGUMENT,
                    "block-wise backward needs the tensor-memory pipeline family: head dims that are multiples of 8 "
                    "up to 128, 16-byte addressable rows, a non-zero scale and at least two keys");
    const bool wide = !pipeline && kfa::wide_backward_supported(p) && wide_extra_bytes(q, k) > 0;
    // Wide heads: the first score kernel (P_low) needs only the forward's statistics, so delta runs on a side
    // stream beside it and joins before the second score kernel.  (Serial while per-kernel timing is on.)
    Side* delta_side = (wide && !g_profile_on.load(std::memory_order_relaxed)) ? side_stream_for(st) : nullptr;
    cudaStream_t delta_stream = st;
    if (delta_side && cudaEventRecord(delta_side->fork, st) == cudaSuccess &&
        cudaStreamWaitEvent(delta_side->stream, delta_side->fork, 0) == cudaSuccess)
        delta_stream = delta_side->stream;
    cudaError_t ce = timed("output_delta", delta_stream, [&] {
        if (wide) return kfa::launch_wide_delta(p, bf16, delta_stream);
        return pipeline ? kfa::launch_pipeline_delta(p, bf16, st) : kfa::launch_output_delta(p, bf16, st);
    });
    bool delta_joined = delta_stream == st;
    auto join_delta = [&]() -> cudaError_t {
        if (delta_joined) return cudaSuccess;
        delta_joined = true;
        cudaError_t e = cudaEventRecord(delta_side->join, delta_stream);
        return e == cudaSuccess ? cudaStreamWaitEvent(st, delta_side->join, 0) : e;
    };
    if (ce != cudaSuccess) {
        join_delta();
        return cuda_fail(ce, "output_delta launch");
    }
    if (pipeline) {
        // The two gradient owners depend on delta only, not on each other: the key owners go to a side
        // stream so that the query owners' CTAs fill the SMs the first grid frees while it drains.
        // (Not while per-kernel timing is on: an event pair must bracket one kernel alone.)
        Side* side = g_profile_on.load(std::memory_order_relaxed) ? nullptr : side_stream_for(st);
        cudaStream_t kv_stream = st;
        if (side && cudaEventRecord(side->fork, st) == cudaSuccess &&
            cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess)
            kv_stream = side->stream;
        ce = timed("pipeline_backward_kv", kv_stream,
                   [&] { return kfa::launch_pipeline_backward(p, bf16, 1, kv_stream); });
        cudaError_t cq = timed("pipeline_backward_q", st, [&] { return kfa::launch_pipeline_backward(p, bf16, 0, st); });
        if (kv_stream != st) {
            // always join, also after a failed launch: the caller's stream must not lose the side stream
            cudaError_t cj = cudaEventRecord(side->join, kv_stream);
            if (cj == cudaSuccess) cj = cudaStreamWaitEvent(st, side->join, 0);
            if (ce == cudaSuccess) ce = cj;
        }
        if (ce != cudaSuccess) return cuda_fail(ce, "pipeline backward (dK/dV) launch");
        if (cq != cudaSuccess) return cuda_fail(cq, "pipeline backward (dQ) launch");
    } else if (wide) {
        void* stored = static_cast<char*>(workspace) + delta_bytes(q);
        static const char* const names[3] = {"wide_scores_p", "wide_scores_ds", "wide_grad"};
        const WidePlan plan = wide_plan(q, k);
        auto run_pass = [&](const kfa::AttnParams& pass) -> int {
            for (int step = 0; step < 3; ++step) {
                cudaError_t e = timed(names[step], st, [&] { return kfa::launch_wide_backward(pass, bf16, step, stored, st); });
                if (e == cudaSuccess && step == 0) e = join_delta();  // dS_low needs delta
                if (e != cudaSuccess) {
                    join_delta();
                    return cuda_fail(e, "wide-head backward launch");
                }
            }
            return 0;
        };
        if (plan.single) {
            if (int e = run_pass(p)) return e;
        } else if (plan.keys_per_pass > 0) {
            // one head group at a time, key range by key range; dQ partial sums live behind the two matrices
            float* dq_acc = reinterpret_cast<float*>(static_cast<char*>(stored) + 2 * plan.matrix_bytes);
            for (int b = 0; b < p.B; ++b)
                for (int h0 = 0; h0 < p.Hkv; ++h0) {
                    const kfa::AttnParams group = wide_slice(p, b, h0, 1);
                    for (int k0 = 0; k0 < p.Sk; k0 += plan.keys_per_pass) {
                        const int n = std::min(plan.keys_per_pass, p.Sk - k0);
                        const bool first = k0 == 0, last = k0 + n >= p.Sk;
                        const int position = first && last ? 0 : first ? 1 : last ? 3 : 2;
                        if (int e = run_pass(wide_key_range(group, k0, n, position, dq_acc))) return e;
                    }
                }
        } else {
            // the stored matrices are reused pass by pass; passes are ordered on the stream
            for (int b = 0; b < p.B; ++b)
                for (int h0 = 0; h0 < p.Hkv; h0 += plan.heads_per_pass) {
                    const int n = std::min(plan.heads_per_pass, p.Hkv - h0);
                    if (int e = run_pass(wide_slice(p, b, h0, n))) return e;
                }
        }
    } else {
        ce = timed("general_backward_q", st, [&] { return kfa::launch_general_backward(p, bf16, 0, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "general backward (dQ) launch");
        ce = timed("general_backward_kv", st, [&] { return kfa::launch_general_backward(p, bf16, 1, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "general backward (dK/dV) launch");
    }
    return 0;
}

}  // namespace

extern "C" {

int kfa_backward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                 const kfa_tensor* out, const kfa_tensor* maximum, const kfa_tensor* logsum, const kfa_tensor* dout,
                 const kfa_tensor* blocks, kfa_tensor* dq, kfa_tensor* dk, kfa_tensor* dv, void* workspace,
                 size_t workspace_bytes, float scale, int causal, void* stream) {
    return backward_impl(q, k, v, mask, out, maximum, logsum, dout, blocks, dq, dk, dv, workspace, workspace_bytes,
                         scale, causal, 0, stream);
}

int kfa_backward_partial(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                         const kfa_tensor* out, const kfa_tensor* maximum, const kfa_tensor* logsum,
                         const kfa_tensor* dout, const kfa_tensor* blocks, kfa_tensor* dq, kfa_tensor* dk,
                         kfa_tensor* dv, void* workspace, size_t workspace_bytes, float scale, int causal,
                         int accumulate_dq, int accumulate_dkv, void* stream) {
    return backward_impl(q, k, v, mask, out, maximum, logsum, dout, blocks, dq, dk, dv, workspace, workspace_bytes,
                         scale, causal, 1 | (accumulate_dq ? 2 : 0) | (accumulate_dkv ? 4 : 0), stream);
}

int kfa_forward_running(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                        kfa_tensor* acc, kfa_tensor* run_maximum, kfa_tensor* run_sum, kfa_tensor* blocks,
                        float scale, int causal, void* stream) {
    if (int e = check_device_ok()) return e;
    if (int e = check_qkv(q, k, v)) return e;
    kfa::AttnParams p;
    if (int e = fill_common(p, q, k, v, mask, scale, causal, static_cast<cudaStream_t>(stream))) return e;
    if (int e = check_f32_like(acc, q, "acc")) return e;
    auto rows3 = [&](const kfa_tensor* t) {
        return t && t->data && t->dtype == KFA_F32 && t->ndim == 3 && t->sizes[0] == p.B && t->sizes[1] == p.Hq &&
               t->sizes[2] == p.Sq && t->strides[2] == 1;
    };
    if (!rows3(run_maximum) || !rows3(run_sum) || run_maximum->strides[0] != run_sum->strides[0] ||
        run_maximum->strides[1] != run_sum->strides[1])
        return fail(KFA_INVALID_ARGUMENT,
                    "running maximum/sum must be float32 [B,Hq,Sq] with unit row stride and equal strides");
    p.ss[0] = run_maximum->strides[0];
    p.ss[1] = run_maximum->strides[1];
    if (int e = bind_blocks(p, blocks)) return e;
    p.out = acc->data;
    copy4(p.os, acc->strides);
    p.maximum = static_cast<float*>(run_maximum->data);
    p.run_sum = static_cast<float*>(run_sum->data);
    p.running = 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf16 = q->dtype == KFA_BF16;
    if (!kfa::pipeline_forward_supported(p, bf16))
        return fail(KFA_INVALID_ARGUMENT,
                    "block-wise forward needs the tensor-memory pipeline family: head dims that are multiples of 8 "
                    "up to 128, 16-byte addressable rows, a non-zero scale and at least two keys");
    cudaError_t ce;
    if (p.has_mask) {
        int64_t n[4];
        block_extents(p, n);
        ce = timed("pack_mask", st, [&] { return kfa::launch_pack_mask(p, (int)n[0], (int)n[1], (int)n[2], (int)n[3], st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "pack_mask launch");
    }
    ce = timed("pipeline_forward", st, [&] { return kfa::launch_pipeline_forward(p, bf16, st); });
    if (ce != cudaSuccess) return cuda_fail(ce, "pipeline forward launch");
    return 0;
}

int kfa_finish_running(const kfa_tensor* acc, const kfa_tensor* run_maximum, const kfa_tensor* run_sum,
                       kfa_tensor* out, kfa_tensor* maximum, kfa_tensor* logsum, void* stream) {
    if (!acc || !out || !acc->data || !out->data || acc->ndim != 4 || out->ndim != 4 || !same_shape(acc, out) ||
        acc->dtype != KFA_F32 || !is_half_type(out) || acc->strides[3] != 1)
        return fail(KFA_INVALID_ARGUMENT, "finish requires a float32 accumulator and an FP16/BF16 output of one 4D shape");
    const int64_t B = acc->sizes[0], H = acc->sizes[1], S = acc->sizes[2], D = acc->sizes[3];
    if (B * H * S > INT32_MAX * int64_t(4)) return fail(KFA_TOO_LARGE, "finish: too many rows");
    if (!contiguous3(run_maximum, B, H, S) || !contiguous3(run_sum, B, H, S) || !contiguous3(maximum, B, H, S) ||
        !contiguous3(logsum, B, H, S))
        return fail(KFA_INVALID_ARGUMENT, "finish statistics must be contiguous float32 [B,H,S]");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t ce = timed("finish_running", st, [&] {
        return kfa::launch_finish_running(out->data, static_cast<float*>(maximum->data),
                                          static_cast<float*>(logsum->data), static_cast<const float*>(acc->data),
                                          static_cast<const float*>(run_maximum->data),
                                          static_cast<const float*>(run_sum->data), out->dtype == KFA_BF16, (int)B,
                                          (int)H, (int)S, (int)D, acc->strides, out->strides, st);
    });
    if (ce != cudaSuccess) return cuda_fail(ce, "finish launch");
    return 0;
}

size_t kfa_center_keys_workspace_bytes(const kfa_tensor* k) {
    if (!k || k->ndim != 4) return 0;
    // 32 sequence splits of partial column sums plus the means
    return ((size_t)k->sizes[0] * k->sizes[1] * k->sizes[3] * sizeof(float) * 33 + 255) / 256 * 256;
}

int kfa_center_keys(const kfa_tensor* k, kfa_tensor* centered, void* workspace, size_t workspace_bytes, void* stream) {
    if (!k || !k->data || k->ndim != 4 || !is_half_type(k))
        return fail(KFA_INVALID_ARGUMENT, "center_keys requires a 4D FP16/BF16 tensor");
    if (int e = check_like(centered, k, "centered")) return e;
    if (!workspace || workspace_bytes < kfa_center_keys_workspace_bytes(k))
        return fail(KFA_INVALID_ARGUMENT, "center_keys workspace too small");
    for (int i = 0; i < 4; ++i)
        if (k->sizes[i] <= 0 || k->sizes[i] > INT32_MAX) return fail(KFA_INVALID_ARGUMENT, "center_keys: bad extent");
    if (k->sizes[0] * k->sizes[1] > INT32_MAX / 8) return fail(KFA_TOO_LARGE, "center_keys: batch*heads exceeds 2^28");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int launches = 0;
    cudaError_t ce = timed("center_keys", st, [&] {
        return kfa::launch_center_keys(k->data, centered->data, static_cast<float*>(workspace), k->dtype == KFA_BF16,
                                       (int)k->sizes[0], (int)k->sizes[1], (int)k->sizes[2], (int)k->sizes[3],
                                       k->strides, centered->strides, st, &launches);
    });
    if (ce != cudaSuccess) return cuda_fail(ce, "center_keys launch");
    // one launch (thread-block clusters) or three (partial sums, means, subtraction)
    if (launches > 1) count_kernel("center_keys", (uint64_t)(launches - 1));
    return 0;
}

int kfa_neighborhood_forward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, kfa_tensor* out,
                             kfa_tensor* maximum, kfa_tensor* logsum, const int64_t* spatial, int nd,
                             const int64_t* window, float scale, void* stream) {
    if (int e = check_device_ok()) return e;
    if (int e = check_qkv(q, k, v)) return e;
    kfa::AttnParams p;
    if (int e = fill_common(p, q, k, v, nullptr, scale, 0, static_cast<cudaStream_t>(stream))) return e;
    if (int e = geometry(p, spatial, nd, window)) return e;
    if (int e = check_like(out, q, "out")) return e;
    if (!contiguous3(maximum, p.B, p.Hq, p.Sq) || !contiguous3(logsum, p.B, p.Hq, p.Sq))
        return fail(KFA_INVALID_ARGUMENT, "maximum/logsum must be contiguous float32 [B,H,S]");
    p.out = out->data;
    copy4(p.os, out->strides);
    p.maximum = static_cast<float*>(maximum->data);
    p.logsum = static_cast<float*>(logsum->data);
    p.two_term = nd == 3 ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf16 = q->dtype == KFA_BF16;
    cudaError_t ce = kfa::na_pipeline_forward_supported(p)
                         ? timed("na_pipeline_forward", st, [&] { return kfa::launch_na_pipeline_forward(p, bf16, st); })
                         : timed("neighborhood_forward", st,
                                 [&] { return kfa::launch_neighborhood_forward(p, bf16, st); });
    if (ce != cudaSuccess) return cuda_fail(ce, "neighborhood forward launch");
    return 0;
}

size_t kfa_neighborhood_backward_workspace_bytes(const kfa_tensor* q) {
    if (!q || q->ndim != 4) return 0;
    const size_t rows = (size_t)q->sizes[0] * q->sizes[1] * q->sizes[2];
    return 2 * (((rows * sizeof(float) + 255) / 256) * 256);
}

int kfa_neighborhood_backward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* out,
                              const kfa_tensor* maximum, const kfa_tensor* logsum, const kfa_tensor* dout,
                              kfa_tensor* dq, kfa_tensor* dk, kfa_tensor* dv, void* workspace, size_t workspace_bytes,
                              const int64_t* spatial, int nd, const int64_t* window, float scale, void* stream) {
    if (int e = check_device_ok()) return e;
    if (int e = check_qkv(q, k, v)) return e;
    kfa::AttnParams p;
    if (int e = fill_common(p, q, k, v, nullptr, scale, 0, static_cast<cudaStream_t>(stream))) return e;
    if (int e = geometry(p, spatial, nd, window)) return e;
    if (int e = check_like(out, q, "out")) return e;
    if (int e = check_like(dout, q, "dout")) return e;
    if (int e = check_like(dq, q, "dq")) return e;
    if (int e = check_like(dk, k, "dk")) return e;
    if (int e = check_like(dv, v, "dv")) return e;
    if (!contiguous3(maximum, p.B, p.Hq, p.Sq) || !contiguous3(logsum, p.B, p.Hq, p.Sq))
        return fail(KFA_INVALID_ARGUMENT, "maximum/logsum must be contiguous float32 [B,H,S]");
    const size_t need = kfa_neighborhood_backward_workspace_bytes(q);
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return fail(KFA_INVALID_ARGUMENT, "neighborhood backward workspace too small or not 256-byte aligned");
    p.out = const_cast<void*>(out->data);
    copy4(p.os, out->strides);
    p.maximum = static_cast<float*>(maximum->data);
    p.logsum = static_cast<float*>(logsum->data);
    p.dout = dout->data;
    copy4(p.gs, dout->strides);
    p.delta = static_cast<float*>(workspace);
    p.aux = reinterpret_cast<float*>(static_cast<char*>(workspace) + need / 2);
    p.dq = dq->data;
    copy4(p.dqs, dq->strides);
    p.dk = dk->data;
    copy4(p.dks, dk->strides);
    p.dv = dv->data;
    copy4(p.dvs, dv->strides);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool bf16 = q->dtype == KFA_BF16;
    const bool tensor_path = kfa::na_pipeline_backward_supported(p);
    cudaError_t ce = timed("output_delta", st, [&] {
        return tensor_path ? kfa::launch_pipeline_delta(p, bf16, st) : kfa::launch_output_delta(p, bf16, st);
    });
    if (ce != cudaSuccess) return cuda_fail(ce, "output_delta launch");
    if (tensor_path) {
        ce = timed("na_pipeline_backward_q", st, [&] { return kfa::launch_na_pipeline_backward(p, bf16, 0, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "neighborhood pipeline backward (dQ) launch");
        ce = timed("na_pipeline_backward_kv", st, [&] { return kfa::launch_na_pipeline_backward(p, bf16, 1, st); });
        if (ce != cudaSuccess) return cuda_fail(ce, "neighborhood pipeline backward (dK/dV) launch");
        return 0;
    }
    ce = timed("neighborhood_backward_q", st, [&] { return kfa::launch_neighborhood_backward(p, bf16, 0, st); });
    if (ce != cudaSuccess) return cuda_fail(ce, "neighborhood backward (dQ) launch");
    ce = timed("neighborhood_backward_kv", st, [&] { return kfa::launch_neighborhood_backward(p, bf16, 1, st); });
    if (ce != cudaSuccess) return cuda_fail(ce, "neighborhood backward (dK/dV) launch");
    return 0;
}

int kfa_merge_splits(kfa_tensor* out, kfa_tensor* maximum, kfa_tensor* logsum, const kfa_tensor* part_out,
                     const kfa_tensor* part_maximum, const kfa_tensor* part_logsum, float scale, void* stream) {
    if (!out || !out->data || out->ndim != 4 || !is_half_type(out))
        return fail(KFA_INVALID_ARGUMENT, "merge_splits requires a 4D FP16/BF16 output");
    if (!part_out || !part_out->data || part_out->ndim != 5 || part_out->dtype != out->dtype)
        return fail(KFA_INVALID_ARGUMENT, "merge_splits requires [splits,B,H,S,D] partial outputs of the output's type");
    const int64_t P = part_out->sizes[0], B = out->sizes[0], H = out->sizes[1], S = out->sizes[2], D = out->sizes[3];
    if (P < 1 || P > 1024 || part_out->sizes[1] != B || part_out->sizes[2] != H || part_out->sizes[3] != S ||
        part_out->sizes[4] != D || part_out->strides[4] != 1 || part_out->strides[3] != D ||
        part_out->strides[2] != S * D || part_out->strides[1] != H * S * D || part_out->strides[0] != B * H * S * D)
        return fail(KFA_INVALID_ARGUMENT, "merge_splits requires contiguous [splits,B,H,S,D] partial outputs");
    auto stats_ok = [&](const kfa_tensor* t) {
        return t && t->data && t->dtype == KFA_F32 && t->ndim == 4 && t->sizes[0] == P && t->sizes[1] == B &&
               t->sizes[2] == H && t->sizes[3] == S && t->strides[3] == 1 && t->strides[2] == S &&
               t->strides[1] == H * S && t->strides[0] == B * H * S;
    };
    if (!stats_ok(part_maximum) || !stats_ok(part_logsum))
        return fail(KFA_INVALID_ARGUMENT, "merge_splits requires contiguous float32 [splits,B,H,S] partial statistics");
    const bool keep = maximum != nullptr || logsum != nullptr;
    if (keep && (!contiguous3(maximum, B, H, S) || !contiguous3(logsum, B, H, S)))
        return fail(KFA_INVALID_ARGUMENT, "maximum/logsum must be contiguous float32 [B,H,S] (or both NULL)");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t ce = timed("merge_splits", st, [&] {
        return kfa::launch_merge_splits(out->data, keep ? static_cast<float*>(maximum->data) : nullptr,
                                        keep ? static_cast<float*>(logsum->data) : nullptr, part_out->data,
                                        static_cast<const float*>(part_maximum->data),
                                        static_cast<const float*>(part_logsum->data), out->dtype == KFA_BF16, (int)P,
                                        (int)B, (int)H, (int)S, (int)D, out->strides, scale, st);
    });
    if (ce != cudaSuccess) return cuda_fail(ce, "merge_splits launch");
    return 0;
}

int kfa_merge_partial(kfa_tensor* acc_out, kfa_tensor* acc_maximum, kfa_tensor* acc_logsum, const kfa_tensor* part_out,
                      const kfa_tensor* part_maximum, const kfa_tensor* part_logsum, float scale, void* stream) {
    if (!acc_out || !part_out || acc_out->ndim != 4 || part_out->ndim != 4 || !same_shape(acc_out, part_out))
        return fail(KFA_INVALID_ARGUMENT, "merge requires matching 4D outputs");
    if (acc_out->dtype != KFA_F32 || !is_half_type(part_out))
        return fail(KFA_INVALID_ARGUMENT, "merge requires an FP32 running output and an FP16/BF16 partial output");
    const int64_t B = acc_out->sizes[0], H = acc_out->sizes[1], S = acc_out->sizes[2], D = acc_out->sizes[3];
    if (acc_out->strides[3] != 1 || acc_out->strides[2] != D || acc_out->strides[1] != S * D ||
        acc_out->strides[0] != H * S * D)
        return fail(KFA_INVALID_ARGUMENT, "merge requires a contiguous running output");
    if (!contiguous3(acc_maximum, B, H, S) || !contiguous3(acc_logsum, B, H, S) ||
        !contiguous3(part_maximum, B, H, S) || !contiguous3(part_logsum, B, H, S))
        return fail(KFA_INVALID_ARGUMENT, "merge statistics must be contiguous float32 [B,H,S]");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t ce = timed("merge_partial", st, [&] {
        return kfa::launch_merge_partial(
            static_cast<float*>(acc_out->data), static_cast<float*>(acc_maximum->data),
            static_cast<float*>(acc_logsum->data), part_out->data, static_cast<const float*>(part_maximum->data),
            static_cast<const float*>(part_logsum->data), part_out->dtype == KFA_BF16, (int)B, (int)H, (int)S, (int)D,
            part_out->strides, scale, st);
    });
    if (ce != cudaSuccess) return cuda_fail(ce, "merge launch");
    return 0;
}

}  // extern "C"
