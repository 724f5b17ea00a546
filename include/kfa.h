/*
 * kfa.h - C ABI of the B200-native attention library (libkfa.so).
 *
 * Every entry point takes plain pointers, sizes and strides; no C++ or PyTorch
 * types cross this boundary.  All tensors live in device memory and are
 * allocated by the caller (outputs and scratch included, except for the one
 * entry point that says otherwise), so that a caller using a caching allocator
 * can capture the calls in a CUDA graph.  The library keeps no tensor pointer
 * between calls.  Kernels are enqueued on the `stream` argument (a
 * cudaStream_t passed as void*; NULL is the legacy default stream) of the
 * device that is current on the calling thread.
 *
 * Return value: 0 on success, non-zero on failure; the message is available
 * from kfa_last_error() on the same thread.  Nothing throws or aborts.
 *
 * Citations of the form `native.cpp:NNN` or `api.py:NNN` name the file and
 * line of the reference project (SimpleTuner-io/KohakuFA-CuTe,
 * src/kohakufa_cute/...) whose host interface the entry point replaces.
 */
#ifndef KFA_H
#define KFA_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define KFA_API __attribute__((visibility("default")))
#else
#define KFA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum kfa_dtype { KFA_F16 = 0, KFA_BF16 = 1, KFA_F32 = 2, KFA_BOOL = 3, KFA_I32 = 4 };

/* Non-owning tensor description; strides are in elements.  The reference passes
 * the same information as non-owning DLTensor views (native.cpp:205-210). */
typedef struct kfa_tensor {
    void* data;
    int32_t dtype; /* enum kfa_dtype */
    int32_t ndim;  /* <= 6 */
    int64_t sizes[6];
    int64_t strides[6];
} kfa_tensor;

/* Error codes. */
enum kfa_status {
    KFA_OK = 0,
    KFA_INVALID_ARGUMENT = 1, /* shapes, dtypes or strides the operator does not accept */
    KFA_CUDA_ERROR = 2,       /* a CUDA runtime/driver call failed */
    KFA_DEVICE_TIMEOUT = 3,   /* a bounded device-side wait ran out (reported by kfa_device_status) */
    KFA_TOO_LARGE = 4         /* problem exceeds a stated fixed capacity */
};

/* Library identity: (major << 16) | minor. */
KFA_API int kfa_version(void);

/* Message of the last failure on the calling thread ("" when none). */
KFA_API const char* kfa_last_error(void);

/*
 * Sets up the per-device state of the device that is current on the calling thread (a status word in
 * mapped host memory and a small flag in device memory).  The first launching call on a device does
 * the same implicitly; call kfa_init() instead when that first call would otherwise fall inside a
 * stream capture, where allocating is not allowed (the launching entry points then fail with
 * KFA_CUDA_ERROR and a message that says so, rather than breaking the capture).  Idempotent.
 * (No counterpart in the reference, whose host launcher allocates through PyTorch.)
 */
KFA_API int kfa_init(void);

/*
 * Attention forward.  Replaces the module function `forward` of the reference's
 * host launcher (native.cpp:1034-1037, forward_canonical native.cpp:294-314).
 *
 *   q [B,Hq,Sq,D], k,v [B,Hkv,Sk,D]  fp16 or bf16, any strides, Hq % Hkv == 0, 1 <= D <= 512
 *   mask     NULL, or a bool tensor already expanded to [B,Hq,Sq,Sk] (stride 0 on broadcast axes)
 *   out      [B,Hq,Sq,D] same dtype as q (the caller gives it q's strides)
 *   maximum  [B,Hq,Sq] f32: row maximum of the unscaled scores times sign(scale)
 *   logsum   [B,Hq,Sq] f32: log2 of the softmax normaliser relative to `maximum`
 *   blocks   int32 tile table [Bm,Hm,ceil(Sq/64) or 1,ceil(Sk/64) or 1] written when mask != NULL
 *            (extent 1 on the mask's stride-0 axes); NULL when mask == NULL
 * A row with no visible key yields out = 0, maximum = -inf, logsum = 0.
 * `maximum` and `logsum` may both be NULL: the statistics exist for the backward pass, and a forward
 * call that nobody will differentiate (inference; the reference lists this mode as an open item,
 * results/README.md:120-129) then writes the output only.
 */
KFA_API int kfa_forward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                kfa_tensor* out, kfa_tensor* maximum, kfa_tensor* logsum, kfa_tensor* blocks, float scale,
                int causal, void* stream);

/*
 * Classifies the 64x64 tiles of an expanded boolean mask (0 hidden, 1 mixed, 2 fully visible) into
 * `blocks`, laid out as kfa_forward documents.  kfa_forward does this itself; the separate entry
 * point serves callers that run kfa_backward against a (query shard, key block) pair for which no
 * forward call produced a table.  Replaces the PackMask kernel launch (kernels.py:3170-3198).
 */
KFA_API int kfa_pack_mask(const kfa_tensor* mask, kfa_tensor* blocks, void* stream);

/* Bytes of scratch kfa_backward needs for these shapes (native.cpp:341-354 sizes the
 * same buffers: delta and its base).  For heads of 256, 384 or 512 channels the figure also
 * covers two 16-bit [B,Hq,Sq,ceil128(Sk)] matrices (rounded probabilities and score gradients)
 * that the wide-head tensor-core backward stores once and multiplies three times.  Above 2 GiB
 * per matrix (environment variable KFA_WIDE_MATRIX_BYTES overrides the limit) the backward runs in
 * passes over batch elements and K/V-head groups that reuse one pass-sized pair of matrices; only
 * when a single K/V head's group exceeds the limit are they left out and the general kernels run. */
KFA_API size_t kfa_backward_workspace_bytes(const kfa_tensor* q, const kfa_tensor* k);

/*
 * Attention backward.  Replaces `backward` (native.cpp:1038-1042, 341-358).
 * Reads the forward's saved out/maximum/logsum/blocks; writes dq (like q) and dk, dv (like k, v).
 * `workspace` must hold kfa_backward_workspace_bytes() bytes, 256-byte aligned.
 */
KFA_API int kfa_backward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                 const kfa_tensor* out, const kfa_tensor* maximum, const kfa_tensor* logsum,
                 const kfa_tensor* dout, const kfa_tensor* blocks, kfa_tensor* dq, kfa_tensor* dk,
                 kfa_tensor* dv, void* workspace, size_t workspace_bytes, float scale, int causal,
                 void* stream);

/*
 * Key centering: centered = round(f32(k) - mean over the sequence axis of f32(k)) per
 * (batch, head, channel).  Replaces the PyTorch expression at api.py:100-103.  The same
 * entry point computes the gradient projection (apply it to the centred-key gradient).
 * `workspace` holds kfa_center_keys_workspace_bytes() bytes (partial column sums and the means).
 */
KFA_API size_t kfa_center_keys_workspace_bytes(const kfa_tensor* k);
KFA_API int kfa_center_keys(const kfa_tensor* k, kfa_tensor* centered, void* workspace, size_t workspace_bytes,
                    void* stream);

/*
 * Key centering for callers that must not allocate: same result as kfa_center_keys, but the
 * scratch lives in a fixed array inside the library image instead of caller memory, and the
 * call makes no allocation of any kind.  (This entry point has no counterpart in the reference
 * project.)  Limits and rules:
 *   - batch * heads * channels must not exceed kfa_center_keys_static_limit() (16384); larger
 *     problems return KFA_TOO_LARGE and launch nothing;
 *   - every GPU that loads the library holds the array (about 2.1 MB) until the process exits;
 *   - shapes the one-launch thread-block-cluster kernel serves (64/128/256/512 channels, >= 64 rows,
 *     16-byte addressable rows, slab fits in shared memory) need no scratch and leave the array alone;
 *     all other calls share the array, and such calls that overlap in time on one GPU race with each other;
 *   - the first call on a device looks up the array's address; make it before any stream capture.
 */
KFA_API size_t kfa_center_keys_static_limit(void);
KFA_API int kfa_center_keys_static(const kfa_tensor* k, kfa_tensor* centered, void* stream);

/*
 * Neighbourhood (shifted-window) attention, head dim 64, equal Q/K/V shapes
 * [B,H,prod(spatial),64].  Replaces `neighborhood_forward` (native.cpp:1043-1054) and the
 * Python-side backward launch (neighborhood_kernels.py:408-411).  `nd` is 2 or 3.
 * The 3-D forward uses the two-term probability product.
 */
KFA_API int kfa_neighborhood_forward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, kfa_tensor* out,
                             kfa_tensor* maximum, kfa_tensor* logsum, const int64_t* spatial, int nd,
                             const int64_t* window, float scale, void* stream);
KFA_API size_t kfa_neighborhood_backward_workspace_bytes(const kfa_tensor* q);
KFA_API int kfa_neighborhood_backward(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v,
                              const kfa_tensor* out, const kfa_tensor* maximum, const kfa_tensor* logsum,
                              const kfa_tensor* dout, kfa_tensor* dq, kfa_tensor* dk, kfa_tensor* dv,
                              void* workspace, size_t workspace_bytes, const int64_t* spatial, int nd,
                              const int64_t* window, float scale, void* stream);

/*
 * Merge step of ring context parallelism: folds the partial result of attending to one
 * more key/value block into a running result.  Each side is (out, maximum, logsum) as
 * kfa_forward returns them; `acc_*` are updated in place.  The arithmetic is the
 * (max, sum) merge of the reference's split forward (split_forward.py:219-245).
 *   acc_out/part_out [B,H,S,D] (acc is f32, part is the 16-bit type), stats [B,H,S] f32
 */
KFA_API int kfa_merge_partial(kfa_tensor* acc_out, kfa_tensor* acc_maximum, kfa_tensor* acc_logsum,
                      const kfa_tensor* part_out, const kfa_tensor* part_maximum,
                      const kfa_tensor* part_logsum, float scale, void* stream);

/*
 * Forward for token-by-token decoding against a key/value cache: at most 8 query rows per K/V head (query positions
 * x grouped-query heads), 64 or 128 channels, at least 512 keys, no mask, not causal.  The reference serves short query
 * sequences with its split forward (split_forward.py:125-245); here the call is a CUDA-core kernel bound by the HBM
 * time of K and V (the keys of a head are split over CTAs, partial results merged with the (maximum, sum)
 * arithmetic of split_forward.py:219-245) instead of one 128-row tensor-core tile per head.  Results and statistics
 * follow kfa_forward's contract; maximum/logsum may both be NULL.  Other operands: KFA_INVALID_ARGUMENT.
 *   workspace: kfa_forward_decode_workspace_bytes(q, k) bytes, 16-byte aligned
 */
KFA_API size_t kfa_forward_decode_workspace_bytes(const kfa_tensor* q, const kfa_tensor* k);
KFA_API int kfa_forward_decode(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, kfa_tensor* out,
                       kfa_tensor* maximum, kfa_tensor* logsum, void* workspace, size_t workspace_bytes, float scale,
                       void* stream);

/*
 * Block-wise forms for callers that hold only one block of a longer sequence at a time (ring context
 * parallelism; no counterpart in the reference, whose split forward keeps FP32 partial outputs with (maximum, sum)
 * pairs and merges them afterwards: split_forward.py:125-245).  Nothing is rounded to the 16-bit type between
 * blocks.  Served by the tensor-memory pipeline family only (head dims that are multiples of 8 up to 128, 16-byte
 * addressable rows, non-zero scale, at least two keys); other operands return KFA_INVALID_ARGUMENT.
 *
 * kfa_forward_running attends q to one block (k, v, mask) and folds the result into a running state with the
 * (maximum, sum) merge of split_forward.py:219-245, inside the kernel's epilogue:
 *   acc [B,Hq,Sq,D] f32, unit channel stride: unnormalised output relative to run_maximum (start: zeros)
 *   run_maximum [B,Hq,Sq] f32, unit row stride: unscaled row maximum so far (start: -inf)
 *   run_sum     [B,Hq,Sq] f32, same strides: sum of 2^((s - run_maximum) |scale| log2e) so far (start: zeros)
 * kfa_finish_running divides once, rounds `out` once and writes the statistics of kfa_forward's contract
 * (maximum = run_maximum, logsum = log2(run_sum); rows that saw no key: zeros, -inf, 0).  `maximum` may be the
 * same tensor as `run_maximum`, `logsum` the same as `run_sum`.
 *
 * kfa_backward_partial is kfa_backward for one (query block, key block) pair against the statistics of the whole
 * sequence, with float32 gradients (unit channel stride, any other strides): dq is overwritten or, with
 * accumulate_dq != 0, added to; dk and dv likewise with accumulate_dkv.  Workspace as for kfa_backward.
 */
KFA_API int kfa_forward_running(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                        kfa_tensor* acc, kfa_tensor* run_maximum, kfa_tensor* run_sum, kfa_tensor* blocks,
                        float scale, int causal, void* stream);
KFA_API int kfa_finish_running(const kfa_tensor* acc, const kfa_tensor* run_maximum, const kfa_tensor* run_sum,
                       kfa_tensor* out, kfa_tensor* maximum, kfa_tensor* logsum, void* stream);
KFA_API int kfa_backward_partial(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v, const kfa_tensor* mask,
                         const kfa_tensor* out, const kfa_tensor* maximum, const kfa_tensor* logsum,
                         const kfa_tensor* dout, const kfa_tensor* blocks, kfa_tensor* dq, kfa_tensor* dk,
                         kfa_tensor* dv, void* workspace, size_t workspace_bytes, float scale, int causal,
                         int accumulate_dq, int accumulate_dkv, void* stream);

/*
 * Merge step of a forward pass split over the key axis (short query sequences against long key
 * sequences, where one CTA per head would leave the GPU idle): the caller runs kfa_forward on `splits`
 * key ranges and this call folds the partial results, with the arithmetic of the reference's split
 * forward (split_forward.py:219-245): out = sum_i w_i O_i / sum_i w_i with
 * w_i = 2^((m_i - m) |scale| log2e + logsum_i), m = max_i m_i; the merged statistics describe the whole
 * key range, so the ordinary backward applies.
 *   out [B,H,S,D] 16-bit (any strides); maximum, logsum [B,H,S] f32 or both NULL;
 *   part_out [splits,B,H,S,D] 16-bit contiguous; part_maximum, part_logsum [splits,B,H,S] f32 contiguous
 */
KFA_API int kfa_merge_splits(kfa_tensor* out, kfa_tensor* maximum, kfa_tensor* logsum, const kfa_tensor* part_out,
                     const kfa_tensor* part_maximum, const kfa_tensor* part_logsum, float scale, void* stream);

/* Number of kernel variants configured so far / forget them.  Replace `cache_size`
 * and `clear_cache` (native.cpp:1055-1065). */
KFA_API int kfa_cache_size(void);
KFA_API void kfa_clear_cache(void);

/* Kernels launched by this library since load (all threads) - observability only. */
KFA_API uint64_t kfa_launch_count(void);
/* The same count per kernel family: entry `index` (0, 1, ...) gives a name such as "pipeline_forward" and
 * its launches since load; returns non-zero once `index` is past the last name seen so far. */
KFA_API int kfa_launch_stats(int index, char* name, size_t name_bytes, uint64_t* launches);

/*
 * Per-kernel timing for benchmarks.  While enabled, every launch is bracketed by CUDA events
 * on its own stream.  kfa_profile_collect() waits for the recorded events, adds them to
 * per-kernel totals and returns the number of distinct kernels seen; kfa_profile_entry()
 * reads one total; kfa_profile_reset() clears the totals.  Do not enable while capturing a
 * CUDA graph.
 */
KFA_API void kfa_profile_enable(int on);
KFA_API int kfa_profile_collect(void);
KFA_API int kfa_profile_entry(int index, char* name, size_t name_bytes, double* total_ms, uint64_t* launches);
KFA_API void kfa_profile_reset(void);

/*
 * Device-side status: 0 when no kernel reported a problem, otherwise the code a bounded
 * wait stored when it gave up.  Reading does not synchronise; call after the stream is
 * idle.  `reset` != 0 clears it.  While the status is non-zero every tensor-memory kernel
 * skips its work, and kfa_forward, kfa_backward and the neighbourhood entry points return
 * KFA_DEVICE_TIMEOUT without launching (so no caller is handed unwritten outputs); acknowledge
 * the report with kfa_device_status(1) to resume.
 */
KFA_API int kfa_device_status(int reset);

/*
 * Self-test of the failure-detection chain (no counterpart in the reference): launches `ctas` CTAs
 * that each wait at most `limit_cycles` SM cycles on a barrier that nothing completes.  No fault is
 * raised: the waits run out, the first CTAs report code 9001 through kfa_device_status() and set the
 * launch-wide abort flag; CTAs that start afterwards skip their wait (their number is returned in
 * `skipped`, which may be null).  Until kfa_device_status(1) clears the condition, every tensor-memory
 * kernel of this library skips its work as well.  Synchronises the stream.
 */
KFA_API int kfa_self_test_wait(long long limit_cycles, int ctas, int* skipped, void* stream);

/* Which kernel family kfa_forward / kfa_backward would select for these operands:
 * 0 = general kernels, 1 = tcgen05 tensor-memory pipeline (heads of 64/128 channels),
 * 2 = tcgen05 wide-head kernels (256/384/512 channels).  (The reference exposes its
 * selection through kernels.kernel_configuration, kernels.py:2593-2637.) */
KFA_API int kfa_selected_family(const kfa_tensor* q, const kfa_tensor* k, const kfa_tensor* v,
                        const kfa_tensor* mask, int causal, int backward);

#ifdef __cplusplus
}
#endif
#endif /* KFA_H */
