// Host-side launch functions implemented by the kernel translation units.
#pragma once
#include "kfa_common.cuh"

namespace kfa {

bool general_vector_path(const AttnParams& p, bool backward);
cudaError_t launch_pack_mask(const AttnParams& p, int nb, int nh, int nq, int nk, cudaStream_t st);
cudaError_t launch_general_forward(const AttnParams& p, bool bf16, cudaStream_t st);
cudaError_t launch_output_delta(const AttnParams& p, bool bf16, cudaStream_t st);
cudaError_t launch_general_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st);
// `launches` (may be null) receives the number of kernels launched: 1 for the cluster kernel, 3 for the
// partial-sum path that uses `workspace`.
cudaError_t launch_center_keys(const void* k, void* out, float* workspace, bool bf16, int B, int H, int S, int D,
                               const int64_t* ks, const int64_t* os, cudaStream_t st, int* launches = nullptr);
bool center_keys_cluster_supported(const void* k, const void* out, int B, int H, int S, int D, const int64_t* ks,
                                   const int64_t* os);
// False when this device cannot co-schedule the cluster the one-launch kernel needs (queried once per device).
bool center_keys_cluster_schedulable(bool bf16, int S, int D);
cudaError_t launch_center_keys_cluster(const void* k, void* out, bool bf16, int B, int H, int S, int D,
                                       const int64_t* ks, const int64_t* os, cudaStream_t st);
cudaError_t launch_merge_partial(float* acc, float* am, float* al, const void* part, const float* pm, const float* pl,
                                 bool bf16, int B, int H, int S, int D, const int64_t* ps, float scale,
                                 cudaStream_t st);

cudaError_t launch_merge_splits(void* out, float* maximum, float* logsum, const void* part, const float* pm,
                                const float* pl, bool bf16, int splits, int B, int H, int S, int D, const int64_t* os,
                                float scale, cudaStream_t st);

cudaError_t launch_finish_running(void* out, float* maximum, float* logsum, const float* acc, const float* run_max,
                                  const float* run_sum, bool bf16, int B, int H, int S, int D, const int64_t* as,
                                  const int64_t* os, cudaStream_t st);

// Forward for at most eight query rows per K/V head against a long key sequence (decoding): CUDA-core kernels bound
// by the HBM time of K and V.  `workspace` holds the partial results of the key ranges.
bool decode_forward_supported(const AttnParams& p);
size_t decode_forward_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Sk, int64_t D);
cudaError_t launch_decode_forward(const AttnParams& p, bool bf16, void* workspace, int* launches, cudaStream_t st);

cudaError_t launch_neighborhood_forward(const AttnParams& p, bool bf16, cudaStream_t st);
cudaError_t launch_neighborhood_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st);

// Tensor-memory pipeline family (tcgen05).  `*_supported` says whether the
// operands meet the family's layout requirements.
bool pipeline_forward_supported(const AttnParams& p, bool bf16);
cudaError_t launch_pipeline_forward(const AttnParams& p, bool bf16, cudaStream_t st);
bool pipeline_backward_supported(const AttnParams& p, bool bf16);
cudaError_t launch_pipeline_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st);
cudaError_t launch_pipeline_delta(const AttnParams& p, bool bf16, cudaStream_t st);

// Wide heads (256/384/512 channels) on the tensor-memory pipeline.  The backward needs two 16-bit
// [B,Hq,Sq,ceil128(Sk)] matrices (`wide_stored_bytes` each) behind the delta scratch.
bool wide_forward_supported(const AttnParams& p);
cudaError_t launch_wide_forward(const AttnParams& p, bool bf16, cudaStream_t st);
size_t wide_stored_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Sk);
bool wide_backward_supported(const AttnParams& p);
cudaError_t launch_wide_delta(const AttnParams& p, bool bf16, cudaStream_t st);
cudaError_t launch_wide_backward(const AttnParams& p, bool bf16, int step, void* stored, cudaStream_t st);

// Neighbourhood attention on the tensor-memory pipeline (dense tiles + per-row window bit masks).
bool na_pipeline_forward_supported(const AttnParams& p);
cudaError_t launch_na_pipeline_forward(const AttnParams& p, bool bf16, cudaStream_t st);
bool na_pipeline_backward_supported(const AttnParams& p);
cudaError_t launch_na_pipeline_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st);

// Failure-detection self-test: CTAs wait `limit` cycles on a barrier nothing completes.
cudaError_t launch_wait_probe(int* status, int* abort_flag, long long limit, int ctas, int* skipped, cudaStream_t st);

int pipeline_configured_variants();
void pipeline_forget_variants();

}  // namespace kfa
