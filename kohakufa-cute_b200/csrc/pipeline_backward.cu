// Attention backward on the tensor-memory pipeline.
#include "kfa_common.cuh"
#include "launchers.h"

namespace kfa {

int pipeline_forward_variants();
void pipeline_forward_forget();

bool pipeline_backward_supported(const AttnParams& p, bool bf16) {
    (void)p;
    (void)bf16;
    return false;
}
cudaError_t launch_pipeline_backward(const AttnParams& p, bool bf16, int which, cudaStream_t st) {
    (void)which;
    (void)p;
    (void)bf16;
    (void)st;
    return cudaErrorNotSupported;
}
int pipeline_configured_variants() { return pipeline_forward_variants(); }
void pipeline_forget_variants() { pipeline_forward_forget(); }

}  // namespace kfa
