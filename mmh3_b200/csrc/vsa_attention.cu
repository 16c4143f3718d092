#include "common.cuh"

namespace mmh3 {

int launch_vsa_attention(const void *, const void *, const void *, const void *, int64_t, void *,
                         int, int, const Mmh3AttentionLayout &, float, int,
                         const Mmh3VsaWorkspace &, cudaStream_t) {
    return NOT_SUPPORTED;
}

int launch_vsa_attention_quantized(const Mmh3QuantizedWorkspace &, void *, int, int,
                                   const Mmh3AttentionLayout &, float, const Mmh3VsaWorkspace &,
                                   int, const void *, int64_t, cudaStream_t) {
    return NOT_SUPPORTED;
}

} // namespace mmh3
