#include "common.cuh"

namespace mmh3 {

int launch_quantized_attention(const Mmh3QuantizedWorkspace &, void *, int, int,
                               const Mmh3AttentionLayout &, float, const Mmh3VsaWorkspace *, int,
                               const void *, int64_t, cudaStream_t) {
    return NOT_SUPPORTED;
}

} // namespace mmh3
