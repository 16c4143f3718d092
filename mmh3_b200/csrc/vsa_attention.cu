#include "common.cuh"

namespace mmh3 {

int launch_vsa_attention(const void *, const void *, const void *, const void *, int64_t, void *,
                         int, int, const Mmh3AttentionLayout &, float, int,
                         const Mmh3VsaWorkspace &, cudaStream_t) {
    return NOT_SUPPORTED;
}

} // namespace mmh3
