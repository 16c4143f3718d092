// Ulysses layout changes around the attention of a head-sharded DiT block: before it a rank holds
// its own tokens and every head, after it every token and its own heads. Both directions are pure
// gathers of 16-byte groups, bound by HBM bandwidth. They compute what the reference's
// shard_pack_kernel and shard_unpack_kernel do (crates/mmh3-cuda/kernels/dit.cu:953-1023).
#include "common.cuh"

namespace mmh3 {

namespace {

constexpr int THREADS = 256;
constexpr int GROUP = 8; // 16-bit elements per 16-byte group

// `packed` [tokens][tensors][span][dim] <- `source` [tokens][tensors][heads][dim] at first_head.
__global__ void __launch_bounds__(THREADS)
    shard_pack_kernel(const uint4 *__restrict__ source, uint4 *__restrict__ packed, int64_t groups,
                      int heads, int dim_groups, int first_head, int span) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * THREADS;
    const int64_t run = static_cast<int64_t>(span) * dim_groups; // contiguous on both sides
    for (int64_t index = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; index < groups;
         index += stride) {
        const int64_t outer = index / run; // token * tensors + tensor
        const int64_t inner = index % run;
        packed[index] = __ldg(source + (outer * heads + first_head) * dim_groups + inner);
    }
}

// `output` [tokens][heads][dim] at first_head <- `part` [tokens][span][dim].
__global__ void __launch_bounds__(THREADS)
    shard_unpack_kernel(const uint4 *__restrict__ part, uint4 *__restrict__ output, int64_t groups,
                        int heads, int dim_groups, int first_head, int span) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * THREADS;
    const int64_t run = static_cast<int64_t>(span) * dim_groups;
    for (int64_t index = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; index < groups;
         index += stride) {
        const int64_t token = index / run;
        const int64_t inner = index % run;
        output[(token * heads + first_head) * dim_groups + inner] = __ldg(part + index);
    }
}

// The kernels move 16-byte groups: a pointer off that boundary would fault on the device, so it is
// refused on the host instead.
bool aligned(const void *first, const void *second) {
    return (reinterpret_cast<uintptr_t>(first) | reinterpret_cast<uintptr_t>(second)) % 16 == 0;
}

// Enough CTAs to fill the device several times over, walked with a grid stride.
unsigned grid_for(int64_t groups) {
    const int64_t wanted = (groups + THREADS - 1) / THREADS;
    const int64_t limit = static_cast<int64_t>(multiprocessor_count()) * 16;
    return static_cast<unsigned>(wanted < 1 ? 1 : (limit > 0 && wanted > limit ? limit : wanted));
}

} // namespace

int launch_shard_pack(const void *source, void *packed, int tokens, int tensors, int heads, int dim,
                      int first_head, int span, cudaStream_t stream) {
    if (dim % GROUP != 0 || tokens < 0 || tensors < 0 || span < 0 || first_head < 0 ||
        first_head + span > heads) {
        return INVALID_VALUE;
    }
    const int dim_groups = dim / GROUP;
    const int64_t groups = static_cast<int64_t>(tokens) * tensors * span * dim_groups;
    if (groups == 0) {
        return 0;
    }
    if (source == nullptr || packed == nullptr || !aligned(source, packed)) {
        return INVALID_VALUE;
    }
    shard_pack_kernel<<<grid_for(groups), THREADS, 0, stream>>>(
        static_cast<const uint4 *>(source), static_cast<uint4 *>(packed), groups, heads,
        dim_groups, first_head, span);
    return static_cast<int>(cudaGetLastError());
}

int launch_shard_unpack(const void *part, void *output, int tokens, int heads, int dim,
                        int first_head, int span, cudaStream_t stream) {
    if (dim % GROUP != 0 || tokens < 0 || span < 0 || first_head < 0 || first_head + span > heads) {
        return INVALID_VALUE;
    }
    const int dim_groups = dim / GROUP;
    const int64_t groups = static_cast<int64_t>(tokens) * span * dim_groups;
    if (groups == 0) {
        return 0;
    }
    if (part == nullptr || output == nullptr || !aligned(part, output)) {
        return INVALID_VALUE;
    }
    shard_unpack_kernel<<<grid_for(groups), THREADS, 0, stream>>>(
        static_cast<const uint4 *>(part), static_cast<uint4 *>(output), groups, heads, dim_groups,
        first_head, span);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mmh3
