// VSA's tile selection: per head and query tile, the pooled scores against every tile, the exact
// set of tiles it attends token by token, and the coarse output softmax(scores) . mean values.
//
// The routes are bit-identical to the reference's select_kernel
// (crates/mmh3-cuda/kernels/vsa_attention.cu:96-273). That fixes the FP32 evaluation order of a
// score: 32 chains of four fused multiply-adds over dimensions l, l + 32, l + 64, l + 96, summed
// over a balanced tree that pairs chains by bit 4 of l first and by bit 0 last, then one multiply
// by the scale. Here one thread evaluates that whole tree: it holds one pooled key in registers and
// scores it against each of its CTA's eight query tiles, whose pooled queries sit in shared
// memory, two chains to a packed operation; the reference spreads a score over the lanes of a warp. The selection itself
// is a function of the scores alone, so it is free to differ: here a warp finds the kept-th
// largest video score with a four-pass radix select over
// order-preserving integer keys (the reference descends one bit at a time), ties go to the lower
// tile index, and the route is an ascending list of uint16 tile indices.
#include <cfloat>

#include "common.cuh"
#include "pooled_score.cuh"

namespace mmh3 {

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int MAX_QUERIES = 8;

// Maps a float to an unsigned integer with the same order.
__device__ __forceinline__ uint32_t ordered_bits(float value) {
    const uint32_t bits = __float_as_uint(value);
    return (bits & 0x80000000u) ? ~bits : bits | 0x80000000u;
}

__device__ __forceinline__ float block_reduce(float value, float *scratch, bool maximum) {
    #pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        value = maximum ? fmaxf(value, other) : value + other;
    }
    if (threadIdx.x % 32 == 0) {
        scratch[threadIdx.x / 32] = value;
    }
    __syncthreads();
    float result = scratch[0];
    for (int warp = 1; warp < WARPS; warp++) {
        result = maximum ? fmaxf(result, scratch[warp]) : result + scratch[warp];
    }
    __syncthreads();
    return result;
}

// One CTA takes QUERIES consecutive query tiles of one head. A thread holds one pooled key in
// registers (read once, straight from L2) and scores it against each of the CTA's queries, which
// sit in shared memory; then the next key, 128 tiles further on.
template <int QUERIES>
__global__ void __launch_bounds__(THREADS, 3)
    select_kernel(Mmh3VsaWorkspace workspace, int tiles, int prefix_tiles, int kept, float scale,
                  int coarse) {
    extern __shared__ __align__(16) float scores[]; // [QUERIES][tiles]
    __shared__ float4 queries[QUERIES][32];
    __shared__ float sums[QUERIES];
    __shared__ float scratch[WARPS];
    __shared__ int histogram[WARPS][256];
    const int first_query = blockIdx.x * QUERIES;
    const int query_count = min(QUERIES, tiles - first_query);
    const int head = blockIdx.y;
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    const size_t first_row = static_cast<size_t>(head) * tiles + first_query;

    for (int index = threadIdx.x; index < QUERIES * 32; index += THREADS) {
        const int query = index / 32, four = index % 32;
        float4 values = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (query < query_count) {
            values = reinterpret_cast<const float4 *>(workspace.pooled_query +
                                                      (first_row + query) * HEAD_DIM)[four];
        }
        queries[query][four] = values;
    }
    __syncthreads();

    const float *head_keys = workspace.pooled_key + static_cast<size_t>(head) * tiles * HEAD_DIM;
    for (int tile = threadIdx.x; tile < tiles; tile += THREADS) {
        float2 key[HEAD_DIM / 2];
        load_row(head_keys + static_cast<size_t>(tile) * HEAD_DIM, key);
        #pragma unroll 1
        for (int query = 0; query < query_count; query++) {
            scores[static_cast<size_t>(query) * tiles + tile] =
                __fmul_rn(score_tree(queries[query], key), scale);
        }
    }
    __syncthreads();

    // Each warp selects the tiles of one query tile: a radix select, one byte of the ordered keys
    // at a time from the top, finds the kept-th largest video score; then one pass emits the
    // prefix tiles, the video tiles above it and the first of those equal to it.
    const int video_tiles = tiles - prefix_tiles;
    for (int query = warp; query < query_count; query += WARPS) {
        const int query_tile = first_query + query;
        const float *query_scores = scores + static_cast<size_t>(query) * tiles;
        const bool everything = query_tile < prefix_tiles || kept >= video_tiles;
        uint32_t threshold = 0;  // ordered key of the kept-th largest video score
        int remaining = kept;    // how many scores equal to the threshold are kept
        if (!everything) {
            int *bins = histogram[warp];
            uint32_t settled = 0; // mask of the key bits `threshold` already holds
            for (int shift = 24; shift >= 0; shift -= 8) {
                for (int bin = lane; bin < 256; bin += 32) {
                    bins[bin] = 0;
                }
                __syncwarp();
                for (int first = prefix_tiles; first < tiles; first += 32) {
                    const int tile = first + lane;
                    const uint32_t bits = tile < tiles ? ordered_bits(query_scores[tile]) : 0;
                    const bool counted = tile < tiles && (bits & settled) == threshold;
                    // Scores crowd into a few bins, so the lanes of a bin add their count once.
                    const uint32_t bin = counted ? (bits >> shift) & 255u : 256u;
                    const unsigned same = __match_any_sync(0xffffffffu, bin);
                    if (counted && lane == __ffs(same) - 1) {
                        bins[bin] += __popc(same);
                    }
                    __syncwarp();
                }
                __syncwarp();
                // Lane l owns bins 8 l .. 8 l + 7. `above` counts the candidates in higher bins.
                int owned[8];
                int total = 0;
                #pragma unroll
                for (int bin = 0; bin < 8; bin++) {
                    owned[bin] = bins[lane * 8 + bin];
                    total += owned[bin];
                }
                int above = total;
                #pragma unroll
                for (int offset = 1; offset < 32; offset *= 2) {
                    const int other = __shfl_down_sync(0xffffffffu, above, offset);
                    if (lane + offset < 32) {
                        above += other;
                    }
                }
                above -= total;
                const bool holds = above < remaining && remaining <= above + total;
                int digit = 0, passed = 0;
                if (holds) {
                    int seen = above;
                    #pragma unroll
                    for (int bin = 7; bin >= 0; bin--) {
                        if (seen < remaining && remaining <= seen + owned[bin]) {
                            digit = lane * 8 + bin;
                            passed = seen;
                        }
                        seen += owned[bin];
                    }
                }
                const int holder = __ffs(__ballot_sync(0xffffffffu, holds)) - 1;
                digit = __shfl_sync(0xffffffffu, digit, holder);
                passed = __shfl_sync(0xffffffffu, passed, holder);
                remaining -= passed;
                threshold |= static_cast<uint32_t>(digit) << shift;
                settled |= 255u << shift;
                __syncwarp();
            }
        }
        uint16_t *route = workspace.routes + (first_row + query) * tiles;
        int count = 0;
        int equal_before = 0;
        for (int start = 0; start < tiles; start += 32) {
            const int tile = start + lane;
            bool keep = tile < tiles;
            bool equal = false;
            if (keep && !everything && tile >= prefix_tiles) {
                const uint32_t bits = ordered_bits(query_scores[tile]);
                equal = bits == threshold;
                keep = bits > threshold;
            }
            const unsigned equal_mask = __ballot_sync(0xffffffffu, equal);
            // Ties go to the lower tile index.
            if (equal && equal_before + __popc(equal_mask & ((1u << lane) - 1)) < remaining) {
                keep = true;
            }
            equal_before += __popc(equal_mask);
            const unsigned kept_mask = __ballot_sync(0xffffffffu, keep);
            if (keep) {
                route[count + __popc(kept_mask & ((1u << lane) - 1))] =
                    static_cast<uint16_t>(tile);
            }
            count += __popc(kept_mask);
        }
        if (lane == 0) {
            workspace.route_counts[first_row + query] = count;
        }
    }
    __syncthreads();

    if (!coarse) {
        return;
    }
    // softmax(scores) . (summed values / tile length), one thread per dimension.
    for (int query = 0; query < query_count; query++) {
        float *query_scores = scores + static_cast<size_t>(query) * tiles;
        float maximum = -FLT_MAX;
        for (int tile = threadIdx.x; tile < tiles; tile += THREADS) {
            maximum = fmaxf(maximum, query_scores[tile]);
        }
        maximum = block_reduce(maximum, scratch, true);
        float sum = 0.0f;
        for (int tile = threadIdx.x; tile < tiles; tile += THREADS) {
            const float weight = expf(query_scores[tile] - maximum);
            query_scores[tile] = weight / static_cast<float>(workspace.tile_lengths[tile]);
            sum += weight;
        }
        sum = block_reduce(sum, scratch, false);
        if (threadIdx.x == 0) {
            sums[query] = sum;
        }
    }
    __syncthreads();
    const float *values =
        workspace.pooled_value + static_cast<size_t>(head) * tiles * HEAD_DIM + threadIdx.x;
    float outputs[QUERIES] = {};
    constexpr int VALUE_BATCH = 8;
    for (int first = 0; first < tiles; first += VALUE_BATCH) {
        float loaded[VALUE_BATCH];
        #pragma unroll
        for (int batch = 0; batch < VALUE_BATCH; batch++) {
            loaded[batch] = first + batch < tiles
                                ? __ldg(values + static_cast<size_t>(first + batch) * HEAD_DIM)
                                : 0.0f;
        }
        #pragma unroll
        for (int batch = 0; batch < VALUE_BATCH; batch++) {
            if (first + batch < tiles) {
                #pragma unroll
                for (int query = 0; query < QUERIES; query++) {
                    if (query < query_count) {
                        outputs[query] =
                            fmaf(scores[static_cast<size_t>(query) * tiles + first + batch],
                                 loaded[batch], outputs[query]);
                    }
                }
            }
        }
    }
    #pragma unroll
    for (int query = 0; query < QUERIES; query++) {
        if (query < query_count) {
            workspace.coarse[(first_row + query) * HEAD_DIM + threadIdx.x] =
                outputs[query] / sums[query];
        }
    }
}

template <int QUERIES>
int launch_queries(const Mmh3VsaWorkspace &workspace, int tiles, int heads, int prefix_tiles,
                   int kept, float scale, int coarse, cudaStream_t stream) {
    const size_t shared = static_cast<size_t>(QUERIES) * tiles * sizeof(float);
    // The opt-in limit only ever grows, and is per device.
    static std::atomic<size_t> configured[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    if (shared > configured[device].load(std::memory_order_relaxed)) {
        const cudaError_t status =
            cudaFuncSetAttribute(select_kernel<QUERIES>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(shared));
        if (status != cudaSuccess) {
            return static_cast<int>(status);
        }
        configured[device].store(shared, std::memory_order_relaxed);
    }
    select_kernel<QUERIES><<<dim3((tiles + QUERIES - 1) / QUERIES, heads), THREADS, shared,
                             stream>>>(workspace, tiles, prefix_tiles, kept, scale, coarse);
    return static_cast<int>(cudaGetLastError());
}

} // namespace

int launch_select(const Mmh3VsaWorkspace &workspace, int tiles, int heads, int prefix_tiles,
                  int kept, float scale, int coarse, cudaStream_t stream) {
    // As many query tiles per CTA as keep its scores within a third of an SM's shared memory
    // (three CTAs per SM), fewer for very long sequences, down to one.
    const size_t row = static_cast<size_t>(tiles) * sizeof(float);
    constexpr size_t SHARE = 66 * 1024, LIMIT = 200 * 1024;
    if (MAX_QUERIES * row <= SHARE) {
        return launch_queries<8>(workspace, tiles, heads, prefix_tiles, kept, scale, coarse, stream);
    }
    if (4 * row <= SHARE) {
        return launch_queries<4>(workspace, tiles, heads, prefix_tiles, kept, scale, coarse, stream);
    }
    if (2 * row <= SHARE) {
        return launch_queries<2>(workspace, tiles, heads, prefix_tiles, kept, scale, coarse, stream);
    }
    if (row <= LIMIT) {
        return launch_queries<1>(workspace, tiles, heads, prefix_tiles, kept, scale, coarse, stream);
    }
    return INVALID_VALUE;
}

} // namespace mmh3
