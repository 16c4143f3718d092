// Sol-Attn for BF16 heads of 128 on sm_100a: block-sparse attention over blocks of 64 tokens in
// which every query block attends a routed subset of the key blocks token by token and every other
// key block through one pooled term (its mean key against the query block's mean query, weighted
// by its length, carrying its summed values). It computes what the reference's
// mmh3_sparse_attention computes (crates/mmh3-cuda/kernels/sparse_attention.cu:72-586; the
// algorithm is stated in crates/mmh3-core/src/dit/sparse.rs:1-9, 103-234) in five steps:
//
// 1. block statistics: mean query, mean key and summed value of every block (the pooling pass of
//    inputs.cu, shared with VSA);
// 2. centre_keys: per head the mean and variance of the block keys, which are then centred;
// 3. route: per head and query block the pooled scores against every key block, the routed key
//    blocks (score above tau standard deviations, the neighbours, the sinks), and the pooled tail
//    of the rest as an online-softmax state (maximum, weighted sum, weighted values);
// 4. row_offsets: per token and head q . key mean, which moves a row's token-level scores into the
//    centred units of the pooled ones;
// 5. the token attention over the routes (vsa_attention.cu, tcgen05; BF16, or INT8/FP8 over a
//    quantized workspace), merged with the tail.
//
// The routes are bit-identical to the reference's. That fixes the FP32 order of everything a route
// depends on: the block sums run down the rows, the key mean and variance down the blocks, the
// spread of a query block over a xor butterfly and then over the four warps, and a pooled score
// over the tree of pooled_score.cuh. The tail sums are free to differ in order and do.
#include <atomic>
#include <cfloat>
#include <cmath>

#include "common.cuh"
#include "pooled_score.cuh"

namespace mmh3 {

namespace {

constexpr int BLOCK = 64;
constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int MAX_QUERIES = 8;
static_assert(THREADS == HEAD_DIM, "the routing kernels give each thread one dimension");

__device__ __forceinline__ int block_rows(int block, int tokens) {
    return min(BLOCK, tokens - block * BLOCK);
}

// Sum or maximum over the CTA: a xor butterfly in each warp, then the warps in order.
__device__ __forceinline__ float cta_reduce(float value, float *scratch, bool maximum) {
    #pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        value = maximum ? fmaxf(value, other) : __fadd_rn(value, other);
    }
    if (threadIdx.x % 32 == 0) {
        scratch[threadIdx.x / 32] = value;
    }
    __syncthreads();
    float result = scratch[0];
    for (int warp = 1; warp < WARPS; warp++) {
        result = maximum ? fmaxf(result, scratch[warp]) : __fadd_rn(result, scratch[warp]);
    }
    __syncthreads();
    return result;
}

// One CTA per head, one thread per dimension: the mean of the block keys, the centred block keys in
// place, and their variance. The blocks are walked in order (the sums are order-dependent), eight
// loads in flight at a time.
__global__ void __launch_bounds__(THREADS)
    centre_keys_kernel(float *__restrict__ block_keys, int blocks, float *__restrict__ key_mean,
                       float *__restrict__ key_variance) {
    const int head = blockIdx.x;
    const int dimension = threadIdx.x;
    float *column = block_keys + static_cast<size_t>(head) * blocks * HEAD_DIM + dimension;
    constexpr int BATCH = 8;
    float total = 0.0f;
    for (int first = 0; first < blocks; first += BATCH) {
        float loaded[BATCH];
        #pragma unroll
        for (int index = 0; index < BATCH; index++) {
            loaded[index] =
                first + index < blocks ? column[static_cast<size_t>(first + index) * HEAD_DIM] : 0.0f;
        }
        #pragma unroll
        for (int index = 0; index < BATCH; index++) {
            if (first + index < blocks) {
                total = __fadd_rn(total, loaded[index]);
            }
        }
    }
    const float count = static_cast<float>(blocks);
    const float mean = __fdiv_rn(total, count);
    float squares = 0.0f;
    for (int first = 0; first < blocks; first += BATCH) {
        float loaded[BATCH];
        #pragma unroll
        for (int index = 0; index < BATCH; index++) {
            loaded[index] =
                first + index < blocks ? column[static_cast<size_t>(first + index) * HEAD_DIM] : 0.0f;
        }
        #pragma unroll
        for (int index = 0; index < BATCH; index++) {
            if (first + index < blocks) {
                const float centred = __fsub_rn(loaded[index], mean);
                column[static_cast<size_t>(first + index) * HEAD_DIM] = centred;
                squares = __fmaf_rn(centred, centred, squares);
            }
        }
    }
    key_mean[head * HEAD_DIM + dimension] = mean;
    key_variance[head * HEAD_DIM + dimension] = __fdiv_rn(squares, count);
}

// One CTA takes QUERIES consecutive query blocks of one head. A thread holds one centred block key
// in registers and scores it against each of the CTA's centroids, which sit in shared memory; then
// the next key block, 128 further on.
template <int QUERIES>
__global__ void __launch_bounds__(THREADS, 3)
    route_kernel(Mmh3SparseWorkspace workspace, int tokens, int blocks, float tau, float log2_scale,
                 int sink_key_start, int sink_key_end, int sink_query_start, int sink_query_end) {
    extern __shared__ __align__(16) float weights[]; // [blocks][QUERIES], scores at first
    uint8_t *routed = reinterpret_cast<uint8_t *>(weights + static_cast<size_t>(QUERIES) * blocks);
    __shared__ float4 centroids[QUERIES][32];
    __shared__ float thresholds[QUERIES];
    __shared__ float tail_maxima[QUERIES];
    __shared__ float tail_sums[QUERIES];
    __shared__ float scratch[WARPS];
    const int first_query = blockIdx.x * QUERIES;
    const int queries = min(QUERIES, blocks - first_query);
    const int head = blockIdx.y;
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    const size_t first_row = static_cast<size_t>(head) * blocks + first_query;

    // The centroids, and per query block the threshold: tau standard deviations of its pooled
    // scores, from the variance of the block keys along each dimension.
    const float variance = workspace.key_variance[head * HEAD_DIM + threadIdx.x];
    for (int query = 0; query < queries; query++) {
        const float centroid = workspace.centroids[(first_row + query) * HEAD_DIM + threadIdx.x];
        reinterpret_cast<float *>(&centroids[query][0])[threadIdx.x] = centroid;
        const float spread =
            cta_reduce(__fmul_rn(__fmul_rn(centroid, centroid), variance), scratch, false);
        if (threadIdx.x == 0) {
            thresholds[query] = __fmul_rn(
                tau, sqrtf(__fmaf_rn(__fmul_rn(spread, log2_scale), log2_scale, 1e-6f)));
        }
    }
    __syncthreads();

    const float *head_keys = workspace.block_keys + static_cast<size_t>(head) * blocks * HEAD_DIM;
    for (int key_block = threadIdx.x; key_block < blocks; key_block += THREADS) {
        float2 key[HEAD_DIM / 2];
        load_row(head_keys + static_cast<size_t>(key_block) * HEAD_DIM, key);
        #pragma unroll 1
        for (int query = 0; query < queries; query++) {
            const int query_block = first_query + query;
            const float score = __fmul_rn(score_tree(centroids[query], key), log2_scale);
            weights[static_cast<size_t>(key_block) * QUERIES + query] = score;
            routed[static_cast<size_t>(query) * blocks + key_block] =
                score > thresholds[query] || abs(query_block - key_block) <= 1 ||
                (key_block >= sink_key_start && key_block < sink_key_end) ||
                (query_block >= sink_query_start && query_block < sink_query_end);
        }
    }
    __syncthreads();

    // The tail of each query block: the key blocks it does not route, as softmax weights against
    // their maximum, each counted once per token it stands for.
    for (int query = 0; query < queries; query++) {
        float *query_weights = weights + query; // QUERIES apart
        const uint8_t *query_routed = routed + static_cast<size_t>(query) * blocks;
        float maximum = -FLT_MAX;
        for (int key_block = threadIdx.x; key_block < blocks; key_block += THREADS) {
            if (!query_routed[key_block]) {
                maximum = fmaxf(maximum, query_weights[static_cast<size_t>(key_block) * QUERIES]);
            }
        }
        maximum = cta_reduce(maximum, scratch, true);
        float sum = 0.0f;
        for (int key_block = threadIdx.x; key_block < blocks; key_block += THREADS) {
            const float weight =
                query_routed[key_block]
                    ? 0.0f
                    : exp2f(query_weights[static_cast<size_t>(key_block) * QUERIES] - maximum);
            query_weights[static_cast<size_t>(key_block) * QUERIES] = weight;
            sum = fmaf(weight, static_cast<float>(block_rows(key_block, tokens)), sum);
        }
        sum = cta_reduce(sum, scratch, false);
        if (threadIdx.x == 0) {
            tail_maxima[query] = maximum;
            tail_sums[query] = sum;
        }
    }
    __syncthreads();

    // The weighted values of the tails: thread d sums dimension d of the summed values of the key
    // blocks, which every query block of the CTA weighs its own way.
    const float *values =
        workspace.value_sums + static_cast<size_t>(head) * blocks * HEAD_DIM + threadIdx.x;
    // A key block's weights for the CTA's query blocks lie side by side, so one or two 16-byte
    // loads bring all of them, and two query blocks share a packed multiply-add. Each sum still
    // runs over the key blocks in order.
    float tails[QUERIES] = {};
    constexpr int BATCH = 16;
    for (int first = 0; first < blocks; first += BATCH) {
        float loaded[BATCH];
        #pragma unroll
        for (int index = 0; index < BATCH; index++) {
            loaded[index] =
                first + index < blocks ? values[static_cast<size_t>(first + index) * HEAD_DIM] : 0.0f;
        }
        #pragma unroll
        for (int index = 0; index < BATCH; index++) {
            if (first + index < blocks) {
                // Routed blocks have weight zero; query blocks past the last one are not stored.
                const float *block_weights = weights + static_cast<size_t>(first + index) * QUERIES;
                if constexpr (QUERIES % 4 == 0) {
                    const float2 value = make_float2(loaded[index], loaded[index]);
                    #pragma unroll
                    for (int four = 0; four < QUERIES / 4; four++) {
                        const float4 weight = reinterpret_cast<const float4 *>(block_weights)[four];
                        const float2 low = __ffma2_rn(make_float2(weight.x, weight.y), value,
                                                      make_float2(tails[four * 4],
                                                                  tails[four * 4 + 1]));
                        const float2 high = __ffma2_rn(make_float2(weight.z, weight.w), value,
                                                       make_float2(tails[four * 4 + 2],
                                                                   tails[four * 4 + 3]));
                        tails[four * 4] = low.x;
                        tails[four * 4 + 1] = low.y;
                        tails[four * 4 + 2] = high.x;
                        tails[four * 4 + 3] = high.y;
                    }
                } else {
                    #pragma unroll
                    for (int query = 0; query < QUERIES; query++) {
                        tails[query] = fmaf(block_weights[query], loaded[index], tails[query]);
                    }
                }
            }
        }
    }
    #pragma unroll
    for (int query = 0; query < QUERIES; query++) {
        if (query < queries) {
            workspace.tail_values[(first_row + query) * HEAD_DIM + threadIdx.x] = tails[query];
        }
    }

    // The routes: ascending key blocks, one warp per query block.
    for (int query = warp; query < queries; query += WARPS) {
        const size_t row = first_row + query;
        uint16_t *route = workspace.routes + row * blocks;
        const uint8_t *query_routed = routed + static_cast<size_t>(query) * blocks;
        int count = 0;
        for (int first = 0; first < blocks; first += 32) {
            const int key_block = first + lane;
            const bool flag = key_block < blocks && query_routed[key_block];
            const unsigned mask = __ballot_sync(0xffffffffu, flag);
            if (flag) {
                route[count + __popc(mask & ((1u << lane) - 1u))] = static_cast<uint16_t>(key_block);
            }
            count += __popc(mask);
        }
        if (lane == 0) {
            workspace.route_counts[row] = count;
            workspace.tail_max[row] = tail_maxima[query];
            workspace.tail_sum[row] = tail_sums[query];
        }
    }
}

template <int QUERIES>
int launch_queries(const Mmh3SparseWorkspace &workspace, int tokens, int blocks, int heads,
                   float tau, float log2_scale, int sink_key_start, int sink_key_end,
                   int sink_query_start, int sink_query_end, cudaStream_t stream) {
    // Scores and flags of the CTA's query blocks against every key block.
    const size_t shared = static_cast<size_t>(QUERIES) * blocks * (sizeof(float) + 1);
    // The opt-in limit only ever grows, and is per device.
    static std::atomic<size_t> configured[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    if (shared > configured[device].load(std::memory_order_relaxed)) {
        const cudaError_t status =
            cudaFuncSetAttribute(route_kernel<QUERIES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(shared));
        if (status != cudaSuccess) {
            return static_cast<int>(status);
        }
        configured[device].store(shared, std::memory_order_relaxed);
    }
    const dim3 grid((blocks + QUERIES - 1) / QUERIES, heads);
    route_kernel<QUERIES><<<grid, THREADS, shared, stream>>>(
        workspace, tokens, blocks, tau, log2_scale, sink_key_start, sink_key_end, sink_query_start,
        sink_query_end);
    return static_cast<int>(cudaGetLastError());
}

// As many query blocks per CTA as keep its scores and flags within a third of an SM's shared
// memory (three CTAs per SM), fewer for very long sequences, down to one.
int launch_route(const Mmh3SparseWorkspace &workspace, int tokens, int blocks, int heads, float tau,
                 float log2_scale, int sink_key_start, int sink_key_end, int sink_query_start,
                 int sink_query_end, cudaStream_t stream) {
    const size_t row = static_cast<size_t>(blocks) * (sizeof(float) + 1);
    constexpr size_t SHARE = 66 * 1024, LIMIT = 200 * 1024;
#define MMH3_ROUTE(QUERIES)                                                                        \
    launch_queries<QUERIES>(workspace, tokens, blocks, heads, tau, log2_scale, sink_key_start,    \
                            sink_key_end, sink_query_start, sink_query_end, stream)
    if (MAX_QUERIES * row <= SHARE) {
        return MMH3_ROUTE(8);
    }
    if (4 * row <= SHARE) {
        return MMH3_ROUTE(4);
    }
    if (2 * row <= SHARE) {
        return MMH3_ROUTE(2);
    }
    if (row <= LIMIT) {
        return MMH3_ROUTE(1);
    }
#undef MMH3_ROUTE
    return INVALID_VALUE;
}

// One warp per (token, head): q . key mean in the units of the exponent. Lane l chains dimensions
// l, l + 32, l + 64, l + 96; the lanes meet over a xor butterfly.
__global__ void __launch_bounds__(256)
    row_offsets_kernel(const __nv_bfloat16 *__restrict__ query, int tokens, int heads,
                       int64_t token_stride, int64_t head_stride,
                       const float *__restrict__ key_mean, float log2_scale,
                       float *__restrict__ row_offsets) {
    const int lane = threadIdx.x % 32;
    const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (item >= static_cast<int64_t>(tokens) * heads) {
        return;
    }
    const int head = static_cast<int>(item % heads);
    const int64_t token = item / heads;
    const __nv_bfloat16 *row = query + token * token_stride + head * head_stride;
    float partial = 0.0f;
    #pragma unroll
    for (int part = 0; part < HEAD_DIM / 32; part++) {
        partial = __fmaf_rn(__bfloat162float(row[lane + part * 32]),
                            key_mean[head * HEAD_DIM + lane + part * 32], partial);
    }
    #pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
        partial = __fadd_rn(partial, __shfl_xor_sync(0xffffffffu, partial, offset));
    }
    if (lane == 0) {
        row_offsets[static_cast<size_t>(head) * tokens + token] = __fmul_rn(partial, log2_scale);
    }
}

} // namespace

int launch_sparse_attention(const void *query, const void *key, const void *value, void *output,
                            int tokens, int heads, const Mmh3AttentionLayout &layout, float scale,
                            float tau, int sink_key_start, int sink_key_end, int sink_query_start,
                            int sink_query_end, const Mmh3SparseWorkspace &workspace,
                            const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                            cudaStream_t stream) {
    if (!(scale > 0.0f) || !std::isfinite(scale)) {
        return INVALID_VALUE;
    }
    const int blocks = (tokens + BLOCK - 1) / BLOCK;
    if (blocks > 65535) {
        return NOT_SUPPORTED; // routes are 16-bit block indices
    }
    const float log2_scale = scale * LOG2_E;
    if (!inputs_ready) {
        const int pooled =
            launch_block_statistics(query, key, value, tokens, heads, layout, workspace, stream);
        if (pooled != 0) {
            return pooled;
        }
    }
    centre_keys_kernel<<<heads, THREADS, 0, stream>>>(workspace.block_keys, blocks,
                                                      workspace.key_mean, workspace.key_variance);
    const int routed = launch_route(workspace, tokens, blocks, heads, tau, log2_scale, sink_key_start,
                                    sink_key_end, sink_query_start, sink_query_end, stream);
    if (routed != 0) {
        return routed;
    }
    const int64_t items = static_cast<int64_t>(tokens) * heads;
    row_offsets_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16 *>(query), tokens, heads, layout.token_stride[QUERY],
        layout.head_stride[QUERY], workspace.key_mean, log2_scale, workspace.row_offsets);
    const cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess) {
        return static_cast<int>(launched);
    }
    if (quantized != nullptr) {
        // As the reference does (sparse_attention.cu:577-580): the quantizer's passes that
        // inputs_ready leaves to do, then the INT8/FP8 token attention.
        const int prepared = launch_quantize(query, key, value, tokens, heads, layout, *quantized,
                                             nullptr, nullptr, 0, inputs_ready, stream);
        if (prepared != 0) {
            return prepared;
        }
        return launch_sol_token_attention_quantized(*quantized, output, tokens, heads, layout,
                                                    scale, workspace, stream);
    }
    return launch_sol_token_attention(query, key, value, output, tokens, heads, layout, scale,
                                      workspace, stream);
}

} // namespace mmh3
