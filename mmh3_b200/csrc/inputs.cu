// The passes over q, k and v that come before the attention: per-head RMSNorm and RoPE, INT8 q and
// k with one scale per head and block, FP8 V transposed, the |v| maxima, and VSA's pooled tiles.
// One kernel template covers them all. It is bound by HBM bandwidth: every element of q, k and v
// is read once and each quantized byte written once.
//
// The results are bit-identical to the reference's (crates/mmh3-cuda/kernels/dit.cu:98-391,
// quantized_attention.cu:85-241, vsa_attention.cu:68-91), which fixes the order of every FP32
// operation: the lane-strided sum of squares with its xor butterfly, the row-ordered sums of the
// pooled tiles, IEEE divisions by the scales, and round-to-nearest-even conversions.
//
// A CTA of 256 threads owns one block of 64 tokens (or one VSA tile of up to 64) of one head. q, k
// and v take turns in a 16 KiB tile of shared memory; the rows of the next turn are already in
// flight in registers while the current one is worked on, and four CTAs share an SM.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mmh3 {

namespace {

constexpr int BLOCK_ROWS = 64;
constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
// A row of 128 BF16 values is 16 chunks of 16 bytes.
constexpr int CHUNKS_PER_THREAD = BLOCK_ROWS * 16 / THREADS;
constexpr int HEADS_PER_CTA = 8;

struct InputsParams {
    const __nv_bfloat16 *source[3];
    // Where normalized q and k go back to, or null.
    __nv_bfloat16 *normalized[2];
    int64_t token_stride[3];
    int64_t head_stride[3];
    const __nv_bfloat16 *weight[2];
    const float *angles;
    int pairs;
    float epsilon;
    int tokens;
    int heads;
    const int32_t *tile_starts;
    const int32_t *tile_lengths;
    uint8_t *quantized[2]; // INT8 q and k, [tokens, heads, 128]
    float *scales[2];      // [heads, blocks]
    uint8_t *value8;       // [heads, 128, blocks * 64]
    float *value_scales;   // [heads]
    float *value_maxima;   // [heads, blocks]
    float *pooled[3];      // mean q, mean k, summed v, [heads, blocks, 128]
    // Per-head maxima of |v| to quantize V with in this pass, or null.
    const float *value_head_maxima;
    // Nonzero quantizes V with value_scales as another kernel left them.
    int value_scales_ready;
    // The first and the last of the turns q (0), k (1), v (2) to take.
    int first_part;
    int last_part;
    // Whether rows can be read in 16-byte chunks.
    int vector_loads;
    // Heads one CTA walks, sharing the cosines and sines of its block's angles.
    int heads_per_cta;
};

__device__ __forceinline__ float warp_max(float value) {
    #pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
        value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
    }
    return value;
}

// x / scale, rounded to nearest as IEEE division rounds it, for many x and one scale: with
// y = RN(1 / scale), q = RN(x * y) and the exact residual r = x - q * scale, RN(q + r * y) is the
// correctly rounded quotient (Markstein) unless the significand of the scale is all ones or the
// residual could underflow; `exact` says whether the scale is one of those, and then the division
// itself is used. The quotient's bits decide an INT8 or FP8 code, so "almost" would not do.
struct Divider {
    float scale;
    float reciprocal;
    bool exact;
    __device__ __forceinline__ explicit Divider(float divisor) : scale(divisor) {
        reciprocal = __frcp_rn(divisor);
        const uint32_t bits = __float_as_uint(divisor);
        exact = (bits & 0x007fffffu) != 0x007fffffu && divisor >= 1e-24f && divisor <= 1e24f;
    }
    __device__ __forceinline__ float operator()(float x) const {
        if (exact) {
            const float quotient = __fmul_rn(x, reciprocal);
            const float residual = __fmaf_rn(-quotient, scale, x);
            return __fmaf_rn(residual, reciprocal, quotient);
        }
        return __fdiv_rn(x, scale);
    }
};

// RMSNorm of the row `row` of the tile with `weight`, then the split-half rotary embedding of its
// first 2 * pairs dimensions from the cosines and sines of the row's angles, written back to the
// tile in BF16. One warp works on the row; lane l holds dimensions l, l + 32, l + 64 and l + 96,
// which is what the order of the additions in the sum of squares depends on. Returns the largest
// magnitude this lane wrote.
__device__ __forceinline__ float normalize_row(__nv_bfloat16 *row, float *scratch,
                                               const __nv_bfloat16 *__restrict__ weight,
                                               const float2 *__restrict__ row_trig, int pairs,
                                               float epsilon) {
    const int lane = threadIdx.x % 32;
    float values[4];
    float squares = 0.0f;
    #pragma unroll
    for (int part = 0; part < 4; part++) {
        values[part] = __bfloat162float(row[lane + part * 32]);
        squares = __fmaf_rn(values[part], values[part], squares);
    }
    #pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
        squares += __shfl_xor_sync(0xffffffffu, squares, offset);
    }
    const float inverse = rsqrtf(__fmaf_rn(squares, 1.0f / HEAD_DIM, epsilon));
    #pragma unroll
    for (int part = 0; part < 4; part++) {
        values[part] = __fmul_rn(
            values[part], __fmul_rn(inverse, __bfloat162float(weight[lane + part * 32])));
    }
    if (row_trig != nullptr) {
        #pragma unroll
        for (int part = 0; part < 4; part++) {
            scratch[lane + part * 32] = values[part];
        }
        __syncwarp();
        for (int pair = lane; pair < pairs; pair += 32) {
            const float2 trig = row_trig[pair]; // (cosine, sine)
            const float first = scratch[pair];
            const float second = scratch[pair + pairs];
            scratch[pair] = __fmaf_rn(trig.x, first, -__fmul_rn(trig.y, second));
            scratch[pair + pairs] = __fmaf_rn(trig.y, first, __fmul_rn(trig.x, second));
        }
        __syncwarp();
        #pragma unroll
        for (int part = 0; part < 4; part++) {
            values[part] = scratch[lane + part * 32];
        }
        __syncwarp();
    }
    float maximum = 0.0f;
    #pragma unroll
    for (int part = 0; part < 4; part++) {
        const __nv_bfloat16 rounded = __float2bfloat16_rn(values[part]);
        row[lane + part * 32] = rounded;
        maximum = fmaxf(maximum, fabsf(__bfloat162float(rounded)));
    }
    return maximum;
}

__device__ __forceinline__ float chunk_max(const uint4 &chunk) {
    const uint32_t words[4] = {chunk.x, chunk.y, chunk.z, chunk.w};
    float maximum = 0.0f;
    #pragma unroll
    for (int word = 0; word < 4; word++) {
        maximum = fmaxf(maximum, fabsf(__uint_as_float(words[word] << 16)));
        maximum = fmaxf(maximum, fabsf(__uint_as_float(words[word] & 0xffff0000u)));
    }
    return maximum;
}

// Dynamic shared memory: the cosines and sines of the block's angles, [rows][pairs] float2, computed
// once per CTA and used by q and k of every head the CTA takes.
template <bool NORMALIZE, bool STATS, bool QUANTIZE>
__global__ void __launch_bounds__(THREADS, 4) inputs_kernel(const InputsParams p) {
    extern __shared__ __align__(16) float2 trig[];
    __shared__ __align__(16) __nv_bfloat16 tile[BLOCK_ROWS][HEAD_DIM];
    __shared__ float scratch[WARPS][HEAD_DIM];
    __shared__ float maxima[WARPS];
    const int block = blockIdx.x;
    const int blocks = gridDim.x;
    const int first_head = blockIdx.y * p.heads_per_cta;
    const int head_count = min(p.heads_per_cta, p.heads - first_head);
    const int64_t first_token =
        p.tile_starts != nullptr ? p.tile_starts[block] : static_cast<int64_t>(block) * BLOCK_ROWS;
    const int rows = p.tile_lengths != nullptr
                         ? p.tile_lengths[block]
                         : min(BLOCK_ROWS, p.tokens - block * BLOCK_ROWS);
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    const bool rotate = NORMALIZE && p.angles != nullptr;
    const bool values_here =
        QUANTIZE && (p.value_head_maxima != nullptr || p.value_scales_ready != 0);
    const int parts = p.last_part - p.first_part + 1;
    const int items = head_count * parts;

    uint4 chunks[CHUNKS_PER_THREAD];
    auto load = [&](int item) {
        const int part = p.first_part + item % parts;
        const int head = first_head + item / parts;
        const __nv_bfloat16 *rows_base =
            p.source[part] + first_token * p.token_stride[part] + head * p.head_stride[part];
        #pragma unroll
        for (int index = 0; index < CHUNKS_PER_THREAD; index++) {
            const int chunk = threadIdx.x + index * THREADS;
            if (chunk / 16 < rows) {
                const __nv_bfloat16 *source =
                    rows_base + (chunk / 16) * p.token_stride[part] + (chunk % 16) * 8;
                if (p.vector_loads) {
                    chunks[index] = __ldg(reinterpret_cast<const uint4 *>(source));
                } else {
                    uint16_t halves[8];
                    #pragma unroll
                    for (int element = 0; element < 8; element++) {
                        halves[element] = __ldg(reinterpret_cast<const uint16_t *>(source) + element);
                    }
                    chunks[index] = make_uint4(halves[0] | (uint32_t(halves[1]) << 16),
                                               halves[2] | (uint32_t(halves[3]) << 16),
                                               halves[4] | (uint32_t(halves[5]) << 16),
                                               halves[6] | (uint32_t(halves[7]) << 16));
                }
            }
        }
    };

    load(0);
    if (rotate) {
        for (int index = threadIdx.x; index < rows * p.pairs; index += THREADS) {
            float sine, cosine;
            sincosf(p.angles[first_token * p.pairs + index], &sine, &cosine);
            trig[index] = make_float2(cosine, sine);
        }
    }
    for (int item = 0; item < items; item++) {
        const int part = p.first_part + item % parts;
        const int head = first_head + item / parts;
        const size_t statistic = (static_cast<size_t>(head) * blocks + block) * HEAD_DIM;
        // The rows go to the tile; the largest magnitude is taken on the way where nothing
        // changes the rows before it is needed.
        float maximum = 0.0f;
        #pragma unroll
        for (int index = 0; index < CHUNKS_PER_THREAD; index++) {
            const int chunk = threadIdx.x + index * THREADS;
            if (chunk / 16 < rows) {
                *reinterpret_cast<uint4 *>(&tile[chunk / 16][(chunk % 16) * 8]) = chunks[index];
                if (QUANTIZE && (!NORMALIZE || part == 2)) {
                    maximum = fmaxf(maximum, chunk_max(chunks[index]));
                }
            }
        }
        __syncthreads();
        if (item + 1 < items) {
            load(item + 1);
        }
        if (NORMALIZE && part < 2) {
            for (int row = warp; row < rows; row += WARPS) {
                maximum = fmaxf(maximum,
                                normalize_row(tile[row], scratch[warp], p.weight[part],
                                              rotate ? trig + row * p.pairs : nullptr, p.pairs,
                                              p.epsilon));
            }
        }
        const bool needs_maximum = QUANTIZE && (part < 2 || !values_here);
        if (needs_maximum) {
            maximum = warp_max(maximum);
            if (lane == 0) {
                maxima[warp] = maximum;
            }
        }
        if (NORMALIZE || needs_maximum) {
            __syncthreads();
        }
        if (needs_maximum) {
            maximum = maxima[0];
            #pragma unroll
            for (int index = 1; index < WARPS; index++) {
                maximum = fmaxf(maximum, maxima[index]);
            }
        }

        if constexpr (STATS) {
            // The sums over the rows in row order, one thread per dimension.
            if (threadIdx.x < HEAD_DIM) {
                const int dimension = threadIdx.x;
                float sum = 0.0f;
                for (int row = 0; row < rows; row++) {
                    sum += __bfloat162float(tile[row][dimension]);
                }
                p.pooled[part][statistic + dimension] = part == 2 ? sum : sum / rows;
            }
        }

        if (part == 2) {
            if (QUANTIZE && !values_here && threadIdx.x == 0) {
                p.value_maxima[head * blocks + block] = maximum;
            }
            if (values_here) {
                // FP8 V transposed into 64 columns per block, zero past the block's rows. Each
                // thread writes one 32-byte sector: 32 rows of one dimension.
                float scale;
                if (p.value_head_maxima != nullptr) {
                    scale = fmaxf(p.value_head_maxima[head] / 448.0f, 1e-30f);
                    if (block == 0 && threadIdx.x == 0) {
                        p.value_scales[head] = scale;
                    }
                } else {
                    scale = p.value_scales[head];
                }
                const Divider divide(scale);
                const int dimension = threadIdx.x % HEAD_DIM;
                const int first_row = threadIdx.x / HEAD_DIM * 32;
                uint32_t words[8];
                #pragma unroll
                for (int word = 0; word < 8; word++) {
                    uint32_t packed = 0;
                    #pragma unroll
                    for (int byte = 0; byte < 4; byte++) {
                        const int row = first_row + word * 4 + byte;
                        const float element =
                            row < rows ? __bfloat162float(tile[row][dimension]) : 0.0f;
                        packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(
                                      divide(element), __NV_SATFINITE, __NV_E4M3))
                                  << (8 * byte);
                    }
                    words[word] = packed;
                }
                uint4 *destination = reinterpret_cast<uint4 *>(
                    p.value8 +
                    (static_cast<int64_t>(head) * HEAD_DIM + dimension) * blocks * BLOCK_ROWS +
                    static_cast<int64_t>(block) * BLOCK_ROWS + first_row);
                destination[0] = make_uint4(words[0], words[1], words[2], words[3]);
                destination[1] = make_uint4(words[4], words[5], words[6], words[7]);
            }
        } else {
            if constexpr (QUANTIZE) {
                const float scale = fmaxf(maximum / 127.0f, 1e-30f);
                if (threadIdx.x == 0) {
                    p.scales[part][head * blocks + block] = scale;
                }
                const Divider divide(scale);
                // A row of 128 INT8 values is 8 chunks of 16 bytes, each from 16 BF16 values.
                uint8_t *destination =
                    p.quantized[part] + (first_token * p.heads + head) * HEAD_DIM;
                for (int chunk = threadIdx.x; chunk < rows * 8; chunk += THREADS) {
                    const uint4 *source =
                        reinterpret_cast<const uint4 *>(&tile[chunk / 8][(chunk % 8) * 16]);
                    const uint4 halves[2] = {source[0], source[1]};
                    const __nv_bfloat16 *elements =
                        reinterpret_cast<const __nv_bfloat16 *>(halves);
                    uint32_t words[4];
                    #pragma unroll
                    for (int word = 0; word < 4; word++) {
                        uint32_t packed = 0;
                        #pragma unroll
                        for (int byte = 0; byte < 4; byte++) {
                            const int8_t value = static_cast<int8_t>(__float2int_rn(
                                divide(__bfloat162float(elements[word * 4 + byte]))));
                            packed |= static_cast<uint32_t>(static_cast<uint8_t>(value))
                                      << (8 * byte);
                        }
                        words[word] = packed;
                    }
                    *reinterpret_cast<uint4 *>(
                        destination + static_cast<int64_t>(chunk / 8) * p.heads * HEAD_DIM +
                        (chunk % 8) * 16) = make_uint4(words[0], words[1], words[2], words[3]);
                }
            }
            if (NORMALIZE && p.normalized[part] != nullptr) {
                __nv_bfloat16 *rows_base = p.normalized[part] +
                                           first_token * p.token_stride[part] +
                                           head * p.head_stride[part];
                for (int chunk = threadIdx.x; chunk < rows * 16; chunk += THREADS) {
                    *reinterpret_cast<uint4 *>(rows_base + (chunk / 16) * p.token_stride[part] +
                                               (chunk % 16) * 8) =
                        *reinterpret_cast<const uint4 *>(&tile[chunk / 16][(chunk % 16) * 8]);
                }
            }
        }
        __syncthreads();
    }
}

// The FP8 scale of each head from its block maxima of |v|
// (crates/mmh3-cuda/kernels/quantized_attention.cu:116-127).
__global__ void value_scales_kernel(const float *__restrict__ maxima, float *__restrict__ scales,
                                    int blocks) {
    float maximum = 0.0f;
    for (int block = threadIdx.x; block < blocks; block += blockDim.x) {
        maximum = fmaxf(maximum, maxima[static_cast<size_t>(blockIdx.x) * blocks + block]);
    }
    __shared__ float partial[32];
    maximum = warp_max(maximum);
    if (threadIdx.x % 32 == 0) {
        partial[threadIdx.x / 32] = maximum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int warp = 1; warp < static_cast<int>(blockDim.x) / 32; warp++) {
            maximum = fmaxf(maximum, partial[warp]);
        }
        scales[blockIdx.x] = fmaxf(maximum / 448.0f, 1e-30f);
    }
}

bool aligned_rows(const void *base, int64_t token_stride, int64_t head_stride) {
    return reinterpret_cast<uintptr_t>(base) % 16 == 0 && token_stride % 8 == 0 &&
           head_stride % 8 == 0;
}

template <bool NORMALIZE, bool STATS, bool QUANTIZE>
int launch(InputsParams params, int blocks, cudaStream_t stream) {
    const bool rotate = NORMALIZE && params.angles != nullptr;
    // With angles a CTA takes several heads so that their sincosf is paid once; the grid still
    // holds several CTAs per SM slot.
    params.heads_per_cta = rotate ? HEADS_PER_CTA : 1;
    const int groups = (params.heads + params.heads_per_cta - 1) / params.heads_per_cta;
    const size_t shared = rotate ? static_cast<size_t>(BLOCK_ROWS) * params.pairs * sizeof(float2)
                                 : 0;
    if (rotate) {
        // Up to 64 pairs: 32 KiB of cosines and sines beside the 20 KiB of static shared memory.
        static SharedMemoryOptIn shared_memory;
        const cudaError_t configured = shared_memory.ensure(
            inputs_kernel<NORMALIZE, STATS, QUANTIZE>, BLOCK_ROWS * (HEAD_DIM / 2) * 8);
        if (configured != cudaSuccess) {
            return static_cast<int>(configured);
        }
    }
    inputs_kernel<NORMALIZE, STATS, QUANTIZE>
        <<<dim3(blocks, groups), THREADS, shared, stream>>>(params);
    return static_cast<int>(cudaGetLastError());
}

} // namespace

// q and k of the fused rows [q | k | v] normalized and rotated in place. A block of 64 tokens of
// one q or k head is one CTA's work; the key heads follow the query heads along blockIdx.y.
int launch_qk_norm_rope(__nv_bfloat16 *qkv, const __nv_bfloat16 *query_weight,
                        const __nv_bfloat16 *key_weight, const float *angles, int pairs,
                        int tokens, int query_heads, int key_heads, float epsilon,
                        cudaStream_t stream) {
    const int64_t row = static_cast<int64_t>(query_heads + 2 * key_heads) * HEAD_DIM;
    const int blocks = (tokens + BLOCK_ROWS - 1) / BLOCK_ROWS;
    // Two launches, one over the query heads and one over the key heads, each a one-turn pass.
    for (int part = 0; part < 2; part++) {
        const int heads = part ? key_heads : query_heads;
        if (heads == 0) {
            continue;
        }
        InputsParams params = {};
        __nv_bfloat16 *base = qkv + (part ? static_cast<int64_t>(query_heads) * HEAD_DIM : 0);
        params.source[0] = base;
        params.normalized[0] = base;
        params.token_stride[0] = row;
        params.head_stride[0] = HEAD_DIM;
        params.weight[0] = part ? key_weight : query_weight;
        params.angles = angles;
        params.pairs = pairs;
        params.epsilon = epsilon;
        params.tokens = tokens;
        params.heads = heads;
        params.first_part = 0;
        params.last_part = 0;
        params.vector_loads = aligned_rows(base, row, HEAD_DIM);
        if (!params.vector_loads) {
            return NOT_SUPPORTED;
        }
        const int status = launch<true, false, false>(params, blocks, stream);
        if (status != 0) {
            return status;
        }
    }
    return 0;
}

int launch_attention_inputs(__nv_bfloat16 *qkv, const __nv_bfloat16 *query_weight,
                            const __nv_bfloat16 *key_weight, const float *angles, int pairs,
                            int tokens, int heads, float epsilon,
                            const Mmh3SparseWorkspace *sparse,
                            const Mmh3QuantizedWorkspace *quantized, const int32_t *tile_starts,
                            const int32_t *tile_lengths, int tiles,
                            const float *value_head_maxima, cudaStream_t stream) {
    const int64_t inner = static_cast<int64_t>(heads) * HEAD_DIM;
    const int blocks = tile_starts != nullptr ? tiles : (tokens + BLOCK_ROWS - 1) / BLOCK_ROWS;
    InputsParams params = {};
    for (int part = 0; part < 3; part++) {
        params.source[part] = qkv + part * inner;
        params.token_stride[part] = 3 * inner;
        params.head_stride[part] = HEAD_DIM;
    }
    if (!aligned_rows(qkv, 3 * inner, HEAD_DIM)) {
        return NOT_SUPPORTED;
    }
    params.vector_loads = 1;
    const bool stats = sparse != nullptr;
    const bool quantize = quantized != nullptr;
    // Normalized q goes back to qkv in BF16 when the attention or the Sol-Attn row offsets read
    // it, and normalized k when the attention reads BF16 keys
    // (crates/mmh3-cuda/kernels/dit.cu:381-388).
    params.normalized[0] =
        (stats && tile_starts == nullptr) || !quantize ? qkv : nullptr;
    params.normalized[1] = !quantize ? qkv + inner : nullptr;
    params.weight[0] = query_weight;
    params.weight[1] = key_weight;
    params.angles = angles;
    params.pairs = pairs;
    params.epsilon = epsilon;
    params.tokens = tokens;
    params.heads = heads;
    params.tile_starts = tile_starts;
    params.tile_lengths = tile_lengths;
    if (quantize) {
        params.quantized[0] = quantized->query;
        params.quantized[1] = quantized->key;
        params.scales[0] = quantized->query_scales;
        params.scales[1] = quantized->key_scales;
        params.value8 = quantized->value;
        params.value_scales = quantized->value_scales;
        params.value_maxima = quantized->value_maxima;
    }
    if (stats) {
        params.pooled[0] = sparse->centroids;
        params.pooled[1] = sparse->block_keys;
        params.pooled[2] = sparse->value_sums;
    }
    params.value_head_maxima = value_head_maxima;
    params.first_part = 0;
    params.last_part = 2;
    if (stats && quantize) {
        return launch<true, true, true>(params, blocks, stream);
    }
    if (stats) {
        return launch<true, true, false>(params, blocks, stream);
    }
    return launch<true, false, true>(params, blocks, stream);
}

// What mmh3_attention_quantized and mmh3_vsa_attention_quantized prepare themselves
// (crates/mmh3-cuda/kernels/quantized_attention.cu:590-604, 624-630): with inputs_ready 0 INT8 q and
// k, their scales and the block maxima of |v|; below 2 the per-head FP8 scale and FP8 V.
int launch_quantize(const void *query, const void *key, const void *value, int tokens, int heads,
                    const Mmh3AttentionLayout &layout, const Mmh3QuantizedWorkspace &workspace,
                    const int32_t *tile_starts, const int32_t *tile_lengths, int tiles,
                    int inputs_ready, cudaStream_t stream) {
    if (inputs_ready == 2) {
        return 0;
    }
    const int blocks = tile_starts != nullptr ? tiles : (tokens + BLOCK_ROWS - 1) / BLOCK_ROWS;
    InputsParams params = {};
    const void *sources[3] = {query, key, value};
    params.vector_loads = 1;
    for (int part = 0; part < 3; part++) {
        params.source[part] = static_cast<const __nv_bfloat16 *>(sources[part]);
        params.token_stride[part] = layout.token_stride[part];
        params.head_stride[part] = layout.head_stride[part];
        if (sources[part] != nullptr &&
            !aligned_rows(sources[part], layout.token_stride[part], layout.head_stride[part])) {
            params.vector_loads = 0;
        }
    }
    params.tokens = tokens;
    params.heads = heads;
    params.tile_starts = tile_starts;
    params.tile_lengths = tile_lengths;
    params.quantized[0] = workspace.query;
    params.quantized[1] = workspace.key;
    params.scales[0] = workspace.query_scales;
    params.scales[1] = workspace.key_scales;
    params.value8 = workspace.value;
    params.value_scales = workspace.value_scales;
    params.value_maxima = workspace.value_maxima;
    if (inputs_ready == 0) {
        params.first_part = 0;
        params.last_part = 2;
        const int status = launch<false, false, true>(params, blocks, stream);
        if (status != 0) {
            return status;
        }
    }
    value_scales_kernel<<<heads, 256, 0, stream>>>(workspace.value_maxima, workspace.value_scales,
                                                   blocks);
    cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess) {
        return static_cast<int>(launched);
    }
    params.first_part = 2;
    params.last_part = 2;
    params.value_scales_ready = 1;
    return launch<false, false, true>(params, blocks, stream);
}

// VSA's pooled tiles from BF16 q, k and v (crates/mmh3-cuda/kernels/vsa_attention.cu:68-91).
int launch_pool(const void *query, const void *key, const void *value, int heads,
                const Mmh3AttentionLayout &layout, int tiles, const Mmh3VsaWorkspace &workspace,
                cudaStream_t stream) {
    InputsParams params = {};
    const void *sources[3] = {query, key, value};
    params.vector_loads = 1;
    for (int part = 0; part < 3; part++) {
        params.source[part] = static_cast<const __nv_bfloat16 *>(sources[part]);
        params.token_stride[part] = layout.token_stride[part];
        params.head_stride[part] = layout.head_stride[part];
        if (!aligned_rows(sources[part], layout.token_stride[part], layout.head_stride[part])) {
            params.vector_loads = 0;
        }
    }
    params.heads = heads;
    params.tile_starts = workspace.tile_starts;
    params.tile_lengths = workspace.tile_lengths;
    params.pooled[0] = workspace.pooled_query;
    params.pooled[1] = workspace.pooled_key;
    params.pooled[2] = workspace.pooled_value;
    params.first_part = 0;
    params.last_part = 2;
    return launch<false, true, false>(params, tiles, stream);
}

// Sol-Attn's block statistics: the same pooling pass over blocks of 64 tokens (no tile tables),
// into the mean query, mean key and summed value of the sparse workspace.
int launch_block_statistics(const void *query, const void *key, const void *value, int tokens,
                            int heads, const Mmh3AttentionLayout &layout,
                            const Mmh3SparseWorkspace &workspace, cudaStream_t stream) {
    InputsParams params = {};
    const void *sources[3] = {query, key, value};
    params.vector_loads = 1;
    for (int part = 0; part < 3; part++) {
        params.source[part] = static_cast<const __nv_bfloat16 *>(sources[part]);
        params.token_stride[part] = layout.token_stride[part];
        params.head_stride[part] = layout.head_stride[part];
        if (!aligned_rows(sources[part], layout.token_stride[part], layout.head_stride[part])) {
            params.vector_loads = 0;
        }
    }
    params.heads = heads;
    params.tokens = tokens;
    params.pooled[0] = workspace.centroids;
    params.pooled[1] = workspace.block_keys;
    params.pooled[2] = workspace.value_sums;
    params.first_part = 0;
    params.last_part = 2;
    return launch<false, true, false>(params, (tokens + BLOCK_ROWS - 1) / BLOCK_ROWS, stream);
}

} // namespace mmh3
