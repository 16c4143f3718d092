// Dense INT8 QK^T / FP8 PV attention for heads of 128 on sm_100a, over a prepared workspace: INT8 q
// and k [tokens, heads, 128] with one scale per head and 64-token block, FP8 E4M3 V transposed to
// [heads, 128, blocks * 64] with one scale per head. Softmax and accumulation are FP32, the output
// BF16. It computes what the reference's quantized attention_kernel<DENSE> computes
// (crates/mmh3-cuda/kernels/quantized_attention.cu:247-549) with the design of the BF16 kernel of
// this library:
//
// - a CTA owns two tiles of 128 query rows of one head and walks the keys in blocks of 128;
// - warp 8 streams Q8 once and then K8 and V8 tiles (16 KiB each) with TMA through a ring;
// - warp 9 issues tcgen05 MMAs: S = Q8 K8^T with kind::i8 into INT32 tensor memory, and
//   O += P8 V8^T with kind::f8f6f4 into FP32 tensor memory, P8 read from tensor memory;
// - warps 0-7 are the softmax, one thread per query row: INT32 scores are dequantized with
//   scale * log2(e) * q_scale[row block] * k_scale[key block] (a 128-key block spans two key
//   scales), the probabilities are scaled and rounded to E4M3 as the reference does, and written
//   over the first 32 columns of S. Maxima are taken on the integers, the FP32 arithmetic runs on
//   pairs (fma.rn.f32x2), and a quarter of the exponentials on a polynomial instead of the MUFU:
//   with MMAs twice as fast as BF16's, this kernel is bound by its softmax instruction stream.
//
// The running maximum may lag the true one by a factor of two before O is rescaled; E4M3
// saturates at 448, so the probabilities are scaled by 224 instead of the reference's 448.
#include <cfloat>
#include <cmath>
#include <cuda_fp8.h>
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace mmh3 {

namespace {

using namespace sm100;

constexpr int TILE_M = 128;
constexpr int QUERY_TILES = 2;
constexpr int TILE_N = 128;
constexpr int STAGES = 8;
constexpr int TILE_BYTES = 128 * 128; // 128 rows of 128 one-byte elements: one swizzled slab
constexpr int SOFTMAX_WARPS = 4 * QUERY_TILES;
constexpr int LOAD_WARP = SOFTMAX_WARPS;
constexpr int MMA_WARP = SOFTMAX_WARPS + 1;
constexpr int THREADS = (SOFTMAX_WARPS + 4) * 32;
constexpr int SOFTMAX_REGISTERS = 208;
constexpr int OTHER_REGISTERS = 88;
// What the third warpgroup releases must cover what the softmax warpgroups take (see the BF16
// kernel): the kernel launches with 168 registers per thread.
constexpr int LAUNCH_REGISTERS = 168;
static_assert((LAUNCH_REGISTERS - OTHER_REGISTERS) * 128 >=
                  (SOFTMAX_REGISTERS - LAUNCH_REGISTERS) * SOFTMAX_WARPS * 32,
              "the softmax warps ask for more registers than the other warps release");

constexpr int SMEM_QUERY = 0;
constexpr int SMEM_RING = QUERY_TILES * TILE_BYTES;
constexpr int SMEM_BARRIERS = SMEM_RING + STAGES * TILE_BYTES;
constexpr int SMEM_BYTES = SMEM_BARRIERS + 256 + 1024;

enum Barrier {
    QUERY_FULL = 0,
    RING_FULL = 1,
    RING_EMPTY = RING_FULL + STAGES,
    SCORES_FULL = RING_EMPTY + STAGES,
    PROBABILITIES_FULL = SCORES_FULL + QUERY_TILES,
    OUTPUT_FULL = PROBABILITIES_FULL + QUERY_TILES,
    BARRIERS = OUTPUT_FULL + 1,
};
static_assert(BARRIERS * 8 + 8 <= 256, "the barriers outgrew their corner of shared memory");

constexpr uint32_t TMEM_COLUMNS = 512;
constexpr uint32_t TMEM_SCORES = 0;
constexpr uint32_t TMEM_OUTPUT = 256;

constexpr uint32_t SCORE_MMA =
    instruction_descriptor(ACCUMULATE_S32, FORMAT_S8, FORMAT_S8, 0, 0, TILE_M, TILE_N);
constexpr uint32_t OUTPUT_MMA =
    instruction_descriptor(ACCUMULATE_F32, FORMAT_E4M3, FORMAT_E4M3, 0, 0, TILE_M, HEAD_DIM);

// The probabilities go to E4M3 times 224: the reference's factor of 448, halved because the running
// maximum here may lag the true one by a factor of two. log2(224) folds it into the exponent.
constexpr float LOG2_224 = 7.807354922057604f;
constexpr float RESCALE_THRESHOLD = 1.0f;
// Of every four pairs of probabilities, how many take the polynomial exp2 instead of the MUFU.
// Measured at L = 66,048 with the integer add below: 0 -> 47.6 ms, 1 -> 50.9 ms, 2 -> 53.0 ms.
constexpr int POLYNOMIAL_PAIRS_OF_4 = 0;
// An integer score s, |s| < 2^22, becomes the float 1.5 * 2^23 + s by adding these bits to it: an
// integer add where a conversion would be, which leaves the conversion unit to the exponentials.
constexpr int32_t MAGIC_BITS = 0x4B400000;
constexpr float MAGIC_VALUE = 12582912.0f;
// What a key past the last token scores, before the scales: below every real score (at most
// 128 * 127 * 127 in magnitude) by far, and small enough to stay finite after scaling.
constexpr int32_t MASKED_SCORE = -(1 << 28);

struct QuantizedMaps {
    CUtensorMap query; // [128, tokens, heads] INT8
    CUtensorMap key;   // [128, tokens, heads] INT8
    CUtensorMap value; // [padded tokens, 128, heads] E4M3
};

// K-major descriptor of a tile of 128-byte rows; contraction step `step` is 32 bytes further on.
__device__ __forceinline__ uint64_t row_operand(uint32_t tile) {
    return smem_descriptor(tile, 16, 1024);
}

__global__ void __launch_bounds__(THREADS, 1)
    quantized_dense_kernel(const __grid_constant__ QuantizedMaps maps,
                           __nv_bfloat16 *__restrict__ output, int tokens, int blocks64,
                           const float *__restrict__ query_scales,
                           const float *__restrict__ key_scales,
                           const float *__restrict__ value_scales, int64_t output_token_stride,
                           int64_t output_head_stride, int vector_stores, float scale_log2,
                           unsigned int *status) {
    extern __shared__ uint8_t shared_memory[];
    const uint32_t base = (smem_u32(shared_memory) + 1023u) & ~1023u;
    uint8_t *aligned = shared_memory + (base - smem_u32(shared_memory));
    const uint32_t barriers = base + SMEM_BARRIERS;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + SMEM_BARRIERS +
                                                                         BARRIERS * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const Watchdog watchdog = {abort_flag, status};
    auto barrier = [&](int index) { return barriers + index * 8; };

    if (*reinterpret_cast<volatile unsigned int *>(status) != 0) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int head = blockIdx.y;
    const int first_query = blockIdx.x * (QUERY_TILES * TILE_M);
    const int blocks = (tokens + TILE_N - 1) / TILE_N;

    if (threadIdx.x == 0) {
        mbar_init(barrier(QUERY_FULL), 1);
        for (int stage = 0; stage < STAGES; stage++) {
            mbar_init(barrier(RING_FULL + stage), 1);
            mbar_init(barrier(RING_EMPTY + stage), 1);
        }
        for (int tile = 0; tile < QUERY_TILES; tile++) {
            mbar_init(barrier(SCORES_FULL + tile), 1);
            mbar_init(barrier(PROBABILITIES_FULL + tile), TILE_M);
        }
        mbar_init(barrier(OUTPUT_FULL), 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), TMEM_COLUMNS);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp >= SOFTMAX_WARPS) {
        register_decrease<OTHER_REGISTERS>();
    }
    if (warp == LOAD_WARP) {
        if (lane == 0) {
            tma_prefetch_descriptor(&maps.query);
            tma_prefetch_descriptor(&maps.key);
            tma_prefetch_descriptor(&maps.value);
            mbar_expect_tx(barrier(QUERY_FULL), QUERY_TILES * TILE_BYTES);
            for (int tile = 0; tile < QUERY_TILES; tile++) {
                tma_load_3d(base + SMEM_QUERY + tile * TILE_BYTES, &maps.query,
                            barrier(QUERY_FULL), 0, first_query + tile * TILE_M, head);
            }
            for (int item = 0; item < 2 * blocks; item++) {
                const int stage = item % STAGES;
                const int use = item / STAGES;
                if (use > 0 && !mbar_wait(barrier(RING_EMPTY + stage), (use - 1) & 1, watchdog,
                                          STATUS_QUANTIZED | 1)) {
                    break;
                }
                mbar_expect_tx(barrier(RING_FULL + stage), TILE_BYTES);
                const uint32_t destination = base + SMEM_RING + stage * TILE_BYTES;
                if (item & 1) {
                    // 128 keys along the rows of all 128 dimensions.
                    tma_load_3d(destination, &maps.value, barrier(RING_FULL + stage),
                                (item / 2) * TILE_N, 0, head);
                } else {
                    tma_load_3d(destination, &maps.key, barrier(RING_FULL + stage), 0,
                                (item / 2) * TILE_N, head);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            const uint32_t query_tiles = base + SMEM_QUERY;
            const uint32_t ring = base + SMEM_RING;
            const uint64_t query_operands[QUERY_TILES] = {row_operand(query_tiles),
                                                          row_operand(query_tiles + TILE_BYTES)};
            auto score = [&](int tile, uint32_t key_tile) {
                const uint64_t key_operand = row_operand(key_tile);
                #pragma unroll
                for (int step = 0; step < HEAD_DIM / 32; step++) {
                    mma_i8_ss(tmem + TMEM_SCORES + tile * TILE_N,
                              advance_descriptor(query_operands[tile], step * 32),
                              advance_descriptor(key_operand, step * 32), SCORE_MMA, step > 0);
                }
                tcgen05_commit(barrier(SCORES_FULL + tile));
            };
            auto accumulate = [&](int tile, uint32_t value_tile, bool first) {
                const uint64_t operand = row_operand(value_tile);
                #pragma unroll
                for (int step = 0; step < TILE_N / 32; step++) {
                    // P is E4M3, four to a column: 32 keys are 8 columns.
                    mma_f8_ts(tmem + TMEM_OUTPUT + tile * HEAD_DIM,
                              tmem + TMEM_SCORES + tile * TILE_N + step * 8,
                              advance_descriptor(operand, step * 32), OUTPUT_MMA,
                              !first || step > 0);
                }
            };
            bool alive = mbar_wait(barrier(QUERY_FULL), 0, watchdog, STATUS_QUANTIZED | 2) &&
                         mbar_wait(barrier(RING_FULL + 0), 0, watchdog, STATUS_QUANTIZED | 3);
            if (alive) {
                tcgen05_fence_after();
                score(0, ring);
                score(1, ring);
                tcgen05_commit(barrier(RING_EMPTY + 0));
            }
            int item = 1;
            for (int block = 0; alive && block < blocks; block++, item += 2) {
                const int value_stage = item % STAGES;
                const int key_stage = (item + 1) % STAGES;
                const bool more = block + 1 < blocks;
                alive = mbar_wait(barrier(RING_FULL + value_stage), (item / STAGES) & 1, watchdog,
                                  STATUS_QUANTIZED | 4) &&
                        (!more || mbar_wait(barrier(RING_FULL + key_stage),
                                            ((item + 1) / STAGES) & 1, watchdog,
                                            STATUS_QUANTIZED | 5));
                if (!alive) {
                    break;
                }
                const uint32_t value_tile = ring + value_stage * TILE_BYTES;
                const uint32_t key_tile = ring + key_stage * TILE_BYTES;
                #pragma unroll
                for (int tile = 0; tile < QUERY_TILES; tile++) {
                    alive = mbar_wait(barrier(PROBABILITIES_FULL + tile), block & 1, watchdog,
                                      STATUS_QUANTIZED | 6);
                    if (!alive) {
                        break;
                    }
                    tcgen05_fence_after();
                    accumulate(tile, value_tile, block == 0);
                    if (tile == QUERY_TILES - 1) {
                        tcgen05_commit(barrier(RING_EMPTY + value_stage));
                    }
                    if (more) {
                        score(tile, key_tile);
                        if (tile == QUERY_TILES - 1) {
                            tcgen05_commit(barrier(RING_EMPTY + key_stage));
                        }
                    }
                }
            }
            if (alive) {
                tcgen05_commit(barrier(OUTPUT_FULL));
            }
        }
    } else if (warp < SOFTMAX_WARPS) {
        register_increase<SOFTMAX_REGISTERS>();
        const int tile = warp / 4;
        const int row = (warp % 4) * 32 + lane;
        const int token = first_query + tile * TILE_M + row;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const uint32_t scores = tmem + lane_base + TMEM_SCORES + tile * TILE_N;
        const uint32_t accumulator = tmem + lane_base + TMEM_OUTPUT + tile * HEAD_DIM;
        const float *head_key_scales = key_scales + static_cast<size_t>(head) * blocks64;
        // Rows past the last token read no scale; their scores are zero and never stored.
        const float query_factor =
            scale_log2 * (token < tokens ? query_scales[static_cast<size_t>(head) * blocks64 +
                                                        token / 64]
                                         : 0.0f);
        float maximum = -FLT_MAX;
        float2 sums[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
        bool alive = true;
        for (int block = 0; block < blocks; block++) {
            // The scales of the two 64-key halves of this block. A half past the last block holds
            // masked scores only and borrows the other's scale.
            const float factor_low = query_factor * __ldg(head_key_scales + 2 * block);
            const float factor_high =
                2 * block + 1 < blocks64 ? query_factor * __ldg(head_key_scales + 2 * block + 1)
                                         : factor_low;
            alive = mbar_wait(barrier(SCORES_FULL + tile), block & 1, watchdog,
                              STATUS_QUANTIZED | 7);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) {
                break;
            }
            tcgen05_fence_after();
            uint32_t raw[4][32];
            #pragma unroll
            for (int chunk = 0; chunk < 4; chunk++) {
                tmem_load_32(scores + chunk * 32, raw[chunk]);
            }
            tmem_wait_load();
            const int valid = tokens - block * TILE_N;
            if (valid < TILE_N) {
                // Keys past the last token: an integer far below any score.
                #pragma unroll
                for (int index = 0; index < TILE_N; index++) {
                    if (index >= valid) {
                        raw[index / 32][index % 32] = static_cast<uint32_t>(MASKED_SCORE);
                    }
                }
            }
            // The maximum of each 64-key half as an integer, three values to an instruction, then
            // the two candidates in FP32 with their scales.
            int maxima[2];
            #pragma unroll
            for (int half = 0; half < 2; half++) {
                int partial[2] = {static_cast<int>(raw[half * 2][0]),
                                  static_cast<int>(raw[half * 2][1])};
                #pragma unroll
                for (int index = 2; index + 1 < 64; index += 2) {
                    const int chain = (index / 2) % 2;
                    partial[chain] = __vimax3_s32(
                        partial[chain], static_cast<int>(raw[half * 2 + index / 32][index % 32]),
                        static_cast<int>(raw[half * 2 + (index + 1) / 32][(index + 1) % 32]));
                }
                maxima[half] = max(partial[0], partial[1]);
            }
            const float block_maximum = fmaxf(static_cast<float>(maxima[0]) * factor_low,
                                              static_cast<float>(maxima[1]) * factor_high);
            // The maximum may lag by up to one (a factor of two in the probabilities), which the
            // factor of 224 instead of 448 leaves room for in E4M3; the division by the row sum
            // makes the result exact again.
            const bool grown = block_maximum - maximum > RESCALE_THRESHOLD;
            if (block == 0) {
                maximum = block_maximum;
            } else if (__any_sync(0xffffffffu, grown)) {
                const float raised = fmaxf(maximum, block_maximum);
                const float correction = exp2_approx(maximum - raised);
                maximum = raised;
                const float2 correction2 = make_float2(correction, correction);
                sums[0] = __fmul2_rn(sums[0], correction2);
                sums[1] = __fmul2_rn(sums[1], correction2);
                #pragma unroll
                for (int chunk = 0; chunk < 4; chunk++) {
                    uint32_t values[32];
                    tmem_load_32(accumulator + chunk * 32, values);
                    tmem_wait_load();
                    #pragma unroll
                    for (int index = 0; index < 32; index++) {
                        values[index] =
                            __float_as_uint(__uint_as_float(values[index]) * correction);
                    }
                    tmem_store_32(accumulator + chunk * 32, values);
                }
            }
            // 224 * exp2(score - maximum) as E4M3, two elements at a time.
            const float offset = LOG2_224 - maximum;
            uint32_t packed[32];
            // MASKED is set for the last block of a sequence that does not fill it: the keys past
            // the last token then get an exponent of minus infinity whatever their scale is (a scale
            // may be zero, which would turn the masked integer into a score of zero).
            auto exponentials = [&](auto masked) {
                constexpr bool MASKED = decltype(masked)::value;
                #pragma unroll
                for (int quad = 0; quad < 32; quad++) {
                    const float factor = quad < 16 ? factor_low : factor_high;
                    const float2 factor2 = make_float2(factor, factor);
                    // (MAGIC + s) * factor + (offset - MAGIC * factor) = s * factor + offset: the
                    // product is exact inside the FMA, and the constant, a few hundred at most,
                    // is off by less than 2^-15 of an exponent.
                    const float shifted = fmaf(-MAGIC_VALUE, factor, offset);
                    const float2 offset2 = make_float2(shifted, shifted);
                    uint16_t halves[2];
                    #pragma unroll
                    for (int pair = 0; pair < 2; pair++) {
                        const int index = quad * 4 + pair * 2;
                        const float2 raw_pair = make_float2(
                            __int_as_float(static_cast<int32_t>(raw[index / 32][index % 32]) +
                                           MAGIC_BITS),
                            __int_as_float(
                                static_cast<int32_t>(raw[(index + 1) / 32][(index + 1) % 32]) +
                                MAGIC_BITS));
                        float2 x = __ffma2_rn(raw_pair, factor2, offset2);
                        if (MASKED) {
                            x.x = index < valid ? x.x : -INFINITY;
                            x.y = index + 1 < valid ? x.y : -INFINITY;
                        }
                        float2 probability;
                        if ((quad * 2 + pair) % 4 < POLYNOMIAL_PAIRS_OF_4) {
                            probability = exp2_polynomial(x);
                        } else {
                            probability = make_float2(exp2_approx(x.x), exp2_approx(x.y));
                        }
                        sums[pair] = __fadd2_rn(sums[pair], probability);
                        // cvt packs its first source into the upper byte.
                        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;"
                            : "=h"(halves[pair])
                            : "f"(probability.y), "f"(probability.x));
                    }
                    packed[quad] = static_cast<uint32_t>(halves[0]) |
                                   (static_cast<uint32_t>(halves[1]) << 16);
                }
            };
            if (valid < TILE_N) {
                exponentials(std::true_type{});
            } else {
                exponentials(std::false_type{});
            }
            tmem_store_32(scores, packed);
            tmem_wait_store();
            tcgen05_fence_before();
            mbar_arrive(barrier(PROBABILITIES_FULL + tile));
        }
        if (alive) {
            alive = mbar_wait(barrier(OUTPUT_FULL), 0, watchdog, STATUS_QUANTIZED | 8);
            alive = __all_sync(0xffffffffu, alive);
        }
        if (alive) {
            tcgen05_fence_after();
            // The sums carry the factor of 448 the probabilities do.
            const float inverse =
                value_scales[head] / ((sums[0].x + sums[0].y) + (sums[1].x + sums[1].y));
            __nv_bfloat16 *output_row =
                output + static_cast<int64_t>(token) * output_token_stride +
                static_cast<int64_t>(head) * output_head_stride;
            #pragma unroll
            for (int chunk = 0; chunk < 4; chunk++) {
                uint32_t values[32];
                tmem_load_32(accumulator + chunk * 32, values);
                tmem_wait_load();
                if (token < tokens) {
                    uint32_t packed[16];
                    #pragma unroll
                    for (int pair = 0; pair < 16; pair++) {
                        packed[pair] = pack_bf16(__uint_as_float(values[pair * 2]) * inverse,
                                                 __uint_as_float(values[pair * 2 + 1]) * inverse);
                    }
                    if (vector_stores) {
                        uint4 *destination = reinterpret_cast<uint4 *>(output_row + chunk * 32);
                        #pragma unroll
                        for (int part = 0; part < 4; part++) {
                            destination[part] =
                                make_uint4(packed[part * 4], packed[part * 4 + 1],
                                           packed[part * 4 + 2], packed[part * 4 + 3]);
                        }
                    } else {
                        uint16_t *destination =
                            reinterpret_cast<uint16_t *>(output_row + chunk * 32);
                        #pragma unroll
                        for (int pair = 0; pair < 16; pair++) {
                            destination[pair * 2] = static_cast<uint16_t>(packed[pair] & 0xffffu);
                            destination[pair * 2 + 1] = static_cast<uint16_t>(packed[pair] >> 16);
                        }
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        if (*abort_flag != 0) {
            for (int spin = 0; spin < 64; spin++) {
                __nanosleep(1000);
            }
        }
        tcgen05_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
}

} // namespace

int launch_quantized_attention(const Mmh3QuantizedWorkspace &workspace, void *output, int tokens,
                               int heads, const Mmh3AttentionLayout &layout, float scale,
                               const Mmh3VsaWorkspace *vsa, int tiles, const void *gate,
                               int64_t gate_stride, cudaStream_t stream) {
    if (vsa != nullptr) {
        return launch_vsa_attention_quantized(workspace, output, tokens, heads, layout, scale, *vsa,
                                              tiles, gate, gate_stride, stream);
    }
    if (!(scale > 0.0f) || !std::isfinite(scale)) {
        return INVALID_VALUE;
    }
    unsigned int *status = status_pointer();
    if (status == nullptr) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    static SharedMemoryOptIn shared_memory;
    const cudaError_t configured = shared_memory.ensure(quantized_dense_kernel, SMEM_BYTES);
    if (configured != cudaSuccess) {
        return static_cast<int>(configured);
    }
    const int blocks64 = (tokens + 63) / 64;
    const uint64_t padded = static_cast<uint64_t>(blocks64) * 64;
    QuantizedMaps maps;
    const uint64_t row_dimensions[3] = {HEAD_DIM, static_cast<uint64_t>(tokens),
                                        static_cast<uint64_t>(heads)};
    const uint64_t row_strides[2] = {static_cast<uint64_t>(heads) * HEAD_DIM, HEAD_DIM};
    const uint32_t row_box[3] = {HEAD_DIM, TILE_M, 1};
    const uint64_t value_dimensions[3] = {padded, HEAD_DIM, static_cast<uint64_t>(heads)};
    const uint64_t value_strides[2] = {padded, padded * HEAD_DIM};
    const uint32_t value_box[3] = {TILE_N, HEAD_DIM, 1};
    if (!encode_tensor_map(&maps.query, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, workspace.query,
                           row_dimensions, row_strides, row_box) ||
        !encode_tensor_map(&maps.key, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, workspace.key,
                           row_dimensions, row_strides, row_box) ||
        !encode_tensor_map(&maps.value, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, workspace.value,
                           value_dimensions, value_strides, value_box)) {
        return NOT_SUPPORTED;
    }
    auto *out = static_cast<__nv_bfloat16 *>(output);
    const int vector_stores = reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                              layout.token_stride[OUTPUT] % 8 == 0 &&
                              layout.head_stride[OUTPUT] % 8 == 0;
    const dim3 grid((tokens + QUERY_TILES * TILE_M - 1) / (QUERY_TILES * TILE_M), heads);
    quantized_dense_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(
        maps, out, tokens, blocks64, workspace.query_scales, workspace.key_scales,
        workspace.value_scales, layout.token_stride[OUTPUT], layout.head_stride[OUTPUT],
        vector_stores, scale * LOG2_E, status);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mmh3
