// The passes over q, k and v that come before the attention: per-head RMSNorm and RoPE, INT8 q and
// k with one scale per head and block, FP8 V transposed, the |v| maxima, and VSA's pooled tiles.
// One kernel template covers them all. Every element of q, k and v is read once and each quantized
// byte written once.
//
// The results are bit-identical to the reference's (crates/mmh3-cuda/kernels/dit.cu:98-391,
// quantized_attention.cu:85-241, vsa_attention.cu:68-91), which fixes the order of every FP32
// operation: the sum of squares as 32 chains over dimensions l, l + 32, l + 64, l + 96 joined by a
// butterfly over l, the row-ordered sums of the pooled tiles, IEEE divisions by the scales, and
// round-to-nearest-even conversions.
//
// A CTA of 256 threads owns one block of 64 tokens (or one VSA tile of up to 64) of one head at a
// time. Four threads share a row; thread c of the four holds dimensions 16 G + 4 c + {0, 1, 2, 3}
// for G = 0 .. 7 and keeps them in registers from the load to the stores. That choice makes eight
// of the 32 chains whole in one thread (two shuffle rounds join the four threads, the rest of the
// butterfly is private), and whenever the rotary pairs are a multiple of 16 it puts both
// dimensions of every pair, and the pair's cosine and sine for the life of the CTA, in one thread
// too. Shared memory is then only the weights, the block maximum, the transposition of V and the
// staging of the pooled sums. The rows of the next turn are in flight in registers while one is
// worked on.
#include <cuda_fp8.h>
#include <type_traits>

#include "common.cuh"

namespace mmh3 {

namespace {

constexpr int BLOCK_ROWS = 64;
constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
// Threads that share a row, and the groups of four neighbouring dimensions each of them holds.
constexpr int ROW_THREADS = THREADS / BLOCK_ROWS;
constexpr int GROUPS = HEAD_DIM / (4 * ROW_THREADS);
constexpr int HEADS_PER_CTA = 16;
// Strides in shared memory that keep the threads served together in different banks: a staged row
// is 128 BF16 values of which a thread touches 8 bytes at a time (16 threads, four rows, at once).
constexpr int STAGED_STRIDE = HEAD_DIM + 16; // BF16 values
constexpr int EXCHANGE_STRIDE = HEAD_DIM + 4; // floats
// INT8 rows on their way out, a warp's eight at a time: 128 bytes of which a thread writes four at
// a time and later reads 16.
constexpr int CODES_STRIDE = HEAD_DIM + 16; // bytes
// Adding 1.5 * 2^23 rounds a float below 2^22 in magnitude to the nearest integer, ties to even,
// and leaves it in two's complement in the low bits of the sum.
constexpr float ROUNDING_MAGIC = 12582912.0f;
// How the rotary embedding finds a dimension's partner.
enum Rotation { NO_ROTATION = 0, IN_THREAD = 1, THROUGH_SHARED_MEMORY = 2 };

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
    // Whether rows can be read in 8-byte pieces.
    int vector_loads;
    // Heads one CTA walks, sharing the cosines and sines of its block's angles.
    int heads_per_cta;
};

// The largest of the warp's values, none of them negative or NaN: such floats order as their bits
// do, and the warp reduces unsigned integers in one instruction.
__device__ __forceinline__ float warp_max(float value) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(value)));
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
    // For a divisor known when compiling, with its reciprocal rounded by the compiler.
    __device__ __forceinline__ constexpr Divider(float divisor, float rounded_reciprocal)
        : scale(divisor), reciprocal(rounded_reciprocal), exact(true) {}
    // The quotient where `exact` holds, and where it does not. A caller with many values asks
    // `exact` once and runs one of two loops.
    template <bool QUICK> __device__ __forceinline__ float quotient(float x) const {
        if (QUICK) {
            const float estimate = __fmul_rn(x, reciprocal);
            const float residual = __fmaf_rn(-estimate, scale, x);
            return __fmaf_rn(residual, reciprocal, estimate);
        }
        return __fdiv_rn(x, scale);
    }
    // Two quotients at a time, as two independent IEEE operations per packed instruction;
    // q * (-scale) + x is the same number as -q * scale + x.
    template <bool QUICK> __device__ __forceinline__ float2 quotients(float2 x) const {
        if (QUICK) {
            const float2 estimate = __fmul2_rn(x, make_float2(reciprocal, reciprocal));
            const float2 residual = __ffma2_rn(estimate, make_float2(-scale, -scale), x);
            return __ffma2_rn(residual, make_float2(reciprocal, reciprocal), estimate);
        }
        return make_float2(__fdiv_rn(x.x, scale), __fdiv_rn(x.y, scale));
    }
    // `body(std::true_type)` where the quick quotient is right, `body(std::false_type)` otherwise.
    template <typename Body> __device__ __forceinline__ void dispatch(const Body &body) const {
        if (exact) {
            body(std::true_type());
        } else {
            body(std::false_type());
        }
    }
};

// maximum / LEVELS as IEEE division gives it wherever the quotient is 1e-30 or more, which is all a
// scale keeps of it; LEVELS is 127 or 448, whose significands are not all ones.
template <int LEVELS> __device__ __forceinline__ float scale_for(float maximum) {
    constexpr Divider divide(static_cast<float>(LEVELS), 1.0f / static_cast<float>(LEVELS));
    return fmaxf(divide.quotient<true>(maximum), 1e-30f);
}

__device__ __forceinline__ float low_half(uint32_t word) { return __uint_as_float(word << 16); }
// The two BF16 values of a word as floats, the low half first.
__device__ __forceinline__ float2 both_halves(uint32_t word) {
    return make_float2(__uint_as_float(word << 16), __uint_as_float(word & 0xffff0000u));
}
__device__ __forceinline__ float high_half(uint32_t word) {
    return __uint_as_float(word & 0xffff0000u);
}

// Two floats rounded to BF16, `low` in the low half.
__device__ __forceinline__ uint32_t pack_bf16(float low, float high) {
    uint32_t word;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(word) : "f"(high), "f"(low));
    return word;
}

// Two floats to saturating E4M3, `low` in the low byte of the 16 bits.
__device__ __forceinline__ uint32_t pack_e4m3(float low, float high) {
    uint16_t pair;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(high), "f"(low));
    return pair;
}

// The integers nearest to four quotients of magnitude at most 127, as four bytes.
__device__ __forceinline__ uint32_t pack_int8(float2 low, float2 high) {
    const float2 magic = make_float2(ROUNDING_MAGIC, ROUNDING_MAGIC);
    const float2 first = __fadd2_rn(low, magic), second = __fadd2_rn(high, magic);
    return __byte_perm(
        __byte_perm(__float_as_uint(first.x), __float_as_uint(first.y), 0x0040),
        __byte_perm(__float_as_uint(second.x), __float_as_uint(second.y), 0x0040), 0x5410);
}

// The largest magnitude among four BF16 values.
__device__ __forceinline__ float group_max(const uint2 &group) {
    return fmaxf(fmaxf(fabsf(low_half(group.x)), fabsf(high_half(group.x))),
                 fmaxf(fabsf(low_half(group.y)), fabsf(high_half(group.y))));
}

// A thread's share of a row as floats: values[G][j] holds dimensions 16 G + 4 c + 2 j and the
// next, c the thread's place among the four of its row. The arithmetic runs on such pairs with
// the packed FP32 instructions, each half an IEEE operation of its own.
struct RowShare {
    float2 values[GROUPS][2];

    __device__ __forceinline__ void unpack(const uint2 (&groups)[GROUPS]) {
        #pragma unroll
        for (int group = 0; group < GROUPS; group++) {
            values[group][0] = both_halves(groups[group].x);
            values[group][1] = both_halves(groups[group].y);
        }
    }

    // The row's sum of squares, the same bits in all four threads of the row. Chain l of the row
    // runs over dimensions l, l + 32, l + 64, l + 96; with l = 16 h + 4 c + i its four dimensions
    // are in groups h, h + 2, h + 4, h + 6 of this thread. The butterfly over l goes 16 (h, in
    // this thread), 8 and 4 (the two bits of c, across the threads of the row), 2 and 1 (the bits
    // of i, in this thread), and an addition gives both of its sides the same bits, so every
    // thread ends with the sum any lane of a 32-lane butterfly would hold.
    __device__ __forceinline__ float sum_of_squares() const {
        float2 sums[2]; // chains i = 0, 1 and i = 2, 3
        #pragma unroll
        for (int two = 0; two < 2; two++) {
            float2 chains[2];
            #pragma unroll
            for (int half = 0; half < 2; half++) {
                float2 squares = make_float2(0.0f, 0.0f);
                #pragma unroll
                for (int step = 0; step < GROUPS / 2; step++) {
                    const float2 value = values[2 * step + half][two];
                    squares = __ffma2_rn(value, value, squares);
                }
                chains[half] = squares;
            }
            sums[two] = __fadd2_rn(chains[0], chains[1]);
        }
        #pragma unroll
        for (int offset = ROW_THREADS / 2; offset > 0; offset /= 2) {
            #pragma unroll
            for (int two = 0; two < 2; two++) {
                sums[two] = __fadd2_rn(
                    sums[two], make_float2(__shfl_xor_sync(0xffffffffu, sums[two].x, offset),
                                           __shfl_xor_sync(0xffffffffu, sums[two].y, offset)));
            }
        }
        // Level 2 pairs i with i ^ 2, level 1 what is left.
        const float2 last = __fadd2_rn(sums[0], sums[1]);
        return last.x + last.y;
    }

    // Every value times `inverse` times its weight, the product of those two first.
    __device__ __forceinline__ void scale(float inverse, const float *weights, int place) {
        const float2 inverses = make_float2(inverse, inverse);
        #pragma unroll
        for (int group = 0; group < GROUPS; group++) {
            const float4 weight = *reinterpret_cast<const float4 *>(weights + 16 * group + 4 * place);
            values[group][0] =
                __fmul2_rn(values[group][0], __fmul2_rn(inverses, make_float2(weight.x, weight.y)));
            values[group][1] =
                __fmul2_rn(values[group][1], __fmul2_rn(inverses, make_float2(weight.z, weight.w)));
        }
    }

    // The largest magnitude among the values, two at a time with the three-input maximum.
    __device__ __forceinline__ float largest() const {
        float maxima[2] = {0.0f, 0.0f};
        #pragma unroll
        for (int group = 0; group < GROUPS; group++) {
            #pragma unroll
            for (int two = 0; two < 2; two++) {
                asm("max.f32 %0, %0, %1, %2;"
                    : "+f"(maxima[two])
                    : "f"(fabsf(values[group][two].x)), "f"(fabsf(values[group][two].y)));
            }
        }
        return fmaxf(maxima[0], maxima[1]);
    }

    // The values rounded to BF16.
    __device__ __forceinline__ void pack(uint2 (&groups)[GROUPS]) const {
        #pragma unroll
        for (int group = 0; group < GROUPS; group++) {
            groups[group] = make_uint2(pack_bf16(values[group][0].x, values[group][0].y),
                                       pack_bf16(values[group][1].x, values[group][1].y));
        }
    }
};

// The cosines and sines of a thread's pairs where pairs are a multiple of 16: pair 16 G + 4 c + i
// for the first pairs / 16 values of G.
struct PairAngles {
    float2 cosines[GROUPS / 2][2];
    float2 sines[GROUPS / 2][2];
};

// The split-half rotary embedding where dimension d < pairs = 16 * SIXTEENTHS turns with
// d + pairs: group G with group G + SIXTEENTHS of the same thread.
template <int SIXTEENTHS>
__device__ __forceinline__ void rotate_in_thread(RowShare &share, const PairAngles &angles) {
    #pragma unroll
    for (int group = 0; group < SIXTEENTHS; group++) {
        #pragma unroll
        for (int two = 0; two < 2; two++) {
            const float2 cosine = angles.cosines[group][two];
            const float2 sine = angles.sines[group][two];
            const float2 first = share.values[group][two];
            const float2 second = share.values[group + SIXTEENTHS][two];
            const float2 crossed = __fmul2_rn(sine, second);
            share.values[group][two] =
                __ffma2_rn(cosine, first, make_float2(-crossed.x, -crossed.y));
            share.values[group + SIXTEENTHS][two] =
                __ffma2_rn(sine, first, __fmul2_rn(cosine, second));
        }
    }
}

// The same for any number of pairs: the four threads of the row leave their values in the row's
// 128 floats of shared memory, `mine`, and find their partners' there; `cosines` and `sines` are
// those of the row's pairs.
__device__ __forceinline__ void rotate_through_shared_memory(RowShare &share, float *mine,
                                                             const float *cosines,
                                                             const float *sines, int pairs,
                                                             int place) {
    #pragma unroll
    for (int group = 0; group < GROUPS; group++) {
        *reinterpret_cast<float4 *>(mine + 16 * group + 4 * place) =
            make_float4(share.values[group][0].x, share.values[group][0].y,
                        share.values[group][1].x, share.values[group][1].y);
    }
    __syncwarp();
    #pragma unroll
    for (int group = 0; group < GROUPS; group++) {
        #pragma unroll
        for (int index = 0; index < 4; index++) {
            const int dimension = 16 * group + 4 * place + index;
            float &value = index % 2 ? share.values[group][index / 2].y
                                     : share.values[group][index / 2].x;
            if (dimension < pairs) {
                value = __fmaf_rn(cosines[dimension], value,
                                  -__fmul_rn(sines[dimension], mine[dimension + pairs]));
            } else if (dimension < 2 * pairs) {
                value = __fmaf_rn(sines[dimension - pairs], mine[dimension - pairs],
                                  __fmul_rn(cosines[dimension - pairs], value));
            }
        }
    }
    __syncwarp();
}

// Dynamic shared memory, only where the rotary pairs are not a multiple of 16: the cosines of the
// block's angles, [64][pairs], then the sines.
//
// SIXTEENTHS is pairs / 16 where the rotary pairs are a multiple of 16, else 0.
template <bool NORMALIZE, bool STATS, bool QUANTIZE, int SIXTEENTHS>
__global__ void __launch_bounds__(THREADS, (NORMALIZE || QUANTIZE) ? 2 : 4)
    inputs_kernel(const InputsParams p) {
    extern __shared__ __align__(16) float trig[];
    // The rows as BF16 where V is transposed or sums are pooled. The same memory holds rows of 128
    // floats for the rotary exchange through shared memory; the two uses take turns, a barrier
    // between them.
    __shared__ __align__(16) float exchange[BLOCK_ROWS][EXCHANGE_STRIDE];
    static_assert(BLOCK_ROWS * STAGED_STRIDE * 2 <= sizeof(exchange), "staged rows fit");
    __shared__ __align__(16) float weights[2][HEAD_DIM];
    __shared__ __align__(16) uint8_t codes[BLOCK_ROWS][CODES_STRIDE];
    __shared__ __align__(16) float maxima[2][WARPS];
    static_assert(WARPS == 8, "the block maximum reads eight warp maxima as two float4");
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
    const int row = threadIdx.x / ROW_THREADS;
    const int place = threadIdx.x % ROW_THREADS;
    const bool row_here = row < rows;
    const int rotation = SIXTEENTHS != 0                                      ? IN_THREAD
                         : !NORMALIZE || p.angles == nullptr || p.pairs == 0 ? NO_ROTATION
                                                                             : THROUGH_SHARED_MEMORY;
    const bool values_here =
        QUANTIZE && (p.value_head_maxima != nullptr || p.value_scales_ready != 0);
    const int items = head_count * (p.last_part - p.first_part + 1);
    // Word `word` (two BF16 values) of staged row `index`. Each run of 16 rows has its words
    // exchanged in eights, so that the threads that later read the same word of rows 16 apart
    // find them in different banks.
    uint32_t *const staged_words = reinterpret_cast<uint32_t *>(&exchange[0][0]);
    const auto staged_word = [](int index, int word) {
        return index * (STAGED_STRIDE / 2) + (word ^ (8 * ((index / 16) % 4)));
    };
    float *const cosines = trig;
    float *const sines = trig + BLOCK_ROWS * p.pairs;

    // The first group of this thread's row of the CTA's first head, in q, k and v, as an offset
    // from the tensor's first element.
    const auto first_group = [&](int part) {
        return (first_token + row) * p.token_stride[part] + first_head * p.head_stride[part] +
               4 * place;
    };
    const int64_t first_groups[3] = {first_group(0), first_group(1), first_group(2)};
    const auto pick = [](int part, const auto &of_three) {
        return part == 0 ? of_three[0] : part == 1 ? of_three[1] : of_three[2];
    };
    // The thread's eight groups of its row of one turn (q, k or v of the CTA's head number
    // `walked`); zeros past the block's rows.
    //
    // A turn that only passes through shared memory (V, and everything where nothing is normalized
    // or quantized) is loaded as whole rows instead, 16 threads to a row and 16 bytes each, four
    // times: groups 2 i and 2 i + 1 then hold piece lane % 16 of row 8 warp + 2 i + lane / 16.
    const auto in_rows = [](int part) { return part == 2 || (!NORMALIZE && !QUANTIZE); };
    uint2 next[GROUPS];
    auto load = [&](int part, int walked) {
        if (in_rows(part)) {
            const int64_t token_stride = pick(part, p.token_stride);
            const __nv_bfloat16 *source = pick(part, p.source) +
                                          (first_token + 8 * warp + lane / 16) * token_stride +
                                          (first_head + walked) * pick(part, p.head_stride) +
                                          8 * (lane % 16);
            #pragma unroll
            for (int two = 0; two < GROUPS / 2; two++) {
                uint4 piece = make_uint4(0, 0, 0, 0);
                if (8 * warp + 2 * two + lane / 16 < rows) {
                    const __nv_bfloat16 *from = source + 2 * two * token_stride;
                    if (p.vector_loads) {
                        piece = __ldg(reinterpret_cast<const uint4 *>(from));
                    } else {
                        uint32_t words[4];
                        #pragma unroll
                        for (int word = 0; word < 4; word++) {
                            const uint16_t *halves = reinterpret_cast<const uint16_t *>(from);
                            words[word] = __ldg(halves + 2 * word) |
                                          (uint32_t(__ldg(halves + 2 * word + 1)) << 16);
                        }
                        piece = make_uint4(words[0], words[1], words[2], words[3]);
                    }
                }
                next[2 * two] = make_uint2(piece.x, piece.y);
                next[2 * two + 1] = make_uint2(piece.z, piece.w);
            }
            return;
        }
        const __nv_bfloat16 *source =
            pick(part, p.source) + pick(part, first_groups) + walked * pick(part, p.head_stride);
        #pragma unroll
        for (int group = 0; group < GROUPS; group++) {
            next[group] = make_uint2(0, 0);
            if (row_here) {
                const __nv_bfloat16 *from = source + 16 * group;
                if (p.vector_loads) {
                    next[group] = __ldg(reinterpret_cast<const uint2 *>(from));
                } else {
                    uint16_t halves[4];
                    #pragma unroll
                    for (int element = 0; element < 4; element++) {
                        halves[element] = __ldg(reinterpret_cast<const uint16_t *>(from) + element);
                    }
                    next[group] = make_uint2(halves[0] | (uint32_t(halves[1]) << 16),
                                             halves[2] | (uint32_t(halves[3]) << 16));
                }
            }
        }
    };

    load(p.first_part, 0);
    PairAngles angles;
    if (NORMALIZE) {
        if (threadIdx.x < HEAD_DIM) {
            #pragma unroll
            for (int part = 0; part < 2; part++) {
                weights[part][threadIdx.x] =
                    p.weight[part] != nullptr ? __bfloat162float(p.weight[part][threadIdx.x]) : 0.0f;
            }
        }
        if (SIXTEENTHS != 0) {
            const float *row_angles = p.angles + (first_token + row) * p.pairs + 4 * place;
            #pragma unroll 1
            for (int group = 0; group < SIXTEENTHS; group++) {
                float found[2][4] = {};
                if (row_here) {
                    #pragma unroll
                    for (int index = 0; index < 4; index++) {
                        sincosf(row_angles[16 * group + index], &found[1][index], &found[0][index]);
                    }
                }
                // The loop is kept a loop for the size of sincosf; its results reach the
                // registers of their group through the unrolled comparison.
                #pragma unroll
                for (int slot = 0; slot < SIXTEENTHS; slot++) {
                    if (slot == group) {
                        #pragma unroll
                        for (int two = 0; two < 2; two++) {
                            angles.cosines[slot][two] =
                                make_float2(found[0][2 * two], found[0][2 * two + 1]);
                            angles.sines[slot][two] =
                                make_float2(found[1][2 * two], found[1][2 * two + 1]);
                        }
                    }
                }
            }
        } else if (rotation == THROUGH_SHARED_MEMORY) {
            for (int index = threadIdx.x; index < rows * p.pairs; index += THREADS) {
                sincosf(p.angles[first_token * p.pairs + index], &sines[index], &cosines[index]);
            }
        }
        __syncthreads();
    }
    // Where this thread's 16 bytes of FP8 V go within a head: the first of its two dimensions,
    // its 16 rows of the block.
    const int64_t value_column = static_cast<int64_t>(2 * (8 * warp + lane % 8)) * blocks * BLOCK_ROWS +
                                 static_cast<int64_t>(block) * BLOCK_ROWS + lane / 8 * 16;
    const int64_t quantized_block = (first_token * p.heads + first_head) * HEAD_DIM;
    int part = p.first_part;
    int walked = 0; // heads of the CTA's that are done
    for (int item = 0; item < items; item++) {
        const int head = first_head + walked;
        const size_t statistic = (static_cast<size_t>(head) * blocks + block) * HEAD_DIM;
        const bool last_part = part == p.last_part;
        const int next_part = last_part ? p.first_part : part + 1;
        uint2 groups[GROUPS];
        #pragma unroll
        for (int group = 0; group < GROUPS; group++) {
            groups[group] = next[group];
        }
        if (item + 1 < items) {
            load(next_part, walked + (last_part ? 1 : 0));
        }
        // Whether the rows of this turn go through shared memory as BF16.
        const bool staged = STATS || part == 2;
        const bool needs_maximum = QUANTIZE && (part < 2 || !values_here);
        float maximum = 0.0f;

        if (NORMALIZE && part < 2) {
            RowShare share;
            share.unpack(groups);
            const float squares = share.sum_of_squares();
            const float inverse = rsqrtf(__fmaf_rn(squares, 1.0f / HEAD_DIM, p.epsilon));
            share.scale(inverse, weights[part], place);
            if (SIXTEENTHS != 0) {
                rotate_in_thread<SIXTEENTHS>(share, angles);
            } else if (rotation == THROUGH_SHARED_MEMORY) {
                rotate_through_shared_memory(share, exchange[row], cosines + row * p.pairs,
                                             sines + row * p.pairs, p.pairs, place);
            }
            // Rounding keeps the order of magnitudes, so the largest rounded magnitude is the
            // rounded largest magnitude.
            if (QUANTIZE && row_here) {
                maximum = __bfloat162float(__float2bfloat16_rn(share.largest()));
            }
            share.pack(groups);
            if (p.normalized[part] != nullptr && row_here) {
                __nv_bfloat16 *target = p.normalized[part] + pick(part, first_groups) +
                                        walked * pick(part, p.head_stride);
                #pragma unroll
                for (int group = 0; group < GROUPS; group++) {
                    *reinterpret_cast<uint2 *>(target + 16 * group) = groups[group];
                }
            }
        } else if (needs_maximum) {
            #pragma unroll
            for (int group = 0; group < GROUPS; group++) {
                maximum = fmaxf(maximum, group_max(groups[group]));
            }
        }
        if (staged) {
            // The staged rows lie over other warps' exchange rows: those warps must be through
            // with their rotations, which a barrier of the turn before only tells for V behind a
            // quantized k.
            if (rotation == THROUGH_SHARED_MEMORY && !(QUANTIZE && part == 2)) {
                __syncthreads();
            }
            if (in_rows(part)) {
                #pragma unroll
                for (int two = 0; two < GROUPS / 2; two++) {
                    *reinterpret_cast<uint4 *>(
                        &staged_words[staged_word(8 * warp + 2 * two + lane / 16,
                                                  4 * (lane % 16))]) =
                        make_uint4(groups[2 * two].x, groups[2 * two].y, groups[2 * two + 1].x,
                                   groups[2 * two + 1].y);
                }
            } else {
                #pragma unroll
                for (int group = 0; group < GROUPS; group++) {
                    *reinterpret_cast<uint2 *>(
                        &staged_words[staged_word(row, 8 * group + 2 * place)]) = groups[group];
                }
            }
        }
        if (needs_maximum) {
            maximum = warp_max(maximum);
            if (lane == 0) {
                maxima[item % 2][warp] = maximum;
            }
        }
        if (staged || needs_maximum) {
            __syncthreads();
        }
        if (needs_maximum) {
            const float4 low = reinterpret_cast<const float4 *>(maxima[item % 2])[0];
            const float4 high = reinterpret_cast<const float4 *>(maxima[item % 2])[1];
            maximum = fmaxf(fmaxf(fmaxf(low.x, low.y), fmaxf(low.z, low.w)),
                            fmaxf(fmaxf(high.x, high.y), fmaxf(high.z, high.w)));
        }

        if constexpr (STATS) {
            // The sums over the rows in row order, one thread per dimension.
            if (threadIdx.x < HEAD_DIM) {
                const int dimension = threadIdx.x;
                // The thread's half of a word as the high half of a float, by one permutation.
                const uint32_t selector = dimension % 2 ? 0x3244u : 0x1044u;
                float sum = 0.0f;
                #pragma unroll
                for (int run = 0; run < BLOCK_ROWS / 16; run++) {
                    const uint32_t *words = staged_words + staged_word(16 * run, dimension / 2);
                    if (16 * run + 16 <= rows) {
                        #pragma unroll
                        for (int index = 0; index < 16; index++) {
                            sum += __uint_as_float(
                                __byte_perm(words[index * (STAGED_STRIDE / 2)], 0u, selector));
                        }
                    } else {
                        for (int index = 0; 16 * run + index < rows; index++) {
                            sum += __uint_as_float(
                                __byte_perm(words[index * (STAGED_STRIDE / 2)], 0u, selector));
                        }
                    }
                }
                p.pooled[part][statistic + dimension] = part == 2 ? sum : sum / rows;
            }
        }

        if (part == 2) {
            if (QUANTIZE && !values_here && threadIdx.x == 0) {
                p.value_maxima[head * blocks + block] = maximum;
            }
            if (values_here) {
                // FP8 V transposed into 64 columns per block, zero past the block's rows. A thread
                // takes 16 rows of two neighbouring dimensions and writes 16 bytes of each; a warp
                // takes all 64 rows of 16 dimensions, so that its stores fill 64-byte runs.
                float scale;
                if (p.value_head_maxima != nullptr) {
                    scale = scale_for<448>(p.value_head_maxima[head]);
                    if (block == 0 && threadIdx.x == 0) {
                        p.value_scales[head] = scale;
                    }
                } else {
                    scale = p.value_scales[head];
                }
                const Divider divide(scale);
                const int pair = 8 * warp + lane % 8;
                const int first_row = lane / 8 * 16;
                uint32_t bytes[2][4];
                divide.dispatch([&](auto quick) {
                    constexpr bool QUICK = decltype(quick)::value;
                    #pragma unroll
                    for (int word = 0; word < 4; word++) {
                        uint32_t halves[2][2];
                        #pragma unroll
                        for (int two = 0; two < 2; two++) {
                            float elements[2][2]; // [row of the two][dimension of the two]
                            #pragma unroll
                            for (int step = 0; step < 2; step++) {
                                // Rows past the block's were staged as zeros.
                                const int index = first_row + word * 4 + two * 2 + step;
                                const uint32_t both = staged_words[staged_word(index, pair)];
                                const float2 divided =
                                    divide.quotients<QUICK>(both_halves(both));
                                elements[step][0] = divided.x;
                                elements[step][1] = divided.y;
                            }
                            halves[0][two] = pack_e4m3(elements[0][0], elements[1][0]);
                            halves[1][two] = pack_e4m3(elements[0][1], elements[1][1]);
                        }
                        bytes[0][word] = __byte_perm(halves[0][0], halves[0][1], 0x5410);
                        bytes[1][word] = __byte_perm(halves[1][0], halves[1][1], 0x5410);
                    }
                });
                #pragma unroll
                for (int which = 0; which < 2; which++) {
                    uint8_t *target = p.value8 + value_column +
                                      (static_cast<int64_t>(head) * HEAD_DIM + which) *
                                          blocks * BLOCK_ROWS;
                    *reinterpret_cast<uint4 *>(target) = make_uint4(
                        bytes[which][0], bytes[which][1], bytes[which][2], bytes[which][3]);
                }
            }
        } else if constexpr (QUANTIZE) {
            const float scale = scale_for<127>(maximum);
            if (threadIdx.x == 0) {
                p.scales[part][head * blocks + block] = scale;
            }
            // A thread's codes are four bytes in each of eight 16-byte pieces of its row. They
            // meet the other threads' in shared memory, a warp's eight rows to itself, and leave
            // as whole 128-byte rows: four rows to a store instead of eight quarter rows.
            const Divider divide(scale);
            divide.dispatch([&](auto quick) {
                constexpr bool QUICK = decltype(quick)::value;
                #pragma unroll
                for (int group = 0; group < GROUPS; group++) {
                    *reinterpret_cast<uint32_t *>(&codes[row][16 * group + 4 * place]) =
                        pack_int8(divide.quotients<QUICK>(both_halves(groups[group].x)),
                                  divide.quotients<QUICK>(both_halves(groups[group].y)));
                }
            });
            __syncwarp();
            #pragma unroll
            for (int half = 0; half < 2; half++) {
                const int leaving = warp * 8 + half * 4 + lane / 8;
                if (leaving < rows) {
                    uint8_t *target = p.quantized[part] + quantized_block +
                                      (static_cast<int64_t>(leaving) * p.heads + walked) * HEAD_DIM;
                    *reinterpret_cast<uint4 *>(target + 16 * (lane % 8)) =
                        *reinterpret_cast<const uint4 *>(&codes[leaving][16 * (lane % 8)]);
                }
            }
            __syncwarp();
        }
        if (staged) {
            __syncthreads();
        }
        part = next_part;
        walked += last_part ? 1 : 0;
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

template <bool NORMALIZE, bool STATS, bool QUANTIZE, int SIXTEENTHS>
int launch_as(const InputsParams &params, int blocks, size_t shared, cudaStream_t stream) {
    const auto kernel = inputs_kernel<NORMALIZE, STATS, QUANTIZE, SIXTEENTHS>;
    if (shared != 0) {
        // Up to 63 pairs: 32 KiB of cosines and sines beside the 35 KiB of static shared memory.
        static SharedMemoryOptIn shared_memory;
        const cudaError_t configured =
            shared_memory.ensure(kernel, 2 * BLOCK_ROWS * (HEAD_DIM / 2) * 4);
        if (configured != cudaSuccess) {
            return static_cast<int>(configured);
        }
    }
    const int groups = (params.heads + params.heads_per_cta - 1) / params.heads_per_cta;
    kernel<<<dim3(blocks, groups), THREADS, shared, stream>>>(params);
    return static_cast<int>(cudaGetLastError());
}

template <bool NORMALIZE, bool STATS, bool QUANTIZE>
int launch(InputsParams params, int blocks, cudaStream_t stream) {
    const bool rotate = NORMALIZE && params.angles != nullptr && params.pairs > 0;
    // With angles a CTA takes several heads so that their sincosf is paid once: as many as leave
    // the grid a few CTAs for every place on the multiprocessors.
    params.heads_per_cta = 1;
    if (rotate) {
        const int wanted = 4 * 2 * max(multiprocessor_count(), 1);
        params.heads_per_cta = HEADS_PER_CTA;
        while (params.heads_per_cta > 1 &&
               static_cast<int64_t>(blocks) *
                       ((params.heads + params.heads_per_cta - 1) / params.heads_per_cta) <
                   wanted) {
            params.heads_per_cta /= 2;
        }
    }
    if constexpr (NORMALIZE) {
        if (rotate && params.pairs % 16 == 0) {
            switch (params.pairs / 16) {
            case 1: return launch_as<NORMALIZE, STATS, QUANTIZE, 1>(params, blocks, 0, stream);
            case 2: return launch_as<NORMALIZE, STATS, QUANTIZE, 2>(params, blocks, 0, stream);
            case 3: return launch_as<NORMALIZE, STATS, QUANTIZE, 3>(params, blocks, 0, stream);
            default: return launch_as<NORMALIZE, STATS, QUANTIZE, 4>(params, blocks, 0, stream);
            }
        }
    }
    // Only pairs that are not a multiple of 16 need the table of cosines and sines.
    const size_t shared =
        rotate ? static_cast<size_t>(2) * BLOCK_ROWS * params.pairs * sizeof(float) : 0;
    return launch_as<NORMALIZE, STATS, QUANTIZE, 0>(params, blocks, shared, stream);
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
