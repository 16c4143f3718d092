// The pooled score of one block mean against another in the FP32 evaluation order both of the
// reference's routing kernels use (crates/mmh3-cuda/kernels/vsa_attention.cu:96-273,
// kernels/sparse_attention.cu:162-206): a warp holds the 128 products lane-strided, every lane
// chains four fused multiply-adds over dimensions l, l + 32, l + 64, l + 96, and the 32 chains are
// summed over a xor butterfly that pairs lanes by bit 4 first and bit 0 last. Evaluated in that
// order, whoever evaluates it, the scores, and therefore the routes, are bit-identical. Here four
// threads share the tree, two chains at a time in the halves of packed FP32 operations
// (fma.rn.f32x2, add.rn.f32x2: two independent IEEE operations each).
#pragma once

#include "common.cuh"

namespace mmh3 {

// The pooled scores of two key means against one query mean by four threads, in the order
// described at the top. Thread c of the four holds the chains
// l = 4 a + c, a = 0 .. 7, that is dimensions 4 m + c with m = a + 8 k for step k: of a key as the
// pairs key[i] = (m = 2 i, m = 2 i + 1), of the query as 16-byte words of four consecutive m.
// Chains a and a + 1 are the halves of packed operations; bits 4, 3, 2 of l are bits 2, 1, 0 of a
// (two packed additions and the sum of the halves), bits 1 and 0 are c: two exchanges among the
// four threads, after which each holds both scores.
__device__ __forceinline__ void score_two_keys(const float4 *__restrict__ query,
                                               const float2 (&keys)[2][HEAD_DIM / 8],
                                               float (&scores)[2]) {
    float2 sums[2][4];
    #pragma unroll
    for (int key = 0; key < 2; key++) {
        #pragma unroll
        for (int pair = 0; pair < 4; pair++) {
            sums[key][pair] = make_float2(0.0f, 0.0f);
        }
    }
    #pragma unroll
    for (int step = 0; step < 4; step++) {
        #pragma unroll
        for (int half = 0; half < 2; half++) {
            const float4 four = query[step * 2 + half];
            #pragma unroll
            for (int key = 0; key < 2; key++) {
                sums[key][half * 2] = __ffma2_rn(make_float2(four.x, four.y),
                                                 keys[key][half * 2 + step * 4],
                                                 sums[key][half * 2]);
                sums[key][half * 2 + 1] = __ffma2_rn(make_float2(four.z, four.w),
                                                     keys[key][half * 2 + 1 + step * 4],
                                                     sums[key][half * 2 + 1]);
            }
        }
    }
    #pragma unroll
    for (int key = 0; key < 2; key++) {
        const float2 folded = __fadd2_rn(__fadd2_rn(sums[key][0], sums[key][2]),
                                         __fadd2_rn(sums[key][1], sums[key][3]));
        float sum = __fadd_rn(folded.x, folded.y);
        sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 2));
        scores[key] = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 1));
    }
}

// The xor butterfly from bit 4 down to bit 0 over eight values a lane at once, narrowing as it
// goes: at bit 4 a lane keeps four of the eight sums and hands its partner the other four, at bit
// 3 two, at bit 2 one, so that each sum is the one the full butterfly leaves in that lane (an
// addition commutes) at 9 exchanges instead of 40. Lane l ends with sum (l / 4) % 8 of the eight.
__device__ __forceinline__ float narrowed_sum(const float (&eight)[8], int lane) {
    const bool upper_four = lane & 16, upper_two = lane & 8, upper_one = lane & 4;
    float four[4], two[2];
    #pragma unroll
    for (int index = 0; index < 4; index++) {
        const float kept = upper_four ? eight[4 + index] : eight[index];
        const float handed = upper_four ? eight[index] : eight[4 + index];
        four[index] = __fadd_rn(kept, __shfl_xor_sync(0xffffffffu, handed, 16));
    }
    #pragma unroll
    for (int index = 0; index < 2; index++) {
        const float kept = upper_two ? four[2 + index] : four[index];
        const float handed = upper_two ? four[index] : four[2 + index];
        two[index] = __fadd_rn(kept, __shfl_xor_sync(0xffffffffu, handed, 8));
    }
    float sum = __fadd_rn(upper_one ? two[1] : two[0],
                          __shfl_xor_sync(0xffffffffu, upper_one ? two[0] : two[1], 4));
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 2));
    return __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 1));
}

} // namespace mmh3
