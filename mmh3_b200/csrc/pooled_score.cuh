// The pooled score of one block mean against another in the FP32 evaluation order both of the
// reference's routing kernels use (crates/mmh3-cuda/kernels/vsa_attention.cu:96-273,
// kernels/sparse_attention.cu:162-206): a warp holds the 128 products lane-strided, every lane
// chains four fused multiply-adds over dimensions l, l + 32, l + 64, l + 96, and the 32 chains are
// summed over a xor butterfly that pairs lanes by bit 4 first and bit 0 last. Here one thread
// evaluates that whole tree, which keeps scores, and therefore routes, bit-identical. It does so
// two chains at a time: chains 2b and 2b + 1 are the two halves of packed FP32 operations
// (fma.rn.f32x2, add.rn.f32x2: two independent IEEE operations each), over the dimension pairs
// (2b + 32k, 2b + 1 + 32k) that sit next to each other in the key's registers and in the query's
// row; the butterfly's last step, bit 0, adds the two halves.
#pragma once

#include "common.cuh"

namespace mmh3 {

// For chains l = BASE, BASE + STRIDE, ... (the even ones in .x, the odd ones after them in .y):
// the sums of the products of one query with one key in the tree order described at the top.
// `key` is the key's 128 values in registers, as pairs; `query` the query's 128 values in order.
template <int STRIDE, int PAIR>
__device__ __forceinline__ float2 score_pairs(const float4 *__restrict__ query,
                                              const float2 (&key)[HEAD_DIM / 2]) {
    if constexpr (STRIDE == 32) {
        // Chains 2 * PAIR and 2 * PAIR + 1 over their four dimensions each.
        float2 sums = make_float2(0.0f, 0.0f);
        #pragma unroll
        for (int step = 0; step < 4; step++) {
            const float4 four = query[(2 * PAIR + 32 * step) / 4];
            const float2 two = PAIR % 2 == 0 ? make_float2(four.x, four.y)
                                             : make_float2(four.z, four.w);
            sums = __ffma2_rn(two, key[PAIR + 16 * step], sums);
        }
        return sums;
    } else {
        return __fadd2_rn(score_pairs<STRIDE * 2, PAIR>(query, key),
                          score_pairs<STRIDE * 2, PAIR + STRIDE / 2>(query, key));
    }
}

// The whole tree: the butterfly down to pairs of chains, then its last step.
__device__ __forceinline__ float score_tree(const float4 *__restrict__ query,
                                            const float2 (&key)[HEAD_DIM / 2]) {
    const float2 halves = score_pairs<2, 0>(query, key);
    return __fadd_rn(halves.x, halves.y);
}

// A row of 128 FP32 values from global memory into registers, as pairs.
__device__ __forceinline__ void load_row(const float *__restrict__ row,
                                         float2 (&values)[HEAD_DIM / 2]) {
    const float4 *source = reinterpret_cast<const float4 *>(row);
    #pragma unroll
    for (int chunk = 0; chunk < HEAD_DIM / 4; chunk++) {
        const float4 loaded = __ldg(source + chunk);
        values[chunk * 2] = make_float2(loaded.x, loaded.y);
        values[chunk * 2 + 1] = make_float2(loaded.z, loaded.w);
    }
}

} // namespace mmh3
