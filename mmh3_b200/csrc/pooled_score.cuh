// The pooled score of one block mean against another in the FP32 evaluation order both of the
// reference's routing kernels use (crates/mmh3-cuda/kernels/vsa_attention.cu:96-273,
// kernels/sparse_attention.cu:162-206): a warp holds the 128 products lane-strided, every lane
// chains four fused multiply-adds over dimensions l, l + 32, l + 64, l + 96, and the 32 chains are
// summed over a xor butterfly that pairs lanes by bit 4 first and bit 0 last. Here one thread
// evaluates that whole tree, which keeps scores, and therefore routes, bit-identical.
#pragma once

#include "common.cuh"

namespace mmh3 {

// The sum over the chains l = BASE, BASE + STRIDE, ... of the products of one query with one key,
// in the tree order described at the top. `key` is the key's 128 values in registers; `query` holds
// the query regrouped by chain: query[l] = (q[l], q[l + 32], q[l + 64], q[l + 96]).
template <int STRIDE, int BASE>
__device__ __forceinline__ float score_tree(const float4 *__restrict__ query,
                                            const float (&key)[HEAD_DIM]) {
    if constexpr (STRIDE == 32) {
        const float4 q = query[BASE];
        float sum = __fmaf_rn(q.x, key[BASE], 0.0f);
        sum = __fmaf_rn(q.y, key[BASE + 32], sum);
        sum = __fmaf_rn(q.z, key[BASE + 64], sum);
        return __fmaf_rn(q.w, key[BASE + 96], sum);
    } else {
        return __fadd_rn(score_tree<STRIDE * 2, BASE>(query, key),
                         score_tree<STRIDE * 2, BASE + STRIDE>(query, key));
    }
}

} // namespace mmh3
