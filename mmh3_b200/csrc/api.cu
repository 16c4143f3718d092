// The extern "C" entry points of libmmh3_attn_b200.so: argument checks in the reference's terms,
// then the launchers. Declarations and the reference function each one replaces are in
// include/mmh3_attention.h.
#include <cstdio>

#include "common.cuh"

using namespace mmh3;

extern "C" int mmh3_attention_roped(int element_type, int head_dim, const void *query,
                                    const void *key, const void *value, void *output, int tokens,
                                    int heads, int batch, const Mmh3AttentionLayout *layout,
                                    float scale, const float *angles, int pairs, float epsilon,
                                    mmh3_stream_t stream) {
    // crates/mmh3-cuda/kernels/attention.cu:507-510
    if (layout == nullptr || tokens <= 0 || heads <= 0 || batch <= 0 ||
        (layout->heads_per_key_value > 0 && heads % layout->heads_per_key_value != 0)) {
        return INVALID_VALUE;
    }
    if ((element_type != 0 && element_type != 1) || (head_dim != 64 && head_dim != 128)) {
        return INVALID_VALUE;
    }
    return launch_dense_bf16(query, key, value, output, tokens, heads, batch, *layout, scale,
                             as_stream(stream), element_type == 1, head_dim, angles, pairs,
                             epsilon);
}

extern "C" int mmh3_attention(int element_type, int head_dim, const void *query, const void *key,
                              const void *value, void *output, int tokens, int heads, int batch,
                              const Mmh3AttentionLayout *layout, float scale,
                              mmh3_stream_t stream) {
    return mmh3_attention_roped(element_type, head_dim, query, key, value, output, tokens, heads,
                                batch, layout, scale, nullptr, 0, 0.0f, stream);
}

extern "C" int mmh3_attention_bf16(const void *query, const void *key, const void *value,
                                   void *output, int tokens, int heads, int64_t query_stride,
                                   int64_t key_stride, int64_t value_stride, int64_t output_stride,
                                   float scale, mmh3_stream_t stream) {
    const Mmh3AttentionLayout layout = {{query_stride, key_stride, value_stride, output_stride},
                                        {128, 128, 128, 128},
                                        {0, 0, 0, 0},
                                        1,
                                        0};
    return mmh3_attention(0, 128, query, key, value, output, tokens, heads, 1, &layout, scale,
                          stream);
}

extern "C" int mmh3_qk_norm_rope(void *qkv, const void *query_weight, const void *key_weight,
                                 const float *angles, int pairs, int tokens, int query_heads,
                                 int key_heads, float epsilon, mmh3_stream_t stream) {
    if (tokens <= 0 || query_heads < 0 || key_heads < 0 || pairs < 0 || 2 * pairs > HEAD_DIM) {
        return INVALID_VALUE;
    }
    return launch_qk_norm_rope(static_cast<__nv_bfloat16 *>(qkv),
                               static_cast<const __nv_bfloat16 *>(query_weight),
                               static_cast<const __nv_bfloat16 *>(key_weight), angles, pairs,
                               tokens, query_heads, key_heads, epsilon, as_stream(stream));
}

extern "C" int mmh3_attention_inputs(void *qkv, const void *query_weight, const void *key_weight,
                                     const float *angles, int pairs, int tokens, int heads,
                                     float epsilon, const Mmh3SparseWorkspace *sparse,
                                     const Mmh3QuantizedWorkspace *quantized,
                                     const int32_t *tile_starts, const int32_t *tile_lengths,
                                     int tiles, const float *value_head_maxima,
                                     mmh3_stream_t stream) {
    // crates/mmh3-cuda/kernels/dit.cu:786-790
    if (tokens <= 0 || heads <= 0 || (sparse == nullptr && quantized == nullptr) ||
        (tile_starts != nullptr && (tile_lengths == nullptr || tiles <= 0)) ||
        (value_head_maxima != nullptr && quantized == nullptr) || pairs < 0 ||
        2 * pairs > HEAD_DIM) {
        return INVALID_VALUE;
    }
    return launch_attention_inputs(static_cast<__nv_bfloat16 *>(qkv),
                                   static_cast<const __nv_bfloat16 *>(query_weight),
                                   static_cast<const __nv_bfloat16 *>(key_weight), angles, pairs,
                                   tokens, heads, epsilon, sparse, quantized, tile_starts,
                                   tile_lengths, tiles, value_head_maxima, as_stream(stream));
}

extern "C" int mmh3_attention_quantized(const void *query, const void *key, const void *value,
                                        void *output, int tokens, int heads,
                                        const Mmh3AttentionLayout *layout, float scale,
                                        const Mmh3SparseWorkspace *sparse,
                                        const Mmh3QuantizedWorkspace *workspace, int inputs_ready,
                                        mmh3_stream_t stream) {
    // crates/mmh3-cuda/kernels/quantized_attention.cu:581-583
    if (layout == nullptr || workspace == nullptr || tokens <= 0 || heads <= 0 ||
        layout->causal != 0 || layout->heads_per_key_value > 1 || inputs_ready < 0 ||
        inputs_ready > 2) {
        return INVALID_VALUE;
    }
    const int prepared = launch_quantize(query, key, value, tokens, heads, *layout, *workspace,
                                         nullptr, nullptr, 0, inputs_ready, as_stream(stream));
    if (prepared != 0) {
        return prepared;
    }
    if (sparse != nullptr) {
        // Sol-Attn: over the routes and tails a call of mmh3_sparse_attention left in `sparse`.
        return launch_sol_token_attention_quantized(*workspace, output, tokens, heads, *layout,
                                                    scale, *sparse, as_stream(stream));
    }
    return launch_quantized_attention(*workspace, output, tokens, heads, *layout, scale, nullptr,
                                      0, nullptr, 0, as_stream(stream));
}

extern "C" int mmh3_vsa_attention_quantized(const void *value, const void *gate,
                                            int64_t gate_stride, void *output, int tokens,
                                            int heads, const Mmh3AttentionLayout *layout,
                                            float scale, int tiles, const Mmh3VsaWorkspace *vsa,
                                            const Mmh3QuantizedWorkspace *workspace,
                                            int inputs_ready, mmh3_stream_t stream) {
    // crates/mmh3-cuda/kernels/quantized_attention.cu:619-622
    if (layout == nullptr || vsa == nullptr || workspace == nullptr || tokens <= 0 || heads <= 0 ||
        tiles <= 0 || layout->causal != 0 || layout->heads_per_key_value > 1) {
        return INVALID_VALUE;
    }
    if (inputs_ready != 2) {
        // INT8 q and k and the |v| maxima are there; FP8 V is still to be made.
        const int prepared =
            launch_quantize(nullptr, nullptr, value, tokens, heads, *layout, *workspace,
                            vsa->tile_starts, vsa->tile_lengths, tiles, 1, as_stream(stream));
        if (prepared != 0) {
            return prepared;
        }
    }
    return launch_quantized_attention(*workspace, output, tokens, heads, *layout, scale, vsa,
                                      tiles, gate, gate_stride, as_stream(stream));
}

extern "C" int mmh3_vsa_attention(const void *query, const void *key, const void *value,
                                  const void *gate, int64_t gate_stride, void *output, int tokens,
                                  int heads, const Mmh3AttentionLayout *layout, float scale,
                                  int tiles, int prefix_tiles, int kept,
                                  const Mmh3VsaWorkspace *workspace,
                                  const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                                  mmh3_stream_t stream) {
    // crates/mmh3-cuda/kernels/vsa_attention.cu:510-513
    if (layout == nullptr || workspace == nullptr || tokens <= 0 || heads <= 0 || tiles <= 0 ||
        tiles > 65536 || prefix_tiles < 0 || prefix_tiles > tiles || kept < 1 ||
        (quantized != nullptr && !inputs_ready)) {
        return INVALID_VALUE;
    }
    if (!inputs_ready) {
        const int pooled =
            launch_pool(query, key, value, heads, *layout, tiles, *workspace, as_stream(stream));
        if (pooled != 0) {
            return pooled;
        }
    }
    const int selected = launch_select(*workspace, tiles, heads, prefix_tiles, kept, scale,
                                       gate != nullptr, as_stream(stream));
    if (selected != 0) {
        return selected;
    }
    if (quantized != nullptr) {
        return mmh3_vsa_attention_quantized(value, gate, gate_stride, output, tokens, heads, layout,
                                            scale, tiles, workspace, quantized, inputs_ready,
                                            stream);
    }
    return launch_vsa_attention(query, key, value, gate, gate_stride, output, tokens, heads,
                                *layout, scale, tiles, *workspace, as_stream(stream));
}

extern "C" int mmh3_sparse_attention(const void *query, const void *key, const void *value,
                                     void *output, int tokens, int heads,
                                     const Mmh3AttentionLayout *layout, float scale, float tau,
                                     int sink_key_start, int sink_key_end, int sink_query_start,
                                     int sink_query_end, const Mmh3SparseWorkspace *workspace,
                                     const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                                     mmh3_stream_t stream) {
    if (tokens <= 0 || heads <= 0) {
        return INVALID_VALUE;
    }
    if (layout == nullptr || workspace == nullptr || query == nullptr || key == nullptr ||
        value == nullptr || output == nullptr) {
        return INVALID_VALUE;
    }
    if (quantized != nullptr && (layout->causal != 0 || layout->heads_per_key_value > 1 ||
                                 inputs_ready < 0 || inputs_ready > 2)) {
        return INVALID_VALUE;
    }
    return launch_sparse_attention(query, key, value, output, tokens, heads, *layout, scale, tau,
                                   sink_key_start, sink_key_end, sink_query_start, sink_query_end,
                                   *workspace, quantized, inputs_ready, as_stream(stream));
}

extern "C" int mmh3_dit_shard_pack(const void *source, void *packed, int tokens, int tensors,
                                   int heads, int dim, int first_head, int span,
                                   mmh3_stream_t stream) {
    return launch_shard_pack(source, packed, tokens, tensors, heads, dim, first_head, span,
                             as_stream(stream));
}

extern "C" int mmh3_dit_shard_unpack(const void *part, void *output, int tokens, int heads,
                                     int dim, int first_head, int span, mmh3_stream_t stream) {
    return launch_shard_unpack(part, output, tokens, heads, dim, first_head, span,
                               as_stream(stream));
}

// The band heights a caller may name, as crates/mmh3-cuda/kernels/int8_gemm.cu:735.
static constexpr int GROUP_HEIGHTS[] = {4, 8, 16};

extern "C" int mmh3_int8_gemm_config_count(void) { return 2; }

extern "C" int mmh3_int8_gemm_group_heights(int *heights, int capacity) {
    constexpr int COUNT = sizeof(GROUP_HEIGHTS) / sizeof(GROUP_HEIGHTS[0]);
    for (int index = 0; index < COUNT && index < capacity; index++) {
        heights[index] = GROUP_HEIGHTS[index];
    }
    return COUNT;
}

extern "C" int mmh3_int8_gemm(int config, int group_m, const int8_t *activations,
                              const int8_t *weights, const float *activation_scales,
                              const float *weight_scales, const float *bias, void *output,
                              int output_is_f16, int swiglu, int m, int n, int k,
                              int output_stride, const void *adapter_down, const void *adapter_up,
                              int rank, int adapter_down_stride, float adapter_scale,
                              unsigned *column_maxima, int maxima_first_column,
                              mmh3_stream_t stream) {
    if (activations == nullptr || weights == nullptr || activation_scales == nullptr ||
        weight_scales == nullptr || output == nullptr) {
        return INVALID_VALUE;
    }
    return launch_int8_gemm(config, group_m, activations, weights, activation_scales,
                            weight_scales, bias, output, output_is_f16 != 0, swiglu != 0, m, n, k,
                            output_stride, adapter_down, adapter_up, rank, adapter_down_stride,
                            adapter_scale, column_maxima, maxima_first_column, as_stream(stream));
}

extern "C" int mmh3_int8_gemm_bf16(int config, int group_m, const int8_t *activations,
                                   const int8_t *weights, const float *activation_scales,
                                   const float *weight_scales, void *output, int m, int n, int k,
                                   mmh3_stream_t stream) {
    return mmh3_int8_gemm(config, group_m, activations, weights, activation_scales, weight_scales,
                          nullptr, output, 0, 0, m, n, k, n, nullptr, nullptr, 0, 0, 0.0f, nullptr,
                          0, stream);
}

extern "C" int mmh3_int8_gemm_tilings(Mmh3Int8Tiling *chosen, int capacity) {
    (void)chosen;
    (void)capacity;
    return 0;
}

extern "C" void mmh3_int8_gemm_adopt(const Mmh3Int8Tiling *chosen, int count) {
    (void)chosen;
    (void)count;
}

extern "C" int mmh3_int8_gemm_tiling_key(char *key, int capacity) {
    int device = 0;
    cudaDeviceProp properties;
    cudaError_t status = cudaGetDevice(&device);
    if (status == cudaSuccess) {
        status = cudaGetDeviceProperties(&properties, device);
    }
    if (status != cudaSuccess) {
        return static_cast<int>(status);
    }
    if (key == nullptr || capacity <= 0) {
        return INVALID_VALUE;
    }
    const int written =
        std::snprintf(key, static_cast<size_t>(capacity), "%s, sm_%d%d, one tcgen05 tiling",
                      properties.name, properties.major, properties.minor);
    return written < 0 || written >= capacity ? INVALID_VALUE : 0;
}

extern "C" int mmh3_interleave_swiglu_rows(const void *source, void *destination, int rows,
                                           int row_bytes, mmh3_stream_t stream) {
    return launch_interleave_swiglu_rows(source, destination, rows, row_bytes, as_stream(stream));
}
