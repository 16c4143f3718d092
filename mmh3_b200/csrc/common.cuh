// Host-side helpers shared by the launchers: error codes, the per-device status word the kernels'
// bounded waits report to, tensor-map encoding and per-device kernel attributes.
#pragma once

#include <atomic>
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/mmh3_attention.h"
#include "../../include/mmh3_int8_gemm.h"

namespace mmh3 {

// The most devices one process computes on, as in the reference
// (crates/mmh3-cuda/kernels/device.cuh:14-16).
constexpr int MAX_DEVICES = 16;

constexpr int INVALID_VALUE = static_cast<int>(cudaErrorInvalidValue);
constexpr int NOT_SUPPORTED = static_cast<int>(cudaErrorNotSupported);

enum Operand { QUERY = 0, KEY = 1, VALUE = 2, OUTPUT = 3 };

constexpr int HEAD_DIM = 128;
constexpr float LOG2_E = 1.4426950408889634f;

// Codes a kernel leaves in the status word when one of its waits runs out: the kernel in the high
// half, the wait in the low half.
constexpr unsigned int STATUS_DENSE = 0x00010000u;
constexpr unsigned int STATUS_QUANTIZED = 0x00020000u;
constexpr unsigned int STATUS_VSA = 0x00030000u;

inline cudaStream_t as_stream(mmh3_stream_t stream) {
    return reinterpret_cast<cudaStream_t>(stream);
}

// The current device, or -1.
inline int current_device() {
    int device = 0;
    return cudaGetDevice(&device) == cudaSuccess && device < MAX_DEVICES ? device : -1;
}

// Device address of the current device's status word, or null.
unsigned int *status_pointer();

// Multiprocessors of the current device, or 0.
int multiprocessor_count();

// Encodes a tiled tensor map of up to five dimensions with a swizzle (128 bytes unless told) and
// zero fill of out-of-range boxes. `strides` are in bytes for dimensions 1 and up. Returns false
// when the driver refuses, e.g. for a base or a stride that is not a multiple of 16 bytes.
bool encode_tensor_map(CUtensorMap *map, CUtensorMapDataType type, int rank, const void *base,
                       const uint64_t *dimensions, const uint64_t *strides, const uint32_t *box,
                       CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per device and kernel. A launcher keeps
// one of these per kernel as a function-local static.
struct SharedMemoryOptIn {
    std::atomic<int> configured[MAX_DEVICES];
    template <typename Kernel> cudaError_t ensure(Kernel kernel, int bytes) {
        const int device = current_device();
        if (device < 0) {
            return cudaErrorInvalidDevice;
        }
        if (const int kept = configured[device].load(std::memory_order_relaxed); kept != 0) {
            return static_cast<cudaError_t>(kept - 1);
        }
        const cudaError_t status =
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        configured[device].store(static_cast<int>(status) + 1, std::memory_order_relaxed);
        return status;
    }
};

// Whether TMA can describe an operand: a base and strides that are multiples of 16 bytes
// (strides in 16-bit elements).
bool tma_aligned(const void *base, int heads, int64_t token_stride, int64_t head_stride);

// Dense copies, in stream-ordered scratch that is given back when this goes out of scope, of the
// 16-bit operands TMA cannot describe (the reference copies such operands with cp.async inside its
// kernels, crates/mmh3-cuda/kernels/attention.cu:386-418).
struct StagedOperands {
    cudaStream_t stream;
    void *buffers[3] = {nullptr, nullptr, nullptr};
    explicit StagedOperands(cudaStream_t on) : stream(on) {}
    StagedOperands(const StagedOperands &) = delete;
    StagedOperands &operator=(const StagedOperands &) = delete;
    ~StagedOperands();
    // Replaces `base` and its strides by a dense [tokens][heads][head_dim] copy when TMA cannot
    // describe them as they are.
    cudaError_t stage(int slot, const uint16_t *&base, int tokens, int heads, int head_dim,
                      int64_t &token_stride, int64_t &head_stride);
};

// Launchers of the kernels, one per .cu file.
// dense_bf16.cu: heads of 64 or 128, BF16 or FP16 (`half`), causal or not, grouped key/value heads;
// non-null `angles` [tokens, pairs] normalize and rotate the query inside the kernel.
int launch_dense_bf16(const void *query, const void *key, const void *value, void *output,
                      int tokens, int heads, int batch, const Mmh3AttentionLayout &layout,
                      float scale, cudaStream_t stream, bool half = false, int head_dim = 128,
                      const float *angles = nullptr, int pairs = 0, float epsilon = 0.0f);


// inputs.cu
int launch_qk_norm_rope(__nv_bfloat16 *qkv, const __nv_bfloat16 *query_weight,
                        const __nv_bfloat16 *key_weight, const float *angles, int pairs,
                        int tokens, int query_heads, int key_heads, float epsilon,
                        cudaStream_t stream);
int launch_attention_inputs(__nv_bfloat16 *qkv, const __nv_bfloat16 *query_weight,
                            const __nv_bfloat16 *key_weight, const float *angles, int pairs,
                            int tokens, int heads, float epsilon,
                            const Mmh3SparseWorkspace *sparse,
                            const Mmh3QuantizedWorkspace *quantized, const int32_t *tile_starts,
                            const int32_t *tile_lengths, int tiles,
                            const float *value_head_maxima, cudaStream_t stream);
int launch_quantize(const void *query, const void *key, const void *value, int tokens, int heads,
                    const Mmh3AttentionLayout &layout, const Mmh3QuantizedWorkspace &workspace,
                    const int32_t *tile_starts, const int32_t *tile_lengths, int tiles,
                    int inputs_ready, cudaStream_t stream);
int launch_pool(const void *query, const void *key, const void *value, int heads,
                const Mmh3AttentionLayout &layout, int tiles, const Mmh3VsaWorkspace &workspace,
                cudaStream_t stream);

int launch_block_statistics(const void *query, const void *key, const void *value, int tokens,
                            int heads, const Mmh3AttentionLayout &layout,
                            const Mmh3SparseWorkspace &workspace, cudaStream_t stream);

// sol_attention.cu: Sol-Attn over BF16 q, k, v (block statistics unless inputs_ready, centring,
// routing, row offsets, token attention merged with the pooled tails). With `quantized`, the token
// attention runs in INT8/FP8 over that workspace, which inputs_ready = 0 fills, 1 completes with
// the FP8 V, and 2 finds complete.
int launch_sparse_attention(const void *query, const void *key, const void *value, void *output,
                            int tokens, int heads, const Mmh3AttentionLayout &layout, float scale,
                            float tau, int sink_key_start, int sink_key_end, int sink_query_start,
                            int sink_query_end, const Mmh3SparseWorkspace &workspace,
                            const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                            cudaStream_t stream);

// vsa_select.cu
int launch_select(const Mmh3VsaWorkspace &workspace, int tiles, int heads, int prefix_tiles,
                  int kept, float scale, int coarse, cudaStream_t stream);

// quantized_attention.cu: dense when `vsa` is null, else over the routes of `vsa`.
int launch_quantized_attention(const Mmh3QuantizedWorkspace &workspace, void *output, int tokens,
                               int heads, const Mmh3AttentionLayout &layout, float scale,
                               const Mmh3VsaWorkspace *vsa, int tiles, const void *gate,
                               int64_t gate_stride, cudaStream_t stream);

// vsa_attention.cu
int launch_vsa_attention(const void *query, const void *key, const void *value, const void *gate,
                         int64_t gate_stride, void *output, int tokens, int heads,
                         const Mmh3AttentionLayout &layout, float scale, int tiles,
                         const Mmh3VsaWorkspace &workspace, cudaStream_t stream);

// Sol-Attn's token attention over the routes in `sparse`, merged with its pooled tails.
int launch_sol_token_attention(const void *query, const void *key, const void *value, void *output,
                               int tokens, int heads, const Mmh3AttentionLayout &layout,
                               float scale, const Mmh3SparseWorkspace &sparse,
                               cudaStream_t stream);

// The INT8/FP8 token attention over the routes of `vsa`.
int launch_vsa_attention_quantized(const Mmh3QuantizedWorkspace &workspace, void *output,
                                   int tokens, int heads, const Mmh3AttentionLayout &layout,
                                   float scale, const Mmh3VsaWorkspace &vsa, int tiles,
                                   const void *gate, int64_t gate_stride, cudaStream_t stream,
                                   const Mmh3SparseWorkspace *tails = nullptr);

// The INT8/FP8 token attention over Sol-Attn's routes, merged with its pooled tails.
int launch_sol_token_attention_quantized(const Mmh3QuantizedWorkspace &workspace, void *output,
                                         int tokens, int heads, const Mmh3AttentionLayout &layout,
                                         float scale, const Mmh3SparseWorkspace &sparse,
                                         cudaStream_t stream);

// int8_gemm.cu: the scaled INT8 product with its optional bias, low-rank adapter, SwiGLU and
// column maxima.
int launch_int8_gemm(int config, int group_m, const int8_t *activations, const int8_t *weights,
                     const float *activation_scales, const float *weight_scales, const float *bias,
                     void *output, bool output_is_f16, bool swiglu, int m, int n, int k,
                     int output_stride, const void *adapter_down, const void *adapter_up, int rank,
                     int adapter_down_stride, float adapter_scale, unsigned *column_maxima,
                     int maxima_first_column, cudaStream_t stream);
int launch_interleave_swiglu_rows(const void *source, void *destination, int rows, int row_bytes,
                                  cudaStream_t stream);

// shard.cu
int launch_shard_pack(const void *source, void *packed, int tokens, int tensors, int heads, int dim,
                      int first_head, int span, cudaStream_t stream);
int launch_shard_unpack(const void *part, void *output, int tokens, int heads, int dim,
                        int first_head, int span, cudaStream_t stream);

} // namespace mmh3
