/* C ABI of the B200 (sm_100a) attention library, libmmh3_attn_b200.so.
 *
 * Every entry point keeps the name, the argument list and the return convention of the function
 * of niw/mmh3's CUDA crate it replaces, so that mmh3's Rust wrappers
 * (crates/mmh3-cuda/src/attention.rs:158-288, crates/mmh3-cuda/src/dit.rs) bind it unchanged.
 *
 * Conventions, as in the reference:
 * - the return value is a cudaError_t as an int, 0 for success; bad arguments give
 *   cudaErrorInvalidValue (1), combinations this library does not implement give
 *   cudaErrorNotSupported (801);
 * - every pointer is caller-owned device memory and the library never synchronizes; the kernels
 *   of one call are ordered on `stream` (NULL is the legacy default stream) and the call returns
 *   once they are enqueued. It allocates nothing, with one exception: BF16 or FP16 operands of the
 *   dense, VSA and Sol-Attn calls whose base or strides are not multiples of 16 bytes, which TMA
 *   cannot describe, are first gathered into dense arrays in stream-ordered scratch
 *   (cudaMallocAsync on `stream`, given back with cudaFreeAsync behind the kernels; the reference
 *   copies such operands with cp.async inside its kernels). The results are the same bits;
 * - strides are in elements; structs are read during the call only;
 * - any host thread may call, for whatever device is current on it.
 */
#ifndef MMH3_ATTENTION_H
#define MMH3_ATTENTION_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *mmh3_stream_t; /* cudaStream_t */

/* Element (batch, token, head, dimension) of the query, key, value and output tensors, in that
 * order, lives at base + batch * batch_stride + token * token_stride + head * head_stride +
 * dimension. Replaces crates/mmh3-cuda/kernels/tensor_core.cuh:15-23. */
typedef struct Mmh3AttentionLayout {
    int64_t token_stride[4];
    int64_t head_stride[4];
    int64_t batch_stride[4];
    int32_t heads_per_key_value; /* query heads per key/value head, 0 means 1 */
    int32_t causal;              /* nonzero masks the keys after each query's own position */
} Mmh3AttentionLayout;

/* Sol-Attn scratch. Only centroids, block_keys and value_sums are used here: the fused input pass
 * delivers VSA's pooled tiles through them. Replaces
 * crates/mmh3-cuda/kernels/attention_workspace.cuh:8-22. */
typedef struct Mmh3SparseWorkspace {
    float *centroids;   /* [heads, blocks, 128] mean query */
    float *block_keys;  /* [heads, blocks, 128] mean key */
    float *value_sums;  /* [heads, blocks, 128] summed value */
    float *key_mean;
    float *key_variance;
    float *row_offsets;
    uint16_t *routes;
    int32_t *route_counts;
    float *tail_max;
    float *tail_sum;
    float *tail_values;
} Mmh3SparseWorkspace;

/* INT8 Q/K, FP8 V and their scales for one sequence. `blocks` below is ceil(tokens / 64) for dense
 * attention and the number of tiles for VSA. Replaces attention_workspace.cuh:24-32. */
typedef struct Mmh3QuantizedWorkspace {
    uint8_t *query;      /* [tokens, heads, 128] INT8 */
    uint8_t *key;        /* [tokens, heads, 128] INT8 */
    uint8_t *value;      /* [heads, 128, blocks * 64] FP8 E4M3, zero past a block's rows */
    float *query_scales; /* [heads, blocks] */
    float *key_scales;   /* [heads, blocks] */
    float *value_scales; /* [heads] */
    float *value_maxima; /* [heads, blocks] max |v| */
} Mmh3QuantizedWorkspace;

/* Tiles of a VSA plan and the scratch of one call. Replaces attention_workspace.cuh:35-44. */
typedef struct Mmh3VsaWorkspace {
    const int32_t *tile_starts;  /* [tiles] */
    const int32_t *tile_lengths; /* [tiles], each at most 64 */
    float *pooled_query;         /* [heads, tiles, 128] mean */
    float *pooled_key;           /* [heads, tiles, 128] mean */
    float *pooled_value;         /* [heads, tiles, 128] sum */
    uint16_t *routes;            /* [heads, tiles, tiles], route_counts entries used per row */
    int32_t *route_counts;       /* [heads, tiles] */
    float *coarse;               /* [heads, tiles, 128] */
} Mmh3VsaWorkspace;

/* Dense softmax(Q K^T * scale) V. element_type 0 is BF16 and 1 is FP16; head_dim 64 or 128.
 * Causal or not, with grouped key/value heads and batches: the DiT's, the text encoder's and the
 * VAE decoder's uses. `scale` must be positive. Operands TMA cannot describe (bases or strides that
 * are not multiples of 16 bytes) are first gathered into dense arrays in stream-ordered scratch
 * (cudaMallocAsync on `stream`, given back with cudaFreeAsync behind the kernel); the result is
 * the same bits.
 * Replaces crates/mmh3-cuda/kernels/attention.cu:531-536. */
int mmh3_attention(int element_type, int head_dim, const void *query, const void *key,
                   const void *value, void *output, int tokens, int heads, int batch,
                   const Mmh3AttentionLayout *layout, float scale, mmh3_stream_t stream);

/* mmh3_attention with a query RMSNorm + RoPE fused in (the video VAE's decoder): `angles` is FP32
 * [tokens, pairs], dimension p of a query row pairs with p + pairs, 2 * pairs <= head_dim. Null
 * `angles` is mmh3_attention.
 * Replaces crates/mmh3-cuda/kernels/attention.cu:502-529. */
int mmh3_attention_roped(int element_type, int head_dim, const void *query, const void *key,
                         const void *value, void *output, int tokens, int heads, int batch,
                         const Mmh3AttentionLayout *layout, float scale, const float *angles,
                         int pairs, float epsilon, mmh3_stream_t stream);

/* The DiT's layout: q, k and v BF16 with their own token strides and heads of 128 packed
 * contiguously. Replaces crates/mmh3-cuda/kernels/attention.cu:539-551. */
int mmh3_attention_bf16(const void *query, const void *key, const void *value, void *output,
                        int tokens, int heads, int64_t query_stride, int64_t key_stride,
                        int64_t value_stride, int64_t output_stride, float scale,
                        mmh3_stream_t stream);

/* Per-head RMSNorm of q and k in rows of [q | k | v] and the split-half rotary embedding of the
 * first 2 * pairs dimensions, in place. Replaces crates/mmh3-cuda/kernels/dit.cu:760-770. */
int mmh3_qk_norm_rope(void *qkv, const void *query_weight, const void *key_weight,
                      const float *angles, int pairs, int tokens, int query_heads, int key_heads,
                      float epsilon, mmh3_stream_t stream);

/* mmh3_qk_norm_rope fused with the attention's per-block work: INT8 q and k with their block
 * scales and the block maxima of |v| (or, with `value_head_maxima`, FP8 V and its scales) when
 * `quantized` is given; the mean query, mean key and summed value per block when `sparse` is.
 * Tile tables replace the 64-token blocks, for VSA.
 * Replaces crates/mmh3-cuda/kernels/dit.cu:778-810. */
int mmh3_attention_inputs(void *qkv, const void *query_weight, const void *key_weight,
                          const float *angles, int pairs, int tokens, int heads, float epsilon,
                          const Mmh3SparseWorkspace *sparse,
                          const Mmh3QuantizedWorkspace *quantized, const int32_t *tile_starts,
                          const int32_t *tile_lengths, int tiles, const float *value_head_maxima,
                          mmh3_stream_t stream);

/* INT8 QK^T and FP8 PV attention with FP32 softmax and BF16 output. inputs_ready: 0 computes the
 * workspace from BF16 q, k, v; 1 finds INT8 q, k, their scales and the |v| block maxima there;
 * 2 also the FP8 V and its scales. With a non-null `sparse` the attention runs over the routes and
 * pooled tails a call of mmh3_sparse_attention left there (Sol-Attn).
 * Replaces crates/mmh3-cuda/kernels/quantized_attention.cu:575-611. */
int mmh3_attention_quantized(const void *query, const void *key, const void *value, void *output,
                             int tokens, int heads, const Mmh3AttentionLayout *layout, float scale,
                             const Mmh3SparseWorkspace *sparse,
                             const Mmh3QuantizedWorkspace *workspace, int inputs_ready,
                             mmh3_stream_t stream);

/* Video sparse attention over a sequence in tile order: pool (unless inputs_ready), select `kept`
 * video tiles per video query tile, token attention over the selected tiles, plus gate * coarse
 * when `gate` (BF16 rows of heads * 128, gate_stride apart) is not null. A non-null `quantized`
 * runs the token attention in INT8/FP8 and needs inputs_ready >= 1.
 * Replaces crates/mmh3-cuda/kernels/vsa_attention.cu:503-536. */
int mmh3_vsa_attention(const void *query, const void *key, const void *value, const void *gate,
                       int64_t gate_stride, void *output, int tokens, int heads,
                       const Mmh3AttentionLayout *layout, float scale, int tiles,
                       int prefix_tiles, int kept, const Mmh3VsaWorkspace *workspace,
                       const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                       mmh3_stream_t stream);

/* The INT8/FP8 token attention of VSA over routes already selected.
 * Replaces crates/mmh3-cuda/kernels/quantized_attention.cu:613-634. */
int mmh3_vsa_attention_quantized(const void *value, const void *gate, int64_t gate_stride,
                                 void *output, int tokens, int heads,
                                 const Mmh3AttentionLayout *layout, float scale, int tiles,
                                 const Mmh3VsaWorkspace *vsa,
                                 const Mmh3QuantizedWorkspace *workspace, int inputs_ready,
                                 mmh3_stream_t stream);

/* Sol-Attn over one sequence of BF16 heads of 128: blocks of 64 tokens; a query block attends the
 * key blocks it routes (pooled score above tau standard deviations, its neighbours, the key sinks
 * [sink_key_start, sink_key_end), every block for the query sinks) token by token and the rest
 * through one pooled term each. inputs_ready != 0: the workspace already holds the block statistics
 * (mmh3_attention_inputs). The routes are bit-identical to the reference's. A non-null `quantized`
 * runs the token attention over the routes in INT8/FP8, with inputs_ready as for
 * mmh3_attention_quantized.
 * Replaces crates/mmh3-cuda/kernels/sparse_attention.cu:546-586. */
int mmh3_sparse_attention(const void *query, const void *key, const void *value, void *output,
                          int tokens, int heads, const Mmh3AttentionLayout *layout, float scale,
                          float tau, int sink_key_start, int sink_key_end, int sink_query_start,
                          int sink_query_end, const Mmh3SparseWorkspace *workspace,
                          const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                          mmh3_stream_t stream);

/* Ulysses layout changes: gather heads [first_head, first_head + span) of
 * [tokens][tensors][heads][dim] into [tokens][tensors][span][dim], and scatter
 * [tokens][span][dim] back into [tokens][heads][dim]. Elements are 16 bits; dim is a multiple of 8.
 * Both buffers are moved in 16-byte groups: a pointer off a 16-byte boundary returns
 * cudaErrorInvalidValue (the reference would fault on the device).
 * Replace crates/mmh3-cuda/kernels/dit.cu:998-1023. */
int mmh3_dit_shard_pack(const void *source, void *packed, int tokens, int tensors, int heads,
                        int dim, int first_head, int span, mmh3_stream_t stream);
int mmh3_dit_shard_unpack(const void *part, void *output, int tokens, int heads, int dim,
                          int first_head, int span, mmh3_stream_t stream);

/* No counterpart in the reference. mmh3_attention_quantized with inputs_ready = 0, for callers that
 * cannot allocate its workspace: a host that accounts for the whole device itself and has given
 * what is left to something else (mmh3 sizes its weight streaming that way), or a loop that cannot
 * take the device-wide stall of a cudaMalloc. The INT8 q and k, the FP8 V and their scales live in a
 * fixed array inside the library's device image (about 12 MiB on every GPU that loads the library,
 * until the process exits), and this call allocates and frees nothing.
 *
 * Limits: heads <= 64 and (tokens rounded up to a multiple of 64) * heads <= 32,768, e.g. 4,096
 * tokens of 8 heads. Anything larger returns cudaErrorInvalidValue and names the limit on stderr.
 * The layout must not be causal nor share key/value heads, as for mmh3_attention_quantized.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call outside any stream capture. With the CUDA runtime's default lazy module loading
 * that first call is also when the driver loads this part of the library and backs the 12 MiB on
 * that device, not the dlopen: a host that budgets every byte should make one small warm-up call
 * per device before it measures what is left. Calls after the first take no device memory. All calls on a device share the one array, which
 * keeps what the last call left in it; every byte a call reads it has written first, so results do
 * not depend on earlier calls, but two calls whose kernels overlap on the GPU (different streams)
 * race and must be ordered by the caller. */
int mmh3_b200_attention_quantized_static(const void *query, const void *key, const void *value,
                                         void *output, int tokens, int heads,
                                         const Mmh3AttentionLayout *layout, float scale,
                                         mmh3_stream_t stream);

/* Not in the reference. The kernels bound every wait on a barrier; one that runs out stores a
 * nonzero code in a per-device status word and the CTA returns without finishing its tile. This
 * synchronizes the current device and returns the word (0 = every kernel ran to completion),
 * clearing it. A negative value is minus a cudaError_t. */
int mmh3_b200_take_status(void);

#ifdef __cplusplus
}
#endif

#endif /* MMH3_ATTENTION_H */
