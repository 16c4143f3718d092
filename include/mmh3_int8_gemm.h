/* C ABI of the scaled INT8 GEMM in libmmh3_attn_b200.so: the DiT's fused qkv projection, the step
 * before attention, whose epilogue leaves the per-head maxima of |v| that mmh3_attention_inputs
 * (mmh3_attention.h) turns into the FP8 V of quantized attention. The functions carry the names and
 * signatures of crates/mmh3-cuda/kernels/int8_gemm.cu, bound by crates/mmh3-cuda/src/gemm.rs:7-60.
 * Every function returns a cudaError_t as int, enqueues on `stream` and does not synchronize. */
#ifndef MMH3_INT8_GEMM_H
#define MMH3_INT8_GEMM_H

#include <stdint.h>

#include "mmh3_attention.h"

#ifdef __cplusplus
extern "C" {
#endif

/* How many tilings `config` can name (0 and 1), and the band heights a caller may try as
 * `group_m`; returns how many there are and writes up to `capacity` of them. This library runs one
 * tiling whatever the config, so the choice changes neither the results nor the speed.
 * Replace crates/mmh3-cuda/kernels/int8_gemm.cu:873-882. */
int mmh3_int8_gemm_config_count(void);
int mmh3_int8_gemm_group_heights(int *heights, int capacity);

/* output[r, c] = round(sum_k activations[r, k] * weights[c, k] * activation_scales[r] *
 * weight_scales[c]) in BF16, activations [m, k] and weights [n, k] INT8 with K contiguous, output
 * rows n elements apart. n must be a multiple of 128 (256 for config 1), k of 128; m may be ragged.
 * Replaces crates/mmh3-cuda/kernels/int8_gemm.cu:887-895. */
int mmh3_int8_gemm_bf16(int config, int group_m, const int8_t *activations, const int8_t *weights,
                        const float *activation_scales, const float *weight_scales, void *output,
                        int m, int n, int k, mmh3_stream_t stream);

/* The same with an optional FP32 bias [n], BF16 or FP16 output whose rows lie output_stride
 * elements apart (0: side by side), and:
 * - swiglu: for weights, scales and bias whose rows went through mmh3_interleave_swiglu_rows, the
 *   output is silu(gate) * up, [m, n / 2];
 * - column_maxima: for BF16 output without swiglu, receives the maximum |output| of each group of
 *   128 columns from maxima_first_column (a multiple of 128) on, as the FP32 bits of the BF16
 *   magnitude, raised with atomicMax; the caller zeroes it first. For the qkv projection with
 *   maxima_first_column = 2 * heads * 128 these are the per-head maxima of |v|.
 * - adapter_down, adapter_up (both non-null, adapter_scale != 0): the low-rank adapter
 *   adapter_scale * adapter_down . adapter_up^T is added in FP32 before the single rounding;
 *   adapter_down is BF16 [m, rank] with rows adapter_down_stride elements apart (a multiple of 8,
 *   at least rank), adapter_up BF16 [n, rank], rank a multiple of 64.
 * A negative config runs the tiling chosen for the shape. Without an adapter, outputs and maxima
 * are bit-identical to the reference's for every config; with one, the BF16 products are summed
 * in FP32 by the tensor cores in an order of their own, and the result is within the bounds of
 * the reference's tests (|error| <= |x| / 256 + 1e-4).
 * Replaces crates/mmh3-cuda/kernels/int8_gemm.cu:905-936. */
int mmh3_int8_gemm(int config, int group_m, const int8_t *activations, const int8_t *weights,
                   const float *activation_scales, const float *weight_scales, const float *bias,
                   void *output, int output_is_f16, int swiglu, int m, int n, int k,
                   int output_stride, const void *adapter_down, const void *adapter_up, int rank,
                   int adapter_down_stride, float adapter_scale, unsigned *column_maxima,
                   int maxima_first_column, mmh3_stream_t stream);

/* The bookkeeping of the reference's tiling search, which times the tilings of a shape on its first
 * call and lets the host save and restore what it chose (bound in
 * crates/mmh3-cuda/src/algorithms.rs:42-44). This library runs one tiling for every shape, so
 * nothing is ever chosen: mmh3_int8_gemm_tilings reports no entries (returns 0 and writes nothing),
 * mmh3_int8_gemm_adopt ignores what it is given, and mmh3_int8_gemm_tiling_key writes a line naming
 * the GPU and this library into `key` (`capacity` bytes; cudaErrorInvalidValue if it does not fit),
 * so that files saved by the reference's search are recognised as foreign.
 * Replace crates/mmh3-cuda/kernels/int8_gemm.cu:864-871, 940-998. */
typedef struct Mmh3Int8Tiling {
    int64_t m;
    int64_t n;
    int64_t k;
    int64_t rank;
    int64_t config;
    int64_t group_m;
} Mmh3Int8Tiling;
int mmh3_int8_gemm_tilings(Mmh3Int8Tiling *chosen, int capacity);
void mmh3_int8_gemm_adopt(const Mmh3Int8Tiling *chosen, int count);
int mmh3_int8_gemm_tiling_key(char *key, int capacity);

/* Reorders the rows of a [rows, row_bytes] matrix whose first half are SwiGLU gates and second half
 * the matching up projections into groups of eight: the gates of four features, then their up
 * projections. Replaces crates/mmh3-cuda/kernels/int8_gemm.cu:1000-1009. */
int mmh3_interleave_swiglu_rows(const void *source, void *destination, int rows, int row_bytes,
                                mmh3_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* MMH3_INT8_GEMM_H */
