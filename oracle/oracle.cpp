// CPU oracle of the attention path: TEST INFRASTRUCTURE ONLY. Nothing the library ships or times as
// its own result may call into this file; tests, the smoke check and the CPU-baseline leg of the
// benchmark are its only users.
//
// Every function restates, in plain scalar C++, what one piece of niw/mmh3 computes, and cites the
// file and lines it follows. Parity status: pinned. The known answers of the reference's own tests
// (tile plans, kept counts, tie-breaking, keep-all == dense, the +-448 uniform means, the LCG) are
// checked in tests/test_oracle.py, and on a GPU the same functions are compared with the
// reference's CUDA kernels compiled from its sources (oracle/_ref).
//
// Build: oracle/Makefile (g++ -O2 -fopenmp -shared).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// crates/mmh3-core/src/numeric.rs:3-13
inline float bf16_to_f32(uint16_t bits) {
    uint32_t word = static_cast<uint32_t>(bits) << 16;
    float value;
    std::memcpy(&value, &word, 4);
    return value;
}

inline uint16_t f32_to_bf16(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    if (std::isnan(value)) {
        return static_cast<uint16_t>((bits >> 16) | 0x40);
    }
    return static_cast<uint16_t>((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16);
}

// FP8 E4M3 (no infinities, maximum 448) from FP32, round to nearest even, saturating: what
// __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) returns
// (crates/mmh3-cuda/kernels/quantized_attention.cu:146).
inline uint8_t f32_to_e4m3(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    const uint8_t sign = static_cast<uint8_t>((bits >> 24) & 0x80);
    if (std::isnan(value)) {
        return sign | 0x7F;
    }
    const float magnitude = std::fabs(value);
    if (magnitude >= 448.0f) {
        // Everything from 448 up saturates; 464 and up would round past the largest value.
        return sign | 0x7E;
    }
    // Values below 2^-6 are subnormal: multiples of 2^-9.
    if (magnitude < 0.015625f) {
        const float scaled = magnitude * 512.0f;
        const float rounded = std::nearbyint(scaled); // ties to even in the default mode
        return sign | static_cast<uint8_t>(rounded);  // 8 rounds up into the first normal, 0x08
    }
    int exponent;
    const float fraction = std::frexp(magnitude, &exponent); // magnitude = fraction * 2^exponent
    // mantissa in [1, 2): fraction * 2, exponent - 1
    const float mantissa = fraction * 2.0f;
    int unbiased = exponent - 1;
    float steps = std::nearbyint((mantissa - 1.0f) * 8.0f);
    if (steps == 8.0f) {
        steps = 0.0f;
        unbiased += 1;
    }
    const int biased = unbiased + 7;
    const uint8_t code = static_cast<uint8_t>((biased << 3) | static_cast<int>(steps));
    return sign | (code > 0x7E ? 0x7E : code);
}

inline float e4m3_to_f32(uint8_t code) {
    const int exponent = (code >> 3) & 0xF;
    const int mantissa = code & 7;
    float magnitude;
    if (exponent == 0) {
        magnitude = std::ldexp(static_cast<float>(mantissa), -9);
    } else if (exponent == 15 && mantissa == 7) {
        magnitude = std::numeric_limits<float>::quiet_NaN();
    } else {
        magnitude = std::ldexp(1.0f + mantissa / 8.0f, exponent - 7);
    }
    return (code & 0x80) ? -magnitude : magnitude;
}

inline int threads_or_all(int threads) {
#ifdef _OPENMP
    return threads > 0 ? threads : omp_get_max_threads();
#else
    (void)threads;
    return 1;
#endif
}

} // namespace

extern "C" {

int oracle_max_threads() { return threads_or_all(0); }

uint16_t oracle_f32_to_bf16(float value) { return f32_to_bf16(value); }
float oracle_bf16_to_f32(uint16_t bits) { return bf16_to_f32(bits); }
uint8_t oracle_f32_to_e4m3(float value) { return f32_to_e4m3(value); }
float oracle_e4m3_to_f32(uint8_t code) { return e4m3_to_f32(code); }

// The generator of the reference's kernel tests (crates/mmh3-cuda/tests/attention.rs:8-16):
// fills `count` values uniform in [low, high) and returns the advanced state.
uint64_t oracle_lcg_uniform(uint64_t state, float low, float high, float *values, int64_t count) {
    for (int64_t index = 0; index < count; index++) {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        values[index] =
            low + (high - low) * (static_cast<float>(state >> 40) / static_cast<float>(1ull << 24));
    }
    return state;
}

// Softmax attention over all tokens with f64 dot products, softmax and weighted sums
// (crates/mmh3-cpu/src/dit.rs:79-118). q, k, v and output are f32 [tokens, heads, dim]. The
// reference fixes scale = 1 / sqrt(dim) and runs on one thread; `threads` > 1 splits the
// (head, query) pairs, which changes no result since every row is independent.
void oracle_attention_f32(const float *query, const float *key, const float *value, float *output,
                          int64_t tokens, int heads, int dim, double scale, int threads) {
    const int64_t inner = static_cast<int64_t>(heads) * dim;
#pragma omp parallel num_threads(threads_or_all(threads))
    {
        std::vector<double> scores(tokens);
#pragma omp for collapse(2) schedule(dynamic, 16)
        for (int head = 0; head < heads; head++) {
            for (int64_t query_token = 0; query_token < tokens; query_token++) {
                const float *query_row = query + query_token * inner + head * dim;
                for (int64_t key_token = 0; key_token < tokens; key_token++) {
                    const float *key_row = key + key_token * inner + head * dim;
                    double dot = 0.0;
                    for (int index = 0; index < dim; index++) {
                        dot += static_cast<double>(query_row[index]) * key_row[index];
                    }
                    scores[key_token] = dot * scale;
                }
                double maximum = std::numeric_limits<double>::lowest();
                for (double score : scores) {
                    maximum = std::max(maximum, score);
                }
                double total = 0.0;
                for (double &score : scores) {
                    score = std::exp(score - maximum);
                    total += score;
                }
                float *output_row = output + query_token * inner + head * dim;
                for (int index = 0; index < dim; index++) {
                    double sum = 0.0;
                    for (int64_t key_token = 0; key_token < tokens; key_token++) {
                        sum += scores[key_token] * value[key_token * inner + head * dim + index];
                    }
                    output_row[index] = static_cast<float>(sum / total);
                }
            }
        }
    }
}

// The same arithmetic on BF16 operands with the strides of Mmh3AttentionLayout (in elements), for
// the query rows [query_begin, query_end) of heads [head_begin, head_end) against all `tokens`
// keys: what the dense kernel tests compare with, and what the CPU baseline times. The output is
// f32, [query_end - query_begin][head_end - head_begin][128], unrounded. The loop nest is reordered
// against oracle_attention_f32 (keys outermost in the weighted sum) for cache locality; each output
// still adds the same f64 products in the same key order.
void oracle_attention_bf16(const uint16_t *query, const uint16_t *key, const uint16_t *value,
                           float *output, int64_t tokens, const int64_t *token_stride,
                           const int64_t *head_stride, int heads_per_key_value, double scale,
                           int64_t query_begin, int64_t query_end, int head_begin, int head_end,
                           int threads) {
    constexpr int DIM = 128;
    const int group = heads_per_key_value > 0 ? heads_per_key_value : 1;
    const int head_count = head_end - head_begin;
#pragma omp parallel num_threads(threads_or_all(threads))
    {
        std::vector<double> scores(tokens);
        std::vector<float> key_rows;
#pragma omp for collapse(2) schedule(dynamic, 4)
        for (int head = head_begin; head < head_end; head++) {
            for (int64_t query_token = query_begin; query_token < query_end; query_token++) {
                const int key_value_head = head / group;
                double query_row[DIM];
                for (int index = 0; index < DIM; index++) {
                    query_row[index] = bf16_to_f32(
                        query[query_token * token_stride[0] + head * head_stride[0] + index]);
                }
                double maximum = std::numeric_limits<double>::lowest();
                for (int64_t key_token = 0; key_token < tokens; key_token++) {
                    const uint16_t *key_row =
                        key + key_token * token_stride[1] + key_value_head * head_stride[1];
                    double dot = 0.0;
                    for (int index = 0; index < DIM; index++) {
                        dot += query_row[index] * bf16_to_f32(key_row[index]);
                    }
                    scores[key_token] = dot * scale;
                    maximum = std::max(maximum, scores[key_token]);
                }
                double total = 0.0;
                double sums[DIM] = {};
                for (int64_t key_token = 0; key_token < tokens; key_token++) {
                    const double weight = std::exp(scores[key_token] - maximum);
                    total += weight;
                    const uint16_t *value_row =
                        value + key_token * token_stride[2] + key_value_head * head_stride[2];
                    for (int index = 0; index < DIM; index++) {
                        sums[index] += weight * bf16_to_f32(value_row[index]);
                    }
                }
                float *output_row =
                    output + ((query_token - query_begin) * head_count + (head - head_begin)) * DIM;
                for (int index = 0; index < DIM; index++) {
                    output_row[index] = static_cast<float>(sums[index] / total);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Quantizer (crates/mmh3-cuda/kernels/quantized_attention.cu:85-206)

// INT8 q or k with one symmetric scale per head and block of 64 tokens (quantize_qk, :157-206), or
// per tile when tile tables are given (crates/mmh3-cuda/kernels/dit.cu:337-379). `source` is BF16
// with `token_stride` and `head_stride` in elements; `destination` is [tokens, heads, 128];
// `scales` is [heads, blocks].
void oracle_quantize_rows(const uint16_t *source, int64_t token_stride, int64_t head_stride,
                          int64_t tokens, int heads, const int32_t *tile_starts,
                          const int32_t *tile_lengths, int tiles, int8_t *destination,
                          float *scales) {
    const int blocks = tile_starts != nullptr ? tiles : static_cast<int>((tokens + 63) / 64);
#pragma omp parallel for collapse(2)
    for (int head = 0; head < heads; head++) {
        for (int block = 0; block < blocks; block++) {
            const int64_t first = tile_starts != nullptr ? tile_starts[block] : block * 64ll;
            const int64_t rows =
                tile_lengths != nullptr ? tile_lengths[block] : std::min<int64_t>(64, tokens - first);
            float maximum = 0.0f;
            for (int64_t row = 0; row < rows; row++) {
                for (int index = 0; index < 128; index++) {
                    maximum = std::fmax(
                        maximum, std::fabs(bf16_to_f32(
                                     source[(first + row) * token_stride + head * head_stride + index])));
                }
            }
            const float scale = std::fmax(maximum / 127.0f, 1e-30f);
            scales[head * blocks + block] = scale;
            for (int64_t row = 0; row < rows; row++) {
                for (int index = 0; index < 128; index++) {
                    const float element = bf16_to_f32(
                        source[(first + row) * token_stride + head * head_stride + index]);
                    // __float2int_rn: round to nearest even.
                    destination[((first + row) * heads + head) * 128 + index] =
                        static_cast<int8_t>(static_cast<int>(std::nearbyint(element / scale)));
                }
            }
        }
    }
}

// Block maxima of |v| (value_max, :85-114), the per-head scale max / 448 (value_scales, :116-127)
// and FP8 E4M3 V transposed to [heads, 128, blocks * 64] with zeroes past each block's rows
// (quantize_value :130-155, quantize_value_tiles :210-241).
void oracle_quantize_value(const uint16_t *source, int64_t token_stride, int64_t head_stride,
                           int64_t tokens, int heads, const int32_t *tile_starts,
                           const int32_t *tile_lengths, int tiles, uint8_t *destination,
                           float *value_scales, float *value_maxima) {
    const int blocks = tile_starts != nullptr ? tiles : static_cast<int>((tokens + 63) / 64);
    const int64_t padded = blocks * 64ll;
#pragma omp parallel for
    for (int head = 0; head < heads; head++) {
        float head_maximum = 0.0f;
        for (int block = 0; block < blocks; block++) {
            const int64_t first = tile_starts != nullptr ? tile_starts[block] : block * 64ll;
            const int64_t rows =
                tile_lengths != nullptr ? tile_lengths[block] : std::min<int64_t>(64, tokens - first);
            float maximum = 0.0f;
            for (int64_t row = 0; row < rows; row++) {
                for (int index = 0; index < 128; index++) {
                    maximum = std::fmax(
                        maximum, std::fabs(bf16_to_f32(
                                     source[(first + row) * token_stride + head * head_stride + index])));
                }
            }
            value_maxima[head * blocks + block] = maximum;
            head_maximum = std::fmax(head_maximum, maximum);
        }
        const float scale = std::fmax(head_maximum / 448.0f, 1e-30f);
        value_scales[head] = scale;
        for (int block = 0; block < blocks; block++) {
            const int64_t first = tile_starts != nullptr ? tile_starts[block] : block * 64ll;
            const int64_t rows =
                tile_lengths != nullptr ? tile_lengths[block] : std::min<int64_t>(64, tokens - first);
            for (int index = 0; index < 128; index++) {
                for (int64_t row = 0; row < 64; row++) {
                    const float element =
                        row < rows ? bf16_to_f32(source[(first + row) * token_stride +
                                                        head * head_stride + index]) /
                                         scale
                                   : 0.0f;
                    destination[(static_cast<int64_t>(head) * 128 + index) * padded + block * 64 +
                                row] = f32_to_e4m3(element);
                }
            }
        }
    }
}

// The INT8 QK / FP8 PV attention over a prepared workspace, block by block in FP32 as the kernel
// walks it (crates/mmh3-cuda/kernels/quantized_attention.cu:357-477, 538-547): integer dot
// products, dequantized with scale * log2(e) * q_scale * k_scale, an online base-2 softmax whose
// probabilities are scaled by 448 and rounded to E4M3 before they meet the FP8 values, and a final
// factor value_scale / 448 / row_sum. With `routes` (VSA) a query tile walks its route list and
// tile tables give the rows; without, every 64-token block in order. `gate`/`coarse` add the VSA
// coarse branch (:521-537). Output BF16 [tokens, heads, 128] with `output_token_stride`.
void oracle_quantized_attention(const int8_t *query8, const int8_t *key8, const uint8_t *value8,
                                const float *query_scales, const float *key_scales,
                                const float *value_scales, int64_t tokens, int heads, float scale,
                                const int32_t *tile_starts, const int32_t *tile_lengths, int tiles,
                                const uint16_t *routes, const int32_t *route_counts,
                                const uint16_t *gate, int64_t gate_stride, const float *coarse,
                                uint16_t *output, int64_t output_token_stride,
                                int64_t output_head_stride) {
    const bool vsa = tile_starts != nullptr;
    const int blocks = vsa ? tiles : static_cast<int>((tokens + 63) / 64);
    const int64_t padded = blocks * 64ll;
    const float scale_log2 = scale * 1.4426950408889634f;
    float e4m3_table[256];
    for (int code = 0; code < 256; code++) {
        e4m3_table[code] = e4m3_to_f32(static_cast<uint8_t>(code));
    }
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int head = 0; head < heads; head++) {
        for (int query_block = 0; query_block < blocks; query_block++) {
            const int64_t first_query = vsa ? tile_starts[query_block] : query_block * 64ll;
            const int64_t query_rows =
                vsa ? tile_lengths[query_block] : std::min<int64_t>(64, tokens - first_query);
            const size_t route_row = static_cast<size_t>(head) * blocks + query_block;
            const int count = routes != nullptr ? route_counts[route_row] : blocks;
            for (int64_t row = 0; row < query_rows; row++) {
                const int8_t *query_row = query8 + ((first_query + row) * heads + head) * 128;
                float row_max = -std::numeric_limits<float>::max();
                float row_sum = 0.0f;
                float accumulators[128] = {};
                for (int entry = 0; entry < count; entry++) {
                    const int key_block =
                        routes != nullptr ? routes[route_row * blocks + entry] : entry;
                    const int64_t first_key = vsa ? tile_starts[key_block] : key_block * 64ll;
                    const int64_t key_count =
                        vsa ? tile_lengths[key_block] : std::min<int64_t>(64, tokens - first_key);
                    const float factor = scale_log2 * query_scales[route_row] *
                                         key_scales[head * blocks + key_block];
                    float scores[64];
                    float block_max = -std::numeric_limits<float>::max();
                    for (int64_t column = 0; column < key_count; column++) {
                        const int8_t *key_row = key8 + ((first_key + column) * heads + head) * 128;
                        int32_t dot = 0;
                        for (int index = 0; index < 128; index++) {
                            dot += static_cast<int32_t>(query_row[index]) * key_row[index];
                        }
                        scores[column] = static_cast<float>(dot) * factor;
                        block_max = std::fmax(block_max, scores[column]);
                    }
                    const float new_max = std::fmax(row_max, block_max);
                    const float correction = std::exp2(row_max - new_max);
                    row_max = new_max;
                    row_sum *= correction;
                    for (float &accumulator : accumulators) {
                        accumulator *= correction;
                    }
                    for (int64_t column = 0; column < key_count; column++) {
                        const float probability = std::exp2(scores[column] - row_max);
                        row_sum += probability;
                        const float rounded = e4m3_table[f32_to_e4m3(probability * 448.0f)];
                        if (rounded == 0.0f) {
                            continue;
                        }
                        const uint8_t *value_column = value8 +
                                                      static_cast<int64_t>(head) * 128 * padded +
                                                      key_block * 64ll + column;
                        for (int index = 0; index < 128; index++) {
                            accumulators[index] +=
                                rounded * e4m3_table[value_column[index * padded]];
                        }
                    }
                }
                const float inverse = value_scales[head] / 448.0f / row_sum;
                const int64_t token = first_query + row;
                uint16_t *output_row =
                    output + token * output_token_stride + head * output_head_stride;
                for (int index = 0; index < 128; index++) {
                    float result = accumulators[index] * inverse;
                    if (gate != nullptr) {
                        result = std::fma(bf16_to_f32(gate[token * gate_stride + head * 128 + index]),
                                          coarse[route_row * 128 + index], result);
                    }
                    output_row[index] = f32_to_bf16(result);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Video sparse attention (crates/mmh3-core/src/dit/vsa.rs)

// VsaPlan::for_layout (vsa.rs:38-103) for PackedLayout::text_to_video(text_tokens, frames,
// latent_height, latent_width, audio_frames) (crates/mmh3-core/src/dit/layout.rs:188-204,
// 300-321): a text segment, 2 * audio_frames audio rows, then frames * (latent_height / 2) *
// (latent_width / 2) video patches. Segments before the video are cut every 64 tokens; the video
// is grouped into 4 x 4 x 4 cubes of (frame, row, column), smaller at the far edges.
// Returns the tile count; with null outputs only counts. `video_order` gets one entry per video
// token, `meta` = {prefix_tiles, video_start, tokens}.
int oracle_vsa_plan(int text_tokens, int frames, int latent_height, int latent_width,
                    int audio_frames, int32_t *tile_starts, int32_t *tile_lengths,
                    int32_t *video_order, int32_t *meta) {
    const int segments[2][2] = {{0, text_tokens}, {text_tokens, text_tokens + 2 * audio_frames}};
    int tiles = 0;
    for (const auto &segment : segments) {
        for (int start = segment[0]; start < segment[1]; start += 64) {
            if (tile_starts != nullptr) {
                tile_starts[tiles] = start;
                tile_lengths[tiles] = std::min(segment[1] - start, 64);
            }
            tiles++;
        }
    }
    const int prefix_tiles = tiles;
    const int video_start = text_tokens + 2 * audio_frames;
    const int grid[3] = {frames, latent_height / 2, latent_width / 2};
    int start = video_start;
    int ordered = 0;
    for (int frame_tile = 0; frame_tile < grid[0]; frame_tile += 4) {
        for (int row_tile = 0; row_tile < grid[1]; row_tile += 4) {
            for (int column_tile = 0; column_tile < grid[2]; column_tile += 4) {
                const int before = ordered;
                for (int frame = frame_tile; frame < std::min(frame_tile + 4, grid[0]); frame++) {
                    for (int row = row_tile; row < std::min(row_tile + 4, grid[1]); row++) {
                        for (int column = column_tile; column < std::min(column_tile + 4, grid[2]);
                             column++) {
                            if (video_order != nullptr) {
                                video_order[ordered] = (frame * grid[1] + row) * grid[2] + column;
                            }
                            ordered++;
                        }
                    }
                }
                if (tile_starts != nullptr) {
                    tile_starts[tiles] = start;
                    tile_lengths[tiles] = ordered - before;
                }
                start += ordered - before;
                tiles++;
            }
        }
    }
    if (meta != nullptr) {
        meta[0] = prefix_tiles;
        meta[1] = video_start;
        meta[2] = start;
    }
    return tiles;
}

// VsaPlan::kept_video_tiles (vsa.rs:103-106).
int oracle_vsa_kept(int video_tiles, double sparsity) {
    const int kept = static_cast<int>(std::ceil((1.0 - sparsity) * video_tiles));
    return std::min(std::max(kept, 1), std::max(video_tiles, 1));
}

// select_tiles (vsa.rs:144-164): every tile for a prefix query tile or when nothing is dropped,
// else the prefix tiles and the `kept` best video tiles by score (total order on floats, ties to
// the lower index), ascending. Returns how many tiles `selected` received.
int oracle_select_tiles(const float *scores, int tiles, int query_tile, int prefix_tiles, int kept,
                        int32_t *selected) {
    if (query_tile < prefix_tiles || kept >= tiles - prefix_tiles) {
        for (int tile = 0; tile < tiles; tile++) {
            selected[tile] = tile;
        }
        return tiles;
    }
    // f32::total_cmp orders by the sign-magnitude bit pattern.
    auto key = [](float value) {
        int32_t bits;
        std::memcpy(&bits, &value, 4);
        return bits ^ static_cast<int32_t>(static_cast<uint32_t>(bits >> 31) >> 1);
    };
    std::vector<int> video(tiles - prefix_tiles);
    for (int index = 0; index < tiles - prefix_tiles; index++) {
        video[index] = prefix_tiles + index;
    }
    std::sort(video.begin(), video.end(), [&](int left, int right) {
        const int32_t left_key = key(scores[left]), right_key = key(scores[right]);
        return left_key != right_key ? left_key > right_key : left < right;
    });
    video.resize(kept);
    std::sort(video.begin(), video.end());
    int count = 0;
    for (int tile = 0; tile < prefix_tiles; tile++) {
        selected[count++] = tile;
    }
    for (int tile : video) {
        selected[count++] = tile;
    }
    return count;
}

// Pooled tiles in FP32 as pool_kernel computes them (crates/mmh3-cuda/kernels/vsa_attention.cu:
// 68-91): sums over the rows in row order, the query and key divided by the row count, the value
// left as a sum. Outputs are [heads, tiles, 128].
void oracle_vsa_pool(const uint16_t *query, const uint16_t *key, const uint16_t *value,
                     const int64_t *token_stride, const int64_t *head_stride, int heads,
                     const int32_t *tile_starts, const int32_t *tile_lengths, int tiles,
                     float *pooled_query, float *pooled_key, float *pooled_value) {
#pragma omp parallel for collapse(2)
    for (int head = 0; head < heads; head++) {
        for (int tile = 0; tile < tiles; tile++) {
            const int rows = tile_lengths[tile];
            for (int index = 0; index < 128; index++) {
                float sums[3] = {0.0f, 0.0f, 0.0f};
                const uint16_t *tensors[3] = {query, key, value};
                for (int row = 0; row < rows; row++) {
                    const int64_t token = tile_starts[tile] + row;
                    for (int tensor = 0; tensor < 3; tensor++) {
                        sums[tensor] += bf16_to_f32(
                            tensors[tensor][token * token_stride[tensor] +
                                            head * head_stride[tensor] + index]);
                    }
                }
                const size_t at = (static_cast<size_t>(head) * tiles + tile) * 128 + index;
                pooled_query[at] = sums[0] / rows;
                pooled_key[at] = sums[1] / rows;
                pooled_value[at] = sums[2];
            }
        }
    }
}

// The FP32 score of one pooled query against one pooled key in the kernel's evaluation order
// (vsa_attention.cu:133-166): lane l chains fused multiply-adds over dimensions l, l + 32, l + 64,
// l + 96, the 32 lane partials are added over an xor butterfly (offsets 16, 8, 4, 2, 1), and the
// sum is multiplied by the scale.
float oracle_vsa_score(const float *pooled_query, const float *pooled_key, float scale) {
    float partials[32];
    for (int lane = 0; lane < 32; lane++) {
        float partial = 0.0f;
        for (int part = 0; part < 4; part++) {
            partial = std::fma(pooled_query[lane + part * 32], pooled_key[lane + part * 32], partial);
        }
        partials[lane] = partial;
    }
    for (int offset = 16; offset > 0; offset /= 2) {
        float next[32];
        for (int lane = 0; lane < 32; lane++) {
            next[lane] = partials[lane] + partials[lane ^ offset];
        }
        std::memcpy(partials, next, sizeof(next));
    }
    return partials[0] * scale;
}

// Scores, routes and route counts of every (head, query tile) as select_kernel leaves them
// (vsa_attention.cu:96-221), through oracle_vsa_score and oracle_select_tiles. `routes` is
// [heads, tiles, tiles] with the first route_counts entries of each row written; `scores_out`
// (nullable) is [heads, tiles, tiles].
void oracle_vsa_select(const float *pooled_query, const float *pooled_key, int heads, int tiles,
                       int prefix_tiles, int kept, float scale, uint16_t *routes,
                       int32_t *route_counts, float *scores_out) {
#pragma omp parallel
    {
        std::vector<float> scores(tiles);
        std::vector<int32_t> selected(tiles);
#pragma omp for collapse(2)
        for (int head = 0; head < heads; head++) {
            for (int query_tile = 0; query_tile < tiles; query_tile++) {
                const size_t row = static_cast<size_t>(head) * tiles + query_tile;
                for (int tile = 0; tile < tiles; tile++) {
                    scores[tile] = oracle_vsa_score(
                        pooled_query + row * 128,
                        pooled_key + (static_cast<size_t>(head) * tiles + tile) * 128, scale);
                }
                if (scores_out != nullptr) {
                    std::memcpy(scores_out + row * tiles, scores.data(), tiles * sizeof(float));
                }
                const int count = oracle_select_tiles(scores.data(), tiles, query_tile,
                                                      prefix_tiles, kept, selected.data());
                route_counts[row] = count;
                for (int entry = 0; entry < count; entry++) {
                    routes[row * tiles + entry] = static_cast<uint16_t>(selected[entry]);
                }
            }
        }
    }
}

// VSA over [tokens, heads, dim] f32 query, key and value in the plan's order, computed in f64
// (reference(), vsa.rs:169-266). A non-null gate, in the same layout, enables the coarse branch.
void oracle_vsa_reference(const float *query, const float *key, const float *value,
                          const float *gate, const int32_t *tile_starts,
                          const int32_t *tile_lengths, int tiles, int prefix_tiles, int heads,
                          int dim, float scale, int kept, float *output) {
    auto at = [&](const float *tensor, int64_t token, int head, int index) {
        return static_cast<double>(tensor[(token * heads + head) * dim + index]);
    };
#pragma omp parallel for
    for (int head = 0; head < heads; head++) {
        std::vector<std::vector<double>> pooled[3];
        const float *tensors[3] = {query, key, value};
        for (int tensor = 0; tensor < 3; tensor++) {
            pooled[tensor].assign(tiles, std::vector<double>(dim));
            for (int tile = 0; tile < tiles; tile++) {
                for (int index = 0; index < dim; index++) {
                    double sum = 0.0;
                    for (int row = 0; row < tile_lengths[tile]; row++) {
                        sum += at(tensors[tensor], tile_starts[tile] + row, head, index);
                    }
                    pooled[tensor][tile][index] = sum / tile_lengths[tile];
                }
            }
        }
        std::vector<double> scores(tiles), weights(tiles), coarse(dim);
        std::vector<float> scores_f32(tiles);
        std::vector<int32_t> selected(tiles);
        for (int query_tile = 0; query_tile < tiles; query_tile++) {
            for (int tile = 0; tile < tiles; tile++) {
                double dot = 0.0;
                for (int index = 0; index < dim; index++) {
                    dot += pooled[0][query_tile][index] * pooled[1][tile][index];
                }
                scores[tile] = dot * static_cast<double>(scale);
                scores_f32[tile] = static_cast<float>(scores[tile]);
            }
            const int count = oracle_select_tiles(scores_f32.data(), tiles, query_tile,
                                                  prefix_tiles, kept, selected.data());
            double maximum = std::numeric_limits<double>::lowest();
            for (double score : scores) {
                maximum = std::max(maximum, score);
            }
            double total = 0.0;
            for (int tile = 0; tile < tiles; tile++) {
                weights[tile] = std::exp(scores[tile] - maximum);
                total += weights[tile];
            }
            for (int index = 0; index < dim; index++) {
                double sum = 0.0;
                for (int tile = 0; tile < tiles; tile++) {
                    sum += weights[tile] * pooled[2][tile][index];
                }
                coarse[index] = sum / total;
            }
            std::vector<int64_t> keys;
            for (int entry = 0; entry < count; entry++) {
                const int tile = selected[entry];
                for (int row = 0; row < tile_lengths[tile]; row++) {
                    keys.push_back(tile_starts[tile] + row);
                }
            }
            std::vector<double> logits(keys.size());
            for (int row = 0; row < tile_lengths[query_tile]; row++) {
                const int64_t token = tile_starts[query_tile] + row;
                double row_maximum = std::numeric_limits<double>::lowest();
                for (size_t other = 0; other < keys.size(); other++) {
                    double dot = 0.0;
                    for (int index = 0; index < dim; index++) {
                        dot += at(query, token, head, index) * at(key, keys[other], head, index);
                    }
                    logits[other] = dot * static_cast<double>(scale);
                    row_maximum = std::max(row_maximum, logits[other]);
                }
                double row_total = 0.0;
                for (double &logit : logits) {
                    logit = std::exp(logit - row_maximum);
                    row_total += logit;
                }
                for (int index = 0; index < dim; index++) {
                    double sum = 0.0;
                    for (size_t other = 0; other < keys.size(); other++) {
                        sum += logits[other] * at(value, keys[other], head, index);
                    }
                    sum /= row_total;
                    if (gate != nullptr) {
                        sum += at(gate, token, head, index) * coarse[index];
                    }
                    output[(token * heads + head) * dim + index] = static_cast<float>(sum);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Sol-Attn (crates/mmh3-core/src/dit/sparse.rs, crates/mmh3-cuda/kernels/sparse_attention.cu)

// Everything the routing of Sol-Attn leaves in its workspace, in FP32 and in the kernels' order
// (sparse_attention.cu:72-290, 315-338), from BF16 query, key and value with strides in elements:
// block_stats (sums down the rows; mean query, mean key, summed value), center_keys (mean and
// variance down the blocks, the block keys centred in place), route (threshold = tau * sqrt(spread
// * log2_scale^2 + 1e-6) with the spread summed over a xor butterfly per warp of 32 dimensions and
// then over the four warps; pooled scores in the order of oracle_vsa_score; a key block is routed
// if its score clears the threshold, if it neighbours the query block, or by the sinks), the
// pooled tail of the unrouted blocks as (maximum, sum of weights times block length, weighted value
// sums), and row_offsets. The tail sums and the offsets are accumulated in FP32 in an order of
// this function's own; the kernels' differ in the last bits. `sinks` = {key start, key end, query
// start, query end}. Any output may be null.
void oracle_sol_route(const uint16_t *query, const uint16_t *key, const uint16_t *value,
                      const int64_t *token_stride, const int64_t *head_stride, int tokens,
                      int heads, float tau, float scale, const int32_t *sinks, float *centroids,
                      float *block_keys, float *value_sums, float *key_mean, float *key_variance,
                      float *row_offsets, uint16_t *routes, int32_t *route_counts,
                      float *tail_max, float *tail_sum, float *tail_values) {
    const int blocks = (tokens + 63) / 64;
    const float log2_scale = scale * 1.4426950408889634f;
    std::vector<int32_t> starts(blocks), lengths(blocks);
    for (int block = 0; block < blocks; block++) {
        starts[block] = block * 64;
        lengths[block] = std::min(64, tokens - block * 64);
    }
    const size_t per_block = static_cast<size_t>(heads) * blocks * 128;
    std::vector<float> mean_query(per_block), mean_key(per_block), sums(per_block);
    oracle_vsa_pool(query, key, value, token_stride, head_stride, heads, starts.data(),
                    lengths.data(), blocks, mean_query.data(), mean_key.data(), sums.data());
    std::vector<float> means(heads * 128), variances(heads * 128);
    for (int head = 0; head < heads; head++) {
        for (int index = 0; index < 128; index++) {
            float *column = mean_key.data() + static_cast<size_t>(head) * blocks * 128 + index;
            float total = 0.0f;
            for (int block = 0; block < blocks; block++) {
                total += column[static_cast<size_t>(block) * 128];
            }
            const float mean = total / blocks;
            float squares = 0.0f;
            for (int block = 0; block < blocks; block++) {
                const float centred = column[static_cast<size_t>(block) * 128] - mean;
                column[static_cast<size_t>(block) * 128] = centred;
                squares = std::fma(centred, centred, squares);
            }
            means[head * 128 + index] = mean;
            variances[head * 128 + index] = squares / blocks;
        }
    }
#pragma omp parallel
    {
        std::vector<float> scores(blocks);
        std::vector<uint8_t> routed(blocks);
#pragma omp for collapse(2)
        for (int head = 0; head < heads; head++) {
            for (int query_block = 0; query_block < blocks; query_block++) {
                const size_t row = static_cast<size_t>(head) * blocks + query_block;
                const float *centroid = mean_query.data() + row * 128;
                float warps[4];
                for (int warp = 0; warp < 4; warp++) {
                    float lanes[32];
                    for (int lane = 0; lane < 32; lane++) {
                        const int index = warp * 32 + lane;
                        lanes[lane] = (centroid[index] * centroid[index]) *
                                      variances[head * 128 + index];
                    }
                    for (int offset = 16; offset > 0; offset /= 2) {
                        float next[32];
                        for (int lane = 0; lane < 32; lane++) {
                            next[lane] = lanes[lane] + lanes[lane ^ offset];
                        }
                        std::memcpy(lanes, next, sizeof(next));
                    }
                    warps[warp] = lanes[0];
                }
                const float spread = ((warps[0] + warps[1]) + warps[2]) + warps[3];
                const float threshold =
                    tau * std::sqrt(std::fma(spread * log2_scale, log2_scale, 1e-6f));
                int count = 0;
                float maximum = -std::numeric_limits<float>::max();
                for (int key_block = 0; key_block < blocks; key_block++) {
                    scores[key_block] = oracle_vsa_score(
                        centroid,
                        mean_key.data() + (static_cast<size_t>(head) * blocks + key_block) * 128,
                        log2_scale);
                    routed[key_block] = scores[key_block] > threshold ||
                                        std::abs(query_block - key_block) <= 1 ||
                                        (key_block >= sinks[0] && key_block < sinks[1]) ||
                                        (query_block >= sinks[2] && query_block < sinks[3]);
                    if (routed[key_block]) {
                        if (routes != nullptr) {
                            routes[row * blocks + count] = static_cast<uint16_t>(key_block);
                        }
                        count++;
                    } else {
                        maximum = std::max(maximum, scores[key_block]);
                    }
                }
                if (route_counts != nullptr) {
                    route_counts[row] = count;
                }
                float total = 0.0f;
                float weighted[128] = {};
                for (int key_block = 0; key_block < blocks; key_block++) {
                    if (routed[key_block]) {
                        continue;
                    }
                    const float weight = std::exp2(scores[key_block] - maximum);
                    total = std::fma(weight, static_cast<float>(lengths[key_block]), total);
                    const float *block_sums =
                        sums.data() + (static_cast<size_t>(head) * blocks + key_block) * 128;
                    for (int index = 0; index < 128; index++) {
                        weighted[index] = std::fma(weight, block_sums[index], weighted[index]);
                    }
                }
                if (tail_max != nullptr) {
                    tail_max[row] = maximum;
                }
                if (tail_sum != nullptr) {
                    tail_sum[row] = total;
                }
                if (tail_values != nullptr) {
                    std::memcpy(tail_values + row * 128, weighted, sizeof(weighted));
                }
            }
        }
    }
    if (row_offsets != nullptr) {
#pragma omp parallel for collapse(2)
        for (int head = 0; head < heads; head++) {
            for (int token = 0; token < tokens; token++) {
                const uint16_t *row = query + static_cast<int64_t>(token) * token_stride[0] +
                                      static_cast<int64_t>(head) * head_stride[0];
                float lanes[32];
                for (int lane = 0; lane < 32; lane++) {
                    float partial = 0.0f;
                    for (int part = 0; part < 4; part++) {
                        partial = std::fma(bf16_to_f32(row[lane + part * 32]),
                                           means[head * 128 + lane + part * 32], partial);
                    }
                    lanes[lane] = partial;
                }
                for (int offset = 16; offset > 0; offset /= 2) {
                    float next[32];
                    for (int lane = 0; lane < 32; lane++) {
                        next[lane] = lanes[lane] + lanes[lane ^ offset];
                    }
                    std::memcpy(lanes, next, sizeof(next));
                }
                row_offsets[static_cast<size_t>(head) * tokens + token] = lanes[0] * log2_scale;
            }
        }
    }
    auto copy = [](float *destination, const std::vector<float> &source) {
        if (destination != nullptr) {
            std::memcpy(destination, source.data(), source.size() * sizeof(float));
        }
    };
    copy(centroids, mean_query);
    copy(block_keys, mean_key);
    copy(value_sums, sums);
    copy(key_mean, means);
    copy(key_variance, variances);
}

// Sol-Attn over [tokens, heads, dim] f32 query, key and value, computed densely in f64
// (reference(), sparse.rs:103-234): block means of the queries and keys and block sums of the
// values; the block keys centred by their mean, whose variance sets each query block's threshold;
// a key block is exact when its pooled score clears the threshold, neighbours the query block, or
// by the sinks; a row's softmax runs over the tokens of the exact blocks (keys centred by the same
// mean) and one term per other block (pooled score, weight = block length, value = block sum).
// Returns the fraction of (head, query block, key block) triples routed exactly.
double oracle_sol_reference(const float *query, const float *key, const float *value, int tokens,
                            int heads, int dim, float tau, float scale, const int32_t *sinks,
                            float *output) {
    const int blocks = (tokens + 63) / 64;
    auto length = [&](int block) { return std::min(64, tokens - block * 64); };
    auto at = [&](const float *tensor, int64_t token, int head, int index) {
        return static_cast<double>(tensor[(token * heads + head) * dim + index]);
    };
    const double log2_scale = static_cast<double>(scale) * 1.4426950408889634074;
    int64_t routed_total = 0;
#pragma omp parallel for reduction(+ : routed_total)
    for (int head = 0; head < heads; head++) {
        auto pool = [&](const float *tensor, bool mean) {
            std::vector<std::vector<double>> pooled(blocks, std::vector<double>(dim));
            for (int block = 0; block < blocks; block++) {
                for (int index = 0; index < dim; index++) {
                    double sum = 0.0;
                    for (int row = 0; row < length(block); row++) {
                        sum += at(tensor, static_cast<int64_t>(block) * 64 + row, head, index);
                    }
                    pooled[block][index] = mean ? sum / length(block) : sum;
                }
            }
            return pooled;
        };
        const auto centroids = pool(query, true);
        auto block_keys = pool(key, true);
        const auto value_sums = pool(value, false);
        std::vector<double> key_mean(dim), key_variance(dim);
        for (int index = 0; index < dim; index++) {
            double sum = 0.0;
            for (int block = 0; block < blocks; block++) {
                sum += block_keys[block][index];
            }
            key_mean[index] = sum / blocks;
        }
        for (int index = 0; index < dim; index++) {
            double squares = 0.0;
            for (int block = 0; block < blocks; block++) {
                block_keys[block][index] -= key_mean[index];
                squares += block_keys[block][index] * block_keys[block][index];
            }
            key_variance[index] = squares / blocks;
        }
        std::vector<double> pooled(blocks), scores, weights;
        std::vector<uint8_t> exact(blocks);
        std::vector<const double *> rows;
        std::vector<double> centred;
        for (int query_block = 0; query_block < blocks; query_block++) {
            const auto &centroid = centroids[query_block];
            double spread = 0.0;
            for (int index = 0; index < dim; index++) {
                spread += centroid[index] * centroid[index] * key_variance[index];
            }
            const double threshold =
                static_cast<double>(tau) * std::sqrt(spread * log2_scale * log2_scale + 1e-6);
            for (int key_block = 0; key_block < blocks; key_block++) {
                double dot = 0.0;
                for (int index = 0; index < dim; index++) {
                    dot += centroid[index] * block_keys[key_block][index];
                }
                pooled[key_block] = dot * log2_scale;
                exact[key_block] = pooled[key_block] > threshold ||
                                   std::abs(query_block - key_block) <= 1 ||
                                   (key_block >= sinks[0] && key_block < sinks[1]) ||
                                   (query_block >= sinks[2] && query_block < sinks[3]);
                routed_total += exact[key_block];
            }
            for (int row = 0; row < length(query_block); row++) {
                const int64_t token = static_cast<int64_t>(query_block) * 64 + row;
                // One term per key token of an exact block, one per other block.
                scores.clear();
                weights.clear();
                std::vector<std::pair<int, int64_t>> sources; // (1, token) or (0, block)
                for (int key_block = 0; key_block < blocks; key_block++) {
                    if (exact[key_block]) {
                        for (int other = 0; other < length(key_block); other++) {
                            const int64_t key_token = static_cast<int64_t>(key_block) * 64 + other;
                            double dot = 0.0;
                            for (int index = 0; index < dim; index++) {
                                dot += at(query, token, head, index) *
                                       (at(key, key_token, head, index) - key_mean[index]);
                            }
                            scores.push_back(dot * log2_scale);
                            weights.push_back(1.0);
                            sources.emplace_back(1, key_token);
                        }
                    } else {
                        scores.push_back(pooled[key_block]);
                        weights.push_back(length(key_block));
                        sources.emplace_back(0, key_block);
                    }
                }
                double maximum = std::numeric_limits<double>::lowest();
                for (double score : scores) {
                    maximum = std::max(maximum, score);
                }
                std::vector<double> numerator(dim, 0.0);
                double denominator = 0.0;
                for (size_t term = 0; term < scores.size(); term++) {
                    const double probability = std::exp2(scores[term] - maximum);
                    denominator += probability * weights[term];
                    for (int index = 0; index < dim; index++) {
                        const double term_value =
                            sources[term].first ? at(value, sources[term].second, head, index)
                                                : value_sums[sources[term].second][index];
                        numerator[index] += probability * term_value;
                    }
                }
                for (int index = 0; index < dim; index++) {
                    output[(token * heads + head) * dim + index] =
                        static_cast<float>(numerator[index] / denominator);
                }
            }
        }
    }
    return static_cast<double>(routed_total) /
           (static_cast<double>(heads) * blocks * static_cast<double>(blocks));
}

// ---------------------------------------------------------------------------------------------
// Ulysses partitioning (crates/mmh3-core/src/shard.rs:168-188): contiguous cuts of `count` items
// (tokens, in units of `alignment`, or heads) over `ranks`, the remainder going to the last rank.
// Writes ranks + 1 boundaries.
void oracle_shard_even(int64_t count, int ranks, int64_t alignment, int64_t *boundaries) {
    const int64_t step = alignment > 0 ? alignment : 1;
    const int64_t each = (count / ranks / step) * step;
    for (int rank = 0; rank < ranks; rank++) {
        boundaries[rank] = rank * each;
    }
    boundaries[ranks] = count;
}

// The scaled INT8 GEMM of the linear layers: the exact integer sums, then the FP32 operations of
// crates/mmh3-cuda/kernels/int8_gemm.cu in their order: (sum * activation scale) * weight scale
// (lines 448-457), + bias (489-508), rounded to BF16 or FP16 (521-525). With `swiglu`, columns come
// in groups of eight, the gates of four features and then their up projections, and the output
// [m, n / 2] is silu(gate) * up of the rounded products, rounded again (297-305, 545-554); expf
// stands where the kernel has __expf, so those bits may differ in the last place. `maxima`, unless
// null, receives the largest |output| of each group of 128 columns from `first_column` on as the
// FP32 bits of the BF16 magnitude (112-116, 556-587). `output_stride` elements lie between rows.
void oracle_int8_gemm(const int8_t *activations, const int8_t *weights,
                      const float *activation_scales, const float *weight_scales,
                      const float *bias, uint16_t *output, int f16, int swiglu, int m, int n, int k,
                      int output_stride, uint32_t *maxima, int first_column) {
    auto round_bits = [f16](float value) -> uint16_t {
        if (f16) {
            const _Float16 half = static_cast<_Float16>(value);
            uint16_t bits;
            std::memcpy(&bits, &half, 2);
            return bits;
        }
        return f32_to_bf16(value);
    };
    auto widen = [f16](uint16_t bits) -> float {
        if (f16) {
            _Float16 half;
            std::memcpy(&half, &bits, 2);
            return static_cast<float>(half);
        }
        return bf16_to_f32(bits);
    };
    const int groups = maxima != nullptr && n > first_column ? (n - first_column) / 128 : 0;
    std::vector<uint32_t> largest(groups, 0);
    #pragma omp parallel
    {
        std::vector<uint16_t> rounded(n);
        std::vector<uint32_t> local(groups, 0);
        #pragma omp for schedule(static)
        for (int row = 0; row < m; row++) {
            const int8_t *a = activations + static_cast<size_t>(row) * k;
            for (int column = 0; column < n; column++) {
                const int8_t *w = weights + static_cast<size_t>(column) * k;
                int32_t sum = 0;
                for (int index = 0; index < k; index++) {
                    sum += static_cast<int32_t>(a[index]) * static_cast<int32_t>(w[index]);
                }
                float value = static_cast<float>(sum) * activation_scales[row];
                value = value * weight_scales[column];
                if (bias != nullptr) {
                    value = value + bias[column];
                }
                rounded[column] = round_bits(value);
            }
            uint16_t *output_row = output + static_cast<size_t>(row) * output_stride;
            if (swiglu) {
                for (int column = 0; column < n; column += 8) {
                    for (int feature = 0; feature < 4; feature++) {
                        const float gate = widen(rounded[column + feature]);
                        const float up = widen(rounded[column + 4 + feature]);
                        output_row[column / 2 + feature] =
                            round_bits(gate / (1.0f + std::exp(-gate)) * up);
                    }
                }
            } else {
                for (int column = 0; column < n; column++) {
                    output_row[column] = rounded[column];
                    if (column >= first_column && groups > 0) {
                        uint32_t &slot = local[(column - first_column) / 128];
                        slot = std::max(slot, static_cast<uint32_t>(rounded[column] & 0x7fffu) << 16);
                    }
                }
            }
        }
        #pragma omp critical
        for (int group = 0; group < groups; group++) {
            largest[group] = std::max(largest[group], local[group]);
        }
    }
    for (int group = 0; group < groups; group++) {
        maxima[group] = std::max(maxima[group], largest[group]);
    }
}

} // extern "C"
