// Dense attention on sm_100a: softmax(Q K^T * scale) V with FP32 accumulation and softmax, for heads
// of 64 or 128 in BF16 or FP16, causal or not, with grouped key/value heads and batches, and
// optionally the query's RMS norm and RoPE applied inside the kernel. Computes what the reference's
// attention_kernel (crates/mmh3-cuda/kernels/attention.cu:62-381) computes, with another design. The
// instance the DiT uses (BF16, heads of 128, no mask, no query transform) is the one the benchmark
// times; the others are the same template for the text encoder and the VAE decoder.
//
// A CTA owns two tiles of 128 query rows of one head and walks the keys in blocks of 128.
//
// - Warp 8 (one thread) streams the tiles with TMA into 128-byte-swizzled shared memory: the two
//   query tiles once, then K0, V0, K1, V1, ... through a ring of five stages (32 KiB each for heads
//   of 128).
// - Warp 9 (one thread) issues the tcgen05 MMAs. S = Q K^T (128 x 128, FP32) of each query tile
//   lands in tensor memory; O += P V accumulates there too, with P read from tensor memory. The
//   two query tiles alternate, so the tensor cores work on one while the softmax of the other runs.
// - Warps 0-3 and 4-7 are the softmax of tile 0 and tile 1, one thread per query row (a row is one
//   TMEM lane, so no reduction crosses threads). A thread reads its row of S, keeps the running
//   maximum and sum, writes P in the element type over the first half of the S columns it has just
//   read, and rescales its row of O only when the maximum has grown by more than 2^8, which the
//   final division by the row sum makes exact again. With a query transform, the same eight warps
//   first normalize and rotate the query tiles where TMA left them.
//
// Tensor memory: S0 | S1 | O0 | O1, S 128 columns each and O one column per head dimension.
#include <cfloat>
#include <cmath>

#include "common.cuh"
#include "sm100.cuh"

namespace mmh3 {

namespace {

using namespace sm100;

constexpr int TILE_M = 128;                   // query rows per tile, one per TMEM lane
constexpr int QUERY_TILES = 2;                // query tiles per CTA
constexpr int TILE_N = 128;                   // keys per block
constexpr int STAGES = 5;                     // ring of K and V tiles
constexpr int SLAB_BYTES = 128 * 128;         // 128 rows of 64 16-bit elements
constexpr int SOFTMAX_WARPS = 4 * QUERY_TILES;
constexpr int LOAD_WARP = SOFTMAX_WARPS;
constexpr int MMA_WARP = SOFTMAX_WARPS + 1;
// Warps 10 and 11 only fill the third warpgroup, whose registers go to the softmax warps.
constexpr int THREADS = (SOFTMAX_WARPS + 4) * 32;
constexpr int SOFTMAX_REGISTERS = 208;
constexpr int OTHER_REGISTERS = 88;
// setmaxnreg.inc blocks until the CTA's own pool holds the registers it asks for, and only what the
// CTA's warps have given back with setmaxnreg.dec goes into that pool: what the third warpgroup
// releases from the 168 registers per thread the kernel launches with must cover what the two
// softmax warpgroups take, or the kernel never gets past the increase.
constexpr int LAUNCH_REGISTERS = 168;
static_assert((LAUNCH_REGISTERS - OTHER_REGISTERS) * 128 >=
                  (SOFTMAX_REGISTERS - LAUNCH_REGISTERS) * SOFTMAX_WARPS * 32,
              "the softmax warps ask for more registers than the other warps release");

// Shared memory for heads of DIM (64 or 128): a tile of 128 rows is one slab of 64 columns per 64
// dimensions.
template <int DIM> struct Shape {
    static constexpr int SLABS = DIM / 64;
    static constexpr int TILE_BYTES = SLABS * SLAB_BYTES;
    static constexpr int SMEM_QUERY = 0;
    static constexpr int SMEM_RING = QUERY_TILES * TILE_BYTES;
    static constexpr int SMEM_BARRIERS = SMEM_RING + STAGES * TILE_BYTES;
    // Barriers, then the TMEM base address and the abort flag. The extra 1024 bytes align the tiles.
    static constexpr int SMEM_BYTES = SMEM_BARRIERS + 256 + 1024;
};

enum Barrier {
    QUERY_FULL = 0,
    RING_FULL = 1,
    RING_EMPTY = RING_FULL + STAGES,
    SCORES_FULL = RING_EMPTY + STAGES,               // one per query tile
    PROBABILITIES_FULL = SCORES_FULL + QUERY_TILES,  // one per query tile
    OUTPUT_FULL = PROBABILITIES_FULL + QUERY_TILES,
    QUERY_READY = OUTPUT_FULL + 1,                   // the query tiles are normalized and rotated
    PROBABILITIES_HALF = QUERY_READY + 1,            // one per query tile: the first 64 keys' P
    BARRIERS = PROBABILITIES_HALF + QUERY_TILES,
};
static_assert(BARRIERS * 8 + 8 <= 256, "the barriers outgrew their corner of shared memory");

constexpr uint32_t TMEM_COLUMNS = 512;
constexpr uint32_t TMEM_SCORES = 0;    // + tile * 128
constexpr uint32_t TMEM_OUTPUT = 256;  // + tile * head dimension

// The 16-bit element of q, k, v, P and the output: BF16, or FP16 (`HALF`).
template <bool HALF, int DIM = 128> struct Element {
    static constexpr uint32_t FORMAT = HALF ? FORMAT_F16 : FORMAT_BF16;
    static constexpr uint32_t SCORE_MMA =
        instruction_descriptor(ACCUMULATE_F32, FORMAT, FORMAT, 0, 0, TILE_M, TILE_N);
    static constexpr uint32_t OUTPUT_MMA =
        instruction_descriptor(ACCUMULATE_F32, FORMAT, FORMAT, 0, 1, TILE_M, DIM);
    static __device__ __forceinline__ float to_float(uint16_t bits) {
        if constexpr (HALF) {
            return __half2float(__ushort_as_half(bits));
        } else {
            return __uint_as_float(static_cast<uint32_t>(bits) << 16);
        }
    }
    static __device__ __forceinline__ uint16_t from_float(float value) {
        if constexpr (HALF) {
            return __half_as_ushort(__float2half_rn(value));
        } else {
            return __bfloat16_as_ushort(__float2bfloat16_rn(value));
        }
    }
    // Two FP32 values rounded to nearest even and packed, the first in the low half.
    static __device__ __forceinline__ uint32_t pack(float low, float high) {
        if constexpr (HALF) {
            uint32_t packed;
            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(high), "f"(low));
            return packed;
        } else {
            return pack_bf16(low, high);
        }
    }
};

// The maximum may lag the true row maximum by this much (in log2 units) before O is rescaled.
constexpr float RESCALE_THRESHOLD = 8.0f;
// Of every four pairs of probabilities, how many take the polynomial exp2 instead of the MUFU.
// One in four costs fewer cycles a block (3,466 against 3,543) and more power: over the twenty
// launches of a benchmark run the GPU sits at its power cap, where none in four runs at 1,627 MHz
// instead of 1,582 and is the faster by 0.6 % (2 % in the token attention over routes).
constexpr int POLYNOMIAL_PAIRS_OF_4 = 0;

struct DenseMaps {
    CUtensorMap query;
    CUtensorMap key;
    CUtensorMap value;
};

// The RMS norm and rotary embedding the VAE decoder's query takes inside the attention
// (crates/mmh3-cuda/kernels/attention.cu:49-111): angles [tokens, pairs], dimension p pairs with
// p + pairs.
struct QueryRope {
    const float *angles;
    int pairs;
    float epsilon;
};

// K-major descriptor of a Q or K tile, and the byte offset of contraction step `step` (16 of the
// 128 dimensions) in it.
__device__ __forceinline__ uint64_t row_operand(uint32_t tile) {
    return smem_descriptor(tile, 16, 1024);
}
__host__ __device__ constexpr uint32_t row_step(int step) {
    return (step / 4) * SLAB_BYTES + (step % 4) * 32;
}

// MN-major descriptor of a V tile (N runs along the rows of both slabs), and the byte offset of
// contraction step `step` (16 of the 128 keys) in it.
__device__ __forceinline__ uint64_t value_operand(uint32_t tile) {
    return smem_descriptor(tile, SLAB_BYTES, 1024);
}
__host__ __device__ constexpr uint32_t value_step(int step) { return step * 16 * 128; }

template <bool HALF, bool CAUSAL, int DIM, bool ROPE>
__global__ void __launch_bounds__(THREADS, 1)
    dense_bf16_kernel(const __grid_constant__ DenseMaps maps, uint16_t *__restrict__ output,
                      int tokens, int heads_per_key_value, int64_t output_token_stride,
                      int64_t output_head_stride, int vector_stores, float scale_log2,
                      QueryRope rope, unsigned int *status) {
    constexpr uint32_t SCORE_MMA = Element<HALF, DIM>::SCORE_MMA;
    constexpr uint32_t OUTPUT_MMA = Element<HALF, DIM>::OUTPUT_MMA;
    constexpr int SLABS = Shape<DIM>::SLABS;
    constexpr int TILE_BYTES = Shape<DIM>::TILE_BYTES;
    constexpr int SMEM_QUERY = Shape<DIM>::SMEM_QUERY;
    constexpr int SMEM_RING = Shape<DIM>::SMEM_RING;
    constexpr int SMEM_BARRIERS = Shape<DIM>::SMEM_BARRIERS;
    extern __shared__ uint8_t shared_memory[];
    const uint32_t base = (smem_u32(shared_memory) + 1023u) & ~1023u;
    uint8_t *aligned = shared_memory + (base - smem_u32(shared_memory));
    const uint32_t barriers = base + SMEM_BARRIERS;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + SMEM_BARRIERS +
                                                                         BARRIERS * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const Watchdog watchdog = {abort_flag, status};
    auto barrier = [&](int index) { return barriers + index * 8; };

    // Once a wait has run out anywhere, the rest of the grid drains instead of waiting too.
    if (*reinterpret_cast<volatile unsigned int *>(status) != 0) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int head = blockIdx.y;
    const int first_query = blockIdx.x * (QUERY_TILES * TILE_M);
    // A causal row sees the keys up to its own token: the CTA's two query tiles need the key
    // blocks up to the second tile's diagonal one (the first tile finds its last block all masked).
    const int blocks = CAUSAL ? min((tokens + TILE_N - 1) / TILE_N,
                                    first_query / TILE_N + QUERY_TILES)
                              : (tokens + TILE_N - 1) / TILE_N;

    if (threadIdx.x == 0) {
        mbar_init(barrier(QUERY_FULL), 1);
        for (int stage = 0; stage < STAGES; stage++) {
            mbar_init(barrier(RING_FULL + stage), 1);
            mbar_init(barrier(RING_EMPTY + stage), 1);
        }
        for (int tile = 0; tile < QUERY_TILES; tile++) {
            mbar_init(barrier(SCORES_FULL + tile), 1);
            mbar_init(barrier(PROBABILITIES_FULL + tile), TILE_M);
            mbar_init(barrier(PROBABILITIES_HALF + tile), TILE_M);
        }
        mbar_init(barrier(OUTPUT_FULL), 1);
        mbar_init(barrier(QUERY_READY), SOFTMAX_WARPS * 32);
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
            const int key_value_head = head / heads_per_key_value;
            mbar_expect_tx(barrier(QUERY_FULL), QUERY_TILES * TILE_BYTES);
            for (int tile = 0; tile < QUERY_TILES; tile++) {
                for (int slab = 0; slab < SLABS; slab++) {
                    tma_load_3d(base + SMEM_QUERY + tile * TILE_BYTES + slab * SLAB_BYTES,
                                &maps.query, barrier(QUERY_FULL), slab * 64,
                                first_query + tile * TILE_M, head);
                }
            }
            // K0, V0, K1, V1, ... in the order the MMA warp consumes and releases them.
            for (int item = 0; item < 2 * blocks; item++) {
                const int stage = item % STAGES;
                const int use = item / STAGES;
                if (use > 0 && !mbar_wait(barrier(RING_EMPTY + stage), (use - 1) & 1, watchdog,
                                          STATUS_DENSE | 1)) {
                    break;
                }
                mbar_expect_tx(barrier(RING_FULL + stage), TILE_BYTES);
                const CUtensorMap *map = (item & 1) ? &maps.value : &maps.key;
                for (int slab = 0; slab < SLABS; slab++) {
                    tma_load_3d(base + SMEM_RING + stage * TILE_BYTES + slab * SLAB_BYTES, map,
                                barrier(RING_FULL + stage), slab * 64, (item / 2) * TILE_N,
                                key_value_head);
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
                for (int step = 0; step < DIM / 16; step++) {
                    mma_f16_ss(tmem + TMEM_SCORES + tile * TILE_N,
                               advance_descriptor(query_operands[tile], row_step(step)),
                               advance_descriptor(key_operand, row_step(step)), SCORE_MMA,
                               step > 0);
                }
                tcgen05_commit(barrier(SCORES_FULL + tile));
            };
            auto accumulate = [&](int tile, uint32_t value_tile, bool first, int from, int to) {
                const uint64_t operand = value_operand(value_tile);
                #pragma unroll
                for (int step = from; step < to; step++) {
                    // P is BF16, two to a column: 16 keys are 8 columns.
                    mma_f16_ts(tmem + TMEM_OUTPUT + tile * DIM,
                               tmem + TMEM_SCORES + tile * TILE_N + step * 8,
                               advance_descriptor(operand, value_step(step)), OUTPUT_MMA,
                               !first || step > 0);
                }
            };
            bool alive = mbar_wait(barrier(ROPE ? QUERY_READY : QUERY_FULL), 0, watchdog,
                                   STATUS_DENSE | 2) &&
                         mbar_wait(barrier(RING_FULL + 0), 0, watchdog, STATUS_DENSE | 3);
            if (alive) {
                tcgen05_fence_after();
                score(0, ring);
                score(1, ring);
                tcgen05_commit(barrier(RING_EMPTY + 0));
            }
            int item = 1; // ring position of V of the current block; K of the next follows it
            for (int block = 0; alive && block < blocks; block++, item += 2) {
                const int value_stage = item % STAGES;
                const int key_stage = (item + 1) % STAGES;
                const bool more = block + 1 < blocks;
                alive = mbar_wait(barrier(RING_FULL + value_stage), (item / STAGES) & 1, watchdog,
                                  STATUS_DENSE | 4) &&
                        (!more || mbar_wait(barrier(RING_FULL + key_stage),
                                            ((item + 1) / STAGES) & 1, watchdog,
                                            STATUS_DENSE | 5));
                if (!alive) {
                    break;
                }
                const uint32_t value_tile = ring + value_stage * TILE_BYTES;
                const uint32_t key_tile = ring + key_stage * TILE_BYTES;
                #pragma unroll
                for (int tile = 0; tile < QUERY_TILES; tile++) {
                    // The first 64 keys' probabilities are handed over first: their four MMAs
                    // run while the softmax threads work on the other 64, which takes a quarter
                    // of O += P V out of the chain softmax -> P V -> S of a tile (62.4 -> 60.8 ms).
                    alive = mbar_wait(barrier(PROBABILITIES_HALF + tile), block & 1, watchdog,
                                      STATUS_DENSE | 11);
                    if (!alive) {
                        break;
                    }
                    tcgen05_fence_after();
                    accumulate(tile, value_tile, block == 0, 0, TILE_N / 32);
                    alive = mbar_wait(barrier(PROBABILITIES_FULL + tile), block & 1, watchdog,
                                      STATUS_DENSE | 6);
                    if (!alive) {
                        break;
                    }
                    tcgen05_fence_after();
                    accumulate(tile, value_tile, false, TILE_N / 32, TILE_N / 16);
                    if (tile == QUERY_TILES - 1) {
                        tcgen05_commit(barrier(RING_EMPTY + value_stage));
                    }
                    if (more) {
                        // Issued after the P V that reads the columns it overwrites.
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
        // Softmax of query tile `tile`; this thread owns row `row`, TMEM lane `row`.
        register_increase<SOFTMAX_REGISTERS>();
        const int tile = warp / 4;
        const int row = (warp % 4) * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        const uint32_t scores = tmem + lane_base + TMEM_SCORES + tile * TILE_N;
        const uint32_t accumulator = tmem + lane_base + TMEM_OUTPUT + tile * DIM;
        float maximum = -INFINITY; // of the raw scores, before the scale
        float2 sums[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
        bool alive = true;
        if constexpr (ROPE) {
            // The eight softmax warps normalize and rotate the 256 query rows where TMA left them,
            // a warp to a row: lane l holds dimensions l, l + 32, ... of the row.
            alive = mbar_wait(barrier(QUERY_FULL), 0, watchdog, STATUS_DENSE | 10);
            alive = __all_sync(0xffffffffu, alive);
            constexpr int SLOTS = DIM / 32;
            for (int query_row = warp; alive && query_row < QUERY_TILES * TILE_M;
                 query_row += SOFTMAX_WARPS) {
                const int token = first_query + query_row;
                if (token >= tokens) {
                    continue;
                }
                const int tile_row = query_row % TILE_M;
                uint32_t addresses[SLOTS];
                float values[SLOTS];
                float squares = 0.0f;
                #pragma unroll
                for (int slot = 0; slot < SLOTS; slot++) {
                    const int index = slot * 32 + lane;
                    // 16-byte chunk c of a row sits at chunk c ^ (row % 8) of its 128-byte line.
                    const int chunk = ((index % 64) / 8) ^ (tile_row % 8);
                    addresses[slot] = base + SMEM_QUERY + (query_row / TILE_M) * TILE_BYTES +
                                      (index / 64) * SLAB_BYTES + tile_row * 128 + chunk * 16 +
                                      (index % 8) * 2;
                    uint16_t bits;
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(bits) : "r"(addresses[slot]));
                    values[slot] = Element<HALF, DIM>::to_float(bits);
                    squares = fmaf(values[slot], values[slot], squares);
                }
                #pragma unroll
                for (int offset = 16; offset > 0; offset /= 2) {
                    squares += __shfl_xor_sync(0xffffffffu, squares, offset);
                }
                const float inverse = rsqrtf(squares / DIM + rope.epsilon);
                #pragma unroll
                for (int slot = 0; slot < SLOTS; slot++) {
                    values[slot] *= inverse;
                }
                float rotated[SLOTS];
                #pragma unroll
                for (int slot = 0; slot < SLOTS; slot++) {
                    const int index = slot * 32 + lane;
                    const bool leads = index < rope.pairs;
                    const bool follows = !leads && index < 2 * rope.pairs;
                    const int partner = leads ? index + rope.pairs
                                              : (follows ? index - rope.pairs : index);
                    float other = 0.0f;
                    #pragma unroll
                    for (int source = 0; source < SLOTS; source++) {
                        const float fetched =
                            __shfl_sync(0xffffffffu, values[source], partner % 32);
                        other = source == partner / 32 ? fetched : other;
                    }
                    float result = values[slot];
                    if (leads || follows) {
                        float sine, cosine;
                        sincosf(rope.angles[static_cast<int64_t>(token) * rope.pairs +
                                            (leads ? index : partner)],
                                &sine, &cosine);
                        result = leads ? values[slot] * cosine - other * sine
                                       : other * sine + values[slot] * cosine;
                    }
                    rotated[slot] = result;
                }
                #pragma unroll
                for (int slot = 0; slot < SLOTS; slot++) {
                    const uint16_t bits = Element<HALF, DIM>::from_float(rotated[slot]);
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addresses[slot]), "h"(bits)
                                 : "memory");
                }
            }
            // The MMAs read the tiles through the async proxy.
            fence_proxy_async();
            mbar_arrive(barrier(QUERY_READY));
        }
        for (int block = 0; alive && block < blocks; block++) {
            alive = mbar_wait(barrier(SCORES_FULL + tile), block & 1, watchdog, STATUS_DENSE | 7);
            // The tensor memory accesses below are warp-wide: the warp goes on or leaves as one.
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
            float s[TILE_N];
            #pragma unroll
            for (int index = 0; index < TILE_N; index++) {
                s[index] = __uint_as_float(raw[index / 32][index % 32]);
            }
            // Keys past the last token arrive as zeroes and are masked, and so are, for a causal
            // row, the keys after its own token: `valid` keys of this block count for this row.
            int valid = tokens - block * TILE_N;
            if constexpr (CAUSAL) {
                valid = min(valid, first_query + tile * TILE_M + row - block * TILE_N + 1);
            }
            if (valid < TILE_N) {
                #pragma unroll
                for (int index = 0; index < TILE_N; index++) {
                    if (index >= valid) {
                        s[index] = -INFINITY;
                    }
                }
            }
            float partial[4] = {s[0], s[1], s[2], s[3]};
            #pragma unroll
            for (int index = 4; index < TILE_N; index++) {
                partial[index % 4] = fmaxf(partial[index % 4], s[index]);
            }
            const float block_maximum =
                fmaxf(fmaxf(partial[0], partial[1]), fmaxf(partial[2], partial[3]));
            if (block == 0) {
                maximum = block_maximum;
            } else {
                const bool grown = (block_maximum - maximum) * scale_log2 > RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffu, grown)) {
                    // S(block) being complete means P V of the block before is too, so O is
                    // at rest until this thread hands over P.
                    const float raised = fmaxf(maximum, block_maximum);
                    const float correction = exp2_approx((maximum - raised) * scale_log2);
                    maximum = raised;
                    const float2 correction2 = make_float2(correction, correction);
                    sums[0] = __fmul2_rn(sums[0], correction2);
                    sums[1] = __fmul2_rn(sums[1], correction2);
                    #pragma unroll
                    for (int chunk = 0; chunk < DIM / 32; chunk++) {
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
            }
            // p = 2^(s * scale - maximum * scale), two elements at a time, on the MUFU (or a share
            // of the pairs on the FMA pipe's polynomial, see POLYNOMIAL_PAIRS_OF_4).
            const float offset = maximum * scale_log2;
            const float2 scale2 = make_float2(scale_log2, scale_log2);
            const float2 offset2 = make_float2(-offset, -offset);
            #pragma unroll
            for (int chunk = 0; chunk < 2; chunk++) {
                uint32_t packed[32];
                #pragma unroll
                for (int pair = 0; pair < 32; pair++) {
                    const int index = chunk * 64 + pair * 2;
                    const float2 x =
                        __ffma2_rn(make_float2(s[index], s[index + 1]), scale2, offset2);
                    float2 probability;
                    if (pair % 4 < POLYNOMIAL_PAIRS_OF_4) {
                        probability = exp2_polynomial(x);
                    } else {
                        probability = make_float2(exp2_approx(x.x), exp2_approx(x.y));
                    }
                    sums[pair % 2] = __fadd2_rn(sums[pair % 2], probability);
                    packed[pair] = Element<HALF, DIM>::pack(probability.x, probability.y);
                }
                tmem_store_32(scores + chunk * 32, packed);
                if (chunk == 0) {
                    tmem_wait_store();
                    tcgen05_fence_before();
                    mbar_arrive(barrier(PROBABILITIES_HALF + tile));
                }
            }
            tmem_wait_store();
            tcgen05_fence_before();
            mbar_arrive(barrier(PROBABILITIES_FULL + tile));
        }
        if (alive) {
            alive = mbar_wait(barrier(OUTPUT_FULL), 0, watchdog, STATUS_DENSE | 8);
            alive = __all_sync(0xffffffffu, alive);
        }
        if (alive) {
            tcgen05_fence_after();
            const float inverse = 1.0f / ((sums[0].x + sums[0].y) + (sums[1].x + sums[1].y));
            const int token = first_query + tile * TILE_M + row;
            uint16_t *output_row = output + static_cast<int64_t>(token) * output_token_stride +
                                   static_cast<int64_t>(head) * output_head_stride;
            #pragma unroll
            for (int chunk = 0; chunk < DIM / 32; chunk++) {
                uint32_t values[32];
                tmem_load_32(accumulator + chunk * 32, values);
                tmem_wait_load();
                if (token < tokens) {
                    uint32_t packed[16];
                    #pragma unroll
                    for (int pair = 0; pair < 16; pair++) {
                        packed[pair] =
                            Element<HALF, DIM>::pack(__uint_as_float(values[pair * 2]) * inverse,
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
            // Give what is still in flight time to land before the columns go back.
            for (int spin = 0; spin < 64; spin++) {
                __nanosleep(1000);
            }
        }
        tcgen05_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
}

bool encode_operand(CUtensorMap *map, bool half, int head_dim, const void *base, int tokens,
                    int heads, int64_t token_stride, int64_t head_stride) {
    const uint64_t dimensions[3] = {static_cast<uint64_t>(head_dim), static_cast<uint64_t>(tokens),
                                    static_cast<uint64_t>(heads)};
    uint64_t strides[2] = {static_cast<uint64_t>(token_stride) * 2,
                           static_cast<uint64_t>(head_stride) * 2};
    if (heads == 1 && strides[1] == 0) {
        // A dimension of one never uses its stride, but the encoder rejects zero.
        strides[1] = strides[0] * static_cast<uint64_t>(tokens);
    }
    const uint32_t box[3] = {64, TILE_M, 1};
    return encode_tensor_map(
        map, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base,
        dimensions, strides, box);
}

// The kernel instance for an element type, mask, head dimension and query transform, and its
// shared memory.
struct Instance {
    void (*kernel)(const DenseMaps, uint16_t *, int, int, int64_t, int64_t, int, float, QueryRope,
                   unsigned int *);
    int shared_bytes;
};

template <bool HALF, bool CAUSAL, int DIM> Instance instance(bool rope) {
    return {rope ? dense_bf16_kernel<HALF, CAUSAL, DIM, true>
                 : dense_bf16_kernel<HALF, CAUSAL, DIM, false>,
            Shape<DIM>::SMEM_BYTES};
}

template <bool HALF, bool CAUSAL> Instance instance(int head_dim, bool rope) {
    return head_dim == 64 ? instance<HALF, CAUSAL, 64>(rope) : instance<HALF, CAUSAL, 128>(rope);
}

} // namespace

int launch_dense_bf16(const void *query, const void *key, const void *value, void *output,
                      int tokens, int heads, int batch, const Mmh3AttentionLayout &layout,
                      float scale, cudaStream_t stream, bool half, int head_dim,
                      const float *angles, int pairs, float epsilon) {
    const int group = layout.heads_per_key_value > 0 ? layout.heads_per_key_value : 1;
    if (!(scale > 0.0f) || !std::isfinite(scale)) {
        return INVALID_VALUE;
    }
    if ((head_dim != 64 && head_dim != 128) ||
        (angles != nullptr && (pairs < 0 || 2 * pairs > head_dim))) {
        return INVALID_VALUE;
    }
    for (int operand = 0; operand < 4; operand++) {
        if (layout.token_stride[operand] <= 0 || layout.head_stride[operand] < 0) {
            return INVALID_VALUE;
        }
    }
    unsigned int *status = status_pointer();
    if (status == nullptr) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    const bool causal = layout.causal != 0;
    const bool rope = angles != nullptr;
    const Instance chosen =
        half ? (causal ? instance<true, true>(head_dim, rope) : instance<true, false>(head_dim, rope))
             : (causal ? instance<false, true>(head_dim, rope)
                       : instance<false, false>(head_dim, rope));
    static SharedMemoryOptIn shared_memory[16];
    const int index = (half ? 8 : 0) + (causal ? 4 : 0) + (head_dim == 64 ? 2 : 0) + (rope ? 1 : 0);
    const cudaError_t configured = shared_memory[index].ensure(chosen.kernel, chosen.shared_bytes);
    if (configured != cudaSuccess) {
        return static_cast<int>(configured);
    }
    const QueryRope query_rope = {angles, pairs, epsilon};
    // Both element types are 16 bits wide: the strides are in elements either way.
    const auto *q = static_cast<const uint16_t *>(query);
    const auto *k = static_cast<const uint16_t *>(key);
    const auto *v = static_cast<const uint16_t *>(value);
    auto *out = static_cast<uint16_t *>(output);
    for (int item = 0; item < batch; item++) {
        const uint16_t *batch_query = q + item * layout.batch_stride[QUERY];
        const uint16_t *batch_key = k + item * layout.batch_stride[KEY];
        const uint16_t *batch_value = v + item * layout.batch_stride[VALUE];
        uint16_t *batch_output = out + item * layout.batch_stride[OUTPUT];
        // Operands off TMA's 16-byte grid go through a dense copy first; the DiT's never do.
        StagedOperands staged(stream);
        const uint16_t *bases[3] = {batch_query, batch_key, batch_value};
        int64_t token_strides[3], head_strides[3];
        for (int operand = 0; operand < 3; operand++) {
            token_strides[operand] = layout.token_stride[operand];
            head_strides[operand] = layout.head_stride[operand];
            const cudaError_t copied =
                staged.stage(operand, bases[operand], tokens, operand == QUERY ? heads : heads / group,
                             head_dim, token_strides[operand], head_strides[operand]);
            if (copied != cudaSuccess) {
                return static_cast<int>(copied);
            }
        }
        DenseMaps maps;
        if (!encode_operand(&maps.query, half, head_dim, bases[QUERY], tokens, heads,
                            token_strides[QUERY], head_strides[QUERY]) ||
            !encode_operand(&maps.key, half, head_dim, bases[KEY], tokens, heads / group,
                            token_strides[KEY], head_strides[KEY]) ||
            !encode_operand(&maps.value, half, head_dim, bases[VALUE], tokens, heads / group,
                            token_strides[VALUE], head_strides[VALUE])) {
            return NOT_SUPPORTED;
        }
        const int vector_stores = reinterpret_cast<uintptr_t>(batch_output) % 16 == 0 &&
                                  layout.token_stride[OUTPUT] % 8 == 0 &&
                                  layout.head_stride[OUTPUT] % 8 == 0;
        const dim3 grid((tokens + QUERY_TILES * TILE_M - 1) / (QUERY_TILES * TILE_M), heads);
        chosen.kernel<<<grid, THREADS, chosen.shared_bytes, stream>>>(
            maps, batch_output, tokens, group, layout.token_stride[OUTPUT],
            layout.head_stride[OUTPUT], vector_stores, scale * LOG2_E, query_rope, status);
        const cudaError_t launched = cudaGetLastError();
        if (launched != cudaSuccess) {
            return static_cast<int>(launched);
        }
    }
    return 0;
}

} // namespace mmh3
