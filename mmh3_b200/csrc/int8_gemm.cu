// The scaled INT8 GEMM of the DiT's linear layers, as the step before attention uses it: the fused
// qkv projection, which also leaves the maximum |v| of each head for the FP8 quantisation of V.
//
//   output[r, c] = round((sum_k activations[r, k] * weights[c, k]) * activation_scales[r]
//                        * weight_scales[c]
//                        + adapter_scale * sum_j adapter_down[r, j] * adapter_up[c, j] + bias[c])
//
// rounded once to BF16 or FP16, activations [m, k] and weights [n, k] INT8 with K contiguous, the
// low-rank adapter (BF16) and the bias optional. It replaces
// crates/mmh3-cuda/kernels/int8_gemm.cu:321-591 (mma.sync over a two-stage ring) and keeps its
// arithmetic: the integer sums are exact, and the FP32 operations after them are the
// same in the same order, so without an adapter the outputs and the column maxima are the same
// bits. With an adapter a tile is 128 rows: its INT32 accumulator and an FP32 accumulator for
// down . up^T sit side by side in tensor memory, and after the K blocks the ring carries blocks of
// 64 ranks of the two BF16 operands, in the same 128-byte rows, for kind::f16 MMAs. Those sums
// come in the tensor cores' own order, so that result is held to the reference's bounds instead.
//
// One persistent CTA per SM walks tiles of 256 rows by 256 columns in bands of rows of tiles, so
// the CTAs in flight share rows of activations and columns of weights in L2. A tile is two
// accumulators of 128 rows by 256 columns of INT32 in tensor memory (all 512 columns of the SM).
// Warp 0 streams stages of 128 bytes of K (32 KB of activations, 32 KB of weights, 128-byte
// swizzle) through a ring of three with TMA; one thread of warp 1 issues tcgen05.mma kind::i8 of
// 128 x 256 x 32 from shared memory; eight warps scale and round the accumulators, turn their rows
// around in a staging tile of shared memory so that the stores cover whole 128-byte runs, and give
// tensor memory back as soon as the last columns are in registers, while the ring fills for the
// next tile. At this tile shape a stage of 64 KB feeds 1,024 cycles of MMA, 64 bytes a cycle,
// which is what an SM can take from L2; a tile of 128 x 256 would leave room for a second pair of
// accumulators and an epilogue hidden behind the next tile's MMAs, but needs 96 bytes a cycle.
#include "common.cuh"
#include "sm100.cuh"

#include <cuda_fp16.h>

namespace mmh3 {
namespace {

using namespace sm100;

constexpr int TILE_M = 128;     // rows of one accumulator
constexpr int TILE_N = 256;
constexpr int BLOCK_K = 128;    // bytes of one stage along K: 128 INT8 values, 64 BF16 ranks
constexpr int COLUMNS_BYTES = TILE_N * BLOCK_K;
// Where an epilogue warp turns its 32 rows of 64 columns around for the stores.
constexpr int STAGING_ROW = 128;
constexpr int STAGING_BYTES = 32 * STAGING_ROW;
constexpr int EPILOGUE_WARPS = 8;
constexpr int MAX_STAGES = 4;

// Without a low-rank adapter a tile is 256 rows: two INT32 accumulators fill tensor memory. With
// one it is 128 rows: one INT32 accumulator, and one FP32 accumulator for down . up^T beside it.
template <bool ADAPTED> struct Shape {
    static constexpr int ROW_TILES = ADAPTED ? 1 : 2;
    static constexpr int STAGES = ADAPTED ? 4 : 3;
    static constexpr int ROWS_BYTES = ROW_TILES * TILE_M * BLOCK_K;
    static constexpr int STAGE_BYTES = ROWS_BYTES + COLUMNS_BYTES;
    static constexpr int SMEM_BYTES =
        STAGES * STAGE_BYTES + EPILOGUE_WARPS * STAGING_BYTES + 1024;
    static_assert(STAGES <= MAX_STAGES, "more stages than barriers");
    static_assert(SMEM_BYTES + 256 <= 227 * 1024, "ring, staging and barriers exceed an SM");
};

constexpr int LOAD_WARP = 0;
constexpr int MMA_WARP = 1;
constexpr int FIRST_EPILOGUE_WARP = 2;
constexpr int THREADS = (FIRST_EPILOGUE_WARP + EPILOGUE_WARPS) * 32;
constexpr int TMEM_COLUMNS = 2 * TILE_N;
constexpr uint32_t TMEM_ADAPTER = TILE_N; // the adapter's accumulator, beside the INT32 one
constexpr int CHUNK = 32; // columns of one tcgen05.ld

constexpr unsigned int STATUS_GEMM = 0x00040000u;

enum Barrier {
    RING_FULL = 0,
    RING_EMPTY = RING_FULL + MAX_STAGES,
    ACCUMULATOR_FULL = RING_EMPTY + MAX_STAGES,
    ACCUMULATOR_EMPTY,
    BARRIERS,
};

constexpr uint32_t PRODUCT_MMA =
    instruction_descriptor(ACCUMULATE_S32, FORMAT_S8, FORMAT_S8, 0, 0, TILE_M, TILE_N);

constexpr uint32_t ADAPTER_MMA =
    instruction_descriptor(ACCUMULATE_F32, FORMAT_BF16, FORMAT_BF16, 0, 0, TILE_M, TILE_N);

struct GemmMaps {
    CUtensorMap activations;  // [m, k] INT8
    CUtensorMap weights;      // [n, k] INT8
    CUtensorMap adapter_down; // [m, rank] BF16, rows down_stride apart
    CUtensorMap adapter_up;   // [n, rank] BF16
};

struct TileWalk {
    int tiles_m;
    int tiles_n;
    int band;

    __device__ int tiles() const { return tiles_m * tiles_n; }

    // Down a band of `band` rows of tiles, then one column of tiles to the right.
    __device__ void locate(int tile, int &tile_m, int &tile_n) const {
        const int band_tiles = band * tiles_n;
        const int band_first = tile / band_tiles * band;
        const int height = min(band, tiles_m - band_first);
        const int within = tile - tile / band_tiles * band_tiles;
        tile_m = band_first + within % height;
        tile_n = within / height;
    }
};

__device__ __forceinline__ uint32_t pack(__nv_bfloat16 *, float2 pair) {
    return pack_bf16(pair.x, pair.y);
}

__device__ __forceinline__ uint32_t pack(__half *, float2 pair) {
    const __half2 value = __floats2half2_rn(pair.x, pair.y);
    return *reinterpret_cast<const uint32_t *>(&value);
}

__device__ __forceinline__ float2 unpack(__nv_bfloat16 *, uint32_t word) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&word));
}

__device__ __forceinline__ float2 unpack(__half *, uint32_t word) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&word));
}

// silu(gate) * up of two features from their rounded products, rounded again, as
// crates/mmh3-cuda/kernels/int8_gemm.cu:297-305 computes it.
template <typename Output>
__device__ __forceinline__ uint32_t gated_pair(Output *output, uint32_t gate_word,
                                               uint32_t up_word) {
    const float2 gate = unpack(output, gate_word);
    const float2 up = unpack(output, up_word);
    return pack(output, make_float2(gate.x / (1.0f + __expf(-gate.x)) * up.x,
                                    gate.y / (1.0f + __expf(-gate.y)) * up.y));
}

template <typename Output, bool SWIGLU, bool ADAPTED>
__global__ void __launch_bounds__(THREADS, 1)
    int8_gemm_kernel(const __grid_constant__ GemmMaps maps,
                     const float *__restrict__ activation_scales,
                     const float *__restrict__ weight_scales, const float *__restrict__ bias,
                     Output *__restrict__ output, int m, int n, int k_blocks, int output_stride,
                     TileWalk walk, unsigned *maxima, int maxima_first_column,
                     int adapter_blocks, float adapter_scale, unsigned int *status) {
    constexpr int ROW_TILES = Shape<ADAPTED>::ROW_TILES;
    constexpr int STAGES = Shape<ADAPTED>::STAGES;
    constexpr int ROWS_BYTES = Shape<ADAPTED>::ROWS_BYTES;
    constexpr int STAGE_BYTES = Shape<ADAPTED>::STAGE_BYTES;
    extern __shared__ uint8_t shared_raw[];
    __shared__ __align__(8) uint64_t barriers[BARRIERS];
    __shared__ uint32_t tmem_slot_storage;
    __shared__ uint32_t abort_storage;
    const uint32_t base = (smem_u32(shared_raw) + 1023u) & ~1023u;
    volatile uint32_t *abort_flag = &abort_storage;
    volatile uint32_t *tmem_slot = &tmem_slot_storage;
    const Watchdog watchdog{abort_flag, status};
    auto barrier = [&](int index) { return smem_u32(&barriers[index]); };
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int tiles = walk.tiles();

    if (threadIdx.x == 0) {
        for (int stage = 0; stage < STAGES; stage++) {
            mbar_init(barrier(RING_FULL + stage), 1);
            mbar_init(barrier(RING_EMPTY + stage), 1);
        }
        mbar_init(barrier(ACCUMULATOR_FULL), 1);
        mbar_init(barrier(ACCUMULATOR_EMPTY), EPILOGUE_WARPS);
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

    if (warp == LOAD_WARP) {
        if (lane == 0) {
            tma_prefetch_descriptor(&maps.activations);
            tma_prefetch_descriptor(&maps.weights);
            if constexpr (ADAPTED) {
                tma_prefetch_descriptor(&maps.adapter_down);
                tma_prefetch_descriptor(&maps.adapter_up);
            }
            int item = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < tiles; tile += gridDim.x) {
                int tile_m, tile_n;
                walk.locate(tile, tile_m, tile_n);
                // The K blocks of the INT8 operands, then the adapter's blocks of 64 ranks: the
                // same 128-byte rows in the same places.
                for (int block = 0; block < k_blocks + adapter_blocks; block++, item++) {
                    const int stage = item % STAGES;
                    const int use = item / STAGES;
                    if (use > 0 && !mbar_wait(barrier(RING_EMPTY + stage), (use - 1) & 1,
                                              watchdog, STATUS_GEMM | 1)) {
                        alive = false;
                        break;
                    }
                    const uint32_t destination = base + stage * STAGE_BYTES;
                    const bool adapter = block >= k_blocks;
                    // Coordinates are in elements: bytes for INT8, BF16 values for the adapter.
                    const int along = adapter ? (block - k_blocks) * (BLOCK_K / 2) : block * BLOCK_K;
                    mbar_expect_tx(barrier(RING_FULL + stage), STAGE_BYTES);
                    tma_load_2d(destination, adapter ? &maps.adapter_down : &maps.activations,
                                barrier(RING_FULL + stage), along, tile_m * (ROW_TILES * TILE_M));
                    tma_load_2d(destination + ROWS_BYTES,
                                adapter ? &maps.adapter_up : &maps.weights,
                                barrier(RING_FULL + stage), along, tile_n * TILE_N);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // The MMAs of one accumulator over one stage: four steps of 32 along K.
            auto multiply = [&](int half, int stage, bool first) {
                const uint32_t stage_base = base + stage * STAGE_BYTES;
                const uint64_t rows =
                    smem_descriptor(stage_base + half * (TILE_M * BLOCK_K), 16, 1024);
                const uint64_t columns = smem_descriptor(stage_base + ROWS_BYTES, 16, 1024);
                #pragma unroll
                for (int step = 0; step < BLOCK_K / 32; step++) {
                    mma_i8_ss(tmem + half * TILE_N, advance_descriptor(rows, step * 32),
                              advance_descriptor(columns, step * 32), PRODUCT_MMA,
                              !first || step > 0);
                }
            };
            // down . up^T over one stage of 64 ranks: four steps of 16 BF16 values along K.
            auto adapt = [&](int stage, bool first) {
                const uint32_t stage_base = base + stage * STAGE_BYTES;
                const uint64_t rows = smem_descriptor(stage_base, 16, 1024);
                const uint64_t columns = smem_descriptor(stage_base + ROWS_BYTES, 16, 1024);
                #pragma unroll
                for (int step = 0; step < BLOCK_K / 32; step++) {
                    mma_f16_ss(tmem + TMEM_ADAPTER, advance_descriptor(rows, step * 32),
                               advance_descriptor(columns, step * 32), ADAPTER_MMA,
                               !first || step > 0);
                }
            };
            int item = 0;
            int round = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < tiles; tile += gridDim.x, round++) {
                for (int block = 0; block < k_blocks + adapter_blocks; block++, item++) {
                    const int stage = item % STAGES;
                    alive = mbar_wait(barrier(RING_FULL + stage), (item / STAGES) & 1, watchdog,
                                      STATUS_GEMM | 2);
                    if (alive && block == 0 && round > 0) {
                        // The epilogue warps have read the last tile out of both accumulators.
                        alive = mbar_wait(barrier(ACCUMULATOR_EMPTY), (round - 1) & 1, watchdog,
                                          STATUS_GEMM | 3);
                    }
                    if (!alive) {
                        break;
                    }
                    tcgen05_fence_after();
                    if (ADAPTED && block >= k_blocks) {
                        adapt(stage, block == k_blocks);
                    } else {
                        #pragma unroll
                        for (int half = 0; half < ROW_TILES; half++) {
                            multiply(half, stage, block == 0);
                        }
                    }
                    tcgen05_commit(barrier(RING_EMPTY + stage));
                }
                if (alive) {
                    tcgen05_commit(barrier(ACCUMULATOR_FULL));
                }
            }
        }
    } else {
        const int epilogue_warp = warp - FIRST_EPILOGUE_WARP;
        // A warp reads the quarter of the lanes of tensor memory its number selects.
        const int quarter = warp % 4;
        const int column_half = epilogue_warp / 4;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        uint8_t *staging = shared_raw + (base - smem_u32(shared_raw)) + STAGES * STAGE_BYTES +
                           epilogue_warp * STAGING_BYTES;
        int round = 0;
        bool alive = true;
        for (int tile = blockIdx.x; alive && tile < tiles; tile += gridDim.x, round++) {
            int tile_m, tile_n;
            walk.locate(tile, tile_m, tile_n);
            // The warp's 128 columns lie in one group of 128.
            const int first_column = tile_n * TILE_N + column_half * (TILE_N / 2);
            const bool inside = first_column < n;
            const bool track =
                !SWIGLU && maxima != nullptr && inside && first_column >= maxima_first_column;
            // While the MMAs run: this warp's column scales, bias and row scales into L1.
            if (inside) {
                const int line = lane % 4;
                const void *wanted = nullptr;
                if (lane < 4) {
                    wanted = weight_scales + first_column + line * 32;
                } else if (lane < 8 && bias != nullptr) {
                    wanted = bias + first_column + line * 32;
                } else if (lane >= 8 && lane < 8 + ROW_TILES) {
                    const int rows = tile_m * (ROW_TILES * TILE_M) + (lane - 8) * TILE_M +
                                     quarter * 32;
                    wanted = rows < m ? activation_scales + rows : nullptr;
                }
                if (wanted != nullptr) {
                    prefetch_l1(wanted);
                }
            }
            alive = mbar_wait(barrier(ACCUMULATOR_FULL), round & 1, watchdog, STATUS_GEMM | 4);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) {
                break;
            }
            tcgen05_fence_after();
            auto accumulator = [&](int half, int chunk) {
                return tmem + lane_base + half * TILE_N + column_half * (TILE_N / 2) +
                       chunk * CHUNK;
            };
            // Two buffers take turns: the load of the next 32 columns is in flight while these
            // are scaled. tcgen05.wait::ld waits for every load, so the next one is issued right
            // after it.
            uint32_t even[CHUNK], odd[CHUNK];
            if constexpr (!ADAPTED) {
                tmem_load_32(accumulator(0, 0), even);
            }
            // adapter_scale * (down . up^T) joins the scaled product as the reference adds it:
            // (product / adapter_scale + down . up^T) * adapter_scale
            // (crates/mmh3-cuda/kernels/int8_gemm.cu:461-487).
            const float inverse_adapter_scale = ADAPTED ? 1.0f / adapter_scale : 0.0f;
            const float2 inverse_adapter_scales =
                make_float2(inverse_adapter_scale, inverse_adapter_scale);
            const float2 adapter_scales = make_float2(adapter_scale, adapter_scale);
            #pragma unroll 1
            for (int half = 0; half < ROW_TILES; half++) {
                const int first_row =
                    tile_m * (ROW_TILES * TILE_M) + half * TILE_M + quarter * 32;
                const int row = first_row + lane;
                // Nothing of these rows and columns exists: the whole warp only drains.
                const bool idle = !inside || first_row >= m;
                const float row_scale = row < m ? __ldg(activation_scales + row) : 0.0f;
                const float2 row_scales = make_float2(row_scale, row_scale);
                uint32_t magnitudes = 0;

                // Scales, rounds and stages 32 columns of the lane's row.
                auto scale = [&](const uint32_t (&products)[CHUNK],
                                 const uint32_t (&low_rank)[CHUNK], int chunk) {
                    const int column = first_column + chunk * CHUNK;
                    const float2 *column_scales =
                        reinterpret_cast<const float2 *>(weight_scales + column);
                    const float2 *column_bias = reinterpret_cast<const float2 *>(bias + column);
                    uint32_t words[CHUNK / 2];
                    #pragma unroll
                    for (int pair = 0; pair < CHUNK / 2; pair++) {
                        float2 scaled = make_float2(
                            static_cast<float>(static_cast<int32_t>(products[pair * 2])),
                            static_cast<float>(static_cast<int32_t>(products[pair * 2 + 1])));
                        scaled = __fmul2_rn(__fmul2_rn(scaled, row_scales),
                                            __ldg(column_scales + pair));
                        if constexpr (ADAPTED) {
                            const float2 added = make_float2(__uint_as_float(low_rank[pair * 2]),
                                                             __uint_as_float(low_rank[pair * 2 + 1]));
                            scaled = __fmul2_rn(
                                __fadd2_rn(__fmul2_rn(scaled, inverse_adapter_scales), added),
                                adapter_scales);
                        }
                        if (bias != nullptr) {
                            scaled = __fadd2_rn(scaled, __ldg(column_bias + pair));
                        }
                        words[pair] = pack(output, scaled);
                    }
                    if (track && row < m) {
                        // Magnitudes of BF16 values order like unsigned integers.
                        #pragma unroll
                        for (int pair = 0; pair < CHUNK / 2; pair++) {
                            magnitudes = __vmaxu2(magnitudes, words[pair] & 0x7fff7fffu);
                        }
                    }
                    // The lane's row goes to the warp's staging tile, 16 bytes at a time, at
                    // positions swizzled by the row so that neither these stores nor the loads
                    // of `store_rows` meet in a bank.
                    const int part = chunk % 2;
                    if constexpr (SWIGLU) {
                        // Eight columns hold the gates of four features, then their up
                        // projections: four outputs, 8 bytes.
                        #pragma unroll
                        for (int group = 0; group < CHUNK / 8; group += 2) {
                            const int slot = part * 2 + group / 2;
                            *reinterpret_cast<uint4 *>(staging + lane * STAGING_ROW +
                                                       ((slot ^ (lane & 7)) << 4)) =
                                make_uint4(
                                    gated_pair(output, words[group * 4], words[group * 4 + 2]),
                                    gated_pair(output, words[group * 4 + 1], words[group * 4 + 3]),
                                    gated_pair(output, words[group * 4 + 4], words[group * 4 + 6]),
                                    gated_pair(output, words[group * 4 + 5], words[group * 4 + 7]));
                        }
                    } else {
                        #pragma unroll
                        for (int group = 0; group < CHUNK / 8; group++) {
                            const int slot = part * 4 + group;
                            *reinterpret_cast<uint4 *>(staging + lane * STAGING_ROW +
                                                       ((slot ^ (lane & 7)) << 4)) =
                                make_uint4(words[group * 4], words[group * 4 + 1],
                                           words[group * 4 + 2], words[group * 4 + 3]);
                        }
                    }
                };
                // The 64 staged columns back out by rows: a store instruction covers whole
                // 128-byte runs of four rows (64-byte runs of eight with SwiGLU) instead of 16
                // bytes of 32 rows.
                auto store_rows = [&](int chunk) {
                    constexpr int SLOTS = SWIGLU ? 4 : 8; // 16-byte pieces of a staged row
                    constexpr int ROWS_AT_ONCE = 32 / SLOTS;
                    const int column = first_column + chunk * CHUNK;
                    const int slot = lane % SLOTS;
                    __syncwarp();
                    #pragma unroll
                    for (int pass = 0; pass < 32 / ROWS_AT_ONCE; pass++) {
                        const int staged_row = pass * ROWS_AT_ONCE + lane / SLOTS;
                        const uint4 piece = *reinterpret_cast<const uint4 *>(
                            staging + staged_row * STAGING_ROW + ((slot ^ (staged_row & 7)) << 4));
                        if (first_row + staged_row < m) {
                            Output *destination =
                                output +
                                static_cast<size_t>(first_row + staged_row) * output_stride +
                                (SWIGLU ? column / 2 : column) + slot * 8;
                            *reinterpret_cast<uint4 *>(destination) = piece;
                        }
                    }
                    __syncwarp();
                };

                if constexpr (ADAPTED) {
                    // The product and the adapter's sum of the same 32 columns, side by side.
                    #pragma unroll
                    for (int chunk = 0; chunk < TILE_N / 2 / CHUNK; chunk++) {
                        tmem_load_32(accumulator(0, chunk), even);
                        tmem_load_32(accumulator(0, chunk) + TMEM_ADAPTER, odd);
                        tmem_wait_load();
                        if (chunk == TILE_N / 2 / CHUNK - 1) {
                            tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) {
                                mbar_arrive(barrier(ACCUMULATOR_EMPTY));
                            }
                        }
                        if (!idle) {
                            scale(even, odd, chunk);
                            if (chunk % 2 == 1) {
                                store_rows(chunk - 1);
                            }
                        }
                    }
                } else {
                    tmem_wait_load();
                    tmem_load_32(accumulator(half, 1), odd);
                    if (!idle) {
                        scale(even, even, 0);
                    }
                    tmem_wait_load();
                    tmem_load_32(accumulator(half, 2), even);
                    if (!idle) {
                        scale(odd, odd, 1);
                        store_rows(0);
                    }
                    tmem_wait_load();
                    tmem_load_32(accumulator(half, 3), odd);
                    if (!idle) {
                        scale(even, even, 2);
                    }
                    tmem_wait_load();
                    if (half + 1 < ROW_TILES) {
                        tmem_load_32(accumulator(half + 1, 0), even);
                    } else {
                        // Everything is out of tensor memory: the next tile's MMAs may start while
                        // the last columns are scaled and stored.
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive(barrier(ACCUMULATOR_EMPTY));
                        }
                    }
                    if (!idle) {
                        scale(odd, odd, 3);
                        store_rows(2);
                    }
                }
                if (track) {
                    const unsigned magnitude = __reduce_max_sync(
                        0xffffffffu, max(magnitudes & 0xffffu, magnitudes >> 16));
                    if (lane == 0 && magnitude != 0) {
                        // As the FP32 bits of the BF16 magnitude.
                        atomicMax(maxima + (first_column - maxima_first_column) / 128,
                                  magnitude << 16);
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        if (*abort_flag != 0) {
            // A wait gave up: let copies and MMAs in flight land before tensor memory goes back.
            for (int spin = 0; spin < 64; spin++) {
                __nanosleep(1000);
            }
        }
        tcgen05_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
}

template <typename Output, bool SWIGLU, bool ADAPTED>
int launch_kernel(const GemmMaps &maps, const float *activation_scales, const float *weight_scales,
                  const float *bias, Output *output, int m, int n, int k, int output_stride,
                  int band, unsigned *maxima, int maxima_first_column, int rank,
                  float adapter_scale, cudaStream_t stream) {
    unsigned int *status = status_pointer();
    const int processors = multiprocessor_count();
    if (status == nullptr || processors == 0) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    constexpr int SMEM_BYTES = Shape<ADAPTED>::SMEM_BYTES;
    static SharedMemoryOptIn shared_memory;
    const cudaError_t configured =
        shared_memory.ensure(int8_gemm_kernel<Output, SWIGLU, ADAPTED>, SMEM_BYTES);
    if (configured != cudaSuccess) {
        return static_cast<int>(configured);
    }
    constexpr int TILE_ROWS = Shape<ADAPTED>::ROW_TILES * TILE_M;
    TileWalk walk;
    walk.tiles_m = (m + TILE_ROWS - 1) / TILE_ROWS;
    walk.tiles_n = (n + TILE_N - 1) / TILE_N;
    walk.band = band;
    const int64_t tiles = static_cast<int64_t>(walk.tiles_m) * walk.tiles_n;
    if (tiles > INT32_MAX) {
        return INVALID_VALUE;
    }
    const int blocks = tiles < processors ? static_cast<int>(tiles) : processors;
    int8_gemm_kernel<Output, SWIGLU, ADAPTED><<<blocks, THREADS, SMEM_BYTES, stream>>>(
        maps, activation_scales, weight_scales, bias, output, m, n, k / BLOCK_K, output_stride,
        walk, maxima, maxima_first_column, ADAPTED ? rank * 2 / BLOCK_K : 0, adapter_scale,
        status);
    return static_cast<int>(cudaGetLastError());
}

__global__ void interleave_rows_kernel(const uint32_t *__restrict__ source,
                                       uint32_t *__restrict__ destination, int rows,
                                       int row_words) {
    // Eight rows to a group: the gates of features 4g to 4g + 3, then their up projections,
    // which the source keeps in its second half.
    const int row = blockIdx.x;
    const int feature = row / 8 * 4 + row % 4;
    const size_t from = static_cast<size_t>(row % 8 < 4 ? feature : rows / 2 + feature) * row_words;
    const size_t to = static_cast<size_t>(row) * row_words;
    for (int word = threadIdx.x; word < row_words; word += blockDim.x) {
        destination[to + word] = source[from + word];
    }
}

} // namespace

int launch_int8_gemm(int config, int group_m, const int8_t *activations, const int8_t *weights,
                     const float *activation_scales, const float *weight_scales, const float *bias,
                     void *output, bool output_is_f16, bool swiglu, int m, int n, int k,
                     int output_stride, const void *adapter_down, const void *adapter_up, int rank,
                     int adapter_down_stride, float adapter_scale, unsigned *column_maxima,
                     int maxima_first_column, cudaStream_t stream) {
    // crates/mmh3-cuda/kernels/int8_gemm.cu:640-645, 700-712, 720-722: config 0 needs N in
    // multiples of 128 and config 1 of 256; a negative config is the tiling chosen for the shape.
    // Here every config runs the one tiling, whose results do not depend on it.
    // int8_gemm.cu:622-624
    const bool adapted = adapter_down != nullptr && adapter_up != nullptr && adapter_scale != 0.0f;
    if (config > 1 || (config >= 0 && group_m <= 0) || m <= 0 || n <= 0 || k <= 0 ||
        n % (config == 1 ? 256 : 128) != 0 || k % BLOCK_K != 0) {
        return INVALID_VALUE;
    }
    // The adapter comes in blocks of 64 ranks, its down rows at a stride that keeps them 16-byte
    // aligned (int8_gemm.cu:642-644).
    if (adapted && (rank <= 0 || rank * 2 % BLOCK_K != 0 || adapter_down_stride < rank ||
                    adapter_down_stride % 8 != 0)) {
        return INVALID_VALUE;
    }
    if (column_maxima != nullptr &&
        (swiglu || output_is_f16 || maxima_first_column < 0 || maxima_first_column % 128 != 0)) {
        return INVALID_VALUE;
    }
    if (output_stride <= 0) {
        output_stride = swiglu ? n / 2 : n;
    }
    // The epilogue stores 16 bytes at a time (8 with SwiGLU) and reads the scales in pairs.
    if (reinterpret_cast<uintptr_t>(output) % 16 != 0 || output_stride % 8 != 0 ||
        reinterpret_cast<uintptr_t>(weight_scales) % 8 != 0 ||
        reinterpret_cast<uintptr_t>(bias) % 8 != 0) {
        return INVALID_VALUE;
    }
    GemmMaps maps;
    const uint64_t row_dimensions[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
    const uint64_t column_dimensions[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t row_box[2] = {BLOCK_K, static_cast<uint32_t>((adapted ? 1 : 2) * TILE_M)};
    const uint32_t column_box[2] = {BLOCK_K, TILE_N};
    if (!encode_tensor_map(&maps.activations, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, activations,
                           row_dimensions, strides, row_box) ||
        !encode_tensor_map(&maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, weights,
                           column_dimensions, strides, column_box)) {
        return INVALID_VALUE;
    }
    maps.adapter_down = maps.activations;
    maps.adapter_up = maps.weights;
    if (adapted) {
        const uint64_t down_dimensions[2] = {static_cast<uint64_t>(rank), static_cast<uint64_t>(m)};
        const uint64_t up_dimensions[2] = {static_cast<uint64_t>(rank), static_cast<uint64_t>(n)};
        const uint64_t down_strides[1] = {static_cast<uint64_t>(adapter_down_stride) * 2};
        const uint64_t up_strides[1] = {static_cast<uint64_t>(rank) * 2};
        const uint32_t down_box[2] = {BLOCK_K / 2, TILE_M};
        const uint32_t up_box[2] = {BLOCK_K / 2, TILE_N};
        if (!encode_tensor_map(&maps.adapter_down, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                               adapter_down, down_dimensions, down_strides, down_box) ||
            !encode_tensor_map(&maps.adapter_up, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, adapter_up,
                               up_dimensions, up_strides, up_box)) {
            return INVALID_VALUE;
        }
    }
    const int band = config >= 0 ? group_m : 8;
#define MMH3_GEMM(OUTPUT, SWIGLU, ADAPTED)                                                         \
    launch_kernel<OUTPUT, SWIGLU, ADAPTED>(                                                        \
        maps, activation_scales, weight_scales, bias, static_cast<OUTPUT *>(output), m, n, k,      \
        output_stride, band, column_maxima, maxima_first_column, rank, adapter_scale, stream)
#define MMH3_GEMM_OUTPUT(OUTPUT)                                                                   \
    (swiglu ? (adapted ? MMH3_GEMM(OUTPUT, true, true) : MMH3_GEMM(OUTPUT, true, false))           \
            : (adapted ? MMH3_GEMM(OUTPUT, false, true) : MMH3_GEMM(OUTPUT, false, false)))
    return output_is_f16 ? MMH3_GEMM_OUTPUT(__half) : MMH3_GEMM_OUTPUT(__nv_bfloat16);
#undef MMH3_GEMM_OUTPUT
#undef MMH3_GEMM
}

int launch_interleave_swiglu_rows(const void *source, void *destination, int rows, int row_bytes,
                                  cudaStream_t stream) {
    // crates/mmh3-cuda/kernels/int8_gemm.cu:1000-1009
    if (rows % 8 != 0 || row_bytes % 4 != 0 || rows <= 0) {
        return INVALID_VALUE;
    }
    interleave_rows_kernel<<<rows, 128, 0, stream>>>(static_cast<const uint32_t *>(source),
                                                     static_cast<uint32_t *>(destination), rows,
                                                     row_bytes / 4);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mmh3
