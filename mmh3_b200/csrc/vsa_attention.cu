// VSA's token attention on sm_100a: every query tile (a run of up to 64 tokens) attends, token by
// token, to the tiles its route lists, plus gate * coarse when a gate is given. BF16 or INT8/FP8
// operands, FP32 softmax and accumulation, BF16 output. It computes what the reference's VSA
// attention kernels compute (crates/mmh3-cuda/kernels/vsa_attention.cu:304-493 and the VSA pattern
// of quantized_attention.cu:247-549) with another design.
//
// The tcgen05 MMA works on 128 rows, a tile has at most 64, so a CTA takes TWO query tiles of one
// head, A in rows 0-63 and B in rows 64-127, and walks their two route lists in step. At step i
// the key block is the i-th routed tile of A (keys 0-63) next to the i-th routed tile of B (keys
// 64-127), fetched by TMA as two boxes of 64 rows. S = Q K^T then holds the wanted scores on its
// diagonal blocks: a softmax thread (one per row) reads only the 64 columns of its own tile's
// keys, and writes P with zeroes in the other tile's columns, so that O += P V adds nothing across
// the pair. Half of each MMA is spent on the off-diagonal blocks; in exchange every row and every
// softmax thread has work, and the tiles keep their own routes.
//
// Key tiles that BOTH route lists hold are taken first, one to a step, for both query tiles at
// once: S is then 128 rows by that tile's 64 keys and nothing of the MMAs is wasted. The CTA finds
// them with one bit per tile and list in shared memory; every role (loader, MMA issuer, softmax
// threads) walks the same schedule from the two lists and the two bitmaps.
//
// Rows of a box past a tile's length belong to the next tile (or are zero past the sequence):
// their scores are masked and their probabilities are zero. A list that ends before its
// partner's loads zero tiles from past the end of the sequence.
//
// Two CTAs share an SM (256 TMEM columns and under 100 KiB of shared memory each): while one
// waits for its softmax, the MMAs of the other run.
#include <cfloat>
#include <climits>
#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "sm100.cuh"

namespace mmh3 {

namespace {

using namespace sm100;

constexpr int TILE = 64;              // rows of a VSA tile
constexpr int PAIR = 2 * TILE;        // rows and keys of one MMA
constexpr int SOFTMAX_WARPS = 4;
constexpr int LOAD_WARP = SOFTMAX_WARPS;
constexpr int MMA_WARP = SOFTMAX_WARPS + 1;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
// Up to this many tiles the two route lists of a CTA are compared (one bit per tile each) and the
// key tiles both lists hold are walked once for both query tiles; longer sequences pair the lists
// entry by entry only.
constexpr int MAX_BITMAP_TILES = 16384;
// Route lists of up to this many tiles are sorted into the schedule's lists once per CTA; longer
// ones are walked entry by entry as the steps come.
constexpr int TABLE_ENTRIES = 1024;
constexpr uint32_t TMEM_COLUMNS = 256;
constexpr uint32_t TMEM_SCORES = 0;
constexpr uint32_t TMEM_OUTPUT = 128;
// How far (in log2 units) the running maximum may lag before O is rescaled: BF16 probabilities
// have the range for 2^8; E4M3 saturates at 448, so there the lag is one and the probabilities are
// scaled by 224 instead of the reference's 448.
template <bool QUANTIZED> constexpr float RESCALE_LAG = QUANTIZED ? 1.0f : 8.0f;
constexpr float LOG2_224 = 7.807354922057604f;
// Of every four pairs of probabilities, how many take the polynomial exp2 instead of the MUFU:
// none, which at the power cap a layer's worth of launches runs into is 2 % faster than one in
// four (fewer instructions, a higher clock), as in dense_bf16.cu.
constexpr int POLYNOMIAL_PAIRS_OF_4 = 0;
// In the INT8/FP8 form every exponential takes the MUFU, and an integer score s, |s| < 2^22,
// becomes the float 1.5 * 2^23 + s by adding these bits to it, as in quantized_attention.cu.
constexpr int32_t MAGIC_BITS = 0x4B400000;
constexpr float MAGIC_VALUE = 12582912.0f;

template <bool QUANTIZED> struct Shape {
    // Bytes of a 128-row operand tile and of the half of it one VSA tile fills.
    static constexpr int TILE_BYTES = QUANTIZED ? PAIR * 128 : 2 * PAIR * 128;
    static constexpr int STAGES = QUANTIZED ? 4 : 2;
    static constexpr int SMEM_QUERY = 0;
    static constexpr int SMEM_RING = TILE_BYTES;
    static constexpr int SMEM_BARRIERS = SMEM_RING + STAGES * TILE_BYTES;
    // After the barriers: one bit per tile for each of the CTA's two route lists.
    static constexpr int SMEM_BITMAPS = SMEM_BARRIERS + 256;
    // Then the schedule's three lists of tiles (common, only in list 0, only in list 1).
    static constexpr int SMEM_TABLES = SMEM_BITMAPS + 2 * (MAX_BITMAP_TILES / 8);
    static constexpr int SMEM_BYTES = SMEM_TABLES + 3 * TABLE_ENTRIES * 2 + 1024;
    static constexpr int QUERY_FULL = 0;
    static constexpr int RING_FULL = 1;
    static constexpr int RING_EMPTY = RING_FULL + STAGES;
    static constexpr int SCORES_FULL = RING_EMPTY + STAGES;
    static constexpr int PROBABILITIES_FULL = SCORES_FULL + 1;
    static constexpr int OUTPUT_FULL = PROBABILITIES_FULL + 1;
    static constexpr int BARRIERS = OUTPUT_FULL + 1;
    static_assert(BARRIERS * 8 + 8 <= 256, "the barriers outgrew their corner of shared memory");
};

struct VsaMaps {
    // BF16: [128, tokens, heads] each, boxes of 64 columns x 64 rows.
    // INT8/FP8: query and key [128, tokens, heads] INT8 in boxes of 128 x 64; value
    // [tiles * 64, 128, heads] E4M3 in boxes of 64 keys x 128 dimensions with the 64-byte swizzle.
    CUtensorMap query;
    CUtensorMap key;
    CUtensorMap value;
};

struct VsaParams {
    __nv_bfloat16 *output;
    int64_t output_token_stride;
    int64_t output_head_stride;
    const __nv_bfloat16 *gate;
    int64_t gate_stride;
    const float *coarse;
    const int32_t *tile_starts;
    const int32_t *tile_lengths;
    const uint16_t *routes;
    const int32_t *route_counts;
    const float *query_scales;
    const float *key_scales;
    const float *value_scales;
    // Sol-Attn: the pooled tail of each query block as an online-softmax state and the centring
    // offset of each row's scores (see the epilogue); null for VSA.
    const float *tail_max;
    const float *tail_sum;
    const float *tail_values;
    const float *row_offsets;
    int tokens;
    int tiles;
    float scale_log2;
    int vector_stores;
    int vector_gates; // gate rows start on 16 bytes
    unsigned int *status;
};

template <bool QUANTIZED>
__global__ void __launch_bounds__(THREADS, 2)
    vsa_attention_kernel(const __grid_constant__ VsaMaps maps, const VsaParams p) {
    using S = Shape<QUANTIZED>;
    extern __shared__ uint8_t shared_memory[];
    const uint32_t base = (smem_u32(shared_memory) + 1023u) & ~1023u;
    uint8_t *aligned = shared_memory + (base - smem_u32(shared_memory));
    const uint32_t barriers = base + S::SMEM_BARRIERS;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(
        aligned + S::SMEM_BARRIERS + S::BARRIERS * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const Watchdog watchdog = {abort_flag, p.status};
    auto barrier = [&](int index) { return barriers + index * 8; };

    if (*reinterpret_cast<volatile unsigned int *>(p.status) != 0) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int head = blockIdx.y;
    // Without tile tables the tiles are the blocks of 64 tokens (Sol-Attn).
    auto tile_start = [&](int tile) {
        return p.tile_starts != nullptr ? p.tile_starts[tile] : tile * TILE;
    };
    auto tile_length = [&](int tile) {
        return p.tile_lengths != nullptr ? p.tile_lengths[tile] : min(TILE, p.tokens - tile * TILE);
    };
    // The two query tiles of this CTA; the second may not exist.
    const int query_tiles[2] = {static_cast<int>(blockIdx.x) * 2,
                                static_cast<int>(blockIdx.x) * 2 + 1};
    const bool exists[2] = {true, query_tiles[1] < p.tiles};
    const size_t route_rows[2] = {static_cast<size_t>(head) * p.tiles + query_tiles[0],
                                  static_cast<size_t>(head) * p.tiles + query_tiles[1]};
    const int counts[2] = {p.route_counts[route_rows[0]],
                           exists[1] ? p.route_counts[route_rows[1]] : 0};
    const uint16_t *lists[2] = {p.routes + route_rows[0] * p.tiles,
                                p.routes + (exists[1] ? route_rows[1] : route_rows[0]) * p.tiles};
    // One bit per tile and list, and how many tiles both lists hold.
    uint32_t *bitmaps = reinterpret_cast<uint32_t *>(aligned + S::SMEM_BITMAPS);
    constexpr int BITMAP_WORDS = MAX_BITMAP_TILES / 32;
    __shared__ int common_tiles;
    const bool compared = exists[1] && p.tiles <= MAX_BITMAP_TILES;
    if (compared) {
        const int words = (p.tiles + 31) / 32;
        for (int word = threadIdx.x; word < words; word += THREADS) {
            bitmaps[word] = 0;
            bitmaps[BITMAP_WORDS + word] = 0;
        }
        if (threadIdx.x == 0) {
            common_tiles = 0;
        }
        __syncthreads();
        for (int half = 0; half < 2; half++) {
            for (int entry = threadIdx.x; entry < counts[half]; entry += THREADS) {
                const int tile = lists[half][entry];
                atomicOr(bitmaps + half * BITMAP_WORDS + tile / 32, 1u << (tile % 32));
            }
        }
        __syncthreads();
        int both = 0;
        for (int word = threadIdx.x; word < words; word += THREADS) {
            both += __popc(bitmaps[word] & bitmaps[BITMAP_WORDS + word]);
        }
        #pragma unroll
        for (int offset = 16; offset > 0; offset /= 2) {
            both += __shfl_xor_sync(0xffffffffu, both, offset);
        }
        if (threadIdx.x % 32 == 0 && both > 0) {
            atomicAdd(&common_tiles, both);
        }
        __syncthreads();
    }
    const int common = compared ? common_tiles : 0;
    // The schedule's lists, in ascending order as the route lists are: the tiles both lists hold,
    // and each list's own. A warp to a list, 32 entries at a time; every role then reads a step's
    // tiles from shared memory instead of walking the route lists in global memory against the
    // bitmaps as the steps come.
    uint16_t *tables = reinterpret_cast<uint16_t *>(aligned + S::SMEM_TABLES);
    const bool tabled = compared && counts[0] <= TABLE_ENTRIES && counts[1] <= TABLE_ENTRIES;
    if (tabled) {
        if (warp < 3) {
            const int half = warp == 2 ? 1 : 0;
            const bool want_common = warp == 0;
            uint16_t *table = tables + warp * TABLE_ENTRIES;
            int written = 0;
            const int entries = half ? counts[1] : counts[0];
            const uint16_t *list = half ? lists[1] : lists[0];
            for (int first = 0; first < entries; first += 32) {
                const int entry = first + lane;
                int tile = 0;
                bool keep = false;
                if (entry < entries) {
                    tile = list[entry];
                    const bool in_other =
                        (bitmaps[(1 - half) * BITMAP_WORDS + tile / 32] >> (tile % 32)) & 1u;
                    keep = in_other == want_common;
                }
                const unsigned kept = __ballot_sync(0xffffffffu, keep);
                if (keep) {
                    table[written + __popc(kept & ((1u << lane) - 1))] = static_cast<uint16_t>(tile);
                }
                written += __popc(kept);
            }
        }
        __syncthreads();
    }
    // The schedule every role walks. First the `common` tiles, two to a step (both query tiles
    // against both key tiles: a full 128 x 128 block of S), then the odd one left over alone (a
    // 128 x 64 block), then the remaining entries of the two lists paired in order, each query
    // tile against its own key tile (the diagonal 64 x 64 blocks of S).
    const int double_steps = common / 2;
    const int single_steps = common % 2;
    const int steps = double_steps + single_steps + max(counts[0], counts[1]) - common;
    enum StepKind { BOTH_BOTH, BOTH_ONE, OWN };
    auto step_kind = [&](int step) {
        return step < double_steps ? BOTH_BOTH
                                   : (step < double_steps + single_steps ? BOTH_ONE : OWN);
    };
    auto in_list = [&](int half, int tile) {
        return (bitmaps[half * BITMAP_WORDS + tile / 32] >> (tile % 32)) & 1u;
    };
    // Positions in the two route lists.
    struct Cursors {
        int at[2];
    };
    // The key tiles of step `step` (-1: none). For the kinds that share, both come from list 0
    // (the next entries that list 1 also holds); BOTH_ONE fills only tiles[0].
    auto next_step = [&](int step, Cursors &cursors, int (&tiles)[2]) {
        const StepKind kind = step_kind(step);
        if (tabled) {
            if (kind == OWN) {
                const int index = step - double_steps - single_steps;
                tiles[0] = index < counts[0] - common ? tables[TABLE_ENTRIES + index] : -1;
                tiles[1] = index < counts[1] - common ? tables[2 * TABLE_ENTRIES + index] : -1;
            } else {
                tiles[0] = tables[2 * step];
                tiles[1] = kind == BOTH_BOTH ? tables[2 * step + 1] : -1;
            }
            return kind;
        }
        if (kind != OWN) {
            int entry = cursors.at[0];
            for (int slot = 0; slot < (kind == BOTH_BOTH ? 2 : 1); slot++) {
                while (!in_list(1, lists[0][entry])) {
                    entry++;
                }
                tiles[slot] = lists[0][entry];
                entry++;
            }
            if (kind == BOTH_ONE) {
                tiles[1] = -1;
            }
            cursors.at[0] = entry;
            return kind;
        }
        if (step == double_steps + single_steps) {
            cursors.at[0] = cursors.at[1] = 0;
        }
        #pragma unroll
        for (int half = 0; half < 2; half++) {
            int entry = cursors.at[half];
            if (common > 0) {
                while (entry < counts[half] && in_list(1 - half, lists[half][entry])) {
                    entry++;
                }
            }
            tiles[half] = entry < counts[half] ? lists[half][entry] : -1;
            cursors.at[half] = entry + 1;
        }
        return kind;
    };

    if (threadIdx.x == 0) {
        mbar_init(barrier(S::QUERY_FULL), 1);
        for (int stage = 0; stage < S::STAGES; stage++) {
            mbar_init(barrier(S::RING_FULL + stage), 1);
            mbar_init(barrier(S::RING_EMPTY + stage), 1);
        }
        mbar_init(barrier(S::SCORES_FULL), 1);
        mbar_init(barrier(S::PROBABILITIES_FULL), PAIR);
        mbar_init(barrier(S::OUTPUT_FULL), 1);
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
            tma_prefetch_descriptor(&maps.query);
            tma_prefetch_descriptor(&maps.key);
            tma_prefetch_descriptor(&maps.value);
            // A box that starts at row `tokens` lies past the tensor and arrives as zeroes.
            auto load_rows = [&](const CUtensorMap *map, uint32_t destination, uint32_t bar,
                                 int row) {
                if constexpr (QUANTIZED) {
                    tma_load_3d(destination, map, bar, 0, row, head);
                } else {
                    tma_load_3d(destination, map, bar, 0, row, head);
                    tma_load_3d(destination + PAIR * 128, map, bar, 64, row, head);
                }
            };
            mbar_expect_tx(barrier(S::QUERY_FULL), S::TILE_BYTES);
            for (int half = 0; half < 2; half++) {
                load_rows(&maps.query, base + S::SMEM_QUERY + half * TILE * 128,
                          barrier(S::QUERY_FULL),
                          exists[half] ? tile_start(query_tiles[half]) : p.tokens);
            }
            Cursors cursors = {{0, 0}};
            for (int step = 0; step < steps; step++) {
                int tiles_now[2];
                const StepKind kind = next_step(step, cursors, tiles_now);
                // A step with one key tile for both query tiles fills only the first half of the
                // stage.
                const int halves = kind == BOTH_ONE ? 1 : 2;
                int rows[2];
                for (int half = 0; half < 2; half++) {
                    rows[half] = tiles_now[half] >= 0 ? tile_start(tiles_now[half]) : p.tokens;
                }
                bool alive = true;
                for (int part = 0; part < 2 && alive; part++) { // K, then V
                    const int item = 2 * step + part;
                    const int stage = item % S::STAGES;
                    const int use = item / S::STAGES;
                    if (use > 0 && !mbar_wait(barrier(S::RING_EMPTY + stage), (use - 1) & 1,
                                              watchdog, STATUS_VSA | 1)) {
                        alive = false;
                        break;
                    }
                    const uint32_t bar = barrier(S::RING_FULL + stage);
                    const uint32_t destination = base + S::SMEM_RING + stage * S::TILE_BYTES;
                    mbar_expect_tx(bar, S::TILE_BYTES / 2 * halves);
                    for (int half = 0; half < halves; half++) {
                        if (QUANTIZED && part == 1) {
                            // FP8 V: 64 keys of tile t are columns t * 64 of [128 dims] rows; each
                            // half is its own tile of 64-byte rows.
                            const int column =
                                tiles_now[half] >= 0 ? tiles_now[half] * TILE : p.tiles * TILE;
                            tma_load_3d(destination + half * (HEAD_DIM * TILE), &maps.value, bar,
                                        column, 0, head);
                        } else {
                            load_rows(part ? &maps.value : &maps.key,
                                      destination + half * TILE * 128, bar, rows[half]);
                        }
                    }
                }
                if (!alive) {
                    break;
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            const uint32_t query_tile = base + S::SMEM_QUERY;
            const uint32_t ring = base + S::SMEM_RING;
            constexpr uint32_t SCORE_MMA =
                QUANTIZED ? instruction_descriptor(ACCUMULATE_S32, FORMAT_S8, FORMAT_S8, 0, 0,
                                                   PAIR, PAIR)
                          : instruction_descriptor(ACCUMULATE_F32, FORMAT_BF16, FORMAT_BF16, 0, 0,
                                                   PAIR, PAIR);
            constexpr uint32_t OUTPUT_MMA =
                QUANTIZED ? instruction_descriptor(ACCUMULATE_F32, FORMAT_E4M3, FORMAT_E4M3, 0, 0,
                                                   PAIR, HEAD_DIM)
                          : instruction_descriptor(ACCUMULATE_F32, FORMAT_BF16, FORMAT_BF16, 0, 1,
                                                   PAIR, HEAD_DIM);
            // A shared step scores all 128 rows against one key tile: 64 columns instead of 128.
            constexpr uint32_t SHARED_SCORE_MMA =
                QUANTIZED ? instruction_descriptor(ACCUMULATE_S32, FORMAT_S8, FORMAT_S8, 0, 0,
                                                   PAIR, TILE)
                          : instruction_descriptor(ACCUMULATE_F32, FORMAT_BF16, FORMAT_BF16, 0, 0,
                                                   PAIR, TILE);
            const uint64_t query_operand = smem_descriptor(query_tile, 16, 1024);
            auto score = [&](uint32_t key_tile, bool shared) {
                const uint64_t key_operand = smem_descriptor(key_tile, 16, 1024);
                const uint32_t shape = shared ? SHARED_SCORE_MMA : SCORE_MMA;
                if constexpr (QUANTIZED) {
                    #pragma unroll
                    for (int step = 0; step < HEAD_DIM / 32; step++) {
                        mma_i8_ss(tmem + TMEM_SCORES, advance_descriptor(query_operand, step * 32),
                                  advance_descriptor(key_operand, step * 32), shape, step > 0);
                    }
                } else {
                    #pragma unroll
                    for (int step = 0; step < HEAD_DIM / 16; step++) {
                        const uint32_t offset = (step / 4) * (PAIR * 128) + (step % 4) * 32;
                        mma_f16_ss(tmem + TMEM_SCORES, advance_descriptor(query_operand, offset),
                                   advance_descriptor(key_operand, offset), shape, step > 0);
                    }
                }
                tcgen05_commit(barrier(S::SCORES_FULL));
            };
            // `keys` of P and V take part: 128, or the 64 of a shared step.
            auto accumulate = [&](uint32_t value_tile, bool first, int keys) {
                if constexpr (QUANTIZED) {
                    // Two tiles of [128 dims][64 keys] in the 64-byte swizzle.
                    const uint64_t operand = smem_descriptor(value_tile, 16, 512, SWIZZLE_64B);
                    #pragma unroll
                    for (int step = 0; step < PAIR / 32; step++) {
                        if (step * 32 < keys) {
                            mma_f8_ts(tmem + TMEM_OUTPUT, tmem + TMEM_SCORES + step * 8,
                                      advance_descriptor(operand, (step / 2) * (HEAD_DIM * TILE) +
                                                                      (step % 2) * 32),
                                      OUTPUT_MMA, !first || step > 0);
                        }
                    }
                } else {
                    const uint64_t operand = smem_descriptor(value_tile, PAIR * 128, 1024);
                    #pragma unroll
                    for (int step = 0; step < PAIR / 16; step++) {
                        if (step * 16 < keys) {
                            mma_f16_ts(tmem + TMEM_OUTPUT, tmem + TMEM_SCORES + step * 8,
                                       advance_descriptor(operand, step * 16 * 128), OUTPUT_MMA,
                                       !first || step > 0);
                        }
                    }
                }
            };
            bool alive = steps == 0 ||
                         (mbar_wait(barrier(S::QUERY_FULL), 0, watchdog, STATUS_VSA | 2) &&
                          mbar_wait(barrier(S::RING_FULL + 0), 0, watchdog, STATUS_VSA | 3));
            if (alive && steps > 0) {
                tcgen05_fence_after();
                score(ring, step_kind(0) == BOTH_ONE);
                tcgen05_commit(barrier(S::RING_EMPTY + 0));
            }
            int item = 1;
            for (int step = 0; alive && step < steps; step++, item += 2) {
                const int value_stage = item % S::STAGES;
                const int key_stage = (item + 1) % S::STAGES;
                const bool more = step + 1 < steps;
                alive = mbar_wait(barrier(S::RING_FULL + value_stage), (item / S::STAGES) & 1,
                                  watchdog, STATUS_VSA | 4) &&
                        (!more || mbar_wait(barrier(S::RING_FULL + key_stage),
                                            ((item + 1) / S::STAGES) & 1, watchdog,
                                            STATUS_VSA | 5)) &&
                        mbar_wait(barrier(S::PROBABILITIES_FULL), step & 1, watchdog,
                                  STATUS_VSA | 6);
                if (!alive) {
                    break;
                }
                tcgen05_fence_after();
                accumulate(ring + value_stage * S::TILE_BYTES, step == 0,
                           step_kind(step) == BOTH_ONE ? TILE : PAIR);
                tcgen05_commit(barrier(S::RING_EMPTY + value_stage));
                if (more) {
                    score(ring + key_stage * S::TILE_BYTES, step_kind(step + 1) == BOTH_ONE);
                    tcgen05_commit(barrier(S::RING_EMPTY + key_stage));
                }
            }
            if (alive) {
                tcgen05_commit(barrier(S::OUTPUT_FULL));
            }
        }
    } else {
        // Softmax: this thread owns row `row` of the pair, which is row `row % 64` of tile `half`.
        const int row = warp * 32 + lane;
        const int half = row / TILE;
        // This thread's tile of the two, picked once: indexing the pairs with `half` would put
        // them in local memory.
        const int count = half ? counts[1] : counts[0];
        const bool own_exists = half ? exists[1] : exists[0];
        const int own_query_tile = half ? query_tiles[1] : query_tiles[0];
        const size_t own_route_row = half ? route_rows[1] : route_rows[0];
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        // The 64 columns of S that hold this tile's keys, and where its P goes: BF16 P packs two
        // keys to a column (own keys in 32 columns), E4M3 P four (16 columns).
        // In a shared step both tiles' threads read columns 0-63 and P fills the first columns
        // alone.
        const uint32_t score_columns = tmem + lane_base + TMEM_SCORES;
        constexpr int P_COLUMNS = QUANTIZED ? TILE / 4 : TILE / 2;
        const uint32_t accumulator = tmem + lane_base + TMEM_OUTPUT;
        float query_factor = p.scale_log2;
        const float *head_key_scales = nullptr;
        if constexpr (QUANTIZED) {
            query_factor *= own_exists ? p.query_scales[own_route_row] : 0.0f;
            head_key_scales = p.key_scales + static_cast<size_t>(head) * p.tiles;
        }
        float maximum = -INFINITY;
        float2 sums[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
        bool first_pass = true;
        // MASKED below: the key tile is shorter than 64 (or this list has ended), so the columns past
        // its length take an exponent of minus infinity. Warps 0-1 and 2-3 may serve different key
        // tiles, but a warp serves one, so the choice is uniform across a warp.
        //
        // The running maximum takes 64 scores in, and O and the sums are rescaled if it grew too
        // far.
        auto take_maximum = [&](auto masked, const uint32_t (&raw)[2][32], int valid, float factor,
                                bool active) {
            constexpr bool MASKED = decltype(masked)::value;
            // The block maximum in the units of the exponent: scale * log2(e) times the score.
            float block_maximum;
            if constexpr (QUANTIZED) {
                int partial[2] = {INT_MIN, INT_MIN};
                #pragma unroll
                for (int index = 0; index + 1 < TILE; index += 2) {
                    const int first = static_cast<int>(raw[index / 32][index % 32]);
                    const int second = static_cast<int>(raw[(index + 1) / 32][(index + 1) % 32]);
                    partial[(index / 2) % 2] = __vimax3_s32(
                        partial[(index / 2) % 2], MASKED && index >= valid ? INT_MIN : first,
                        MASKED && index + 1 >= valid ? INT_MIN : second);
                }
                const int largest = max(partial[0], partial[1]);
                block_maximum =
                    largest == INT_MIN ? -INFINITY : static_cast<float>(largest) * factor;
            } else {
                float partial[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                #pragma unroll
                for (int index = 0; index < TILE; index++) {
                    const float score = __uint_as_float(raw[index / 32][index % 32]);
                    partial[index % 4] =
                        fmaxf(partial[index % 4], MASKED && index >= valid ? -INFINITY : score);
                }
                block_maximum =
                    fmaxf(fmaxf(partial[0], partial[1]), fmaxf(partial[2], partial[3])) * factor;
            }
            // The first step of a list always has keys, so the maximum is finite from then on.
            const bool grown = active && block_maximum - maximum > RESCALE_LAG<QUANTIZED>;
            if (first_pass) {
                maximum = active ? block_maximum : 0.0f;
            } else if (__any_sync(0xffffffffu, grown)) {
                const float raised = fmaxf(maximum, block_maximum);
                const float correction = exp2_approx(maximum - raised);
                maximum = raised;
                const float2 correction2 = make_float2(correction, correction);
                sums[0] = __fmul2_rn(sums[0], correction2);
                sums[1] = __fmul2_rn(sums[1], correction2);
                #pragma unroll
                for (int chunk = 0; chunk < 4; chunk++) {
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
            first_pass = false;
        };
        // The probabilities of 64 scores against the running maximum go to `own_p`, and zeroes to
        // `other_p` when the other query tile has its own key tile in this step.
        auto write_probabilities = [&](auto masked, const uint32_t (&raw)[2][32], int valid,
                                       float factor, uint32_t own_p, uint32_t other_p,
                                       bool shared) {
            constexpr bool MASKED = decltype(masked)::value;
            // p = 2^(factor * score - maximum), times 224 for E4M3; pairs of elements.
            // (MAGIC + s) * factor + (offset - MAGIC * factor) = s * factor + offset, the product
            // exact inside the FMA.
            const float offset =
                QUANTIZED ? fmaf(-MAGIC_VALUE, factor, LOG2_224 - maximum) : -maximum;
            const float2 factor2 = make_float2(factor, factor);
            const float2 offset2 = make_float2(offset, offset);
            constexpr int WORDS = QUANTIZED ? TILE / 4 : TILE / 2;
            uint32_t packed[WORDS], zeroes[WORDS];
            #pragma unroll
            for (int pair = 0; pair < TILE / 2; pair++) {
                const uint32_t words[2] = {raw[(pair * 2) / 32][(pair * 2) % 32],
                                           raw[(pair * 2 + 1) / 32][(pair * 2 + 1) % 32]};
                const float2 score =
                    QUANTIZED ? make_float2(__int_as_float(static_cast<int32_t>(words[0]) + MAGIC_BITS),
                                            __int_as_float(static_cast<int32_t>(words[1]) + MAGIC_BITS))
                              : make_float2(__uint_as_float(words[0]),
                                            __uint_as_float(words[1]));
                float2 x = __ffma2_rn(score, factor2, offset2);
                if (MASKED) {
                    x.x = pair * 2 < valid ? x.x : -INFINITY;
                    x.y = pair * 2 + 1 < valid ? x.y : -INFINITY;
                }
                float2 probability;
                if (!QUANTIZED && pair % 4 < POLYNOMIAL_PAIRS_OF_4) {
                    probability = exp2_polynomial(x);
                } else {
                    probability = make_float2(exp2_approx(x.x), exp2_approx(x.y));
                }
                sums[pair % 2] = __fadd2_rn(sums[pair % 2], probability);
                if constexpr (QUANTIZED) {
                    uint16_t two;
                    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;"
                        : "=h"(two)
                        : "f"(probability.y), "f"(probability.x));
                    if (pair % 2 == 0) {
                        packed[pair / 2] = two;
                    } else {
                        packed[pair / 2] |= static_cast<uint32_t>(two) << 16;
                    }
                } else {
                    packed[pair] = pack_bf16(probability.x, probability.y);
                }
            }
            #pragma unroll
            for (int word = 0; word < WORDS; word++) {
                zeroes[word] = 0;
            }
            if constexpr (QUANTIZED) {
                tmem_store_16(own_p, packed);
                if (!shared) {
                    tmem_store_16(other_p, zeroes);
                }
            } else {
                tmem_store_32(own_p, packed);
                if (!shared) {
                    tmem_store_32(other_p, zeroes);
                }
            }
        };
        bool alive = true;
        Cursors cursors = {{0, 0}};
        for (int step = 0; step < steps; step++) {
            int tiles_now[2];
            const StepKind kind = next_step(step, cursors, tiles_now);
            // What the step's key tiles bring (their lengths, and their scales in INT8) is read
            // while the scores are still being taken.
            const int first_tile = tiles_now[0], second_tile = tiles_now[1];
            const int first_valid = first_tile >= 0 ? tile_length(first_tile) : 0;
            const int second_valid = second_tile >= 0 ? tile_length(second_tile) : 0;
            float first_factor = query_factor, second_factor = query_factor;
            if constexpr (QUANTIZED) {
                first_factor *= first_tile >= 0 ? __ldg(head_key_scales + first_tile) : 0.0f;
                second_factor *= second_tile >= 0 ? __ldg(head_key_scales + second_tile) : 0.0f;
            }
            alive = mbar_wait(barrier(S::SCORES_FULL), step & 1, watchdog, STATUS_VSA | 7);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) {
                break;
            }
            tcgen05_fence_after();
            // A thread takes 64 columns of S at a time: its own tile's key tile in a step of kind
            // OWN (and zeroes go into the other tile's columns of P); the one key tile of a
            // BOTH_ONE step; and both key tiles, one after the other, in a BOTH_BOTH step.
            // BOTH_BOTH: passes 0 and 1 take the two key tiles into the maximum, passes 2 and 3 write
            // their probabilities.
            const int passes = kind == BOTH_BOTH ? 4 : 1;
            for (int pass = 0; pass < passes; pass++) {
                const bool maximum_phase = kind != BOTH_BOTH || pass < 2;
                const bool probability_phase = kind != BOTH_BOTH || pass >= 2;
                const int slot = kind == OWN ? half : pass % 2;
                const bool shared = kind != OWN;
                const bool active = (slot == 0 ? first_tile : second_tile) >= 0;
                const int valid = slot == 0 ? first_valid : second_valid;
                const float factor = slot == 0 ? first_factor : second_factor;
                const uint32_t scores = score_columns + slot * TILE;
                const uint32_t own_p = score_columns + slot * P_COLUMNS;
                const uint32_t other_p = score_columns + (1 - half) * P_COLUMNS;
                uint32_t raw[2][32];
                tmem_load_32(scores, raw[0]);
                tmem_load_32(scores + 32, raw[1]);
                tmem_wait_load();
                if (valid < TILE) {
                    if (maximum_phase) {
                        take_maximum(std::true_type{}, raw, valid, factor, active);
                    }
                    if (probability_phase) {
                        write_probabilities(std::true_type{}, raw, valid, factor, own_p, other_p,
                                            shared);
                    }
                } else {
                    if (maximum_phase) {
                        take_maximum(std::false_type{}, raw, valid, factor, active);
                    }
                    if (probability_phase) {
                        write_probabilities(std::false_type{}, raw, valid, factor, own_p, other_p,
                                            shared);
                    }
                }
            }
            tmem_wait_store();
            tcgen05_fence_before();
            mbar_arrive(barrier(S::PROBABILITIES_FULL));
        }
        if (alive && steps > 0) {
            alive = mbar_wait(barrier(S::OUTPUT_FULL), 0, watchdog, STATUS_VSA | 8);
            alive = __all_sync(0xffffffffu, alive);
        }
        if (alive && steps > 0) {
            tcgen05_fence_after();
            const int tile_row = row % TILE;
            const bool stored =
                own_exists && tile_row < tile_length(own_query_tile) && count > 0;
            const int64_t token = stored ? tile_start(own_query_tile) + tile_row : 0;
            const float sum = (sums[0].x + sums[0].y) + (sums[1].x + sums[1].y);
            float value_scale = 1.0f;
            if constexpr (QUANTIZED) {
                value_scale = p.value_scales[head];
            }
            float inverse = value_scale / sum;
            // Sol-Attn: every key block the list leaves out contributes one pooled term; their
            // sum arrives as a softmax state (maximum, sum of weights, weighted values) in the
            // units of the centred scores, which this row's scores reach by its offset.
            const bool tailed = p.tail_max != nullptr;
            const float *tail_values = tailed ? p.tail_values + own_route_row * HEAD_DIM : nullptr;
            float tail_weight = 0.0f;
            if (tailed && stored) {
                const float centred =
                    maximum - p.row_offsets[static_cast<size_t>(head) * p.tokens + token];
                const float tail_maximum = p.tail_max[own_route_row];
                const float merged = fmaxf(centred, tail_maximum);
                const float routed_weight = exp2f(centred - merged);
                // E4M3 probabilities, and with them the sum and O, carry a factor of 224.
                constexpr float CARRIED = QUANTIZED ? 224.0f : 1.0f;
                tail_weight = CARRIED * exp2f(tail_maximum - merged);
                const float total =
                    1.0f / (sum * routed_weight + p.tail_sum[own_route_row] * tail_weight);
                tail_weight *= total;
                inverse = value_scale * routed_weight * total;
            }
            __nv_bfloat16 *output_row = p.output + token * p.output_token_stride +
                                        static_cast<int64_t>(head) * p.output_head_stride;
            const bool gated = p.gate != nullptr;
            const __nv_bfloat16 *gate_row =
                gated ? p.gate + token * p.gate_stride + static_cast<int64_t>(head) * HEAD_DIM
                      : nullptr;
            const float *coarse = gated ? p.coarse + own_route_row * HEAD_DIM : nullptr;
            #pragma unroll
            for (int chunk = 0; chunk < 4; chunk++) {
                uint32_t values[32];
                tmem_load_32(accumulator + chunk * 32, values);
                tmem_wait_load();
                if (stored) {
                    float results[32];
                    #pragma unroll
                    for (int index = 0; index < 32; index++) {
                        results[index] = __uint_as_float(values[index]) * inverse;
                    }
                    if (gated) {
                        // 32 gates (eight to a 16-byte load where the rows allow it) times the
                        // tile's 32 coarse values.
                        float gates[32];
                        if (p.vector_gates) {
                            #pragma unroll
                            for (int part = 0; part < 4; part++) {
                                const uint4 eight =
                                    __ldg(reinterpret_cast<const uint4 *>(gate_row + chunk * 32) + part);
                                const uint32_t words[4] = {eight.x, eight.y, eight.z, eight.w};
                                #pragma unroll
                                for (int word = 0; word < 4; word++) {
                                    gates[part * 8 + word * 2] = __uint_as_float(words[word] << 16);
                                    gates[part * 8 + word * 2 + 1] =
                                        __uint_as_float(words[word] & 0xffff0000u);
                                }
                            }
                        } else {
                            #pragma unroll
                            for (int index = 0; index < 32; index++) {
                                gates[index] = __bfloat162float(gate_row[chunk * 32 + index]);
                            }
                        }
                        #pragma unroll
                        for (int part = 0; part < 8; part++) {
                            const float4 four =
                                __ldg(reinterpret_cast<const float4 *>(coarse + chunk * 32) + part);
                            results[part * 4] = fmaf(gates[part * 4], four.x, results[part * 4]);
                            results[part * 4 + 1] =
                                fmaf(gates[part * 4 + 1], four.y, results[part * 4 + 1]);
                            results[part * 4 + 2] =
                                fmaf(gates[part * 4 + 2], four.z, results[part * 4 + 2]);
                            results[part * 4 + 3] =
                                fmaf(gates[part * 4 + 3], four.w, results[part * 4 + 3]);
                        }
                    }
                    if (tailed) {
                        #pragma unroll
                        for (int part = 0; part < 8; part++) {
                            const float4 four = __ldg(
                                reinterpret_cast<const float4 *>(tail_values + chunk * 32) + part);
                            results[part * 4] = fmaf(four.x, tail_weight, results[part * 4]);
                            results[part * 4 + 1] = fmaf(four.y, tail_weight, results[part * 4 + 1]);
                            results[part * 4 + 2] = fmaf(four.z, tail_weight, results[part * 4 + 2]);
                            results[part * 4 + 3] = fmaf(four.w, tail_weight, results[part * 4 + 3]);
                        }
                    }
                    uint32_t packed[16];
                    #pragma unroll
                    for (int pair = 0; pair < 16; pair++) {
                        packed[pair] = pack_bf16(results[pair * 2], results[pair * 2 + 1]);
                    }
                    if (p.vector_stores) {
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
            for (int spin = 0; spin < 64; spin++) {
                __nanosleep(1000);
            }
        }
        tcgen05_fence_after();
        tmem_dealloc(tmem, TMEM_COLUMNS);
    }
}

template <bool QUANTIZED>
int launch(const VsaMaps &maps, const VsaParams &params, int heads, cudaStream_t stream) {
    using S = Shape<QUANTIZED>;
    static SharedMemoryOptIn shared_memory;
    const cudaError_t configured =
        shared_memory.ensure(vsa_attention_kernel<QUANTIZED>, S::SMEM_BYTES);
    if (configured != cudaSuccess) {
        return static_cast<int>(configured);
    }
    const dim3 grid((params.tiles + 1) / 2, heads);
    vsa_attention_kernel<QUANTIZED><<<grid, THREADS, S::SMEM_BYTES, stream>>>(maps, params);
    return static_cast<int>(cudaGetLastError());
}

bool fill_params(VsaParams &params, void *output, int tokens, const Mmh3AttentionLayout &layout,
                 float scale, const Mmh3VsaWorkspace &workspace, int tiles, const void *gate,
                 int64_t gate_stride) {
    params.output = static_cast<__nv_bfloat16 *>(output);
    params.output_token_stride = layout.token_stride[OUTPUT];
    params.output_head_stride = layout.head_stride[OUTPUT];
    params.gate = static_cast<const __nv_bfloat16 *>(gate);
    params.gate_stride = gate_stride;
    params.coarse = workspace.coarse;
    params.tile_starts = workspace.tile_starts;
    params.tile_lengths = workspace.tile_lengths;
    params.routes = workspace.routes;
    params.route_counts = workspace.route_counts;
    params.tokens = tokens;
    params.tiles = tiles;
    params.scale_log2 = scale * LOG2_E;
    params.vector_gates = gate != nullptr && reinterpret_cast<uintptr_t>(gate) % 16 == 0 &&
                          gate_stride % 8 == 0;
    params.vector_stores = reinterpret_cast<uintptr_t>(output) % 16 == 0 &&
                           layout.token_stride[OUTPUT] % 8 == 0 &&
                           layout.head_stride[OUTPUT] % 8 == 0;
    params.status = status_pointer();
    return params.status != nullptr;
}

// BF16 q, k, v as [128, tokens, heads] in boxes of 64 columns x 64 rows. Operands off TMA's
// 16-byte grid are gathered into dense arrays in `staged` first.
int encode_bf16_maps(VsaMaps &maps, const void *query, const void *key, const void *value,
                     int tokens, int heads, const Mmh3AttentionLayout &layout,
                     StagedOperands &staged) {
    const uint16_t *bases[3] = {static_cast<const uint16_t *>(query),
                                static_cast<const uint16_t *>(key),
                                static_cast<const uint16_t *>(value)};
    CUtensorMap *targets[3] = {&maps.query, &maps.key, &maps.value};
    for (int operand = 0; operand < 3; operand++) {
        int64_t token_stride = layout.token_stride[operand];
        int64_t head_stride = layout.head_stride[operand];
        const cudaError_t copied = staged.stage(operand, bases[operand], tokens, heads, HEAD_DIM,
                                                token_stride, head_stride);
        if (copied != cudaSuccess) {
            return static_cast<int>(copied);
        }
        const uint64_t dimensions[3] = {HEAD_DIM, static_cast<uint64_t>(tokens),
                                        static_cast<uint64_t>(heads)};
        uint64_t strides[2] = {static_cast<uint64_t>(token_stride) * 2,
                               static_cast<uint64_t>(head_stride) * 2};
        if (heads == 1 && strides[1] == 0) {
            strides[1] = strides[0] * static_cast<uint64_t>(tokens);
        }
        const uint32_t box[3] = {64, TILE, 1};
        if (!encode_tensor_map(targets[operand], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                               bases[operand], dimensions, strides, box)) {
            return NOT_SUPPORTED;
        }
    }
    return 0;
}

} // namespace

int launch_vsa_attention(const void *query, const void *key, const void *value, const void *gate,
                         int64_t gate_stride, void *output, int tokens, int heads,
                         const Mmh3AttentionLayout &layout, float scale, int tiles,
                         const Mmh3VsaWorkspace &workspace, cudaStream_t stream) {
    if (!(scale > 0.0f) || !std::isfinite(scale)) {
        return INVALID_VALUE;
    }
    VsaParams params = {};
    if (!fill_params(params, output, tokens, layout, scale, workspace, tiles, gate, gate_stride)) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    VsaMaps maps;
    StagedOperands staged(stream);
    const int encoded = encode_bf16_maps(maps, query, key, value, tokens, heads, layout, staged);
    if (encoded != 0) {
        return encoded;
    }
    return launch<false>(maps, params, heads, stream);
}

int launch_sol_token_attention(const void *query, const void *key, const void *value, void *output,
                               int tokens, int heads, const Mmh3AttentionLayout &layout,
                               float scale, const Mmh3SparseWorkspace &sparse,
                               cudaStream_t stream) {
    // The routes of Sol-Attn in the form the kernel walks: blocks of 64 tokens for tiles, no gate.
    Mmh3VsaWorkspace workspace = {};
    workspace.routes = sparse.routes;
    workspace.route_counts = sparse.route_counts;
    VsaParams params = {};
    const int blocks = (tokens + TILE - 1) / TILE;
    if (!fill_params(params, output, tokens, layout, scale, workspace, blocks, nullptr, 0)) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    params.tail_max = sparse.tail_max;
    params.tail_sum = sparse.tail_sum;
    params.tail_values = sparse.tail_values;
    params.row_offsets = sparse.row_offsets;
    VsaMaps maps;
    StagedOperands staged(stream);
    const int encoded = encode_bf16_maps(maps, query, key, value, tokens, heads, layout, staged);
    if (encoded != 0) {
        return encoded;
    }
    return launch<false>(maps, params, heads, stream);
}

int launch_sol_token_attention_quantized(const Mmh3QuantizedWorkspace &quantized, void *output,
                                         int tokens, int heads, const Mmh3AttentionLayout &layout,
                                         float scale, const Mmh3SparseWorkspace &sparse,
                                         cudaStream_t stream) {
    // Blocks of 64 tokens for tiles: the dense quantizer's blocks, scales and FP8 V layout.
    Mmh3VsaWorkspace workspace = {};
    workspace.routes = sparse.routes;
    workspace.route_counts = sparse.route_counts;
    return launch_vsa_attention_quantized(quantized, output, tokens, heads, layout, scale,
                                          workspace, (tokens + TILE - 1) / TILE, nullptr, 0, stream,
                                          &sparse);
}

int launch_vsa_attention_quantized(const Mmh3QuantizedWorkspace &quantized, void *output,
                                   int tokens, int heads, const Mmh3AttentionLayout &layout,
                                   float scale, const Mmh3VsaWorkspace &workspace, int tiles,
                                   const void *gate, int64_t gate_stride, cudaStream_t stream,
                                   const Mmh3SparseWorkspace *tails) {
    if (!(scale > 0.0f) || !std::isfinite(scale)) {
        return INVALID_VALUE;
    }
    VsaParams params = {};
    if (!fill_params(params, output, tokens, layout, scale, workspace, tiles, gate, gate_stride)) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    if (tails != nullptr) {
        params.tail_max = tails->tail_max;
        params.tail_sum = tails->tail_sum;
        params.tail_values = tails->tail_values;
        params.row_offsets = tails->row_offsets;
    }
    params.query_scales = quantized.query_scales;
    params.key_scales = quantized.key_scales;
    params.value_scales = quantized.value_scales;
    VsaMaps maps;
    const uint64_t row_dimensions[3] = {HEAD_DIM, static_cast<uint64_t>(tokens),
                                        static_cast<uint64_t>(heads)};
    const uint64_t row_strides[2] = {static_cast<uint64_t>(heads) * HEAD_DIM, HEAD_DIM};
    const uint32_t row_box[3] = {HEAD_DIM, TILE, 1};
    const uint64_t padded = static_cast<uint64_t>(tiles) * TILE;
    const uint64_t value_dimensions[3] = {padded, HEAD_DIM, static_cast<uint64_t>(heads)};
    const uint64_t value_strides[2] = {padded, padded * HEAD_DIM};
    const uint32_t value_box[3] = {TILE, HEAD_DIM, 1};
    if (!encode_tensor_map(&maps.query, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, quantized.query,
                           row_dimensions, row_strides, row_box) ||
        !encode_tensor_map(&maps.key, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, quantized.key,
                           row_dimensions, row_strides, row_box) ||
        !encode_tensor_map(&maps.value, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, quantized.value,
                           value_dimensions, value_strides, value_box,
                           CU_TENSOR_MAP_SWIZZLE_64B)) {
        return NOT_SUPPORTED;
    }
    return launch<true>(maps, params, heads, stream);
}

} // namespace mmh3
