// VSA's tile selection: for every head and query tile the exact set of tiles it attends token by
// token, and, when the layer is gated, the coarse output softmax(scores) . mean values.
//
// What has to come out is what the reference's select_kernel leaves
// (crates/mmh3-cuda/kernels/vsa_attention.cu:96-273): every prefix tile, then the `kept` video
// tiles with the largest pooled scores, ties to the lower tile index, as an ascending list of
// uint16 tile indices, bit for bit. A pooled score there is one particular FP32 evaluation of
// (mean q) . (mean k) * scale: 32 chains of four fused multiply-adds over dimensions l, l + 32,
// l + 64, l + 96, summed over a butterfly that pairs the chains by bit 4 of l first and bit 0 last.
// Scoring every pair of tiles that way is 128 FMAs a pair on the CUDA cores, and almost all of it
// decides nothing: a route only depends on the scores close to its own threshold.
//
// So the work is split by what it needs:
//
// 1. `cosine_kernel`: all pairs on the tensor cores. tcgen05.mma kind::tf32 over the FP32 tile
//    means (TMA into swizzled shared memory, accumulators in tensor memory) gives every score to
//    about 2^-9 of |q| |k|. A CTA keeps a panel of query means and walks key panels through a ring
//    of two with two accumulators. The epilogue divides by the two norms and stores the cosine as
//    a signed 16-bit fraction in the very slot of the route table the pair owns (the table is
//    [heads][tiles][tiles] uint16, one slot a pair), so no other scratch is needed.
// 2. `route_kernel`: a warp per query tile. It rebuilds the approximate scores from its row of
//    cosines, finds the bin of a 512-bin histogram that holds the kept-th largest, and from the
//    proven bound B >= |approximate - exact| sorts the tiles into "certainly kept" (more than 2 B
//    above that bin), "certainly dropped" (more than 2 B below) and the few in between. Only those
//    are scored again, exactly, in the reference's FP32 order, a lane to a chain; a radix select
//    over their order-preserving bit patterns finds the threshold among them and how many ties at
//    it are kept; and the ascending list is written from a bit per kept tile. If the counts ever
//    fail to add up (they cannot while the bound holds) or the open tiles outgrow their list, the
//    row is redone with every tile scored exactly.
// 3. `coarse_kernel`, only for gated layers: eight query tiles to a warp in registers, the tiles
//    32 at a time through shared memory, an online softmax in FP32 (this output is held to a
//    tolerance, not to bits).
#include <algorithm>
#include <cfloat>

#include "common.cuh"
#include "pooled_score.cuh"
#include "sm100.cuh"

namespace mmh3 {

namespace {

using namespace sm100;

// ---------------------------------------------------------------------------------------------
// 1. Cosines of all pairs of tile means, on the tensor cores.

constexpr int PANEL = 128;                     // query tiles and key tiles to a CTA
constexpr int PANEL_SLAB = PANEL * 128;        // 128 rows of 32 floats
constexpr int PANEL_SLABS = HEAD_DIM / 32;
constexpr int PANEL_BYTES = PANEL_SLABS * PANEL_SLAB;
constexpr int COSINE_STAGES = 2;               // key panels and accumulators in flight
constexpr int COSINE_STORING_WARPS = 8;        // two to a quarter of the TMEM lanes, 64 columns each
constexpr int COSINE_THREADS = (COSINE_STORING_WARPS + 1) * 32; // the ninth warp loads and issues
constexpr int COSINE_SMEM_KEYS = PANEL_BYTES;
constexpr int COSINE_SMEM_NORMS = (1 + COSINE_STAGES) * PANEL_BYTES;
constexpr int COSINE_SMEM_BARRIERS = COSINE_SMEM_NORMS + COSINE_STAGES * PANEL * 4;
constexpr int COSINE_SMEM_BYTES = COSINE_SMEM_BARRIERS + 128 + 1024;
constexpr float COSINE_ONE = 32767.0f;
constexpr uint32_t FORMAT_TF32 = 2;            // kind::tf32
constexpr uint32_t COSINE_MMA =
    instruction_descriptor(ACCUMULATE_F32, FORMAT_TF32, FORMAT_TF32, 0, 0, PANEL, PANEL);
constexpr unsigned int STATUS_SELECT = 0x00040000u;

struct CosineMaps {
    CUtensorMap query; // [128, tiles, heads] FP32
    CUtensorMap key;
};

__device__ __forceinline__ void mma_tf32(uint32_t d, uint64_t a, uint64_t b, uint32_t accumulate) {
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
                 "}" ::"r"(d),
                 "l"(a), "l"(b), "r"(COSINE_MMA), "r"(accumulate)
                 : "memory");
}

// The sum of the squares of row `row` of a panel as TMA left it: 32 floats to a 128-byte line,
// 16-byte chunk c of a line at c ^ (row % 8).
__device__ __forceinline__ float panel_row_square(const uint8_t *panel, int row) {
    float sum = 0.0f;
    #pragma unroll
    for (int slab = 0; slab < PANEL_SLABS; slab++) {
        const uint8_t *line = panel + slab * PANEL_SLAB + row * 128;
        #pragma unroll
        for (int chunk = 0; chunk < 8; chunk++) {
            const float4 four = *reinterpret_cast<const float4 *>(line + ((chunk ^ (row & 7)) * 16));
            sum = fmaf(four.x, four.x, sum);
            sum = fmaf(four.y, four.y, sum);
            sum = fmaf(four.z, four.z, sum);
            sum = fmaf(four.w, four.w, sum);
        }
    }
    return sum;
}

// A CTA keeps one panel of 128 query means and walks the key panels blockIdx.x, blockIdx.x +
// gridDim.x, ...: the ninth warp's first lane loads them into a ring of two and issues each
// panel's 16 MMAs into one of two accumulators, and the eight storing warps take a panel's norms
// and store the finished accumulator's cosines while the next panel's MMAs run.
__global__ void __launch_bounds__(COSINE_THREADS, 1)
    cosine_kernel(const __grid_constant__ CosineMaps maps, uint16_t *__restrict__ table, int tiles,
                  unsigned int *status) {
    extern __shared__ uint8_t shared_memory[];
    const uint32_t base = (smem_u32(shared_memory) + 1023u) & ~1023u;
    uint8_t *aligned = shared_memory + (base - smem_u32(shared_memory));
    // Barriers: the query panel; per stage the key panel loaded and free again, its norms written,
    // the accumulator full and read out.
    const uint32_t barriers = base + COSINE_SMEM_BARRIERS;
    const uint32_t query_loaded = barriers;
    const auto key_loaded = [&](int stage) { return barriers + 8 + stage * 8; };
    const auto key_free = [&](int stage) { return barriers + 8 + (COSINE_STAGES + stage) * 8; };
    const auto norms_written = [&](int stage) { return barriers + 8 + (2 * COSINE_STAGES + stage) * 8; };
    const auto multiplied = [&](int stage) { return barriers + 8 + (3 * COSINE_STAGES + stage) * 8; };
    const auto read_out = [&](int stage) { return barriers + 8 + (4 * COSINE_STAGES + stage) * 8; };
    float *inverse_key_norms = reinterpret_cast<float *>(aligned + COSINE_SMEM_NORMS);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(
        aligned + COSINE_SMEM_BARRIERS + 8 + 5 * COSINE_STAGES * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const Watchdog watchdog = {abort_flag, status};
    if (*reinterpret_cast<volatile unsigned int *>(status) != 0) {
        return;
    }
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    const int first_query = blockIdx.y * PANEL;
    const int head = blockIdx.z;
    const int panels = (tiles + PANEL - 1) / PANEL;
    // The key panels of this CTA: blockIdx.x + turn * gridDim.x.
    const int turns = (panels - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                      static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        mbar_init(query_loaded, 1);
        for (int stage = 0; stage < COSINE_STAGES; stage++) {
            mbar_init(key_loaded(stage), 1);
            mbar_init(key_free(stage), 1 + COSINE_STORING_WARPS / 2); // the MMAs and the norms' readers
            mbar_init(norms_written(stage), COSINE_STORING_WARPS / 2);
            mbar_init(multiplied(stage), 1);
            mbar_init(read_out(stage), COSINE_STORING_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == COSINE_STORING_WARPS) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), COSINE_STAGES * PANEL);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == COSINE_STORING_WARPS) {
        if (lane == 0) {
            const auto load_keys = [&](int turn) {
                const int stage = turn % COSINE_STAGES;
                const int first_key = (static_cast<int>(blockIdx.x) + turn * static_cast<int>(gridDim.x)) * PANEL;
                mbar_expect_tx(key_loaded(stage), PANEL_BYTES);
                for (int slab = 0; slab < PANEL_SLABS; slab++) {
                    tma_load_3d(base + COSINE_SMEM_KEYS + stage * PANEL_BYTES + slab * PANEL_SLAB,
                                &maps.key, key_loaded(stage), slab * 32, first_key, head);
                }
            };
            mbar_expect_tx(query_loaded, PANEL_BYTES);
            for (int slab = 0; slab < PANEL_SLABS; slab++) {
                tma_load_3d(base + slab * PANEL_SLAB, &maps.query, query_loaded, slab * 32,
                            first_query, head);
            }
            for (int turn = 0; turn < min(turns, COSINE_STAGES); turn++) {
                load_keys(turn);
            }
            bool alive = mbar_wait(query_loaded, 0, watchdog, STATUS_SELECT | 1);
            for (int turn = 0; alive && turn < turns; turn++) {
                const int stage = turn % COSINE_STAGES;
                const uint32_t parity = (turn / COSINE_STAGES) & 1;
                alive = mbar_wait(key_loaded(stage), parity, watchdog, STATUS_SELECT | 2) &&
                        mbar_wait(read_out(stage), parity ^ 1, watchdog, STATUS_SELECT | 4);
                if (!alive) {
                    break;
                }
                tcgen05_fence_after();
                // Eight floats, 32 bytes, to an MMA: four steps to a slab of 32 dimensions.
                const uint32_t keys = base + COSINE_SMEM_KEYS + stage * PANEL_BYTES;
                #pragma unroll
                for (int step = 0; step < HEAD_DIM / 8; step++) {
                    const uint32_t offset = (step / 4) * PANEL_SLAB + (step % 4) * 32;
                    mma_tf32(tmem + stage * PANEL, smem_descriptor(base + offset, 16, 1024),
                             smem_descriptor(keys + offset, 16, 1024), step > 0);
                }
                tcgen05_commit(multiplied(stage));
                tcgen05_commit(key_free(stage));
                // The panel after this one goes where the panel before this one was, once the
                // MMAs and the norms are done with that.
                if (turn >= 1 && turn + 1 < turns) {
                    const int refilled = (turn + 1) % COSINE_STAGES;
                    const uint32_t emptied = ((turn + 1) / COSINE_STAGES - 1) & 1;
                    alive = mbar_wait(key_free(refilled), emptied, watchdog, STATUS_SELECT | 5);
                    if (alive) {
                        load_keys(turn + 1);
                    }
                }
            }
        }
    } else {
        // Thread r of the first four warps: the norm of key row r of every panel; every thread: the
        // norm of its query row and half of that row of the products.
        const int row = (warp % 4) * 32 + lane;
        const int half = warp / 4;
        bool alive = __all_sync(0xffffffffu, mbar_wait(query_loaded, 0, watchdog, STATUS_SELECT | 2));
        float inverse_query_norm = 0.0f;
        if (alive) {
            const float query_square = panel_row_square(aligned, row);
            inverse_query_norm = query_square > 0.0f ? rsqrtf(query_square) : 0.0f;
        }
        const float query_factor = inverse_query_norm * COSINE_ONE;
        const int query_tile = first_query + row;
        const uint32_t lane_base = static_cast<uint32_t>((warp % 4) * 32) << 16;
        // Whole 16-byte groups of a row can be stored as such when every row starts on one.
        const bool vector_stores = tiles % 8 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0;
        for (int turn = 0; alive && turn < turns; turn++) {
            const int stage = turn % COSINE_STAGES;
            const uint32_t parity = (turn / COSINE_STAGES) & 1;
            const int first_key = (static_cast<int>(blockIdx.x) + turn * static_cast<int>(gridDim.x)) * PANEL;
            float *norms = inverse_key_norms + stage * PANEL;
            if (half == 0) {
                // The norms of this stage's last panel have been read by every warp once its
                // accumulator is read out.
                alive = __all_sync(0xffffffffu,
                                   mbar_wait(key_loaded(stage), parity, watchdog, STATUS_SELECT | 6) &&
                                       mbar_wait(read_out(stage), parity ^ 1, watchdog,
                                                 STATUS_SELECT | 7));
                if (!alive) {
                    break;
                }
                const float key_square =
                    panel_row_square(aligned + COSINE_SMEM_KEYS + stage * PANEL_BYTES, row);
                norms[row] = key_square > 0.0f ? rsqrtf(key_square) : 0.0f;
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(norms_written(stage));
                    mbar_arrive(key_free(stage));
                }
            }
            alive = __all_sync(0xffffffffu,
                               mbar_wait(norms_written(stage), parity, watchdog, STATUS_SELECT | 8) &&
                                   mbar_wait(multiplied(stage), parity, watchdog, STATUS_SELECT | 3));
            if (!alive) {
                break;
            }
            tcgen05_fence_after();
            uint16_t *slots = table + (static_cast<size_t>(head) * tiles + query_tile) * tiles + first_key;
            #pragma unroll
            for (int chunk = half * 2; chunk < half * 2 + 2; chunk++) {
                uint32_t values[32];
                tmem_load_32(tmem + lane_base + stage * PANEL + chunk * 32, values);
                tmem_wait_load();
                // product / (|q| |k|) * 32767, rounded, the two of a pair saturated into 16 bits
                // each by one instruction (a cosine is within a rounding of +-1 already).
                uint32_t packed[16];
                #pragma unroll
                for (int four = 0; four < 8; four++) {
                    const float4 key_norms =
                        *reinterpret_cast<const float4 *>(norms + chunk * 32 + four * 4);
                    const float inverse[4] = {key_norms.x, key_norms.y, key_norms.z, key_norms.w};
                    int fractions[4];
                    #pragma unroll
                    for (int index = 0; index < 4; index++) {
                        fractions[index] = __float2int_rn(__uint_as_float(values[four * 4 + index]) *
                                                          query_factor * inverse[index]);
                    }
                    #pragma unroll
                    for (int pair = 0; pair < 2; pair++) {
                        asm("cvt.pack.sat.s16.s32 %0, %1, %2;"
                            : "=r"(packed[four * 2 + pair])
                            : "r"(fractions[pair * 2 + 1]), "r"(fractions[pair * 2]));
                    }
                }
                if (query_tile < tiles) {
                    const int column = first_key + chunk * 32;
                    if (vector_stores && column + 32 <= tiles) {
                        uint4 *destination = reinterpret_cast<uint4 *>(slots + chunk * 32);
                        #pragma unroll
                        for (int part = 0; part < 4; part++) {
                            destination[part] = make_uint4(packed[part * 4], packed[part * 4 + 1],
                                                           packed[part * 4 + 2],
                                                           packed[part * 4 + 3]);
                        }
                    } else {
                        #pragma unroll
                        for (int index = 0; index < 32; index++) {
                            if (column + index < tiles) {
                                slots[chunk * 32 + index] = static_cast<uint16_t>(
                                    packed[index / 2] >> (16 * (index % 2)));
                            }
                        }
                    }
                }
            }
            // This warp is done with the accumulator and with the stage's norms.
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(read_out(stage));
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == COSINE_STORING_WARPS) {
        if (*abort_flag != 0) {
            for (int spin = 0; spin < 64; spin++) {
                __nanosleep(1000);
            }
        }
        tcgen05_fence_after();
        tmem_dealloc(tmem, COSINE_STAGES * PANEL);
    }
}

// ---------------------------------------------------------------------------------------------
// 2. Routes from the cosines.

constexpr int ROUTE_WARPS = 8;
constexpr int ROUTE_THREADS = ROUTE_WARPS * 32;
constexpr int BINS = 512;
constexpr int LISTED = 1024; // open tiles a warp can list; a row with more is scored whole
// |approximate - exact| <= BOUND * |q| |k| * scale. Operands cut to TF32 are each off by less
// than 2^-10 of themselves, so a product by less than 2^-8.99 of its size, and the sum of the 128
// sizes is at most |q| |k|; the FP32 accumulation, the 16-bit cosine (2^-16) and the rounding of
// the exact evaluation itself add less than 2^-13 together. 2^-8 leaves a factor of 1.8.
constexpr float BOUND = 0.00390625f;
// A tile's fate once its approximate score is placed: certain tiles carry it in the row of scores
// itself, as an infinity that any threshold among the open ones sorts the right way.
constexpr uint32_t KEPT_BITS = 0x7f800000u, DROPPED_BITS = 0xff800000u;

// The open tiles of a row: those listed, or, when the whole row is open, every video tile.
struct OpenTiles {
    const uint16_t *list;
    int first_video_tile;
    __device__ __forceinline__ int operator[](int index) const {
        return list != nullptr ? list[index] : first_video_tile + index;
    }
};

__device__ __forceinline__ uint32_t order_preserving(float value) {
    const uint32_t bits = __float_as_uint(value);
    return bits ^ ((bits >> 31) ? 0xffffffffu : 0x80000000u);
}

__device__ __forceinline__ float warp_sum(float value) {
    #pragma unroll
    for (int offset = 16; offset > 0; offset /= 2) {
        value += __shfl_xor_sync(0xffffffffu, value, offset);
    }
    return value;
}

// The pooled scores of eight tiles in the reference's FP32 order, by a whole warp: lane l holds
// dimensions l, l + 32, l + 64, l + 96 of the query and reads the same of each key (coalesced
// loads, all eight tiles' in flight together: a route's open tiles are scattered over a head's
// megabyte of means, and one tile at a time would wait for L2 a hundred times a row), chains four
// fused multiply-adds from zero, and a xor butterfly from bit 4 down to bit 0 adds the 32 chains
// in the reference's tree. The butterfly narrows as it goes: at bit 4 a lane keeps four of the
// eight tiles' sums and hands the other four to its partner, at bit 3 two, at bit 2 one, so that
// each sum is still the one the full butterfly leaves in that lane (an addition commutes) at 9
// exchanges instead of 40. Lane l ends with the score of tile (l / 4) % 8 of the eight.
// In three steps, so that the next eight tiles' loads can go between the second and the third.
constexpr int EXACT_BATCH = 8;
// Lane l's dimensions l, l + 32, l + 64, l + 96 of the key means of the tiles first .. first + 7
// of `tiles` (the last one again past `count`).
__device__ __forceinline__ void load_open_keys(const float *__restrict__ head_keys,
                                               const OpenTiles &tiles, int first, int count,
                                               int lane, float (&loaded)[EXACT_BATCH][4]) {
    #pragma unroll
    for (int index = 0; index < EXACT_BATCH; index++) {
        const int listed = min(first + index, count - 1);
        const float *key = head_keys + static_cast<size_t>(tiles[listed]) * HEAD_DIM + lane;
        #pragma unroll
        for (int part = 0; part < 4; part++) {
            loaded[index][part] = __ldg(key + part * 32);
        }
    }
}
// This lane's chains of the eight tiles.
__device__ __forceinline__ void chain_sums(const float (&query)[4],
                                           const float (&loaded)[EXACT_BATCH][4],
                                           float (&eight)[EXACT_BATCH]) {
    #pragma unroll
    for (int index = 0; index < EXACT_BATCH; index++) {
        float chain = 0.0f;
        #pragma unroll
        for (int part = 0; part < 4; part++) {
            chain = __fmaf_rn(query[part], loaded[index][part], chain);
        }
        eight[index] = chain;
    }
}
// The narrowing butterfly over the eight tiles' chains: the score of tile (lane / 4) % 8.
__device__ __forceinline__ float narrowed_score(const float (&eight)[EXACT_BATCH], int lane,
                                                float scale) {
    return __fmul_rn(narrowed_sum(eight, lane), scale);
}

// Among the `count` tiles listed in `list`, whose exact scores are in `values`: the order-preserving
// bits of the `wanted`-th largest score, and how many of the tiles equal to it belong to the
// `wanted` largest. One byte of the bits at a time from the top; `bins` is 256 counters.
__device__ __forceinline__ void select_among(const OpenTiles &list, int count, const float *values,
                                             int wanted, int *bins, int lane, uint32_t &threshold,
                                             int &ties) {
    uint32_t settled = 0;
    threshold = 0;
    ties = wanted;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int bin = lane; bin < 256; bin += 32) {
            bins[bin] = 0;
        }
        __syncwarp();
        for (int first = 0; first < count; first += 32) {
            const int index = first + lane;
            const uint32_t bits = index < count ? order_preserving(values[list[index]]) : 0;
            const bool counted = index < count && (bits & settled) == threshold;
            // Equal scores crowd into one counter: the lanes that share one add their number once.
            const uint32_t digit = counted ? (bits >> shift) & 255u : 256u;
            const unsigned same = __match_any_sync(0xffffffffu, digit);
            if (counted && lane == __ffs(same) - 1) {
                bins[digit] += __popc(same);
            }
            __syncwarp();
        }
        // Lane l looks after counters 255 - 8 l down to 248 - 8 l, so that lane order is score
        // order; `before` is how many candidates sit in counters above this lane's.
        int own[8];
        int total = 0;
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            own[index] = bins[255 - (lane * 8 + index)];
            total += own[index];
        }
        int before = total;
        #pragma unroll
        for (int offset = 1; offset < 32; offset *= 2) {
            const int other = __shfl_up_sync(0xffffffffu, before, offset);
            if (lane >= offset) {
                before += other;
            }
        }
        before -= total;
        int digit = -1, passed = 0;
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            if (digit < 0 && before + own[index] >= ties) {
                digit = 255 - (lane * 8 + index);
                passed = before;
            }
            before += own[index];
        }
        const int holder = __ffs(__ballot_sync(0xffffffffu, digit >= 0)) - 1;
        digit = __shfl_sync(0xffffffffu, digit, max(holder, 0));
        passed = __shfl_sync(0xffffffffu, passed, max(holder, 0));
        ties -= passed;
        threshold |= static_cast<uint32_t>(digit & 255) << shift;
        settled |= 255u << shift;
        __syncwarp();
    }
}

__global__ void __launch_bounds__(ROUTE_THREADS, 2)
    route_kernel(Mmh3VsaWorkspace workspace, int tiles, int prefix_tiles, int kept, float scale) {
    // [tiles] key norms, then per warp: [tiles] scores, [BINS] counters, [LISTED] tile numbers.
    extern __shared__ __align__(16) uint8_t route_memory[];
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    const int head = blockIdx.y;
    const int padded = (tiles + 3) & ~3;
    float *key_norms = reinterpret_cast<float *>(route_memory);
    uint8_t *mine = route_memory + padded * 4 +
                    static_cast<size_t>(warp) * (padded * 4 + BINS * 4 + LISTED * 2);
    float *values = reinterpret_cast<float *>(mine);
    int *bins = reinterpret_cast<int *>(mine + padded * 4);
    uint16_t *list = reinterpret_cast<uint16_t *>(mine + padded * 4 + BINS * 4);
    __shared__ float warp_maxima[ROUTE_WARPS];

    const float *head_keys = workspace.pooled_key + static_cast<size_t>(head) * tiles * HEAD_DIM;
    const int video_tiles = tiles - prefix_tiles;

    // The norms of this head's key means, a warp to a tile and eight tiles' loads in flight,
    // and the largest of them.
    float largest = 0.0f;
    for (int first = warp * 8; first < tiles; first += ROUTE_WARPS * 8) {
        float4 loaded[8];
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            const int tile = min(first + index, tiles - 1);
            loaded[index] = __ldg(
                reinterpret_cast<const float4 *>(head_keys + static_cast<size_t>(tile) * HEAD_DIM) +
                lane);
        }
        float squares[8];
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            const float4 four = loaded[index];
            squares[index] =
                fmaf(four.x, four.x, fmaf(four.y, four.y, fmaf(four.z, four.z, four.w * four.w)));
        }
        #pragma unroll
        for (int offset = 16; offset > 0; offset /= 2) {
            #pragma unroll
            for (int index = 0; index < 8; index++) {
                squares[index] += __shfl_xor_sync(0xffffffffu, squares[index], offset);
            }
        }
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            const float norm = sqrtf(squares[index]);
            if (lane == index && first + index < tiles) {
                key_norms[first + index] = norm;
            }
            largest = fmaxf(largest, norm);
        }
    }
    if (lane == 0) {
        warp_maxima[warp] = largest;
    }
    __syncthreads();
    largest = warp_maxima[0];
    #pragma unroll
    for (int other = 1; other < ROUTE_WARPS; other++) {
        largest = fmaxf(largest, warp_maxima[other]);
    }

    // The CTAs of a head share its query tiles round robin, a warp to a tile.
    for (int query_tile = blockIdx.x * ROUTE_WARPS + warp; query_tile < tiles;
         query_tile += gridDim.x * ROUTE_WARPS) {
        const size_t row = static_cast<size_t>(head) * tiles + query_tile;
        uint16_t *route = workspace.routes + row * tiles;
        if (query_tile < prefix_tiles || kept >= video_tiles) {
            // Every tile, in order.
            for (int tile = lane; tile < tiles; tile += 32) {
                route[tile] = static_cast<uint16_t>(tile);
            }
            if (lane == 0) {
                workspace.route_counts[row] = tiles;
            }
            continue;
        }
        float query[4];
        float square = 0.0f;
        #pragma unroll
        for (int part = 0; part < 4; part++) {
            query[part] = __ldg(workspace.pooled_query + row * HEAD_DIM + lane + part * 32);
            square = fmaf(query[part], query[part], square);
        }
        const float query_norm = sqrtf(warp_sum(square));
        const float unit = query_norm * scale / COSINE_ONE;
        const float bound = BOUND * query_norm * largest * scale;

        // The approximate scores of the video tiles, counted into BINS equal steps down from the
        // largest value a score of this row can have.
        const float reach = query_norm * largest * scale;
        const float step = 2.0f * reach / BINS;
        float keep_above = FLT_MAX, drop_below = -FLT_MAX;
        const bool binned = step > 0.0f && step < FLT_MAX;
        if (binned) {
            const float steps_per_unit = 1.0f / step;
            for (int bin = lane; bin < BINS; bin += 32) {
                bins[bin] = 0;
            }
            __syncwarp();
            // Eight of a lane's cosines are read before any is used: the row comes from L2.
            for (int first = prefix_tiles + lane; first < tiles; first += 8 * 32) {
                uint16_t cosines[8];
                #pragma unroll
                for (int index = 0; index < 8; index++) {
                    const int tile = first + index * 32;
                    cosines[index] = tile < tiles ? route[tile] : 0;
                }
                #pragma unroll
                for (int index = 0; index < 8; index++) {
                    const int tile = first + index * 32;
                    if (tile < tiles) {
                        const float value = static_cast<float>(static_cast<int16_t>(cosines[index])) *
                                            (unit * key_norms[tile]);
                        values[tile] = value;
                        const int bin = static_cast<int>((reach - value) * steps_per_unit);
                        atomicAdd(&bins[min(max(bin, 0), BINS - 1)], 1);
                    }
                }
            }
            __syncwarp();
            // Which bin holds the kept-th largest: lane l owns bins 16 l .. 16 l + 15, and
            // `before` counts the scores in the bins above its own.
            int total = 0;
            for (int index = 0; index < BINS / 32; index++) {
                total += bins[lane * (BINS / 32) + index];
            }
            int before = total;
            #pragma unroll
            for (int offset = 1; offset < 32; offset *= 2) {
                const int other = __shfl_up_sync(0xffffffffu, before, offset);
                if (lane >= offset) {
                    before += other;
                }
            }
            before -= total;
            int found = -1;
            for (int index = 0; index < BINS / 32; index++) {
                const int held = bins[lane * (BINS / 32) + index];
                if (found < 0 && before + held >= kept) {
                    found = lane * (BINS / 32) + index;
                }
                before += held;
            }
            const int holder = __ffs(__ballot_sync(0xffffffffu, found >= 0)) - 1;
            found = __shfl_sync(0xffffffffu, found, max(holder, 0));
            if (holder >= 0) {
                // A bin to either side allows for the rounding of the binning itself.
                keep_above = reach - static_cast<float>(found - 1) * step + 2.0f * bound;
                drop_below = reach - static_cast<float>(found + 2) * step - 2.0f * bound;
            }
            __syncwarp();
        }

        // Every tile's fate, and the open ones listed in ascending order: a certain tile's score
        // gives way to the infinity that stands for its fate. Everything is open when the scores
        // could not be binned, the counts do not add up or the list overflows.
        // A bit per video tile says that it is kept: 32 consecutive tiles to a word, in the upper
        // half of the counters, which the binning is done with.
        uint32_t *kept_words = reinterpret_cast<uint32_t *>(bins + BINS / 2);
        const int words = (video_tiles + 31) / 32;
        int certain = 0, listed = 0;
        for (int first = prefix_tiles; first < tiles; first += 32) {
            const int tile = first + lane;
            bool kept_for_certain = false, open = false;
            if (tile < tiles) {
                const float value = binned ? values[tile] : 0.0f;
                kept_for_certain = value > keep_above;
                open = !kept_for_certain && !(value < drop_below);
                if (!open) {
                    values[tile] = __uint_as_float(kept_for_certain ? KEPT_BITS : DROPPED_BITS);
                }
            }
            const unsigned kept_mask = __ballot_sync(0xffffffffu, kept_for_certain);
            if (lane == 0) {
                kept_words[(first - prefix_tiles) / 32] = kept_mask;
            }
            certain += __popc(kept_mask);
            const unsigned open_mask = __ballot_sync(0xffffffffu, open);
            const int slot = listed + __popc(open_mask & ((1u << lane) - 1));
            if (open && slot < LISTED) {
                list[slot] = static_cast<uint16_t>(tile);
            }
            listed += __popc(open_mask);
        }
        OpenTiles open_tiles = {list, prefix_tiles};
        if (kept - certain < 1 || kept - certain > listed || listed > LISTED) {
            open_tiles.list = nullptr;
            certain = 0;
            listed = video_tiles;
            for (int word = lane; word < words; word += 32) {
                kept_words[word] = 0;
            }
        }
        __syncwarp();

        // The open tiles scored exactly, eight at a time; the first of the four lanes that end
        // with a tile's score puts it in the tile's place.
        // The next eight tiles' loads go out as soon as these eight's chains are summed, ahead of
        // the butterfly.
        if (listed > 0) {
            float loaded[EXACT_BATCH][4];
            load_open_keys(head_keys, open_tiles, 0, listed, lane, loaded);
            for (int first = 0; first < listed; first += EXACT_BATCH) {
                float eight[EXACT_BATCH];
                chain_sums(query, loaded, eight);
                const int index = first + lane / 4;
                const int own_tile = open_tiles[min(index, listed - 1)];
                if (first + EXACT_BATCH < listed) {
                    load_open_keys(head_keys, open_tiles, first + EXACT_BATCH, listed, lane, loaded);
                }
                const float score = narrowed_score(eight, lane, scale);
                if (lane % 4 == 0 && index < listed) {
                    values[own_tile] = score;
                }
            }
        }
        __syncwarp();
        uint32_t threshold;
        int ties;
        select_among(open_tiles, listed, values, kept - certain, bins, lane, threshold, ties);

        // Of the open tiles those above the threshold and the first `ties` at it join the kept
        // ones: the list is in ascending order, so ties go to the lower index.
        int ties_seen = 0;
        for (int first = 0; first < listed; first += 32) {
            const int index = first + lane;
            int tile = prefix_tiles;
            bool keep = false, tie = false;
            if (index < listed) {
                tile = open_tiles[index];
                const uint32_t bits = order_preserving(values[tile]);
                keep = bits > threshold;
                tie = bits == threshold;
            }
            const unsigned tie_mask = __ballot_sync(0xffffffffu, tie);
            if (tie && ties_seen + __popc(tie_mask & ((1u << lane) - 1)) < ties) {
                keep = true;
            }
            ties_seen += __popc(tie_mask);
            if (keep) {
                atomicOr(&kept_words[(tile - prefix_tiles) / 32], 1u << ((tile - prefix_tiles) % 32));
            }
        }
        __syncwarp();

        // The route: the prefix tiles, then the set bits in ascending order, a lane to a word. The
        // list lands on the cosines it was computed from, which are all read by now.
        for (int tile = lane; tile < prefix_tiles; tile += 32) {
            route[tile] = static_cast<uint16_t>(tile);
        }
        int count = prefix_tiles;
        for (int first = 0; first < words; first += 32) {
            const int index = first + lane;
            uint32_t word = index < words ? kept_words[index] : 0u;
            const int own = __popc(word);
            int before = own;
            #pragma unroll
            for (int offset = 1; offset < 32; offset *= 2) {
                const int other = __shfl_up_sync(0xffffffffu, before, offset);
                if (lane >= offset) {
                    before += other;
                }
            }
            const int total = __shfl_sync(0xffffffffu, before, 31);
            int position = count + before - own;
            while (word != 0) {
                const int bit = __ffs(word) - 1;
                word &= word - 1;
                route[position++] = static_cast<uint16_t>(prefix_tiles + index * 32 + bit);
            }
            count += total;
        }
        if (lane == 0) {
            workspace.route_counts[row] = count;
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------
// 3. The coarse output of a gated layer: softmax over all tiles of the pooled scores, times the
// tiles' mean values (the workspace holds their sums).

constexpr int COARSE_WARPS = 8;
constexpr int COARSE_QUERIES = 8;                      // query tiles to a warp
constexpr int COARSE_KEYS = 32 / COARSE_QUERIES;       // key tiles to a butterfly
constexpr int COARSE_CHUNK = 32;    // key tiles staged at a time, twice over
constexpr int COARSE_STAGE = 2 * COARSE_CHUNK * HEAD_DIM; // floats: the chunk's key means, its value sums

// 16 bytes from global to shared memory without passing through registers; a thread's copies
// complete, in order, by the time its wait returns.
__device__ __forceinline__ void copy_16_bytes_async(float *destination, const float *source) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(destination)),
                 "l"(source)
                 : "memory");
}
__device__ __forceinline__ void wait_for_own_copies() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// The sums over the 32 lanes of 32 values a lane, one sum to a lane: a xor butterfly that halves
// what a lane holds at every step (16 + 8 + 4 + 2 + 1 exchanges). Lane l ends with the sum of
// value l: at the step over lane bit b a lane keeps the values whose own bit b equals the lane's.
template <int HALF>
__device__ __forceinline__ void halve_to_own_lanes(float (&values)[32], int lane) {
    const bool upper = lane & HALF;
    #pragma unroll
    for (int index = 0; index < HALF; index++) {
        const float kept = upper ? values[HALF + index] : values[index];
        const float handed = upper ? values[index] : values[HALF + index];
        values[index] = kept + __shfl_xor_sync(0xffffffffu, handed, HALF);
    }
}
__device__ __forceinline__ float sum_to_own_lane(float (&values)[32], int lane) {
    halve_to_own_lanes<16>(values, lane);
    halve_to_own_lanes<8>(values, lane);
    halve_to_own_lanes<4>(values, lane);
    halve_to_own_lanes<2>(values, lane);
    halve_to_own_lanes<1>(values, lane);
    return values[0];
}

// A CTA of eight warps takes 64 query tiles of a head, a warp eight of them, and walks the head's
// tiles 32 at a time through two stages of shared memory (asynchronous copies, the next chunk on
// its way while this one is used). Scores: lane l keeps dimensions 4 l .. 4 l + 3 of its warp's
// eight query means in registers (times scale and log2 e), reads the same dimensions of a key
// mean, and the 32 partial products of eight queries with four keys go through one halving
// butterfly, which leaves lane l the score of query l / 4 against key l % 4 of the four. Softmax:
// online, a lane over its query's eight scores of the chunk and the four lanes of a query
// together. Values: the weights (over the tiles' lengths: the workspace holds sums, not means) go
// through shared memory, eight queries' side by side, and a lane accumulates its four dimensions
// of the eight outputs.
__global__ void __launch_bounds__(COARSE_WARPS * 32, 2)
    coarse_kernel(Mmh3VsaWorkspace workspace, int tiles, float scale) {
    extern __shared__ __align__(16) float coarse_memory[];
    // Two stages, then per warp [COARSE_CHUNK][COARSE_QUERIES] weights and [COARSE_QUERIES]
    // corrections, then [tiles] inverse lengths.
    float *stages = coarse_memory;
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    float *weights = coarse_memory + 2 * COARSE_STAGE +
                     warp * (COARSE_CHUNK + 1) * COARSE_QUERIES;
    float *corrections = weights + COARSE_CHUNK * COARSE_QUERIES;
    float *inverse_lengths =
        coarse_memory + 2 * COARSE_STAGE + COARSE_WARPS * (COARSE_CHUNK + 1) * COARSE_QUERIES;
    const int head = blockIdx.y;
    const size_t head_rows = static_cast<size_t>(head) * tiles;
    const int first_query = (blockIdx.x * COARSE_WARPS + warp) * COARSE_QUERIES;
    const float *head_keys = workspace.pooled_key + head_rows * HEAD_DIM;
    const float *head_values = workspace.pooled_value + head_rows * HEAD_DIM;

    // A chunk's rows are contiguous in both arrays: 2 * 32 * 32 16-byte pieces, eight to a thread.
    const auto stage_chunk = [&](int chunk) {
        float *stage = stages + (chunk % 2) * COARSE_STAGE;
        const int first = chunk * COARSE_CHUNK;
        #pragma unroll
        for (int turn = 0; turn < 2 * COARSE_CHUNK * (HEAD_DIM / 4) / (COARSE_WARPS * 32); turn++) {
            const int piece = turn * COARSE_WARPS * 32 + static_cast<int>(threadIdx.x);
            const int row = (piece / (HEAD_DIM / 4)) % COARSE_CHUNK;
            const bool values = piece >= COARSE_CHUNK * (HEAD_DIM / 4);
            if (first + row < tiles) {
                copy_16_bytes_async(stage + piece * 4,
                                    (values ? head_values : head_keys) +
                                        static_cast<size_t>(first + row) * HEAD_DIM +
                                        (piece % (HEAD_DIM / 4)) * 4);
            } else {
                // Past the last tile: zeros, which a weight of zero leaves zero.
                *reinterpret_cast<float4 *>(stage + piece * 4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    };
    stage_chunk(0);
    for (int tile = threadIdx.x; tile < tiles; tile += COARSE_WARPS * 32) {
        inverse_lengths[tile] = 1.0f / static_cast<float>(workspace.tile_lengths[tile]);
    }
    float4 queries[COARSE_QUERIES];
    const float factor = scale * LOG2_E;
    #pragma unroll
    for (int query = 0; query < COARSE_QUERIES; query++) {
        float4 four = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (first_query + query < tiles) {
            four = __ldg(reinterpret_cast<const float4 *>(
                             workspace.pooled_query + (head_rows + first_query + query) * HEAD_DIM) +
                         lane);
        }
        queries[query] = make_float4(four.x * factor, four.y * factor, four.z * factor, four.w * factor);
    }
    // This lane's query (lane / 4) and its keys of a chunk (lane % 4 of every four).
    float maximum = -FLT_MAX, sum = 0.0f;
    float4 outputs[COARSE_QUERIES];
    #pragma unroll
    for (int query = 0; query < COARSE_QUERIES; query++) {
        outputs[query] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    const int chunks = (tiles + COARSE_CHUNK - 1) / COARSE_CHUNK;
    for (int chunk = 0; chunk < chunks; chunk++) {
        wait_for_own_copies();
        __syncthreads();
        if (chunk + 1 < chunks) {
            stage_chunk(chunk + 1);
        }
        const float4 *keys = reinterpret_cast<const float4 *>(stages + (chunk % 2) * COARSE_STAGE);
        const float4 *values = keys + COARSE_CHUNK * (HEAD_DIM / 4);
        const int first = chunk * COARSE_CHUNK;

        float scores[COARSE_CHUNK / COARSE_KEYS];
        #pragma unroll
        for (int group = 0; group < COARSE_CHUNK / COARSE_KEYS; group++) {
            float partial[32];
            #pragma unroll
            for (int key = 0; key < COARSE_KEYS; key++) {
                const float4 four = keys[(group * COARSE_KEYS + key) * (HEAD_DIM / 4) + lane];
                #pragma unroll
                for (int query = 0; query < COARSE_QUERIES; query++) {
                    partial[query * COARSE_KEYS + key] =
                        fmaf(queries[query].w, four.w,
                             fmaf(queries[query].z, four.z,
                                  fmaf(queries[query].y, four.y, queries[query].x * four.x)));
                }
            }
            const float score = sum_to_own_lane(partial, lane);
            scores[group] =
                first + group * COARSE_KEYS + lane % COARSE_KEYS < tiles ? score : -FLT_MAX;
        }
        // The chunk's maximum for this lane's query, over the lane's eight keys and the four lanes.
        float chunk_maximum = scores[0];
        #pragma unroll
        for (int group = 1; group < COARSE_CHUNK / COARSE_KEYS; group++) {
            chunk_maximum = fmaxf(chunk_maximum, scores[group]);
        }
        #pragma unroll
        for (int reach = 1; reach < COARSE_KEYS; reach *= 2) {
            chunk_maximum = fmaxf(chunk_maximum, __shfl_xor_sync(0xffffffffu, chunk_maximum, reach));
        }
        const float raised = fmaxf(maximum, chunk_maximum);
        const float correction = exp2f(maximum - raised);
        maximum = raised;
        float chunk_sum = 0.0f;
        #pragma unroll
        for (int group = 0; group < COARSE_CHUNK / COARSE_KEYS; group++) {
            const int key = group * COARSE_KEYS + lane % COARSE_KEYS;
            const float weight = first + key < tiles ? exp2f(scores[group] - maximum) : 0.0f;
            chunk_sum += weight;
            weights[key * COARSE_QUERIES + lane / COARSE_KEYS] =
                weight * inverse_lengths[min(first + key, tiles - 1)];
        }
        #pragma unroll
        for (int reach = 1; reach < COARSE_KEYS; reach *= 2) {
            chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, reach);
        }
        sum = sum * correction + chunk_sum;
        if (lane % COARSE_KEYS == 0) {
            corrections[lane / COARSE_KEYS] = correction;
        }
        __syncwarp();
        {
            float all[COARSE_QUERIES];
            #pragma unroll
            for (int four = 0; four < COARSE_QUERIES / 4; four++) {
                const float4 loaded = *reinterpret_cast<const float4 *>(corrections + four * 4);
                all[four * 4] = loaded.x, all[four * 4 + 1] = loaded.y;
                all[four * 4 + 2] = loaded.z, all[four * 4 + 3] = loaded.w;
            }
            #pragma unroll
            for (int query = 0; query < COARSE_QUERIES; query++) {
                outputs[query].x *= all[query];
                outputs[query].y *= all[query];
                outputs[query].z *= all[query];
                outputs[query].w *= all[query];
            }
        }
        #pragma unroll 4
        for (int key = 0; key < COARSE_CHUNK; key++) {
            const float4 four = values[key * (HEAD_DIM / 4) + lane];
            float all[COARSE_QUERIES];
            #pragma unroll
            for (int four = 0; four < COARSE_QUERIES / 4; four++) {
                const float4 loaded =
                    *reinterpret_cast<const float4 *>(weights + key * COARSE_QUERIES + four * 4);
                all[four * 4] = loaded.x, all[four * 4 + 1] = loaded.y;
                all[four * 4 + 2] = loaded.z, all[four * 4 + 3] = loaded.w;
            }
            #pragma unroll
            for (int query = 0; query < COARSE_QUERIES; query++) {
                outputs[query].x = fmaf(all[query], four.x, outputs[query].x);
                outputs[query].y = fmaf(all[query], four.y, outputs[query].y);
                outputs[query].z = fmaf(all[query], four.z, outputs[query].z);
                outputs[query].w = fmaf(all[query], four.w, outputs[query].w);
            }
        }
        __syncwarp();
    }
    #pragma unroll
    for (int query = 0; query < COARSE_QUERIES; query++) {
        const float inverse = 1.0f / __shfl_sync(0xffffffffu, sum, query * COARSE_KEYS);
        if (first_query + query < tiles) {
            reinterpret_cast<float4 *>(workspace.coarse +
                                       (head_rows + first_query + query) * HEAD_DIM)[lane] =
                make_float4(outputs[query].x * inverse, outputs[query].y * inverse,
                            outputs[query].z * inverse, outputs[query].w * inverse);
        }
    }
}

size_t coarse_shared_bytes(int tiles) {
    return sizeof(float) * (2 * COARSE_STAGE + COARSE_WARPS * (COARSE_CHUNK + 1) * COARSE_QUERIES +
                            static_cast<size_t>(tiles));
}

size_t route_shared_bytes(int tiles) {
    const size_t padded = (static_cast<size_t>(tiles) + 3) & ~static_cast<size_t>(3);
    return padded * 4 + ROUTE_WARPS * (padded * 4 + BINS * 4 + LISTED * 2);
}

} // namespace

int launch_select(const Mmh3VsaWorkspace &workspace, int tiles, int heads, int prefix_tiles,
                  int kept, float scale, int coarse, cudaStream_t stream) {
    // The route kernel keeps a row of scores per warp in shared memory.
    const size_t shared = route_shared_bytes(tiles);
    if (shared > 200 * 1024 || tiles > 32 * (BINS / 2)) {
        return INVALID_VALUE; // the second: a bit per tile in half of a warp's counters
    }
    unsigned int *status = status_pointer();
    if (status == nullptr) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    const int video_tiles = tiles - prefix_tiles;
    if (kept < video_tiles) {
        static SharedMemoryOptIn cosine_memory;
        const cudaError_t configured = cosine_memory.ensure(cosine_kernel, COSINE_SMEM_BYTES);
        if (configured != cudaSuccess) {
            return static_cast<int>(configured);
        }
        CosineMaps maps;
        const uint64_t dimensions[3] = {HEAD_DIM, static_cast<uint64_t>(tiles),
                                        static_cast<uint64_t>(heads)};
        const uint64_t strides[2] = {HEAD_DIM * sizeof(float),
                                     static_cast<uint64_t>(tiles) * HEAD_DIM * sizeof(float)};
        const uint32_t box[3] = {32, PANEL, 1};
        if (!encode_tensor_map(&maps.query, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                               workspace.pooled_query, dimensions, strides, box) ||
            !encode_tensor_map(&maps.key, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, workspace.pooled_key,
                               dimensions, strides, box)) {
            return NOT_SUPPORTED;
        }
        // A CTA walks a share of the key panels of its query panel: as few shares as fill the
        // device four times over, so that the last round of CTAs costs little.
        const int panels = (tiles + PANEL - 1) / PANEL;
        const int wanted = 4 * multiprocessor_count();
        const int shares =
            std::max(1, std::min(panels, (wanted + panels * heads - 1) / (panels * heads)));
        cosine_kernel<<<dim3(shares, panels, heads), COSINE_THREADS, COSINE_SMEM_BYTES, stream>>>(
            maps, workspace.routes, tiles, status);
        const cudaError_t launched = cudaGetLastError();
        if (launched != cudaSuccess) {
            return static_cast<int>(launched);
        }
    }
    // The opt-in limit only ever grows, and is per device.
    static std::atomic<size_t> configured[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    if (shared > configured[device].load(std::memory_order_relaxed)) {
        const cudaError_t raised = cudaFuncSetAttribute(
            route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        if (raised != cudaSuccess) {
            return static_cast<int>(raised);
        }
        configured[device].store(shared, std::memory_order_relaxed);
    }
    // Every CTA computes its head's key norms once, so there are only as many CTAs as the device
    // holds at a time (two to an SM), shared out evenly over the heads.
    const int resident = 2 * multiprocessor_count();
    const int per_head = std::max(1, std::min((tiles + ROUTE_WARPS - 1) / ROUTE_WARPS, resident / heads));
    route_kernel<<<dim3(per_head, heads), ROUTE_THREADS, shared, stream>>>(
        workspace, tiles, prefix_tiles, kept, scale);
    cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess || !coarse) {
        return static_cast<int>(launched);
    }
    const size_t coarse_shared = coarse_shared_bytes(tiles);
    if (coarse_shared > 200 * 1024) {
        return INVALID_VALUE;
    }
    static std::atomic<size_t> coarse_configured[MAX_DEVICES];
    if (coarse_shared > coarse_configured[device].load(std::memory_order_relaxed)) {
        const cudaError_t raised =
            cudaFuncSetAttribute(coarse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(coarse_shared));
        if (raised != cudaSuccess) {
            return static_cast<int>(raised);
        }
        coarse_configured[device].store(coarse_shared, std::memory_order_relaxed);
    }
    const int per_cta = COARSE_WARPS * COARSE_QUERIES;
    coarse_kernel<<<dim3((tiles + per_cta - 1) / per_cta, heads), COARSE_WARPS * 32, coarse_shared,
                    stream>>>(workspace, tiles, scale);
    return static_cast<int>(cudaGetLastError());
}

} // namespace mmh3
