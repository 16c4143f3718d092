// Sol-Attn for BF16 heads of 128 on sm_100a: block-sparse attention over blocks of 64 tokens in
// which every query block attends a routed subset of the key blocks token by token and every other
// key block through one pooled term (its mean key against the query block's mean query, weighted
// by its length, carrying its summed values). It computes what the reference's
// mmh3_sparse_attention computes (crates/mmh3-cuda/kernels/sparse_attention.cu:72-586; the
// algorithm is stated in crates/mmh3-core/src/dit/sparse.rs:1-9, 103-234) in five steps:
//
// 1. block statistics: mean query, mean key and summed value of every block (the pooling pass of
//    inputs.cu, shared with VSA);
// 2. centre_keys: per head the mean and variance of the block keys, which are then centred;
// 3. route: per head and query block the pooled scores against every key block, the routed key
//    blocks (score above tau standard deviations, the neighbours, the sinks), and the pooled tail
//    of the rest as an online-softmax state (maximum, weighted sum, weighted values);
// 4. row_offsets: per token and head q . key mean, which moves a row's token-level scores into the
//    centred units of the pooled ones;
// 5. the token attention over the routes (vsa_attention.cu, tcgen05; BF16, or INT8/FP8 over a
//    quantized workspace), merged with the tail.
//
// The routes are bit-identical to the reference's. That fixes the FP32 order of everything a route
// depends on: the block sums run down the rows, the key mean and variance down the blocks, the
// spread of a query block over four butterflies of 32 dimensions each that are then added in
// order, and a pooled score over the tree of pooled_score.cuh. The tail sums are free to differ in
// order and do.
//
// How the routing kernel is cut: a CTA of eight warps takes eight query blocks of a head, a warp
// looking after one block's threshold, route list and tail statistics. While the scores are
// taken, four threads own two key blocks: the blocks' centred means come through a staging buffer
// in shared memory (asynchronous 16-byte copies, the next rows in flight while these are used),
// each of the four threads keeps a quarter of both means in registers and meets the same quarter
// of the eight query means in shared memory, and two exchanges among the four finish the sums.
// Two of the four then decide a block's fate each for the eight queries and cast its vote into
// the bit mask of routed blocks (a ballot is 16 key blocks of one query: half a word of the
// mask). The maxima of the tails come from the stored scores, the weighted values of the tails
// a warp to four key blocks with its loads four groups ahead, and the route lists are expanded
// from the mask words, a lane to a word.
#include <atomic>
#include <cfloat>
#include <cmath>

#include "common.cuh"
#include "pooled_score.cuh"
#include "sm100.cuh"

namespace mmh3 {

namespace {

constexpr int BLOCK = 64;
constexpr int MOST_QUERIES = 8;          // query blocks to a CTA, where their scores fit
constexpr int ROUTE_WARPS = 8;           // each looks after one of them
constexpr int ROUTE_THREADS = ROUTE_WARPS * 32;
constexpr int STEP_KEYS = 16;            // key blocks a warp scores at a time: two to four threads
constexpr int PASS_KEYS = ROUTE_WARPS * STEP_KEYS;

// Tokens in block `block` of a sequence of `tokens`.
__device__ __forceinline__ int tokens_in(int block, int tokens) {
    return min(BLOCK, tokens - block * BLOCK);
}

// One warp per 32 dimensions of a head: lane l walks the block keys of dimension d = 32 w + l down
// the blocks, in order (the sums depend on it), eight rows in flight: their mean, then the keys
// centred in place and their variance.
__global__ void __launch_bounds__(32)
    centre_keys_kernel(float *__restrict__ block_keys, int blocks, float *__restrict__ key_mean,
                       float *__restrict__ key_variance) {
    const int head = blockIdx.y;
    const int dimension = blockIdx.x * 32 + threadIdx.x;
    float *column = block_keys + static_cast<size_t>(head) * blocks * HEAD_DIM + dimension;
    constexpr int ROWS = 8;
    float total = 0.0f;
    for (int first = 0; first < blocks; first += ROWS) {
        float rows[ROWS];
        #pragma unroll
        for (int index = 0; index < ROWS; index++) {
            rows[index] = column[static_cast<size_t>(min(first + index, blocks - 1)) * HEAD_DIM];
        }
        #pragma unroll
        for (int index = 0; index < ROWS; index++) {
            total = first + index < blocks ? __fadd_rn(total, rows[index]) : total;
        }
    }
    const float mean = __fdiv_rn(total, static_cast<float>(blocks));
    float squares = 0.0f;
    for (int first = 0; first < blocks; first += ROWS) {
        float rows[ROWS];
        #pragma unroll
        for (int index = 0; index < ROWS; index++) {
            rows[index] = column[static_cast<size_t>(min(first + index, blocks - 1)) * HEAD_DIM];
        }
        #pragma unroll
        for (int index = 0; index < ROWS; index++) {
            if (first + index < blocks) {
                const float centred = __fsub_rn(rows[index], mean);
                column[static_cast<size_t>(first + index) * HEAD_DIM] = centred;
                squares = __fmaf_rn(centred, centred, squares);
            }
        }
    }
    key_mean[head * HEAD_DIM + dimension] = mean;
    key_variance[head * HEAD_DIM + dimension] = __fdiv_rn(squares, static_cast<float>(blocks));
}

// The block ranges that are always exact: keys every query attends token by token, queries that
// attend every key so.
struct ExactRanges {
    int first_key, keys_end, first_query, queries_end;
    __host__ __device__ bool key(int block) const { return block >= first_key && block < keys_end; }
    __host__ __device__ bool query(int block) const {
        return block >= first_query && block < queries_end;
    }
};

// What the routing kernel is told besides its workspace.
struct RouteTask {
    int tokens, blocks;
    float tau, log2_scale;
    ExactRanges exact;
};

// a + the same value of the lanes 16, 8, 4, 2 and 1 away, in that order.
__device__ __forceinline__ float butterfly_sum(float value) {
    #pragma unroll
    for (int reach = 16; reach != 0; reach >>= 1) {
        value = __fadd_rn(value, __shfl_xor_sync(0xffffffffu, value, reach));
    }
    return value;
}
__device__ __forceinline__ float butterfly_max(float value) {
    #pragma unroll
    for (int reach = 16; reach != 0; reach >>= 1) {
        value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, reach));
    }
    return value;
}

// 16 bytes from global to shared memory without passing through registers; a thread's copies
// complete, in order, by the time its wait returns.
__device__ __forceinline__ void copy_16_bytes_async(float *destination, const float *source) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm100::smem_u32(destination)),
                 "l"(source)
                 : "memory");
}
__device__ __forceinline__ void wait_for_own_copies() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// A row of key means staged in shared memory: 128 values and a pad of four words, and the rows of
// a warp's 16 key blocks in the order 0, 2, 4, .., 14, 1, 3, .., 15, so that the eight fours of
// threads, each reading one word of its own row, meet no bank twice.
constexpr int STAGED_ROW = HEAD_DIM + 4;
constexpr int STAGED_FLOATS = PASS_KEYS * STAGED_ROW;
__device__ __forceinline__ int staged_row(int key) { return key / 2 + 8 * (key % 2); }
// A query mean in shared memory: four runs of 32 values, run c holding dimensions c, c + 4,
// c + 8, ..., each with a pad of four words (four threads read a 16-byte word of their own run each).
constexpr int QUARTER_ROW = HEAD_DIM / 4 + 4;
// Where the score of key block `key` against the CTA's query block `query` lies: 32 consecutive
// key blocks of one query side by side (a warp's stores and loads meet no bank twice), and
// four consecutive key blocks of a query in one 16-byte word.
template <int GROUP>
__device__ __forceinline__ int score_slot(int key, int query) {
    return (key / 32) * (32 * GROUP) + query * 32 + key % 32;
}
// The 16 bits that `votes` has at lanes 4 i and 4 i + 1, side by side.
__device__ __forceinline__ uint32_t two_of_every_four(uint32_t votes) {
    votes &= 0x33333333u;
    votes = (votes | (votes >> 2)) & 0x0f0f0f0fu;
    votes = (votes | (votes >> 4)) & 0x00ff00ffu;
    return (votes | (votes >> 8)) & 0x0000ffffu;
}

// Static shared memory of the routing kernel; the dynamic part holds the scores (a slot for each
// of `words` * 32 key blocks and GROUP queries), the staged key means ([PASS_KEYS][STAGED_ROW],
// later the warps' shares of the tails) and the masks of routed key blocks ([GROUP][words]).
template <int GROUP>
struct __align__(16) RouteShared {
    float query_quarters[GROUP][4][QUARTER_ROW];
    float thresholds[GROUP];
    float maxima[ROUTE_WARPS][GROUP]; // [warp][query]: each warp's share of the tails' maxima
    float sums[ROUTE_WARPS][GROUP];
};

template <int GROUP>
__global__ void __launch_bounds__(ROUTE_THREADS, 2)
    route_kernel(const Mmh3SparseWorkspace workspace, const RouteTask task) {
    const int tokens = task.tokens, blocks = task.blocks;
    const float tau = task.tau, log2_scale = task.log2_scale;
    extern __shared__ __align__(16) float scores[];
    const int words = (blocks + 31) / 32;
    float *staged = scores + static_cast<size_t>(words) * 32 * GROUP;
    uint32_t *masks = reinterpret_cast<uint32_t *>(staged + STAGED_FLOATS);
    __shared__ RouteShared<GROUP> shared;
    const int lane = threadIdx.x % 32;
    const int warp = threadIdx.x / 32;
    const int head = blockIdx.y;
    const int first_query = blockIdx.x * GROUP;
    const size_t head_rows = static_cast<size_t>(head) * blocks;
    const float *head_keys = workspace.block_keys + head_rows * HEAD_DIM;

    // The key means of the 16 key blocks from `first_key` on into this warp's rows of the staging
    // buffer: a row is 512 contiguous bytes, 16 to a lane.
    float *own_rows = staged + warp * STEP_KEYS * STAGED_ROW;
    const auto stage_keys = [&](int first_key) {
        #pragma unroll
        for (int row = 0; row < STEP_KEYS; row++) {
            if (first_key + row < blocks) {
                copy_16_bytes_async(
                    own_rows + staged_row(row) * STAGED_ROW + lane * 4,
                    head_keys + static_cast<size_t>(first_key + row) * HEAD_DIM + lane * 4);
            }
        }
    };
    stage_keys(warp * STEP_KEYS);

    // This warp's query mean into shared memory, and its threshold: tau standard deviations of a
    // query block's pooled scores, from the variance of the block keys along each dimension. Lane
    // l holds dimensions l, l + 32, l + 64, l + 96; each group of 32 is added over a butterfly and
    // the four groups then in order, which is the order the reference's 128 threads add them in.
    for (int slot = warp; slot < GROUP; slot += ROUTE_WARPS) {
        const int own_query = first_query + slot;
        float groups[4];
        #pragma unroll
        for (int group = 0; group < 4; group++) {
            const int dimension = group * 32 + lane;
            const float mean =
                own_query < blocks ? workspace.centroids[(head_rows + own_query) * HEAD_DIM + dimension]
                                   : 0.0f;
            shared.query_quarters[slot][dimension % 4][dimension / 4] = mean;
            groups[group] = __fmul_rn(__fmul_rn(mean, mean),
                                      workspace.key_variance[head * HEAD_DIM + dimension]);
        }
        #pragma unroll
        for (int group = 0; group < 4; group++) {
            groups[group] = butterfly_sum(groups[group]);
        }
        const float spread =
            __fadd_rn(__fadd_rn(__fadd_rn(groups[0], groups[1]), groups[2]), groups[3]);
        if (lane == 0) {
            shared.thresholds[slot] =
                __fmul_rn(tau, sqrtf(__fmaf_rn(__fmul_rn(spread, log2_scale), log2_scale, 1e-6f)));
        }
    }
    __syncthreads();

    // Four threads to two key blocks: thread c of the four holds dimensions c, c + 4, c + 8, ...
    // of both centred means in registers and meets the same dimensions of the eight query means
    // in shared memory. The first two of the four then decide a block's fate each for the eight
    // queries and cast its vote into the bit mask of routed blocks (a warp's votes are 16 key
    // blocks of one query: half a word). The means arrive through the staging buffer (threads
    // reading their own rows straight from global memory would touch a cache line each), and
    // the next 16 rows are on their way while these meet the queries.
    {
        const int four = lane / 4, part = lane % 4;
        uint16_t *half_words = reinterpret_cast<uint16_t *>(masks);
        uint32_t exact_queries = 0;
        #pragma unroll
        for (int query = 0; query < GROUP; query++) {
            exact_queries |= (task.exact.query(first_query + query) ? 1u : 0u) << query;
        }
        for (int first = warp * STEP_KEYS; first < words * 32; first += PASS_KEYS) {
            float2 keys[2][HEAD_DIM / 8];
            wait_for_own_copies();
            __syncwarp();
            #pragma unroll
            for (int key = 0; key < 2; key++) {
                const float *row = own_rows + staged_row(four * 2 + key) * STAGED_ROW + part;
                #pragma unroll
                for (int pair = 0; pair < HEAD_DIM / 8; pair++) {
                    keys[key][pair] = make_float2(row[pair * 8], row[pair * 8 + 4]);
                }
            }
            __syncwarp();
            stage_keys(first + PASS_KEYS);
            // What this thread decides: the first of the two blocks in thread 0, the second in
            // thread 1, nothing in the other two. Bit q of `fated` says that the block is exact
            // for query q whatever its score: a key every query attends so, a neighbour of the
            // query block, a query block that attends every key so.
            const int key_block = first + four * 2 + part;
            const bool decides = part < 2 && key_block < blocks;
            const int ahead = key_block - first_query;
            const uint32_t fated =
                task.exact.key(key_block)
                    ? (1u << GROUP) - 1u
                    : (exact_queries |
                       (ahead >= -1 && ahead <= GROUP ? ((7u << (ahead + 1)) >> 2) & ((1u << GROUP) - 1u)
                                                      : 0u));
            float *slots = scores + score_slot<GROUP>(key_block, 0);
            uint32_t routed = 0;
            #pragma unroll 1
            for (int query = 0; query < GROUP; query++) {
                float both[2];
                score_two_keys(reinterpret_cast<const float4 *>(shared.query_quarters[query][part]),
                               keys, both);
                if (decides) {
                    const float score = __fmul_rn(part == 0 ? both[0] : both[1], log2_scale);
                    slots[query * 32] = score;
                    routed |= (score > shared.thresholds[query] ? 1u : 0u) << query;
                }
            }
            routed = decides ? routed | fated : 0u;
            // A ballot per query: 16 key blocks' votes, which lane q packs into query q's half
            // word of the mask.
            uint32_t votes = 0;
            #pragma unroll
            for (int query = 0; query < GROUP; query++) {
                const uint32_t cast = __ballot_sync(0xffffffffu, (routed >> query) & 1u);
                votes = lane == query ? cast : votes;
            }
            if (lane < GROUP) {
                half_words[(lane * words) * 2 + first / STEP_KEYS] =
                    static_cast<uint16_t>(two_of_every_four(votes));
            }
        }
    }
    __syncthreads();

    // The maxima of what stays in the tails: thread t looks at key blocks t, t + 256, ...
    float maxima[GROUP];
    #pragma unroll
    for (int query = 0; query < GROUP; query++) {
        maxima[query] = -FLT_MAX;
    }
    for (int key_block = threadIdx.x; key_block < blocks; key_block += ROUTE_THREADS) {
        const float *slots = scores + score_slot<GROUP>(key_block, 0);
        #pragma unroll
        for (int query = 0; query < GROUP; query++) {
            const bool routed = (masks[query * words + key_block / 32] >> lane) & 1u;
            maxima[query] = routed ? maxima[query] : fmaxf(maxima[query], slots[query * 32]);
        }
    }
    #pragma unroll
    for (int query = 0; query < GROUP; query++) {
        const float maximum = butterfly_max(maxima[query]);
        if (lane == 0) {
            shared.maxima[warp][query] = maximum;
        }
    }
    __syncthreads();
    #pragma unroll
    for (int query = 0; query < GROUP; query++) {
        float maximum = shared.maxima[0][query];
        #pragma unroll
        for (int other = 1; other < ROUTE_WARPS; other++) {
            maximum = fmaxf(maximum, shared.maxima[other][query]);
        }
        maxima[query] = maximum;
    }

    // The tails: what is not routed, as softmax weights against its maximum, each key block
    // counted once per token it stands for. The weights replace the scores; the slots past the
    // last key block get weight zero.
    float sums[GROUP];
    #pragma unroll
    for (int query = 0; query < GROUP; query++) {
        sums[query] = 0.0f;
    }
    for (int key_block = threadIdx.x; key_block < words * 32; key_block += ROUTE_THREADS) {
        const bool present = key_block < blocks;
        const float length = present ? static_cast<float>(tokens_in(key_block, tokens)) : 0.0f;
        float *slots = scores + score_slot<GROUP>(key_block, 0);
        #pragma unroll
        for (int query = 0; query < GROUP; query++) {
            const bool routed = (masks[query * words + key_block / 32] >> lane) & 1u;
            const float weight =
                routed || !present ? 0.0f : exp2f(slots[query * 32] - maxima[query]);
            slots[query * 32] = weight;
            sums[query] = fmaf(weight, length, sums[query]);
        }
    }
    #pragma unroll
    for (int query = 0; query < GROUP; query++) {
        const float sum = butterfly_sum(sums[query]);
        if (lane == 0) {
            shared.sums[warp][query] = sum;
        }
    }
    __syncthreads();

    // The weighted values of the tails. A warp takes every eighth group of four key blocks: a lane
    // loads four dimensions of their summed values (a row is one coalesced 512-byte load) and the
    // four weights each of the eight query blocks gives them (one 16-byte word a query), and keeps
    // its four dimensions of the eight sums. Routed blocks have weight zero. The warps' shares
    // meet in the staging buffer, which the scores are done with.
    {
        const float4 *values =
            reinterpret_cast<const float4 *>(workspace.value_sums + head_rows * HEAD_DIM) + lane;
        float2 tails[GROUP][2];
        #pragma unroll
        for (int query = 0; query < GROUP; query++) {
            tails[query][0] = tails[query][1] = make_float2(0.0f, 0.0f);
        }
        // The summed values come from L2, hundreds of cycles away, which a few warps a scheduler
        // do not hide: the loads run AHEAD groups before their use.
        constexpr int AHEAD = 4, STRIDE = ROUTE_WARPS * 4;
        float4 rows[AHEAD][4];
        const auto load_group = [&](int first, float4 (&into)[4]) {
            #pragma unroll
            for (int index = 0; index < 4; index++) {
                into[index] = first + index < blocks
                                  ? __ldg(values + static_cast<size_t>(first + index) * (HEAD_DIM / 4))
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        };
        #pragma unroll
        for (int stage = 0; stage < AHEAD; stage++) {
            load_group(warp * 4 + stage * STRIDE, rows[stage]);
        }
        for (int base = warp * 4; base < blocks; base += AHEAD * STRIDE) {
            #pragma unroll
            for (int stage = 0; stage < AHEAD; stage++) {
                const int first = base + stage * STRIDE;
                if (first < blocks) {
                    #pragma unroll
                    for (int query = 0; query < GROUP; query++) {
                        const float4 four =
                            *reinterpret_cast<const float4 *>(scores + score_slot<GROUP>(first, query));
                        const float weights[4] = {four.x, four.y, four.z, four.w};
                        #pragma unroll
                        for (int index = 0; index < 4; index++) {
                            const float2 weight = make_float2(weights[index], weights[index]);
                            const float4 row = rows[stage][index];
                            tails[query][0] =
                                __ffma2_rn(weight, make_float2(row.x, row.y), tails[query][0]);
                            tails[query][1] =
                                __ffma2_rn(weight, make_float2(row.z, row.w), tails[query][1]);
                        }
                    }
                }
                load_group(first + AHEAD * STRIDE, rows[stage]);
            }
        }
        float4 *shares = reinterpret_cast<float4 *>(staged);
        #pragma unroll
        for (int query = 0; query < GROUP; query++) {
            shares[(warp * GROUP + query) * (HEAD_DIM / 4) + lane] = make_float4(
                tails[query][0].x, tails[query][0].y, tails[query][1].x, tails[query][1].y);
        }
        __syncthreads();
        for (int item = threadIdx.x; item < GROUP * HEAD_DIM; item += ROUTE_THREADS) {
            const int query = item / HEAD_DIM;
            float total = staged[item];
            #pragma unroll
            for (int other = 1; other < ROUTE_WARPS; other++) {
                total += staged[other * GROUP * HEAD_DIM + item];
            }
            if (first_query + query < blocks) {
                workspace.tail_values[(head_rows + first_query) * HEAD_DIM + item] = total;
            }
        }
    }

    // The routes of this warp's query blocks: the set bits of a mask in ascending order, a lane to
    // a word.
    for (int slot = warp; slot < GROUP && first_query + slot < blocks; slot += ROUTE_WARPS) {
        const size_t row = head_rows + first_query + slot;
        uint16_t *route = workspace.routes + row * blocks;
        const uint32_t *mask = masks + slot * words;
        int written = 0;
        for (int first = 0; first < words; first += 32) {
            const int index = first + lane;
            uint32_t word = index < words ? mask[index] : 0u;
            // How many key blocks the words before this lane's hold.
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
            int position = written + before - own;
            while (word != 0) {
                const int bit = __ffs(word) - 1;
                word &= word - 1;
                route[position++] = static_cast<uint16_t>(index * 32 + bit);
            }
            written += total;
        }
        if (lane == 0) {
            float sum = shared.sums[0][slot], maximum = shared.maxima[0][slot];
            for (int other = 1; other < ROUTE_WARPS; other++) {
                sum += shared.sums[other][slot];
                maximum = fmaxf(maximum, shared.maxima[other][slot]);
            }
            workspace.route_counts[row] = written;
            workspace.tail_max[row] = maximum;
            workspace.tail_sum[row] = sum;
        }
    }
}

// The dynamic shared memory of route_kernel<GROUP>: a score and a mask bit per key block and
// query, and the staged key means.
template <int GROUP>
size_t route_shared_bytes(int blocks) {
    const size_t words = (blocks + 31) / 32;
    return words * 32 * GROUP * sizeof(float) + STAGED_FLOATS * sizeof(float) +
           GROUP * words * sizeof(uint32_t);
}
constexpr size_t MOST_ROUTE_SHARED = 200 * 1024;

// Launches route_kernel with as many query blocks per CTA as their scores leave room for, halving
// them as the sequence grows, as the reference does (sparse_attention.cu:289-315).
template <int GROUP>
int launch_route_with(const Mmh3SparseWorkspace &workspace, const RouteTask &task, int heads,
                      cudaStream_t stream) {
    const int blocks = task.blocks;
    const size_t shared = route_shared_bytes<GROUP>(blocks);
    if (shared > MOST_ROUTE_SHARED) {
        if constexpr (GROUP > 1) {
            return launch_route_with<GROUP / 2>(workspace, task, heads, stream);
        } else {
            return INVALID_VALUE;
        }
    }
    // The opt-in limit only ever grows, and is per device.
    static std::atomic<size_t> configured[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    if (shared > configured[device].load(std::memory_order_relaxed)) {
        const cudaError_t raised =
            cudaFuncSetAttribute(route_kernel<GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(shared));
        if (raised != cudaSuccess) {
            return static_cast<int>(raised);
        }
        configured[device].store(shared, std::memory_order_relaxed);
    }
    route_kernel<GROUP><<<dim3((blocks + GROUP - 1) / GROUP, heads), ROUTE_THREADS, shared, stream>>>(
        workspace, task);
    return static_cast<int>(cudaGetLastError());
}

int launch_route(const Mmh3SparseWorkspace &workspace, const RouteTask &task, int heads,
                 cudaStream_t stream) {
    return launch_route_with<MOST_QUERIES>(workspace, task, heads, stream);
}

// q . key mean of every token and head, in the units of the exponent: what moves a row's
// token-level scores into the centred units of the pooled ones. A warp keeps a head's key mean in
// registers (lane l dimensions 4 l .. 4 l + 3) and walks tokens with it, one 8-byte load a lane.
constexpr int OFFSET_WARPS = 8;
constexpr int OFFSET_TOKENS = 64; // tokens to a warp

__global__ void __launch_bounds__(OFFSET_WARPS * 32)
    row_offsets_kernel(const __nv_bfloat16 *__restrict__ query, int tokens, int64_t token_stride,
                       int64_t head_stride, const float *__restrict__ key_mean, float log2_scale,
                       float *__restrict__ row_offsets) {
    const int lane = threadIdx.x % 32;
    const int head = blockIdx.y;
    const int first =
        (blockIdx.x * OFFSET_WARPS + static_cast<int>(threadIdx.x) / 32) * OFFSET_TOKENS;
    const float4 mean = reinterpret_cast<const float4 *>(key_mean + head * HEAD_DIM)[lane];
    const __nv_bfloat16 *column = query + head * head_stride + lane * 4;
    // Eight tokens at a time: their loads in flight together, and one narrowing butterfly for the
    // eight sums (lane l ends with the sum of token (l / 4) % 8).
    const int end = min(first + OFFSET_TOKENS, tokens);
    for (int token = first; token < end; token += 8) {
        uint2 loaded[8];
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            loaded[index] = __ldg(reinterpret_cast<const uint2 *>(
                column + static_cast<int64_t>(min(token + index, end - 1)) * token_stride));
        }
        float dots[8];
        #pragma unroll
        for (int index = 0; index < 8; index++) {
            const uint2 four = loaded[index];
            float dot = __uint_as_float(four.x << 16) * mean.x;
            dot = fmaf(__uint_as_float(four.x & 0xffff0000u), mean.y, dot);
            dot = fmaf(__uint_as_float(four.y << 16), mean.z, dot);
            dots[index] = fmaf(__uint_as_float(four.y & 0xffff0000u), mean.w, dot);
        }
        const float dot = narrowed_sum(dots, lane);
        const int own = token + lane / 4;
        if (lane % 4 == 0 && own < end) {
            row_offsets[static_cast<size_t>(head) * tokens + own] = dot * log2_scale;
        }
    }
}

int launch_sparse_attention_aligned(const void *query, const void *key, const void *value,
                                    void *output, int heads, const Mmh3AttentionLayout &layout,
                                    float scale, const RouteTask &task,
                                    const Mmh3SparseWorkspace &workspace,
                                    const Mmh3QuantizedWorkspace *precision, int prepared_inputs,
                                    cudaStream_t stream);

} // namespace

int launch_sparse_attention(const void *query, const void *key, const void *value, void *output,
                            int tokens, int heads, const Mmh3AttentionLayout &layout, float scale,
                            float tau, int sink_key_start, int sink_key_end, int sink_query_start,
                            int sink_query_end, const Mmh3SparseWorkspace &workspace,
                            const Mmh3QuantizedWorkspace *quantized, int inputs_ready,
                            cudaStream_t stream) {
    if (!(scale > 0.0f) || !std::isfinite(scale)) {
        return INVALID_VALUE;
    }
    const int blocks = (tokens + BLOCK - 1) / BLOCK;
    if (blocks > 65535) {
        return NOT_SUPPORTED; // routes are 16-bit block indices
    }
    const float log2_scale = scale * LOG2_E;
    // Operands off TMA's 16-byte grid are gathered into dense arrays once, for every kernel below
    // (the row offsets read q eight bytes at a time, the token attention through TMA).
    StagedOperands staged(stream);
    Mmh3AttentionLayout dense_layout = layout;
    const uint16_t *operands[3] = {static_cast<const uint16_t *>(query),
                                   static_cast<const uint16_t *>(key),
                                   static_cast<const uint16_t *>(value)};
    for (int operand = 0; operand < 3; operand++) {
        const cudaError_t copied =
            staged.stage(operand, operands[operand], tokens, heads, HEAD_DIM,
                         dense_layout.token_stride[operand], dense_layout.head_stride[operand]);
        if (copied != cudaSuccess) {
            return static_cast<int>(copied);
        }
    }
    const RouteTask task = {tokens, blocks, tau, log2_scale,
                            {sink_key_start, sink_key_end, sink_query_start, sink_query_end}};
    return launch_sparse_attention_aligned(operands[QUERY], operands[KEY], operands[VALUE], output,
                                           heads, dense_layout, scale, task, workspace, quantized,
                                           inputs_ready, stream);
}

namespace {

int launch_sparse_attention_aligned(const void *query, const void *key, const void *value,
                                    void *output, int heads, const Mmh3AttentionLayout &layout,
                                    float scale, const RouteTask &task,
                                    const Mmh3SparseWorkspace &workspace,
                                    const Mmh3QuantizedWorkspace *precision, int prepared_inputs,
                                    cudaStream_t stream) {
    const int tokens = task.tokens, blocks = task.blocks;
    const float log2_scale = task.log2_scale;
    const Mmh3QuantizedWorkspace *const quantized = precision;
    const int inputs_ready = prepared_inputs;
    if (!inputs_ready) {
        const int pooled =
            launch_block_statistics(query, key, value, tokens, heads, layout, workspace, stream);
        if (pooled != 0) {
            return pooled;
        }
    }
    centre_keys_kernel<<<dim3(HEAD_DIM / 32, heads), 32, 0, stream>>>(
        workspace.block_keys, blocks, workspace.key_mean, workspace.key_variance);
    if (const int code = launch_route(workspace, task, heads, stream); code != 0) {
        return code;
    }
    const int per_cta = OFFSET_WARPS * OFFSET_TOKENS;
    row_offsets_kernel<<<dim3((tokens + per_cta - 1) / per_cta, heads), OFFSET_WARPS * 32, 0,
                         stream>>>(static_cast<const __nv_bfloat16 *>(query), tokens,
                                   layout.token_stride[QUERY], layout.head_stride[QUERY],
                                   workspace.key_mean, log2_scale, workspace.row_offsets);
    const cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess) {
        return static_cast<int>(launched);
    }
    if (quantized != nullptr) {
        // As the reference does (sparse_attention.cu:577-580): the quantizer's passes that
        // inputs_ready leaves to do, then the INT8/FP8 token attention.
        const int prepared = launch_quantize(query, key, value, tokens, heads, layout, *quantized,
                                             nullptr, nullptr, 0, inputs_ready, stream);
        if (prepared != 0) {
            return prepared;
        }
        return launch_sol_token_attention_quantized(*quantized, output, tokens, heads, layout,
                                                    scale, workspace, stream);
    }
    return launch_sol_token_attention(query, key, value, output, tokens, heads, layout, scale,
                                      workspace, stream);
}

} // namespace

} // namespace mmh3
