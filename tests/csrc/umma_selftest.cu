// Test-only kernel that exercises the tcgen05 building blocks of the attention kernels in
// isolation, on one 128 x 128 x 128 problem per call, so that a failing attention test can be told
// apart from a wrong descriptor:
//
//   scores = A . B^T   A and B K-major in 128-byte-swizzled shared memory (TMA), both from smem
//   output = P . V     P written to tensor memory by the threads (as the softmax does), V from smem
//
// mode 0: BF16 operands, FP32 accumulators, V [keys][dims] MN-major (kind::f16)
// mode 1: INT8 A and B with INT32 accumulators (kind::i8); E4M3 P and V^T [dims][keys] K-major with
//         FP32 accumulators (kind::f8f6f4)
#include "../../mmh3_b200/csrc/common.cuh"
#include "../../mmh3_b200/csrc/sm100.cuh"

namespace {

using namespace sm100;

constexpr int N = 128;
constexpr int THREADS = 160; // four warps own the TMEM lanes, warp 4 loads and issues
constexpr int SMEM_BYTES = 3 * 32768 + 256 + 1024;
constexpr unsigned int STATUS_SELFTEST = 0x00ff0000u;

struct SelftestMaps {
    CUtensorMap a, b, v;
};

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
    selftest_kernel(const __grid_constant__ SelftestMaps maps, const uint32_t *__restrict__ p,
                    uint32_t *__restrict__ scores, float *__restrict__ output,
                    unsigned int *status) {
    extern __shared__ uint8_t shared_memory[];
    const uint32_t base = (smem_u32(shared_memory) + 1023u) & ~1023u;
    uint8_t *aligned = shared_memory + (base - smem_u32(shared_memory));
    const uint32_t barriers = base + 3 * 32768;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + 3 * 32768 + 64);
    volatile uint32_t *abort_flag = tmem_slot + 1;
    const Watchdog watchdog = {abort_flag, status};
    const int warp = threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    // Bytes of one operand tile and of one 128-byte-wide slab of it.
    constexpr int ELEMENT = MODE == 0 ? 2 : 1;
    constexpr int SLABS = N * ELEMENT / 128;
    constexpr int SLAB_BYTES = N * 128;
    constexpr int TILE_BYTES = SLABS * SLAB_BYTES;
    const uint32_t a_tile = base, b_tile = base + 32768, v_tile = base + 65536;

    if (threadIdx.x == 0) {
        mbar_init(barriers + 0, 1);  // tiles loaded
        mbar_init(barriers + 8, 1);  // scores done
        mbar_init(barriers + 16, N); // P written
        mbar_init(barriers + 24, 1); // output done
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_scores = tmem, tmem_p = tmem + 128, tmem_output = tmem + 256;

    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(barriers + 0, 3 * TILE_BYTES);
            for (int slab = 0; slab < SLABS; slab++) {
                const int column = slab * (128 / ELEMENT);
                tma_load_2d(a_tile + slab * SLAB_BYTES, &maps.a, barriers + 0, column, 0);
                tma_load_2d(b_tile + slab * SLAB_BYTES, &maps.b, barriers + 0, column, 0);
                tma_load_2d(v_tile + slab * SLAB_BYTES, &maps.v, barriers + 0, column, 0);
            }
            if (mbar_wait(barriers + 0, 0, watchdog, STATUS_SELFTEST | 1)) {
                tcgen05_fence_after();
                constexpr int K_STEP = MODE == 0 ? 16 : 32; // elements per MMA, 32 bytes
                for (int step = 0; step < N / K_STEP; step++) {
                    const uint32_t offset = (step / 4) * SLAB_BYTES + (step % 4) * 32;
                    const uint64_t a = smem_descriptor(a_tile + offset, 16, 1024);
                    const uint64_t b = smem_descriptor(b_tile + offset, 16, 1024);
                    if (MODE == 0) {
                        mma_f16_ss(tmem_scores, a, b,
                                   instruction_descriptor(ACCUMULATE_F32, FORMAT_BF16, FORMAT_BF16,
                                                          0, 0, N, N),
                                   step > 0);
                    } else {
                        mma_i8_ss(tmem_scores, a, b,
                                  instruction_descriptor(ACCUMULATE_S32, FORMAT_S8, FORMAT_S8, 0, 0,
                                                         N, N),
                                  step > 0);
                    }
                }
                tcgen05_commit(barriers + 8);
                if (mbar_wait(barriers + 16, 0, watchdog, STATUS_SELFTEST | 2)) {
                    tcgen05_fence_after();
                    for (int step = 0; step < N / K_STEP; step++) {
                        if (MODE == 0) {
                            // V [keys][dims]: 16 keys down the rows of both slabs of 64 dims.
                            const uint64_t v =
                                smem_descriptor(v_tile + step * 16 * 128, SLAB_BYTES, 1024);
                            mma_f16_ts(tmem_output, tmem_p + step * 8, v,
                                       instruction_descriptor(ACCUMULATE_F32, FORMAT_BF16,
                                                              FORMAT_BF16, 0, 1, N, N),
                                       step > 0);
                        } else {
                            // V^T [dims][keys]: 32 keys along the row.
                            const uint64_t v = smem_descriptor(v_tile + step * 32, 16, 1024);
                            mma_f8_ts(tmem_output, tmem_p + step * 8, v,
                                      instruction_descriptor(ACCUMULATE_F32, FORMAT_E4M3,
                                                             FORMAT_E4M3, 0, 0, N, N),
                                      step > 0);
                        }
                    }
                    tcgen05_commit(barriers + 24);
                }
            }
        }
    } else {
        const int row = warp * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        // P first: 128 BF16 are 64 columns, 128 E4M3 are 32.
        constexpr int P_WORDS = MODE == 0 ? 64 : 32;
        for (int chunk = 0; chunk < P_WORDS / 32; chunk++) {
            uint32_t words[32];
            for (int index = 0; index < 32; index++) {
                words[index] = p[row * P_WORDS + chunk * 32 + index];
            }
            tmem_store_32(tmem_p + lane_base + chunk * 32, words);
        }
        tmem_wait_store();
        tcgen05_fence_before();
        mbar_arrive(barriers + 16);
        bool alive = mbar_wait(barriers + 8, 0, watchdog, STATUS_SELFTEST | 3);
        alive = __all_sync(0xffffffffu, alive);
        if (alive) {
            tcgen05_fence_after();
            for (int chunk = 0; chunk < 4; chunk++) {
                uint32_t words[32];
                tmem_load_32(tmem_scores + lane_base + chunk * 32, words);
                tmem_wait_load();
                for (int index = 0; index < 32; index++) {
                    scores[row * N + chunk * 32 + index] = words[index];
                }
            }
            alive = mbar_wait(barriers + 24, 0, watchdog, STATUS_SELFTEST | 4);
            alive = __all_sync(0xffffffffu, alive);
        }
        if (alive) {
            tcgen05_fence_after();
            for (int chunk = 0; chunk < 4; chunk++) {
                uint32_t words[32];
                tmem_load_32(tmem_output + lane_base + chunk * 32, words);
                tmem_wait_load();
                for (int index = 0; index < 32; index++) {
                    output[row * N + chunk * 32 + index] = __uint_as_float(words[index]);
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 4) {
        tcgen05_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

} // namespace

// a, b: [128][128] row-major (BF16 in mode 0, INT8 in mode 1). v: mode 0 BF16 [keys][dims],
// mode 1 E4M3 [dims][keys]. p: row-major [128][128] BF16 or E4M3. scores: [128][128] FP32 bits or
// INT32. output: [128][128] FP32. Returns a cudaError_t.
extern "C" int mmh3_b200_umma_selftest(int mode, const void *a, const void *b, const void *v,
                                       const void *p, void *scores, void *output) {
    using namespace mmh3;
    const int element = mode == 0 ? 2 : 1;
    const CUtensorMapDataType type =
        mode == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const uint64_t dimensions[2] = {N, N};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * element};
    const uint32_t box[2] = {static_cast<uint32_t>(128 / element), N};
    SelftestMaps maps;
    if (!encode_tensor_map(&maps.a, type, 2, a, dimensions, strides, box) ||
        !encode_tensor_map(&maps.b, type, 2, b, dimensions, strides, box) ||
        !encode_tensor_map(&maps.v, type, 2, v, dimensions, strides, box)) {
        return INVALID_VALUE;
    }
    unsigned int *status = status_pointer();
    if (status == nullptr) {
        return static_cast<int>(cudaErrorInvalidDevice);
    }
    auto run = [&](auto kernel) {
        cudaError_t error = cudaFuncSetAttribute(
            kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (error != cudaSuccess) {
            return static_cast<int>(error);
        }
        kernel<<<1, THREADS, SMEM_BYTES>>>(maps, static_cast<const uint32_t *>(p),
                                           static_cast<uint32_t *>(scores),
                                           static_cast<float *>(output), status);
        return static_cast<int>(cudaGetLastError());
    };
    return mode == 0 ? run(selftest_kernel<0>) : run(selftest_kernel<1>);
}

namespace {

// Every thread waits for a phase of a barrier that nothing completes: the bounded wait gives up
// after about a second, records `code` in the status word, raises the CTA's abort flag, and the
// kernel returns; the context stays usable.
__global__ void expired_wait_kernel(unsigned int *status, unsigned int code, int *gave_up) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        sm100::mbar_init(sm100::smem_u32(&bar), 1);
        abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncthreads();
    const sm100::Watchdog watchdog = {&abort_flag, status};
    const bool completed = sm100::mbar_wait(sm100::smem_u32(&bar), 0, watchdog, code);
    if (!completed) {
        atomicAdd(gave_up, 1);
    }
}

} // namespace

// Launches the kernel above with 64 threads and returns how many of them gave up their wait (after
// synchronizing), or a negative cudaError_t. The status word afterwards holds `code`.
extern "C" int mmh3_b200_expired_wait_selftest(unsigned int code) {
    unsigned int *status = mmh3::status_pointer();
    if (status == nullptr) {
        return -static_cast<int>(cudaErrorInvalidDevice);
    }
    int *gave_up = nullptr;
    cudaError_t error = cudaMalloc(&gave_up, sizeof(int));
    if (error != cudaSuccess) {
        return -static_cast<int>(error);
    }
    cudaMemset(gave_up, 0, sizeof(int));
    expired_wait_kernel<<<1, 64>>>(status, code, gave_up);
    int count = 0;
    error = cudaMemcpy(&count, gave_up, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(gave_up);
    return error == cudaSuccess ? count : -static_cast<int>(error);
}
