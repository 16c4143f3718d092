// Thin wrappers over the Blackwell (sm_100a) instructions the attention kernels are built from:
// mbarrier, TMA tile loads (cp.async.bulk.tensor), tensor memory (TMEM) allocation and access, and
// the tcgen05 UMMA with its shared-memory and instruction descriptors.
//
// Every wait in here is bounded. A wait that runs out records a code in a status word and raises a
// flag in shared memory that every other wait of the CTA polls, so that a broken pipeline drains
// and returns instead of hanging the device.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace sm100 {

// About one second at the clocks a B200 runs at: far longer than any wait of a healthy pipeline.
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void *pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

// ---------------------------------------------------------------------------------------------
// mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes the initialised barriers visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}

// What a CTA shares about a wait that gave up: a flag in shared memory that its other waits poll,
// and the status word in global memory the host reads.
struct Watchdog {
    volatile uint32_t *abort_flag;
    unsigned int *status;
};

// Waits for the phase of `bar` with parity `parity` to complete. Returns false when the wait ran
// out or another wait of the CTA already had; `code` then says which wait this was.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Watchdog &watchdog,
                                          unsigned int code) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    for (;;) {
        #pragma unroll 1
        for (int spin = 0; spin < 64; spin++) {
            if (mbar_try_wait(bar, parity)) {
                return true;
            }
        }
        if (*watchdog.abort_flag != 0) {
            return false;
        }
        if (clock64() - start > WAIT_LIMIT_CYCLES) {
            *watchdog.abort_flag = 1;
            atomicCAS(watchdog.status, 0u, code);
            return false;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// TMA: one box of a tiled tensor map into shared memory, completing `bar` by its byte count.

__device__ __forceinline__ void tma_load_2d(uint32_t destination, const CUtensorMap *map,
                                            uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];" ::"r"(destination),
                 "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t destination, const CUtensorMap *map,
                                            uint32_t bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(destination),
                 "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// A hint: the 128-byte line holding `address` into L1.
__device__ __forceinline__ void prefetch_l1(const void *address) {
    asm volatile("prefetch.global.L1 [%0];" ::"l"(address));
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor memory

// Allocates `columns` (a power of two, at least 32) TMEM columns and writes their base address to
// shared memory. One whole warp calls it, and the same warp frees the columns.
__device__ __forceinline__ void tmem_alloc(uint32_t destination, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     destination),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Makes `bar` complete once every MMA this thread has issued so far has.
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::
                     "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_wait_load() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_store() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 consecutive 32-bit columns of this thread's TMEM lane (the warp's lane quarter plus the lane
// index), starting at `address`. The registers are valid after tmem_wait_load.
__device__ __forceinline__ void tmem_load_32(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address)
        : "memory");
}

__device__ __forceinline__ void tmem_store_32(uint32_t address, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
            address),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_store_16(uint32_t address, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(
                     address),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
                 "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
                 "r"(r[14]), "r"(r[15])
                 : "memory");
}

__device__ __forceinline__ void tmem_store_8(uint32_t address, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(address),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
                 "r"(r[7])
                 : "memory");
}

// ---------------------------------------------------------------------------------------------
// UMMA descriptors

// Shared-memory matrix descriptor of a tile in the 128-byte swizzle TMA writes (rows of 128 bytes,
// eight rows to a 1024-byte swizzle atom). `leading` and `stride` are byte offsets:
//
// - K-major operand (the contraction runs along a row): `stride` is the distance between groups
//   of eight rows, and `leading` is not used.
// - MN-major operand (the contraction runs down the rows): `stride` is the distance between
//   groups of eight rows of the contraction, and `leading` the distance between slabs of 128
//   bytes (64 16-bit elements) along M or N.
//
// `swizzle` is the layout code of the descriptor: SWIZZLE_128B for rows of 128 bytes, SWIZZLE_64B
// for rows of 64 bytes (eight rows to a 512-byte atom).
constexpr uint64_t SWIZZLE_128B = 2, SWIZZLE_64B = 4;

__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address, uint32_t leading,
                                                    uint32_t stride,
                                                    uint64_t swizzle = SWIZZLE_128B) {
    uint64_t descriptor = 0;
    descriptor |= static_cast<uint64_t>((address >> 4) & 0x3fffu);
    descriptor |= static_cast<uint64_t>((leading >> 4) & 0x3fffu) << 16;
    descriptor |= static_cast<uint64_t>((stride >> 4) & 0x3fffu) << 32;
    descriptor |= 1ull << 46; // descriptor version of sm_100
    descriptor |= swizzle << 61;
    return descriptor;
}

// The same descriptor `bytes` further on in shared memory: the address field is the low 14 bits, in
// units of 16 bytes, and shared memory is smaller than the field, so the addition never carries
// into the next field. The MMA-issuing thread builds each tile's descriptor once and steps through
// it with this, which keeps its instruction stream short.
__device__ __forceinline__ uint64_t advance_descriptor(uint64_t descriptor, uint32_t bytes) {
    return descriptor + (bytes >> 4);
}

// Operand formats of the instruction descriptor.
constexpr uint32_t FORMAT_F16 = 0, FORMAT_BF16 = 1;   // kind::f16
constexpr uint32_t FORMAT_U8 = 0, FORMAT_S8 = 1;      // kind::i8
constexpr uint32_t FORMAT_E4M3 = 0, FORMAT_E5M2 = 1;  // kind::f8f6f4
constexpr uint32_t ACCUMULATE_F16 = 0, ACCUMULATE_F32 = 1, ACCUMULATE_S32 = 2;

// Instruction descriptor of a dense M × N UMMA. A major flag of one says the operand is MN-major.
__host__ __device__ constexpr uint32_t instruction_descriptor(uint32_t accumulator, uint32_t a_format,
                                          uint32_t b_format, uint32_t a_mn_major,
                                          uint32_t b_mn_major, uint32_t m, uint32_t n) {
    return (accumulator << 4) | (a_format << 7) | (b_format << 10) | (a_mn_major << 15) |
           (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D (TMEM) = A (smem) · B (smem), or D += A · B when `accumulate` is nonzero. One thread issues it.
#define MMH3_DEFINE_MMA(KIND, NAME)                                                               \
    __device__ __forceinline__ void NAME##_ss(uint32_t d, uint64_t a, uint64_t b,                 \
                                              uint32_t instruction, uint32_t accumulate) {        \
        asm volatile("{\n"                                                                        \
                     ".reg .pred p;\n"                                                            \
                     "setp.ne.b32 p, %4, 0;\n"                                                    \
                     "tcgen05.mma.cta_group::1.kind::" KIND " [%0], %1, %2, %3, p;\n"             \
                     "}" ::"r"(d),                                                                \
                     "l"(a), "l"(b), "r"(instruction), "r"(accumulate)                            \
                     : "memory");                                                                 \
    }                                                                                             \
    /* The same with A in tensor memory at `a`. */                                                \
    __device__ __forceinline__ void NAME##_ts(uint32_t d, uint32_t a, uint64_t b,                 \
                                              uint32_t instruction, uint32_t accumulate) {        \
        asm volatile("{\n"                                                                        \
                     ".reg .pred p;\n"                                                            \
                     "setp.ne.b32 p, %4, 0;\n"                                                    \
                     "tcgen05.mma.cta_group::1.kind::" KIND " [%0], [%1], %2, %3, p;\n"           \
                     "}" ::"r"(d),                                                                \
                     "r"(a), "l"(b), "r"(instruction), "r"(accumulate)                            \
                     : "memory");                                                                 \
    }

MMH3_DEFINE_MMA("f16", mma_f16)
MMH3_DEFINE_MMA("i8", mma_i8)
MMH3_DEFINE_MMA("f8f6f4", mma_f8)
#undef MMH3_DEFINE_MMA

// Moves registers between the warpgroups of a CTA: every warp of a warpgroup (four consecutive
// warps) executes the same one.
template <int REGISTERS> __device__ __forceinline__ void register_increase() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}

template <int REGISTERS> __device__ __forceinline__ void register_decrease() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}

__device__ __forceinline__ float exp2_approx(float value) {
    float result;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(result) : "f"(value));
    return result;
}

// 2^x for both halves of a pair on the FMA pipe instead of the MUFU: x is split into its nearest
// integer n (the low mantissa bits after adding 1.5 * 2^23) and a fraction f in [-0.5, 0.5], 2^f is
// a cubic (relative error under 8e-5, far below what BF16 or E4M3 keep), and n goes into the
// exponent field. x must not be far above zero. Anything below -125 gives 2^-125: the cubic lies in
// [0.7, 1.42], so its exponent field is 126 or 127 and n = -125 still leaves a positive one.
__device__ __forceinline__ float2 exp2_polynomial(float2 x) {
    constexpr float MAGIC = 12582912.0f;
    x.x = fmaxf(x.x, -125.0f);
    x.y = fmaxf(x.y, -125.0f);
    const float2 shifted = __fadd2_rn(x, make_float2(MAGIC, MAGIC));
    const float2 whole = __fadd2_rn(shifted, make_float2(-MAGIC, -MAGIC));
    const float2 fraction = __ffma2_rn(whole, make_float2(-1.0f, -1.0f), x);
    float2 power = __ffma2_rn(fraction, make_float2(0.05520550534129143f, 0.05520550534129143f),
                              make_float2(0.24261397123336792f, 0.24261397123336792f));
    power = __ffma2_rn(power, fraction, make_float2(0.6932547688484192f, 0.6932547688484192f));
    power = __ffma2_rn(power, fraction, make_float2(0.9999276995658875f, 0.9999276995658875f));
    power.x = __int_as_float(__float_as_int(power.x) + (__float_as_int(shifted.x) << 23));
    power.y = __int_as_float(__float_as_int(power.y) + (__float_as_int(shifted.y) << 23));
    return power;
}

__device__ __forceinline__ uint32_t pack_bf16(float low, float high) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(high), "f"(low));
    return packed;
}

} // namespace sm100
