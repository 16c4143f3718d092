// INT8/FP8 dense attention for callers that cannot allocate device memory.
//
// mmh3_attention_quantized needs scratch (INT8 q and k, FP8 V, their scales) that the caller
// allocates and passes in as an Mmh3QuantizedWorkspace. Some callers have no way to do that: a host
// that accounts for every byte of the device itself and has handed the rest to its weight
// streaming (mmh3 sizes its streaming window by what its own counters say is left, and a
// cudaMalloc behind its back either fails or eats that window), or a caller inside a loop where
// cudaMalloc's device-wide synchronization would stall every other stream. For them this entry
// point keeps the scratch in a fixed array that is part of the library's device image. Nothing is
// allocated or freed here, by the CUDA runtime or by anything else.
//
// The price: the array has a fixed, modest size, every GPU that loads the library carries it until
// the process exits, and all calls share it. With lazy module loading (the runtime's default) the
// driver backs the array on a device when the first call there looks up its address, not when the
// library is opened; calls after that take no device memory at all.
#include <atomic>
#include <cstdio>

#include "common.cuh"

namespace {

using namespace mmh3;

// Largest problem: tokens rounded up to 64, times heads, at most this many (4,096 tokens of 8 heads,
// or any other shape with as many rows).
constexpr int64_t MAX_ROWS = 4096 * 8;
constexpr int MAX_HEADS = 64;
constexpr int64_t TENSOR_BYTES = MAX_ROWS * HEAD_DIM;       // one of q8, k8, v8: 4 MiB
constexpr int64_t SCALE_FLOATS = MAX_ROWS / 64;             // one scale per head and 64-token block
constexpr int64_t OFFSET_QUERY = 0;
constexpr int64_t OFFSET_KEY = OFFSET_QUERY + TENSOR_BYTES;
constexpr int64_t OFFSET_VALUE = OFFSET_KEY + TENSOR_BYTES;
constexpr int64_t OFFSET_QUERY_SCALES = OFFSET_VALUE + TENSOR_BYTES;
constexpr int64_t OFFSET_KEY_SCALES = OFFSET_QUERY_SCALES + SCALE_FLOATS * 4;
constexpr int64_t OFFSET_VALUE_MAXIMA = OFFSET_KEY_SCALES + SCALE_FLOATS * 4;
constexpr int64_t OFFSET_VALUE_SCALES = OFFSET_VALUE_MAXIMA + SCALE_FLOATS * 4;
constexpr int64_t SCRATCH_BYTES = OFFSET_VALUE_SCALES + 256; // 12 MiB and a few KiB
static_assert(MAX_HEADS * 4 <= 256, "the per-head scales have 256 bytes");
static_assert(OFFSET_KEY % 256 == 0 && OFFSET_VALUE % 256 == 0 && OFFSET_QUERY_SCALES % 256 == 0,
              "the tensors the TMA reads start on 256-byte boundaries");

// The scratch itself. In host code this name is only a handle for the runtime's symbol calls, not
// an address a kernel can use: the device address comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) unsigned char scratch[SCRATCH_BYTES];

// The device address of `scratch` on the current device, looked up on the first call there.
unsigned char *scratch_on_this_device(cudaError_t *error) {
    static std::atomic<unsigned char *> addresses[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        *error = cudaErrorInvalidDevice;
        return nullptr;
    }
    if (unsigned char *known = addresses[device].load(std::memory_order_acquire);
        known != nullptr) {
        return known;
    }
    unsigned char *address = nullptr;
    *error = cudaGetSymbolAddress(reinterpret_cast<void **>(&address), scratch);
    if (*error != cudaSuccess) {
        return nullptr;
    }
    addresses[device].store(address, std::memory_order_release);
    return address;
}

} // namespace

extern "C" int mmh3_b200_attention_quantized_static(const void *query, const void *key,
                                                    const void *value, void *output, int tokens,
                                                    int heads, const Mmh3AttentionLayout *layout,
                                                    float scale, mmh3_stream_t stream) {
    if (layout == nullptr || tokens <= 0 || heads <= 0 || layout->causal != 0 ||
        layout->heads_per_key_value > 1) {
        return INVALID_VALUE;
    }
    const int64_t blocks = (static_cast<int64_t>(tokens) + 63) / 64;
    if (heads > MAX_HEADS || blocks * 64 * heads > MAX_ROWS) {
        std::fprintf(stderr,
                     "mmh3_b200_attention_quantized_static: %d tokens x %d heads is past the "
                     "built-in scratch (tokens rounded up to 64, times heads, at most %lld; at "
                     "most %d heads); use mmh3_attention_quantized with a workspace of your own\n",
                     tokens, heads, static_cast<long long>(MAX_ROWS), MAX_HEADS);
        return INVALID_VALUE;
    }
    cudaError_t error = cudaSuccess;
    unsigned char *base = scratch_on_this_device(&error);
    if (base == nullptr) {
        return static_cast<int>(error);
    }
    Mmh3QuantizedWorkspace workspace;
    workspace.query = base + OFFSET_QUERY;
    workspace.key = base + OFFSET_KEY;
    workspace.value = base + OFFSET_VALUE;
    workspace.query_scales = reinterpret_cast<float *>(base + OFFSET_QUERY_SCALES);
    workspace.key_scales = reinterpret_cast<float *>(base + OFFSET_KEY_SCALES);
    workspace.value_maxima = reinterpret_cast<float *>(base + OFFSET_VALUE_MAXIMA);
    workspace.value_scales = reinterpret_cast<float *>(base + OFFSET_VALUE_SCALES);
    // Every byte the attention reads is written first by the passes below (the FP8 V including the
    // zeroes past the last token of the last block), so nothing of an earlier call shows through
    // and nothing needs clearing.
    return mmh3_attention_quantized(query, key, value, output, tokens, heads, layout, scale,
                                    nullptr, &workspace, 0, stream);
}
