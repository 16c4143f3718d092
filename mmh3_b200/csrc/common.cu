#include "common.cuh"

#include <cudaTypedefs.h>
#include <mutex>

namespace mmh3 {

namespace {

// One word per device that loads the library; the kernels' bounded waits write to it.
__device__ unsigned int status_word;

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 encoder = [] {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault,
                                    &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess) {
            return static_cast<PFN_cuTensorMapEncodeTiled_v12000>(nullptr);
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(entry);
    }();
    return encoder;
}

} // namespace

unsigned int *status_pointer() {
    static std::atomic<unsigned int *> pointers[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        return nullptr;
    }
    if (unsigned int *kept = pointers[device].load(std::memory_order_acquire); kept != nullptr) {
        return kept;
    }
    void *address = nullptr;
    if (cudaGetSymbolAddress(&address, status_word) != cudaSuccess) {
        return nullptr;
    }
    pointers[device].store(static_cast<unsigned int *>(address), std::memory_order_release);
    return static_cast<unsigned int *>(address);
}

int multiprocessor_count() {
    static std::atomic<int> counts[MAX_DEVICES];
    const int device = current_device();
    if (device < 0) {
        return 0;
    }
    if (const int kept = counts[device].load(std::memory_order_relaxed); kept != 0) {
        return kept;
    }
    int processors = 0;
    if (cudaDeviceGetAttribute(&processors, cudaDevAttrMultiProcessorCount, device) !=
        cudaSuccess) {
        return 0;
    }
    counts[device].store(processors, std::memory_order_relaxed);
    return processors;
}

bool encode_tensor_map(CUtensorMap *map, CUtensorMapDataType type, int rank, const void *base,
                       const uint64_t *dimensions, const uint64_t *strides, const uint32_t *box,
                       CUtensorMapSwizzle swizzle) {
    PFN_cuTensorMapEncodeTiled_v12000 encoder = tensor_map_encoder();
    if (encoder == nullptr || reinterpret_cast<uintptr_t>(base) % 16 != 0 || rank < 2 ||
        rank > 5) {
        return false;
    }
    cuuint64_t global_dimensions[5];
    cuuint64_t global_strides[4];
    cuuint32_t box_dimensions[5];
    cuuint32_t element_strides[5];
    for (int index = 0; index < rank; index++) {
        global_dimensions[index] = dimensions[index];
        box_dimensions[index] = box[index];
        element_strides[index] = 1;
        if (index + 1 < rank) {
            if (strides[index] == 0 || strides[index] % 16 != 0) {
                return false;
            }
            global_strides[index] = strides[index];
        }
    }
    return encoder(map, type, static_cast<cuuint32_t>(rank), const_cast<void *>(base),
                   global_dimensions, global_strides, box_dimensions, element_strides,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tma_aligned(const void *base, int heads, int64_t token_stride, int64_t head_stride) {
    return reinterpret_cast<uintptr_t>(base) % 16 == 0 && token_stride % 8 == 0 &&
           (heads == 1 || head_stride % 8 == 0);
}

namespace {

// An operand copied 16 bits at a time into a dense [tokens][heads][dim] array.
__global__ void gather_operand_kernel(const uint16_t *__restrict__ source,
                                      uint16_t *__restrict__ target, int64_t elements, int heads,
                                      int head_dim, int64_t token_stride, int64_t head_stride) {
    for (int64_t index = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
         index < elements; index += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int dimension = static_cast<int>(index % head_dim);
        const int64_t row = index / head_dim;
        const int head = static_cast<int>(row % heads);
        const int64_t token = row / heads;
        target[index] = source[token * token_stride + head * head_stride + dimension];
    }
}

} // namespace

StagedOperands::~StagedOperands() {
    for (void *buffer : buffers) {
        if (buffer != nullptr) {
            cudaFreeAsync(buffer, stream);
        }
    }
}

cudaError_t StagedOperands::stage(int slot, const uint16_t *&base, int tokens, int heads,
                                  int head_dim, int64_t &token_stride, int64_t &head_stride) {
    if (tma_aligned(base, heads, token_stride, head_stride)) {
        return cudaSuccess;
    }
    const int64_t elements = static_cast<int64_t>(tokens) * heads * head_dim;
    const cudaError_t allocated = cudaMallocAsync(&buffers[slot], elements * 2, stream);
    if (allocated != cudaSuccess) {
        return allocated;
    }
    const int64_t wanted = (elements + 255) / 256;
    const int64_t most = 8 * static_cast<int64_t>(multiprocessor_count() > 0 ? multiprocessor_count() : 1);
    const int blocks = static_cast<int>(wanted < most ? wanted : most);
    gather_operand_kernel<<<blocks, 256, 0, stream>>>(base, static_cast<uint16_t *>(buffers[slot]),
                                                      elements, heads, head_dim, token_stride,
                                                      head_stride);
    base = static_cast<const uint16_t *>(buffers[slot]);
    token_stride = static_cast<int64_t>(heads) * head_dim;
    head_stride = head_dim;
    return cudaGetLastError();
}

} // namespace mmh3

extern "C" int mmh3_b200_take_status(void) {
    cudaError_t error = cudaDeviceSynchronize();
    if (error != cudaSuccess) {
        return -static_cast<int>(error);
    }
    unsigned int *word = mmh3::status_pointer();
    if (word == nullptr) {
        return -static_cast<int>(cudaErrorInvalidDevice);
    }
    unsigned int value = 0;
    error = cudaMemcpy(&value, word, sizeof(value), cudaMemcpyDeviceToHost);
    if (error != cudaSuccess) {
        return -static_cast<int>(error);
    }
    if (value != 0) {
        const unsigned int zero = 0;
        cudaMemcpy(word, &zero, sizeof(zero), cudaMemcpyHostToDevice);
    }
    return static_cast<int>(value);
}
