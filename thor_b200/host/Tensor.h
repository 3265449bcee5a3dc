// Minimal stand-ins for the reference's boundary types Tensor and Stream
// (DeepLearning/Implementation/Tensor/Tensor.h:56-266, Utilities/Common/Stream.h:35-118): a device
// pointer with dtype + dense row-major dimensions, and a cudaStream_t with its device ordinal.
// Device memory comes from the C ABI (thor_b200_device_alloc); the host layer never links CUDA.
#pragma once

#include <cstdint>
#include <memory>
#include <vector>

#include "DataType.h"

namespace ThorB200 {

struct Stream {
    void* handle = nullptr;  // cudaStream_t
    int gpu_num = 0;
    Stream() = default;
    Stream(void* h, int gpu) : handle(h), gpu_num(gpu) {}
    int getGpuNum() const { return gpu_num; }
};

class Tensor {
   public:
    Tensor() = default;
    // Adopts memory owned by the caller (a torch tensor, a Thor tensor, ...).
    static Tensor wrap(void* device_ptr, DataType dtype, std::vector<uint64_t> dims, int gpu_num = 0);
    // Allocates dense device memory on gpu_num (used at stamp time for intermediates and outputs).
    static Tensor allocate(DataType dtype, std::vector<uint64_t> dims, int gpu_num = 0);

    // Plan-only mode (thread local): allocate() hands out distinct placeholder addresses instead of
    // device memory and every kernel is compiled without being loaded, so that a plan (stages,
    // kernel shapes, emitted sources, intermediate bytes) can be produced on a machine without a
    // GPU.  A plan stamped in this mode refuses to run.
    static void setPlanOnly(bool on);
    static bool planOnly();

    // Host (pinned) memory owned by the caller: gpu_num is -1.
    static Tensor wrapHost(void* host_ptr, DataType dtype, std::vector<uint64_t> dims) { return wrap(host_ptr, dtype, std::move(dims), -1); }
    // Tensor::copyFromAsync (Tensor.cpp:700-860) for dense tensors: same element count; a dtype change across placements
    // copies in the source dtype and converts in place on the destination GPU, and is refused when the destination
    // dtype is the smaller one; conversions into host memory are refused (no CPU path here).
    void copyFromAsync(const Tensor& source, const Stream& stream);

    bool isInitialized() const { return ptr_ != nullptr; }
    void* getMemPtr() const { return ptr_; }
    DataType getDataType() const { return dtype_; }
    const std::vector<uint64_t>& getDimensions() const { return dims_; }
    int getGpuNum() const { return gpu_num_; }
    uint64_t getTotalNumElements() const {
        uint64_t n = 1;
        for (uint64_t d : dims_) n *= d;
        return n;
    }
    uint64_t getArraySizeInBytes() const { return getTotalNumElements() * dataTypeSize(dtype_); }

    // Zero-copy view of this tensor's storage (Tensor::aliasView, Tensor.h:146-152): dims and element strides of the
    // view, element offset of its first element from this tensor's first element.  getMemPtr() of the view already
    // includes the offset; the view keeps the storage alive.
    Tensor aliasView(std::vector<uint64_t> dims, std::vector<uint64_t> strides_elements, uint64_t element_offset = 0) const;
    // Element strides: those of the view, or the dense row-major strides of dims.
    std::vector<uint64_t> getStridesElements() const;
    uint64_t getStorageElementOffset() const { return storage_offset_; }
    bool isDenseRowMajor() const;

   private:
    void* ptr_ = nullptr;
    DataType dtype_ = DataType::FP32;
    std::vector<uint64_t> dims_;
    int gpu_num_ = 0;
    std::vector<uint64_t> strides_;  // empty = dense row-major
    uint64_t storage_offset_ = 0;
    std::shared_ptr<void> owner_;
};

}  // namespace ThorB200
