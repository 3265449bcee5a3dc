#include "Tensor.h"

#include <stdexcept>
#include <string>

#include "thor_b200.h"

namespace ThorB200 {

Tensor Tensor::wrap(void* device_ptr, DataType dtype, std::vector<uint64_t> dims, int gpu_num) {
    Tensor t;
    t.ptr_ = device_ptr;
    t.dtype_ = dtype;
    t.dims_ = std::move(dims);
    t.gpu_num_ = gpu_num;
    return t;
}

namespace {
thread_local bool g_plan_only = false;
thread_local uint64_t g_placeholder = 0x100000000000ull;  // never dereferenced
}  // namespace

void Tensor::setPlanOnly(bool on) { g_plan_only = on; }
bool Tensor::planOnly() { return g_plan_only; }

Tensor Tensor::allocate(DataType dtype, std::vector<uint64_t> dims, int gpu_num) {
    Tensor t;
    t.dtype_ = dtype;
    t.dims_ = std::move(dims);
    t.gpu_num_ = gpu_num;
    if (g_plan_only) {
        t.ptr_ = reinterpret_cast<void*>(g_placeholder);
        g_placeholder += (t.getArraySizeInBytes() + 511) / 256 * 256;
        return t;
    }
    void* p = nullptr;
    // the caller has made gpu_num current (the reference wraps allocation in ScopedGpu)
    if (thor_b200_device_alloc(t.getArraySizeInBytes(), &p) != THOR_B200_OK)
        throw std::runtime_error(std::string("Tensor::allocate: ") + thor_b200_last_error());
    t.ptr_ = p;
    t.owner_ = std::shared_ptr<void>(p, [](void* q) { thor_b200_device_free(q); });
    return t;
}

Tensor Tensor::aliasView(std::vector<uint64_t> dims, std::vector<uint64_t> strides_elements, uint64_t element_offset) const {
    if (!isInitialized()) throw std::logic_error("Tensor::aliasView: uninitialised tensor");
    if (dims.size() != strides_elements.size()) throw std::invalid_argument("Tensor::aliasView: one stride per dimension");
    // the view must stay inside the storage this tensor describes
    uint64_t last = element_offset;
    for (size_t i = 0; i < dims.size(); ++i) {
        if (dims[i] == 0) throw std::invalid_argument("Tensor::aliasView: zero-sized dimension");
        last += (dims[i] - 1) * strides_elements[i];
    }
    uint64_t extent = 1;
    const std::vector<uint64_t> own = getStridesElements();
    for (size_t i = 0; i < dims_.size(); ++i) extent += (dims_[i] - 1) * own[i];
    if (last >= extent) throw std::invalid_argument("Tensor::aliasView: the view reaches beyond the tensor's storage");
    Tensor v = *this;
    v.dims_ = std::move(dims);
    v.strides_ = std::move(strides_elements);
    v.storage_offset_ = storage_offset_ + element_offset;
    v.ptr_ = static_cast<char*>(ptr_) + element_offset * dataTypeSize(dtype_);
    return v;
}

std::vector<uint64_t> Tensor::getStridesElements() const {
    if (!strides_.empty()) return strides_;
    std::vector<uint64_t> s(dims_.size(), 1);
    for (size_t i = dims_.size(); i-- > 1;) s[i - 1] = s[i] * dims_[i];
    return s;
}

bool Tensor::isDenseRowMajor() const {
    if (strides_.empty()) return true;
    uint64_t expect = 1;
    for (size_t i = dims_.size(); i-- > 0;) {
        if (dims_[i] != 1 && strides_[i] != expect) return false;
        expect *= dims_[i];
    }
    return true;
}

void Tensor::copyFromAsync(const Tensor& source, const Stream& stream) {
    if (!isInitialized() || !source.isInitialized()) throw std::logic_error("Tensor::copyFromAsync: uninitialised tensor");
    if (source.getTotalNumElements() != getTotalNumElements()) throw std::logic_error("Tensor::copyFromAsync: total number of elements does not match");
    if (gpu_num_ >= 0 && gpu_num_ != stream.getGpuNum()) throw std::logic_error("Tensor::copyFromAsync: the stream belongs to another GPU than the destination");
    const int status = thor_b200_copy_convert_launch(ptr_, static_cast<int>(dtype_), gpu_num_, source.ptr_, static_cast<int>(source.dtype_), source.gpu_num_,
                                                     static_cast<int64_t>(getTotalNumElements()), stream.handle);
    if (status == THOR_B200_INVALID_ARGUMENT || status == THOR_B200_UNSUPPORTED) throw std::logic_error(std::string("Tensor::copyFromAsync: ") + thor_b200_last_error());
    if (status != THOR_B200_OK) throw std::runtime_error(std::string("Tensor::copyFromAsync: ") + thor_b200_last_error());
}

}  // namespace ThorB200
