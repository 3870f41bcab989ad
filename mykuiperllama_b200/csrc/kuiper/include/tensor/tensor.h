// Shape + dtype + shared Buffer handle passed to every kernel by const reference.
// Public interface of the reference's tensor::Tensor (kuiper/include/tensor/tensor.h:8-86;
// behaviour pinned by test/test_tensor/test_tensor.cpp), including the historical
// spelling of assgin().
#ifndef KUIPER_INCLUDE_TENSOR_TENSOR_H
#define KUIPER_INCLUDE_TENSOR_TENSOR_H

#include <cuda_runtime_api.h>

#include <vector>

#include "base/buffer.h"

namespace tensor {

class Tensor {
public:
    explicit Tensor() = default;

    // need_alloc: allocate through `allocator` now.  allocator == nullptr borrows `ptr`;
    // allocator + ptr adopts `ptr` (released through the allocator).
    explicit Tensor(base::DataType data_type, int32_t dim0, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr, void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr, void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr, void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, int32_t dim3,
                    bool need_alloc = false, std::shared_ptr<base::DeviceAllocator> allocator = nullptr,
                    void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, std::vector<int32_t> dims, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr, void* ptr = nullptr);

    void init_buffer(std::shared_ptr<base::DeviceAllocator> allocator, bool need_alloc, void* ptr);
    bool allocate(std::shared_ptr<base::DeviceAllocator> allocator, bool need_realloc);
    bool assgin(std::shared_ptr<base::Buffer> buffer);

    void to_cpu();
    void to_cuda(cudaStream_t stream = nullptr);

    void reshape(const std::vector<int32_t>& dims);
    int32_t dims_size() const;
    int32_t get_dim(int32_t index) const;
    const std::vector<int32_t>& dims() const;
    std::vector<size_t> strides() const;  // row-major, in elements

    Tensor clone() const;
    void reset(base::DataType data_type, const std::vector<int32_t>& dims);

    bool is_empty() const;
    size_t size() const;
    size_t byte_size() const;
    base::DataType data_type() const;
    base::DeviceType device_type() const;
    void set_device_type(base::DeviceType device_type) const;
    std::shared_ptr<base::Buffer> get_buffer() const;

    template <typename T> T* ptr();
    template <typename T> const T* ptr() const;
    template <typename T> T* ptr(int64_t index);
    template <typename T> const T* ptr(int64_t index) const;
    template <typename T> T& index(int64_t offset);
    template <typename T> const T& index(int64_t offset) const;

private:
    size_t size_ = 0;
    std::vector<int32_t> dims_;
    std::shared_ptr<base::Buffer> buffer_;
    base::DataType data_type_ = base::DataType::DataTypeUnknown;
};

template <typename T>
T* Tensor::ptr() {
    return buffer_ ? reinterpret_cast<T*>(buffer_->ptr()) : nullptr;
}

template <typename T>
const T* Tensor::ptr() const {
    return buffer_ ? reinterpret_cast<const T*>(buffer_->ptr()) : nullptr;
}

template <typename T>
T* Tensor::ptr(int64_t index) {
    CHECK(buffer_ && buffer_->ptr()) << "The data area buffer of this tensor is empty or it points to a null pointer.";
    return reinterpret_cast<T*>(buffer_->ptr()) + index;
}

template <typename T>
const T* Tensor::ptr(int64_t index) const {
    CHECK(buffer_ && buffer_->ptr()) << "The data area buffer of this tensor is empty or it points to a null pointer.";
    return reinterpret_cast<const T*>(buffer_->ptr()) + index;
}

template <typename T>
T& Tensor::index(int64_t offset) {
    CHECK_GE(offset, 0);
    CHECK_LT(size_t(offset), size_);
    return reinterpret_cast<T*>(buffer_->ptr())[offset];
}

template <typename T>
const T& Tensor::index(int64_t offset) const {
    CHECK_GE(offset, 0);
    CHECK_LT(size_t(offset), size_);
    return reinterpret_cast<const T*>(buffer_->ptr())[offset];
}

}  // namespace tensor

#endif  // KUIPER_INCLUDE_TENSOR_TENSOR_H
