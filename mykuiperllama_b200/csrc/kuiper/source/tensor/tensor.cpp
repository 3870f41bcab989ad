// tensor::Tensor (interface: kuiper/include/tensor/tensor.h:8-86 of the reference; the
// ownership rules of init_buffer / allocate / assgin and the grow-and-copy reshape follow
// kuiper/source/tensor/tensor.cpp:61-177, which test/test_tensor/test_tensor.cpp pins).
#include "tensor/tensor.h"

#include <functional>
#include <numeric>

namespace tensor {
namespace {
size_t element_count(const std::vector<int32_t>& dims) {
    if (dims.empty()) return 0;
    return std::accumulate(dims.begin(), dims.end(), size_t(1),
                           [](size_t acc, int32_t d) { return acc * size_t(d); });
}
}  // namespace

Tensor::Tensor(base::DataType data_type, int32_t dim0, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0}, need_alloc, std::move(allocator), ptr) {}

Tensor::Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0, dim1}, need_alloc, std::move(allocator), ptr) {}

Tensor::Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0, dim1, dim2}, need_alloc, std::move(allocator), ptr) {}

Tensor::Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, int32_t dim3, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0, dim1, dim2, dim3}, need_alloc, std::move(allocator), ptr) {}

Tensor::Tensor(base::DataType data_type, std::vector<int32_t> dims, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : size_(element_count(dims)), dims_(std::move(dims)), data_type_(data_type) {
    // a default-constructed-like call (no allocator, no pointer, no allocation) leaves the buffer empty
    if (!allocator && !ptr && !need_alloc) return;
    init_buffer(std::move(allocator), need_alloc, ptr);
}

void Tensor::init_buffer(std::shared_ptr<base::DeviceAllocator> allocator, bool need_alloc, void* ptr) {
    if (!allocator) {
        // borrowed memory: the tensor never frees it
        CHECK_NE(ptr, nullptr);
        CHECK_EQ(need_alloc, false);
        buffer_ = std::make_shared<base::Buffer>(byte_size(), nullptr, ptr, true);
        return;
    }
    if (need_alloc) {
        allocate(allocator, false);
    } else if (ptr) {
        // adopt: released through the allocator with the last handle
        buffer_ = std::make_shared<base::Buffer>(byte_size(), allocator, ptr, false);
        buffer_->set_device_type(allocator->device_type());
    } else {
        allocate(allocator, true);
    }
}

bool Tensor::allocate(std::shared_ptr<base::DeviceAllocator> allocator, bool need_realloc) {
    if (!allocator) {
        LOG(ERROR) << "The allocator parameter in the allocate function is null pointer!";
        return false;
    }
    const size_t bytes = byte_size();
    if (bytes == 0) {
        LOG(ERROR) << "The byte_size parameter in the allocate function is equal to zero!";
        return false;
    }
    if (buffer_ && bytes <= buffer_->byte_size() && !need_realloc) return true;
    buffer_ = std::make_shared<base::Buffer>(bytes, allocator, nullptr);
    if (!buffer_->ptr()) {
        LOG(ERROR) << "The memory allocated is a null pointer!";
        return false;
    }
    return true;
}

bool Tensor::assgin(std::shared_ptr<base::Buffer> buffer) {
    if (!buffer) {
        LOG(ERROR) << "The buffer parameter in the assign function is null pointer!";
        return false;
    }
    if (buffer_ && buffer_->device_type() != buffer->device_type()) {
        LOG(ERROR) << "The device type of the new buffer is different from the original one.";
    }
    if (buffer->byte_size() < byte_size()) {
        LOG(ERROR) << "The size of buffer is too small for the tensor!";
        return false;
    }
    buffer_ = std::move(buffer);
    return true;
}

void Tensor::to_cpu() {
    CHECK_NE(buffer_, nullptr);
    const base::DeviceType dev = device_type();
    if (dev == base::DeviceType::DeviceCUDA) {
        auto alloc = base::CPUDeviceAllocatorFactory::get_instance();
        auto host = std::make_shared<base::Buffer>(byte_size(), alloc);
        alloc->memcpy(host->ptr(), buffer_->ptr(), byte_size(), base::MemcpyKind::MemcpyCUDA2CPU);
        buffer_ = host;
    } else if (dev == base::DeviceType::DeviceCPU) {
        LOG(INFO) << "The device type of the tensor is already cpu.";
    } else {
        LOG(ERROR) << "The device type of the tensor is unknown.";
    }
}

void Tensor::to_cuda(cudaStream_t stream) {
    CHECK_NE(buffer_, nullptr);
    const base::DeviceType dev = device_type();
    if (dev == base::DeviceType::DeviceCPU) {
        auto alloc = base::CUDADeviceAllocatorFactory::get_instance();
        auto devbuf = std::make_shared<base::Buffer>(byte_size(), alloc);
        // with a stream the copy is asynchronous on it (pageable host memory makes the
        // runtime stage it); the source buffer is kept alive until the copy is enqueued
        alloc->memcpy(devbuf->ptr(), buffer_->ptr(), byte_size(), base::MemcpyKind::MemcpyCPU2CUDA, stream);
        if (stream) cudaStreamSynchronize(stream);
        buffer_ = devbuf;
    } else if (dev == base::DeviceType::DeviceCUDA) {
        LOG(INFO) << "The device type of the tensor is already cuda.";
    } else {
        LOG(ERROR) << "The device type of the tensor is unknown.";
    }
}

void Tensor::reshape(const std::vector<int32_t>& dims) {
    const size_t new_size = element_count(dims);
    if (buffer_ && new_size > size_) {
        // growing: move the contents into a larger buffer from the same allocator
        auto bigger = std::make_shared<base::Buffer>(new_size * base::data_type_size(data_type_), buffer_->allocator());
        bigger->copy_from(buffer_.get());
        buffer_ = bigger;
    }
    dims_ = dims;
    size_ = new_size;
}

int32_t Tensor::dims_size() const { return int32_t(dims_.size()); }

int32_t Tensor::get_dim(int32_t index) const {
    CHECK_GE(index, 0);
    CHECK_LT(size_t(index), dims_.size());
    return dims_[size_t(index)];
}

const std::vector<int32_t>& Tensor::dims() const { return dims_; }

std::vector<size_t> Tensor::strides() const {
    std::vector<size_t> out(dims_.size(), 1);
    for (size_t i = dims_.size(); i-- > 1;) out[i - 1] = out[i] * size_t(dims_[i]);
    return out;
}

Tensor Tensor::clone() const {
    Tensor copy = *this;
    copy.buffer_ = std::make_shared<base::Buffer>(byte_size(), buffer_->allocator());
    copy.buffer_->copy_from(buffer_.get());
    return copy;
}

void Tensor::reset(base::DataType data_type, const std::vector<int32_t>& dims) {
    data_type_ = data_type;
    dims_ = dims;
    size_ = element_count(dims);
    buffer_ = nullptr;
}

bool Tensor::is_empty() const { return size_ == 0 || !buffer_ || !buffer_->ptr(); }
size_t Tensor::size() const { return size_; }
size_t Tensor::byte_size() const { return size_ * base::data_type_size(data_type_); }
base::DataType Tensor::data_type() const { return data_type_; }

base::DeviceType Tensor::device_type() const {
    return buffer_ ? buffer_->device_type() : base::DeviceType::DeviceUnknown;
}

void Tensor::set_device_type(base::DeviceType device_type) const {
    if (buffer_ && buffer_->device_type() != device_type) buffer_->set_device_type(device_type);
}

std::shared_ptr<base::Buffer> Tensor::get_buffer() const { return buffer_; }

}  // namespace tensor
