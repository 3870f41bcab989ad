// Buffer: owned or borrowed byte range (interface: kuiper/include/base/buffer.h:17-45 of the
// reference; ownership and copy rules as kuiper/source/base/buffer.cpp:4-71).
#include "base/buffer.h"

namespace base {

Buffer::Buffer(size_t byte_size, std::shared_ptr<DeviceAllocator> allocator, void* ptr, bool use_external)
    : byte_size_(byte_size), ptr_(ptr), use_external_(use_external), allocator_(std::move(allocator)) {
    // no pointer given: allocate now and own the result; a supplied pointer keeps the
    // device tag Unknown until the caller sets it (the reference's tests do so by hand)
    if (ptr_ == nullptr && allocator_) {
        device_type_ = allocator_->device_type();
        use_external_ = false;
        ptr_ = allocator_->allocate(byte_size_);
    }
}

Buffer::~Buffer() {
    if (use_external_ || !ptr_ || !allocator_) return;
    allocator_->release(ptr_);
    ptr_ = nullptr;
}

bool Buffer::allocate() {
    if (!allocator_ || byte_size_ == 0) return false;
    use_external_ = false;
    ptr_ = allocator_->allocate(byte_size_);
    return ptr_ != nullptr;
}

void Buffer::copy_from(const Buffer& buffer) const { copy_from(&buffer); }

void Buffer::copy_from(const Buffer* buffer) const {
    CHECK(allocator_ != nullptr);
    CHECK(buffer != nullptr && buffer->ptr_ != nullptr);
    const DeviceType src = buffer->device_type_, dst = device_type_;
    CHECK(src != DeviceType::DeviceUnknown && dst != DeviceType::DeviceUnknown);
    const size_t n = byte_size_ < buffer->byte_size_ ? byte_size_ : buffer->byte_size_;
    const bool src_cuda = src == DeviceType::DeviceCUDA, dst_cuda = dst == DeviceType::DeviceCUDA;
    MemcpyKind kind = MemcpyKind::MemcpyCPU2CPU;
    if (src_cuda && dst_cuda) kind = MemcpyKind::MemcpyCUDA2CUDA;
    else if (src_cuda) kind = MemcpyKind::MemcpyCUDA2CPU;
    else if (dst_cuda) kind = MemcpyKind::MemcpyCPU2CUDA;
    allocator_->memcpy(ptr_, buffer->ptr_, n, kind);
}

void* Buffer::ptr() { return ptr_; }
const void* Buffer::ptr() const { return ptr_; }
size_t Buffer::byte_size() const { return byte_size_; }
std::shared_ptr<DeviceAllocator> Buffer::allocator() const { return allocator_; }
DeviceType Buffer::device_type() const { return device_type_; }
void Buffer::set_device_type(DeviceType device_type) { device_type_ = device_type; }
std::shared_ptr<Buffer> Buffer::get_shared_from_this() { return shared_from_this(); }
bool Buffer::is_external() const { return use_external_; }

}  // namespace base
