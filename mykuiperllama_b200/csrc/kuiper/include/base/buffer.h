// A byte range on one device, owned (released through its allocator on destruction) or
// borrowed (use_external: never released).  Interface of the reference's
// kuiper/include/base/buffer.h:17-45.  One deliberate difference: the reference inherits
// enable_shared_from_this privately (buffer.h:17), which makes get_shared_from_this()
// throw; here the base is public so the call works.
#ifndef KUIPER_INCLUDE_BASE_BUFFER_H
#define KUIPER_INCLUDE_BASE_BUFFER_H

#include "base/alloc.h"

namespace base {

class Buffer : public NoCopyable, public std::enable_shared_from_this<Buffer> {
public:
    explicit Buffer() = default;
    explicit Buffer(size_t byte_size, std::shared_ptr<DeviceAllocator> allocator = nullptr, void* ptr = nullptr,
                    bool use_external = false);
    virtual ~Buffer();

    bool allocate();
    // copies min(byte sizes); the direction comes from the two device tags
    void copy_from(const Buffer& buffer) const;
    void copy_from(const Buffer* buffer) const;

    void* ptr();
    const void* ptr() const;
    size_t byte_size() const;
    std::shared_ptr<DeviceAllocator> allocator() const;
    DeviceType device_type() const;
    void set_device_type(DeviceType device_type);
    std::shared_ptr<Buffer> get_shared_from_this();
    bool is_external() const;

private:
    size_t byte_size_ = 0;
    void* ptr_ = nullptr;
    bool use_external_ = false;
    DeviceType device_type_ = DeviceType::DeviceUnknown;
    std::shared_ptr<DeviceAllocator> allocator_;
};

}  // namespace base

#endif  // KUIPER_INCLUDE_BASE_BUFFER_H
