// Allocators: copy / clear helpers shared by all devices, the malloc-backed CPU
// allocator, the cudaMalloc-backed CUDA allocator and the arena.  Behaviour follows the
// reference's kuiper/source/base/alloc.cpp:6-74, alloc_cpu.cpp:7-20, alloc_cu.cpp:8-23.
#include "base/alloc.h"

#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>

namespace base {

void DeviceAllocator::memcpy(void* dest_ptr, const void* src_ptr, size_t byte_size, MemcpyKind memcpy_kind,
                             void* stream, bool need_sync) const {
    CHECK_NE(dest_ptr, nullptr);
    CHECK_NE(src_ptr, nullptr);
    if (byte_size == 0) return;

    if (memcpy_kind == MemcpyKind::MemcpyCPU2CPU) {
        std::memcpy(dest_ptr, src_ptr, byte_size);
    } else {
        cudaMemcpyKind kind;
        switch (memcpy_kind) {
            case MemcpyKind::MemcpyCPU2CUDA: kind = cudaMemcpyHostToDevice; break;
            case MemcpyKind::MemcpyCUDA2CPU: kind = cudaMemcpyDeviceToHost; break;
            case MemcpyKind::MemcpyCUDA2CUDA: kind = cudaMemcpyDeviceToDevice; break;
            default: LOG(FATAL) << "Unknown memcpy kind: " << int(memcpy_kind); return;
        }
        cudaError_t err = stream ? cudaMemcpyAsync(dest_ptr, src_ptr, byte_size, kind, static_cast<cudaStream_t>(stream))
                                 : cudaMemcpy(dest_ptr, src_ptr, byte_size, kind);
        CHECK_EQ(int(err), int(cudaSuccess)) << "memcpy failed: " << cudaGetErrorString(err);
    }
    if (need_sync) cudaDeviceSynchronize();
}

void DeviceAllocator::memset_zero(void* ptr, size_t byte_size, void* stream, bool need_sync) {
    CHECK(device_type_ != DeviceType::DeviceUnknown);
    if (device_type_ == DeviceType::DeviceCPU) {
        std::memset(ptr, 0, byte_size);
    } else if (stream) {
        cudaMemsetAsync(ptr, 0, byte_size, static_cast<cudaStream_t>(stream));
    } else {
        cudaMemset(ptr, 0, byte_size);
    }
    if (need_sync) cudaDeviceSynchronize();
}

// ---- CPU
CPUDeviceAllocator::CPUDeviceAllocator() : DeviceAllocator(DeviceType::DeviceCPU) {}

void* CPUDeviceAllocator::allocate(size_t byte_size) const { return byte_size ? std::malloc(byte_size) : nullptr; }

void CPUDeviceAllocator::release(void* ptr) const {
    if (ptr) std::free(ptr);
}

// ---- CUDA
CUDADeviceAllocator::CUDADeviceAllocator() : DeviceAllocator(DeviceType::DeviceCUDA) {}

void* CUDADeviceAllocator::allocate(size_t byte_size) const {
    if (byte_size == 0) return nullptr;
    void* ptr = nullptr;
    cudaError_t err = cudaMalloc(&ptr, byte_size);
    CHECK_EQ(int(err), int(cudaSuccess)) << "cudaMalloc of " << byte_size << " bytes failed: " << cudaGetErrorString(err);
    return ptr;
}

void CUDADeviceAllocator::release(void* ptr) const {
    if (ptr) cudaFree(ptr);
}

// ---- arena
CUDAArenaAllocator::CUDAArenaAllocator(size_t capacity_bytes)
    : DeviceAllocator(DeviceType::DeviceCUDA), capacity_(capacity_bytes) {
    if (capacity_ == 0) return;
    void* ptr = nullptr;
    cudaError_t err = cudaMalloc(&ptr, capacity_);
    CHECK_EQ(int(err), int(cudaSuccess)) << "arena of " << capacity_ << " bytes failed: " << cudaGetErrorString(err);
    base_ = static_cast<char*>(ptr);
}

CUDAArenaAllocator::~CUDAArenaAllocator() {
    if (base_) cudaFree(base_);
}

void* CUDAArenaAllocator::allocate(size_t byte_size) const {
    if (byte_size == 0) return nullptr;
    const size_t rounded = (byte_size + 255) / 256 * 256;
    CHECK_LE(offset_ + rounded, capacity_) << "arena exhausted: " << offset_ << " + " << rounded << " > " << capacity_;
    void* ptr = base_ + offset_;
    offset_ += rounded;
    return ptr;
}

void CUDAArenaAllocator::release(void*) const {}

std::shared_ptr<CPUDeviceAllocator> CPUDeviceAllocatorFactory::instance = nullptr;
std::shared_ptr<CUDADeviceAllocator> CUDADeviceAllocatorFactory::instance = nullptr;

}  // namespace base
