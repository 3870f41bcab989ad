// Built-in checks of the base / tensor / op classes, reachable through kuiper_selftest().
//
// They restate, against this implementation, what the reference's unit tests pin:
// buffers (test/test_tensor/test_buffer.cpp:7-114: ownership flags, allocator identity,
// device tags, copy_from in the three CUDA directions), tensors
// (test/test_tensor/test_tensor.cpp:6-276: constructors of every rank, strides, clone,
// to_cpu / to_cuda, borrowed pointers, assgin) and the add operator through the kernel
// registry (test/test_op/test_op_add.cpp:7-91) plus the VecAddLayer the reference never
// exercises.  gtest is not a dependency here: each EXPECT appends a line to the report.
#include <cstring>
#include <numeric>
#include <sstream>
#include <vector>

#include "kuiper_llama.h"
#include "op/add.h"
#include "op/kernel/kernel_interface.h"
#include "op/matmul.h"
#include "tensor/tensor.h"

namespace {

struct Report {
    std::ostringstream out;
    int failed = 0;
    int passed = 0;
    void expect(bool ok, const char* expr, const char* file, int line) {
        if (ok) {
            passed++;
        } else {
            failed++;
            out << "FAILED " << file << ":" << line << " " << expr << "\n";
        }
    }
};

#define EXPECT(cond) rep.expect((cond), #cond, __FILE__, __LINE__)

using base::DataType;
using base::DeviceType;
using tensor::Tensor;

void fill_device(float* dev, size_t n, float v) {
    std::vector<float> h(n, v);
    cudaMemcpy(dev, h.data(), n * sizeof(float), cudaMemcpyHostToDevice);
}

bool all_equal_device(const float* dev, size_t n, float v, float tol = 0.f) {
    std::vector<float> h(n);
    cudaMemcpy(h.data(), dev, n * sizeof(float), cudaMemcpyDeviceToHost);
    for (float x : h)
        if (!(x >= v - tol && x <= v + tol)) return false;
    return true;
}

void test_status(Report& rep) {
    base::Status ok = base::error::success();
    base::Status bad = base::error::invalid_argument("nope");
    EXPECT(bool(ok) && int(ok) == 0);
    EXPECT(!bool(bad) && bad == base::StatusCode::InvalidArgument && bad.get_err_msg() == "nope");
    EXPECT(base::error::key_has_exits().get_err_code() == 6 && base::error::internal_error().get_err_code() == 5);
    EXPECT(base::data_type_size(DataType::DataTypeFp32) == 4 && base::data_type_size(DataType::DataTypeInt8) == 1 &&
           base::data_type_size(DataType::DataTypeInt32) == 4 && base::data_type_size(DataType::DataTypeBf16) == 2 &&
           base::data_type_size(DataType::DataTypeFp16) == 2);
}

void test_buffer_cpu(Report& rep) {
    auto alloc = base::CPUDeviceAllocatorFactory::get_instance();
    base::Buffer buffer(32, alloc);
    EXPECT(buffer.ptr() != nullptr && buffer.byte_size() == 32 && !buffer.is_external());
    EXPECT(buffer.allocator() == alloc && buffer.device_type() == DeviceType::DeviceCPU);
    buffer.set_device_type(DeviceType::DeviceCUDA);
    EXPECT(buffer.device_type() == DeviceType::DeviceCUDA);

    float* raw = new float[32];
    {
        base::Buffer ext(32, nullptr, raw, true);
        EXPECT(ext.is_external() && ext.byte_size() == 32 && ext.ptr() == raw);
    }
    raw[0] = 1.f;  // still ours: a borrowed buffer never frees
    delete[] raw;

    auto shared = std::make_shared<base::Buffer>(16, alloc);
    EXPECT(shared->get_shared_from_this() == shared);
}

void test_tensor_cpu(Report& rep) {
    auto alloc = base::CPUDeviceAllocatorFactory::get_instance();
    Tensor t3(DataType::DataTypeFp32, 32, 32, 3, true, alloc);
    EXPECT(!t3.is_empty() && t3.dims_size() == 3 && t3.size() == 32u * 32 * 3);
    EXPECT(t3.strides() == std::vector<size_t>({96, 3, 1}));
    EXPECT(t3.byte_size() == t3.size() * 4 && t3.device_type() == DeviceType::DeviceCPU);

    Tensor t5(DataType::DataTypeFp32, std::vector<int32_t>{2, 3, 4, 5, 6}, true, alloc);
    EXPECT(t5.dims_size() == 5 && t5.size() == 720 && t5.strides() == std::vector<size_t>({360, 120, 30, 6, 1}));

    // borrowed pointer: device tag is set by hand, pointer arithmetic in elements
    float* raw = new float[32];
    raw[0] = 31;
    raw[1] = 32;
    Tensor tb(DataType::DataTypeFp32, 32, false, nullptr, raw);
    EXPECT(tb.device_type() == DeviceType::DeviceUnknown);
    tb.set_device_type(DeviceType::DeviceCPU);
    EXPECT(tb.device_type() == DeviceType::DeviceCPU && tb.ptr<float>() == raw && *tb.ptr<float>(1) == 32);
    EXPECT(tb.get_buffer()->is_external());

    // clone is deep
    Tensor t1(DataType::DataTypeFp32, 32, 32, true, alloc);
    for (size_t i = 0; i < t1.size(); i++) t1.index<float>(int64_t(i)) = 1.f;
    Tensor t2 = t1.clone();
    t2.index<float>(0) = 7.f;
    EXPECT(t1.index<float>(0) == 1.f && t2.index<float>(1) == 1.f && t2.ptr<float>() != t1.ptr<float>());
    EXPECT(t2.dims() == t1.dims() && t2.data_type() == t1.data_type() && t2.byte_size() == t1.byte_size());

    // assgin accepts a buffer that is large enough, refuses one that is too small
    auto big = std::make_shared<base::Buffer>(32 * 32 * 4, nullptr, new float[32 * 32], true);
    big->set_device_type(DeviceType::DeviceCPU);
    EXPECT(t1.assgin(big) && t1.ptr<void>() == big->ptr() && t1.size() == 32u * 32);
    auto small = std::make_shared<base::Buffer>(16, alloc);
    EXPECT(!t1.assgin(small));
    delete[] static_cast<float*>(big->ptr());

    // reshape grows by copy and keeps contents
    Tensor tr(DataType::DataTypeFp32, 4, true, alloc);
    for (int i = 0; i < 4; i++) tr.index<float>(i) = float(i);
    tr.reshape({2, 4});
    EXPECT(tr.size() == 8 && tr.index<float>(3) == 3.f && tr.dims() == std::vector<int32_t>({2, 4}));
    tr.reset(DataType::DataTypeInt32, {3});
    EXPECT(tr.is_empty() && tr.size() == 3 && tr.data_type() == DataType::DataTypeInt32);
    delete[] raw;
}

void test_layer_cpu(Report& rep) {
    // slot bookkeeping and argument checking need no device
    op::MatmulLayer mm(DeviceType::DeviceCUDA, 256, 128, true);
    EXPECT(mm.weights_size() == 2 && mm.input_size() == 1 && mm.output_size() == 1 && mm.group_size() == 128);
    EXPECT(mm.layer_type() == op::LayerType::LayerMatmul && mm.data_type() == DataType::DataTypeFp32);
    mm.set_residual(true);
    EXPECT(mm.input_size() == 2);
    base::Status st = mm.check();  // nothing bound yet
    EXPECT(!st && st == base::StatusCode::InvalidArgument);
    auto alloc = base::CPUDeviceAllocatorFactory::get_instance();
    Tensor wrong(DataType::DataTypeFp32, 4, true, alloc);
    EXPECT(!mm.set_weight(0, wrong));  // fp32 is not the packed INT4 word type
    op::VecAddLayer add(DeviceType::DeviceCUDA);
    EXPECT(add.input_size() == 2 && add.output_size() == 1 && add.layer_name() == "Add");
    EXPECT(!add.forward());  // empty tensors are rejected by check()
}

void test_cuda(Report& rep) {
    auto cu = base::CUDADeviceAllocatorFactory::get_instance();
    auto cpu = base::CPUDeviceAllocatorFactory::get_instance();
    {
        base::Buffer b(32, cu);
        EXPECT(b.ptr() != nullptr && !b.is_external() && b.device_type() == DeviceType::DeviceCUDA && b.allocator() == cu);
    }
    {  // copy_from: host -> device -> device -> host
        const int n = 32;
        base::Buffer host(n * 4, cpu), d1(n * 4, cu), d2(n * 4, cu), back(n * 4, cpu);
        float* hp = static_cast<float*>(host.ptr());
        for (int i = 0; i < n; i++) hp[i] = float(i);
        d1.copy_from(host);
        d2.copy_from(&d1);
        back.copy_from(d2);
        bool same = true;
        for (int i = 0; i < n; i++) same = same && static_cast<float*>(back.ptr())[i] == float(i);
        EXPECT(same);
    }
    {  // to_cpu / to_cuda / clone on the device
        Tensor t(DataType::DataTypeFp32, 32, 32, true, cu);
        fill_device(t.ptr<float>(), t.size(), 1.f);
        Tensor c = t.clone();
        EXPECT(c.device_type() == DeviceType::DeviceCUDA && c.ptr<float>() != t.ptr<float>() &&
               all_equal_device(c.ptr<float>(), c.size(), 1.f));
        t.to_cpu();
        EXPECT(t.device_type() == DeviceType::DeviceCPU && t.index<float>(1023) == 1.f);
        t.to_cuda();
        EXPECT(t.device_type() == DeviceType::DeviceCUDA && all_equal_device(t.ptr<float>(), t.size(), 1.f));
    }
    {  // arena: no driver call per allocation, 256-byte granularity, exhaustion is reported by CHECK
        auto arena = std::make_shared<base::CUDAArenaAllocator>(4096);
        Tensor a(DataType::DataTypeFp32, 10, true, arena), b(DataType::DataTypeFp32, 10, true, arena);
        EXPECT(a.ptr<char>() + 256 == b.ptr<char>() && arena->used() == 512);
    }
    // add through the registry, default stream and user stream, plus the unaligned tail case
    for (int variant = 0; variant < 3; variant++) {
        const bool big = variant == 2;
        Tensor a = big ? Tensor(DataType::DataTypeFp32, 32, 151, 13, true, cu) : Tensor(DataType::DataTypeFp32, 32, 151, true, cu);
        Tensor b = a.clone(), out = a.clone();
        fill_device(a.ptr<float>(), a.size(), big ? 2.1f : 2.f);
        fill_device(b.ptr<float>(), b.size(), big ? 3.3f : 3.f);
        cudaStream_t s = nullptr;
        if (variant == 1) cudaStreamCreate(&s);
        kernel::get_add_kernel(DeviceType::DeviceCUDA)(a, b, out, s);
        cudaDeviceSynchronize();
        EXPECT(all_equal_device(out.ptr<float>(), out.size(), big ? 5.4f : 5.f, big ? 1e-4f : 0.f));
        if (s) cudaStreamDestroy(s);
    }
    {  // the layer path the reference never tests
        op::VecAddLayer add(DeviceType::DeviceCUDA);
        auto cfg = std::make_shared<kernel::CudaConfig>();
        cfg->create();
        add.set_cuda_config(cfg);
        Tensor a(DataType::DataTypeFp32, 1000, true, cu), b(DataType::DataTypeFp32, 1000, true, cu),
            out(DataType::DataTypeFp32, 1000, true, cu);
        fill_device(a.ptr<float>(), 1000, 2.f);
        fill_device(b.ptr<float>(), 1000, 3.f);
        EXPECT(bool(add.forward(a, b, out)));
        cudaStreamSynchronize(cfg->stream());
        EXPECT(all_equal_device(out.ptr<float>(), 1000, 5.f));
        Tensor short_out(DataType::DataTypeFp32, 999, true, cu);
        EXPECT(!add.forward(a, b, short_out));
    }
}

}  // namespace

extern "C" int kuiper_selftest(int use_cuda, char* report, size_t report_bytes) {
    Report rep;
    test_status(rep);
    test_buffer_cpu(rep);
    test_tensor_cpu(rep);
    test_layer_cpu(rep);
    if (use_cuda) test_cuda(rep);
    rep.out << rep.passed << " checks passed, " << rep.failed << " failed\n";
    if (report && report_bytes > 0) {
        const std::string s = rep.out.str();
        const size_t n = s.size() < report_bytes - 1 ? s.size() : report_bytes - 1;
        std::memcpy(report, s.data(), n);
        report[n] = '\0';
    }
    return rep.failed;
}
