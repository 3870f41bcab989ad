// Status codes, device / data type tags and the decode-step buffer names.
//
// Same public names and numeric values as the reference's kuiper/include/base/base.h
// (ModelBufferType :12-31, DeviceType :35-39, DataType :41-46, StatusCode :76-84,
// Status :92-110, STATUS_CHECK :115-126, error factories :128-134), extended with the
// 16-bit float tags the INT4 path needs (the reference stops at Fp32 / Int8 / Int32).
// Packed INT4 has no tag of its own: a [K, N] 4-bit matrix is an Int32 tensor of dims
// [K, N/8], because data_type_size() is in whole bytes.
#ifndef KUIPER_INCLUDE_BASE_BASE_H
#define KUIPER_INCLUDE_BASE_BASE_H

#include <glog/logging.h>

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <ostream>
#include <string>

#define UNUSED(expr) \
    do {             \
        (void)(expr); \
    } while (0)

namespace model {
// names of the intermediate buffers of one forward pass
enum class ModelBufferType {
    InputTokens = 0,
    InputEmbeddings = 1,
    OutputRMSNorm = 2,
    KeyCache = 3,
    ValueCache = 4,
    Query = 5,
    InputPos = 6,
    ScoreStorage = 7,  // kept for API compatibility; flash-decoding never materialises scores
    OutputMHA = 8,
    AttnOutput = 9,
    W1Output = 10,
    W2Output = 11,
    W3Output = 12,
    FFNRMSNorm = 13,
    ForwardOutput = 15,
    ForwardOutputCPU = 16,
    SinCache = 17,
    CosCache = 18,
    // additions of this engine (values above the reference's range)
    QKVOutput = 32,     // fused q|k|v projection output
    SeqLen = 33,        // per-row attention length (pos + 1)
    SeqSlot = 34,       // per-row KV-cache sequence slot
    NextTokens = 35,    // greedy ids on the device
    MatmulWorkspace = 36,
    MHAWorkspace = 37,
    GemmWorkspace = 38,  // fp16 copy of the activation rows for the tensor-core matmul
    LogitsShard = 39,    // tensor parallelism: this rank's slice of the logits [rows, vocab / tp]
    LogitsGather = 40,   // tensor parallelism: the slices of all ranks [tp, rows, vocab / tp]
};
}  // namespace model

namespace base {

enum class DeviceType : uint8_t { DeviceUnknown = 0, DeviceCPU = 1, DeviceCUDA = 2 };

enum class DataType : uint8_t {
    DataTypeUnknown = 0,
    DataTypeFp32 = 1,
    DataTypeInt8 = 2,
    DataTypeInt32 = 3,
    DataTypeBf16 = 4,  // extension
    DataTypeFp16 = 5,  // extension
};

enum class ModelType : uint8_t {
    ModelTypeUnown = 0,
    ModelTypeLLama2 = 1,
    ModelTypeQwen3 = 2,  // extension
};

inline size_t data_type_size(DataType data_type) {
    switch (data_type) {
        case DataType::DataTypeFp32: return sizeof(float);
        case DataType::DataTypeInt8: return sizeof(int8_t);
        case DataType::DataTypeInt32: return sizeof(int32_t);
        case DataType::DataTypeBf16:
        case DataType::DataTypeFp16: return sizeof(uint16_t);
        default: break;
    }
    LOG(FATAL) << "Unknown data type size for " << int(data_type);
    return 0;
}

class NoCopyable {
protected:
    NoCopyable() = default;
    ~NoCopyable() = default;
    NoCopyable(const NoCopyable&) = delete;
    NoCopyable& operator=(const NoCopyable&) = delete;
};

enum StatusCode : uint8_t {
    Success = 0,
    FunctionUnImplement = 1,
    PathNotValid = 2,
    ModelParseError = 3,
    InternalError = 5,
    KeyValueHasExist = 6,
    InvalidArgument = 7,
};

enum class TokenizerType { EncodeUnknown = -1, EncodeSpe = 0, EncodeBpe = 1 };

class Status {
public:
    Status(int code = StatusCode::Success, std::string err_msg = "");
    Status(const Status& other) = default;
    Status& operator=(const Status& other) = default;
    Status& operator=(int code);
    bool operator==(int code) const;
    bool operator!=(int code) const;
    operator int() const;
    operator bool() const;  // true on success
    int get_err_code() const;
    const std::string& get_err_msg() const;
    void set_err_msg(const std::string& err_msg);

private:
    int code_ = StatusCode::Success;
    std::string err_msg_;
};

namespace error {
// evaluates `call`; on failure logs file, line, code and message and aborts
#define STATUS_CHECK(call)                                                                             \
    do {                                                                                               \
        const base::Status& status = call;                                                             \
        if (!status) {                                                                                 \
            char buf[512];                                                                             \
            snprintf(buf, sizeof(buf) - 1, "Infer error\n File: %s Line: %d\n Error code: %d\n Error msg: %s\n", \
                     __FILE__, __LINE__, int(status), status.get_err_msg().c_str());                   \
            LOG(FATAL) << buf;                                                                         \
        }                                                                                              \
    } while (0)

Status success(const std::string& err_msg = "");
Status function_not_implement(const std::string& err_msg = "");
Status path_not_valid(const std::string& err_msg = "");
Status model_parse_error(const std::string& err_msg = "");
Status internal_error(const std::string& err_msg = "");
Status key_has_exits(const std::string& err_msg = "");
Status invalid_argument(const std::string& err_msg = "");
}  // namespace error

std::ostream& operator<<(std::ostream& os, const Status& status);

}  // namespace base

#endif  // KUIPER_INCLUDE_BASE_BASE_H
