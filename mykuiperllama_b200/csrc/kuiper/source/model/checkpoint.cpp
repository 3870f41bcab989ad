// safetensors container: header parse (a small JSON reader, enough for the header's grammar) + mmap.
#include "model/checkpoint.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>

namespace model {
namespace {

// recursive-descent reader over the header text; only what a safetensors header can contain
class HeaderReader {
public:
    HeaderReader(const char* p, size_t n) : p_(p), end_(p + n) {}

    bool fail() const { return failed_; }
    const std::string& why() const { return why_; }

    void skip_ws() {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) p_++;
    }
    bool consume(char c) {
        skip_ws();
        if (p_ < end_ && *p_ == c) {
            p_++;
            return true;
        }
        return false;
    }
    void expect(char c) {
        if (!consume(c)) error(std::string("expected '") + c + "'");
    }
    bool peek(char c) {
        skip_ws();
        return p_ < end_ && *p_ == c;
    }
    std::string string() {
        std::string out;
        skip_ws();
        if (p_ >= end_ || *p_ != '"') {
            error("expected a string");
            return out;
        }
        p_++;
        while (p_ < end_ && *p_ != '"') {
            if (*p_ == '\\') {
                p_++;
                if (p_ >= end_) break;
                switch (*p_) {
                    case 'n': out.push_back('\n'); break;
                    case 't': out.push_back('\t'); break;
                    case 'r': out.push_back('\r'); break;
                    case 'b': out.push_back('\b'); break;
                    case 'f': out.push_back('\f'); break;
                    case 'u': {  // kept verbatim: tensor names are ASCII, metadata is only passed through
                        out += "\\u";
                        break;
                    }
                    default: out.push_back(*p_); break;
                }
                p_++;
            } else {
                out.push_back(*p_++);
            }
        }
        if (p_ >= end_) {
            error("unterminated string");
            return out;
        }
        p_++;
        return out;
    }
    int64_t integer() {
        skip_ws();
        bool neg = false;
        if (p_ < end_ && *p_ == '-') {
            neg = true;
            p_++;
        }
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') {
            error("expected an integer");
            return 0;
        }
        int64_t v = 0;
        while (p_ < end_ && *p_ >= '0' && *p_ <= '9') {
            if (v > (INT64_MAX - 9) / 10) {
                error("integer overflow");
                return 0;
            }
            v = v * 10 + (*p_++ - '0');
        }
        return neg ? -v : v;
    }
    std::vector<int64_t> int_array() {
        std::vector<int64_t> out;
        expect('[');
        if (consume(']')) return out;
        do {
            out.push_back(integer());
        } while (!failed_ && consume(','));
        expect(']');
        return out;
    }
    // skips any value (used for unknown keys)
    void skip_value() {
        skip_ws();
        if (p_ >= end_) return error("unexpected end of header");
        if (*p_ == '"') {
            string();
        } else if (*p_ == '{') {
            p_++;
            if (consume('}')) return;
            do {
                string();
                expect(':');
                skip_value();
            } while (!failed_ && consume(','));
            expect('}');
        } else if (*p_ == '[') {
            p_++;
            if (consume(']')) return;
            do {
                skip_value();
            } while (!failed_ && consume(','));
            expect(']');
        } else {
            while (p_ < end_ && *p_ != ',' && *p_ != '}' && *p_ != ']') p_++;
        }
    }
    void error(const std::string& what) {
        if (!failed_) {
            failed_ = true;
            why_ = what;
        }
    }

private:
    const char* p_;
    const char* end_;
    bool failed_ = false;
    std::string why_;
};

size_t dtype_bytes(const std::string& dt) {
    if (dt == "F64" || dt == "I64" || dt == "U64") return 8;
    if (dt == "F32" || dt == "I32" || dt == "U32") return 4;
    if (dt == "F16" || dt == "BF16" || dt == "I16" || dt == "U16") return 2;
    if (dt == "I8" || dt == "U8" || dt == "BOOL" || dt == "F8_E4M3" || dt == "F8_E5M2") return 1;
    return 0;
}

}  // namespace

int64_t CheckpointTensor::element_count() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, map_bytes_);
}

const CheckpointTensor* SafetensorsFile::find(const std::string& name) const {
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}

base::Status SafetensorsFile::open(const std::string& path, std::unique_ptr<SafetensorsFile>* out) {
    if (!out) return base::error::invalid_argument("null output");
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) return base::error::path_not_valid("cannot open " + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
        ::close(fd);
        return base::error::model_parse_error(path + " is too short for a safetensors file");
    }
    const size_t file_bytes = size_t(st.st_size);
    void* map = mmap(nullptr, file_bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (map == MAP_FAILED) return base::error::internal_error("mmap of " + path + " failed");
    std::unique_ptr<SafetensorsFile> f(new SafetensorsFile());
    f->map_ = map;
    f->map_bytes_ = file_bytes;
    const unsigned char* base_ptr = static_cast<const unsigned char*>(map);
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; i--) header_len = (header_len << 8) | base_ptr[i];  // little endian
    if (header_len == 0 || header_len > file_bytes - 8 || header_len > (uint64_t(1) << 30))
        return base::error::model_parse_error("header length of " + path + " exceeds the file");
    const unsigned char* data0 = base_ptr + 8 + header_len;
    const size_t data_bytes = file_bytes - 8 - size_t(header_len);

    HeaderReader r(reinterpret_cast<const char*>(base_ptr + 8), size_t(header_len));
    r.expect('{');
    if (!r.peek('}')) {
        do {
            const std::string name = r.string();
            r.expect(':');
            if (name == "__metadata__") {
                r.expect('{');
                if (!r.consume('}')) {
                    do {
                        const std::string k = r.string();
                        r.expect(':');
                        if (r.peek('"')) f->metadata_[k] = r.string();
                        else r.skip_value();
                    } while (!r.fail() && r.consume(','));
                    r.expect('}');
                }
                continue;
            }
            CheckpointTensor t;
            std::vector<int64_t> offsets;
            r.expect('{');
            if (!r.consume('}')) {
                do {
                    const std::string k = r.string();
                    r.expect(':');
                    if (k == "dtype") t.dtype = r.string();
                    else if (k == "shape") t.shape = r.int_array();
                    else if (k == "data_offsets") offsets = r.int_array();
                    else r.skip_value();
                } while (!r.fail() && r.consume(','));
                r.expect('}');
            }
            if (r.fail()) break;
            const size_t esz = dtype_bytes(t.dtype);
            if (esz == 0) return base::error::model_parse_error("tensor " + name + " has an unknown dtype " + t.dtype);
            if (offsets.size() != 2 || offsets[0] < 0 || offsets[1] < offsets[0] || uint64_t(offsets[1]) > data_bytes)
                return base::error::model_parse_error("tensor " + name + " lies outside the file");
            int64_t n = 1;
            for (int64_t d : t.shape) {
                if (d < 0 || (d > 0 && n > INT64_MAX / d)) return base::error::model_parse_error("tensor " + name + " has a bad shape");
                n *= d;
            }
            t.bytes = size_t(offsets[1] - offsets[0]);
            if (uint64_t(n) * esz != t.bytes) return base::error::model_parse_error("tensor " + name + ": shape and byte range disagree");
            t.data = data0 + offsets[0];
            f->tensors_[name] = std::move(t);
        } while (!r.fail() && r.consume(','));
    }
    r.expect('}');
    if (r.fail()) return base::error::model_parse_error("header of " + path + " is not valid: " + r.why());
    *out = std::move(f);
    return base::error::success();
}

}  // namespace model
