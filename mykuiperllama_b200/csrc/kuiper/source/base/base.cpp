// Status value type and its factories (interface: kuiper/include/base/base.h:92-135 of the reference).
#include "base/base.h"

namespace base {

Status::Status(int code, std::string err_msg) : code_(code), err_msg_(std::move(err_msg)) {}

Status& Status::operator=(int code) {
    code_ = code;
    return *this;
}

bool Status::operator==(int code) const { return code_ == code; }
bool Status::operator!=(int code) const { return code_ != code; }
Status::operator int() const { return code_; }
Status::operator bool() const { return code_ == StatusCode::Success; }
int Status::get_err_code() const { return code_; }
const std::string& Status::get_err_msg() const { return err_msg_; }
void Status::set_err_msg(const std::string& err_msg) { err_msg_ = err_msg; }

namespace error {
namespace {
Status make(StatusCode code, const std::string& msg) { return Status(int(code), msg); }
}  // namespace

Status success(const std::string& err_msg) { return make(StatusCode::Success, err_msg); }
Status function_not_implement(const std::string& err_msg) { return make(StatusCode::FunctionUnImplement, err_msg); }
Status path_not_valid(const std::string& err_msg) { return make(StatusCode::PathNotValid, err_msg); }
Status model_parse_error(const std::string& err_msg) { return make(StatusCode::ModelParseError, err_msg); }
Status internal_error(const std::string& err_msg) { return make(StatusCode::InternalError, err_msg); }
Status key_has_exits(const std::string& err_msg) { return make(StatusCode::KeyValueHasExist, err_msg); }
Status invalid_argument(const std::string& err_msg) { return make(StatusCode::InvalidArgument, err_msg); }
}  // namespace error

std::ostream& operator<<(std::ostream& os, const Status& status) { return os << status.get_err_msg(); }

}  // namespace base
