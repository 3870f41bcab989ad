// Minimal logging / assertion macros with the glog spelling: LOG(INFO|WARNING|ERROR|FATAL)
// streams a line to stderr, FATAL aborts; CHECK(cond) and CHECK_{EQ,NE,LT,LE,GT,GE}(a, b)
// abort with the failed expression and accept a trailing `<< message`.
#ifndef KUIPER_BASE_LOG_H
#define KUIPER_BASE_LOG_H

#include <cstdlib>
#include <iostream>
#include <sstream>

namespace kuiper_log {

enum Severity { INFO = 0, WARNING = 1, ERROR = 2, FATAL = 3 };

// set to WARNING to silence LOG(INFO) (environment variable KUIPER_LOG_LEVEL, 0..3)
inline int min_severity() {
    static const int level = [] {
        const char* env = std::getenv("KUIPER_LOG_LEVEL");
        return env ? std::atoi(env) : 0;
    }();
    return level;
}

class Message {
public:
    Message(const char* file, int line, Severity sev) : sev_(sev) {
        static const char tag[] = {'I', 'W', 'E', 'F'};
        stream_ << tag[sev] << ' ' << file << ':' << line << "] ";
    }
    ~Message() {
        if (sev_ >= min_severity()) std::cerr << stream_.str() << std::endl;
        if (sev_ == FATAL) std::abort();
    }
    std::ostream& stream() { return stream_; }

private:
    Severity sev_;
    std::ostringstream stream_;
};

// swallows the stream expression of a CHECK that held
struct Voidify {
    void operator&(std::ostream&) {}
};

}  // namespace kuiper_log

#define LOG(severity) ::kuiper_log::Message(__FILE__, __LINE__, ::kuiper_log::severity).stream()

#define CHECK(cond)  \
    (cond) ? (void)0 \
           : ::kuiper_log::Voidify() & ::kuiper_log::Message(__FILE__, __LINE__, ::kuiper_log::FATAL).stream() << "Check failed: " #cond " "

#define KUIPER_CHECK_OP(a, b, op) CHECK((a)op(b))
#define CHECK_EQ(a, b) KUIPER_CHECK_OP(a, b, ==)
#define CHECK_NE(a, b) KUIPER_CHECK_OP(a, b, !=)
#define CHECK_LT(a, b) KUIPER_CHECK_OP(a, b, <)
#define CHECK_LE(a, b) KUIPER_CHECK_OP(a, b, <=)
#define CHECK_GT(a, b) KUIPER_CHECK_OP(a, b, >)
#define CHECK_GE(a, b) KUIPER_CHECK_OP(a, b, >=)

#endif  // KUIPER_BASE_LOG_H
