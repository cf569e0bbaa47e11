// Logging and checking macros of the public API: CHECK / CHECK_xx / LOG(sev) /
// DLOG / DCHECK with glog-like spelling.  A failed CHECK or LOG(FATAL) writes
// the message to stderr and throws caffe::Error (it does not abort), which the
// C API turns into a -1 return code.  Same contract as mini-caffe's
// include/caffe/logging.hpp:22-28,200-213.
#ifndef CAFFE_LOGGING_H_
#define CAFFE_LOGGING_H_

#include <ctime>
#include <iostream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>

namespace caffe {

/*! \brief thrown by every failed CHECK and by LOG(FATAL) */
struct Error : public std::runtime_error {
  explicit Error(const std::string& what) : std::runtime_error(what) {}
};

namespace logging {

inline std::string Prefix(const char* file, int line) {
  char stamp[16];
  std::time_t now = std::time(nullptr);
  std::tm parts;
  localtime_r(&now, &parts);
  std::snprintf(stamp, sizeof(stamp), "%02d:%02d:%02d", parts.tm_hour, parts.tm_min, parts.tm_sec);
  std::ostringstream os;
  os << "[" << stamp << "] " << file << ":" << line << ": ";
  return os.str();
}

/*! \brief one line to stderr, flushed when the temporary dies */
class Line {
 public:
  Line(const char* file, int line) { buf_ << Prefix(file, line); }
  ~Line() { std::cerr << buf_.str() << '\n'; }
  std::ostream& stream() { return buf_; }

 private:
  std::ostringstream buf_;
  Line(const Line&) = delete;
  void operator=(const Line&) = delete;
};

/*! \brief like Line, but the destructor throws caffe::Error with the text */
class FatalLine {
 public:
  FatalLine(const char* file, int line) { buf_ << Prefix(file, line); }
  ~FatalLine() noexcept(false) {
    std::cerr << buf_.str() << '\n';
    throw Error(buf_.str());
  }
  std::ostringstream& stream() { return buf_; }

 private:
  std::ostringstream buf_;
  FatalLine(const FatalLine&) = delete;
  void operator=(const FatalLine&) = delete;
};

/*! \brief swallows a stream expression in the disabled branch of LOG_IF / DLOG */
struct Voidify {
  void operator&(std::ostream&) {}
};

#define CAFFE_DEFINE_CMP_(name, op)                                      \
  struct name {                                                          \
    template <typename X, typename Y>                                    \
    bool operator()(const X& x, const Y& y) const { return x op y; }     \
  }
CAFFE_DEFINE_CMP_(CmpLT, <);
CAFFE_DEFINE_CMP_(CmpGT, >);
CAFFE_DEFINE_CMP_(CmpLE, <=);
CAFFE_DEFINE_CMP_(CmpGE, >=);
CAFFE_DEFINE_CMP_(CmpEQ, ==);
CAFFE_DEFINE_CMP_(CmpNE, !=);
#undef CAFFE_DEFINE_CMP_

/*! \brief null when the comparison holds, else " (x vs. y) " */
template <typename Cmp, typename X, typename Y>
inline std::unique_ptr<std::string> Compare(const X& x, const Y& y) {
  if (Cmp()(x, y)) return std::unique_ptr<std::string>();
  std::ostringstream os;
  os << " (" << x << " vs. " << y << ") ";
  return std::unique_ptr<std::string>(new std::string(os.str()));
}

}  // namespace logging
}  // namespace caffe

#define CAFFE_CHECK_OP_(cmp, op, x, y)                                                               \
  if (std::unique_ptr<std::string> caffe_check_msg_ =                                                \
          ::caffe::logging::Compare< ::caffe::logging::cmp>((x), (y)))                               \
  ::caffe::logging::FatalLine(__FILE__, __LINE__).stream() << "Check failed: " #x " " #op " " #y     \
                                                            << *caffe_check_msg_

#define CHECK(cond) \
  if (!(cond)) ::caffe::logging::FatalLine(__FILE__, __LINE__).stream() << "Check failed: " #cond << ' '
#define CHECK_LT(x, y) CAFFE_CHECK_OP_(CmpLT, <, x, y)
#define CHECK_GT(x, y) CAFFE_CHECK_OP_(CmpGT, >, x, y)
#define CHECK_LE(x, y) CAFFE_CHECK_OP_(CmpLE, <=, x, y)
#define CHECK_GE(x, y) CAFFE_CHECK_OP_(CmpGE, >=, x, y)
#define CHECK_EQ(x, y) CAFFE_CHECK_OP_(CmpEQ, ==, x, y)
#define CHECK_NE(x, y) CAFFE_CHECK_OP_(CmpNE, !=, x, y)
#define CHECK_NOTNULL(x)                                                                                      \
  ((x) == NULL ? ::caffe::logging::FatalLine(__FILE__, __LINE__).stream() << "Check  notnull: " #x << ' ', (x) \
               : (x))

#define LOG_INFO ::caffe::logging::Line(__FILE__, __LINE__)
#define LOG_WARNING LOG_INFO
#define LOG_ERROR LOG_INFO
#define LOG_FATAL ::caffe::logging::FatalLine(__FILE__, __LINE__)
#define LOG_QFATAL LOG_FATAL
#define LOG(severity) LOG_##severity.stream()
#define LG LOG_INFO.stream()
#define VLOG(level) LOG_INFO.stream()
#define LOG_IF(severity, cond) !(cond) ? (void)0 : ::caffe::logging::Voidify() & LOG(severity)
#define LOG_EVERY_N(severity, n) LOG(severity)

#ifdef NDEBUG
#define DCHECK(x) while (false) CHECK(x)
#define DCHECK_LT(x, y) while (false) CHECK((x) < (y))
#define DCHECK_GT(x, y) while (false) CHECK((x) > (y))
#define DCHECK_LE(x, y) while (false) CHECK((x) <= (y))
#define DCHECK_GE(x, y) while (false) CHECK((x) >= (y))
#define DCHECK_EQ(x, y) while (false) CHECK((x) == (y))
#define DCHECK_NE(x, y) while (false) CHECK((x) != (y))
#define LOG_DFATAL LOG_ERROR
#define DFATAL ERROR
#define DLOG(severity) true ? (void)0 : ::caffe::logging::Voidify() & LOG(severity)
#define DLOG_IF(severity, cond) (true || !(cond)) ? (void)0 : ::caffe::logging::Voidify() & LOG(severity)
#else
#define DCHECK(x) CHECK(x)
#define DCHECK_LT(x, y) CHECK((x) < (y))
#define DCHECK_GT(x, y) CHECK((x) > (y))
#define DCHECK_LE(x, y) CHECK((x) <= (y))
#define DCHECK_GE(x, y) CHECK((x) >= (y))
#define DCHECK_EQ(x, y) CHECK((x) == (y))
#define DCHECK_NE(x, y) CHECK((x) != (y))
#define LOG_DFATAL LOG_FATAL
#define DFATAL FATAL
#define DLOG(severity) LOG(severity)
#define DLOG_IF(severity, cond) LOG_IF(severity, cond)
#endif  // NDEBUG

#endif  // CAFFE_LOGGING_H_
