// File-descriptor backed streams (whole-file reads and writes).
#ifndef MCB200_PROTO_RUNTIME_ZERO_COPY_STREAM_IMPL_H_
#define MCB200_PROTO_RUNTIME_ZERO_COPY_STREAM_IMPL_H_

#include <string>

#include "google/protobuf/io/coded_stream.h"

namespace google {
namespace protobuf {
namespace io {

class FileInputStream : public ZeroCopyInputStream {
 public:
  explicit FileInputStream(int fd) : fd_(fd), drained_(false) {}
  const std::string& ReadAll() override;
 private:
  int fd_;
  bool drained_;
  std::string buf_;
};

class FileOutputStream : public ZeroCopyOutputStream {
 public:
  explicit FileOutputStream(int fd) : fd_(fd) {}
  bool WriteAll(const std::string& data) override;
 private:
  int fd_;
};

}  // namespace io
}  // namespace protobuf
}  // namespace google

#endif  // MCB200_PROTO_RUNTIME_ZERO_COPY_STREAM_IMPL_H_
