// Byte-source adapters with the upstream spelling (CodedInputStream,
// FileInputStream ...) on top of the small wire reader in message.h.
#ifndef MCB200_PROTO_RUNTIME_CODED_STREAM_H_
#define MCB200_PROTO_RUNTIME_CODED_STREAM_H_

#include <string>

#include "google/protobuf/message.h"

namespace google {
namespace protobuf {
namespace io {

class ZeroCopyInputStream {
 public:
  virtual ~ZeroCopyInputStream() {}
  // Drains the source; the returned buffer lives as long as the stream.
  virtual const std::string& ReadAll() = 0;
};

class ZeroCopyOutputStream {
 public:
  virtual ~ZeroCopyOutputStream() {}
  virtual bool WriteAll(const std::string& data) = 0;
};

class CodedInputStream {
 public:
  CodedInputStream(const uint8* buffer, int size) : data_(buffer), size_(size) {}
  explicit CodedInputStream(ZeroCopyInputStream* in) {
    const std::string& all = in->ReadAll();
    data_ = reinterpret_cast<const uint8*>(all.data());
    size_ = all.size();
  }
  // Accepted for source compatibility; this reader has no size limit.
  void SetTotalBytesLimit(int, int) {}
  void SetTotalBytesLimit(int) {}
  const uint8* data() const { return data_; }
  std::size_t size() const { return size_; }

 private:
  const uint8* data_;
  std::size_t size_;
};

}  // namespace io
}  // namespace protobuf
}  // namespace google

#endif  // MCB200_PROTO_RUNTIME_CODED_STREAM_H_
