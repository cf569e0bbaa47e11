// Text-format entry points with the upstream spelling.
#ifndef MCB200_PROTO_RUNTIME_TEXT_FORMAT_H_
#define MCB200_PROTO_RUNTIME_TEXT_FORMAT_H_

#include <string>

#include "google/protobuf/io/zero_copy_stream_impl.h"
#include "google/protobuf/message.h"

namespace google {
namespace protobuf {

class TextFormat {
 public:
  static bool ParseFromString(const std::string& input, Message* output);
  static bool Parse(io::ZeroCopyInputStream* input, Message* output);
  static bool PrintToString(const Message& message, std::string* output);
  static bool Print(const Message& message, io::ZeroCopyOutputStream* output);
  // Message of the last failed parse on this thread ("" if none).
  static const std::string& LastError();
};

}  // namespace protobuf
}  // namespace google

#endif  // MCB200_PROTO_RUNTIME_TEXT_FORMAT_H_
