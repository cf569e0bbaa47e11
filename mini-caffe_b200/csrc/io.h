// Model-file readers and writers (prototxt text format, caffemodel wire
// format) and the upgrade of legacy net definitions.  Counterpart of
// mini-caffe's src/util/io.{hpp,cpp} and src/util/upgrade_proto.{hpp,cpp}.
#ifndef MCB200_IO_H_
#define MCB200_IO_H_

#include <string>

#include "caffe.pb.h"
#include "caffe/base.hpp"
#include "google/protobuf/message.h"

namespace caffe {

using ::google::protobuf::Message;

// A missing file is a CHECK failure ("File not found: ..."); a file that does
// not parse returns false.
bool ReadProtoFromTextFile(const char* filename, Message* proto);
bool ReadProtoFromBinaryFile(const char* filename, Message* proto);
void ReadProtoFromBinaryFileOrDie(const char* filename, Message* proto);
void WriteProtoToTextFile(const Message& proto, const char* filename);
void WriteProtoToBinaryFile(const Message& proto, const char* filename);

// Rewrites deprecated constructs in place:
//  * top-level `input:` / `input_shape` / `input_dim` become an "Input" layer
//    placed first (src/util/upgrade_proto.cpp:271-306);
//  * V1 `layers { type: CONVOLUTION }` entries become `layer { type: "Convolution" }`
//    entries (src/util/upgrade_proto.cpp:18-44, 61-262); a definition with both
//    kinds is refused.
bool UpgradeNetAsNeeded(const string& source, NetParameter* param);
void ReadNetParamsFromTextFileOrDie(const string& file, NetParameter* param);
void ReadNetParamsFromBinaryFileOrDie(const string& file, NetParameter* param);

}  // namespace caffe

#endif  // MCB200_IO_H_
