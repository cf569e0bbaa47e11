// Implementation of the small protobuf-compatible runtime declared under
// google/protobuf/: varint wire codec, text-format tokenizer and printer, file
// streams.
#include <unistd.h>

#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <ostream>
#include <sstream>

#include "google/protobuf/io/coded_stream.h"
#include "google/protobuf/io/zero_copy_stream_impl.h"
#include "google/protobuf/message.h"
#include "google/protobuf/text_format.h"

namespace google {
namespace protobuf {

// ------------------------------------------------------------------ wire

namespace wire {

uint64 Reader::Varint() {
  uint64 v = 0;
  int shift = 0;
  while (p_ < end_ && shift < 70) {
    uint8 b = *p_++;
    if (shift < 64) v |= static_cast<uint64>(b & 0x7f) << shift;
    if (!(b & 0x80)) return v;
    shift += 7;
  }
  fail();
  return 0;
}

uint32 Reader::Fixed32() {
  if (remaining() < 4) { fail(); return 0; }
  uint32 v;
  std::memcpy(&v, p_, 4);  // little-endian hosts only
  p_ += 4;
  return v;
}

uint64 Reader::Fixed64() {
  if (remaining() < 8) { fail(); return 0; }
  uint64 v;
  std::memcpy(&v, p_, 8);
  p_ += 8;
  return v;
}

Reader Reader::Len() {
  uint64 n = Varint();
  if (!ok_ || n > remaining()) { fail(); return Reader(end_, 0); }
  Reader sub(p_, static_cast<std::size_t>(n));
  p_ += n;
  return sub;
}

std::string Reader::Bytes() {
  Reader sub = Len();
  return std::string(reinterpret_cast<const char*>(sub.pos()), sub.remaining());
}

bool Reader::Skip(int wire_type) {
  switch (wire_type) {
    case kVarint: Varint(); break;
    case kFixed64: Fixed64(); break;
    case kLen: Len(); break;
    case kFixed32: Fixed32(); break;
    case kStartGroup: {
      // Skip nested fields until the matching end-group tag.
      while (ok_ && !done()) {
        uint64 tag = Varint();
        int wt = static_cast<int>(tag & 7);
        if (wt == kEndGroup) return ok_;
        if (!Skip(wt)) return false;
      }
      fail();
      break;
    }
    default: fail();
  }
  return ok_;
}

void PutVarint(std::string* out, uint64 v) {
  while (v >= 0x80) {
    out->push_back(static_cast<char>((v & 0x7f) | 0x80));
    v >>= 7;
  }
  out->push_back(static_cast<char>(v));
}

void PutTag(std::string* out, int field, int wire_type) {
  PutVarint(out, (static_cast<uint64>(field) << 3) | static_cast<uint64>(wire_type));
}

void PutFixed32(std::string* out, uint32 v) { out->append(reinterpret_cast<const char*>(&v), 4); }
void PutFixed64(std::string* out, uint64 v) { out->append(reinterpret_cast<const char*>(&v), 8); }
void PutLen(std::string* out, const std::string& payload) {
  PutVarint(out, payload.size());
  out->append(payload);
}

}  // namespace wire

// ------------------------------------------------------------------ text

namespace text {

Parser::Parser(const char* data, std::size_t n) : p_(data), end_(data + n), line_(1) { Lex(); }

void Parser::Fail(const std::string& why) {
  if (err_.empty()) {
    std::ostringstream os;
    os << "line " << tok_.line << ": " << why;
    if (tok_.kind != Token::kEnd) os << " (at '" << tok_.text << "')";
    err_ = os.str();
  }
}

static bool IsIdentStart(char c) { return std::isalpha(static_cast<unsigned char>(c)) || c == '_'; }
static bool IsIdentChar(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.'; }

void Parser::Lex() {
  // Skip blanks and '#' comments.
  for (;;) {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\r' || *p_ == '\n' || *p_ == '\f' || *p_ == '\v')) {
      if (*p_ == '\n') ++line_;
      ++p_;
    }
    if (p_ < end_ && *p_ == '#') {
      while (p_ < end_ && *p_ != '\n') ++p_;
      continue;
    }
    break;
  }
  tok_.text.clear();
  tok_.line = line_;
  if (p_ >= end_) { tok_.kind = Token::kEnd; return; }
  char c = *p_;
  if (IsIdentStart(c)) {
    tok_.kind = Token::kIdent;
    while (p_ < end_ && IsIdentChar(*p_)) tok_.text.push_back(*p_++);
    return;
  }
  if (std::isdigit(static_cast<unsigned char>(c)) || c == '-' || c == '+' ||
      (c == '.' && p_ + 1 < end_ && std::isdigit(static_cast<unsigned char>(p_[1])))) {
    tok_.kind = Token::kNumber;
    tok_.text.push_back(*p_++);
    // "-" may be followed by blanks and then a number or identifier (-inf).
    if ((c == '-' || c == '+')) {
      while (p_ < end_ && (*p_ == ' ' || *p_ == '\t')) ++p_;
    }
    while (p_ < end_) {
      char d = *p_;
      bool exp_sign = (d == '-' || d == '+') && !tok_.text.empty() &&
                      (tok_.text.back() == 'e' || tok_.text.back() == 'E') &&
                      !(tok_.text.size() > 1 && (tok_.text[1] == 'x' || tok_.text[1] == 'X'));
      if (std::isalnum(static_cast<unsigned char>(d)) || d == '.' || exp_sign) {
        tok_.text.push_back(d);
        ++p_;
      } else {
        break;
      }
    }
    return;
  }
  if (c == '"' || c == '\'') {
    tok_.kind = Token::kString;
    char q = c;
    ++p_;
    while (p_ < end_ && *p_ != q) {
      char d = *p_++;
      if (d == '\n') { ++line_; }
      if (d != '\\' || p_ >= end_) { tok_.text.push_back(d); continue; }
      char e = *p_++;
      switch (e) {
        case 'n': tok_.text.push_back('\n'); break;
        case 't': tok_.text.push_back('\t'); break;
        case 'r': tok_.text.push_back('\r'); break;
        case 'a': tok_.text.push_back('\a'); break;
        case 'b': tok_.text.push_back('\b'); break;
        case 'f': tok_.text.push_back('\f'); break;
        case 'v': tok_.text.push_back('\v'); break;
        case 'x': case 'X': {
          int v = 0, nd = 0;
          while (p_ < end_ && nd < 2 && std::isxdigit(static_cast<unsigned char>(*p_))) {
            char h = *p_++;
            v = v * 16 + (std::isdigit(static_cast<unsigned char>(h)) ? h - '0' : (std::tolower(h) - 'a' + 10));
            ++nd;
          }
          tok_.text.push_back(static_cast<char>(v));
          break;
        }
        default:
          if (e >= '0' && e <= '7') {
            int v = e - '0', nd = 1;
            while (p_ < end_ && nd < 3 && *p_ >= '0' && *p_ <= '7') { v = v * 8 + (*p_++ - '0'); ++nd; }
            tok_.text.push_back(static_cast<char>(v));
          } else {
            tok_.text.push_back(e);  // \\ \' \" \? and anything else: literal
          }
      }
    }
    if (p_ >= end_) { tok_.kind = Token::kEnd; Fail("unterminated string"); return; }
    ++p_;  // closing quote
    return;
  }
  tok_.kind = Token::kSymbol;
  tok_.text.push_back(*p_++);
}

Token Parser::next() {
  Token t = tok_;
  if (tok_.kind != Token::kEnd) Lex();
  return t;
}

bool Parser::TryConsume(const char* symbol) {
  if (tok_.kind == Token::kSymbol && tok_.text == symbol) { Lex(); return true; }
  return false;
}

static bool ParseInteger(const std::string& s, bool allow_neg, uint64* mag, bool* neg) {
  std::size_t i = 0;
  *neg = false;
  if (i < s.size() && (s[i] == '-' || s[i] == '+')) { *neg = (s[i] == '-'); ++i; }
  if (*neg && !allow_neg) return false;
  if (i >= s.size()) return false;
  int base = 10;
  if (s.size() > i + 1 && s[i] == '0' && (s[i + 1] == 'x' || s[i + 1] == 'X')) { base = 16; i += 2; }
  else if (s.size() > i + 1 && s[i] == '0') { base = 8; }
  errno = 0;
  char* endp = nullptr;
  unsigned long long v = std::strtoull(s.c_str() + i, &endp, base);
  if (errno != 0 || endp == s.c_str() + i || *endp != '\0') return false;
  *mag = v;
  return true;
}

bool Parser::ReadInt64(int64* v) {
  if (tok_.kind != Token::kNumber) { Fail("expected integer"); return false; }
  uint64 mag; bool neg;
  if (!ParseInteger(tok_.text, true, &mag, &neg)) { Fail("bad integer"); return false; }
  *v = neg ? -static_cast<int64>(mag) : static_cast<int64>(mag);
  Lex();
  return true;
}

bool Parser::ReadUInt64(uint64* v) {
  if (tok_.kind != Token::kNumber) { Fail("expected unsigned integer"); return false; }
  uint64 mag; bool neg;
  if (!ParseInteger(tok_.text, false, &mag, &neg)) { Fail("bad unsigned integer"); return false; }
  *v = mag;
  Lex();
  return true;
}

bool Parser::ReadDouble(double* v) {
  if (tok_.kind == Token::kIdent) {
    std::string s = tok_.text;
    for (auto& ch : s) ch = static_cast<char>(std::tolower(ch));
    if (s == "inf" || s == "infinity") { *v = INFINITY; Lex(); return true; }
    if (s == "nan") { *v = NAN; Lex(); return true; }
    Fail("expected number");
    return false;
  }
  if (tok_.kind != Token::kNumber) { Fail("expected number"); return false; }
  std::string s = tok_.text;
  bool neg = false;
  std::size_t i = 0;
  if (!s.empty() && (s[0] == '-' || s[0] == '+')) { neg = s[0] == '-'; i = 1; }
  std::string body = s.substr(i);
  std::string low = body;
  for (auto& ch : low) ch = static_cast<char>(std::tolower(ch));
  double val;
  if (low == "inf" || low == "infinity") {
    val = INFINITY;
  } else if (low == "nan") {
    val = NAN;
  } else {
    if (!body.empty() && (body.back() == 'f' || body.back() == 'F') &&
        !(body.size() > 1 && (body[1] == 'x' || body[1] == 'X'))) {
      body.pop_back();  // "1.0f"
    }
    char* endp = nullptr;
    if (body.size() > 1 && body[0] == '0' && (body[1] == 'x' || body[1] == 'X')) {
      val = static_cast<double>(std::strtoull(body.c_str(), &endp, 16));
    } else {
      val = std::strtod(body.c_str(), &endp);
    }
    if (endp == body.c_str() || *endp != '\0') { Fail("bad number"); return false; }
  }
  *v = neg ? -val : val;
  Lex();
  return true;
}

bool Parser::ReadBool(bool* v) {
  if (tok_.kind == Token::kIdent) {
    const std::string& s = tok_.text;
    if (s == "true" || s == "True" || s == "t") { *v = true; Lex(); return true; }
    if (s == "false" || s == "False" || s == "f") { *v = false; Lex(); return true; }
  } else if (tok_.kind == Token::kNumber) {
    if (tok_.text == "1") { *v = true; Lex(); return true; }
    if (tok_.text == "0") { *v = false; Lex(); return true; }
  }
  Fail("expected boolean");
  return false;
}

bool Parser::ReadString(std::string* v) {
  if (tok_.kind != Token::kString) { Fail("expected string"); return false; }
  v->clear();
  while (tok_.kind == Token::kString) {  // adjacent literals concatenate
    v->append(tok_.text);
    Lex();
  }
  return ok();
}

bool Parser::ReadIdentOrInt(std::string* ident, int64* num, bool* is_ident) {
  if (tok_.kind == Token::kIdent) {
    *ident = tok_.text;
    *is_ident = true;
    Lex();
    return true;
  }
  *is_ident = false;
  return ReadInt64(num);
}

void Printer::Field(const char* name, const std::string& rendered) {
  out_.append(static_cast<std::size_t>(indent_) * 2, ' ');
  out_.append(name);
  out_.append(": ");
  out_.append(rendered);
  out_.push_back('\n');
}

void Printer::Open(const char* name) {
  out_.append(static_cast<std::size_t>(indent_) * 2, ' ');
  out_.append(name);
  out_.append(" {\n");
  ++indent_;
}

void Printer::Close() {
  --indent_;
  out_.append(static_cast<std::size_t>(indent_) * 2, ' ');
  out_.append("}\n");
}

std::string Printer::Quote(const std::string& s) {
  std::string r = "\"";
  for (unsigned char c : s) {
    switch (c) {
      case '\n': r += "\\n"; break;
      case '\r': r += "\\r"; break;
      case '\t': r += "\\t"; break;
      case '"': r += "\\\""; break;
      case '\'': r += "\\'"; break;
      case '\\': r += "\\\\"; break;
      default:
        if (c < 0x20 || c >= 0x7f) {
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\%03o", c);
          r += buf;
        } else {
          r.push_back(static_cast<char>(c));
        }
    }
  }
  r.push_back('"');
  return r;
}

static std::string RenderFloating(double v, int short_digits, int long_digits, bool is_float) {
  if (std::isnan(v)) return "nan";
  if (std::isinf(v)) return v > 0 ? "inf" : "-inf";
  char buf[40];
  std::snprintf(buf, sizeof(buf), "%.*g", short_digits, v);
  bool same = is_float ? (std::strtof(buf, nullptr) == static_cast<float>(v)) : (std::strtod(buf, nullptr) == v);
  if (!same) std::snprintf(buf, sizeof(buf), "%.*g", long_digits, v);
  return buf;
}

std::string Printer::Num(double v) { return RenderFloating(v, 15, 17, false); }
std::string Printer::Num(float v) { return RenderFloating(v, 6, 9, true); }

}  // namespace text

// ------------------------------------------------------------------ Message

bool Message::ParseFromArray(const void* data, int size) {
  Clear();
  wire::Reader r(static_cast<const uint8*>(data), static_cast<std::size_t>(size));
  return MergeFromWire(&r) && r.ok();
}

bool Message::ParseFromCodedStream(io::CodedInputStream* in) {
  Clear();
  wire::Reader r(in->data(), in->size());
  return MergeFromWire(&r) && r.ok();
}

bool Message::SerializeToOstream(std::ostream* out) const {
  std::string s;
  AppendToWire(&s);
  out->write(s.data(), static_cast<std::streamsize>(s.size()));
  return out->good();
}

std::string Message::DebugString() const {
  text::Printer p;
  PrintText(&p);
  return p.str();
}

bool Message::ParseTextBody(text::Parser* in, const char* closer) {
  for (;;) {
    if (!in->ok()) return false;
    const text::Token& t = in->peek();
    if (t.kind == text::Token::kEnd) {
      if (closer) { in->Fail(std::string("missing '") + closer + "'"); return false; }
      return true;
    }
    if (closer && t.kind == text::Token::kSymbol && t.text == closer) {
      in->next();
      return true;
    }
    if (t.kind != text::Token::kIdent) { in->Fail("expected field name"); return false; }
    std::string name = in->next().text;
    if (!ParseTextField(name, in)) {
      in->Fail("in " + std::string(GetTypeName()) + ": cannot set field '" + name + "'");
      return false;
    }
    // Optional separators between fields.
    if (!in->TryConsume(",")) in->TryConsume(";");
  }
}

// ------------------------------------------------------------------ streams

namespace io {

const std::string& FileInputStream::ReadAll() {
  if (!drained_) {
    drained_ = true;
    char chunk[1 << 16];
    for (;;) {
      ssize_t n = ::read(fd_, chunk, sizeof(chunk));
      if (n < 0 && errno == EINTR) continue;
      if (n <= 0) break;
      buf_.append(chunk, static_cast<std::size_t>(n));
    }
  }
  return buf_;
}

bool FileOutputStream::WriteAll(const std::string& data) {
  std::size_t off = 0;
  while (off < data.size()) {
    ssize_t n = ::write(fd_, data.data() + off, data.size() - off);
    if (n < 0 && errno == EINTR) continue;
    if (n <= 0) return false;
    off += static_cast<std::size_t>(n);
  }
  return true;
}

}  // namespace io

// ------------------------------------------------------------------ TextFormat

static std::string& TextError() {
  static thread_local std::string err;
  return err;
}

const std::string& TextFormat::LastError() { return TextError(); }

bool TextFormat::ParseFromString(const std::string& input, Message* output) {
  output->Clear();
  text::Parser p(input.data(), input.size());
  bool ok = output->ParseTextBody(&p, nullptr) && p.ok();
  TextError() = ok ? std::string() : p.error();
  if (!ok) std::fprintf(stderr, "[text-format] %s: %s\n", output->GetTypeName(), p.error().c_str());
  return ok;
}

bool TextFormat::Parse(io::ZeroCopyInputStream* input, Message* output) {
  return ParseFromString(input->ReadAll(), output);
}

bool TextFormat::PrintToString(const Message& message, std::string* output) {
  *output = message.DebugString();
  return true;
}

bool TextFormat::Print(const Message& message, io::ZeroCopyOutputStream* output) {
  return output->WriteAll(message.DebugString());
}

}  // namespace protobuf
}  // namespace google
