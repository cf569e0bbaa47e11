#!/usr/bin/env python3
"""Generate C++ message classes (caffe.pb.h / caffe.pb.cc) from caffe_schema.def.

The image this library is built in has no protoc and no libprotobuf, so the
model-file classes are produced by this script instead.  The emitted classes
expose the accessor spelling protoc would give a proto2 file (x(), has_x(),
set_x(), x_size(), add_x(), mutable_x(), clear_x(), Message_Enum_VALUE ...),
and derive from the small runtime in runtime/google/protobuf/message.h, which
supplies wire-format and text-format parsing.

usage: protogen.py <schema.def> <out_dir>
"""
import os
import sys

SCALARS = {
    # type: (c++ type, wire kind)
    "int32": ("::google::protobuf::int32", "varint"),
    "int64": ("::google::protobuf::int64", "varint"),
    "uint32": ("::google::protobuf::uint32", "varint"),
    "uint64": ("::google::protobuf::uint64", "varint"),
    "bool": ("bool", "varint"),
    "float": ("float", "fixed32"),
    "double": ("double", "fixed64"),
    "string": ("::std::string", "len"),
    "bytes": ("::std::string", "len"),
}


class Enum:
    def __init__(self, name, values, owner=None):
        self.name, self.values, self.owner = name, values, owner

    @property
    def cpp(self):
        return f"{self.owner}_{self.name}" if self.owner else self.name

    def const(self, value_name):
        return f"{self.owner}_{self.name}_{value_name}" if self.owner else value_name


class Field:
    def __init__(self, label, ftype, name, number, packed, default):
        self.label, self.ftype, self.name = label, ftype, name
        self.number, self.packed, self.default = number, packed, default
        self.kind = None  # scalar | enum | message
        self.enum = None


class Message:
    def __init__(self, name):
        self.name, self.fields, self.enums = name, [], []


def parse_schema(path):
    messages, enums = [], []
    cur = None
    for raw in open(path):
        line = raw.split("#", 1)[0].rstrip() if not raw.lstrip().startswith("#") else ""
        if not line.strip():
            continue
        indented = line[0] in " \t"
        toks = line.split()
        if toks[0] == "message":
            cur = Message(toks[1])
            messages.append(cur)
        elif toks[0] == "enum":
            vals = [(t.split("=")[0], int(t.split("=")[1])) for t in toks[2:]]
            if indented:
                cur.enums.append(Enum(toks[1], vals, cur.name))
            else:
                enums.append(Enum(toks[1], vals))
        elif toks[0] in ("opt", "rep"):
            label, ftype, name, number = toks[0], toks[1], toks[2], int(toks[3])
            rest = toks[4:]
            packed = "packed" in rest
            default = None
            if "=" in rest:
                default = line.split("=", 1)[1].strip()
            cur.fields.append(Field(label, ftype, name, number, packed, default))
        else:
            raise SystemExit(f"bad schema line: {raw!r}")
    msg_names = {m.name for m in messages}
    top_enums = {e.name: e for e in enums}
    for m in messages:
        local = {e.name: e for e in m.enums}
        for f in m.fields:
            if f.ftype in SCALARS:
                f.kind = "scalar"
            elif f.ftype in local:
                f.kind, f.enum = "enum", local[f.ftype]
            elif f.ftype in top_enums:
                f.kind, f.enum = "enum", top_enums[f.ftype]
            elif f.ftype in msg_names:
                f.kind = "message"
            elif "." in f.ftype and f.ftype.split(".")[0] in msg_names:
                owner, ename = f.ftype.split(".")
                scoped = {e.name: e for mm in messages if mm.name == owner for e in mm.enums}
                if ename not in scoped:
                    raise SystemExit(f"{m.name}.{f.name}: unknown type {f.ftype}")
                f.kind, f.enum = "enum", scoped[ename]
            else:
                raise SystemExit(f"{m.name}.{f.name}: unknown type {f.ftype}")
    return messages, enums


def cpp_type(f):
    if f.kind == "scalar":
        return SCALARS[f.ftype][0]
    if f.kind == "enum":
        return f.enum.cpp
    return f.ftype


def default_expr(f):
    if f.kind == "message":
        return None
    if f.kind == "enum":
        return f.enum.const(f.default) if f.default is not None else f.enum.const(f.enum.values[0][0])
    t = f.ftype
    if t in ("string", "bytes"):
        return f.default if f.default is not None else '""'
    if f.default is None:
        return "false" if t == "bool" else "0"
    d = f.default
    if t == "float":
        low = d.lower()
        if low in ("inf", "-inf", "nan"):
            return {"inf": "INFINITY", "-inf": "-INFINITY", "nan": "NAN"}[low]
        if not any(c in d for c in ".eE"):
            d += ".0"
        return d + "f"
    if t == "double":
        if not any(c in d for c in ".eE"):
            d += ".0"
        return d
    if t in ("uint32", "uint64"):
        return d + "u"
    if t == "int64":
        return f"static_cast<::google::protobuf::int64>({d}LL)"
    return d


def gen_header(messages, enums, guard="MCB200_CAFFE_PB_H_"):
    o = []
    w = o.append
    w("// Generated by protogen.py from caffe_schema.def -- do not edit.")
    w(f"#ifndef {guard}\n#define {guard}\n")
    w("#include <string>\n\n#include \"google/protobuf/message.h\"\n")
    w("namespace caffe {\n")
    for m in messages:
        w(f"class {m.name};")
    w("")

    def emit_enum(e):
        w(f"enum {e.cpp} {{")
        for n, v in e.values:
            w(f"  {e.const(n)} = {v},")
        w("};")
        w(f"const char* {e.cpp}_Name(int value);")
        w(f"bool {e.cpp}_Parse(const ::std::string& name, {e.cpp}* value);")
        w(f"bool {e.cpp}_IsValid(int value);\n")

    for e in enums:
        emit_enum(e)
    for m in messages:
        for e in m.enums:
            emit_enum(e)

    for m in messages:
        w(f"class {m.name} : public ::google::protobuf::Message {{")
        w(" public:")
        w(f"  {m.name}();")
        w(f"  static const {m.name}& default_instance();")
        w(f"  const char* GetTypeName() const override {{ return \"caffe.{m.name}\"; }}")
        w("  void Clear() override;")
        w("  bool MergeFromWire(::google::protobuf::wire::Reader* in) override;")
        w("  void AppendToWire(::std::string* out) const override;")
        w("  bool ParseTextField(const ::std::string& name, ::google::protobuf::text::Parser* in) override;")
        w("  void PrintText(::google::protobuf::text::Printer* out) const override;")
        w(f"  void CopyFrom(const {m.name}& other) {{ if (this != &other) *this = other; }}")
        w(f"  void Swap({m.name}* other) {{ {m.name} tmp(*other); *other = *this; *this = tmp; }}")
        for e in m.enums:
            w(f"  typedef {e.cpp} {e.name};")
            for n, _ in e.values:
                w(f"  static const {e.name} {n} = {e.const(n)};")
            w(f"  static const char* {e.name}_Name(int v) {{ return {e.cpp}_Name(v); }}")
        for f in m.fields:
            n, T = f.name, cpp_type(f)
            w(f"  // {f.label} {f.ftype} {n} = {f.number}")
            if f.label == "opt":
                if f.kind == "message":
                    w(f"  bool has_{n}() const {{ return {n}_.get() != nullptr; }}")
                    w(f"  const {T}& {n}() const;")
                    w(f"  {T}* mutable_{n}();")
                    w(f"  void clear_{n}() {{ {n}_.reset(); }}")
                else:
                    w(f"  bool has_{n}() const {{ return has_{n}_; }}")
                    if f.ftype in ("string", "bytes"):
                        w(f"  const ::std::string& {n}() const {{ return {n}_; }}")
                        w(f"  void set_{n}(const ::std::string& v) {{ {n}_ = v; has_{n}_ = true; }}")
                        w(f"  void set_{n}(const char* v) {{ {n}_ = v; has_{n}_ = true; }}")
                        w(f"  ::std::string* mutable_{n}() {{ has_{n}_ = true; return &{n}_; }}")
                    else:
                        w(f"  {T} {n}() const {{ return {n}_; }}")
                        w(f"  void set_{n}({T} v) {{ {n}_ = v; has_{n}_ = true; }}")
                    w(f"  void clear_{n}() {{ {n}_ = {default_expr(f)}; has_{n}_ = false; }}")
            else:
                w(f"  int {n}_size() const {{ return {n}_.size(); }}")
                w(f"  void clear_{n}() {{ {n}_.Clear(); }}")
                if f.kind == "message":
                    w(f"  const {T}& {n}(int i) const;")
                    w(f"  {T}* mutable_{n}(int i);")
                    w(f"  {T}* add_{n}();")
                    w(f"  const ::google::protobuf::RepeatedPtrField<{T}>& {n}() const {{ return {n}_; }}")
                    w(f"  ::google::protobuf::RepeatedPtrField<{T}>* mutable_{n}() {{ return &{n}_; }}")
                else:
                    if f.ftype in ("string", "bytes"):
                        w(f"  const ::std::string& {n}(int i) const {{ return {n}_.Get(i); }}")
                        w(f"  void set_{n}(int i, const ::std::string& v) {{ {n}_.Set(i, v); }}")
                        w(f"  void add_{n}(const ::std::string& v) {{ {n}_.Add(v); }}")
                        w(f"  ::std::string* add_{n}() {{ {n}_.Add(::std::string()); return {n}_.Mutable({n}_.size() - 1); }}")
                        w(f"  ::std::string* mutable_{n}(int i) {{ return {n}_.Mutable(i); }}")
                    else:
                        w(f"  {T} {n}(int i) const {{ return {n}_.Get(i); }}")
                        w(f"  void set_{n}(int i, {T} v) {{ {n}_.Set(i, v); }}")
                        w(f"  void add_{n}({T} v) {{ {n}_.Add(v); }}")
                    w(f"  const ::google::protobuf::RepeatedField<{T}>& {n}() const {{ return {n}_; }}")
                    w(f"  ::google::protobuf::RepeatedField<{T}>* mutable_{n}() {{ return &{n}_; }}")
        w(" private:")
        for f in m.fields:
            n, T = f.name, cpp_type(f)
            if f.label == "opt":
                if f.kind == "message":
                    w(f"  ::google::protobuf::MsgHolder<{T}> {n}_;")
                else:
                    w(f"  {T} {n}_;")
                    w(f"  bool has_{n}_;")
            elif f.kind == "message":
                w(f"  ::google::protobuf::RepeatedPtrField<{T}> {n}_;")
            else:
                w(f"  ::google::protobuf::RepeatedField<{T}> {n}_;")
        w("};\n")
    w("}  // namespace caffe\n")
    w(f"#endif  // {guard}")
    return "\n".join(o) + "\n"


def wire_read_scalar(f, src="in"):
    """C++ expression decoding one scalar of field f from reader `src`."""
    t = f.ftype
    if f.kind == "enum":
        return f"static_cast<{f.enum.cpp}>(static_cast<int>({src}->Varint()))"
    if t == "float":
        return f"::google::protobuf::wire::BitsFloat({src}->Fixed32())"
    if t == "double":
        return f"::google::protobuf::wire::BitsDouble({src}->Fixed64())"
    if t == "bool":
        return f"({src}->Varint() != 0)"
    return f"static_cast<{SCALARS[t][0]}>({src}->Varint())"


def wire_kind(f):
    if f.kind == "enum":
        return "varint"
    if f.kind == "message":
        return "len"
    return SCALARS[f.ftype][1]


WT = {"varint": 0, "fixed64": 1, "len": 2, "fixed32": 5}


def wire_put_scalar(f, val, out="out"):
    t = f.ftype
    if f.kind == "enum":
        return f"::google::protobuf::wire::PutVarint({out}, static_cast<::google::protobuf::uint64>(static_cast<::google::protobuf::int64>({val})));"
    if t == "float":
        return f"::google::protobuf::wire::PutFixed32({out}, ::google::protobuf::wire::FloatBits({val}));"
    if t == "double":
        return f"::google::protobuf::wire::PutFixed64({out}, ::google::protobuf::wire::DoubleBits({val}));"
    if t == "bool":
        return f"::google::protobuf::wire::PutVarint({out}, {val} ? 1 : 0);"
    if t in ("int32", "int64"):
        return f"::google::protobuf::wire::PutVarint({out}, static_cast<::google::protobuf::uint64>(static_cast<::google::protobuf::int64>({val})));"
    return f"::google::protobuf::wire::PutVarint({out}, static_cast<::google::protobuf::uint64>({val}));"


def text_read_scalar(f, target):
    """C++ statements reading one text value into lvalue `target`; uses `in`."""
    t = f.ftype
    if f.kind == "enum":
        e = f.enum.cpp
        return (f"{{ ::std::string id; ::google::protobuf::int64 num = 0; bool is_id = false; "
                f"if (!in->ReadIdentOrInt(&id, &num, &is_id)) return false; {e} ev; "
                f"if (is_id) {{ if (!{e}_Parse(id, &ev)) return false; }} "
                f"else {{ if (!{e}_IsValid(static_cast<int>(num))) return false; ev = static_cast<{e}>(num); }} "
                f"{target} = ev; }}")
    if t in ("string", "bytes"):
        return f"{{ if (!in->ReadString(&{target})) return false; }}"
    if t == "bool":
        return f"{{ bool b; if (!in->ReadBool(&b)) return false; {target} = b; }}"
    if t in ("float", "double"):
        return f"{{ double d; if (!in->ReadDouble(&d)) return false; {target} = static_cast<{SCALARS[t][0]}>(d); }}"
    if t in ("uint32", "uint64"):
        return f"{{ ::google::protobuf::uint64 u; if (!in->ReadUInt64(&u)) return false; {target} = static_cast<{SCALARS[t][0]}>(u); }}"
    return f"{{ ::google::protobuf::int64 s; if (!in->ReadInt64(&s)) return false; {target} = static_cast<{SCALARS[t][0]}>(s); }}"


def text_render(f, val):
    t = f.ftype
    if f.kind == "enum":
        return f"::std::string({f.enum.cpp}_Name({val}))"
    if t in ("string", "bytes"):
        return f"::google::protobuf::text::Printer::Quote({val})"
    if t == "bool":
        return f"::std::string({val} ? \"true\" : \"false\")"
    if t in ("float", "double"):
        return f"::google::protobuf::text::Printer::Num({val})"
    return f"::std::to_string({val})"


def gen_source(messages, enums):
    o = []
    w = o.append
    w("// Generated by protogen.py from caffe_schema.def -- do not edit.")
    w("#include \"caffe.pb.h\"\n\n#include <cmath>\n#include <string>\n")
    w("namespace caffe {\n")

    def emit_enum(e):
        w(f"const char* {e.cpp}_Name(int value) {{\n  switch (value) {{")
        seen = set()
        for n, v in e.values:
            if v in seen:
                continue
            seen.add(v)
            w(f"    case {v}: return \"{n}\";")
        w("    default: return \"\";\n  }\n}")
        w(f"bool {e.cpp}_Parse(const ::std::string& name, {e.cpp}* value) {{")
        for n, v in e.values:
            w(f"  if (name == \"{n}\") {{ *value = {e.const(n)}; return true; }}")
        w("  return false;\n}")
        w(f"bool {e.cpp}_IsValid(int value) {{ return {e.cpp}_Name(value)[0] != '\\0'; }}\n")

    for e in enums:
        emit_enum(e)
    for m in messages:
        for e in m.enums:
            emit_enum(e)

    for m in messages:
        M = m.name
        inits = []
        for f in m.fields:
            if f.label == "opt" and f.kind != "message":
                inits.append(f"{f.name}_({default_expr(f)})")
                inits.append(f"has_{f.name}_(false)")
        w(f"{M}::{M}()" + ((" : " + ", ".join(inits)) if inits else "") + " {}")
        w(f"const {M}& {M}::default_instance() {{ static const {M} inst; return inst; }}")
        for f in m.fields:
            n, T = f.name, cpp_type(f)
            if f.kind != "message":
                continue
            if f.label == "opt":
                w(f"const {T}& {M}::{n}() const {{ return {n}_.get() ? *{n}_.get() : {T}::default_instance(); }}")
                w(f"{T}* {M}::mutable_{n}() {{ return {n}_.mut(); }}")
            else:
                w(f"const {T}& {M}::{n}(int i) const {{ return {n}_.Get(i); }}")
                w(f"{T}* {M}::mutable_{n}(int i) {{ return {n}_.Mutable(i); }}")
                w(f"{T}* {M}::add_{n}() {{ return {n}_.Add(); }}")
        # Clear
        w(f"void {M}::Clear() {{")
        for f in m.fields:
            w(f"  clear_{f.name}();")
        w("}")
        # MergeFromWire
        w(f"bool {M}::MergeFromWire(::google::protobuf::wire::Reader* in) {{")
        w("  while (in->ok() && !in->done()) {")
        w("    ::google::protobuf::uint64 tag = in->Varint();")
        w("    if (!in->ok()) return false;")
        w("    const int field = static_cast<int>(tag >> 3);")
        w("    const int wt = static_cast<int>(tag & 7);")
        w("    switch (field) {")
        for f in m.fields:
            n = f.name
            w(f"      case {f.number}: {{")
            if f.kind == "message":
                w("        if (wt != 2) { if (!in->Skip(wt)) return false; break; }")
                w("        ::google::protobuf::wire::Reader sub = in->Len();")
                w("        if (!in->ok()) return false;")
                target = f"mutable_{n}()" if f.label == "opt" else f"add_{n}()"
                w(f"        if (!{target}->MergeFromWire(&sub) || !sub.ok()) return false;")
            elif f.kind == "scalar" and f.ftype in ("string", "bytes"):
                w("        if (wt != 2) { if (!in->Skip(wt)) return false; break; }")
                if f.label == "opt":
                    w(f"        set_{n}(in->Bytes());")
                else:
                    w(f"        add_{n}(in->Bytes());")
            else:
                k = WT[wire_kind(f)]
                if f.label == "opt":
                    w(f"        if (wt != {k}) {{ if (!in->Skip(wt)) return false; break; }}")
                    w(f"        set_{n}({wire_read_scalar(f)});")
                else:
                    w("        if (wt == 2) {  // packed")
                    w("          ::google::protobuf::wire::Reader sub = in->Len();")
                    w("          if (!in->ok()) return false;")
                    if f.ftype == "float":
                        w(f"          {n}_.Reserve({n}_.size() + static_cast<int>(sub.remaining() / 4));")
                    w(f"          while (sub.ok() && !sub.done()) {n}_.Add({wire_read_scalar(f, '(&sub)')});")
                    w("          if (!sub.ok()) return false;")
                    w(f"        }} else if (wt == {k}) {{")
                    w(f"          {n}_.Add({wire_read_scalar(f)});")
                    w("        } else if (!in->Skip(wt)) {")
                    w("          return false;")
                    w("        }")
            w("        break;\n      }")
        w("      default:\n        if (!in->Skip(wt)) return false;")
        w("    }\n  }\n  return in->ok();\n}")
        # AppendToWire
        w(f"void {M}::AppendToWire(::std::string* out) const {{")
        for f in sorted(m.fields, key=lambda x: x.number):
            n = f.name
            if f.kind == "message":
                if f.label == "opt":
                    w(f"  if (has_{n}()) {{ ::std::string sub; {n}().AppendToWire(&sub); "
                      f"::google::protobuf::wire::PutTag(out, {f.number}, 2); ::google::protobuf::wire::PutLen(out, sub); }}")
                else:
                    w(f"  for (int i = 0; i < {n}_size(); ++i) {{ ::std::string sub; {n}(i).AppendToWire(&sub); "
                      f"::google::protobuf::wire::PutTag(out, {f.number}, 2); ::google::protobuf::wire::PutLen(out, sub); }}")
            elif f.kind == "scalar" and f.ftype in ("string", "bytes"):
                if f.label == "opt":
                    w(f"  if (has_{n}()) {{ ::google::protobuf::wire::PutTag(out, {f.number}, 2); ::google::protobuf::wire::PutLen(out, {n}_); }}")
                else:
                    w(f"  for (int i = 0; i < {n}_size(); ++i) {{ ::google::protobuf::wire::PutTag(out, {f.number}, 2); ::google::protobuf::wire::PutLen(out, {n}_.Get(i)); }}")
            else:
                k = WT[wire_kind(f)]
                if f.label == "opt":
                    w(f"  if (has_{n}()) {{ ::google::protobuf::wire::PutTag(out, {f.number}, {k}); {wire_put_scalar(f, n + '_')} }}")
                elif f.packed:
                    w(f"  if ({n}_size() > 0) {{ ::std::string sub; for (int i = 0; i < {n}_size(); ++i) {{ {wire_put_scalar(f, n + '_.Get(i)', '(&sub)')} }} "
                      f"::google::protobuf::wire::PutTag(out, {f.number}, 2); ::google::protobuf::wire::PutLen(out, sub); }}")
                else:
                    w(f"  for (int i = 0; i < {n}_size(); ++i) {{ ::google::protobuf::wire::PutTag(out, {f.number}, {k}); {wire_put_scalar(f, n + '_.Get(i)')} }}")
        w("}")
        # ParseTextField
        w(f"bool {M}::ParseTextField(const ::std::string& name, ::google::protobuf::text::Parser* in) {{")
        for f in m.fields:
            n, T = f.name, cpp_type(f)
            w(f"  if (name == \"{n}\") {{")
            if f.kind == "message":
                target = f"mutable_{n}()" if f.label == "opt" else f"add_{n}()"
                w("    in->TryConsume(\":\");")
                if f.label == "rep":
                    # `field: [ {..}, {..} ]` list form
                    w("    if (in->TryConsume(\"[\")) {")
                    w("      if (in->TryConsume(\"]\")) return true;")
                    w("      do {")
                    w("        const char* c = nullptr;")
                    w("        if (in->TryConsume(\"{\")) c = \"}\"; else if (in->TryConsume(\"<\")) c = \">\"; else return false;")
                    w(f"        if (!add_{n}()->ParseTextBody(in, c)) return false;")
                    w("      } while (in->TryConsume(\",\"));")
                    w("      return in->TryConsume(\"]\");")
                    w("    }")
                w("    const char* closer = nullptr;")
                w("    if (in->TryConsume(\"{\")) closer = \"}\"; else if (in->TryConsume(\"<\")) closer = \">\"; else return false;")
                w(f"    return {target}->ParseTextBody(in, closer);")
            else:
                w("    if (!in->TryConsume(\":\")) return false;")
                if f.label == "opt":
                    w(f"    {T} v = {default_expr(f)};")
                    w(f"    {text_read_scalar(f, 'v')}")
                    w(f"    set_{n}(v);")
                    w("    return true;")
                else:
                    w("    if (in->TryConsume(\"[\")) {")
                    w("      if (in->TryConsume(\"]\")) return true;")
                    w("      do {")
                    w(f"        {T} v = {default_expr(f)};")
                    w(f"        {text_read_scalar(f, 'v')}")
                    w(f"        {n}_.Add(v);")
                    w("      } while (in->TryConsume(\",\"));")
                    w("      return in->TryConsume(\"]\");")
                    w("    }")
                    w(f"    {T} v = {default_expr(f)};")
                    w(f"    {text_read_scalar(f, 'v')}")
                    w(f"    {n}_.Add(v);")
                    w("    return true;")
            w("  }")
        w("  return false;\n}")
        # PrintText
        w(f"void {M}::PrintText(::google::protobuf::text::Printer* out) const {{")
        for f in sorted(m.fields, key=lambda x: x.number):
            n = f.name
            if f.kind == "message":
                if f.label == "opt":
                    w(f"  if (has_{n}()) {{ out->Open(\"{n}\"); {n}().PrintText(out); out->Close(); }}")
                else:
                    w(f"  for (int i = 0; i < {n}_size(); ++i) {{ out->Open(\"{n}\"); {n}(i).PrintText(out); out->Close(); }}")
            elif f.label == "opt":
                w(f"  if (has_{n}()) out->Field(\"{n}\", {text_render(f, n + '_')});")
            else:
                w(f"  for (int i = 0; i < {n}_size(); ++i) out->Field(\"{n}\", {text_render(f, n + '_.Get(i)')});")
        w("}\n")
    w("}  // namespace caffe")
    return "\n".join(o) + "\n"


def write_if_changed(path, text):
    if os.path.exists(path) and open(path).read() == text:
        return
    with open(path, "w") as fh:
        fh.write(text)


def main(argv):
    if len(argv) != 3:
        raise SystemExit(__doc__)
    messages, enums = parse_schema(argv[1])
    os.makedirs(argv[2], exist_ok=True)
    write_if_changed(os.path.join(argv[2], "caffe.pb.h"), gen_header(messages, enums))
    write_if_changed(os.path.join(argv[2], "caffe.pb.cc"), gen_source(messages, enums))


if __name__ == "__main__":
    main(sys.argv)
