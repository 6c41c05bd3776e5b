// Zero-copy FlatBuffers access primitives and a bounds-checking verifier.
//
// The TTNN binary is a size-prefixed FlatBuffer with file identifier "TTNN"
// (reference: include/ttmlir/Target/TTNN/binary.fbs:8-19, read there through
// flatc-generated code in runtime/lib/binary.cpp:126-131).  No flatbuffers library
// or flatc exists on the build machine, so the few primitives the format needs are
// written here from the published wire-format description:
//   table   : i32 soffset to vtable at the table start; vtable = {u16 vtable bytes,
//             u16 table bytes, u16 field offset per field id (0 = absent)}
//   offsets : u32, relative to the position of the offset itself, always forward
//   vector  : u32 count then elements; string : u32 length, bytes, NUL
//   union   : u8 type in slot i, offset to the member table in slot i+1
// All accessors assume a buffer that passed `Verifier`; loading verifies first.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <optional>
#include <string>
#include <string_view>
#include <type_traits>

namespace fb {

template <typename T>
inline T readScalar(const void *p) {
  T v;
  std::memcpy(&v, p, sizeof(T));
  return v;
}

struct String {
  uint32_t size() const { return readScalar<uint32_t>(this); }
  const char *c_str() const { return reinterpret_cast<const char *>(this) + 4; }
  std::string str() const { return std::string(c_str(), size()); }
  std::string_view view() const { return std::string_view(c_str(), size()); }
};

// Element access for vectors of scalars / structs (T stored inline).
template <typename T>
struct Vector {
  uint32_t size() const { return readScalar<uint32_t>(this); }
  const uint8_t *data() const { return reinterpret_cast<const uint8_t *>(this) + 4; }
  T Get(uint32_t i) const { return readScalar<T>(data() + sizeof(T) * i); }
  T operator[](uint32_t i) const { return Get(i); }
  struct It {
    const Vector *v;
    uint32_t i;
    T operator*() const { return v->Get(i); }
    It &operator++() { ++i; return *this; }
    bool operator!=(const It &o) const { return i != o.i; }
  };
  It begin() const { return {this, 0}; }
  It end() const { return {this, size()}; }
};

// Vectors of tables / strings store u32 offsets; Get follows the offset.
template <typename T>
struct OffsetVector {
  uint32_t size() const { return readScalar<uint32_t>(this); }
  const T *Get(uint32_t i) const {
    const uint8_t *p = reinterpret_cast<const uint8_t *>(this) + 4 + 4 * i;
    return reinterpret_cast<const T *>(p + readScalar<uint32_t>(p));
  }
  const T *operator[](uint32_t i) const { return Get(i); }
  struct It {
    const OffsetVector *v;
    uint32_t i;
    const T *operator*() const { return v->Get(i); }
    It &operator++() { ++i; return *this; }
    bool operator!=(const It &o) const { return i != o.i; }
  };
  It begin() const { return {this, 0}; }
  It end() const { return {this, size()}; }
};

struct Table {
  const uint8_t *self() const { return reinterpret_cast<const uint8_t *>(this); }
  const uint8_t *vtable() const { return self() - readScalar<int32_t>(self()); }
  // Byte offset of field `id` inside the table, 0 when absent.
  uint16_t fieldOffset(uint32_t id) const {
    const uint8_t *vt = vtable();
    uint32_t at = 4 + 2 * id;
    if (at >= readScalar<uint16_t>(vt)) {
      return 0;
    }
    return readScalar<uint16_t>(vt + at);
  }
  bool has(uint32_t id) const { return fieldOffset(id) != 0; }
  template <typename T>
  T scalar(uint32_t id, T dflt) const {
    uint16_t off = fieldOffset(id);
    return off ? readScalar<T>(self() + off) : dflt;
  }
  template <typename T>
  std::optional<T> optScalar(uint32_t id) const {
    uint16_t off = fieldOffset(id);
    if (!off) {
      return std::nullopt;
    }
    return readScalar<T>(self() + off);
  }
  template <typename T>
  const T *structPtr(uint32_t id) const {
    uint16_t off = fieldOffset(id);
    return off ? reinterpret_cast<const T *>(self() + off) : nullptr;
  }
  template <typename T>
  const T *child(uint32_t id) const {
    uint16_t off = fieldOffset(id);
    if (!off) {
      return nullptr;
    }
    const uint8_t *p = self() + off;
    return reinterpret_cast<const T *>(p + readScalar<uint32_t>(p));
  }
};

// Bounds checker.  Every generated `verify` goes through these helpers so a corrupt
// or truncated file is rejected with a message instead of being dereferenced.
class Verifier {
public:
  Verifier(const uint8_t *buf, size_t size) : buf_(buf), size_(size) {}

  bool ok() const { return error_.empty(); }
  const std::string &error() const { return error_; }
  bool fail(const std::string &what) {
    if (error_.empty()) {
      error_ = what;
    }
    return false;
  }

  bool inBounds(const void *p, size_t n) const {
    const uint8_t *q = reinterpret_cast<const uint8_t *>(p);
    return q >= buf_ && n <= size_ && static_cast<size_t>(q - buf_) <= size_ - n;
  }

  // Checks table header + vtable; must precede any field check on that table.
  bool tableStart(const Table *t, const char *name) {
    if (++depth_ > kMaxDepth) {
      return fail(std::string("nesting too deep at ") + name);
    }
    if (++tables_ > kMaxTables) {
      return fail("too many tables");
    }
    const uint8_t *p = reinterpret_cast<const uint8_t *>(t);
    if (!inBounds(p, 4) || (reinterpret_cast<uintptr_t>(p) - reinterpret_cast<uintptr_t>(buf_)) % 4) {
      return fail(std::string("table out of bounds or misaligned: ") + name);
    }
    int64_t vtPos = static_cast<int64_t>(p - buf_) - readScalar<int32_t>(p);
    if (vtPos < 0 || static_cast<size_t>(vtPos) + 4 > size_ || (vtPos & 1)) {
      return fail(std::string("vtable out of bounds: ") + name);
    }
    const uint8_t *vt = buf_ + vtPos;
    uint16_t vtSize = readScalar<uint16_t>(vt);
    uint16_t tblSize = readScalar<uint16_t>(vt + 2);
    if (vtSize < 4 || (vtSize & 1) || !inBounds(vt, vtSize) || !inBounds(p, tblSize)) {
      return fail(std::string("bad vtable: ") + name);
    }
    return true;
  }
  void tableEnd() { --depth_; }

  template <typename T>
  bool scalarField(const Table *t, uint32_t id, const char *name) {
    uint16_t off = t->fieldOffset(id);
    if (off && !fieldInTable(t, off, sizeof(T))) {
      return fail(std::string("scalar field out of bounds: ") + name);
    }
    return true;
  }
  bool structField(const Table *t, uint32_t id, size_t size, const char *name) {
    uint16_t off = t->fieldOffset(id);
    if (off && !fieldInTable(t, off, size)) {
      return fail(std::string("struct field out of bounds: ") + name);
    }
    return true;
  }
  // Resolves an offset field; returns nullptr when absent, sets `bad` when invalid.
  const uint8_t *offsetField(const Table *t, uint32_t id, const char *name, bool &bad) {
    uint16_t off = t->fieldOffset(id);
    if (!off) {
      return nullptr;
    }
    if (!fieldInTable(t, off, 4)) {
      bad = true;
      fail(std::string("offset field out of bounds: ") + name);
      return nullptr;
    }
    return follow(t->self() + off, name, bad);
  }
  const uint8_t *follow(const uint8_t *p, const char *name, bool &bad) {
    uint32_t rel = readScalar<uint32_t>(p);
    if (rel == 0 || !inBounds(p + rel, 4)) {
      bad = true;
      fail(std::string("offset target out of bounds: ") + name);
      return nullptr;
    }
    return p + rel;
  }
  bool string(const uint8_t *p, const char *name) {
    uint32_t n = readScalar<uint32_t>(p);
    if (!inBounds(p + 4, static_cast<size_t>(n) + 1) || p[4 + n] != 0) {
      return fail(std::string("bad string: ") + name);
    }
    return true;
  }
  bool vector(const uint8_t *p, size_t elemSize, const char *name) {
    uint32_t n = readScalar<uint32_t>(p);
    if (!inBounds(p + 4, static_cast<size_t>(n) * elemSize)) {
      return fail(std::string("vector out of bounds: ") + name);
    }
    return true;
  }

private:
  bool fieldInTable(const Table *t, uint16_t off, size_t n) const {
    uint16_t tblSize = readScalar<uint16_t>(t->vtable() + 2);
    return static_cast<size_t>(off) + n <= tblSize;
  }
  static constexpr int kMaxDepth = 64;
  static constexpr size_t kMaxTables = 1u << 24;
  const uint8_t *buf_;
  size_t size_;
  int depth_ = 0;
  size_t tables_ = 0;
  std::string error_;
};

// ---- JSON text (used by the generated toJson members) ---------------------------------------
inline void jsonString(std::string_view v, std::string &out) {
  out += '"';
  for (char ch : v) {
    const unsigned char c = static_cast<unsigned char>(ch);
    switch (c) {
    case '"': out += "\\\""; break;
    case '\\': out += "\\\\"; break;
    case '\n': out += "\\n"; break;
    case '\r': out += "\\r"; break;
    case '\t': out += "\\t"; break;
    default:
      if (c < 0x20) {
        char buf[8];
        std::snprintf(buf, sizeof(buf), "\\u%04x", c);
        out += buf;
      } else {
        out += ch;
      }
    }
  }
  out += '"';
}
inline void jsonScalar(bool v, std::string &out) { out += v ? "true" : "false"; }
inline void jsonScalar(float v, std::string &out) {
  if (v != v) { out += "NaN"; return; }
  if (v - v != 0.0f) { out += v > 0 ? "Infinity" : "-Infinity"; return; }
  char buf[32];
  std::snprintf(buf, sizeof(buf), "%.9g", static_cast<double>(v));
  out += buf;
}
inline void jsonScalar(double v, std::string &out) {
  if (v != v) { out += "NaN"; return; }
  if (v - v != 0.0) { out += v > 0 ? "Infinity" : "-Infinity"; return; }
  char buf[40];
  std::snprintf(buf, sizeof(buf), "%.17g", v);
  out += buf;
}
template <typename T, typename = std::enable_if_t<std::is_integral_v<T> && !std::is_same_v<T, bool>>>
inline void jsonScalar(T v, std::string &out) {
  out += std::to_string(v);
}
// An enum value by name, or by number when the schema does not know it.
inline void jsonEnum(const char *name, long long value, std::string &out) {
  if (name && name[0]) jsonString(name, out);
  else out += std::to_string(value);
}

} // namespace fb
