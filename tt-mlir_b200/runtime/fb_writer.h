// A small back-to-front flatbuffer writer (the format's published layout: tables with vtables,
// vectors, strings, inline structs), enough for the few buffers this runtime has to PRODUCE: the
// system descriptor of tt::runtime::getCurrentSystemDesc.  Reading is fb.h; there is no flatbuffers
// library in the build.  Offsets returned by the create* functions count from the END of the buffer,
// as in the reference implementation of the format, so that children are written before parents.
#pragma once

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace tt::runtime::cuda::fb {

class Writer {
public:
  explicit Writer(size_t initial = 4096) : buf_(initial), head_(initial) {}

  uint32_t offset() const { return static_cast<uint32_t>(buf_.size() - head_); }

  uint32_t createString(const std::string &s) {
    prep(4, s.size() + 1);
    push<uint8_t>(0);
    pushBytes(s.data(), s.size());
    push<uint32_t>(static_cast<uint32_t>(s.size()));
    return offset();
  }

  template <typename T> uint32_t createScalarVector(const std::vector<T> &v) {
    prep(4, v.size() * sizeof(T));
    prep(sizeof(T), v.size() * sizeof(T));
    pushBytes(v.data(), v.size() * sizeof(T));
    push<uint32_t>(static_cast<uint32_t>(v.size()));
    return offset();
  }

  // `count` structs of `structSize` bytes each, already laid out as the schema's struct.
  uint32_t createStructVector(const void *data, size_t count, size_t structSize, size_t align) {
    prep(4, count * structSize);
    prep(align, count * structSize);
    pushBytes(data, count * structSize);
    push<uint32_t>(static_cast<uint32_t>(count));
    return offset();
  }

  uint32_t createOffsetVector(const std::vector<uint32_t> &targets) {
    prep(4, 4 * targets.size());
    for (size_t i = targets.size(); i-- > 0;) pushUOffset(targets[i]);
    push<uint32_t>(static_cast<uint32_t>(targets.size()));
    return offset();
  }

  // ---- tables: startTable(n fields); add*(id, ...) in any order; endTable() ----------------------
  void startTable(size_t fields) {
    slots_.assign(fields, 0);
    objectEnd_ = offset();
  }
  template <typename T> void addScalar(size_t id, T v, T dflt = T()) {
    if (v == dflt) return; // defaults are not stored
    prep(sizeof(T), 0);
    push<T>(v);
    slots_[id] = offset();
  }
  void addStruct(size_t id, const void *data, size_t size, size_t align) {
    prep(align, size);
    pushBytes(data, size);
    slots_[id] = offset();
  }
  void addOffset(size_t id, uint32_t target) {
    if (!target) return;
    pushUOffset(target);
    slots_[id] = offset();
  }
  uint32_t endTable() {
    prep(4, 0);
    push<int32_t>(0); // patched below with the distance to the vtable
    const uint32_t objectOffset = offset();
    size_t n = slots_.size();
    while (n > 0 && slots_[n - 1] == 0) --n;
    std::vector<uint16_t> vt;
    vt.push_back(static_cast<uint16_t>((n + 2) * 2));
    vt.push_back(static_cast<uint16_t>(objectOffset - objectEnd_));
    for (size_t i = 0; i < n; ++i) vt.push_back(slots_[i] ? static_cast<uint16_t>(objectOffset - slots_[i]) : 0);
    prep(2, vt.size() * 2);
    pushBytes(vt.data(), vt.size() * 2);
    const int32_t toVtable = static_cast<int32_t>(offset()) - static_cast<int32_t>(objectOffset);
    std::memcpy(&buf_[buf_.size() - objectOffset], &toVtable, 4);
    return objectOffset;
  }

  // Size-prefixed buffer with a 4-character file identifier: [u32 size][u32 root][identifier]...
  std::vector<uint8_t> finish(uint32_t root, const char identifier[4]) {
    prep(minAlign_, 4 + 4 + 4);
    pushBytes(identifier, 4);
    pushUOffset(root);
    push<uint32_t>(offset());
    return std::vector<uint8_t>(buf_.begin() + static_cast<std::ptrdiff_t>(head_), buf_.end());
  }

private:
  std::vector<uint8_t> buf_;
  size_t head_;
  size_t minAlign_ = 1;
  std::vector<uint32_t> slots_;
  uint32_t objectEnd_ = 0;

  void grow(size_t need) {
    while (head_ < need) {
      const size_t old = buf_.size();
      std::vector<uint8_t> bigger(old * 2);
      std::memcpy(bigger.data() + old, buf_.data(), old); // content stays at the end
      buf_.swap(bigger);
      head_ += old;
    }
  }
  // Makes the position after writing `additional` more bytes a multiple of `size`.
  void prep(size_t size, size_t additional) {
    if (size > minAlign_) minAlign_ = size;
    const size_t pad = (~(offset() + additional) + 1) & (size - 1);
    grow(pad + size + additional);
    for (size_t i = 0; i < pad; ++i) buf_[--head_] = 0;
  }
  template <typename T> void push(T v) {
    grow(sizeof(T));
    head_ -= sizeof(T);
    std::memcpy(&buf_[head_], &v, sizeof(T));
  }
  void pushBytes(const void *p, size_t n) {
    grow(n);
    head_ -= n;
    if (n) std::memcpy(&buf_[head_], p, n);
  }
  void pushUOffset(uint32_t target) {
    prep(4, 0);
    push<uint32_t>(offset() - target + 4);
  }
};

} // namespace tt::runtime::cuda::fb
