// Handle and option types of the tt::runtime API, as the B200 target provides them.
//
// Names, members and semantics follow the reference header
// runtime/include/tt/runtime/types.h (handle model :112-150, TensorDesc :187-208,
// MeshDeviceOptions :221-231, Flatbuffer/Binary :302-386, Device/Event/Tensor/Layout :392-481)
// so that code written against tt::runtime compiles against this target unchanged.  The
// flatbuffer accessor types come from this repo's own generated header instead of flatc's.
#ifndef TT_RUNTIME_TYPES_H
#define TT_RUNTIME_TYPES_H

#include <cassert>
#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

#include "generated/ttnn_schema.h"

namespace tt::runtime {

// The reference keeps this enum in runtime/include/tt/runtime/flatbuffer/types.fbs:8-12
// (Disabled, TTNN, TTMetal).  CUDA is appended, which keeps the existing values stable.
enum class DeviceRuntime : uint32_t { Disabled = 0, TTNN = 1, TTMetal = 2, CUDA = 3 };
enum class HostRuntime : uint32_t { Local = 0, Distributed = 1 };
enum class DispatchCoreType : uint32_t { WORKER = 0, ETH = 1 };
enum class FabricConfig : uint32_t { DISABLED = 0, FABRIC_1D = 1, FABRIC_1D_RING = 2, FABRIC_2D = 3 };
enum class MemoryLogLevel : uint32_t { NONE = 0, PROGRAM = 1, OPERATION = 2, ANY = 3 };

inline const char *toString(DeviceRuntime r) {
  switch (r) {
  case DeviceRuntime::Disabled: return "Disabled";
  case DeviceRuntime::TTNN: return "TTNN";
  case DeviceRuntime::TTMetal: return "TTMetal";
  case DeviceRuntime::CUDA: return "CUDA";
  }
  return "";
}

enum class MemoryBufferType { DRAM, L1, L1_SMALL, TRACE };

using Scalar = std::variant<uint32_t, int32_t, uint16_t, int16_t, uint8_t, int8_t, bool, float>;

namespace detail {

struct ObjectImpl {
  std::shared_ptr<void> handle;
  ObjectImpl(std::shared_ptr<void> handle) : handle(std::move(handle)) {}
  template <typename T> T &as() {
    assert(handle && "Handle should not be null");
    return *static_cast<T *>(handle.get());
  }
  template <typename T> const T &as() const {
    assert(handle && "Handle should not be null");
    return *static_cast<const T *>(handle.get());
  }
};

// A handle tagged with the device runtime that created it; casting with another runtime's tag
// is a programming error (reference: types.h:112-150).
struct RuntimeCheckedObjectImpl {
  std::shared_ptr<void> handle;
  DeviceRuntime associatedRuntime;

  RuntimeCheckedObjectImpl() : handle(nullptr), associatedRuntime(DeviceRuntime::Disabled) {}
  RuntimeCheckedObjectImpl(std::shared_ptr<void> handle, DeviceRuntime runtime)
      : handle(std::move(handle)), associatedRuntime(runtime) {}

  bool matchesRuntime(DeviceRuntime runtime) const { return associatedRuntime == runtime; }
  void assertMatchesRuntime(DeviceRuntime expected) const;

  template <typename T> T &as(DeviceRuntime expected) {
    assertMatchesRuntime(expected);
    return *static_cast<T *>(handle.get());
  }
  template <typename T> const T &as(DeviceRuntime expected) const {
    assertMatchesRuntime(expected);
    return *static_cast<const T *>(handle.get());
  }
  template <typename T> std::shared_ptr<T> asSharedPtr(DeviceRuntime expected) const {
    assertMatchesRuntime(expected);
    return std::static_pointer_cast<T>(handle);
  }
};

} // namespace detail

struct TensorDesc {
  std::vector<uint32_t> shape = {};
  ::tt::target::DataType dataType = ::tt::target::DataType::MAX;
  std::vector<int64_t> stride = {};
  uint64_t physicalVolume = 0;

  TensorDesc() = default;
  TensorDesc(const std::vector<uint32_t> &shape, ::tt::target::DataType dataType,
             const std::optional<std::vector<int64_t>> &stride = {},
             std::optional<uint64_t> physicalVolume = {});

  size_t volume() const;
  size_t sizeBytes() const;
  uint32_t elementSize() const;
  bool isPadded() const { return physicalVolume > volume(); }
};

struct MeshDeviceOptions {
  std::vector<uint32_t> meshOffset{0, 0};
  // CUDA device ordinals backing the mesh coordinates this process owns (row-major).
  // Empty: device i of the process backs mesh coordinate i.
  std::vector<int> deviceIds{};
  size_t numHWCQs = 1;
  bool enableProgramCache = true;
  std::optional<std::vector<uint32_t>> meshShape = std::nullopt;
  std::optional<size_t> l1SmallSize = std::nullopt;
  std::optional<size_t> traceRegionSize = std::nullopt;
  std::optional<DispatchCoreType> dispatchCoreType = std::nullopt;

  // --- additions of this target: one process per GPU ---------------------------------------
  // When processCount > 1 the mesh is spread over `processCount` processes, this one owning
  // mesh coordinate `processRank` only; `ncclUniqueId` (128 bytes, identical in all
  // processes, made by getNcclUniqueId() in one of them) bootstraps the communicator.
  uint32_t processRank = 0;
  uint32_t processCount = 1;
  std::string ncclUniqueId;
};

struct Flatbuffer : public detail::ObjectImpl {
  using detail::ObjectImpl::ObjectImpl;

  static Flatbuffer loadFromPath(const char *path);
  static Flatbuffer loadFromMemory(const void *memory, size_t size);

  void store(const char *path) const;
  void storeToMemory(std::vector<std::byte> &serializedFlatbuffer) const;

  size_t size() const; // bytes including the 4-byte size prefix
  std::string getFileIdentifier() const;
  std::string getVersion() const;
  std::string getSchemaHash() const;
  bool checkSchemaHash() const;
  std::string getTTMLIRGitHash() const;
  std::string asJson() const;
};

struct SystemDesc : public Flatbuffer {
  using Flatbuffer::Flatbuffer;
};

struct Binary : public Flatbuffer {
  Binary(Flatbuffer fb);
  Binary(std::shared_ptr<void> handle);
  Binary(const Binary &) = default;
  Binary(Binary &&) = default;
  Binary &operator=(const Binary &) = default;
  Binary &operator=(Binary &&) = default;

  static Binary loadFromPath(const char *path);
  static Binary loadFromMemory(const void *memory, size_t size);

  const ::tt::target::ttnn::TTNNBinary *get() const;

  std::uint32_t getNumPrograms() const;
  std::string getProgramName(std::uint32_t programIndex) const;
  bool isProgramPrivate(std::uint32_t programIndex) const;
  std::string getProgramOpsAsJson(std::uint32_t programIndex) const;
  std::string getProgramInputsAsJson(std::uint32_t programIndex) const;
  std::string getProgramOutputsAsJson(std::uint32_t programIndex) const;
  std::string getMlirAsJson() const;
  std::string getSystemDescAsJson() const;
  std::uint32_t getNumProgramInputs(std::uint32_t programIndex) const;
  std::uint32_t getNumProgramOutputs(std::uint32_t programIndex) const;
  std::vector<TensorDesc> getProgramInputs(std::uint32_t programIndex) const;
  std::vector<TensorDesc> getProgramOutputs(std::uint32_t programIndex) const;
  std::unordered_map<std::uint32_t, const ::tt::target::GoldenTensor *>
  getDebugInfoGolden(std::string &loc) const;
  const std::pair<std::uint32_t, std::uint32_t> getProgramMeshShape(std::uint32_t programIndex) const;

  void setId(std::uint64_t id) { binaryId = id; }
  std::uint64_t id() const { return binaryId; }

private:
  std::uint64_t binaryId;
};

struct Device : public detail::RuntimeCheckedObjectImpl {
  Device(DeviceRuntime runtime) : detail::RuntimeCheckedObjectImpl(nullptr, runtime), globalId(nextId()) {}
  Device(std::shared_ptr<void> handle, DeviceRuntime runtime)
      : detail::RuntimeCheckedObjectImpl(std::move(handle), runtime), globalId(nextId()) {}
  std::uint32_t getGlobalId() const { return globalId; }

private:
  static std::uint32_t nextId();
  std::uint32_t globalId;
};

struct Event : public detail::RuntimeCheckedObjectImpl {
  using detail::RuntimeCheckedObjectImpl::RuntimeCheckedObjectImpl;
};

struct Tensor : public detail::RuntimeCheckedObjectImpl {
  std::shared_ptr<void> data;
  Event event;
  Tensor() : globalId(nextId()) {}
  Tensor(std::shared_ptr<void> handle, std::shared_ptr<void> data, DeviceRuntime runtime,
         std::optional<std::shared_ptr<void>> eventHandle = std::nullopt)
      : detail::RuntimeCheckedObjectImpl(std::move(handle), runtime), data(std::move(data)),
        event(eventHandle.value_or(nullptr), runtime), globalId(nextId()) {}
  std::uint64_t getGlobalId() const { return globalId; }

private:
  static std::uint64_t nextId();
  std::uint64_t globalId;
};

struct TensorRef : public detail::RuntimeCheckedObjectImpl {
  using detail::RuntimeCheckedObjectImpl::RuntimeCheckedObjectImpl;
};

struct Layout : public detail::RuntimeCheckedObjectImpl {
  using detail::RuntimeCheckedObjectImpl::RuntimeCheckedObjectImpl;
};

struct CallbackContext : public detail::RuntimeCheckedObjectImpl {
  using detail::RuntimeCheckedObjectImpl::RuntimeCheckedObjectImpl;
};

struct OpContext : public detail::RuntimeCheckedObjectImpl {
  using detail::RuntimeCheckedObjectImpl::RuntimeCheckedObjectImpl;
};

} // namespace tt::runtime

#endif
