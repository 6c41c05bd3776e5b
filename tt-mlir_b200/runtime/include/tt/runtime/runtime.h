// Free functions of the tt::runtime API served by the B200 target.
//
// Signatures follow runtime/include/tt/runtime/runtime.h:31-308 of the reference.  Functions
// that only make sense on Tenstorrent silicon (L1 sizes, fabric configuration, trace regions,
// the distributed controller) are kept where callers such as ttrt invoke them
// unconditionally, and return neutral values.
#ifndef TT_RUNTIME_RUNTIME_H
#define TT_RUNTIME_RUNTIME_H

#include <cstdint>
#include <functional>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "tt/runtime/types.h"

namespace tt::runtime {

namespace detail {
uint32_t getNumShards(Tensor tensor);
} // namespace detail

std::vector<DeviceRuntime> getAvailableDeviceRuntimes();
DeviceRuntime getCurrentDeviceRuntime();
void setCurrentDeviceRuntime(const DeviceRuntime &runtime);
void setCompatibleDeviceRuntime(const Binary &binary);

std::vector<HostRuntime> getAvailableHostRuntimes();
HostRuntime getCurrentHostRuntime();
void setCurrentHostRuntime(const HostRuntime &runtime);

void setMlirHome(std::string_view mlirHome);
void setMetalHome(std::string_view metalHome);
void setMemoryLogLevel(const MemoryLogLevel &logLevel);

// Synthesised descriptor: one chip per visible GPU, HBM as a single DRAM channel.
SystemDesc getCurrentSystemDesc(std::optional<DispatchCoreType> dispatchCoreType = std::nullopt,
                                std::optional<Device> meshDevice = std::nullopt);

Tensor createBorrowedHostTensor(void *data, const std::vector<std::uint32_t> &shape,
                                const std::vector<std::int64_t> &stride, std::uint32_t itemsize,
                                ::tt::target::DataType dataType);
Tensor createOwnedHostTensor(const void *data, const std::vector<std::uint32_t> &shape,
                             const std::vector<std::int64_t> &stride, std::uint32_t itemsize,
                             ::tt::target::DataType dataType);
Tensor createMultiDeviceHostTensor(const std::vector<const void *> &data,
                                   const std::vector<std::uint32_t> &shape,
                                   const std::vector<std::int64_t> &stride, std::uint32_t itemsize,
                                   ::tt::target::DataType dataType,
                                   const std::unordered_map<std::string, std::string> &strategy,
                                   const std::vector<uint32_t> &meshShape);
Tensor createMultiDeviceHostTensor(const std::vector<Tensor> &tensorShards,
                                   const std::unordered_map<std::string, std::string> &strategy,
                                   const std::vector<uint32_t> &meshShape);
Tensor createMultiDeviceBorrowedHostTensor(std::vector<void *> &data,
                                           const std::vector<std::uint32_t> &shape,
                                           const std::vector<std::int64_t> &stride,
                                           std::uint32_t itemsize, ::tt::target::DataType dataType,
                                           const std::unordered_map<std::string, std::string> &strategy,
                                           const std::vector<uint32_t> &meshShape);
Tensor createEmptyTensor(Device device, Layout layout, const std::vector<std::uint32_t> &shape,
                         const std::vector<std::int64_t> &stride, std::uint32_t itemsize);

inline Tensor createBorrowedHostTensor(void *data, const TensorDesc &desc) {
  return createBorrowedHostTensor(data, desc.shape, desc.stride, desc.elementSize(), desc.dataType);
}
inline Tensor createOwnedHostTensor(const void *data, const TensorDesc &desc) {
  return createOwnedHostTensor(data, desc.shape, desc.stride, desc.elementSize(), desc.dataType);
}

bool isTensorAllocated(Tensor tensor);
tt::target::DataType getTensorDataType(Tensor tensor);
std::vector<std::byte> getTensorDataBuffer(Tensor tensor);
std::uint32_t getTensorElementSize(Tensor tensor);
std::uint32_t getTensorVolume(Tensor tensor);
std::uint32_t getTensorLogicalVolume(Tensor tensor);
std::vector<std::uint32_t> getTensorShape(Tensor tensor);
std::vector<std::int64_t> getTensorStride(Tensor tensor);
TensorDesc getTensorDesc(Tensor tensor);
bool getTensorRetain(Tensor tensor);
void setTensorRetain(Tensor tensor, bool retain);

tt::target::Arch getArch();
size_t getNumAvailableDevices();
// 128 opaque bytes that every process of a one-process-per-GPU mesh passes in
// MeshDeviceOptions::ncclUniqueId (addition of this target).
std::string getNcclUniqueId();

Device openMeshDevice(const MeshDeviceOptions &options = {});
void closeMeshDevice(Device parentMesh);
Device createSubMeshDevice(Device parentMesh, const std::vector<uint32_t> &meshShape,
                           const std::optional<const std::vector<uint32_t>> &meshOffset = std::nullopt);
void releaseSubMeshDevice(Device subMesh);
void reshapeMeshDevice(Device meshDevice, const std::vector<uint32_t> &meshShape);
std::vector<uint32_t> getMeshShape(Device meshDevice);
std::vector<int> getDeviceIds(Device meshDevice);
size_t getNumHwCqs(Device meshDevice);
bool isProgramCacheEnabled(Device meshDevice);
void clearProgramCache(Device meshDevice);
size_t getL1SmallSize(Device meshDevice);
size_t getTraceRegionSize(Device meshDevice);
// Drops the traces recorded for one main program of one binary (runtime/include/tt/runtime/
// runtime.h:182-183): graphs and slots are freed; the next submit records them again.
void releaseTrace(Device meshDevice, std::uint64_t binaryId, size_t mainProgramId);
size_t getNumDramChannels(Device meshDevice);
size_t getDramSizePerChannel(Device meshDevice);
size_t getL1SizePerCore(Device meshDevice);
void deallocateBuffers(Device device);
void dumpMemoryReport(Device device);
void readDeviceProfilerResults(Device device);
void setFabricConfig(FabricConfig config);

void wait(Event event);
void wait(Tensor tensor, std::optional<uint8_t> cqId = std::nullopt);
void wait(const std::vector<Tensor> &tensors, std::optional<uint8_t> cqId = std::nullopt);

std::vector<Tensor> toHost(Tensor tensor, bool untilize = false, bool blocking = true);
std::vector<Tensor> getDeviceTensors(Tensor tensor);
Tensor toLayout(Tensor tensor, Device device, Layout layout, std::optional<bool> retain = std::nullopt);
bool hasLayout(Tensor tensor, Layout layout);
Layout getTensorLayout(Tensor tensor);
Layout getLayout(Binary executableHandle, std::uint32_t programIndex, std::uint32_t inputIndex);

void memcpy(void *dst, Tensor src, std::optional<tt::target::DataType> targetDataType = std::nullopt);
void memcpy(Tensor dst, Tensor src);
void deallocateTensor(Tensor &tensor, bool force = false);

std::string getOpDebugString(OpContext opContextHandle);
std::string getOpLocInfo(OpContext opContextHandle);
std::unordered_map<std::uint32_t, Tensor> getOpOutputTensor(OpContext opContextHandle,
                                                            CallbackContext programContextHandle);
std::vector<TensorRef> getOpOutputRefs(OpContext opContextHandle);
std::vector<TensorRef> getOpInputRefs(OpContext opContextHandle);
std::vector<uint32_t> getTensorRefShape(TensorRef tensorRef);
::tt::target::DataType getTensorRefDataType(TensorRef tensorRef);
std::optional<Tensor> retrieveTensorFromPool(CallbackContext programContextHandle, TensorRef tensorRef,
                                             bool untilize);
void updateTensorInPool(CallbackContext programContextHandle, TensorRef tensorRef, Tensor srcTensor);
size_t getProgramIndex(CallbackContext programContextHandle);

using OpWalkFn = std::function<void(OpContext)>;
void walkProgram(Binary executableHandle, uint32_t programIndex, const OpWalkFn &cb);

std::vector<Tensor> submit(Device deviceHandle, Binary executableHandle, std::uint32_t programIndex,
                           std::vector<Tensor> &inputs);

void dumpTensor(Tensor tensor, const std::string &filePath);
Tensor loadTensor(const std::string &filePath, std::optional<Device> device = std::nullopt);

} // namespace tt::runtime

#endif
