// Internal object model of the B200 runtime target: what sits behind the opaque handles of
// tt/runtime/types.h.  The reference keeps the equivalent state in TTNNTensorWrapper,
// LayoutDesc and the MeshDevice (runtime/include/tt/runtime/detail/ttnn/types/types.h:36-135).
#pragma once

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/ttb_kernels.h"
#include "tt/runtime/types.h"

namespace tt::runtime::cuda {

using ::tt::target::DataType;

// ---- errors / logging ------------------------------------------------------------------
// Same convention as the reference's LOG_FATAL (runtime/include/tt/runtime/detail/common/
// logger.h:301-321): the message goes to stderr and a std::runtime_error is thrown.
[[noreturn]] void fatal(const std::string &msg);
void logDebug(const std::string &msg);

template <typename... Args> std::string strcat_(Args &&...args) {
  std::ostringstream os;
  (os << ... << args);
  return os.str();
}

// The schema hash this runtime writes and accepts (binary.cpp).
const char *schemaHashString();

#define TTRT_FATAL(...) ::tt::runtime::cuda::fatal(::tt::runtime::cuda::strcat_(__VA_ARGS__))
#define TTRT_ASSERT(cond, ...)                                                           \
  do {                                                                                   \
    if (!(cond)) {                                                                       \
      ::tt::runtime::cuda::fatal(::tt::runtime::cuda::strcat_("Assertion `" #cond "` failed: ", __VA_ARGS__)); \
    }                                                                                    \
  } while (0)
// Turns a C-ABI status into an exception carrying the kernel library's message.
#define TTB_CALL(expr)                                                                   \
  do {                                                                                   \
    int _rc = (expr);                                                                    \
    if (_rc != TTB_OK) {                                                                 \
      ::tt::runtime::cuda::fatal(::tt::runtime::cuda::strcat_(#expr " failed (", _rc, "): ", ttb_last_error())); \
    }                                                                                    \
  } while (0)

// ---- dtype helpers ---------------------------------------------------------------------
uint32_t dataTypeSize(DataType dt); // 0 for block formats
bool isSupportedDataType(DataType dt);
const char *dataTypeName(DataType dt);
inline int ttbDtype(DataType dt) { return static_cast<int>(dt); }

// ---- device ----------------------------------------------------------------------------
// One mesh coordinate owned by this process: a CUDA device, a stream and (for meshes of more
// than one device) an NCCL communicator rank.
struct RankCtx {
  int cudaDevice = 0;
  uint32_t meshRank = 0;
  void *stream = nullptr;   // compute: every kernel of every program, in submission order
  void *copyIn = nullptr;   // host -> device copies from pinned memory (overlap the previous step's compute)
  void *copyOut = nullptr;  // non-blocking device -> host copies (overlap the next step's compute)
  void *comm = nullptr;
  void *symm = nullptr;     // peer-memory workspace for all-reduce (created at the first one), or null
};

// A CUDA event owned by whoever holds the last reference.
struct EventHolder {
  void *event = nullptr;
  int cudaDevice = 0;
  EventHolder(int device);
  ~EventHolder();
  EventHolder(const EventHolder &) = delete;
  EventHolder &operator=(const EventHolder &) = delete;
};
using EventPtr = std::shared_ptr<EventHolder>;

// Upload staging memory that went out of use, kept per device for the next upload of the same
// size: `lastUse` (recorded on the compute stream when the block was released) gates its reuse
// on the upload stream.  Keeps the stream-ordered allocator, whose cross-stream reuse would make
// the upload wait for the compute stream, out of a pipelined loop.
struct StagingBlock {
  void *ptr = nullptr;
  size_t bytes = 0;
  EventPtr lastUse;
};

// A recorded trace: one executable CUDA graph per coordinate this process owns.
struct TraceGraph {
  std::vector<void *> execs;
};
// What CaptureOrExecuteTraceOp keeps per (binary, main program, capture program, execute program),
// as the reference's TraceData (runtime/include/tt/runtime/detail/ttnn/types/trace_cache.h).
struct TraceData {
  uint32_t traceId = 0;
  std::vector<std::shared_ptr<struct TensorImpl>> inputSlots, outputSlots;
};
using TraceKey = std::tuple<uint64_t, uint32_t, uint32_t, uint32_t>;

struct DeviceImpl {
  std::map<uint32_t, TraceGraph> traces; // by trace id
  uint32_t nextTraceId = 1;
  uint32_t recordingTrace = 0;           // id of the trace being recorded, or 0
  std::map<TraceKey, TraceData> traceCache;
  void releaseTraceGraph(uint32_t id);
  std::vector<std::vector<StagingBlock>> stagingCache; // per entry of `locals`
  std::mutex stagingMutex;
  std::vector<uint32_t> meshShape{1, 1};
  uint32_t worldSize = 1;          // mesh volume
  std::vector<RankCtx> locals;     // coordinates this process owns
  bool multiProcess = false;
  bool open = false;
  bool ranIndexOp = false; // a gather / scatter ran: ask the kernel library for bad indices at the next wait
  bool ranEmbedding = false, ranUpdateCache = false; // their kernels flag indices outside the table / cache; wait() reports it
  bool symmTried = false;          // the peer workspaces are set up (or found unavailable) once
  std::mutex submitMutex;          // submit is serialised per device
  ~DeviceImpl();
  void close();
};

// ---- tensors ---------------------------------------------------------------------------
struct Buffer {
  void *ptr = nullptr;
  size_t bytes = 0;
  int cudaDevice = -1;   // -1: host memory
  void *stream = nullptr; // stream that orders the free of device memory
  std::shared_ptr<struct DeviceImpl> owner; // keeps the stream's device alive; closed device -> plain free
  enum class Kind { Borrowed, HostMalloc, HostPinned, HostPinnedPooled, Device, DeviceStaging } kind = Kind::Borrowed;
  size_t localIndex = 0; // DeviceStaging: which entry of owner->locals the block belongs to
  std::shared_ptr<void> keepAlive; // another object owning the memory (views)
  // Work on a copy stream that the compute stream does not know about yet:
  //  device buffer: its contents are complete once `ready` fires (an upload in flight), and
  //                 `pendingRead` is a download still reading it (the free waits for it);
  //  host buffer:   `ready` is the download that fills it (wait(tensor) blocks on it).
  EventPtr ready, pendingRead;
  ~Buffer();
};
using BufferPtr = std::shared_ptr<Buffer>;

enum class Storage { Host, Device };

struct TensorImpl {
  std::vector<uint32_t> shape;     // per-shard logical shape
  std::vector<int64_t> stride;     // dense row-major, in elements
  DataType dtype = DataType::Float32;
  Storage storage = Storage::Host;
  ::tt::target::TensorLayout layout = ::tt::target::TensorLayout::RowMajor; // metadata only
  // Host: 1 shard, or one per mesh coordinate (multi-device host tensor).
  // Device: one per mesh coordinate owned by this process, in DeviceImpl::locals order.
  std::vector<BufferPtr> shards;
  std::shared_ptr<DeviceImpl> device; // set for device tensors
  bool retain = false;
  // Identifies the tensor's contents: unique per tensor and renewed by every write through the
  // API, as in the reference (TTNNTensorWrapper::version, runtime/include/tt/runtime/detail/ttnn/
  // types/types.h:43,75-83).  Key of the const-eval cache and of the trace input slots.
  std::atomic<uint64_t> version{nextTensorVersion()};
  static uint64_t nextTensorVersion();
  // A reshaped alias made for a program input shares its memory with `base`, the caller's tensor.
  std::shared_ptr<TensorImpl> base;
  // Run when the tensor dies (const-eval cache entries keyed by it are dropped).
  std::vector<std::function<void()>> onDestroy;
  void *readyEvent = nullptr;      // recorded after the producing work was enqueued
  // The tensor was never assembled: its producer scattered it, row block by row block, into the
  // all-reduce workspaces of the ranks that will sum the blocks.  Only that all-reduce may read it.
  bool pushedForAllReduce = false;
  // Result of prepare_conv2d_weights / prepare_conv2d_bias: the tensor the op was given, handed on unchanged (the
  // preparation TTNN does is a Tenstorrent tile / shard layout; these kernels take the weights as they are).
  // conv2d uses it in place of the declared operand.
  std::shared_ptr<TensorImpl> preparedFrom;

  size_t volume() const {
    size_t v = 1;
    for (uint32_t d : shape) v *= d;
    return v;
  }
  size_t bytes() const { return volume() * dataTypeSize(dtype); }
  // True while at least one shard still has memory (shards of other processes stay null).
  bool allocated() const {
    for (const BufferPtr &b : shards) {
      if (b && b->ptr) return true;
    }
    return false;
  }
  ~TensorImpl();
};
using TensorPtr = std::shared_ptr<TensorImpl>;

struct LayoutImpl {
  Storage storage = Storage::Host;
  ::tt::target::TensorLayout layout = ::tt::target::TensorLayout::RowMajor;
  DataType dtype = DataType::Float32;
  bool operator==(const LayoutImpl &o) const {
    return storage == o.storage && layout == o.layout && dtype == o.dtype;
  }
};

std::vector<int64_t> denseStrides(const std::vector<uint32_t> &shape);

TensorPtr makeHostTensor(const std::vector<uint32_t> &shape, DataType dt, size_t nshards, bool pinned = false);
// Makes the compute stream wait for uploads of `t` that are still in flight on the copy stream.
void orderAfterUploads(const TensorPtr &t);
TensorPtr makeDeviceTensor(const std::shared_ptr<DeviceImpl> &dev, const std::vector<uint32_t> &shape, DataType dt);
Tensor wrapTensor(const TensorPtr &t);
TensorPtr unwrapTensor(const Tensor &t);

// Host <-> device movement shared by the API functions and the executor's layout ops.
TensorPtr toDevice(const TensorPtr &host, const std::shared_ptr<DeviceImpl> &dev, DataType dt);
TensorPtr toHostTensor(const TensorPtr &devTensor, bool blocking);
TensorPtr castOnDevice(const TensorPtr &t, DataType dt);

// ---- const-eval cache --------------------------------------------------------------------
// Results of const-eval sub-programs, shared by every binary that carries a function with the
// same hash (the reference's GlobalTensorCache, runtime/include/tt/runtime/detail/ttnn/types/
// global_tensor_cache.h:26-104).  An entry lives until one of the tensors it was computed from
// dies, the device closes, or clear().
struct ConstEvalKey {
  const void *device = nullptr;
  std::string hash;
  std::vector<uint64_t> inputVersions;
  bool operator<(const ConstEvalKey &o) const {
    return std::tie(device, hash, inputVersions) < std::tie(o.device, o.hash, o.inputVersions);
  }
};
class ConstEvalCache {
public:
  static ConstEvalCache &get();
  bool find(const ConstEvalKey &key, std::vector<TensorPtr> &outputs) const;
  void store(const ConstEvalKey &key, const std::vector<TensorPtr> &inputs, const std::vector<TensorPtr> &outputs);
  void remove(const ConstEvalKey &key);
  void removeDevice(const void *device);
  void clear();
  size_t size() const;

private:
  mutable std::mutex mutex;
  std::map<ConstEvalKey, std::vector<TensorPtr>> entries;
};

// ---- program execution -----------------------------------------------------------------
std::vector<Tensor> runProgram(const std::shared_ptr<DeviceImpl> &dev, Binary &binary, uint32_t programIndex,
                               std::vector<Tensor> &inputs);

// Tensor refs an op reads / writes, in schema order (used by hooks and by fusion legality).
void collectOpRefs(const ::tt::target::ttnn::Operation *op,
                   std::vector<const ::tt::target::ttnn::TensorRef *> &ins,
                   std::vector<const ::tt::target::ttnn::TensorRef *> &outs);

struct OpContextImpl {
  const ::tt::target::ttnn::Operation *op = nullptr;
};
struct ProgramContextImpl; // defined in executor.cpp

} // namespace tt::runtime::cuda
