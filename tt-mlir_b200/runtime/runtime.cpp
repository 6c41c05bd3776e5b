// tt::runtime API of the B200 target: devices, tensors, layouts, host<->device movement.
// Counterpart of runtime/lib/ttnn/runtime.cpp in the reference (createBorrowed/OwnedHostTensor
// :237-314, multi-device host tensors :316-368, tensor queries :428-560, openMeshDevice
// :582-624, wait :824-853, toHost :861-884, toLayout :906-933, getLayout :953-983, memcpy
// :985-1076, deallocateTensor :1078-1087) and of the dispatcher runtime/lib/runtime.cpp.
#include <cstring>
#include <iostream>

#include "fb_writer.h"
#include "impl.h"
#include "tt/runtime/debug.h"
#include "tt/runtime/runtime.h"

namespace tt::runtime {

using namespace ::tt::runtime::cuda;
namespace fbt = ::tt::target::ttnn;
using ::tt::target::TensorLayout;

// ---- handle bookkeeping ------------------------------------------------------------------
void detail::RuntimeCheckedObjectImpl::assertMatchesRuntime(DeviceRuntime expected) const {
  if (!matchesRuntime(expected)) {
    TTRT_FATAL("handle belongs to runtime ", toString(associatedRuntime), ", expected ", toString(expected));
  }
  if (!handle) {
    TTRT_FATAL("null handle");
  }
}

std::uint32_t Device::nextId() {
  static std::atomic<std::uint32_t> id{0};
  return id.fetch_add(1);
}
std::uint64_t Tensor::nextId() {
  static std::atomic<std::uint64_t> id{0};
  return id.fetch_add(1);
}

// ---- TensorDesc --------------------------------------------------------------------------
TensorDesc::TensorDesc(const std::vector<uint32_t> &shape, ::tt::target::DataType dataType,
                       const std::optional<std::vector<int64_t>> &stride, std::optional<uint64_t> physicalVolume)
    : shape(shape), dataType(dataType) {
  this->stride = stride ? *stride : denseStrides(shape);
  this->physicalVolume = physicalVolume ? *physicalVolume : volume();
}
size_t TensorDesc::volume() const {
  size_t v = 1;
  for (uint32_t d : shape) v *= d;
  return v;
}
uint32_t TensorDesc::elementSize() const {
  uint32_t s = dataTypeSize(dataType);
  if (!s) {
    TTRT_FATAL("data type ", ::tt::target::EnumNameDataType(dataType), " has no per-element size");
  }
  return s;
}
size_t TensorDesc::sizeBytes() const { return volume() * elementSize(); }

namespace cuda {

// ---- logging -----------------------------------------------------------------------------
void fatal(const std::string &msg) {
  std::cerr << "[tt::runtime::cuda] FATAL: " << msg << std::endl;
  throw std::runtime_error("Fatal error: " + msg);
}

void logDebug(const std::string &msg) {
  static const bool on = [] {
    const char *e = std::getenv("TTMLIR_RUNTIME_LOGGER_LEVEL");
    return e && (std::strcmp(e, "DEBUG") == 0 || std::strcmp(e, "TRACE") == 0);
  }();
  if (on) {
    std::cerr << "[tt::runtime::cuda] " << msg << std::endl;
  }
}

uint32_t dataTypeSize(DataType dt) {
  switch (dt) {
  case DataType::Float32: case DataType::UInt32: case DataType::Int32: return 4;
  case DataType::Float16: case DataType::BFloat16: case DataType::UInt16: case DataType::Int16: return 2;
  case DataType::UInt8: case DataType::Int8: case DataType::Bool: return 1;
  case DataType::Float64: case DataType::Int64: case DataType::UInt64: return 8;
  default: return 0;
  }
}

bool isSupportedDataType(DataType dt) {
  switch (dt) {
  case DataType::Float32: case DataType::Float16: case DataType::BFloat16: case DataType::UInt32:
  case DataType::UInt16: case DataType::UInt8: case DataType::Int32: case DataType::Int8:
    return true;
  default:
    return false;
  }
}

const char *dataTypeName(DataType dt) { return ::tt::target::EnumNameDataType(dt); }

std::vector<int64_t> denseStrides(const std::vector<uint32_t> &shape) {
  std::vector<int64_t> s(shape.size());
  int64_t acc = 1;
  for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) {
    s[i] = acc;
    acc *= shape[i];
  }
  return s;
}

EventHolder::EventHolder(int device) : cudaDevice(device) {
  TTB_CALL(ttb_set_device(device));
  TTB_CALL(ttb_event_create(&event));
}
EventHolder::~EventHolder() {
  if (event) ttb_event_destroy(event);
}

// Page-locked staging buffers for non-blocking downloads are recycled: pinning memory costs
// milliseconds, a step of a pipelined loop needs one buffer of the same size every time.
namespace {
struct PinnedPool {
  std::mutex mu;
  std::unordered_map<size_t, std::vector<void *>> free;
  size_t cachedBytes = 0;
  static constexpr size_t kMaxCached = size_t(2) << 30;
  static PinnedPool &get() {
    static PinnedPool *p = new PinnedPool(); // never destroyed: buffers may outlive static teardown
    return *p;
  }
  void *take(size_t bytes) {
    {
      std::lock_guard<std::mutex> g(mu);
      auto it = free.find(bytes);
      if (it != free.end() && !it->second.empty()) {
        void *p = it->second.back();
        it->second.pop_back();
        cachedBytes -= bytes;
        return p;
      }
    }
    void *p = nullptr;
    TTB_CALL(ttb_host_alloc_pinned(&p, bytes));
    return p;
  }
  void give(void *p, size_t bytes) {
    {
      std::lock_guard<std::mutex> g(mu);
      if (cachedBytes + bytes <= kMaxCached) {
        free[bytes].push_back(p);
        cachedBytes += bytes;
        return;
      }
    }
    ttb_host_free_pinned(p);
  }
};
} // namespace

Buffer::~Buffer() {
  if (!ptr) {
    return;
  }
  switch (kind) {
  case Kind::HostMalloc: std::free(ptr); break;
  case Kind::HostPinned: ttb_host_free_pinned(ptr); break;
  case Kind::HostPinnedPooled:
    // A download that still writes this buffer must land before the memory is handed out again.
    if (ready) ttb_event_sync(ready->event);
    PinnedPool::get().give(ptr, bytes);
    break;
  case Kind::Device: {
    // Stream-ordered free: safe while kernels using the block are still queued on `stream`.
    // After the device was closed its stream is gone: free on the default stream instead.
    ttb_set_device(cudaDevice);
    void *st = (owner && owner->open) ? stream : nullptr;
    // Copies on the copy streams are not in `stream`'s order: the free waits for them.
    if (ready) ttb_stream_wait_event(st, ready->event);
    if (pendingRead) ttb_stream_wait_event(st, pendingRead->event);
    ttb_free(ptr, st);
    break;
  }
  case Kind::DeviceStaging: {
    ttb_set_device(cudaDevice);
    if (owner && owner->open) {
      // Back to the device's cache; the next upload into it waits for the work queued so far.
      void *st = stream;
      if (ready) ttb_stream_wait_event(st, ready->event);
      if (pendingRead) ttb_stream_wait_event(st, pendingRead->event);
      StagingBlock blk;
      blk.ptr = ptr;
      blk.bytes = bytes;
      blk.lastUse = std::make_shared<EventHolder>(cudaDevice);
      ttb_event_record(blk.lastUse->event, st);
      std::lock_guard<std::mutex> g(owner->stagingMutex);
      if (localIndex < owner->stagingCache.size() && owner->stagingCache[localIndex].size() < 8) {
        owner->stagingCache[localIndex].push_back(std::move(blk));
        break;
      }
      ttb_free(ptr, st);
    } else {
      ttb_free(ptr, nullptr);
    }
    break;
  }
  case Kind::Borrowed: break;
  }
}

uint64_t TensorImpl::nextTensorVersion() {
  static std::atomic<uint64_t> latest{1};
  return latest.fetch_add(1, std::memory_order_relaxed);
}

TensorImpl::~TensorImpl() {
  for (auto &fn : onDestroy) {
    try {
      fn();
    } catch (...) {
    }
  }
  if (readyEvent) {
    ttb_event_destroy(readyEvent);
  }
}

ConstEvalCache &ConstEvalCache::get() {
  static ConstEvalCache *c = new ConstEvalCache(); // never destroyed: tensors may outlive static teardown
  return *c;
}

bool ConstEvalCache::find(const ConstEvalKey &key, std::vector<TensorPtr> &outputs) const {
  std::lock_guard<std::mutex> g(mutex);
  auto it = entries.find(key);
  if (it == entries.end()) {
    debug::Stats::get().incrementStat("ConstEvalCacheMiss");
    return false;
  }
  debug::Stats::get().incrementStat("ConstEvalCacheHit");
  outputs = it->second;
  return true;
}

void ConstEvalCache::store(const ConstEvalKey &key, const std::vector<TensorPtr> &inputs,
                           const std::vector<TensorPtr> &outputs) {
  {
    std::lock_guard<std::mutex> g(mutex);
    entries[key] = outputs;
  }
  for (const TensorPtr &in : inputs) {
    in->onDestroy.push_back([key] { ConstEvalCache::get().remove(key); });
  }
}

void ConstEvalCache::remove(const ConstEvalKey &key) {
  std::vector<TensorPtr> dying; // released after the lock: their own callbacks may come back here
  {
    std::lock_guard<std::mutex> g(mutex);
    auto it = entries.find(key);
    if (it == entries.end()) return;
    dying = std::move(it->second);
    entries.erase(it);
  }
}

void ConstEvalCache::removeDevice(const void *device) {
  std::vector<std::vector<TensorPtr>> dying;
  {
    std::lock_guard<std::mutex> g(mutex);
    for (auto it = entries.begin(); it != entries.end();) {
      if (it->first.device == device) {
        dying.push_back(std::move(it->second));
        it = entries.erase(it);
      } else {
        ++it;
      }
    }
  }
}

void ConstEvalCache::clear() {
  std::map<ConstEvalKey, std::vector<TensorPtr>> dying;
  {
    std::lock_guard<std::mutex> g(mutex);
    dying.swap(entries);
  }
}

size_t ConstEvalCache::size() const {
  std::lock_guard<std::mutex> g(mutex);
  return entries.size();
}

void DeviceImpl::releaseTraceGraph(uint32_t id) {
  auto it = traces.find(id);
  if (it == traces.end()) return;
  for (size_t i = 0; i < it->second.execs.size() && i < locals.size(); ++i) {
    if (it->second.execs[i]) {
      ttb_set_device(locals[i].cudaDevice);
      if (locals[i].stream) ttb_stream_sync(locals[i].stream); // a replay may still be running
      ttb_trace_destroy(it->second.execs[i]);
    }
  }
  traces.erase(it);
}

DeviceImpl::~DeviceImpl() { close(); }

void DeviceImpl::close() {
  if (!open) {
    return;
  }
  // Cached const-eval results and trace slots live in this device's memory.
  ConstEvalCache::get().removeDevice(this);
  traceCache.clear();
  while (!traces.empty()) releaseTraceGraph(traces.begin()->first);
  open = false;
  for (RankCtx &r : locals) {
    ttb_set_device(r.cudaDevice);
    for (void *st : {r.copyIn, r.copyOut, r.stream}) {
      if (st) ttb_stream_sync(st);
    }
    {
      std::lock_guard<std::mutex> g(stagingMutex);
      size_t idx = static_cast<size_t>(&r - locals.data());
      if (idx < stagingCache.size()) {
        for (StagingBlock &b : stagingCache[idx]) ttb_free(b.ptr, r.stream);
        stagingCache[idx].clear();
      }
      if (r.stream) ttb_stream_sync(r.stream);
    }
    if (r.symm) {
      ttb_symm_destroy(r.symm);
      r.symm = nullptr;
    }
    if (r.comm) {
      ttb_comm_destroy(r.comm);
      r.comm = nullptr;
    }
    for (void **st : {&r.copyIn, &r.copyOut, &r.stream}) {
      if (*st) {
        ttb_stream_destroy(*st);
        *st = nullptr;
      }
    }
  }
}

TensorPtr makeHostTensor(const std::vector<uint32_t> &shape, DataType dt, size_t nshards, bool pinned) {
  auto t = std::make_shared<TensorImpl>();
  t->shape = shape;
  t->stride = denseStrides(shape);
  t->dtype = dt;
  t->storage = Storage::Host;
  size_t bytes = t->bytes();
  for (size_t i = 0; i < nshards; ++i) {
    auto b = std::make_shared<Buffer>();
    b->bytes = bytes;
    if (pinned) {
      b->ptr = PinnedPool::get().take(bytes ? bytes : 16);
      b->bytes = bytes ? bytes : 16;
      b->kind = Buffer::Kind::HostPinnedPooled;
      t->shards.push_back(b);
      continue;
    }
    b->ptr = std::aligned_alloc(64, (bytes + 63) / 64 * 64 + 64);
    b->kind = Buffer::Kind::HostMalloc;
    if (!b->ptr) {
      TTRT_FATAL("out of host memory allocating ", bytes, " bytes");
    }
    t->shards.push_back(b);
  }
  return t;
}

TensorPtr makeDeviceTensor(const std::shared_ptr<DeviceImpl> &dev, const std::vector<uint32_t> &shape, DataType dt) {
  TTRT_ASSERT(dev && dev->open, "device is closed");
  TTRT_ASSERT(isSupportedDataType(dt), "data type ", dataTypeName(dt), " is not supported on device");
  auto t = std::make_shared<TensorImpl>();
  t->shape = shape;
  t->stride = denseStrides(shape);
  t->dtype = dt;
  t->storage = Storage::Device;
  t->layout = TensorLayout::Tile;
  t->device = dev;
  size_t bytes = t->bytes();
  for (const RankCtx &r : dev->locals) {
    auto b = std::make_shared<Buffer>();
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_malloc(&b->ptr, bytes, r.stream));
    b->bytes = bytes;
    b->cudaDevice = r.cudaDevice;
    b->stream = r.stream;
    b->owner = dev;
    b->kind = Buffer::Kind::Device;
    t->shards.push_back(b);
  }
  return t;
}

Tensor wrapTensor(const TensorPtr &t) {
  return Tensor(std::static_pointer_cast<void>(t), nullptr, DeviceRuntime::CUDA);
}

TensorPtr unwrapTensor(const Tensor &t) { return t.asSharedPtr<TensorImpl>(DeviceRuntime::CUDA); }

TensorPtr castOnDevice(const TensorPtr &t, DataType dt) {
  if (t->dtype == dt) {
    return t;
  }
  orderAfterUploads(t);
  auto out = makeDeviceTensor(t->device, t->shape, dt);
  out->layout = t->layout;
  for (size_t i = 0; i < t->shards.size(); ++i) {
    const RankCtx &r = t->device->locals[i];
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_typecast(t->shards[i]->ptr, ttbDtype(t->dtype), out->shards[i]->ptr, ttbDtype(dt), t->volume(),
                          r.stream));
  }
  return out;
}

// Host tensor -> device tensor.  A single-shard host tensor is replicated to every mesh
// coordinate; a multi-device host tensor supplies coordinate i from shard i.
TensorPtr toDevice(const TensorPtr &host, const std::shared_ptr<DeviceImpl> &dev, DataType dt) {
  TTRT_ASSERT(host->storage == Storage::Host, "toDevice expects a host tensor");
  TTRT_ASSERT(host->allocated(), "host tensor has no data");
  TTRT_ASSERT(host->shards.size() == 1 || host->shards.size() == dev->worldSize,
              "host tensor has ", host->shards.size(), " shards, mesh has ", dev->worldSize, " devices");
  // Page-locked sources are copied on the upload stream without stopping the host: the copy
  // overlaps whatever the compute stream is doing, and the tensor carries an event that the
  // first consumer on the compute stream waits for.  The caller keeps the source unchanged until
  // then (as with any asynchronous copy).  Pageable sources are copied before this returns.
  bool pinned = true;
  for (const RankCtx &r : dev->locals) {
    const BufferPtr &src = host->shards.size() == 1 ? host->shards[0] : host->shards[r.meshRank];
    TTRT_ASSERT(src && src->ptr, "host tensor has no shard for mesh coordinate ", r.meshRank);
    int isPinned = 0;
    TTB_CALL(ttb_host_is_pinned(src->ptr, &isPinned));
    pinned = pinned && isPinned != 0;
  }
  if (pinned) {
    auto staged = std::make_shared<TensorImpl>();
    staged->shape = host->shape;
    staged->stride = denseStrides(host->shape);
    staged->dtype = host->dtype;
    staged->storage = Storage::Device;
    staged->layout = TensorLayout::Tile;
    staged->device = dev;
    size_t bytes = staged->bytes();
    for (const RankCtx &r : dev->locals) {
      const BufferPtr &src = host->shards.size() == 1 ? host->shards[0] : host->shards[r.meshRank];
      auto b = std::make_shared<Buffer>();
      TTB_CALL(ttb_set_device(r.cudaDevice));
      size_t li = static_cast<size_t>(&r - dev->locals.data());
      {
        std::lock_guard<std::mutex> g(dev->stagingMutex);
        auto &cache = dev->stagingCache[li];
        for (size_t c = 0; c < cache.size(); ++c) {
          if (cache[c].bytes == bytes) {
            // Oldest matching block first: its last use is the most likely to be over.
            StagingBlock blk = std::move(cache[c]);
            cache.erase(cache.begin() + static_cast<long>(c));
            TTB_CALL(ttb_stream_wait_event(r.copyIn, blk.lastUse->event));
            b->ptr = blk.ptr;
            break;
          }
        }
      }
      // A new block is allocated in the upload stream's order, so that the copy does not wait for compute.
      if (!b->ptr) TTB_CALL(ttb_malloc(&b->ptr, bytes, r.copyIn));
      b->bytes = bytes;
      b->cudaDevice = r.cudaDevice;
      b->stream = r.stream; // released in compute order, after its consumers
      b->owner = dev;
      b->localIndex = li;
      b->kind = Buffer::Kind::DeviceStaging;
      TTB_CALL(ttb_memcpy_h2d(b->ptr, src->ptr, bytes, r.copyIn));
      b->ready = std::make_shared<EventHolder>(r.cudaDevice);
      TTB_CALL(ttb_event_record(b->ready->event, r.copyIn));
      b->keepAlive = src; // the source stays alive while the copy may still read it
      staged->shards.push_back(b);
    }
    return castOnDevice(staged, dt);
  }
  auto staged = makeDeviceTensor(dev, host->shape, host->dtype);
  for (size_t i = 0; i < dev->locals.size(); ++i) {
    const RankCtx &r = dev->locals[i];
    const BufferPtr &src = host->shards.size() == 1 ? host->shards[0] : host->shards[r.meshRank];
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_memcpy_h2d(staged->shards[i]->ptr, src->ptr, host->bytes(), r.stream));
  }
  // Pageable host memory may be reused by the caller as soon as this returns.
  for (const RankCtx &r : dev->locals) {
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_stream_sync(r.stream));
  }
  return castOnDevice(staged, dt);
}

void orderAfterUploads(const TensorPtr &t) {
  if (!t || t->storage != Storage::Device || !t->device) return;
  for (size_t i = 0; i < t->shards.size() && i < t->device->locals.size(); ++i) {
    const BufferPtr &b = t->shards[i];
    if (b && b->ready) {
      const RankCtx &r = t->device->locals[i];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_stream_wait_event(r.stream, b->ready->event));
      b->ready.reset(); // from here on the compute stream's order covers the upload
      b->keepAlive.reset();
    }
  }
}

TensorPtr toHostTensor(const TensorPtr &d, bool blocking) {
  TTRT_ASSERT(d->storage == Storage::Device, "toHost expects a device tensor");
  TTRT_ASSERT(d->allocated(), "device tensor was deallocated");
  orderAfterUploads(d);
  if (blocking) {
    auto h = makeHostTensor(d->shape, d->dtype, d->shards.size());
    h->layout = TensorLayout::RowMajor;
    for (size_t i = 0; i < d->shards.size(); ++i) {
      const RankCtx &r = d->device->locals[i];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_memcpy_d2h(h->shards[i]->ptr, d->shards[i]->ptr, d->bytes(), r.stream));
    }
    for (const RankCtx &r : d->device->locals) {
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_stream_sync(r.stream));
    }
    return h;
  }
  // Non-blocking: the download stream waits for the work enqueued so far on the compute stream,
  // then copies into page-locked memory while later submissions run.  wait(tensor) blocks on
  // the copy alone.
  auto h = makeHostTensor(d->shape, d->dtype, d->shards.size(), /*pinned=*/true);
  h->layout = TensorLayout::RowMajor;
  h->device = d->device;
  for (size_t i = 0; i < d->shards.size(); ++i) {
    const RankCtx &r = d->device->locals[i];
    TTB_CALL(ttb_set_device(r.cudaDevice));
    EventHolder produced(r.cudaDevice);
    TTB_CALL(ttb_event_record(produced.event, r.stream));
    TTB_CALL(ttb_stream_wait_event(r.copyOut, produced.event));
    TTB_CALL(ttb_memcpy_d2h(h->shards[i]->ptr, d->shards[i]->ptr, d->bytes(), r.copyOut));
    auto done = std::make_shared<EventHolder>(r.cudaDevice);
    TTB_CALL(ttb_event_record(done->event, r.copyOut));
    h->shards[i]->ready = done;
    h->shards[i]->keepAlive = d->shards[i]; // the source outlives the copy
    d->shards[i]->pendingRead = done;       // and is not reused before the copy has read it
  }
  return h;
}

} // namespace cuda

// ---- runtime selection -------------------------------------------------------------------
static DeviceRuntime g_currentRuntime = DeviceRuntime::CUDA;

std::vector<DeviceRuntime> getAvailableDeviceRuntimes() { return {DeviceRuntime::CUDA}; }
DeviceRuntime getCurrentDeviceRuntime() { return g_currentRuntime; }
void setCurrentDeviceRuntime(const DeviceRuntime &runtime) {
  if (runtime != DeviceRuntime::CUDA) {
    TTRT_FATAL("device runtime ", toString(runtime), " is not built into this library");
  }
  g_currentRuntime = runtime;
}
// The reference maps the file identifier to a runtime (runtime/lib/runtime.cpp:184-201);
// here "TTNN" binaries select the CUDA target.
void setCompatibleDeviceRuntime(const Binary &binary) {
  if (binary.getFileIdentifier() != "TTNN") {
    TTRT_FATAL("no device runtime for flatbuffer identifier ", binary.getFileIdentifier());
  }
  g_currentRuntime = DeviceRuntime::CUDA;
}
std::vector<HostRuntime> getAvailableHostRuntimes() { return {HostRuntime::Local}; }
HostRuntime getCurrentHostRuntime() { return HostRuntime::Local; }
void setCurrentHostRuntime(const HostRuntime &runtime) {
  if (runtime != HostRuntime::Local) {
    TTRT_FATAL("only the local host runtime exists in this target");
  }
}
void setMlirHome(std::string_view) {}
void setMetalHome(std::string_view) {}
void setMemoryLogLevel(const MemoryLogLevel &) {}
void setFabricConfig(FabricConfig) {}
tt::target::Arch getArch() { return tt::target::Arch::Blackhole; }

size_t getNumAvailableDevices() {
  int n = 0;
  TTB_CALL(ttb_device_count(&n));
  return static_cast<size_t>(n);
}

std::string getNcclUniqueId() {
  std::string id(128, '\0');
  TTB_CALL(ttb_nccl_unique_id(id.data()));
  return id;
}

// ---- devices -----------------------------------------------------------------------------
Device openMeshDevice(const MeshDeviceOptions &options) {
  std::vector<uint32_t> mesh = options.meshShape.value_or(std::vector<uint32_t>{1, 1});
  TTRT_ASSERT(mesh.size() == 2, "mesh shape must have two entries");
  uint32_t world = mesh[0] * mesh[1];
  TTRT_ASSERT(world >= 1, "empty mesh");
  TTRT_ASSERT(mesh[0] == 1 || mesh[1] == 1, "only 1xN and Nx1 meshes are supported, got ", mesh[0], "x", mesh[1]);
  auto dev = std::make_shared<DeviceImpl>();
  dev->meshShape = mesh;
  dev->worldSize = world;
  size_t avail = getNumAvailableDevices();
  TTRT_ASSERT(avail > 0, "no CUDA device is visible");
  if (options.processCount > 1) {
    TTRT_ASSERT(options.processCount == world, "processCount ", options.processCount, " != mesh volume ", world);
    TTRT_ASSERT(options.processRank < world, "processRank out of range");
    TTRT_ASSERT(options.ncclUniqueId.size() == 128, "ncclUniqueId must be 128 bytes");
    dev->multiProcess = true;
    RankCtx r;
    r.cudaDevice = options.deviceIds.empty() ? 0 : options.deviceIds[0];
    r.meshRank = options.processRank;
    dev->locals.push_back(r);
  } else {
    TTRT_ASSERT(options.deviceIds.empty() || options.deviceIds.size() == world,
                "deviceIds must name one CUDA device per mesh coordinate");
    for (uint32_t i = 0; i < world; ++i) {
      RankCtx r;
      r.cudaDevice = options.deviceIds.empty() ? static_cast<int>(i) : options.deviceIds[i];
      r.meshRank = i;
      TTRT_ASSERT(static_cast<size_t>(r.cudaDevice) < avail, "mesh needs CUDA device ", r.cudaDevice, " but only ",
                  avail, " are visible");
      dev->locals.push_back(r);
    }
  }
  dev->open = true;
  for (RankCtx &r : dev->locals) {
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_stream_create(&r.stream));
    TTB_CALL(ttb_stream_create(&r.copyIn));
    TTB_CALL(ttb_stream_create(&r.copyOut));
  }
  dev->stagingCache.resize(dev->locals.size());
  if (world > 1) {
    if (dev->multiProcess) {
      RankCtx &r = dev->locals[0];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_comm_init_rank(&r.comm, static_cast<int>(world), options.ncclUniqueId.data(),
                                  static_cast<int>(r.meshRank)));
    } else {
      std::vector<void *> comms(world);
      std::vector<int> ids;
      for (const RankCtx &r : dev->locals) ids.push_back(r.cudaDevice);
      TTB_CALL(ttb_comm_init_all(comms.data(), static_cast<int>(world), ids.data()));
      for (uint32_t i = 0; i < world; ++i) dev->locals[i].comm = comms[i];
    }
  }
  return Device(std::static_pointer_cast<void>(dev), DeviceRuntime::CUDA);
}

static std::shared_ptr<DeviceImpl> deviceImpl(const Device &d) { return d.asSharedPtr<DeviceImpl>(DeviceRuntime::CUDA); }

void closeMeshDevice(Device parentMesh) { deviceImpl(parentMesh)->close(); }

Device createSubMeshDevice(Device parentMesh, const std::vector<uint32_t> &meshShape,
                           const std::optional<const std::vector<uint32_t>> &meshOffset) {
  // A sub-mesh is its own set of streams over a slice of the parent's devices, so that
  // several threads can submit to disjoint sub-meshes concurrently
  // (runtime/test/ttnn/python/n300/test_data_parallel.py:25-37).
  auto parent = deviceImpl(parentMesh);
  TTRT_ASSERT(!parent->multiProcess, "sub-meshes need all devices in one process");
  TTRT_ASSERT(meshShape.size() == 2, "mesh shape must have two entries");
  uint32_t vol = meshShape[0] * meshShape[1];
  uint32_t off = 0;
  if (meshOffset) {
    TTRT_ASSERT(meshOffset->size() == 2, "mesh offset must have two entries");
    off = (*meshOffset)[0] * parent->meshShape[1] + (*meshOffset)[1];
  }
  TTRT_ASSERT(off + vol <= parent->worldSize, "sub-mesh exceeds the parent mesh");
  MeshDeviceOptions o;
  o.meshShape = meshShape;
  for (uint32_t i = 0; i < vol; ++i) o.deviceIds.push_back(parent->locals[off + i].cudaDevice);
  return openMeshDevice(o);
}

void releaseSubMeshDevice(Device subMesh) { deviceImpl(subMesh)->close(); }

void reshapeMeshDevice(Device meshDevice, const std::vector<uint32_t> &meshShape) {
  auto d = deviceImpl(meshDevice);
  TTRT_ASSERT(meshShape.size() == 2 && meshShape[0] * meshShape[1] == d->worldSize, "reshape must keep the volume");
  d->meshShape = meshShape;
}

std::vector<uint32_t> getMeshShape(Device meshDevice) { return deviceImpl(meshDevice)->meshShape; }
std::vector<int> getDeviceIds(Device meshDevice) {
  std::vector<int> ids;
  for (const RankCtx &r : deviceImpl(meshDevice)->locals) ids.push_back(r.cudaDevice);
  return ids;
}
size_t getNumHwCqs(Device) { return 1; }
bool isProgramCacheEnabled(Device) { return true; }
void clearProgramCache(Device) {}
size_t getL1SmallSize(Device) { return 0; }
size_t getTraceRegionSize(Device) { return 0; }
void releaseTrace(Device meshDevice, std::uint64_t binaryId, size_t mainProgramId) {
  auto d = deviceImpl(meshDevice);
  std::lock_guard<std::mutex> g(d->submitMutex);
  for (auto it = d->traceCache.begin(); it != d->traceCache.end();) {
    if (std::get<0>(it->first) == binaryId && std::get<1>(it->first) == mainProgramId) {
      d->releaseTraceGraph(it->second.traceId);
      it = d->traceCache.erase(it);
    } else {
      ++it;
    }
  }
}
size_t getNumDramChannels(Device) { return 1; }
size_t getDramSizePerChannel(Device meshDevice) {
  size_t total = 0;
  auto d = deviceImpl(meshDevice);
  TTB_CALL(ttb_device_info(d->locals.at(0).cudaDevice, nullptr, &total, nullptr, nullptr));
  return total;
}
size_t getL1SizePerCore(Device) { return 227 * 1024; } // shared memory per SM
void deallocateBuffers(Device) {}
void dumpMemoryReport(Device) {}
void readDeviceProfilerResults(Device) {}

// A descriptor of the machine in the reference's wire format ("TTSY", Common/system_desc.fbs), so
// that callers which fetch, print, store or compare system descriptors keep working (`ttrt query`,
// tools/ttrt/common/util.py:868-912).  The schema describes Tenstorrent chips, so the GPU is put in
// its terms: one ChipDesc per visible GPU (or per device of `meshDevice`), the SMs as a y x x worker
// grid (2 dies of SMs / 2 on B200), shared memory per SM as the L1 size, HBM as ONE DRAM channel of the
// device's total memory, 32 x 32 tiles, the data types this runtime computes in.  The `arch` field is an
// enum of Tenstorrent architectures with no spare value; Blackhole is written and the product
// identifier says what the device really is.  A binary compiled for Tenstorrent silicon carries a
// different descriptor: callers must skip the comparison for this target (ttrt: --ignore-system-desc).
SystemDesc getCurrentSystemDesc(std::optional<DispatchCoreType>, std::optional<Device> meshDevice) {
  std::vector<int> ordinals;
  if (meshDevice) {
    ordinals = getDeviceIds(*meshDevice);
  } else {
    int n = 0;
    TTB_CALL(ttb_device_count(&n));
    for (int i = 0; i < n; ++i) ordinals.push_back(i);
  }
  // A machine without a visible GPU gets a descriptor with no chips.
  fb::Writer w;
  struct Dim2d { int32_t y, x; };
  struct ChipCoord { uint32_t rack, shelf, y, x; };
  std::vector<uint32_t> chipDescs, indices, capabilities;
  std::vector<ChipCoord> coords;
  std::string product = "NVIDIA-CUDA";
  for (size_t i = 0; i < ordinals.size(); ++i) {
    int sms = 0, major = 0, minor = 0;
    size_t total = 0;
    TTB_CALL(ttb_device_info(ordinals[i], &sms, &total, &major, &minor));
    if (i == 0) product = "NVIDIA-CUDA-sm_" + std::to_string(major) + std::to_string(minor) + "-" + std::to_string(sms) + "SM";
    const std::vector<uint16_t> dtypes = {
        static_cast<uint16_t>(DataType::Float32), static_cast<uint16_t>(DataType::Float16), static_cast<uint16_t>(DataType::BFloat16),
        static_cast<uint16_t>(DataType::UInt32),  static_cast<uint16_t>(DataType::UInt16),  static_cast<uint16_t>(DataType::UInt8),
        static_cast<uint16_t>(DataType::Int32),   static_cast<uint16_t>(DataType::Int8)};
    const uint32_t dtypeVec = w.createScalarVector(dtypes);
    const Dim2d tile{32, 32};
    const uint32_t tileVec = w.createStructVector(&tile, 1, sizeof(Dim2d), 4);
    const Dim2d bank{0, 0};
    const uint32_t bank0 = w.createStructVector(&bank, 1, sizeof(Dim2d), 4);
    const uint32_t bank1 = w.createStructVector(&bank, 1, sizeof(Dim2d), 4);
    const Dim2d grid{sms % 2 == 0 ? 2 : 1, sms % 2 == 0 ? sms / 2 : sms}, zero{0, 0}, dramGrid{1, 1};
    w.startTable(22);
    w.addScalar<uint32_t>(0, 1 /* Arch::Blackhole: see above */, 0);
    w.addStruct(1, &grid, sizeof(grid), 4);
    w.addStruct(2, &zero, sizeof(zero), 4);
    w.addScalar<uint64_t>(3, 227 * 1024);                 // shared memory per SM
    w.addScalar<uint32_t>(4, 1);                          // HBM as one DRAM channel
    w.addScalar<uint64_t>(5, static_cast<uint64_t>(total));
    w.addScalar<uint32_t>(6, 16);                         // alignment of bulk (TMA) copies
    w.addScalar<uint32_t>(7, 64);
    w.addScalar<uint32_t>(8, 256);                        // allocation granularity of the memory pool
    w.addOffset(13, dtypeVec);
    w.addOffset(14, tileVec);
    w.addScalar<uint32_t>(15, 512);                       // tensor-memory columns per SM
    w.addScalar<uint32_t>(16, 0);
    w.addScalar<uint32_t>(17, 4);                         // warp schedulers per SM
    w.addScalar<uint32_t>(18, 1);
    w.addStruct(19, &dramGrid, sizeof(dramGrid), 4);
    w.addOffset(20, bank0);
    w.addOffset(21, bank1);
    chipDescs.push_back(w.endTable());
    indices.push_back(static_cast<uint32_t>(i));
    capabilities.push_back(1);                            // HostMMIO: every GPU is reachable from the host
    coords.push_back(ChipCoord{0, 0, 0, static_cast<uint32_t>(i)});
  }
  const uint32_t triple = w.createString("x86_64-pc-linux-gnu");
  w.startTable(2);
  w.addScalar<uint8_t>(0, 0);                             // CPURole::Host
  w.addOffset(1, triple);
  const uint32_t cpu = w.endTable();
  const uint32_t cpuVec = w.createOffsetVector({cpu});
  const uint32_t chipVec = w.createOffsetVector(chipDescs);
  const uint32_t idxVec = w.createScalarVector(indices);
  const uint32_t capVec = w.createScalarVector(capabilities);
  const uint32_t coordVec = w.createStructVector(coords.data(), coords.size(), sizeof(ChipCoord), 4);
  w.startTable(6);
  w.addOffset(0, cpuVec);
  w.addOffset(1, chipVec);
  w.addOffset(2, idxVec);
  w.addOffset(3, capVec);
  w.addOffset(4, coordVec);
  const uint32_t desc = w.endTable();
  const uint32_t hash = w.createString(schemaHashString());
  const uint32_t git = w.createString("b200-runtime");
  const uint32_t prod = w.createString(product);
  struct Version { uint16_t major, minor; uint32_t patch; } version{0, 1, 0};
  w.startTable(5);
  w.addStruct(0, &version, sizeof(version), 4);
  w.addOffset(1, hash);
  w.addOffset(2, git);
  w.addOffset(3, prod);
  w.addOffset(4, desc);
  const uint32_t root = w.endTable();
  std::vector<uint8_t> bytes = w.finish(root, "TTSY");
  return SystemDesc(Flatbuffer::loadFromMemory(bytes.data(), bytes.size()).handle);
}

// ---- host tensors ------------------------------------------------------------------------
static void checkHostArgs(const std::vector<std::uint32_t> &shape, const std::vector<std::int64_t> &stride,
                          std::uint32_t itemsize, DataType dt) {
  TTRT_ASSERT(shape.size() == stride.size(), "shape and stride rank differ");
  TTRT_ASSERT(itemsize > 0, "itemsize must be positive");
  uint32_t es = dataTypeSize(dt);
  TTRT_ASSERT(es == itemsize, "itemsize ", itemsize, " does not match data type ", dataTypeName(dt));
}

static bool isDense(const std::vector<std::uint32_t> &shape, const std::vector<std::int64_t> &stride) {
  int64_t acc = 1;
  for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) {
    if (shape[i] != 1 && stride[i] != acc) {
      return false;
    }
    acc *= shape[i];
  }
  return true;
}

Tensor createBorrowedHostTensor(void *data, const std::vector<std::uint32_t> &shape,
                                const std::vector<std::int64_t> &stride, std::uint32_t itemsize, DataType dataType) {
  checkHostArgs(shape, stride, itemsize, dataType);
  size_t vol = 1;
  for (uint32_t d : shape) vol *= d;
  TTRT_ASSERT(data != nullptr || vol == 0, "cannot borrow null data");
  // Same restriction as the reference (runtime/lib/ttnn/runtime.cpp:250-256).
  TTRT_ASSERT(isDense(shape, stride), "borrowed host tensors must be contiguous row-major");
  auto t = std::make_shared<TensorImpl>();
  t->shape = shape;
  t->stride = denseStrides(shape);
  t->dtype = dataType;
  t->storage = Storage::Host;
  static char emptyPlaceholder[16];
  auto b = std::make_shared<Buffer>();
  b->ptr = data ? data : emptyPlaceholder; // empty tensors may come with a null pointer
  b->bytes = t->bytes();
  b->kind = Buffer::Kind::Borrowed;
  t->shards.push_back(b);
  return wrapTensor(t);
}

// Owned tensors copy; strided input is gathered element by element (reference :68-103).
static void gatherStrided(uint8_t *dst, const uint8_t *src, const std::vector<std::uint32_t> &shape,
                          const std::vector<std::int64_t> &stride, uint32_t es) {
  size_t n = 1;
  for (uint32_t d : shape) n *= d;
  std::vector<uint32_t> idx(shape.size(), 0);
  for (size_t i = 0; i < n; ++i) {
    int64_t off = 0;
    for (size_t k = 0; k < shape.size(); ++k) off += static_cast<int64_t>(idx[k]) * stride[k];
    std::memcpy(dst + i * es, src + off * es, es);
    for (int k = static_cast<int>(shape.size()) - 1; k >= 0; --k) {
      if (++idx[k] < shape[k]) break;
      idx[k] = 0;
    }
  }
}

Tensor createOwnedHostTensor(const void *data, const std::vector<std::uint32_t> &shape,
                             const std::vector<std::int64_t> &stride, std::uint32_t itemsize, DataType dataType) {
  checkHostArgs(shape, stride, itemsize, dataType);
  auto t = makeHostTensor(shape, dataType, 1);
  if (data && t->bytes()) {
    if (isDense(shape, stride)) {
      std::memcpy(t->shards[0]->ptr, data, t->bytes());
    } else {
      gatherStrided(static_cast<uint8_t *>(t->shards[0]->ptr), static_cast<const uint8_t *>(data), shape, stride,
                    itemsize);
    }
  }
  return wrapTensor(t);
}

Tensor createMultiDeviceHostTensor(const std::vector<const void *> &data, const std::vector<std::uint32_t> &shape,
                                   const std::vector<std::int64_t> &stride, std::uint32_t itemsize, DataType dataType,
                                   const std::unordered_map<std::string, std::string> &,
                                   const std::vector<uint32_t> &meshShape) {
  checkHostArgs(shape, stride, itemsize, dataType);
  size_t vol = 1;
  for (uint32_t m : meshShape) vol *= m;
  TTRT_ASSERT(data.size() == vol, "need one data pointer per mesh coordinate");
  auto t = makeHostTensor(shape, dataType, vol);
  for (size_t i = 0; i < vol; ++i) {
    if (isDense(shape, stride)) {
      std::memcpy(t->shards[i]->ptr, data[i], t->bytes());
    } else {
      gatherStrided(static_cast<uint8_t *>(t->shards[i]->ptr), static_cast<const uint8_t *>(data[i]), shape, stride,
                    itemsize);
    }
  }
  return wrapTensor(t);
}

Tensor createMultiDeviceHostTensor(const std::vector<Tensor> &tensorShards,
                                   const std::unordered_map<std::string, std::string> &,
                                   const std::vector<uint32_t> &meshShape) {
  size_t vol = 1;
  for (uint32_t m : meshShape) vol *= m;
  TTRT_ASSERT(tensorShards.size() == vol && vol > 0, "need one shard per mesh coordinate");
  auto first = unwrapTensor(tensorShards[0]);
  auto t = std::make_shared<TensorImpl>();
  t->shape = first->shape;
  t->stride = first->stride;
  t->dtype = first->dtype;
  t->storage = Storage::Host;
  for (const Tensor &s : tensorShards) {
    auto impl = unwrapTensor(s);
    TTRT_ASSERT(impl->storage == Storage::Host && impl->shards.size() == 1, "shards must be single host tensors");
    TTRT_ASSERT(impl->shape == first->shape && impl->dtype == first->dtype, "shards must agree in shape and type");
    t->shards.push_back(impl->shards[0]);
  }
  return wrapTensor(t);
}

Tensor createMultiDeviceBorrowedHostTensor(std::vector<void *> &data, const std::vector<std::uint32_t> &shape,
                                           const std::vector<std::int64_t> &stride, std::uint32_t itemsize,
                                           DataType dataType,
                                           const std::unordered_map<std::string, std::string> &strategy,
                                           const std::vector<uint32_t> &meshShape) {
  std::vector<Tensor> shards;
  for (void *p : data) shards.push_back(createBorrowedHostTensor(p, shape, stride, itemsize, dataType));
  return createMultiDeviceHostTensor(shards, strategy, meshShape);
}

Tensor createEmptyTensor(Device device, Layout layout, const std::vector<std::uint32_t> &shape,
                         const std::vector<std::int64_t> &, std::uint32_t) {
  const auto &l = layout.as<LayoutImpl>(DeviceRuntime::CUDA);
  if (l.storage == Storage::Host) {
    return wrapTensor(makeHostTensor(shape, l.dtype, 1));
  }
  return wrapTensor(makeDeviceTensor(deviceImpl(device), shape, l.dtype));
}

// ---- tensor queries ------------------------------------------------------------------------
bool isTensorAllocated(Tensor tensor) { return unwrapTensor(tensor)->allocated(); }
DataType getTensorDataType(Tensor tensor) { return unwrapTensor(tensor)->dtype; }
std::uint32_t getTensorElementSize(Tensor tensor) { return dataTypeSize(unwrapTensor(tensor)->dtype); }
std::uint32_t getTensorVolume(Tensor tensor) { return static_cast<uint32_t>(unwrapTensor(tensor)->volume()); }
std::uint32_t getTensorLogicalVolume(Tensor tensor) { return getTensorVolume(tensor); }
std::vector<std::uint32_t> getTensorShape(Tensor tensor) { return unwrapTensor(tensor)->shape; }
std::vector<std::int64_t> getTensorStride(Tensor tensor) { return unwrapTensor(tensor)->stride; }
TensorDesc getTensorDesc(Tensor tensor) {
  auto t = unwrapTensor(tensor);
  return TensorDesc(t->shape, t->dtype, t->stride);
}
bool getTensorRetain(Tensor tensor) { return unwrapTensor(tensor)->retain; }
void setTensorRetain(Tensor tensor, bool retain) { unwrapTensor(tensor)->retain = retain; }
uint32_t detail::getNumShards(Tensor tensor) { return static_cast<uint32_t>(unwrapTensor(tensor)->shards.size()); }

std::vector<std::byte> getTensorDataBuffer(Tensor tensor) {
  auto t = unwrapTensor(tensor);
  TensorPtr h = t->storage == Storage::Device ? toHostTensor(t, true) : t;
  TTRT_ASSERT(h->allocated(), "tensor has no data");
  std::vector<std::byte> out(h->bytes());
  std::memcpy(out.data(), h->shards[0]->ptr, out.size());
  return out;
}

// ---- sync ----------------------------------------------------------------------------------
static void syncDevice(const std::shared_ptr<DeviceImpl> &d) {
  if (!d || !d->open) {
    return;
  }
  for (const RankCtx &r : d->locals) {
    TTB_CALL(ttb_set_device(r.cudaDevice));
    for (void *st : {r.copyIn, r.stream, r.copyOut}) {
      if (st) TTB_CALL(ttb_stream_sync(st));
    }
    if (d->ranEmbedding) {
      int bad = 0;
      TTB_CALL(ttb_embedding_status(&bad));
      TTRT_ASSERT(bad == 0, "an embedding lookup saw an index outside its table (row 0 was used instead)");
    }
    if (d->ranIndexOp) {
      int bad = 0;
      TTB_CALL(ttb_index_status(&bad));
      TTRT_ASSERT(bad == 0, "a gather / scatter saw an index outside its dimension (the element was skipped)");
    }
    if (d->ranUpdateCache) {
      int bad = 0;
      TTB_CALL(ttb_update_cache_status(&bad));
      TTRT_ASSERT(bad == 0, "an update_cache position was outside the cache (nothing was written)");
    }
    if (r.symm) {
      int status = 0;
      TTB_CALL(ttb_symm_status(r.symm, &status));
      if (status != 0) {
        // Reported once: the word is cleared so that the collectives after this one are judged on their own.
        TTB_CALL(ttb_symm_clear_status(r.symm));
        TTRT_FATAL("a peer-memory all-reduce gave up waiting for rank ", (status & 0xff) - 1, " in phase ", status >> 8,
                   "; results since that launch are invalid");
      }
    }
    // The tensor-core kernels (GEMM, convolution, attention) bound every wait; one that ran out left
    // output tiles unwritten.  Reported once per timeout (the words are cleared on reading).
    int gemmStatus = 0, sdpaStatus = 0;
    TTB_CALL(ttb_tcgen05_status(&gemmStatus, &sdpaStatus, /*clear=*/1));
    TTRT_ASSERT(gemmStatus == 0, "a tensor-core GEMM / convolution launch gave up waiting (role ", gemmStatus >> 8,
                ": 1 loader, 2-3 MMA issuer, 4-5 epilogue); its output is incomplete");
    TTRT_ASSERT(sdpaStatus == 0, "a tensor-core attention launch gave up waiting (site ", sdpaStatus >> 8,
                "); its output is incomplete");
  }
}

void wait(Event) { TTRT_FATAL("wait(Event) is not supported; wait on tensors (as in the reference TTNN target)"); }
void wait(Tensor tensor, std::optional<uint8_t>) {
  auto t = unwrapTensor(tensor);
  if (t->storage == Storage::Host) {
    // The result of a non-blocking toHost: wait for its copy only.
    bool pending = false;
    for (const BufferPtr &b : t->shards) {
      if (b && b->ready) {
        TTB_CALL(ttb_event_sync(b->ready->event));
        b->ready.reset();
        b->keepAlive.reset();
        pending = true;
      }
    }
    if (pending || !t->device) return;
  }
  syncDevice(t->device);
}
void wait(const std::vector<Tensor> &tensors, std::optional<uint8_t> cqId) {
  for (const Tensor &t : tensors) wait(t, cqId);
}

// ---- layouts / movement ----------------------------------------------------------------------
static Layout makeLayout(const LayoutImpl &l) {
  return Layout(std::static_pointer_cast<void>(std::make_shared<LayoutImpl>(l)), DeviceRuntime::CUDA);
}

Layout getLayout(Binary executableHandle, std::uint32_t programIndex, std::uint32_t inputIndex) {
  const auto *programs = executableHandle.get()->programs();
  TTRT_ASSERT(programs && programIndex < programs->size(), "program index out of range");
  const auto *inputs = programs->Get(programIndex)->inputs();
  TTRT_ASSERT(inputs && inputIndex < inputs->size(), "input index out of range");
  const auto *desc = inputs->Get(inputIndex)->desc();
  TTRT_ASSERT(desc && desc->layout() && desc->layout()->memory_desc(), "program input has no layout");
  const auto *md = desc->layout()->memory_desc();
  LayoutImpl l;
  l.storage = md->storage_type() == fbt::StorageType::Device ? Storage::Device : Storage::Host;
  // Tile shape 32x32 means TILE, 1x1 ROW_MAJOR (runtime/lib/ttnn/utils/utils.cpp:57-60); on the
  // GPU both are the same dense row-major memory and the tag is only carried along.
  const auto *ts = md->tile_shape();
  l.layout = (ts && ts->y() == 32 && ts->x() == 32) ? TensorLayout::Tile : TensorLayout::RowMajor;
  l.dtype = md->data_type();
  return makeLayout(l);
}

Layout getTensorLayout(Tensor tensor) {
  auto t = unwrapTensor(tensor);
  LayoutImpl l;
  l.storage = t->storage;
  l.layout = t->layout;
  l.dtype = t->dtype;
  return makeLayout(l);
}

bool hasLayout(Tensor tensor, Layout layout) {
  auto t = unwrapTensor(tensor);
  const auto &l = layout.as<LayoutImpl>(DeviceRuntime::CUDA);
  return t->storage == l.storage && t->layout == l.layout && t->dtype == l.dtype;
}

// Host-side dtype conversion for host -> host layout changes (rare; small tensors).
static TensorPtr castOnHost(const TensorPtr &t, DataType dt);

Tensor toLayout(Tensor tensor, Device device, Layout layout, std::optional<bool> retain) {
  auto t = unwrapTensor(tensor);
  const auto &l = layout.as<LayoutImpl>(DeviceRuntime::CUDA);
  auto dev = deviceImpl(device);
  TensorPtr out;
  if (l.storage == Storage::Device) {
    if (t->storage == Storage::Host) {
      out = toDevice(t, dev, l.dtype);
    } else {
      out = castOnDevice(t, l.dtype);
    }
  } else {
    if (t->storage == Storage::Device) {
      out = toHostTensor(castOnDevice(t, l.dtype), true);
    } else {
      out = castOnHost(t, l.dtype);
    }
  }
  if (out == t) {
    // Same storage and dtype: hand back a new handle onto the same buffers.
    auto alias = std::make_shared<TensorImpl>();
    alias->shape = t->shape;
    alias->stride = t->stride;
    alias->dtype = t->dtype;
    alias->storage = t->storage;
    alias->shards = t->shards;
    alias->device = t->device;
    out = alias;
  }
  out->layout = l.layout;
  out->retain = retain.value_or(false);
  // The source is released unless the caller asked to keep it (reference :929-931).
  if (!t->retain && t->storage == Storage::Device && out->shards != t->shards) {
    t->shards.clear();
  }
  return wrapTensor(out);
}

std::vector<Tensor> toHost(Tensor tensor, bool, bool blocking) {
  auto t = unwrapTensor(tensor);
  std::vector<Tensor> out;
  if (t->storage == Storage::Host) {
    out.push_back(tensor);
    return out;
  }
  auto h = toHostTensor(t, blocking);
  // One host tensor per shard, as the reference returns (:861-884).
  for (size_t i = 0; i < h->shards.size(); ++i) {
    auto s = std::make_shared<TensorImpl>();
    s->shape = h->shape;
    s->stride = h->stride;
    s->dtype = h->dtype;
    s->storage = Storage::Host;
    s->shards.push_back(h->shards[i]);
    s->device = h->device;
    out.push_back(wrapTensor(s));
  }
  return out;
}

std::vector<Tensor> getDeviceTensors(Tensor tensor) {
  auto t = unwrapTensor(tensor);
  std::vector<Tensor> out;
  for (size_t i = 0; i < t->shards.size(); ++i) {
    auto s = std::make_shared<TensorImpl>();
    s->shape = t->shape;
    s->stride = t->stride;
    s->dtype = t->dtype;
    s->storage = t->storage;
    s->layout = t->layout;
    s->shards.push_back(t->shards[i]);
    out.push_back(wrapTensor(s));
  }
  return out;
}

// Element conversions on the host for memcpy(void*, Tensor, dtype) and host layout changes.
static double loadAsDouble(const void *p, DataType dt, size_t i) {
  switch (dt) {
  case DataType::Float32: return static_cast<const float *>(p)[i];
  case DataType::BFloat16: {
    uint32_t bits = static_cast<uint32_t>(static_cast<const uint16_t *>(p)[i]) << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
  }
  case DataType::UInt32: return static_cast<const uint32_t *>(p)[i];
  case DataType::Int32: return static_cast<const int32_t *>(p)[i];
  case DataType::UInt16: return static_cast<const uint16_t *>(p)[i];
  case DataType::UInt8: return static_cast<const uint8_t *>(p)[i];
  case DataType::Int8: return static_cast<const int8_t *>(p)[i];
  default: TTRT_FATAL("host conversion from ", dataTypeName(dt), " is not supported");
  }
}

static void storeFromDouble(void *p, DataType dt, size_t i, double v) {
  switch (dt) {
  case DataType::Float32: static_cast<float *>(p)[i] = static_cast<float>(v); break;
  case DataType::BFloat16: {
    float f = static_cast<float>(v);
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) {
      bits |= 0x00400000u; // quiet NaN
    } else {
      bits += 0x7fffu + ((bits >> 16) & 1u); // round to nearest even
    }
    static_cast<uint16_t *>(p)[i] = static_cast<uint16_t>(bits >> 16);
    break;
  }
  case DataType::UInt32: static_cast<uint32_t *>(p)[i] = static_cast<uint32_t>(static_cast<int64_t>(v)); break;
  case DataType::Int32: static_cast<int32_t *>(p)[i] = static_cast<int32_t>(static_cast<int64_t>(v)); break;
  case DataType::UInt16: static_cast<uint16_t *>(p)[i] = static_cast<uint16_t>(static_cast<int64_t>(v)); break;
  case DataType::UInt8: static_cast<uint8_t *>(p)[i] = static_cast<uint8_t>(static_cast<int64_t>(v)); break;
  case DataType::Int8: static_cast<int8_t *>(p)[i] = static_cast<int8_t>(static_cast<int64_t>(v)); break;
  default: TTRT_FATAL("host conversion to ", dataTypeName(dt), " is not supported");
  }
}

static TensorPtr castOnHost(const TensorPtr &t, DataType dt) {
  if (t->dtype == dt) {
    return t;
  }
  auto out = makeHostTensor(t->shape, dt, t->shards.size());
  for (size_t s = 0; s < t->shards.size(); ++s) {
    for (size_t i = 0; i < t->volume(); ++i) {
      storeFromDouble(out->shards[s]->ptr, dt, i, loadAsDouble(t->shards[s]->ptr, t->dtype, i));
    }
  }
  return out;
}

void memcpy(void *dst, Tensor src, std::optional<DataType> targetDataType) {
  TTRT_ASSERT(dst != nullptr, "null destination");
  auto t = unwrapTensor(src);
  TTRT_ASSERT(t->allocated(), "tensor has no data");
  if (t->storage == Storage::Device && (!targetDataType || *targetDataType == t->dtype)) {
    // straight into the caller's buffer (a true DMA when that buffer is pinned)
    orderAfterUploads(t);
    const RankCtx &r = t->device->locals[0];
    TTB_CALL(ttb_set_device(r.cudaDevice));
    TTB_CALL(ttb_memcpy_d2h(dst, t->shards[0]->ptr, t->bytes(), r.stream));
    TTB_CALL(ttb_stream_sync(r.stream));
    return;
  }
  TensorPtr h = t->storage == Storage::Device ? toHostTensor(t, true) : t;
  if (!targetDataType || *targetDataType == h->dtype) {
    std::memcpy(dst, h->shards[0]->ptr, h->bytes());
    return;
  }
  for (size_t i = 0; i < h->volume(); ++i) {
    storeFromDouble(dst, *targetDataType, i, loadAsDouble(h->shards[0]->ptr, h->dtype, i));
  }
}

void memcpy(Tensor dst, Tensor src) {
  auto d = unwrapTensor(dst);
  auto s = unwrapTensor(src);
  TTRT_ASSERT(d->allocated() && s->allocated(), "tensor has no data");
  TTRT_ASSERT(d->volume() == s->volume() && d->dtype == s->dtype, "memcpy needs equal size and data type");
  TTRT_ASSERT(d->shards.size() == s->shards.size(), "memcpy needs equal shard counts");
  orderAfterUploads(d);
  orderAfterUploads(s);
  for (size_t i = 0; i < d->shards.size(); ++i) {
    void *dp = d->shards[i]->ptr;
    const void *sp = s->shards[i]->ptr;
    if (d->storage == Storage::Host && s->storage == Storage::Host) {
      std::memcpy(dp, sp, d->bytes());
    } else if (d->storage == Storage::Host) {
      const RankCtx &r = s->device->locals[i];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_memcpy_d2h(dp, sp, d->bytes(), r.stream));
      TTB_CALL(ttb_stream_sync(r.stream));
    } else if (s->storage == Storage::Host) {
      const RankCtx &r = d->device->locals[i];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_memcpy_h2d(dp, sp, d->bytes(), r.stream));
      TTB_CALL(ttb_stream_sync(r.stream));
    } else {
      const RankCtx &r = d->device->locals[i];
      TTB_CALL(ttb_set_device(r.cudaDevice));
      TTB_CALL(ttb_memcpy_d2d(dp, sp, d->bytes(), r.stream));
    }
  }
  d->version.store(TensorImpl::nextTensorVersion());
  if (d->base) d->base->version.store(d->version.load());
}

void deallocateTensor(Tensor &tensor, bool force) {
  auto t = unwrapTensor(tensor);
  if (t->retain && !force) {
    return;
  }
  if (!t->shards.empty() && t->shards[0] && t->shards[0]->kind == Buffer::Kind::Borrowed) {
    return; // borrowed host memory belongs to the caller
  }
  t->shards.clear();
}

// ---- tensor files ----------------------------------------------------------------------------
void dumpTensor(Tensor tensor, const std::string &filePath) {
  auto t = unwrapTensor(tensor);
  TensorPtr h = t->storage == Storage::Device ? toHostTensor(t, true) : t;
  FILE *f = std::fopen(filePath.c_str(), "wb");
  TTRT_ASSERT(f != nullptr, "cannot open ", filePath);
  uint32_t rank = static_cast<uint32_t>(h->shape.size()), dt = static_cast<uint32_t>(h->dtype);
  std::fwrite("TTBT", 1, 4, f);
  std::fwrite(&dt, 4, 1, f);
  std::fwrite(&rank, 4, 1, f);
  std::fwrite(h->shape.data(), 4, rank, f);
  std::fwrite(h->shards[0]->ptr, 1, h->bytes(), f);
  std::fclose(f);
}

Tensor loadTensor(const std::string &filePath, std::optional<Device> device) {
  FILE *f = std::fopen(filePath.c_str(), "rb");
  TTRT_ASSERT(f != nullptr, "cannot open ", filePath);
  char magic[4];
  uint32_t dt = 0, rank = 0;
  bool ok = std::fread(magic, 1, 4, f) == 4 && std::memcmp(magic, "TTBT", 4) == 0 && std::fread(&dt, 4, 1, f) == 1 &&
            std::fread(&rank, 4, 1, f) == 1 && rank <= 8;
  std::vector<uint32_t> shape(ok ? rank : 0);
  ok = ok && std::fread(shape.data(), 4, rank, f) == rank;
  if (!ok) {
    std::fclose(f);
    TTRT_FATAL("not a tensor file: ", filePath);
  }
  auto t = makeHostTensor(shape, static_cast<DataType>(dt), 1);
  size_t got = std::fread(t->shards[0]->ptr, 1, t->bytes(), f);
  std::fclose(f);
  TTRT_ASSERT(got == t->bytes(), "tensor file is truncated: ", filePath);
  if (device) {
    return wrapTensor(toDevice(t, deviceImpl(*device), t->dtype));
  }
  return wrapTensor(t);
}

// ---- submit ----------------------------------------------------------------------------------
std::vector<Tensor> submit(Device deviceHandle, Binary executableHandle, std::uint32_t programIndex,
                           std::vector<Tensor> &inputs) {
  auto dev = deviceImpl(deviceHandle);
  TTRT_ASSERT(dev->open, "device is closed");
  return runProgram(dev, executableHandle, programIndex, inputs);
}

// ---- debug singletons ------------------------------------------------------------------------
namespace debug {

const Hooks &Hooks::get(std::optional<OperationCallbackFn> pre, std::optional<OperationCallbackFn> post,
                        std::optional<ProgramCallbackFn> preProgram, std::optional<ProgramCallbackFn> postProgram) {
  static Hooks hooks;
  if (pre) hooks.preOperatorCallback = pre;
  if (post) hooks.postOperatorCallback = post;
  if (preProgram) hooks.preProgramCallback = preProgram;
  if (postProgram) hooks.postProgramCallback = postProgram;
  return hooks;
}

Stats &Stats::get() {
  static Stats s;
  return s;
}
void Stats::incrementStat(const std::string &stat, std::int64_t value) {
  std::lock_guard<std::mutex> g(mutex);
  counters[stat] += value;
}
std::int64_t Stats::getStat(const std::string &stat) const {
  std::lock_guard<std::mutex> g(mutex);
  auto it = counters.find(stat);
  return it == counters.end() ? 0 : it->second;
}
void Stats::removeStat(const std::string &stat) {
  std::lock_guard<std::mutex> g(mutex);
  counters.erase(stat);
}
void Stats::clear() {
  std::lock_guard<std::mutex> g(mutex);
  counters.clear();
}
std::string Stats::toString() const {
  std::lock_guard<std::mutex> g(mutex);
  std::string s = "DebugStats{";
  for (const auto &kv : counters) s += "\n\t" + kv.first + ": " + std::to_string(kv.second);
  return s + "\n}";
}

static bool envFlag(const char *name) {
  const char *e = std::getenv(name);
  return e && e[0] && std::strcmp(e, "0") != 0;
}

const Env &Env::get() {
  static const Env env{envFlag("TT_RUNTIME_SYNC_AFTER_OP"), envFlag("TTB_DISABLE_FUSION"),
                       envFlag("TTB_DISABLE_TCGEN05")};
  return env;
}

} // namespace debug

} // namespace tt::runtime
