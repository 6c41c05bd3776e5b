// Device, stream, memory and event entry points of the C ABI, plus error bookkeeping.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

#include <atomic>
#include <map>
#include <mutex>
#include <vector>

namespace ttb {

static thread_local std::string g_lastError;
std::atomic<uint64_t> g_launchCount{0};

void setLastError(const std::string &msg) { g_lastError = msg; }

int cudaFail(cudaError_t e, const char *what, const char *file, int line) {
  g_lastError = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e) + " at " +
                file + ":" + std::to_string(line) + " in " + what;
  return TTB_ERR_CUDA;
}

int smCount() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    return 148;
  }
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      n = 148;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

bool pdlEnabled() {
  static const bool on = [] {
    const char *e = std::getenv("TTB_DISABLE_PDL");
    return !(e && e[0] == '1');
  }();
  return on;
}

void countLaunch(uint64_t n) { g_launchCount.fetch_add(n, std::memory_order_relaxed); }

// ---- per-launch profiling ----------------------------------------------------------------
struct ProfRecord {
  const char *tag;
  double flops, bytes;
  cudaEvent_t start, stop;
};
static std::atomic<bool> g_profOn{false};
static std::mutex g_profMutex;
static std::vector<ProfRecord> g_profRecords;

ProfScope::ProfScope(const char *tag, double flops, double bytes, cudaStream_t st) : slot(-1), stream(st) {
  if (!g_profOn.load(std::memory_order_relaxed)) return;
  cudaEvent_t start = nullptr, stop = nullptr;
  if (cudaEventCreate(&start) != cudaSuccess) return;
  if (cudaEventCreate(&stop) != cudaSuccess) {
    cudaEventDestroy(start);
    return;
  }
  cudaEventRecord(start, st);
  std::lock_guard<std::mutex> g(g_profMutex);
  g_profRecords.push_back(ProfRecord{tag, flops, bytes, start, stop});
  slot = static_cast<int>(g_profRecords.size()) - 1;
}

ProfScope::~ProfScope() {
  if (slot < 0) return;
  std::lock_guard<std::mutex> g(g_profMutex);
  if (slot < static_cast<int>(g_profRecords.size())) cudaEventRecord(g_profRecords[slot].stop, stream);
}

} // namespace ttb

using namespace ttb;

extern "C" {

const char *ttb_last_error(void) { return g_lastError.c_str(); }

size_t ttb_dtype_size(int dtype) { return dtypeSize(dtype); }

uint64_t ttb_launch_count(void) { return g_launchCount.load(std::memory_order_relaxed); }

int ttb_prof_enable(int on) {
  std::lock_guard<std::mutex> g(g_profMutex);
  for (ProfRecord &r : g_profRecords) {
    if (r.start) cudaEventDestroy(r.start);
    if (r.stop) cudaEventDestroy(r.stop);
  }
  g_profRecords.clear();
  g_profOn.store(on != 0);
  return TTB_OK;
}

int ttb_prof_summary(char *json_out, size_t cap) {
  TTB_CHECK(json_out && cap > 2, "output buffer missing");
  std::lock_guard<std::mutex> g(g_profMutex);
  struct Agg { long launches = 0; double ms = 0, flops = 0, bytes = 0; };
  std::map<std::string, Agg> agg;
  for (ProfRecord &r : g_profRecords) {
    TTB_CUDA(cudaEventSynchronize(r.stop));
    float ms = 0.0f;
    TTB_CUDA(cudaEventElapsedTime(&ms, r.start, r.stop));
    Agg &a = agg[r.tag];
    a.launches++;
    a.ms += ms;
    a.flops += r.flops;
    a.bytes += r.bytes;
  }
  std::string s = "[";
  bool first = true;
  for (const auto &kv : agg) {
    char buf[256];
    snprintf(buf, sizeof buf, "%s{\"tag\": \"%s\", \"launches\": %ld, \"ms\": %.6f, \"flops\": %.6e, \"bytes\": %.6e}",
             first ? "" : ", ", kv.first.c_str(), kv.second.launches, kv.second.ms, kv.second.flops, kv.second.bytes);
    s += buf;
    first = false;
  }
  s += "]";
  TTB_CHECK(s.size() + 1 <= cap, "output buffer too small");
  memcpy(json_out, s.c_str(), s.size() + 1);
  return TTB_OK;
}

int ttb_device_count(int *count) {
  TTB_CHECK(count != nullptr, "count is null");
  cudaError_t e = cudaGetDeviceCount(count);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
    *count = 0;
    (void)cudaGetLastError();
    return TTB_OK;
  }
  TTB_CUDA(e);
  return TTB_OK;
}

int ttb_set_device(int device) {
  TTB_CUDA(cudaSetDevice(device));
  return TTB_OK;
}

int ttb_device_info(int device, int *sm_count, size_t *total_mem, int *cc_major, int *cc_minor) {
  cudaDeviceProp p;
  TTB_CUDA(cudaGetDeviceProperties(&p, device));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (total_mem) *total_mem = p.totalGlobalMem;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return TTB_OK;
}

int ttb_stream_create(void **stream) {
  TTB_CHECK(stream != nullptr, "stream is null");
  cudaStream_t s;
  TTB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  // Keep freed blocks in the pool: tensors of a program are re-allocated every submit.
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  cudaMemPool_t pool;
  TTB_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
  uint64_t threshold = UINT64_MAX;
  TTB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
  *stream = s;
  return TTB_OK;
}

int ttb_stream_destroy(void *stream) {
  TTB_CUDA(cudaStreamDestroy(asStream(stream)));
  return TTB_OK;
}

int ttb_stream_sync(void *stream) {
  TTB_CUDA(cudaStreamSynchronize(asStream(stream)));
  return TTB_OK;
}

int ttb_device_sync(void) {
  TTB_CUDA(cudaDeviceSynchronize());
  return TTB_OK;
}

int ttb_malloc(void **ptr, size_t bytes, void *stream) {
  TTB_CHECK(ptr != nullptr, "ptr is null");
  if (bytes == 0) {
    bytes = 16; // distinct non-null pointers for empty tensors
  }
  TTB_CUDA(cudaMallocAsync(ptr, bytes, asStream(stream)));
  return TTB_OK;
}

int ttb_free(void *ptr, void *stream) {
  if (ptr) {
    TTB_CUDA(cudaFreeAsync(ptr, asStream(stream)));
  }
  return TTB_OK;
}

int ttb_mempool_stats(uint64_t *reserved, uint64_t *used, uint64_t *used_high, int reset_high) {
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  cudaMemPool_t pool;
  TTB_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
  uint64_t v = 0;
  if (reserved) {
    TTB_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &v));
    *reserved = v;
  }
  if (used) {
    TTB_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &v));
    *used = v;
  }
  if (used_high) {
    TTB_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &v));
    *used_high = v;
  }
  if (reset_high) {
    uint64_t zero = 0; // the only value the attribute accepts: the mark falls back to the current use
    TTB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &zero));
  }
  return TTB_OK;
}

int ttb_host_alloc_pinned(void **ptr, size_t bytes) {
  TTB_CHECK(ptr != nullptr, "ptr is null");
  TTB_CUDA(cudaMallocHost(ptr, bytes ? bytes : 16));
  return TTB_OK;
}

int ttb_host_is_pinned(const void *ptr, int *pinned) {
  TTB_CHECK(pinned != nullptr, "pinned is null");
  *pinned = 0;
  if (!ptr) return TTB_OK;
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) {
    (void)cudaGetLastError(); // plain malloc memory on older drivers reports an error: not pinned
    return TTB_OK;
  }
  *pinned = attr.type == cudaMemoryTypeHost ? 1 : 0;
  return TTB_OK;
}

int ttb_host_free_pinned(void *ptr) {
  if (ptr) {
    TTB_CUDA(cudaFreeHost(ptr));
  }
  return TTB_OK;
}

int ttb_memcpy_h2d(void *dst, const void *host_src, size_t bytes, void *stream) {
  if (bytes) {
    TTB_CUDA(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, asStream(stream)));
  }
  return TTB_OK;
}

int ttb_memcpy_d2h(void *host_dst, const void *src, size_t bytes, void *stream) {
  if (bytes) {
    TTB_CUDA(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, asStream(stream)));
  }
  return TTB_OK;
}

int ttb_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes) {
    TTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, asStream(stream)));
  }
  return TTB_OK;
}

int ttb_memset(void *dst, int byte, size_t bytes, void *stream) {
  if (bytes) {
    TTB_CUDA(cudaMemsetAsync(dst, byte, bytes, asStream(stream)));
  }
  return TTB_OK;
}

// ---- traces: a stretch of a stream's work recorded once and replayed as one CUDA graph ----
int ttb_trace_begin(void *stream) {
  // Thread-local mode: other threads may keep allocating and copying while this one records.
  TTB_CUDA(cudaStreamBeginCapture(asStream(stream), cudaStreamCaptureModeThreadLocal));
  return TTB_OK;
}

int ttb_trace_end(void *stream, void **trace) {
  TTB_CHECK(trace != nullptr, "trace is null");
  *trace = nullptr;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(asStream(stream), &graph);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    ::ttb::setLastError(std::string("the recording was invalidated: ") + cudaGetErrorString(e));
    return TTB_ERR_CUDA;
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    ::ttb::setLastError(std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
    return TTB_ERR_CUDA;
  }
  *trace = exec;
  return TTB_OK;
}

int ttb_trace_abort(void *stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(asStream(stream), &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return TTB_OK;
  }
  if (st != cudaStreamCaptureStatusNone) {
    cudaGraph_t graph = nullptr;
    (void)cudaStreamEndCapture(asStream(stream), &graph);
    (void)cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
  }
  return TTB_OK;
}

int ttb_trace_launch(void *trace, void *stream) {
  TTB_CHECK(trace != nullptr, "trace is null");
  TTB_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(trace), asStream(stream)));
  return TTB_OK;
}

int ttb_trace_destroy(void *trace) {
  if (trace) TTB_CUDA(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(trace)));
  return TTB_OK;
}

int ttb_stream_is_recording(void *stream, int *recording) {
  TTB_CHECK(recording != nullptr, "recording is null");
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  TTB_CUDA(cudaStreamIsCapturing(asStream(stream), &st));
  *recording = st == cudaStreamCaptureStatusActive ? 1 : 0;
  return TTB_OK;
}

int ttb_event_create(void **event) {
  TTB_CHECK(event != nullptr, "event is null");
  cudaEvent_t e;
  TTB_CUDA(cudaEventCreate(&e));
  *event = e;
  return TTB_OK;
}

int ttb_event_destroy(void *event) {
  TTB_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return TTB_OK;
}

int ttb_event_record(void *event, void *stream) {
  TTB_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), asStream(stream)));
  return TTB_OK;
}

int ttb_event_sync(void *event) {
  TTB_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
  return TTB_OK;
}

int ttb_stream_wait_event(void *stream, void *event) {
  TTB_CUDA(cudaStreamWaitEvent(asStream(stream), reinterpret_cast<cudaEvent_t>(event), 0));
  return TTB_OK;
}

int ttb_event_elapsed_ms(void *start, void *stop, float *ms) {
  TTB_CHECK(ms != nullptr, "ms is null");
  TTB_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start),
                                reinterpret_cast<cudaEvent_t>(stop)));
  return TTB_OK;
}

} // extern "C"
