// C ABI over the tt::runtime API (declarations and reference citations: include/ttb_runtime.h).
// Every entry point converts exceptions into a status code plus a thread-local message.
#include <cstring>
#include <string>

#include "../../include/ttb_runtime.h"
#include "impl.h"
#include "tt/runtime/debug.h"
#include "tt/runtime/perf.h"
#include "tt/runtime/runtime.h"

using namespace tt::runtime;

static thread_local std::string g_err;

#define TTRT_TRY try {
#define TTRT_CATCH                                                                       \
  }                                                                                      \
  catch (const std::exception &e) {                                                      \
    g_err = e.what();                                                                    \
    return 1;                                                                            \
  }                                                                                      \
  catch (...) {                                                                          \
    g_err = "unknown exception";                                                         \
    return 1;                                                                            \
  }                                                                                      \
  return 0;

#define TTRT_ARG(cond)                                                                   \
  if (!(cond)) {                                                                         \
    g_err = "invalid argument: " #cond;                                                  \
    return 2;                                                                            \
  }

static Binary &B(ttrt_binary_t b) { return *static_cast<Binary *>(b); }
static Device &D(ttrt_device_t d) { return *static_cast<Device *>(d); }
static Tensor &T(ttrt_tensor_t t) { return *static_cast<Tensor *>(t); }
static Layout &L(ttrt_layout_t l) { return *static_cast<Layout *>(l); }

static int copyOut(const std::string &s, char *out, size_t cap) {
  if (!out || cap == 0) {
    g_err = "output buffer missing";
    return 2;
  }
  size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
  std::memcpy(out, s.data(), n);
  out[n] = 0;
  return 0;
}

static char *dupString(const std::string &s) {
  char *p = static_cast<char *>(std::malloc(s.size() + 1));
  if (p) {
    std::memcpy(p, s.c_str(), s.size() + 1);
  }
  return p;
}

extern "C" {

const char *ttrt_last_error(void) { return g_err.c_str(); }
void ttrt_free_string(char *s) { std::free(s); }

// ---- Binary ---------------------------------------------------------------------------------
int ttrt_binary_load_from_path(const char *path, ttrt_binary_t *out) {
  TTRT_ARG(path && out)
  TTRT_TRY
  *out = new Binary(Binary::loadFromPath(path));
  TTRT_CATCH
}

int ttrt_binary_load_from_memory(const void *mem, size_t size, ttrt_binary_t *out) {
  TTRT_ARG(mem && out)
  TTRT_TRY
  *out = new Binary(Binary::loadFromMemory(mem, size));
  TTRT_CATCH
}

void ttrt_binary_free(ttrt_binary_t bin) { delete static_cast<Binary *>(bin); }

int ttrt_binary_store(ttrt_binary_t bin, const char *path) {
  TTRT_ARG(bin && path)
  TTRT_TRY
  B(bin).store(path);
  TTRT_CATCH
}

int ttrt_binary_file_identifier(ttrt_binary_t bin, char out[5]) {
  TTRT_ARG(bin && out)
  TTRT_TRY
  return copyOut(B(bin).getFileIdentifier(), out, 5);
  TTRT_CATCH
}

int ttrt_binary_version(ttrt_binary_t bin, char *out, size_t cap) {
  TTRT_ARG(bin)
  TTRT_TRY
  return copyOut(B(bin).getVersion(), out, cap);
  TTRT_CATCH
}

int ttrt_binary_check_schema_hash(ttrt_binary_t bin, int *ok) {
  TTRT_ARG(bin && ok)
  TTRT_TRY
  *ok = B(bin).checkSchemaHash() ? 1 : 0;
  TTRT_CATCH
}

int ttrt_binary_as_json(ttrt_binary_t bin, char **out) {
  TTRT_ARG(bin && out)
  TTRT_TRY
  *out = dupString(B(bin).asJson());
  TTRT_CATCH
}

int ttrt_binary_num_programs(ttrt_binary_t bin, uint32_t *n) {
  TTRT_ARG(bin && n)
  TTRT_TRY
  *n = B(bin).getNumPrograms();
  TTRT_CATCH
}

int ttrt_binary_program_name(ttrt_binary_t bin, uint32_t program, char *out, size_t cap) {
  TTRT_ARG(bin)
  TTRT_TRY
  return copyOut(B(bin).getProgramName(program), out, cap);
  TTRT_CATCH
}

int ttrt_binary_is_program_private(ttrt_binary_t bin, uint32_t program, int *priv) {
  TTRT_ARG(bin && priv)
  TTRT_TRY
  *priv = B(bin).isProgramPrivate(program) ? 1 : 0;
  TTRT_CATCH
}

int ttrt_binary_num_program_inputs(ttrt_binary_t bin, uint32_t program, uint32_t *n) {
  TTRT_ARG(bin && n)
  TTRT_TRY
  *n = B(bin).getNumProgramInputs(program);
  TTRT_CATCH
}

int ttrt_binary_num_program_outputs(ttrt_binary_t bin, uint32_t program, uint32_t *n) {
  TTRT_ARG(bin && n)
  TTRT_TRY
  *n = B(bin).getNumProgramOutputs(program);
  TTRT_CATCH
}

int ttrt_binary_program_io_desc(ttrt_binary_t bin, uint32_t program, int is_output, uint32_t index, uint32_t *rank,
                                uint32_t shape[TTRT_MAX_RANK], int *dtype) {
  TTRT_ARG(bin && rank && shape && dtype)
  TTRT_TRY
  std::vector<TensorDesc> descs = is_output ? B(bin).getProgramOutputs(program) : B(bin).getProgramInputs(program);
  if (index >= descs.size()) {
    g_err = "descriptor index out of range";
    return 2;
  }
  const TensorDesc &d = descs[index];
  if (d.shape.size() > TTRT_MAX_RANK) {
    g_err = "rank above TTRT_MAX_RANK";
    return 2;
  }
  *rank = static_cast<uint32_t>(d.shape.size());
  for (size_t i = 0; i < d.shape.size(); ++i) shape[i] = d.shape[i];
  *dtype = static_cast<int>(d.dataType);
  TTRT_CATCH
}

int ttrt_binary_program_mesh_shape(ttrt_binary_t bin, uint32_t program, uint32_t *y, uint32_t *x) {
  TTRT_ARG(bin && y && x)
  TTRT_TRY
  auto m = B(bin).getProgramMeshShape(program);
  *y = m.first;
  *x = m.second;
  TTRT_CATCH
}

int ttrt_binary_program_ops_as_json(ttrt_binary_t bin, uint32_t program, char **out) {
  TTRT_ARG(bin && out)
  TTRT_TRY
  *out = dupString(B(bin).getProgramOpsAsJson(program));
  TTRT_CATCH
}

int ttrt_binary_query_string(ttrt_binary_t bin, int what, uint32_t program, char **out) {
  TTRT_ARG(bin && out)
  TTRT_TRY
  std::string s;
  switch (what) {
  case TTRT_Q_PROGRAM_INPUTS_JSON: s = B(bin).getProgramInputsAsJson(program); break;
  case TTRT_Q_PROGRAM_OUTPUTS_JSON: s = B(bin).getProgramOutputsAsJson(program); break;
  case TTRT_Q_MLIR_JSON: s = B(bin).getMlirAsJson(); break;
  case TTRT_Q_SYSTEM_DESC_JSON: s = B(bin).getSystemDescAsJson(); break;
  case TTRT_Q_SCHEMA_HASH: s = B(bin).getSchemaHash(); break;
  case TTRT_Q_TTMLIR_GIT_HASH: s = B(bin).getTTMLIRGitHash(); break;
  default: g_err = "unknown query"; return 2;
  }
  *out = dupString(s);
  TTRT_CATCH
}

// ---- devices ----------------------------------------------------------------------------------
int ttrt_set_compatible_device_runtime(ttrt_binary_t bin) {
  TTRT_ARG(bin)
  TTRT_TRY
  setCompatibleDeviceRuntime(B(bin));
  TTRT_CATCH
}

int ttrt_get_num_available_devices(size_t *n) {
  TTRT_ARG(n)
  TTRT_TRY
  *n = getNumAvailableDevices();
  TTRT_CATCH
}

int ttrt_get_nccl_unique_id(char id128[128]) {
  TTRT_ARG(id128)
  TTRT_TRY
  std::string id = getNcclUniqueId();
  std::memcpy(id128, id.data(), 128);
  TTRT_CATCH
}

int ttrt_open_mesh_device(uint32_t mesh_y, uint32_t mesh_x, const int *device_ids, uint32_t n_device_ids,
                          uint32_t process_rank, uint32_t process_count, const char *nccl_id128, ttrt_device_t *out) {
  TTRT_ARG(out)
  TTRT_TRY
  MeshDeviceOptions o;
  o.meshShape = std::vector<uint32_t>{mesh_y, mesh_x};
  if (device_ids) {
    o.deviceIds.assign(device_ids, device_ids + n_device_ids);
  }
  o.processRank = process_rank;
  o.processCount = process_count ? process_count : 1;
  if (nccl_id128) {
    o.ncclUniqueId.assign(nccl_id128, 128);
  }
  *out = new Device(openMeshDevice(o));
  TTRT_CATCH
}

int ttrt_close_mesh_device(ttrt_device_t dev) {
  TTRT_ARG(dev)
  TTRT_TRY
  closeMeshDevice(D(dev));
  TTRT_CATCH
}

void ttrt_device_free(ttrt_device_t dev) { delete static_cast<Device *>(dev); }

int ttrt_device_mesh_shape(ttrt_device_t dev, uint32_t *y, uint32_t *x) {
  TTRT_ARG(dev && y && x)
  TTRT_TRY
  auto m = getMeshShape(D(dev));
  *y = m[0];
  *x = m[1];
  TTRT_CATCH
}

int ttrt_device_num_local(ttrt_device_t dev, uint32_t *n) {
  TTRT_ARG(dev && n)
  TTRT_TRY
  *n = static_cast<uint32_t>(D(dev).as<cuda::DeviceImpl>(DeviceRuntime::CUDA).locals.size());
  TTRT_CATCH
}

int ttrt_device_stream(ttrt_device_t dev, uint32_t index, void **stream, int *cuda_device) {
  TTRT_ARG(dev && stream)
  TTRT_TRY
  auto &impl = D(dev).as<cuda::DeviceImpl>(DeviceRuntime::CUDA);
  if (index >= impl.locals.size()) {
    g_err = "local coordinate index out of range";
    return 2;
  }
  *stream = impl.locals[index].stream;
  if (cuda_device) {
    *cuda_device = impl.locals[index].cudaDevice;
  }
  TTRT_CATCH
}

// ---- tensors ----------------------------------------------------------------------------------
int ttrt_create_borrowed_host_tensor(void *data, const uint32_t *shape, const int64_t *stride, uint32_t rank,
                                     uint32_t itemsize, int dtype, ttrt_tensor_t *out) {
  TTRT_ARG(out && (rank == 0 || (shape && stride)))
  TTRT_TRY
  *out = new Tensor(createBorrowedHostTensor(data, std::vector<uint32_t>(shape, shape + rank),
                                             std::vector<int64_t>(stride, stride + rank), itemsize,
                                             static_cast<tt::target::DataType>(dtype)));
  TTRT_CATCH
}

int ttrt_create_owned_host_tensor(const void *data, const uint32_t *shape, const int64_t *stride, uint32_t rank,
                                  uint32_t itemsize, int dtype, ttrt_tensor_t *out) {
  TTRT_ARG(out && (rank == 0 || (shape && stride)))
  TTRT_TRY
  *out = new Tensor(createOwnedHostTensor(data, std::vector<uint32_t>(shape, shape + rank),
                                          std::vector<int64_t>(stride, stride + rank), itemsize,
                                          static_cast<tt::target::DataType>(dtype)));
  TTRT_CATCH
}

int ttrt_create_multi_device_host_tensor(const ttrt_tensor_t *shards, uint32_t n_shards, uint32_t mesh_y,
                                         uint32_t mesh_x, ttrt_tensor_t *out) {
  TTRT_ARG(shards && out)
  TTRT_TRY
  std::vector<Tensor> v;
  for (uint32_t i = 0; i < n_shards; ++i) v.push_back(T(shards[i]));
  *out = new Tensor(createMultiDeviceHostTensor(v, {}, {mesh_y, mesh_x}));
  TTRT_CATCH
}

void ttrt_tensor_free(ttrt_tensor_t t) { delete static_cast<Tensor *>(t); }

int ttrt_tensor_info(ttrt_tensor_t t, uint32_t *rank, uint32_t shape[TTRT_MAX_RANK], int *dtype, int *storage,
                     uint32_t *n_shards, int *allocated) {
  TTRT_ARG(t)
  TTRT_TRY
  auto impl = cuda::unwrapTensor(T(t));
  if (impl->shape.size() > TTRT_MAX_RANK) {
    g_err = "rank above TTRT_MAX_RANK";
    return 2;
  }
  if (rank) *rank = static_cast<uint32_t>(impl->shape.size());
  if (shape) {
    for (size_t i = 0; i < impl->shape.size(); ++i) shape[i] = impl->shape[i];
  }
  if (dtype) *dtype = static_cast<int>(impl->dtype);
  if (storage) *storage = impl->storage == cuda::Storage::Device ? 1 : 0;
  if (n_shards) *n_shards = static_cast<uint32_t>(impl->shards.size());
  if (allocated) *allocated = impl->allocated() ? 1 : 0;
  TTRT_CATCH
}

int ttrt_tensor_get_retain(ttrt_tensor_t t, int *retain) {
  TTRT_ARG(t && retain)
  TTRT_TRY
  *retain = getTensorRetain(T(t)) ? 1 : 0;
  TTRT_CATCH
}

int ttrt_tensor_set_retain(ttrt_tensor_t t, int retain) {
  TTRT_ARG(t)
  TTRT_TRY
  setTensorRetain(T(t), retain != 0);
  TTRT_CATCH
}

int ttrt_deallocate_tensor(ttrt_tensor_t t, int force) {
  TTRT_ARG(t)
  TTRT_TRY
  deallocateTensor(T(t), force != 0);
  TTRT_CATCH
}

// ---- layouts / movement -----------------------------------------------------------------------
int ttrt_get_layout(ttrt_binary_t bin, uint32_t program, uint32_t input, ttrt_layout_t *out) {
  TTRT_ARG(bin && out)
  TTRT_TRY
  *out = new Layout(getLayout(B(bin), program, input));
  TTRT_CATCH
}

void ttrt_layout_free(ttrt_layout_t l) { delete static_cast<Layout *>(l); }

int ttrt_to_layout(ttrt_tensor_t t, ttrt_device_t dev, ttrt_layout_t layout, int retain, ttrt_tensor_t *out) {
  TTRT_ARG(t && dev && layout && out)
  TTRT_TRY
  std::optional<bool> r = retain < 0 ? std::nullopt : std::optional<bool>(retain != 0);
  *out = new Tensor(toLayout(T(t), D(dev), L(layout), r));
  TTRT_CATCH
}

int ttrt_has_layout(ttrt_tensor_t t, ttrt_layout_t layout, int *yes) {
  TTRT_ARG(t && layout && yes)
  TTRT_TRY
  *yes = hasLayout(T(t), L(layout)) ? 1 : 0;
  TTRT_CATCH
}

int ttrt_to_host(ttrt_tensor_t t, int untilize, int blocking, ttrt_tensor_t *out, uint32_t cap, uint32_t *n) {
  TTRT_ARG(t && out && n)
  TTRT_TRY
  std::vector<Tensor> v = toHost(T(t), untilize != 0, blocking != 0);
  if (v.size() > cap) {
    g_err = "output array too small for the shards";
    return 2;
  }
  for (size_t i = 0; i < v.size(); ++i) out[i] = new Tensor(v[i]);
  *n = static_cast<uint32_t>(v.size());
  TTRT_CATCH
}

int ttrt_memcpy_to_ptr(void *dst, ttrt_tensor_t src, int target_dtype) {
  TTRT_ARG(dst && src)
  TTRT_TRY
  std::optional<tt::target::DataType> dt;
  if (target_dtype >= 0) dt = static_cast<tt::target::DataType>(target_dtype);
  tt::runtime::memcpy(dst, T(src), dt);
  TTRT_CATCH
}

int ttrt_memcpy_tensor(ttrt_tensor_t dst, ttrt_tensor_t src) {
  TTRT_ARG(dst && src)
  TTRT_TRY
  tt::runtime::memcpy(T(dst), T(src));
  TTRT_CATCH
}

int ttrt_tensor_host_ptr(ttrt_tensor_t t, void **ptr) {
  TTRT_ARG(t && ptr)
  TTRT_TRY
  auto impl = tt::runtime::cuda::unwrapTensor(T(t));
  if (impl->storage != tt::runtime::cuda::Storage::Host || impl->shards.empty() || !impl->shards[0]) {
    throw std::runtime_error("tensor_host_ptr needs a host tensor with data");
  }
  *ptr = impl->shards[0]->ptr;
  TTRT_CATCH
}

int ttrt_wait_tensor(ttrt_tensor_t t) {
  TTRT_ARG(t)
  TTRT_TRY
  wait(T(t));
  TTRT_CATCH
}

// ---- execution ----------------------------------------------------------------------------------
int ttrt_submit(ttrt_device_t dev, ttrt_binary_t bin, uint32_t program, const ttrt_tensor_t *inputs, uint32_t n_inputs,
                ttrt_tensor_t *outputs, uint32_t cap, uint32_t *n_outputs) {
  TTRT_ARG(dev && bin && n_outputs && (n_inputs == 0 || inputs))
  TTRT_TRY
  std::vector<Tensor> in;
  for (uint32_t i = 0; i < n_inputs; ++i) {
    if (!inputs[i]) {
      g_err = "null input tensor";
      return 2;
    }
    in.push_back(T(inputs[i]));
  }
  std::vector<Tensor> out = submit(D(dev), B(bin), program, in);
  if (out.size() > cap || (out.size() && !outputs)) {
    g_err = "output array too small";
    return 2;
  }
  for (size_t i = 0; i < out.size(); ++i) outputs[i] = new Tensor(out[i]);
  *n_outputs = static_cast<uint32_t>(out.size());
  TTRT_CATCH
}

// ---- sub-program state --------------------------------------------------------------------------
int ttrt_binary_id(ttrt_binary_t bin, uint64_t *id) {
  TTRT_ARG(bin && id)
  TTRT_TRY
  *id = B(bin).id();
  TTRT_CATCH
}

int ttrt_release_trace(ttrt_device_t dev, uint64_t binary_id, size_t main_program) {
  TTRT_ARG(dev)
  TTRT_TRY
  releaseTrace(D(dev), binary_id, main_program);
  TTRT_CATCH
}

int ttrt_const_eval_cache_size(size_t *n) {
  TTRT_ARG(n)
  TTRT_TRY
  *n = ::tt::runtime::cuda::ConstEvalCache::get().size();
  TTRT_CATCH
}

int ttrt_const_eval_cache_clear(void) {
  TTRT_TRY
  ::tt::runtime::cuda::ConstEvalCache::get().clear();
  TTRT_CATCH
}

int ttrt_stat_get(const char *name, int64_t *value) {
  TTRT_ARG(name && value)
  TTRT_TRY
  *value = debug::Stats::get().getStat(name);
  TTRT_CATCH
}

int ttrt_stats_clear(void) {
  TTRT_TRY
  debug::Stats::get().clear();
  TTRT_CATCH
}

// ---- hooks --------------------------------------------------------------------------------------
int ttrt_register_op_hooks(ttrt_op_callback_t pre, ttrt_op_callback_t post, void *user) {
  TTRT_TRY
  auto wrap = [user](ttrt_op_callback_t cb) -> std::optional<debug::Hooks::OperationCallbackFn> {
    if (!cb) {
      return std::nullopt;
    }
    return debug::Hooks::OperationCallbackFn([cb, user](Binary b, CallbackContext pc, OpContext oc) {
      cb(&b, &pc, &oc, user);
    });
  };
  debug::Hooks::get(wrap(pre), wrap(post));
  TTRT_CATCH
}

int ttrt_unregister_hooks(void) {
  TTRT_TRY
  debug::Hooks::get().unregisterHooks();
  TTRT_CATCH
}

int ttrt_op_loc_info(void *op_ctx, char *out, size_t cap) {
  TTRT_ARG(op_ctx)
  TTRT_TRY
  return copyOut(getOpLocInfo(*static_cast<OpContext *>(op_ctx)), out, cap);
  TTRT_CATCH
}

int ttrt_op_debug_string(void *op_ctx, char *out, size_t cap) {
  TTRT_ARG(op_ctx)
  TTRT_TRY
  return copyOut(getOpDebugString(*static_cast<OpContext *>(op_ctx)), out, cap);
  TTRT_CATCH
}

int ttrt_op_output_tensor(void *op_ctx, void *program_ctx, ttrt_tensor_t *out) {
  TTRT_ARG(op_ctx && program_ctx && out)
  TTRT_TRY
  auto m = getOpOutputTensor(*static_cast<OpContext *>(op_ctx), *static_cast<CallbackContext *>(program_ctx));
  *out = nullptr;
  if (!m.empty()) {
    uint32_t best = UINT32_MAX;
    for (const auto &kv : m) best = kv.first < best ? kv.first : best;
    *out = new Tensor(m.at(best));
  }
  TTRT_CATCH
}

int ttrt_program_index(void *program_ctx, size_t *index) {
  TTRT_ARG(program_ctx && index)
  TTRT_TRY
  *index = getProgramIndex(*static_cast<CallbackContext *>(program_ctx));
  TTRT_CATCH
}

// ---- system descriptor, sub-meshes, embedded goldens, tensor references -----------------------------
int ttrt_get_current_system_desc(ttrt_device_t dev, ttrt_binary_t *out) {
  TTRT_ARG(out)
  TTRT_TRY
  SystemDesc d = dev ? getCurrentSystemDesc(std::nullopt, D(dev)) : getCurrentSystemDesc();
  *out = new Binary(Flatbuffer(d.handle));
  TTRT_CATCH
}

int ttrt_create_sub_mesh_device(ttrt_device_t parent, uint32_t mesh_y, uint32_t mesh_x, int has_offset, uint32_t off_y,
                                uint32_t off_x, ttrt_device_t *out) {
  TTRT_ARG(parent && out)
  TTRT_TRY
  std::optional<const std::vector<uint32_t>> off;
  if (has_offset) off.emplace(std::vector<uint32_t>{off_y, off_x});
  *out = new Device(createSubMeshDevice(D(parent), {mesh_y, mesh_x}, off));
  TTRT_CATCH
}

int ttrt_release_sub_mesh_device(ttrt_device_t sub) {
  TTRT_ARG(sub)
  TTRT_TRY
  releaseSubMeshDevice(D(sub));
  TTRT_CATCH
}

int ttrt_reshape_mesh_device(ttrt_device_t dev, uint32_t mesh_y, uint32_t mesh_x) {
  TTRT_ARG(dev)
  TTRT_TRY
  reshapeMeshDevice(D(dev), {mesh_y, mesh_x});
  TTRT_CATCH
}

int ttrt_device_ids(ttrt_device_t dev, int *ids, uint32_t cap, uint32_t *n) {
  TTRT_ARG(dev && n)
  TTRT_TRY
  std::vector<int> v = getDeviceIds(D(dev));
  *n = static_cast<uint32_t>(v.size());
  for (uint32_t i = 0; ids && i < cap && i < v.size(); ++i) ids[i] = v[i];
  TTRT_CATCH
}

int ttrt_binary_golden_devices(ttrt_binary_t bin, const char *loc, uint32_t *devices, uint32_t cap, uint32_t *n) {
  TTRT_ARG(bin && loc && n)
  TTRT_TRY
  std::string key(loc);
  auto m = B(bin).getDebugInfoGolden(key);
  *n = static_cast<uint32_t>(m.size());
  uint32_t i = 0;
  for (const auto &kv : m) {
    if (devices && i < cap) devices[i] = kv.first;
    ++i;
  }
  TTRT_CATCH
}

int ttrt_binary_golden_tensor(ttrt_binary_t bin, const char *loc, uint32_t device, uint32_t *rank, int64_t shape[TTRT_MAX_RANK],
                              int64_t stride[TTRT_MAX_RANK], int *dtype, const void **data, size_t *size) {
  TTRT_ARG(bin && loc && rank && shape && stride && dtype && data && size)
  TTRT_TRY
  std::string key(loc);
  auto m = B(bin).getDebugInfoGolden(key);
  auto it = m.find(device);
  *data = nullptr;
  *size = 0;
  *rank = 0;
  if (it != m.end() && it->second) {
    const auto *g = it->second;
    const uint32_t r = g->shape() ? g->shape()->size() : 0;
    if (r > TTRT_MAX_RANK) {
      g_err = "golden tensor rank exceeds TTRT_MAX_RANK";
      return 1;
    }
    *rank = r;
    for (uint32_t i = 0; i < r; ++i) {
      shape[i] = g->shape()->Get(i);
      stride[i] = g->stride() && i < g->stride()->size() ? g->stride()->Get(i) : 0;
    }
    *dtype = static_cast<int>(g->dtype());
    if (g->data()) {
      *data = g->data()->data();
      *size = g->data()->size();
    }
  }
  TTRT_CATCH
}

static int copyRefs(const std::vector<TensorRef> &refs, ttrt_tensor_ref_t *out, uint32_t cap, uint32_t *n) {
  *n = static_cast<uint32_t>(refs.size());
  for (uint32_t i = 0; out && i < cap && i < refs.size(); ++i) out[i] = new TensorRef(refs[i]);
  return 0;
}

int ttrt_op_input_refs(void *op_ctx, ttrt_tensor_ref_t *out, uint32_t cap, uint32_t *n) {
  TTRT_ARG(op_ctx && n)
  TTRT_TRY
  return copyRefs(getOpInputRefs(*static_cast<OpContext *>(op_ctx)), out, cap, n);
  TTRT_CATCH
}

int ttrt_op_output_refs(void *op_ctx, ttrt_tensor_ref_t *out, uint32_t cap, uint32_t *n) {
  TTRT_ARG(op_ctx && n)
  TTRT_TRY
  return copyRefs(getOpOutputRefs(*static_cast<OpContext *>(op_ctx)), out, cap, n);
  TTRT_CATCH
}

void ttrt_tensor_ref_free(ttrt_tensor_ref_t ref) { delete static_cast<TensorRef *>(ref); }

int ttrt_tensor_ref_info(ttrt_tensor_ref_t ref, uint32_t *rank, uint32_t shape[TTRT_MAX_RANK], int *dtype) {
  TTRT_ARG(ref && rank && shape && dtype)
  TTRT_TRY
  auto &r = *static_cast<TensorRef *>(ref);
  std::vector<uint32_t> s = getTensorRefShape(r);
  TTRT_ARG(s.size() <= TTRT_MAX_RANK)
  *rank = static_cast<uint32_t>(s.size());
  for (size_t i = 0; i < s.size(); ++i) shape[i] = s[i];
  *dtype = static_cast<int>(getTensorRefDataType(r));
  TTRT_CATCH
}

int ttrt_retrieve_tensor_from_pool(void *program_ctx, ttrt_tensor_ref_t ref, int untilize, ttrt_tensor_t *out) {
  TTRT_ARG(program_ctx && ref && out)
  TTRT_TRY
  auto t = retrieveTensorFromPool(*static_cast<CallbackContext *>(program_ctx), *static_cast<TensorRef *>(ref), untilize != 0);
  *out = t ? new Tensor(*t) : nullptr;
  TTRT_CATCH
}

int ttrt_update_tensor_in_pool(void *program_ctx, ttrt_tensor_ref_t ref, ttrt_tensor_t src) {
  TTRT_ARG(program_ctx && ref && src)
  TTRT_TRY
  updateTensorInPool(*static_cast<CallbackContext *>(program_ctx), *static_cast<TensorRef *>(ref), T(src));
  TTRT_CATCH
}

// ---- perf::Env (runtime/include/tt/runtime/perf.h) ----------------------------------------------------
int ttrt_perf_env_get(uint32_t dump_device_rate, int enable_perf_trace, const char *program_metadata, int *enabled) {
  TTRT_TRY
  perf::Env &e = perf::Env::get(dump_device_rate, enable_perf_trace != 0, program_metadata ? program_metadata : "");
  if (enabled) *enabled = e.enablePerfTrace ? 1 : 0;
  TTRT_CATCH
}

int ttrt_perf_message(int tag, const char *text) {
  TTRT_ARG(text)
  TTRT_TRY
  perf::Env &e = perf::Env::get();
  switch (tag) {
  case 0: e.tracyLogOpLocation(text); break;
  case 1: e.tracyLogConstEvalProgram(std::strcmp(text, "true") == 0); break;
  case 2: e.tracyLogProgramMetadata(text); break;
  case 3: e.tracyLogInputLayoutConversion(std::strcmp(text, "true") == 0); break;
  case 4: e.setProgramMetadata(text); break;
  default: g_err = "unknown perf tag"; return 2;
  }
  TTRT_CATCH
}

uint64_t ttrt_perf_emitted(void) { return perf::Env::emitted(); }

} // extern "C"
