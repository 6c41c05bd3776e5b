// Collectives over NVLink / NVSwitch through NCCL, for the mesh ops of a 1xN device mesh
// (reference call sites: ::ttnn::all_reduce / all_gather / reduce_scatter in
// runtime/lib/ttnn/operations/ccl/{all_reduce,all_gather,reduce_scatter}.cpp, which ride on
// tt-fabric).  NCCL is opened with dlopen on first use so that the kernel library loads on
// machines without it and single-GPU programs never touch it.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

namespace ttb {

struct NcclApi {
  void *lib = nullptr;
  decltype(&ncclGetUniqueId) getUniqueId = nullptr;
  decltype(&ncclCommInitRank) commInitRank = nullptr;
  decltype(&ncclCommInitAll) commInitAll = nullptr;
  decltype(&ncclCommDestroy) commDestroy = nullptr;
  decltype(&ncclAllReduce) allReduce = nullptr;
  decltype(&ncclAllGather) allGather = nullptr;
  decltype(&ncclReduceScatter) reduceScatter = nullptr;
  decltype(&ncclBroadcast) broadcast = nullptr;
  decltype(&ncclGroupStart) groupStart = nullptr;
  decltype(&ncclGroupEnd) groupEnd = nullptr;
  decltype(&ncclGetErrorString) getErrorString = nullptr;
  decltype(&ncclGetVersion) getVersion = nullptr;
  std::string error;
};

static NcclApi &nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    // A libnccl already mapped into the process (for instance the one bundled with torch) is
    // found first; otherwise the system library.
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
      api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.lib) break;
    }
    if (!api.lib) {
      api.error = std::string("cannot load NCCL: ") + dlerror();
      return;
    }
#define TTB_SYM(field, name)                                                             \
  api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.lib, #name));              \
  if (!api.field) {                                                                      \
    api.error = "NCCL symbol missing: " #name;                                           \
    return;                                                                              \
  }
    TTB_SYM(getUniqueId, ncclGetUniqueId)
    TTB_SYM(commInitRank, ncclCommInitRank)
    TTB_SYM(commInitAll, ncclCommInitAll)
    TTB_SYM(commDestroy, ncclCommDestroy)
    TTB_SYM(allReduce, ncclAllReduce)
    TTB_SYM(allGather, ncclAllGather)
    TTB_SYM(reduceScatter, ncclReduceScatter)
    TTB_SYM(broadcast, ncclBroadcast)
    TTB_SYM(groupStart, ncclGroupStart)
    TTB_SYM(groupEnd, ncclGroupEnd)
    TTB_SYM(getErrorString, ncclGetErrorString)
    TTB_SYM(getVersion, ncclGetVersion)
#undef TTB_SYM
  });
  return api;
}

#define TTB_NCCL_READY()                                                                 \
  NcclApi &api = nccl();                                                                 \
  if (!api.error.empty()) {                                                              \
    setLastError(api.error);                                                             \
    return TTB_ERR_NCCL;                                                                 \
  }

#define TTB_NCCL(expr)                                                                   \
  do {                                                                                   \
    ncclResult_t _r = (expr);                                                            \
    if (_r != ncclSuccess) {                                                             \
      setLastError(std::string("NCCL: ") + api.getErrorString(_r) + " in " #expr);      \
      return TTB_ERR_NCCL;                                                               \
    }                                                                                    \
  } while (0)

static bool ncclType(int dt, ncclDataType_t &out) {
  switch (dt) {
  case kF32: out = ncclFloat32; return true;
  case kF16: out = ncclFloat16; return true;
  case kBF16: out = ncclBfloat16; return true;
  case kI32: out = ncclInt32; return true;
  case kU32: out = ncclUint32; return true;
  case kU8: out = ncclUint8; return true;
  case kI8: out = ncclInt8; return true;
  default: return false;
  }
}

// ttcore::ReduceType as serialised in AllReduceOp.reduce_type (0 Sum, 1 Mean, 2 Max, 3 Min;
// runtime/lib/ttnn/utils/utils.cpp:149-166).
static bool ncclOp(int reduceType, ncclRedOp_t &out) {
  switch (reduceType) {
  case 0: out = ncclSum; return true;
  case 1: out = ncclAvg; return true;
  case 2: out = ncclMax; return true;
  case 3: out = ncclMin; return true;
  default: return false;
  }
}

} // namespace ttb

using namespace ttb;

extern "C" {

int ttb_nccl_version(int *version) {
  TTB_NCCL_READY();
  TTB_NCCL(api.getVersion(version));
  return TTB_OK;
}

int ttb_nccl_unique_id(char *id128) {
  TTB_CHECK(id128 != nullptr, "id buffer is null");
  TTB_NCCL_READY();
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  ncclUniqueId id;
  TTB_NCCL(api.getUniqueId(&id));
  memcpy(id128, &id, 128);
  return TTB_OK;
}

int ttb_comm_init_rank(void **comm, int nranks, const char *id128, int rank) {
  TTB_CHECK(comm && id128, "null argument");
  TTB_NCCL_READY();
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  ncclComm_t c;
  TTB_NCCL(api.commInitRank(&c, nranks, id, rank));
  *comm = c;
  return TTB_OK;
}

int ttb_comm_init_all(void **comms, int ndev, const int *devices) {
  TTB_CHECK(comms && devices && ndev > 0, "bad argument");
  TTB_NCCL_READY();
  TTB_NCCL(api.commInitAll(reinterpret_cast<ncclComm_t *>(comms), ndev, devices));
  return TTB_OK;
}

int ttb_comm_destroy(void *comm) {
  if (!comm) return TTB_OK;
  TTB_NCCL_READY();
  TTB_NCCL(api.commDestroy(static_cast<ncclComm_t>(comm)));
  return TTB_OK;
}

int ttb_group_start(void) {
  TTB_NCCL_READY();
  TTB_NCCL(api.groupStart());
  return TTB_OK;
}

int ttb_group_end(void) {
  TTB_NCCL_READY();
  TTB_NCCL(api.groupEnd());
  return TTB_OK;
}

int ttb_all_reduce(void *comm, const void *in, void *out, size_t count, int dtype, int reduce_type, void *stream) {
  TTB_CHECK(comm && in && out, "null argument");
  TTB_NCCL_READY();
  ncclDataType_t dt;
  ncclRedOp_t op;
  if (!ncclType(dtype, dt)) { setLastError("all_reduce: unsupported dtype"); return TTB_ERR_UNSUPPORTED; }
  if (!ncclOp(reduce_type, op)) { setLastError("all_reduce: unsupported reduce type (Std/Var)"); return TTB_ERR_UNSUPPORTED; }
  ProfScope prof("nccl_all_reduce", 0, double(count) * dtypeSize(dtype), asStream(stream));
  TTB_NCCL(api.allReduce(in, out, count, dt, op, static_cast<ncclComm_t>(comm), asStream(stream)));
  countLaunch();
  return TTB_OK;
}

int ttb_all_gather(void *comm, const void *in, void *out, size_t send_count, int dtype, void *stream) {
  TTB_CHECK(comm && in && out, "null argument");
  TTB_NCCL_READY();
  ncclDataType_t dt;
  if (!ncclType(dtype, dt)) { setLastError("all_gather: unsupported dtype"); return TTB_ERR_UNSUPPORTED; }
  ProfScope prof("nccl_all_gather", 0, double(send_count) * dtypeSize(dtype), asStream(stream));
  TTB_NCCL(api.allGather(in, out, send_count, dt, static_cast<ncclComm_t>(comm), asStream(stream)));
  countLaunch();
  return TTB_OK;
}

int ttb_reduce_scatter(void *comm, const void *in, void *out, size_t recv_count, int dtype, int reduce_type,
                       void *stream) {
  TTB_CHECK(comm && in && out, "null argument");
  TTB_NCCL_READY();
  ncclDataType_t dt;
  ncclRedOp_t op;
  if (!ncclType(dtype, dt)) { setLastError("reduce_scatter: unsupported dtype"); return TTB_ERR_UNSUPPORTED; }
  if (!ncclOp(reduce_type, op)) { setLastError("reduce_scatter: unsupported reduce type"); return TTB_ERR_UNSUPPORTED; }
  ProfScope prof("nccl_reduce_scatter", 0, double(recv_count) * dtypeSize(dtype), asStream(stream));
  TTB_NCCL(api.reduceScatter(in, out, recv_count, dt, op, static_cast<ncclComm_t>(comm), asStream(stream)));
  countLaunch();
  return TTB_OK;
}

int ttb_broadcast(void *comm, const void *in, void *out, size_t count, int dtype, int root, void *stream) {
  TTB_CHECK(comm && in && out, "null argument");
  TTB_NCCL_READY();
  ncclDataType_t dt;
  if (!ncclType(dtype, dt)) { setLastError("broadcast: unsupported dtype"); return TTB_ERR_UNSUPPORTED; }
  TTB_NCCL(api.broadcast(in, out, count, dt, root, static_cast<ncclComm_t>(comm), asStream(stream)));
  countLaunch();
  return TTB_OK;
}

} // extern "C"
