// Collectives over NVLink / NVSwitch through NCCL, for the mesh ops of a 1xN device mesh
// (reference call sites: ::ttnn::all_reduce / all_gather / reduce_scatter in
// runtime/lib/ttnn/operations/ccl/{all_reduce,all_gather,reduce_scatter}.cpp, which ride on
// tt-fabric).  NCCL is opened with dlopen on first use so that the kernel library loads on
// machines without it and single-GPU programs never touch it.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

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
  decltype(&ncclSend) send = nullptr;
  decltype(&ncclRecv) recv = nullptr;
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
    TTB_SYM(send, ncclSend)
    TTB_SYM(recv, ncclRecv)
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


// ---- all-reduce over peer memory ------------------------------------------------------------
// Every rank of a 1xN mesh owns a workspace that all other ranks map (CUDA IPC between
// processes, peer access inside one process).  One kernel per rank does the whole all-reduce:
//   A  copy the local operand into the own workspace (skipped when the producer already wrote
//      it there, see ttb_symm_input_buffer); peers can now read it
//   B  reduce slice `rank`: read that slice from every rank over NVLink, sum in f32 in rank
//      order (the same bits on every rank), optionally add a residual; the result goes to the
//      local output and is pushed into every peer's workspace
//   C  copy the slices the peers pushed from the own workspace to the local output
// with a flag barrier between A/B and B/C.  Remote traffic per rank is (n-1)/n of the operand
// in each direction, loads and stores in the same loop, so both directions of the links work at
// once.  Work is split so that block b touches the same elements in every phase on every rank;
// a barrier is then per block (block b waits for block b of the peers), which needs no
// grid-wide synchronisation.  Flags carry a launch counter and the data and result regions
// alternate between two copies per launch, so nothing is ever reset.
// Pushed mode (MODE 2): the GEMM that produces the operand has already stored, from its epilogue,
// every row block of its partial result into the workspace of the rank that owns the block
// (ttb_symm_push_targets), so phase A is empty, phase B sums n local copies (no remote read), and
// only the push of the reduced slice and phase C remain after the barrier: the reduce-scatter
// half of the exchange has overlapped the GEMM.
// Waits are bounded: when a peer does not show up within about a second the kernel records it
// in the status word and carries on (the result of that launch is then invalid).
constexpr int SYMM_MAX_RANKS = 8;
constexpr int SYMM_MAX_BLOCKS = 512;
constexpr int SYMM_THREADS = 512;
constexpr size_t SYMM_FLAG_BYTES = 2 * SYMM_MAX_BLOCKS * SYMM_MAX_RANKS * sizeof(uint32_t);

struct SymmParams {
  int rank, n;
  char *ws[SYMM_MAX_RANKS]; // every rank's workspace as mapped on this device; ws[rank] is local
  size_t dataOff, resultOff; // this launch's regions inside a workspace
  uint32_t token;            // first barrier waits for token, second for token + 1
  int oneShot;               // every rank reduces the whole operand itself: no push, no second barrier
  int ownOnly;               // reduce-scatter: only the own slice is wanted (stored densely at out[0..]); no push, no second barrier
  int *status;
  long long waitCycles; // how long a barrier may spin on a peer's flag before it gives up (SM clock cycles)
};

__device__ __forceinline__ void symmStoreFlag(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t symmLoadFlag(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-level barrier across ranks: block b of every rank has finished the phase before it.
// The poll is a relaxed load (hundreds of blocks spin at once); one fence after it orders the
// reads that follow.
__device__ __forceinline__ void symmBarrier(const SymmParams &p, int which, uint32_t token) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < p.n && t != p.rank) {
    const size_t slot = (static_cast<size_t>(which) * SYMM_MAX_BLOCKS + blockIdx.x) * SYMM_MAX_RANKS;
    symmStoreFlag(reinterpret_cast<uint32_t *>(p.ws[t]) + slot + p.rank, token); // release: orders the block's writes
    const uint32_t *mine = reinterpret_cast<const uint32_t *>(p.ws[p.rank]) + slot + t;
    const long long start = clock64();
    uint32_t spins = 0;
    while (static_cast<int32_t>(symmLoadFlag(mine) - token) < 0) {
      if ((++spins & 255u) == 0 && clock64() - start > p.waitCycles) {
        atomicCAS(p.status, 0, ((which + 1) << 8) | (t + 1));
        break;
      }
    }
    __threadfence_system();
  }
  __syncthreads();
}

template <typename T> struct SymmVec { static constexpr int N = 16 / sizeof(T); };

// NR: compile-time bound on the rank count (2, 4 or 8), which sizes the registers that hold the
// loads in flight.
// MODE: 0 the operand is copied into the workspace, 1 the producer wrote it there, 2 pushed.
template <typename T, bool RESIDUAL, int MODE, int NR>
__global__ void __launch_bounds__(SYMM_THREADS)
    symmAllReduceKernel(SymmParams p, const uint4 *__restrict__ in, const uint4 *__restrict__ residual,
                        uint4 *__restrict__ out, size_t nvec) {
  constexpr int V = SymmVec<T>::N;
  constexpr int U = NR == 8 ? 2 : 4;
  constexpr bool STAGED = MODE != 0;
  const size_t per = (nvec + p.n - 1) / p.n; // vectors per slice
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t first = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;

  // A: publish the local operand (already in place when the producer wrote into the workspace).
  if (!STAGED) {
    uint4 *myData = reinterpret_cast<uint4 *>(p.ws[p.rank] + p.dataOff);
    if (p.oneShot) {
      // the peers read everything, with the element-to-block map of the reduce loop below
      for (size_t i = first; i < nvec; i += stride) myData[i] = __ldcs(in + i);
    } else {
      for (int s = 0; s < p.n; ++s) {
        if (s == p.rank) continue; // the own slice is read from `in`
        const size_t lo = s * per, hi = lo + per < nvec ? lo + per : nvec;
        for (size_t i = lo + first; i < hi; i += stride) myData[i] = __ldcs(in + i);
      }
    }
  }
  symmBarrier(p, 0, p.token);

  // B: reduce the own slice, U vectors per thread and iteration with every load issued before
  // the first use, so that a thread has U * n remote loads in flight.
  // One-shot mode (two ranks, or operands so small that latency dominates): the same loop over
  // the whole operand, nothing pushed, and the launch ends here.
  {
    const size_t lo = p.oneShot ? 0 : p.rank * per;
    const size_t hi = p.oneShot ? nvec : (lo + per < nvec ? lo + per : nvec);
    const bool push = !p.oneShot && !p.ownOnly;
    const size_t outShift = p.ownOnly ? lo : 0; // reduce-scatter: `out` holds the own slice only
    for (size_t i0 = lo + first; i0 < hi; i0 += stride * U) {
      uint4 v[U][NR];
      uint4 rv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + u * stride;
        if (i < hi) {
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            if (r < p.n) {
              if (MODE == 2) {
                // rank r's partial of the own slice, pushed here by r's GEMM
                v[u][r] = __ldcg(reinterpret_cast<const uint4 *>(p.ws[p.rank] + p.dataOff) + r * per + (i - lo));
              } else {
                v[u][r] = (r == p.rank && !STAGED) ? __ldcs(in + i)
                                                   : __ldcg(reinterpret_cast<const uint4 *>(p.ws[r] + p.dataOff) + i);
              }
            }
          }
          if (RESIDUAL) rv[u] = __ldcs(residual + i);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + u * stride;
        if (i < hi) {
          float acc[V];
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] = 0.0f;
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            if (r < p.n) {
              const T *e = reinterpret_cast<const T *>(&v[u][r]);
#pragma unroll
              for (int j = 0; j < V; ++j) acc[j] = __fadd_rn(acc[j], toF32(e[j]));
            }
          }
          uint4 o;
          T *oe = reinterpret_cast<T *>(&o);
          if (RESIDUAL) {
            const T *re = reinterpret_cast<const T *>(&rv[u]);
#pragma unroll
            for (int j = 0; j < V; ++j) oe[j] = fromF32<T>(__fadd_rn(toF32(fromF32<T>(acc[j])), toF32(re[j])));
          } else {
#pragma unroll
            for (int j = 0; j < V; ++j) oe[j] = fromF32<T>(acc[j]);
          }
          out[i - outShift] = o;
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            if (push && r < p.n && r != p.rank) reinterpret_cast<uint4 *>(p.ws[r] + p.resultOff)[i] = o;
          }
        }
      }
    }
  }
  if (p.oneShot || p.ownOnly) return;
  symmBarrier(p, 1, p.token + 1);

  // C: the slices the peers pushed.
  {
    const uint4 *mine = reinterpret_cast<const uint4 *>(p.ws[p.rank] + p.resultOff);
    for (int s = 0; s < p.n; ++s) {
      if (s == p.rank) continue;
      const size_t lo = s * per, hi = lo + per < nvec ? lo + per : nvec;
      for (size_t i = lo + first; i < hi; i += stride) out[i] = __ldcg(mine + i);
    }
  }
}

template <typename T, bool RESIDUAL, int MODE, int NR>
static int symmLaunch(const SymmParams &p, const void *in, const void *residual, void *out, size_t nvec, cudaStream_t st) {
  // All blocks of all ranks have to be resident at the same time (they wait for each other).
  static std::mutex mu;
  static int perSmOf[64] = {};
  int dev = 0;
  TTB_CUDA(cudaGetDevice(&dev));
  TTB_CHECK(dev >= 0 && dev < 64, "device ordinal out of range");
  int perSm[64];
  {
    std::lock_guard<std::mutex> lock(mu); // several threads may drive different devices of one mesh
    if (!perSmOf[dev]) {
      int n = 0;
      TTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, symmAllReduceKernel<T, RESIDUAL, MODE, NR>, SYMM_THREADS, 0));
      TTB_CHECK(n >= 1, "all-reduce kernel does not fit on an SM");
      perSmOf[dev] = n > 2 ? 2 : n;
    }
    perSm[dev] = perSmOf[dev];
  }
  const size_t work = p.oneShot ? nvec : (nvec + p.n - 1) / p.n;
  size_t blocks = (work + SYMM_THREADS - 1) / SYMM_THREADS;
  size_t cap = static_cast<size_t>(smCount()) * perSm[dev];
  if (cap > SYMM_MAX_BLOCKS) cap = SYMM_MAX_BLOCKS;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  symmAllReduceKernel<T, RESIDUAL, MODE, NR><<<static_cast<unsigned>(blocks), SYMM_THREADS, 0, st>>>(
      p, static_cast<const uint4 *>(in), static_cast<const uint4 *>(residual), static_cast<uint4 *>(out), nvec);
  countLaunch();
  TTB_LAUNCH_CHECK();
  return TTB_OK;
}

template <typename T>
static int symmDispatch(const SymmParams &p, const void *in, const void *residual, void *out, size_t nvec, int mode,
                        cudaStream_t st) {
#define TTB_SYMM_MODE(RES, NRv)                                                                       \
  switch (mode) {                                                                                     \
  case 0: return symmLaunch<T, RES, 0, NRv>(p, in, residual, out, nvec, st);                          \
  case 1: return symmLaunch<T, RES, 1, NRv>(p, in, residual, out, nvec, st);                          \
  default: return symmLaunch<T, RES, 2, NRv>(p, in, residual, out, nvec, st);                         \
  }
#define TTB_SYMM_NR(NRv)                                                                              \
  if (residual) { TTB_SYMM_MODE(true, NRv) }                                                          \
  TTB_SYMM_MODE(false, NRv)
  if (p.n <= 2) { TTB_SYMM_NR(2) }
  if (p.n <= 4) { TTB_SYMM_NR(4) }
  TTB_SYMM_NR(8)
#undef TTB_SYMM_NR
#undef TTB_SYMM_MODE
}

struct Symm {
  int rank = 0, n = 1, device = 0;
  bool ipc = false;
  char *ws[SYMM_MAX_RANKS] = {};
  size_t maxBytes = 0; // largest operand
  uint32_t launches = 0;
  int *status = nullptr;
  long long waitCycles = 2000000000ll; // about a second
};

static size_t symmTotalBytes(size_t maxBytes) { return SYMM_FLAG_BYTES + 4 * maxBytes; }

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

// One-directional copy between two ranks (point_to_point).  Sender and receiver call their half; when one process
// drives both ranks the two calls sit inside one ttb_group_start / ttb_group_end pair.
int ttb_send(void *comm, const void *in, size_t count, int dtype, int peer, void *stream) {
  TTB_CHECK(comm && in, "null argument");
  TTB_NCCL_READY();
  ncclDataType_t dt;
  if (!ncclType(dtype, dt)) { setLastError("send: unsupported dtype"); return TTB_ERR_UNSUPPORTED; }
  TTB_NCCL(api.send(in, count, dt, peer, static_cast<ncclComm_t>(comm), asStream(stream)));
  countLaunch();
  return TTB_OK;
}

int ttb_recv(void *comm, void *out, size_t count, int dtype, int peer, void *stream) {
  TTB_CHECK(comm && out, "null argument");
  TTB_NCCL_READY();
  ncclDataType_t dt;
  if (!ncclType(dtype, dt)) { setLastError("recv: unsupported dtype"); return TTB_ERR_UNSUPPORTED; }
  TTB_NCCL(api.recv(out, count, dt, peer, static_cast<ncclComm_t>(comm), asStream(stream)));
  countLaunch();
  return TTB_OK;
}

// ---- all-reduce over peer memory: host side -----------------------------------------------------
int ttb_symm_create_rank(void **symm, void *comm, int rank, int nranks, size_t max_bytes, void *stream) {
  TTB_CHECK(symm && comm, "null argument");
  TTB_CHECK(nranks >= 2 && nranks <= SYMM_MAX_RANKS && rank >= 0 && rank < nranks, "bad rank / world size");
  TTB_NCCL_READY();
  max_bytes = (max_bytes + 255) / 256 * 256;
  auto *s = new Symm();
  // Whatever has been built is torn down again on every error return below.
  struct Guard {
    Symm *s;
    char *handles = nullptr;
    ~Guard() {
      if (handles) cudaFree(handles);
      if (s) ttb_symm_destroy(s);
    }
  } guard{s};
  s->rank = rank;
  s->n = nranks;
  s->ipc = true;
  s->maxBytes = max_bytes;
  TTB_CUDA(cudaGetDevice(&s->device));
  char *local = nullptr;
  TTB_CUDA(cudaMalloc(reinterpret_cast<void **>(&local), symmTotalBytes(max_bytes)));
  s->ws[rank] = local;
  TTB_CUDA(cudaMemset(local, 0, SYMM_FLAG_BYTES));
  TTB_CUDA(cudaMalloc(reinterpret_cast<void **>(&s->status), 128));
  TTB_CUDA(cudaMemset(s->status, 0, 128));
  s->ws[rank] = local;
  // Exchange the IPC handles through the communicator the mesh already has.
  cudaIpcMemHandle_t mine;
  TTB_CUDA(cudaIpcGetMemHandle(&mine, local));
  char *devHandles = nullptr;
  TTB_CUDA(cudaMalloc(reinterpret_cast<void **>(&devHandles), sizeof(mine) * (nranks + 1)));
  guard.handles = devHandles;
  cudaStream_t st = asStream(stream);
  TTB_CUDA(cudaMemcpyAsync(devHandles + sizeof(mine) * nranks, &mine, sizeof(mine), cudaMemcpyHostToDevice, st));
  TTB_NCCL(api.allGather(devHandles + sizeof(mine) * nranks, devHandles, sizeof(mine), ncclChar,
                         static_cast<ncclComm_t>(comm), st));
  std::vector<cudaIpcMemHandle_t> all(nranks);
  TTB_CUDA(cudaMemcpyAsync(all.data(), devHandles, sizeof(mine) * nranks, cudaMemcpyDeviceToHost, st));
  TTB_CUDA(cudaStreamSynchronize(st));
  for (int r = 0; r < nranks; ++r) {
    if (r == rank) continue;
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      setLastError(std::string("cannot map the workspace of rank ") + std::to_string(r) + ": " + cudaGetErrorString(e));
      return TTB_ERR_CUDA;
    }
    s->ws[r] = static_cast<char *>(p);
  }
  // Nobody may touch a peer before every rank has cleared its flags and mapped the others.
  TTB_NCCL(api.allGather(devHandles + sizeof(mine) * nranks, devHandles, sizeof(mine), ncclChar,
                         static_cast<ncclComm_t>(comm), st));
  TTB_CUDA(cudaStreamSynchronize(st));
  guard.handles = nullptr;
  guard.s = nullptr; // handed to the caller
  TTB_CUDA(cudaFree(devHandles));
  *symm = s;
  return TTB_OK;
}

int ttb_symm_create_all(void **symms, int ndev, const int *devices, size_t max_bytes) {
  TTB_CHECK(symms && devices, "null argument");
  TTB_CHECK(ndev >= 2 && ndev <= SYMM_MAX_RANKS, "bad device count");
  max_bytes = (max_bytes + 255) / 256 * 256;
  int before = 0;
  TTB_CUDA(cudaGetDevice(&before));
  std::vector<Symm *> all(ndev);
  for (int i = 0; i < ndev; ++i) {
    TTB_CUDA(cudaSetDevice(devices[i]));
    auto *s = new Symm();
    s->rank = i;
    s->n = ndev;
    s->device = devices[i];
    s->maxBytes = max_bytes;
    char *local = nullptr;
    TTB_CUDA(cudaMalloc(reinterpret_cast<void **>(&local), symmTotalBytes(max_bytes)));
    TTB_CUDA(cudaMemset(local, 0, SYMM_FLAG_BYTES));
    TTB_CUDA(cudaMalloc(reinterpret_cast<void **>(&s->status), 128));
    TTB_CUDA(cudaMemset(s->status, 0, 128));
    s->ws[i] = local;
    all[i] = s;
    for (int j = 0; j < ndev; ++j) {
      if (j == i) continue;
      int can = 0;
      TTB_CUDA(cudaDeviceCanAccessPeer(&can, devices[i], devices[j]));
      if (!can) {
        setLastError("devices " + std::to_string(devices[i]) + " and " + std::to_string(devices[j]) + " have no peer access");
        return TTB_ERR_UNSUPPORTED;
      }
      cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) TTB_CUDA(e);
      (void)cudaGetLastError();
    }
    TTB_CUDA(cudaDeviceSynchronize());
  }
  for (int i = 0; i < ndev; ++i) {
    for (int j = 0; j < ndev; ++j) all[i]->ws[j] = all[j]->ws[j];
    symms[i] = all[i];
  }
  TTB_CUDA(cudaSetDevice(before));
  return TTB_OK;
}

int ttb_symm_destroy(void *symm) {
  if (!symm) return TTB_OK;
  auto *s = static_cast<Symm *>(symm);
  int before = 0;
  cudaGetDevice(&before);
  cudaSetDevice(s->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < s->n; ++r) {
    if (r == s->rank || !s->ws[r]) continue;
    if (s->ipc) cudaIpcCloseMemHandle(s->ws[r]);
  }
  if (s->ws[s->rank]) cudaFree(s->ws[s->rank]);
  if (s->status) cudaFree(s->status);
  (void)cudaGetLastError();
  cudaSetDevice(before);
  delete s;
  return TTB_OK;
}

size_t ttb_symm_max_bytes(void *symm) { return symm ? static_cast<Symm *>(symm)->maxBytes : 0; }

int ttb_symm_input_buffer(void *symm, size_t bytes, void **ptr) {
  TTB_CHECK(symm && ptr, "null argument");
  auto *s = static_cast<Symm *>(symm);
  TTB_CHECK(bytes <= s->maxBytes, "operand larger than the workspace allows");
  *ptr = s->ws[s->rank] + SYMM_FLAG_BYTES + static_cast<size_t>(s->launches & 1u) * s->maxBytes;
  return TTB_OK;
}

int ttb_symm_set_wait_limit(void *symm, long long cycles) {
  TTB_CHECK(symm != nullptr, "null argument");
  static_cast<Symm *>(symm)->waitCycles = cycles > 0 ? cycles : 2000000000ll;
  return TTB_OK;
}

int ttb_symm_launch_count(void *symm, uint32_t *launches) {
  TTB_CHECK(symm && launches, "null argument");
  *launches = static_cast<Symm *>(symm)->launches;
  return TTB_OK;
}

int ttb_symm_set_launch_count(void *symm, uint32_t launches) {
  TTB_CHECK(symm != nullptr, "null argument");
  static_cast<Symm *>(symm)->launches = launches;
  return TTB_OK;
}

int ttb_symm_clear_status(void *symm) {
  TTB_CHECK(symm != nullptr, "null argument");
  auto *s = static_cast<Symm *>(symm);
  TTB_CUDA(cudaMemset(s->status, 0, sizeof(int)));
  return TTB_OK;
}

int ttb_symm_status(void *symm, int *status) {
  TTB_CHECK(symm && status, "null argument");
  auto *s = static_cast<Symm *>(symm);
  TTB_CUDA(cudaMemcpy(status, s->status, sizeof(int), cudaMemcpyDeviceToHost));
  return TTB_OK;
}

int ttb_symm_push_targets(void *symm, size_t bytes, void **targets, int *rank, int *nranks) {
  TTB_CHECK(symm && targets && rank && nranks, "null argument");
  auto *s = static_cast<Symm *>(symm);
  TTB_CHECK(bytes <= s->maxBytes, "operand larger than the workspace allows");
  TTB_CHECK(bytes % (16 * static_cast<size_t>(s->n)) == 0, "operand does not split into 16-byte aligned slices");
  const size_t slice = bytes / s->n;
  for (int o = 0; o < s->n; ++o) {
    targets[o] = s->ws[o] + SYMM_FLAG_BYTES + static_cast<size_t>(s->launches & 1u) * s->maxBytes + s->rank * slice;
  }
  *rank = s->rank;
  *nranks = s->n;
  return TTB_OK;
}

static int symmAllReduceImpl(void *symm, const void *in, const void *residual, void *out, size_t count, int dtype,
                             void *stream, bool pushed, bool ownOnly = false);

int ttb_symm_all_reduce_pushed(void *symm, const void *residual, void *out, size_t count, int dtype, void *stream) {
  TTB_CHECK(symm && out, "null argument");
  return symmAllReduceImpl(symm, out /* unused */, residual, out, count, dtype, stream, true);
}

int ttb_symm_all_reduce(void *symm, const void *in, const void *residual, void *out, size_t count, int dtype,
                        void *stream) {
  TTB_CHECK(symm && in && out, "null argument");
  return symmAllReduceImpl(symm, in, residual, out, count, dtype, stream, false);
}

// The reduce-scatter half alone: `out` receives only this rank's slice of the sum (count / nranks elements: block
// `rank` of the flattened operand) plus the matching part of `residual` (full size, nullable).  Nothing is pushed to
// the peers and the second barrier and the final copy fall away, which is what an all_reduce whose result is only
// read through a mesh_partition of the same axis needs.
int ttb_symm_reduce_scatter(void *symm, const void *in, const void *residual, void *out, size_t count, int dtype,
                            void *stream) {
  TTB_CHECK(symm && in && out, "null argument");
  return symmAllReduceImpl(symm, in, residual, out, count, dtype, stream, false, true);
}

int ttb_symm_reduce_scatter_pushed(void *symm, const void *residual, void *out, size_t count, int dtype, void *stream) {
  TTB_CHECK(symm && out, "null argument");
  return symmAllReduceImpl(symm, out /* unused */, residual, out, count, dtype, stream, true, true);
}

} // extern "C"

static int symmAllReduceImpl(void *symm, const void *in, const void *residual, void *out, size_t count, int dtype,
                             void *stream, bool pushed, bool ownOnly) {
  auto *s = static_cast<Symm *>(symm);
  const size_t es = dtypeSize(dtype);
  const size_t bytes = count * es;
  if ((dtype != kBF16 && dtype != kF16 && dtype != kF32) || bytes % 16 != 0 || bytes > s->maxBytes || !aligned16(in) ||
      !aligned16(out) || (residual && !aligned16(residual))) {
    setLastError("symm_all_reduce: operand type, size or alignment not supported");
    return TTB_ERR_UNSUPPORTED;
  }
  if (count == 0) return TTB_OK;
  SymmParams p;
  p.rank = s->rank;
  p.n = s->n;
  for (int r = 0; r < SYMM_MAX_RANKS; ++r) p.ws[r] = s->ws[r];
  const uint32_t launch = s->launches++;
  const size_t parity = launch & 1u;
  p.dataOff = SYMM_FLAG_BYTES + parity * s->maxBytes;
  p.resultOff = SYMM_FLAG_BYTES + (2 + parity) * s->maxBytes;
  p.token = 2 * launch + 1;
  p.status = s->status;
  p.oneShot = (!pushed && !ownOnly && (s->n == 2 || bytes <= (size_t(256) << 10))) ? 1 : 0;
  p.ownOnly = ownOnly ? 1 : 0;
  if ((pushed || ownOnly) && bytes % (16 * static_cast<size_t>(s->n)) != 0) {
    setLastError("symm_all_reduce: operand does not split into 16-byte aligned slices");
    return TTB_ERR_UNSUPPORTED;
  }
  p.waitCycles = s->waitCycles;
  const size_t nvec = bytes / 16;
  cudaStream_t st = asStream(stream);
  // The producer wrote the operand into this launch's data region (ttb_symm_input_buffer).
  const bool staged = static_cast<const char *>(in) == s->ws[s->rank] + p.dataOff;
  // per rank: (n-1)/n of the operand read from peers and as much pushed to them, the operand and
  // the result once each locally, plus the staging copies
  ProfScope prof("symm_all_reduce", 0, double(bytes) * (2.0 + 2.0 * (s->n - 1) / s->n), st);
  const int mode = pushed ? 2 : (staged ? 1 : 0);
  if (dtype == kBF16) return symmDispatch<__nv_bfloat16>(p, in, residual, out, nvec, mode, st);
  if (dtype == kF16) return symmDispatch<__half>(p, in, residual, out, nvec, mode, st);
  return symmDispatch<float>(p, in, residual, out, nvec, mode, st);
}
