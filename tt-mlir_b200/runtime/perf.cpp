// perf::Env: the reference's Tracy messages (runtime/lib/common/perf.cpp) as NVTX marks and ranges.
// nvtx3 is header-only: without a profiler attached a call is one pointer check.
#include "tt/runtime/perf.h"

#include <atomic>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

namespace tt::runtime::perf {

static std::atomic<std::uint64_t> g_emitted{0};

static bool envSwitch() {
  const char *e = std::getenv("TT_RUNTIME_ENABLE_PERF_TRACE");
  return e && e[0] && std::strcmp(e, "0") != 0;
}

Env &Env::get(std::uint32_t dumpDeviceRate, bool enablePerfTrace, const std::string &tracyProgramMetadata) {
  static Env config(dumpDeviceRate, enablePerfTrace || envSwitch(), tracyProgramMetadata);
  return config;
}

static void mark(const Env &env, TracyLogTag tag, const std::string &text) {
  if (!env.enablePerfTrace) return;
  const std::string message = toString(tag) + ";" + text;
  nvtxMarkA(message.c_str());
  g_emitted.fetch_add(1, std::memory_order_relaxed);
}

void Env::tracyLogOpLocation(const std::string &locInfo) const { mark(*this, TracyLogTag::MLIR_OP_LOCATION, locInfo); }
void Env::tracyLogConstEvalProgram(bool constEvalOp) const { mark(*this, TracyLogTag::MLIR_CONST_EVAL_OP, constEvalOp ? "true" : "false"); }
void Env::tracyLogInputLayoutConversion(bool conv) const { mark(*this, TracyLogTag::MLIR_INPUT_LAYOUT_CONVERSION_OP, conv ? "true" : "false"); }
void Env::tracyLogProgramMetadata(const std::string &metaData) const { mark(*this, TracyLogTag::MLIR_PROGRAM_METADATA, metaData); }
void Env::setProgramMetadata(const std::string &programMetadata) { tracyProgramMetadata = programMetadata; }

void Env::rangePush(const std::string &name) const {
  if (!enablePerfTrace) return;
  nvtxRangePushA(name.c_str());
  g_emitted.fetch_add(1, std::memory_order_relaxed);
}
void Env::rangePop() const {
  if (!enablePerfTrace) return;
  nvtxRangePop();
}
std::uint64_t Env::emitted() { return g_emitted.load(std::memory_order_relaxed); }

} // namespace tt::runtime::perf
