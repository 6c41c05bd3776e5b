// perf::Env of the tt::runtime API for the B200 target.
//
// Same members as runtime/include/tt/runtime/perf.h:13-53 of the reference.  There the messages go
// to Tracy ("MLIR_OP_LOCATION;<loc>", ... -- `ttrt perf` parses them out of the capture); here they are
// NVTX marks with the same text, and while tracing is enabled the executor also brackets every op
// with an NVTX range named "<OpType> <loc>", so that a timeline (Nsight Systems, or any NVTX consumer)
// shows the flatbuffer's ops over the kernels they launched.  With tracing off nothing is emitted.
// Tracing is switched on by Env::get(rate, /*enablePerfTrace=*/true, ...) on its first call, or by the
// environment variable TT_RUNTIME_ENABLE_PERF_TRACE=1.
#ifndef TT_RUNTIME_PERF_H
#define TT_RUNTIME_PERF_H

#include <cstdint>
#include <ostream>
#include <string>

namespace tt::runtime::perf {

enum class TracyLogTag { MLIR_OP_LOCATION, MLIR_CONST_EVAL_OP, MLIR_PROGRAM_METADATA, MLIR_INPUT_LAYOUT_CONVERSION_OP };

inline std::string toString(TracyLogTag tag) {
  switch (tag) {
  case TracyLogTag::MLIR_OP_LOCATION: return "MLIR_OP_LOCATION";
  case TracyLogTag::MLIR_CONST_EVAL_OP: return "MLIR_CONST_EVAL_OP";
  case TracyLogTag::MLIR_PROGRAM_METADATA: return "MLIR_PROGRAM_METADATA";
  case TracyLogTag::MLIR_INPUT_LAYOUT_CONVERSION_OP: return "MLIR_INPUT_LAYOUT_CONVERSION_OP";
  }
  return "";
}

struct Env {
  // The first call fixes the settings (as the reference's function-local static does).
  static Env &get(std::uint32_t dumpDeviceRate = 1000, bool enablePerfTrace = false,
                  const std::string &tracyProgramMetadata = "");

  std::uint32_t dumpDeviceRate;
  bool enablePerfTrace;
  std::string tracyProgramMetadata;

  Env(const Env &) = delete;
  Env &operator=(const Env &) = delete;

  void tracyLogOpLocation(const std::string &locInfo) const;
  void tracyLogConstEvalProgram(bool constEvalOp) const;
  void tracyLogInputLayoutConversion(bool inputLayoutConversionOp) const;
  void tracyLogProgramMetadata(const std::string &metaData) const;
  void setProgramMetadata(const std::string &programMetadata);

  // Additions of this target: the per-op range the executor opens, and a count of everything emitted
  // (what tests look at: NVTX itself has no read-back).
  void rangePush(const std::string &name) const;
  void rangePop() const;
  static std::uint64_t emitted();

private:
  Env(std::uint32_t rate, bool trace, const std::string &meta)
      : dumpDeviceRate(rate), enablePerfTrace(trace), tracyProgramMetadata(meta) {}
};

inline std::ostream &operator<<(std::ostream &os, const Env &env) {
  os << "perf::Env{\n"
     << "\tdumpDeviceRate: " << env.dumpDeviceRate << "\n"
     << "\tenablePerfTrace: " << env.enablePerfTrace << "\n"
     << "\ttracyProgramMetadata: " << env.tracyProgramMetadata << "\n"
     << "}";
  return os;
}

} // namespace tt::runtime::perf

#endif
