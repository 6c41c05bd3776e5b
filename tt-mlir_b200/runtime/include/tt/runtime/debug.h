// Debug hooks and counters of the tt::runtime API (reference: runtime/include/tt/runtime/debug.h,
// Hooks :77-158, Stats :175-208).  Hooks are a process-wide singleton; when any operator
// callback is registered the executor runs op by op (no cross-op fusion) so that every
// intermediate tensor a callback may ask for exists.
#ifndef TT_RUNTIME_DEBUG_H
#define TT_RUNTIME_DEBUG_H

#include <functional>
#include <mutex>
#include <optional>
#include <string>
#include <unordered_map>

#include "tt/runtime/types.h"

namespace tt::runtime::debug {

struct Hooks {
  using OperationCallbackFn = std::function<void(Binary, CallbackContext, OpContext)>;
  using ProgramCallbackFn = std::function<void(Binary, CallbackContext)>;

  // Registers the given callbacks (a nullopt argument leaves that slot unchanged) and returns
  // the singleton.
  static const Hooks &get(std::optional<OperationCallbackFn> preOperatorCallback = std::nullopt,
                          std::optional<OperationCallbackFn> postOperatorCallback = std::nullopt,
                          std::optional<ProgramCallbackFn> preProgramCallback = std::nullopt,
                          std::optional<ProgramCallbackFn> postProgramCallback = std::nullopt);

  const std::optional<OperationCallbackFn> &getPreOperatorCallback() const { return preOperatorCallback; }
  const std::optional<OperationCallbackFn> &getPostOperatorCallback() const { return postOperatorCallback; }
  const std::optional<ProgramCallbackFn> &getpreProgramCallback() const { return preProgramCallback; }
  const std::optional<ProgramCallbackFn> &getpostProgramCallback() const { return postProgramCallback; }

  void unregisterHooks() const {
    preOperatorCallback = std::nullopt;
    postOperatorCallback = std::nullopt;
    preProgramCallback = std::nullopt;
    postProgramCallback = std::nullopt;
  }

private:
  Hooks() = default;
  mutable std::optional<OperationCallbackFn> preOperatorCallback;
  mutable std::optional<OperationCallbackFn> postOperatorCallback;
  mutable std::optional<ProgramCallbackFn> preProgramCallback;
  mutable std::optional<ProgramCallbackFn> postProgramCallback;
};

struct Stats {
  static Stats &get();
  void incrementStat(const std::string &stat, std::int64_t value = 1);
  std::int64_t getStat(const std::string &stat) const;
  void removeStat(const std::string &stat);
  void clear();
  std::string toString() const;

private:
  Stats() = default;
  mutable std::mutex mutex;
  std::unordered_map<std::string, std::int64_t> counters;
};

// Runtime switches read from the environment once (names follow the reference where one
// exists: TT_RUNTIME_SYNC_AFTER_OP, runtime/lib/ttnn/program_executor.cpp:781-789).
struct Env {
  static const Env &get();
  bool syncAfterOp;     // TT_RUNTIME_SYNC_AFTER_OP=1: synchronise the stream after every op
  bool disableFusion;   // TTB_DISABLE_FUSION=1: execute the op list one op per launch
  bool disableTcgen05;  // TTB_DISABLE_TCGEN05=1: route every contraction to the SIMT kernel
};

} // namespace tt::runtime::debug

#endif
