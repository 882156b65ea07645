#ifndef GLOW_BACKENDS_B200_B200FUNCTION_H
#define GLOW_BACKENDS_B200_B200FUNCTION_H

#include "glow/Backend/CompiledFunction.h"
#include "glow/IR/IR.h"

#include "glow_b200.h"

namespace glow {

/// A Glow IR function translated, instruction by instruction, into a glowb200_function.
class B200Function final : public CompiledFunction {
  std::unique_ptr<IRFunction> F_;
  glowb200_function *fn_{nullptr};
  /// Set by the device manager that loaded the function: the library's handle and the Glow
  /// object (the owner of tensors resident on this device).
  glowb200_device_manager *dm_{nullptr};
  const void *owner_{nullptr};

public:
  B200Function(std::unique_ptr<IRFunction> F, runtime::RuntimeBundle &&bundle);
  ~B200Function() override;

  /// Walks the IR once and builds the runtime function; constants are read from \p module
  /// (Provisioner compiles with collectConstants=false and the device manager translates from
  /// addNetwork, before the module may be stripped: lib/Runtime/Provisioner/Provisioner.cpp:
  /// 270-283).  An instruction without a translation, or a view that is not a contiguous piece
  /// of its tensor, is COMPILE_UNSUPPORTED_NODE_AFTER_OPTIMIZE -- returned, never fatal.
  Error translate(const Module *module);
  /// The CompiledFunction hook; errors cannot leave it, so the device manager calls translate()
  /// itself and this only covers callers that compiled with collectConstants=true.
  void collectConstants(const Module *module) override;
  Error execute(ExecutionContext *context) override;
  std::string getCompileBackendName() const override { return "B200"; }

  glowb200_function *handle() const { return fn_; }
  void setDeviceManager(glowb200_device_manager *dm, const void *owner) {
    dm_ = dm;
    owner_ = owner;
  }
};

} // namespace glow
#endif
