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
  /// Set by the device manager that loaded the function.
  glowb200_device_manager *dm_{nullptr};

  Error translate(const Module *module);

public:
  B200Function(std::unique_ptr<IRFunction> F, runtime::RuntimeBundle &&bundle);
  ~B200Function() override;

  /// Constants are read from the module once (Provisioner compiles with collectConstants=false and
  /// the device manager calls this from addNetwork: lib/Runtime/Provisioner/Provisioner.cpp:270-283).
  void collectConstants(const Module *module) override;
  Error execute(ExecutionContext *context) override;
  std::string getCompileBackendName() const override { return "B200"; }

  glowb200_function *handle() const { return fn_; }
  void setDeviceManager(glowb200_device_manager *dm) { dm_ = dm; }
};

} // namespace glow
#endif
