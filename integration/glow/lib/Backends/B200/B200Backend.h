// glow::Backend for NVIDIA B200, on the glow_b200 kernel library.
// Not compiled in the glow_b200 repository (Glow needs LLVM, folly, glog); it is the glue a
// maintainer drops into lib/Backends/B200 of a Glow tree.
#ifndef GLOW_BACKENDS_B200_B200BACKEND_H
#define GLOW_BACKENDS_B200_B200BACKEND_H

#include "glow/Backend/Backend.h"
#include "glow/Backends/DeviceManager.h"

namespace glow {

class B200Backend final : public BackendUsingGlowIR {
public:
  ~B200Backend() override = default;

  std::string getBackendName() const override { return getName(); }
  static std::string getName() { return "B200"; }
  static unsigned numDevices();                    // cudaGetDeviceCount
  static std::vector<unsigned> scanDeviceIDs();

  Expected<std::unique_ptr<CompiledFunction>> compile(Function *F, const BackendOptions &opts) const override;
  std::unique_ptr<CompiledFunction> compileIR(std::unique_ptr<IRFunction> IR) const override;

  bool isOpSupported(const NodeInfo &NI) const override;
  // Keep FullyConnected / Convolution / SparseLengthsSum / Relu whole, as the CPU backend does
  // (lib/Backends/CPU/CPUBackend.cpp:71-84).
  bool shouldLower(const Node *N) const override;
  // Relu and Clip fold into (channelwise) convolutions and rowwise FCs.
  bool supportsFusedActivation(Node *parent, Node *activation) const override;
  bool supportsPartialTensors() const override { return true; }
  bool supportsStaticPlaceholders() const override { return true; }
  // int64 index tensors may be demoted to int32, the SLS family included (the CPU backend keeps
  // theirs, CPUBackend.cpp:147-160): tables have fewer than 2^31 rows and the host link carries
  // half the bytes.
  bool canDoIndexTypeDemotion(ElemKind fromTy, ElemKind toTy, PrecisionConfiguration &precConfig) const override;

  unsigned getContextCount(CompilationContext &cctx) const override;
  Error bindContexts(llvm::ArrayRef<runtime::ContextBinding> bindings, const runtime::DAGNode *root, bool enableP2P,
                     bool enableDRT, int64_t stateId) override;

  runtime::DeviceManager *createDeviceManager(const runtime::DeviceConfig &deviceConfig) override;
};

} // namespace glow
#endif
