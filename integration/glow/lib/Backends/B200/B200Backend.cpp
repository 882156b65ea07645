#include "B200Backend.h"
#include "B200DeviceManager.h"
#include "B200Function.h"

#include "glow/Backend/BackendUtils.h"
#include "glow/Graph/Nodes.h"
#include "glow/IR/IR.h"
#include "glow/Optimizer/IROptimizer/IROptimizer.h"

#include <cuda_runtime.h>

using namespace glow;

unsigned B200Backend::numDevices() {
  int n = 0;
  return cudaGetDeviceCount(&n) == cudaSuccess ? (unsigned)n : 0u;
}

std::vector<unsigned> B200Backend::scanDeviceIDs() {
  std::vector<unsigned> ids(numDevices());
  for (unsigned i = 0; i < ids.size(); i++) ids[i] = i;
  return ids;
}

Expected<std::unique_ptr<CompiledFunction>> B200Backend::compile(Function *F, const BackendOptions &opts) const {
  auto IR = generateAndOptimizeIR(F, *this, shouldShareBuffers());
  if (opts.autoInstrument) autoInstrument(getTraceInfo(), IR.get());
  return compileIR(std::move(IR));
}

std::unique_ptr<CompiledFunction> B200Backend::compileIR(std::unique_ptr<IRFunction> IR) const {
  // One allocator per slab, like LLVMBackend::compileIRWithoutConstants (LLVMBackend.cpp:687-712).
  MemoryAllocator constants("ConstantWeights", 0), placeholders("MutableWeights", 0), activations("Activations", 0);
  runtime::RuntimeBundle bundle = runtime::RuntimeBundle::create(*IR, constants, placeholders, activations);
  return glow::make_unique<B200Function>(std::move(IR), std::move(bundle));
}

// The predicates of B200Ops.def.
namespace {
bool supportsAny(const NodeInfo &) { return true; }
bool supportsInt8(const NodeInfo &NI) {
  // all inputs and outputs Int8QTy; the bias of FullyConnected / Convolution may be Int32QTy
  return NI.allInputsAndOutputsHaveSameElemKind({ElemKind::Int8QTy}, /*ignoreIn*/ {FullyConnectedNode::BiasIdx}) ||
         NI.allInputsAndOutputsHaveSameElemKind({ElemKind::Int8QTy});
}
bool supportsFusedPool(const NodeInfo &NI) {
  // every fused / rowwise kind, fp32 or fp16 result, int32 / int64 indices -- the lengths are int32
  for (unsigned i = 0, e = NI.getNumInputs(); i < e; i++)
    if (NI.getInName(i) == "Lengths") return NI.getInElemTy(i) == ElemKind::Int32ITy;
  return true;
}
bool supportsF32Table(const NodeInfo &NI) { return NI.getInElemTy(SparseLengthsSumNode::DataIdx) == ElemKind::FloatTy; }
bool supportsSplitEmbedding(const NodeInfo &NI) {
  return NI.getInElemTy(IntNBitSplitEmbeddingBagsNode::IndicesIdx) == NI.getInElemTy(IntNBitSplitEmbeddingBagsNode::OffsetsIdx);
}
bool supportsDynamicFC(const NodeInfo &NI) {
  // fp16 activations and result, int8 weights, fp32 bias (what the Interpreter implements)
  return NI.getInElemTy(DynamicQuantizedFullyConnectedNode::InputIdx) == ElemKind::Float16Ty &&
         NI.getOutElemTy(DynamicQuantizedFullyConnectedNode::ResultIdx) == ElemKind::Float16Ty;
}
bool supportsPool(const NodeInfo &NI) { return NI.allInputsAndOutputsHaveSameElemKind({ElemKind::Int8QTy}); }
} // namespace

bool B200Backend::isOpSupported(const NodeInfo &NI) const {
  switch (NI.getKind()) {
#define B200_OP(NODE, INST, RUNTIME, PRED)                                                                                      \
  case Kinded::Kind::NODE##NodeKind:                                                                                            \
    return supports##PRED(NI);
#include "B200Ops.def"
#undef B200_OP
  // no instruction of their own: Save becomes a Copy, Reshape a TensorView, Concat a run of
  // InsertTensor (Lower.cpp), all of which B200Function::translate handles
  case Kinded::Kind::SaveNodeKind:
  case Kinded::Kind::ReshapeNodeKind:
  case Kinded::Kind::ConcatNodeKind:
    return true;
  default:
    return false;  // the heterogeneous partitioner routes everything else to another backend
  }
}

bool B200Backend::shouldLower(const Node *N) const {
  switch (N->getKind()) {
  case Kinded::Kind::ReluNodeKind:
  case Kinded::Kind::ClipNodeKind:
  case Kinded::Kind::FullyConnectedNodeKind:
  case Kinded::Kind::ConvolutionNodeKind:
  case Kinded::Kind::SparseLengthsSumNodeKind:
    return false;
  default:
    return true;
  }
}

bool B200Backend::supportsFusedActivation(Node *parent, Node *activation) const {
  const bool conv = parent->getKind() == Kinded::Kind::ConvolutionNodeKind ||
                    parent->getKind() == Kinded::Kind::ChannelwiseQuantizedConvolutionNodeKind;
  const bool act = activation->getKind() == Kinded::Kind::ReluNodeKind || activation->getKind() == Kinded::Kind::ClipNodeKind ||
                   activation->getKind() == Kinded::Kind::LeakyReluNodeKind;
  return conv && act;
}

bool B200Backend::canDoIndexTypeDemotion(ElemKind fromTy, ElemKind toTy, PrecisionConfiguration &precConfig) const {
  precConfig.precisionModeKindSet.insert(Kinded::Kind::FusedRowwiseQuantizedSparseLengthsWeightedSumNodeKind);
  precConfig.precisionModeKindSet.insert(Kinded::Kind::EmbeddingBagByteRowwiseOffsetsNodeKind);
  return fromTy == ElemKind::Int64ITy && toTy == ElemKind::Int32ITy;
}

// Two execution contexts per network: the inputs of the next request arrive while this one runs.
unsigned B200Backend::getContextCount(CompilationContext &) const { return 2; }

// Device-resident tensors: with enableDRT the tensors bound to a network's placeholders are
// declared resident at the placeholders' device addresses, so that a tensor one partition wrote
// is read by the next from where it lies (B200Function::execute copies nothing for a tensor that
// is resident on its own device).  enableP2P needs nothing here: partitions on other B200s get
// their inputs from peer memory through the same addresses (glowb200_peer_buffer_*).
Error B200Backend::bindContexts(llvm::ArrayRef<runtime::ContextBinding> bindings, const runtime::DAGNode *root, bool enableP2P,
                                bool enableDRT, int64_t stateId) {
  (void)root; (void)enableP2P; (void)stateId;
  if (!enableDRT) return Error::success();
  for (const auto &cb : bindings) {
    auto *dm = dynamic_cast<runtime::B200DeviceManager *>(cb.device);
    if (!dm) continue;  // another backend's partition
    for (auto &PH : cb.context->getPlaceholderBindings()->pairs()) {
      if (PH.first->isStatic()) continue;
      void *where = dm->placeholderAddress(cb.networkName, PH.first->getName().str());
      if (where) PH.second.moveToDevice(dm, where);
    }
  }
  return Error::success();
}

runtime::DeviceManager *B200Backend::createDeviceManager(const runtime::DeviceConfig &deviceConfig) {
  return new runtime::B200DeviceManager(deviceConfig);
}
