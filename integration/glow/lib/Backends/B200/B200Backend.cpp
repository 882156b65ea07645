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

bool B200Backend::isOpSupported(const NodeInfo &NI) const {
  switch (NI.getKind()) {
  case Kinded::Kind::FusedRowwiseQuantizedSparseLengthsWeightedSumNodeKind:
    // all four fused kinds, fp32 or fp16 result, int32/int64 indices, int32 lengths
    return NI.getInElemTy(FusedRowwiseQuantizedSparseLengthsWeightedSumNode::LengthsIdx) == ElemKind::Int32ITy;
  case Kinded::Kind::IntNBitSplitEmbeddingBagsNodeKind:
  case Kinded::Kind::IntNBitSplitEmbeddingWeightedBagsNodeKind:
    // int32 / int64 indices and offsets of one type; fp32 or fp16 result
    return NI.getInElemTy(IntNBitSplitEmbeddingBagsNode::IndicesIdx) == NI.getInElemTy(IntNBitSplitEmbeddingBagsNode::OffsetsIdx);
  case Kinded::Kind::DynamicRowwiseQuantizedFullyConnectedNodeKind:
  case Kinded::Kind::DynamicQuantizedFullyConnectedNodeKind:
    // fp16 activations and result, int8 weights, fp32 bias (what the Interpreter implements)
    return NI.getInElemTy(DynamicQuantizedFullyConnectedNode::InputIdx) == ElemKind::Float16Ty &&
           NI.getOutElemTy(DynamicQuantizedFullyConnectedNode::ResultIdx) == ElemKind::Float16Ty;
  case Kinded::Kind::EmbeddingBagByteRowwiseOffsetsNodeKind:
  case Kinded::Kind::RowwiseQuantizedFullyConnectedNodeKind:
  case Kinded::Kind::ChannelwiseQuantizedConvolutionNodeKind:
    return true;
  case Kinded::Kind::FullyConnectedNodeKind:
  case Kinded::Kind::MatMulNodeKind:
  case Kinded::Kind::ConvolutionNodeKind:
  case Kinded::Kind::AddNodeKind:
  case Kinded::Kind::SubNodeKind:
  case Kinded::Kind::MaxNodeKind:
  case Kinded::Kind::MinNodeKind:
  case Kinded::Kind::MulNodeKind:
  case Kinded::Kind::DivNodeKind:
  case Kinded::Kind::BatchedAddNodeKind:
  case Kinded::Kind::ReluNodeKind:
  case Kinded::Kind::MaxPoolNodeKind:
  case Kinded::Kind::AvgPoolNodeKind:
  case Kinded::Kind::RescaleQuantizedNodeKind:
    return NI.allInputsAndOutputsHaveSameElemKind({ElemKind::Int8QTy}, /*ignoreIn*/ {FullyConnectedNode::BiasIdx});
  case Kinded::Kind::SparseLengthsWeightedSumNodeKind:
    return NI.getInElemTy(SparseLengthsWeightedSumNode::DataIdx) == ElemKind::FloatTy;
  case Kinded::Kind::SplatNodeKind:
  case Kinded::Kind::InsertTensorNodeKind:
  case Kinded::Kind::QuantizeNodeKind:
  case Kinded::Kind::DequantizeNodeKind:
  case Kinded::Kind::TransposeNodeKind:
  case Kinded::Kind::SaveNodeKind:
  case Kinded::Kind::ReshapeNodeKind:
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

runtime::DeviceManager *B200Backend::createDeviceManager(const runtime::DeviceConfig &deviceConfig) {
  return new runtime::B200DeviceManager(deviceConfig);
}
