#include "B200Function.h"

#include "glow/Graph/Graph.h"
#include "glow/Flags/Flags.h"
#include "glow/IR/Instrs.h"
#include "glow/Support/Error.h"

using namespace glow;

namespace {
int fusedKind(ElemKind k) {
  switch (k) {
  case ElemKind::UInt8FusedQTy: return GLOWB200_UINT8_FUSED;
  case ElemKind::UInt8FusedFP16QTy: return GLOWB200_UINT8_FUSED_FP16;
  case ElemKind::UInt4FusedQTy: return GLOWB200_UINT4_FUSED;
  default: return GLOWB200_UINT4_FUSED_FP16;
  }
}
Error fromRuntime(int rc) {
  if (rc == GLOWB200_OK) return Error::success();
  auto code = rc == GLOWB200_RUNTIME_NET_NOT_FOUND             ? ErrorValue::ErrorCode::RUNTIME_NET_NOT_FOUND
              : rc == GLOWB200_RUNTIME_OUT_OF_DEVICE_MEMORY    ? ErrorValue::ErrorCode::RUNTIME_OUT_OF_DEVICE_MEMORY
              : rc == GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE   ? ErrorValue::ErrorCode::RUNTIME_DEVICE_NONRECOVERABLE
                                                               : ErrorValue::ErrorCode::RUNTIME_ERROR;
  return MAKE_ERR(code, glowb200_last_error());
}
} // namespace

B200Function::B200Function(std::unique_ptr<IRFunction> F, runtime::RuntimeBundle &&bundle)
    : CompiledFunction(std::move(bundle)), F_(std::move(F)) {}

B200Function::~B200Function() { glowb200_function_destroy(fn_); }

void B200Function::collectConstants(const Module *module) {
  if (fn_) return;
  EXIT_ON_ERR(translate(module));
}

Error B200Function::translate(const Module *module) {
  fn_ = glowb200_function_create(F_->getGraph()->getName().str().c_str());
  std::unordered_map<const Value *, int> sym;
  // WeightVars: constants carry their payload, placeholders are bound per request.
  for (auto *W : F_->getWeights()) {
    const size_t bytes = W->getType()->getSizeInBytes();
    if (auto *C = module->getConstantByName(W->getName())) {
      sym[W] = glowb200_function_add_symbol(fn_, W->getName().str().c_str(), GLOWB200_SYMBOL_CONSTANT, bytes,
                                            C->getPayload().getUnsafePtr());
    } else {
      sym[W] = glowb200_function_add_symbol(fn_, W->getName().str().c_str(), GLOWB200_SYMBOL_PLACEHOLDER, bytes, nullptr);
    }
  }
  auto S = [&](const Value *v) {  // symbol of a value, looking through tensor views
    while (auto *TV = llvm::dyn_cast<TensorViewInst>(v)) v = TV->getSrc();
    return sym.at(v);
  };
  for (const auto &I : F_->getInstrs()) {
    switch (I.getKind()) {
    case Kinded::Kind::AllocActivationInstKind:
      sym[&I] = glowb200_function_add_symbol(fn_, I.getName().str().c_str(), GLOWB200_SYMBOL_ACTIVATION,
                                             llvm::cast<AllocActivationInst>(&I)->getTy()->getSizeInBytes(), nullptr);
      break;
    case Kinded::Kind::DeallocActivationInstKind:
    case Kinded::Kind::TensorViewInstKind:
    case Kinded::Kind::TouchInstKind:
      break;
    case Kinded::Kind::FusedRowwiseQuantizedSparseLengthsWeightedSumInstKind: {
      auto *N = llvm::cast<FusedRowwiseQuantizedSparseLengthsWeightedSumInst>(&I);
      auto *D = N->getData();
      const int32_t ops[5] = {S(N->getDest()), S(D), S(N->getWeights()), S(N->getIndices()), S(N->getLengths())};
      const int64_t ia[9] = {fusedKind(D->getElementType()), (int64_t)D->dims()[0], (int64_t)D->dims()[1],
                             (int64_t)N->getDest()->dims()[1], (int64_t)N->getLengths()->dims()[0],
                             (int64_t)N->getIndices()->dims()[0], N->getIndices()->getElementType() == ElemKind::Int64ITy,
                             N->getDest()->getElementType() == ElemKind::Float16Ty, N->getUseFP16Accumulation()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_FRWQ_SLWS, ops, 5, ia, 9, nullptr, 0)));
      break;
    }
    case Kinded::Kind::RowwiseQuantizedFullyConnectedInstKind: {
      auto *N = llvm::cast<RowwiseQuantizedFullyConnectedInst>(&I);
      const int32_t ops[6] = {S(N->getDest()), S(N->getSrc()), S(N->getWeights()), S(N->getScales()), S(N->getOffsets()), S(N->getBias())};
      const int64_t ia[7] = {(int64_t)N->getSrc()->dims()[0], (int64_t)N->getSrc()->dims()[1], (int64_t)N->getWeights()->dims()[0],
                             N->getSrc()->getType()->getOffset(), N->getBias()->getType()->getOffset(),
                             N->getDest()->getType()->getOffset(), 0};
      const float fa[3] = {N->getSrc()->getType()->getScale(), N->getBias()->getType()->getScale(), N->getDest()->getType()->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_RWQ_FC, ops, 6, ia, 7, fa, 3)));
      break;
    }
    case Kinded::Kind::ChannelwiseQuantizedConvolutionInstKind: {
      auto *N = llvm::cast<ChannelwiseQuantizedConvolutionInst>(&I);
      const int32_t ops[8] = {S(N->getDest()), S(N->getSrc()), S(N->getFilter()), S(N->getBias()), S(N->getFilterScales()),
                              S(N->getFilterOffsets()), S(N->getBiasScales()), S(N->getBiasOffsets())};
      auto in = N->getSrc()->dims(), out = N->getDest()->dims();
      auto k = N->getKernels(), s = N->getStrides(), p = N->getPads(), d = N->getDilation();
      const int64_t ia[21] = {(int64_t)in[0], (int64_t)in[1], (int64_t)in[2], (int64_t)in[3], (int64_t)out[1], (int64_t)out[2],
                              (int64_t)out[3], k[0], k[1], s[0], s[1], p[0], p[1], p[2], p[3], N->getGroup(), d[0], d[1],
                              N->getSrc()->getType()->getOffset(), N->getDest()->getType()->getOffset(),
                              (int64_t)N->getFusedActivation()};
      const float fa[2] = {N->getSrc()->getType()->getScale(), N->getDest()->getType()->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_CWQ_CONV, ops, 8, ia, 21, fa, 2)));
      break;
    }
    case Kinded::Kind::ElementAddInstKind: {
      auto *N = llvm::cast<ElementAddInst>(&I);
      const int32_t ops[3] = {S(N->getDest()), S(N->getLHS()), S(N->getRHS())};
      const int64_t ia[4] = {(int64_t)N->getDest()->size(), N->getDest()->getType()->getOffset(), N->getLHS()->getType()->getOffset(),
                             N->getRHS()->getType()->getOffset()};
      const float fa[3] = {N->getLHS()->getType()->getScale(), N->getRHS()->getType()->getScale(), N->getDest()->getType()->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_ADD, ops, 3, ia, 4, fa, 3)));
      break;
    }
    case Kinded::Kind::ElementSubInstKind:
    case Kinded::Kind::ElementMaxInstKind:
    case Kinded::Kind::ElementMinInstKind:
    case Kinded::Kind::ElementMulInstKind:
    case Kinded::Kind::ElementDivInstKind: {
      // dest, lhs, rhs are operands 0..2 of every arithmetic instruction
      const Value *dst = I.getOperand(0).first, *lhs = I.getOperand(1).first, *rhs = I.getOperand(2).first;
      const auto k = I.getKind();
      const bool muldiv = k == Kinded::Kind::ElementMulInstKind || k == Kinded::Kind::ElementDivInstKind;
      const int64_t sel = k == Kinded::Kind::ElementSubInstKind   ? GLOWB200_BINARY_SUB
                          : k == Kinded::Kind::ElementMaxInstKind ? GLOWB200_BINARY_MAX
                          : k == Kinded::Kind::ElementMinInstKind ? GLOWB200_BINARY_MIN
                                                                  : (k == Kinded::Kind::ElementDivInstKind);
      const int32_t ops[3] = {S(dst), S(lhs), S(rhs)};
      const int64_t ia[5] = {(int64_t)dst->size(), dst->getType()->getOffset(), lhs->getType()->getOffset(),
                             rhs->getType()->getOffset(), sel};
      const float fa[3] = {lhs->getType()->getScale(), rhs->getType()->getScale(), dst->getType()->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, muldiv ? GLOWB200_INSTR_MULDIV_I8 : GLOWB200_INSTR_BINARY_I8,
                                                                  ops, 3, ia, 5, fa, 3)));
      break;
    }
    case Kinded::Kind::BatchedAddInstKind: {
      auto *N = llvm::cast<BatchedAddInst>(&I);
      auto *B = N->getBatch();
      const int64_t slices = (int64_t)B->dims()[0];
      const int32_t ops[3] = {S(N->getDest()), S(B), S(N->getSlice())};
      const int64_t ia[6] = {slices, slices ? (int64_t)B->size() / slices : 0, N->getDest()->getType()->getOffset(),
                             B->getType()->getOffset(), N->getSlice()->getType()->getOffset(),
                             N->getSlice()->getElementType() == ElemKind::Int32QTy};
      const float fa[3] = {B->getType()->getScale(), N->getSlice()->getType()->getScale(), N->getDest()->getType()->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_BATCHED_ADD_I8, ops, 3, ia, 6, fa, 3)));
      break;
    }
    case Kinded::Kind::QuantizeInstKind:
    case Kinded::Kind::DequantizeInstKind: {
      const bool q = I.getKind() == Kinded::Kind::QuantizeInstKind;
      const Value *dst = I.getOperand(0).first, *src = I.getOperand(1).first;
      const Type *qt = q ? dst->getType() : src->getType();
      const int32_t ops[2] = {S(dst), S(src)};
      const int64_t ia[2] = {(int64_t)dst->size(), qt->getOffset()};
      const float fa[1] = {qt->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, q ? GLOWB200_INSTR_QUANTIZE : GLOWB200_INSTR_DEQUANTIZE, ops, 2, ia, 2, fa, 1)));
      break;
    }
    case Kinded::Kind::CopyInstKind: {
      auto *N = llvm::cast<CopyInst>(&I);
      const int32_t ops[2] = {S(N->getDest()), S(N->getSrc())};
      const int64_t ia[1] = {(int64_t)N->getDest()->getType()->getSizeInBytes()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_COPY, ops, 2, ia, 1, nullptr, 0)));
      break;
    }
    case Kinded::Kind::FullyConnectedInstKind: {
      auto *N = llvm::cast<FullyConnectedInst>(&I);
      const int32_t ops[4] = {S(N->getDest()), S(N->getSrc()), S(N->getWeights()), S(N->getBias())};
      const Type *in = N->getSrc()->getType(), *w = N->getWeights()->getType(), *b = N->getBias()->getType(), *o = N->getDest()->getType();
      const int64_t ia[7] = {(int64_t)in->dims()[0], (int64_t)in->dims()[1], (int64_t)w->dims()[1], in->getOffset(), w->getOffset(),
                             b->getOffset(), o->getOffset()};
      const float fa[4] = {in->getScale(), w->getScale(), b->getScale(), o->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_FC_I8, ops, 4, ia, 7, fa, 4)));
      break;
    }
    case Kinded::Kind::MatMulInstKind: {
      auto *N = llvm::cast<MatMulInst>(&I);
      const int32_t ops[3] = {S(N->getDest()), S(N->getLHS()), S(N->getRHS())};
      const Type *l = N->getLHS()->getType(), *r = N->getRHS()->getType(), *o = N->getDest()->getType();
      const int64_t ia[6] = {(int64_t)l->dims()[0], (int64_t)l->dims()[1], (int64_t)r->dims()[1], l->getOffset(), r->getOffset(), o->getOffset()};
      const float fa[3] = {l->getScale(), r->getScale(), o->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_MATMUL_I8, ops, 3, ia, 6, fa, 3)));
      break;
    }
    case Kinded::Kind::ReluInstKind:
    case Kinded::Kind::RescaleQuantizedInstKind: {
      const bool relu = I.getKind() == Kinded::Kind::ReluInstKind;
      const Value *dst = I.getOperand(0).first, *src = I.getOperand(1).first;
      const int32_t ops[2] = {S(dst), S(src)};
      const int64_t ia[3] = {(int64_t)dst->size(), src->getType()->getOffset(), dst->getType()->getOffset()};
      const float fa[2] = {src->getType()->getScale(), dst->getType()->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, relu ? GLOWB200_INSTR_RELU : GLOWB200_INSTR_RESCALE, ops, 2, ia, 3, fa, 2)));
      break;
    }
    case Kinded::Kind::SplatInstKind: {
      auto *N = llvm::cast<SplatInst>(&I);
      const int32_t ops[1] = {S(N->getDest())};
      const int64_t ia[2] = {(int64_t)N->getDest()->size(), N->getDest()->getElementType() == ElemKind::Float16Ty};
      const float fa[1] = {N->getValue()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_SPLAT, ops, 1, ia, 2, fa, 1)));
      break;
    }
    case Kinded::Kind::SparseLengthsWeightedSumInstKind: {
      auto *N = llvm::cast<SparseLengthsWeightedSumInst>(&I);
      const int32_t ops[5] = {S(N->getDest()), S(N->getData()), S(N->getWeights()), S(N->getIndices()), S(N->getLengths())};
      const int64_t ia[5] = {(int64_t)N->getData()->dims()[0], (int64_t)N->getDest()->dims()[1], (int64_t)N->getLengths()->dims()[0],
                             (int64_t)N->getIndices()->dims()[0], N->getIndices()->getElementType() == ElemKind::Int64ITy};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_SLWS_F32, ops, 5, ia, 5, nullptr, 0)));
      break;
    }
    case Kinded::Kind::EmbeddingBagByteRowwiseOffsetsInstKind: {
      auto *N = llvm::cast<EmbeddingBagByteRowwiseOffsetsInst>(&I);
      auto *D = N->getData();
      const int32_t ops[5] = {S(N->getDest()), S(D), S(N->getWeights()), S(N->getIndices()), S(N->getOffsets())};
      const int64_t ia[10] = {fusedKind(D->getElementType()), (int64_t)D->dims()[0], (int64_t)D->dims()[1], (int64_t)N->getDest()->dims()[1],
                              (int64_t)N->getOffsets()->dims()[0], (int64_t)N->getIndices()->dims()[0],
                              N->getIndices()->getElementType() == ElemKind::Int64ITy, N->getHasEndOffset(),
                              N->getDest()->getElementType() == ElemKind::Float16Ty, N->getUseFP16Accumulation()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_EMBEDDING_BAG, ops, 5, ia, 10, nullptr, 0)));
      break;
    }
    case Kinded::Kind::IntNBitSplitEmbeddingBagsInstKind:
    case Kinded::Kind::IntNBitSplitEmbeddingWeightedBagsInstKind: {
      // the two instructions differ by the IndiceWeight operand only
      auto *W = llvm::dyn_cast<IntNBitSplitEmbeddingWeightedBagsInst>(&I);
      auto *U = llvm::dyn_cast<IntNBitSplitEmbeddingBagsInst>(&I);
      Value *dest = W ? W->getDest() : U->getDest(), *dev = W ? W->getDevWeights() : U->getDevWeights();
      Value *uvm = W ? W->getUvmWeights() : U->getUvmWeights(), *pl = W ? W->getWeightsPlacements() : U->getWeightsPlacements();
      Value *wo = W ? W->getWeightsOffsets() : U->getWeightsOffsets(), *tys = W ? W->getWeightsTys() : U->getWeightsTys();
      Value *dimo = W ? W->getDimOffsets() : U->getDimOffsets(), *idx = W ? W->getIndices() : U->getIndices();
      Value *off = W ? W->getOffsets() : U->getOffsets();
      const int64_t tables = (int64_t)dimo->dims()[0] - 1;
      const int32_t ops[10] = {S(dest), S(dev), S(uvm), S(pl), S(wo), S(tys), S(dimo), S(idx), S(off), W ? S(W->getIndiceWeight()) : -1};
      const int64_t ia[13] = {(int64_t)dev->getType()->getSizeInBytes(), (int64_t)uvm->getType()->getSizeInBytes(), tables,
                              W ? W->getTotalDims() : U->getTotalDims(), (int64_t)idx->dims()[0],
                              tables ? ((int64_t)off->dims()[0] - 1) / tables : 0, idx->getElementType() == ElemKind::Int64ITy,
                              wo->getElementType() == ElemKind::Int64ITy, (int64_t)(W ? W->getPoolingMode() : U->getPoolingMode()),
                              W && W->getIndiceWeight()->getElementType() == ElemKind::Float16Ty,
                              dest->getElementType() == ElemKind::Float16Ty, glow::flags::ConvertFusedScaleOffsetToFP32,
                              glow::interpreter::flags::RowAlignmentBytes};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_SPLIT_EMBEDDING, ops, 10, ia, 13, nullptr, 0)));
      break;
    }
    case Kinded::Kind::DynamicRowwiseQuantizedFullyConnectedInstKind: {
      auto *N = llvm::cast<DynamicRowwiseQuantizedFullyConnectedInst>(&I);
      if (!N->getIsSymmetric() || !N->getIsPerBatchElement())  // the Interpreter asserts the same (InterpreterNodes.cpp:4713-4714)
        return MAKE_ERR(ErrorValue::ErrorCode::COMPILE_UNSUPPORTED_NODE_AFTER_OPTIMIZE, "B200: only symmetric per-batch-element dynamic quantization");
      const int32_t ops[6] = {S(N->getDest()), S(N->getSrc()), S(N->getWeights()), S(N->getBias()), S(N->getScales()), S(N->getOffsets())};
      const int64_t ia[4] = {(int64_t)N->getSrc()->dims()[0], (int64_t)N->getSrc()->dims()[1], (int64_t)N->getDest()->dims()[1], 0};
      const float fa[1] = {0.f};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_DYN_QUANTIZED_FC, ops, 6, ia, 4, fa, 1)));
      break;
    }
    case Kinded::Kind::DynamicQuantizedFullyConnectedInstKind: {
      auto *N = llvm::cast<DynamicQuantizedFullyConnectedInst>(&I);
      if (!N->getIsSymmetric() || !N->getIsPerBatchElement())
        return MAKE_ERR(ErrorValue::ErrorCode::COMPILE_UNSUPPORTED_NODE_AFTER_OPTIMIZE, "B200: only symmetric per-batch-element dynamic quantization");
      auto *WT = N->getWeights()->getType();
      const int32_t ops[6] = {S(N->getDest()), S(N->getSrc()), S(N->getWeights()), S(N->getBias()), -1, -1};
      const int64_t ia[4] = {(int64_t)N->getSrc()->dims()[0], (int64_t)N->getSrc()->dims()[1], (int64_t)N->getDest()->dims()[1], WT->getOffset()};
      const float fa[1] = {WT->getScale()};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_DYN_QUANTIZED_FC, ops, 6, ia, 4, fa, 1)));
      break;
    }
    case Kinded::Kind::InsertTensorInstKind: {
      // the lowered Concat of pooled vectors: a [rows, width] block into a wider row-major tensor
      auto *N = llvm::cast<InsertTensorInst>(&I);
      const auto dd = N->getDest()->dims(), sd = N->getSrc()->dims();
      const size_t eb = N->getDest()->getType()->getElementSize();
      if (dd.size() != 2 || N->getCount() != 1 || N->getOffsets()[0] != 0)
        return MAKE_ERR(ErrorValue::ErrorCode::COMPILE_UNSUPPORTED_NODE_AFTER_OPTIMIZE, "B200: only column-wise InsertTensor is supported");
      const int32_t ops[2] = {S(N->getDest()), S(N->getSrc())};
      const int64_t ia[4] = {(int64_t)sd[0], (int64_t)(sd[1] * eb), (int64_t)(dd[1] * eb), (int64_t)(N->getOffsets()[1] * eb)};
      RETURN_IF_ERR(fromRuntime(glowb200_function_add_instruction(fn_, GLOWB200_INSTR_INSERT_TENSOR, ops, 2, ia, 4, nullptr, 0)));
      break;
    }
    // MaxPool / AvgPool / Transpose / CPUMaxSplat-style max-with-immediate follow the same pattern
    // with GLOWB200_INSTR_MAXPOOL / _AVGPOOL / _TRANSPOSE / _MAXSPLAT (attribute lists in runtime.cu).
    default:
      return MAKE_ERR(ErrorValue::ErrorCode::COMPILE_UNSUPPORTED_NODE_AFTER_OPTIMIZE,
                      "B200: instruction " + std::string(I.getKindName()) + " is not supported");
    }
  }
  return fromRuntime(glowb200_function_compile(fn_));
}

Error B200Function::execute(ExecutionContext *context) {
  // Bind every placeholder the function uses to its host tensor; the device manager copies in,
  // runs, and copies back (a shorter tensor is a partial tensor).
  std::vector<std::string> names;
  std::vector<const char *> cnames;
  std::vector<void *> bufs;
  std::vector<size_t> bytes;
  std::vector<int> dirs;
  const auto &table = getRuntimeBundle().getSymbolTable();
  for (auto &PH : context->getPlaceholderBindings()->pairs()) {
    auto it = table.find(PH.first->getName().str());
    if (it == table.end() || it->second.symbolCategory != glow::runtime::SymbolCategory::Placeholder) continue;
    if (PH.first->isStatic()) continue;  // moved once by transferStaticPlaceholderToDevice
    names.push_back(PH.first->getName().str());
    bufs.push_back(PH.second.getUnsafePtr());
    bytes.push_back(PH.second.getUnpaddedSizeInBytes());
    // the input / output marks of the symbol table decide which way a tensor travels
    dirs.push_back((it->second.input ? GLOWB200_BINDING_INPUT : 0) | (it->second.output ? GLOWB200_BINDING_OUTPUT : 0));
  }
  for (auto &n : names) cnames.push_back(n.c_str());
  return fromRuntime(glowb200_device_manager_run_function_io(dm_, F_->getGraph()->getName().str().c_str(), cnames.data(),
                                                             bufs.data(), bytes.data(), dirs.data(), (int)names.size()));
}
