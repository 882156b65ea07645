#include "B200Function.h"

#include "glow/Flags/Flags.h"
#include "glow/Graph/Graph.h"
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
Error unsupported(const std::string &what) {
  return MAKE_ERR(ErrorValue::ErrorCode::COMPILE_UNSUPPORTED_NODE_AFTER_OPTIMIZE, "B200: " + what);
}
int64_t I64(dim_t v) { return (int64_t)v; }

/// Walks one IR function and emits runtime instructions.  One emit method per IR instruction of
/// B200Ops.def; translate() dispatches through the same list.
class Translator {
  glowb200_function *fn_;
  const Module *module_;
  std::unordered_map<const Value *, int> sym_;
  std::string bad_;  // why the last operand could not be resolved
  unsigned derived_ = 0;

  /// An operand: the symbol behind \p v and the byte offset of \p v inside it.  A TensorView
  /// with offsets is a piece of its source; it can be addressed by an offset alone when the
  /// piece is contiguous there: a reshape (all offsets zero, same number of elements), or a
  /// slice of leading dimensions (every dimension behind the first one that is narrower than
  /// the source's is taken whole, and the ones before it have extent 1).
  bool resolve(const Value *v, int32_t &id, int64_t &off) {
    off = 0;
    while (auto *TV = llvm::dyn_cast<TensorViewInst>(v)) {
      const Value *src = TV->getSrc();
      auto sd = src->dims(), vd = TV->getTy()->dims();
      auto offs = TV->getOffsets();
      bool zero = true;
      for (auto o : offs) zero = zero && o == 0;
      if (!zero || TV->getTy()->size() != src->getType()->size()) {
        if (vd.size() != sd.size() || offs.size() != sd.size()) {
          bad_ = "a TensorView that changes rank and has offsets (" + TV->getName().str() + ")";
          return false;
        }
        size_t k = 0;  // first dimension the view narrows
        while (k < sd.size() && vd[k] == sd[k]) k++;
        for (size_t i = 0; i < k; i++)
          if (vd[i] != 1 && k < sd.size()) {
            bad_ = "a TensorView that is not a contiguous piece of its tensor (" + TV->getName().str() + ")";
            return false;
          }
        for (size_t i = k + 1; i < sd.size(); i++)
          if (vd[i] != sd[i] || offs[i] != 0) {
            bad_ = "a TensorView that is not a contiguous piece of its tensor (" + TV->getName().str() + ")";
            return false;
          }
        int64_t linear = 0, stride = 1;
        for (size_t i = sd.size(); i-- > 0;) {
          linear += I64(offs[i]) * stride;
          stride *= I64(sd[i]);
        }
        off += linear * (int64_t)src->getType()->getElementSize();
      }
      v = src;
    }
    auto it = sym_.find(v);
    if (it == sym_.end()) {
      bad_ = "an operand that is neither a weight nor an activation (" + v->getName().str() + ")";
      return false;
    }
    id = it->second;
    return true;
  }

  /// Emits one runtime instruction; \p operands may hold nullptr for an operand left out.
  Error emit(int kind, llvm::ArrayRef<const Value *> operands, llvm::ArrayRef<int64_t> ia, llvm::ArrayRef<float> fa = {}) {
    std::vector<int32_t> ids(operands.size(), -1);
    std::vector<int64_t> offs(operands.size(), 0);
    for (size_t i = 0; i < operands.size(); i++)
      if (operands[i] && !resolve(operands[i], ids[i], offs[i])) return unsupported(bad_);
    return fromRuntime(glowb200_function_add_instruction_views(fn_, kind, ids.data(), offs.data(), (int)ids.size(), ia.data(),
                                                               (int)ia.size(), fa.data(), (int)fa.size()));
  }

  /// A constant the translator makes up (per-channel copies of a per-tensor scale, the unit
  /// weights of an unweighted sum): a symbol of its own, registered under a fresh Value key.
  std::vector<std::unique_ptr<WeightVar>> made_;
  const Value *makeConstant(const std::string &tag, TypeRef ty, const void *data, size_t bytes) {
    const std::string name = tag + ".b200." + std::to_string(derived_++);
    made_.push_back(glow::make_unique<WeightVar>(name, ty, WeightVar::MutabilityKind::Constant));
    sym_[made_.back().get()] = glowb200_function_add_symbol(fn_, name.c_str(), GLOWB200_SYMBOL_CONSTANT, bytes, data);
    return made_.back().get();
  }

public:
  Translator(glowb200_function *fn, const Module *module) : fn_(fn), module_(module) {}

  Error addWeight(const WeightVar *W, const IRFunction &F) {
    const size_t bytes = W->getType()->getSizeInBytes();
    int id;
    if (auto *C = module_->getConstantByName(W->getName())) {
      id = glowb200_function_add_symbol(fn_, W->getName().str().c_str(), GLOWB200_SYMBOL_CONSTANT, bytes, C->getPayload().getUnsafePtr());
    } else {
      // a static placeholder is written once and shared by the execution contexts
      auto *PH = module_->getPlaceholderByNameSlow(W->getName());
      id = glowb200_function_add_symbol(fn_, W->getName().str().c_str(),
                                        PH && PH->isStatic() ? GLOWB200_SYMBOL_STATIC : GLOWB200_SYMBOL_PLACEHOLDER, bytes, nullptr);
    }
    if (id < 0) return fromRuntime(GLOWB200_RUNTIME_ERROR);
    sym_[W] = id;
    return Error::success();
  }

  Error addActivation(const AllocActivationInst *A) {
    const int id = glowb200_function_add_symbol(fn_, A->getName().str().c_str(), GLOWB200_SYMBOL_ACTIVATION,
                                                A->getTy()->getSizeInBytes(), nullptr);
    if (id < 0) return fromRuntime(GLOWB200_RUNTIME_ERROR);
    sym_[A] = id;
    return Error::success();
  }

  // ---- embedding gather-pool family ---------------------------------------------------------
  Error fusedPool(const Value *dest, const Value *data, const Value *weights, const Value *indices, const Value *lengths,
                  bool fp16Accumulation) {
    const int64_t ia[9] = {fusedKind(data->getElementType()), I64(data->dims()[0]), I64(data->dims()[1]), I64(dest->dims()[1]),
                           I64(lengths->dims()[0]), I64(indices->dims()[0]), indices->getElementType() == ElemKind::Int64ITy,
                           dest->getElementType() == ElemKind::Float16Ty, fp16Accumulation};
    return emit(GLOWB200_INSTR_FRWQ_SLWS, {dest, data, weights, indices, lengths}, ia);
  }
  Error emitFusedRowwiseQuantizedSparseLengthsWeightedSum(const FusedRowwiseQuantizedSparseLengthsWeightedSumInst *N) {
    return fusedPool(N->getDest(), N->getData(), N->getWeights(), N->getIndices(), N->getLengths(), N->getUseFP16Accumulation());
  }
  Error emitFusedRowwiseQuantizedSparseLengthsSum(const FusedRowwiseQuantizedSparseLengthsSumInst *N) {
    // the sum is the weighted sum with unit weights (lib/Optimizer/Lower/Lower.cpp:1576-1606), in
    // the result's element type
    const dim_t n = N->getIndices()->dims()[0];
    const bool half = N->getDest()->getElementType() == ElemKind::Float16Ty;
    std::vector<uint16_t> ones16(half ? n : 0, 0x3C00);
    std::vector<float> ones32(half ? 0 : n, 1.0f);
    auto ty = module_->uniqueType(half ? ElemKind::Float16Ty : ElemKind::FloatTy, {n});
    const Value *ones = makeConstant(N->getName().str(), ty, half ? (const void *)ones16.data() : (const void *)ones32.data(),
                                     n * (half ? 2 : 4));
    return fusedPool(N->getDest(), N->getData(), ones, N->getIndices(), N->getLengths(), N->getUseFP16Accumulation());
  }
  Error emitRowwiseQuantizedSparseLengthsWeightedSum(const RowwiseQuantizedSparseLengthsWeightedSumInst *N) {
    auto *D = N->getData();
    const int64_t ia[5] = {I64(D->dims()[0]), I64(D->dims()[1]), I64(N->getLengths()->dims()[0]), I64(N->getIndices()->dims()[0]),
                           N->getIndices()->getElementType() == ElemKind::Int64ITy};
    return emit(GLOWB200_INSTR_RWQ_SLWS, {N->getDest(), D, N->getScales(), N->getOffsets(), N->getWeights(), N->getIndices(), N->getLengths()}, ia);
  }
  Error plainPool(const Value *dest, const Value *data, const Value *weights, const Value *indices, const Value *lengths) {
    const int64_t ia[5] = {I64(data->dims()[0]), I64(dest->dims()[1]), I64(lengths->dims()[0]), I64(indices->dims()[0]),
                           indices->getElementType() == ElemKind::Int64ITy};
    return emit(GLOWB200_INSTR_SLWS_F32, {dest, data, weights, indices, lengths}, ia);
  }
  Error emitSparseLengthsWeightedSum(const SparseLengthsWeightedSumInst *N) {
    return plainPool(N->getDest(), N->getData(), N->getWeights(), N->getIndices(), N->getLengths());
  }
  Error emitSparseLengthsSum(const SparseLengthsSumInst *N) {
    return plainPool(N->getDest(), N->getData(), nullptr, N->getIndices(), N->getLengths());
  }
  Error emitEmbeddingBagByteRowwiseOffsets(const EmbeddingBagByteRowwiseOffsetsInst *N) {
    auto *D = N->getData();
    const int64_t ia[10] = {fusedKind(D->getElementType()), I64(D->dims()[0]), I64(D->dims()[1]), I64(N->getDest()->dims()[1]),
                            I64(N->getOffsets()->dims()[0]), I64(N->getIndices()->dims()[0]),
                            N->getIndices()->getElementType() == ElemKind::Int64ITy, N->getHasEndOffset(),
                            N->getDest()->getElementType() == ElemKind::Float16Ty, N->getUseFP16Accumulation()};
    return emit(GLOWB200_INSTR_EMBEDDING_BAG, {N->getDest(), D, N->getWeights(), N->getIndices(), N->getOffsets()}, ia);
  }
  template <class InstT> Error splitEmbedding(const InstT *N, const Value *indiceWeight) {
    const Value *dev = N->getDevWeights(), *uvm = N->getUvmWeights(), *wo = N->getWeightsOffsets(), *idx = N->getIndices();
    const Value *off = N->getOffsets(), *dimo = N->getDimOffsets();
    const int64_t tables = I64(dimo->dims()[0]) - 1;
    const int64_t ia[13] = {(int64_t)dev->getType()->getSizeInBytes(), (int64_t)uvm->getType()->getSizeInBytes(), tables,
                            (int64_t)N->getTotalDims(), I64(idx->dims()[0]), tables ? (I64(off->dims()[0]) - 1) / tables : 0,
                            idx->getElementType() == ElemKind::Int64ITy, wo->getElementType() == ElemKind::Int64ITy,
                            (int64_t)N->getPoolingMode(), indiceWeight && indiceWeight->getElementType() == ElemKind::Float16Ty,
                            N->getDest()->getElementType() == ElemKind::Float16Ty, glow::flags::ConvertFusedScaleOffsetToFP32,
                            glow::interpreter::flags::RowAlignmentBytes};
    return emit(GLOWB200_INSTR_SPLIT_EMBEDDING,
                {N->getDest(), dev, uvm, N->getWeightsPlacements(), wo, N->getWeightsTys(), dimo, idx, off, indiceWeight}, ia);
  }
  Error emitIntNBitSplitEmbeddingBags(const IntNBitSplitEmbeddingBagsInst *N) { return splitEmbedding(N, nullptr); }
  Error emitIntNBitSplitEmbeddingWeightedBags(const IntNBitSplitEmbeddingWeightedBagsInst *N) {
    return splitEmbedding(N, N->getIndiceWeight());
  }

  // ---- contractions -------------------------------------------------------------------------
  Error emitRowwiseQuantizedFullyConnected(const RowwiseQuantizedFullyConnectedInst *N) {
    const Type *in = N->getSrc()->getType(), *b = N->getBias()->getType(), *o = N->getDest()->getType();
    const int64_t ia[7] = {I64(in->dims()[0]), I64(in->dims()[1]), I64(N->getWeights()->dims()[0]), in->getOffset(), b->getOffset(),
                           o->getOffset(), 0};
    const float fa[3] = {in->getScale(), b->getScale(), o->getScale()};
    return emit(GLOWB200_INSTR_RWQ_FC, {N->getDest(), N->getSrc(), N->getWeights(), N->getScales(), N->getOffsets(), N->getBias()}, ia, fa);
  }
  Error emitDynamicRowwiseQuantizedFullyConnected(const DynamicRowwiseQuantizedFullyConnectedInst *N) {
    if (!N->getIsSymmetric() || !N->getIsPerBatchElement())  // the Interpreter asserts the same (InterpreterNodes.cpp:4713-4714)
      return unsupported("only symmetric per-batch-element dynamic quantization");
    const int64_t ia[4] = {I64(N->getSrc()->dims()[0]), I64(N->getSrc()->dims()[1]), I64(N->getDest()->dims()[1]), 0};
    const float fa[1] = {0.f};
    return emit(GLOWB200_INSTR_DYN_QUANTIZED_FC, {N->getDest(), N->getSrc(), N->getWeights(), N->getBias(), N->getScales(), N->getOffsets()}, ia, fa);
  }
  Error emitDynamicQuantizedFullyConnected(const DynamicQuantizedFullyConnectedInst *N) {
    if (!N->getIsSymmetric() || !N->getIsPerBatchElement()) return unsupported("only symmetric per-batch-element dynamic quantization");
    auto *WT = N->getWeights()->getType();
    const int64_t ia[4] = {I64(N->getSrc()->dims()[0]), I64(N->getSrc()->dims()[1]), I64(N->getDest()->dims()[1]), WT->getOffset()};
    const float fa[1] = {WT->getScale()};
    return emit(GLOWB200_INSTR_DYN_QUANTIZED_FC, {N->getDest(), N->getSrc(), N->getWeights(), N->getBias(), nullptr, nullptr}, ia, fa);
  }
  template <class InstT>
  Error conv(const InstT *N, const Value *fScales, const Value *fOffsets, const Value *bScales, const Value *bOffsets) {
    auto in = N->getSrc()->dims(), out = N->getDest()->dims();
    auto k = N->getKernels(), s = N->getStrides(), p = N->getPads(), d = N->getDilation();
    if (in.size() != 4) return unsupported("only 2-D NHWC convolutions");
    const int64_t ia[21] = {I64(in[0]), I64(in[1]), I64(in[2]), I64(in[3]), I64(out[1]), I64(out[2]), I64(out[3]), k[0], k[1], s[0],
                            s[1], p[0], p[1], p[2], p[3], N->getGroup(), d[0], d[1], N->getSrc()->getType()->getOffset(),
                            N->getDest()->getType()->getOffset(), (int64_t)N->getFusedActivation()};
    const float fa[2] = {N->getSrc()->getType()->getScale(), N->getDest()->getType()->getScale()};
    return emit(GLOWB200_INSTR_CWQ_CONV, {N->getDest(), N->getSrc(), N->getFilter(), N->getBias(), fScales, fOffsets, bScales, bOffsets}, ia, fa);
  }
  Error emitChannelwiseQuantizedConvolution(const ChannelwiseQuantizedConvolutionInst *N) {
    return conv(N, N->getFilterScales(), N->getFilterOffsets(), N->getBiasScales(), N->getBiasOffsets());
  }
  Error emitConvolution(const ConvolutionInst *N) {
    // The per-tensor quantized convolution (libjit_conv2d_i8_i32, LLVMIRGen.cpp:2501-2599) is the
    // channelwise one with every channel given the tensor's scale and offset.
    if (N->getLayout() != NHWC) return unsupported("only NHWC convolutions");
    const Type *f = N->getFilter()->getType(), *b = N->getBias()->getType();
    const dim_t oc = N->getDest()->dims()[3];
    std::vector<float> fs(oc, f->getScale()), bs(oc, b->getScale());
    std::vector<int32_t> fo(oc, f->getOffset()), bo(oc, b->getOffset());
    auto fty = module_->uniqueType(ElemKind::FloatTy, {oc}), ity = module_->uniqueType(ElemKind::Int32ITy, {oc});
    const std::string tag = N->getName().str();
    return conv(N, makeConstant(tag, fty, fs.data(), oc * 4), makeConstant(tag, ity, fo.data(), oc * 4),
                makeConstant(tag, fty, bs.data(), oc * 4), makeConstant(tag, ity, bo.data(), oc * 4));
  }
  Error emitFullyConnected(const FullyConnectedInst *N) {
    const Type *in = N->getSrc()->getType(), *w = N->getWeights()->getType(), *b = N->getBias()->getType(), *o = N->getDest()->getType();
    const int64_t ia[7] = {I64(in->dims()[0]), I64(in->dims()[1]), I64(w->dims()[1]), in->getOffset(), w->getOffset(), b->getOffset(),
                           o->getOffset()};
    const float fa[4] = {in->getScale(), w->getScale(), b->getScale(), o->getScale()};
    return emit(GLOWB200_INSTR_FC_I8, {N->getDest(), N->getSrc(), N->getWeights(), N->getBias()}, ia, fa);
  }
  Error emitMatMul(const MatMulInst *N) {
    const Type *l = N->getLHS()->getType(), *r = N->getRHS()->getType(), *o = N->getDest()->getType();
    const int64_t ia[6] = {I64(l->dims()[0]), I64(l->dims()[1]), I64(r->dims()[1]), l->getOffset(), r->getOffset(), o->getOffset()};
    const float fa[3] = {l->getScale(), r->getScale(), o->getScale()};
    return emit(GLOWB200_INSTR_MATMUL_I8, {N->getDest(), N->getLHS(), N->getRHS()}, ia, fa);
  }

  // ---- quantized glue -----------------------------------------------------------------------
  Error emitElementAdd(const ElementAddInst *N) {
    const Type *d = N->getDest()->getType(), *l = N->getLHS()->getType(), *r = N->getRHS()->getType();
    const int64_t ia[4] = {I64(d->size()), d->getOffset(), l->getOffset(), r->getOffset()};
    const float fa[3] = {l->getScale(), r->getScale(), d->getScale()};
    return emit(GLOWB200_INSTR_ADD, {N->getDest(), N->getLHS(), N->getRHS()}, ia, fa);
  }
  Error binary(const Instruction *I, int kind, int64_t selector) {  // dest, lhs, rhs are operands 0..2
    const Value *dst = I->getOperand(0).first, *lhs = I->getOperand(1).first, *rhs = I->getOperand(2).first;
    const int64_t ia[5] = {I64(dst->getType()->size()), dst->getType()->getOffset(), lhs->getType()->getOffset(),
                           rhs->getType()->getOffset(), selector};
    const float fa[3] = {lhs->getType()->getScale(), rhs->getType()->getScale(), dst->getType()->getScale()};
    return emit(kind, {dst, lhs, rhs}, ia, fa);
  }
  Error emitElementSub(const ElementSubInst *N) { return binary(N, GLOWB200_INSTR_BINARY_I8, GLOWB200_BINARY_SUB); }
  Error emitElementMax(const ElementMaxInst *N) { return binary(N, GLOWB200_INSTR_BINARY_I8, GLOWB200_BINARY_MAX); }
  Error emitElementMin(const ElementMinInst *N) { return binary(N, GLOWB200_INSTR_BINARY_I8, GLOWB200_BINARY_MIN); }
  Error emitElementMul(const ElementMulInst *N) { return binary(N, GLOWB200_INSTR_MULDIV_I8, 0); }
  Error emitElementDiv(const ElementDivInst *N) { return binary(N, GLOWB200_INSTR_MULDIV_I8, 1); }
  Error emitBatchedAdd(const BatchedAddInst *N) {
    auto *B = N->getBatch();
    const int64_t slices = I64(B->dims()[0]);
    const int64_t ia[6] = {slices, slices ? I64(B->getType()->size()) / slices : 0, N->getDest()->getType()->getOffset(),
                           B->getType()->getOffset(), N->getSlice()->getType()->getOffset(),
                           N->getSlice()->getElementType() == ElemKind::Int32QTy};
    const float fa[3] = {B->getType()->getScale(), N->getSlice()->getType()->getScale(), N->getDest()->getType()->getScale()};
    return emit(GLOWB200_INSTR_BATCHED_ADD_I8, {N->getDest(), B, N->getSlice()}, ia, fa);
  }
  Error rescaling(const Instruction *I, int kind) {  // Relu and RescaleQuantized: dest, src
    const Value *dst = I->getOperand(0).first, *src = I->getOperand(1).first;
    const int64_t ia[3] = {I64(dst->getType()->size()), src->getType()->getOffset(), dst->getType()->getOffset()};
    const float fa[2] = {src->getType()->getScale(), dst->getType()->getScale()};
    return emit(kind, {dst, src}, ia, fa);
  }
  Error emitRelu(const ReluInst *N) { return rescaling(N, GLOWB200_INSTR_RELU); }
  Error emitRescaleQuantized(const RescaleQuantizedInst *N) { return rescaling(N, GLOWB200_INSTR_RESCALE); }
  Error emitMaxPool(const MaxPoolInst *N) {
    // libjit_max_pool_i8 (libjit.cpp:2592-2600): NHWC, top/left pads, the result keeps the input's type
    if (N->getLayout() != NHWC) return unsupported("only NHWC pooling");
    auto in = N->getSrc()->dims(), out = N->getDest()->dims();
    auto k = N->getKernels(), s = N->getStrides(), p = N->getPads();
    const int64_t ia[13] = {I64(in[0]), I64(in[1]), I64(in[2]), I64(in[3]), I64(out[1]), I64(out[2]), k[0], k[1], s[0], s[1], p[0], p[1],
                            N->getDest()->getType()->getOffset()};
    return emit(GLOWB200_INSTR_MAXPOOL, {N->getDest(), N->getSrc()}, ia);
  }
  Error emitAvgPool(const AvgPoolInst *N) {
    // libjit_avg_pool_i8 (libjit.cpp:2812-2897; scale derivation LLVMIRGen.cpp:3003-3046)
    if (N->getLayout() != NHWC) return unsupported("only NHWC pooling");
    auto in = N->getSrc()->dims(), out = N->getDest()->dims();
    auto k = N->getKernels(), s = N->getStrides(), p = N->getPads();
    const Type *it = N->getSrc()->getType(), *ot = N->getDest()->getType();
    const int64_t ia[15] = {I64(in[0]), I64(in[1]), I64(in[2]), I64(in[3]), I64(out[1]), I64(out[2]), k[0], k[1], s[0], s[1], p[0], p[1],
                            it->getOffset(), ot->getOffset(), N->getCountIncludePads()};
    const float fa[2] = {it->getScale(), ot->getScale()};
    return emit(GLOWB200_INSTR_AVGPOOL, {N->getDest(), N->getSrc()}, ia, fa);
  }
  Error emitQuantize(const QuantizeInst *N) {
    const Type *qt = N->getDest()->getType();
    const int64_t ia[2] = {I64(qt->size()), qt->getOffset()};
    const float fa[1] = {qt->getScale()};
    return emit(GLOWB200_INSTR_QUANTIZE, {N->getDest(), N->getSrc()}, ia, fa);
  }
  Error emitDequantize(const DequantizeInst *N) {
    const Type *qt = N->getSrc()->getType();
    const int64_t ia[2] = {I64(qt->size()), qt->getOffset()};
    const float fa[1] = {qt->getScale()};
    return emit(GLOWB200_INSTR_DEQUANTIZE, {N->getDest(), N->getSrc()}, ia, fa);
  }

  // ---- data movement ------------------------------------------------------------------------
  Error emitTranspose(const TransposeInst *N) {
    auto d = N->getSrc()->dims();
    auto sh = N->getShuffle();
    if (d.size() < 1 || d.size() > 4) return unsupported("transposes of 1 to 4 dimensions only");
    int64_t ia[10] = {I64(d.size()), (int64_t)N->getSrc()->getType()->getElementSize(), 1, 1, 1, 1, 0, 0, 0, 0};
    for (size_t i = 0; i < d.size(); i++) {
      ia[2 + i] = I64(d[i]);
      ia[6 + i] = sh[i];
    }
    return emit(GLOWB200_INSTR_TRANSPOSE, {N->getDest(), N->getSrc()}, ia);
  }
  Error emitSplat(const SplatInst *N) {
    const ElemKind e = N->getDest()->getElementType();
    if (e != ElemKind::FloatTy && e != ElemKind::Float16Ty) return unsupported("only fp32 / fp16 splats");
    const int64_t ia[2] = {I64(N->getDest()->getType()->size()), e == ElemKind::Float16Ty};
    const float fa[1] = {N->getValue()};
    return emit(GLOWB200_INSTR_SPLAT, {N->getDest()}, ia, fa);
  }
  Error emitInsertTensor(const InsertTensorInst *N) {
    // the lowered Concat of pooled vectors: a [rows, width] block into a wider row-major tensor
    const auto dd = N->getDest()->dims(), sd = N->getSrc()->dims();
    const size_t eb = N->getDest()->getType()->getElementSize();
    if (dd.size() != 2 || N->getCount() != 1 || N->getOffsets()[0] != 0) return unsupported("only column-wise InsertTensor");
    const int64_t ia[4] = {I64(sd[0]), (int64_t)(sd[1] * eb), (int64_t)(dd[1] * eb), (int64_t)(N->getOffsets()[1] * eb)};
    return emit(GLOWB200_INSTR_INSERT_TENSOR, {N->getDest(), N->getSrc()}, ia);
  }
  Error emitCopy(const CopyInst *N) {
    const int64_t ia[1] = {(int64_t)N->getDest()->getType()->getSizeInBytes()};
    return emit(GLOWB200_INSTR_COPY, {N->getDest(), N->getSrc()}, ia);
  }
};
} // namespace

B200Function::B200Function(std::unique_ptr<IRFunction> F, runtime::RuntimeBundle &&bundle)
    : CompiledFunction(std::move(bundle)), F_(std::move(F)) {}

B200Function::~B200Function() { glowb200_function_destroy(fn_); }

void B200Function::collectConstants(const Module *module) {
  if (fn_) return;
  // errors cannot leave this hook: a failed translation leaves fn_ empty, and the device manager,
  // which calls translate() itself, reports it through the readyCB of addNetwork
  if (auto err = translate(module)) {
    LOG(ERROR) << "B200: translation failed: " << ERR_TO_STRING(std::move(err));
    glowb200_function_destroy(fn_);
    fn_ = nullptr;
  }
}

Error B200Function::translate(const Module *module) {
  if (fn_) return Error::success();
  fn_ = glowb200_function_create(F_->getGraph()->getName().str().c_str());
  Translator T(fn_, module);
  // WeightVars: constants carry their payload, placeholders are bound per request
  for (auto *W : F_->getWeights()) RETURN_IF_ERR(T.addWeight(W, *F_));
  for (const auto &I : F_->getInstrs()) {
    switch (I.getKind()) {
    case Kinded::Kind::AllocActivationInstKind:
      RETURN_IF_ERR(T.addActivation(llvm::cast<AllocActivationInst>(&I)));
      break;
    case Kinded::Kind::DeallocActivationInstKind:
    case Kinded::Kind::TensorViewInstKind:  // resolved where it is used, offsets included
    case Kinded::Kind::TouchInstKind:
      break;
    case Kinded::Kind::CopyInstKind:  // IR only (Save, and copies the optimizer leaves)
      RETURN_IF_ERR(T.emitCopy(llvm::cast<CopyInst>(&I)));
      break;
#define B200_OP(NODE, INST, RUNTIME, PRED)                                                                                      \
    case Kinded::Kind::INST##InstKind:                                                                                          \
      RETURN_IF_ERR(T.emit##INST(llvm::cast<INST##Inst>(&I)));                                                                  \
      break;
#include "B200Ops.def"
#undef B200_OP
    default:
      return unsupported("instruction " + std::string(I.getKindName()) + " (" + I.getName().str() + ") has no translation");
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
    // device resident on this device: already where the kernels read it, or the result stays there
    if (PH.second.isDeviceResident() && (const void *)PH.second.getDeviceManager() == owner_) continue;
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
