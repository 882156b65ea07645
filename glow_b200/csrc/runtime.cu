// Host runtime above the kernel ABI: the part of a Glow backend that sits between
// DeviceManager::runFunction and the kernels, written against this library instead of Glow's
// headers (Glow itself needs LLVM, folly and glog to compile; the thin glue that adapts these
// classes to glow::CompiledFunction / glow::DeviceManager ships as source under integration/glow/lib/Backends/B200).
//
//   Function       what Backend::compile produces: a symbol table with byte offsets into three
//                  slabs -- constants, placeholders ("mutable weights") and activations -- like
//                  glow::RuntimeBundle (include/glow/Backend/BackendUtils.h:66-170), and a flat,
//                  control-flow-free instruction list like Glow's low-level IR (docs/IR.md).
//                  compile() does what LLVMIRGen does while emitting a call: it turns the float
//                  scales of the node types into the integer pre/post/scale triples
//                  (LLVMIRGen.cpp:2222-2320, 2695-2798, 1716-1771, 3003-3046).
//   DeviceManager  one GPU: addNetwork uploads the constants slab and accounts its memory,
//                  evictNetwork frees it, runFunction copies the bound inputs in, walks the
//                  instructions, copies the outputs back and turns the kernels' status word into
//                  an error -- the contract of CPUDeviceManager (lib/Backends/CPU/
//                  CPUDeviceManager.cpp:65-179) with the copies of OpenCLDeviceManager
//                  (lib/Backends/OpenCL/OpenCLDeviceManager.cpp:775-853).
// Error codes carry the names of glow::ErrorValue::ErrorCode (include/glow/Support/Error.h).
#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace glowb200 {
void quantize_scale_32to8(float scale, int32_t &pre, int32_t &post, int32_t &iscale);
}

namespace {

using glowb200::align_up;
using glowb200::set_error;

// kStatic: a placeholder that is written once and then stays put (Placeholder::isStatic: the
// embedding tables of a recommendation model).  It lives beside the constants, shared by all
// execution contexts of a network; ordinary placeholders and activations exist once per context.
enum SymbolKind { kConstant = 0, kPlaceholder = 1, kActivation = 2, kStatic = 3 };
constexpr int kSlabs = 4;

struct Symbol {
  std::string name;
  int kind;
  size_t bytes, offset;
  std::vector<uint8_t> host;  // constants only
};

struct Instruction {
  int kind;
  std::vector<int> ops;       // symbol ids
  std::vector<int64_t> off;   // byte offset of each operand inside its symbol (a view of a larger tensor)
  int group = -1;             // FRWQ_SLWS: index of the batched launch this instruction is part of
  bool group_leader = false;  // ... and whether it is the one that launches it
  bool absorbed = false;      // QUANTIZE: done by the TRANSPOSE behind it (nothing to launch)
  bool quantizes = false;     // TRANSPOSE: reads floats (operand 2) and quantizes them on the way (fa[0], ia[10])
  std::vector<int64_t> ia;    // integer attributes
  std::vector<float> fa;      // float attributes
  std::vector<int> derived;   // ids of constants compile() added (triples, row sums ...)
};

}  // namespace

struct glowb200_function {
  std::string name;
  std::vector<Symbol> symbols;
  std::vector<Instruction> instrs;
  bool compiled = false;
  size_t slab_bytes[kSlabs] = {0, 0, 0, 0};
  size_t workspace_bytes = 0;
  // Runs of pooling instructions that become ONE batched launch each: their members, in order.
  std::vector<std::vector<int>> slws_groups;
  int fused_quantize_transposes = 0;
  std::map<std::string, int> by_name;

  int add_symbol(const std::string &n, int kind, size_t bytes, const void *data) {
    if (by_name.count(n)) return -1;
    Symbol s;
    s.name = n;
    s.kind = kind;
    s.bytes = bytes;
    s.offset = 0;
    if (data) s.host.assign(static_cast<const uint8_t *>(data), static_cast<const uint8_t *>(data) + bytes);
    symbols.push_back(std::move(s));
    by_name[n] = (int)symbols.size() - 1;
    return (int)symbols.size() - 1;
  }
  int add_i32_constant(const std::string &n, const std::vector<int32_t> &v) {
    return add_symbol(n, kConstant, v.size() * 4, v.data());
  }
};

namespace {

// One execution context of a loaded network (Backend::getContextCount / bindContexts,
// include/glow/Backend/Backend.h:272-276): its own placeholders and activations, so that the
// inputs of the next request can arrive while this one runs and the last one's results leave.
struct Context {
  uint8_t *slab[kSlabs] = {nullptr, nullptr, nullptr, nullptr};  // [kConstant], [kStatic]: the network's, shared
  uint8_t *workspace = nullptr;
  int32_t *status_dev = nullptr;
  int32_t *status_host = nullptr;      // pinned
  std::vector<glowb200_slws_job *> jobs;  // device descriptor arrays, one per batched pooling launch
  cudaEvent_t in_done = nullptr, run_done = nullptr, out_done = nullptr;
  int64_t ticket = 0;                  // the request in flight on this context (0: none)
};

struct LoadedNetwork {
  glowb200_function *fn;
  uint8_t *shared[2] = {nullptr, nullptr};  // constants, static placeholders
  std::vector<Context> ctx;
  size_t next_ctx = 0;
  size_t device_bytes = 0;
};

const float *host_f32(const glowb200_function *f, int id) { return reinterpret_cast<const float *>(f->symbols[id].host.data()); }

// Triples for n rows from float scales: what LLVMIRGen bakes into the rowwise FC / channelwise
// conv call.  Returns the ids of six int32 constants.
std::vector<int> add_row_triples(glowb200_function *f, const std::string &tag, const float *row_scales, int64_t n, float in_scale,
                                 const float *bias_scales, int64_t nb, float out_scale) {
  std::vector<int32_t> v[6];
  for (auto &x : v) x.resize(n);
  for (int64_t j = 0; j < n; j++) {
    const float mm = in_scale * row_scales[j];
    glowb200::quantize_scale_32to8(bias_scales[nb == 1 ? 0 : j] / mm, v[0][j], v[1][j], v[2][j]);
    glowb200::quantize_scale_32to8(mm / out_scale, v[3][j], v[4][j], v[5][j]);
  }
  std::vector<int> ids;
  const char *names[6] = {".bias_pre", ".bias_post", ".bias_scale", ".out_pre", ".out_post", ".out_scale"};
  for (int i = 0; i < 6; i++) ids.push_back(f->add_i32_constant(tag + names[i], v[i]));
  return ids;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Function building
// ---------------------------------------------------------------------------------------------
extern "C" glowb200_function *glowb200_function_create(const char *name) {
  auto *f = new glowb200_function();
  f->name = name ? name : "";
  return f;
}

extern "C" void glowb200_function_destroy(glowb200_function *f) { delete f; }

extern "C" int glowb200_function_add_symbol(glowb200_function *f, const char *name, int kind, size_t bytes, const void *host_data) {
  if (!f || !name || f->compiled || kind < 0 || kind >= kSlabs || (kind == kConstant) != (host_data != nullptr)) {
    set_error(GLOWB200_RUNTIME_ERROR, "bad symbol '%s'", name ? name : "?");
    return -1;
  }
  const int id = f->add_symbol(name, kind, bytes, host_data);
  if (id < 0) set_error(GLOWB200_RUNTIME_ERROR, "symbol '%s' already exists", name);
  return id;
}

extern "C" int glowb200_function_add_instruction(glowb200_function *f, int kind, const int32_t *operands, int num_operands,
                                                 const int64_t *int_attrs, int num_int_attrs, const float *float_attrs,
                                                 int num_float_attrs) {
  return glowb200_function_add_instruction_views(f, kind, operands, nullptr, num_operands, int_attrs, num_int_attrs,
                                                 float_attrs, num_float_attrs);
}

extern "C" int glowb200_function_add_instruction_views(glowb200_function *f, int kind, const int32_t *operands,
                                                       const int64_t *operand_byte_offsets, int num_operands,
                                                       const int64_t *int_attrs, int num_int_attrs, const float *float_attrs,
                                                       int num_float_attrs) {
  if (!f || f->compiled) return set_error(GLOWB200_RUNTIME_ERROR, "function is NULL or already compiled");
  Instruction in;
  in.kind = kind;
  for (int i = 0; i < num_operands; i++) {
    if (operands[i] < -1 || operands[i] >= (int)f->symbols.size()) return set_error(GLOWB200_RUNTIME_ERROR, "operand %d: no such symbol", i);
    const int64_t o = operand_byte_offsets ? operand_byte_offsets[i] : 0;
    if (o < 0 || (operands[i] < 0 && o != 0)) return set_error(GLOWB200_RUNTIME_ERROR, "operand %d: bad byte offset", i);
    in.ops.push_back(operands[i]);
    in.off.push_back(o);
  }
  in.ia.assign(int_attrs, int_attrs + num_int_attrs);
  in.fa.assign(float_attrs, float_attrs + num_float_attrs);
  f->instrs.push_back(std::move(in));
  return GLOWB200_OK;
}

namespace {

// What an instruction addresses, checked against the sizes of the symbols it names: a
// malformed or mistranslated instruction must fail here, not overwrite a neighbour in the slab.
// Layouts as in the table above glowb200_function_compile.
int validate_instruction(const glowb200_function *f, const Instruction &in, size_t ii) {
  const auto &a = in.ia;
  struct Need { int op; int64_t bytes; bool optional; };
  std::vector<Need> needs;
  auto need = [&](int op, int64_t bytes, bool optional = false) { needs.push_back({op, bytes, optional}); };
  auto bad = [&](const char *what) { return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: %s", ii, what); };
  auto nonneg = [&](std::initializer_list<int> idx) {
    for (int i : idx)
      if (a[i] < 0) return false;
    return true;
  };
  switch (in.kind) {
    case GLOWB200_INSTR_FRWQ_SLWS: {
      if (!nonneg({1, 2, 3, 4, 5})) return bad("negative size");
      const int64_t es = a[7] ? 2 : 4;
      need(0, a[4] * a[3] * es); need(1, a[1] * a[2]); need(2, a[5] * es); need(3, a[5] * (a[6] ? 8 : 4)); need(4, a[4] * 4);
      break;
    }
    case GLOWB200_INSTR_RWQ_FC:
      if (!nonneg({0, 1, 2})) return bad("negative size");
      need(0, a[0] * a[2]); need(1, a[0] * a[1]); need(2, a[2] * a[1]); need(3, a[2] * 4); need(4, a[2] * 4); need(5, a[2] * 4);
      break;
    case GLOWB200_INSTR_CWQ_CONV: {
      if (!nonneg({0, 1, 2, 3, 4, 5, 6, 7, 8})) return bad("negative size");
      if (a[15] <= 0 || a[3] % a[15] || a[6] % a[15]) return bad("group must be positive and divide the channel counts");
      const int64_t OC = a[6];
      need(0, a[0] * a[4] * a[5] * OC); need(1, a[0] * a[1] * a[2] * a[3]); need(2, OC * a[7] * a[8] * (a[3] / a[15]));
      need(3, OC * 4); need(4, OC * 4); need(5, OC * 4); need(6, OC * 4); need(7, OC * 4);
      break;
    }
    case GLOWB200_INSTR_ADD: case GLOWB200_INSTR_ADD_MAXSPLAT: case GLOWB200_INSTR_BINARY_I8: case GLOWB200_INSTR_MULDIV_I8:
      if (a[0] < 0) return bad("negative size");
      need(0, a[0]); need(1, a[0]); need(2, a[0]);
      break;
    case GLOWB200_INSTR_MAXSPLAT: case GLOWB200_INSTR_RELU: case GLOWB200_INSTR_RESCALE:
      if (a[0] < 0) return bad("negative size");
      need(0, a[0]); need(1, a[0]);
      break;
    case GLOWB200_INSTR_QUANTIZE:
      if (a[0] < 0) return bad("negative size");
      need(0, a[0]); need(1, a[0] * 4);
      break;
    case GLOWB200_INSTR_DEQUANTIZE:
      if (a[0] < 0) return bad("negative size");
      need(0, a[0] * 4); need(1, a[0]);
      break;
    case GLOWB200_INSTR_MAXPOOL: case GLOWB200_INSTR_AVGPOOL:
      if (!nonneg({0, 1, 2, 3, 4, 5})) return bad("negative size");
      need(0, a[0] * a[4] * a[5] * a[3]); need(1, a[0] * a[1] * a[2] * a[3]);
      break;
    case GLOWB200_INSTR_TRANSPOSE: {
      if (a[0] < 1 || a[0] > 4 || a[1] < 1) return bad("transpose of 1 to 4 dimensions");
      int64_t n = a[1];
      for (int i = 0; i < a[0]; i++) {
        if (a[2 + i] < 0 || a[6 + i] < 0 || a[6 + i] >= a[0]) return bad("bad transpose shape or shuffle");
        n *= a[2 + i];
      }
      need(0, n); need(1, n);
      break;
    }
    case GLOWB200_INSTR_COPY:
      if (a[0] < 0) return bad("negative size");
      need(0, a[0]); need(1, a[0]);
      break;
    case GLOWB200_INSTR_FC_I8:
      if (!nonneg({0, 1, 2})) return bad("negative size");
      need(0, a[0] * a[2]); need(1, a[0] * a[1]); need(2, a[1] * a[2]); need(3, a[2] * 4);
      break;
    case GLOWB200_INSTR_MATMUL_I8:
      if (!nonneg({0, 1, 2})) return bad("negative size");
      need(0, a[0] * a[2]); need(1, a[0] * a[1]); need(2, a[1] * a[2]);
      break;
    case GLOWB200_INSTR_SPLAT:
      if (a[0] < 0) return bad("negative size");
      need(0, a[0] * (a[1] ? 2 : 4));
      break;
    case GLOWB200_INSTR_INSERT_TENSOR:
      if (!nonneg({0, 1, 2, 3}) || a[2] < a[1]) return bad("bad insert-tensor pitch or offset");
      need(0, a[0] > 0 ? a[3] + (a[0] - 1) * a[2] + a[1] : 0); need(1, a[0] * a[1]);
      break;
    case GLOWB200_INSTR_PAIRWISE_DOT: {
      if (!nonneg({0, 1, 2, 3, 4, 5})) return bad("negative size");
      const int64_t B = a[0], T = a[1], D = a[2], width = D + (T + 1) * T / 2;
      if (a[3] < D || a[4] < T * D || a[5] < width) return bad("leading dimension smaller than a row");
      need(0, B > 0 ? ((B - 1) * a[5] + width) * (a[6] ? 1 : 4) : 0); need(1, B > 0 ? ((B - 1) * a[3] + D) * 4 : 0);
      need(2, B > 0 ? ((B - 1) * a[4] + T * D) * 4 : 0);
      break;
    }
    case GLOWB200_INSTR_SLWS_F32:
      if (!nonneg({0, 1, 2, 3})) return bad("negative size");
      need(0, a[2] * a[1] * 4); need(1, a[0] * a[1] * 4); need(2, a[3] * 4, true); need(3, a[3] * (a[4] ? 8 : 4)); need(4, a[2] * 4);
      break;
    case GLOWB200_INSTR_RWQ_SLWS:
      if (!nonneg({0, 1, 2, 3})) return bad("negative size");
      need(0, a[2] * a[1] * 4); need(1, a[0] * a[1]); need(2, a[0] * 4); need(3, a[0] * 4); need(4, a[3] * 4);
      need(5, a[3] * (a[4] ? 8 : 4)); need(6, a[2] * 4);
      break;
    case GLOWB200_INSTR_EMBEDDING_BAG: {
      if (!nonneg({1, 2, 3, 4, 5})) return bad("negative size");
      const int64_t es = a[8] ? 2 : 4, bags = a[7] ? (a[4] > 0 ? a[4] - 1 : 0) : a[4], ib = a[6] ? 8 : 4;
      need(0, bags * a[3] * es); need(1, a[1] * a[2]); need(2, a[5] * es); need(3, a[5] * ib); need(4, a[4] * ib);
      break;
    }
    case GLOWB200_INSTR_SPLIT_EMBEDDING: {
      if (!nonneg({0, 1, 2, 3, 4, 5})) return bad("negative size");
      const int64_t ib = a[6] ? 8 : 4, T = a[2];
      need(0, a[5] * a[3] * (a[10] ? 2 : 4)); need(1, a[0], a[0] == 0); need(2, a[1], a[1] == 0); need(3, T * 4);
      need(4, T * (a[7] ? 8 : 4)); need(5, T); need(6, (T + 1) * 4); need(7, a[4] * ib); need(8, (T * a[5] + 1) * ib);
      need(9, a[4] * (a[9] ? 2 : 4), true);
      break;
    }
    case GLOWB200_INSTR_DYN_QUANTIZED_FC:
      if (!nonneg({0, 1, 2})) return bad("negative size");
      need(0, a[0] * a[2] * 2); need(1, a[0] * a[1] * 2); need(2, a[1] * a[2]); need(3, a[2] * 4); need(4, a[2] * 4, true);
      need(5, a[2] * 4, true);
      break;
    case GLOWB200_INSTR_BATCHED_ADD_I8:
      if (!nonneg({0, 1})) return bad("negative size");
      need(0, a[0] * a[1]); need(1, a[0] * a[1]); need(2, a[1] * (a[5] ? 4 : 1));
      break;
    default: break;
  }
  if (needs.size() != in.ops.size()) return bad("operand table out of step with the instruction");
  for (const Need &n : needs) {
    const int id = in.ops[n.op];
    if (id < 0) {
      if (!n.optional) return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: operand %d is required", ii, n.op);
      continue;
    }
    const Symbol &s = f->symbols[id];
    if ((int64_t)s.bytes < in.off[n.op] + n.bytes)
      return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: operand %d ('%s', %zu bytes) is smaller than the %lld bytes the instruction addresses at offset %lld",
                       ii, n.op, s.name.c_str(), s.bytes, (long long)n.bytes, (long long)in.off[n.op]);
    if (n.op == 0 && s.kind == kConstant) return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: the destination '%s' is a constant", ii, s.name.c_str());
  }
  return GLOWB200_OK;
}

}  // namespace

// Instruction operand / attribute layouts (ia = integer attributes, fa = float attributes):
//  FRWQ_SLWS   ops {dest, data, weights, indices, lengths}  ia {kind, rows, in_line, out_line, segments, num_indices, idx64, out_fp16, fp16_acc}
//  RWQ_FC      ops {dest, src, weights, scales(f32 const), offsets, bias}  ia {M, K, N, in_off, bias_off, out_off, relu}  fa {in_scale, bias_scale, out_scale}
//  CWQ_CONV    ops {dest, src, filter, bias, filter_scales(f32 const), filter_offsets, bias_scales(f32 const), bias_offsets}
//              ia {N,H,W,C, OH,OW,OC, KH,KW, SH,SW, PT,PL,PB,PR, group, DH,DW, in_off, out_off, act}  fa {in_scale, out_scale}
//  ADD         ops {dest, lhs, rhs}  ia {n, dest_off, lhs_off, rhs_off}  fa {lhs_scale, rhs_scale, dest_scale}
//  MAXSPLAT    ops {dest, src}  ia {n, splat}
//  QUANTIZE    ops {dest, src}  ia {n, offset}  fa {scale}
//  DEQUANTIZE  ops {dest, src}  ia {n, offset}  fa {scale}
//  MAXPOOL     ops {dest, src}  ia {N,H,W,C, OH,OW, KH,KW, SH,SW, PT,PL, out_off}
//  AVGPOOL     ops {dest, src}  ia {N,H,W,C, OH,OW, KH,KW, SH,SW, PT,PL, in_off, out_off, count_include_pads}  fa {in_scale, out_scale}
//  TRANSPOSE   ops {dest, src}  ia {ndims, elem_bytes, d0..d3, s0..s3}
//  COPY        ops {dest, src}  ia {bytes}
//  ADD_MAXSPLAT ops {dest, lhs, rhs}  ia {n, dest_off, lhs_off, rhs_off, splat}  fa {lhs_scale, rhs_scale, dest_scale}
//  RELU        ops {dest, src}  ia {n, src_off, dest_off}  fa {src_scale, dest_scale}
//  RESCALE     ops {dest, src}  ia {n, in_off, out_off}  fa {in_scale, out_scale}
//  FC_I8       ops {dest, src, weights [K,N], bias}  ia {M, K, N, in_off, w_off, bias_off, out_off}  fa {in_scale, w_scale, bias_scale, out_scale}
//  MATMUL_I8   ops {dest, lhs, rhs [K,N]}  ia {M, K, N, lhs_off, rhs_off, out_off}  fa {lhs_scale, rhs_scale, out_scale}
//  SPLAT       ops {dest}  ia {n, is_fp16}  fa {value}
//  INSERT_TENSOR ops {dest, src}  ia {rows, width_bytes, dest_pitch_bytes, dest_offset_bytes}
//  PAIRWISE_DOT ops {dest, dense, pooled}  ia {batch, tables, dim, ld_dense, ld_pooled, ld_out, out_is_i8, q_offset}  fa {q_scale}
//  SLWS_F32    ops {dest, data, weights (-1: unweighted), indices, lengths}  ia {rows, line, segments, num_indices, idx64}
//  RWQ_SLWS    ops {dest, data, scales, offsets, weights, indices, lengths}  ia {rows, line, segments, num_indices, idx64}
//  EMBEDDING_BAG ops {dest, data, weights, indices, offsets}  ia {kind, rows, in_line, out_line, num_offsets, num_indices, idx64, has_end_offset, out_fp16, fp16_acc}
//  SPLIT_EMBEDDING ops {dest, dev_weights, uvm_weights, placements, weights_offsets, weights_tys, dim_offsets, indices, offsets,
//                   indice_weights (-1: unweighted)}
//              ia {dev_bytes, uvm_bytes, num_tables, total_dims, num_indices, bags_per_table, idx64, weights_offsets_are_int64,
//                  pooling_mode, indice_weights_are_fp16, out_fp16, scale_offset_is_fp32, row_alignment}
//  DYN_QUANTIZED_FC ops {dest (fp16), src (fp16), weights [K,N], bias (fp32), scales (-1: per tensor), offsets (-1: per tensor)}
//              ia {M, K, N, weights_offset}  fa {weights_scale}
//  BINARY_I8   ops {dest, lhs, rhs}  ia {n, dest_off, lhs_off, rhs_off, op (GLOWB200_BINARY_*)}  fa {lhs_scale, rhs_scale, dest_scale}
//  MULDIV_I8   ops {dest, lhs, rhs}  ia {n, dest_off, lhs_off, rhs_off, is_div}  fa {lhs_scale, rhs_scale, dest_scale}
//  BATCHED_ADD_I8 ops {dest, batch, slice}  ia {num_slices, slice_size, dest_off, batch_off, slice_off, slice_is_int32}
//              fa {batch_scale, slice_scale, dest_scale}
extern "C" int glowb200_function_compile(glowb200_function *f) {
  if (!f || f->compiled) return set_error(GLOWB200_RUNTIME_ERROR, "function is NULL or already compiled");
  size_t ws = 256;
  bool sizes_bad = false;  // validate_instruction has set the message
  for (size_t ii = 0; ii < f->instrs.size(); ii++) {
    Instruction &in = f->instrs[ii];
    const std::string tag = "i" + std::to_string(ii);
    bool counts_ok = false;
    auto need = [&](size_t nops, size_t nia, size_t nfa) {
      counts_ok = in.ops.size() == nops && in.ia.size() == nia && in.fa.size() == nfa;
      if (counts_ok && validate_instruction(f, in, ii) != GLOWB200_OK) {
        counts_ok = false;
        sizes_bad = true;
      }
      return counts_ok;
    };
    auto malformed = [&](const char *what) {
      if (sizes_bad) return (int)GLOWB200_RUNTIME_ERROR;  // validate_instruction's message stands
      return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: malformed %s", ii, what);
    };
    switch (in.kind) {
      case GLOWB200_INSTR_FRWQ_SLWS:
        if (!need(5, 9, 0)) return malformed("FRWQ_SLWS");
        ws = std::max(ws, glowb200_slws_workspace_bytes(in.ia[4], 1));
        break;
      case GLOWB200_INSTR_RWQ_FC: {
        if (!need(6, 7, 3)) return malformed("RWQ_FC");
        const int64_t N = in.ia[2];
        if (f->symbols[in.ops[3]].host.size() != (size_t)N * 4) return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: scales must be a float constant of N entries", ii);
        in.derived = add_row_triples(f, tag, host_f32(f, in.ops[3]), N, in.fa[0], &in.fa[1], 1, in.fa[2]);
        // row sums of the constant weights, computed once on the host
        const Symbol &w = f->symbols[in.ops[2]];
        if (w.host.size() != (size_t)N * in.ia[1]) return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: weights must be an int8 constant [N,K]", ii);
        std::vector<int32_t> rs(N);
        for (int64_t j = 0; j < N; j++) {
          int32_t s = 0;
          for (int64_t k = 0; k < in.ia[1]; k++) s += (int8_t)w.host[j * in.ia[1] + k];
          rs[j] = s;
        }
        in.derived.push_back(f->add_i32_constant(tag + ".row_sums", rs));
        ws = std::max(ws, glowb200_i8_gemm_workspace_bytes(in.ia[0], in.ia[1], N));
        break;
      }
      case GLOWB200_INSTR_CWQ_CONV: {
        if (!need(8, 21, 2)) return malformed("CWQ_CONV");
        const int64_t OC = in.ia[6];
        if (f->symbols[in.ops[4]].host.size() != (size_t)OC * 4 || f->symbols[in.ops[6]].host.size() != (size_t)OC * 4)
          return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: filter/bias scales must be float constants of outC entries", ii);
        in.derived = add_row_triples(f, tag, host_f32(f, in.ops[4]), OC, in.fa[0], host_f32(f, in.ops[6]), OC, in.fa[1]);
        const int64_t od[4] = {in.ia[0], in.ia[4], in.ia[5], in.ia[6]}, id[4] = {in.ia[0], in.ia[1], in.ia[2], in.ia[3]};
        const int64_t fd[4] = {in.ia[6], in.ia[7], in.ia[8], in.ia[3] / in.ia[15]}, k[2] = {in.ia[7], in.ia[8]}, s[2] = {in.ia[9], in.ia[10]};
        const int64_t p[4] = {in.ia[11], in.ia[12], in.ia[13], in.ia[14]}, d[2] = {in.ia[16], in.ia[17]};
        ws = std::max(ws, glowb200_conv2d_workspace_bytes(od, id, fd, k, s, p, in.ia[15], d));
        break;
      }
      case GLOWB200_INSTR_ADD: {
        if (!need(3, 4, 3)) return malformed("ADD");
        std::vector<int32_t> t(6);
        glowb200::quantize_scale_32to8(in.fa[0] / in.fa[2], t[0], t[1], t[2]);  // LLVMIRGen.cpp:1740-1743
        glowb200::quantize_scale_32to8(in.fa[1] / in.fa[2], t[3], t[4], t[5]);
        for (int32_t x : t) in.ia.push_back(x);
        break;
      }
      case GLOWB200_INSTR_AVGPOOL: {
        if (!need(2, 15, 2)) return malformed("AVGPOOL");
        // LLVMIRGen.cpp:3003-3046: the kernel area is folded into the scale when pads are counted
        float sc = in.fa[0] / in.fa[1];
        if (in.ia[14]) sc = sc / (float)(in.ia[6] * in.ia[7]);
        int32_t a, b, c;
        glowb200::quantize_scale_32to8(sc, a, b, c);
        in.ia.push_back(a); in.ia.push_back(b); in.ia.push_back(c);
        break;
      }
      case GLOWB200_INSTR_MAXSPLAT: if (!need(2, 2, 0)) return malformed("MAXSPLAT"); break;
      case GLOWB200_INSTR_QUANTIZE:
      case GLOWB200_INSTR_DEQUANTIZE: if (!need(2, 2, 1)) return malformed("(de)quantize"); break;
      case GLOWB200_INSTR_MAXPOOL: if (!need(2, 13, 0)) return malformed("MAXPOOL"); break;
      case GLOWB200_INSTR_TRANSPOSE: if (!need(2, 10, 0)) return malformed("TRANSPOSE"); break;
      case GLOWB200_INSTR_COPY: if (!need(2, 1, 0)) return malformed("COPY"); break;
      case GLOWB200_INSTR_ADD_MAXSPLAT: {
        if (!need(3, 5, 3)) return malformed("ADD_MAXSPLAT");
        int32_t t[6];
        glowb200::quantize_scale_32to8(in.fa[0] / in.fa[2], t[0], t[1], t[2]);
        glowb200::quantize_scale_32to8(in.fa[1] / in.fa[2], t[3], t[4], t[5]);
        for (int32_t x : t) in.ia.push_back(x);
        break;
      }
      case GLOWB200_INSTR_RELU:
      case GLOWB200_INSTR_RESCALE: {
        // LLVMIRGen.cpp:1465-1499, 1630-1698: one triple from srcScale / destScale
        if (!need(2, 3, 2)) return malformed("RELU / RESCALE");
        int32_t a, b, c;
        glowb200::quantize_scale_32to8(in.fa[0] / in.fa[1], a, b, c);
        in.ia.push_back(a); in.ia.push_back(b); in.ia.push_back(c);
        break;
      }
      case GLOWB200_INSTR_FC_I8: {
        // LLVMIRGen.cpp:2098-2137: bias from biasScale / (inScale * wScale), result from inScale * wScale / outScale
        if (!need(4, 7, 4)) return malformed("FC_I8");
        const float mm = in.fa[0] * in.fa[1];
        int32_t t[6];
        glowb200::quantize_scale_32to8(in.fa[2] / mm, t[0], t[1], t[2]);
        glowb200::quantize_scale_32to8(mm / in.fa[3], t[3], t[4], t[5]);
        for (int32_t x : t) in.ia.push_back(x);
        ws = std::max(ws, glowb200_i8_gemm_workspace_bytes(in.ia[0], in.ia[1], in.ia[2]));
        break;
      }
      case GLOWB200_INSTR_MATMUL_I8: {
        // LLVMIRGen.cpp:2161-2220: one triple from lhsScale * rhsScale / destScale
        if (!need(3, 6, 3)) return malformed("MATMUL_I8");
        int32_t a, b, c;
        glowb200::quantize_scale_32to8(in.fa[0] * in.fa[1] / in.fa[2], a, b, c);
        in.ia.push_back(a); in.ia.push_back(b); in.ia.push_back(c);
        ws = std::max(ws, glowb200_i8_gemm_workspace_bytes(in.ia[0], in.ia[1], in.ia[2]));
        break;
      }
      case GLOWB200_INSTR_SPLAT: if (!need(1, 2, 1)) return malformed("SPLAT"); break;
      case GLOWB200_INSTR_INSERT_TENSOR: if (!need(2, 4, 0)) return malformed("INSERT_TENSOR"); break;
      case GLOWB200_INSTR_PAIRWISE_DOT: if (!need(3, 8, 1)) return malformed("PAIRWISE_DOT"); break;
      case GLOWB200_INSTR_SLWS_F32:
        if (!need(5, 5, 0)) return malformed("SLWS_F32");
        ws = std::max(ws, glowb200_slws_workspace_bytes(in.ia[2], 1));
        break;
      case GLOWB200_INSTR_RWQ_SLWS:
        if (!need(7, 5, 0)) return malformed("RWQ_SLWS");
        ws = std::max(ws, glowb200_slws_workspace_bytes(in.ia[2], 1));
        break;
      case GLOWB200_INSTR_EMBEDDING_BAG:
        if (!need(5, 10, 0)) return malformed("EMBEDDING_BAG");
        ws = std::max(ws, glowb200_slws_workspace_bytes(in.ia[4], 1));
        break;
      case GLOWB200_INSTR_BINARY_I8: {
        // LLVMIRGen.cpp:1716-1776: each side rescaled by sideScale / destScale
        if (!need(3, 5, 3)) return malformed("BINARY_I8");
        int32_t t[6];
        glowb200::quantize_scale_32to8(in.fa[0] / in.fa[2], t[0], t[1], t[2]);
        glowb200::quantize_scale_32to8(in.fa[1] / in.fa[2], t[3], t[4], t[5]);
        for (int32_t x : t) in.ia.push_back(x);
        break;
      }
      case GLOWB200_INSTR_MULDIV_I8: {
        // LLVMIRGen.cpp:1927-2035: lhsScale * rhsScale / destScale, or lhsScale / (rhsScale * destScale)
        if (!need(3, 5, 3)) return malformed("MULDIV_I8");
        int32_t a, b, c;
        glowb200::quantize_scale_32to8(in.ia[4] ? in.fa[0] / (in.fa[1] * in.fa[2]) : in.fa[0] * in.fa[1] / in.fa[2], a, b, c);
        in.ia.push_back(a); in.ia.push_back(b); in.ia.push_back(c);
        break;
      }
      case GLOWB200_INSTR_BATCHED_ADD_I8: {
        // LLVMIRGen.cpp:2322-2375: batchScale / destScale and sliceScale / destScale
        if (!need(3, 6, 3)) return malformed("BATCHED_ADD_I8");
        int32_t t[6];
        glowb200::quantize_scale_32to8(in.fa[0] / in.fa[2], t[0], t[1], t[2]);
        glowb200::quantize_scale_32to8(in.fa[1] / in.fa[2], t[3], t[4], t[5]);
        for (int32_t x : t) in.ia.push_back(x);
        break;
      }
      case GLOWB200_INSTR_SPLIT_EMBEDDING:
        if (!need(10, 13, 0)) return malformed("SPLIT_EMBEDDING");
        break;
      case GLOWB200_INSTR_DYN_QUANTIZED_FC:
        if (!need(6, 4, 1)) return malformed("DYN_QUANTIZED_FC");
        if ((in.ops[4] < 0) != (in.ops[5] < 0))
          return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: DYN_QUANTIZED_FC needs both scales and offsets, or neither", ii);
        ws = std::max(ws, glowb200_dynamic_fc_workspace_bytes(in.ia[0], in.ia[1], in.ia[2]));
        break;
      default: return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu: unsupported kind %d (isOpSupported would refuse the node)", ii, in.kind);
    }
  }
  // Pooling instructions that follow one another, read the same kind of table with the same row
  // width and do not feed each other become ONE batched launch (a recommendation model's tables
  // are so many independent SparseLengthsSum nodes): the descriptors are built when the network
  // is loaded.  The batched kernels want 16-byte aligned operands; views at other offsets stay
  // single launches.
  {
    auto groupable = [&](const Instruction &in) {
      if (in.kind != GLOWB200_INSTR_FRWQ_SLWS) return false;
      for (int64_t o : in.off)
        if (o % 16) return false;
      return true;
    };
    auto same_shape = [](const Instruction &a, const Instruction &b) {
      return a.ia[0] == b.ia[0] && a.ia[2] == b.ia[2] && a.ia[3] == b.ia[3] && a.ia[6] == b.ia[6] && a.ia[7] == b.ia[7] &&
             a.ia[8] == b.ia[8];
    };
    size_t i = 0;
    while (i < f->instrs.size()) {
      if (!groupable(f->instrs[i])) { i++; continue; }
      std::vector<int> members{(int)i};
      size_t j = i + 1;
      for (; j < f->instrs.size() && groupable(f->instrs[j]) && same_shape(f->instrs[i], f->instrs[j]); j++) {
        // an earlier member must not write what this one reads, nor the bytes it writes
        auto dest_range = [](const Instruction &in, int64_t &lo, int64_t &hi) {
          lo = in.off[0];
          hi = lo + in.ia[4] * in.ia[3] * (in.ia[7] ? 2 : 4);
        };
        bool feeds = false;
        const Instruction &cand = f->instrs[j];
        for (int m : members) {
          const Instruction &prev = f->instrs[m];
          for (size_t o = 1; o < cand.ops.size(); o++) feeds = feeds || cand.ops[o] == prev.ops[0];
          for (size_t o = 1; o < prev.ops.size(); o++) feeds = feeds || prev.ops[o] == cand.ops[0];
          if (cand.ops[0] == prev.ops[0]) {
            int64_t a0, a1, b0, b1;
            dest_range(cand, a0, a1);
            dest_range(prev, b0, b1);
            feeds = feeds || (a0 < b1 && b0 < a1);
          }
        }
        if (feeds) break;
        members.push_back((int)j);
      }
      if (members.size() > 1 && members.size() <= 65535) {
        int64_t max_segments = 0;
        for (int m : members) {
          f->instrs[m].group = (int)f->slws_groups.size();
          max_segments = std::max(max_segments, f->instrs[m].ia[4]);
        }
        f->instrs[members[0]].group_leader = true;
        ws = std::max(ws, glowb200_slws_workspace_bytes(max_segments, (int64_t)members.size()));
        f->slws_groups.push_back(members);
      }
      i = j;
    }
  }
  // A Quantize whose result nothing reads but the Transpose right behind it (the NCHW float input
  // of a network on its way to NHWC int8; Glow's optimizer leaves the pair in this order,
  // GraphOptimizer.cpp:1076-1086) becomes one kernel: the Transpose reads the floats and quantizes.
  for (size_t i = 0; i + 1 < f->instrs.size(); i++) {
    Instruction &q = f->instrs[i], &t = f->instrs[i + 1];
    if (q.kind != GLOWB200_INSTR_QUANTIZE || t.kind != GLOWB200_INSTR_TRANSPOSE || t.ia[1] != 1) continue;
    const int mid = q.ops[0];
    if (mid < 0 || t.ops[1] != mid || t.off[1] != q.off[0] || f->symbols[mid].kind != kActivation) continue;
    int64_t n = 1;
    for (int d = 0; d < t.ia[0]; d++) n *= t.ia[2 + d];
    if (n != q.ia[0]) continue;
    bool read_elsewhere = false;
    for (size_t k = 0; k < f->instrs.size(); k++) {
      if (k == i || k == i + 1) continue;
      for (int o : f->instrs[k].ops) read_elsewhere = read_elsewhere || o == mid;
    }
    if (read_elsewhere) continue;
    q.absorbed = true;
    t.quantizes = true;
    t.ops.push_back(q.ops[1]);
    t.off.push_back(q.off[1]);
    t.fa.assign(1, q.fa[0]);
    t.ia.resize(11, 0);
    t.ia[10] = q.ia[1];
    f->fused_quantize_transposes++;
  }
  // slab offsets: 64-byte alignment like glow::TensorAlignment (include/glow/Support/Memory.h:29)
  for (Symbol &s : f->symbols) {
    s.offset = f->slab_bytes[s.kind];
    f->slab_bytes[s.kind] += align_up(s.bytes ? s.bytes : 1, 64);
  }
  f->workspace_bytes = align_up(ws, 256);
  f->compiled = true;
  return GLOWB200_OK;
}

extern "C" size_t glowb200_function_constant_bytes(const glowb200_function *f) { return f ? f->slab_bytes[kConstant] : 0; }
extern "C" int glowb200_function_fused_quantize_transposes(const glowb200_function *f) {
  return (f && f->compiled) ? f->fused_quantize_transposes : 0;
}
extern "C" int glowb200_function_batched_pooling_launches(const glowb200_function *f) {
  return (f && f->compiled) ? (int)f->slws_groups.size() : 0;
}

// ---------------------------------------------------------------------------------------------
// Device manager
// ---------------------------------------------------------------------------------------------
struct glowb200_device_manager {
  int device = 0;
  uint64_t max_memory = 0, used_memory = 0;
  bool running = false;
  cudaStream_t stream = nullptr;      // kernels
  cudaStream_t in_stream = nullptr;   // host-to-device copies of asynchronous requests
  cudaStream_t out_stream = nullptr;  // device-to-host copies of asynchronous requests
  int contexts = 1;                   // execution contexts every network is loaded with
  int64_t next_ticket = 1;
  std::map<int64_t, int> finished;    // results of requests that were completed on behalf of a later one
  std::map<std::string, LoadedNetwork> networks;
  std::mutex lock;
};

extern "C" glowb200_device_manager *glowb200_device_manager_create(int device_id, uint64_t max_memory_bytes) {
  auto *dm = new glowb200_device_manager();
  dm->device = device_id;
  dm->max_memory = max_memory_bytes;
  return dm;
}

// DeviceManager::init: the CUDA context, the stream and the status word exist after this call, so
// that the first request does not pay for them (Glow's tests wait 2 s for a run).
extern "C" int glowb200_device_manager_init(glowb200_device_manager *dm) {
  if (!dm) return set_error(GLOWB200_RUNTIME_ERROR, "NULL device manager");
  std::lock_guard<std::mutex> g(dm->lock);
  if (dm->running) return GLOWB200_OK;
  if (cudaSetDevice(dm->device) != cudaSuccess) return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "cannot select CUDA device %d", dm->device);
  if (dm->max_memory == 0) {
    size_t fr = 0, tot = 0;
    if (cudaMemGetInfo(&fr, &tot) != cudaSuccess) return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "cudaMemGetInfo failed");
    dm->max_memory = fr;
  }
  if (cudaStreamCreateWithFlags(&dm->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&dm->in_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&dm->out_stream, cudaStreamNonBlocking) != cudaSuccess)
    return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "cannot create the streams of device %d", dm->device);
  dm->running = true;
  return GLOWB200_OK;
}

extern "C" uint64_t glowb200_device_manager_maximum_memory(glowb200_device_manager *dm) { return dm ? dm->max_memory : 0; }
extern "C" uint64_t glowb200_device_manager_available_memory(glowb200_device_manager *dm) {
  return dm ? dm->max_memory - dm->used_memory : 0;
}
extern "C" int glowb200_device_manager_is_memory_available(glowb200_device_manager *dm, uint64_t estimate) {
  return dm && dm->max_memory >= dm->used_memory + estimate;
}

static void free_network(LoadedNetwork &n) {
  for (auto &p : n.shared) if (p) cudaFree(p);
  for (Context &c : n.ctx) {
    if (c.slab[kPlaceholder]) cudaFree(c.slab[kPlaceholder]);
    if (c.slab[kActivation]) cudaFree(c.slab[kActivation]);
    if (c.workspace) cudaFree(c.workspace);
    if (c.status_dev) cudaFree(c.status_dev);
    if (c.status_host) cudaFreeHost(c.status_host);
    for (auto *j : c.jobs) if (j) cudaFree(j);
    if (c.in_done) cudaEventDestroy(c.in_done);
    if (c.run_done) cudaEventDestroy(c.run_done);
    if (c.out_done) cudaEventDestroy(c.out_done);
  }
  n.ctx.clear();
}

// Number of execution contexts networks are loaded with from now on (1 by default: one set of
// placeholders and activations, requests one after the other).
extern "C" int glowb200_device_manager_set_context_count(glowb200_device_manager *dm, int contexts) {
  if (!dm || contexts < 1 || contexts > 8) return set_error(GLOWB200_RUNTIME_ERROR, "context count must be in [1, 8]");
  std::lock_guard<std::mutex> g(dm->lock);
  dm->contexts = contexts;
  return GLOWB200_OK;
}

// addNetwork: name must be new, the network must fit the memory budget; uploads the constants.
extern "C" int glowb200_device_manager_add_network(glowb200_device_manager *dm, glowb200_function *f) {
  if (!dm || !f) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  std::lock_guard<std::mutex> g(dm->lock);
  if (!dm->running) return set_error(GLOWB200_RUNTIME_ERROR, "device manager is not initialised");
  if (!f->compiled) return set_error(GLOWB200_RUNTIME_ERROR, "function %s is not compiled", f->name.c_str());
  if (dm->networks.count(f->name)) return set_error(GLOWB200_RUNTIME_ERROR, "Failed to add network: already have a function called %s", f->name.c_str());
  size_t jobs_bytes = 0;
  for (const auto &grp : f->slws_groups) jobs_bytes += align_up(grp.size() * sizeof(glowb200_slws_job), 256);
  const uint64_t per_context = f->slab_bytes[kPlaceholder] + f->slab_bytes[kActivation] + f->workspace_bytes + jobs_bytes + 256;
  const uint64_t total = f->slab_bytes[kConstant] + f->slab_bytes[kStatic] + (uint64_t)dm->contexts * per_context;
  if (dm->used_memory + total > dm->max_memory) return set_error(GLOWB200_RUNTIME_OUT_OF_DEVICE_MEMORY, "Failed to add network: not enough memory");
  cudaSetDevice(dm->device);
  LoadedNetwork n;
  n.fn = f;
  n.device_bytes = total;
  bool ok = true;
  if (f->slab_bytes[kConstant]) ok = cudaMalloc(&n.shared[0], f->slab_bytes[kConstant]) == cudaSuccess;
  if (ok && f->slab_bytes[kStatic]) ok = cudaMalloc(&n.shared[1], f->slab_bytes[kStatic]) == cudaSuccess;
  n.ctx.resize(dm->contexts);
  for (Context &c : n.ctx) {
    if (!ok) break;
    c.slab[kConstant] = n.shared[0];
    c.slab[kStatic] = n.shared[1];
    if (f->slab_bytes[kPlaceholder]) ok = ok && cudaMalloc(&c.slab[kPlaceholder], f->slab_bytes[kPlaceholder]) == cudaSuccess;
    if (f->slab_bytes[kActivation]) ok = ok && cudaMalloc(&c.slab[kActivation], f->slab_bytes[kActivation]) == cudaSuccess;
    ok = ok && cudaMalloc(&c.workspace, f->workspace_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&c.status_dev, 4) == cudaSuccess && cudaMemsetAsync(c.status_dev, 0, 4, dm->stream) == cudaSuccess;
    ok = ok && cudaMallocHost(&c.status_host, 4) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&c.in_done, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&c.run_done, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&c.out_done, cudaEventDisableTiming) == cudaSuccess;
    // descriptors of the batched pooling launches: device addresses of this context's operands
    for (const auto &grp : f->slws_groups) {
      if (!ok) break;
      std::vector<glowb200_slws_job> jobs(grp.size());
      for (size_t k = 0; k < grp.size(); k++) {
        const Instruction &in = f->instrs[grp[k]];
        auto at = [&](int o) -> uint8_t * { const Symbol &sy = f->symbols[in.ops[o]]; return c.slab[sy.kind] + sy.offset + in.off[o]; };
        glowb200_slws_job &j = jobs[k];
        memset(&j, 0, sizeof(j));
        j.dest = at(0); j.data = at(1); j.weights = at(2); j.indices = at(3);
        j.lengths = reinterpret_cast<const int32_t *>(at(4));
        j.rows = in.ia[1]; j.num_indices = in.ia[5]; j.dest_stride = in.ia[3]; j.segments = in.ia[4];
      }
      glowb200_slws_job *dj = nullptr;
      ok = cudaMalloc(&dj, jobs.size() * sizeof(glowb200_slws_job)) == cudaSuccess &&
           cudaMemcpy(dj, jobs.data(), jobs.size() * sizeof(glowb200_slws_job), cudaMemcpyHostToDevice) == cudaSuccess;
      c.jobs.push_back(dj);
    }
  }
  if (ok)
    for (const Symbol &s : f->symbols)
      if (s.kind == kConstant && s.bytes)
        ok = ok && cudaMemcpyAsync(n.shared[0] + s.offset, s.host.data(), s.bytes, cudaMemcpyHostToDevice, dm->stream) == cudaSuccess;
  if (ok) ok = cudaStreamSynchronize(dm->stream) == cudaSuccess;
  if (!ok) {
    free_network(n);
    cudaGetLastError();
    return set_error(GLOWB200_RUNTIME_OUT_OF_DEVICE_MEMORY, "Failed to add network: device allocation or upload failed");
  }
  dm->used_memory += total;
  dm->networks[f->name] = std::move(n);
  return GLOWB200_OK;
}

extern "C" int glowb200_device_manager_evict_network(glowb200_device_manager *dm, const char *name) {
  if (!dm || !name) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  std::lock_guard<std::mutex> g(dm->lock);
  auto it = dm->networks.find(name);
  if (it == dm->networks.end()) return set_error(GLOWB200_RUNTIME_NET_NOT_FOUND, "Could not find function with name %s to evict", name);
  cudaSetDevice(dm->device);
  cudaStreamSynchronize(dm->in_stream);
  cudaStreamSynchronize(dm->stream);
  cudaStreamSynchronize(dm->out_stream);
  free_network(it->second);
  dm->used_memory -= it->second.device_bytes;
  dm->networks.erase(it);
  return GLOWB200_OK;
}

extern "C" int glowb200_device_manager_stop(glowb200_device_manager *dm) {
  if (!dm) return GLOWB200_OK;
  std::lock_guard<std::mutex> g(dm->lock);
  if (!dm->running) return GLOWB200_OK;
  cudaSetDevice(dm->device);
  cudaStreamSynchronize(dm->in_stream);
  cudaStreamSynchronize(dm->stream);
  cudaStreamSynchronize(dm->out_stream);
  for (auto &kv : dm->networks) free_network(kv.second);
  dm->networks.clear();
  dm->finished.clear();
  dm->used_memory = 0;
  cudaStreamDestroy(dm->stream);
  cudaStreamDestroy(dm->in_stream);
  cudaStreamDestroy(dm->out_stream);
  dm->stream = dm->in_stream = dm->out_stream = nullptr;
  dm->running = false;
  return GLOWB200_OK;
}

extern "C" void glowb200_device_manager_destroy(glowb200_device_manager *dm) {
  if (dm) {
    glowb200_device_manager_stop(dm);
    delete dm;
  }
}

namespace {

int execute(glowb200_device_manager *dm, LoadedNetwork &n, Context &c) {
  glowb200_function *f = n.fn;
  auto ptr = [&](int id) -> void * {  // a whole symbol (the constants compile() derived)
    if (id < 0) return nullptr;
    const Symbol &s = f->symbols[id];
    return c.slab[s.kind] + s.offset;
  };
  void *st = dm->stream;
  for (size_t ii = 0; ii < f->instrs.size(); ii++) {
    const Instruction &in = f->instrs[ii];
    const auto &a = in.ia;
    auto P = [&](int o) -> void * {  // operand o: its symbol's address plus the view's offset
      const int id = in.ops[o];
      if (id < 0) return nullptr;
      const Symbol &s = f->symbols[id];
      return c.slab[s.kind] + s.offset + in.off[o];
    };
    int rc = GLOWB200_OK;
    switch (in.kind) {
      case GLOWB200_INSTR_FRWQ_SLWS:
        if (in.group >= 0) {  // part of a batched launch: the first member launches it for all
          if (in.group_leader) {
            const auto &grp = f->slws_groups[in.group];
            int64_t max_segments = 0;
            for (int m : grp) max_segments = std::max(max_segments, f->instrs[m].ia[4]);
            rc = glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum_batched(
                c.jobs[in.group], (int64_t)grp.size(), max_segments, (int)a[0], (int)a[6], a[2], a[3], (int)a[7], (int)a[8],
                c.workspace, f->workspace_bytes, c.status_dev, st);
          }
          break;
        }
        rc = glowb200_fused_rowwise_quantized_sparse_lengths_weighted_sum(
            P(0), P(1), (int)a[0], a[1], P(2), P(3), (int)a[6],
            (const int32_t *)P(4), a[4], a[5], a[2], a[3], (int)a[7], (int)a[8], c.workspace, f->workspace_bytes,
            c.status_dev, st);
        break;
      case GLOWB200_INSTR_RWQ_FC: {
        auto d = [&](int i) { return (const int32_t *)ptr(in.derived[i]); };
        rc = glowb200_rowwise_quantized_fc_i8_i32(
            (int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2), (const int32_t *)P(5),
            (const int32_t *)P(4), d(0), d(1), d(2), d(3), d(4), d(5), a[0], a[1], a[2], (int32_t)a[5], (int32_t)a[3],
            (int32_t)a[4], d(6), a[6] ? GLOWB200_FC_FUSE_RELU : 0, c.workspace, f->workspace_bytes, c.status_dev, st);
        break;
      }
      case GLOWB200_INSTR_CWQ_CONV: {
        auto d = [&](int i) { return (const int32_t *)ptr(in.derived[i]); };
        const int64_t od[4] = {a[0], a[4], a[5], a[6]}, id[4] = {a[0], a[1], a[2], a[3]}, fd[4] = {a[6], a[7], a[8], a[3] / a[15]};
        const int64_t k[2] = {a[7], a[8]}, s[2] = {a[9], a[10]}, p[4] = {a[11], a[12], a[13], a[14]}, dl[2] = {a[16], a[17]};
        rc = glowb200_channelwise_quantized_conv2d_i8_i32(
            (int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2), (const int32_t *)P(3),
            od, id, fd, k, s, p, a[15], dl, (int32_t)a[19], (int32_t)a[18], (const int32_t *)P(5),
            (const int32_t *)P(7), d(0), d(1), d(2), d(3), d(4), d(5), (int32_t)a[20], nullptr, nullptr, 0, c.workspace,
            f->workspace_bytes, c.status_dev, st);
        break;
      }
      case GLOWB200_INSTR_ADD:
        rc = glowb200_element_add_i8((int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2), a[0],
                                     (int32_t)a[1], (int32_t)a[2], (int32_t)a[3], (int32_t)a[4], (int32_t)a[5], (int32_t)a[6],
                                     (int32_t)a[7], (int32_t)a[8], (int32_t)a[9], st);
        break;
      case GLOWB200_INSTR_MAXSPLAT:
        rc = glowb200_element_maxsplat_i8((int8_t *)P(0), (const int8_t *)P(1), a[0], (int32_t)a[1], st);
        break;
      case GLOWB200_INSTR_QUANTIZE:
        if (in.absorbed) break;  // the Transpose behind it does both
        rc = glowb200_element_quantize_i8((int8_t *)P(0), (const float *)P(1), a[0], in.fa[0], (int32_t)a[1], st);
        break;
      case GLOWB200_INSTR_DEQUANTIZE:
        rc = glowb200_element_dequantize_i8((float *)P(0), (const int8_t *)P(1), a[0], in.fa[0], (int32_t)a[1], st);
        break;
      case GLOWB200_INSTR_MAXPOOL: {
        const int64_t id[4] = {a[0], a[1], a[2], a[3]}, od[4] = {a[0], a[4], a[5], a[3]}, k[2] = {a[6], a[7]}, s[2] = {a[8], a[9]};
        const int64_t p[4] = {a[10], a[11], a[10], a[11]};
        rc = glowb200_max_pool_i8((const int8_t *)P(1), (int8_t *)P(0), id, od, k, s, p, (int32_t)a[12], st);
        break;
      }
      case GLOWB200_INSTR_AVGPOOL: {
        const int64_t id[4] = {a[0], a[1], a[2], a[3]}, od[4] = {a[0], a[4], a[5], a[3]}, k[2] = {a[6], a[7]}, s[2] = {a[8], a[9]};
        const int64_t p[4] = {a[10], a[11], a[10], a[11]};
        rc = glowb200_avg_pool_i8((const int8_t *)P(1), (int8_t *)P(0), id, od, k, s, p, (int)a[14], (int32_t)a[13],
                                  (int32_t)a[12], (int32_t)a[15], (int32_t)a[16], (int32_t)a[17], st);
        break;
      }
      case GLOWB200_INSTR_TRANSPOSE: {
        const int nd = (int)a[0];
        int64_t dims[4];
        int32_t sh[4];
        for (int i = 0; i < nd; i++) { dims[i] = a[2 + i]; sh[i] = (int32_t)a[6 + i]; }
        if (in.quantizes) rc = glowb200_quantize_transpose_i8((int8_t *)P(0), (const float *)P(2), dims, sh, nd, in.fa[0], (int32_t)a[10], st);
        else rc = glowb200_transpose(P(1), P(0), dims, sh, nd, (int)a[1], st);
        break;
      }
      case GLOWB200_INSTR_COPY:
        if (cudaMemcpyAsync(P(0), P(1), (size_t)a[0], cudaMemcpyDeviceToDevice, dm->stream) != cudaSuccess)
          rc = set_error(GLOWB200_RUNTIME_ERROR, "copy failed");
        break;
      case GLOWB200_INSTR_ADD_MAXSPLAT:
        rc = glowb200_element_add_maxsplat_i8((int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2),
                                              a[0], (int32_t)a[1], (int32_t)a[2], (int32_t)a[3], (int32_t)a[5], (int32_t)a[6],
                                              (int32_t)a[7], (int32_t)a[8], (int32_t)a[9], (int32_t)a[10], (int32_t)a[4], st);
        break;
      case GLOWB200_INSTR_RELU:
        rc = glowb200_element_relu_i8((int8_t *)P(0), (const int8_t *)P(1), a[0], (int32_t)a[1], (int32_t)a[2],
                                      (int32_t)a[3], (int32_t)a[4], (int32_t)a[5], st);
        break;
      case GLOWB200_INSTR_RESCALE:
        rc = glowb200_element_rescale_i8((int8_t *)P(0), (const int8_t *)P(1), a[0], (int32_t)a[2], (int32_t)a[1],
                                         (int32_t)a[3], (int32_t)a[4], (int32_t)a[5], st);
        break;
      case GLOWB200_INSTR_FC_I8:
        rc = glowb200_fc_i8_i32((int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2),
                                (const int32_t *)P(3), a[0], a[1], a[2], (int32_t)a[6], (int32_t)a[3], (int32_t)a[4],
                                (int32_t)a[5], (int32_t)a[7], (int32_t)a[8], (int32_t)a[9], (int32_t)a[10], (int32_t)a[11],
                                (int32_t)a[12], nullptr, 0, c.workspace, f->workspace_bytes, c.status_dev, st);
        break;
      case GLOWB200_INSTR_MATMUL_I8:
        rc = glowb200_matmul_i8((int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2), a[0], a[1],
                                a[2], (int32_t)a[5], (int32_t)a[3], (int32_t)a[4], (int32_t)a[6], (int32_t)a[7], (int32_t)a[8], 0,
                                c.workspace, f->workspace_bytes, c.status_dev, st);
        break;
      case GLOWB200_INSTR_SPLAT:
        rc = glowb200_splat_f(P(0), a[0], in.fa[0], (int)a[1], st);
        break;
      case GLOWB200_INSTR_INSERT_TENSOR:
        if (cudaMemcpy2DAsync((uint8_t *)P(0) + a[3], (size_t)a[2], P(1), (size_t)a[1], (size_t)a[1], (size_t)a[0],
                              cudaMemcpyDeviceToDevice, dm->stream) != cudaSuccess)
          rc = set_error(GLOWB200_RUNTIME_ERROR, "insert-tensor copy failed");
        break;
      case GLOWB200_INSTR_PAIRWISE_DOT:
        rc = glowb200_pairwise_dot_interaction((const float *)P(1), a[3], (const float *)P(2), a[4], a[0], a[1], a[2],
                                               a[6] ? nullptr : (float *)P(0), a[6] ? (int8_t *)P(0) : nullptr, a[5],
                                               in.fa[0], (int32_t)a[7], st);
        break;
      case GLOWB200_INSTR_SLWS_F32:
        rc = glowb200_sparse_lengths_weighted_sum_f32((float *)P(0), (const float *)P(1), a[0],
                                                      (const float *)P(2), P(3), (int)a[4],
                                                      (const int32_t *)P(4), a[2], a[3], a[1], c.workspace,
                                                      f->workspace_bytes, c.status_dev, st);
        break;
      case GLOWB200_INSTR_RWQ_SLWS:
        rc = glowb200_rowwise_quantized_sparse_lengths_weighted_sum_f32(
            (float *)P(0), (const uint8_t *)P(1), (const float *)P(2), (const float *)P(3), a[0],
            (const float *)P(4), P(5), (int)a[4], (const int32_t *)P(6), a[2], a[3], a[1], c.workspace,
            f->workspace_bytes, c.status_dev, st);
        break;
      case GLOWB200_INSTR_BINARY_I8:
        rc = glowb200_element_binary_i8((int)a[4], (int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2),
                                        a[0], (int32_t)a[1], (int32_t)a[2], (int32_t)a[3], (int32_t)a[5], (int32_t)a[6], (int32_t)a[7],
                                        (int32_t)a[8], (int32_t)a[9], (int32_t)a[10], st);
        break;
      case GLOWB200_INSTR_MULDIV_I8:
        rc = glowb200_element_muldiv_i8((int)a[4], (int8_t *)P(0), (const int8_t *)P(1), (const int8_t *)P(2),
                                        a[0], (int32_t)a[1], (int32_t)a[2], (int32_t)a[3], (int32_t)a[5], (int32_t)a[6], (int32_t)a[7], st);
        break;
      case GLOWB200_INSTR_BATCHED_ADD_I8:
        rc = glowb200_batched_add_i8((int8_t *)P(0), (const int8_t *)P(1), P(2), (int)a[5], a[0], a[1],
                                     (int32_t)a[2], (int32_t)a[3], (int32_t)a[4], (int32_t)a[6], (int32_t)a[7], (int32_t)a[8],
                                     (int32_t)a[9], (int32_t)a[10], (int32_t)a[11], st);
        break;
      case GLOWB200_INSTR_SPLIT_EMBEDDING:
        rc = glowb200_int_nbit_split_embedding_bags(
            P(0), P(1), a[0], P(2), a[1], (const int32_t *)P(3), P(4), (int)a[7],
            (const uint8_t *)P(5), (const int32_t *)P(6), a[2], a[3], P(7), P(8), (int)a[6],
            a[4], a[5], (int)a[8], P(9), (int)a[9], (int)a[10], (int)a[11], (int)a[12], c.status_dev, st);
        break;
      case GLOWB200_INSTR_DYN_QUANTIZED_FC:
        if (in.ops[4] >= 0)
          rc = glowb200_dynamic_rowwise_quantized_fc(P(0), P(1), (const int8_t *)P(2),
                                                     (const float *)P(3), (const float *)P(4),
                                                     (const int32_t *)P(5), a[0], a[1], a[2], nullptr, 0, c.workspace,
                                                     f->workspace_bytes, c.status_dev, st);
        else
          rc = glowb200_dynamic_quantized_fc(P(0), P(1), (const int8_t *)P(2),
                                             (const float *)P(3), in.fa[0], (int32_t)a[3], a[0], a[1], a[2], nullptr, 0,
                                             c.workspace, f->workspace_bytes, c.status_dev, st);
        break;
      case GLOWB200_INSTR_EMBEDDING_BAG:
        rc = glowb200_embedding_bag_byte_rowwise_offsets(P(0), P(1), (int)a[0], a[1], P(2), P(3),
                                                         P(4), (int)a[6], a[4], a[5], a[2], a[3], (int)a[7], (int)a[8],
                                                         (int)a[9], c.workspace, f->workspace_bytes, c.status_dev, st);
        break;
    }
    if (rc != GLOWB200_OK) {
      // keep the kernel ABI's message, report it as a runtime error of this instruction
      char msg[400];
      snprintf(msg, sizeof(msg), "%s", glowb200_last_error());
      return set_error(GLOWB200_RUNTIME_ERROR, "instruction %zu of %s failed: %s", ii, f->name.c_str(), msg);
    }
  }
  return GLOWB200_OK;
}

}  // namespace

// runFunction: `bindings` pairs placeholder names with HOST buffers (the PlaceholderBindings of
// an ExecutionContext).  Every bound placeholder is copied to the device before the run and
// every bound placeholder is copied back after it -- inputs come back unchanged, outputs carry
// the results (LLVMCompiledFunction::loadPlaceholders / updatePlaceholders,
// lib/LLVMIRCodeGen/LLVMCompiledFunction.cpp:33-71, do the same with memcpy).  A binding may be
// shorter than the placeholder (a partial tensor, supportsPartialTensors): the rest is zeroed.
extern "C" int glowb200_device_manager_run_function(glowb200_device_manager *dm, const char *name, const char *const *placeholder_names,
                                                    void *const *host_buffers, const size_t *buffer_bytes, int num_bindings) {
  return glowb200_device_manager_run_function_io(dm, name, placeholder_names, host_buffers, buffer_bytes, nullptr, num_bindings);
}

namespace {
int status_to_error(int32_t status, const char *name) {
  if (status & GLOWB200_STATUS_WAIT_TIMEOUT) return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "a device-side wait gave up while running %s", name);
  if (status) return set_error(GLOWB200_RUNTIME_ERROR, "invalid sparse input to %s (status bits 0x%x: index out of range 1, lengths overrun 2, negative length 4, bad offsets 8, unsupported table 32)", name, status);
  return GLOWB200_OK;
}

// Finishes a synchronous request: the status word, the stream, the mapping of what went wrong.
int finish_request(glowb200_device_manager *dm, Context &c, const char *name) {
  int32_t status = 0;
  cudaMemcpyAsync(&status, c.status_dev, 4, cudaMemcpyDeviceToHost, dm->stream);
  cudaMemsetAsync(c.status_dev, 0, 4, dm->stream);
  const cudaError_t e = cudaStreamSynchronize(dm->stream);
  if (e != cudaSuccess) return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "device error while running %s: %s", name, cudaGetErrorString(e));
  return status_to_error(status, name);
}

// A request that failed on the host part-way through: kernels and copies already queued are
// waited for (the caller may reuse its buffers as soon as the error returns) and whatever they
// raised in the status word is dropped with the request, so the next one starts clean.  The
// message of the failure that led here is kept.
int abort_request(glowb200_device_manager *dm, Context &c, int rc) {
  char msg[512];
  snprintf(msg, sizeof(msg), "%s", glowb200_last_error());
  bool ok = cudaStreamSynchronize(dm->in_stream) == cudaSuccess;
  cudaMemsetAsync(c.status_dev, 0, 4, dm->stream);
  ok = cudaStreamSynchronize(dm->stream) == cudaSuccess && ok;
  ok = cudaStreamSynchronize(dm->out_stream) == cudaSuccess && ok;
  c.ticket = 0;
  if (!ok) {
    cudaGetLastError();
    return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "device error after a failed request (%s)", msg);
  }
  return set_error(rc, "%s", msg);
}

// Completes the asynchronous request in flight on a context (if any) and returns its result.
int complete_context(glowb200_device_manager *dm, Context &c, const char *name) {
  if (c.ticket == 0) return GLOWB200_OK;
  const cudaError_t e = cudaEventSynchronize(c.out_done);
  c.ticket = 0;
  if (e != cudaSuccess) return set_error(GLOWB200_RUNTIME_DEVICE_NONRECOVERABLE, "device error while running %s: %s", name, cudaGetErrorString(e));
  const int32_t status = *c.status_host;
  return status_to_error(status, name);
}

// Where a placeholder of a loaded network lives (context 0 for the per-context kind); dm->lock
// is held by the caller.
int find_placeholder(glowb200_device_manager *dm, const char *name, const char *placeholder, void **device_ptr, size_t *bytes) {
  auto it = dm->networks.find(name);
  if (it == dm->networks.end()) return set_error(GLOWB200_RUNTIME_NET_NOT_FOUND, "Function %s not found", name);
  glowb200_function *f = it->second.fn;
  auto s = f->by_name.find(placeholder);
  if (s == f->by_name.end() || (f->symbols[s->second].kind != kPlaceholder && f->symbols[s->second].kind != kStatic))
    return set_error(GLOWB200_RUNTIME_ERROR, "%s is not a placeholder of %s", placeholder, name);
  const Symbol &sym = f->symbols[s->second];
  *device_ptr = it->second.ctx[0].slab[sym.kind] + sym.offset;
  if (bytes) *bytes = sym.bytes;
  return GLOWB200_OK;
}

// Resolves the bindings of a request against the network's placeholders.
int resolve_bindings(glowb200_function *f, const char *name, const char *const *placeholder_names, const size_t *buffer_bytes,
                     int num_bindings, std::vector<int> &ids) {
  ids.resize(num_bindings);
  for (int b = 0; b < num_bindings; b++) {
    auto s = f->by_name.find(placeholder_names[b]);
    if (s == f->by_name.end() || f->symbols[s->second].kind != kPlaceholder)
      return set_error(GLOWB200_RUNTIME_ERROR, "%s is not a placeholder of %s", placeholder_names[b], name);
    ids[b] = s->second;
    if (buffer_bytes[b] > f->symbols[ids[b]].bytes)
      return set_error(GLOWB200_RUNTIME_ERROR, "binding of %s is larger than the placeholder", f->symbols[ids[b]].name.c_str());
  }
  return GLOWB200_OK;
}
}  // namespace

// Device-resident tensors and static placeholders (DeviceManager::transferToDevice /
// transferFromDevice / transferStaticPlaceholderToDevice, include/glow/Backends/DeviceManager.h:
// 163-231): where a placeholder of a loaded network lives on the device.
extern "C" int glowb200_device_manager_placeholder_address(glowb200_device_manager *dm, const char *name, const char *placeholder,
                                                           void **device_ptr, size_t *bytes) {
  if (!dm || !name || !placeholder || !device_ptr) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  std::lock_guard<std::mutex> g(dm->lock);
  return find_placeholder(dm, name, placeholder, device_ptr, bytes);
}

extern "C" int glowb200_device_manager_transfer_static_placeholder(glowb200_device_manager *dm, const char *name,
                                                                   const char *placeholder, const void *host, size_t bytes) {
  if (!dm || !name || !placeholder) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  void *d = nullptr;
  size_t cap = 0;
  // one critical section from the lookup to the end of the copy: an eviction in between would
  // free the slab the copy writes
  std::lock_guard<std::mutex> g(dm->lock);
  if (int rc = find_placeholder(dm, name, placeholder, &d, &cap)) return rc;
  if (!host || bytes > cap) return set_error(GLOWB200_RUNTIME_ERROR, "static placeholder %s: NULL buffer or more bytes than the placeholder holds", placeholder);
  cudaSetDevice(dm->device);
  if (cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, dm->stream) != cudaSuccess || cudaStreamSynchronize(dm->stream) != cudaSuccess)
    return set_error(GLOWB200_RUNTIME_ERROR, "host-to-device copy of %s failed", placeholder);
  return GLOWB200_OK;
}

extern "C" int glowb200_device_manager_run_function_resident(glowb200_device_manager *dm, const char *name) {
  if (!dm || !name) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  std::lock_guard<std::mutex> g(dm->lock);
  if (!dm->running) return set_error(GLOWB200_RUNTIME_ERROR, "device manager is not initialised");
  auto it = dm->networks.find(name);
  if (it == dm->networks.end()) return set_error(GLOWB200_RUNTIME_NET_NOT_FOUND, "Function %s not found", name);
  cudaSetDevice(dm->device);
  Context &c = it->second.ctx[0];
  if (c.ticket) {  // an asynchronous request still owns the context: let it finish, keep its result
    const int64_t t = c.ticket;
    dm->finished[t] = complete_context(dm, c, name);
  }
  if (int rc = execute(dm, it->second, c)) return abort_request(dm, c, rc);
  return finish_request(dm, c, name);
}

extern "C" int glowb200_device_manager_run_function_io(glowb200_device_manager *dm, const char *name, const char *const *placeholder_names,
                                                       void *const *host_buffers, const size_t *buffer_bytes, const int *directions,
                                                       int num_bindings) {
  if (!dm || !name) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  std::lock_guard<std::mutex> g(dm->lock);
  if (!dm->running) return set_error(GLOWB200_RUNTIME_ERROR, "device manager is not initialised");
  auto it = dm->networks.find(name);
  if (it == dm->networks.end()) return set_error(GLOWB200_RUNTIME_NET_NOT_FOUND, "Function %s not found", name);
  LoadedNetwork &n = it->second;
  glowb200_function *f = n.fn;
  cudaSetDevice(dm->device);
  std::vector<int> ids;
  if (int rc = resolve_bindings(f, name, placeholder_names, buffer_bytes, num_bindings, ids)) return rc;
  Context &c = n.ctx[0];
  if (c.ticket) {
    const int64_t t = c.ticket;
    dm->finished[t] = complete_context(dm, c, name);
  }
  for (int b = 0; b < num_bindings; b++) {
    const Symbol &sym = f->symbols[ids[b]];
    uint8_t *d = c.slab[kPlaceholder] + sym.offset;
    if (directions && !(directions[b] & GLOWB200_BINDING_INPUT)) continue;  // an output: nothing to copy in
    bool ok = cudaMemcpyAsync(d, host_buffers[b], buffer_bytes[b], cudaMemcpyHostToDevice, dm->stream) == cudaSuccess;
    if (ok && buffer_bytes[b] < sym.bytes) ok = cudaMemsetAsync(d + buffer_bytes[b], 0, sym.bytes - buffer_bytes[b], dm->stream) == cudaSuccess;
    if (!ok) return abort_request(dm, c, set_error(GLOWB200_RUNTIME_ERROR, "host-to-device copy of %s failed", sym.name.c_str()));
  }
  if (int rc = execute(dm, n, c)) return abort_request(dm, c, rc);
  for (int b = 0; b < num_bindings; b++) {
    const Symbol &sym = f->symbols[ids[b]];
    if (directions && !(directions[b] & GLOWB200_BINDING_OUTPUT)) continue;  // an input: nothing to copy back
    if (cudaMemcpyAsync(host_buffers[b], c.slab[kPlaceholder] + sym.offset, buffer_bytes[b], cudaMemcpyDeviceToHost, dm->stream) != cudaSuccess)
      return abort_request(dm, c, set_error(GLOWB200_RUNTIME_ERROR, "device-to-host copy of %s failed", sym.name.c_str()));
  }
  return finish_request(dm, c, name);
}

// The asynchronous request: the inputs go in on one stream, the kernels run on a second, the
// results leave on a third, ordered by events -- so that with two or more execution contexts
// (glowb200_device_manager_set_context_count) the inputs of request i + 1 arrive while request
// i runs and the results of request i - 1 leave, as Glow's executor overlaps them when a
// backend offers several contexts.  The host buffers must stay valid, and should be pinned,
// until glowb200_device_manager_wait has returned the ticket's result.  Contexts are taken in
// turn; a context whose last request has not been waited for is completed first (its result is
// kept for its own wait call).
extern "C" int glowb200_device_manager_run_function_async(glowb200_device_manager *dm, const char *name,
                                                          const char *const *placeholder_names, void *const *host_buffers,
                                                          const size_t *buffer_bytes, const int *directions, int num_bindings,
                                                          int64_t *ticket) {
  if (!dm || !name || !ticket) return set_error(GLOWB200_RUNTIME_ERROR, "NULL argument");
  std::lock_guard<std::mutex> g(dm->lock);
  if (!dm->running) return set_error(GLOWB200_RUNTIME_ERROR, "device manager is not initialised");
  auto it = dm->networks.find(name);
  if (it == dm->networks.end()) return set_error(GLOWB200_RUNTIME_NET_NOT_FOUND, "Function %s not found", name);
  LoadedNetwork &n = it->second;
  glowb200_function *f = n.fn;
  cudaSetDevice(dm->device);
  std::vector<int> ids;
  if (int rc = resolve_bindings(f, name, placeholder_names, buffer_bytes, num_bindings, ids)) return rc;
  Context &c = n.ctx[n.next_ctx];
  n.next_ctx = (n.next_ctx + 1) % n.ctx.size();
  if (c.ticket) {
    const int64_t t = c.ticket;
    dm->finished[t] = complete_context(dm, c, name);
  }
  // inputs: the context's previous kernels and copies are complete (completed above, or waited
  // for by the caller), so nothing still reads or writes these placeholders
  for (int b = 0; b < num_bindings; b++) {
    const Symbol &sym = f->symbols[ids[b]];
    uint8_t *d = c.slab[kPlaceholder] + sym.offset;
    if (directions && !(directions[b] & GLOWB200_BINDING_INPUT)) continue;
    bool ok = cudaMemcpyAsync(d, host_buffers[b], buffer_bytes[b], cudaMemcpyHostToDevice, dm->in_stream) == cudaSuccess;
    if (ok && buffer_bytes[b] < sym.bytes) ok = cudaMemsetAsync(d + buffer_bytes[b], 0, sym.bytes - buffer_bytes[b], dm->in_stream) == cudaSuccess;
    if (!ok) return abort_request(dm, c, set_error(GLOWB200_RUNTIME_ERROR, "host-to-device copy of %s failed", sym.name.c_str()));
  }
  bool ok = cudaEventRecord(c.in_done, dm->in_stream) == cudaSuccess && cudaStreamWaitEvent(dm->stream, c.in_done, 0) == cudaSuccess;
  if (!ok) return abort_request(dm, c, set_error(GLOWB200_RUNTIME_ERROR, "cannot order the streams of %s", name));
  if (int rc = execute(dm, n, c)) return abort_request(dm, c, rc);
  ok = cudaEventRecord(c.run_done, dm->stream) == cudaSuccess && cudaStreamWaitEvent(dm->out_stream, c.run_done, 0) == cudaSuccess;
  for (int b = 0; b < num_bindings && ok; b++) {
    const Symbol &sym = f->symbols[ids[b]];
    if (directions && !(directions[b] & GLOWB200_BINDING_OUTPUT)) continue;
    ok = cudaMemcpyAsync(host_buffers[b], c.slab[kPlaceholder] + sym.offset, buffer_bytes[b], cudaMemcpyDeviceToHost, dm->out_stream) == cudaSuccess;
  }
  ok = ok && cudaMemcpyAsync(c.status_host, c.status_dev, 4, cudaMemcpyDeviceToHost, dm->out_stream) == cudaSuccess &&
       cudaMemsetAsync(c.status_dev, 0, 4, dm->out_stream) == cudaSuccess && cudaEventRecord(c.out_done, dm->out_stream) == cudaSuccess;
  if (!ok) return abort_request(dm, c, set_error(GLOWB200_RUNTIME_ERROR, "device-to-host copies of %s failed", name));
  c.ticket = dm->next_ticket++;
  *ticket = c.ticket;
  return GLOWB200_OK;
}

// Blocks until the request behind `ticket` is complete (its outputs are in the host buffers)
// and returns its result: GLOWB200_OK, or the error the synchronous call would have returned.
extern "C" int glowb200_device_manager_wait(glowb200_device_manager *dm, int64_t ticket) {
  if (!dm || ticket <= 0) return set_error(GLOWB200_RUNTIME_ERROR, "bad ticket");
  std::lock_guard<std::mutex> g(dm->lock);
  auto done = dm->finished.find(ticket);
  if (done != dm->finished.end()) {
    const int rc = done->second;
    dm->finished.erase(done);
    if (rc != GLOWB200_OK) return set_error(rc, "request %lld failed (completed on behalf of a later request)", (long long)ticket);
    return GLOWB200_OK;
  }
  cudaSetDevice(dm->device);
  for (auto &kv : dm->networks)
    for (Context &c : kv.second.ctx)
      if (c.ticket == ticket) return complete_context(dm, c, kv.first.c_str());
  return set_error(GLOWB200_RUNTIME_ERROR, "no request with ticket %lld is in flight", (long long)ticket);
}

// Pinned host memory for the buffers of asynchronous requests (DeviceManager::allocateDeviceIOBuffer,
// include/glow/Backends/DeviceManager.h:150-160).
extern "C" void *glowb200_device_manager_allocate_io_buffer(glowb200_device_manager *dm, size_t bytes) {
  if (!dm || bytes == 0) return nullptr;
  cudaSetDevice(dm->device);
  void *p = nullptr;
  if (cudaMallocHost(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    set_error(GLOWB200_RUNTIME_ERROR, "cannot allocate %zu bytes of pinned host memory", bytes);
    return nullptr;
  }
  return p;
}

extern "C" void glowb200_device_manager_free_io_buffer(glowb200_device_manager *dm, void *buffer) {
  if (dm && buffer) cudaFreeHost(buffer);
}
