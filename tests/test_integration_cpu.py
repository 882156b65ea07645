"""The Glow-side glue under integration/ cannot be compiled here (Glow needs LLVM, folly, glog);
these checks keep its pieces in step with each other and with the library's header by reading
the sources."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B200 = os.path.join(ROOT, "integration", "glow", "lib", "Backends", "B200")

# runtime instructions no Glow IR instruction maps to: fusions the library offers to callers that
# build functions themselves (the models under glow_b200/), and the interaction kernel
NOT_FROM_GLOW_IR = {"MAXSPLAT", "ADD_MAXSPLAT", "PAIRWISE_DOT"}
# emitted for an IR-only instruction outside the operator table
IR_ONLY = {"COPY"}


def _ops():
    text = open(os.path.join(B200, "B200Ops.def")).read()
    return re.findall(r"^B200_OP\((\w+),\s*(\w+),\s*(\w+),\s*(\w+)\)", text, re.M)


def test_every_runtime_instruction_has_an_adapter_case():
    header = open(os.path.join(ROOT, "include", "glow_b200.h")).read()
    kinds = set(re.findall(r"#define GLOWB200_INSTR_(\w+)\s+\d+", header))
    assert len(kinds) >= 27
    emitted = {r for _, _, r, _ in _ops()} | IR_ONLY
    assert kinds - emitted == NOT_FROM_GLOW_IR, "instruction kinds without an adapter case: %s" % sorted(kinds - emitted - NOT_FROM_GLOW_IR)
    assert emitted <= kinds


def test_every_table_entry_has_its_translation_and_its_predicate():
    fn = open(os.path.join(B200, "B200Function.cpp")).read()
    be = open(os.path.join(B200, "B200Backend.cpp")).read()
    assert '#include "B200Ops.def"' in fn and '#include "B200Ops.def"' in be
    for node, inst, runtime, pred in _ops():
        assert re.search(r"Error emit%s\(const %sInst \*" % (inst, inst), fn), "no translation of %sInst" % inst
        assert "GLOWB200_INSTR_%s" % runtime in fn
        assert re.search(r"bool supports%s\(" % pred, be), "no predicate %s" % pred
    # translation errors are returned, never fatal, and reach addNetwork's callback
    assert "EXIT_ON_ERR" not in fn
    dm = open(os.path.join(B200, "B200DeviceManager.cpp")).read()
    assert "F->translate(module)" in dm and "readyCB(module, std::move(err))" in dm
    for hook in ("transferToDevice", "transferFromDevice", "transferStaticPlaceholderToDevice", "allocateDeviceIOBuffer"):
        assert "B200DeviceManager::%s" % hook in dm
    assert "B200Backend::bindContexts" in be and "B200Backend::getContextCount" in be


def test_blacklist_is_generated_and_names_the_tests_kept():
    bl = open(os.path.join(B200, "tests", "B200OperatorTest.cpp")).read()
    names = set(re.findall(r'"(\w+)/0"', bl))
    assert len(names) > 500
    for kept in ("FusedRowwiseQuantizedSparseLengthsWeightedSum_Float", "rowwiseQuantizedFCTest_Int8_BiasInt32",
                 "ChannelwiseQuantizedConv2D", "EmbeddingBag4BitRowwiseOffsets_Float16", "IntMatMul"):
        assert kept not in names
    for dropped in ("less_float", "Conv3DQuantizedTest_Int8_BiasInt8", "SparseLengthsSum_BFloat16"):
        assert dropped in names
