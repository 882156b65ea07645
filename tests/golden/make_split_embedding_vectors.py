"""Extracts the IntNBitSplitEmbedding(Weighted)Bags cases of pytorch/glow's own operator tests
into split_embedding_vectors.json.

usage: python make_split_embedding_vectors.py <glow checkout>/tests/unittests/OperatorTest.cpp

The test file is read as text: the initialiser lists of the helper functions (table bytes,
indices, offsets, per-index weights) and of every TEST_P (expected tensor, pooling mode, types,
tolerance) are copied as numbers.  Nothing of the reference is compiled or run.
"""
import json
import os
import re
import sys


def numbers(block):
    block = re.sub(r"//[^\n]*", "", block)
    return [float(x) for x in re.findall(r"-?\d+\.?\d*(?:[eE][-+]?\d+)?", block)]


def init_list(text, start, marker):
    """Numbers of the first `marker ... = { ... };` initialiser at or after `start`."""
    at = text.index(marker, start)
    lo = text.index("{", text.index("=", at))
    hi = text.index("}", lo)
    return numbers(text[lo + 1:hi]), hi


def function_body(text, signature):
    at = text.index(signature)
    end = text.index("\n}\n", at)
    return text[at:end], at


SPARSE = {"EST_FLOAT": 0, "EST_FLOAT16": 1, "EST_INT8": 2, "EST_INT4": 3}
POOL = {"EP_SUM": 0, "EP_MEAN": 1}


def main(path):
    text = open(path).read()
    line_of = lambda pos: text.count("\n", 0, pos) + 1
    out = {"_about": "IntNBitSplitEmbeddingBags / IntNBitSplitEmbeddingWeightedBags cases of "
                     "pytorch/glow tests/unittests/OperatorTest.cpp, extracted as numbers by "
                     "make_split_embedding_vectors.py; weights_tys / pooling / output_dtype use the "
                     "enum values of include/glow/Graph/Nodes.h:296-309; placements 3 = HOST "
                     "(dev_weights), 1 = MANAGED (uvm_weights)."}

    body, at = function_body(text, "static void testIntNBitSplitEmbeddingBagsSingle(")
    single = {"source_line": line_of(at)}
    single["weights"], _ = init_list(body, 0, "devWeightsTensorReal.getHandle<uint8_t>()")
    single["indices"], _ = init_list(body, 0, "indicesTensorReal.getHandle<IndexTy>()")
    single["offsets"], _ = init_list(body, 0, "offsetsTensorReal.getHandle<IndexTy>()")
    single["dim_offsets"], _ = init_list(body, 0, "dimOffsetsTensorReal.getHandle<int32_t>()")
    single["placements"], _ = init_list(body, 0, "weightsPlacementReal.getHandle<int32_t>()")
    single["weights_offsets"], _ = init_list(body, 0, "weightsOffsetsReal.getHandle<int32_t>()")
    single["total_dims"] = 1
    out["single_setup"] = single

    body, at = function_body(text, "static void testIntNBitSplitEmbeddingBags(")
    multi = {"source_line": line_of(at)}
    multi["indices"], _ = init_list(body, 0, "indicesTensorReal.getHandle<IndexTy>()")
    multi["offsets"], _ = init_list(body, 0, "offsetsTensorReal.getHandle<IndexTy>()")
    multi["dim_offsets"], _ = init_list(body, 0, "dimOffsetsTensorReal.getHandle<int32_t>()")
    multi["placements"], _ = init_list(body, 0, "weightsPlacementReal.getHandle<int32_t>()")
    multi["total_dims"] = 10
    body, at = function_body(text, "static void testIntNBitSplitEmbeddingWeightedBags(")
    multi["indice_weights"], _ = init_list(body, 0, "indiceWeightsTensorReal.getHandle<IndexWeightTy>()")
    assert init_list(body, 0, "indicesTensorReal.getHandle<IndexTy>()")[0] == multi["indices"]
    out["multi_setup"] = multi

    for name, key in (("getIntNBitSplitEmbeddingBagsWeightsFloat()", "weights_float"),
                      ("getIntNBitSplitEmbeddingBagsWeightsFloat16()", "weights_float16")):
        body, at = function_body(text, "static Tensor " + name)
        out[key], _ = init_list(body, 0, "weights.getHandle<uint8_t>()")

    cases = []
    for m in re.finditer(r"TEST_P\(OperatorTest,\s*(IntNBitSplitEmbedding\w+)\)\s*\{", text):
        end = text.index("\n}\n", m.end())
        body = text[m.end():end]
        case = {"name": m.group(1), "source_line": line_of(m.start())}
        kind = "f16" if re.search(r"expected\(ElemKind::Float16Ty", body) else "f32"
        case["expected_dtype"] = kind
        dims = numbers(re.search(r"expected\(ElemKind::\w+,\s*\{([^}]*)\}", body).group(1))
        case["expected_dims"] = [int(x) for x in dims]
        case["expected"], _ = init_list(body, 0, "expected.getHandle<")
        if "weightsOffsets.getHandle<int32_t>()" in body:
            case["weights_offsets"], _ = init_list(body, 0, "weightsOffsets.getHandle<int32_t>()")
        call = body[body.index("testIntNBitSplitEmbedding"):]
        case["weighted"] = call.startswith("testIntNBitSplitEmbeddingWeightedBags")
        case["single"] = call.startswith("testIntNBitSplitEmbeddingBagsSingle")
        tys = re.findall(r"SplitEmbeddingSparseType::(EST_\w+)", call)
        pools = re.findall(r"SplitEmbeddingPoolingMode::(EP_\w+)", call)
        case["pooling"] = POOL[pools[0]] if pools else 0
        if case["single"]:
            case["weights_ty"] = SPARSE[tys[0]]
            case["output_dtype"] = SPARSE[tys[1]]
        else:
            case["table"] = "weights_float16" if "WeightsFloat16()" in call else "weights_float"
            case["weights_ty"] = 1 if case["table"] == "weights_float16" else 0
            case["output_dtype"] = SPARSE[tys[-1]]
        if case["weighted"]:
            tmpl = re.search(r"<([^>]*)>", call).group(1).replace("\n", " ")
            case["indice_weights_dtype"] = "f16" if tmpl.split(",")[-1].strip() == "float16_t" else "f32"
        case["tol"] = numbers(call[call.rindex(","):])[0]
        cases.append(case)
    out["cases"] = cases
    dest = os.path.join(os.path.dirname(os.path.abspath(__file__)), "split_embedding_vectors.json")
    with open(dest, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", dest, "with", len(cases), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
