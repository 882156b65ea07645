"""Inputs of the reference's IntNBitSplitEmbedding(Weighted)Bags unit tests
(tests/golden/split_embedding_vectors.json) as numpy arrays, shared by the oracle test and the
GPU parity test."""
import json
import os

import numpy as np

G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "split_embedding_vectors.json")))
CASES = [c["name"] for c in G["cases"]]


def case_inputs(name, idx_dtype=np.int32):
    c = next(c for c in G["cases"] if c["name"] == name)
    s = G["single_setup"] if c["single"] else G["multi_setup"]
    T = len(s["dim_offsets"]) - 1
    table = np.array(s["weights"] if c["single"] else G[c["table"]], np.uint8)
    a = dict(
        dev_weights=table, uvm_weights=table.copy(),
        placements=np.array(s["placements"], np.int32),
        weights_offsets=np.array(s["weights_offsets"] if c["single"] else c["weights_offsets"], np.int32),
        weights_tys=np.full(T, c["weights_ty"], np.uint8),
        dim_offsets=np.array(s["dim_offsets"], np.int32),
        total_dims=s["total_dims"],
        indices=np.array(s["indices"], idx_dtype), offsets=np.array(s["offsets"], idx_dtype),
        pooling_mode=c["pooling"], out_fp16=c["output_dtype"] == 1, indice_weights=None)
    if c["weighted"]:
        a["indice_weights"] = np.array(s["indice_weights"],
                                       np.float16 if c["indice_weights_dtype"] == "f16" else np.float32)
    expected = np.array(c["expected"], np.float32).reshape(c["expected_dims"])
    return a, expected, c["tol"]
