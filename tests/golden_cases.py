"""Loaders that turn the committed golden vectors (made by tests/golden/make_golden.py from the
reference's own code) into LI cases for the oracle and the CUDA path."""
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"


def li_fixture_case(name):
    """The reference fixture as a one-request, four-query LI case in PHYSICAL order.
    Returns (case, expected_bits_or_scores [4, history] in physical order, data)."""
    data = np.load(GOLDEN / name)
    query, keys = data["query"], data["keys"]
    queries, heads = query.shape[0], query.shape[1]
    storage = keys.shape[0]
    order = data["physical_to_logical"]
    visible = data["visible"].astype(np.int32)
    case = dict(
        query=query, keys=np.ascontiguousarray(keys), weights=data["weights"].astype(np.float32),
        query_scale=data["query_scale"].astype(np.float32), key_scale=data["key_scale"].astype(np.float32),
        key_lengths=np.array([int(visible.max())], np.int32), query_ends=visible.reshape(1, queries),
        block_table=np.arange(storage // 128, dtype=np.int32).reshape(1, -1), heads=heads, queries=queries, batch=1,
        history=storage, key_dtype="fp8", weight_dtype="fp32")
    logical = data["logical_scores"]
    expected = logical[:, order[: logical.shape[1]]] if logical.shape[1] <= len(order) else logical[:, order]
    return case, expected, data
