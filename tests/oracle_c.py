"""ctypes access to oracle/_build/libkvip_oracle.so (the C restatement). Test infrastructure."""
import ctypes
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parents[1] / "oracle"
LIB = ORACLE_DIR / "_build" / "libkvip_oracle.so"
_lib = None


def library():
    global _lib
    if _lib is None:
        if not LIB.exists():
            subprocess.run(["make", "-C", str(ORACLE_DIR), "all"], check=True, capture_output=True)
        _lib = ctypes.CDLL(str(LIB))
    return _lib


def _p(array):
    return None if array is None else array.ctypes.data_as(ctypes.c_void_p)


def li_scores(case, score_mode=0, stride=None):
    lib = library()
    batch, queries = case["query_ends"].shape
    pages = case["block_table"].shape[1]
    stride = stride or pages * 128
    scores = np.zeros((batch * queries, stride), dtype=np.float32)
    arrays = [np.ascontiguousarray(case[k]) if case[k] is not None else None
              for k in ("query", "keys", "weights", "query_scale", "key_scale", "key_lengths", "query_ends", "block_table")]
    lib.kvip_oracle_li_scores(*[_p(a) for a in arrays], _p(scores), batch, queries, case["heads"], pages, stride,
                              int(case["key_dtype"] == "bf16"), int(case["weight_dtype"] == "bf16"), score_mode)
    return scores


def topk(scores, key_lengths, query_ends, base_index=0):
    lib = library()
    rows = scores.shape[0]
    queries = rows // len(key_lengths)
    out = np.empty((rows, 2048), dtype=np.int32)
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    lib.kvip_oracle_topk(_p(scores), _p(np.ascontiguousarray(key_lengths, dtype=np.int32)),
                         _p(np.ascontiguousarray(query_ends, dtype=np.int32).reshape(-1)), _p(out), rows, queries,
                         scores.shape[1], base_index)
    return out
