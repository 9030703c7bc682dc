"""ABC tail maps: ring-buffer slots for the newest tokens of a request.

Same call as the reference's update_abc (python/kvip/cache/abc.py:5-33); on a CUDA device the maps
are written by one kernel launch on the current stream (the reference used a Triton kernel)."""
import ctypes

import torch

from .. import _lib


def update_abc(token_to_slot, slot_to_token, descriptors, requests, history, tail):
    """token_to_slot[layer, owner, tok] = history + tok % tail for tok in [begin, end) and the reverse
    ring slot_to_token[layer, owner, history:history+tail] (-1 where empty), for every descriptor row
    (layer, owner, begin, end) of descriptors[group, :requests]."""
    for name, tensor in (("token_to_slot", token_to_slot), ("slot_to_token", slot_to_token), ("descriptors", descriptors)):
        if not tensor.is_cuda or tensor.dtype != torch.int32 or not tensor.is_contiguous():
            raise ValueError(f"update_abc: {name} must be a contiguous int32 CUDA tensor")
    if token_to_slot.ndim != 3 or slot_to_token.ndim != 3 or descriptors.ndim != 3 or descriptors.shape[2] != 4:
        raise ValueError("update_abc: maps are [layers, pool, n] and descriptors [groups, rows, 4]")
    lib = _lib.load_library()
    stream = ctypes.c_void_p(torch.cuda.current_stream(token_to_slot.device).cuda_stream)
    code = lib.kvip_b200_update_abc(
        token_to_slot.data_ptr(), slot_to_token.data_ptr(), descriptors.data_ptr(), descriptors.shape[0],
        descriptors.shape[1], requests, token_to_slot.shape[1], token_to_slot.shape[2], slot_to_token.shape[2],
        history, tail, stream)
    _lib.check(code, "update_abc", lib)
