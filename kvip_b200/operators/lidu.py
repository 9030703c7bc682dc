"""kvip.lidu: the serial-chain slot resolver with the reference's out-parameter ABI.

`lidu(*args)` takes the same 24 positional arguments, in the same order, as the reference op
nanovllm_dsa::lidu_fused_batch_get_prepare_mtp_out
(csrc/operators/lidu/torch_extension/csrc/lidu_fused_batch_get_prepare_mtp_ops.cpp:385-398; call site
tests/operators/lifetch/support/execution.py:1432-1457), checks them like CheckInputs/CheckOutputs
(:41-190) and enqueues the CUDA kernels on torch's current stream. The op is also registered as
torch.ops.nanovllm_dsa.lidu_fused_batch_get_prepare_mtp_out with the reference schema."""
import ctypes

import torch

from .. import _lib

SPARSE_COUNT = 2048
MTP_MISS_CAPACITY = 4 * SPARSE_COUNT
MAX_SOURCE_CAPACITY = (1 << 20) + 20 * 128
MAX_CACHE_TOKENS = (1 << 17) + 20 * 128
MISS_SLOT_BITMAP_WORDS = ((MAX_CACHE_TOKENS + 31) // 32 + 7) // 8 * 8  # 4176
_SCRATCH = {}

_SCHEMA = (
    "lidu_fused_batch_get_prepare_mtp_out(Tensor topk_indices, Tensor actual_seq_lengths_query, "
    "Tensor req_pool_entries, Tensor(a!) token_to_slot_pool, Tensor(b!) slot_to_token_pool, "
    "Tensor(c!) eviction_cursors, Tensor cache_tokens, Tensor candidate_lens, Tensor miss_slots, "
    "Tensor miss_slot_bitmap, Tensor resident_block_table, Tensor logical_seq_lengths, Tensor profile_enabled, "
    "Tensor(d!) destination_slots, Tensor(e!) miss_counts, Tensor(f!) indices, Tensor(g!) offsets, "
    "Tensor(h!) output_indices, Tensor(i!) resident_seq_lengths, Tensor(j!) profiling, int layer_id, "
    "int num_layers, int max_num_reqs, int qcap) -> (Tensor(d!), Tensor(e!), Tensor(f!), Tensor(g!), Tensor(h!), "
    "Tensor(i!))")


def _check(condition, message):
    if not condition:
        raise ValueError(f"lidu: {message}")


def _validate(topk, ends, pools, t2s, s2t, cursors, cache_tokens, candidate_lens, miss_slots, bitmap, block_table,
              logical, profile, dest, counts, indices, offsets, outputs, resident, profiling, layer_id, num_layers,
              max_num_reqs, qcap):
    _check(topk.dim() == 3 and topk.size(0) > 0 and topk.size(1) == 1 and topk.size(2) == SPARSE_COUNT,
           "topk_indices must be int32 [T,1,2048]")
    _check(ends.dim() == 1 and ends.size(0) > 0, "actual_seq_lengths_query must be int32 [B]")
    batch, packed = ends.size(0), topk.size(0)
    _check(batch <= packed <= 4 * batch, "requires 1--4 packed queries per request")
    _check(all(t.dim() == 1 and t.size(0) == batch for t in (pools, cache_tokens, candidate_lens, logical))
           and profile.dim() == 1 and profile.size(0) == 1,
           "request metadata must be int32 [B], with profile_enabled int32 [1]")
    _check(tuple(miss_slots.shape) == (batch, SPARSE_COUNT), "miss_slots must be int32 [B,2048]")
    _check(tuple(bitmap.shape) == (batch, MISS_SLOT_BITMAP_WORDS), "miss_slot_bitmap must be int32 [B,4176]")
    _check(t2s.dim() == 2 and t2s.size(0) > 0 and 0 < t2s.size(1) <= MAX_SOURCE_CAPACITY,
           "token_to_slot_pool must be [pool,source_capacity]")
    _check(s2t.dim() == 2 and s2t.size(0) == t2s.size(0) and s2t.size(1) >= SPARSE_COUNT,
           "slot_to_token_pool must be [pool,resident_capacity >= 2048]")
    _check(cursors.dim() == 1 and cursors.size(0) == t2s.size(0), "eviction_cursors must be int32 [pool]")
    _check(block_table.dim() == 2 and block_table.size(0) == batch and block_table.size(1) > 0,
           "resident_block_table must be int32 [B,resident_blocks]")
    _check(0 <= layer_id < num_layers and max_num_reqs >= batch and qcap > 0
           and max_num_reqs * num_layers * qcap <= 2**31 - 1 and block_table.size(1) * 128 <= 2**31 - 1,
           "AccessTable geometry is invalid")
    device = topk.device
    _check(device.type == "cuda", "inputs must be on a CUDA device")
    for t in (topk, ends, pools, t2s, s2t, cursors, cache_tokens, candidate_lens, miss_slots, bitmap, block_table,
              logical, profile, dest, counts, indices, offsets, outputs, resident):
        _check(t.dtype == torch.int32 and t.device == device and t.is_contiguous(),
               "tensors must be contiguous int32 on one device")
    _check(dest.shape == topk.shape, "destination_slots must be int32 [T,1,2048]")
    capacity = batch * MTP_MISS_CAPACITY
    _check(counts.dim() == 1 and counts.size(0) == batch + 1 and all(t.dim() == 1 and t.numel() == capacity
                                                                      for t in (indices, offsets, outputs))
           and resident.dim() == 1 and resident.size(0) == batch,
           "descriptors must be int32 [B*8192], with miss_counts int32 [B+1] and resident_seq_lengths int32 [B]")
    _check(tuple(profiling.shape) == (batch, 8, 32) and profiling.dtype == torch.int64 and profiling.device == device
           and profiling.is_contiguous(), "profiling must be contiguous int64 [B,8,32]")
    return batch, packed


def lidu(topk_indices, actual_seq_lengths_query, req_pool_entries, token_to_slot_pool, slot_to_token_pool,
         eviction_cursors, cache_tokens, candidate_lens, miss_slots, miss_slot_bitmap, resident_block_table,
         logical_seq_lengths, profile_enabled, destination_slots, miss_counts, indices, offsets, output_indices,
         resident_seq_lengths, profiling, layer_id, num_layers, max_num_reqs, qcap):
    """Call the LIDU kernels on torch's current CUDA stream; returns the six output tensors."""
    batch, packed = _validate(
        topk_indices, actual_seq_lengths_query, req_pool_entries, token_to_slot_pool, slot_to_token_pool,
        eviction_cursors, cache_tokens, candidate_lens, miss_slots, miss_slot_bitmap, resident_block_table,
        logical_seq_lengths, profile_enabled, destination_slots, miss_counts, indices, offsets, output_indices,
        resident_seq_lengths, profiling, layer_id, num_layers, max_num_reqs, qcap)
    lib = _lib.load_library()
    device = topk_indices.device
    key = (str(device), batch)
    if key not in _SCRATCH:  # allocated on first use per (device, batch): call once before graph capture
        _SCRATCH[key] = torch.zeros(lib.kvip_b200_lidu_scratch_words(batch), dtype=torch.int32, device=device)
    p = lambda t: t.data_ptr()  # noqa: E731
    args = _lib.LiduArgs(
        topk_indices=p(topk_indices), actual_seq_lengths_query=p(actual_seq_lengths_query),
        req_pool_entries=p(req_pool_entries), token_to_slot_pool=p(token_to_slot_pool),
        slot_to_token_pool=p(slot_to_token_pool), eviction_cursors=p(eviction_cursors), cache_tokens=p(cache_tokens),
        candidate_lens=p(candidate_lens), miss_slots=p(miss_slots), miss_slot_bitmap=p(miss_slot_bitmap),
        resident_block_table=p(resident_block_table), logical_seq_lengths=p(logical_seq_lengths),
        profile_enabled=p(profile_enabled), destination_slots=p(destination_slots), miss_counts=p(miss_counts),
        indices=p(indices), offsets=p(offsets), output_indices=p(output_indices),
        resident_seq_lengths=p(resident_seq_lengths), profiling=p(profiling), layer_id=layer_id,
        num_layers=num_layers, max_num_reqs=max_num_reqs, qcap=qcap, packed_queries=packed, batch=batch,
        pool_size=token_to_slot_pool.size(0), source_capacity=token_to_slot_pool.size(1),
        resident_capacity=slot_to_token_pool.size(1), resident_blocks=resident_block_table.size(1),
        bitmap_words=miss_slot_bitmap.size(1), scratch=p(_SCRATCH[key]))
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    _lib.check(lib.kvip_b200_lidu(ctypes.byref(args), stream), "lidu", lib)
    return destination_slots, miss_counts, indices, offsets, output_indices, resident_seq_lengths


def _register():
    try:
        library = torch.library.Library("nanovllm_dsa", "FRAGMENT")
        library.define(_SCHEMA)
        library.impl("lidu_fused_batch_get_prepare_mtp_out", lidu, "CUDA")
        return library
    except RuntimeError:  # already defined by another copy of this module
        return None


_TORCH_LIBRARY = _register()
