"""Stage-level operators: thin torch-tensor wrappers over the C ABI, each enqueued on the
current CUDA stream. Nothing here computes on the host: inputs are checked, pointers are
packed into the argument struct of include/kvip_b200.h and the kernel is launched."""
import ctypes

import torch

from . import _lib
from ._lib import TOPK, SLOTS, CHANGE_CAPACITY, BLOCK_TOKENS


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(tensor):
    return None if tensor is None else tensor.data_ptr()


def _require(tensor, name, dtype=None, device=None):
    if tensor is None:
        return
    if not tensor.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device (kvip_b200 has no CPU path)")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise ValueError(f"{name} must have dtype {dtype}, got {tensor.dtype}")
    if device is not None and tensor.device != device:
        raise ValueError(f"{name} must be on {device}")


def li_score(query, keys, weights, query_scale, key_scale, key_lengths, query_ends, block_table, scores=None, *,
             status=None, score_mode=_lib.SCORE_FP32, ctas=0, stages=0, simt=False, withhold_tile=0,
             wait_kilocycles=0):
    """scores[t, s] = kscale[s] * sum_h W[t,h] * relu(q[t,h,:] . k[s,:]) over the paged Index cache.

    query [B*Q, H, 128] float8_e4m3fn/uint8 or bfloat16; keys [rows, 128] same element type;
    weights [B*Q, H] bfloat16 or float32; query_ends [B, Q]. Returns (scores, status)."""
    device = query.device
    batch, queries = query_ends.shape
    heads = weights.shape[1]
    bf16 = query.dtype == torch.bfloat16
    for name, t, dt in (("query", query, None), ("keys", keys, None), ("weights", weights, (torch.bfloat16, torch.float32)),
                        ("query_scale", query_scale, torch.float32), ("key_scale", key_scale, torch.float32),
                        ("key_lengths", key_lengths, torch.int32), ("query_ends", query_ends, torch.int32),
                        ("block_table", block_table, torch.int32)):
        _require(t, name, dt, device)
    if (keys.dtype == torch.bfloat16) != bf16 or query.element_size() != keys.element_size():
        raise ValueError("query and keys must share one element type (FP8 e4m3 or bfloat16)")
    if tuple(query.shape) != (batch * queries, heads, 128) or keys.shape[-1] != 128:
        raise ValueError("query must be [B*Q, H, 128] and keys [..., 128]")
    pages = block_table.shape[1]
    stride = pages * BLOCK_TOKENS
    if scores is None:
        scores = torch.zeros((batch * queries, stride), dtype=torch.float32, device=device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=device)
    _require(scores, "scores", torch.float32, device)
    args = _lib.LiArgs(
        query=_ptr(query), keys=_ptr(keys), weights=_ptr(weights), query_scale=_ptr(query_scale),
        key_scale=_ptr(key_scale), key_lengths=_ptr(key_lengths), query_ends=_ptr(query_ends),
        block_table=_ptr(block_table), scores=_ptr(scores), status=_ptr(status), batch=batch, queries=queries,
        heads=heads, pagesPerRequest=pages, keyRows=keys.numel() // 128, scoreStride=scores.shape[1],
        keyDtype=_lib.KEY_BF16 if bf16 else _lib.KEY_FP8,
        weightDtype=_lib.WEIGHT_FP32 if weights.dtype == torch.float32 else _lib.WEIGHT_BF16,
        scoreMode=score_mode, ctas=ctas, stages=stages, withhold_tile=withhold_tile,
        wait_kilocycles=wait_kilocycles)
    lib = _lib.load_library()
    fn = lib.kvip_b200_li_score_simt if simt else lib.kvip_b200_li_score
    _lib.check(fn(ctypes.byref(args), _stream(device)), "li_score")
    return scores, status


def topk(scores, key_lengths, query_ends, out=None, *, out_scores=None, base_index=0, histogram=None,
         split_scratch=None):
    """Canonical TopK-2048 per score row. query_ends [B, Q] or flat [B*Q]. `histogram` is an all-zero int32
    [rows, 4096] scratch (returned all-zero): with it the first radix pass is spread over the whole GPU;
    `split_scratch` is an int32 [rows, 20544] scratch whose first 4160 words per row are zero (and are
    zero again afterwards): with it every pass is."""
    device = scores.device
    rows = scores.shape[0]
    queries = rows // key_lengths.numel()
    for name, t, dt in (("scores", scores, torch.float32), ("key_lengths", key_lengths, torch.int32),
                        ("query_ends", query_ends, torch.int32)):
        _require(t, name, dt, device)
    if out is None:
        out = torch.empty((rows, TOPK), dtype=torch.int32, device=device)
    args = _lib.TopkArgs(scores=_ptr(scores), key_lengths=_ptr(key_lengths), query_ends=_ptr(query_ends),
                         topk=_ptr(out), topk_scores=_ptr(out_scores), histogram=_ptr(histogram), rows=rows,
                         queries=queries, scoreStride=scores.shape[1], base_index=base_index,
                         split_scratch=_ptr(split_scratch))
    _lib.check(_lib.load_library().kvip_b200_topk(ctypes.byref(args), _stream(device)), "topk")
    return out


def cold_predicate(scores, key_lengths, query_ends, resident):
    """Resident threshold and cold predicate of every score row: the TopK of the resident prefix (positions
    below `resident`), the threshold key (smallest selected key; 0 while the prefix holds fewer than 2048 valid
    positions), one bit per cold position whose score beats it, and the number of such positions.
    Returns (prefix_topk [rows, 2048], threshold_keys [rows] int32 holding u32 bits, bitmap [rows, words] int32,
    counts [rows])."""
    device = scores.device
    rows, stride = scores.shape
    queries = rows // key_lengths.numel()
    if resident % 32 or resident > stride:
        raise ValueError("resident must be a multiple of 32 inside the score row")
    clipped = torch.clamp(query_ends.reshape(-1), max=resident).to(torch.int32)
    prefix_scores = torch.zeros((rows, TOPK), dtype=torch.float32, device=device)
    prefix_topk = topk(scores, key_lengths, clipped, out_scores=prefix_scores)
    words = max(1, (stride - resident + 31) // 32)
    thresholds = torch.zeros(rows, dtype=torch.int32, device=device)
    bitmap = torch.zeros((rows, words), dtype=torch.int32, device=device)
    counts = torch.zeros(rows, dtype=torch.int32, device=device)
    ends = query_ends.reshape(-1).contiguous()
    args = _lib.ColdArgs(scores=_ptr(scores), key_lengths=_ptr(key_lengths), query_ends=_ptr(ends),
                         prefix_topk=_ptr(prefix_topk), prefix_scores=_ptr(prefix_scores), threshold_keys=_ptr(thresholds),
                         bitmap=_ptr(bitmap), counts=_ptr(counts), rows=rows, queries=queries, scoreStride=stride,
                         resident=resident, bitmap_words=words)
    _lib.check(_lib.load_library().kvip_b200_cold_predicate(ctypes.byref(args), _stream(device)), "cold_predicate")
    return prefix_topk, thresholds, bitmap, counts


def topk_merge(cand_scores, cand_index, out=None):
    """Global top-2048 of [rows, shards*2048] (score, index) candidates."""
    device = cand_scores.device
    _require(cand_scores, "cand_scores", torch.float32, device)
    _require(cand_index, "cand_index", torch.int32, device)
    rows = cand_scores.shape[0]
    shards = cand_scores.shape[1] // TOPK
    if out is None:
        out = torch.empty((rows, TOPK), dtype=torch.int32, device=device)
    args = _lib.MergeArgs(cand_scores=_ptr(cand_scores), cand_index=_ptr(cand_index), topk=_ptr(out), rows=rows,
                          shards=shards)
    _lib.check(_lib.load_library().kvip_b200_topk_merge(ctypes.byref(args), _stream(device)), "topk_merge")
    return out


def topk_merge_gathered(gathered, out=None):
    """Global top-2048 straight from the all-gather buffer: `gathered` int32 [shards, 2, rows, 2048], block r = rank
    r's (score bits, indices). No repacking between the collective and the merge."""
    device = gathered.device
    _require(gathered, "gathered", torch.int32, device)
    shards, two, rows, width = gathered.shape
    if two != 2 or width != TOPK:
        raise ValueError("gathered candidates must be int32 [shards, 2, rows, 2048]")
    if out is None:
        out = torch.empty((rows, TOPK), dtype=torch.int32, device=device)
    args = _lib.MergeArgs(cand_scores=gathered.data_ptr(), cand_index=gathered[0, 1].data_ptr(), topk=_ptr(out),
                          rows=rows, shards=shards, shard_stride=2 * rows * TOPK, row_stride=TOPK)
    _lib.check(_lib.load_library().kvip_b200_topk_merge(ctypes.byref(args), _stream(device)), "topk_merge")
    return out


def peer_exchange(send, peer_blocks, rank):
    """Deliver this rank's candidate block (`send`, int32 [2, rows, 2048]) into every rank's exchange block over peer
    memory and raise this rank's flag there. `peer_blocks`: device addresses of all ranks' blocks as mapped in this
    process (kvip_b200.sharding.PeerBlocks)."""
    device = send.device
    _require(send, "send", torch.int32, device)
    args = _lib.PeerExchangeArgs(send=_ptr(send), block_bytes=send.numel() * 4, rank=rank, world=len(peer_blocks))
    for r, address in enumerate(peer_blocks):
        args.peer_block[r] = address
    _lib.check(_lib.load_library().kvip_b200_peer_exchange(ctypes.byref(args), _stream(device)), "peer_exchange")


def topk_merge_peer(own_block, rows, world, out, status, wait_kilocycles=0):
    """Global top-2048 of the candidates the ranks delivered into this rank's exchange block (device address
    `own_block`) with `peer_exchange`; waits, bounded, for every rank's flag of the current step."""
    device = out.device
    _require(out, "out", torch.int32, device)
    _require(status, "status", torch.int32, device)
    args = _lib.MergeArgs(topk=_ptr(out), rows=rows, shards=world, shard_stride=2 * rows * TOPK, row_stride=TOPK,
                          peer_block=own_block, status=_ptr(status), wait_ranks=world, wait_kilocycles=wait_kilocycles)
    _lib.check(_lib.load_library().kvip_b200_topk_merge(ctypes.byref(args), _stream(device)), "topk_merge")
    return out


class ResolveState:
    """Per-launch resolver scratch and outputs (shapes of operators/lifetch/workspace.py:9-32)."""

    def __init__(self, batch, queries, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.locations = torch.full((batch, queries, TOPK), -1, **i32)
        self.changes = torch.full((batch, CHANGE_CAPACITY), -1, **i32)
        self.change_slots = torch.full((batch, CHANGE_CAPACITY), -1, **i32)
        self.change_count = torch.zeros(batch, **i32)
        self.events_src = torch.zeros((batch, SLOTS), **i32)
        self.events_dst = torch.zeros((batch, SLOTS), **i32)
        self.query_counts = torch.zeros((batch, 8), **i32)
        self.fetch_sources = torch.zeros((batch, SLOTS), dtype=torch.int64, device=device)
        self.fetch_destinations = torch.zeros((batch, SLOTS), **i32)
        self.row_status = torch.zeros((batch, 32), **i32)
        self.logical_output = torch.full((batch * queries, TOPK), -1, **i32)
        self.slot_output = torch.full((batch * queries, TOPK), -1, **i32)
        self.final_posts = torch.zeros((batch * 4, 32), **i32)   # KvipFinalPost records, one per (request, query)


def resolve(selected, hot_valid, reserved_hot, lru_slots, logical_ids, addresses, state, *, history, resident,
            output_stride=None, row_owners=None, unpack_indices=None, output_valid=None, query_ends=None,
            tail_bounds=None, source_bytes=0, token_bytes=0):
    """Classify, resolve and publish one round. selected [B, Q, 2048] int32. `tail_bounds` [B, 2] int32 marks the
    ABC tail of every request (its rows live in the output_stride - resident slots behind the hot ones);
    `source_bytes` / `token_bytes` switch on the range check of the missing rows' source addresses."""
    device = selected.device
    batch, queries = selected.shape[0], selected.shape[1]
    for name, t, dt in (("selected", selected, torch.int32), ("hot_valid", hot_valid, torch.int32),
                        ("reserved_hot", reserved_hot, torch.int32), ("lru_slots", lru_slots, torch.int32),
                        ("logical_ids", logical_ids, torch.int64), ("addresses", addresses, torch.int64),
                        ("row_owners", row_owners, torch.int32), ("unpack_indices", unpack_indices, torch.int64),
                        ("output_valid", output_valid, torch.int64), ("query_ends", query_ends, torch.int32),
                        ("tail_bounds", tail_bounds, torch.int32)):
        _require(t, name, dt, device)
    s = state
    args = _lib.ResolveArgs(
        topk=_ptr(selected), row_owners=_ptr(row_owners), hot_valid=_ptr(hot_valid), reserved_hot=_ptr(reserved_hot),
        lru_slots=_ptr(lru_slots), tail_bounds=_ptr(tail_bounds), logical_ids=_ptr(logical_ids), addresses=_ptr(addresses),
        locations=_ptr(s.locations), changes=_ptr(s.changes), change_slots=_ptr(s.change_slots),
        change_count=_ptr(s.change_count), events_src=_ptr(s.events_src), events_dst=_ptr(s.events_dst),
        query_counts=_ptr(s.query_counts), fetch_sources=_ptr(s.fetch_sources),
        fetch_destinations=_ptr(s.fetch_destinations), logical_output=_ptr(s.logical_output),
        slot_output=_ptr(s.slot_output), unpack_indices=_ptr(unpack_indices), output_valid=_ptr(output_valid),
        query_ends=_ptr(query_ends), row_status=_ptr(s.row_status), batch=batch, queries=queries, history=history,
        resident=resident, address_stride=addresses.stride(0), outputStride=output_stride or resident,
        tokenBytes=token_bytes, source_bytes=source_bytes, final_posts=_ptr(getattr(s, "final_posts", None)))
    _lib.check(_lib.load_library().kvip_b200_resolve(ctypes.byref(args), _stream(device)), "resolve")
    return state


def exchange(keys, scales, addresses, logical_ids, hot_valid, state, shadow, status, *, history, resident,
             queries, row_owners=None):
    """Apply one round of (position, slot) events to the Index rows."""
    device = keys.device
    batch = state.events_src.shape[0]
    for name, t, dt in (("scales", scales, torch.float32), ("addresses", addresses, torch.int64),
                        ("logical_ids", logical_ids, torch.int64), ("hot_valid", hot_valid, torch.int32),
                        ("shadow", shadow, torch.int32), ("status", status, torch.int32)):
        _require(t, name, dt, device)
    _require(keys, "keys", None, device)
    args = _lib.ExchangeArgs(
        keys=_ptr(keys), scales=_ptr(scales), addresses=_ptr(addresses), logical_ids=_ptr(logical_ids),
        hot_valid=_ptr(hot_valid), events_src=_ptr(state.events_src), events_dst=_ptr(state.events_dst),
        query_counts=_ptr(state.query_counts), row_owners=_ptr(row_owners), row_status=_ptr(state.row_status),
        shadow=_ptr(shadow), status=_ptr(status), batch=batch, queries=queries, history=history, resident=resident,
        address_stride=addresses.stride(0), key_row_bytes=128 * keys.element_size())
    _lib.check(_lib.load_library().kvip_b200_exchange(ctypes.byref(args), _stream(device)), "exchange")


def make_shadow(batch, history, device):
    """Identity row<->position maps the exchange kernel works on (it restores them on exit)."""
    identity = torch.arange(history, dtype=torch.int32, device=device)
    return identity.repeat(batch, 2).contiguous()


def fetch(source, source_bytes, pool, hot_valid, state, *, resident, output_stride, token_bytes, row_owners=None,
          status=None):
    """Copy every descriptor's row from `source` (a device-visible tensor or a raw device pointer to
    the mapped host pool) into its resident slot and publish residency. `status` [B] int32 (the Index-update
    status) receives code 4 for a request with a descriptor outside the source."""
    device = pool.device
    batch = state.fetch_sources.shape[0]
    _require(pool, "pool", torch.uint8, device)
    _require(hot_valid, "hot_valid", torch.int32, device)
    base = source if isinstance(source, int) else source.data_ptr()
    args = _lib.FetchArgs(
        source_base=base, fetch_sources=_ptr(state.fetch_sources), fetch_destinations=_ptr(state.fetch_destinations),
        query_counts=_ptr(state.query_counts), row_owners=_ptr(row_owners), row_status=_ptr(state.row_status),
        pool=_ptr(pool), hot_valid=_ptr(hot_valid), source_bytes=source_bytes, batch=batch, resident=resident,
        outputStride=output_stride, tokenBytes=token_bytes, status=_ptr(status))
    _lib.check(_lib.load_library().kvip_b200_fetch(ctypes.byref(args), _stream(device)), "fetch")


def gather(pool, slots, out=None, *, queries, output_stride, token_bytes, row_owners=None):
    """out[t, k, :] = pool[owner*stride + slots[t, k], :]; zero rows where the slot is negative."""
    device = pool.device
    rows = slots.shape[0]
    _require(pool, "pool", torch.uint8, device)
    _require(slots, "slots", torch.int32, device)
    if out is None:
        out = torch.empty((rows, TOPK, token_bytes), dtype=torch.uint8, device=device)
    args = _lib.GatherArgs(pool=_ptr(pool), slots=_ptr(slots), row_owners=_ptr(row_owners), out=_ptr(out), rows=rows,
                           queries=queries, outputStride=output_stride, tokenBytes=token_bytes)
    _lib.check(_lib.load_library().kvip_b200_gather(ctypes.byref(args), _stream(device)), "gather")
    return out


def ingest(keys, scales, source_keys, source_scales, slot_mapping, gather_indices, query_ends, row_owners, *,
           queries, history):
    """Scatter the new tokens' Index rows into persistent storage (quantising bf16 sources)."""
    device = keys.device
    bf16 = source_keys.dtype == torch.bfloat16
    for name, t, dt in (("slot_mapping", slot_mapping, torch.int64), ("gather_indices", gather_indices, torch.int64),
                        ("query_ends", query_ends, torch.int32), ("row_owners", row_owners, torch.int32),
                        ("scales", scales, torch.float32), ("source_scales", source_scales, torch.float32)):
        _require(t, name, dt, device)
    args = _lib.IngestArgs(
        source_keys=_ptr(source_keys), source_scales=_ptr(source_scales), slot_mapping=_ptr(slot_mapping),
        gather_indices=_ptr(gather_indices), query_ends=_ptr(query_ends), row_owners=_ptr(row_owners),
        keys=_ptr(keys), scales=_ptr(scales), batch=row_owners.numel(), queries=queries, history=history,
        source_is_bf16=int(bf16))
    _lib.check(_lib.load_library().kvip_b200_ingest(ctypes.byref(args), _stream(device)), "ingest")


def ingest_spans(keys, scales, source_keys, source_scales, block_table, slot_mapping, positions, spans, *, history,
                 block, max_tokens, errors=None):
    """Import whole spans of Index rows in one launch (prefill): `spans` int32 [n, 8] rows of
    (owner, block-table row, kind, first, tokens, 0, 0, 0); kind 0 restores cached history through the block
    table, kind 1 writes this forward's tokens through slot_mapping / positions."""
    device = keys.device
    for name, t, dt in (("keys", keys, torch.uint8), ("scales", scales, torch.float32),
                        ("source_keys", source_keys, torch.uint8), ("source_scales", source_scales, torch.float32),
                        ("block_table", block_table, torch.int32), ("slot_mapping", slot_mapping, torch.int64),
                        ("positions", positions, torch.int64), ("spans", spans, torch.int32),
                        ("errors", errors, torch.int32)):
        _require(t, name, dt, device)
    table = block_table.reshape(-1, block_table.shape[-1])
    args = _lib.IngestSpanArgs(
        source_keys=_ptr(source_keys), source_scales=_ptr(source_scales), block_table=_ptr(table),
        slot_mapping=_ptr(slot_mapping), positions=_ptr(positions), spans=_ptr(spans), keys=_ptr(keys),
        scales=_ptr(scales), errors=_ptr(errors), source_rows=source_scales.numel(), count=spans.shape[0],
        max_tokens=max_tokens, owners=keys.shape[0], history=history, block=block, table_rows=table.shape[0],
        table_stride=table.shape[1], batch_tokens=min(slot_mapping.numel(), positions.numel()))
    _lib.check(_lib.load_library().kvip_b200_ingest_spans(ctypes.byref(args), _stream(device)), "ingest_spans")


def lru_commit(order, slots, bitmap, unique, reserved_hot, touched, active):
    device = order.device
    for name, t in (("order", order), ("slots", slots), ("bitmap", bitmap), ("unique", unique),
                    ("reserved_hot", reserved_hot), ("touched", touched), ("active", active)):
        _require(t, name, torch.int32, device)
    args = _lib.LruArgs(order=_ptr(order), slots=_ptr(slots), bitmap=_ptr(bitmap), unique=_ptr(unique),
                        reserved_hot=_ptr(reserved_hot), touched=_ptr(touched), active=_ptr(active),
                        rows=order.shape[0], capacity=order.shape[1], words=bitmap.shape[1],
                        touched_stride=touched.shape[1],
                        resident=0 if reserved_hot is None else reserved_hot.shape[1])
    _lib.check(_lib.load_library().kvip_b200_lru_commit(ctypes.byref(args), _stream(device)), "lru_commit")
