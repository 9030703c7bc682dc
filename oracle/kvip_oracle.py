"""CPU oracle for the LI -> TopK -> resolver -> fetch -> Index-update path.

TEST INFRASTRUCTURE ONLY. Nothing under ``kvip_b200/`` imports this module; only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``
may use it, and only as the checker or as the timed CPU arm.

Every function restates, in NumPy, behaviour read from the reference project
(zxdgongjue-spec/KVIP); paths below are relative to that project. Parity status:

* LI score / TopK set: pinned by the reference's own fixture generators, imported from the
  reference's test support when the golden vectors under ``tests/golden`` were made
  (``tests/operators/lifetch/support/workloads.py:196-283, 975-1076``;
  ``correctness.py:22-36, 170-213``).
* SlotLRU, ABC maps, Index ingest, hot-slot bitmap scan: pinned against the reference's own
  Python / C++ code executed in this container (``tests/golden/make_golden.py``).
* TopK output ORDER, resolver victim choice, LIDU victim choice, Index exchange: the reference
  tests pin sets and invariants, not orders (``execution.py:1833-1836, 2102-2131, 2216-2224``);
  the deterministic restatement below is checked against those invariants.
"""
from __future__ import annotations

import numpy as np

TOPK = 2048
SLOTS = 8192
LRU_SLOTS = 2048
CHANGE_CAPACITY = 10240
BLOCK = 128
MISSING = -1

ERR_TOKEN_RANGE, ERR_NO_SLOT, ERR_HASH, ERR_SOURCE = 1, 4, 8, 64


# ---------------------------------------------------------------------------------------------
# number formats
# ---------------------------------------------------------------------------------------------
def e4m3_table() -> np.ndarray:
    """Value of every FP8 E4M3 (fn) code; same decode as workloads.py:1063-1068 / unpack()."""
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exponent = ((codes >> 3) & 0xF).astype(np.int32)
    mantissa = (codes & 7).astype(np.float64)
    values = np.where(exponent == 0, mantissa * 2.0**-9, (1 + mantissa / 8) * np.exp2(exponent - 7.0))
    values = sign * values
    values[(codes & 0x7F) == 0x7F] = np.nan
    return values.astype(np.float32)


_E4M3 = e4m3_table()


def decode_e4m3(codes: np.ndarray) -> np.ndarray:
    return _E4M3[np.asarray(codes, dtype=np.uint8)]


def encode_e4m3(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even, saturating fp32 -> E4M3 code (what cuda_fp8's SATFINITE does)."""
    x = np.asarray(values, dtype=np.float32)
    finite = np.sort(np.unique(_E4M3[np.isfinite(_E4M3) & (_E4M3 >= 0)]))  # 127 magnitudes incl. 0
    mag = np.minimum(np.abs(x).astype(np.float64), 448.0)
    hi = np.searchsorted(finite, mag, side="left").clip(0, len(finite) - 1)
    lo = (hi - 1).clip(0)
    d_lo, d_hi = mag - finite[lo], finite[hi] - mag
    code_of = {float(v): int(c) for c, v in enumerate(_E4M3[:127])}
    codes_sorted = np.array([code_of[float(v)] for v in finite], dtype=np.uint8)
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & ((codes_sorted[hi] & 1) == 0))
    code = np.where(pick_hi, codes_sorted[hi], codes_sorted[lo]).astype(np.uint8)
    return np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_rne(values: np.ndarray) -> np.ndarray:
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    rounded = bits + 0x7FFF + ((bits >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def bf16_away(values: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 with ties away from zero, widened back (indexer_score.h:119-139;
    golden: workloads.py:233-235)."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    return ((bits + np.uint32(0x8000)) & np.uint32(0xFFFF0000)).view(np.float32)


def sortable_key(values: np.ndarray) -> np.ndarray:
    """Order-preserving u32 image of fp32 (score_common.h:66-97 does the same on bf16)."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    key = np.where(bits & 0x80000000, ~bits, bits | np.uint32(0x80000000)).astype(np.uint32)
    key[(bits & 0x7FFFFFFF) > 0x7F800000] = 0xFFFFFFFF
    return key


# ---------------------------------------------------------------------------------------------
# LI score (golden: workloads.py:406-413, 1228-1237; kernel: indexer_score.h:59-140, 384-426)
# ---------------------------------------------------------------------------------------------
def head_weights(weights, query_scale, weight_is_bf16):
    w = bf16_to_f32(weights) if weight_is_bf16 else np.asarray(weights, dtype=np.float32)
    if query_scale is not None:
        w = (w * np.asarray(query_scale, dtype=np.float32)).astype(np.float32)
    return w


def li_scores(query, keys, weights, query_scale, key_scale, key_lengths, query_ends, block_table, *,
              key_is_bf16=False, weight_is_bf16=True, score_mode=0, score_stride=None, chunk=4096):
    """Scores [T, stride] (fp32). query [T,H,128] (u8 codes or bf16 bits), keys [rows,128] paged,
    block_table [B,pages], query_ends [B,Q]. Positions >= the valid length are left at 0."""
    query_ends = np.asarray(query_ends, dtype=np.int64)
    batch, queries = query_ends.shape
    pages = block_table.shape[1]
    stride = score_stride or pages * BLOCK
    q = bf16_to_f32(query) if key_is_bf16 else decode_e4m3(query)
    w = head_weights(weights, query_scale, weight_is_bf16).reshape(batch * queries, -1)
    out = np.zeros((batch * queries, stride), dtype=np.float32)
    for b in range(batch):
        ends = query_ends[b]
        if not (ends > 0).any():
            continue
        length = int(min(key_lengths[b], ends.max(), pages * BLOCK))
        if length <= 0:
            continue
        padded = -(-length // BLOCK) * BLOCK
        rows = (block_table[b, : padded // BLOCK].astype(np.int64)[:, None] * BLOCK + np.arange(BLOCK)).reshape(-1)
        k = bf16_to_f32(keys[rows]) if key_is_bf16 else decode_e4m3(keys[rows])
        ks = np.ones(padded, np.float32) if key_scale is None else np.asarray(key_scale, np.float32)[rows]
        for qi in range(queries):
            if ends[qi] <= 0:
                continue
            t = b * queries + qi
            for begin in range(0, padded, chunk):
                end = min(begin + chunk, padded)
                dots = np.einsum("hd,nd->hn", q[t], k[begin:end], optimize=True)
                out[t, begin:end] = (np.maximum(dots, 0) * w[t][:, None]).sum(0, dtype=np.float32) * ks[begin:end]
    if score_mode == 1:
        out = bf16_away(out)
    return out


# ---------------------------------------------------------------------------------------------
# TopK-2048 (topk_common.h:1136-1187; bounds indexer_vector.h:826-957)
# ---------------------------------------------------------------------------------------------
def topk_row(scores_row, valid_len, base_index=0):
    out = np.full(TOPK, -1, dtype=np.int32)
    length = int(min(valid_len, len(scores_row)))
    if length <= 0:
        return out
    if length <= TOPK:
        out[:length] = np.arange(length) + base_index
        return out
    keys = sortable_key(scores_row[:length])
    kth = np.partition(keys, length - TOPK)[length - TOPK]
    above = np.flatnonzero(keys > kth)
    equal = np.flatnonzero(keys == kth)
    out[: len(above)] = above + base_index
    out[len(above):] = equal[: TOPK - len(above)] + base_index
    return out


def topk(scores, key_lengths, query_ends, base_index=0):
    query_ends = np.asarray(query_ends).reshape(len(key_lengths), -1)
    queries = query_ends.shape[1]
    rows = scores.shape[0]
    out = np.empty((rows, TOPK), dtype=np.int32)
    for t in range(rows):
        b = t // queries
        out[t] = topk_row(scores[t], min(int(key_lengths[b]), int(query_ends[b, t % queries])), base_index)
    return out


def cold_predicate(scores, key_lengths, query_ends, resident):
    """Resident threshold + cold predicate (ProcessResidentTopK / SaveResident, indexer_vector.h:100-105, 162-177;
    ClassifyScore / BatchClassifyScore, indexer_score.h:784-792, 976-1017): TopK of the positions below
    `resident`, threshold = smallest selected key (0 while that prefix holds fewer than 2048 valid positions),
    one bit per cold position whose key beats it (bit i of word w = position resident + 32 w + i), their count."""
    query_ends = np.asarray(query_ends).reshape(len(key_lengths), -1)
    queries = query_ends.shape[1]
    rows, stride = scores.shape
    words = max(1, (stride - resident + 31) // 32)
    prefix = np.empty((rows, TOPK), dtype=np.int32)
    thresholds = np.zeros(rows, dtype=np.uint32)
    bitmap = np.zeros((rows, words), dtype=np.uint32)
    counts = np.zeros(rows, dtype=np.int32)
    for t in range(rows):
        b = t // queries
        length = max(0, min(int(key_lengths[b]), int(query_ends[b, t % queries]), stride))
        prefix[t] = topk_row(scores[t], min(length, resident), 0)
        if (prefix[t] >= 0).all():
            thresholds[t] = sortable_key(scores[t, prefix[t]]).min()
        cold = np.arange(resident, length)
        marked = cold[sortable_key(scores[t, cold]) > thresholds[t]] - resident
        np.bitwise_or.at(bitmap[t], marked // 32, np.uint32(1) << (marked % 32).astype(np.uint32))
        counts[t] = len(marked)
    return prefix, thresholds, bitmap, counts


def topk_merge(cand_scores, cand_index):
    """Global top-2048 of sharded candidates under (score desc, index asc), canonical order. With at most 2048
    valid candidates nothing is cut and the input order is kept: the shards are in position order and every
    shard's list is canonical for its slice (ascending positions for a slice of at most 2048 keys; the whole answer
    when a single shard contributes), which is what the TopK of the unsharded row gives."""
    rows = cand_scores.shape[0]
    out = np.full((rows, TOPK), -1, dtype=np.int32)
    for r in range(rows):
        live = np.flatnonzero(cand_index[r] >= 0)
        if len(live) <= TOPK:
            out[r, : len(live)] = cand_index[r, live]
            continue
        keys = sortable_key(cand_scores[r, live]).astype(np.int64)
        index = cand_index[r, live].astype(np.int64)
        order = np.lexsort((index, -keys))[:TOPK]
        if len(order) == 0:
            continue
        cut = keys[order[-1]]
        chosen_keys, chosen_index = keys[order], index[order]
        final = np.lexsort((chosen_index, (chosen_keys == cut).astype(np.int64)))
        out[r, : len(order)] = chosen_index[final]
    return out


def validate_topk(ids, scores):
    """The reference's TopK validity oracle (correctness.py:22-36), for full rows."""
    ids = np.asarray(ids).reshape(-1, TOPK)
    scores = np.asarray(scores).reshape(-1, scores.shape[-1])
    for i, selected in enumerate(ids):
        row = scores[i % len(scores)]
        if selected.min() < 0 or selected.max() >= len(row) or len(np.unique(selected)) != TOPK:
            raise AssertionError("TopK has invalid/duplicate positions")
        cutoff = np.partition(row, -TOPK)[-TOPK]
        tolerance = max(float(abs(cutoff)) * 2**-7, np.finfo(np.float32).tiny)
        if row[selected].min() < cutoff - tolerance:
            raise AssertionError("TopK selected a score below the cutoff")
        mandatory = np.flatnonzero(row > cutoff + tolerance)
        if not np.isin(mandatory, selected).all():
            raise AssertionError("TopK omitted a score above the cutoff")


# ---------------------------------------------------------------------------------------------
# hot-slot bitmap scan (lidu/op_kernel/hot_slot_selection.h:6-137)
# ---------------------------------------------------------------------------------------------
def free_slots_ring(protected_words, budget, begin, count):
    """First `count` slots whose bit is clear, scanning [begin, budget) then [0, begin)."""
    bits = np.unpackbits(np.asarray(protected_words, dtype="<u4").view(np.uint8), bitorder="little")[:budget]
    order = np.concatenate((np.arange(begin, budget), np.arange(0, begin)))
    free = order[bits[order] == 0]
    return free[:count].astype(np.int32), len(free)


# ---------------------------------------------------------------------------------------------
# classification + resolver (staged_topk_classify.h:9-46; resolver_staged_dma2.h:83-237;
# staged_urma_pack.h:6-71; streaming.cpp:66-90)
# ---------------------------------------------------------------------------------------------
def resolve_request(selected, hot_valid, reserved_hot, lru_slots, history, resident, *, tail_bounds=None,
                    output_stride=None, addresses=None, source_bytes=0, token_bytes=0, request=0):
    """One request. selected [Q,2048] positions (-1 = none). Returns a dict with locations [Q,2048],
    events (src, dst), per-query counts, change records, the final posts and the error word.

    ABC tail (common/lifetch/cache_metadata.h:22-26, 100-105; prefetch.h:26-44): with tail_bounds = (begin, end)
    and ring = output_stride - resident dedicated slots, a position begin <= p < end is never hot by position;
    while p - begin < ring its location is resident + p % ring (the reference's mapping code
    resident + 8192 + p % ring, resolved by ResolvePhysicalSlot), otherwise it is resolved like a cold position.
    Source check (streaming.cpp:399-400): with source_bytes, a new slot whose source address is negative, not
    16-byte aligned or beyond the pool fails the request with ERR_SOURCE before anything moves.
    Final posts (common/lifetch/final_post.h:5-12): per query {count, pending 0, error, deferred 0, first
    descriptor = request * 8192 + descriptors of earlier queries, nonconflicting = count}."""
    queries = selected.shape[0]
    ring = (output_stride or resident) - resident
    tail_begin, tail_end = (int(tail_bounds[0]), int(tail_bounds[1])) if tail_bounds is not None and ring else (0, 0)
    tail_begin, tail_end = max(tail_begin, 0), max(tail_end, 0)
    loc = np.full((queries, TOPK), MISSING, dtype=np.int64)
    protect = np.zeros(resident, dtype=bool)
    error = 0
    for q in range(queries):
        for k in range(TOPK):
            p = int(selected[q, k])
            if p < 0:
                continue
            if p >= history:
                error |= ERR_TOKEN_RANGE
                continue
            if tail_begin <= p < tail_end:
                if p - tail_begin < ring:
                    loc[q, k] = resident + p % ring
                continue
            if p < resident and hot_valid[p] != 0 and reserved_hot[p] < 0:
                loc[q, k] = p
                protect[p] = True
    changes = np.full(CHANGE_CAPACITY, -1, dtype=np.int32)
    change_slots = np.full(CHANGE_CAPACITY, -1, dtype=np.int32)
    change_slots[:LRU_SLOTS] = lru_slots
    ev_src, ev_dst, counts = [], [], [0] * 4
    assigned = {}
    for q in range(queries):
        if error:
            break
        new_tokens = []
        for k in range(TOPK):
            p = int(selected[q, k])
            if p < 0 or p >= history or loc[q, k] != MISSING:
                continue
            if p not in assigned and p not in new_tokens:
                new_tokens.append(p)
        added = len(new_tokens)
        victims = []
        if added:
            for slot in lru_slots:  # every candidate is range-checked, free ones are taken in list order
                slot = int(slot)
                if slot < 0 or slot >= resident:
                    if slot != -1:
                        error |= ERR_NO_SLOT
                    continue
                if not protect[slot] and len(victims) < added:
                    victims.append(slot)
            for slot in victims:
                protect[slot] = True
            if len(victims) < added:
                free = np.flatnonzero(~protect)
                need = added - len(victims)
                if len(free) < need:
                    error |= ERR_NO_SLOT
                else:
                    extra = [int(s) for s in free[:need]]
                    for slot in extra:
                        protect[slot] = True
                    victims += extra
        if error:
            break
        base = len(ev_src)
        if source_bytes and addresses is not None:
            for token in new_tokens:
                source = int(addresses[token])
                if source < 0 or source % 16 or source + token_bytes > source_bytes:
                    error |= ERR_SOURCE
        if error:
            break
        for i, (token, slot) in enumerate(zip(new_tokens, victims)):
            assigned[token] = slot
            ordinal = int(reserved_hot[slot])
            record = ordinal if ordinal >= 0 else LRU_SLOTS + base + i
            change_slots[record] = slot
            changes[record] = token
        ev_src += new_tokens
        ev_dst += victims
        counts[q] = added
        for k in range(TOPK):
            p = int(selected[q, k])
            if p >= 0 and loc[q, k] == MISSING:
                loc[q, k] = assigned[p]
    if error:
        counts = [0] * 4
    posts = np.zeros((4, 32), dtype=np.uint32)
    for q in range(4):
        posts[q, 0] = posts[q, 5] = counts[q]
        posts[q, 2] = error
        posts[q, 4] = request * SLOTS + sum(counts[:q])
    return dict(final_posts=posts, locations=loc.astype(np.int32), events_src=np.array(ev_src, dtype=np.int32),
                events_dst=np.array(ev_dst, dtype=np.int32), counts=counts, total=0 if error else len(ev_src),
                changes=changes, change_slots=change_slots,
                change_count=LRU_SLOTS + (0 if error else len(ev_src)), error=error)


# ---------------------------------------------------------------------------------------------
# Index exchange (shadow_exchange_parallel.h:27-198; driver streaming.cpp:205-274)
# ---------------------------------------------------------------------------------------------
def exchange_request(keys, scales, addresses, logical_ids, hot_valid, events_src, events_dst, counts,
                     history, resident, chunk=512):
    """Applies one request's events in place. Arrays are that owner's rows. Returns the error word."""
    row_pos, pos_row = {}, {}
    begin = 0
    for count in counts:
        for base in range(0, count, chunk):
            n = min(chunk, count - base)
            orig = [int(x) for x in events_src[begin + base : begin + base + n]]
            dst = [int(x) for x in events_dst[begin + base : begin + base + n]]
            if any(o < 0 or o >= history for o in orig) or any(d < 0 or d >= resident for d in dst):
                return 1
            src = [row_pos.get(o, o) for o in orig]
            if len(set(src)) != n or len(set(dst)) != n:
                return 1
            src_set, dst_set = set(src), set(dst)
            displaced = [d for d in dst if d not in src_set]
            freed = [s for s in src if s not in dst_set]
            move_src, move_dst = src + displaced, dst + freed
            snap = [(keys[s].copy(), scales[s].copy(), addresses[s].copy(), logical_ids[s].copy(), pos_row.get(s, s))
                    for s in move_src]
            for (k, sc, ad, lg, row), d in zip(snap, move_dst):
                keys[d], scales[d], addresses[d], logical_ids[d] = k, sc, ad, lg
                pos_row[d] = row
                row_pos[row] = d
            for d in freed:
                if d < resident:
                    hot_valid[d] = 0
        begin += count
    return 0


# ---------------------------------------------------------------------------------------------
# fetch and gather (patches/kvaf-ubmem-device-get.patch: fused_batch_get_device.h:21-61;
# streaming.cpp:300-328)
# ---------------------------------------------------------------------------------------------
def fetch_request(pool, hot_valid, source, sources, destinations, owner, output_stride, resident, token_bytes):
    """pool [rows, token_bytes] u8, source flat u8, sources byte offsets, destinations pool rows."""
    for address, dest in zip(sources, destinations):
        pool[int(dest)] = source[int(address) : int(address) + token_bytes]
        slot = int(dest) - owner * output_stride
        if 0 <= slot < resident:
            hot_valid[slot] = 1


def gather(pool, slots, owners, queries, output_stride):
    rows = slots.shape[0]
    out = np.zeros((rows, TOPK, pool.shape[1]), dtype=np.uint8)
    for t in range(rows):
        owner = int(owners[t // queries])
        live = (slots[t] >= 0) & (slots[t] < output_stride)
        out[t, live] = pool[owner * output_stride + slots[t, live]]
    return out


# ---------------------------------------------------------------------------------------------
# paged Index-cache update (python/kvip/adapters/vllm/index_import.py:38-52)
# ---------------------------------------------------------------------------------------------
def quantize_rows(rows_bf16_bits):
    x = bf16_to_f32(rows_bf16_bits)
    amax = np.abs(x).max(axis=-1)
    scale = np.where(amax > 0, (amax / np.float32(448.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    return encode_e4m3((x / scale[..., None]).astype(np.float32)), scale


def ingest_decode(keys, scales, source_keys, source_scales, slot_mapping, gather_indices, query_ends, row_owners,
                  queries, history, source_is_bf16=False):
    flat_keys, flat_scales = keys.reshape(-1, 128), scales.reshape(-1)
    for row in range(len(query_ends)):
        live = query_ends[row] > 0
        source = int(slot_mapping[gather_indices[row]]) if live else 0
        target = int(row_owners[row // queries]) * history + int(query_ends[row]) - 1 if live else row
        if source_is_bf16:
            code, scale = quantize_rows(source_keys[source][None])
            flat_keys[target], flat_scales[target] = code[0], scale[0]
        else:
            flat_keys[target], flat_scales[target] = source_keys[source], source_scales[source]


# ---------------------------------------------------------------------------------------------
# SlotLRU as an ordered array (python/kvip/cache/lru.py:33-118; _lru_kernel.py:32-199)
# ---------------------------------------------------------------------------------------------
class SlotLRUOracle:
    def __init__(self):
        self.order = np.empty(0, dtype=np.int32)
        self.active = 0
        self.version = 0

    def resize(self, capacity, committed):
        if not 0 <= committed <= capacity:
            raise ValueError("Committed slots must fit HBM capacity")
        if committed < self.active or self.active == 0 < committed:
            self.order = np.arange(committed, dtype=np.int32)
            self.active = committed
            self.version += 1
        elif committed > self.active:
            self.order = np.concatenate((self.order, np.arange(self.active, committed, dtype=np.int32)))
            self.active = committed
            self.version += 1

    def commit(self, destinations):
        feedback = np.asarray(destinations)
        feedback = np.unique(feedback[(feedback >= 0) & (feedback < self.active)]).astype(np.int32)
        if not feedback.size:
            return 0
        self.order = np.concatenate((self.order[~np.isin(self.order, feedback)], feedback))
        self.version += 1
        return int(feedback.size)

    @property
    def slots(self):
        out = np.full(LRU_SLOTS, -1, dtype=np.int32)
        count = min(LRU_SLOTS, self.active)
        out[:count] = self.order[:count]
        return out

    def reserved_hot(self, resident):
        inverse = np.full(resident, -1, dtype=np.int32)
        victims = self.slots
        live = victims >= 0
        inverse[victims[live]] = np.flatnonzero(live)
        return inverse


def update_abc(token_to_slot, slot_to_token, descriptors, requests, history, tail):
    """python/kvip/cache/abc.py:23-33 (CPU branch)."""
    for group in range(descriptors.shape[0]):
        for row in range(requests):
            layer, owner, begin, end = (int(x) for x in descriptors[group, row])
            tokens = np.arange(begin, end, dtype=np.int32)
            token_to_slot[layer, owner, begin:end] = history + tokens % tail
            reverse = slot_to_token[layer, owner, history : history + tail]
            reverse[:] = -1
            reverse[tokens % tail] = tokens


def publish_pages(rows, addresses, valid, token_to_slot, fused=(), widths=(), token_bytes=656, block=128):
    """python/kvip/cache/page_updates.py:49-62 (CPU branch), rows applied in order; the per-token table of a
    fused group is clipped at its history length as the device program does
    (python/kvip/cache/_page_updates_kernel.py:33-40)."""
    owners, groups, pages = addresses.shape
    for index, address, clear in np.asarray(rows, dtype=np.int64).reshape(-1, 3):
        owner, rem = divmod(int(index), groups * pages)
        group, page = divmod(rem, pages)
        addresses.reshape(-1)[index] = address
        valid.reshape(-1)[index] = 1
        if clear >= 0:
            token_to_slot.reshape(-1)[clear : clear + block] = -1
        if len(fused):
            history = fused[group].shape[1]
            first = page * block
            live = max(0, min(block, history - first))
            fused[group][owner, first : first + live] = address + np.arange(live, dtype=np.int64) * widths[group] * token_bytes


# ---------------------------------------------------------------------------------------------
# LIDU (csrc/operators/lidu/op_kernel/a5_lidu_fused_batch_get_prepare_mtp.cpp, lines cited in
# kvip_b200/csrc/lidu.cu); unique misses ordered by (query, TopK position) of first occurrence
# ---------------------------------------------------------------------------------------------
MAX_CACHE_TOKENS = (1 << 17) + 20 * 128


def lidu(topk_indices, ends, pool_entries, t2s, s2t, cursors, cache_tokens, candidate_lens, miss_slots,
         miss_bitmap, block_table, logical_lens, layer_id, num_layers, max_num_reqs, qcap):
    """Mutates t2s, s2t, cursors. Returns destination_slots, miss_counts, indices, offsets,
    output_indices, resident_seq_lengths."""
    packed = topk_indices.shape[0]
    batch = len(ends)
    topk_indices = topk_indices.reshape(packed, TOPK)
    dest = np.full((packed, TOPK), -1, dtype=np.int32)
    counts = np.zeros(batch + 1, dtype=np.int32)
    indices = np.zeros(batch * SLOTS, dtype=np.int32)
    offsets = np.zeros(batch * SLOTS, dtype=np.int32)
    outputs = np.zeros(batch * SLOTS, dtype=np.int32)
    resident_len = np.zeros(batch, dtype=np.int32)
    lows = np.concatenate(([0], ends[:-1]))
    layout_bad = any(h - l < 1 or h - l > 4 or h > packed or l < 0 for l, h in zip(lows, ends))
    written = 0
    for r in range(batch):
        if layout_bad:
            counts[r] = -1
            continue
        budget, cand, pool, logical = (int(cache_tokens[r]), int(candidate_lens[r]), int(pool_entries[r]),
                                      int(logical_lens[r]))
        rows = range(int(lows[r]), int(ends[r]))
        ok = (TOPK <= budget <= min(MAX_CACHE_TOKENS, s2t.shape[1]) and TOPK <= cand <= t2s.shape[1]
              and (cand + 127) // 128 <= qcap and (budget + 127) // 128 <= block_table.shape[1]
              and 0 <= pool < t2s.shape[0] and pool < max_num_reqs)
        if not ok:
            padding = budget == 0 and cand == 0 and logical == 1 and pool == max_num_reqs
            counts[r] = 0 if padding else -1
            if padding:
                resident_len[r] = logical
            continue
        status = 0
        if any(i != r and int(pool_entries[i]) == pool and int(cache_tokens[i]) >= TOPK for i in range(batch)):
            status = -102
        protect = np.unpackbits(np.asarray(miss_bitmap[r], dtype="<i4").view(np.uint8), bitorder="little").astype(bool)
        protect = protect.copy()
        unique, seen, per_query = [], set(), []
        for row in rows:
            tokens = topk_indices[row]
            slots = np.full(TOPK, -1, dtype=np.int64)
            for k, token in enumerate(tokens):
                token = int(token)
                if 0 <= token < cand:
                    mapped = int(t2s[pool, token])
                    if 0 <= mapped < budget and not protect[mapped]:
                        slots[k] = mapped
                else:
                    status = min(status, -103)
            miss = np.flatnonzero(slots < 0)
            hit = np.flatnonzero(slots >= 0)
            per_query.append((row, miss, hit, slots))
            for k in miss:
                token = int(tokens[k])
                if 0 <= token < cand and token not in seen:
                    seen.add(token)
                    unique.append(token)
        for _, _, hit, slots in per_query:
            protect[slots[hit]] = True
        victims, new_cursor = [], None
        if status == 0:
            for i in range(min(len(unique), LRU_SLOTS)):
                s = int(miss_slots[r, i])
                if s < 0 or s >= budget:
                    status = -109
                victims.append(s)
        if status == 0 and len(unique) > LRU_SLOTS:
            extra = len(unique) - LRU_SLOTS
            cursor = int(cursors[pool]) % budget
            order = np.concatenate((np.arange(cursor, budget), np.arange(0, cursor)))
            free = order[~protect[order]]
            if len(free) < extra:
                status = -107
            else:
                victims += [int(s) for s in free[:extra]]
                new_cursor = (victims[-1] + 1) % budget
        if status:
            counts[r] = status and -1
            continue
        for d in victims:
            v = int(s2t[pool, d])
            if 0 <= v < t2s.shape[1] and t2s[pool, v] == d:
                t2s[pool, v] = -1
        for token, d in zip(unique, victims):
            t2s[pool, token] = d
            s2t[pool, d] = token
        for row, miss, hit, slots in per_query:
            tokens = topk_indices[row]
            dest[row, : len(miss)] = t2s[pool, tokens[miss]]
            dest[row, len(miss):] = slots[hit]
        for token, d in zip(unique, victims):
            indices[written] = (pool * num_layers + layer_id) * qcap + (token >> 7)
            offsets[written] = (token & 127) * 656
            block = int(block_table[r, d >> 7])
            outputs[written] = -1 if block < 0 else block * 128 + (d & 127)
            written += 1
        counts[r] = len(unique)
        if budget >= TOPK and cand >= TOPK and logical >= cand:
            resident_len[r] = budget + logical - cand
        if new_cursor is not None:
            cursors[pool] = new_cursor
    counts[batch] = written
    return dest.reshape(packed, 1, TOPK), counts, indices, offsets, outputs, resident_len
