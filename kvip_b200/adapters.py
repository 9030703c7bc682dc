"""The serving-side caller of the path, and the names of the reference's adapter that lie outside this build.

`IndexSelector` is the reference's `VllmIndexSelector` without its vLLM-Ascend bindings; `PagedIndexer` stands
in for the model's indexer object on the prefill rows of a mixed batch. `bind_selectors` needs vLLM-Ascend
policy/writer objects and `build_libraries` drives the Ascend toolchain (reference
python/kvip/adapters/vllm/binding.py:20-200, python/kvip/runtime/build.py:40-91); both names exist so that
`import kvip_b200` offers the reference's surface, and say what to use instead."""


def bind_selectors(*_args, **_kwargs):
    raise NotImplementedError(
        "bind_selectors binds vLLM-Ascend layer objects; on CUDA build the path from LIFetchWorkspace, "
        "IndexCacheStorage, CudaBinding, IndexUpdate and LIFetch, or use IndexSelector")


def build_libraries(force=False):
    """Build the CUDA library in-tree and return its path (the reference built three Ascend libraries)."""
    from .build import build_library

    return {"lifetch": build_library(force=force)}


# ---- serving-side caller of the path -----------------------------------------------------------------
class RequestPlan:
    """One request of a forward batch, as the selector sees it (reference selector.py:94-104 reads
    `.decode .begin .stop .owner .request .start .query_end .key_end` of the caller's plan objects).

    `begin:stop` is the request's token range in the flattened query batch, `owner` its stable Index owner,
    `start` the number of tokens already cached before this forward, `key_end` the context length after it."""

    def __init__(self, request, owner, begin, stop, *, decode, start=0, key_end=0):
        self.request, self.owner, self.begin, self.stop = request, int(owner), int(begin), int(stop)
        self.decode, self.start, self.key_end = bool(decode), int(start), int(key_end)
        self.query_end = self.stop - self.begin


class PagedIndexer:
    """The model-side indexer the selector falls back to for prefill rows: Index keys in the model's own paged
    cache (`k_cache.kv_cache = (keys [blocks, block, 128] FP8-as-u8, scales [blocks, block] f32)`), selected with
    the same LI-score and TopK kernels (reference: `indexer.select_topk_native`, selector.py:116, 146-151).

    The LI kernel takes at most four query slots per row, so a chunk of n tokens runs as ceil(n / 4) rows that
    all read the request's pages through copies of its block-table row; at most 1024 rows per launch."""

    ROWS_PER_LAUNCH = 1024

    def __init__(self, torch, keys, scales, *, index_heads=64):
        if keys.shape[-1] != 128 or keys.element_size() != 1 or scales.dtype != torch.float32:
            raise ValueError("PagedIndexer takes FP8 (one byte) keys [..., 128] and float32 scales")
        self.torch, self.index_heads = torch, index_heads
        self.k_cache = type("KCache", (), {"kv_cache": (keys, scales)})()
        self.keys = keys.view(torch.float8_e4m3fn).reshape(-1, 128)
        self.scales = scales.reshape(-1)
        self.scratch = {}

    def select_topk_native(self, query, weights, metadata, query_scale):
        """query [n, H, 128] FP8, weights [n, H], query_scale [n, H]; metadata.block_table [1, pages] and
        metadata.seq_lens = context length after the chunk. Token i of the chunk sees seq_lens - n + i + 1 keys.
        Returns int32 [n, 1, 2048] positions inside the request (-1 padded)."""
        from . import ops

        torch, heads = self.torch, self.index_heads
        n = weights.shape[0]
        device = weights.device
        key_end = int(metadata.seq_lens)
        table_row = metadata.block_table.reshape(1, -1).to(torch.int32)
        pages = table_row.shape[1]
        if key_end > pages * 128 or key_end < n:
            raise ValueError("prefill chunk does not fit the request's block table")
        out = torch.full((n, 1, 2048), -1, dtype=torch.int32, device=device)
        per_launch = self.ROWS_PER_LAUNCH * 4
        key = (str(device), pages)
        if key not in self.scratch:   # eager path (prefill is not graph-captured): sized once per table width
            self.scratch[key] = dict(
                scores=torch.zeros((per_launch, pages * 128), dtype=torch.float32, device=device),
                status=torch.zeros(1, dtype=torch.int32, device=device))
        scratch = self.scratch[key]
        query = query.view(torch.float8_e4m3fn).reshape(n, heads, 128)
        for lo in range(0, n, per_launch):
            count = min(per_launch, n - lo)
            rows = (count + 3) // 4
            padded = rows * 4
            q = torch.zeros((padded, heads, 128), dtype=torch.uint8, device=device)
            q[:count] = query[lo:lo + count].view(torch.uint8)
            w = torch.zeros((padded, heads), dtype=weights.dtype, device=device)
            w[:count] = weights[lo:lo + count]
            s = torch.ones((padded, heads), dtype=torch.float32, device=device)
            s[:count] = query_scale.reshape(n, heads)[lo:lo + count]
            ends = torch.zeros(padded, dtype=torch.int32, device=device)
            ends[:count] = key_end - n + lo + 1 + torch.arange(count, dtype=torch.int32, device=device)
            lengths = torch.full((rows,), key_end, dtype=torch.int32, device=device)
            scores = scratch["scores"][:padded]
            ops.li_score(q.view(torch.float8_e4m3fn), self.keys, w, s, self.scales, lengths, ends.view(rows, 4),
                         table_row.expand(rows, pages).contiguous(), scores, status=scratch["status"])
            picked = ops.topk(scores, lengths, ends.view(rows, 4))
            out[lo:lo + count, 0] = picked[:count]
        return out


class IndexSelector:
    """Indexer selector over the fused path (reference `VllmIndexSelector`, adapters/vllm/selector.py:46-161):
    `prepare(plans)` lays the decode rows out on the host once per forward, `__call__(query, weights, indexer,
    metadata, query_scale)` ingests the new Index rows, packs the decode queries into the bound buffers, runs
    `LIFetch` and returns the logical TopK per query token; prefill rows of a mixed batch are selected by the
    model-side indexer over its own paged cache. `slots(n)` are the resident slots for the attention kernel.

    The caller binds `inputs.bind_positions(positions)` before the call, as in the reference."""

    def __init__(self, torch, *, inputs, rotating, update, logical_ids, row_owners, storage=None, forward=None,
                 lru=None):
        from .operators.lifetch import LIFetch

        self.torch = torch
        self.inputs, self.rotating, self.update = inputs, rotating, update
        self.forward = forward if forward is not None else LIFetch(rotating, update, lru=lru)
        self.logical_ids, self.row_owners, self.storage = logical_ids, row_owners, storage
        self.positions = None
        if logical_ids.ndim != 2 or not logical_ids.is_contiguous() or logical_ids.dtype != torch.int64:
            raise ValueError("LIFetch logical IDs require contiguous int64 owner/history rows")
        if tuple(row_owners.shape) != (inputs.batch,) or row_owners.dtype != torch.int32:
            raise ValueError("LIFetch row owners must match the bound batch")
        for actual, expected in ((rotating.arguments[0], inputs.query), (rotating.arguments[2], inputs.weights),
                                 (rotating.arguments[3], inputs.scale)):
            if actual.data_ptr() != expected.data_ptr():
                raise ValueError("LIFetch kernel must bind the persistent packed query buffers")
        self.attention_indices = None
        self.plans, self.decodes = None, ()

    def prepare(self, plans, *, prepare_inputs=True):
        """Host-side request layout, once per forward; no device readback."""
        self.plans = tuple(plans)
        self.decodes = tuple(p for p in self.plans if p.decode)
        owners = [p.owner for p in self.decodes if p.stop > p.begin]
        if len(owners) != len(set(owners)):
            raise ValueError("active decode rows must have distinct stable owners")
        if self.storage is not None:
            self.storage.prepare(self.plans)
        if prepare_inputs:
            self.inputs.prepare([int(p.stop - p.begin) for p in self.decodes],
                                query_starts=[int(p.begin) for p in self.decodes],
                                query_owners=[int(p.owner) for p in self.decodes])
        if self.row_owners.data_ptr() != self.inputs.row_owners.data_ptr():
            self.row_owners.copy_(self.inputs.row_owners)

    def __call__(self, query, weights, indexer, metadata, query_scale):
        torch = self.torch
        mixed = bool(self.plans) and len(self.decodes) != len(self.plans)
        if self.storage is not None:
            if mixed:
                self.storage.ingest_prefill(indexer.k_cache.kv_cache, metadata, self.plans, self.positions)
            else:
                self.storage.ingest_decode(indexer.k_cache.kv_cache, metadata, self.inputs, self.row_owners)
        heads = self.inputs.index_heads
        query_rows = query.view(weights.shape[0], heads, 128)
        scale_rows = query_scale.view(weights.shape[0], heads)
        if self.plans and not self.decodes:
            return self._prefill_rows(query_rows, weights, indexer, metadata, scale_rows, None)
        self.inputs.pack(query_rows, weights, scale_rows)
        self.forward()
        token_count = (self.inputs.token_count if mixed or weights.shape[0] > self.inputs.batch * self.inputs.queries
                       else weights.shape[0])
        logical = self.update.logical_output[:token_count]
        self.attention_indices = self.update.slot_output[:token_count]
        if not mixed:
            return logical
        return self._prefill_rows(query_rows, weights, indexer, metadata, scale_rows, logical)

    def _prefill_rows(self, query_rows, weights, indexer, metadata, scale_rows, decode_logical):
        torch = self.torch
        result = torch.full((weights.shape[0], 1, 2048), -1, dtype=torch.int32, device=weights.device)
        offset = 0
        for row, plan in enumerate(self.plans):
            count = plan.stop - plan.begin
            if plan.decode:
                result[plan.begin:plan.stop].copy_(decode_logical[offset:offset + count])
                offset += count
                continue
            prefill = type("PrefillMetadata", (), {})()
            prefill.block_table = metadata.block_table[row:row + 1]
            prefill.num_actual_tokens = count
            prefill.seq_lens = plan.key_end
            result[plan.begin:plan.stop].copy_(indexer.select_topk_native(
                query_rows[plan.begin:plan.stop], weights[plan.begin:plan.stop], prefill,
                scale_rows[plan.begin:plan.stop]))
        return result

    def slots(self, token_count):
        if self.attention_indices is None:
            raise RuntimeError("LIFetch selection must execute before the attention kernel reads its slots")
        if token_count > self.attention_indices.shape[0]:
            raise ValueError("attention query count exceeds the fused selection")
        return self.attention_indices[:token_count]
