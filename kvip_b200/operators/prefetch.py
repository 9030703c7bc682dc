"""Speculative prefetch windows for `LIFetch` (reference: the prefetch role of the fused forward,
csrc/operators/lightning_indexer_with_fetch/op_kernel/prefetch.h:577-821; budgets prefetch_budget.h:7-17;
window geometry python/kvip/operators/lifetch/geometry.py:4-12, 49-55).

The score pass is issued as one launch per key window: the resident prefix first, then the cold positions in
`cold_windows` pieces. On a second stream, as soon as the resident prefix is scored, its TopK gives every score
row a threshold (its 2048th best resident score); after each cold window, positions that beat the threshold of
any query row of their request are listed (at most `limit` per request and round, `window_limit` more per
window) and their rows are copied from the host pool into a staging area in HBM, while the score kernel is
already working on the next window. Every cold position of the final TopK beats the threshold, so the list is
a superset of the step's misses as long as the limit lasts.

Unlike the reference, staged rows do not go into victim slots: the resolver, the Index exchange and the slot
maps run exactly as without speculation (same outputs, same pool bytes), and the final fetch reads a missing
row from the staging area when its source address is listed there. There is therefore no split of the final
descriptors into a conflicting and a non-conflicting part."""
import ctypes

from .. import _lib

TOPK = 2048
BLOCK = 128


class PrefetchWindows:
    def __init__(self, forward, *, limit=512, window_limit=480, cold_windows=3, li_ctas=0, last_window=False):
        rotating, torch = forward.rotating, forward.torch
        shape = rotating.runtime_shape
        if not 1 <= limit <= 512 or not 1 <= window_limit <= limit:
            raise ValueError("prefetch limit: 1..512 rows per request and round, window limit no larger")
        if shape.liVariant:
            raise ValueError("prefetch windows need the tensor-core score kernel")
        batch, queries, history, resident = shape.batch, shape.queries, shape.history, shape.resident
        cold = history - resident
        if cold < BLOCK:
            raise ValueError("prefetch windows need cold positions: history must exceed resident")
        cold_windows = max(1, min(cold_windows, 7, cold // BLOCK))
        per = -(-cold // (cold_windows * BLOCK)) * BLOCK
        first = [0, resident]
        while first[-1] < history:
            first.append(min(history, first[-1] + per))
        self.first, self.windows = first, len(first) - 1
        self.torch, self.library = torch, rotating.library   # no reference back to `forward`: it owns this object
        self.limit, self.window_limit = limit, window_limit
        # rows listed after the last window cannot be copied behind the score pass any more: by default they are
        # left to the final fetch, which reads exactly the missing ones
        self.staged_windows = self.windows if last_window or self.windows == 2 else self.windows - 1
        device, rows = rotating.device, batch * queries
        i32 = dict(dtype=torch.int32, device=device)
        self.window_lengths = torch.zeros((self.windows, batch), **i32)
        self.window_ends = torch.zeros((self.windows, rows), **i32)
        self.staged_count, self.staged_rows, self.staged_hits = (torch.zeros(batch, **i32) for _ in range(3))
        self.staged_sources = torch.full((batch, limit), -1, dtype=torch.int64, device=device)
        self.staging = torch.zeros((batch, limit, shape.tokenBytes), dtype=torch.uint8, device=device)
        self.prefix_topk = torch.full((rows, TOPK), -1, **i32)
        self.prefix_scores = torch.zeros((rows, TOPK), dtype=torch.float32, device=device)
        self.thresholds = torch.zeros(rows, **i32)   # u32 keys
        self.side = torch.cuda.Stream(device)
        self.scored = [torch.cuda.Event() for _ in range(self.windows)]
        self.staged = torch.cuda.Event()
        arguments = rotating.arguments
        pointer = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        scores, block_table = arguments[12], arguments[7]
        self.bounds = _lib.WindowArgs(
            key_lengths=pointer(arguments[6]), query_ends=pointer(rotating.query_ends),
            window_lengths=pointer(self.window_lengths), window_ends=pointer(self.window_ends),
            staged_count=pointer(self.staged_count), staged_rows=pointer(self.staged_rows),
            staged_hits=pointer(self.staged_hits), batch=batch, queries=queries, windows=self.windows,
            first=(ctypes.c_uint32 * 9)(*(first + [0] * (9 - len(first)))))
        self.score_args = [_lib.LiArgs(
            query=pointer(arguments[0]), keys=pointer(arguments[1]), weights=pointer(arguments[2]),
            query_scale=pointer(arguments[3]), key_scale=pointer(arguments[4]),
            key_lengths=self.window_lengths.data_ptr() + 4 * w * batch, query_ends=self.window_ends.data_ptr() + 4 * w * rows,
            block_table=block_table.data_ptr() + 4 * (first[w] // BLOCK), scores=scores.data_ptr() + 4 * first[w],
            status=forward.li_status.data_ptr(), batch=batch, queries=queries, heads=shape.indexHeads,
            pagesPerRequest=shape.pagesPerRequest, keyRows=shape.keyRows, scoreStride=shape.scoreStride,
            keyDtype=shape.keyDtype, weightDtype=shape.weightDtype, scoreMode=shape.scoreMode,
            ctas=li_ctas or shape.smCount, stages=0, withhold_tile=0) for w in range(self.windows)]
        self.prefix_args = _lib.TopkArgs(
            scores=pointer(scores), key_lengths=pointer(self.window_lengths), query_ends=pointer(self.window_ends),
            topk=pointer(self.prefix_topk), topk_scores=pointer(self.prefix_scores), histogram=None, rows=rows,
            queries=queries, scoreStride=shape.scoreStride, base_index=0, split_scratch=None)
        self.threshold_args = _lib.ThresholdArgs(prefix_topk=pointer(self.prefix_topk),
                                                 prefix_scores=pointer(self.prefix_scores),
                                                 thresholds=pointer(self.thresholds), rows=rows)
        addresses = rotating.token_addresses
        self.window_args = [_lib.SpeculateArgs(
            scores=pointer(scores), thresholds=pointer(self.thresholds), key_lengths=pointer(arguments[6]),
            query_ends=pointer(rotating.query_ends), row_owners=pointer(rotating.row_owners), addresses=pointer(addresses),
            source_base=rotating.source_base, staged_sources=pointer(self.staged_sources),
            staged_count=pointer(self.staged_count), staged_rows=pointer(self.staged_rows), staging=pointer(self.staging),
            source_bytes=rotating.source_bytes, batch=batch, queries=queries, scoreStride=shape.scoreStride,
            address_stride=addresses.stride(0), first=first[w], last=first[w + 1], capacity=limit,
            limit=min(limit, window_limit * w), tokenBytes=shape.tokenBytes) for w in range(1, self.windows)]
        # the final fetch learns about the staging area through the workspace record (host memory)
        record = forward.workspace.numpy()
        for name, value in (("staged_sources", self.staged_sources.data_ptr()), ("staged_rows", self.staged_rows.data_ptr()),
                            ("staging", self.staging.data_ptr()), ("staged_hits", self.staged_hits.data_ptr())):
            offset = getattr(_lib.Workspace, name).offset
            record[offset:offset + 8].view("<u8")[0] = value
        offset = _lib.Workspace.staged_capacity.offset
        record[offset:offset + 4].view("<u4")[0] = limit

    def _check(self, code, what):
        _lib.check(code, what, self.library)

    def enqueue(self, main):
        """Windowed score launches on `main`; thresholds, candidate lists and row copies on the side stream.
        `self.staged` is recorded when the last window's rows are in the staging area."""
        lib, ref = self.library, ctypes.byref
        stream = ctypes.c_void_p(main.cuda_stream)
        side = ctypes.c_void_p(self.side.cuda_stream)
        self._check(lib.kvip_b200_window_bounds(ref(self.bounds), stream), "window_bounds")
        for w in range(self.windows):
            self._check(lib.kvip_b200_li_score(ref(self.score_args[w]), stream), "li_score window")
            self.scored[w].record(main)
        self.side.wait_event(self.scored[0])
        self._check(lib.kvip_b200_topk(ref(self.prefix_args), side), "prefix topk")
        self._check(lib.kvip_b200_resident_threshold(ref(self.threshold_args), side), "resident_threshold")
        for w in range(1, self.staged_windows):
            self.side.wait_event(self.scored[w])
            self._check(lib.kvip_b200_speculate_window(ref(self.window_args[w - 1]), side), "speculate_window")
        self.staged.record(self.side)

    @property
    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (
            self.window_lengths, self.window_ends, self.staged_count, self.staged_rows, self.staged_hits,
            self.staged_sources, self.staging, self.prefix_topk, self.prefix_scores, self.thresholds))
