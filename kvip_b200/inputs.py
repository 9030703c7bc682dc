"""Stable query-slot input views for the LIFetch kernels.

Mirrors the reference's QueryInputs (python/kvip/adapters/vllm/inputs.py:31-152): every request owns a
fixed number of query slots (4 in the reference; 1..4 here), scheduler row packing is uploaded once per
step from double-buffered pinned staging, positions come from a device tensor, and `pack` gathers the
projected queries into the persistent buffers the captured graph reads. No host read is needed."""
import numpy as np

QUERIES_PER_REQUEST = 4
INDEX_WIDTH = 128


def committed_candidates(candidates, committed, resident):
    """Keep victim candidates inside the committed prefix (reference inputs.py:14-28)."""
    limit = min(committed, resident)
    if limit == resident:
        return candidates
    eligible = candidates[candidates < limit]
    missing = np.setdiff1d(np.arange(limit, dtype=np.int32), eligible, assume_unique=True)
    return np.concatenate((eligible, missing, candidates[candidates >= limit]))[: len(candidates)]


class QueryInputs:
    def __init__(self, torch, batch, device, *, pin_memory=True, history=0, index_heads=64,
                 queries=QUERIES_PER_REQUEST, query_dtype=None, weight_dtype=None):
        if index_heads not in (32, 64):
            raise ValueError("LIFetch supports 32 or 64 Indexer heads")
        if not 1 <= queries <= QUERIES_PER_REQUEST:
            raise ValueError("LIFetch rows hold one to four query slots per request")
        self.index_heads, self.queries = index_heads, queries
        self.torch, self.batch, self.device = torch, batch, torch.device(device)
        capacity = batch * queries
        on_gpu = self.device.type == "cuda"
        # Fields share one upload, including output padding validity.
        self.metadata = torch.zeros((5, capacity), dtype=torch.int64, device=device)
        self.host = [torch.zeros((5, capacity), dtype=torch.int64, pin_memory=pin_memory and on_gpu) for _ in range(2)]
        self.host_events = [None, None]
        self.turn = 0
        self.gather_indices, self.query_valid, self.unpack_indices, self.output_valid = self.metadata[:4].unbind(0)
        # int32 owners share the int64 upload: the last row is reinterpreted.
        self.row_owners = self.metadata[4].view(torch.int32)[:batch]
        query_dtype = query_dtype or torch.float8_e4m3fn
        self.query = torch.zeros((capacity, index_heads, INDEX_WIDTH), dtype=torch.uint8 if query_dtype == torch.float8_e4m3fn
                                 else query_dtype, device=device)
        if query_dtype == torch.float8_e4m3fn:
            self.query = self.query.view(torch.float8_e4m3fn)
        self.weights = torch.zeros((capacity, index_heads), dtype=weight_dtype or torch.bfloat16, device=device)
        self.scale = torch.ones((capacity, index_heads), dtype=torch.float32, device=device)
        self.position_scratch = torch.zeros(capacity, dtype=torch.int64, device=device)
        self.query_ends = torch.zeros(capacity, dtype=torch.int32, device=device)
        self.token_count = 0
        self.block_offsets = torch.arange(history // 128, dtype=torch.int32, device=device)
        self.block_table = torch.zeros((batch, history // 128), dtype=torch.int32, device=device)
        self.block_bases = torch.zeros((batch, 1), dtype=torch.int32, device=device)

    @property
    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (
            self.metadata, self.query, self.weights, self.scale, self.position_scratch, self.query_ends,
            self.block_offsets, self.block_table, self.block_bases))

    def prepare(self, query_counts, *, query_starts=None, query_owners=None):
        """Input preparation, outside capture; no device-dependent branching."""
        q = self.queries
        counts = tuple(query_counts)
        if len(counts) > self.batch or any(type(n) is not int or not 0 <= n <= q for n in counts):
            raise ValueError(f"LIFetch rows require zero to {q} queries per request")
        starts = None if query_starts is None else tuple(query_starts)
        if starts is not None and (len(starts) != len(counts) or any(type(n) is not int or n < 0 for n in starts)):
            raise ValueError("Decode query starts must match request rows and be nonnegative")
        owners = None if query_owners is None else tuple(query_owners)
        if owners is not None and (
                len(owners) != len(counts) or any(type(n) is not int or not 0 <= n < (1 << 31) for n in owners)):
            raise ValueError("Decode owners must match request rows and fit nonnegative int32")
        ring = self.turn % 2
        event = self.host_events[ring]
        if event is not None and not event.query():
            event.synchronize()
        values = self.host[ring].numpy()
        values.fill(0)
        if owners is not None:
            self.host[ring][4].view(self.torch.int32)[: len(owners)].numpy()[...] = owners
        begin = 0
        for row, count in enumerate(counts):
            start = row * q
            source = begin if starts is None else starts[row]
            values[0, start: start + count] = np.arange(source, source + count)
            values[1, start: start + count] = 1
            values[2, begin: begin + count] = np.arange(start, start + count)
            values[3, begin: begin + count] = 1
            begin += count
        self.token_count = begin
        self.metadata.copy_(self.host[ring], non_blocking=True)
        if self.block_offsets.numel():
            self.torch.mul(self.row_owners[:, None], self.block_offsets.numel(), out=self.block_bases)
            self.torch.add(self.block_bases, self.block_offsets, out=self.block_table)
        if self.device.type == "cuda":
            event = self.host_events[ring]
            if event is None:
                event = self.host_events[ring] = self.torch.cuda.Event()
            event.record(self.torch.cuda.current_stream(self.device))
        self.turn += 1

    def _pack_kernel(self, *, query=None, weights=None, scale=None, positions=None, tokens):
        """One gather launch on the bound device (kvip_b200_pack_inputs)."""
        import ctypes

        from . import _lib
        p = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
        args = _lib.PackArgs(
            query_src=p(query), weights_src=p(weights), scale_src=p(scale), positions_src=p(positions),
            gather_indices=p(self.gather_indices), query_valid=p(self.query_valid), query_dst=p(self.query),
            weights_dst=p(self.weights), scale_dst=p(self.scale), position_scratch=p(self.position_scratch),
            query_ends=p(self.query_ends), rows=self.batch * self.queries, tokens=tokens, heads=self.index_heads,
            query_row_bytes=self.index_heads * INDEX_WIDTH * self.query.element_size(),
            weights_row_bytes=self.index_heads * self.weights.element_size())
        stream = ctypes.c_void_p(self.torch.cuda.current_stream(self.device).cuda_stream)
        lib = _lib.load_library()
        _lib.check(lib.kvip_b200_pack_inputs(ctypes.byref(args), stream), "pack_inputs", lib)

    def bind_positions(self, positions):
        """Enqueue once per forward, after the runner corrects MTP positions."""
        if self.device.type == "cuda" and positions.is_cuda and positions.dtype == self.torch.int64 and positions.is_contiguous():
            self._pack_kernel(positions=positions, tokens=positions.numel())
            return self.query_ends.view(self.batch, self.queries)
        self.torch.index_select(positions, 0, self.gather_indices, out=self.position_scratch)
        self.position_scratch.add_(1).mul_(self.query_valid)
        self.query_ends.copy_(self.position_scratch)
        return self.query_ends.view(self.batch, self.queries)

    def pack(self, query, weights, scale):
        """Graph-safe gather into the fixed buffers."""
        torch = self.torch
        if weights.ndim != 2 or weights.shape[1] != self.index_heads:
            raise ValueError("LIFetch weights require [tokens,index_heads]")
        tokens = weights.shape[0]
        if tuple(query.shape) == (tokens * self.index_heads, INDEX_WIDTH):
            query = query.view(tokens, self.index_heads, INDEX_WIDTH)
        if tuple(query.shape) != (tokens, self.index_heads, INDEX_WIDTH) or query.dtype != self.query.dtype:
            raise ValueError("LIFetch requires Index queries of the bound dtype, head count and width 128")
        if weights.dtype != self.weights.dtype:
            raise ValueError("LIFetch weights must have the bound dtype")
        if scale is not None:
            if scale.dtype != self.scale.dtype:
                raise ValueError("LIFetch requires float32 query scales")
            if tuple(scale.shape) in ((tokens * self.index_heads,), (tokens * self.index_heads, 1)):
                scale = scale.view(tokens, self.index_heads)
            if tuple(scale.shape) != (tokens, self.index_heads):
                raise ValueError("LIFetch requires one scale per token/head")
        if (self.device.type == "cuda" and query.is_cuda and query.is_contiguous() and weights.is_contiguous()
                and (scale is None or scale.is_contiguous())):
            self._pack_kernel(query=query, weights=weights, scale=scale, tokens=tokens)
            return self.query, self.weights, self.scale
        if scale is not None:
            torch.index_select(scale, 0, self.gather_indices, out=self.scale)
        raw = torch.uint8 if self.query.element_size() == 1 else torch.int16
        torch.index_select(query.view(raw), 0, self.gather_indices, out=self.query.view(raw))
        torch.index_select(weights, 0, self.gather_indices, out=self.weights)
        return self.query, self.weights, self.scale
