"""Query-slot inputs of the fused LIFetch call.

The role of the reference's QueryInputs (python/kvip/adapters/vllm/inputs.py:31-152) with the same attribute
names, because the operator objects and the selector read them: every request owns a fixed number of query
slots (4 in the reference, 1..4 here); once per step the scheduler's row packing is laid out on the host
(`slot_layout`, plain NumPy), uploaded with ONE copy from double-buffered pinned staging, and two gather
launches (`bind_positions`, `pack`: kvip_b200_pack_inputs) fill the persistent device buffers that the
captured graph reads. Nothing here reads device memory back, and there is no CPU path: the buffers live on
a CUDA device and the gathers are kernels."""
import ctypes

import numpy as np

from . import _lib

QUERIES_PER_REQUEST = 4
INDEX_WIDTH = 128
# rows of the metadata block, in upload order
GATHER, QUERY_VALID, UNPACK, OUTPUT_VALID, OWNERS = range(5)


def committed_candidates(candidates, committed, resident):
    """Victim candidates restricted to the committed prefix of the resident pool (reference inputs.py:14-28):
    candidates below `min(committed, resident)` keep their order and come first, then the committed slots that
    are no candidates (ascending), then the rest; the list keeps its length."""
    limit = min(int(committed), int(resident))
    candidates = np.asarray(candidates)
    if limit >= resident:
        return candidates
    inside = candidates < limit
    listed = np.zeros(limit, dtype=bool)
    listed[candidates[inside]] = True
    fill = np.flatnonzero(~listed).astype(candidates.dtype)
    return np.concatenate((candidates[inside], fill, candidates[~inside]))[: candidates.size]


def slot_layout(query_counts, *, batch, queries=QUERIES_PER_REQUEST, query_starts=None, query_owners=None):
    """Host layout of one step: int64 [5, batch * queries].

    Row GATHER: token index each query slot reads (request r's tokens are `query_starts[r] + 0..count-1`, or
    the running token offset when no starts are given); QUERY_VALID: 1 for a live slot; UNPACK: for packed
    output row t (tokens in request order) the slot it comes from; OUTPUT_VALID: 1 for the first
    `sum(counts)` output rows; OWNERS: the requests' stable owners as int32 values packed two per word.
    Returns (layout, token_count). Raises ValueError for what the reference rejects (inputs.py:75-92)."""
    counts = tuple(query_counts)
    if len(counts) > batch or any(type(n) is not int or not 0 <= n <= queries for n in counts):
        raise ValueError(f"LIFetch rows require zero to {queries} queries per request")
    rows = len(counts)
    if query_starts is not None:
        query_starts = tuple(query_starts)
        if len(query_starts) != rows or any(type(n) is not int or n < 0 for n in query_starts):
            raise ValueError("Decode query starts must match request rows and be nonnegative")
    if query_owners is not None:
        query_owners = tuple(query_owners)
        if len(query_owners) != rows or any(type(n) is not int or not 0 <= n < (1 << 31) for n in query_owners):
            raise ValueError("Decode owners must match request rows and fit nonnegative int32")
    layout = np.zeros((5, batch * queries), dtype=np.int64)
    count = np.asarray(counts, dtype=np.int64).reshape(-1)
    offsets = np.cumsum(count) - count                       # first packed token of every request
    total = int(count.sum())
    first = offsets if query_starts is None else np.asarray(query_starts, dtype=np.int64)
    request = np.repeat(np.arange(rows, dtype=np.int64), count)   # request of every packed token
    within = np.arange(total, dtype=np.int64) - offsets[request]   # its query slot inside the request
    slot = request * queries + within
    layout[GATHER, slot] = first[request] + within
    layout[QUERY_VALID, slot] = 1
    layout[UNPACK, :total] = slot
    layout[OUTPUT_VALID, :total] = 1
    if query_owners is not None:
        layout[OWNERS].view(np.int32)[:rows] = query_owners
    return layout, total


class QueryInputs:
    def __init__(self, torch, batch, device, *, pin_memory=True, history=0, index_heads=64,
                 queries=QUERIES_PER_REQUEST, query_dtype=None, weight_dtype=None):
        if index_heads not in (32, 64):
            raise ValueError("LIFetch supports 32 or 64 Indexer heads")
        if not 1 <= queries <= QUERIES_PER_REQUEST:
            raise ValueError("LIFetch rows hold one to four query slots per request")
        self.torch, self.batch, self.device = torch, batch, torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("QueryInputs buffers live on a CUDA device (kvip_b200 has no CPU path)")
        self.index_heads, self.queries = index_heads, queries
        slots = batch * queries
        self.metadata = torch.zeros((5, slots), dtype=torch.int64, device=device)
        self.gather_indices, self.query_valid, self.unpack_indices, self.output_valid = (
            self.metadata[row] for row in (GATHER, QUERY_VALID, UNPACK, OUTPUT_VALID))
        self.row_owners = self.metadata[OWNERS].view(torch.int32)[:batch]   # int32 owners inside the int64 block
        # two pinned staging blocks: the upload of step i may still be in flight while step i + 1 is laid out
        self.host = [torch.zeros((5, slots), dtype=torch.int64, pin_memory=pin_memory) for _ in range(2)]
        self.host_events = [None, None]
        self.turn = 0
        fp8 = query_dtype in (None, torch.float8_e4m3fn)
        self.query = torch.zeros((slots, index_heads, INDEX_WIDTH), dtype=torch.uint8 if fp8 else query_dtype, device=device)
        if fp8:
            self.query = self.query.view(torch.float8_e4m3fn)
        self.weights = torch.zeros((slots, index_heads), dtype=weight_dtype or torch.bfloat16, device=device)
        self.scale = torch.ones((slots, index_heads), dtype=torch.float32, device=device)
        self.position_scratch = torch.zeros(slots, dtype=torch.int64, device=device)
        self.query_ends = torch.zeros(slots, dtype=torch.int32, device=device)
        self.token_count = 0
        pages = history // 128
        self.block_offsets = torch.arange(pages, dtype=torch.int32, device=device)
        self.block_table = torch.zeros((batch, pages), dtype=torch.int32, device=device)
        self.block_bases = torch.zeros((batch, 1), dtype=torch.int32, device=device)

    @property
    def nbytes(self):
        tensors = (self.metadata, self.query, self.weights, self.scale, self.position_scratch, self.query_ends,
                   self.block_offsets, self.block_table, self.block_bases)
        return sum(t.numel() * t.element_size() for t in tensors)

    def prepare(self, query_counts, *, query_starts=None, query_owners=None):
        """Lay the step out on the host and enqueue its upload; outside capture, no device read."""
        layout, self.token_count = slot_layout(query_counts, batch=self.batch, queries=self.queries,
                                               query_starts=query_starts, query_owners=query_owners)
        ring = self.turn % 2
        self.turn += 1
        pending = self.host_events[ring]
        if pending is not None:
            pending.synchronize()          # the copy that last used this staging block (two steps ago) has finished
        self.host[ring].numpy()[...] = layout
        self.metadata.copy_(self.host[ring], non_blocking=True)
        if self.block_offsets.numel():     # per-owner contiguous Index storage: page p of a request = owner * pages + p
            self.torch.mul(self.row_owners[:, None], self.block_offsets.numel(), out=self.block_bases)
            self.torch.add(self.block_bases, self.block_offsets, out=self.block_table)
        if pending is None:
            pending = self.host_events[ring] = self.torch.cuda.Event()
        pending.record(self.torch.cuda.current_stream(self.device))

    def _gather(self, *, query=None, weights=None, scale=None, positions=None, tokens):
        """One gather launch on the bound device (kvip_b200_pack_inputs)."""
        def pointer(tensor):
            return 0 if tensor is None else tensor.data_ptr()

        args = _lib.PackArgs(
            query_src=pointer(query), weights_src=pointer(weights), scale_src=pointer(scale),
            positions_src=pointer(positions), gather_indices=pointer(self.gather_indices),
            query_valid=pointer(self.query_valid), query_dst=pointer(self.query), weights_dst=pointer(self.weights),
            scale_dst=pointer(self.scale), position_scratch=pointer(self.position_scratch),
            query_ends=pointer(self.query_ends), rows=self.batch * self.queries, tokens=tokens, heads=self.index_heads,
            query_row_bytes=self.index_heads * INDEX_WIDTH * self.query.element_size(),
            weights_row_bytes=self.index_heads * self.weights.element_size())
        stream = ctypes.c_void_p(self.torch.cuda.current_stream(self.device).cuda_stream)
        library = _lib.load_library()
        _lib.check(library.kvip_b200_pack_inputs(ctypes.byref(args), stream), "pack_inputs", library)

    def _on_device(self, tensor, what):
        if tensor.device != self.device or not tensor.is_contiguous():
            raise ValueError(f"LIFetch {what} must be contiguous on {self.device}")

    def bind_positions(self, positions):
        """query_ends[slot] = (positions[token of the slot] + 1) * valid: one launch, once per forward, after the
        runner has corrected the MTP positions."""
        if positions.dtype != self.torch.int64 or positions.ndim != 1:
            raise ValueError("LIFetch positions must be a flat int64 tensor")
        self._on_device(positions, "positions")
        self._gather(positions=positions, tokens=positions.numel())
        return self.query_ends.view(self.batch, self.queries)

    def pack(self, query, weights, scale):
        """Gather the projected queries, head weights and query scales of the step into the bound buffers: one
        launch, graph-capturable."""
        heads = self.index_heads
        if weights.ndim != 2 or weights.shape[1] != heads:
            raise ValueError("LIFetch weights require [tokens,index_heads]")
        tokens = weights.shape[0]
        if tuple(query.shape) == (tokens * heads, INDEX_WIDTH):
            query = query.view(tokens, heads, INDEX_WIDTH)
        if tuple(query.shape) != (tokens, heads, INDEX_WIDTH) or query.dtype != self.query.dtype:
            raise ValueError("LIFetch requires Index queries of the bound dtype, head count and width 128")
        if weights.dtype != self.weights.dtype:
            raise ValueError("LIFetch weights must have the bound dtype")
        if scale is not None:
            if scale.dtype != self.scale.dtype:
                raise ValueError("LIFetch requires float32 query scales")
            if scale.numel() == tokens * heads and scale.ndim <= 2:
                scale = scale.view(tokens, heads)
            if tuple(scale.shape) != (tokens, heads):
                raise ValueError("LIFetch requires one scale per token/head")
            self._on_device(scale, "query scales")
        self._on_device(query, "queries")
        self._on_device(weights, "weights")
        self._gather(query=query, weights=weights, scale=scale, tokens=tokens)
        return self.query, self.weights, self.scale
