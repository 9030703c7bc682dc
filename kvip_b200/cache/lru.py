"""SlotLRU on the device: one eviction chain per request/layer row.

Same semantics and attribute names as the reference's host class (python/kvip/cache/lru.py:14-118,
numba kernels _lru_kernel.py:32-199), but the chain is an ordered array in HBM ("oldest first")
instead of next/previous links, so `commit` is one parallel stream compaction per row and the
victim list / its inverse map are written straight into the tensors the resolver reads
(`slots` -> rotating.lru_slots, `reserved_hot` -> rotating.reserved_hot): no host round trip
between forwards. `next`, `previous`, `head`, `tail` are derived views for inspection."""
import numpy as np
import torch

from .. import ops

TOPK = 2048
BITMAP_WORD_BITS = 32
BITMAP_ALIGNMENT_WORDS = 8


class SlotLRU:
    """Only the committed slot prefix is evictable; ABC slots live outside ``active``."""

    def __init__(self, device=None, rows=1, *, slots=None, reserved_hot=None):
        self.device = torch.device("cuda" if device is None else device)
        if self.device.type != "cuda":
            raise ValueError("SlotLRU keeps its state on a CUDA device")
        self.rows_count = rows
        self.version = 0
        self.active = 0                      # committed slots (max over rows; per-row in active_rows)
        self.capacity = 0
        i32 = dict(dtype=torch.int32, device=self.device)
        self.order = torch.empty((rows, 0), **i32)
        self.slots = torch.full((rows, TOPK), -1, **i32) if slots is None else slots
        self.reserved_hot = reserved_hot
        if self.slots.shape != (rows, TOPK) or self.slots.dtype != torch.int32 or not self.slots.is_contiguous():
            raise ValueError("SlotLRU victims must be contiguous int32 [rows, 2048]")
        if slots is not None:
            self.slots.fill_(-1)
        if reserved_hot is not None:
            reserved_hot.fill_(-1)
        self.bitmap = torch.empty((rows, 0), **i32)
        self.unique = torch.zeros(rows, **i32)
        self.rows = torch.zeros(rows, dtype=torch.int64, device=self.device)
        self.active_rows = torch.zeros(rows, **i32)
        self._active_host = [0] * rows
        self._no_touch = torch.full((rows, 1), -1, **i32)

    # ---- lifecycle --------------------------------------------------------------------------
    def resize(self, capacity, committed):
        """Grow storage and append newly committed slots, preserving LRU order; shrinking (or the
        first use) resets a row to ascending slot order. `committed` is an int or one int per row."""
        committed = [int(committed)] * self.rows_count if np.isscalar(committed) else [int(c) for c in committed]
        if len(committed) != self.rows_count or any(not 0 <= c <= capacity for c in committed):
            raise ValueError("Committed slots must fit HBM capacity")
        changed = False
        if capacity > self.capacity:
            capacity = max(capacity, 2 * self.capacity)
            grown = torch.full((self.rows_count, capacity), -1, dtype=torch.int32, device=self.device)
            grown[:, : self.capacity] = self.order
            self.order = grown
            words = (capacity + BITMAP_WORD_BITS - 1) // BITMAP_WORD_BITS
            words = (words + BITMAP_ALIGNMENT_WORDS - 1) // BITMAP_ALIGNMENT_WORDS * BITMAP_ALIGNMENT_WORDS
            self.bitmap = torch.zeros((self.rows_count, words), dtype=torch.int32, device=self.device)
            self.capacity = capacity
            changed = True
        identity = None
        for row, target in enumerate(committed):
            current = self._active_host[row]
            if target < current or current == 0 < target:
                identity = torch.arange(self.capacity, dtype=torch.int32, device=self.device) if identity is None else identity
                self.order[row, :target] = identity[:target]
                changed = True
            elif target > current:
                identity = torch.arange(self.capacity, dtype=torch.int32, device=self.device) if identity is None else identity
                self.order[row, current:target] = identity[current:target]
                changed = True
            self._active_host[row] = target
        self.active = max(self._active_host)
        self.active_rows.copy_(torch.tensor(self._active_host, dtype=torch.int32), non_blocking=False)
        if changed:
            self._select()

    def _select(self):
        self.version += 1
        ops.lru_commit(self.order, self.slots, self.bitmap, self.unique, self.reserved_hot, self._no_touch,
                       self.active_rows)

    def commit(self, destinations):
        """Consume the slots actually accessed in this step (any int32 tensor/array with one row of
        slots per LRU row, or a flat vector for a single row). Slots outside [0, active) are ignored."""
        if not torch.is_tensor(destinations):
            destinations = torch.from_numpy(np.ascontiguousarray(destinations, dtype=np.int32))
        touched = destinations.to(self.device, torch.int32).reshape(self.rows_count, -1).contiguous()
        if touched.shape[1] == 0 or self.capacity == 0:
            return
        ops.lru_commit(self.order, self.slots, self.bitmap, self.unique, self.reserved_hot, touched, self.active_rows)
        self.version += 1

    # ---- derived linked-list views (host, inspection only) -------------------------------------
    def _links(self):
        order = self.order.cpu().numpy()
        nxt = np.full((self.rows_count, self.capacity), -1, np.int32)
        prev = np.full((self.rows_count, self.capacity), -1, np.int32)
        head = np.full(self.rows_count, -1, np.int32)
        tail = np.full(self.rows_count, -1, np.int32)
        for row, active in enumerate(self._active_host):
            chain = order[row, :active]
            if active:
                head[row], tail[row] = chain[0], chain[-1]
                nxt[row, chain[:-1]] = chain[1:]
                prev[row, chain[1:]] = chain[:-1]
        return nxt, prev, head, tail

    next = property(lambda self: self._links()[0])
    previous = property(lambda self: self._links()[1])
    head = property(lambda self: self._links()[2])
    tail = property(lambda self: self._links()[3])


def warmup(device=None):
    """Touch the kernels once before serving (the reference compiles its numba kernels here)."""
    row = SlotLRU(device)
    row.resize(32, 16)
    row.commit(np.array([1], dtype=np.int32))
    row.resize(32, 24)
