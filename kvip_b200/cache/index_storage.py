"""Persistent Index rows, ownership and committed host-pool addresses.

Mirrors the reference's IndexCacheStorage / VllmIndexCacheStorage
(python/kvip/cache/index_storage.py:9-61, python/kvip/adapters/vllm/index_import.py:6-56): per stable
owner, `history` Index rows (128-byte key, fp32 scale, int64 source address, int64 logical id) whose
first `resident` positions describe the hot KV slots. The decode-time update of new tokens is one
CUDA launch (`ingest_decode`); bf16 sources are quantised to FP8 e4m3 on the way in."""
from .. import ops


class IndexCacheStorage:
    def __init__(self, torch, owners, history, resident, device, *, key_dtype=None):
        self.torch, self.history, self.resident, self.device = torch, history, resident, device
        key_dtype = key_dtype or torch.uint8
        self.keys = torch.zeros((owners, history, 128), dtype=key_dtype, device=device)
        self.scales = torch.ones((owners, history), dtype=torch.float32, device=device)
        self.addresses = torch.zeros((owners, history), dtype=torch.int64, device=device)
        self.identity = torch.arange(history, dtype=torch.int64, device=device)
        self.logical_ids = self.identity.expand(owners, -1).clone()
        self.hot_valid = torch.zeros((owners, resident), dtype=torch.int32, device=device)
        self.requests = {}
        self.imported = set()
        self.published = {}

    @property
    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (
            self.keys, self.scales, self.addresses, self.identity, self.logical_ids, self.hot_valid))

    def prepare(self, plans):
        """Invalidate recycled owner metadata before this step is queued."""
        for plan in plans:
            if self.requests.get(plan.owner) == plan.request:
                continue
            self.requests[plan.owner] = plan.request
            self.imported.discard(plan.owner)
            self.published[plan.owner] = 0
            self.logical_ids[plan.owner].copy_(self.identity)
            self.hot_valid[plan.owner].zero_()
            self.addresses[plan.owner].zero_()

    def publish(self, owner, page_addresses, *, block_size, token_bytes):
        """Append newly committed host pages; entries that were already permuted are never rewritten."""
        count = len(page_addresses)
        previous = self.published.get(owner, 0)
        if count < previous or count * block_size > self.history:
            raise ValueError("Committed Index address range shrank or exceeds bound history")
        if count == previous:
            return
        pages = self.torch.tensor(page_addresses[previous:], dtype=self.torch.int64, device=self.device)
        offsets = self.identity[:block_size] * token_bytes
        self.addresses[owner, previous * block_size: count * block_size].copy_(
            (pages[:, None] + offsets[None, :]).reshape(-1))
        self.published[owner] = count

    # ---- paged-cache import (reference: adapters/vllm/index_import.py) --------------------------
    def _sources(self, cache):
        keys, scales = cache
        torch = self.torch
        if keys.shape[-1] != 128:
            raise ValueError("LIFetch Index import requires 128-wide keys")
        if keys.dtype == torch.bfloat16:
            return keys.reshape(-1, 128), None
        if keys.element_size() != 1 or scales is None or scales.dtype != torch.float32:
            raise ValueError("LIFetch Index import requires C8 keys and float32 scales (or bfloat16 keys)")
        source_keys, source_scales = keys.view(torch.uint8).reshape(-1, 128), scales.reshape(-1)
        if source_keys.shape[0] != source_scales.numel():
            raise ValueError("Paged Index key and scale capacities differ")
        return source_keys, source_scales

    def ingest_prefill(self, cache, metadata, plans, positions):
        """Eager prefill: import restored history once, then the current writes (not graph-captured)."""
        torch = self.torch
        source_keys, source_scales = self._sources(cache)
        if source_scales is None:
            raise ValueError("Prefill import takes quantised (C8) pages")
        for row, plan in enumerate(plans):
            owner = plan.owner
            if self.requests.get(owner) != plan.request:
                raise RuntimeError("Index owner must be prepared before ingestion")
            if owner not in self.imported and plan.start:
                tokens = self.identity[: plan.start]
                pages = torch.index_select(metadata.block_table[row], 0, tokens // metadata.block_size)
                sources = pages.long() * metadata.block_size + tokens % metadata.block_size
                self.keys[owner, : plan.start].copy_(torch.index_select(source_keys, 0, sources).view(self.keys.dtype))
                self.scales[owner, : plan.start].copy_(torch.index_select(source_scales, 0, sources))
            self.imported.add(owner)
            sources = metadata.slot_mapping[plan.begin: plan.stop].long()
            targets = positions[plan.begin: plan.stop].long()
            self.keys[owner].index_copy_(0, targets, torch.index_select(source_keys, 0, sources).view(self.keys.dtype))
            self.scales[owner].index_copy_(0, targets, torch.index_select(source_scales, 0, sources))

    def ingest_decode(self, cache, metadata, inputs, row_owners):
        """Fixed-shape, graph-capturable write of the B*Q new rows: one kernel launch. Invalid graph rows
        write distinct positions of reserved owner zero, leaving every live request untouched."""
        source_keys, source_scales = self._sources(cache)
        ops.ingest(self.keys.view(self.torch.uint8), self.scales, source_keys, source_scales, metadata.slot_mapping,
                   inputs.gather_indices, inputs.query_ends, row_owners, queries=inputs.queries, history=self.history)
