"""Persistent Index rows of every stable owner, and the two ways rows get into them.

The role of the reference's IndexCacheStorage / VllmIndexCacheStorage (python/kvip/cache/index_storage.py:9-61,
python/kvip/adapters/vllm/index_import.py:6-56), with the attribute names its consumers read: per owner,
`history` Index rows (128-byte key, fp32 scale, int64 source address in the host pool, int64 logical id) whose
first `resident` positions describe the hot KV slots. Rows arrive from the model's paged Index cache: the new
tokens of a decode step with one launch (`ingest_decode`, kvip_b200_ingest, graph-capturable; bf16 sources are
quantised to FP8 e4m3 on the way), whole requests of a prefill batch with one launch (`ingest_prefill`,
kvip_b200_ingest_spans). The host keeps only the bookkeeping that needs no device read."""
import numpy as np

from .. import ops


class IndexCacheStorage:
    def __init__(self, torch, owners, history, resident, device, *, key_dtype=None):
        self.torch, self.history, self.resident, self.device = torch, history, resident, device
        self.keys = torch.zeros((owners, history, 128), dtype=key_dtype or torch.uint8, device=device)
        self.scales = torch.ones((owners, history), dtype=torch.float32, device=device)
        self.addresses = torch.zeros((owners, history), dtype=torch.int64, device=device)
        self.identity = torch.arange(history, dtype=torch.int64, device=device)
        self.logical_ids = self.identity.repeat(owners, 1)
        self.hot_valid = torch.zeros((owners, resident), dtype=torch.int32, device=device)
        self.requests = {}     # owner -> request currently bound to it
        self.imported = set()  # owners whose cached history has been restored
        self.published = {}    # owner -> committed host pages
        self.ingest_errors = torch.zeros(1, dtype=torch.int32, device=device)

    @property
    def nbytes(self):
        tensors = (self.keys, self.scales, self.addresses, self.identity, self.logical_ids, self.hot_valid)
        return sum(t.numel() * t.element_size() for t in tensors)

    def prepare(self, plans):
        """Owners that changed hands since the last step lose their permutation, residency and addresses,
        before the step is queued. All recycled owners are reset together (three indexed writes)."""
        recycled = []
        for plan in plans:
            if self.requests.get(plan.owner) != plan.request:
                self.requests[plan.owner] = plan.request
                self.imported.discard(plan.owner)
                self.published[plan.owner] = 0
                recycled.append(plan.owner)
        if not recycled:
            return
        rows = self.torch.tensor(sorted(set(recycled)), dtype=self.torch.int64, device=self.device)
        self.logical_ids[rows] = self.identity
        self.hot_valid[rows] = 0
        self.addresses[rows] = 0

    def publish(self, owner, page_addresses, *, block_size, token_bytes):
        """Append the owner's newly committed host pages as per-token addresses. Positions published earlier may
        have been permuted by the Index exchange since, so they are never rewritten."""
        done, total = self.published.get(owner, 0), len(page_addresses)
        if total < done or total * block_size > self.history:
            raise ValueError("Committed Index address range shrank or exceeds bound history")
        if total == done:
            return
        pages = np.asarray(page_addresses[done:], dtype=np.int64)
        tokens = (pages[:, None] + np.arange(block_size, dtype=np.int64)[None, :] * token_bytes).reshape(-1)
        self.addresses[owner, done * block_size: total * block_size] = self.torch.from_numpy(tokens).to(self.device)
        self.published[owner] = total

    # ---- import from the model's paged Index cache ----------------------------------------------------
    def _sources(self, cache):
        keys, scales = cache
        torch = self.torch
        if keys.shape[-1] != 128:
            raise ValueError("LIFetch Index import requires 128-wide keys")
        if keys.dtype == torch.bfloat16:
            return keys.reshape(-1, 128), None
        if keys.element_size() != 1 or scales is None or scales.dtype != torch.float32:
            raise ValueError("LIFetch Index import requires C8 keys and float32 scales (or bfloat16 keys)")
        rows = keys.view(torch.uint8).reshape(-1, 128)
        if rows.shape[0] != scales.numel():
            raise ValueError("Paged Index key and scale capacities differ")
        return rows, scales.reshape(-1)

    def ingest_prefill(self, cache, metadata, plans, positions):
        """Eager (not captured) import for a batch with prefill rows: for every request, its cached history once
        (through its block-table row), then the tokens this forward writes (through slot_mapping / positions). The
        span list is host bookkeeping; the rows move in ONE launch."""
        source_keys, source_scales = self._sources(cache)
        if source_scales is None:
            raise ValueError("Prefill import takes quantised (C8) pages")
        spans = []
        for row, plan in enumerate(plans):
            if self.requests.get(plan.owner) != plan.request:
                raise RuntimeError("Index owner must be prepared before ingestion")
            if plan.owner not in self.imported and plan.start:
                spans.append((plan.owner, row, 0, 0, plan.start, 0, 0, 0))
            self.imported.add(plan.owner)
            if plan.stop > plan.begin:
                spans.append((plan.owner, row, 1, plan.begin, plan.stop - plan.begin, 0, 0, 0))
        if not spans:
            return
        torch = self.torch
        table = torch.from_numpy(np.asarray(spans, dtype=np.int32)).to(self.device)
        ops.ingest_spans(self.keys.view(torch.uint8), self.scales, source_keys, source_scales,
                         metadata.block_table.to(torch.int32), metadata.slot_mapping.to(torch.int64),
                         positions.to(torch.int64), table, history=self.history, block=int(metadata.block_size),
                         max_tokens=max(span[4] for span in spans), errors=self.ingest_errors)

    def ingest_decode(self, cache, metadata, inputs, row_owners):
        """Fixed-shape, graph-capturable write of the B*Q new rows: one launch. Padding rows of the graph write
        distinct positions of reserved owner zero, so no live request is touched."""
        source_keys, source_scales = self._sources(cache)
        ops.ingest(self.keys.view(self.torch.uint8), self.scales, source_keys, source_scales, metadata.slot_mapping,
                   inputs.gather_indices, inputs.query_ends, row_owners, queries=inputs.queries, history=self.history)
