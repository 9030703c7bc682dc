"""Harness of bench.py, the smoke check and the end-to-end tests; not part of the `kvip_b200` package.

Seeded synthetic decode workloads with the shapes and value distributions of the benchmark
configs, built directly in device memory, and a `DecodePipeline` that wires the public objects
(IndexCacheStorage, LIFetchWorkspace, HostKVPool, CudaBinding, IndexUpdate, SlotLRU, LIFetch) the way
a serving adapter would.

The reference measures on captured decode traces and a calibrated generator that are not shipped;
these inputs stand in for them: q_I / k_I ~ N(0,1) (bf16, or FP8 e4m3 with per-token key scales and
per-(token, head) query scales drawn log-uniformly from [1e-3, 1e-1]), head weights ~ N(0, 1/64),
context lengths uniform in [len_lo, len_hi], KV rows that identify (owner, token) in every 8-byte word."""
import numpy as np
import torch

from kvip_b200 import _lib
from kvip_b200.cache.index_storage import IndexCacheStorage
from kvip_b200.cache.lru import SlotLRU
from kvip_b200.operators.lifetch import CudaBinding, HostKVPool, IndexUpdate, LIFetch, LIFetchWorkspace

TOPK = 2048


def payload_rows(owner, tokens, token_bytes):
    """Self-identifying KV rows (NumPy, host): word w of row (owner, token) mixes all three."""
    tokens = np.asarray(tokens, dtype=np.uint64).reshape(-1, 1)
    words = np.arange(token_bytes // 8, dtype=np.uint64)[None, :]
    value = ((np.uint64(owner + 1) << np.uint64(48)) ^ (tokens << np.uint64(16)) ^ words
             ^ (tokens * np.uint64(0x9E3779B97F4A7C15)))
    return value.view(np.uint8).reshape(len(tokens), token_bytes)


def _log_uniform(shape, lo, hi, generator, device):
    u = torch.rand(shape, generator=generator, device=device, dtype=torch.float32)
    return torch.exp(u * (np.log(hi) - np.log(lo)) + np.log(lo))


def lidu_state(batch, queries_per_request, source, hot, *, resident_fraction=0.5, hit_fraction=0.9, seed=0):
    """Seeded inputs of one `lidu` call (NumPy): `batch` requests with `queries_per_request` query rows each,
    `source` logical tokens, `hot` resident slots of which `resident_fraction` are mapped; every query selects
    2048 distinct tokens, `hit_fraction` of them resident. Keys are the argument names of `kvip_b200.lidu`."""
    rng = np.random.default_rng(seed)
    t2s = np.full((batch, source), -1, np.int32)
    s2t = np.full((batch, hot), -1, np.int32)
    rows = []
    for r in range(batch):
        resident = rng.choice(source, int(hot * resident_fraction), replace=False)
        slots = rng.permutation(hot)[: len(resident)]
        t2s[r, resident], s2t[r, slots] = slots, resident
        cold = np.setdiff1d(np.arange(source), resident, assume_unique=False)
        hits = int(TOPK * hit_fraction)
        for _ in range(queries_per_request):
            picked = np.concatenate((rng.choice(resident, hits, replace=False),
                                     rng.choice(cold, TOPK - hits, replace=False)))
            rows.append(rng.permutation(picked))
    miss_slots = np.stack([rng.permutation(hot)[:TOPK] for _ in range(batch)]).astype(np.int32)
    bitmap = np.zeros((batch, 4176), np.int32)
    for r in range(batch):  # the victim candidates are also marked in the bitmap: their tokens count as misses
        bits = np.zeros(4176 * 32, np.uint8)
        bits[miss_slots[r]] = 1
        bitmap[r] = np.packbits(bits, bitorder="little").view("<i4")
    return dict(
        topk_indices=np.stack(rows).astype(np.int32).reshape(-1, 1, TOPK),
        actual_seq_lengths_query=np.cumsum([queries_per_request] * batch).astype(np.int32),
        req_pool_entries=np.arange(batch, dtype=np.int32), token_to_slot_pool=t2s, slot_to_token_pool=s2t,
        eviction_cursors=rng.integers(0, hot, batch).astype(np.int32), cache_tokens=np.full(batch, hot, np.int32),
        candidate_lens=np.full(batch, source, np.int32), miss_slots=miss_slots, miss_slot_bitmap=bitmap,
        resident_block_table=rng.permutation(batch * hot // 128).astype(np.int32).reshape(batch, -1),
        logical_seq_lengths=np.full(batch, source, np.int32))


class DecodePipeline:
    def __init__(self, device, *, batch, queries=1, heads=64, history, resident, len_lo, len_hi, key_dtype="fp8",
                 weight_dtype="bf16", token_bytes=1152, seed=0, gather=True, host_pool=True, fill_payload=False,
                 score_mode=_lib.SCORE_FP32, li_variant=0, owners=None, permute_owners=True, sm_count=0,
                 overlap_lru=True, prefetch_limit=0, prefetch_windows=3, prefetch_ctas=0,
                 prefetch_last_window=False, tail_slots=0, overlap_fetch=False):
        self.device = device = torch.device(device)
        self.batch, self.queries, self.heads, self.history, self.resident = batch, queries, heads, history, resident
        self.token_bytes, self.key_dtype = token_bytes, key_dtype
        owners = owners or batch
        self.owners = owners
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        rng = np.random.default_rng(seed)
        bf16 = key_dtype == "bf16"
        self.storage = IndexCacheStorage(torch, owners, history, resident, device,
                                         key_dtype=torch.bfloat16 if bf16 else torch.uint8)
        self.workspace = LIFetchWorkspace(
            torch, batch=batch, history=history, device=device, index_heads=heads, queries=queries,
            query_dtype=torch.bfloat16 if bf16 else torch.float8_e4m3fn,
            weight_dtype=torch.float32 if weight_dtype == "fp32" else torch.bfloat16)
        # ---- Index keys and scales, one owner at a time to bound temporaries ------------------------
        for owner in range(owners):
            if bf16:
                self.storage.keys[owner].copy_(torch.randn((history, 128), generator=g, device=device).to(torch.bfloat16))
            else:
                scale = _log_uniform((history,), 1e-3, 1e-1, g, device)
                values = (torch.randn((history, 128), generator=g, device=device) * 8).clamp_(-448, 448)
                self.storage.keys[owner].copy_(values.to(torch.float8_e4m3fn).view(torch.uint8))
                self.storage.scales[owner].copy_(scale)
        # ---- requests --------------------------------------------------------------------------------
        self.lengths = rng.integers(len_lo, len_hi + 1, batch).astype(np.int32)
        owner_order = rng.permutation(owners)[:batch] if permute_owners else np.arange(batch)
        self.row_owner_list = [int(o) for o in owner_order]
        inputs = self.workspace.inputs
        inputs.prepare((queries,) * batch, query_owners=tuple(self.row_owner_list))
        positions = np.zeros(batch * queries, dtype=np.int64)
        for b in range(batch):
            for q in range(queries):
                positions[b * queries + q] = max(0, int(self.lengths[b]) - (queries - q))  # MTP: len-Q .. len-1
        self.positions = torch.from_numpy(positions).to(device)
        inputs.bind_positions(self.positions)
        self.workspace.key_lengths.copy_(torch.from_numpy(self.lengths))
        self.new_queries(seed)
        # ---- KV pools ----------------------------------------------------------------------------------
        # ABC tail: `tail_slots` dedicated slots per owner behind the hot ones, bounds [B, 2] set by the caller
        self.tail_slots = tail_slots
        self.output_stride = resident + tail_slots
        self.tail_bounds = torch.zeros((batch, 2), dtype=torch.int32, device=device) if tail_slots else None
        self.pool_hbm = torch.zeros((owners * self.output_stride, token_bytes), dtype=torch.uint8, device=device)
        self.host_pool = None
        source = None
        if host_pool:
            self.host_pool = HostKVPool(torch, owners, history, token_bytes, device)
            if fill_payload:
                for owner in range(owners):
                    self.host_pool.tensor[owner].copy_(torch.from_numpy(payload_rows(owner, np.arange(history), token_bytes)))
            for owner in range(owners):
                self.storage.addresses[owner].copy_(self.host_pool.addresses(owner))
        else:
            source = torch.zeros((owners * history, token_bytes), dtype=torch.uint8, device=device)
            if fill_payload:
                for owner in range(owners):
                    source[owner * history:(owner + 1) * history].copy_(
                        torch.from_numpy(payload_rows(owner, np.arange(history), token_bytes)))
            identity = torch.arange(history, dtype=torch.int64, device=device)
            for owner in range(owners):
                self.storage.addresses[owner].copy_((identity + owner * history) * token_bytes)
        self.source = source
        self.gather_out = (torch.zeros((batch * queries, TOPK, token_bytes), dtype=torch.uint8, device=device)
                           if gather else None)
        # ---- bindings -----------------------------------------------------------------------------------
        self.workspace.allocate_rotation(torch, batch=batch, history=history, resident=resident)
        self.rotating = CudaBinding(
            torch, self.workspace.arguments(self.storage), self.host_pool, self.pool_hbm, batch=batch, history=history,
            resident=resident, query_ends=inputs.query_ends, hot_valid=self.storage.hot_valid,
            token_addresses=self.storage.addresses, row_owners=inputs.row_owners, scratch=self.workspace.scratch,
            token_bytes=token_bytes, queries=queries, score_mode=score_mode, gather_output=self.gather_out,
            li_variant=li_variant, source=source, sm_count=sm_count, tail_bounds=self.tail_bounds,
            output_stride=self.output_stride)
        self.update = IndexUpdate(
            torch, keys=self.storage.keys, scales=self.storage.scales, addresses=self.storage.addresses,
            logical_ids=self.storage.logical_ids, row_owners=inputs.row_owners, rotating=self.rotating,
            query_inputs=inputs)
        self.lru = SlotLRU(device, rows=batch, slots=self.rotating.lru_slots, reserved_hot=self.rotating.reserved_hot)
        self.lru.resize(resident, resident)
        # LRU feedback inside the call (beside fetch + gather) or, as in the reference, after it
        self.overlap_lru = overlap_lru
        self.forward = LIFetch(self.rotating, self.update, lru=self.lru if overlap_lru else None,
                               prefetch_limit=prefetch_limit, prefetch_windows=prefetch_windows, prefetch_ctas=prefetch_ctas,
                               prefetch_last_window=prefetch_last_window, overlap_fetch=overlap_fetch)

    def new_queries(self, seed):
        """Fresh projected queries / head weights for all rows, packed through QueryInputs.pack."""
        device, heads = self.device, self.heads
        tokens = self.batch * self.queries
        g = torch.Generator(device=device)
        g.manual_seed(1000003 + seed)
        inputs = self.workspace.inputs
        w = torch.randn((tokens, heads), generator=g, device=device) / 8
        weights = w if inputs.weights.dtype == torch.float32 else w.to(torch.bfloat16)
        if self.key_dtype == "bf16":
            query = torch.randn((tokens, heads, 128), generator=g, device=device).to(torch.bfloat16)
            scale = None
        else:
            query = (torch.randn((tokens, heads, 128), generator=g, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
            scale = _log_uniform((tokens, heads), 1e-3, 1e-1, g, device)
        inputs.pack(query, weights, scale)

    def step(self, ingest=False):
        """One decode step of the path: (the paged Index update of the new tokens,) the fused forward, then
        the LRU feedback of the slots it used."""
        if ingest:
            self.ingest_new_tokens()
        self.forward()
        if not self.overlap_lru:
            self.lru.commit(self.update.slot_output.view(self.batch, -1))

    def ingest_new_tokens(self):
        """Write one new bf16 k_I row per query token into the Index cache (quantised to FP8 + scale)."""
        if self.key_dtype != "fp8":
            raise ValueError("the Index update quantises into FP8 storage")
        if not hasattr(self, "new_keys"):
            from types import SimpleNamespace
            tokens = self.batch * self.queries
            g = torch.Generator(device=self.device)
            g.manual_seed(777)
            self.new_keys = torch.randn((tokens, 128), generator=g, device=self.device).to(torch.bfloat16)
            self.new_meta = SimpleNamespace(slot_mapping=torch.arange(tokens, dtype=torch.int64, device=self.device))
        inputs = self.workspace.inputs
        self.storage.ingest_decode((self.new_keys, None), self.new_meta, inputs, inputs.row_owners)

    def make_query_bank(self, count, correlation=0.9, seed=0):
        """`count` query sets whose selections overlap from one step to the next: an AR(1) drift
        q[k] = rho * q[k-1] + sqrt(1 - rho^2) * noise on the unquantised queries, fixed head weights."""
        device, heads = self.device, self.heads
        tokens = self.batch * self.queries
        g = torch.Generator(device=device)
        g.manual_seed(2000003 + seed)
        weights = (torch.randn((tokens, heads), generator=g, device=device) / 8).to(self.workspace.inputs.weights.dtype)
        scale = _log_uniform((tokens, heads), 1e-3, 1e-1, g, device)
        state = torch.randn((tokens, heads, 128), generator=g, device=device)
        bank = []
        for _ in range(count):
            noise = torch.randn((tokens, heads, 128), generator=g, device=device)
            state = correlation * state + (1 - correlation ** 2) ** 0.5 * noise
            if self.key_dtype == "bf16":
                bank.append((state.to(torch.bfloat16), weights, None))
            else:
                bank.append(((state * 8).clamp(-448, 448).to(torch.float8_e4m3fn), weights, scale))
        self.query_bank = bank
        return bank

    def load_queries(self, index):
        """Pack query set `index` of the bank into the bound input buffers (device copies, in stream order)."""
        query, weights, scale = self.query_bank[index % len(self.query_bank)]
        self.workspace.inputs.pack(query, weights, scale)

    def query_tokens(self):
        return self.batch * self.queries

    def close(self):
        if self.host_pool is not None:
            self.host_pool.close()
