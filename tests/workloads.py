"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

They stand in for the reference's calibrated generator and captured traces
(tests/operators/lifetch/support/workloads.py:399-490, 555-658 in the reference project), which are
not shipped. Everything is NumPy so that the oracle and the CUDA path see the same bytes."""
import numpy as np

import kvip_oracle as oracle

BLOCK, TOPK = 128, 2048


def li_case(seed=0, batch=4, queries=1, heads=64, len_lo=2048, len_hi=4096, key_dtype="fp8", weight_dtype="bf16",
            active=None, history=None, scale_lo=1e-3, scale_hi=1e-1, permute=True, owners=None):
    """One LI problem. Returns a dict of NumPy arrays:
    query [B*Q,H,128] (u8 E4M3 codes or u16 bf16 bits), keys [owners*history,128], weights [B*Q,H] (u16 bf16 bits or
    f32), query_scale [B*Q,H] f32 or None, key_scale [rows] f32 or None, key_lengths [B], query_ends [B,Q],
    block_table [B, history/128]."""
    rng = np.random.default_rng(seed)
    history = history or -(-len_hi // BLOCK) * BLOCK
    owners = owners or batch
    pages = history // BLOCK
    lengths = rng.integers(len_lo, len_hi + 1, batch).astype(np.int32)
    active = np.full(batch, queries) if active is None else np.asarray(active)
    query_ends = np.zeros((batch, queries), dtype=np.int32)
    for b in range(batch):
        for q in range(int(active[b])):
            query_ends[b, q] = max(1, int(lengths[b]) - (int(active[b]) - 1 - q))  # MTP: len-k+1 .. len
    rows = owners * history
    tokens = batch * queries
    if key_dtype == "fp8":
        key_scale = np.exp(rng.uniform(np.log(scale_lo), np.log(scale_hi), rows)).astype(np.float32)
        query_scale = np.exp(rng.uniform(np.log(scale_lo), np.log(scale_hi), (tokens, heads))).astype(np.float32)
        keys = oracle.encode_e4m3(np.clip(rng.standard_normal((rows, 128), dtype=np.float32) * 8, -448, 448))
        query = oracle.encode_e4m3(np.clip(rng.standard_normal((tokens, heads, 128), dtype=np.float32) * 8, -448, 448))
    else:
        key_scale = query_scale = None
        keys = oracle.f32_to_bf16_rne(rng.standard_normal((rows, 128), dtype=np.float32))
        query = oracle.f32_to_bf16_rne(rng.standard_normal((tokens, heads, 128), dtype=np.float32))
    w = (rng.standard_normal((tokens, heads)) / 8).astype(np.float32)  # N(0, 1/64)
    weights = oracle.f32_to_bf16_rne(w) if weight_dtype == "bf16" else w
    if permute:
        table = rng.permutation(owners * pages)[: batch * pages].reshape(batch, pages).astype(np.int32)
    else:
        table = np.arange(batch * pages, dtype=np.int32).reshape(batch, pages)
    return dict(query=query, keys=keys, weights=weights, query_scale=query_scale, key_scale=key_scale,
                key_lengths=lengths, query_ends=query_ends, block_table=table, heads=heads, queries=queries,
                batch=batch, history=history, key_dtype=key_dtype, weight_dtype=weight_dtype)


def prefill_case(seed=0, chunk=64, context=8192, heads=64, scale_lo=1e-3, scale_hi=1e-1):
    """A chunked-prefill LI problem in the layout of `li_case`: one owner's `context` FP8 keys, the last `chunk`
    tokens as queries (query i sees context - chunk + i + 1 keys), packed four query slots per row; every row
    reads the same pages through its own copy of one permuted block table."""
    assert chunk % 4 == 0 and context % BLOCK == 0
    rng = np.random.default_rng(seed)
    batch, queries, pages = chunk // 4, 4, context // BLOCK
    ends = (context - chunk + 1 + np.arange(chunk)).astype(np.int32).reshape(batch, queries)
    key_scale = np.exp(rng.uniform(np.log(scale_lo), np.log(scale_hi), context)).astype(np.float32)
    query_scale = np.exp(rng.uniform(np.log(scale_lo), np.log(scale_hi), (chunk, heads))).astype(np.float32)
    keys = oracle.encode_e4m3(np.clip(rng.standard_normal((context, 128), dtype=np.float32) * 8, -448, 448))
    query = oracle.encode_e4m3(np.clip(rng.standard_normal((chunk, heads, 128), dtype=np.float32) * 8, -448, 448))
    weights = oracle.f32_to_bf16_rne((rng.standard_normal((chunk, heads)) / 8).astype(np.float32))
    table = np.tile(rng.permutation(pages).astype(np.int32), (batch, 1))
    return dict(query=query, keys=keys, weights=weights, query_scale=query_scale, key_scale=key_scale,
                key_lengths=np.full(batch, context, np.int32), query_ends=ends, block_table=table, heads=heads,
                queries=queries, batch=batch, history=context, key_dtype="fp8", weight_dtype="bf16")


def to_torch(case, device):
    """Device tensors for the keys of a case (FP8 codes viewed as float8_e4m3fn, bf16 bits as bfloat16)."""
    import torch

    out = {}
    for name, value in case.items():
        if not isinstance(value, np.ndarray):
            out[name] = value
            continue
        t = torch.from_numpy(value.view(np.int16) if value.dtype == np.uint16 else value).to(device)
        if value.dtype == np.uint16:
            t = t.view(torch.bfloat16)
        elif value.dtype == np.uint8 and name in ("query", "keys"):
            t = t.view(torch.float8_e4m3fn)
        out[name] = t
    return out


def oracle_scores(case, score_mode=0, exact=False):
    """Oracle scores: NumPy golden formula, or the C restatement with the kernel's accumulation order."""
    kw = dict(key_is_bf16=case["key_dtype"] == "bf16", weight_is_bf16=case["weight_dtype"] == "bf16",
              score_mode=score_mode)
    if not exact:
        return oracle.li_scores(case["query"], case["keys"], case["weights"], case["query_scale"], case["key_scale"],
                                case["key_lengths"], case["query_ends"], case["block_table"], **kw)
    import oracle_c
    return oracle_c.li_scores(case, score_mode)


def li_tolerance(case, reference):
    """Allowed |device - reference| per score: the relative tolerance of the input format (1e-2 for FP8 inputs, 2e-3
    for bf16) plus a floor of 1e-2 of that (1e-4 / 2e-5) of the row's largest score, for sums that cancel."""
    rtol = 2e-3 if case["key_dtype"] == "bf16" else 1e-2
    return rtol * np.abs(reference) + rtol * 1e-2 * np.abs(reference).max(axis=1, keepdims=True)


def payload(owner, tokens, token_bytes):
    """Self-identifying KV rows: every 8-byte word of a row encodes (owner, token, word index), so any
    misplaced, torn or stale row is detected by value (the idea of workloads.py:493-502)."""
    tokens = np.asarray(tokens, dtype=np.uint64).reshape(-1, 1)
    words = np.arange(token_bytes // 8, dtype=np.uint64)[None, :]
    value = (np.uint64(owner + 1) << np.uint64(48)) ^ (tokens << np.uint64(16)) ^ words ^ (tokens * np.uint64(0x9E3779B97F4A7C15))
    return value.view(np.uint8).reshape(len(tokens), token_bytes)


def resolver_case(seed=0, batch=2, queries=4, history=8192, resident=4096, hot_fraction=0.5, overlap=0.5,
                  reserved=True, lru_valid=2048):
    """Selected positions with controlled hit/miss mix, cross-query duplicates and LRU state."""
    rng = np.random.default_rng(seed)
    selected = np.empty((batch, queries, TOPK), dtype=np.int32)
    hot_valid = (rng.random((batch, resident)) < 0.8).astype(np.int32)
    lru = np.full((batch, 2048), -1, dtype=np.int32)
    reserved_hot = np.full((batch, resident), -1, dtype=np.int32)
    for b in range(batch):
        victims = rng.permutation(resident)[:lru_valid].astype(np.int32)
        lru[b, :lru_valid] = victims
        if reserved:
            reserved_hot[b, victims] = np.arange(lru_valid)
        base = None
        for q in range(queries):
            hot_n = int(TOPK * hot_fraction)
            hot = rng.choice(resident, hot_n, replace=False)
            cold = rng.choice(np.arange(resident, history), TOPK - hot_n, replace=False)
            row = np.concatenate((hot, cold))
            if base is not None:
                keep = rng.random(TOPK) < overlap
                row = np.where(keep, base, row)
                _, first = np.unique(row, return_index=True)  # keep rows duplicate-free
                dup = np.setdiff1d(np.arange(TOPK), first)
                spare = np.setdiff1d(np.arange(history), row)
                row[dup] = rng.choice(spare, len(dup), replace=False)
            rng.shuffle(row)
            selected[b, q] = row
            base = row
    return dict(selected=selected, hot_valid=hot_valid, lru_slots=lru, reserved_hot=reserved_hot, history=history,
                resident=resident, batch=batch, queries=queries)
