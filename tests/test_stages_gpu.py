"""Parity of every CUDA stage with the CPU oracle, called through the C ABI (B200 only).

Bit-exact for indices, slot maps, Index rows and bytes; LI scores within the tolerance of the
north star: rtol 1e-2 for FP8 inputs and 2e-3 for bf16 inputs, measured against the score scale
of the row (scores are signed sums, so a pure element-wise rtol is meaningless near zero)."""
import numpy as np
import pytest
import torch

import kvip_oracle as oracle
import oracle_c
import workloads
from kvip_b200 import _lib, ops

pytestmark = pytest.mark.gpu
TOPK = 2048


def _valid_mask(case, stride):
    ends = case["query_ends"].reshape(-1)
    lens = np.repeat(case["key_lengths"], case["queries"])
    valid = np.minimum(ends, lens)
    return np.arange(stride)[None, :] < valid[:, None]


def _li(case, device, **kw):
    t = workloads.to_torch(case, device)
    scores, status = ops.li_score(t["query"], t["keys"], t["weights"], t["query_scale"], t["key_scale"],
                                  t["key_lengths"], t["query_ends"], t["block_table"], **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"LI kernel status {int(status.item())}"
    return scores, t


LI_CASES = [
    # C1 of the benchmark configs: B=4, 1 query, ctx U[2048,4096], 64 heads, bf16 q/k, fp32 weights
    dict(seed=0, batch=4, queries=1, heads=64, len_lo=2048, len_hi=4096, key_dtype="bf16", weight_dtype="fp32"),
    # FP8 keys with per-token scales, 2 MTP queries, bf16 weights x per-(token, head) query scale
    dict(seed=1, batch=3, queries=2, heads=64, len_lo=3000, len_hi=6000, key_dtype="fp8", weight_dtype="bf16"),
    # 32 heads, the reference's 4 query slots with ragged activity (0..4 active, padding rows)
    dict(seed=2, batch=5, queries=4, heads=32, len_lo=130, len_hi=2500, key_dtype="fp8", weight_dtype="bf16",
         active=[4, 0, 1, 3, 2]),
    dict(seed=3, batch=2, queries=4, heads=64, len_lo=1000, len_hi=1500, key_dtype="bf16", weight_dtype="bf16"),
]


@pytest.mark.parametrize("spec", LI_CASES, ids=lambda s: f"seed{s['seed']}")
def test_li_simt_matches_c_oracle_bit_exact(spec, device):
    case = workloads.li_case(**spec)
    expected = workloads.oracle_scores(case, exact=True)
    scores, _ = _li(case, device, simt=True)
    mask = _valid_mask(case, expected.shape[1])
    got = scores.cpu().numpy()
    assert np.array_equal(got[mask].view(np.uint32), expected[mask].view(np.uint32))


@pytest.mark.parametrize("spec", LI_CASES, ids=lambda s: f"seed{s['seed']}")
@pytest.mark.parametrize("score_mode", [0, 1])
def test_li_tcgen05_within_tolerance(spec, score_mode, device):
    """Against the NumPy golden formula."""
    case = workloads.li_case(**spec)
    expected = workloads.oracle_scores(case, score_mode=score_mode)
    scores, _ = _li(case, device, score_mode=score_mode)
    got = scores.cpu().numpy()
    mask = _valid_mask(case, expected.shape[1])
    allowed = workloads.li_tolerance(case, np.where(mask, expected, 0))
    if score_mode == 1:
        allowed = allowed + 2**-7 * np.abs(expected)  # one bf16 spacing: a rounding boundary may fall between the two sums
    err = np.abs(got - expected)
    assert (err[mask] <= allowed[mask]).all(), (err[mask].max(), np.abs(expected[mask]).max())


RING_CASES = [(1, 64, "fp8"), (2, 64, "fp8"), (4, 64, "fp8"), (4, 32, "fp8"), (1, 64, "bf16"), (4, 64, "bf16")]


@pytest.mark.parametrize("stages", [0, 2, 3, 5, 8])
@pytest.mark.parametrize("queries,heads,key_dtype", RING_CASES)
def test_li_tcgen05_rings_wrap(queries, heads, key_dtype, stages, device):
    """Two CTAs for ~170 key pages: every CTA walks its key-stage ring and its accumulator ring many
    times and crosses request boundaries, for each accumulator count (8, 4, 2) and for stage counts that
    allow four, two and one MMA issuers. Checked against the CUDA-core kernel, which matches the C
    oracle bit for bit."""
    case = workloads.li_case(seed=40 + queries, batch=3, queries=queries, heads=heads, len_lo=5000, len_hi=9000,
                             key_dtype=key_dtype, weight_dtype="bf16")
    expected, _ = _li(case, device, simt=True)
    expected = expected.cpu().numpy()
    mask = _valid_mask(case, expected.shape[1])
    allowed = workloads.li_tolerance(case, np.where(mask, expected, 0))
    scores, _ = _li(case, device, ctas=2, stages=stages)
    assert (np.abs(scores.cpu().numpy() - expected)[mask] <= allowed[mask]).all(), (queries, heads, stages)


@pytest.mark.parametrize("key_dtype", ["fp8", "bf16"])
def test_li_tcgen05_ragged_query_slots_two_units(key_dtype, device):
    """Four query slots of 64 heads are reduced as two 128-column units per key page; requests with one, two or
    three live slots leave the second unit partly or wholly empty, and a request without live slots has no
    tiles at all."""
    case = workloads.li_case(seed=77, batch=5, queries=4, heads=64, len_lo=3000, len_hi=6000, key_dtype=key_dtype,
                             weight_dtype="bf16", active=[3, 1, 4, 0, 2])
    expected, _ = _li(case, device, simt=True)
    expected = expected.cpu().numpy()
    mask = _valid_mask(case, expected.shape[1])
    allowed = workloads.li_tolerance(case, np.where(mask, expected, 0))
    for kw in (dict(), dict(ctas=2), dict(ctas=3, stages=3)):
        scores, _ = _li(case, device, **kw)
        assert (np.abs(scores.cpu().numpy() - expected)[mask] <= allowed[mask]).all(), kw


def test_li_bounded_wait_gives_up_and_reports(device):
    """Every wait inside the tensor-core kernel is bounded. With the test hook one key page of CTA 0 is never
    loaded: the wait for it runs out (the limit is a launch argument: 20 million cycles, about 10 ms, here), the CTA
    leaves its pipeline in order, the
    kernel returns with KVIP_ERR_PIPELINE in the status word, and the next ordinary call on the same context
    is correct again."""
    case = workloads.li_case(seed=12, batch=2, queries=1, heads=64, len_lo=4000, len_hi=5000, key_dtype="fp8",
                             weight_dtype="bf16")
    t = workloads.to_torch(case, device)
    args = (t["query"], t["keys"], t["weights"], t["query_scale"], t["key_scale"], t["key_lengths"], t["query_ends"],
            t["block_table"])
    _, status = ops.li_score(*args, ctas=2, withhold_tile=3, wait_kilocycles=20000)
    torch.cuda.synchronize()
    assert int(status.item()) & 32, "the kernel must report the abandoned wait"
    expected, _ = _li(case, device, simt=True)
    scores, status = ops.li_score(*args, ctas=2)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    mask = _valid_mask(case, expected.shape[1])
    ref, out = expected.cpu().numpy(), scores.cpu().numpy()
    for row in range(out.shape[0]):
        scale = np.abs(ref[row][mask[row]]).max()
        assert (np.abs(out[row][mask[row]] - ref[row][mask[row]]) <= 1e-2 * np.abs(ref[row][mask[row]]) + 1e-4 * scale).all()


def test_chunked_prefill_li_and_topk(device):
    """The chunked-prefill configuration at test size: 128 query tokens of one request against a causal
    8192-token context, four query slots per row, all rows reading the same key pages. Scores within the FP8
    tolerance of the golden formula; TopK of the kernel's own scores bit-exact with the oracle's TopK of them."""
    case = workloads.prefill_case(seed=3, chunk=128, context=8192)
    expected = workloads.oracle_scores(case)
    scores, t = _li(case, device)
    got = scores.cpu().numpy()
    mask = _valid_mask(case, expected.shape[1])
    allowed = workloads.li_tolerance(case, np.where(mask, expected, 0))
    assert (np.abs(got - expected)[mask] <= allowed[mask]).all()
    ends = case["query_ends"].reshape(-1, 1)
    picked = ops.topk(scores, t["key_lengths"], t["query_ends"])
    torch.cuda.synchronize()
    assert np.array_equal(picked.cpu().numpy(), oracle_c.topk(got, case["key_lengths"], ends))


def test_li_exact_binary_fraction_fixture(device):
    """Exact-arithmetic inputs in the style of the reference fixture (workloads.py:196-283: FP8 codes
    {0, 0x38, 0x40, 0x44}, power-of-two scales): every partial sum is exact in fp32, so the tensor-core
    path must agree with the oracle bit for bit, in both score modes."""
    rng = np.random.default_rng(73121)
    batch, queries, heads, history = 2, 4, 64, 4096
    case = workloads.li_case(seed=5, batch=batch, queries=queries, heads=heads, len_lo=history, len_hi=history)
    codes = np.array([0, 0x38, 0x40, 0x44], np.uint8)
    case["keys"] = codes[rng.integers(0, 4, case["keys"].shape)]
    query = np.zeros_like(case["query"])
    for t in range(batch * queries):
        columns = (np.arange(heads) + t * 16) % 128
        query[t, np.arange(heads), columns] = 0x38
    case["query"] = query
    head = np.arange(heads)[None, :]
    qi = np.arange(batch * queries)[:, None]
    case["query_scale"] = np.array([0.5, 1.0, 2.0], np.float32)[(head + qi) % 3]
    case["weights"] = oracle.f32_to_bf16_rne(np.array([1.0, 2.0, 0.5], np.float32)[(head * 2 + qi) % 3])
    case["key_scale"] = np.exp2(rng.integers(-2, 2, case["key_scale"].shape)).astype(np.float32)
    for mode in (0, 1):
        expected = workloads.oracle_scores(case, score_mode=mode)
        mask = _valid_mask(case, expected.shape[1])
        scores, _ = _li(case, device, score_mode=mode)
        assert np.array_equal(scores.cpu().numpy()[mask], expected[mask]), mode


def _topk_check(scores_np, key_lengths, query_ends, device, base_index=0):
    scores = torch.from_numpy(scores_np).to(device)
    out_scores = torch.zeros((scores.shape[0], TOPK), dtype=torch.float32, device=device)
    lengths_t, ends_t = torch.from_numpy(key_lengths).to(device), torch.from_numpy(query_ends).to(device)
    got = ops.topk(scores, lengths_t, ends_t, out_scores=out_scores, base_index=base_index)
    # second path: first radix pass in its own kernel + shared-memory candidates; run twice to prove the
    # histogram scratch is handed back all-zero
    histogram = torch.zeros((scores.shape[0], 4096), dtype=torch.int32, device=device)
    for _ in range(2):
        split = ops.topk(scores, lengths_t, ends_t, base_index=base_index, histogram=histogram)
        torch.cuda.synchronize()
        assert torch.equal(split, got)
        assert int(histogram.abs().sum()) == 0
    # third path: every pass on several CTAs per row
    scratch = torch.zeros((scores.shape[0], 20544), dtype=torch.int32, device=device)
    split_scores = torch.zeros_like(out_scores)
    for _ in range(2):
        split = ops.topk(scores, lengths_t, ends_t, base_index=base_index, split_scratch=scratch, out_scores=split_scores)
        torch.cuda.synchronize()
        assert torch.equal(split, got) and torch.equal(split_scores, out_scores)
        assert int(scratch[:, :4160].abs().sum()) == 0   # histogram + header are handed back all-zero
    expected = oracle_c.topk(scores_np, key_lengths, query_ends, base_index)
    got = got.cpu().numpy()
    assert np.array_equal(got, expected)
    live = got >= 0
    rows = np.nonzero(live)[0]
    assert np.array_equal(out_scores.cpu().numpy()[live], scores_np[rows, got[live] - base_index])
    return got


def test_topk_random_rows(device):
    rng = np.random.default_rng(0)
    batch, queries, stride = 6, 2, 40960
    scores = rng.standard_normal((batch * queries, stride)).astype(np.float32)
    key_lengths = np.array([40960, 2048, 2049, 100, 0, 33333], np.int32)
    query_ends = np.stack((key_lengths - 1, key_lengths), 1).astype(np.int32).clip(0)
    _topk_check(scores, key_lengths, query_ends, device)


def test_topk_ties_and_special_values(device):
    rng = np.random.default_rng(1)
    stride = 16384
    rows = []
    rows.append(np.zeros(stride, np.float32))                                   # all equal: lowest indices win
    rows.append(rng.integers(0, 3, stride).astype(np.float32))                  # massive ties at the cut
    bf = oracle.bf16_away(rng.standard_normal(stride).astype(np.float32))       # bf16-rounded scores
    rows.append(bf)
    special = rng.standard_normal(stride).astype(np.float32)
    special[::97] = -0.0
    special[5::1013] = np.inf
    special[7::1013] = -np.inf
    rows.append(special)
    rows.append(-np.abs(rng.standard_normal(stride)).astype(np.float32))        # all negative
    rows.append(np.arange(stride, dtype=np.float32))                             # ascending: the tail wins
    scores = np.stack(rows)
    key_lengths = np.full(len(rows), stride, np.int32)
    got = _topk_check(scores, key_lengths, key_lengths.copy().reshape(-1, 1), device)
    assert np.array_equal(got[0], np.arange(TOPK))


def test_topk_long_row_and_base_index(device):
    rng = np.random.default_rng(2)
    scores = (rng.standard_normal((2, 131072)) * np.exp(rng.uniform(-3, 3, (2, 131072)))).astype(np.float32)
    key_lengths = np.array([131072, 131071], np.int32)
    _topk_check(scores, key_lengths, key_lengths.reshape(-1, 1).copy(), device, base_index=131072 * 3)


def test_topk_many_rows_one_cta_each(device):
    """More rows than half the SMs: the selection runs one CTA per row instead of a pair per row."""
    rng = np.random.default_rng(9)
    rows, stride = 96, 20480
    scores = (rng.standard_normal((rows, stride)) * np.exp(rng.uniform(-2, 2, (rows, 1)))).astype(np.float32)
    scores[5] = 1.0                                  # constant row: the kept list overflows -> three-pass path
    scores[6] = rng.integers(0, 2, stride)           # two values: the cut falls inside a long run of ties
    key_lengths = rng.integers(2048, stride + 1, rows).astype(np.int32)
    key_lengths[:8] = stride
    _topk_check(scores, key_lengths, key_lengths.reshape(-1, 1).copy(), device)


@pytest.mark.parametrize("stride", [200704, 300032])
def test_topk_wide_rows(stride, device):
    """Rows beyond 131072 scores: 32 scores per thread in the cluster kernel, and (beyond 262144) the
    one-CTA-per-row kernel. A constant row overflows every candidate list; a two-valued row puts the cut
    inside a run of ties that spans all eight slices."""
    rng = np.random.default_rng(stride)
    rows = [rng.standard_normal(stride).astype(np.float32),
            np.full(stride, 0.25, np.float32),
            rng.integers(0, 2, stride).astype(np.float32),
            (rng.standard_normal(stride) * np.exp(rng.uniform(-3, 3, stride))).astype(np.float32)]
    scores = np.stack(rows)
    key_lengths = np.array([stride, stride, stride - 5, stride // 2 + 1], np.int32)
    _topk_check(scores, key_lengths, key_lengths.reshape(-1, 1).copy(), device, base_index=7)


def test_cold_predicate_matches_oracle_and_covers_the_final_topk(device):
    """Resident threshold + cold predicate: prefix TopK, threshold key, bitmap and count bit-exact with the
    oracle; and the property that makes the stage useful - every cold position of the row's final TopK is marked."""
    rng = np.random.default_rng(21)
    stride, resident = 24576, 8192
    scores = (rng.standard_normal((6, stride)) * np.exp(rng.uniform(-2, 2, (6, 1)))).astype(np.float32)
    scores[1, :resident] -= 3.0                       # cold tokens dominate this row
    scores[2] = rng.integers(0, 4, stride)            # heavy ties around the threshold
    key_lengths = np.array([stride, stride, stride - 77, 9000, 4096, 1500], np.int32)   # the last two: no cold part
    ends = key_lengths.reshape(-1, 1).copy()
    prefix, thresholds, bitmap, counts = ops.cold_predicate(
        torch.from_numpy(scores).to(device), torch.from_numpy(key_lengths).to(device), torch.from_numpy(ends).to(device),
        resident)
    torch.cuda.synchronize()
    want_prefix, want_thresholds, want_bitmap, want_counts = oracle.cold_predicate(scores, key_lengths, ends, resident)
    assert np.array_equal(prefix.cpu().numpy(), want_prefix)
    assert np.array_equal(thresholds.cpu().numpy().view(np.uint32), want_thresholds)
    assert np.array_equal(bitmap.cpu().numpy().view(np.uint32), want_bitmap)
    assert np.array_equal(counts.cpu().numpy(), want_counts)
    final = oracle.topk(scores, key_lengths, ends)
    marked = np.unpackbits(want_bitmap.view(np.uint8), axis=1, bitorder="little").astype(bool)
    for row in range(6):
        cold = final[row][final[row] >= resident] - resident
        assert marked[row][cold].all()
    assert want_counts[4] == 0 and want_counts[5] == 0 and want_thresholds[5] == 0


def test_topk_merge_equals_unsharded(device):
    """Sequence sharding: per-shard top-2048 + merge == top-2048 of the whole row (canonical order)."""
    rng = np.random.default_rng(3)
    shards, per = 8, 16384
    whole = rng.integers(-50, 50, (2, shards * per)).astype(np.float32)  # many ties across shards
    whole[1] = rng.standard_normal(shards * per).astype(np.float32)
    expected = oracle_c.topk(whole, np.full(2, shards * per, np.int32), np.full(2, shards * per, np.int32))
    cand_scores = np.zeros((2, shards * TOPK), np.float32)
    cand_index = np.full((2, shards * TOPK), -1, np.int32)
    for s in range(shards):
        part = np.ascontiguousarray(whole[:, s * per:(s + 1) * per])
        local = oracle_c.topk(part, np.full(2, per, np.int32), np.full(2, per, np.int32), base_index=s * per)
        cand_index[:, s * TOPK:(s + 1) * TOPK] = local
        cand_scores[:, s * TOPK:(s + 1) * TOPK] = np.take_along_axis(whole, local, 1)
    assert np.array_equal(oracle.topk_merge(cand_scores, cand_index), expected)
    got = ops.topk_merge(torch.from_numpy(cand_scores).to(device), torch.from_numpy(cand_index).to(device))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), expected)
    # the same candidates in the layout an all-gather of per-rank [2, rows, 2048] blocks leaves: merged in place
    gathered = np.empty((shards, 2, 2, TOPK), np.int32)
    for s in range(shards):
        gathered[s, 0] = cand_scores[:, s * TOPK:(s + 1) * TOPK].view(np.int32)
        gathered[s, 1] = cand_index[:, s * TOPK:(s + 1) * TOPK]
    got = ops.topk_merge_gathered(torch.from_numpy(gathered).to(device))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), expected)
    # fewer shards (other candidate counts, odd ones included): the leading shards against the TopK of their keys
    for fewer in (2, 3, 4, 5):     # 2, 4 and 8 shards merge on a cluster of CTAs, the others on one CTA
        keys_here = fewer * per
        part = np.ascontiguousarray(whole[:, :keys_here])
        expected_part = oracle_c.topk(part, np.full(2, keys_here, np.int32), np.full(2, keys_here, np.int32))
        got = ops.topk_merge(torch.from_numpy(np.ascontiguousarray(cand_scores[:, :fewer * TOPK])).to(device),
                             torch.from_numpy(np.ascontiguousarray(cand_index[:, :fewer * TOPK])).to(device))
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), expected_part), fewer
    # one shard alone: its list is the answer and comes back unchanged (ties at the cut stay behind the rest)
    single = oracle_c.topk(whole[:, :per].copy(), np.full(2, per, np.int32), np.full(2, per, np.int32))
    got = ops.topk_merge(torch.from_numpy(np.take_along_axis(whole, single, 1)).to(device), torch.from_numpy(single).to(device))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), single)
    # a context shorter than 2048 keys spread over three shards: ascending positions, then -1
    short_index = np.full((1, 3 * TOPK), -1, np.int32)
    short_index[0, :700] = np.arange(700)
    short_index[0, TOPK:TOPK + 650] = 700 + np.arange(650)
    short_index[0, 2 * TOPK:2 * TOPK + 3] = 1350 + np.arange(3)
    short_scores = rng.standard_normal((1, 3 * TOPK)).astype(np.float32)
    got = ops.topk_merge(torch.from_numpy(short_scores).to(device), torch.from_numpy(short_index).to(device))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy()[0], np.concatenate((np.arange(1353), np.full(TOPK - 1353, -1))).astype(np.int32))
    assert np.array_equal(oracle.topk_merge(short_scores, short_index)[0], got.cpu().numpy()[0])
    # the same short context over four shards (the cluster kernel's way out without a cut), the last shard empty
    wide_index = np.full((1, 4 * TOPK), -1, np.int32)
    wide_index[0, :3 * TOPK] = short_index[0]
    wide_scores = rng.standard_normal((1, 4 * TOPK)).astype(np.float32)
    got = ops.topk_merge(torch.from_numpy(wide_scores).to(device), torch.from_numpy(wide_index).to(device))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy()[0], np.concatenate((np.arange(1353), np.full(TOPK - 1353, -1))).astype(np.int32))


RESOLVER_CASES = [
    dict(seed=0, batch=3, queries=4, history=16384, resident=8192, hot_fraction=0.5, overlap=0.5),
    dict(seed=1, batch=2, queries=1, history=16384, resident=2048, hot_fraction=0.0, overlap=0.0),   # all miss
    dict(seed=2, batch=2, queries=2, history=8192, resident=8192, hot_fraction=1.0, overlap=0.3),    # mostly hits
    dict(seed=3, batch=2, queries=4, history=32768, resident=16384, hot_fraction=0.3, overlap=0.5,
         lru_valid=1024),                                                                            # fallback scan
    dict(seed=4, batch=1, queries=4, history=32768, resident=2048, hot_fraction=0.0, overlap=0.0),   # no slots: error 4
]


def _resolve(case, device):
    batch, queries, history, resident = case["batch"], case["queries"], case["history"], case["resident"]
    rng = np.random.default_rng(99)
    logical = np.stack([rng.permutation(history) for _ in range(batch)]).astype(np.int64)
    addresses = (logical * 1152).astype(np.int64)
    state = ops.ResolveState(batch, queries, device)
    dev = {k: torch.from_numpy(v).to(device) for k, v in case.items() if isinstance(v, np.ndarray)}
    ops.resolve(dev["selected"], dev["hot_valid"], dev["reserved_hot"], dev["lru_slots"],
                torch.from_numpy(logical).to(device), torch.from_numpy(addresses).to(device), state,
                history=history, resident=resident)
    torch.cuda.synchronize()
    return state, logical, addresses


@pytest.mark.parametrize("spec", RESOLVER_CASES, ids=lambda s: f"seed{s['seed']}")
def test_resolver_matches_oracle(spec, device):
    case = workloads.resolver_case(**spec)
    state, logical, addresses = _resolve(case, device)
    resident, history = case["resident"], case["history"]
    for b in range(case["batch"]):
        ref = oracle.resolve_request(case["selected"][b], case["hot_valid"][b], case["reserved_hot"][b],
                                     case["lru_slots"][b], history, resident)
        status = state.row_status[b].cpu().numpy()
        assert int(status[0]) == ref["error"]
        counts = state.query_counts[b].cpu().numpy()
        assert list(counts[:4]) == ref["counts"] and int(counts[4]) == ref["total"]
        assert int(state.change_count[b]) == ref["change_count"]
        if ref["error"]:
            assert spec["seed"] == 4 and ref["error"] == oracle.ERR_NO_SLOT
            assert (state.slot_output.view(case["batch"], -1, TOPK)[b].cpu().numpy() == -1).all()
            continue
        n = ref["total"]
        assert np.array_equal(state.locations[b].cpu().numpy(), ref["locations"])
        assert np.array_equal(state.events_src[b, :n].cpu().numpy(), ref["events_src"])
        assert np.array_equal(state.events_dst[b, :n].cpu().numpy(), ref["events_dst"])
        assert np.array_equal(state.changes[b].cpu().numpy(), ref["changes"])
        assert np.array_equal(state.change_slots[b].cpu().numpy(), ref["change_slots"])
        assert np.array_equal(state.fetch_sources[b, :n].cpu().numpy(), addresses[b][ref["events_src"]])
        assert np.array_equal(state.fetch_destinations[b, :n].cpu().numpy(), b * resident + ref["events_dst"])
        posts = state.final_posts.view(case["batch"], 4, 32)[b].cpu().numpy().view(np.uint32)
        expected_posts = oracle.resolve_request(case["selected"][b], case["hot_valid"][b], case["reserved_hot"][b],
                                                case["lru_slots"][b], history, resident, request=b)["final_posts"]
        assert np.array_equal(posts, expected_posts), "final posts (count, first descriptor, error) differ"
        q = case["queries"]
        assert np.array_equal(state.slot_output.view(-1, q, TOPK)[b].cpu().numpy(), ref["locations"])
        assert np.array_equal(state.logical_output.view(-1, q, TOPK)[b].cpu().numpy(),
                              logical[b][case["selected"][b]].astype(np.int32))
        # the reference's invariants (execution.py:2102-2131): slots in range, one slot per token
        loc, sel = ref["locations"].reshape(-1), case["selected"][b].reshape(-1)
        assert loc.min() >= 0 and loc.max() < resident
        pairs = set(zip(sel.tolist(), loc.tolist()))
        assert len(pairs) == len(set(sel.tolist())) == len({s for _, s in pairs})
    if spec["seed"] == 3:
        assert (state.events_dst[0, : int(state.query_counts[0, 4])].cpu().numpy()[:, None]
                != case["lru_slots"][0][None, :]).all(1).any(), "fallback slots were not exercised"


def test_resolver_padding_rows_and_range_error(device):
    case = workloads.resolver_case(seed=7, batch=2, queries=4, history=8192, resident=4096)
    case["selected"][0, 2:] = -1            # inactive query rows
    case["selected"][0, 1, 1000:] = -1      # short row
    case["selected"][1, 0, 5] = 8192        # out of range -> error 1
    state, _, _ = _resolve(case, device)
    ref = oracle.resolve_request(case["selected"][0], case["hot_valid"][0], case["reserved_hot"][0],
                                 case["lru_slots"][0], 8192, 4096)
    assert np.array_equal(state.locations[0].cpu().numpy(), ref["locations"])
    assert (state.locations[0, 2:].cpu().numpy() == -1).all()
    assert int(state.row_status[1, 0]) == oracle.ERR_TOKEN_RANGE
    assert int(state.query_counts[1, 4]) == 0


def test_resolver_abc_tail_matches_oracle(device):
    """ABC tail (reference cache_metadata.h:22-26, 100-105; prefetch.h:26-44): positions [begin, end) of a request
    live in the ring of output_stride - resident dedicated slots. They are never hot by position, never misses and
    never victims; their location is resident + p % ring while the ring holds them, and a tail position beyond
    the ring is resolved like a cold one. Bit-exact against the restatement, plus the properties themselves."""
    batch, queries, history, resident, ring = 3, 4, 16384, 8192, 512
    case = workloads.resolver_case(seed=21, batch=batch, queries=queries, history=history, resident=resident)
    rng = np.random.default_rng(5)
    # request 0: tail of 300 cold positions; request 1: a tail that reaches below `resident` and is longer than the
    # ring; request 2: empty tail. Every request selects some tail positions in every query.
    bounds = np.array([[9000, 9300], [7900, 8700], [12000, 12000]], dtype=np.int32)
    for b in range(batch):
        lo, hi = bounds[b]
        if hi > lo:
            for q in range(queries):
                row = case["selected"][b, q]
                tail = rng.choice(np.arange(lo, hi), 64, replace=False)
                fresh = tail[~np.isin(tail, row)]
                row[rng.choice(TOPK, len(fresh), replace=False)] = fresh
    logical = np.stack([np.arange(history) for _ in range(batch)]).astype(np.int64)
    addresses = logical * 1152
    state = ops.ResolveState(batch, queries, device)
    dev = {k: torch.from_numpy(v).to(device) for k, v in case.items() if isinstance(v, np.ndarray)}
    ops.resolve(dev["selected"], dev["hot_valid"], dev["reserved_hot"], dev["lru_slots"], torch.from_numpy(logical).to(device),
                torch.from_numpy(addresses).to(device), state, history=history, resident=resident,
                output_stride=resident + ring, tail_bounds=torch.from_numpy(bounds).to(device))
    torch.cuda.synchronize()
    for b in range(batch):
        ref = oracle.resolve_request(case["selected"][b], case["hot_valid"][b], case["reserved_hot"][b],
                                     case["lru_slots"][b], history, resident, tail_bounds=bounds[b],
                                     output_stride=resident + ring, request=b)
        assert ref["error"] == 0 and int(state.row_status[b, 0]) == 0
        loc = state.locations[b].cpu().numpy()
        n = ref["total"]
        assert np.array_equal(loc, ref["locations"])
        assert np.array_equal(state.events_src[b, :n].cpu().numpy(), ref["events_src"])
        assert np.array_equal(state.events_dst[b, :n].cpu().numpy(), ref["events_dst"])
        assert np.array_equal(state.final_posts.view(batch, 4, 32)[b].cpu().numpy().view(np.uint32), ref["final_posts"])
        sel = case["selected"][b]
        lo, hi = bounds[b]
        in_ring = (sel >= lo) & (sel < hi) & (sel - lo < ring)
        assert np.array_equal(loc[in_ring], resident + sel[in_ring] % ring)
        assert (loc[~in_ring] < resident).all() and (loc[~in_ring] >= 0).all()
        events = set(ref["events_src"].tolist())
        assert not events & set(sel[in_ring].tolist()), "a ring position must not be fetched"
        assert (ref["events_dst"] < resident).all(), "ring slots are never victims"
        if b == 1:  # tail positions below `resident` are not hot hits even where hot_valid says so
            low = in_ring & (sel < resident)
            assert low.any() and (loc[low] >= resident).all()
            beyond = (sel >= lo + ring) & (sel < hi)
            assert beyond.any() and (loc[beyond] < resident).all(), "beyond the ring: resolved like a cold position"
    with pytest.raises(ValueError):  # fewer than 384 dedicated slots (reference binding.py:163-164)
        ops.resolve(dev["selected"], dev["hot_valid"], dev["reserved_hot"], dev["lru_slots"], torch.from_numpy(logical).to(device),
                    torch.from_numpy(addresses).to(device), state, history=history, resident=resident,
                    output_stride=resident + 256, tail_bounds=torch.from_numpy(bounds).to(device))


def test_resolver_rejects_a_source_outside_the_pool(device):
    """A missing row whose source address lies outside the miss source fails its request in the resolver, before
    any Index row moves (the reference range-checks the same descriptors, streaming.cpp:399-400): status
    KVIP_ERR_SOURCE, no descriptors, outputs -1; the other request is untouched."""
    case = workloads.resolver_case(seed=31, batch=2, queries=2, history=8192, resident=4096)
    history, resident = 8192, 4096
    logical = np.stack([np.arange(history) for _ in range(2)]).astype(np.int64)
    addresses = logical * 1152
    cold = case["selected"][1][case["selected"][1] >= resident][0]
    addresses[1, cold] = history * 1152          # one row past the end of the source
    state = ops.ResolveState(2, 2, device)
    dev = {k: torch.from_numpy(v).to(device) for k, v in case.items() if isinstance(v, np.ndarray)}
    ops.resolve(dev["selected"], dev["hot_valid"], dev["reserved_hot"], dev["lru_slots"], torch.from_numpy(logical).to(device),
                torch.from_numpy(addresses).to(device), state, history=history, resident=resident,
                source_bytes=history * 1152, token_bytes=1152)
    torch.cuda.synchronize()
    for b in range(2):
        ref = oracle.resolve_request(case["selected"][b], case["hot_valid"][b], case["reserved_hot"][b],
                                     case["lru_slots"][b], history, resident, addresses=addresses[b],
                                     source_bytes=history * 1152, token_bytes=1152, request=b)
        assert int(state.row_status[b, 0]) == ref["error"] == (oracle.ERR_SOURCE if b == 1 else 0)
        assert int(state.query_counts[b, 4]) == ref["total"]
        assert np.array_equal(state.final_posts.view(2, 4, 32)[b].cpu().numpy().view(np.uint32), ref["final_posts"])
    assert (state.slot_output.view(2, 2, TOPK)[1].cpu().numpy() == -1).all()
    assert np.array_equal(state.locations[0].cpu().numpy(),
                          oracle.resolve_request(case["selected"][0], case["hot_valid"][0], case["reserved_hot"][0],
                                                 case["lru_slots"][0], history, resident)["locations"])


def test_fetch_bad_descriptor_revokes_residency(device):
    """A descriptor that fails the fetch's own range check is skipped, and its destination slot must not keep the
    residency of the row it evicted (the Index row of the new token already sits there): hot_valid of the slot is
    cleared, row_status[2] is set and the update status gets code 4 (reference CompleteEarlyUpdate,
    index_cache_update.h:6-20). The other descriptors of the request still land."""
    batch, resident, token_bytes, rows = 2, 4096, 1152, 32
    state = ops.ResolveState(batch, 1, device)
    source = torch.from_numpy(workloads.payload(0, np.arange(256), token_bytes)).to(device)
    pool = torch.zeros((batch * resident, token_bytes), dtype=torch.uint8, device=device)
    hot_valid = torch.ones((batch, resident), dtype=torch.int32, device=device)
    status = torch.zeros(batch, dtype=torch.int32, device=device)
    tokens = torch.arange(rows, device=device)
    for b in range(batch):
        state.fetch_sources[b, :rows] = (tokens + 10 * b) * token_bytes
        state.fetch_destinations[b, :rows] = (b * resident + 100 + tokens).int()
        state.query_counts[b, 4] = rows
    state.fetch_sources[1, 7] = 256 * token_bytes     # one row past the end of the source
    ops.fetch(source, source.numel(), pool, hot_valid, state, resident=resident, output_stride=resident,
              token_bytes=token_bytes, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 4] and int(state.row_status[1, 2]) == 1 and int(state.row_status[0, 2]) == 0
    valid = hot_valid.cpu().numpy()
    assert valid[1, 107] == 0 and valid[1].sum() == resident - 1 and valid[0].all()
    got = pool.cpu().numpy()
    for b in range(batch):
        for i in range(rows):
            expected = np.zeros(token_bytes, np.uint8) if (b, i) == (1, 7) else workloads.payload(0, [i + 10 * b], token_bytes)[0]
            assert np.array_equal(got[b * resident + 100 + i], expected), (b, i)


def _index_state(batch, history, resident, seed, bf16=False):
    rng = np.random.default_rng(seed)
    if bf16:
        keys = rng.integers(0, 2**16, (batch, history, 128), dtype=np.uint16)
    else:
        keys = rng.integers(0, 256, (batch, history, 128), dtype=np.uint8)
    scales = rng.random((batch, history), dtype=np.float32)
    logical = np.stack([rng.permutation(history) for _ in range(batch)]).astype(np.int64)
    addresses = logical * 1152 + 7 * 1152
    hot_valid = np.ones((batch, resident), dtype=np.int32)
    return keys, scales, addresses, logical, hot_valid


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("spec", RESOLVER_CASES[:4], ids=lambda s: f"seed{s['seed']}")
def test_exchange_matches_oracle(spec, bf16, device):
    case = workloads.resolver_case(**spec)
    batch, queries, history, resident = case["batch"], case["queries"], case["history"], case["resident"]
    keys, scales, addresses, logical, _ = _index_state(batch, history, resident, 5, bf16)
    hot_valid = case["hot_valid"].copy()
    state = ops.ResolveState(batch, queries, device)
    dev = {k: torch.from_numpy(v).to(device) for k, v in case.items() if isinstance(v, np.ndarray)}
    keys_t = torch.from_numpy(keys.view(np.int16) if bf16 else keys).to(device)
    scales_t, addr_t, logical_t = (torch.from_numpy(x).to(device) for x in (scales, addresses, logical))
    valid_t = torch.from_numpy(hot_valid).to(device)
    ops.resolve(dev["selected"], valid_t, dev["reserved_hot"], dev["lru_slots"], logical_t, addr_t, state,
                history=history, resident=resident)
    shadow = ops.make_shadow(batch, history, device)
    status = torch.zeros(batch, dtype=torch.int32, device=device)
    ops.exchange(keys_t, scales_t, addr_t, logical_t, valid_t, state, shadow, status, history=history,
                 resident=resident, queries=queries)
    torch.cuda.synchronize()
    assert (status.cpu().numpy() == 0).all()
    assert torch.equal(shadow, ops.make_shadow(batch, history, device)), "row/position maps not restored"
    seed_keys, seed_scales, seed_addr = keys.copy(), scales.copy(), addresses.copy()
    for b in range(batch):
        ref = oracle.resolve_request(case["selected"][b], hot_valid[b], case["reserved_hot"][b], case["lru_slots"][b],
                                     history, resident)
        valid_ref = hot_valid[b].copy()
        err = oracle.exchange_request(keys[b], scales[b], addresses[b], logical[b], valid_ref, ref["events_src"],
                                      ref["events_dst"], ref["counts"], history, resident)
        assert err == 0
        got_keys = keys_t[b].cpu().numpy()
        assert np.array_equal(got_keys.view(keys.dtype), keys[b])
        assert np.array_equal(scales_t[b].cpu().numpy(), scales[b])
        assert np.array_equal(addr_t[b].cpu().numpy(), addresses[b])
        assert np.array_equal(logical_t[b].cpu().numpy(), logical[b])
        assert np.array_equal(valid_t[b].cpu().numpy(), valid_ref)
        # the reference's invariant (execution.py:2216-2224, 2773-2778): rows stay a joint permutation and
        # every selected token now sits at the position equal to its slot
        ids = logical[b]
        assert np.array_equal(np.sort(ids), np.arange(history))
        inverse_seed = np.empty(history, np.int64)
        rng_logical = np.stack([np.random.default_rng(5).permutation(history)])  # noqa: F841 (documented seed)
        first_ids = (seed_addr[b] - 7 * 1152) // 1152
        inverse_seed[first_ids] = np.arange(history)
        assert np.array_equal(keys[b], seed_keys[b][inverse_seed[ids]])
        assert np.array_equal(scales[b], seed_scales[b][inverse_seed[ids]])
        assert np.array_equal(addresses[b], ids * 1152 + 7 * 1152)
        loc, sel = ref["locations"].reshape(-1), case["selected"][b].reshape(-1)
        assert np.array_equal(ids[loc], first_ids[sel])


def test_exchange_rejects_bad_events(device):
    batch, queries, history, resident = 1, 1, 4096, 2048
    keys, scales, addresses, logical, hot_valid = _index_state(batch, history, resident, 6)
    state = ops.ResolveState(batch, queries, device)
    state.events_src[0, :2] = torch.tensor([3000, 3001], dtype=torch.int32)
    state.events_dst[0, :2] = torch.tensor([5, 5], dtype=torch.int32)   # duplicate destination
    state.query_counts[0, 0] = 2
    t = [torch.from_numpy(x).to(device) for x in (keys, scales, addresses, logical, hot_valid)]
    status = torch.zeros(batch, dtype=torch.int32, device=device)
    shadow = ops.make_shadow(batch, history, device)
    ops.exchange(*t, state, shadow, status, history=history, resident=resident, queries=queries)
    torch.cuda.synchronize()
    assert int(status[0]) == 1
    assert (t[4].cpu().numpy() == 0).all(), "a failed owner must lose hot residency"
    assert np.array_equal(t[0].cpu().numpy(), keys), "rows must not move on a rejected plan"
    assert torch.equal(shadow, ops.make_shadow(batch, history, device))


@pytest.mark.parametrize("token_bytes", [1152, 656, 2624])
def test_fetch_and_gather_bytes(token_bytes, device):
    """Fetched bytes == payload(token) for every descriptor, hot_valid published, gather returns the rows of
    the selected slots (the byte-equality checks of execution.py:2122-2131)."""
    case = workloads.resolver_case(seed=11, batch=3, queries=2, history=8192, resident=4096, hot_fraction=0.4)
    batch, queries, history, resident = 3, 2, 8192, 4096
    stride = resident + 384
    host = np.concatenate([workloads.payload(b, np.arange(history), token_bytes) for b in range(batch)])
    addresses = (np.arange(batch * history, dtype=np.int64).reshape(batch, history)) * token_bytes
    logical = np.broadcast_to(np.arange(history, dtype=np.int64), (batch, history)).copy()
    pool = np.zeros((batch * stride, token_bytes), np.uint8)
    for b in range(batch):   # hot slots hold their own token (identity layout at round start)
        pool[b * stride: b * stride + resident] = workloads.payload(b, np.arange(resident), token_bytes)
    state = ops.ResolveState(batch, queries, device)
    dev = {k: torch.from_numpy(v).to(device) for k, v in case.items() if isinstance(v, np.ndarray)}
    pool_t, source_t = torch.from_numpy(pool).to(device), torch.from_numpy(host.reshape(-1)).to(device)
    valid_t = dev["hot_valid"].clone()
    ops.resolve(dev["selected"], valid_t, dev["reserved_hot"], dev["lru_slots"], torch.from_numpy(logical).to(device),
                torch.from_numpy(addresses).to(device), state, history=history, resident=resident,
                output_stride=stride)
    ops.fetch(source_t, host.size, pool_t, valid_t, state, resident=resident, output_stride=stride,
              token_bytes=token_bytes)
    out = ops.gather(pool_t, state.slot_output, queries=queries, output_stride=stride, token_bytes=token_bytes)
    torch.cuda.synchronize()
    got_pool, got_valid, got_out = pool_t.cpu().numpy(), valid_t.cpu().numpy(), out.cpu().numpy()
    for b in range(batch):
        ref = oracle.resolve_request(case["selected"][b], case["hot_valid"][b], case["reserved_hot"][b],
                                     case["lru_slots"][b], history, resident)
        valid_ref = case["hot_valid"][b].copy()
        oracle.fetch_request(pool, valid_ref, host.reshape(-1), addresses[b][ref["events_src"]],
                             b * stride + ref["events_dst"], b, stride, resident, token_bytes)
        assert np.array_equal(got_valid[b], valid_ref)
        assert int(state.row_status[b, 2]) == 0
        for q in range(queries):
            expect = workloads.payload(b, case["selected"][b, q], token_bytes)
            hit_or_fetched = (ref["locations"][q] >= 0)
            assert hit_or_fetched.all()
            assert np.array_equal(got_out[b * queries + q], expect)
    assert np.array_equal(got_pool, pool)
    assert np.array_equal(got_out, oracle.gather(pool, state.slot_output.cpu().numpy(), np.arange(batch), queries, stride))


def test_fetch_rejects_out_of_window_source(device):
    batch, queries, resident = 1, 1, 2048
    state = ops.ResolveState(batch, queries, device)
    state.fetch_sources[0, :3] = torch.tensor([0, 1152 * 10, 1152 * 100], dtype=torch.int64)  # the last is outside
    state.fetch_destinations[0, :3] = torch.tensor([0, 1, 2], dtype=torch.int32)
    state.query_counts[0, 4] = 3
    source = torch.arange(1152 * 50, dtype=torch.int32, device=device).to(torch.uint8)
    pool = torch.zeros((resident, 1152), dtype=torch.uint8, device=device)
    valid = torch.zeros((1, resident), dtype=torch.int32, device=device)
    ops.fetch(source, source.numel(), pool, valid, state, resident=resident, output_stride=resident, token_bytes=1152)
    torch.cuda.synchronize()
    assert int(state.row_status[0, 2]) == 1 and valid[0, :3].tolist() == [1, 1, 0]
    assert torch.equal(pool[1], source[1152 * 10: 1152 * 11]) and int(pool[2].sum()) == 0


def test_gather_negative_slots_are_zero_rows(device):
    pool = torch.randint(0, 255, (4096, 1152), dtype=torch.uint8, device=device)
    slots = torch.randint(0, 4096, (2, TOPK), dtype=torch.int32, device=device)
    slots[0, ::3] = -1
    out = ops.gather(pool, slots, queries=1, output_stride=2048, token_bytes=1152)
    torch.cuda.synchronize()
    ref = oracle.gather(pool.cpu().numpy(), slots.cpu().numpy(), np.arange(2), 1, 2048)
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("bf16_source", [False, True])
def test_ingest_decode(bf16_source, device):
    rng = np.random.default_rng(4)
    batch, queries, history, owners, source_rows = 5, 4, 1024, 8, 4096
    keys = rng.integers(0, 256, (owners, history, 128), dtype=np.uint8)
    scales = rng.random((owners, history), dtype=np.float32)
    if bf16_source:
        src = oracle.f32_to_bf16_rne(rng.standard_normal((source_rows, 128)).astype(np.float32) * 3)
        src[17] = 0  # an all-zero row quantises with scale 1
        src_scales = None
    else:
        src = rng.integers(0, 256, (source_rows, 128), dtype=np.uint8)
        src_scales = rng.random(source_rows, dtype=np.float32)
    tokens = 13
    slot_mapping = rng.permutation(source_rows)[:tokens].astype(np.int64)
    slot_mapping[3] = 17
    gather_idx = rng.integers(0, tokens, batch * queries).astype(np.int64)
    gather_idx[0] = 3
    query_ends = rng.integers(1, history, (batch, queries)).astype(np.int32)
    query_ends[1, 2:] = 0
    query_ends[4, :] = 0
    owners_row = rng.permutation(np.arange(1, owners))[:batch].astype(np.int32)
    keys_t, scales_t = torch.from_numpy(keys).to(device), torch.from_numpy(scales).to(device)
    src_t = torch.from_numpy(src.view(np.int16) if bf16_source else src).to(device)
    if bf16_source:
        src_t = src_t.view(torch.bfloat16)
    ops.ingest(keys_t, scales_t, src_t, None if src_scales is None else torch.from_numpy(src_scales).to(device),
               torch.from_numpy(slot_mapping).to(device), torch.from_numpy(gather_idx).to(device),
               torch.from_numpy(query_ends.reshape(-1)).to(device), torch.from_numpy(owners_row).to(device),
               queries=queries, history=history)
    torch.cuda.synchronize()
    oracle.ingest_decode(keys, scales, src, src_scales, slot_mapping, gather_idx, query_ends.reshape(-1), owners_row,
                         queries, history, source_is_bf16=bf16_source)
    assert np.array_equal(keys_t.cpu().numpy(), keys)
    assert np.array_equal(scales_t.cpu().numpy().view(np.uint32), scales.view(np.uint32))


@pytest.mark.gpu
def test_maximum_history_scores_and_topk(device):
    """The largest history the shape check admits (2^21 keys in one request, random block table): tensor-core scores
    against the CUDA-core cross-check kernel, then the TopK of those scores against the C oracle, bit for bit."""
    history, heads, short = 1 << 21, 64, 77
    g = torch.Generator(device=device)
    g.manual_seed(3)
    keys = (torch.randn((history, 128), generator=g, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
    key_scale = torch.exp(torch.rand((history,), generator=g, device=device) * 4.6052 - 6.9078)
    query = (torch.randn((1, heads, 128), generator=g, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
    query_scale = torch.exp(torch.rand((1, heads), generator=g, device=device) * 4.6052 - 6.9078)
    weights = (torch.randn((1, heads), generator=g, device=device) / 8).to(torch.bfloat16)
    lengths = torch.full((1,), history - short, dtype=torch.int32, device=device)
    ends = torch.full((1, 1), history - short, dtype=torch.int32, device=device)
    table = torch.randperm(history // 128, generator=g, device=device).to(torch.int32).view(1, -1).contiguous()
    scores, status = ops.li_score(query, keys, weights, query_scale, key_scale, lengths, ends, table)
    check, _ = ops.li_score(query, keys, weights, query_scale, key_scale, lengths, ends, table, simt=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got, want = scores[0, :history - short].cpu().numpy(), check[0, :history - short].cpu().numpy()
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()
    top = ops.topk(scores, lengths, ends)
    torch.cuda.synchronize()
    host_scores = scores.cpu().numpy()
    expected = oracle_c.topk(host_scores, lengths.cpu().numpy(), ends.cpu().numpy().reshape(-1))
    assert np.array_equal(top.cpu().numpy(), expected)
    assert top.max().item() < history - short   # nothing beyond the valid length
