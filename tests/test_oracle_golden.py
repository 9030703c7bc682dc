"""CPU: the oracle against the golden vectors produced by the reference's own code, so that the
checker the GPU parity tests rely on is itself pinned."""
import numpy as np
import pytest

import kvip_oracle as oracle
import oracle_c
import workloads
from golden_cases import GOLDEN, li_fixture_case

TOPK = 2048


def _bf16_bits(scores):
    return (oracle.bf16_away(scores).view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("name", ["li_exact_fixture.npz", "li_exact_causal_fixture.npz", "li_full_chain_fixture.npz"])
def test_li_score_matches_reference_fixture_bits(name):
    """prepare_fixture / prepare_full_chain_fixture (reference workloads.py:196-283, 975-1076) publish the
    expected score of every token as bf16 bits, rounded ties-away. Exact binary fractions: must match bit
    for bit, with both the NumPy and the C restatement."""
    case, expected, data = li_fixture_case(name)
    history = int(data["history"])
    for exact in (False, True):
        scores = workloads.oracle_scores(case, score_mode=1, exact=exact)
        for q in range(case["queries"]):
            visible = int(case["query_ends"][0, q])
            n = min(visible, expected.shape[1])
            assert np.array_equal(_bf16_bits(scores[q, :n]), expected[q, :n]), (name, q, exact)
    assert history % 256 == 0


def test_topk_on_unique_cutoff_fixture_is_the_reference_set():
    """prepare_full_chain_fixture guarantees exactly 2048 scores at or above the cutoff
    (workloads.py:1049-1051), so the selected SET is pinned (execution.py:1833-1836)."""
    case, expected, _ = li_fixture_case("li_full_chain_fixture.npz")
    scores = workloads.oracle_scores(case, score_mode=1)
    got = oracle.topk(scores, case["key_lengths"], case["query_ends"])
    assert np.array_equal(got, oracle_c.topk(scores, case["key_lengths"], case["query_ends"]))
    for q in range(4):
        bits = expected[q]
        cutoff = np.partition(bits, -TOPK)[-TOPK]
        want = np.flatnonzero(bits >= cutoff)
        assert len(want) == TOPK
        assert np.array_equal(np.sort(got[q]), want)
    oracle.validate_topk(got, scores[:, : expected.shape[1]])


def test_li_score_matches_reference_compact_golden():
    """prepare_compact_fixture (workloads.py:399-457) stores scores = bf16(golden einsum formula) for the
    calibrated generator. Accumulation order differs between two fp32 einsums, so equality is required up
    to one bf16 spacing, and the reference's own validity oracle must accept the oracle's TopK."""
    case, expected, _ = li_fixture_case("li_compact_fixture.npz")
    scores = workloads.oracle_scores(case)
    rounded = oracle.bf16_to_f32(oracle.f32_to_bf16_rne(scores[:, : expected.shape[1]]))
    spacing = np.maximum(np.abs(expected), np.finfo(np.float32).tiny) * 2.0**-7
    assert (np.abs(rounded - expected) <= spacing).all()
    assert (rounded == expected).mean() > 0.995
    got = oracle.topk(oracle.bf16_away(scores), case["key_lengths"], case["query_ends"])
    oracle.validate_topk(got, expected)


def test_topk_short_rows_and_padding():
    scores = np.random.default_rng(0).standard_normal((4, 4096)).astype(np.float32)
    got = oracle.topk(scores, np.array([4096, 100, 0, 2048], np.int32), np.array([4096, 4096, 5, 4096], np.int32))
    assert np.array_equal(got[1, :100], np.arange(100)) and (got[1, 100:] == -1).all()
    assert (got[2] == -1).all() and np.array_equal(got[3], np.arange(2048))
    assert np.array_equal(got, oracle_c.topk(scores, np.array([4096, 100, 0, 2048], np.int32),
                                             np.array([4096, 4096, 5, 4096], np.int32)))


def test_slot_lru_matches_reference_trace():
    """The ordered-array LRU against the reference's numba linked list (python/kvip/cache/lru.py,
    _lru_kernel.py) replayed by make_golden.py: same victims, same full order, same unique counts."""
    data = np.load(GOLDEN / "slot_lru_trace.npz")
    lru = oracle.SlotLRUOracle()
    for i in range(int(data["steps"])):
        op = bytes(data[f"s{i}_op"]).decode()
        capacity, committed, _version, active, unique = (int(x) for x in data[f"s{i}_args"])
        if op == "resize":
            lru.resize(capacity, committed)
        else:
            count = lru.commit(data[f"s{i}_touched"])
            assert count == unique
        assert lru.active == active
        assert np.array_equal(lru.order, data[f"s{i}_order"]), (i, op)
        assert np.array_equal(lru.slots, data[f"s{i}_slots"]), (i, op)


def test_abc_matches_reference():
    data = np.load(GOLDEN / "abc_maps.npz")
    t2s = np.full((3, 5, 2048), 99, np.int32)
    s2t = t2s.copy()
    for stage in (0, 1):
        oracle.update_abc(t2s, s2t, data[f"d{stage}"], 2, 1024, 384)
        assert np.array_equal(t2s, data[f"t{stage}"]) and np.array_equal(s2t, data[f"s{stage}"])


def test_publish_pages_matches_reference():
    """Two submits recorded from the reference's PageUpdates (python/kvip/cache/page_updates.py, CPU branch)."""
    data = np.load(GOLDEN / "page_updates.npz")
    owners, groups, pages, block = (int(x) for x in data["shape"])
    addresses = np.zeros((owners, groups, pages), np.int64)
    valid = np.zeros((owners, groups, pages), np.int32)
    token_to_slot = data["map0"].copy()
    fused = [np.full((owners, pages * block), -7, np.int64) for _ in range(groups)]
    for ring in (0, 1):
        oracle.publish_pages(data[f"rows{ring}"], addresses, valid, token_to_slot, fused, (1, 4), 656, block)
        assert np.array_equal(addresses, data[f"addresses{ring}"]) and np.array_equal(valid, data[f"valid{ring}"])
        assert np.array_equal(token_to_slot, data[f"map{ring + 1}"])
        assert all(np.array_equal(fused[g], data[f"fused{ring}_{g}"]) for g in range(groups))


def test_ingest_decode_matches_reference():
    """VllmIndexCacheStorage.ingest_decode (python/kvip/adapters/vllm/index_import.py:38-52) on CPU torch."""
    d = np.load(GOLDEN / "ingest_decode.npz")
    keys, scales = d["before_keys"].copy(), d["before_scales"].copy()
    gather, ends = d["metadata"][0], d["query_ends"]
    oracle.ingest_decode(keys, scales, d["cache_keys"].reshape(-1, 128), d["cache_scales"].reshape(-1),
                         d["slot_mapping"], gather, ends, d["owners"].astype(np.int32), 4, keys.shape[1])
    assert np.array_equal(keys, d["after_keys"]) and np.array_equal(scales, d["after_scales"])


def test_hot_slot_scan_matches_reference_header():
    """free-slot ring scan against the reference's hot_slot_selection.h compiled by oracle/Makefile (cases of
    tests/operators/lidu/test_hot_slot_selection.py:43-51)."""
    d = np.load(GOLDEN / "hot_slot_scan.npz")
    for i in range(int(d["cases"])):
        budget, begin, n = (int(x) for x in d[f"c{i}_args"])
        got, free = oracle.free_slots_ring(d[f"c{i}_words"], budget, begin, n)
        assert np.array_equal(got, d[f"c{i}_slots"]), (budget, begin)
        assert free >= n


def test_stateful_bands_select_and_evict():
    """The reference's stateful case (correctness.py:170-228): three 2048-token key bands, queries A/A/B+C/A;
    reads per request must be [2048, 0, 4096, 2048] and B+C must evict A."""
    history, resident, heads = 12288, 4096, 32
    keys = np.zeros((history, 128), np.uint8)
    for feature, begin in enumerate((4096, 6144, 8192)):
        keys[begin:begin + 2048, feature] = 0x38
    hot_valid = np.ones(resident, np.int32)
    logical = np.arange(history, dtype=np.int64)
    scales = np.ones(history, np.float32)
    addresses = logical * 656
    lru = oracle.SlotLRUOracle()
    lru.resize(resident, resident)
    reads = []
    for number in range(1, 5):
        features = (1, 2, 1, 2) if number == 3 else (0, 0, 0, 0)
        query = np.zeros((4, heads, 128), np.uint8)
        for q, feature in enumerate(features):
            query[q, :, feature] = 0x38
        case = dict(query=query, keys=keys, weights=np.ones((4, heads), np.float32), query_scale=None,
                    key_scale=scales, key_lengths=np.array([history], np.int32),
                    query_ends=np.arange(history - 3, history + 1, dtype=np.int32).reshape(1, 4),
                    block_table=np.arange(history // 128, dtype=np.int32).reshape(1, -1), heads=heads, queries=4,
                    batch=1, history=history, key_dtype="fp8", weight_dtype="fp32")
        scores = workloads.oracle_scores(case, score_mode=1)
        selected = oracle.topk(scores, case["key_lengths"], case["query_ends"])
        expected_ids = set(range(6144, 10240)) if number == 3 else set(range(4096, 6144))
        assert set(logical[selected.reshape(-1)].tolist()) == expected_ids
        ref = oracle.resolve_request(selected, hot_valid, lru.reserved_hot(resident), lru.slots, history, resident)
        assert ref["error"] == 0
        reads.append(ref["total"])
        for d in ref["events_dst"]:
            hot_valid[d] = 1
        assert oracle.exchange_request(keys, scales, addresses, logical, hot_valid, ref["events_src"],
                                       ref["events_dst"], ref["counts"], history, resident) == 0
        lru.commit(ref["locations"].reshape(-1))
        hot_ids = set(logical[:resident][hot_valid[:resident] != 0].tolist())
        assert expected_ids <= hot_ids
        if number == 3:
            assert not hot_ids & set(range(4096, 6144)), "B/C failed to evict A"
        assert np.array_equal(np.sort(logical), np.arange(history))
    assert reads == [2048, 0, 4096, 2048]
