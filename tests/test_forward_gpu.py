"""End-to-end parity of `kvip_b200.LIFetch` (one C call per step) with the oracle chain, on the
benchmark's CPU-golden configuration and on FP8/MTP variants, plus CUDA-graph replay (B200 only)."""
import numpy as np
import pytest
import torch

import kvip_oracle as oracle
import oracle_c
from kvip_b200 import _lib
from decode_harness import DecodePipeline, payload_rows

pytestmark = pytest.mark.gpu
TOPK = 2048


def snapshot(p):
    s = p.storage
    keys = s.keys.view(torch.int16) if s.keys.dtype == torch.bfloat16 else s.keys
    return dict(
        keys=keys.cpu().numpy().copy(), scales=s.scales.cpu().numpy().copy(),
        addresses=s.addresses.cpu().numpy().copy(), logical=s.logical_ids.cpu().numpy().copy(),
        hot_valid=s.hot_valid.cpu().numpy().copy(), pool=p.pool_hbm.cpu().numpy().copy(),
        lru_slots=p.rotating.lru_slots.cpu().numpy().copy(), reserved=p.rotating.reserved_hot.cpu().numpy().copy(),
        order=p.lru.order.cpu().numpy().copy())


def oracle_step(p, before, scores):
    """The whole step on the CPU, from the device's own fp32 scores (so that everything downstream of
    the LI tolerance is compared bit for bit)."""
    batch, queries, history, resident = p.batch, p.queries, p.history, p.resident
    key_lengths = p.workspace.key_lengths.cpu().numpy()
    query_ends = p.workspace.inputs.query_ends.cpu().numpy()
    owners = p.workspace.inputs.row_owners.cpu().numpy()
    topk = oracle_c.topk(scores, key_lengths, query_ends).reshape(batch, queries, TOPK)
    state = {k: v.copy() for k, v in before.items()}
    host = p.host_pool.flat.numpy() if p.host_pool is not None else p.source.cpu().numpy().reshape(-1)
    logical_out = np.full((batch * queries, TOPK), -1, np.int32)
    slot_out = np.full((batch * queries, TOPK), -1, np.int32)
    reads, posts = [], []
    for b in range(batch):
        owner = int(owners[b])
        tail = None if p.tail_bounds is None else p.tail_bounds[b].cpu().numpy()
        ref = oracle.resolve_request(topk[b], state["hot_valid"][owner], state["reserved"][b], state["lru_slots"][b],
                                     history, resident, tail_bounds=tail, output_stride=p.output_stride, request=b)
        assert ref["error"] == 0
        posts.append(ref["final_posts"])
        for q in range(queries):
            live = topk[b, q] >= 0
            logical_out[b * queries + q, live] = state["logical"][owner][topk[b, q][live]]
            slot_out[b * queries + q] = ref["locations"][q]
        sources = state["addresses"][owner][ref["events_src"]]
        err = oracle.exchange_request(state["keys"][owner], state["scales"][owner], state["addresses"][owner],
                                      state["logical"][owner], state["hot_valid"][owner], ref["events_src"],
                                      ref["events_dst"], ref["counts"], history, resident)
        assert err == 0
        oracle.fetch_request(state["pool"], state["hot_valid"][owner], host, sources,
                             owner * p.output_stride + ref["events_dst"], owner, p.output_stride, resident,
                             p.token_bytes)
        reads.append(ref["total"])
    state["final_posts"] = np.stack(posts)
    gathered = oracle.gather(state["pool"], slot_out, owners, queries, p.output_stride)
    # LRU feedback: touched slots move to the tail in ascending slot order
    for b in range(batch):
        lru = oracle.SlotLRUOracle()
        lru.order, lru.active = state["order"][b][:resident].copy(), resident
        lru.commit(slot_out[b * queries:(b + 1) * queries].reshape(-1))
        state["order"][b][:resident] = lru.order
        state["lru_slots"][b] = lru.slots
        state["reserved"][b] = lru.reserved_hot(resident)
    return state, topk, logical_out, slot_out, gathered, reads


def li_tolerance_check(p, scores, before):
    """Device LI scores against the NumPy golden formula, on the valid prefix of every row. Keys and scales
    come from the snapshot taken before the step: the step itself permutes the Index rows."""
    inputs = p.workspace.inputs
    bf16 = p.key_dtype == "bf16"
    as_np = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else (  # noqa: E731
        t.cpu().view(torch.uint8).numpy() if t.element_size() == 1 else t.cpu().numpy())
    query_ends = inputs.query_ends.cpu().numpy().reshape(p.batch, p.queries)
    expected = oracle.li_scores(
        as_np(inputs.query), before["keys"].view(np.uint16 if bf16 else np.uint8).reshape(-1, 128),
        as_np(inputs.weights), None if bf16 else inputs.scale.cpu().numpy(),
        None if bf16 else before["scales"].reshape(-1),
        p.workspace.key_lengths.cpu().numpy(), query_ends, inputs.block_table.cpu().numpy(), key_is_bf16=bf16,
        weight_is_bf16=inputs.weights.dtype == torch.bfloat16)
    rtol = 2e-3 if bf16 else 1e-2
    for t in range(scores.shape[0]):
        n = int(min(query_ends.reshape(-1)[t], p.workspace.key_lengths[t // p.queries]))
        if n <= 0:
            continue
        ref, out = expected[t, :n], scores[t, :n]
        assert (np.abs(out - ref) <= rtol * np.abs(ref) + rtol * 1e-2 * np.abs(ref).max()).all()
    return expected


CONFIGS = [
    # C1, the CPU-golden decode: B=4, 1 query, ctx U[2048,4096], 64 heads bf16, fp32 weights, 576-dim bf16 KV rows,
    # 8192-slot resident pool that starts empty, SlotLRU fresh, seed 0
    dict(batch=4, queries=1, heads=64, history=16384, resident=8192, len_lo=2048, len_hi=4096, key_dtype="bf16",
         weight_dtype="fp32", token_bytes=1152, seed=0),
    # FP8 keys + per-token scales, 2 MTP queries, cold context beyond the resident prefix, more owners than rows
    dict(batch=3, queries=2, heads=64, history=12288, resident=4096, len_lo=9000, len_hi=12288, key_dtype="fp8",
         weight_dtype="bf16", token_bytes=1152, seed=1, owners=5),
    # the reference's 4 query slots, 32 heads, 656-byte rows, misses served from a device-resident source
    dict(batch=2, queries=4, heads=32, history=8192, resident=6144, len_lo=7000, len_hi=8192, key_dtype="fp8",
         weight_dtype="bf16", token_bytes=656, seed=2, host_pool=False),
]


@pytest.mark.parametrize("config", CONFIGS, ids=["c1_bf16", "fp8_mtp2", "q4_h32"])
def test_forward_matches_oracle_over_steps(config, device):
    p = DecodePipeline(device, fill_payload=True, **config)
    try:
        total_reads = []
        for step in range(3):
            if step == 2:
                p.new_queries(config["seed"])      # repeat the first step's queries: mostly hits now
            elif step:
                p.new_queries(config["seed"] + 100 * step)
            before = snapshot(p)
            p.step()
            torch.cuda.synchronize()
            assert int(p.forward.li_status.item()) == 0
            assert (p.update.status.cpu().numpy() == 0).all() and (p.rotating.row_status[:, 0].cpu().numpy() == 0).all()
            scores = p.workspace.scores.cpu().numpy()
            li_tolerance_check(p, scores, before)
            state, topk, logical_out, slot_out, gathered, reads = oracle_step(p, before, scores)
            total_reads.append(reads)
            assert np.array_equal(p.workspace.topk.cpu().numpy(), topk)
            assert np.array_equal(p.update.logical_output.cpu().numpy().reshape(-1, TOPK), logical_out)
            assert np.array_equal(p.update.slot_output.cpu().numpy().reshape(-1, TOPK), slot_out)
            after = snapshot(p)
            for name in ("keys", "scales", "addresses", "logical", "hot_valid", "pool", "lru_slots", "reserved"):
                assert np.array_equal(after[name], state[name]), (step, name)
            assert np.array_equal(after["order"][:, :p.resident], state["order"][:, :p.resident])
            assert np.array_equal(p.gather_out.cpu().numpy(), gathered)
            assert np.array_equal(p.rotating.query_counts[:, 4].cpu().numpy(), np.asarray(reads))
            assert np.array_equal(p.rotating.final_posts.cpu().numpy().view(np.uint32).reshape(p.batch, 4, 32),
                                  state["final_posts"]), "final posts differ from the restatement"
            # fetched bytes identify the selected logical token of the right owner
            owners = p.workspace.inputs.row_owners.cpu().numpy()
            got = p.gather_out.cpu().numpy()
            for t in range(p.batch * p.queries):
                live = logical_out[t] >= 0
                want = payload_rows(int(owners[t // p.queries]), logical_out[t][live], p.token_bytes)
                assert np.array_equal(got[t][live], want)
            # Index rows stay a permutation of the logical tokens
            for owner in set(int(o) for o in owners):
                assert np.array_equal(np.sort(after["logical"][owner]), np.arange(p.history))
        assert sum(total_reads[2]) < sum(total_reads[0]), "a repeated query must mostly hit the resident pool"
    finally:
        p.close()


def test_forward_with_abc_tail(device):
    """The fused call with ABC tail bounds bound (reference binding.py:150-164, cache_metadata.h:22-26, 100-105): the
    last tokens of every request live in a ring of dedicated slots behind the hot ones. Those positions are served
    from the ring (location resident + p % ring), never fetched and never evicted; everything else behaves as
    without a tail. Checked against the restatement over three steps, and by the fetched bytes themselves."""
    ring = 512
    config = dict(batch=3, queries=2, heads=64, history=12288, resident=4096, len_lo=9000, len_hi=12288,
                  key_dtype="fp8", weight_dtype="bf16", token_bytes=1152, seed=3)
    p = DecodePipeline(device, fill_payload=True, tail_slots=ring, **config)
    try:
        owners = p.workspace.inputs.row_owners.cpu().numpy()
        bounds = np.zeros((p.batch, 2), np.int32)
        for b in range(p.batch):
            length, owner = int(p.lengths[b]), int(owners[b])
            bounds[b] = (length - 300 - 40 * b, length)     # the newest 300..380 tokens are uncommitted
            tail = np.arange(bounds[b, 0], bounds[b, 1])
            # the owner of the ring wrote these rows when the tokens were generated (update_abc's slot rule)
            rows = torch.from_numpy(payload_rows(owner, tail, p.token_bytes)).to(device)
            slots = torch.from_numpy(owner * p.output_stride + p.resident + tail % ring).to(device)
            p.pool_hbm[slots] = rows
            # scores of recent tokens are large in practice; here the host pool simply has no valid copy of them
            p.host_pool.tensor[owner, bounds[b, 0]:bounds[b, 1]] = 0xEE
        p.tail_bounds.copy_(torch.from_numpy(bounds))
        in_tail_total = 0
        for step in range(3):
            if step:
                p.new_queries(config["seed"] + 7 * step)
            before = snapshot(p)
            p.step()
            torch.cuda.synchronize()
            assert int(p.forward.li_status.item()) == 0 and int(p.update.status.abs().sum()) == 0
            scores = p.workspace.scores.cpu().numpy()
            state, topk, logical_out, slot_out, gathered, reads = oracle_step(p, before, scores)
            assert np.array_equal(p.workspace.topk.cpu().numpy(), topk)
            assert np.array_equal(p.update.slot_output.cpu().numpy().reshape(-1, TOPK), slot_out)
            assert np.array_equal(p.update.logical_output.cpu().numpy().reshape(-1, TOPK), logical_out)
            after = snapshot(p)
            for name in ("keys", "scales", "addresses", "logical", "hot_valid", "pool", "lru_slots", "reserved"):
                assert np.array_equal(after[name], state[name]), (step, name)
            assert np.array_equal(p.gather_out.cpu().numpy(), gathered)
            got = p.gather_out.cpu().numpy()
            for t in range(p.batch * p.queries):
                b = t // p.queries
                positions = topk.reshape(-1, TOPK)[t]
                live = positions >= 0
                in_tail = live & (positions >= bounds[b, 0]) & (positions < bounds[b, 1])
                in_tail_total += int(in_tail.sum())
                assert (slot_out[t][in_tail] == p.resident + positions[in_tail] % ring).all()
                assert (slot_out[t][live & ~in_tail] < p.resident).all()
                want = payload_rows(int(owners[b]), logical_out[t][live], p.token_bytes)
                assert np.array_equal(got[t][live], want), "tail rows must come from the ring, not from the host pool"
        assert in_tail_total > 0, "the case must select tail positions"
    finally:
        p.close()


def test_stage_times_and_option_bits(device):
    """KVIP_OPTION_DIAGNOSTICS makes the call stamp the GPU timer between its stages (reference: the `times`
    buffer, streaming.cpp:107-108, 390-465); the reference's scheduling-hint bits are accepted and change nothing;
    its legacy-layout bit is refused; the outputs do not depend on any of them."""
    config = dict(batch=2, queries=2, heads=64, history=8192, resident=4096, len_lo=6000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=1152, seed=9, host_pool=False, fill_payload=True)
    plain, timed = DecodePipeline(device, **config), DecodePipeline(device, **config)
    library = _lib.load_library()
    assert library.kvip_b200_abi_version() == 3
    timed.forward.set_options(diagnostics=True)
    timed.forward._options |= _lib.OPTION_SCHEDULING_HINTS      # parallel finalize + prepare metadata + UBmem overlap
    timed.forward._options_word[0] = timed.forward._options
    before = library.kvip_b200_launch_count()
    timed.step()
    assert library.kvip_b200_launch_count() - before == 8 + 8   # the eight kernels of a step + eight stamps
    plain.step()
    torch.cuda.synchronize()
    assert torch.equal(plain.update.outputs, timed.update.outputs) and torch.equal(plain.gather_out, timed.gather_out)
    times = timed.forward.stage_times()
    assert set(times) == set(_lib.TIME_STAGES) | {"total"}
    assert all(value >= 0 for value in times.values()) and times["li_score"] > 0 and times["gather"] > 0
    assert abs(sum(times[name] for name in _lib.TIME_STAGES) - times["total"]) < 1e-6
    assert 1 < times["total"] < 1e6, "a small step takes microseconds to milliseconds"
    assert int(plain.forward.times.abs().sum()) == 0, "without the option nothing is stamped"
    plain.forward._options_word[0] = plain.forward._options | _lib.OPTION_LEGACY_LAYOUT
    code = plain.forward.function(plain.rotating.bindings.data_ptr(), plain.update.bindings.data_ptr(),
                                  plain.forward.workspace.data_ptr(), None, plain.forward.shape_pointer, 2)
    assert code == _lib.BAD_ARGUMENT and "legacy" in _lib.last_error(library)
    plain.forward._options_word[0] = plain.forward._options


def test_forward_is_graph_capturable_and_allocation_free(device):
    config = dict(batch=3, queries=2, heads=64, history=8192, resident=4096, len_lo=6000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=1152, seed=5, host_pool=False)
    eager = DecodePipeline(device, fill_payload=True, **config)
    graphed = DecodePipeline(device, fill_payload=True, **config)
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        graphed.step()                       # warm-up outside capture (lazy function attributes)
        eager.step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = torch.cuda.memory_allocated(device)
        launches = _lib.load_library().kvip_b200_launch_count()
        with torch.cuda.graph(graph, stream=stream):
            graphed.step()
        assert _lib.load_library().kvip_b200_launch_count() - launches == 8  # LI, TopK, resolve, outputs, exchange, fetch, gather, LRU
        for replay in range(3):
            for p in (eager, graphed):
                p.new_queries(40 + replay)   # in-place update of the captured input buffers
            eager.step()
            graph.replay()
            stream.synchronize()
            assert torch.equal(eager.workspace.topk, graphed.workspace.topk)
            assert torch.equal(eager.update.slot_output, graphed.update.slot_output)
            assert torch.equal(eager.update.logical_output, graphed.update.logical_output)
            assert torch.equal(eager.gather_out, graphed.gather_out)
            assert torch.equal(eager.storage.logical_ids, graphed.storage.logical_ids)
            assert torch.equal(eager.rotating.lru_slots, graphed.rotating.lru_slots)
        after = torch.cuda.memory_allocated(device)
        eager.forward()
        assert torch.cuda.memory_allocated(device) == after, "forward() must not allocate"
        assert after - before < (64 << 20)


def test_two_phase_call_and_serial_lru_equal_the_fused_call(device):
    """`select()` + `commit()` with the LRU feedback after the step (the reference's order) leave the same
    outputs, Index rows, pool bytes and LRU order as `__call__()` with the feedback enqueued beside fetch and
    gather."""
    config = dict(batch=3, queries=2, heads=64, history=8192, resident=4096, len_lo=6000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=656, seed=11, host_pool=False, fill_payload=True)
    fused = DecodePipeline(device, **config)
    split = DecodePipeline(device, overlap_lru=False, **config)
    for step in range(4):
        for p in (fused, split):
            p.new_queries(100 + step)
        fused.step()
        split.forward.select()
        split.forward.commit()
        split.lru.commit(split.update.slot_output.view(split.batch, -1))
        torch.cuda.synchronize()
        assert torch.equal(fused.update.outputs, split.update.outputs)
        assert torch.equal(fused.gather_out, split.gather_out)
        assert torch.equal(fused.pool_hbm, split.pool_hbm)
        assert torch.equal(fused.storage.logical_ids, split.storage.logical_ids)
        assert torch.equal(fused.lru.order, split.lru.order)
        assert torch.equal(fused.rotating.lru_slots, split.rotating.lru_slots)
        assert int(fused.update.status.abs().sum()) == 0


@pytest.mark.parametrize("host_pool", [False, True])
def test_overlapped_commit_phase_equals_the_serial_one(host_pool, device):
    """`LIFetch(overlap_fetch=True)`: outputs, Index exchange and the gather of the hit entries run on a side stream
    beside the fetch of the missing rows; residency is published and the missed entries are gathered after both.
    Every observable result must equal the serial call's over steps with misses, evictions and repeats - eagerly
    and replayed from one CUDA graph (the fork and the join are part of the capture)."""
    config = dict(batch=3, queries=2, heads=64, history=12288, resident=4096, len_lo=9000, len_hi=12288, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=1152, seed=21, host_pool=host_pool, fill_payload=True)
    serial = DecodePipeline(device, **config)
    overlapped = DecodePipeline(device, overlap_fetch=True, **config)
    stream = torch.cuda.Stream(device)
    try:
        with torch.cuda.stream(stream):
            graph = None
            for step, seed in enumerate((21, 22, 23, 21, 24, 22)):
                for p in (serial, overlapped):
                    p.new_queries(seed)
                serial.step()
                if graph is None:
                    overlapped.step()
                else:
                    graph.replay()
                stream.synchronize()
                for name in ("outputs",):
                    assert torch.equal(getattr(serial.update, name), getattr(overlapped.update, name)), (step, name)
                assert torch.equal(serial.gather_out, overlapped.gather_out), step
                assert torch.equal(serial.pool_hbm, overlapped.pool_hbm), step
                assert torch.equal(serial.storage.hot_valid, overlapped.storage.hot_valid), step
                assert torch.equal(serial.storage.logical_ids, overlapped.storage.logical_ids), step
                assert torch.equal(serial.storage.keys, overlapped.storage.keys), step
                assert torch.equal(serial.lru.order, overlapped.lru.order), step
                assert torch.equal(serial.rotating.query_counts, overlapped.rotating.query_counts), step
                assert int(overlapped.update.status.abs().sum()) == 0
                if step == 0:
                    assert int(serial.rotating.query_counts[:, 4].sum()) > 0, "the case must have misses"
                    # the miss mask marks exactly the entries whose slot this step's fetch filled
                    mask = overlapped.rotating.miss_mask.cpu().numpy().view(np.uint32)
                    bits = ((mask[:, :, None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(mask.shape[0], TOPK)
                    assert bits.sum() == 3 * 2 * TOPK, "an empty pool misses every entry"
                if step == 1:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):   # recorded, not run: the states stay equal
                        overlapped.step()
    finally:
        serial.close()
        overlapped.close()


def _host_inputs(p):
    inputs = p.workspace.inputs
    pin = lambda t: t.cpu().pin_memory()  # noqa: E731
    return dict(host_query=pin(inputs.query.view(torch.uint8)).view(torch.float8_e4m3fn), host_weights=pin(inputs.weights),
                host_scale=pin(inputs.scale), host_positions=pin(p.positions))


@pytest.mark.parametrize("prefetch", [False, True])
def test_host_decode_loop_equals_serial_steps(prefetch, device):
    """Copies overlapped with neighbouring steps (and both halves replayed from graphs) change nothing: the
    rows read back on the host, the pool and the LRU order equal those of steps issued on one stream. Without
    prefetch the queries change every step; with it they are the same every step, as the caller must have
    the next step's inputs in host memory one step early."""
    from kvip_b200 import HostDecodeLoop
    config = dict(batch=4, queries=1, heads=64, history=8192, resident=4096, len_lo=6000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=656, seed=21, host_pool=False, fill_payload=True, permute_owners=False)
    serial, looped = DecodePipeline(device, **config), DecodePipeline(device, **config)
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        host = _host_inputs(serial)
        host_out = torch.empty(tuple(looped.update.outputs.shape), dtype=torch.int32).pin_memory()
        loop = HostDecodeLoop(torch, looped.forward, looped.workspace.inputs, looped.update.outputs,
                              host_outputs=host_out, **host)
        serial.step()   # the step the loop ran while it was built
        for step in range(4):
            if not prefetch:
                serial.new_queries(300 + step)
                stream.synchronize()
                for name, tensor in _host_inputs(serial).items():
                    host[name].view(torch.uint8).copy_(tensor.view(torch.uint8))
            serial.step()
            loop.step(prefetch_next=prefetch)
            loop.drain()
            stream.synchronize()
            assert torch.equal(host_out, serial.update.outputs.cpu())
            assert torch.equal(looped.update.outputs, serial.update.outputs)
            assert torch.equal(looped.pool_hbm, serial.pool_hbm)
            assert torch.equal(looped.lru.order, serial.lru.order)
            assert torch.equal(looped.gather_out, serial.gather_out)
    assert loop.steps == 4 and loop.h2d_bytes > 0 and loop.d2h_bytes == host_out.numel() * 4


def test_index_selector_mixed_batch(device):
    """The serving-side caller: a forward batch of three decode tokens and one 64-token prefill chunk. Decode
    rows go through QueryInputs.pack + LIFetch and must equal a plain pipeline step on the same queries; the
    prefill rows are selected by the paged indexer over the model's own cache and must satisfy the reference's
    TopK validity oracle against the golden scores; `slots()` returns the resident slots of the decode tokens."""
    import workloads
    from kvip_b200 import IndexSelector, PagedIndexer, RequestPlan
    config = dict(batch=3, queries=1, heads=64, history=8192, resident=4096, len_lo=6000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=656, seed=31, host_pool=False, fill_payload=True)
    plain, served = DecodePipeline(device, **config), DecodePipeline(device, **config)
    plain.step()
    inputs = served.workspace.inputs
    owners = served.row_owner_list
    chunk, context = 64, 4096
    case = workloads.prefill_case(seed=8, chunk=chunk, context=context)
    t = workloads.to_torch(case, device)
    # flattened forward batch: [decode 0 | prefill chunk | decode 1 | decode 2]
    where = [0, chunk + 1, chunk + 2]
    total = chunk + 3
    query = torch.zeros((total, 64, 128), dtype=torch.uint8, device=device)
    weights = torch.zeros((total, 64), dtype=torch.bfloat16, device=device)
    scale = torch.ones((total, 64), dtype=torch.float32, device=device)
    positions = torch.zeros(total, dtype=torch.int64, device=device)
    query[where] = inputs.query.view(torch.uint8)[:3]
    weights[where] = inputs.weights[:3]
    scale[where] = inputs.scale[:3]
    positions[where] = served.positions[:3]
    query[1:chunk + 1] = t["query"].view(torch.uint8)
    weights[1:chunk + 1] = t["weights"]
    scale[1:chunk + 1] = t["query_scale"]
    plans = [RequestPlan("d0", owners[0], 0, 1, decode=True),
             RequestPlan("p", 0, 1, chunk + 1, decode=False, start=context - chunk, key_end=context),
             RequestPlan("d1", owners[1], chunk + 1, chunk + 2, decode=True),
             RequestPlan("d2", owners[2], chunk + 2, chunk + 3, decode=True)]
    selector = IndexSelector(torch, inputs=inputs, rotating=served.rotating, update=served.update,
                             logical_ids=served.storage.logical_ids, row_owners=inputs.row_owners,
                             forward=served.forward)
    indexer = PagedIndexer(torch, t["keys"].view(torch.uint8).view(-1, 128, 128), t["key_scale"].view(-1, 128))
    metadata = type("Metadata", (), {})()
    metadata.block_table = torch.zeros((4, context // 128), dtype=torch.int32, device=device)
    metadata.block_table[1] = t["block_table"][0]
    selector.prepare(plans)
    inputs.bind_positions(positions)
    result = selector(query.view(torch.float8_e4m3fn), weights, indexer, metadata, scale)
    torch.cuda.synchronize()
    assert tuple(result.shape) == (total, 1, 2048)
    assert torch.equal(result[where], plain.update.logical_output[:3])
    assert torch.equal(selector.slots(3), plain.update.slot_output[:3])
    assert torch.equal(served.pool_hbm, plain.pool_hbm)
    expected = workloads.oracle_scores(case)
    picked = result[1:chunk + 1, 0].cpu().numpy()
    ends = case["query_ends"].reshape(-1)
    for i in range(chunk):
        assert picked[i].max() < ends[i]
        oracle.validate_topk(picked[i], expected[i:i + 1, :ends[i]])


def test_full_size_step_properties(device):
    """The benchmark's context length (131072 keys per request, FP8, 2048 x 1152-byte rows gathered per query) at
    batch 8, checked through properties that need no oracle pass over 128k keys: the selection is the TopK of the
    step's own scores (values against torch.topk, canonical order by definition), the Index rows stay a
    permutation that carries keys and scales along, every selected token sits in a valid resident slot holding
    its payload, the dense gather returns those payloads, and repeating the step fetches nothing."""
    p = DecodePipeline(device, batch=8, queries=1, heads=64, history=131072, resident=32768, len_lo=100000,
                       len_hi=131072, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152, seed=4, host_pool=False,
                       fill_payload=True)
    keys_before, scales_before = p.storage.keys.clone(), p.storage.scales.clone()
    p.step()
    torch.cuda.synchronize()
    assert int(p.forward.li_status.item()) == 0 and int(p.update.status.abs().sum()) == 0
    scores, topk = p.workspace.scores, p.workspace.topk.view(-1, 2048)
    lengths = torch.from_numpy(p.lengths).to(device)
    for row in range(8):
        n = int(lengths[row])
        picked = topk[row].long()
        assert int(picked.min()) >= 0 and int(picked.max()) < n and picked.unique().numel() == 2048
        values = scores[row, :n]
        best = torch.topk(values, 2048).values
        assert torch.equal(torch.sort(values[picked], descending=True).values, best)
        cut = best[-1]
        above = picked[values[picked] > cut]
        ties = picked[values[picked] == cut]
        assert torch.equal(torch.cat((above, ties)), picked)                      # all > cut first, then the ties
        assert bool((above[1:] > above[:-1]).all()) and bool((ties[1:] > ties[:-1]).all())   # each in position order
        lower_ties = torch.nonzero(values == cut).view(-1)[: ties.numel()]
        assert torch.equal(ties, lower_ties)                                        # ties go to the lower positions
    owners = torch.tensor(p.row_owner_list, device=device)
    logical_ids = p.storage.logical_ids
    identity = torch.arange(131072, device=device)
    for row in range(8):
        owner = int(owners[row])
        ids = logical_ids[owner]
        assert torch.equal(torch.sort(ids).values, identity)
        assert torch.equal(p.storage.keys[owner], keys_before[owner][ids])
        assert torch.equal(p.storage.scales[owner], scales_before[owner][ids])
        logical = p.update.logical_output[row, 0].long()
        slots = p.update.slot_output[row, 0].long()
        assert torch.equal(torch.sort(logical).values, torch.sort(topk[row].long()).values)  # first step: ids = positions
        assert int(slots.min()) >= 0 and int(slots.max()) < 32768 and slots.unique().numel() == 2048
        assert bool((p.storage.hot_valid[owner][slots] == 1).all())
        assert torch.equal(ids[slots], logical)                                  # slot p holds Index row p
        expected_rows = p.source[owner * 131072 + logical]
        assert torch.equal(p.pool_hbm[owner * p.output_stride + slots], expected_rows)
        assert torch.equal(p.gather_out[row], expected_rows)
    first_logical = p.update.logical_output.clone()
    p.step()
    torch.cuda.synchronize()
    assert int(p.rotating.query_counts[:, 4].sum()) == 0, "a repeated query must find every row resident"
    assert torch.equal(torch.sort(p.update.logical_output, dim=-1).values, torch.sort(first_logical, dim=-1).values)


def test_full_size_steps_with_evictions_from_the_host_pool(device):
    """Benchmark context length (131072 keys, FP8, 1152-byte rows) with misses served from the pinned host pool and a
    resident pool small enough (4096 slots) that rows are evicted and fetched again: independent queries in steps
    1-3 fill the pool and push the first step's rows out, step 4 repeats the first step's queries. After EVERY step
    the invariants the reference's harness checks (execution.py:2102-2131, 2183-2198, 2216-2224) must hold: the
    Index rows stay a joint permutation, every selected token sits in a distinct valid slot whose pool row is that
    token's host row, the dense gather returns those rows, statuses are zero."""
    batch, history, resident = 8, 131072, 4096
    p = DecodePipeline(device, batch=batch, queries=1, heads=64, history=history, resident=resident, len_lo=100000,
                       len_hi=131072, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152, seed=6, host_pool=True,
                       fill_payload=True)
    try:
        keys_before, scales_before = p.storage.keys.clone(), p.storage.scales.clone()
        identity = torch.arange(history, device=device)
        owners = p.row_owner_list
        lengths = torch.from_numpy(p.lengths).to(device)
        reads = []
        for step, seed in enumerate((6, 60, 600, 6)):
            p.new_queries(seed)
            p.step()
            torch.cuda.synchronize()
            assert int(p.forward.li_status.item()) == 0 and int(p.update.status.abs().sum()) == 0
            assert int(p.rotating.row_status[:, 0].abs().sum()) == 0 and int(p.rotating.row_status[:, 2].abs().sum()) == 0
            reads.append(int(p.rotating.query_counts[:, 4].sum()))
            topk = p.workspace.topk.view(-1, 2048)
            for row in range(batch):
                owner, n = owners[row], int(lengths[row])
                values = p.workspace.scores[row, :n]
                picked = topk[row].long()
                assert torch.equal(torch.sort(values[picked], descending=True).values, torch.topk(values, 2048).values)
                ids = p.storage.logical_ids[owner]
                assert torch.equal(torch.sort(ids).values, identity), (step, row)
                assert torch.equal(p.storage.keys[owner], keys_before[owner][ids])
                assert torch.equal(p.storage.scales[owner], scales_before[owner][ids])
                assert torch.equal(p.storage.addresses[owner], (ids + owner * history) * p.token_bytes)
                logical = p.update.logical_output[row, 0].long()
                slots = p.update.slot_output[row, 0].long()
                assert int(slots.min()) >= 0 and int(slots.max()) < resident and slots.unique().numel() == 2048
                assert bool((p.storage.hot_valid[owner][slots] == 1).all())
                assert torch.equal(ids[slots], logical), "slot p must hold Index row p"
                expected_rows = p.host_pool.tensor[owner][logical.cpu()]
                assert torch.equal(p.pool_hbm[owner * p.output_stride + slots].cpu(), expected_rows), (step, row)
                assert torch.equal(p.gather_out[row].cpu(), expected_rows)
                # every valid hot slot (not only the selected ones) still holds the row its Index position names
                valid = torch.nonzero(p.storage.hot_valid[owner]).view(-1)
                sample = valid[:: max(1, valid.numel() // 256)]
                assert torch.equal(p.pool_hbm[owner * p.output_stride + sample].cpu(),
                                   p.host_pool.tensor[owner][ids[sample].cpu()])
        assert reads[0] == batch * 2048, "an empty pool misses everything"
        assert reads[2] > 0 and int(p.storage.hot_valid.sum()) <= batch * resident
        # step 3 took the least recently used slots, i.e. step 1's rows: the repeated query fetches them again
        assert batch * 1024 < reads[3] <= batch * 2048, "the repeated query must find its rows evicted"
    finally:
        p.close()


def test_two_devices_in_one_process(device):
    """Function attributes (the dynamic shared-memory limits) and the SM count are kept per device: a process that
    drives a second GPU gets the same results there. Skipped on a one-GPU box."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    config = dict(batch=2, queries=2, heads=64, history=8192, resident=4096, len_lo=6000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=1152, seed=13, host_pool=False, fill_payload=True)
    results = []
    for index in (0, 1):
        with torch.cuda.device(index):
            p = DecodePipeline(torch.device("cuda", index), **config)
            p.step()
            torch.cuda.synchronize()
            assert int(p.forward.li_status.item()) == 0 and int(p.update.status.abs().sum()) == 0
            results.append((p.update.outputs.cpu(), p.gather_out.cpu()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


def test_forward_rejects_mismatched_shape(device):
    config = dict(batch=2, queries=1, heads=64, history=4096, resident=2048, len_lo=3000, len_hi=4096, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=1152, seed=3, host_pool=False, gather=False)
    p = DecodePipeline(device, **config)
    p.forward()
    other = _lib.RuntimeShape.prepare(p.rotating.library, batch=2, history=8192, resident=2048, indexHeads=64, queries=1,
                                      tokenBytes=1152)
    import ctypes
    p.forward.shape_pointer = ctypes.byref(other)
    with pytest.raises(RuntimeError, match="100000"):
        p.forward()
    torch.cuda.synchronize()


def test_status_reports_exhausted_pool(device):
    """All-miss rounds larger than the pool: the request fails closed - error 4, outputs -1, residency dropped."""
    config = dict(batch=1, queries=4, heads=32, history=32768, resident=2048, len_lo=32768, len_hi=32768,
                  key_dtype="fp8", weight_dtype="bf16", token_bytes=656, seed=9, host_pool=False, gather=False)
    p = DecodePipeline(device, **config)
    p.forward()
    torch.cuda.synchronize()
    assert int(p.rotating.row_status[0, 0]) == oracle.ERR_NO_SLOT
    assert int(p.update.status[0]) == oracle.ERR_NO_SLOT
    assert (p.update.slot_output.cpu().numpy() == -1).all()
    assert int(p.storage.hot_valid.sum()) == 0


def _sparse_attention(query, rows):
    """The consumer's arithmetic over 2048 selected KV rows of 576 bf16 values (512 latent + 64 rotary): keys are
    the whole row, values its first 512 entries; softmax in fp32, probabilities rounded to bf16 before the
    value product, as the reference's check does (tests/operators/lifetch/support/correctness.py:281-296)."""
    kv = rows.view(torch.bfloat16).float()                       # [2048, 576]
    logits = query.float() @ kv.T * 576 ** -0.5                   # [8, 2048]
    prob = torch.softmax(logits, dim=-1).to(torch.bfloat16).float()
    return prob @ kv[:, :512]


def test_sparse_attention_over_slot_output_equals_attention_over_logical_tokens(device):
    """End-to-end consumer check (reference: check_sfa, tests/operators/lifetch/support/correctness.py:262-339):
    sparse attention that reads the resident pool through `slot_output` (and, separately, the dense gathered
    rows) must give what attention over the same logical tokens' rows of the backing pool gives. Tolerances are
    the reference's (atol 0.006, rtol 0.025); since the rows must be the same bytes in the same order, the
    results are also required to be identical. Steps mix misses (first step, new queries) and hits (repeat)."""
    history, resident = 8192, 4096
    p = DecodePipeline(device, batch=3, queries=2, heads=64, history=history, resident=resident, len_lo=6000,
                       len_hi=8192, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152, seed=41, host_pool=False)
    generator = torch.Generator(device=device).manual_seed(181)
    kv = torch.rand(p.source.shape[0], 576, generator=generator, device=device) * 2 - 1
    p.source.view(torch.bfloat16).copy_(kv.to(torch.bfloat16))
    query = (torch.rand(p.batch * 2, 8, 576, generator=generator, device=device) * 0.4 - 0.2).to(torch.bfloat16)
    fetched = []
    for step, seed in enumerate((41, 141, 41)):
        p.new_queries(seed)
        p.step()
        torch.cuda.synchronize()
        assert int(p.update.status.abs().sum()) == 0
        fetched.append(int(p.rotating.query_counts[:, 4].sum()))
        for row in range(p.batch * 2):
            owner = p.row_owner_list[row // 2]
            logical = p.update.logical_output[row, 0].long()
            slots = p.update.slot_output[row, 0].long()
            assert int(logical.min()) >= 0 and int(slots.min()) >= 0 and int(slots.max()) < resident
            expected = _sparse_attention(query[row], p.source[owner * history + logical])
            through_slots = _sparse_attention(query[row], p.pool_hbm[owner * p.output_stride + slots])
            through_gather = _sparse_attention(query[row], p.gather_out[row])
            assert bool(torch.isfinite(through_slots).all())
            for actual in (through_slots, through_gather):
                assert torch.allclose(actual, expected, atol=0.006, rtol=0.025)
                assert torch.equal(actual, expected)
    assert fetched[0] > 0 and fetched[1] > 0 and fetched[2] < fetched[0]   # misses, misses, mostly hits


@pytest.mark.parametrize("len_lo", [6000, 1500], ids=["long", "some_shorter_than_the_pool"])
def test_prefetch_windows_change_only_where_missing_rows_come_from(len_lo, device):
    """Speculative prefetch windows (reference: op_kernel/prefetch.h:577-821; predicate indexer_score.h:976-1017):
    the score pass runs window by window, rows of cold positions that beat the resident threshold are staged
    meanwhile, and the final fetch takes listed rows from the staging area. Scores, outputs, Index rows, pool
    bytes and LRU order must equal those of the plain forward bit for bit; thresholds and candidate lists must
    equal the oracle's cold predicate; the rows served from the staging area are exactly the final descriptors
    whose source is listed."""
    config = dict(batch=5 if len_lo < 4096 else 3, queries=2, heads=64, history=8192, resident=4096, len_lo=len_lo,
                  len_hi=8192, key_dtype="fp8", weight_dtype="bf16", token_bytes=656, seed=51, host_pool=False,
                  fill_payload=True)
    plain = DecodePipeline(device, **config)
    spec = DecodePipeline(device, prefetch_limit=512, prefetch_last_window=True, **config)   # every cold window staged
    prefetch = spec.forward.prefetch
    assert prefetch.first == [0, 4096, 5504, 6912, 8192]
    lengths = spec.workspace.key_lengths.cpu().numpy()
    total_hits = total_listed = 0
    for step in range(4):
        for p in (plain, spec):
            p.new_queries(500 + step)
        addresses_before = spec.storage.addresses.cpu().numpy().copy()
        plain.step()
        spec.step()
        torch.cuda.synchronize()
        assert int(spec.forward.li_status.item()) == 0 and int(spec.update.status.abs().sum()) == 0
        assert torch.equal(spec.workspace.scores, plain.workspace.scores)
        assert torch.equal(spec.workspace.topk, plain.workspace.topk)
        assert torch.equal(spec.update.outputs, plain.update.outputs)
        assert torch.equal(spec.gather_out, plain.gather_out)
        assert torch.equal(spec.pool_hbm, plain.pool_hbm)
        assert torch.equal(spec.storage.logical_ids, plain.storage.logical_ids)
        assert torch.equal(spec.storage.keys, plain.storage.keys)
        assert torch.equal(spec.lru.order, plain.lru.order)
        scores = spec.workspace.scores.cpu().numpy()
        ends = spec.workspace.inputs.query_ends.cpu().numpy().reshape(spec.batch, -1)[:, :2]
        _, thresholds, bitmap, _ = oracle.cold_predicate(scores, lengths, ends, 4096)
        assert np.array_equal(prefetch.thresholds.cpu().numpy().view(np.uint32), thresholds)
        staged_rows = prefetch.staged_rows.cpu().numpy()
        staged_sources = prefetch.staged_sources.cpu().numpy()
        hits = prefetch.staged_hits.cpu().numpy()
        counts = spec.rotating.query_counts.cpu().numpy()[:, 4]
        descriptors = spec.rotating.fallback_addresses.cpu().numpy()
        for b in range(spec.batch):
            owner = spec.row_owner_list[b]
            marked = np.bitwise_or.reduce(bitmap[2 * b: 2 * b + 2], axis=0)
            positions = 4096 + np.flatnonzero(np.unpackbits(marked.view(np.uint8), bitorder="little"))
            expected = set(addresses_before[owner, positions].tolist())
            listed = staged_sources[b, :staged_rows[b]].tolist()
            assert len(set(listed)) == len(listed) and set(listed) <= expected
            if len(expected) <= 480:
                assert set(listed) == expected
            else:
                assert len(listed) >= 480
            wanted = descriptors[b, :counts[b]].tolist()
            assert hits[b] == sum(1 for source in wanted if source in set(listed))
            total_hits += int(hits[b])
            total_listed += len(listed)
    assert total_listed > 0 and total_hits > 0


def test_prefetch_windows_replay_from_a_graph(device):
    """The windowed score launches, the second stream's work and both joins are captured in one CUDA graph; its
    replays equal the eager steps of a plain pipeline."""
    config = dict(batch=2, queries=1, heads=64, history=8192, resident=4096, len_lo=7000, len_hi=8192, key_dtype="fp8",
                  weight_dtype="bf16", token_bytes=1152, seed=61, host_pool=False, fill_payload=True)
    plain = DecodePipeline(device, **config)
    spec = DecodePipeline(device, prefetch_limit=256, prefetch_windows=2, **config)
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        plain.step()
        spec.step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            spec.step()
        for step in range(3):
            for p in (plain, spec):
                p.new_queries(700 + step)
            plain.step()
            graph.replay()
            stream.synchronize()
            assert torch.equal(spec.update.outputs, plain.update.outputs)
            assert torch.equal(spec.pool_hbm, plain.pool_hbm)
            assert torch.equal(spec.gather_out, plain.gather_out)
            assert torch.equal(spec.lru.order, plain.lru.order)
    assert int(spec.forward.prefetch.staged_rows.sum()) > 0


_SHARDED_WORKER = r"""
import os, sys
import torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from kvip_b200 import ops
from kvip_b200.sharding import ShardedTopk
device = torch.device("cuda", 0)
torch.cuda.set_device(device)
dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
g = torch.Generator(device=device)
g.manual_seed(11)
keys_here, rows = 40960, 2
scores = torch.randn((rows, keys_here), generator=g, device=device)
scores[0, ::7] = 0.5                      # ties across the cut
lengths = torch.full((1,), keys_here, dtype=torch.int32, device=device)
ends = torch.full((1, rows), keys_here, dtype=torch.int32, device=device)
expected = ops.topk(scores, lengths, ends)
sharded = ShardedTopk(rows, device)
eager = sharded(scores, lengths, ends, 0).clone()
calls = []
try:
    sharded.capture(lambda: calls.append(1), scores, lengths, ends, 0)
    raise SystemExit("capture on the default stream must be refused")
except ValueError:
    pass
torch.cuda.synchronize()
with torch.cuda.stream(torch.cuda.Stream(device)):
    sharded.capture(lambda: calls.append(1), scores, lengths, ends, 0)
    sharded.merged.fill_(-7)
    replayed = sharded.replay().clone()
torch.cuda.synchronize()
assert torch.equal(eager, expected), "eager sharded TopK differs from the unsharded one"
assert torch.equal(replayed, expected), "captured sharded TopK differs from the unsharded one"
assert calls, "the score step was not captured"
# the same over this library's peer-memory exchange (one rank: the block is its own), eagerly and as ONE graph
peer = ShardedTopk(rows, device, transport="peer")
assert torch.equal(peer(scores, lengths, ends, 0), expected), "peer transport, eager"
with torch.cuda.stream(torch.cuda.Stream(device)):
    peer.capture(lambda: None, scores, lengths, ends, 0)
    for _ in range(3):                      # odd and even steps: both halves of the block
        peer.merged.fill_(-7)
        assert torch.equal(peer.replay(), expected), "peer transport, graph replay"
torch.cuda.synchronize()
assert int(peer.status.item()) == 0
# bounded wait: a block that claims two ranks, of which only rank 0 ever delivers
import ctypes
from kvip_b200 import _lib
lib = _lib.load_library()
block, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
_lib.check(lib.kvip_b200_peer_alloc(_lib.PEER_HEADER_BYTES + 2 * 2 * peer.send.numel() * 4, ctypes.byref(block), handle), "alloc")
ops.peer_exchange(peer.send, [block.value, block.value], 0)
out = torch.zeros((rows, 2048), dtype=torch.int32, device=device)
status = torch.zeros(1, dtype=torch.int32, device=device)
ops.topk_merge_peer(block.value, rows, 2, out, status, wait_kilocycles=2000)    # about a millisecond
torch.cuda.synchronize()
assert int(status.item()) == _lib.ERR_PEER and bool((out == -1).all()), "the wait for the absent rank must give up"
assert torch.equal(peer(scores, lengths, ends, 0), expected), "the context stays usable after a wait ran out"
_lib.check(lib.kvip_b200_peer_free(block), "free")
peer.close()
dist.destroy_process_group()
print("ok")
"""


_TWO_RANK_WORKER = r"""
import os, sys
import torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from kvip_b200 import ops
from kvip_b200.sharding import ShardedTopk, shard_bounds
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
device = torch.device("cuda", rank)
torch.cuda.set_device(device)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
total, rows = 5 * 16384, 2
g = torch.Generator(device=device)
g.manual_seed(5)                                   # the same whole row on every rank
whole = torch.randn((rows, total), generator=g, device=device)
whole[0, ::5] = 0.25                               # ties across the shard border and the cut
begin, end = shard_bounds(total, world, rank)
scores = whole[:, begin:end].contiguous()
lengths = torch.full((1,), end - begin, dtype=torch.int32, device=device)
ends = torch.full((1, rows), end - begin, dtype=torch.int32, device=device)
whole_len = torch.full((1,), total, dtype=torch.int32, device=device)
expected = ops.topk(whole, whole_len, torch.full((1, rows), total, dtype=torch.int32, device=device))
over_nccl = ShardedTopk(rows, device)(scores, lengths, ends, begin).clone()
peer = ShardedTopk(rows, device, transport="peer")
eager = peer(scores, lengths, ends, begin).clone()
with torch.cuda.stream(torch.cuda.Stream(device)):
    peer.capture(lambda: None, scores, lengths, ends, begin)
    for _ in range(4):
        peer.merged.fill_(-7)
        replayed = peer.replay().clone()
        assert torch.equal(replayed, expected), "peer transport, graph replay"
torch.cuda.synchronize()
assert torch.equal(over_nccl, expected) and torch.equal(eager, expected)
assert int(peer.status.item()) == 0
peer.close()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.gpu
def test_sharded_topk_eager_and_captured_forms_on_one_rank(tmp_path):
    """ShardedTopk over NCCL with one rank: local TopK -> all-gather -> merge equals the plain TopK, eagerly and as two
    graph replays around the eager all-gather. A child process, so that the process group does not outlive the test."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    script = tmp_path / "sharded_worker.py"
    script.write_text(_SHARDED_WORKER.format(root=str(Path(__file__).resolve().parents[1])))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_sharded_topk_over_peer_memory_on_two_gpus(tmp_path):
    """Two ranks on two GPUs: local TopK -> candidates written into the other rank's exchange block over NVLink ->
    merge behind a bounded wait equals the unsharded TopK and the NCCL transport, eagerly and from one graph per rank.
    Child processes; NVLS off (plain peer stores only)."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_rank_worker.py"
    script.write_text(_TWO_RANK_WORKER.format(root=str(Path(__file__).resolve().parents[1])))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29643", WORLD_SIZE="2", NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    for proc in procs:
        out, _ = proc.communicate(timeout=300)
        assert proc.returncode == 0, out
