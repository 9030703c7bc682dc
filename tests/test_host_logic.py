"""CPU tests of the host side: the C ABI loads and exports every declared symbol, geometry validation,
ABI record layouts, QueryInputs packing against the reference's golden, request partitioning, and the
sequence-shard exchange among two gloo ranks. No kernel is launched here."""
import ctypes
import json
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import kvip_oracle as oracle
from golden_cases import GOLDEN
from kvip_b200 import _lib, sharding

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def library():
    from kvip_b200.build import build_library
    build_library()
    return _lib.load_library()


def test_library_exports_every_declared_symbol(library):
    header = (ROOT / "include" / "kvip_b200.h").read_text()
    declared = set(re.findall(r"\b(kvip_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(library, name), name


def test_abi_record_sizes(library):
    assert ctypes.sizeof(_lib.RuntimeShape) == 80
    assert ctypes.sizeof(_lib.Workspace) == 256 == library.kvip_b200_workspace_bytes()
    assert ctypes.sizeof(_lib.Context) == library.kvip_b200_context_bytes()
    assert _lib.Workspace.options.offset == 96            # reference streaming.py:146 writes the options word there
    assert _lib.RuntimeShape.tokenBytes.offset == 14 * 4  # same index as the reference's tokenBytes
    assert library.kvip_streaming_resolver_cores() == 3 and library.kvip_streaming_flag_count() == 16


def test_prepare_shape_accepts_benchmark_geometries_and_derives_fields(library):
    for batch, history, resident, queries in ((4, 16384, 8192, 1), (64, 32768, 8192, 2), (64, 131072, 32768, 1),
                                              (256, 131072, 65536, 1), (1, 1 << 20, 2048, 4)):
        shape = _lib.RuntimeShape.prepare(library, batch=batch, history=history, resident=resident, indexHeads=64,
                                          queries=queries, tokenBytes=1152)
        assert (shape.pagesPerRequest, shape.scoreStride, shape.outputStride, shape.owners, shape.finalWorkers) == (
            history // 128, history, resident, batch, 4)
        assert shape.keyRows == batch * history


@pytest.mark.parametrize("bad", [
    dict(batch=0), dict(batch=1025), dict(indexHeads=16), dict(queries=0), dict(queries=5), dict(history=131073),
    dict(resident=16385), dict(resident=1024), dict(resident=262144, history=262144), dict(history=8192, resident=16384),
    dict(tokenBytes=100), dict(tokenBytes=0), dict(keyDtype=2), dict(outputStride=1000)])
def test_prepare_shape_rejects(bad, library):
    """Same contract failures as the reference's check suite (correctness.py:68-109): ValueError, no launch."""
    fields = dict(batch=2, history=131072, resident=16384, indexHeads=64, queries=4, tokenBytes=656)
    fields.update(bad)
    with pytest.raises(ValueError):
        _lib.RuntimeShape.prepare(library, **fields)


def test_stage_entry_points_reject_null_arguments(library):
    """Argument checks run before any CUDA call, so they are testable without a device."""
    for name, struct in _lib._STAGES.items():
        assert getattr(library, name)(ctypes.byref(struct()), None) == _lib.BAD_ARGUMENT, name
    assert library.kvip_lifetch_streaming_forward(None, None, None, None, None, 2) == _lib.BAD_ARGUMENT
    assert b"null" in library.kvip_b200_last_error()


def test_option_bits_do_not_collide_with_the_reference(library):
    """The reference's option word (python/kvip/operators/lifetch/streaming.py:133-146) owns 0x80000000 diagnostics,
    0x40000000 deferred fetch, 0x20000000 legacy layout, 0x10000000 parallel finalize, 0x08000000 prepare metadata,
    0x04000000 UBmem overlap, bits 16-18 workers and bits 0-15 the prefetch limit. The bits this build adds lie
    elsewhere; the legacy layout is refused before anything is enqueued (checked here without a device)."""
    reference_bits = 0xFC000000 | (7 << 16) | 0xFFFF
    added = (_lib.OPTION_SELECT_ONLY, _lib.OPTION_COMMIT_ONLY, _lib.OPTION_SCORES_READY)
    assert all(bit & reference_bits == 0 for bit in added) and len({*added}) == 3
    assert _lib.OPTION_SCHEDULING_HINTS == 0x10000000 | 0x08000000 | 0x04000000
    assert library.kvip_b200_abi_version() == 3
    shape = _lib.RuntimeShape.prepare(library, batch=2, history=8192, resident=4096, indexHeads=64, queries=1, tokenBytes=1152)
    context = _lib.Context(shape=shape)
    workspace = _lib.Workspace(history=8192, resident=4096, max_events=10240, options=_lib.OPTION_LEGACY_LAYOUT | (2 << 16))
    bindings = (ctypes.c_uint64 * 16)(*([0] * 14), ctypes.addressof(context), ctypes.addressof(workspace))
    update = (ctypes.c_int64 * 28)()
    update[24], update[25] = 8192, 4096
    code = library.kvip_lifetch_streaming_forward(ctypes.addressof(bindings), ctypes.addressof(update),
                                                  ctypes.addressof(workspace), None, ctypes.byref(shape), 2)
    assert code == _lib.BAD_ARGUMENT and b"legacy" in library.kvip_b200_last_error()
    # with a scheduling hint instead, the call passes the option check and stops at the first unbound operand
    workspace.options = _lib.OPTION_SCHEDULING_HINTS | (2 << 16)
    code = library.kvip_lifetch_streaming_forward(ctypes.addressof(bindings), ctypes.addressof(update),
                                                  ctypes.addressof(workspace), None, ctypes.byref(shape), 2)
    assert code == _lib.BAD_ARGUMENT and b"unbound" in library.kvip_b200_last_error()


def test_product_has_no_cpu_fallback():
    from kvip_b200 import ops
    with pytest.raises(ValueError, match="CUDA"):
        ops.topk(torch.zeros((1, 4096)), torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="missing"):
        _lib.load_library(ROOT / "kvip_b200" / "no_such_library.so")
    for path in (ROOT / "kvip_b200").rglob("*.py"):
        text = path.read_text()
        assert "import kvip_oracle" not in text and "oracle_c" not in text and "oracle/" not in text, (
            f"{path} must not reach into the oracle")


def test_query_slot_layout_matches_reference_golden():
    """The host layout of a step (`slot_layout`, what QueryInputs.prepare uploads) against the metadata block the
    reference produced (python/kvip/adapters/vllm/inputs.py:73-113; tests/adapters/test_inputs.py). The device
    half (query ends, block table) is checked on the GPU against the same golden."""
    from kvip_b200.inputs import QueryInputs, slot_layout
    d = np.load(GOLDEN / "ingest_decode.npz")
    layout, tokens = slot_layout(tuple(int(x) for x in d["counts"]), batch=3,
                                 query_starts=tuple(int(x) for x in d["starts"]),
                                 query_owners=tuple(int(x) for x in d["owners"]))
    assert np.array_equal(layout, d["metadata"]) and tokens == int(d["token_count"])
    for bad in (dict(query_counts=(5,)), dict(query_counts=(1, 1, 1, 1)), dict(query_counts=(1,), query_starts=(-1,)),
                dict(query_counts=(1, 2), query_starts=(0,)), dict(query_counts=(1,), query_owners=(1 << 31,)),
                dict(query_counts=(1.0,))):
        with pytest.raises(ValueError):
            slot_layout(batch=3, **bad)
    with pytest.raises(ValueError, match="CUDA"):   # the buffers live on the GPU: no CPU path
        QueryInputs(torch, 1, torch.device("cpu"))


def test_query_slot_layout_generalised_slots():
    from kvip_b200.inputs import slot_layout
    layout, tokens = slot_layout((2, 1, 0, 2), batch=4, queries=2, query_owners=(3, 1, 0, 2))
    assert tokens == 5
    assert layout[0].tolist() == [0, 1, 2, 0, 0, 0, 3, 4]
    assert layout[1].tolist() == [1, 1, 1, 0, 0, 0, 1, 1]
    assert layout[2].tolist()[:5] == [0, 1, 2, 6, 7] and layout[3].tolist() == [1] * 5 + [0] * 3
    assert layout[4].view(np.int32)[:4].tolist() == [3, 1, 0, 2]


def test_committed_candidates_keep_the_committed_prefix_first():
    from kvip_b200.inputs import committed_candidates
    candidates = np.array([7, 2, 9, 4, 11, 0], dtype=np.int32)
    assert committed_candidates(candidates, 16, 12) is candidates               # whole pool committed
    assert committed_candidates(candidates, 5, 12).tolist() == [2, 4, 0, 1, 3, 7]   # inside, missing inside, rest; cut


def test_partition_requests_balances_cost():
    rng = np.random.default_rng(0)
    lengths = rng.integers(65536, 131073, 256)
    bins = sharding.partition_requests(lengths, 8)
    assert sorted(i for b in bins for i in b) == list(range(256))
    loads = [int(lengths[b].sum()) for b in bins]
    assert max(loads) - min(loads) <= int(lengths.max())
    assert sharding.partition_requests([5, 5, 5], 2) == [[0, 2], [1]]
    assert sharding.partition_requests([], 4) == [[], [], [], []]


def test_shard_bounds_cover_the_sequence():
    for total, world in ((1 << 20, 8), (1000003, 8), (300, 4), (128, 2)):
        spans = [sharding.shard_bounds(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(begin % 128 == 0 or begin == total for begin, _ in spans)


_WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path[:0] = [{root!r}, {root!r} + "/oracle", {root!r} + "/tests"]
import kvip_oracle as oracle
from kvip_b200 import sharding
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
rng = np.random.default_rng(42)
total = 5 * 4096 + 77
whole = rng.integers(-40, 40, (2, total)).astype(np.float32)       # heavy ties across shard borders
begin, end = sharding.shard_bounds(total, world, rank)
def local_topk(scores, length, base):
    idx = oracle.topk(scores.numpy(), np.full(2, length, np.int32), np.full(2, length, np.int32), base)
    sc = np.where(idx >= 0, np.take_along_axis(whole, np.maximum(idx, 0), 1), 0).astype(np.float32)
    return torch.from_numpy(idx), torch.from_numpy(sc)
merge = lambda s, i: torch.from_numpy(oracle.topk_merge(s.numpy(), i.numpy()))
local = torch.from_numpy(np.ascontiguousarray(whole[:, begin:end]))
got = sharding.sequence_sharded_topk(local, end - begin, begin, local_topk=local_topk, merge=merge)
expected = oracle.topk(whole, np.full(2, total, np.int32), np.full(2, total, np.int32))
assert np.array_equal(got.numpy(), expected), "sharded TopK differs from the unsharded one"
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_sequence_shard_exchange_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=str(ROOT)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    for proc in procs:
        out, _ = proc.communicate(timeout=240)
        assert proc.returncode == 0, out


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "decode_16k_b16",
                          "--steps", "1", "--warmup", "3", "--cpu-requests-per-step", "1"], capture_output=True, text=True,
                         timeout=300, check=True).stdout.strip().splitlines()
    assert len(out) == 1
    line = json.loads(out[0])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0


def test_serving_caller_objects_validate_their_inputs():
    """RequestPlan / PagedIndexer of the serving-side caller: host-side checks only."""
    import torch

    from kvip_b200 import PagedIndexer, RequestPlan
    plan = RequestPlan("r", 3, 10, 14, decode=False, start=100, key_end=104)
    assert (plan.owner, plan.begin, plan.stop, plan.query_end, plan.decode, plan.key_end) == (3, 10, 14, 4, False, 104)
    keys = torch.zeros((2, 128, 128), dtype=torch.uint8)
    indexer = PagedIndexer(torch, keys, torch.ones((2, 128), dtype=torch.float32))
    assert indexer.k_cache.kv_cache[0] is keys and tuple(indexer.keys.shape) == (256, 128)
    with pytest.raises(ValueError):
        PagedIndexer(torch, torch.zeros((2, 128, 128), dtype=torch.bfloat16), torch.ones((2, 128)))
    with pytest.raises(ValueError):
        PagedIndexer(torch, keys, torch.ones((2, 128), dtype=torch.float16))
