"""Regenerates the golden vectors under tests/golden/ by RUNNING THE REFERENCE's own CPU code.

Run it only where a checkout of the reference is available; its path is the first argument, or $KVIP_REFERENCE:

    python tests/golden/make_golden.py /path/to/reference [--only=page_updates|ingest_prefill]

What is imported and executed (paths inside the reference project):
  * tests/operators/lifetch/support/workloads.py: prepare_fixture, prepare_full_chain_fixture,
    prepare_compact_fixture (their logical_scores.npy are the reference's score goldens);
  * tests/operators/lifetch/support/correctness.py: validate_topk (kept as a cross-check here);
  * python/kvip/cache/lru.py (+ numba kernels), python/kvip/cache/abc.py (CPU branch),
    python/kvip/cache/page_updates.py (CPU branch);
  * python/kvip/adapters/vllm/inputs.py + index_import.py (QueryInputs, ingest_decode and ingest_prefill on CPU);
  * oracle/_ref/hot_slot_ref: the reference's csrc/operators/lidu/op_kernel/hot_slot_selection.h
    compiled by oracle/Makefile, fed the cases of tests/operators/lidu/test_hot_slot_selection.py.
Only inputs the CUDA path needs and the reference's outputs are stored (compressed .npz); the
reference sources themselves are not copied.
"""
import json
import random
import subprocess
import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]


def li_fixture(workloads, maker, **kwargs):
    with tempfile.TemporaryDirectory() as tmp:
        root = Path(tmp) / "fixture"
        info = maker(root, **kwargs)
        config = json.loads((root / "fixture.json").read_text())
        history, queries, storage = config["history"], config["queries"], config["storage"]
        heads = kwargs.get("index_heads", 64)
        weights_dtype = np.float32
        out = dict(
            query=np.fromfile(root / "arg0.bin", np.uint8).reshape(queries, heads, 128),
            keys=np.fromfile(root / "arg1.bin", np.uint8).reshape(-1, 128)[:storage],
            weights=np.fromfile(root / "arg2.bin", weights_dtype).reshape(queries, heads),
            query_scale=np.fromfile(root / "arg3.bin", np.float32).reshape(queries, heads),
            key_scale=np.fromfile(root / "arg4.bin", np.float32)[:storage],
            logical_scores=np.load(root / "logical_scores.npy"),
            physical_to_logical=np.load(root / "physical_to_logical.npy"),
            history=np.int64(history), resident=np.int64(config["resident"]),
            visible=np.asarray(config["visible_lengths"], np.int64),
        )
        if isinstance(info, dict):
            out["info"] = np.frombuffer(json.dumps(info).encode(), np.uint8)
        return out


def lru_trace(SlotLRU):
    rng = np.random.default_rng(7)
    lru = SlotLRU()
    steps, snapshots = [], []

    def order_of(l):
        out, slot = [], int(l.head[0])
        while slot >= 0:
            out.append(slot)
            slot = int(l.next[0, slot])
        return np.asarray(out, np.int32)

    def snap():
        snapshots.append(dict(slots=lru.slots[0].copy(), order=order_of(lru), version=lru.version, active=lru.active,
                              unique=int(lru.unique[0])))

    for op, a, b in (("resize", 6000, 3000), ("commit", 500, 0), ("commit", 4096, 0), ("resize", 6000, 5000),
                     ("commit", 2048, 0), ("commit", 8192, 0), ("resize", 20000, 16384), ("commit", 8192, 0),
                     ("commit", 3, 0), ("resize", 20000, 100), ("commit", 64, 0), ("resize", 20000, 4000),
                     ("commit", 8192, 0)):
        if op == "resize":
            lru.resize(a, b)
            steps.append(dict(op=op, capacity=a, committed=b, touched=np.zeros(0, np.int32)))
        else:
            touched = rng.integers(0, max(lru.active, 1) + 50, a).astype(np.int32)  # in-contract: no negative slots
            lru.commit(touched)
            steps.append(dict(op=op, capacity=0, committed=0, touched=touched))
        snap()
    return steps, snapshots


def page_updates_fixture(torch):
    """Two submits through the reference's PageUpdates on CPU tensors (its sequential branch): two groups with
    656- and 2624-byte rows, per-token address tables, and map ranges to clear."""
    from kvip.cache.page_updates import PageUpdates
    rng = np.random.default_rng(31)
    owners, groups, pages, block = 3, 2, 8, 128
    addresses = torch.zeros((owners, groups, pages), dtype=torch.int64)
    valid = torch.zeros((owners, groups, pages), dtype=torch.int32)
    token_to_slot = torch.from_numpy(rng.integers(0, 4096, owners * 2048).astype(np.int32))
    fused = [torch.full((owners, pages * block), -7, dtype=torch.int64) for _ in range(groups)]
    updates = PageUpdates(torch, addresses, valid, token_to_slot, fused=fused, widths=(1, 4), token_bytes=656,
                          block_size=block)
    store = dict(map0=token_to_slot.numpy().copy(), shape=np.asarray([owners, groups, pages, block], np.int64))
    for ring in (0, 1):
        indices = rng.permutation(owners * groups * pages)[:11]
        rows = [[int(i), int(rng.integers(1, 1 << 40)) & ~0xFF, int(rng.choice([-1, 128 * int(rng.integers(0, 47))]))]
                for i in indices]
        updates.submit(rows, ring)
        store.update({f"rows{ring}": np.asarray(rows, np.int64), f"addresses{ring}": addresses.numpy().copy(),
                      f"valid{ring}": valid.numpy().copy(), f"map{ring + 1}": token_to_slot.numpy().copy(),
                      f"fused{ring}_0": fused[0].numpy().copy(), f"fused{ring}_1": fused[1].numpy().copy()})
    np.savez_compressed(HERE / "page_updates.npz", **store)


def ingest_prefill_fixture(torch):
    """A mixed batch through the reference's VllmIndexCacheStorage.ingest_prefill on CPU (index_import.py:17-36):
    a request with cached history that is restored once, a fresh prefill, a decode row, and a second forward of the
    first request (its history is not imported again)."""
    from kvip.adapters.vllm.index_import import VllmIndexCacheStorage
    rng = np.random.default_rng(23)
    owners, history, block, blocks = 5, 512, 128, 12
    storage = VllmIndexCacheStorage(torch, owners, history, 256, torch.device("cpu"))
    # few distinct byte values: the fixture compresses well and every row is still distinguishable by its scale
    storage.keys.copy_(torch.from_numpy(rng.integers(0, 4, tuple(storage.keys.shape), dtype=np.uint8)))
    storage.scales.copy_(torch.from_numpy(rng.random(tuple(storage.scales.shape), dtype=np.float32)))
    cache_keys = torch.from_numpy(rng.integers(4, 12, (blocks, block, 1, 128), dtype=np.uint8))
    cache_scales = torch.from_numpy(rng.random((blocks, block, 1), dtype=np.float32))
    table = torch.from_numpy(rng.permutation(blocks).astype(np.int32).reshape(3, 4))
    store = dict(before_keys=storage.keys.numpy().copy(), before_scales=storage.scales.numpy().copy(),
                 cache_keys=cache_keys.numpy(), cache_scales=cache_scales.numpy(), block_table=table.numpy(),
                 block_size=np.int64(block))
    # plan rows: (request, owner, begin, stop, decode, start)
    forwards = [[("a", 3, 0, 40, 0, 300), ("b", 1, 40, 100, 0, 0), ("c", 4, 100, 101, 1, 450)],
                [("a", 3, 0, 25, 0, 340), ("b", 1, 25, 26, 1, 60), ("c", 4, 26, 27, 1, 451)]]
    for step, rows in enumerate(forwards):
        plans = [SimpleNamespace(request=r, owner=o, begin=b, stop=e, decode=bool(d), start=s) for r, o, b, e, d, s in rows]
        storage.prepare(plans)
        tokens = rows[-1][3]
        positions = torch.cat([torch.arange(s, s + (e - b), dtype=torch.int64) for _, _, b, e, _, s in rows])
        slot_mapping = torch.cat([table[i].long()[(positions[b:e] // block)] * block + positions[b:e] % block
                                  for i, (_, _, b, e, _, _) in enumerate(rows)])
        metadata = SimpleNamespace(block_table=table, block_size=block, slot_mapping=slot_mapping)
        storage.ingest_prefill((cache_keys, cache_scales), metadata, plans, positions)
        store.update({f"plans{step}": np.asarray([[o, b, e, d, s] for _, o, b, e, d, s in rows], np.int64),
                      f"requests{step}": np.frombuffer("".join(r for r, *_ in rows).encode(), np.uint8),
                      f"positions{step}": positions.numpy(), f"slot_mapping{step}": slot_mapping.numpy(),
                      f"after_keys{step}": storage.keys.numpy().copy(), f"after_scales{step}": storage.scales.numpy().copy(),
                      f"tokens{step}": np.int64(tokens)})
    np.savez_compressed(HERE / "ingest_prefill.npz", **store)


def main():
    """python tests/golden/make_golden.py REFERENCE_CHECKOUT [--only=NAME]  (or the checkout in $KVIP_REFERENCE)"""
    import os
    arguments = [a for a in sys.argv[1:] if not a.startswith("--only=")]
    only = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--only=")]
    checkout = arguments[0] if arguments else os.environ.get("KVIP_REFERENCE")
    if not checkout:
        raise SystemExit(main.__doc__)
    reference = Path(checkout)
    sys.path[:0] = [str(reference / "python"), str(reference / "tests/operators/lifetch/support")]
    import torch
    if only == ["page_updates"]:  # regenerate this fixture alone
        page_updates_fixture(torch)
        return
    if only == ["ingest_prefill"]:
        ingest_prefill_fixture(torch)
        return
    import workloads
    from correctness import validate_topk

    # ---- LI score / TopK fixtures ------------------------------------------------------------
    exact = li_fixture(workloads, workloads.prepare_fixture, history=4096, resident=2048, queries=4)
    np.savez_compressed(HERE / "li_exact_fixture.npz", **exact)
    causal = li_fixture(workloads, workloads.prepare_fixture, history=4096, resident=2048, queries=4, causal=True)
    np.savez_compressed(HERE / "li_exact_causal_fixture.npz", **causal)
    chain = li_fixture(workloads, workloads.prepare_full_chain_fixture, history=8192, resident=4096, miss_percent=10)
    np.savez_compressed(HERE / "li_full_chain_fixture.npz", **chain)
    # cross-check with the reference's own validity oracle: the unique-cutoff fixture selects a unique set
    bits = chain["logical_scores"].astype(np.uint32) << 16
    scores = bits.view(np.float32)
    ids = np.argsort(-scores, axis=1, kind="stable")[:, :2048]
    validate_topk(ids, scores)
    compact = li_fixture(workloads, workloads.prepare_compact_fixture, history=16384, resident=8192, miss_percent=10,
                         index_heads=32)
    np.savez_compressed(HERE / "li_compact_fixture.npz", **compact)

    # ---- SlotLRU ------------------------------------------------------------------------------
    from kvip.cache.lru import SlotLRU
    steps, snaps = lru_trace(SlotLRU)
    flat = {}
    for i, (step, snapshot) in enumerate(zip(steps, snaps)):
        flat[f"s{i}_op"] = np.frombuffer(step["op"].encode(), np.uint8)
        flat[f"s{i}_args"] = np.asarray([step["capacity"], step["committed"], snapshot["version"], snapshot["active"],
                                         snapshot["unique"]], np.int64)
        flat[f"s{i}_touched"] = step["touched"]
        flat[f"s{i}_slots"] = snapshot["slots"]
        flat[f"s{i}_order"] = snapshot["order"]
    flat["steps"] = np.int64(len(steps))
    np.savez_compressed(HERE / "slot_lru_trace.npz", **flat)

    # ---- ABC maps -------------------------------------------------------------------------------
    from kvip.cache.abc import update_abc
    descriptors = torch.tensor([[[2, 4, 350, 734], [2, 1, 768, 768]], [[0, 3, 383, 390], [0, 2, 128, 140]]],
                               dtype=torch.int32)
    t2s = torch.full((3, 5, 2048), 99, dtype=torch.int32)
    s2t = t2s.clone()
    stages = []
    for shift in (0, 128):
        descriptors[:, :, 2:] += shift
        update_abc(t2s, s2t, descriptors, 2, 1024, 384)
        stages.append((descriptors.numpy().copy(), t2s.numpy().copy(), s2t.numpy().copy()))
    np.savez_compressed(HERE / "abc_maps.npz", d0=stages[0][0], t0=stages[0][1], s0=stages[0][2], d1=stages[1][0],
                        t1=stages[1][1], s1=stages[1][2])

    page_updates_fixture(torch)
    ingest_prefill_fixture(torch)

    # ---- QueryInputs + paged Index ingest --------------------------------------------------------
    from kvip.adapters.vllm.index_import import VllmIndexCacheStorage
    from kvip.adapters.vllm.inputs import QueryInputs
    rng = np.random.default_rng(11)
    batch, history, owners = 3, 512, 6
    inputs = QueryInputs(torch, batch, torch.device("cpu"), pin_memory=False, history=history)
    counts, starts, row_owners = (2, 0, 4), (5, 0, 9), (4, 0, 2)
    inputs.prepare(counts, query_starts=starts, query_owners=row_owners)
    positions = torch.from_numpy(rng.integers(10, history - 1, 32).astype(np.int64))
    inputs.bind_positions(positions)
    storage = VllmIndexCacheStorage(torch, owners, history, 256, torch.device("cpu"))
    cache_keys = torch.from_numpy(rng.integers(0, 256, (8, 128, 1, 128), dtype=np.uint8))
    cache_scales = torch.from_numpy(rng.random((8, 128, 1), dtype=np.float32))
    metadata = SimpleNamespace(slot_mapping=torch.from_numpy(rng.permutation(8 * 128)[:32].astype(np.int64)))
    storage.keys.copy_(torch.from_numpy(rng.integers(0, 256, tuple(storage.keys.shape), dtype=np.uint8)))
    before_keys, before_scales = storage.keys.numpy().copy(), storage.scales.numpy().copy()
    storage.ingest_decode((cache_keys, cache_scales), metadata, inputs, inputs.row_owners)
    np.savez_compressed(
        HERE / "ingest_decode.npz", counts=np.asarray(counts), starts=np.asarray(starts), owners=np.asarray(row_owners),
        metadata=inputs.metadata.numpy(), query_ends=inputs.query_ends.numpy(), positions=positions.numpy(),
        block_table=inputs.block_table.numpy(), cache_keys=cache_keys.numpy(), cache_scales=cache_scales.numpy(),
        slot_mapping=metadata.slot_mapping.numpy(), before_keys=before_keys, before_scales=before_scales,
        after_keys=storage.keys.numpy(), after_scales=storage.scales.numpy(), token_count=np.int64(inputs.token_count))

    # ---- hot-slot bitmap scan, with the reference's own header ---------------------------------------
    binary = ROOT / "oracle" / "_ref" / "hot_slot_ref"
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref", f"REFERENCE={reference}"], check=True)
    rnd = random.Random(21)  # the case list of tests/operators/lidu/test_hot_slot_selection.py:43-51
    cases = []
    for budget in (1, 31, 32, 33, 8192, 16384, 32768):
        for begin in (0, budget // 2, budget - 1):
            protected = {i for i in range(budget) if rnd.random() < 0.65}
            free = sum(1 for i in range(budget) if i not in protected)
            n = min(free, 4096)
            words = [sum(1 << (i % 32) for i in protected if i // 32 == w) for w in range((budget + 31) // 32)]
            cases.append((budget, begin, n, words))
    data = "".join(" ".join(map(str, [b, c, n, *w])) + "\n" for b, c, n, w in cases)
    result = subprocess.run([str(binary)], input=data, text=True, capture_output=True, check=True)
    store = {"cases": np.int64(len(cases))}
    for i, ((budget, begin, n, words), line) in enumerate(zip(cases, result.stdout.splitlines())):
        store[f"c{i}_args"] = np.asarray([budget, begin, n], np.int64)
        store[f"c{i}_words"] = np.asarray(words, np.uint32)
        store[f"c{i}_slots"] = np.asarray(list(map(int, line.split())), np.int32)
    np.savez_compressed(HERE / "hot_slot_scan.npz", **store)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
