#!/usr/bin/env python
"""Benchmark of the LI -> TopK -> resolve -> Index exchange -> fetch -> gather decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line. Metric: query tokens/s of the decode step at 128k context (workload
`decode_128k_b64`: batch 64 per GPU, 1 query token per request, 64 heads x 128, FP8 Index keys with
per-token scales, TopK 2048, 25 % resident pool of 1152-byte KV rows, dense gather of the selected rows).
Requests are partitioned over GPUs (one process per GPU, no data-path collective): weak scaling.
`value` times CUDA-graph replays of the step with every input resident in HBM; `e2e` times the public
API with host inputs (pinned H2D of the step's queries and positions, D2H of the slot/logical outputs).
`--impl reference` times the reference's CPU golden path (the oracle restatement) on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # the headline: BASELINE.json metric (128k context, batch 64 on one B200)
    "decode_128k_b64": dict(batch=64, queries=1, heads=64, history=131072, resident=32768, len_lo=131072,
                            len_hi=131072, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152),
    # configs[1]: decode LI+TopK, B=64, 2 MTP tokens, ctx U[16k,32k]
    "decode_32k_b64_mtp2": dict(batch=64, queries=2, heads=64, history=32768, resident=8192, len_lo=16384,
                                len_hi=32768, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152),
    # one GPU's share of the 8-GPU serving configuration: 256 requests over 8 GPUs, ctx U[64k,128k], 50 % pool
    "decode_64k_128k_b32": dict(batch=32, queries=1, heads=64, history=131072, resident=65536, len_lo=65536,
                                len_hi=131072, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152),
    # small cases for profiler captures and smoke runs
    "decode_16k_b16": dict(batch=16, queries=1, heads=64, history=16384, resident=4096, len_lo=16384, len_hi=16384,
                           key_dtype="fp8", weight_dtype="bf16", token_bytes=1152),
    "decode_128k_b8": dict(batch=8, queries=1, heads=64, history=131072, resident=32768, len_lo=131072,
                           len_hi=131072, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152),
    "decode_64k_b16_mtp2": dict(batch=16, queries=2, heads=64, history=65536, resident=8192, len_lo=65536, len_hi=65536,
                                key_dtype="fp8", weight_dtype="bf16", token_bytes=1152),
}
METRIC = "LI+TopK+Fetch query tokens/s at 128k ctx"


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, maxes, reasons = [], [], set()
        for line in out.splitlines():
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 9:
                continue
            try:
                clocks.append(float(cells[1]))
                maxes.append(float(cells[2]))
            except ValueError:
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), cells[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            self.result = {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxes), "reasons": sorted(reasons),
                           "samples": len(clocks)}


def li_algorithmic_bytes(lengths, queries, heads, key_bytes):
    """Bytes the LI kernel must move per launch: every request's keys and key scales once, the query rows with
    their head weights and query scales, and the fp32 score rows it writes."""
    keys = sum(int(n) * (128 * key_bytes + 4) for n in lengths)
    tokens = len(lengths) * queries
    query = tokens * heads * (128 * key_bytes + 2 + 4)
    scores = sum(int(n) * 4 * queries for n in lengths)
    return keys + query + scores


def time_region(torch, stream, fn, steps):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / 1e3


def time_blocks(torch, stream, fn, steps, first_block_s, *, least=10, most=200, target_s=1.0):
    """Back-to-back blocks of `steps` calls, each between its own pair of CUDA events. A block of 20 replays lasts a
    few milliseconds, less than one sample of the clock monitor and short enough for one stray clock step to move
    it: enough blocks are timed to fill about a second, and the caller reports their median, minimum and maximum."""
    count = max(least, min(most, int(target_s / max(first_block_s, 1e-6)) + 1))
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(count + 1)]
    marks[0].record(stream)
    for block in range(count):
        for _ in range(steps):
            fn()
        marks[block + 1].record(stream)
    marks[-1].synchronize()
    return [marks[i].elapsed_time(marks[i + 1]) / 1e3 for i in range(count)]


def run_ours(args):
    import torch
    import torch.distributed as dist

    from kvip_b200 import _lib, ops
    from decode_harness import DecodePipeline

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = dict(WORKLOADS[args.workload])
    if args.batch:
        cfg["batch"] = args.batch
    lib = _lib.load_library()
    miss_source = "device tensor" if args.device_source else "pinned mapped host pool"
    try:
        p = DecodePipeline(device, seed=rank, gather=True, host_pool=not args.device_source, **cfg)
    except (RuntimeError, MemoryError) as failure:
        # the host pool of one rank is owners x history x token_bytes (9.7 GB at the headline): when the box cannot
        # pin that much for every rank, the miss rows come from a device tensor instead, and the line says so
        if args.device_source:
            raise
        torch.cuda.empty_cache()
        p = DecodePipeline(device, seed=rank, gather=True, host_pool=False, **cfg)
        miss_source = f"device tensor (host pool unavailable: {str(failure)[:80]})"
    stream = torch.cuda.Stream(device)
    tokens = p.query_tokens()

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    with torch.cuda.stream(stream):
        # cold start: the first step fetches every selected row from the host pool
        t0 = time.perf_counter()
        p.step()
        stream.synchronize()
        cold_s = time.perf_counter() - t0
        cold_reads = int(p.rotating.query_counts[:, 4].sum().item())
        for _ in range(max(args.warmup - 1, 2)):
            p.step()
        stream.synchronize()
        status = int(p.forward.li_status.item()) | int(p.update.status.max().item())
        if status:
            raise RuntimeError(f"device status {status} during warm-up")
        before = lib.kvip_b200_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            p.step()
        launches_per_step = lib.kvip_b200_launch_count() - before
        for _ in range(2):
            graph.replay()
        barrier()

        def soak(seconds):  # the same replays, long enough for the 100 ms clock sampler to see the load
            end = time.perf_counter() + seconds
            while time.perf_counter() < end:
                for _ in range(20):
                    graph.replay()
                stream.synchronize()

        first_block = time_region(torch, stream, graph.replay, args.steps)
        with ClockSampler(local) as clocks:
            soak(0.3)
            barrier()
            block_seconds = time_blocks(torch, stream, graph.replay, args.steps, first_block,
                                        **(dict(least=1, most=1) if args.quick else {}))
            barrier()
            soak(0.3)
        steady_reads = int(p.rotating.query_counts[:, 4].sum().item())
        if args.quick:   # profiler captures: the warm-up and the timed replays only
            median = sorted(block_seconds)[len(block_seconds) // 2]
            if rank == 0:
                print(json.dumps({"metric": METRIC, "value": world * tokens * args.steps / median, "unit": "tokens/s",
                                  "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                                  "ms_per_step": median / args.steps * 1e3, "config": {"workload": args.workload, "quick": True},
                                  "gpu_launches": launches_per_step * args.steps, "cold_step_reads": cold_reads}), flush=True)
            p.close()
            if world > 1:
                dist.destroy_process_group()
            return
        blocks = torch.tensor(block_seconds, dtype=torch.float64, device=device)
        if world > 1:   # every block as slow as its slowest rank (all ranks time the same number of blocks)
            counts = torch.tensor([len(block_seconds)], dtype=torch.int64, device=device)
            dist.all_reduce(counts, op=dist.ReduceOp.MIN)
            blocks = blocks[: int(counts.item())].contiguous()
            dist.all_reduce(blocks, op=dist.ReduceOp.MAX)
        block_seconds = sorted(blocks.tolist())
        elapsed = block_seconds[len(block_seconds) // 2]   # the median block of `steps` replays

        # ---- per-stage device time (each stage alone, K launches, inputs larger than L2) ------------
        inputs, s, r, ws = p.workspace.inputs, p.storage, p.rotating, p.workspace
        stages = {}
        qe2d = inputs.query_ends.view(p.batch, p.queries)
        keys_view = s.keys.view(torch.float8_e4m3fn) if p.key_dtype == "fp8" else s.keys
        li = lambda: ops.li_score(inputs.query, keys_view.view(-1, 128), inputs.weights,  # noqa: E731
                                  inputs.scale if p.key_dtype == "fp8" else None,
                                  s.scales.view(-1) if p.key_dtype == "fp8" else None, ws.key_lengths, qe2d,
                                  inputs.block_table, ws.scores, status=p.forward.li_status)
        tk = lambda: ops.topk(ws.scores, ws.key_lengths, inputs.query_ends, ws.topk.view(-1, 2048))  # noqa: E731
        ga = lambda: ops.gather(p.pool_hbm, p.update.slot_output.view(-1, 2048), p.gather_out,  # noqa: E731
                                queries=p.queries, output_stride=p.output_stride, token_bytes=p.token_bytes,
                                row_owners=inputs.row_owners)
        split_scratch = torch.zeros((p.batch * p.queries, _lib.TOPK_SPLIT_WORDS), dtype=torch.int32, device=device)
        histogram = torch.zeros((p.batch * p.queries, 4096), dtype=torch.int32, device=device)
        tk_hist = lambda: ops.topk(ws.scores, ws.key_lengths, inputs.query_ends, ws.topk.view(-1, 2048),  # noqa: E731
                                   histogram=histogram)
        tk_split = lambda: ops.topk(ws.scores, ws.key_lengths, inputs.query_ends, ws.topk.view(-1, 2048),  # noqa: E731
                                    split_scratch=split_scratch)
        lru = lambda: p.lru.commit(p.update.slot_output.view(p.batch, -1))  # noqa: E731
        for name, fn in (("li_score", li), ("topk", tk), ("topk_histogram_select", tk_hist), ("topk_all_passes_split", tk_split),
                         ("gather", ga), ("lru_commit", lru)):
            for _ in range(2):
                fn()
            stream.synchronize()
            stages[name] = time_region(torch, stream, fn, args.steps) / args.steps
        stages["step_graph"] = elapsed / args.steps
        stages["resolve_outputs_exchange_fetch"] = max(0.0, stages["step_graph"] - stages["li_score"] - stages["topk"]
                                                       - stages["gather"] - stages["lru_commit"])

        # ---- end to end: host inputs in, host outputs out, through the public objects ----------------
        heads, T = p.heads, tokens
        host_q = torch.empty((T, heads, 128), dtype=torch.uint8).pin_memory()
        host_q.copy_(inputs.query.view(torch.uint8).cpu())
        host_w = inputs.weights.cpu().pin_memory()
        host_s = inputs.scale.cpu().pin_memory()
        host_pos = p.positions.cpu().pin_memory()
        dev_q = torch.empty_like(host_q, device=device).view(torch.float8_e4m3fn)
        dev_w, dev_s, dev_pos = (torch.empty_like(x, device=device) for x in (host_w, host_s, host_pos))
        host_out = torch.empty((2, T, 1, 2048), dtype=torch.int32).pin_memory()

        def serial_step():  # everything on one stream, one after the other
            dev_q.view(torch.uint8).copy_(host_q, non_blocking=True)
            dev_w.copy_(host_w, non_blocking=True)
            dev_s.copy_(host_s, non_blocking=True)
            dev_pos.copy_(host_pos, non_blocking=True)
            inputs.bind_positions(dev_pos)
            inputs.pack(dev_q, dev_w, dev_s)
            graph.replay()  # the captured step: forward + LRU feedback
            host_out.copy_(p.update.outputs, non_blocking=True)

        for _ in range(3):
            serial_step()
        barrier()
        serial_elapsed = time_region(torch, stream, serial_step, args.steps)
        barrier()

        # the same work per step through HostDecodeLoop: copies overlap the neighbouring steps' kernels
        from kvip_b200 import HostDecodeLoop
        loop = HostDecodeLoop(torch, p.forward, inputs, p.update.outputs, host_query=host_q.view(torch.float8_e4m3fn),
                              host_weights=host_w, host_scale=host_s, host_positions=host_pos, host_outputs=host_out)

        def looped_steps():
            loop.step()
            if loop.steps % args.steps == 0:
                loop.drain()  # the timed region ends when the last read-back has landed

        for _ in range(3):
            loop.step()
        loop.drain()
        loop.steps = 0
        barrier()
        e2e_elapsed = time_region(torch, stream, looped_steps, args.steps)
        barrier()
        h2d = sum(x.numel() * x.element_size() for x in (host_q, host_w, host_s, host_pos))
        d2h = host_out.numel() * host_out.element_size()

        miss_path = None
        if world == 1 and not args.no_miss_path:
            miss_path = measure_miss_path(torch, ops, p, stream, args)

    worst = torch.tensor([e2e_elapsed, serial_elapsed], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    e2e_elapsed, serial_elapsed = (float(x) for x in worst.tolist())
    hbm_peak, peak_kind = peaks()
    key_bytes = 1 if p.key_dtype == "fp8" else 2
    li_bytes = li_algorithmic_bytes(p.lengths, p.queries, p.heads, key_bytes)
    achieved = li_bytes / stages["li_score"] / 1e9
    step_bytes = li_bytes + 2 * tokens * 2048 * p.token_bytes  # + dense gather read and write
    line = {
        "metric": METRIC, "value": world * tokens * args.steps / elapsed, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32",
        "data": "synthetic",
        "blocks": {"count": len(block_seconds), "steps_per_block": args.steps, "reported": "median block",
                   "min_ms_per_step": block_seconds[0] / args.steps * 1e3,
                   "max_ms_per_step": block_seconds[-1] / args.steps * 1e3,
                   # time x clock: comparable between a box at full clock and one under its power cap
                   "median_ms_x_sm_mhz": (elapsed / args.steps * 1e3 * clocks.result["sm_mhz"]
                                          if clocks.result.get("sm_mhz") else None)},
        "config": {"workload": args.workload, "batch_per_gpu": p.batch, "queries_per_request": p.queries,
                   "context": int(p.lengths.max()), "index_heads": p.heads, "topk": 2048,
                   "resident_slots": p.resident, "token_bytes": p.token_bytes, "cuda_graph": True,
                   "partition": "by request, no collective",
                   "l2": "inputs larger than L2 (keys %.0f MB per step)" % (li_bytes / 1e6),
                   "miss_source": miss_source,
                   "steady_state": "the captured step is replayed with fixed queries: after warm-up every selected row "
                                   "is resident, the timed steps fetch nothing from the host pool and 'Fetch' is the "
                                   "dense gather of 2048 resident rows per query; value_with_misses is the same step "
                                   "with drifting queries"},
        "e2e": {"value": world * tokens * args.steps / e2e_elapsed, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_elapsed / args.steps * 1e3,
                "api": "HostDecodeLoop.step: copies of steps i-1 / i+1 overlap the kernels of step i",
                "one_stream": {"value": world * tokens * args.steps / serial_elapsed,
                               "ms_per_step": serial_elapsed / args.steps * 1e3}},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"kernel": "li_score_tcgen05", "bound": "hbm", "achieved": achieved, "peak": hbm_peak,
                     "unit": "GB/s", "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": li_bytes, "us_per_launch": stages["li_score"] * 1e6,
                     # dram__bytes_read.sum + dram__bytes_write.sum of this kernel on THIS workload: a one-pass ncu
                     # capture of three full-size launches (1108.8 MB read + 30.5-34.6 MB written each); other
                     # workloads have no capture
                     "traffic": 1140829269 if args.workload == "decode_128k_b64" and p.key_dtype == "fp8" else None,
                     "traffic_kind": "measured on this workload: dram__bytes_read.sum + dram__bytes_write.sum per launch, "
                                     "mean of three launches of a one-pass ncu capture (0.9995 x the algorithmic bytes)",
                     "step_frac": step_bytes / stages["step_graph"] / 1e9 / hbm_peak},
        "stages_us": {k: v * 1e6 for k, v in stages.items()},
        "fetch": {"cold_step_reads": cold_reads, "cold_step_ms": cold_s * 1e3,
                  "cold_host_link_gbs": cold_reads * p.token_bytes / cold_s / 1e9, "steady_reads_per_step": steady_reads},
        "clocks": clocks.result,
    }
    if miss_path:
        line["miss_path"] = miss_path
        line["value_with_misses"] = {"value": world * miss_path["tokens_per_s"], "unit": "tokens/s",
                                     "ms_per_step": miss_path["ms_per_step"], "miss_fraction": miss_path["miss_fraction"],
                                     "note": "drifting queries, misses read from the pinned host pool inside the step"}
    if rank == 0:
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(cfg, args.cpu_requests)
        print(json.dumps(line), flush=True)
    p.close()
    if world > 1:
        dist.destroy_process_group()


def measure_miss_path(torch, ops, p, stream, args):
    """Steps whose selections drift (AR(1) queries), so that part of every selection misses the resident pool
    and is fetched from the pinned host pool, with the Index update of one new bf16 row per token in the
    step; plus the host link alone (the fetch kernel over synthetic descriptors)."""
    from kvip_b200 import LIFetch

    steps, warm = 8, 4
    p.make_query_bank(2 * (steps + warm), correlation=0.95)

    def drifting(first):
        for i in range(warm):
            p.load_queries(first + i)
            p.step(ingest=True)
        stream.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        counts = torch.zeros(steps, dtype=torch.int64, device=p.device)
        start.record(stream)
        for i in range(steps):
            p.load_queries(first + warm + i)
            p.step(ingest=True)
            counts[i] = p.rotating.query_counts[:, 4].sum()
        stop.record(stream)
        stop.synchronize()
        return start.elapsed_time(stop) / 1e3, counts.tolist()

    serial_seconds, serial_misses = drifting(0)
    # the same pipeline with the commit phase overlapped: a second call object over the same state (the first one is
    # not used again: the bindings now name the new object's workspace record)
    p.forward = LIFetch(p.rotating, p.update, lru=p.lru, overlap_fetch=True)
    seconds, misses = drifting(steps + warm)
    status = int(p.update.status.max().item()) | int(p.rotating.row_status[:, 2].max().item())
    out = {"steps": steps, "ms_per_step": seconds / steps * 1e3, "tokens_per_s": p.query_tokens() * steps / seconds,
           "misses_per_step": sum(misses) / steps, "miss_fraction": sum(misses) / steps / (p.query_tokens() * 2048),
           "miss_bytes_per_step": sum(misses) / steps * p.token_bytes, "status": status,
           "commit_phase": "overlapped (LIFetch(overlap_fetch=True)): outputs, Index exchange and the gather of hit "
                           "entries on a side stream beside the fetch",
           "serial_commit_phase": {"ms_per_step": serial_seconds / steps * 1e3,
                                   "misses_per_step": sum(serial_misses) / steps,
                                   "note": "the two variants run consecutive pieces of one drifting stream, so their miss "
                                           "counts differ; --workload decode_128k_b32_zipf compares them on identical "
                                           "selections"},
           "query_drift": "AR(1), rho = 0.95, new bf16 k_I row per token quantised to FP8; eager launches"}
    if p.host_pool is not None:
        # host link alone: 16384 rows per request from distinct host rows into the resident slots
        rows = min(8192, p.resident)
        state = ops.ResolveState(p.batch, p.queries, p.device)
        gen = torch.Generator(device=p.device)
        gen.manual_seed(5)
        tokens = torch.stack([torch.randperm(p.history, generator=gen, device=p.device)[:rows] for _ in range(p.batch)])
        owners = p.workspace.inputs.row_owners.long()[:, None]
        state.fetch_sources[:, :rows] = (owners * p.history + tokens) * p.token_bytes
        state.fetch_destinations[:, :rows] = (owners * p.output_stride + torch.arange(rows, device=p.device)[None, :]).int()
        state.query_counts[:, 4] = rows
        valid = torch.zeros_like(p.storage.hot_valid)
        fetch = lambda: ops.fetch(p.host_pool.device_pointer, p.host_pool.nbytes, p.pool_hbm, valid, state,  # noqa: E731
                                  resident=p.resident, output_stride=p.output_stride, token_bytes=p.token_bytes,
                                  row_owners=p.workspace.inputs.row_owners)
        fetch()
        stream.synchronize()
        t = time_region(torch, stream, fetch, 3) / 3
        out["host_link"] = {"rows": rows * p.batch, "bytes": rows * p.batch * p.token_bytes, "ms": t * 1e3,
                            "gbs": rows * p.batch * p.token_bytes / t / 1e9}
    return out


def zipf_selections(rng, length, steps, reuse, exponent=1.1):
    """`steps` selections of 2048 logical tokens of one request (NumPy, host). Every selection is an ordered list:
    index = score rank. Selection k keeps `reuse` of selection k-1, sampled without replacement with probability
    proportional to rank^-exponent (a high-ranked token is likelier to be selected again), and fills up with
    tokens drawn uniformly from the rest of the context; kept tokens stay in rank order ahead of the new ones."""
    import numpy as np
    keep = int(round(2048 * reuse))
    weights = np.arange(1, 2049, dtype=np.float64) ** -exponent
    weights /= weights.sum()
    lists = [rng.choice(length, 2048, replace=False)]
    for _ in range(steps - 1):
        previous = lists[-1]
        kept = previous[np.sort(rng.choice(2048, keep, replace=False, p=weights))]
        taken = np.zeros(length, dtype=bool)
        taken[previous] = True                       # new tokens come from outside the previous selection
        fresh = rng.choice(np.flatnonzero(~taken), 2048 - keep, replace=False)
        lists.append(np.concatenate((kept, fresh)))
    return np.stack(lists)


def zipf_variant(torch, device, stream, cfg, chosen_host, steps, warm, overlap):
    """One pipeline of the Zipf-reuse workload (commit phase serial or overlapped): timed steps, a second pass with
    stage stamps, an end-to-end pass. Returns the measurements as a dict."""
    from decode_harness import DecodePipeline
    from kvip_b200 import ops

    lib = _load_counter()
    local = device.index or 0
    with torch.cuda.stream(stream):
        p = DecodePipeline(device, seed=0, gather=True, host_pool=True, overlap_fetch=overlap, **cfg)
        chosen = torch.from_numpy(chosen_host).to(device)                 # [total, B, 2048] logical tokens
        inputs, s, ws = p.workspace.inputs, p.storage, p.workspace
        owners = inputs.row_owners.long()
        tokens_now = torch.zeros((p.batch, 2048), dtype=torch.int64, device=device)   # static: read by the graph
        inverse = torch.zeros((p.batch, p.history), dtype=torch.int64, device=device)
        positions = torch.zeros((p.batch, 2048), dtype=torch.int64, device=device)
        arange = torch.arange(p.history, dtype=torch.int64, device=device).expand(p.batch, -1).contiguous()
        boost = torch.full((p.batch, 2048), 3.0e38, dtype=torch.float32, device=device)
        keys_view = s.keys.view(torch.float8_e4m3fn).view(-1, 128)
        qe2d = inputs.query_ends.view(p.batch, p.queries)

        def steer():  # where does each chosen logical token sit now, and lift its score
            inverse.scatter_(1, s.logical_ids[owners], arange)
            torch.gather(inverse, 1, tokens_now, out=positions)
            ws.scores.scatter_(1, positions, boost)

        def step():
            p.ingest_new_tokens()
            ops.li_score(inputs.query, keys_view, inputs.weights, inputs.scale, s.scales.view(-1), ws.key_lengths, qe2d,
                         inputs.block_table, ws.scores, status=p.forward.li_status)
            steer()
            p.forward(scores_ready=True)

        def run(index, replay):
            tokens_now.copy_(chosen[index])
            replay()

        for i in range(2):     # eager: lazy set-up outside capture
            run(i, step)
        stream.synchronize()
        before = lib.kvip_b200_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        launches_per_step = lib.kvip_b200_launch_count() - before
        for i in range(2, warm):
            run(i, graph.replay)
        stream.synchronize()
        misses = torch.zeros(steps, dtype=torch.int64, device=device)
        with ClockSampler(local) as clocks:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for k in range(steps):
                run(warm + k, graph.replay)
                misses[k] = p.rotating.query_counts[:, 4].sum()
            stop.record(stream)
            stop.synchronize()
        seconds = start.elapsed_time(stop) / 1e3
        status = (int(p.update.status.abs().max().item()) | int(p.rotating.row_status[:, 0].abs().max().item())
                  | int(p.rotating.row_status[:, 2].abs().max().item()) | int(p.forward.li_status.item()))
        selected = torch.sort(p.update.logical_output.view(p.batch, 2048).long(), dim=1).values
        verified = bool(torch.equal(selected, torch.sort(chosen[warm + steps - 1], dim=1).values))
        harness = time_region(torch, stream, steer, 20) / 20
        # the same chain, as many steps again, with the call's own stage stamps (a profiling pass: extra launches)
        p.forward.set_options(diagnostics=True)
        stage_sum, link = {}, []
        for k in range(steps):
            run(warm + steps + k, step)
            stream.synchronize()
            stamps = p.forward.times[:8].cpu().tolist()
            count = int(p.rotating.query_counts[:, 4].sum().item())
            # serial: the fetch starts when the exchange has finished; overlapped: when the resolver has
            fetch_us = (stamps[6] - (stamps[3] if overlap else stamps[5])) / 1e3
            for name, value in (("li_to_resolve", (stamps[3] - stamps[0]) / 1e3), ("fetch", fetch_us),
                                ("resolve_to_end", (stamps[7] - stamps[3]) / 1e3), ("total", (stamps[7] - stamps[0]) / 1e3)):
                stage_sum[name] = stage_sum.get(name, 0.0) + value / steps
            if fetch_us > 0:
                link.append(count * p.token_bytes / (fetch_us * 1e-6) / 1e9)
        p.forward.set_options()
        # end to end: the step fed from and drained to pinned host memory on one stream
        T = p.query_tokens()
        host_q = inputs.query.view(torch.uint8).cpu().pin_memory()
        host_out = torch.empty((2, T, 1, 2048), dtype=torch.int32).pin_memory()
        host_tokens = chosen[warm + 2 * steps:warm + 3 * steps].cpu().pin_memory()   # the chain goes on: new misses

        def e2e_steps():
            for k in range(steps):
                inputs.query.view(torch.uint8).copy_(host_q, non_blocking=True)
                tokens_now.copy_(host_tokens[k], non_blocking=True)
                graph.replay()
                host_out.copy_(p.update.outputs, non_blocking=True)

        e2e_seconds = time_region(torch, stream, e2e_steps, 1)
    miss_list = misses.tolist()
    result = dict(seconds=seconds, e2e_seconds=e2e_seconds, misses=miss_list, status=status, verified=verified,
                  harness_us=harness * 1e6, stages_us=stage_sum, link_gbs=(sum(link) / len(link)) if link else None,
                  launches_per_step=launches_per_step, clocks=clocks.result, tokens=T, lengths=p.lengths.copy(),
                  h2d=host_q.numel() + 2048 * 8 * p.batch, d2h=host_out.numel() * 4)
    p.close()
    del p, graph
    torch.cuda.empty_cache()
    return result


def run_zipf(args):
    """`--workload decode_128k_b32_zipf`: the full decode step WITH misses of the benchmark configurations - batch 32,
    131072-token context, FP8 Index keys, TopK 2048, a resident pool of 25 % of the context (32768 slots of 1152
    bytes), misses read from the pinned, mapped host pool, LRU feedback, and one new bf16 Index row per token
    quantised to FP8; 8 timed steps whose selections reuse the previous step's tokens with Zipf(1.1) rank weights.

    The selection is steered by biasing the scores (no trace of real queries ships with the reference): every step
    runs the real score kernel over the whole context, then the harness raises the scores of the step's chosen
    tokens above all others (three small torch ops: inverse of the Index permutation, position lookup, scatter) and
    the fused call continues from those score rows (KVIP_OPTION_SCORES_READY): TopK, resolver, Index exchange,
    fetch, gather and LRU feedback are the product path on real state. The whole step is one CUDA graph; the
    step's token list is copied into a static buffer before each replay. The harness ops are timed alone and
    reported so that their share can be subtracted. Measured twice, on the same selections: with the commit phase
    on one stream, and with `LIFetch(overlap_fetch=True)`; `value` is the overlapped variant."""
    import numpy as np
    import torch

    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    stream = torch.cuda.Stream(device)
    steps, warm = 8, max(args.warmup, 4)
    cfg = dict(batch=args.batch or 32, queries=1, heads=64, history=131072, resident=32768, len_lo=131072,
               len_hi=131072, key_dtype="fp8", weight_dtype="bf16", token_bytes=1152)
    rng = np.random.default_rng(0)
    total = warm + 3 * steps   # warm-up, the timed steps, as many with stage stamps, as many fed from the host
    chosen = np.stack([zipf_selections(rng, cfg["len_hi"], total, args.reuse) for _ in range(cfg["batch"])], axis=1)
    # the first pipeline of a process reads the freshly pinned host pool several times slower than later ones
    # (mapping warm-up of the host link): it is run and dropped
    zipf_variant(torch, device, stream, cfg, chosen, steps, warm, overlap=False)
    serial = zipf_variant(torch, device, stream, cfg, chosen, steps, warm, overlap=False)
    best = zipf_variant(torch, device, stream, cfg, chosen, steps, warm, overlap=True)
    T, seconds = best["tokens"], best["seconds"]
    per_step = sum(best["misses"]) / steps
    li_bytes = li_algorithmic_bytes(best["lengths"], cfg["queries"], cfg["heads"], 1)
    print(json.dumps({
        "metric": METRIC + ", with misses (Zipf reuse)", "value": T * steps / seconds, "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warm, "ms_per_step": seconds / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": {"workload": args.workload, "batch_per_gpu": cfg["batch"], "context": cfg["len_hi"], "topk": 2048,
                   "resident_slots": cfg["resident"], "token_bytes": cfg["token_bytes"], "cuda_graph": True,
                   "reuse_of_previous_selection": args.reuse, "zipf_exponent": 1.1,
                   "selection": "scores of the step's chosen tokens raised after the real score pass",
                   "index_update": "one new bf16 row per token quantised to FP8, every step",
                   "commit_phase": "overlapped: outputs, exchange and the gather of hit entries beside the fetch",
                   "l2": "inputs larger than L2 (keys %.0f MB per step)" % (li_bytes / 1e6),
                   "miss_source": "pinned mapped host pool"},
        "misses_per_step": per_step, "misses_by_step": best["misses"], "miss_fraction": per_step / (T * 2048),
        "miss_bytes_per_step": per_step * cfg["token_bytes"], "status": best["status"] | serial["status"],
        "selection_verified": best["verified"] and serial["verified"],
        "same_misses_in_both_variants": best["misses"] == serial["misses"],
        "harness_us_per_step": best["harness_us"], "stages_us": best["stages_us"],
        "serial_commit_phase": {"ms_per_step": serial["seconds"] / steps * 1e3, "tokens_per_s": T * steps / serial["seconds"],
                                "stages_us": serial["stages_us"], "host_link_gbs_inside_the_step": serial["link_gbs"]},
        "host_link": {"gbs_inside_the_step": best["link_gbs"],
                      "how": "missing bytes of a step / device time of its fetch stage (the call's stage stamps), mean "
                             "over the steps of the stamped pass"},
        "e2e": {"value": T * steps / best["e2e_seconds"], "unit": "tokens/s", "h2d_bytes_per_step": best["h2d"],
                "d2h_bytes_per_step": best["d2h"], "ms_per_step": best["e2e_seconds"] / steps * 1e3},
        "gpu_launches": best["launches_per_step"] * steps,
        "roofline": {"kernel": "fetch_rows", "bound": "host link", "achieved": best["link_gbs"], "peak": None,
                     "unit": "GB/s", "frac": None, "traffic": None,
                     "note": "the step is bound by the host link; its HBM-bound part is reported by decode_128k_b64"},
        "clocks": best["clocks"],
    }), flush=True)


def cpu_step(cfg, requests, seed=0, budget_s=1e9):
    """One pass of the reference's CPU golden path over `requests` requests of the workload:
    NumPy einsum LI (tests/operators/lifetch/support/workloads.py:406-413 in the reference), canonical
    TopK, resolver, Index exchange, row fetch and gather. Returns (seconds, query tokens)."""
    import numpy as np
    sys.path.insert(0, str(ROOT / "oracle"))
    import kvip_oracle as oracle

    rng = np.random.default_rng(seed)
    heads, history, resident, queries = cfg["heads"], cfg["history"], cfg["resident"], cfg["queries"]
    token_bytes = cfg["token_bytes"]
    keys = oracle.encode_e4m3(np.clip(rng.standard_normal((history, 128), dtype=np.float32) * 8, -448, 448))
    key_scale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), history)).astype(np.float32)
    query = oracle.encode_e4m3(np.clip(rng.standard_normal((queries, heads, 128), dtype=np.float32) * 8, -448, 448))
    qscale = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), (queries, heads))).astype(np.float32)
    weights = oracle.f32_to_bf16_rne((rng.standard_normal((queries, heads)) / 8).astype(np.float32))
    length = cfg["len_hi"]
    ends = np.array([[max(1, length - (queries - 1 - q)) for q in range(queries)]], np.int32)
    table = np.arange(history // 128, dtype=np.int32).reshape(1, -1)
    pool = np.zeros((resident, token_bytes), np.uint8)
    host = np.zeros((history, token_bytes), np.uint8)
    scales = key_scale.copy()
    addresses = np.arange(history, dtype=np.int64) * token_bytes
    logical = np.arange(history, dtype=np.int64)
    lru = oracle.SlotLRUOracle()
    lru.resize(resident, resident)
    hot_valid = np.ones(resident, np.int32)
    start = time.perf_counter()
    done = 0
    while done < requests and (done == 0 or time.perf_counter() - start < budget_s):
        done += 1
        scores = oracle.li_scores(query, keys, weights, qscale, scales, np.array([length], np.int32), ends, table)
        selected = oracle.topk(scores, np.array([length], np.int32), ends)
        ref = oracle.resolve_request(selected, hot_valid, lru.reserved_hot(resident), lru.slots, history, resident)
        sources = addresses[ref["events_src"]]
        oracle.exchange_request(keys, scales, addresses, logical, hot_valid, ref["events_src"], ref["events_dst"],
                                ref["counts"], history, resident)
        oracle.fetch_request(pool, hot_valid, host.reshape(-1), sources, ref["events_dst"], 0, resident, resident,
                             token_bytes)
        oracle.gather(pool, ref["locations"], np.zeros(1, np.int64), queries, resident)
        lru.commit(ref["locations"].reshape(-1))
    return time.perf_counter() - start, done * queries


def cpu_baseline(cfg, requests):
    seconds, tokens = cpu_step(cfg, requests, budget_s=15.0)
    return {"value": tokens / seconds, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{tokens // cfg['queries']} requests of the workload (1 step each, about 15 s of CPU work), NumPy "
                      f"golden LI + TopK + resolver + exchange + fetch + gather, {seconds:.2f} s"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(WORKLOADS[args.workload])
    for _ in range(min(args.warmup, 1)):
        cpu_step(cfg, 1)
    seconds, tokens = 0.0, 0
    for step in range(args.steps):
        s, t = cpu_step(cfg, args.cpu_requests_per_step, seed=step)
        seconds, tokens = seconds + s, tokens + t
    value = tokens / seconds
    sample = (f"{args.cpu_requests_per_step} request(s) of the workload per step instead of {cfg['batch']}; "
              f"NumPy golden LI + TopK + resolver + exchange + fetch + gather")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (NumPy)", "data": "synthetic",
        "config": {"workload": args.workload, "context": cfg["len_hi"], "queries_per_request": cfg["queries"],
                   "index_heads": cfg["heads"], "topk": 2048, "resident_slots": cfg["resident"],
                   "token_bytes": cfg["token_bytes"]},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def measure_fp8_peak(torch, device, local):
    """Dense FP8 (e4m3 x e4m3 -> bf16) tensor throughput of this GPU, measured the way the bf16 figure of
    MEASURED_PEAKS.json was: torch._scaled_mm (cuBLASLt) on 8192^3, best of 10 as the burst figure and a
    four-second back-to-back loop as the sustained one, with the SM clock sampled during the loop. Only a
    denominator for the roofline of the prefill workload: nothing of the product path calls it."""
    n = 8192
    a = (torch.randn((n, n), device=device) * 0.5).to(torch.float8_e4m3fn)
    b = (torch.randn((n, n), device=device) * 0.5).to(torch.float8_e4m3fn).t()    # column-major operand
    one = torch.ones((), dtype=torch.float32, device=device)
    out = torch.empty((n, n), dtype=torch.bfloat16, device=device)
    run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=out)  # noqa: E731
    flops = 2.0 * n ** 3
    for _ in range(3):
        run()
    torch.cuda.synchronize(device)
    best = float("inf")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(10):
        start.record()
        run()
        stop.record()
        stop.synchronize()
        best = min(best, start.elapsed_time(stop) / 1e3)
    with ClockSampler(local) as sampler:
        begin, count = time.perf_counter(), 0
        start.record()
        while time.perf_counter() - begin < 4.0:
            for _ in range(50):
                run()
            count += 50
            torch.cuda.synchronize(device)
        stop.record()
        stop.synchronize()
        sustained = start.elapsed_time(stop) / 1e3 / count
    return {"fp8_tflops": flops / best / 1e12, "fp8_tflops_sustained": flops / sustained / 1e12,
            "how": "torch._scaled_mm e4m3 x e4m3 -> bf16, 8192^3: best of 10 (burst), 4 s back to back (sustained)",
            "clocks_under_load": sampler.result}


def run_prefill(args):
    """`--workload prefill_16k_128k`: LI score + TopK of one request's 16384-token query chunk against its causal
    131072-token context (FP8), the dense-contraction stress of the benchmark configs. The reference packs at
    most four query slots per row, so the chunk runs as 4 launches of 1024 rows x 4 queries that all read the
    same key pages; the score rows of one launch (2.1 GB) are reused by the next."""
    import torch

    from kvip_b200 import ops

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    chunk, context, heads, rows = 16384, 131072, 64, 4096
    g = torch.Generator(device=device)
    g.manual_seed(0)
    log_uniform = lambda shape: torch.exp(torch.rand(shape, generator=g, device=device) * 4.6052 - 6.9078)  # noqa: E731
    keys = (torch.randn((context, 128), generator=g, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
    key_scale = log_uniform((context,))
    query = (torch.randn((chunk, heads, 128), generator=g, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
    query_scale = log_uniform((chunk, heads))
    weights = (torch.randn((chunk, heads), generator=g, device=device) / 8).to(torch.bfloat16)
    batch = rows // 4
    key_lengths = torch.full((batch,), context, dtype=torch.int32, device=device)
    ends = (context - chunk + 1 + torch.arange(chunk, device=device)).to(torch.int32).view(chunk // 4, 4)
    table = torch.arange(context // 128, dtype=torch.int32, device=device).repeat(batch, 1)
    scores = torch.zeros((rows, context), dtype=torch.float32, device=device)
    picked = torch.empty((chunk, 2048), dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    host_query = query.view(torch.uint8).cpu().pin_memory()
    host_picked = torch.empty((chunk, 2048), dtype=torch.int32).pin_memory()
    stream = torch.cuda.Stream(device)
    lib = _load_counter()

    def li(part):
        lo, hi = part * rows, (part + 1) * rows
        ops.li_score(query[lo:hi], keys, weights[lo:hi], query_scale[lo:hi], key_scale, key_lengths,
                     ends[lo // 4:hi // 4], table, scores, status=status)

    def step(li_only=False):
        for part in range(chunk // rows):
            li(part)
            if not li_only:
                lo, hi = part * rows, (part + 1) * rows
                ops.topk(scores, key_lengths, ends[lo // 4:hi // 4], picked[lo:hi])

    # End to end: the chunk's queries come from pinned host memory and its TopK lists go back there. The four launch
    # groups of a chunk are independent, so the copies are pipelined with them on two copy streams: the queries of
    # group i + 1 arrive while group i is scored, the lists of group i leave while group i + 1 is scored; only the first
    # copy in and the last copy out are exposed.
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    parts = chunk // rows
    arrived = [torch.cuda.Event() for _ in range(parts)]
    selected = [torch.cuda.Event() for _ in range(parts)]
    query_bytes = query.view(torch.uint8)

    def e2e_step():
        copy_in.wait_stream(stream)    # the previous chunk's launches have read their queries
        copy_out.wait_stream(stream)
        with torch.cuda.stream(copy_in):
            for part in range(parts):
                lo, hi = part * rows, (part + 1) * rows
                query_bytes[lo:hi].copy_(host_query[lo:hi], non_blocking=True)
                arrived[part].record(copy_in)
        for part in range(parts):
            lo, hi = part * rows, (part + 1) * rows
            stream.wait_event(arrived[part])
            li(part)
            ops.topk(scores, key_lengths, ends[lo // 4:hi // 4], picked[lo:hi])
            selected[part].record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(selected[part])
                host_picked[lo:hi].copy_(picked[lo:hi], non_blocking=True)
        stream.wait_stream(copy_out)   # the chunk is done when its lists are on the host

    steps = max(1, min(args.steps, 5))
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
        stream.synchronize()
        if int(status.item()):
            raise RuntimeError(f"device status {int(status.item())}")
        with ClockSampler(device.index or 0) as sampler:
            before = lib.kvip_b200_launch_count()
            elapsed = time_region(torch, stream, step, steps)
            launches = lib.kvip_b200_launch_count() - before
            li_elapsed = time_region(torch, stream, lambda: step(li_only=True), steps)
            e2e_elapsed = time_region(torch, stream, e2e_step, steps)
        clocks = sampler.result
    flops = 2.0 * heads * 128 * float(ends.to(torch.float64).sum().item())
    del scores, picked
    torch.cuda.empty_cache()
    fp8 = measure_fp8_peak(torch, device, device.index or 0)
    # a launch lasts milliseconds and a chunk tens of them: the sustained figure is the fair denominator
    fp8_peak = fp8["fp8_tflops_sustained"]
    achieved = flops / (li_elapsed / steps) / 1e12
    print(json.dumps({
        "metric": "LI+TopK query tokens/s, chunked prefill 16384 x 131072 causal", "value": chunk * steps / elapsed,
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 3, "ms_per_step": elapsed / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32",
        "data": "synthetic",
        "config": {"workload": args.workload, "chunk": chunk, "context": context, "index_heads": heads, "topk": 2048,
                   "launches_per_chunk": chunk // rows, "l2": "score rows of one launch (2.1 GB) exceed L2"},
        "e2e": {"value": chunk * steps / e2e_elapsed, "unit": "tokens/s", "h2d_bytes_per_step": host_query.numel(),
                "d2h_bytes_per_step": host_picked.numel() * 4, "ms_per_step": e2e_elapsed / steps * 1e3,
                "api": "ops.li_score + ops.topk per launch group, copies of neighbouring groups on two copy streams"},
        "gpu_launches": launches,
        "roofline": {"kernel": "li_score_tcgen05", "bound": "tensor", "achieved": achieved, "peak": fp8_peak,
                     "unit": "TFLOP/s", "frac": achieved / fp8_peak,
                     "peak_kind": "of measured: dense FP8 GEMM throughput measured in this run (sustained figure)",
                     "peak_measurement": fp8,
                     "flops_per_chunk": flops, "ms_li_per_chunk": li_elapsed / steps * 1e3, "traffic": None},
        "clocks": clocks,
    }), flush=True)


def run_seqshard(args):
    """`--workload seqshard_1m`: one decode request with a 1,048,576-token context whose keys are sharded along
    the sequence over the ranks. Per step and rank: LI score of the shard with the replicated query, local
    top-2048 with global indices, ONE all-gather of the (score, index) candidates, merge to the global
    top-2048. Checked once, outside the timed region, against the TopK of the gathered full score row."""
    import torch
    import torch.distributed as dist

    from kvip_b200 import ops
    from kvip_b200.sharding import ShardedTopk, shard_bounds

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if not dist.is_initialized():
        if world == 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    total, heads = 1 << 20, 64
    begin, end = shard_bounds(total, world, rank)
    keys_here = end - begin
    g = torch.Generator(device=device)
    g.manual_seed(100 + rank)
    keys = (torch.randn((keys_here, 128), generator=g, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
    key_scale = torch.exp(torch.rand((keys_here,), generator=g, device=device) * 4.6052 - 6.9078)
    q = torch.Generator(device=device)
    q.manual_seed(7)  # the query is replicated: same seed on every rank
    query = (torch.randn((1, heads, 128), generator=q, device=device) * 8).clamp_(-448, 448).to(torch.float8_e4m3fn)
    query_scale = torch.exp(torch.rand((1, heads), generator=q, device=device) * 4.6052 - 6.9078)
    weights = (torch.randn((1, heads), generator=q, device=device) / 8).to(torch.bfloat16)
    lengths = torch.full((1,), keys_here, dtype=torch.int32, device=device)
    ends = torch.full((1, 1), keys_here, dtype=torch.int32, device=device)
    table = torch.arange(keys_here // 128, dtype=torch.int32, device=device).view(1, -1)
    scores = torch.zeros((1, keys_here), dtype=torch.float32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    sharded = ShardedTopk(1, device, transport=args.transport)
    merged = sharded.merged
    host_merged = torch.empty((1, 2048), dtype=torch.int32).pin_memory()
    host_query = query.view(torch.uint8).cpu().pin_memory()
    lib = _load_counter()
    stream = torch.cuda.Stream(device)

    def step():
        ops.li_score(query, keys, weights, query_scale, key_scale, lengths, ends, table, scores, status=status)
        sharded(scores, lengths, ends, begin)   # local TopK -> one all-gather -> merge in place

    def phases(rounds=50):
        """Device time of the four phases of the eager step, from CUDA events between them (mean of `rounds`)."""
        import torch.distributed as dist
        names = ("shard_li_score", "local_topk", "exchange", "merge")
        total = dict.fromkeys(names, 0.0)
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        for _ in range(rounds):
            marks[0].record(stream)
            ops.li_score(query, keys, weights, query_scale, key_scale, lengths, ends, table, scores, status=status)
            marks[1].record(stream)
            ops.topk(scores, lengths, ends, sharded.local_index, out_scores=sharded.local_scores, base_index=begin)
            marks[2].record(stream)
            sharded._exchange()
            marks[3].record(stream)
            sharded._merge()   # with the peer transport this includes the wait for the other ranks' candidates
            marks[4].record(stream)
            marks[4].synchronize()
            for i, name in enumerate(names):
                total[name] += marks[i].elapsed_time(marks[i + 1]) * 1e3 / rounds
        return total

    def e2e_step():
        query.view(torch.uint8).copy_(host_query, non_blocking=True)
        step()
        host_merged.copy_(merged, non_blocking=True)

    def barrier():
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        # check: the merged list equals the TopK of the whole row (scores gathered once)
        rows = [torch.empty((1, shard_bounds(total, world, r)[1] - shard_bounds(total, world, r)[0]),
                            dtype=torch.float32, device=device) for r in range(world)]
        dist.all_gather(rows, scores)
        whole = torch.cat(rows, dim=1).contiguous()
        whole_len = torch.full((1,), total, dtype=torch.int32, device=device)
        expected = ops.topk(whole, whole_len, whole_len.view(1, 1))
        stream.synchronize()
        verified = bool(torch.equal(expected, merged)) and int(status.item()) == 0
        barrier()
        before = lib.kvip_b200_launch_count()
        step()
        launches = (lib.kvip_b200_launch_count() - before) * args.steps
        stream.synchronize()
        # One rank, or the peer-memory exchange: the step is replayed from one CUDA graph. Several ranks over NCCL: two
        # graphs of this library's kernels (LI + local TopK, merge) with the all-gather issued eagerly between them;
        # capturing the all-gather itself made a two-rank run of this bench stop responding, so it stays outside graphs.
        graph, replay = None, step
        if world == 1 or args.transport == "peer":
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
            replay = graph.replay
        else:
            sharded.capture(lambda: ops.li_score(query, keys, weights, query_scale, key_scale, lengths, ends, table,
                                                 scores, status=status), scores, lengths, ends, begin)
            replay = sharded.replay

        def e2e_step():  # noqa: F811 - same name on purpose: the graph version replaces the eager one
            query.view(torch.uint8).copy_(host_query, non_blocking=True)
            replay()
            host_merged.copy_(merged, non_blocking=True)

        for _ in range(3):
            replay()
        barrier()
        with ClockSampler(local) as sampler:
            elapsed = time_region(torch, stream, replay, args.steps)
            barrier()
            e2e_elapsed = time_region(torch, stream, e2e_step, args.steps)
            barrier()
        clocks = sampler.result
        replay()
        stream.synchronize()
        verified = verified and bool(torch.equal(expected, merged))
        phase_us = phases()
        barrier()
    worst = torch.tensor([elapsed, e2e_elapsed, 0.0 if verified else 1.0] + [phase_us[k] for k in sorted(phase_us)],
                         dtype=torch.float64, device=device)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    elapsed, e2e_elapsed, failed, *slowest = (float(x) for x in worst.tolist())
    phase_us = dict(zip(sorted(phase_us), slowest))
    if rank == 0:
        print(json.dumps({
            "metric": "LI+TopK query tokens/s, one 1,048,576-token request sharded along the sequence",
            "value": args.steps / elapsed, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
            "config": {"workload": args.workload, "context": total, "keys_per_rank": keys_here, "index_heads": heads,
                       "topk": 2048,
                       "exchange": ("one NCCL all-gather of 2048 x (f32, i32) per rank, then merge" if args.transport == "nccl"
                                    else "this library's kernel: every rank stores its 2048 x (f32, i32) into every rank's "
                                         "exchange block over NVLink peer memory; the merge waits for the flags"),
                       "transport": args.transport,
                       "cuda_graph": True if graph is not None else "kernels on either side of the eager all-gather",
                       "l2": "shard keys %.0f MB per step" % (keys_here * 132 / 1e6)},
            "e2e": {"value": args.steps / e2e_elapsed, "unit": "tokens/s", "h2d_bytes_per_step": host_query.numel(),
                    "d2h_bytes_per_step": host_merged.numel() * 4, "ms_per_step": e2e_elapsed / args.steps * 1e3},
            "gpu_launches": launches, "verified_against_unsharded_topk": failed == 0.0,
            "peer_status": int(sharded.status.item()),
            "phases_us": dict(phase_us, note="eager launches, CUDA events between the phases, slowest rank of each; the "
                                             "events keep the launches from overlapping, so the sum exceeds the step"),
            "roofline": {"kernel": "li_score_tcgen05", "bound": "hbm", "achieved": None, "peak": peaks()[0],
                         "unit": "GB/s", "frac": None, "traffic": None,
                         "note": "latency-bound step: about %d key pages per CTA; see ms_per_step" % round(keys_here / 128 / 148)},
            "clocks": clocks,
        }), flush=True)
    sharded.close()
    dist.destroy_process_group()


def run_merge(args):
    """`--workload topk_merge`: the merge of shard candidates alone, one row, at 1 to 8 shards (random scores, every
    list full): `--steps` launches captured in one graph, CUDA events around one replay."""
    import torch

    from kvip_b200 import ops

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    stream = torch.cuda.Stream(device)
    g = torch.Generator(device=device)
    g.manual_seed(0)
    per_shards = {}
    lib = _load_counter()
    before = lib.kvip_b200_launch_count()
    with torch.cuda.stream(stream):
        for shards in (1, 2, 3, 4, 8):
            scores = torch.randn((1, shards * 2048), generator=g, device=device)
            index = torch.arange(shards * 2048, dtype=torch.int32, device=device).view(1, -1).contiguous()
            out = torch.empty((1, 2048), dtype=torch.int32, device=device)
            for _ in range(max(args.warmup, 3)):
                ops.topk_merge(scores, index, out)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(args.steps):
                    ops.topk_merge(scores, index, out)
            graph.replay()
            stream.synchronize()
            per_shards[shards] = time_region(torch, stream, graph.replay, 1) / args.steps * 1e6
    launches = lib.kvip_b200_launch_count() - before
    print(json.dumps({
        "metric": "topk_merge kernel time at eight shards", "value": per_shards[8], "unit": "us", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": per_shards[8] / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 keys, int32 indices", "data": "synthetic",
        "config": {"workload": args.workload, "rows": 1, "candidates_per_shard": 2048,
                   "kernels": "2, 4, 8 shards: one CTA per shard on a cluster; 1, 3 shards: one CTA"},
        "us_by_shards": {str(k): v for k, v in per_shards.items()}, "gpu_launches": launches,
    }), flush=True)


LIDU_PUBLISHED_US = {1: 20.99, 4: 30.70, 8: 36.00, 12: 35.78}   # csrc/operators/lidu/DESIGN_V2_LOW.md:56-63 (V2, Ascend A5)


def run_lidu(args):
    """`--workload lidu`: kernel time of `kvip.lidu` at the batches the reference publishes (B = 1, 4, 8, 12; four
    query rows per request, 131072 logical tokens, 16384 resident slots, 10 % misses). The call mutates its maps,
    so they are restored before every call; the duration comes from the kernel's own device-time stamps."""
    import torch

    from kvip_b200 import lidu
    from decode_harness import lidu_state

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    stream = torch.cuda.Stream(device)
    lib = _load_counter()
    results, launches = {}, 0
    with torch.cuda.stream(stream):
        for batch in sorted(LIDU_PUBLISHED_US):
            state = {k: torch.from_numpy(v).to(device) for k, v in lidu_state(batch, 4, 131072, 16384, seed=batch).items()}
            mutable = ("token_to_slot_pool", "slot_to_token_pool", "eviction_cursors")
            pristine = {k: state[k].clone() for k in mutable}
            i32 = dict(dtype=torch.int32, device=device)
            packed = batch * 4
            outs = (torch.zeros((packed, 1, 2048), **i32), torch.zeros(batch + 1, **i32), torch.zeros(batch * 8192, **i32),
                    torch.zeros(batch * 8192, **i32), torch.zeros(batch * 8192, **i32), torch.zeros(batch, **i32),
                    torch.zeros((batch, 8, 32), dtype=torch.int64, device=device))
            profile = torch.zeros(1, **i32)

            def restore():
                for k in mutable:
                    state[k].copy_(pristine[k])

            def call():
                lidu(state["topk_indices"], state["actual_seq_lengths_query"], state["req_pool_entries"],
                     state["token_to_slot_pool"], state["slot_to_token_pool"], state["eviction_cursors"],
                     state["cache_tokens"], state["candidate_lens"], state["miss_slots"], state["miss_slot_bitmap"],
                     state["resident_block_table"], state["logical_seq_lengths"], profile, *outs, 0, 1, batch, 131072 // 128)

            restore()
            before = lib.kvip_b200_launch_count()
            call()          # first call allocates the scratch: outside capture
            per_call = lib.kvip_b200_launch_count() - before
            stream.synchronize()
            misses = int(outs[1][batch].item())
            # Kernel-only duration from the kernel's own device-time stamps (`profile_enabled` = 1: every CTA
            # stamps its start and end into `profiling`): last end - first start, replayed from a graph at full
            # clocks with the maps restored before every call. The median of the replays is reported.
            profile.fill_(1)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                restore()
                call()
            reps = max(args.steps, 50)
            for _ in range(1000):   # long enough for the SM clock to settle under load
                graph.replay()
            durations = []
            for _ in range(reps):
                graph.replay()
                stream.synchronize()
                stamps = outs[6][:, 0, :3].cpu()
                durations.append(float(stamps[:, 1:].max() - stamps[:, 0].min()) / 1e3)
            durations.sort()
            launches += per_call * (reps + 1000)
            results[batch] = {"us": durations[len(durations) // 2], "min_us": durations[0], "misses": misses,
                              "published_us": LIDU_PUBLISHED_US[batch]}
    mean = sum(r["us"] for r in results.values()) / len(results)
    published_mean = sum(LIDU_PUBLISHED_US.values()) / len(LIDU_PUBLISHED_US)
    print(json.dumps({
        "metric": "LIDU kernel time, mean of B = 1, 4, 8, 12", "value": mean, "unit": "us", "n_gpus": 1,
        "steps": max(args.steps, 50), "warmup": 1000, "ms_per_step": mean / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": mean / published_mean, "dtype": "int32", "data": "synthetic",
        "config": {"workload": "lidu", "queries_per_request": 4, "logical_tokens": 131072, "resident_slots": 16384,
                   "miss_fraction": 0.1, "published": "Ascend A5 950DT kernel-only task durations, V2"},
        "per_batch": {str(k): v for k, v in results.items()}, "gpu_launches": launches,
    }), flush=True)


def run_miss_prefetch(args):
    """`--workload miss_path_prefetch`: the drifting-query miss path (AR(1) queries, rho = 0.95; 128k context,
    25 % resident pool, misses from the pinned host pool, one new Index row per token) with and without
    speculative prefetch windows, the forward replayed from a CUDA graph. Not a headline line: it reports what the
    windows cost (extra score launches) and what they move off the post-score fetch."""
    import torch

    from decode_harness import DecodePipeline

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    stream = torch.cuda.Stream(device)
    lib = _load_counter()
    batch = args.batch or 32
    cfg = dict(batch=batch, queries=1, heads=64, history=131072, resident=32768, len_lo=131072, len_hi=131072,
               key_dtype="fp8", weight_dtype="bf16", token_bytes=1152)
    variants = [("plain", {}), ("plain", {})] + [
        (f"windows{w}_limit{n}", dict(prefetch_limit=n, prefetch_windows=w)) for n in (512, 128) for w in (2, 3)]
    steps, warm, results = max(args.steps, 8), max(args.warmup, 4), []
    launches_before = lib.kvip_b200_launch_count()
    for name, extra in variants:   # the first plain run also warms the host pool mapping and is dropped below
        with torch.cuda.stream(stream):
            p = DecodePipeline(device, seed=0, gather=True, host_pool=True, **cfg, **extra)
            p.make_query_bank(steps + warm, correlation=0.95)
            for i in range(warm):
                p.load_queries(i)
                p.step(ingest=True)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                p.forward()
            counts = torch.zeros((3, steps), dtype=torch.int64, device=device)

            def drifting():
                for i in range(steps):
                    p.load_queries(warm + i)
                    p.ingest_new_tokens()
                    graph.replay()
                    counts[0, i] = p.rotating.query_counts[:, 4].sum()
                    if p.forward.prefetch is not None:
                        counts[1, i] = p.forward.prefetch.staged_rows.sum()
                        counts[2, i] = p.forward.prefetch.staged_hits.sum()

            stream.synchronize()
            seconds = time_region(torch, stream, drifting, 1)
            p.load_queries(0)
            for _ in range(3):
                graph.replay()
            steady = time_region(torch, stream, graph.replay, 10) / 10
            misses, listed, served = (counts.float().mean(dim=1)).tolist()
            results.append({"variant": name, "ms_per_step": seconds / steps * 1e3, "misses_per_step": misses,
                            "rows_staged_per_step": listed, "misses_served_from_staging": served,
                            "steady_no_miss_ms": steady * 1e3,
                            "status": int(p.update.status.max().item()) | int(p.forward.li_status.item())})
            p.close()
            del p, graph
            torch.cuda.empty_cache()
    print(json.dumps({"metric": "miss-path step time with and without prefetch windows", "unit": "ms", "n_gpus": 1,
                      "higher_is_better": False, "data": "synthetic", "dtype": "fp8_e4m3 x fp8_e4m3 -> f32",
                      "config": {"workload": "miss_path_prefetch", **{k: cfg[k] for k in ("batch", "history", "resident", "token_bytes")},
                                 "query_drift": "AR(1), rho = 0.95", "cuda_graph": True, "steps": steps},
                      "results": results[1:], "gpu_launches": lib.kvip_b200_launch_count() - launches_before}), flush=True)


def _load_counter():
    from kvip_b200 import _lib
    return _lib.load_library()


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--workload", choices=sorted(WORKLOADS) + ["prefill_16k_128k", "seqshard_1m", "lidu", "topk_merge", "miss_path_prefetch",
                                                       "decode_128k_b32_zipf"], default="decode_128k_b64")
    parser.add_argument("--transport", choices=("peer", "nccl"), default="peer",
                        help="seqshard_1m: how the ranks exchange their TopK candidates")
    parser.add_argument("--quick", action="store_true",
                        help="warm-up and timed replays only (for profiler captures): no stage timings, no end-to-end leg")
    parser.add_argument("--reuse", type=float, default=0.75,
                        help="decode_128k_b32_zipf: share of a selection kept from the previous step")
    parser.add_argument("--batch", type=int, default=0, help="override the per-GPU batch of the workload")
    parser.add_argument("--device-source", action="store_true", help="serve misses from HBM instead of the host pool")
    parser.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    parser.add_argument("--no-miss-path", action="store_true", help="skip the drifting-query / host-link measurement")
    parser.add_argument("--cpu-requests", type=int, default=4096, help="upper bound; the leg stops after ~15 s")
    parser.add_argument("--cpu-requests-per-step", type=int, default=2)
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference" and args.workload not in WORKLOADS:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm times the decode workloads only"}), flush=True)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill_16k_128k":
        run_prefill(args)
    elif args.workload == "seqshard_1m":
        run_seqshard(args)
    elif args.workload == "lidu":
        run_lidu(args)
    elif args.workload == "topk_merge":
        run_merge(args)
    elif args.workload == "miss_path_prefetch":
        run_miss_prefetch(args)
    elif args.workload == "decode_128k_b32_zipf":
        run_zipf(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
