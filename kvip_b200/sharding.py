"""Multi-GPU partitioning of the path. One process per GPU.

* Requests are independent (per-request Index rows, resident pool, LRU and host-pool slice), so a batch is
  split over ranks with no data-path collective: `partition_requests` balances the LI cost, which is
  proportional to the context length.
* The one exception is a single very long request: its keys are sharded along the sequence, every rank
  scores its shard with the replicated query and takes a local top-2048 with global indices, the
  (score, index) candidates are exchanged with ONE all-gather (16 KiB per rank) and every rank merges them
  with the same total order (score descending, index ascending) - the result equals the unsharded TopK.
  The reference has no multi-device code; its on-chip two-shard sequence split is the precedent
  (csrc/operators/common/lifetch/sequence_schedule.h:9-37)."""
import torch

TOPK = 2048


def partition_requests(lengths, world):
    """Longest-processing-time-first assignment of request indices to `world` ranks.
    Returns a list of index lists; deterministic (ties by request index)."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    bins, loads = [[] for _ in range(world)], [0] * world
    for i in order:
        target = min(range(world), key=lambda r: (loads[r], len(bins[r]), r))
        bins[target].append(i)
        loads[target] += int(lengths[i])
    return [sorted(b) for b in bins]


def shard_bounds(total_tokens, world, rank, block=128):
    """Contiguous, block-aligned key range [begin, end) of a rank for a sequence-sharded request."""
    blocks = (total_tokens + block - 1) // block
    per, extra = divmod(blocks, world)
    begin_block = rank * per + min(rank, extra)
    end_block = begin_block + per + (1 if rank < extra else 0)
    return min(begin_block * block, total_tokens), min(end_block * block, total_tokens)


def gather_candidates(local_scores, local_index, group=None):
    """ONE all-gather of the per-rank candidates: [rows, 2048] scores and indices each, exchanged as one packed
    int32 tensor [2, rows, 2048] per rank -> ([rows, world*2048] scores, same shape indices) in rank order."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    packed = torch.stack((local_scores.contiguous().view(torch.int32), local_index.contiguous()))
    parts = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(parts, packed, group=group)
    scores = torch.cat([p[0] for p in parts], dim=1).contiguous().view(torch.float32)
    index = torch.cat([p[1] for p in parts], dim=1).contiguous()
    return scores, index


class ShardedTopk:
    """Preallocated buffers of the sequence-sharded TopK of `rows` score rows: the local TopK writes its scores and
    global indices straight into this rank's send block, ONE all-gather fills [world, 2, rows, 2048], and the merge
    kernel reads that buffer in place. Per step: local TopK, all-gather, merge - three launches, no repacking."""

    def __init__(self, rows, device, group=None):
        import torch.distributed as dist

        self.group, self.world = group, dist.get_world_size(group)
        self.send = torch.zeros((2, rows, TOPK), dtype=torch.int32, device=device)
        self.gathered = torch.zeros((self.world, 2, rows, TOPK), dtype=torch.int32, device=device)
        self.merged = torch.empty((rows, TOPK), dtype=torch.int32, device=device)
        self.local_scores, self.local_index = self.send[0].view(torch.float32), self.send[1]

        self._before = self._after = None

    def __call__(self, scores, lengths, ends, base_index):
        import torch.distributed as dist

        from . import ops
        ops.topk(scores, lengths, ends, self.local_index, out_scores=self.local_scores, base_index=base_index)
        dist.all_gather_into_tensor(self.gathered, self.send, group=self.group)
        return ops.topk_merge_gathered(self.gathered, self.merged)

    def capture(self, score_step, scores, lengths, ends, base_index, warmup=3):
        """Capture this rank's launches on either side of the exchange into two CUDA graphs: `score_step()` (the
        caller's LI launch into `scores`) with the local TopK before it, the merge after it. Only kernels of this
        library are captured; the all-gather stays an eager NCCL call between the two replays (`replay`). On a step
        this short the host's launch cost is what the graphs remove. Call it, and `replay`, under the same non-default
        stream."""
        from . import ops

        if torch.cuda.current_stream() == torch.cuda.default_stream():
            raise ValueError("ShardedTopk.capture() must run under a non-default stream (torch.cuda.stream(...)): "
                             "CUDA graphs cannot be captured on the default stream")

        def before():
            score_step()
            ops.topk(scores, lengths, ends, self.local_index, out_scores=self.local_scores, base_index=base_index)

        def after():
            ops.topk_merge_gathered(self.gathered, self.merged)

        for _ in range(max(warmup, 1)):
            before()
            after()
        torch.cuda.current_stream().synchronize()
        self._before, self._after = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._before, stream=torch.cuda.current_stream()):
            before()
        with torch.cuda.graph(self._after, stream=torch.cuda.current_stream()):
            after()

    def replay(self):
        """One step of the captured form: graph (LI + local TopK), eager all-gather, graph (merge)."""
        import torch.distributed as dist

        if self._before is None:
            raise RuntimeError("ShardedTopk.replay() before capture()")
        self._before.replay()
        dist.all_gather_into_tensor(self.gathered, self.send, group=self.group)
        self._after.replay()
        return self.merged


def sequence_sharded_topk(local_scores, local_length, base_index, *, queries=1, group=None, local_topk=None,
                          merge=None):
    """Global TopK-2048 of a request whose score rows are sharded along the sequence.

    local_scores [rows, shard_stride] fp32 on this rank, `local_length` valid keys in the shard, `base_index`
    the global position of the shard's first key. `local_topk` / `merge` default to the CUDA kernels; the
    CPU tests of the exchange logic inject host functions instead."""
    from . import ops

    rows = local_scores.shape[0]
    device = local_scores.device
    if local_topk is None:
        lengths = torch.full((rows // queries,), local_length, dtype=torch.int32, device=device)
        ends = torch.full((rows,), local_length, dtype=torch.int32, device=device)
        cand_scores = torch.zeros((rows, TOPK), dtype=torch.float32, device=device)
        cand_index = ops.topk(local_scores, lengths, ends, out_scores=cand_scores, base_index=base_index)
    else:
        cand_index, cand_scores = local_topk(local_scores, local_length, base_index)
    all_scores, all_index = gather_candidates(cand_scores, cand_index, group)
    return (merge or ops.topk_merge)(all_scores, all_index)
