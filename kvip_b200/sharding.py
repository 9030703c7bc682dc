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


class PeerBlocks:
    """Exchange blocks for `kvip_b200_peer_exchange`: one per rank, allocated by the library on this rank's GPU and
    mapped into every other rank's process through CUDA IPC handles (exchanged once over `torch.distributed`).
    `addresses[r]` is rank r's block as seen from this process. One process per GPU: two ranks on one GPU would have
    one rank's merge kernel wait for another's exchange kernel on the same device, which nothing guarantees to run."""

    def __init__(self, rows, device, group=None):
        import ctypes

        import torch.distributed as dist

        from . import _lib
        self.lib = _lib.load_library()
        self.group, self.rank, self.world = group, dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("the candidate exchange block has flags for at most 8 ranks")
        self.block_bytes = 2 * rows * TOPK * 4
        self.bytes = _lib.PEER_HEADER_BYTES + 2 * self.world * self.block_bytes
        with torch.cuda.device(device):
            own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            _lib.check(self.lib.kvip_b200_peer_alloc(self.bytes, ctypes.byref(own), handle), "peer_alloc")
            self.own = own.value
            identity = str(torch.cuda.get_device_properties(device).uuid)
            everyone = [None] * self.world
            dist.all_gather_object(everyone, (handle.raw, identity), group=group)
            if len({uuid for _, uuid in everyone}) != self.world:
                self.lib.kvip_b200_peer_free(self.own)
                raise ValueError("the peer exchange needs one GPU per rank")
            self.addresses, self._opened = [], []
            for r, (raw, _) in enumerate(everyone):
                if r == self.rank:
                    self.addresses.append(self.own)
                    continue
                mapped = ctypes.c_void_p()
                _lib.check(self.lib.kvip_b200_peer_open(raw, ctypes.byref(mapped)), "peer_open")
                self.addresses.append(mapped.value)
                self._opened.append(mapped.value)
        dist.barrier(group=group)   # every block is mapped everywhere before the first exchange

    def close(self):
        import torch.distributed as dist

        if self.own is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)   # nobody is still writing into a block that is about to go
        for mapped in self._opened:
            self.lib.kvip_b200_peer_close(mapped)
        dist.barrier(group=self.group)
        self.lib.kvip_b200_peer_free(self.own)
        self.own, self._opened = None, []


class ShardedTopk:
    """Preallocated buffers of the sequence-sharded TopK of `rows` score rows: the local TopK writes its scores and
    global indices straight into this rank's send block, one exchange delivers every rank's block to every rank, and
    the merge kernel reads the delivered blocks in place. Per step: local TopK, exchange, merge - no repacking.

    `transport="nccl"`: the exchange is ONE `all_gather_into_tensor` (eager; the kernels on either side of it may be
    captured, `capture` / `replay`). `transport="peer"`: the exchange is this library's kernel over NVLink peer memory
    (`PeerBlocks`): no collective call, the merge waits (bounded) for the other ranks' flags, and the whole step -
    score, local TopK, exchange, merge - captures into ONE graph per rank."""

    def __init__(self, rows, device, group=None, transport="nccl"):
        import torch.distributed as dist

        if transport not in ("nccl", "peer"):
            raise ValueError("transport must be 'nccl' or 'peer'")
        self.group, self.world, self.rows, self.transport = group, dist.get_world_size(group), rows, transport
        self.send = torch.zeros((2, rows, TOPK), dtype=torch.int32, device=device)
        self.merged = torch.empty((rows, TOPK), dtype=torch.int32, device=device)
        self.local_scores, self.local_index = self.send[0].view(torch.float32), self.send[1]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)   # KVIP_ERR_PEER: a wait for a rank ran out
        self._before = self._after = None
        self.peers = self.gathered = None
        if transport == "peer":
            self.peers = PeerBlocks(rows, device, group)
        else:
            self.gathered = torch.zeros((self.world, 2, rows, TOPK), dtype=torch.int32, device=device)

    def close(self):
        """Unmap and free the exchange blocks (peer transport); collective: every rank calls it."""
        if self.peers is not None:
            self.peers.close()
            self.peers = None

    def _merge(self, wait_kilocycles=0):
        from . import ops
        if self.peers is not None:
            return ops.topk_merge_peer(self.peers.own, self.rows, self.world, self.merged, self.status, wait_kilocycles)
        return ops.topk_merge_gathered(self.gathered, self.merged)

    def _exchange(self):
        import torch.distributed as dist

        from . import ops
        if self.peers is not None:
            ops.peer_exchange(self.send, self.peers.addresses, self.peers.rank)
        else:
            dist.all_gather_into_tensor(self.gathered, self.send, group=self.group)

    def __call__(self, scores, lengths, ends, base_index, wait_kilocycles=0):
        from . import ops
        ops.topk(scores, lengths, ends, self.local_index, out_scores=self.local_scores, base_index=base_index)
        self._exchange()
        return self._merge(wait_kilocycles)

    def capture(self, score_step, scores, lengths, ends, base_index, warmup=3):
        """Capture the step into CUDA graphs: `score_step()` (the caller's LI launch into `scores`) with the local TopK,
        then the exchange and the merge. With the peer transport everything is one graph. With NCCL only kernels of
        this library are captured, in two graphs, and the all-gather stays an eager call between the two replays
        (`replay`): on a step this short the host's launch cost is what the graphs remove. Call it, and `replay`, under
        the same non-default stream. The warm-up steps exchange candidates, so every rank must make the same calls."""
        from . import ops

        if torch.cuda.current_stream() == torch.cuda.default_stream():
            raise ValueError("ShardedTopk.capture() must run under a non-default stream (torch.cuda.stream(...)): "
                             "CUDA graphs cannot be captured on the default stream")

        def before():
            score_step()
            ops.topk(scores, lengths, ends, self.local_index, out_scores=self.local_scores, base_index=base_index)

        for _ in range(max(warmup, 1)):
            before()
            self._exchange()
            self._merge()
        torch.cuda.current_stream().synchronize()
        self._before, self._after = torch.cuda.CUDAGraph(), None
        with torch.cuda.graph(self._before, stream=torch.cuda.current_stream()):
            before()
            if self.peers is not None:
                self._exchange()
                self._merge()
        if self.peers is None:
            self._after = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._after, stream=torch.cuda.current_stream()):
                self._merge()

    def replay(self):
        """One step of the captured form: one graph (peer transport), or graph (LI + local TopK), eager all-gather,
        graph (merge)."""
        if self._before is None:
            raise RuntimeError("ShardedTopk.replay() before capture()")
        self._before.replay()
        if self._after is not None:
            self._exchange()
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
