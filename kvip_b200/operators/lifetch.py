"""The fused LIFetch operator: bindings, workspace, host KV pool and the graph-capturable forward.

Python mirror of the reference's operator layer for this path
(python/kvip/operators/lifetch/{workspace,binding,index_update,streaming,forward}.py and
python/kvip/operators/lifetch_ubmem/binding.py): the same object model - a `rotating` binding built
from the 14-tensor argument tuple, an `update` object carrying the 28-word Index-update ABI, and
`LIFetch(rotating, update)` whose `__call__()` is one C call that only enqueues kernels on the current
CUDA stream. All scratch is allocated in the constructors; nothing allocates, synchronises or copies to
the host inside `__call__`, so the call can be captured in a CUDA graph.

Differences that follow from the hardware: the ABI blobs live in (pinned) HOST memory and are read at
enqueue time, where the reference kept them in device memory for its kernels to chase; the transport
service is a pinned, mapped host pool (`HostKVPool`) instead of KVAF queues; batch, history and
query-slot limits are lifted (include/kvip_b200.h)."""
import ctypes

import numpy as np

from .. import _lib, ops
from ..inputs import QueryInputs

TOPK, SLOTS, CHANGE_CAPACITY = _lib.TOPK, _lib.SLOTS, _lib.CHANGE_CAPACITY


def _host_blob(torch, raw, pin=True):
    """A stable host copy of an ABI record; its data_ptr() is what the C entry point receives."""
    tensor = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()
    if pin and torch.cuda.is_available():
        tensor = tensor.pin_memory()
    return tensor


def rotation_spec(batch, history, resident, queries=4):
    """Single source of truth for the persistent-address scratch (reference workspace.py:9-32; the
    Ascend queue/event records are gone, the resolver's records keep their names and shapes)."""
    shapes = dict(
        rows=(batch, 256),
        locations=(batch, queries, TOPK),
        destinations=(batch * SLOTS,),
        lru_slots=(batch, TOPK),
        reserved_hot=(batch, resident),
        changes=(batch, CHANGE_CAPACITY),
        change_slots=(batch, CHANGE_CAPACITY),
        change_count=(batch,),
        row_status=(batch, 32),
        query_counts=(batch, 8),
    )
    spec = {name: (shape, "int32") for name, shape in shapes.items()}
    spec["fallback_addresses"] = ((batch, SLOTS), "int64")
    return spec


class LIFetchWorkspace:
    """Graph-stable LI work buffers shared by sequential layer groups (reference workspace.py:34-132)."""

    def __init__(self, torch, *, batch, history, device, aics=0, windows=0, pin_memory=True, index_heads=64,
                 queries=4, query_dtype=None, weight_dtype=None):
        if history % 128:
            raise ValueError("LIFetch history must align to 128 tokens")
        self.torch, self.batch, self.history, self.queries = torch, batch, history, queries
        self.inputs = self._make_inputs(torch, batch, device, pin_memory=pin_memory, history=history,
                                        index_heads=index_heads, queries=queries, query_dtype=query_dtype,
                                        weight_dtype=weight_dtype)
        self.query_lengths = torch.full((batch,), queries, dtype=torch.int32, device=device)
        self.key_lengths = torch.full((batch,), history, dtype=torch.int32, device=device)
        self.topk = torch.full((batch, queries, TOPK), -1, dtype=torch.int32, device=device)
        self.dummy = torch.zeros(16, dtype=torch.uint8, device=device)
        self.tail_bounds = torch.zeros((batch, 2), dtype=torch.int32, device=device)
        # fp32 score rows [B*Q, history]: written by the LI kernel, read back from L2 by TopK
        self.scores = torch.zeros((batch * queries, history), dtype=torch.float32, device=device)
        self.compute = self.scores.view(torch.uint8).reshape(-1)
        self.prefix_storage = torch.zeros(1024, dtype=torch.uint8, device=device)
        self.scratch = {}

    def _make_inputs(self, torch, batch, device, **kwargs):
        return QueryInputs(torch, batch, device, **kwargs)

    def allocate_rotation(self, torch, *, batch, history, resident, **_unused):
        """Reserve the resolver work memory once; bindings of every layer group point at it."""
        if self.scratch:
            raise RuntimeError("Rotation workspace already allocated")
        self.scratch = {name: torch.zeros(shape, dtype=getattr(torch, dtype), device=self.topk.device)
                        for name, (shape, dtype) in rotation_spec(batch, history, resident, self.queries).items()}

    @property
    def nbytes(self):
        scratch = sum(t.numel() * t.element_size() for t in self.scratch.values())
        own = sum(t.numel() * t.element_size() for t in (
            self.query_lengths, self.key_lengths, self.topk, self.dummy, self.scores, self.prefix_storage,
            self.tail_bounds))
        return self.inputs.nbytes + scratch + own

    def arguments(self, storage):
        """The 14 operator arguments, in the reference's order (workspace.py:105-123)."""
        if storage.history != int(self.block_history):
            raise ValueError("Index storage differs from the bound LI workspace")
        return (self.inputs.query, storage.keys, self.inputs.weights, self.inputs.scale, storage.scales,
                self.query_lengths, self.key_lengths, self.inputs.block_table, self.dummy, self.topk, self.dummy,
                self.dummy, self.compute, self.prefix_storage)

    @property
    def block_history(self):
        return self.inputs.block_table.shape[1] * 128


class HostKVPool:
    """Host-DDR KV rows, pinned and mapped into the device address space.

    Stands where the reference leases a KVAF UBmem mapping (python/kvip/adapters/kvaf.py: UbmemLease,
    LeasedRuntime): the pool owns the registration, hands out the device alias, remembers the stream its
    users run on and must outlive every graph captured against it. Miss rows are read by the fetch kernel
    straight through the alias (zero-copy over the host link)."""

    PAGE = 4096

    def __init__(self, torch, owners, tokens, token_bytes, device):
        if token_bytes % 16:
            raise ValueError("KV rows must be a multiple of 16 bytes")
        self.torch, self.device = torch, torch.device(device)
        self.owners, self.tokens, self.token_bytes = owners, tokens, token_bytes
        self.nbytes = owners * tokens * token_bytes
        self._backing = torch.empty(self.nbytes + self.PAGE, dtype=torch.uint8)
        offset = (-self._backing.data_ptr()) % self.PAGE
        self.flat = self._backing[offset: offset + self.nbytes]
        self.tensor = self.flat.view(owners, tokens, token_bytes)
        self.library = _lib.load_library()
        alias = ctypes.c_uint64(0)
        with torch.cuda.device(self.device):
            _lib.check(self.library.kvip_b200_host_register(self.flat.data_ptr(), self.nbytes, ctypes.byref(alias)),
                       "host pool registration", self.library)
        self.device_pointer = int(alias.value)
        self.stream = None
        self.bindings = []
        self.closed = False
        self.context = dict(token_bytes=token_bytes, tokens_per_block=128)

    def address(self, owner, token):
        """Byte offset of a row from the pool base: what IndexCacheStorage.addresses holds."""
        return (owner * self.tokens + token) * self.token_bytes

    def addresses(self, owner):
        return (self.torch.arange(self.tokens, dtype=self.torch.int64) + owner * self.tokens) * self.token_bytes

    def check_stream(self):
        """Everything that touches the pool is ordered on one stream (reference kvaf.py:119-125)."""
        if self.closed:
            raise RuntimeError("host KV pool is closed")
        stream = self.torch.cuda.current_stream(self.device)
        if self.stream is None:
            self.stream = stream
        elif stream != self.stream:
            raise RuntimeError("LIFetch must run on the stream its host pool was first used on")
        return stream

    def close(self):
        if self.closed:
            return
        self.torch.cuda.synchronize(self.device)
        _lib.check(self.library.kvip_b200_host_unregister(self.flat.data_ptr()), "host pool release", self.library)
        self.closed = True


class CudaBinding:
    """The `rotating` object: geometry, resolver scratch and the context record for one layer group.

    Built from the same 14-tensor argument tuple as the reference's LIFetchBinding / UbmemBinding
    (operators/lifetch/binding.py:12-243, operators/lifetch_ubmem/binding.py:13-171) and exposing the
    attribute names their consumers read."""

    def __init__(self, torch, arguments, lease, output, *, batch, history, resident, query_ends, hot_valid,
                 token_addresses, row_owners=None, tail_bounds=None, output_stride=None, scratch=None,
                 token_bytes=None, queries=None, score_mode=_lib.SCORE_FP32, sm_count=0, gather_output=None,
                 li_variant=0, prefetch_limit=0, source=None, library=None):
        self.torch, self.lease = torch, lease
        self.library = _lib.load_library(library)
        if len(arguments) != 14:
            raise ValueError("LIFetch requires 14 input buffers")
        self.device = arguments[0].device
        if self.device.type != "cuda" or any(x.device != self.device or not x.is_contiguous() for x in arguments):
            raise ValueError("LIFetch requires 14 contiguous input buffers on the same CUDA device")
        if not 0 <= prefetch_limit <= 512:
            raise ValueError("prefetch_limit: at most 512 speculative rows per request and round")
        query, keys, weights = arguments[0], arguments[1], arguments[2]
        queries = queries or query.shape[0] // batch
        heads = query.numel() // (batch * queries * 128)
        output_stride = output_stride or resident
        tail_tokens = output_stride - resident
        if tail_tokens < 0 or tail_tokens % 128:
            raise ValueError("Output stride must preserve hot and optional ABC slots")
        if tail_bounds is not None:
            if tail_tokens < 384:
                raise ValueError("Serving ABC bounds require at least 384 dedicated output slots")
            if (tail_bounds.device != self.device or tail_bounds.dtype != torch.int32
                    or tuple(tail_bounds.shape) != (batch, 2) or not tail_bounds.is_contiguous()):
                raise ValueError("LIFetch tail_bounds must be contiguous int32 [batch, 2]")
        token_bytes = token_bytes or (lease.token_bytes if lease is not None else output.shape[-1])
        owners = hot_valid.shape[0]
        self.runtime_shape = _lib.RuntimeShape.prepare(
            self.library, batch=batch, history=history, resident=resident, indexHeads=heads, smCount=sm_count,
            queries=queries, keyDtype=_lib.KEY_BF16 if keys.dtype == torch.bfloat16 else _lib.KEY_FP8,
            weightDtype=_lib.WEIGHT_FP32 if weights.dtype == torch.float32 else _lib.WEIGHT_BF16,
            scoreMode=score_mode, outputStride=output_stride, owners=owners, tokenBytes=token_bytes,
            keyRows=keys.numel() // 128, gatherRows=int(gather_output is not None), liVariant=li_variant)
        self.shape = self.runtime_shape
        self.shape_pointer = ctypes.byref(self.runtime_shape)
        self.prefetch_limit = prefetch_limit
        self.final_workers = 4
        self.queries, self.batch = queries, batch
        for name, (shape, dtype_name) in rotation_spec(batch, history, resident, queries).items():
            dtype = getattr(torch, dtype_name)
            value = torch.zeros(shape, dtype=dtype, device=self.device) if scratch is None else scratch[name]
            if value.device != self.device or value.dtype != dtype or tuple(value.shape) != shape or not value.is_contiguous():
                raise ValueError(f"Shared LIFetch scratch mismatch: {name}")
            setattr(self, name, value)
        self.reserved_hot.fill_(-1)
        # one 128-byte record per (request, query): count, first descriptor, error (include/kvip_b200.h: KvipFinalPost)
        self.final_posts = torch.zeros((batch * self.final_workers, 32), dtype=torch.int32, device=self.device)
        # one bit per TopK entry: filled by this round's fetch (lets the gather run in two phases around the fetch)
        self.miss_mask = torch.zeros((batch * queries, TOPK // 32), dtype=torch.int32, device=self.device)
        self.mapping = self.final_status = self.prefetch_status = None
        self.output, self.query_ends, self.hot_valid, self.row_owners = output, query_ends, hot_valid, row_owners
        self.token_addresses, self.tail_bounds, self.gather_output = token_addresses, tail_bounds, gather_output
        for name, tensor, expected in (("query_ends", query_ends, (batch * queries,)),
                                       ("hot_valid", hot_valid, (owners, resident))):
            if (tensor.device != self.device or tensor.dtype != torch.int32 or tensor.numel() != int(np.prod(expected))
                    or not tensor.is_contiguous()):
                raise ValueError(f"LIFetch {name} must be contiguous int32 with shape {expected}")
        if row_owners is not None and (row_owners.device != self.device or row_owners.dtype != torch.int32
                                       or tuple(row_owners.shape) != (batch,) or not row_owners.is_contiguous()):
            raise ValueError("LIFetch row_owners must be contiguous int32 [batch]")
        if (token_addresses.device != self.device or token_addresses.dtype != torch.int64
                or tuple(token_addresses.shape) != (owners, history) or not token_addresses.is_contiguous()):
            raise ValueError("Token addresses must match the stable-owner Index rows")
        self.output_stride = self.runtime_shape.outputStride
        if output.device != self.device or output.dtype != torch.uint8 or not output.is_contiguous():
            raise ValueError("The resident KV pool must be a contiguous uint8 CUDA tensor")
        if output.numel() < owners * self.output_stride * token_bytes or output.data_ptr() % 16:
            raise ValueError("The resident KV pool does not cover every stable owner")
        if gather_output is not None and (gather_output.device != self.device or gather_output.dtype != torch.uint8
                                          or gather_output.numel() != batch * queries * TOPK * token_bytes
                                          or not gather_output.is_contiguous()):
            raise ValueError("The gather output must be contiguous uint8 [B*Q, 2048, token_bytes]")
        if lease is not None:
            if lease.device != self.device or lease.token_bytes != token_bytes:
                raise ValueError("Host pool and kernel slot geometry differ")
            source_base, source_bytes = lease.device_pointer, lease.nbytes
            lease.bindings.append(self)
        elif source is not None:  # any device-visible byte tensor can stand in for the host pool
            source_base, source_bytes = source.data_ptr(), source.numel() * source.element_size()
            self.source = source
        else:
            raise ValueError("LIFetch needs a host KV pool (lease) or a device-visible source tensor")
        self.source_base, self.source_bytes = source_base, source_bytes
        context = _lib.Context(
            locations=self.locations.data_ptr(), lru_slots=self.lru_slots.data_ptr(),
            reserved_hot=self.reserved_hot.data_ptr(), changes=self.changes.data_ptr(),
            change_slots=self.change_slots.data_ptr(), change_count=self.change_count.data_ptr(),
            query_ends=query_ends.data_ptr(), fetch_sources=self.fallback_addresses.data_ptr(),
            fetch_destinations=self.destinations.data_ptr(), hot_valid=hot_valid.data_ptr(),
            row_owners=0 if row_owners is None else row_owners.data_ptr(), token_addresses=token_addresses.data_ptr(),
            address_stride=token_addresses.stride(0), output_stride=self.output_stride,
            tail_bounds=0 if tail_bounds is None else tail_bounds.data_ptr(),
            row_status=self.row_status.data_ptr(), query_counts=self.query_counts.data_ptr(),
            pool=output.data_ptr(), source_base=source_base, source_bytes=source_bytes, shape=self.runtime_shape,
            final_posts=self.final_posts.data_ptr(), miss_mask=self.miss_mask.data_ptr())
        self.context = _host_blob(torch, bytes(context))
        self.arguments = tuple(arguments) + (self.context,)
        self.bindings = None  # completed by LIFetch (needs the workspace record)
        self.owner = type("Owner", (), {"abi_sizes": {"status": 128}})()
        self.reset()

    def reset(self):
        for tensor in (self.rows, self.row_status, self.query_counts, self.change_count):
            tensor.zero_()
        self.changes.fill_(-1)
        self.locations.fill_(-1)


class IndexUpdate:
    """The `update` object: Index rows + service outputs behind the 28-word ABI
    (reference operators/lifetch/index_update.py:7-149)."""

    def __init__(self, torch, *, keys, scales, addresses, logical_ids, row_owners, rotating, status=None,
                 query_inputs=None, outputs=None):
        self.torch, self.device = torch, keys.device
        self.batch = rotating.batch
        queries = rotating.queries
        owners_tensor = row_owners if row_owners is not None else torch.arange(self.batch, dtype=torch.int32, device=self.device)
        self.storage = keys, scales, addresses, logical_ids, owners_tensor, rotating, query_inputs, outputs
        if any(t.device != self.device for t in (scales, addresses, logical_ids, owners_tensor)) or any(
                not t.is_contiguous() for t in (keys, scales, logical_ids, owners_tensor)):
            raise ValueError("LIFetch Index storage must be contiguous on one device")
        if owners_tensor.dtype != torch.int32 or owners_tensor.ndim != 1:
            raise ValueError("Request owners must be a flat int32 vector")
        if keys.ndim != 3 or keys.shape[-1] != 128 or keys.element_size() not in (1, 2):
            raise ValueError("LIFetch Index keys require [owner,history,128] FP8 (byte) or bfloat16 storage")
        if any(t.shape != keys.shape[:2] for t in (scales, addresses, logical_ids)):
            raise ValueError("Index key, scale, address and logical-ID rows must match")
        if addresses.stride(1) != 1 or addresses.stride(0) < keys.shape[1]:
            raise ValueError("Index addresses require contiguous, nonoverlapping rows")
        if scales.dtype != torch.float32 or addresses.dtype != torch.int64 or logical_ids.dtype != torch.int64:
            raise ValueError("Index scales require float32; address and logical IDs require int64")
        for name, shape in (("change_slots", (self.batch, CHANGE_CAPACITY)), ("changes", (self.batch, CHANGE_CAPACITY)),
                            ("change_count", (self.batch,)), ("rows", (self.batch, 256))):
            tensor = getattr(rotating, name)
            if (tensor.device != self.device or not tensor.is_contiguous() or tensor.dtype != torch.int32
                    or tuple(tensor.shape) != shape):
                raise ValueError(f"LIFetch producer {name} must be contiguous int32 with shape {shape}")
        self.status = torch.zeros(self.batch, dtype=torch.int32, device=self.device) if status is None else status
        if (self.status.device != self.device or self.status.dtype != torch.int32 or self.status.shape != (self.batch,)
                or not self.status.is_contiguous()):
            raise ValueError("Index update status must be contiguous int32 [batch] on the cache device")
        if outputs is None:
            outputs = torch.full((2, self.batch * queries, 1, TOPK), -1, dtype=torch.int32, device=self.device)
        if (tuple(outputs.shape) != (2, self.batch * queries, 1, TOPK) or outputs.dtype != torch.int32
                or outputs.device != self.device or not outputs.is_contiguous()):
            raise ValueError("Service outputs must be contiguous int32 [2, B*Q, 1, 2048]")
        self.outputs = outputs
        self.logical_output, self.slot_output = outputs.unbind(0)
        words = [keys.data_ptr(), scales.data_ptr(), addresses.data_ptr(), logical_ids.data_ptr(),
                 rotating.change_slots.data_ptr(), rotating.changes.data_ptr(), self.status.data_ptr(),
                 addresses.stride(0), rotating.rows.data_ptr(), owners_tensor.data_ptr(), rotating.row_status.data_ptr(),
                 rotating.final_posts.data_ptr(), 0, 0, rotating.final_workers, 128, rotating.hot_valid.data_ptr(), 0,
                 rotating.arguments[9].data_ptr(), rotating.locations.data_ptr(),
                 0 if query_inputs is None else query_inputs.unpack_indices.data_ptr(),
                 0 if query_inputs is None else query_inputs.output_valid.data_ptr(),
                 self.logical_output.data_ptr(), self.slot_output.data_ptr(), keys.shape[1],
                 rotating.hot_valid.shape[1], rotating.change_count.data_ptr(), 0]
        self.bindings = torch.from_numpy(np.asarray(words, dtype="<u8").view("<i8").copy())
        if torch.cuda.is_available():
            self.bindings = self.bindings.pin_memory()


class LIFetch:
    """`kvip.LIFetch(rotating, update)`: allocate once, then `__call__()` enqueues the whole
    LI -> TopK -> resolve -> Index exchange -> fetch (-> gather) chain with one C call
    (reference operators/lifetch/streaming.py:9-146, forward.py:7-17).

    With `lru=SlotLRU` the LRU feedback of the slots the step used is part of the call: it is enqueued on a
    side stream as soon as the output rows are written and runs beside the fetch and the gather (the reference
    feeds its numba LRU from the host after the step, cache/lru.py:87-96). `select()` and `commit()` are the
    two halves of `__call__()` for callers that overlap host copies with the step: `select()` reads the query
    inputs and writes no output row, `commit()` reads no query input."""

    def __init__(self, rotating, update, *, q_workers=2, lru=None, prefetch_limit=None, prefetch_windows=3, prefetch_ctas=0,
                 prefetch_last_window=False, overlap_fetch=False):
        if rotating.device != update.device:
            raise ValueError("Fetch and Index update must use the same device")
        if update.bindings.numel() != 28:
            raise ValueError("LIFetch requires the 28-field Index update/output binding ABI")
        if q_workers not in (1, 2, 4):
            raise ValueError("LIFetch requires 1/2/4 Fetch workers per query")
        torch = rotating.torch
        self.rotating, self.update, self.torch = rotating, update, torch
        shape = rotating.runtime_shape
        self.batch, self.history, self.resident = shape.batch, shape.history, shape.resident
        self.shape_pointer = ctypes.byref(shape)
        self.q_workers, self.prefetch_limit = q_workers, 0
        self.lru = lru
        self._slots_ready = self._lru_done = self._side = self._fork = self._join = None
        self.overlap_fetch = bool(overlap_fetch)
        current = torch.cuda.current_stream(rotating.device)
        if lru is not None and (lru.device != rotating.device or lru.rows_count != self.batch):
            raise ValueError("the SlotLRU must have one row per request on the cache device")
        if lru is not None or overlap_fetch:
            self._side = torch.cuda.Stream(rotating.device)
            self._slots_ready, self._lru_done = torch.cuda.Event(), torch.cuda.Event()
            self._slots_ready.record(current)   # an event has no handle before its first record
            self._lru_done.record(current)
        if overlap_fetch:
            # the commit phase forks here: outputs, Index exchange and the gather of the hit entries run on the side
            # stream beside the fetch of the missing rows (include/kvip_b200.h: KvipWorkspace.side_stream)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
            self._fork.record(current)
            self._join.record(current)
        library = rotating.library
        self.resolver_cores, flag_count = int(library.kvip_streaming_resolver_cores()), int(library.kvip_streaming_flag_count())
        if self.resolver_cores != 3 or flag_count != 16:
            raise ValueError("Rebuild kvip_b200: the public LIFetch pipeline requires the shared three-role ABI")
        self.function = library.kvip_lifetch_streaming_forward
        keys, scales, addresses, logical = update.storage[:4]
        b, device = self.batch, rotating.device
        pool = getattr(rotating, "streaming_scratch", {})

        def allocate(name, shape_, dtype, fill=None):
            key = (name, tuple(shape_), dtype, str(device))
            if key not in pool:
                pool[key] = torch.zeros(shape_, dtype=dtype, device=device) if fill is None else fill()
            return pool[key]

        self.events_src = allocate("event_sources", (b, SLOTS), torch.int32)
        self.events_dst = allocate("event_destinations", (b, SLOTS), torch.int32)
        self.worker_status = allocate("worker_status", (b, 32), torch.int32)
        self.times = allocate("times", (b * 256,), torch.int64)
        self.li_status = allocate("li_status", (1,), torch.int32)
        # TopK scratch is optional: without it the forward selects with the sampled-pivot kernel
        self.topk_histogram = None
        self.dense_shadow = allocate("dense_shadow", (b, 2 * self.history), torch.int32,
                                     lambda: ops.make_shadow(b, self.history, device))
        workspace = _lib.Workspace(
            context=rotating.context.data_ptr(), keys=keys.data_ptr(), scales=scales.data_ptr(),
            addresses=addresses.data_ptr(), logical_ids=logical.data_ptr(), hot_valid=rotating.hot_valid.data_ptr(),
            flags=0, events_src=self.events_src.data_ptr(), events_dst=self.events_dst.data_ptr(),
            worker_status=self.worker_status.data_ptr(), times=self.times.data_ptr(), history=self.history,
            resident=self.resident, options=q_workers << 16, max_events=CHANGE_CAPACITY, query_bitmaps=0,
            query_errors=0, update_bindings=update.bindings.data_ptr(), dense_shadow=self.dense_shadow.data_ptr(),
            packed_fetch=0, gather_out=0 if rotating.gather_output is None else rotating.gather_output.data_ptr(),
            topk_scores=0, li_status=self.li_status.data_ptr(), topk_histogram=0, topk_split=0,
            slots_ready_event=0 if self._slots_ready is None or lru is None else int(self._slots_ready.cuda_event),
            side_stream=int(self._side.cuda_stream) if overlap_fetch else 0,
            fork_event=int(self._fork.cuda_event) if overlap_fetch else 0,
            join_event=int(self._join.cuda_event) if overlap_fetch else 0)
        self.workspace = _host_blob(torch, bytes(workspace))
        words = [x.data_ptr() for x in rotating.arguments] + [self.workspace.data_ptr()]
        rotating.bindings = torch.from_numpy(np.asarray(words, dtype="<u8").view("<i8").copy())
        if torch.cuda.is_available():
            rotating.bindings = rotating.bindings.pin_memory()
        self.set_options()
        # speculative prefetch windows: `prefetch_limit` rows per request and round (0 = off, at most 512)
        self.prefetch = None
        if prefetch_limit is None:
            prefetch_limit = rotating.prefetch_limit
        if prefetch_limit:
            from .prefetch import PrefetchWindows
            self.prefetch = PrefetchWindows(self, limit=prefetch_limit, window_limit=min(480, prefetch_limit),
                                            cold_windows=prefetch_windows, li_ctas=prefetch_ctas,
                                            last_window=prefetch_last_window)
            self.prefetch_limit = prefetch_limit
            self.set_options()

    def _enqueue(self, phase):
        lease = self.rotating.lease
        stream = lease.check_stream() if lease is not None else self.torch.cuda.current_stream(self.rotating.device)
        self._options_word[0] = self._options | phase   # host memory, read by the call below
        result = self.function(self.rotating.bindings.data_ptr(), self.update.bindings.data_ptr(),
                               self.workspace.data_ptr(), ctypes.c_void_p(stream.cuda_stream), self.shape_pointer,
                               self.q_workers)
        self._options_word[0] = self._options
        if result:
            raise RuntimeError(f"streaming LIFetch launch failed: {result} ({_lib.last_error(self.rotating.library)})")
        if self.lru is not None and not phase & _lib.OPTION_SELECT_ONLY:
            # fork: LRU feedback beside fetch + gather; join before the caller's next work on this stream. (With
            # overlap_fetch the side stream already carries the output rows: the wait is then a no-op.)
            self._side.wait_event(self._slots_ready)
            with self.torch.cuda.stream(self._side):
                self.lru.commit(self.update.slot_output.view(self.batch, -1))
                self._lru_done.record(self._side)
            stream.wait_event(self._lru_done)

    def __call__(self, scores_ready=False):
        """The whole step. `scores_ready=True`: the score rows were written by the caller (an `ops.li_score` launch of
        its own, or a test that supplies scores): the call starts at TopK."""
        if scores_ready:
            if self.prefetch is not None:
                raise ValueError("prefetch windows issue the score pass themselves")
            self._enqueue(_lib.OPTION_SCORES_READY)
        elif self.prefetch is None:
            self._enqueue(0)
        else:
            self.select()
            self.commit()

    def select(self):
        """First half: LI score -> TopK -> resolver. Reads the query inputs; writes no output row. With
        prefetch windows the score pass is issued window by window here, and rows of likely misses are staged
        on a second stream meanwhile."""
        if self.prefetch is None:
            self._enqueue(_lib.OPTION_SELECT_ONLY)
            return
        lease = self.rotating.lease
        main = lease.check_stream() if lease is not None else self.torch.cuda.current_stream(self.rotating.device)
        self.prefetch.enqueue(main)
        self._enqueue(_lib.OPTION_SELECT_ONLY | _lib.OPTION_SCORES_READY)

    def commit(self):
        """Second half: output rows -> Index exchange -> fetch (-> gather) and the LRU feedback."""
        if self.prefetch is not None:   # the fetch reads the staging area: join the second stream
            self.torch.cuda.current_stream(self.rotating.device).wait_event(self.prefetch.staged)
        self._enqueue(_lib.OPTION_COMMIT_ONLY)

    def set_options(self, *, diagnostics=False, deferred_fetch=False):
        """Startup/profile-only update of the options word (byte 96 of the workspace record). The record
        is read when the call is enqueued: a graph captured earlier keeps the options it was captured with."""
        self._options = (self.prefetch_limit | (self.q_workers << 16) | (_lib.OPTION_DIAGNOSTICS if diagnostics else 0)
                         | (_lib.OPTION_DEFERRED_FETCH if deferred_fetch else 0))
        self._options_word = self.workspace.numpy()[96:100].view("<u4")   # same host memory as the record
        self._options_word[0] = self._options

    def stage_times(self):
        """Device time of every stage of the last call made with `set_options(diagnostics=True)`, in microseconds,
        plus `total`. Reads the `times` buffer on the host (a synchronising copy): for use after the step, outside
        any capture. A stage includes the gap to its predecessor; a stage the call skipped reports 0."""
        stamps = self.times[: len(_lib.TIME_STAGES) + 1].cpu().tolist()
        result = {name: (stamps[i + 1] - stamps[i]) / 1e3 for i, name in enumerate(_lib.TIME_STAGES)}
        result["total"] = (stamps[-1] - stamps[0]) / 1e3
        return result
