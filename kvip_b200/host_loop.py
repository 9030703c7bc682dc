"""Decode steps fed from and drained to pinned host memory, with both copies overlapped with device work.

One step of the path, seen from the host, is: copy the step's queries, head weights, scales and positions
to the device; pack them into the bound input buffers (`QueryInputs.bind_positions` + `pack`); run
`LIFetch`; copy the two output rows per query back. Issued on one stream these run one after the other,
and at 128k context the copies and the pack add about a third to the step. `HostDecodeLoop` keeps the same
work per step but lets the copies of neighbouring steps run beside the kernels:

    copy-in stream :                        H2D(i+1) ....
    main stream    : pack(i) -> select(i) -> [outputs of i-1 read?] -> commit(i) -> pack(i+1) -> ...
    copy-out stream: D2H(i-1) ....                                                   D2H(i) ....

* the staging buffers are free again once pack(i) + select(i) have run, so H2D(i+1) overlaps commit(i);
* `LIFetch.select()` (LI score, TopK, resolver) writes no output row, so D2H(i-1) may still be reading the
  output rows while it runs; `LIFetch.commit()` waits for that copy;
* both halves are captured in CUDA graphs when `capture=True` (construction then runs one step on what the
  host tensors hold).

The caller must have step i+1's inputs in host memory when step i is submitted (two micro-batches in
flight); with strictly dependent steps use `LIFetch` directly."""


class HostDecodeLoop:
    def __init__(self, torch, forward, inputs, outputs, *, host_query, host_weights, host_scale, host_positions,
                 host_outputs, capture=True):
        device = outputs.device
        if getattr(forward, "prefetch", None) is not None:
            # select() would leave the prefetch stream unjoined at the end of its graph
            raise ValueError("HostDecodeLoop captures select() and commit() separately: use a forward without prefetch windows")
        for name, tensor in (("host_query", host_query), ("host_weights", host_weights),
                             ("host_positions", host_positions), ("host_outputs", host_outputs)):
            if tensor.device.type != "cpu" or not tensor.is_pinned():
                raise ValueError(f"{name} must be a pinned host tensor")
        if host_scale is not None and (host_scale.device.type != "cpu" or not host_scale.is_pinned()):
            raise ValueError("host_scale must be a pinned host tensor")
        if tuple(host_outputs.shape) != tuple(outputs.shape) or host_outputs.dtype != outputs.dtype:
            raise ValueError("host_outputs must have the shape and dtype of the bound output rows")
        self.torch, self.forward, self.inputs, self.outputs = torch, forward, inputs, outputs
        self.host = (host_query, host_weights, host_scale, host_positions)
        self.host_outputs = host_outputs
        self.stage = tuple(None if t is None else torch.empty(t.shape, dtype=t.dtype, device=device) for t in self.host)
        self.main = torch.cuda.current_stream(device)
        if self.main == torch.cuda.default_stream(device):
            self.main = torch.cuda.Stream(device)   # graphs cannot be captured on the default stream
            self.main.wait_stream(torch.cuda.default_stream(device))
        self.copy_in, self.copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.h2d_done, self.pack_done, self.step_done, self.d2h_done = (torch.cuda.Event() for _ in range(4))
        self.d2h_done.record(self.main)
        self.steps = 0
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in self.host if t is not None)
        self.d2h_bytes = host_outputs.numel() * host_outputs.element_size()
        self._prefetched = False
        self._select = self._commit = None
        if capture:
            # One real step on the host tensors' present contents: lazy attributes and allocations happen
            # outside capture, and the staging buffers hold valid inputs while the graphs are recorded.
            with torch.cuda.stream(self.main):
                for staged, host in zip(self.stage, self.host):
                    if host is not None:
                        staged.copy_(host, non_blocking=True)
                self._pack_and_select()
                forward.commit()
            self.main.synchronize()
            self._select, self._commit = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._select, stream=self.main):
                self._pack_and_select()
            with torch.cuda.graph(self._commit, stream=self.main):
                forward.commit()

    def _pack_and_select(self):
        query, weights, scale, positions = self.stage
        self.inputs.bind_positions(positions)
        self.inputs.pack(query, weights, scale)
        self.forward.select()

    def _copy_in(self):
        self.copy_in.wait_event(self.pack_done)  # the previous pack has read the staging buffers
        with self.torch.cuda.stream(self.copy_in):
            for staged, host in zip(self.stage, self.host):
                if host is not None:
                    staged.copy_(host, non_blocking=True)
            self.h2d_done.record(self.copy_in)
        self._prefetched = True

    def step(self, prefetch_next=True):
        """Enqueue one step on the host tensors' current contents. With `prefetch_next` the next step's
        inputs are copied while this step runs: they must already be in the host tensors."""
        torch = self.torch
        if not self._prefetched:
            self.pack_done.record(self.main)
            self._copy_in()
        with torch.cuda.stream(self.main):
            self.main.wait_event(self.h2d_done)
            if self._select is not None:
                self._select.replay()
            else:
                self._pack_and_select()
            self.pack_done.record(self.main)     # the staging buffers have been read
            self._prefetched = False
            if prefetch_next:
                self._copy_in()
            self.main.wait_event(self.d2h_done)  # the previous step's output rows have left the device
            if self._commit is not None:
                self._commit.replay()
            else:
                self.forward.commit()
            self.step_done.record(self.main)
        self.copy_out.wait_event(self.step_done)
        with torch.cuda.stream(self.copy_out):
            self.host_outputs.copy_(self.outputs, non_blocking=True)
            self.d2h_done.record(self.copy_out)
        self.steps += 1

    def drain(self):
        """Make the main stream wait for the copies still in flight (the last read-back and a pending prefetch)."""
        self.main.wait_event(self.d2h_done)
        if self._prefetched:
            self.main.wait_event(self.h2d_done)
