"""Publish host-pool pages appended this step, over all requests and groups, with one upload and one launch.

Same constructor and `submit(rows, ring)` as the reference's PageUpdates (python/kvip/cache/page_updates.py:5-62).
Each row is `[flat page index, host address, old map offset or -1]`: the page's committed address is stored,
its valid flag set, the `block_size` token-to-slot entries that start at the old map offset are reset to -1,
and for groups that keep per-token addresses (`fused`) the page's tokens get `address + lane * width *
token_bytes`. The reference ran a Triton program per page (python/kvip/cache/_page_updates_kernel.py:8-40);
here the rows go to the device from one of two pinned host buffers and `publish_pages` runs once on the
current stream. There is no host fallback: the tensors must live on a CUDA device."""
import ctypes

import numpy as np

from .. import _lib


class PageUpdates:
    def __init__(self, torch, addresses, valid, token_to_slot, *, fused=(), widths=(), token_bytes=656, block_size=128):
        if addresses.ndim != 3 or tuple(valid.shape) != tuple(addresses.shape):
            raise ValueError("PageUpdates: addresses and valid are [owners, groups, pages]")
        for name, tensor, dtype in (("addresses", addresses, torch.int64), ("valid", valid, torch.int32),
                                    ("token_to_slot", token_to_slot, torch.int32)):
            if not tensor.is_cuda or tensor.dtype != dtype or not tensor.is_contiguous():
                raise ValueError(f"PageUpdates: {name} must be a contiguous {dtype} CUDA tensor")
        self.torch = torch
        self.addresses, self.valid, self.token_to_slot = addresses, valid, token_to_slot
        self.block_size = block_size
        self.fused = tuple(fused)
        self.widths, self.token_bytes = tuple(widths), token_bytes
        if self.fused:
            if len(self.fused) != addresses.shape[1] or len(self.widths) != len(self.fused):
                raise ValueError("PageUpdates: one fused table and one width per group")
            history = self.fused[0].shape[1]
            for table in self.fused:
                if (not table.is_cuda or table.dtype != torch.int64 or not table.is_contiguous()
                        or tuple(table.shape) != (addresses.shape[0], history)):
                    raise ValueError("PageUpdates: fused tables are contiguous int64 [owners, history] CUDA tensors")
        # Each row contains [flat page index, host address, old map offset/-1].
        shape = (addresses.numel(), 3)
        self.device = torch.empty(shape, dtype=torch.int64, device=addresses.device)
        self.host = [torch.empty(shape, dtype=torch.int64, pin_memory=True) for _ in range(2)]
        self.fused_table = torch.tensor(
            [(t.data_ptr(), width * token_bytes) for t, width in zip(self.fused, self.widths)] or [(0, 0)],
            dtype=torch.int64, device=addresses.device)
        self.errors = torch.zeros(1, dtype=torch.int32, device=addresses.device)
        self._args = _lib.PagesArgs(
            rows=self.device.data_ptr(), addresses=addresses.data_ptr(), valid=valid.data_ptr(),
            token_to_slot=token_to_slot.data_ptr(), fused_table=self.fused_table.data_ptr() if self.fused else None,
            errors=self.errors.data_ptr(), map_entries=token_to_slot.numel(), count=0, owners=addresses.shape[0],
            groups=addresses.shape[1], pages=addresses.shape[2], block=block_size,
            history=self.fused[0].shape[1] if self.fused else 0)

    @property
    def nbytes(self):
        return self.device.numel() * self.device.element_size() + self.fused_table.numel() * 8

    def submit(self, rows, ring):
        """Upload `rows` through pinned buffer `ring` (0 or 1) and publish them on the current stream. The
        caller alternates `ring` between steps and synchronises before a buffer's second-next use."""
        if not rows:
            return
        table = np.asarray(rows, dtype=np.int64).reshape(-1, 3)
        if table[:, 0].min() < 0 or table[:, 0].max() >= self.addresses.numel():
            raise IndexError("PageUpdates.submit: flat page index out of range")
        clears = table[:, 2]
        if (clears < -1).any() or (clears + self.block_size > self.token_to_slot.numel()).any():
            raise IndexError("PageUpdates.submit: map offset out of range")
        if len(np.unique(table[:, 0])) != len(table):
            # one program per row, as in the reference's device path: two rows for one page would race
            raise ValueError("PageUpdates.submit: a page may be listed once per call")
        count = len(table)
        host = self.host[ring][:count]
        host.numpy()[:] = table
        self.device[:count].copy_(host, non_blocking=True)
        self._args.count = count
        lib = _lib.load_library()
        stream = ctypes.c_void_p(self.torch.cuda.current_stream(self.addresses.device).cuda_stream)
        _lib.check(lib.kvip_b200_publish_pages(ctypes.byref(self._args), stream), "publish_pages", lib)
