"""Device-side consumers of the reference's two batch sources.

* ``SharedBufferBatches`` reads a ``SharedActivationBuffer``
  (crosslayer_transcoder/data/shared_memory.py:23-214): a ``[buffer_size, 2, L, D]`` tensor in host shared
  memory with a validity mask, filled by generator processes.  The reference's ``get_activations`` picks
  ``batch_size`` random valid rows under the buffer lock, copies them into a new pageable tensor on one CPU
  thread and invalidates them; Lightning then uploads that tensor.  Here the choice of rows is the same
  (same calls on torch's CPU generator, so the same rows for the same seed), but the rows are moved by the
  GPU: the shared mapping is registered with the CUDA driver once and ``clt_gather_batch_rows`` reads the
  chosen rows over PCIe straight into a device batch, on a side stream, one batch ahead of the step.
* ``TensorBatches`` / ``TensorDataModule`` iterate a ``[n_samples, 2, L, D]`` tensor like
  ``InfiniteTensorDataset`` / ``TensorDataModule`` (crosslayer_transcoder/data/tensor_datamodule.py:14-121):
  the tensor lives in HBM when it fits (the default on a 180 GB device), else in registered host memory,
  and each batch is one row-gather kernel.

Both yield device tensors that ``module.training_step`` consumes directly.  A yielded batch stays valid
until the iterator has been advanced ``depth`` more times.
"""
from __future__ import annotations

import ctypes
import time
from typing import Iterator, Optional

import torch

from ._lib import CltError, lib


def draw_rows(store, batch_size: int) -> Optional[torch.Tensor]:
    """The row choice of ``SharedActivationBuffer.get_activations`` (shared_memory.py:184-195), to be called
    with ``store.buffer_lock`` held: None while the store is below its fill threshold or holds fewer than
    ``batch_size`` valid rows, else ``batch_size`` distinct valid row indices drawn with ``torch.randperm``."""
    with store.validity_lock:
        valid = torch.nonzero(store.validity_tensor, as_tuple=False).squeeze(-1)
    if len(valid) / store.buffer_size < store.minimum_fill_threshold or batch_size > len(valid):
        return None
    return valid[torch.randperm(len(valid))[:batch_size]]


def retire_rows(store, rows: torch.Tensor) -> None:
    """Mark ``rows`` as consumed (shared_memory.py:199-204, 259-267)."""
    with store.validity_lock:
        store.validity_tensor[rows] = False
    stats = getattr(store, "stats", None)
    if isinstance(stats, dict):
        stats["total_reads"] = stats.get("total_reads", 0) + 1
        stats["last_read_time"] = time.time()


class HostMapping:
    """A host tensor's memory registered with the CUDA driver and mapped into the device's address space."""

    def __init__(self, tensor: torch.Tensor):
        if tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("HostMapping needs a contiguous CPU tensor")
        self.tensor = tensor
        self.host_ptr = tensor.data_ptr()
        dev = ctypes.c_void_p()
        lib().check_device()
        lib().call("clt_host_register", self.host_ptr, tensor.numel() * tensor.element_size(), ctypes.byref(dev))
        self.device_ptr = dev.value

    def close(self):
        if self.host_ptr is not None:
            lib().call("clt_host_unregister", self.host_ptr)
            self.host_ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _RowGather:
    """``dst[i] = src[rows[i]]`` on a side stream; src in device memory or a registered host mapping."""

    def __init__(self, src_ptr: int, n_src_rows: int, row_shape, dtype, device, depth: int, max_rows: int):
        self.src_ptr, self.n_src_rows = src_ptr, n_src_rows
        self.row_bytes = int(torch.Size(row_shape).numel()) * torch.empty((), dtype=dtype).element_size()
        if self.row_bytes % 16 != 0:
            raise ValueError("batch rows must be a multiple of 16 bytes")
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.depth = depth
        self.out = [torch.empty((max_rows, *row_shape), dtype=dtype, device=self.device) for _ in range(depth)]
        self.rows_host = [torch.empty(max_rows, dtype=torch.int64).pin_memory() for _ in range(depth)]
        self.rows_dev = [torch.empty(max_rows, dtype=torch.int64, device=self.device) for _ in range(depth)]
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self.freed = [torch.cuda.Event() for _ in range(depth)]
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        for e in self.freed:
            e.record(torch.cuda.current_stream(self.device))

    def launch(self, slot: int, rows: torch.Tensor) -> torch.cuda.Event:
        n = len(rows)
        self.rows_host[slot][:n].copy_(rows)
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(self.freed[slot])
            self.rows_dev[slot][:n].copy_(self.rows_host[slot][:n], non_blocking=True)
            lib().call("clt_gather_batch_rows", self.src_ptr, self.rows_dev[slot], self.out[slot], self.row_bytes, n,
                       self.n_src_rows, self.status, self.stream.cuda_stream)
            self.done[slot].record(self.stream)
        return self.done[slot]

    def check(self):
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise CltError(f"batch gather: device status {code:#x} (a row index was out of range)")


class SharedBufferBatches:
    """Iterator over device batches ``[batch_size, 2, L, D]`` drawn from a ``SharedActivationBuffer`` (or any
    object with its ``buffer_tensor``, ``validity_tensor``, ``buffer_lock``, ``validity_lock``,
    ``buffer_size`` and ``minimum_fill_threshold``).

    ``mode="mapped"``: the GPU gathers from the registered shared mapping (no CPU copy).
    ``mode="staged"``: a CPU ``index_select`` into pinned memory, then one host-to-device copy (for stores
    whose memory cannot be registered, e.g. under a locked-memory limit).

    One batch is always in flight: ``__next__`` hands out the batch whose gather was launched by the previous
    call and launches the next one on a side stream before it returns, so the gather runs under the step
    that consumes the current batch.  Rows are chosen under the buffer lock and stay VALID while the GPU
    reads them — generator processes only refill invalid rows, so they cannot overwrite a row in flight —
    and are invalidated once the gather has completed (one consumer per store, as in the reference).  No
    thread is used: the host work per batch is the row choice (``nonzero`` + ``randperm``), which runs
    while the device executes the step that was just enqueued."""

    def __init__(self, store, batch_size: Optional[int] = None, device="cuda", depth: int = 2, mode: str = "mapped",
                 timeout: float = 1000.0):
        batch_size = batch_size or store.batch_size
        if not batch_size or batch_size <= 0:
            raise ValueError("batch_size must be positive")
        if mode not in ("mapped", "staged"):
            raise ValueError("mode is 'mapped' or 'staged'")
        self.store, self.batch_size, self.timeout, self.mode = store, batch_size, timeout, mode
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        buf = store.buffer_tensor
        row_shape = tuple(buf.shape[1:])
        self.depth = depth
        self.n_slots = depth + 1           # `depth` batches with the caller, one in flight
        with torch.cuda.device(self.device):
            if mode == "mapped":
                self.mapping = HostMapping(buf)
                src = self.mapping.device_ptr
            else:
                self.mapping = None
                self.pinned = [torch.empty((batch_size, *row_shape), dtype=buf.dtype).pin_memory()
                               for _ in range(self.n_slots)]
                src = 0
            self.gather = _RowGather(src, buf.shape[0], row_shape, buf.dtype, self.device, self.n_slots, batch_size)
        self._slot = 0
        self._held = []
        self._flight = None                # (slot, rows) of the gather in flight

    def _move(self, slot: int, rows: torch.Tensor) -> torch.cuda.Event:
        g = self.gather
        if self.mode == "mapped":
            return g.launch(slot, rows)
        torch.index_select(self.store.buffer_tensor, 0, rows, out=self.pinned[slot])
        with torch.cuda.stream(g.stream):
            g.stream.wait_event(g.freed[slot])
            g.out[slot].copy_(self.pinned[slot], non_blocking=True)
            g.done[slot].record(g.stream)
        return g.done[slot]

    def _launch(self, block: bool) -> bool:
        """Choose the next batch's rows and start moving them; with ``block`` wait (up to ``timeout``) for
        the store to hold enough valid rows, as ``get_activations`` does."""
        t0 = time.time()
        while True:
            with self.store.buffer_lock:
                rows = draw_rows(self.store, self.batch_size)
                if rows is not None:
                    slot = self._slot
                    self._slot = (slot + 1) % self.n_slots
                    self._move(slot, rows)
                    self._flight = (slot, rows)
                    return True
            if not block:
                return False
            if time.time() - t0 > self.timeout:
                raise TimeoutError("Timeout waiting for valid indices")
            time.sleep(0.01)

    def _land(self) -> int:
        """Wait for the gather in flight, invalidate its rows, return its slot."""
        slot, rows = self._flight
        self._flight = None
        self.gather.done[slot].synchronize()
        with self.store.buffer_lock:
            retire_rows(self.store, rows)
        return slot

    def __iter__(self) -> Iterator[torch.Tensor]:
        return self

    def __next__(self) -> torch.Tensor:
        cur = torch.cuda.current_stream(self.device)
        # the batch handed out `depth` calls ago is released; work already enqueued on it still runs first
        if len(self._held) >= self.depth:
            self.gather.freed[self._held.pop(0)].record(cur)
        if self._flight is None:
            self._launch(block=True)
        slot = self._land()
        cur.wait_event(self.gather.done[slot])
        self._held.append(slot)
        self._launch(block=False)          # the next batch, if the store can supply it already
        return self.gather.out[slot]

    def close(self):
        if self._flight is not None:
            self._land()
        torch.cuda.synchronize(self.device)
        if self.mapping is not None:
            self.mapping.close()
            self.mapping = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TensorBatches:
    """``InfiniteTensorDataset`` (tensor_datamodule.py:14-34) with the gather on the device: every epoch
    draws ``torch.randperm(n)`` on the CPU generator (or 0..n-1 without shuffling) and yields
    ``tensor[indices[i : i + batch_size]]`` — the epoch's last batch may be shorter — as device tensors.

    ``resident=None`` keeps the tensor in device memory when it takes less than half of the free memory,
    otherwise in registered host memory that the gather kernel reads over PCIe."""

    def __init__(self, tensor: torch.Tensor, batch_size: int, shuffle: bool = True, device="cuda", depth: int = 2,
                 resident: Optional[bool] = None):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.batch_size, self.shuffle = batch_size, shuffle
        self.device = torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        tensor = tensor.contiguous()
        self.n = tensor.shape[0]
        nbytes = tensor.numel() * tensor.element_size()
        with torch.cuda.device(self.device):
            if resident is None:
                resident = tensor.is_cuda or nbytes < torch.cuda.mem_get_info()[0] // 2
            if resident:
                self.src, self.mapping = tensor.to(self.device), None
                src_ptr = self.src.data_ptr()
            else:
                self.src = tensor
                self.mapping = HostMapping(tensor)
                src_ptr = self.mapping.device_ptr
            self.depth = depth
            self.gather = _RowGather(src_ptr, self.n, tuple(tensor.shape[1:]), tensor.dtype, self.device, depth + 1,
                                     min(batch_size, self.n))
        self._slot = 0
        self._held = []

    def __iter__(self) -> Iterator[torch.Tensor]:
        while True:
            order = torch.randperm(self.n) if self.shuffle else torch.arange(self.n)
            for i in range(0, self.n, self.batch_size):
                rows = order[i:i + self.batch_size]
                cur = torch.cuda.current_stream(self.device)
                if len(self._held) >= self.depth:
                    self.gather.freed[self._held.pop(0)].record(cur)
                slot = self._slot
                self._slot = (slot + 1) % (self.depth + 1)
                cur.wait_event(self.gather.launch(slot, rows))
                self._held.append(slot)
                yield self.gather.out[slot][:len(rows)]

    def close(self):
        torch.cuda.synchronize(self.device)
        if self.mapping is not None:
            self.mapping.close()


class TensorDataModule:
    """The reference's ``TensorDataModule`` surface (tensor_datamodule.py:37-121: same constructor arguments,
    ``setup`` / ``train_dataloader`` / ``val_dataloader`` / ``teardown``) over ``TensorBatches``.
    ``num_workers`` and ``pin_memory`` are accepted and unused: there are no loader workers and no staging
    copy."""

    def __init__(self, tensor_file: str, batch_size: int = 16, shuffle: bool = True, num_workers: int = 0,
                 pin_memory: bool = False, device="cuda"):
        self.tensor_file, self.batch_size, self.shuffle = tensor_file, batch_size, shuffle
        self.num_workers, self.pin_memory, self.device = num_workers, pin_memory, device
        self.dataset = None
        self.train_loader = None

    def setup(self, stage: Optional[str] = None):
        if stage == "fit" or stage is None:
            tensor = torch.load(self.tensor_file, weights_only=True)
            self.dataset = TensorBatches(tensor, self.batch_size, self.shuffle, device=self.device)
            self.train_loader = self.dataset

    def train_dataloader(self):
        return self.train_loader

    def val_dataloader(self):
        return self.train_loader

    def teardown(self, stage: Optional[str] = None):
        if self.dataset is not None:
            self.dataset.close()
            self.dataset = None
