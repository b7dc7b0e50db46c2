"""Feature-axis sharding of the training step over the GPUs of one node.

The reference shards ``d_features`` with DTensor styles (column-parallel encoder,
sharded nonlinearity, row-parallel decoder whose partial outputs are all-reduced:
crosslayer_transcoder/model/parallel.py:157-339).  Here each rank simply constructs
its module with its own contiguous slice of the feature axis

    encoder.W[:, :, lo:hi]  encoder.b[:, lo:hi]  theta[:, :, lo:hi]  decoder.W_t[:, lo:hi, :]

(``decoder.b`` and the standardizers are replicated), every rank receives the same
batch, and the step's exchange is the sum of the partial normalised reconstructions
(NCCL all-reduce over NVLink).  The TopK selections, which the reference's plan does not
support, add one all-gather of each shard's k best values per row, from which every
rank derives the row's global threshold.  Backward needs no collective: the
reconstruction gradient is replicated and every parameter gradient is shard-local.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def feature_shard(d_features: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of the feature axis owned by ``rank``."""
    if d_features % world:
        raise ValueError(f"d_features={d_features} is not divisible by the {world} ranks")
    per = d_features // world
    return rank * per, (rank + 1) * per


def attach(module, group: Optional[dist.ProcessGroup] = None, fused="auto") -> None:
    """Mark ``module`` (built with this rank's feature slice) as one shard of a group.  With no
    group the default process group is used.

    ``fused`` asks for the exchange that is fused into the kernels over peer memory (the decoder of the
    JumpReLU / TopK step adds its partial rows straight into the owning rank's buffer, the loss backward
    writes its rows into every rank's buffer): "auto" uses it on an NCCL group when the ranks can map each other's
    memory, ``False`` keeps the NCCL all-reduce, ``True`` raises if peer mapping is not available."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    module.tp_group = group if group is not None else dist.group.WORLD
    module.tp_rank = dist.get_rank(module.tp_group)
    module.tp_world = dist.get_world_size(module.tp_group)
    module.tp_fused = False
    if fused and module.tp_world > 1 and dist.get_backend(module.tp_group) == "nccl":
        try:
            _symm()
            module.tp_fused = True
        except Exception:
            if fused is True:
                raise


def shard_module(module, rank: int, world: int) -> None:
    """Cut an unsharded training module down to ``rank``'s feature slice, in place: ``encoder.W`` /
    ``encoder.b``, the JumpReLU ``theta``, every decoder block and the ``last_active`` counters keep
    ``[lo, hi)`` of the feature axis (the placement of the reference's plan:
    crosslayer_transcoder/model/parallel.py:186-192, 235-246, 303-310); ``decoder.b``, the standardizers
    and the BatchTopK thresholds stay replicated.  Call it before the optimizer is created."""
    from torch import nn

    from .engine import StepEngine

    model = module.model
    enc, dec, nl = model.encoder, model.decoder, model.nonlinearity
    lo, hi = feature_shard(enc.d_features, rank, world)

    def cut(owner, name, axis):
        t = getattr(owner, name)
        new = t.detach().narrow(axis, lo, hi - lo).clone()
        if isinstance(t, nn.Parameter):
            setattr(owner, name, nn.Parameter(new, requires_grad=t.requires_grad))
        else:
            setattr(owner, name, new)

    cut(enc, "W", 2)
    cut(enc, "b", 1)
    if dec.crosslayer:
        for t in range(dec.n_layers):
            cut(dec, f"W_{t}", 1)
    else:
        cut(dec, "W", 1)
    if isinstance(getattr(nl, "theta", None), nn.Parameter):
        cut(nl, "theta", 2)
        nl.d_features = hi - lo
    enc.d_features = dec.d_features = hi - lo
    cut(module, "last_active", 1)
    module._engine = StepEngine(module)         # flat buffers are rebuilt for the new shapes
    enc.__dict__["_kernel_engine"] = dec.__dict__["_kernel_engine"] = module._engine


def _symm():
    """torch's symmetric-memory module, set up for plain peer pointers (no NVLink multicast binding:
    the kernels here use peer loads / stores / reductions only)."""
    import os

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem


class PeerBuffer:
    """A tensor of the same shape on every rank of ``group``, each rank's copy mapped into every other
    rank's address space.  ``local`` is this rank's tensor; ``bases`` is a CPU int64 tensor with the
    device address of every rank's copy (this rank's own at index ``rank``), in the form the C ABI's
    ``*_push`` entry points take.  Construction is collective over the group."""

    def __init__(self, shape, dtype, device, group):
        symm_mem = _symm()
        self.local = symm_mem.empty(*shape, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.local, group)
        rank = dist.get_rank(group)
        off = self.local.data_ptr() - int(self.handle.buffer_ptrs[rank])
        if off < 0 or off + self.local.numel() * self.local.element_size() > int(self.handle.buffer_size):
            raise RuntimeError("symmetric-memory tensor lies outside its registered buffer")
        self.bases = torch.tensor([int(p) + off for p in self.handle.buffer_ptrs], dtype=torch.int64)
        self._offset_bytes = off

    def peer(self, rank: int) -> torch.Tensor:
        """Rank ``rank``'s copy as a tensor of THIS device (its storage is the peer's memory, mapped here):
        plain copies into it travel over NVLink."""
        return self.handle.get_buffer(rank, tuple(self.local.shape), self.local.dtype,
                                      self._offset_bytes // self.local.element_size())


def all_reduce_sum(buf: torch.Tensor, group, async_op: bool = False):
    """Sum ``buf`` over the group in place.  With ``async_op`` the collective is only enqueued and a
    work handle is returned; ``handle.wait()`` orders the current stream after it."""
    return dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def all_gather(out: torch.Tensor, part: torch.Tensor, group, async_op: bool = False):
    """out[r] = rank r's ``part`` (out has a leading axis of the group size)."""
    if dist.get_backend(group) == "nccl":
        return dist.all_gather_into_tensor(out, part.contiguous(), group=group, async_op=async_op)
    return dist.all_gather(list(out.unbind(0)), part.contiguous(), group=group, async_op=async_op)


def upload_batch(batch_host: torch.Tensor, staging: torch.Tensor, group) -> torch.Tensor:
    """Bring a pinned host batch ``[B, ...]`` that every rank holds onto every GPU while crossing
    PCIe only once per row: rank r copies rows ``[r c, (r+1) c)`` (c = ceil(B / R)) host-to-device
    and the slices are all-gathered over NVLink.  ``staging`` is a device buffer ``[R c, ...]``;
    returns its first B rows."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B = batch_host.shape[0]
    c = (B + world - 1) // world
    lo, hi = min(rank * c, B), min((rank + 1) * c, B)
    mine = staging[rank * c:(rank + 1) * c]
    if hi > lo:
        mine[: hi - lo].copy_(batch_host[lo:hi], non_blocking=True)
    all_gather(staging.view(world, c, *staging.shape[1:]), mine, group)
    return staging[:B]


class ShardedBatchUploader:
    """Batch ingestion for a feature-shard group that uses the exchange fused into the kernels
    (``attach(module)`` with ``module.tp_fused``): every rank holds the pinned host batch ``[B, 2, L, D]``
    (what the reference's loader hands every tensor-parallel rank,
    crosslayer_transcoder/data/shared_memory.py:168-214), but each row crosses PCIe only once and NVLink
    carries only what the step reads.

    Rank r copies its own token rows ``[r c, (r+1) c)`` (c = ceil(B / R), both halves) host-to-device into
    its double-buffered device batch and copies the INPUT half of those rows into every peer's buffer
    (device-to-device copies on a side stream, no collective, no communicator): in this exchange form a
    rank standardises and encodes all tokens but computes the loss only for its own rows, so the target
    half of the other rows is never read.  ``full=True`` pushes both halves (for the first batch, from
    which the standardizers take their statistics).

    Ordering between the ranks.  The pushes of batch i+1 are enqueued while step i runs.  For small uploads
    the step's own last collective (the all-reduce of the decoder-bias gradient, at the start of backward)
    is made to wait for this rank's pushes (``StepEngine.before_last_collective``), so when that collective
    has completed on a rank, every peer's rows for batch i+1 have landed in its buffer, at no extra cost.
    An upload that may take longer than the forward pass (more than ``late_join_bytes`` per rank) would stall
    that collective; it is joined at the END of backward instead (``StepEngine.after_backward``), by a
    one-element all-reduce of its own, so that the copies have the whole step to finish.  Either way a buffer
    is overwritten only after the step that read it has finished on every rank, which the same collective of
    that step guarantees.

        up = ShardedBatchUploader(module, batch_host.shape, batch_host.dtype, device)
        up.upload(first, full=True); up.fence()     # then, per step:
        batch = up.take()                           # current stream waits for the newest upload
        up.upload(next_host_batch)                  # prefetch while the step runs
        loss = module.training_step(batch, i); loss.backward(); opt.step()
        up.release()                                # the step's work on `batch` is enqueued
    """

    late_join_bytes = 48 << 20

    def __init__(self, module, shape, dtype, device):
        if not getattr(module, "tp_fused", False) or not module._engine.has_fused_exchange():
            raise RuntimeError("ShardedBatchUploader needs a module attached with the fused exchange "
                               "(and a step kind that has it)")
        self.module, self.group = module, module.tp_group
        self.world, self.rank = module.tp_world, module.tp_rank
        B = shape[0]
        self.B, self.c = B, (B + self.world - 1) // self.world
        self.lo, self.hi = min(self.rank * self.c, B), min((self.rank + 1) * self.c, B)
        self.bufs = [PeerBuffer(tuple(shape), dtype, device, self.group) for _ in range(2)]
        self.peers = [[b.peer(r) for r in range(self.world)] for b in self.bufs]
        self.stream = torch.cuda.Stream(device=device)
        self.pushed = [torch.cuda.Event(), torch.cuda.Event()]
        self.freed = [torch.cuda.Event(), torch.cuda.Event()]
        for e in self.freed:
            e.record()
        self._next, self._ready, self._in_use = 0, [], []
        row_bytes = int(torch.Size(shape[1:]).numel()) * torch.empty((), dtype=dtype).element_size()
        self.late_join = (self.hi - self.lo) * row_bytes > self.late_join_bytes
        if self.late_join:
            module._engine.after_backward = self._join_and_fence
        else:
            module._engine.before_last_collective = self._join

    def upload(self, batch_host: torch.Tensor, full: bool = False) -> None:
        slot = self._next
        self._next ^= 1
        lo, hi = self.lo, self.hi
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(self.freed[slot])
            if hi > lo:
                mine = self.bufs[slot].local[lo:hi]
                mine.copy_(batch_host[lo:hi], non_blocking=True)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    dst = self.peers[slot][r][lo:hi]
                    if full:
                        dst.copy_(mine, non_blocking=True)
                    else:
                        dst[:, 0].copy_(mine[:, 0], non_blocking=True)
            self.pushed[slot].record(self.stream)
        self._ready.append(slot)

    def _join(self):
        """Called by the engine right before the last collective of a step: this rank takes part in it
        only after its pushes of the next batch have been written."""
        for slot in self._ready:
            torch.cuda.current_stream().wait_event(self.pushed[slot])

    def _join_and_fence(self):
        """Called by the engine when a backward pass has been enqueued (large uploads): wait for this rank's
        pushes of the next batch, then a one-element all-reduce waits for everyone's."""
        if self._ready:
            self.fence()

    def detach(self) -> None:
        """Take the uploader's hooks out of the engine (its buffers stay valid until they are dropped)."""
        eng = self.module._engine
        eng.before_last_collective = None
        eng.after_backward = None

    def fence(self) -> None:
        """Stream-ordered barrier for a batch that no step's collective has ordered yet (the first one): the
        current stream waits for this rank's pushes, then a one-element all-reduce waits for everyone's."""
        self._join()
        if not hasattr(self, "_token"):
            self._token = torch.zeros(1, dtype=torch.float32, device=self.bufs[0].local.device)
        all_reduce_sum(self._token, self.group)

    def take(self) -> torch.Tensor:
        """The oldest uploaded batch not yet handed out; the current stream waits for this rank's part of it.
        (The peers' parts are ordered by the previous step's last collective; before the first step the
        caller calls ``fence()`` once.)"""
        slot = self._ready.pop(0)
        torch.cuda.current_stream().wait_event(self.pushed[slot])
        self._in_use.append(slot)
        return self.bufs[slot].local[: self.B]

    def release(self) -> None:
        slot = self._in_use.pop(0)
        self.freed[slot].record()


# --------------------------------------------------------------------------------------------------
# checkpoints of feature-sharded modules in the reference's (unsharded) layout
# --------------------------------------------------------------------------------------------------
def _feature_axis(key: str, ndim: int):
    """Axis of the feature dimension for a state-dict key of the transcoder, or None if replicated.
    encoder.W [L,D,F] -> 2, encoder.b [L,F] -> 1, decoder.W_t [(t+1),F,D] / decoder.W [L,F,D] -> 1,
    nonlinearity.theta [1,L,F] -> 2, last_active [L,F] -> 1; decoder.b, standardizers, thresholds: replicated."""
    leaf = key.split(".")[-1]
    owner = key.split(".")[-2] if "." in key else ""
    if owner == "encoder":
        return {"W": 2, "b": 1}.get(leaf)
    if owner == "decoder":
        return 1 if leaf.startswith("W") else None
    if leaf == "theta":
        return 2
    if leaf == "last_active":
        return 1
    return None


def gather_state_dict(module: torch.nn.Module, group=None) -> dict:
    """State dict of a feature-sharded module with every sharded tensor concatenated over the ranks, i.e.
    the keys and shapes of the reference's unsharded module (what ``save_pretrained`` / ``load_state_dict``
    of the reference expect).  Every rank gets the full dict."""
    group = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    out = {}
    for key, t in module.state_dict().items():
        ax = _feature_axis(key, t.dim())
        if ax is None or world == 1:
            out[key] = t.detach().clone()
            continue
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.detach().contiguous(), group=group)
        out[key] = torch.cat(parts, dim=ax)
    return out


def shard_state_dict(full: dict, rank: int, world: int) -> dict:
    """The slice of an unsharded (reference-layout) state dict that ``rank`` of ``world`` holds."""
    out = {}
    for key, t in full.items():
        ax = _feature_axis(key, t.dim())
        if ax is None or world == 1:
            out[key] = t
        else:
            lo, hi = feature_shard(t.shape[ax], rank, world)
            out[key] = t.narrow(ax, lo, hi - lo).contiguous()
    return out
