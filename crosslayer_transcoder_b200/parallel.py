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
