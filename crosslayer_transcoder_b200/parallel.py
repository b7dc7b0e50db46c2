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


def attach(module, group: Optional[dist.ProcessGroup] = None) -> None:
    """Mark ``module`` (built with this rank's feature slice) as one shard of a group.  With no
    group the default process group is used."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    module.tp_group = group if group is not None else dist.group.WORLD
    module.tp_rank = dist.get_rank(module.tp_group)
    module.tp_world = dist.get_world_size(module.tp_group)


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
