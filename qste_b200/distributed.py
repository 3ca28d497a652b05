"""Data-parallel training of binary surfaces.

Coordinate evidence is not an autograd gradient: coordinates carry
``requires_grad=False``, so DDP's bucketed all-reduce never sees it.  Without an
explicit reduction every rank would step its coordinates from its own batch and
the ranks' signs would drift apart while the loss keeps falling.  The reducers
here are that reduction; ``QSTEOptimizer`` installs ``mean_evidence()`` by default
whenever a process group exists.  After the reduction every rank runs the same
deterministic update (the rounding stream depends only on seed, step and index)
and holds byte-identical coordinates, so nothing else needs to be exchanged.

``mean_evidence(overlap=True)`` runs the NCCL all-reduce (the mean rides the collective
for power-of-two worlds) and -- when the caller is ``QSTEOptimizer`` -- the coordinate
update of that surface on a side stream, so that the rest of backward on the compute stream waits
for none of them; ``QSTEOptimizer.step()`` joins the side stream.  Called by
anything else the reducer makes the compute stream wait for the reduced tensor
(``join=True``), which is always safe.

API follows ``src/qste/distributed.py`` of the reference (reducers :46-75,
broadcast :78-95, digest :98-116, FSDP helpers :125-172).
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
from torch import Tensor

from .convert import surfaces as _surfaces
from .surface import Surface


def _distributed_ready() -> bool:
    return torch.distributed.is_available() and torch.distributed.is_initialized()


_side_streams: dict[int, torch.cuda.Stream] = {}


def _side_stream(device: torch.device) -> torch.cuda.Stream:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _side_streams:
        _side_streams[index] = torch.cuda.Stream(device=device)
    return _side_streams[index]


def _all_reduce(evidence: Tensor, group, average: bool, overlap: bool, join: bool = True) -> Tensor:
    world = torch.distributed.get_world_size(group)
    if overlap and evidence.is_cuda:
        # The evidence GEMM that produced `evidence` ran on the current stream.  The
        # collective goes to the side stream, after that GEMM.  With
        # `join` the compute stream then waits for the result; without it the result is
        # valid on the side stream only and the caller carries on there.
        compute = torch.cuda.current_stream(evidence.device)
        side = _side_stream(evidence.device)
        wait_for_producer(side, compute, evidence)
        with torch.cuda.stream(side):
            _reduce(evidence, group, average, world)
        evidence.record_stream(side)
        if join:
            compute.wait_stream(side)
        return evidence
    return _reduce(evidence, group, average, world)


def wait_for_producer(side: torch.cuda.Stream, compute: torch.cuda.Stream, evidence: Tensor) -> None:
    """Make `side` wait until `evidence` is complete.  The fused backward tags the evidence with
    the event it records right after the evidence product (``_qste_ready``): waiting for that
    instead of for the whole compute stream lets the side stream start while the dX product of
    the same layer is still running."""

    ready = getattr(evidence, "_qste_ready", None)
    if ready is not None:
        side.wait_event(ready)
    else:
        side.wait_stream(compute)


def _reduce(evidence: Tensor, group, average: bool, world: int) -> Tensor:
    """Sum over ranks, then the mean (src/qste/distributed.py:53-59 of the reference: all_reduce
    then div_).  With NCCL and a power-of-two world the division rides the collective (ncclAvg
    scales every rank's contribution by 1/world, which is exact for a power of two, so the
    result is bit for bit the sum divided afterwards) and the separate pass over the 4 bytes per
    coordinate disappears."""

    if average and evidence.is_cuda and world & (world - 1) == 0 and \
            torch.distributed.get_backend(group) == "nccl":
        torch.distributed.all_reduce(evidence, op=torch.distributed.ReduceOp.AVG, group=group)
        return evidence
    torch.distributed.all_reduce(evidence, op=torch.distributed.ReduceOp.SUM, group=group)
    return evidence.div_(world) if average else evidence


def _reserve_for_overlap(reserve_sms: int | None) -> None:
    """An overlapped reducer's collective runs beside the persistent GEMMs of backward, which
    otherwise hold every SM: keep a few out of their grids (8 unless told otherwise; the
    environment variable QSTE_B200_RESERVED_SMS overrides the default)."""

    import os

    from . import kernels

    if reserve_sms is None:
        reserve_sms = int(os.environ.get("QSTE_B200_RESERVED_SMS", "8"))
    kernels.set_backward_reserve(reserve_sms)


def mean_evidence(group=None, *, overlap: bool = False, reserve_sms: int | None = None) -> Callable[[Tensor], Tensor]:
    """Reducer that averages evidence over ranks (what DDP does to gradients).

    ``overlap`` (not in the reference) runs the collective on a side stream beside the rest of
    backward; ``reserve_sms`` is how many SMs the backward GEMMs then leave free for it."""

    def reduce(evidence: Tensor, *, join: bool = True) -> Tensor:
        if not _distributed_ready():
            return evidence
        return _all_reduce(evidence, group, average=True, overlap=overlap, join=join)

    reduce.side_stream = _side_stream if overlap else None
    if overlap and _distributed_ready() and torch.distributed.get_world_size(group) > 1:
        _reserve_for_overlap(reserve_sms)
    return reduce


def sum_evidence(group=None, *, overlap: bool = False, reserve_sms: int | None = None) -> Callable[[Tensor], Tensor]:
    """Reducer that sums evidence, for hosts that sum gradients."""

    def reduce(evidence: Tensor, *, join: bool = True) -> Tensor:
        if not _distributed_ready():
            return evidence
        return _all_reduce(evidence, group, average=False, overlap=overlap, join=join)

    reduce.side_stream = _side_stream if overlap else None
    if overlap and _distributed_ready() and torch.distributed.get_world_size(group) > 1:
        _reserve_for_overlap(reserve_sms)
    return reduce


@torch.no_grad()
def broadcast_surfaces(model: nn.Module, src: int = 0, group=None) -> int:
    """Make every rank's binary state equal to ``src``'s; returns tensors sent."""

    if not _distributed_ready():
        return 0
    sent = 0
    for surface in _surfaces(model):
        for tensor in (surface.coordinate.data, surface.packed_sign.data, surface.log_scale.data):
            torch.distributed.broadcast(tensor, src=src, group=group)
            sent += 1
    return sent


@torch.no_grad()
def surfaces_agree(model: nn.Module, group=None) -> bool:
    """True when every rank holds the same signs and coordinates (a debug assert)."""

    if not _distributed_ready():
        return True
    digest = torch.zeros((), dtype=torch.float64, device=_first_device(model))
    for surface in _surfaces(model):
        digest += surface.packed_sign.data.to(torch.float64).sum()
        digest += surface.coordinate.data.to(torch.float64).sum()
    lowest, highest = digest.clone(), digest.clone()
    torch.distributed.all_reduce(lowest, op=torch.distributed.ReduceOp.MIN, group=group)
    torch.distributed.all_reduce(highest, op=torch.distributed.ReduceOp.MAX, group=group)
    return bool(torch.equal(lowest, highest))


def _first_device(model: nn.Module) -> torch.device:
    for parameter in model.parameters():
        return parameter.device
    return torch.device("cpu")


def fsdp_ignored_states(model: nn.Module) -> list[nn.Parameter]:
    """Parameters FSDP must not flatten (``ignored_states=``): int8 coordinates, uint8
    signs and the row scales of every surface.  They stay replicated and are kept in
    sync by an evidence reducer."""

    ignored: list[nn.Parameter] = []
    for surface in _surfaces(model):
        ignored += [surface.coordinate, surface.packed_sign, surface.log_scale]
    return ignored


def fsdp_ignored_modules(model: nn.Module) -> list[Surface]:
    """The surfaces themselves, for FSDP versions that take ``ignored_modules``."""

    return list(_surfaces(model))


def replicated_bytes(model: nn.Module) -> int:
    """Per-rank bytes of the surfaces that FSDP leaves replicated."""

    total = 0
    for surface in _surfaces(model):
        cost = surface.memory()
        total += cost["packed_sign"] + cost["coordinate"] + cost["log_scale"]
    return total


__all__ = [
    "broadcast_surfaces", "fsdp_ignored_modules", "fsdp_ignored_states", "mean_evidence",
    "replicated_bytes", "sum_evidence", "surfaces_agree",
]
