"""Warm-up and retention hooks of the reference's public API, for this backend.

The reference chooses between kernel variants with a stopwatch and caches
expanded weights; ``warmup / decisions / undecided / retain / retained_stats /
invalidate`` (``src/qste/capture.py:38-140``) exist there to move that measuring
and caching out of a training step or a CUDA-graph capture.  This build picks
kernels from the shape alone and never materialises an expanded weight, so there
is nothing to measure and nothing to cache.  The functions keep the reference's
signatures and return types -- ``undecided(model, *args, **kwargs) -> bool``,
``retain(budget_bytes) -> None``, ``retained_stats()`` with its five keys -- so
host code written against the reference runs unchanged and gets the answers of
a backend whose every decision is already made.
"""

from __future__ import annotations

import torch

from . import kernels
from .convert import surfaces


def warmup(model, *args, **kwargs) -> dict:
    """Load the kernel library and run one forward; returns ``decisions()``."""

    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("warmup() must run before a CUDA-graph capture, not inside it")
    for surface in surfaces(model):
        kernels.warm(surface.coordinate.device)
    with torch.no_grad():
        model(*args, **kwargs)
    return decisions()


def decisions() -> dict:
    """Choices made by measurement, keyed ``(device, rows, columns, samples, has_bias,
    dtype)`` in the reference: always empty here, the choice is a function of the shape."""

    return {}


def undecided(model, *args, **kwargs) -> bool:
    """Whether this call would still have to measure something: never.  The forward is
    run all the same (without gradients), as the reference's does, so a host that uses
    this as its pre-capture dry run still gets one."""

    with torch.no_grad():
        model(*args, **kwargs)
    return False


_budget = {"bytes": 0}


def retain(budget_bytes: int) -> None:
    """Budget for expanded weights kept across calls.  Recorded and reported back by
    :func:`retained_stats`; nothing is ever held against it, because no kernel of this
    build expands a weight into memory."""

    budget_bytes = int(budget_bytes)
    if budget_bytes < 0:
        raise ValueError("retain() budget must be >= 0 bytes")
    _budget["bytes"] = budget_bytes


def retained_stats() -> dict[str, int]:
    return {"hits": 0, "misses": 0, "resident_bytes": 0, "budget_bytes": _budget["bytes"], "entries": 0}


def invalidate(packed) -> None:
    """Drop anything expanded from these packed bits: nothing is, so nothing to do."""

    del packed
