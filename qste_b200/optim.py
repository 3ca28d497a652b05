"""The coordinate optimizer.

Owns the int8 coordinates and nothing else: row scales and biases are ordinary
float parameters that the host's own optimizer steps.  State per surface
(``rows x columns``):

    moment_q      int8  rows x columns    first moment, block-quantised
    moment_scale  fp16  ceil(n / block)   one scale per block, initially 1/127
    row_v, col_v  fp16  rows / columns    factored second moment, initially 0

One byte per weight.  By default the update of a surface runs inside backward, as
soon as that surface's evidence exists (``Surface.consume_evidence`` calls
``_apply``); ``step()`` applies whatever was deferred, clamps the row scales,
advances the step counter and returns the number of flipped signs.  Flip counts
are accumulated on the device and read once per ``step()``.

API, state layout, seeds and ``state_dict`` format follow ``src/qste/optim.py`` of
the reference (state :79-92, reducer default :101-116, _apply :156-178, step
:180-201, checkpoint :212-232).
"""

from __future__ import annotations

import contextlib
import math
import os
from typing import Callable, Iterable, Mapping

import torch
import torch.nn as nn
from torch import Tensor

from . import kernels
from .config import QSTEConfig, coerce_config
from .convert import surfaces as _model_surfaces
from .surface import Surface

_SURFACE_SEED_STRIDE = 1_000_003
# default of QSTEOptimizer(async_update=None)
_ASYNC_UPDATE = os.environ.get("QSTE_B200_ASYNC_UPDATE", "0") == "1"


def _reducer_is_live() -> bool:
    return torch.distributed.is_available() and torch.distributed.is_initialized()


class QSTEOptimizer:
    """Steps int8 coordinates from the evidence backward produced.

    model             a converted model, or an iterable of surfaces
    config            numerics; defaults to the config ``convert`` recorded
    gradient_reducer  called on each surface's fp32 evidence before it is applied.
                      ``None`` / ``True``: ``distributed.mean_evidence()`` when a
                      process group is initialised, nothing otherwise.  ``False``:
                      no reduction.  A callable: used as given.
    async_update      (not in the reference) run the coordinate updates that backward
                      triggers on a side CUDA stream, joined by ``step()``: their small
                      memory-bound kernels then fill in beside the next layer's backward
                      (3 % of a step on one B200).  The coordinates and signs are only
                      guaranteed up to date after ``step()``; anything that reads them
                      between ``backward()`` and ``step()`` must not use this.  Default
                      off (``QSTE_B200_ASYNC_UPDATE=1`` turns it on).  An overlapped
                      reducer (``mean_evidence(overlap=True)``) implies it.
    """

    def __init__(self, model: nn.Module | Iterable[Surface], config: QSTEConfig | None = None, *,
                 gradient_reducer: Callable[[Tensor], Tensor] | None | bool = None,
                 async_update: bool | None = None):
        if isinstance(model, nn.Module):
            self.surfaces = _model_surfaces(model)
            config = config or getattr(model, "_qste_config", None)
        else:
            self.surfaces = list(model)
        if not self.surfaces:
            raise ValueError("no QSTE surfaces found; call qste.convert(model, ...) first")
        self.cfg = coerce_config(config)
        self.gradient_reducer = self._resolve_reducer(gradient_reducer)
        self.step_number = 0
        self._flips = 0
        self._device_flips: dict[torch.device, Tensor] = {}
        self._side_streams: set = set()
        self._async_update = _ASYNC_UPDATE if async_update is None else bool(async_update)
        self._deferred = False
        self.state: dict[int, dict[str, Tensor]] = {}
        self._index: dict[int, int] = {}

        block = self.cfg.momentum_block_size
        for position, surface in enumerate(self.surfaces):
            device = surface.coordinate.device
            count = surface.coordinate.numel()
            self._index[id(surface)] = position
            self.state[id(surface)] = {
                "moment_q": torch.zeros_like(surface.coordinate, dtype=torch.int8),
                "moment_scale": torch.full(((count + block - 1) // block,), 1 / 127,
                                           dtype=torch.float16, device=device),
                "row_v": torch.zeros(surface.rows, dtype=torch.float16, device=device),
                "col_v": torch.zeros(surface.columns, dtype=torch.float16, device=device),
            }
            surface._immediate = self._apply
            if device.type == "cuda" and device not in self._device_flips:
                # made here, on the stream the model was built on, so that its zero fill is
                # long done before any side stream first adds to it
                self._device_flips[device] = torch.zeros((), dtype=torch.int64, device=device)
        for surface in self.surfaces:
            kernels.warm(surface.coordinate.device)
            kernels.warn_if_slow(surface.coordinate.device.type)

    @staticmethod
    def _resolve_reducer(requested):
        if requested is False:
            return None
        if requested is not None and requested is not True:
            return requested
        from .distributed import _distributed_ready, mean_evidence

        return mean_evidence() if _distributed_ready() else None

    # -- accumulation control --------------------------------------------------------

    def defer(self, deferred: bool = True) -> None:
        """Hold evidence until :meth:`step` (gradient accumulation, AMP unscaling, graph
        capture) instead of applying it inside backward."""

        self._deferred = deferred
        for surface in self.surfaces:
            surface._immediate = None if deferred else self._apply

    def prepare_accumulation(self) -> None:
        """Preallocate one fixed evidence buffer per surface, then defer into them."""

        self.defer(True)
        for surface in self.surfaces:
            surface.prepare_accumulator()

    def unscale_(self, scale: float | Tensor) -> None:
        """Divide held evidence by an AMP loss scale."""

        divisor = float(scale)
        for surface in self.surfaces:
            surface.scale_evidence_(divisor)

    def zero_grad(self, set_to_none: bool = True) -> None:
        """Drop evidence that was retained but not applied."""

        del set_to_none
        for surface in self.surfaces:
            surface.flush_evidence()
            surface.reset_tracking()
        self._flips = 0
        for counter in self._device_flips.values():
            counter.zero_()

    # -- the step ------------------------------------------------------------------

    @torch.no_grad()
    def _apply(self, surface: Surface, evidence: Tensor) -> None:
        state = self.state[id(surface)]
        evidence = evidence.float()
        side = None
        if self.gradient_reducer is not None:
            side_stream_of = getattr(self.gradient_reducer, "side_stream", None)
            if side_stream_of is not None and evidence.is_cuda and _reducer_is_live():
                # An overlapped reducer: the collective runs on a side stream, and so does the
                # update below -- nothing on the compute stream waits for either until step().
                evidence = self.gradient_reducer(evidence, join=False)
                side = side_stream_of(evidence.device)
                self._side_streams.add(side)
            else:
                evidence = self.gradient_reducer(evidence)
        elif evidence.is_cuda and self._async_update:
            # No reduction to wait for: the update still goes to the side stream, where its small
            # memory-bound kernels fill in beside the next layer's backward (3 % of the step on
            # one GPU).  Same kernels, same inputs: the result does not depend on the stream.
            from .distributed import _side_stream, wait_for_producer

            side = _side_stream(evidence.device)
            wait_for_producer(side, torch.cuda.current_stream(evidence.device), evidence)
            evidence.record_stream(side)
            self._side_streams.add(side)
        arguments = dict(
            beta1=self.cfg.beta1, beta2=self.cfg.beta2, update_clip=self.cfg.update_rms_clip,
            coordinate_lr=self.cfg.coordinate_lr, block_size=self.cfg.momentum_block_size,
            seed=self.cfg.seed + _SURFACE_SEED_STRIDE * self._index[id(surface)],
            step=self.step_number,
        )
        tensors = (evidence, surface.coordinate.data, surface.packed_sign.data, state["moment_q"],
                   state["moment_scale"], state["row_v"], state["col_v"])
        if evidence.is_cuda:
            # keep the count on the device: one host read per step(), not per surface
            device = evidence.device
            total = self._device_flips.get(device)
            if total is None:
                # a surface moved to another device after construction: make the counter where the
                # zero fill is ordered before the add below, whichever stream that runs on
                with torch.cuda.stream(side) if side is not None else contextlib.nullcontext():
                    total = self._device_flips[device] = torch.zeros((), dtype=torch.int64, device=device)
            with torch.cuda.stream(side) if side is not None else contextlib.nullcontext():
                scratch = torch.empty((), dtype=torch.int64, device=device)
                kernels.coordinate_update(*tensors, flips=scratch, **arguments)
                total.add_(scratch)
        else:
            self._flips += int(kernels.coordinate_update(*tensors, **arguments))

    @torch.no_grad()
    def step(self) -> int:
        """Apply retained evidence, clamp the row scales, advance the step.

        Returns the number of sign flips of this step.
        """

        low, high = math.log(self.cfg.scale_min), math.log(self.cfg.scale_max)
        for surface in self.surfaces:
            evidence = surface.flush_evidence(keep_buffer=self._deferred)
            if evidence is not None:
                self._apply(surface, evidence)
            surface.log_scale.data.clamp_(low, high)
        # updates that ran on a side stream: the signs they wrote are read by the next forward
        for side in self._side_streams:
            torch.cuda.current_stream(side.device).wait_stream(side)
        self._side_streams.clear()
        flips = self._flips
        for device, counter in self._device_flips.items():
            flips += int(counter.item())
            counter.zero_()
            # the read above synchronised with everything this step launched on the device: if a
            # GEMM's bounded wait gave up anywhere in it, say so instead of training on
            kernels.check_waits(device)
        self._flips = 0
        self.step_number += 1
        return flips

    # -- reporting and checkpointing -----------------------------------------------------

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for s in self.state.values() for t in s.values())

    def state_dict(self) -> dict[str, object]:
        return {
            "config": self.cfg.metadata(),
            "step_number": self.step_number,
            "surfaces": [{key: tensor.detach().cpu() for key, tensor in self.state[id(s)].items()}
                         for s in self.surfaces],
        }

    def load_state_dict(self, state_dict: Mapping[str, object]) -> None:
        entries = state_dict["surfaces"]
        if len(entries) != len(self.surfaces):
            raise ValueError(
                f"checkpoint holds {len(entries)} surfaces, model has {len(self.surfaces)}")
        for surface, entry in zip(self.surfaces, entries):
            state = self.state[id(surface)]
            for key, tensor in entry.items():
                state[key].copy_(tensor.to(state[key].device))
        self.step_number = int(state_dict.get("step_number", 0))
