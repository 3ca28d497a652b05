"""Modules that stand where ``nn.Linear`` / ``nn.Embedding`` stood.

Two families over the same packed sign bits:

* trainable -- ``QSTELinear`` and ``QSTEEmbedding`` own a ``Surface`` (int8 coordinates, sign
  bits, row scales) and route forward and backward through ``functional``;
* frozen -- ``PackedLinear`` and ``PackedEmbedding`` are what ``export_packed`` leaves behind:
  bits, scales and an optional bias as buffers, forward only.

The attribute names a host framework introspects (``in_features``, ``out_features``,
``num_embeddings``, ``embedding_dim``, ``padding_idx``, ``weight``, ``bias``, ``scale``,
``packed_sign``) and the constructors' signatures follow ``src/qste/modules.py:21-140`` of the
reference; the trainable forward tags its output the way ``src/qste/nn.py:100-104`` expects, so
the activation that follows can tell it came from a converted layer.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional
from .config import QSTEConfig, coerce_config
from .nn import _mark_activation_input
from .surface import Surface


def _surface_of(module: nn.Module, cfg: QSTEConfig | None, surface: Surface | None) -> Surface:
    """The surface a converted copy of `module` should use: the one handed in (tied weights
    share one) or a fresh one built from the float weight."""

    return surface if surface is not None else Surface(module.weight, coerce_config(cfg))


class _Trainable(nn.Module):
    """What both trainable modules share: the surface and the views onto it."""

    surface: Surface

    def __init__(self, surface: Surface):
        super().__init__()
        self.surface = surface

    @property
    def weight(self) -> Tensor:
        """A differentiable dense ``sign * scale`` matrix, for code that reads ``.weight`` (to
        fuse, slice or tie).  Built on every access -- rows x columns floats -- and never used by
        the module's own forward; gradients that reach it become coordinate evidence."""

        return functional.qste_weight(self.surface)

    @property
    def scale(self) -> Tensor:
        return self.surface.scale

    @property
    def packed_sign(self) -> Tensor:
        return self.surface.packed_sign


class QSTELinear(_Trainable):
    """``y = (x @ sign(W)^T) * scale + bias`` with W held as a binary surface."""

    def __init__(self, surface: Surface, bias: Tensor | None = None):
        super().__init__(surface)
        self.out_features, self.in_features = surface.rows, surface.columns
        # the bias stays an ordinary fp32 parameter of the host's optimizer
        self.register_parameter("bias", None if bias is None else nn.Parameter(bias.detach().to(torch.float32).clone()))

    @classmethod
    def from_linear(cls, module: nn.Linear, cfg: QSTEConfig | None = None,
                    surface: Surface | None = None) -> "QSTELinear":
        return cls(_surface_of(module, cfg, surface), module.bias)

    def forward(self, inputs: Tensor) -> Tensor:
        return _mark_activation_input(functional.qste_linear(inputs, self.surface, self.bias))

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class QSTEEmbedding(_Trainable):
    """An embedding table of sign bits: row ``i`` is ``sign[i] * scale[i]``."""

    def __init__(self, surface: Surface, padding_idx: int | None = None):
        super().__init__(surface)
        self.num_embeddings, self.embedding_dim = surface.rows, surface.columns
        self.padding_idx = padding_idx

    @classmethod
    def from_embedding(cls, module: nn.Embedding, cfg: QSTEConfig | None = None,
                       surface: Surface | None = None) -> "QSTEEmbedding":
        return cls(_surface_of(module, cfg, surface), getattr(module, "padding_idx", None))

    def forward(self, ids: Tensor) -> Tensor:
        return _mark_activation_input(functional.qste_embedding(ids, self.surface))

    def extra_repr(self) -> str:
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}"


class _Frozen(nn.Module):
    """Bits and row scales as buffers: they move with ``.to()`` and land in ``state_dict``, and
    nothing about them is trainable."""

    def __init__(self, packed: Tensor, scale: Tensor, columns: int):
        super().__init__()
        self.register_buffer("packed_sign", packed)
        self.register_buffer("scale", scale)
        self.rows, self.columns = int(packed.shape[0]), int(columns)


class PackedLinear(_Frozen):
    """Inference-only Linear over exported bits (one bit per weight plus a float per row)."""

    def __init__(self, packed: Tensor, scale: Tensor, columns: int, bias: Tensor | None):
        super().__init__(packed, scale, columns)
        self.register_buffer("bias", bias)
        self.in_features, self.out_features = self.columns, self.rows

    @torch.no_grad()
    def forward(self, inputs: Tensor) -> Tensor:
        from . import kernels

        out = kernels.packed_linear_affine(inputs, self.packed_sign, self.scale, self.bias, self.columns)
        return out.to(inputs.dtype)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}"


class PackedEmbedding(_Frozen):
    """Inference-only embedding over exported bits."""

    def __init__(self, packed: Tensor, scale: Tensor, columns: int):
        super().__init__(packed, scale, columns)
        self.num_embeddings, self.embedding_dim = self.rows, self.columns

    @torch.no_grad()
    def forward(self, ids: Tensor) -> Tensor:
        from . import kernels

        return kernels.packed_embedding(ids, self.packed_sign, self.scale, self.columns)

    def extra_repr(self) -> str:
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}"
