"""Activations that retain bits (or bytes) for backward instead of floats.

torch's ReLU keeps its full-precision output for backward, and in a
Linear -> ReLU -> Linear stack that tensor is also the next layer's input, so it
stays resident whatever the binary Linear saves.  The functions here keep only
what the gradient needs:

* saturating activations (ReLU, ReLU6, LeakyReLU, Hardtanh, Dropout) keep ONE
  BIT per element -- "did the gradient pass here" -- packed by the library's
  ``pack_bits`` and applied by ``apply_bits``; forward and gradient are identical
  to torch's;
* Hardsigmoid, linear in pieces but not a clamp, keeps the same one bit plus its
  two slopes;
* smooth activations (GELU, SiLU, Tanh, Sigmoid, ELU, CELU, SELU, Softplus,
  Mish, Hardswish) keep their local derivative as int8 with one fp32 scale per
  row; the forward is torch's, the gradient multiplier carries about 0.2 %
  relative error;
* ``relu(x).square()`` keeps ``relu(x)`` as one UNSIGNED byte per element (the
  value is never negative, so all 255 levels resolve magnitude);
* ``elementwise(f, x)`` / ``packed(f)`` do the int8-derivative trick for any
  elementwise ``f`` by asking autograd for ``f'`` once in forward.

Module twins, the replacement tables used by ``convert(activations=...)`` and the
``packed_activations()`` context for functional call sites mirror
``src/qste/nn.py`` of the reference (masks :116-136, piecewise :139-187, fusable
ReLU :190-247, relu_square :292-343, int8 derivative :483-507, any elementwise
:510-586, tables :776-800, context :879-932).
"""

from __future__ import annotations

import math
from contextlib import contextmanager

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor
from torch.autograd import Function

from . import kernels

_TORCH_RELU = F.relu
_TORCH_RELU6 = F.relu6
_TORCH_GELU = F.gelu
_TORCH_SILU = F.silu
_TORCH_LEAKY_RELU = F.leaky_relu
_TORCH_HARDTANH = F.hardtanh
_TORCH_DROPOUT = F.dropout
_TORCH_TORCH_RELU = torch.relu
_TORCH_HARDSIGMOID = F.hardsigmoid
_TORCH_ELU = F.elu
_TORCH_CELU = F.celu
_TORCH_SELU = F.selu
_TORCH_SOFTPLUS = F.softplus
_TORCH_MISH = F.mish
_TORCH_HARDSWISH = F.hardswish


def _rows(value: Tensor) -> tuple[Tensor, torch.Size, int]:
    """``(matrix, original shape, columns)``: the tensor as contiguous rows over its last
    dimension, which is what the bit and int8 tapes are packed along.  A scalar counts as one
    row of one column, a vector as one row."""

    columns = value.shape[-1] if value.ndim else 1
    return value.reshape(-1, columns).contiguous(), value.shape, columns


def _mark_activation_input(value: Tensor) -> Tensor:
    """Tag the output of a converted layer (a plain attribute; it does not propagate)."""

    value._qste_activation_input = True
    return value


def _take_activation_input(value: Tensor) -> Tensor | None:
    return value if getattr(value, "_qste_activation_input", False) else None


# -- one bit per element -----------------------------------------------------------


class _MaskedFn(Function):
    """clamp(x, lower, upper); backward is ``grad`` where the retained bit is set."""

    @staticmethod
    def forward(ctx, inputs, lower, upper):
        output = inputs.clamp_min(lower) if upper is None else inputs.clamp(lower, upper)
        flat, shape, columns = _rows(output)
        # strict: an element sitting on the clamp has zero gradient
        keep = flat > lower if upper is None else (flat > lower) & (flat < upper)
        ctx.save_for_backward(kernels.pack_bits(keep))
        ctx.shape, ctx.columns = shape, columns
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (bits,) = ctx.saved_tensors
        flat = grad_output.reshape(-1, ctx.columns).contiguous()
        return kernels.apply_bits(flat, bits, ctx.columns).view(ctx.shape), None, None


class _LeakyFn(Function):
    """LeakyReLU: the bit says which slope applied."""

    @staticmethod
    def forward(ctx, inputs, negative_slope):
        output = _TORCH_LEAKY_RELU(inputs, negative_slope)
        flat, shape, columns = _rows(inputs)
        ctx.save_for_backward(kernels.pack_bits(flat > 0))
        ctx.shape, ctx.columns, ctx.slope = shape, columns, negative_slope
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (bits,) = ctx.saved_tensors
        flat = grad_output.reshape(-1, ctx.columns).contiguous()
        passed = kernels.apply_bits(flat, bits, ctx.columns)
        return (passed + (flat - passed) * ctx.slope).view(ctx.shape), None


class _DropoutFn(Function):
    """Dropout that keeps its own mask as bits."""

    @staticmethod
    def forward(ctx, inputs, probability):
        flat, shape, columns = _rows(inputs)
        keep = torch.rand_like(flat, dtype=torch.float32) >= probability
        ctx.save_for_backward(kernels.pack_bits(keep))
        ctx.shape, ctx.columns = shape, columns
        ctx.gain = 1.0 / (1.0 - probability)
        return (flat * keep.to(flat.dtype) * ctx.gain).view(shape)

    @staticmethod
    def backward(ctx, grad_output):
        (bits,) = ctx.saved_tensors
        flat = grad_output.reshape(-1, ctx.columns).contiguous()
        return (kernels.apply_bits(flat, bits, ctx.columns) * ctx.gain).view(ctx.shape), None


class _KneeFn(Function):
    """An activation that is linear on each side of its knees and is not a clamp.

    What backward needs is the same single bit as for a clamp -- inside the interval or
    not -- plus the slope on each side, which depend on the activation only
    (``_KNEES``).  An element exactly on a knee counts as outside, like torch.
    """

    @staticmethod
    def forward(ctx, inputs, kind, lower, upper):
        function, inner_slope, outer_slope = _KNEES[kind]
        flat, shape, columns = _rows(inputs)
        inside = flat > lower if upper is None else (flat > lower) & (flat < upper)
        ctx.save_for_backward(kernels.pack_bits(inside))
        ctx.shape, ctx.columns = shape, columns
        ctx.inner_slope, ctx.outer_slope = inner_slope, outer_slope
        return function(inputs)

    @staticmethod
    def backward(ctx, grad_output):
        (bits,) = ctx.saved_tensors
        flat = grad_output.reshape(-1, ctx.columns).contiguous()
        inside = kernels.apply_bits(flat, bits, ctx.columns).view(ctx.shape)
        if ctx.outer_slope == 0.0:
            return inside * ctx.inner_slope, None, None, None
        return grad_output * ctx.outer_slope + inside * (ctx.inner_slope - ctx.outer_slope), None, None, None


_KNEES = {"hardsigmoid": (lambda x: _TORCH_HARDSIGMOID(x), 1.0 / 6.0, 0.0)}


class _ReluSquareFn(Function):
    """``relu(x) ** 2`` as one node.  Its gradient is ``2 relu(x) grad``: a magnitude, so a
    bit is not enough, but an unsigned byte against the row maximum is (255 levels)."""

    @staticmethod
    def forward(ctx, inputs):
        positive = inputs.clamp_min(0)
        flat, shape, columns = _rows(positive)
        step = flat.amax(dim=1).clamp_min(1e-8).div_(255.0)
        levels = flat.div(step.unsqueeze(1)).round_().clamp_(0, 255).to(torch.uint8)
        ctx.save_for_backward(levels, step)
        ctx.shape = shape
        return positive * positive

    @staticmethod
    def backward(ctx, grad_output):
        levels, step = ctx.saved_tensors
        positive = levels.to(grad_output.dtype).mul_(step.to(grad_output.dtype).unsqueeze(1))
        return grad_output * 2.0 * positive.view(ctx.shape)


class _SquarableReLU(Tensor):
    """What ``relu`` returns: the ReLU output, which also remembers the ReLU's input.

    Squared (``.square()``, ``torch.square``, ``** 2``) it re-runs as the fused
    ``_ReluSquareFn`` from that input, so the float ReLU output is not retained for
    the square's backward.  Every other operation sees, and returns, a plain tensor.
    Pickles as a plain tensor.
    """

    @staticmethod
    def __new__(cls, activated: Tensor, pre_activation: Tensor):
        wrapped = activated.as_subclass(cls)
        wrapped._pre_activation = pre_activation
        return wrapped

    def plain(self) -> Tensor:
        with torch._C.DisableTorchFunctionSubclass():
            return self.as_subclass(Tensor)

    def __reduce_ex__(self, protocol):
        return self.plain().__reduce_ex__(protocol)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        first = args[0] if args else None
        source = getattr(first, "_pre_activation", None) if isinstance(first, cls) else None
        if source is not None:
            squares = func in (Tensor.square, torch.square) and len(args) == 1
            squares = squares or (func is Tensor.__pow__ and len(args) == 2 and args[1] == 2)
            if squares:
                return _ReluSquareFn.apply(source)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))


def relu(inputs: Tensor) -> Tensor:
    return _SquarableReLU(_MaskedFn.apply(inputs, 0.0, None), inputs)


def relu_square(inputs: Tensor) -> Tensor:
    """``relu(inputs) ** 2`` retaining one byte per element (what ``relu(x).square()``
    becomes under this module, callable directly)."""

    return _ReluSquareFn.apply(inputs)


def hardsigmoid(inputs: Tensor, inplace: bool = False) -> Tensor:
    if inplace:  # cannot retain what it overwrites
        return _TORCH_HARDSIGMOID(inputs, True)
    return _KneeFn.apply(inputs, "hardsigmoid", -3.0, 3.0)


def relu6(inputs: Tensor) -> Tensor:
    return _MaskedFn.apply(inputs, 0.0, 6.0)


def hardtanh(inputs: Tensor, min_val: float = -1.0, max_val: float = 1.0, inplace: bool = False) -> Tensor:
    del inplace
    return _MaskedFn.apply(inputs, float(min_val), float(max_val))


def leaky_relu(inputs: Tensor, negative_slope: float = 0.01, inplace: bool = False) -> Tensor:
    del inplace
    return _LeakyFn.apply(inputs, float(negative_slope))


def dropout(inputs: Tensor, p: float = 0.5, training: bool = True) -> Tensor:
    if not 0.0 <= p <= 1.0:
        raise ValueError(f"dropout probability has to be between 0 and 1, but got {p}")
    if not training or p == 0.0:
        return inputs
    if p == 1.0:
        return inputs * 0.0
    return _DropoutFn.apply(inputs, float(p))


# -- int8 derivative ------------------------------------------------------------------

_TANH_COEFFICIENT = 0.044715


def _gelu_derivative(x: Tensor, approximate: str) -> Tensor:
    if approximate == "tanh":
        k = math.sqrt(2.0 / math.pi)
        inner = k * (x + _TANH_COEFFICIENT * x.pow(3))
        t = torch.tanh(inner)
        return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * k * (1.0 + 3.0 * _TANH_COEFFICIENT * x * x)
    cdf = 0.5 * (1.0 + torch.erf(x / math.sqrt(2.0)))
    pdf = torch.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)
    return cdf + x * pdf


def _silu_derivative(x: Tensor) -> Tensor:
    s = torch.sigmoid(x)
    return s * (1.0 + x * (1.0 - s))


_SELU_ALPHA = 1.6732632423543772
_SELU_SCALE = 1.0507009873554805


def _mish_derivative(x: Tensor) -> Tensor:
    t = torch.tanh(F.softplus(x))
    return t + x * (1.0 - t * t) * torch.sigmoid(x)


def _hardswish_derivative(x: Tensor) -> Tensor:
    # x * hardsigmoid(x): 0 up to -3, 1 from 3, (2x + 3) / 6 between
    middle = (2.0 * x + 3.0) / 6.0
    return torch.where(x <= -3.0, torch.zeros_like(x), torch.where(x >= 3.0, torch.ones_like(x), middle))


# kind -> (forward(x, parameter), derivative(x, y, parameter)); the derivative is taken from
# whichever of input and output gives it cheaper
_SMOOTH = {
    "gelu": (lambda x, a: _TORCH_GELU(x, approximate=a), lambda x, y, a: _gelu_derivative(x, a)),
    "silu": (lambda x, a: _TORCH_SILU(x), lambda x, y, a: _silu_derivative(x)),
    "tanh": (lambda x, a: torch.tanh(x), lambda x, y, a: 1.0 - y * y),
    "sigmoid": (lambda x, a: torch.sigmoid(x), lambda x, y, a: y * (1.0 - y)),
    # alpha (exp(x) - 1) has derivative alpha exp(x) = y + alpha
    "elu": (lambda x, a: _TORCH_ELU(x, a), lambda x, y, a: torch.where(x > 0, torch.ones_like(x), y + a)),
    "celu": (lambda x, a: _TORCH_CELU(x, a), lambda x, y, a: torch.where(x > 0, torch.ones_like(x), y / a + 1.0)),
    "selu": (lambda x, a: _TORCH_SELU(x),
             lambda x, y, a: torch.where(x > 0, torch.full_like(x, _SELU_SCALE), y + _SELU_SCALE * _SELU_ALPHA)),
    "softplus": (lambda x, a: _TORCH_SOFTPLUS(x, a), lambda x, y, a: torch.sigmoid(a * x)),
    "mish": (lambda x, a: _TORCH_MISH(x), lambda x, y, a: _mish_derivative(x)),
    "hardswish": (lambda x, a: _TORCH_HARDSWISH(x), lambda x, y, a: _hardswish_derivative(x)),
}


def _fused_kind(kind: str, approximate) -> tuple[str, float] | None:
    """(kernel kind, parameter) when the library's one-pass kernel covers this activation."""

    if kind == "gelu":
        return ("gelu_tanh", 1.0) if approximate == "tanh" else ("gelu", 1.0)
    if kind in ("elu", "celu", "softplus"):
        return kind, float(approximate)
    return (kind, 1.0) if kind in kernels.SMOOTH_KINDS else None


class _SmoothFn(Function):
    """The local derivative is retained as int8 + a row scale (nn.py:483-507 of the reference).

    On the GPU forward is ONE library kernel (``kernels.smooth_forward``: activation, derivative,
    row maximum and int8 tape in a single pass over the input) and backward another; elsewhere
    the same arithmetic is composed from torch operations."""

    @staticmethod
    def forward(ctx, inputs, kind, approximate):
        fused = _fused_kind(kind, approximate) if kernels.smooth_supported(inputs) else None
        ctx.fused = fused is not None
        if fused is not None:
            output, payload, scale = kernels.smooth_forward(inputs, *fused)
            ctx.save_for_backward(payload, scale)
            ctx.shape = inputs.shape
            return output
        forward, derivative_of = _SMOOTH[kind]
        output = forward(inputs, approximate)
        derivative = derivative_of(inputs.float(), output.float(), approximate)
        flat, shape, columns = _rows(derivative)
        scale = flat.abs().amax(dim=1).clamp_min(1e-8).div_(127.0)
        payload = flat.div_(scale.unsqueeze(1)).round_().clamp_(-127, 127).to(torch.int8)
        ctx.save_for_backward(payload, scale)
        ctx.shape = shape
        return output

    @staticmethod
    def backward(ctx, grad_output):
        payload, scale = ctx.saved_tensors
        if ctx.fused and grad_output.is_cuda:
            return kernels.smooth_backward(grad_output, payload, scale), None, None
        derivative = payload.to(grad_output.dtype).mul_(scale.to(grad_output.dtype).unsqueeze(1))
        return grad_output * derivative.view(ctx.shape), None, None


def gelu(inputs: Tensor, approximate: str = "none") -> Tensor:
    return _SmoothFn.apply(inputs, "gelu", approximate)


def silu(inputs: Tensor) -> Tensor:
    return _SmoothFn.apply(inputs, "silu", None)


def tanh(inputs: Tensor) -> Tensor:
    return _SmoothFn.apply(inputs, "tanh", None)


def sigmoid(inputs: Tensor) -> Tensor:
    return _SmoothFn.apply(inputs, "sigmoid", None)


def elu(inputs: Tensor, alpha: float = 1.0, inplace: bool = False) -> Tensor:
    return _TORCH_ELU(inputs, alpha, True) if inplace else _SmoothFn.apply(inputs, "elu", alpha)


def celu(inputs: Tensor, alpha: float = 1.0, inplace: bool = False) -> Tensor:
    return _TORCH_CELU(inputs, alpha, True) if inplace else _SmoothFn.apply(inputs, "celu", alpha)


def selu(inputs: Tensor, inplace: bool = False) -> Tensor:
    return _TORCH_SELU(inputs, True) if inplace else _SmoothFn.apply(inputs, "selu", 1.0)


def softplus(inputs: Tensor, beta: float = 1.0, threshold: float = 20.0) -> Tensor:
    del threshold  # torch's linear branch above it has the same derivative to within the tape's precision
    return _SmoothFn.apply(inputs, "softplus", beta)


def mish(inputs: Tensor, inplace: bool = False) -> Tensor:
    return _TORCH_MISH(inputs, True) if inplace else _SmoothFn.apply(inputs, "mish", 1.0)


def hardswish(inputs: Tensor, inplace: bool = False) -> Tensor:
    return _TORCH_HARDSWISH(inputs, True) if inplace else _SmoothFn.apply(inputs, "hardswish", 1.0)


class _AnyElementwiseFn(Function):
    """The int8-derivative tape for a function nobody tabulated.

    ``f'(x)`` is ``grad(f(x).sum(), x)`` whenever each output depends on its own input
    only, so forward runs ``f`` once on a detached copy under autograd, asks for that
    gradient and quantises it like ``_SmoothFn``.  A function that changes the shape
    cannot be elementwise and is refused; one that keeps the shape but mixes elements
    (a softmax) is the caller's to avoid.
    """

    @staticmethod
    def forward(ctx, inputs, function):
        with torch.enable_grad():
            probe = inputs.detach().requires_grad_(True)
            output = function(probe)
            if output.shape != probe.shape:
                raise ValueError("qste.nn.packed() needs an elementwise function; this one maps "
                                 f"{tuple(probe.shape)} to {tuple(output.shape)}")
            (derivative,) = torch.autograd.grad(output.sum(), probe)
        flat, shape, _ = _rows(derivative.float())
        scale = flat.abs().amax(dim=1).clamp_min(1e-8).div_(127.0)
        payload = flat.div_(scale.unsqueeze(1)).round_().clamp_(-127, 127).to(torch.int8)
        ctx.save_for_backward(payload, scale)
        ctx.shape = shape
        return output.detach()

    @staticmethod
    def backward(ctx, grad_output):
        payload, scale = ctx.saved_tensors
        derivative = payload.to(grad_output.dtype).mul_(scale.to(grad_output.dtype).unsqueeze(1))
        return grad_output * derivative.view(ctx.shape), None


def elementwise(function, inputs: Tensor) -> Tensor:
    """``function(inputs)`` for any elementwise ``function``, retaining one byte per element."""

    return _AnyElementwiseFn.apply(inputs, function)


def packed(function):
    """``function`` wrapped so that it retains one byte per element.  Elementwise only."""

    def wrapper(inputs: Tensor) -> Tensor:
        return elementwise(function, inputs)

    wrapper.__name__ = getattr(function, "__name__", "packed")
    wrapper.__doc__ = f"Packed: {getattr(function, '__doc__', None) or function!r}"
    return wrapper


# -- module twins -------------------------------------------------------------------


class ReLU(nn.Module):
    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = False  # cannot retain what it overwrites

    def forward(self, inputs: Tensor) -> Tensor:
        return relu(inputs)


class ReLU6(nn.Module):
    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = False

    def forward(self, inputs: Tensor) -> Tensor:
        return relu6(inputs)


class LeakyReLU(nn.Module):
    def __init__(self, negative_slope: float = 0.01):
        super().__init__()
        self.negative_slope = negative_slope

    def forward(self, inputs: Tensor) -> Tensor:
        return leaky_relu(inputs, self.negative_slope)


class Hardtanh(nn.Module):
    def __init__(self, min_val: float = -1.0, max_val: float = 1.0):
        super().__init__()
        self.min_val, self.max_val = min_val, max_val

    def forward(self, inputs: Tensor) -> Tensor:
        return hardtanh(inputs, self.min_val, self.max_val)


class Dropout(nn.Module):
    def __init__(self, p: float = 0.5, inplace: bool = False):
        super().__init__()
        if not 0.0 <= p <= 1.0:
            raise ValueError(f"dropout probability has to be between 0 and 1, but got {p}")
        self.p = p
        self.inplace = False

    def forward(self, inputs: Tensor) -> Tensor:
        return dropout(inputs, self.p, self.training)

    def extra_repr(self) -> str:
        return f"p={self.p}"


class GELU(nn.Module):
    def __init__(self, approximate: str = "none"):
        super().__init__()
        self.approximate = approximate

    def forward(self, inputs: Tensor) -> Tensor:
        return gelu(inputs, self.approximate)

    def extra_repr(self) -> str:
        return f"approximate={self.approximate!r}"


class SiLU(nn.Module):
    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = False

    def forward(self, inputs: Tensor) -> Tensor:
        return silu(inputs)


class Tanh(nn.Module):
    def forward(self, inputs: Tensor) -> Tensor:
        return tanh(inputs)


class Sigmoid(nn.Module):
    def forward(self, inputs: Tensor) -> Tensor:
        return sigmoid(inputs)


class Hardsigmoid(nn.Module):
    def forward(self, inputs: Tensor) -> Tensor:
        return hardsigmoid(inputs)


class ELU(nn.Module):
    def __init__(self, alpha: float = 1.0):
        super().__init__()
        self.alpha = alpha

    def forward(self, inputs: Tensor) -> Tensor:
        return elu(inputs, self.alpha)


class CELU(nn.Module):
    def __init__(self, alpha: float = 1.0):
        super().__init__()
        self.alpha = alpha

    def forward(self, inputs: Tensor) -> Tensor:
        return celu(inputs, self.alpha)


class SELU(nn.Module):
    def forward(self, inputs: Tensor) -> Tensor:
        return selu(inputs)


class Softplus(nn.Module):
    def __init__(self, beta: float = 1.0, threshold: float = 20.0):
        super().__init__()
        self.beta, self.threshold = beta, threshold

    def forward(self, inputs: Tensor) -> Tensor:
        return softplus(inputs, self.beta, self.threshold)


class Mish(nn.Module):
    def forward(self, inputs: Tensor) -> Tensor:
        return mish(inputs)


class Hardswish(nn.Module):
    def forward(self, inputs: Tensor) -> Tensor:
        return hardswish(inputs)


EXACT_REPLACEMENTS: dict[type, type] = {
    nn.ReLU: ReLU, nn.ReLU6: ReLU6, nn.LeakyReLU: LeakyReLU, nn.Hardtanh: Hardtanh,
    nn.Hardsigmoid: Hardsigmoid, nn.Dropout: Dropout,
}
SMOOTH_REPLACEMENTS: dict[type, type] = {
    nn.GELU: GELU, nn.SiLU: SiLU, nn.Tanh: Tanh, nn.Sigmoid: Sigmoid, nn.ELU: ELU, nn.CELU: CELU,
    nn.SELU: SELU, nn.Softplus: Softplus, nn.Mish: Mish, nn.Hardswish: Hardswish,
}
REPLACEMENTS: dict[type, type] = {**EXACT_REPLACEMENTS, **SMOOTH_REPLACEMENTS}


# hyper-parameters a twin takes over from the module it replaces, in constructor order
_CARRIED: dict[type, tuple[str, ...]] = {
    GELU: ("approximate",), Dropout: ("p",), LeakyReLU: ("negative_slope",), Hardtanh: ("min_val", "max_val"),
    ELU: ("alpha",), CELU: ("alpha",), Softplus: ("beta", "threshold"),
}


def replace(module: nn.Module) -> nn.Module | None:
    """The packed twin of ``module`` carrying its hyper-parameters, or ``None`` when the
    module has no twin."""

    twin = REPLACEMENTS.get(type(module))
    if twin is None:
        return None
    carried = {name: getattr(module, name) for name in _CARRIED.get(twin, ()) if hasattr(module, name)}
    return twin(**carried)


# -- functional call sites ----------------------------------------------------------


def _only_after_converted(original, packed_version):
    """Route to ``packed_version`` only for a tensor a converted layer just emitted."""

    def routed(inputs: Tensor, *args, **kwargs) -> Tensor:
        if _take_activation_input(inputs) is None:
            return original(inputs, *args, **kwargs)
        return packed_version(inputs, *args, **kwargs)

    return routed


def _relu_site(inputs, inplace=False):
    return _TORCH_RELU(inputs, True) if inplace else relu(inputs)


def _relu6_site(inputs, inplace=False):
    return _TORCH_RELU6(inputs, True) if inplace else relu6(inputs)


def _silu_site(inputs, inplace=False):
    return _TORCH_SILU(inputs, True) if inplace else silu(inputs)


def _dropout_site(inputs, p=0.5, training=True, inplace=False):
    return _TORCH_DROPOUT(inputs, p, training, True) if inplace else dropout(inputs, p, training)


_PATCHES = (
    (F, "relu", _only_after_converted(_TORCH_RELU, _relu_site)),
    (F, "relu6", _only_after_converted(_TORCH_RELU6, _relu6_site)),
    (F, "leaky_relu", _only_after_converted(_TORCH_LEAKY_RELU, leaky_relu)),
    (F, "hardtanh", _only_after_converted(_TORCH_HARDTANH, hardtanh)),
    (F, "hardsigmoid", _only_after_converted(_TORCH_HARDSIGMOID, hardsigmoid)),
    (torch, "relu", _only_after_converted(_TORCH_TORCH_RELU, relu)),
    (F, "gelu", _only_after_converted(_TORCH_GELU, gelu)),
    (F, "silu", _only_after_converted(_TORCH_SILU, _silu_site)),
    (F, "elu", _only_after_converted(_TORCH_ELU, elu)),
    (F, "celu", _only_after_converted(_TORCH_CELU, celu)),
    (F, "selu", _only_after_converted(_TORCH_SELU, selu)),
    (F, "softplus", _only_after_converted(_TORCH_SOFTPLUS, softplus)),
    (F, "mish", _only_after_converted(_TORCH_MISH, mish)),
    (F, "hardswish", _only_after_converted(_TORCH_HARDSWISH, hardswish)),
    (F, "dropout", _only_after_converted(_TORCH_DROPOUT, _dropout_site)),
)


@contextmanager
def packed_activations():
    """Inside the context, ``F.relu`` / ``F.gelu`` / ... called directly on the output of a
    converted layer use the packed versions; every other call is untouched.  Whatever was
    patched is put back on exit -- in reverse order, and also when the body or the patching
    itself raises."""

    undo: list[tuple[object, str, object]] = []
    try:
        for owner, name, replacement in _PATCHES:
            undo.append((owner, name, getattr(owner, name)))
            setattr(owner, name, replacement)
        yield
    finally:
        while undo:
            owner, name, original = undo.pop()
            setattr(owner, name, original)


__all__ = [
    "CELU", "Dropout", "ELU", "EXACT_REPLACEMENTS", "GELU", "Hardsigmoid", "Hardswish", "Hardtanh", "LeakyReLU",
    "Mish", "REPLACEMENTS", "ReLU", "ReLU6", "SELU", "SMOOTH_REPLACEMENTS", "SiLU", "Sigmoid", "Softplus",
    "Tanh", "celu", "dropout", "elementwise", "elu", "gelu", "hardsigmoid", "hardswish", "hardtanh",
    "leaky_relu", "mish", "packed", "packed_activations", "relu", "relu6", "relu_square", "replace", "selu",
    "sigmoid", "silu", "softplus", "tanh",
]
