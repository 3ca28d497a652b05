"""Packed activations (``qste_b200.nn``): forward equals torch's, gradients equal torch's
(exactly for the one-bit family, within the int8 tape's precision for the others), module twins
and the functional-call-site context.  Follows the reference's ``tests/test_nn.py`` strategy.

The CPU tests run the host logic over the oracle's pack_bits / apply_bits (fixture
``cpu_kernels``); the GPU test runs the same checks through the CUDA library.
"""

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import qste_b200 as qste
from qste_b200 import nn as qnn

EXACT = [
    ("relu", qnn.relu, F.relu, {}),
    ("relu6", qnn.relu6, F.relu6, {}),
    ("leaky_relu", qnn.leaky_relu, F.leaky_relu, {"negative_slope": 0.1}),
    ("hardtanh", qnn.hardtanh, F.hardtanh, {"min_val": -0.5, "max_val": 0.7}),
    ("hardsigmoid", qnn.hardsigmoid, F.hardsigmoid, {}),
]
SMOOTH = [
    ("gelu", qnn.gelu, F.gelu, {}),
    ("gelu_tanh", qnn.gelu, F.gelu, {"approximate": "tanh"}),
    ("silu", qnn.silu, F.silu, {}),
    ("tanh", qnn.tanh, torch.tanh, {}),
    ("sigmoid", qnn.sigmoid, torch.sigmoid, {}),
    ("elu", qnn.elu, F.elu, {"alpha": 1.3}),
    ("celu", qnn.celu, F.celu, {"alpha": 0.7}),
    ("selu", qnn.selu, F.selu, {}),
    ("softplus", qnn.softplus, F.softplus, {"beta": 2.0}),
    ("mish", qnn.mish, F.mish, {}),
    ("hardswish", qnn.hardswish, F.hardswish, {}),
]


def _both(ours, theirs, kwargs, device, shape=(7, 5, 40)):
    generator = torch.Generator().manual_seed(3)
    x = (torch.randn(*shape, generator=generator) * 3).to(device)
    weight = torch.randn(*shape, generator=generator).to(device)
    a = x.clone().requires_grad_(True)
    b = x.clone().requires_grad_(True)
    ya = ours(a, **kwargs)
    yb = theirs(b, **kwargs)
    (ya * weight).sum().backward()
    (yb * weight).sum().backward()
    return ya.detach(), yb.detach(), a.grad, b.grad


def _check_exact(device):
    for name, ours, theirs, kwargs in EXACT:
        ya, yb, ga, gb = _both(ours, theirs, kwargs, device)
        assert torch.equal(torch.as_tensor(ya), yb), name
        assert torch.allclose(ga, gb, rtol=0, atol=1e-6), name


def _check_smooth(device):
    for name, ours, theirs, kwargs in SMOOTH:
        ya, yb, ga, gb = _both(ours, theirs, kwargs, device)
        if device == "cpu":
            assert torch.equal(ya, yb), name      # composed from torch's own operations
        else:
            # one fused kernel with its own exp / erf / tanh: the last bit of an fp32 result may differ
            assert torch.allclose(ya, yb, rtol=1e-5, atol=1e-6), name
        error = (ga - gb).norm() / gb.norm()
        assert error < 1e-2, (name, float(error))


def _check_relu_square(device):
    for ours in (lambda t: qnn.relu(t).square(), lambda t: qnn.relu(t) ** 2, qnn.relu_square,
                 lambda t: torch.square(qnn.relu(t))):
        ya, yb, ga, gb = _both(ours, lambda t: F.relu(t).square(), {}, device)
        assert torch.allclose(torch.as_tensor(ya), yb), "relu_square forward"
        assert (ga - gb).norm() / gb.norm() < 5e-3
    # anything else done to a ReLU output behaves like a plain tensor
    x = torch.randn(6, 16, device=device, requires_grad=True)
    y = qnn.relu(x)
    assert isinstance(y, torch.Tensor)
    assert type(y * 2.0) is torch.Tensor and type(y.sum()) is torch.Tensor
    assert torch.equal((y + 1).detach(), F.relu(x).detach() + 1)
    assert type(y.plain()) is torch.Tensor


def _check_elementwise(device):
    function = lambda t: t * torch.tanh(F.softplus(t))  # noqa: E731  (mish, written out)
    ya, yb, ga, gb = _both(lambda t: qnn.elementwise(function, t), function, {}, device)
    assert torch.allclose(ya, yb)
    assert (ga - gb).norm() / gb.norm() < 1e-2
    wrapped = qnn.packed(lambda t: F.relu(t) ** 3)
    ya, yb, ga, gb = _both(wrapped, lambda t: F.relu(t) ** 3, {}, device)
    assert torch.allclose(ya, yb) and (ga - gb).norm() / gb.norm() < 1e-2
    with pytest.raises(ValueError, match="elementwise"):
        qnn.elementwise(lambda t: t.sum(dim=-1), torch.randn(3, 4, device=device))


def _check_modules_and_context(device):
    twins = [(nn.Hardsigmoid(), qnn.Hardsigmoid), (nn.ELU(0.5), qnn.ELU), (nn.CELU(2.0), qnn.CELU),
             (nn.SELU(), qnn.SELU), (nn.Softplus(3.0), qnn.Softplus), (nn.Mish(), qnn.Mish),
             (nn.Hardswish(), qnn.Hardswish), (nn.ReLU(), qnn.ReLU), (nn.GELU("tanh"), qnn.GELU)]
    x = torch.randn(5, 24, device=device)
    for original, twin in twins:
        replaced = qnn.replace(original)
        assert isinstance(replaced, twin)
        assert torch.allclose(torch.as_tensor(replaced(x)), original(x))
    assert qnn.replace(nn.Softmax(dim=-1)) is None

    # functional call sites are rerouted only for the output of a converted layer
    model = nn.Sequential(nn.Linear(24, 24)).to(device)
    qste.convert(model, include=["0"])
    with qste.packed_activations():
        for name in ("elu", "mish", "hardswish", "hardsigmoid", "selu", "softplus", "celu"):
            marked = model(x)  # the tag lives on the tensor a converted layer has just returned
            out = getattr(F, name)(marked)
            assert type(out.grad_fn).__name__ in ("_SmoothFnBackward", "_KneeFnBackward"), name
            plain = getattr(F, name)(x.clone().requires_grad_(True))
            assert type(plain.grad_fn).__name__ not in ("_SmoothFnBackward", "_KneeFnBackward"), name
    assert F.elu is qnn._TORCH_ELU and F.mish is qnn._TORCH_MISH  # restored


def test_one_bit_activations_match_torch(cpu_kernels):
    _check_exact("cpu")


def test_int8_derivative_activations_match_torch(cpu_kernels):
    _check_smooth("cpu")


def test_relu_square_fuses_and_everything_else_is_a_plain_tensor(cpu_kernels):
    _check_relu_square("cpu")


def test_any_elementwise_function_can_be_packed(cpu_kernels):
    _check_elementwise("cpu")


def test_module_twins_and_functional_call_sites(cpu_kernels):
    _check_modules_and_context("cpu")


@pytest.mark.gpu
def test_a_module_left_on_the_host_is_refused():
    model = nn.Sequential(nn.Linear(24, 24))
    qste.convert(model, include=["0"])
    with pytest.raises(RuntimeError, match="on the GPU"):
        model(torch.randn(5, 24, device="cuda"))


@pytest.mark.gpu
def test_activations_on_the_device():
    _check_exact("cuda")
    _check_smooth("cuda")
    _check_relu_square("cuda")
    _check_elementwise("cuda")
    _check_modules_and_context("cuda")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(37, 1000), (16, 14336), (5, 77), (3, 4, 96), (1, 8)])
def test_fused_smooth_kernels_against_the_torch_composition(dtype, shape):
    """kernels.smooth_forward / smooth_backward (one pass each) against the reference's own
    sequence of torch operations (src/qste/nn.py:483-507): activation to the last bit or two of
    the dtype, row scales to 1e-5, the int8 tape equal except where a derivative sits within
    rounding of a half, the gradient within the tape's own resolution."""

    from qste_b200 import kernels

    generator = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=generator) * 3).to("cuda", dtype)
    grad = torch.randn(*shape, generator=generator).to("cuda", dtype)
    ulp = {torch.float32: 2e-6, torch.bfloat16: 8e-3, torch.float16: 1e-3}[dtype]
    for kind, approximate in [("gelu", "none"), ("gelu", "tanh"), ("silu", None), ("tanh", None), ("sigmoid", None),
                              ("elu", 1.3), ("celu", 0.7), ("selu", 1.0), ("softplus", 2.0), ("mish", 1.0),
                              ("hardswish", 1.0)]:
        forward, derivative_of = qnn._SMOOTH[kind]
        want_y = forward(x, approximate)
        derivative = derivative_of(x.float(), want_y.float(), approximate).reshape(-1, shape[-1])
        want_scale = derivative.abs().amax(dim=1).clamp_min(1e-8) / 127.0
        want_q = (derivative / want_scale[:, None]).round().clamp(-127, 127).to(torch.int8)
        fused_kind, parameter = qnn._fused_kind(kind, approximate)
        y, q, scale = kernels.smooth_forward(x, fused_kind, parameter)
        assert y.dtype == dtype and y.shape == x.shape and q.shape == want_q.shape, kind
        assert torch.allclose(y.float(), want_y.float(), rtol=ulp, atol=ulp), kind
        assert torch.allclose(scale, want_scale, rtol=1e-4 if dtype == torch.float32 else 2e-2, atol=1e-9), kind
        apart = (q.int() - want_q.int()).abs()
        if dtype == torch.float32:
            assert int(apart.max()) <= 1 and float((apart > 0).float().mean()) < 0.01, kind
        else:
            # derivatives formed from an output rounded to 16 bits differ in their last bits
            assert int(apart.max()) <= 2, kind
        got = kernels.smooth_backward(grad, q, scale)
        want = grad * (q.to(dtype) * scale.to(dtype)[:, None]).view(shape)
        assert torch.allclose(got.float(), want.float(), rtol=ulp, atol=ulp), kind
        exact = grad.float() * derivative.view(shape)
        assert float((got.float() - exact).norm() / exact.norm()) < 2e-2, kind
