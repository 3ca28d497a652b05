"""The converted Linear end to end on the GPU: the reference's golden training
steps, BASELINE config 1 against the oracle, mixed precision, and the public
model-level API (convert / QSTEOptimizer) on CUDA tensors."""

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle
import qste_b200 as qste
from qste_b200 import kernels

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("case,use_bias", [("layer0", True), ("layer1", False)])
def test_golden_training_steps_on_the_gpu(golden, case, use_bias):
    """Same two steps as the CPU host-logic test, but every kernel is the CUDA one."""

    weight = torch.from_numpy(golden(case, "weight"))
    rows, columns = weight.shape
    linear = nn.Linear(columns, rows, bias=use_bias)
    with torch.no_grad():
        linear.weight.copy_(weight)
        if use_bias:
            linear.bias.copy_(torch.from_numpy(golden(case, "bias")))
    model = nn.Sequential(linear).to(DEVICE)
    qste.convert(model, include=["0"], activations=False)
    layer = model[0]
    assert np.array_equal(layer.surface.coordinate.cpu().numpy(), golden(case, "init_coordinate"))
    assert np.array_equal(layer.surface.packed_sign.cpu().numpy(), golden(case, "init_packed"))
    coordinates = qste.QSTEOptimizer(model)
    host = torch.optim.AdamW(qste.continuous_parameters(model), lr=1e-3)
    # the evidence each step hands the optimizer, so the oracle can be walked beside the GPU
    captured = []
    apply = coordinates._apply
    layer.surface._immediate = lambda s, e: (captured.append(e.detach().cpu().numpy().copy()), apply(s, e))
    shadow = {key: golden(case, f"init_{key}").copy() for key in ("coordinate", "packed")}
    blocks = (rows * columns + 255) // 256
    shadow.update(moment_q=np.zeros((rows, columns), np.int8), moment_scale=np.full(blocks, 1 / 127, np.float16),
                  row_v=np.zeros(rows, np.float16), col_v=np.zeros(columns, np.float16))
    for number in range(2):
        x = torch.from_numpy(golden(case, f"x{number}")).to(DEVICE).requires_grad_(True)
        y = model(x)
        assert np.allclose(y.detach().cpu().numpy(), golden(case, f"y{number}"), atol=1e-4)
        y.backward(torch.from_numpy(golden(case, f"dy{number}")).to(DEVICE))
        assert np.allclose(x.grad.cpu().numpy(), golden(case, f"dx{number}"), atol=1e-4)
        assert np.allclose(layer.surface.log_scale.grad.cpu().numpy(), golden(case, f"g_log_scale{number}"),
                           rtol=1e-4, atol=1e-4)
        if use_bias:
            assert np.allclose(layer.bias.grad.cpu().numpy(), golden(case, f"g_bias{number}"), atol=1e-4)
        host.step()
        flips = coordinates.step()
        host.zero_grad(set_to_none=True)
        coordinates.zero_grad()
        state = coordinates.state[id(layer.surface)]
        # the evidence GEMM sums in another order than MKL did, so a coordinate whose
        # rounding draw sits within an ulp of its threshold may land on the other side
        mine = layer.surface.coordinate.cpu().numpy()
        difference = np.abs(mine.astype(np.int32) - golden(case, f"coordinate{number}").astype(np.int32))
        assert difference.max() <= 1 and (difference > 0).mean() < 0.002
        assert abs(flips - int(np.ravel(golden(case, f"flips{number}"))[0])) <= 4
        assert (state["moment_q"].cpu().numpy() != golden(case, f"moment_q{number}")).mean() < 0.01

        # Given the SAME evidence the oracle lands on the GPU's state byte for byte ...
        want_flips = oracle.coordinate_update(
            captured[number].copy(), shadow["coordinate"], shadow["packed"], shadow["moment_q"], shadow["moment_scale"],
            shadow["row_v"], shadow["col_v"], beta1=0.9, beta2=0.99, update_clip=2.0, coordinate_lr=1.0,
            block_size=256, seed=1, step=number)
        assert np.array_equal(mine, shadow["coordinate"]) and flips == want_flips
        assert np.array_equal(state["moment_q"].cpu().numpy(), shadow["moment_q"])
        # ... and where the result differs from the reference's own run, the coordinate is a
        # near-tie of the stochastic rounding.  Start the oracle from the REFERENCE's state before
        # this step and give it the GPU's evidence (which depends on the step's inputs, not on the
        # coordinates): every coordinate that then differs from the reference's has its uniform
        # draw within a hair of the fractional part of its target (cpu.cpp:762-772), so the last
        # bits of the evidence sum -- the order MKL happened to add in -- decide it.
        def reference_state(name):
            if number > 0:
                array = golden(case, f"{name}{number - 1}").copy()
                return array.view(np.float16) if array.dtype == np.uint16 else array
            if name in ("coordinate", "packed"):
                return golden(case, f"init_{name}").copy()
            return {"moment_q": np.zeros((rows, columns), np.int8), "moment_scale": np.full(blocks, 1 / 127, np.float16),
                    "row_v": np.zeros(rows, np.float16), "col_v": np.zeros(columns, np.float16)}[name]

        start = {key: reference_state(key) for key in ("coordinate", "packed", "moment_q", "moment_scale", "row_v", "col_v")}
        before = start["coordinate"].astype(np.float32)
        moment = captured[number].copy()
        _, taps = oracle.coordinate_update(
            moment, start["coordinate"], start["packed"], start["moment_q"], start["moment_scale"], start["row_v"],
            start["col_v"], beta1=0.9, beta2=0.99, update_clip=2.0, coordinate_lr=1.0, block_size=256, seed=1,
            step=number, taps=True)
        apart = np.abs(start["coordinate"].astype(np.int32) - golden(case, f"coordinate{number}").astype(np.int32))
        assert apart.max() <= 1
        target = before - moment * np.float32(taps["coordinate_step"])
        fraction = target - np.floor(target)
        for row, column in zip(*np.nonzero(apart)):
            draw = oracle.uniform(1, number, int(row) * columns + int(column))
            f = float(fraction[row, column])
            assert min(abs(draw - f), f, 1.0 - f) < 1e-4, (number, int(row), int(column), draw, f)


def test_config_one_layer_matches_the_oracle():
    """BASELINE config 1: R = C = 2048, batch 256, fp32, one forward, one backward,
    one coordinate step.  Float results within 1e-3 relative Frobenius; the integer
    state equals the oracle's when the oracle is fed the same evidence."""

    rows = columns = 2048
    batch = 256
    generator = torch.Generator().manual_seed(1)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    x = torch.randn(batch, columns, generator=generator)
    dy = torch.randn(batch, rows, generator=generator)
    surface = qste.Surface(torch.zeros(rows, columns)).to(DEVICE)
    with torch.no_grad():
        surface.coordinate.copy_(coordinate)
        surface.refresh_packed()
        surface.log_scale.fill_(float(np.log(0.02)))
    layer = qste.QSTELinear(surface, torch.zeros(rows)).to(DEVICE)
    packed = oracle.pack_coordinate(coordinate)
    assert np.array_equal(surface.packed_sign.cpu().numpy(), packed)

    captured = {}
    coordinates = qste.QSTEOptimizer([surface])
    apply = coordinates._apply
    surface._immediate = lambda s, e: (captured.setdefault("evidence", e.clone()), apply(s, e))
    xg = x.to(DEVICE).requires_grad_(True)
    y = layer(xg)
    y.backward(dy.to(DEVICE))
    flips = coordinates.step()

    scale = np.full(rows, np.float32(np.exp(np.float32(np.log(0.02)))), np.float32)
    scale = surface.scale.detach().cpu().numpy()
    want_y = oracle.packed_linear_affine(x, packed, scale, np.zeros(rows, np.float32), columns)
    assert rel(y.detach().cpu().numpy(), want_y) <= 1e-5
    assert rel(xg.grad.cpu().numpy(), oracle.packed_transpose(dy, packed, columns, scale)) <= 1e-5
    bits, offset, act_scale = oracle.pack_affine_rows(x)
    decoded = oracle.decoded_evidence(dy, bits, offset, act_scale, columns)
    assert rel(captured["evidence"].cpu().numpy(), decoded * scale[:, None]) <= 1e-5
    g_scale = oracle.packed_row_inner(decoded, packed, columns) * scale  # chain through exp()
    assert rel(surface.log_scale.grad.cpu().numpy(), g_scale) <= 1e-4
    assert rel(layer.bias.grad.cpu().numpy(), dy.sum(0).numpy()) <= 1e-5

    blocks = rows * columns // 256
    state = dict(coordinate=coordinate.numpy().copy(), packed=packed.copy(),
                 moment_q=np.zeros((rows, columns), np.int8),
                 moment_scale=np.full(blocks, 1 / 127, np.float16), row_v=np.zeros(rows, np.float16),
                 col_v=np.zeros(columns, np.float16))
    want_flips = oracle.coordinate_update(
        captured["evidence"].cpu().numpy().copy(), state["coordinate"], state["packed"], state["moment_q"],
        state["moment_scale"], state["row_v"], state["col_v"], beta1=0.9, beta2=0.99, update_clip=2.0,
        coordinate_lr=1.0, block_size=256, seed=1, step=0)
    mine = coordinates.state[id(surface)]
    assert np.array_equal(surface.coordinate.cpu().numpy(), state["coordinate"])
    assert np.array_equal(surface.packed_sign.cpu().numpy(), state["packed"])
    assert np.array_equal(mine["moment_q"].cpu().numpy(), state["moment_q"])
    assert np.array_equal(mine["moment_scale"].cpu().numpy().view(np.uint16), state["moment_scale"].view(np.uint16))
    assert np.array_equal(mine["row_v"].cpu().numpy().view(np.uint16), state["row_v"].view(np.uint16))
    assert np.array_equal(mine["col_v"].cpu().numpy().view(np.uint16), state["col_v"].view(np.uint16))
    assert flips == want_flips


class Mlp(nn.Module):
    def __init__(self, dim=256, hidden=512):
        super().__init__()
        self.up = nn.Linear(dim, hidden)
        self.act = nn.GELU()
        self.down = nn.Linear(hidden, dim)

    def forward(self, x):
        return x + self.down(self.act(self.up(x)))


def test_converted_model_trains_under_autocast_and_checkpoints():
    torch.manual_seed(0)
    model = nn.Sequential(Mlp(), Mlp()).to(DEVICE)
    qste.convert(model, include=["*.up", "*.down"])
    assert isinstance(model[0].act, qste.nn.GELU)
    assert len(qste.surfaces(model)) == 4
    coordinates = qste.QSTEOptimizer(model)
    host = torch.optim.AdamW(qste.continuous_parameters(model), lr=1e-3)
    generator = torch.Generator(device=DEVICE).manual_seed(4)
    target = torch.randn(512, 256, device=DEVICE, generator=generator)
    losses, total_flips = [], 0
    for _ in range(6):
        x = torch.randn(512, 256, device=DEVICE, generator=generator)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = (model(x) - target).float().square().mean()
        loss.backward()
        host.step()
        total_flips += coordinates.step()
        host.zero_grad(set_to_none=True)
        coordinates.zero_grad()
        losses.append(float(loss))
    assert all(np.isfinite(losses)) and total_flips > 0
    for surface in qste.surfaces(model):
        assert torch.equal(surface.packed_sign.data, kernels.pack_coordinate(surface.coordinate.data))
    saved = coordinates.state_dict()
    assert saved["step_number"] == 6 and all(t.device.type == "cpu" for t in saved["surfaces"][0].values())
    exported = qste.export_packed(model)
    with torch.no_grad():
        x = torch.randn(8, 256, device=DEVICE)
        assert torch.allclose(exported(x), model(x), atol=1e-4, rtol=1e-4)
    assert kernels.wait_timeouts() == 0


def test_async_update_reaches_the_same_state():
    """QSTEOptimizer(async_update=True) runs the updates on a side stream and joins it in
    step(): coordinates, signs, moments and flip counts equal those of the in-stream optimizer."""

    def train(async_update):
        torch.manual_seed(5)
        model = nn.Sequential(nn.Linear(256, 512, bias=False), nn.ReLU(), nn.Linear(512, 256)).to(DEVICE)
        qste.convert(model, include=["0", "2"])
        coordinates = qste.QSTEOptimizer(model, async_update=async_update)
        generator = torch.Generator(device=DEVICE).manual_seed(6)
        flips = []
        for _ in range(3):
            x = torch.randn(192, 256, device=DEVICE, generator=generator)
            model(x).square().mean().backward()
            flips.append(coordinates.step())
            coordinates.zero_grad()
            for parameter in model.parameters():
                parameter.grad = None
        state = [(s.coordinate.clone(), s.packed_sign.clone(), coordinates.state[id(s)]["moment_q"].clone())
                 for s in coordinates.surfaces]
        return flips, state

    flips_a, state_a = train(False)
    flips_b, state_b = train(True)
    assert flips_a == flips_b and sum(flips_a) > 0
    for left, right in zip(state_a, state_b):
        for a, b in zip(left, right):
            assert torch.equal(a, b)
