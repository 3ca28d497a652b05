"""Host-side behaviour that needs no GPU: configuration, planning and reports,
conversion, the surface's evidence state machine, optimizer bookkeeping and
checkpoints.  Where a test has to run kernels it uses the ``cpu_kernels`` fixture
(the CPU oracle standing in for the kernel namespace).  The cases follow the
reference's tests/test_convert.py, tests/test_autograd.py:208-257,
tests/test_memory.py and tests/test_learning.py:259-292.
"""

import copy

import numpy as np
import pytest
import torch
import torch.nn as nn

import qste_b200 as qste
from qste_b200 import kernels


class Block(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.fc1 = nn.Linear(dim, dim * 2)
        self.fc2 = nn.Linear(dim * 2, dim)
        self.gate = nn.Linear(dim, dim, bias=False)
        self.act = nn.ReLU()

    def forward(self, x):
        return x + self.fc2(self.act(self.fc1(x))) * torch.sigmoid(self.gate(x))


class Tiny(nn.Module):
    def __init__(self, vocab=48, dim=16, depth=2, tie=True):
        super().__init__()
        self.embed = nn.Embedding(vocab, dim)
        self.blocks = nn.ModuleList([Block(dim) for _ in range(depth)])
        self.head = nn.Linear(dim, vocab, bias=False)
        if tie:
            self.head.weight = self.embed.weight
        self.register_buffer("marker", torch.arange(4))

    def forward(self, ids):
        h = self.embed(ids)
        for block in self.blocks:
            h = block(h)
        return self.head(h)


# -- config ------------------------------------------------------------------------

def test_config_defaults_and_validation():
    cfg = qste.QSTEConfig()
    assert cfg.metadata() == {
        "coordinate_clip": 1.5, "coordinate_lr": 1.0, "beta1": 0.9, "beta2": 0.99,
        "update_rms_clip": 2.0, "momentum_block_size": 256, "seed": 1, "scale_min": 1e-6,
        "scale_max": 4.0, "evidence_accum_dtype": "fp16",
    }
    for bad in ({"coordinate_lr": 0}, {"beta1": 1.0}, {"beta2": -0.1}, {"update_rms_clip": 0},
                {"momentum_block_size": 0}, {"scale_min": 5.0}, {"evidence_accum_dtype": "bf16"}):
        with pytest.raises(ValueError):
            qste.QSTEConfig(**bad)
    with pytest.raises(TypeError):
        qste.coerce_config({"no_such_field": 1})
    assert qste.coerce_config(None) == cfg
    assert qste.coerce_config({"seed": 9}).seed == 9
    assert qste.coerce_config(cfg) is cfg
    with pytest.raises(Exception):
        cfg.seed = 3  # frozen


# -- planning and reports (golden strings from the reference) -----------------------------

def test_plan_table_and_memory_report_match_the_reference(golden, cpu_kernels):
    torch.manual_seed(5)
    model = Tiny()
    candidates = qste.plan(model, include=["blocks.*.fc1", "blocks.*.fc2", "embed", "head"])
    assert qste.format_plan(candidates) == bytes(golden("plan", "table")).decode()
    assert {c.name for c in candidates if c.selected} == {
        "embed", "head", "blocks.0.fc1", "blocks.0.fc2", "blocks.1.fc1", "blocks.1.fc2"}
    head = next(c for c in candidates if c.name == "head")
    assert head.tied_to == "embed" and head.kind == "Linear"
    fc1 = next(c for c in candidates if c.name == "blocks.0.fc1")
    assert (fc1.parameters, fc1.float_bytes, fc1.qste_bytes, fc1.packed_bytes) == (512, 2048, 704, 192)
    qste.convert(model, include=["blocks.*.fc1", "blocks.*.fc2"])
    report = qste.memory_report(model)
    assert ",".join(report) == bytes(golden("plan", "report_keys")).decode()
    assert np.allclose(list(report.values()), golden("plan", "report_values"))
    assert qste.format_plan([]) == "no convertible layers found"


def test_plan_does_not_touch_the_model(cpu_kernels):
    model = Tiny()
    before = copy.deepcopy(model.state_dict())
    qste.plan(model, include=["blocks.*.fc1"])
    assert all(torch.equal(before[k], v) for k, v in model.state_dict().items())


# -- conversion ---------------------------------------------------------------------------

def test_convert_is_surgical_in_place_and_idempotent(cpu_kernels):
    model = Tiny(tie=False)
    assert qste.convert(model, include=["blocks.*.fc1", "blocks.*.fc2"]) is model
    assert isinstance(model.blocks[0].fc1, qste.QSTELinear)
    assert isinstance(model.blocks[1].fc2, qste.QSTELinear)
    assert isinstance(model.blocks[0].gate, nn.Linear) and isinstance(model.head, nn.Linear)
    assert isinstance(model.embed, nn.Embedding)
    assert isinstance(model.blocks[0].act, qste.nn.ReLU)  # activations swap by default
    assert torch.equal(model.marker, torch.arange(4))
    assert model._qste_converted[:4] == ("blocks.0.fc1", "blocks.0.fc2", "blocks.1.fc1", "blocks.1.fc2")
    surfaces = qste.surfaces(model)
    qste.convert(model, include=["blocks.*.fc1", "blocks.*.fc2"])
    assert [id(s) for s in qste.surfaces(model)] == [id(s) for s in surfaces]


def test_convert_errors_and_options(cpu_kernels):
    with pytest.raises(ValueError, match="selected no layers"):
        qste.convert(Tiny(), include=["does.not.exist"])
    with pytest.raises(ValueError, match="activations"):
        qste.convert(Tiny(), include=["head"], activations="some")
    model = Tiny(tie=False)
    qste.convert(model, include=["blocks.*"], exclude=["*.gate"], activations=False)
    assert isinstance(model.blocks[0].fc1, qste.QSTELinear)
    assert isinstance(model.blocks[0].gate, nn.Linear)
    assert isinstance(model.blocks[0].act, nn.ReLU)
    everything = qste.convert(Tiny(tie=False))
    assert not [m for m in everything.modules() if isinstance(m, nn.Linear)]
    assert isinstance(everything.embed, qste.QSTEEmbedding)


def test_tied_weights_share_one_surface_and_names_are_stable(cpu_kernels):
    model = Tiny(tie=True)
    qste.convert(model, include=["embed", "head"])
    assert model.embed.surface is model.head.surface
    assert len(qste.surfaces(model)) == 1
    names = set(model.state_dict())
    assert {"embed.surface.coordinate", "embed.surface.packed_sign", "embed.surface.log_scale"} <= names
    trainable = {id(p) for p in qste.continuous_parameters(model)}
    surface = model.embed.surface
    assert id(surface.coordinate) not in trainable and id(surface.packed_sign) not in trainable
    assert id(surface.log_scale) in trainable


def test_surface_construction_matches_reference(golden, cpu_kernels):
    for case in ("surface0", "surface1"):
        surface = qste.Surface(torch.from_numpy(golden(case, "weight")))
        assert np.array_equal(surface.coordinate.numpy(), golden(case, "coordinate"))
        assert np.array_equal(surface.packed_sign.numpy(), golden(case, "packed"))
        assert np.allclose(surface.log_scale.detach().numpy(), golden(case, "log_scale"), atol=1e-6)
        assert np.allclose(surface.dense_weight().numpy(), golden(case, "dense"), atol=1e-6)
        assert surface.memory() == {
            "packed_sign": surface.rows * ((surface.columns + 7) // 8),
            "coordinate": surface.rows * surface.columns,
            "log_scale": 4 * surface.rows,
            "float_equivalent": 4 * surface.rows * surface.columns,
        }
    with pytest.raises(ValueError):
        qste.Surface(torch.zeros(3))


# -- the converted Linear end to end, against the reference's own numbers ---------------------

@pytest.mark.parametrize("case,use_bias", [("layer0", True), ("layer1", False)])
def test_layer_training_steps_reproduce_the_reference(golden, cpu_kernels, case, use_bias):
    """Two forward/backward/AdamW/coordinate steps of one converted Linear: outputs and
    float gradients within 1e-4, integer state identical (functional.py:153-205,
    optim.py:156-201 of the reference)."""

    weight = torch.from_numpy(golden(case, "weight"))
    rows, columns = weight.shape
    linear = nn.Linear(columns, rows, bias=use_bias)
    with torch.no_grad():
        linear.weight.copy_(weight)
        if use_bias:
            linear.bias.copy_(torch.from_numpy(golden(case, "bias")))
    model = nn.Sequential(linear)
    qste.convert(model, include=["0"], activations=False)
    layer = model[0]
    assert np.array_equal(layer.surface.coordinate.numpy(), golden(case, "init_coordinate"))
    assert np.array_equal(layer.surface.packed_sign.numpy(), golden(case, "init_packed"))
    coordinates = qste.QSTEOptimizer(model)
    host = torch.optim.AdamW(qste.continuous_parameters(model), lr=1e-3)
    for number in range(2):
        x = torch.from_numpy(golden(case, f"x{number}")).requires_grad_(True)
        y = model(x)
        assert np.allclose(y.detach().numpy(), golden(case, f"y{number}"), atol=1e-4)
        y.backward(torch.from_numpy(golden(case, f"dy{number}")))
        assert np.allclose(x.grad.numpy(), golden(case, f"dx{number}"), atol=1e-4)
        assert np.allclose(layer.surface.log_scale.grad.numpy(), golden(case, f"g_log_scale{number}"),
                           rtol=1e-4, atol=1e-4)
        if use_bias:
            assert np.allclose(layer.bias.grad.numpy(), golden(case, f"g_bias{number}"), atol=1e-4)
        host.step()
        flips = coordinates.step()
        host.zero_grad(set_to_none=True)
        coordinates.zero_grad()
        state = coordinates.state[id(layer.surface)]
        assert flips == int(np.ravel(golden(case, f"flips{number}"))[0])
        assert np.array_equal(layer.surface.coordinate.numpy(), golden(case, f"coordinate{number}"))
        assert np.array_equal(layer.surface.packed_sign.numpy(), golden(case, f"packed{number}"))
        assert np.array_equal(state["moment_q"].numpy(), golden(case, f"moment_q{number}"))
        assert np.array_equal(state["moment_scale"].numpy().view(np.uint16), golden(case, f"moment_scale{number}"))
        assert np.allclose(layer.surface.log_scale.detach().numpy(), golden(case, f"log_scale{number}"), atol=1e-6)


# -- evidence state machine ---------------------------------------------------------------

def _one_layer(rows=12, columns=20, seed=0):
    torch.manual_seed(seed)
    model = nn.Sequential(nn.Linear(columns, rows))
    qste.convert(model, include=["0"])
    return model, model[0]


def test_single_use_surface_applies_in_backward_without_a_buffer(cpu_kernels):
    model, layer = _one_layer()
    coordinates = qste.QSTEOptimizer(model)
    before = layer.surface.coordinate.clone()
    model(torch.randn(6, 20)).square().mean().backward()
    assert layer.surface._evidence is None and layer.surface._call_evidence is None
    assert layer.surface._pending_calls == 0
    assert not torch.equal(before, layer.surface.coordinate)  # already applied
    assert coordinates.step() > 0
    assert coordinates.step_number == 1


def test_tied_surface_sums_its_uses_and_applies_once(cpu_kernels):
    torch.manual_seed(1)
    first, second = nn.Linear(16, 16, bias=False), nn.Linear(16, 16, bias=False)
    second.weight = first.weight
    model = nn.Sequential(first, second)
    qste.convert(model, include=["0", "1"], activations=False)
    assert model[0].surface is model[1].surface
    applied = []
    coordinates = qste.QSTEOptimizer(model)
    original = coordinates._apply
    model[0].surface._immediate = lambda s, e: (applied.append(e.clone()), original(s, e))
    model(torch.randn(5, 16)).square().mean().backward()
    assert len(applied) == 1  # one application for two uses
    assert model[0].surface._pending_calls == 0


def test_deferred_mode_accumulates_and_step_applies(cpu_kernels):
    model, layer = _one_layer()
    coordinates = qste.QSTEOptimizer(model)
    coordinates.prepare_accumulation()
    assert layer.surface._evidence is not None and layer.surface._evidence.dtype == torch.float16
    before = layer.surface.coordinate.clone()
    for _ in range(2):
        model(torch.randn(6, 20)).square().mean().backward()
    assert torch.equal(before, layer.surface.coordinate)  # nothing applied yet
    assert float(layer.surface._evidence.abs().sum()) > 0
    coordinates.unscale_(2.0)
    with pytest.raises(ValueError):
        coordinates.unscale_(0.0)
    coordinates.step()
    assert not torch.equal(before, layer.surface.coordinate)
    assert float(layer.surface._evidence.abs().sum()) == 0  # buffer kept, zeroed
    coordinates.defer(False)
    assert layer.surface._immediate is not None


def test_flush_is_the_backstop_for_unbalanced_forwards(cpu_kernels):
    model, layer = _one_layer()
    coordinates = qste.QSTEOptimizer(model)
    model(torch.randn(4, 20))                      # a forward whose backward never comes
    model(torch.randn(4, 20)).sum().backward()     # pending count is now off by one
    assert layer.surface._call_evidence is not None
    before = layer.surface.coordinate.clone()
    coordinates.step()
    assert layer.surface._pending_calls == 0 and layer.surface._call_evidence is None
    assert not torch.equal(before, layer.surface.coordinate)
    coordinates.zero_grad()


def test_optimizer_api_state_and_checkpoint_round_trip(cpu_kernels):
    with pytest.raises(ValueError, match="no QSTE surfaces"):
        qste.QSTEOptimizer(nn.Linear(4, 4))
    model, layer = _one_layer(rows=16, columns=24)
    coordinates = qste.QSTEOptimizer(model, config={"coordinate_lr": 4.0})
    assert coordinates.cfg.coordinate_lr == 4.0 and coordinates.gradient_reducer is None
    state = coordinates.state[id(layer.surface)]
    assert state["moment_q"].dtype == torch.int8 and state["moment_q"].shape == (16, 24)
    assert state["moment_scale"].dtype == torch.float16 and state["moment_scale"].numel() == 2
    assert float(state["moment_scale"][0]) == pytest.approx(1 / 127, rel=1e-3)
    assert coordinates.state_bytes() == 16 * 24 + 2 * 2 + 2 * 16 + 2 * 24
    assert coordinates.state_bytes() < 1.1 * 16 * 24 + 200
    generator = torch.Generator().manual_seed(3)
    for _ in range(2):
        model(torch.randn(8, 24, generator=generator)).square().mean().backward()
        coordinates.step()
    saved_model, saved_opt = copy.deepcopy(model.state_dict()), copy.deepcopy(coordinates.state_dict())
    assert set(saved_opt) == {"config", "step_number", "surfaces"} and saved_opt["step_number"] == 2
    assert set(saved_opt["surfaces"][0]) == {"moment_q", "moment_scale", "row_v", "col_v"}
    batch = torch.randn(8, 24, generator=generator)
    model(batch).square().mean().backward()
    coordinates.step()
    expected = layer.surface.coordinate.clone()

    restored, restored_layer = _one_layer(rows=16, columns=24, seed=99)
    restored.load_state_dict(saved_model)
    again = qste.QSTEOptimizer(restored, config={"coordinate_lr": 4.0})
    again.load_state_dict(saved_opt)
    restored(batch).square().mean().backward()
    again.step()
    assert torch.equal(restored_layer.surface.coordinate, expected)
    assert torch.equal(restored_layer.surface.packed_sign, layer.surface.packed_sign)
    with pytest.raises(ValueError, match="surfaces"):
        again.load_state_dict({"surfaces": [], "step_number": 0})


def test_weight_view_trains_the_coordinate_like_the_module_path(cpu_kernels):
    """Hosts that read ``layer.weight`` and call F.linear themselves produce the same
    evidence (functional.py:213-252; tests/test_autograd.py:166-205 of the reference)."""

    torch.manual_seed(2)
    with qste.exact_evidence():
        records = []
        for use_weight in (False, True):
            model, layer = _one_layer(rows=10, columns=14, seed=7)
            layer.surface._immediate = lambda s, e, r=records: r.append(e.clone())
            x = torch.randn(6, 14, generator=torch.Generator().manual_seed(5))
            out = torch.nn.functional.linear(x, layer.weight, layer.bias) if use_weight else model(x)
            out.square().mean().backward()
    assert torch.allclose(records[0], records[1], atol=1e-5)


def test_retained_bytes_per_sample_are_one_bit_plus_two_floats(cpu_kernels):
    """tests/test_memory.py:95-101 of the reference: C/8 + 8 bytes per sample."""

    model, layer = _one_layer(rows=32, columns=1024)
    sizes = []

    def pack(tensor):
        sizes.append((tuple(tensor.shape), tensor.numel() * tensor.element_size()))
        return tensor

    x = torch.randn(16, 1024)
    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        model(x)
    per_sample = sum(size for shape, size in sizes if shape and shape[-1] == 16 or shape == (16, 128)) / 16
    assert per_sample == 1024 / 8 + 8


def test_forward_without_grad_keeps_no_activation_bits(cpu_kernels, monkeypatch):
    """Evaluation through a trainable module: with autograd off nothing is packed or saved, and
    the output is the training forward's."""

    model, layer = _one_layer(rows=32, columns=256)
    packs = []
    original = kernels.pack_affine_rows
    monkeypatch.setattr(kernels, "pack_affine_rows", lambda values: (packs.append(values.shape), original(values))[1])
    x = torch.randn(5, 256, generator=torch.Generator().manual_seed(1))
    trained = model(x)
    assert len(packs) == 1
    with torch.no_grad():
        evaluated = model(x)
    assert len(packs) == 1 and torch.equal(evaluated, trained.detach())


def test_product_kernels_refuse_cpu_tensors():
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        kernels.pack_coordinate(torch.zeros(4, 8, dtype=torch.int8))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        kernels.packed_linear_affine(torch.zeros(2, 8), torch.zeros(4, 1, dtype=torch.uint8),
                                     torch.ones(4), None, 8)


def _update_arguments(rows=6, columns=16, block=64):
    blocks = (rows * columns + block - 1) // block
    return dict(gradient=torch.zeros(rows, columns), coordinate=torch.zeros(rows, columns, dtype=torch.int8),
                packed=torch.zeros(rows, (columns + 7) // 8, dtype=torch.uint8),
                moment_q=torch.zeros(rows, columns, dtype=torch.int8),
                moment_scale=torch.zeros(blocks, dtype=torch.float16), row_v=torch.zeros(rows, dtype=torch.float16),
                col_v=torch.zeros(columns, dtype=torch.float16))


@pytest.mark.parametrize("entry", ["coordinate_update", "coordinate_update_static"])
@pytest.mark.parametrize("change,error,match", [
    (dict(gradient=torch.zeros(6, 16, dtype=torch.float64)), RuntimeError, "float32"),
    (dict(coordinate=torch.zeros(6, 16, dtype=torch.int16)), RuntimeError, "dtypes"),
    (dict(moment_q=torch.zeros(6, 8, dtype=torch.int8)), RuntimeError, "coordinate state shape"),
    (dict(packed=torch.zeros(6, 1, dtype=torch.uint8)), RuntimeError, "packed sign shape"),
    (dict(moment_scale=torch.zeros(1, dtype=torch.float16)), RuntimeError, "momentum scale shape"),
    (dict(moment_scale=torch.zeros(2, dtype=torch.float32)), RuntimeError, "float16"),
    (dict(row_v=torch.zeros(5, dtype=torch.float16)), RuntimeError, "factored statistics"),
    (dict(col_v=torch.zeros(17, dtype=torch.float16)), RuntimeError, "factored statistics"),
    (dict(coordinate=torch.zeros(16, 6, dtype=torch.int8).t()), RuntimeError, "contiguous"),
    (dict(block_size=48), ValueError, "power of two"),
    (dict(flips=torch.zeros((), dtype=torch.int32)), RuntimeError, "flips must be an int64"),
    (dict(flips=torch.zeros(2, dtype=torch.int64)), RuntimeError, "flips must be an int64"),
])
def test_both_update_wrappers_refuse_malformed_state_before_the_library_is_called(entry, change, error, match):
    """Short, strided or wrongly typed state must never reach a kernel as a raw pointer: both
    wrappers run the same checks (those of cpu.cpp:584-606 of the reference) first."""

    arguments = _update_arguments()
    options = dict(beta1=0.9, beta2=0.99, update_clip=2.0, coordinate_lr=1.0, block_size=64, seed=1, step=0,
                   flips=torch.zeros((), dtype=torch.int64))
    for key, value in change.items():
        (options if key in options else arguments)[key] = value
    with pytest.raises(error, match=match):
        getattr(kernels, entry)(*arguments.values(), **options)


def test_the_allocation_free_update_refuses_what_it_cannot_copy():
    arguments = _update_arguments()
    options = dict(beta1=0.9, beta2=0.99, update_clip=2.0, coordinate_lr=1.0, block_size=64, seed=1, step=0)
    with pytest.raises(RuntimeError, match="needs `flips`"):
        kernels.coordinate_update_static(*arguments.values(), flips=None, **options)
    arguments["gradient"] = torch.zeros(16, 6).t()
    with pytest.raises(RuntimeError, match="must be contiguous"):
        kernels.coordinate_update_static(*arguments.values(), flips=torch.zeros((), dtype=torch.int64), **options)


# -- the overlap plumbing of the evidence exchange, on fakes ------------------------------------


class _RecordingStream:
    def __init__(self):
        self.calls = []

    def wait_event(self, event):
        self.calls.append(("event", event))

    def wait_stream(self, stream):
        self.calls.append(("stream", stream))


def test_side_stream_waits_for_the_evidence_event_when_there_is_one():
    """The fused backward tags the evidence with the event recorded after the evidence product;
    the side stream must wait for that event alone, and for the whole compute stream otherwise."""

    from qste_b200.distributed import wait_for_producer

    side, compute = _RecordingStream(), _RecordingStream()
    tagged = torch.zeros(4)
    tagged._qste_ready = "evidence-done"
    wait_for_producer(side, compute, tagged)
    assert side.calls == [("event", "evidence-done")]
    side.calls.clear()
    wait_for_producer(side, compute, torch.zeros(4))
    assert side.calls == [("stream", compute)]


def test_backward_reserve_setting(monkeypatch):
    """The reserve is a setting of the backward GEMMs only: the setter returns the previous value,
    never goes negative, and the overlapped reducer's default is 8 unless the environment says
    otherwise."""

    from qste_b200 import distributed, kernels

    first = kernels.set_backward_reserve(5)
    try:
        assert kernels.set_backward_reserve(-3) == 5
        assert kernels.set_backward_reserve(0) == 0
        monkeypatch.delenv("QSTE_B200_RESERVED_SMS", raising=False)
        distributed._reserve_for_overlap(None)
        assert kernels.set_backward_reserve(0) == 8
        monkeypatch.setenv("QSTE_B200_RESERVED_SMS", "12")
        distributed._reserve_for_overlap(None)
        assert kernels.set_backward_reserve(0) == 12
        distributed._reserve_for_overlap(4)
        assert kernels.set_backward_reserve(0) == 4
    finally:
        kernels.set_backward_reserve(first)


def test_reserved_sms_of_the_library_are_per_thread():
    """qste_b200_set_reserved_sms changes the calling thread's GEMM grids only (the side stream's
    host thread must not shrink the forward of another)."""

    import os
    import threading

    from qste_b200.kernels import _cabi

    library = _cabi.load()
    before = library.qste_b200_set_reserved_sms(6)
    seen = {}

    def other():
        seen["initial"] = library.qste_b200_set_reserved_sms(3)
        seen["own"] = library.qste_b200_set_reserved_sms(0)

    worker = threading.Thread(target=other)
    worker.start()
    worker.join()
    try:
        # the other thread started from the environment's value (0 when unset), not from this thread's 6
        assert seen["initial"] == max(0, int(os.environ.get("QSTE_B200_RESERVED_SMS", "0"))) and seen["own"] == 3
        assert library.qste_b200_set_reserved_sms(before) == 6     # untouched by the other thread
    finally:
        library.qste_b200_set_reserved_sms(before)
