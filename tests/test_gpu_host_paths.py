"""The paths either side of the converted Linear, on the GPU, through the CUDA kernels:
hosts that read ``.weight``, binary embeddings, gradient checkpointing, deferred and
accumulated evidence, AMP unscaling and a checkpoint round trip.

They follow the reference's own host-behaviour tests (tests/test_host_frameworks.py:51-147,
tests/test_learning.py:173-213, src/qste/optim.py:120-152, 212-232).  Where a result must
equal another run of the same device code it is compared bit for bit; where the yardstick is the
CPU oracle (the same model stepped on CPU tensors through ``tests/_oracle_backend``) integer
state may differ in rounding near-ties, as in test_gpu_layer.py: by at most 1, on well under
1 % of the coordinates.
"""

from __future__ import annotations

import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import _oracle_backend
import qste_b200 as qste

pytestmark = pytest.mark.gpu
DEVICE = "cuda"


class FusedHost(nn.Module):
    """Reads ``.weight`` off its children and multiplies by the concatenation (what a fused
    attention projection does)."""

    def __init__(self, dim):
        super().__init__()
        self.q = nn.Linear(dim, dim, bias=False)
        self.k = nn.Linear(dim, dim, bias=False)
        self.v = nn.Linear(dim, dim, bias=False)

    def forward(self, x):
        return F.linear(x, torch.cat([self.q.weight, self.k.weight, self.v.weight], dim=0))


def close_integer_state(mine, theirs, what):
    apart = (mine.cpu().int() - theirs.cpu().int()).abs()
    assert int(apart.max()) <= 1 and float((apart > 0).float().mean()) < 0.01, what


def on_the_oracle(monkeypatch, run):
    """`run("cpu")` with the kernel namespace replaced by the CPU oracle for its duration."""

    with monkeypatch.context() as patch:
        _oracle_backend.install(patch)
        return run("cpu")


def test_weight_reading_host_trains_like_the_oracle(monkeypatch):
    def run(device):
        torch.manual_seed(0)
        model = FusedHost(64)
        qste.convert(model)
        model.to(device)
        coordinates = qste.QSTEOptimizer(model, config={"coordinate_lr": 8.0})
        before = [s.packed_sign.clone() for s in qste.surfaces(model)]
        x = torch.randn(32, 64, generator=torch.Generator().manual_seed(1)).to(device)
        model(x).square().mean().backward()
        flips = coordinates.step()
        moved = sum(int(not torch.equal(s.packed_sign, b)) for s, b in zip(qste.surfaces(model), before))
        return flips, moved, [s.coordinate.detach().clone() for s in qste.surfaces(model)], \
            [s.log_scale.grad.detach().clone() for s in qste.surfaces(model)]

    flips, moved, coordinates, scale_grads = run(DEVICE)
    assert moved == 3 and flips > 0
    want_flips, _, want_coordinates, want_grads = on_the_oracle(monkeypatch, run)
    assert abs(flips - want_flips) <= max(4, want_flips // 50)
    for mine, theirs, g, wg in zip(coordinates, want_coordinates, scale_grads, want_grads):
        close_integer_state(mine, theirs, "weight-view coordinates")
        assert torch.allclose(g.cpu(), wg, rtol=1e-3, atol=1e-5)


def test_binary_embedding_forward_backward_and_step(monkeypatch):
    def run(device):
        torch.manual_seed(2)
        model = nn.Sequential(nn.Embedding(97, 48), nn.Linear(48, 16))
        qste.convert(model, types=(nn.Linear, nn.Embedding))
        model.to(device)
        coordinates = qste.QSTEOptimizer(model, config={"coordinate_lr": 8.0})
        ids = torch.randint(0, 97, (6, 11), generator=torch.Generator().manual_seed(3)).to(device)
        out = model(ids)
        out.square().mean().backward()
        flips = coordinates.step()
        return out.detach().clone(), flips, [s.coordinate.detach().clone() for s in qste.surfaces(model)]

    out, flips, coordinates = run(DEVICE)
    want_out, want_flips, want_coordinates = on_the_oracle(monkeypatch, run)
    assert flips > 0 and torch.allclose(out.cpu(), want_out, rtol=1e-4, atol=1e-5)
    assert abs(flips - want_flips) <= max(4, want_flips // 50)
    for mine, theirs in zip(coordinates, want_coordinates):
        close_integer_state(mine, theirs, "embedding model coordinates")


@pytest.mark.parametrize("reentrant", [False, True])
def test_gradient_checkpointing_gives_the_same_coordinates(reentrant):
    """Recomputation runs forward twice; the stepped signs must not depend on that."""

    def run(checkpointed):
        torch.manual_seed(4)
        block = nn.Sequential(nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 64))
        qste.convert(block)
        block.to(DEVICE)
        coordinates = qste.QSTEOptimizer(block, config={"coordinate_lr": 8.0})
        inputs = torch.randn(16, 64, generator=torch.Generator().manual_seed(5)).to(DEVICE).requires_grad_(True)
        if checkpointed:
            output = torch.utils.checkpoint.checkpoint(block, inputs, use_reentrant=reentrant)
        else:
            output = block(inputs)
        output.square().mean().backward()
        flips = coordinates.step()
        return [s.packed_sign.clone() for s in qste.surfaces(block)], flips

    plain, plain_flips = run(False)
    recomputed, recomputed_flips = run(True)
    assert plain_flips > 0 and recomputed_flips == plain_flips
    for a, b in zip(plain, recomputed):
        assert torch.equal(a, b)


def _two_layer(device, seed=7):
    torch.manual_seed(seed)
    model = nn.Sequential(nn.Linear(96, 128), nn.GELU(), nn.Linear(128, 32))
    qste.convert(model)
    return model.to(device)


def test_deferred_evidence_matches_the_oracle_and_the_immediate_mode(monkeypatch):
    """defer(): backward parks the evidence, step() applies it (src/qste/optim.py:120-129)."""

    def run(device, deferred=True):
        model = _two_layer(device)
        coordinates = qste.QSTEOptimizer(model, config={"coordinate_lr": 6.0})
        if deferred:
            coordinates.defer()
        x = torch.randn(40, 96, generator=torch.Generator().manual_seed(8)).to(device)
        model(x).square().mean().backward()
        untouched = [s.coordinate.detach().clone() for s in qste.surfaces(model)]
        flips = coordinates.step()
        return flips, untouched, [s.coordinate.detach().clone() for s in qste.surfaces(model)]

    initial = [s.coordinate.detach().clone() for s in qste.surfaces(_two_layer(DEVICE))]
    flips, untouched, stepped = run(DEVICE)
    for before, held in zip(initial, untouched):
        assert torch.equal(before, held)          # nothing moved inside backward
    assert flips > 0
    # held in fp16 between backward and step (evidence_accum_dtype), so close to, not equal to, immediate mode
    immediate_flips, _, immediate = run(DEVICE, deferred=False)
    for a, b in zip(stepped, immediate):
        close_integer_state(a, b, "deferred vs immediate")
    want_flips, _, want = on_the_oracle(monkeypatch, run)
    assert abs(flips - want_flips) <= max(4, want_flips // 50)
    for a, b in zip(stepped, want):
        close_integer_state(a, b, "deferred vs oracle")


def test_accumulation_over_micro_batches_and_amp_unscale():
    """prepare_accumulation(): fixed buffers summed over micro-batches; unscale_() divides what
    is held by the loss scale (src/qste/optim.py:131-152).  Two half batches with a loss scale
    of 1024 must land where the full batch without a scale lands, up to the fp16 buffer."""

    x = torch.randn(64, 96, generator=torch.Generator().manual_seed(9)).to(DEVICE)

    def run(micro_batches, loss_scale):
        model = _two_layer(DEVICE)
        coordinates = qste.QSTEOptimizer(model, config={"coordinate_lr": 6.0, "evidence_accum_dtype": "fp32"})
        coordinates.prepare_accumulation()
        for chunk in x.chunk(micro_batches):
            (model(chunk).square().sum() / x.shape[0] * loss_scale).backward()
        if loss_scale != 1.0:
            coordinates.unscale_(loss_scale)
        flips = coordinates.step()
        buffers = [s._evidence for s in qste.surfaces(model)]
        return flips, [s.coordinate.detach().clone() for s in qste.surfaces(model)], buffers

    flips, whole, buffers = run(1, 1.0)
    assert flips > 0 and all(b is not None for b in buffers)   # the accumulators are kept for the next step
    split_flips, split, _ = run(2, 1024.0)
    assert abs(split_flips - flips) <= max(4, flips // 50)
    for a, b in zip(whole, split):
        close_integer_state(a, b, "accumulated and unscaled vs whole batch")


def test_checkpoint_round_trip_continues_bit_for_bit():
    """state_dict()/load_state_dict() of model and QSTEOptimizer (src/qste/optim.py:212-232):
    a run restored after one step lands exactly where the uninterrupted run lands."""

    batches = [torch.randn(24, 96, generator=torch.Generator().manual_seed(20 + i)).to(DEVICE) for i in range(3)]

    def one_step(model, coordinates, host, x):
        model(x).square().mean().backward()
        host.step()
        coordinates.step()
        host.zero_grad(set_to_none=True)
        coordinates.zero_grad()

    model = _two_layer(DEVICE)
    coordinates = qste.QSTEOptimizer(model)
    host = torch.optim.AdamW(qste.continuous_parameters(model), lr=1e-3)
    one_step(model, coordinates, host, batches[0])
    saved = copy.deepcopy({"model": model.state_dict(), "coordinates": coordinates.state_dict(), "host": host.state_dict()})
    assert all(not t.is_cuda for entry in saved["coordinates"]["surfaces"] for t in entry.values())
    for x in batches[1:]:
        one_step(model, coordinates, host, x)

    restored = _two_layer(DEVICE, seed=99)                # different init: everything must come from the checkpoint
    restored.load_state_dict(saved["model"])
    again = qste.QSTEOptimizer(restored)
    again.load_state_dict(saved["coordinates"])
    host_again = torch.optim.AdamW(qste.continuous_parameters(restored), lr=1e-3)
    host_again.load_state_dict(saved["host"])
    assert again.step_number == 1
    for x in batches[1:]:
        one_step(restored, again, host_again, x)
    for a, b in zip(qste.surfaces(model), qste.surfaces(restored)):
        assert torch.equal(a.coordinate, b.coordinate) and torch.equal(a.packed_sign, b.packed_sign)
        assert torch.equal(a.log_scale, b.log_scale)
    for a, b in zip(coordinates.state.values(), again.state.values()):
        for key in a:
            assert torch.equal(a[key], b[key]), key


def test_exported_model_runs_the_trained_signs_in_every_dtype():
    """export_packed(): bits, scales and biases only; its forward equals the training module's
    (src/qste/convert.py:327-357, src/qste/modules.py:100-140), also through the small-batch kernels in
    fp16 and bf16 (the decode case)."""

    import oracle

    model = _two_layer(DEVICE)
    coordinates = qste.QSTEOptimizer(model, config={"coordinate_lr": 6.0})
    x = torch.randn(40, 96, generator=torch.Generator().manual_seed(11)).to(DEVICE)
    model(x).square().mean().backward()
    coordinates.step()
    frozen = qste.export_packed(model)
    assert not any(p.requires_grad for p in frozen.parameters())
    for dtype, bar in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2), (torch.float16, 2e-3)):
        for batch in (1, 3, 40):
            inputs = x[:batch].to(dtype)
            with torch.no_grad():
                want = model(inputs)
                got = frozen(inputs)
            assert got.dtype == dtype
            assert float((got.float() - want.float()).norm() / want.float().norm()) <= bar, (dtype, batch)
    # the first exported layer against the oracle, from its own buffers
    layer = frozen[0]
    want = oracle.packed_linear_affine(x.cpu(), layer.packed_sign.cpu(), layer.scale.cpu(), layer.bias.cpu(), 96)
    assert torch.allclose(layer(x).cpu(), torch.from_numpy(want), rtol=1e-4, atol=1e-5)
