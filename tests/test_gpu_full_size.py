"""The path at the full sizes of the headline configuration (16384 tokens, 4096 <-> 14336).

The oracle finishes the memory-bound operators at this size in seconds, so those are
compared with it byte for byte.  The three GEMMs are 1.9 TFLOP each, far beyond the oracle:
they are checked through properties that do not depend on the size (exact scaling by a power
of two, exact negation under a flip of every sign, invariance of a row under a permutation of
the batch, additivity over a split of the batch) and against an fp32 product of a sample of
rows formed by torch on the same device.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from qste_b200 import kernels

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
TOKENS, DIM, FFN = 16384, 4096, 14336
ORDER = ("coordinate", "packed", "moment_q", "moment_scale", "row_v", "col_v")


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


def _layer(rows, columns, seed):
    generator = torch.Generator().manual_seed(seed)
    bits = torch.randint(0, 256, (rows, columns // 8), generator=generator, dtype=torch.int32).to(torch.uint8)
    scale = torch.rand(rows, generator=generator) * 0.04 + 0.01
    return bits.to(DEVICE), scale.to(DEVICE), generator


@pytest.mark.parametrize("columns", [DIM, FFN])
def test_pack_affine_rows_full_size_equals_the_oracle(columns):
    """Every bit, offset and scale of 16384 rows (cpu.cpp:143-203 of the reference)."""

    x = torch.randn(TOKENS, columns, generator=torch.Generator().manual_seed(21)).to(torch.bfloat16)
    want_bits, want_offset, want_scale = oracle.pack_affine_rows(x.float())
    bits, offset, scale = kernels.pack_affine_rows(x.to(DEVICE))
    assert np.array_equal(bits.cpu().numpy(), want_bits)
    assert np.array_equal(offset.cpu().numpy().view(np.uint32), np.asarray(want_offset, dtype=np.float32).view(np.uint32))
    assert np.array_equal(scale.cpu().numpy().view(np.uint32), np.asarray(want_scale, dtype=np.float32).view(np.uint32))


@pytest.mark.parametrize("rows,columns", [(FFN, DIM), (DIM, FFN)])
def test_coordinate_update_full_size_equals_the_oracle(rows, columns):
    """58.7 M coordinates, two steps: every byte of the six state arrays and the flip count
    (cpu.cpp:578-808 of the reference)."""

    generator = torch.Generator().manual_seed(31)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    cpu = {
        "coordinate": coordinate,
        "packed": torch.from_numpy(oracle.pack_coordinate(coordinate)),
        "moment_q": torch.zeros(rows, columns, dtype=torch.int8),
        "moment_scale": torch.full((rows * columns // 256,), 1 / 127, dtype=torch.float16),
        "row_v": torch.zeros(rows, dtype=torch.float16),
        "col_v": torch.zeros(columns, dtype=torch.float16),
    }
    gpu = {k: v.clone().to(DEVICE) for k, v in cpu.items()}
    arrays = {k: v.numpy() for k, v in cpu.items()}
    assert torch.equal(kernels.pack_coordinate(gpu["coordinate"]), gpu["packed"])
    for step in range(2):
        evidence = torch.randn(rows, columns, generator=generator) * (0.1 if step else 3.0)
        want = oracle.coordinate_update(
            evidence.clone().numpy(), *[arrays[k] for k in ORDER], beta1=0.9, beta2=0.99, update_clip=2.0,
            coordinate_lr=1.0, block_size=256, seed=5, step=step)
        got = kernels.coordinate_update(
            evidence.to(DEVICE), *[gpu[k] for k in ORDER], beta1=0.9, beta2=0.99, update_clip=2.0,
            coordinate_lr=1.0, block_size=256, seed=5, step=step)
        for key in ORDER:
            mine, theirs = gpu[key].cpu().numpy(), arrays[key]
            if mine.dtype == np.float16:
                mine, theirs = mine.view(np.uint16), theirs.view(np.uint16)
            assert np.array_equal(mine, theirs), (key, step, int((mine != theirs).sum()))
        assert got == want
        assert torch.equal(kernels.pack_coordinate(gpu["coordinate"]), gpu["packed"])


def _sample(count, limit, generator):
    return torch.randperm(limit, generator=generator)[:count].to(DEVICE)


def test_forward_full_size_properties():
    """16384 x 4096 -> 14336, bf16 (packed_linear_affine, loader.py:292-296 of the reference)."""

    bits, scale, generator = _layer(FFN, DIM, 41)
    x = torch.randn(TOKENS, DIM, generator=generator).to(DEVICE, torch.bfloat16)
    y = kernels.packed_linear_affine(x, bits, scale, None, DIM)
    assert y.shape == (TOKENS, FFN) and y.dtype == torch.bfloat16 and bool(torch.isfinite(y).all())
    # scaling by a power of two and a flip of every sign are exact in floating point
    assert torch.equal(kernels.packed_linear_affine(x, bits, scale * 2.0, None, DIM), y * 2.0)
    assert torch.equal(kernels.packed_linear_affine(x, bits ^ 0xFF, scale, None, DIM), -y)
    # An output row depends on its own input row only, wherever it sits in the batch.  Not bit
    # for bit: the tiles of the last round are cut along the contraction, so a row that moves
    # into or out of them has its fp32 sum formed in another order before the bf16 rounding.
    order = torch.randperm(TOKENS, generator=generator).to(DEVICE)
    moved = kernels.packed_linear_affine(x[order], bits, scale, None, DIM)
    assert rel(moved, y[order]) <= 1e-4
    assert float((moved != y[order]).float().mean()) <= 1e-3
    # a sample of rows against torch's fp32 product with the unpacked signs
    picked = _sample(128, TOKENS, generator)
    signs = kernels.unpack_rows(bits, DIM, dtype=torch.float32)
    want = (x[picked].float() @ signs.t()) * scale
    assert rel(y[picked], want) <= 4e-3            # bf16 rounding of the output: 1.7e-3
    assert rel(y[picked], want.to(torch.bfloat16)) <= 1e-3
    assert kernels.wait_timeouts() == 0


def test_transpose_full_size_properties():
    """dX = (dY * scale) @ sign(W), 16384 x 14336 -> 4096 (packed_transpose, loader.py:299-303)."""

    bits, scale, generator = _layer(FFN, DIM, 43)
    dy = torch.randn(TOKENS, FFN, generator=generator).to(DEVICE, torch.bfloat16)
    dx = kernels.packed_transpose(dy, bits, DIM, scale)
    assert dx.shape == (TOKENS, DIM) and dx.dtype == torch.bfloat16 and bool(torch.isfinite(dx).all())
    assert torch.equal(kernels.packed_transpose(dy * 4.0, bits, DIM, scale), dx * 4.0)
    assert torch.equal(kernels.packed_transpose(dy, bits ^ 0xFF, DIM, scale), -dx)
    order = torch.randperm(TOKENS, generator=generator).to(DEVICE)
    moved = kernels.packed_transpose(dy[order], bits, DIM, scale)
    assert rel(moved, dx[order]) <= 1e-4
    assert float((moved != dx[order]).float().mean()) <= 1e-3
    picked = _sample(128, TOKENS, generator)
    signs = kernels.unpack_rows(bits, DIM, dtype=torch.float32)
    want = (dy[picked].float() * scale) @ signs
    assert rel(dx[picked], want) <= 4e-3
    assert rel(dx[picked], want.to(torch.bfloat16)) <= 1e-3
    assert kernels.wait_timeouts() == 0


def test_evidence_full_size_properties():
    """E0 = (dY * x_scale)^T @ sign(x), fp32 14336 x 4096 from 16384 tokens
    (evidence_from_packed, loader.py:306-312), and the whole backward in one call."""

    bits, scale, generator = _layer(FFN, DIM, 47)
    x = torch.randn(TOKENS, DIM, generator=generator).to(DEVICE, torch.bfloat16)
    dy = torch.randn(TOKENS, FFN, generator=generator).to(DEVICE, torch.bfloat16)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
    evidence = kernels.evidence_from_packed(dy, act_bits, DIM, act_scale)
    assert evidence.shape == (FFN, DIM) and evidence.dtype == torch.float32
    assert torch.equal(kernels.evidence_from_packed(dy * 2.0, act_bits, DIM, act_scale), evidence * 2.0)
    assert torch.equal(kernels.evidence_from_packed(dy, act_bits ^ 0xFF, DIM, act_scale), -evidence)
    # additive over a split of the batch; not bit for bit: the order of the sums differs, and the
    # tensor core's fp32 accumulation over 256 k-blocks is itself only good to about 1e-5
    half = TOKENS // 2
    parts = (kernels.evidence_from_packed(dy[:half], act_bits[:half], DIM, act_scale[:half]) +
             kernels.evidence_from_packed(dy[half:], act_bits[half:], DIM, act_scale[half:]))
    assert rel(parts, evidence) <= 1e-4
    picked = _sample(128, FFN, generator)
    decoded = kernels.unpack_rows(act_bits, DIM, dtype=torch.float32) * act_scale[:, None]
    want = dy[:, picked].float().t() @ decoded
    assert rel(evidence[picked], want) <= 1e-3
    # the fused backward against the separate calls and against the same sample
    aux = torch.stack((act_offset, act_scale))
    dx, fused, g_scale, g_bias = kernels.linear_backward(dy, bits, scale, DIM, act_bits, aux, want_bias=True)
    offset_term = (dy[:, picked].float() * act_offset[:, None]).sum(0)
    want_fused = (want + offset_term[:, None]) * scale[picked, None]
    assert rel(fused[picked], want_fused) <= 1e-3
    signs = kernels.unpack_rows(bits, DIM, dtype=torch.float32)
    want_g_scale = ((want + offset_term[:, None]) * signs[picked]).sum(1)
    assert rel(g_scale[picked], want_g_scale) <= 1e-3
    assert rel(g_bias, dy.float().sum(0)) <= 1e-5
    assert rel(dx, kernels.packed_transpose(dy, bits, DIM, scale)) <= 2e-3
    assert kernels.wait_timeouts() == 0


# ---------------------------------------------------------------------------------------
# the CUDA kernels against the reference's own compiled CPU kernels (no restatement between)
# ---------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def compiled_reference():
    from oracle import build_ref

    module = build_ref.load()
    if module is None:
        pytest.skip("oracle/_ref/qste_cpu.so was not built (no reference checkout where this tree was built)")
    return module


def test_pack_affine_rows_full_size_equals_the_compiled_reference(compiled_reference):
    x = torch.randn(TOKENS, DIM, generator=torch.Generator().manual_seed(23)).to(torch.bfloat16)
    want = compiled_reference.pack_affine_rows(x.float())
    got = kernels.pack_affine_rows(x.to(DEVICE))
    for mine, theirs in zip(got, want):
        assert torch.equal(mine.cpu(), theirs)


@pytest.mark.parametrize("rows,columns,steps", [(2048, 2048, 3), (FFN, DIM, 1)])
def test_coordinate_update_equals_the_compiled_reference(compiled_reference, rows, columns, steps):
    """cpu.cpp:578-808 itself, compiled: the single-layer configuration over three steps and
    one step of the 58.7 M-coordinate surface."""

    generator = torch.Generator().manual_seed(37)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    cpu = {
        "coordinate": coordinate,
        "packed": compiled_reference.pack_coordinate(coordinate),
        "moment_q": torch.zeros(rows, columns, dtype=torch.int8),
        "moment_scale": torch.full((rows * columns // 256,), 1 / 127, dtype=torch.float16),
        "row_v": torch.zeros(rows, dtype=torch.float16),
        "col_v": torch.zeros(columns, dtype=torch.float16),
    }
    gpu = {k: v.clone().to(DEVICE) for k, v in cpu.items()}
    for step in range(steps):
        evidence = torch.randn(rows, columns, generator=generator) * (3.0 if step == 0 else 0.1)
        want = compiled_reference.coordinate_update(evidence.clone(), *[cpu[k] for k in ORDER], 0.9, 0.99, 2.0, 1.0, 256, 5, step)
        got = kernels.coordinate_update(evidence.to(DEVICE), *[gpu[k] for k in ORDER], beta1=0.9, beta2=0.99,
                                        update_clip=2.0, coordinate_lr=1.0, block_size=256, seed=5, step=step)
        assert got == int(want)
        for key in ORDER:
            mine, theirs = gpu[key].cpu(), cpu[key]
            if mine.dtype == torch.float16:
                mine, theirs = mine.view(torch.int16), theirs.view(torch.int16)
            assert torch.equal(mine, theirs), (key, step, int((mine != theirs).sum()))
