"""The C oracle against the reference's own compiled CPU kernels, at configuration scale.

``oracle/build_ref.py`` compiles the reference's ``src/qste/kernels/cpu.cpp`` into
``oracle/_ref/qste_cpu.so`` wherever the reference checkout is present; the built file
travels with the tree.  These tests load it and demand that the oracle's integer and bit
outputs equal the reference's byte for byte: activation packing, sign packing, the
row-inner product and the whole optimizer state over several steps, up to the 2048 x 2048
single-layer configuration (three steps, one and eight torch threads) and one step at
14336 x 4096.  GEMM outputs are compared to 1e-5 (the reference's come out of ``at::mm``).
Skipped when the compiled reference is absent.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from oracle import build_ref

ORDER = ("coordinate", "packed", "moment_q", "moment_scale", "row_v", "col_v")


@pytest.fixture(scope="module")
def reference():
    module = build_ref.load()
    if module is None:
        pytest.skip("oracle/_ref/qste_cpu.so was not built (no reference checkout on this machine)")
    return module


def raw(array):
    """Bytes of a tensor or array, so fp16 state compares by bit pattern."""

    if isinstance(array, torch.Tensor):
        array = array.view(torch.int16).numpy() if array.dtype == torch.float16 else array.numpy()
    return array.view(np.int16) if array.dtype == np.float16 else array


def fresh_state(reference, rows, columns, block, seed=11):
    generator = torch.Generator().manual_seed(seed)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    blocks = (rows * columns + block - 1) // block
    return {
        "coordinate": coordinate,
        "packed": reference.pack_coordinate(coordinate),
        "moment_q": torch.zeros(rows, columns, dtype=torch.int8),
        "moment_scale": torch.full((blocks,), 1 / 127, dtype=torch.float16),
        "row_v": torch.zeros(rows, dtype=torch.float16),
        "col_v": torch.zeros(columns, dtype=torch.float16),
    }


@pytest.mark.parametrize("rows,columns", [(17, 13), (64, 64), (128, 96), (33, 8), (5, 1), (7, 65), (256, 2048),
                                          (300, 1000), (512, 4096), (128, 14336)])
def test_packing_and_row_inner_are_byte_identical(reference, rows, columns):
    generator = torch.Generator().manual_seed(rows * 31 + columns)
    for x in (torch.randn(rows, columns, generator=generator),
              torch.nn.functional.gelu(torch.randn(rows, columns, generator=generator)) * 3 + 0.25,
              torch.randn(rows, columns, generator=generator).to(torch.bfloat16).float()):
        theirs = reference.pack_affine_rows(x)
        mine = oracle.pack_affine_rows(x)
        for a, b in zip(theirs, mine):
            assert np.array_equal(raw(a), raw(b))
        matrix = torch.randn(rows, columns, generator=generator)
        assert np.array_equal(reference.packed_row_inner(matrix, theirs[0], columns).numpy(),
                              oracle.packed_row_inner(matrix, mine[0], columns))
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    assert np.array_equal(reference.pack_coordinate(coordinate).numpy(), oracle.pack_coordinate(coordinate))


@pytest.mark.parametrize("rows,columns,block,steps", [
    (16, 32, 64, 3), (24, 40, 64, 3), (7, 13, 16, 3), (300, 1000, 256, 3), (129, 77, 64, 3), (1, 4097, 256, 3),
    (2048, 2048, 256, 3), (14336, 4096, 256, 1)])
@pytest.mark.parametrize("threads", [1, 8])
def test_optimizer_state_is_byte_identical(reference, rows, columns, block, steps, threads):
    if rows * columns > 1 << 24 and threads != 8:
        pytest.skip("the largest case runs once")
    saved = torch.get_num_threads()
    torch.set_num_threads(threads)
    try:
        theirs = fresh_state(reference, rows, columns, block)
        mine = {key: value.clone().numpy() for key, value in theirs.items()}
        for step in range(steps):
            evidence = torch.randn(rows, columns, generator=torch.Generator().manual_seed(100 + step)) * (10.0 ** (step - 1))
            want = reference.coordinate_update(evidence.clone(), *[theirs[k] for k in ORDER], 0.9, 0.99, 2.0, 1.0, block, 7, step)
            got = oracle.coordinate_update(evidence.clone().numpy(), *[mine[k] for k in ORDER], beta1=0.9, beta2=0.99,
                                           update_clip=2.0, coordinate_lr=1.0, block_size=block, seed=7, step=step)
            assert int(want) == got, step
            for key in ORDER:
                assert np.array_equal(raw(theirs[key]), raw(mine[key])), (key, step)
    finally:
        torch.set_num_threads(saved)


@pytest.mark.parametrize("rows,columns,samples", [(17, 13, 5), (128, 96, 40), (512, 1024, 64), (3072, 768, 32)])
def test_projections_agree_to_fp32_accuracy(reference, rows, columns, samples):
    generator = torch.Generator().manual_seed(rows + samples)
    x = torch.randn(samples, columns, generator=generator)
    dy = torch.randn(samples, rows, generator=generator)
    packed = reference.pack_affine_rows(torch.randn(rows, columns, generator=generator))[0]
    scale = torch.rand(rows, generator=generator) + 0.5
    bias = torch.randn(rows, generator=generator)

    def rel(a, b):
        return float(np.linalg.norm(np.asarray(a, np.float64) - b) / np.linalg.norm(b))

    assert rel(reference.packed_linear_affine(x, packed, scale, bias, columns).numpy(),
               oracle.packed_linear_affine(x, packed, scale, bias, columns)) <= 1e-5
    assert rel(reference.packed_transpose(dy, packed, columns, scale).numpy(),
               oracle.packed_transpose(dy, packed, columns, scale)) <= 1e-5
    bits, _, act_scale = reference.pack_affine_rows(x)
    assert rel(reference.evidence_from_packed(dy, bits, columns, act_scale).numpy(),
               oracle.evidence_from_packed(dy, bits, columns, act_scale)) <= 1e-5
