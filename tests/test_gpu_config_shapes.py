"""The three packed-sign GEMMs at the shapes of every benchmark configuration, against
the CPU oracle.

* the GEMM sweep: (K, N) in {(4096, 11008), (11008, 4096), (4096, 14336), (14336, 4096)};
  batches of 1, 16 and 128 tokens are compared with the oracle in full (they are where the
  library switches between the bit-streaming kernel, the small-batch kernels and the
  tensor-core tiles), 4096 and 16384 tokens on 128 sampled rows of every output plus the
  exact properties that do not depend on size;
* the GPT-2-small shape (8192 tokens, 768 <-> 3072) and the Llama-1.1B shape (16384 tokens
  per GPU at 8 GPUs, 2048 <-> 5632) the same way.

Reference interfaces: kernels.packed_linear_affine / packed_transpose /
evidence_from_packed (src/qste/kernels/loader.py:292-312, cpu.cpp:342-456) and
QSTELinearFn.backward (src/qste/functional.py:173-194).  The reference's own GPU tests run
"every batch size" and "awkward shapes" the same way (tests/test_gpu.py:33-41, 248-258).

Bar: relative Frobenius error <= 1e-3 against the oracle's fp32 result rounded to the
kernel's output dtype (bf16 for Y and dX, fp32 for the evidence).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from qste_b200 import kernels

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
BAR = 1e-3

SWEEP = [(4096, 11008), (11008, 4096), (4096, 14336), (14336, 4096)]
GPT2 = [(768, 3072), (3072, 768)]
LLAMA = [(2048, 5632), (5632, 2048)]


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def host(tensor):
    return tensor.detach().float().cpu().numpy()


def like_bf16(array):
    return torch.from_numpy(np.ascontiguousarray(array)).to(torch.bfloat16).float().numpy()


def problem(samples, columns, rows, seed):
    """Sweep inputs as the benchmark words them: bf16 N(0,1) activations and gradients,
    Bernoulli(1/2) sign bits, per-row scale uniform in [0.01, 0.05]."""

    generator = torch.Generator().manual_seed(seed)
    x = torch.randn(samples, columns, generator=generator).to(torch.bfloat16)
    dy = torch.randn(samples, rows, generator=generator).to(torch.bfloat16)
    bits = torch.randint(0, 256, (rows, columns // 8), generator=generator, dtype=torch.int32).to(torch.uint8)
    scale = torch.rand(rows, generator=generator) * 0.04 + 0.01
    return x, dy, bits, scale, generator


def check_against_oracle(samples, columns, rows, seed, sample_rows=None):
    """Forward, dX, plain evidence and the fused backward of one layer shape.  With
    `sample_rows`, that many rows of every output are compared (the oracle's cost is then
    that of a small batch); otherwise everything is."""

    x, dy, bits, scale, generator = problem(samples, columns, rows, seed)
    xd, dyd, bitsd, scaled = x.to(DEVICE), dy.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE)
    y = kernels.packed_linear_affine(xd, bitsd, scaled, None, columns)
    dx = kernels.packed_transpose(dyd, bitsd, columns, scaled)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(xd)
    plain = kernels.evidence_from_packed(dyd, act_bits, columns, act_scale)
    aux = torch.stack((act_offset, act_scale))
    dx_fused, fused, g_scale, g_bias = kernels.linear_backward(dyd, bitsd, scaled, columns, act_bits, aux, want_bias=True)
    assert y.dtype == torch.bfloat16 and y.shape == (samples, rows)
    assert dx.dtype == torch.bfloat16 and dx.shape == (samples, columns)
    assert plain.dtype == torch.float32 and plain.shape == (rows, columns)
    torch.cuda.synchronize()
    assert kernels.wait_timeouts() == 0, kernels.first_wait_timeout()

    # the activation encoding is bit-exact at every one of these widths
    want_bits, want_offset, want_scale = oracle.pack_affine_rows(x.float())
    assert np.array_equal(act_bits.cpu().numpy(), want_bits)
    assert np.array_equal(act_offset.cpu().numpy(), want_offset)
    assert np.array_equal(act_scale.cpu().numpy(), want_scale)

    if sample_rows is None or sample_rows >= samples:
        tokens = torch.arange(samples)
    else:
        tokens = torch.randperm(samples, generator=generator)[:sample_rows].sort().values
    if sample_rows is None or sample_rows >= rows:
        outputs = torch.arange(rows)
    else:
        outputs = torch.randperm(rows, generator=generator)[:sample_rows].sort().values

    want_y = oracle.packed_linear_affine(x[tokens].float(), bits, scale, None, columns)
    assert rel(host(y[tokens.to(DEVICE)]), like_bf16(want_y)) <= BAR, "forward"
    want_dx = oracle.packed_transpose(dy[tokens].float(), bits, columns, scale)
    assert rel(host(dx[tokens.to(DEVICE)]), like_bf16(want_dx)) <= BAR, "dX"
    assert rel(host(dx_fused[tokens.to(DEVICE)]), like_bf16(want_dx)) <= BAR, "dX of the fused backward"

    picked_dy = dy[:, outputs].float().contiguous()
    want_plain = oracle.evidence_from_packed(picked_dy, want_bits, columns, want_scale)
    assert rel(host(plain[outputs.to(DEVICE)]), want_plain) <= BAR, "evidence"
    correction = picked_dy.double().t().numpy() @ want_offset.astype(np.float64)
    decoded = want_plain.astype(np.float64) + correction[:, None]
    picked_scale = scale[outputs].double().numpy()
    assert rel(host(fused[outputs.to(DEVICE)]), decoded * picked_scale[:, None]) <= BAR, "fused evidence"
    want_g_scale = oracle.packed_row_inner(decoded.astype(np.float32), bits[outputs].contiguous(), columns)
    assert rel(host(g_scale[outputs.to(DEVICE)]), want_g_scale) <= BAR, "scale gradient"
    assert rel(host(g_bias), dy.double().sum(0).numpy()) <= 1e-5, "bias gradient"
    return xd, dyd, bitsd, scaled, (y, dx, plain), (act_bits, act_scale)


def check_exact_properties(xd, dyd, bitsd, scaled, outputs, saved, columns):
    """What holds bit for bit at any size: scaling by a power of two, and a flip of every
    sign bit negates the result."""

    y, dx, plain = outputs
    act_bits, act_scale = saved
    assert torch.equal(kernels.packed_linear_affine(xd, bitsd, scaled * 2.0, None, columns), y * 2.0)
    assert torch.equal(kernels.packed_linear_affine(xd, bitsd ^ 0xFF, scaled, None, columns), -y)
    assert torch.equal(kernels.packed_transpose(dyd, bitsd ^ 0xFF, columns, scaled), -dx)
    assert torch.equal(kernels.evidence_from_packed(dyd, act_bits ^ 0xFF, columns, act_scale), -plain)
    torch.cuda.synchronize()
    assert kernels.wait_timeouts() == 0, kernels.first_wait_timeout()


@pytest.mark.parametrize("columns,rows", SWEEP)
@pytest.mark.parametrize("samples", [1, 16, 128])
def test_sweep_small_batches_equal_the_oracle_in_full(samples, columns, rows):
    check_against_oracle(samples, columns, rows, seed=1000 + samples + rows)


@pytest.mark.parametrize("columns,rows", SWEEP)
@pytest.mark.parametrize("samples", [2, 3, 4, 5, 8, 31, 64, 100])
def test_sweep_forward_every_small_batch_equals_the_oracle(samples, columns, rows):
    """The batch sizes between the benchmark's, where the forward dispatch changes kernel."""

    x, _, bits, scale, generator = problem(samples, columns, rows, seed=2000 + samples)
    bias = torch.randn(rows, generator=generator)
    y = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
    want = oracle.packed_linear_affine(x.float(), bits, scale, bias, columns)
    assert rel(host(y), like_bf16(want)) <= BAR
    assert kernels.wait_timeouts() == 0, kernels.first_wait_timeout()


@pytest.mark.parametrize("columns,rows", SWEEP)
@pytest.mark.parametrize("samples", [4096, 16384])
def test_sweep_large_batches_on_sampled_rows_and_exact_properties(samples, columns, rows):
    xd, dyd, bitsd, scaled, outputs, saved = check_against_oracle(
        samples, columns, rows, seed=3000 + rows, sample_rows=128)
    check_exact_properties(xd, dyd, bitsd, scaled, outputs, saved, columns)


@pytest.mark.parametrize("columns,rows", GPT2)
def test_gpt2_small_mlp_shapes(columns, rows):
    """8 sequences x 1024 tokens through a 768 <-> 3072 MLP."""

    xd, dyd, bitsd, scaled, outputs, saved = check_against_oracle(8192, columns, rows, seed=4000 + rows, sample_rows=128)
    check_exact_properties(xd, dyd, bitsd, scaled, outputs, saved, columns)


@pytest.mark.parametrize("columns,rows", LLAMA)
@pytest.mark.parametrize("samples", [16384, 2048])
def test_llama_1b_mlp_shapes(samples, columns, rows):
    """2048 <-> 5632: one rank's 8 sequences of 2048 tokens at 8 GPUs, and one sequence (the
    micro-batch of an accumulating run)."""

    xd, dyd, bitsd, scaled, outputs, saved = check_against_oracle(samples, columns, rows, seed=5000 + rows, sample_rows=128)
    check_exact_properties(xd, dyd, bitsd, scaled, outputs, saved, columns)
