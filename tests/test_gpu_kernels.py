"""Parity of every CUDA kernel with the CPU oracle and with the reference's golden
vectors, called through the C ABI (qste_b200.kernels is a ctypes shim over it).

Bars: bit-exact for sign bits, activation bit packs, int8 coordinates / moments and
flip counts; relative Frobenius error <= 1e-3 for GEMM outputs and float gradients
(fp32 accumulation); 1e-4 absolute where the reference's own tests use it on
small fp32 cases (tests/test_kernels.py:73-152 of the reference).
"""

import os

import numpy as np
import pytest
import torch

import oracle
from qste_b200 import kernels

pytestmark = pytest.mark.gpu

ORDER = ("coordinate", "packed", "moment_q", "moment_scale", "row_v", "col_v")
DEVICE = "cuda"


def dev(array, dtype=None):
    tensor = torch.from_numpy(np.ascontiguousarray(array)).to(DEVICE)
    return tensor if dtype is None else tensor.to(dtype)


def host(tensor):
    return tensor.detach().float().cpu().numpy() if tensor.dtype in (torch.bfloat16, torch.float16) \
        else tensor.detach().cpu().numpy()


def like(array, dtype):
    """The oracle's fp32 result rounded to the kernel's output dtype: outputs are
    compared like for like, so only the fp32 accumulators are under test."""

    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype).float().numpy()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


class forced_path:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.saved = os.environ.get("QSTE_B200_PATH")
        os.environ["QSTE_B200_PATH"] = self.name

    def __exit__(self, *exc):
        if self.saved is None:
            os.environ.pop("QSTE_B200_PATH", None)
        else:
            os.environ["QSTE_B200_PATH"] = self.saved


def tensor_path_or_skip(call):
    """Run `call` with the tcgen05 path forced; skip when the shape is not eligible."""

    with forced_path("tensor"):
        try:
            return call()
        except RuntimeError as error:
            if "unsupported" in str(error):
                pytest.skip("shape not eligible for the tensor-core path")
            raise


# ---------------------------------------------------------------------------------------
# packing
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("case", [f"pack{i}" for i in range(6)])
def test_packing_golden(golden, case):
    x = golden(case, "x")
    columns = x.shape[1]
    bits, offset, scale = kernels.pack_affine_rows(dev(x))
    assert np.array_equal(host(bits), golden(case, "bits"))
    assert np.array_equal(host(offset), golden(case, "offset"))
    assert np.array_equal(host(scale), golden(case, "scale"))
    assert np.array_equal(host(kernels.pack_coordinate(dev(golden(case, "coordinate")))), golden(case, "coordinate_bits"))
    mask_bits = kernels.pack_bits(dev(golden(case, "mask")).bool())
    assert np.array_equal(host(mask_bits), golden(case, "mask_bits"))
    assert np.array_equal(host(kernels.apply_bits(dev(golden(case, "values")), mask_bits, columns)), golden(case, "applied"))
    assert np.array_equal(host(kernels.unpack_rows(bits, columns)), golden(case, "unpacked"))
    assert np.array_equal(host(kernels.unpack_bits(mask_bits, columns)), golden(case, "unpacked_bits"))


@pytest.mark.parametrize("rows,columns", [(1, 1), (5, 7), (9, 255), (3, 257), (70, 1000), (33, 2048), (257, 4096), (64, 515), (9, 1028), (3, 132), (17, 8), (40, 520)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_pack_affine_rows_is_bit_exact_for_every_dtype_and_ragged_width(rows, columns, dtype):
    generator = torch.Generator().manual_seed(rows * 1000 + columns)
    x = torch.randn(rows, columns, generator=generator)
    if rows % 2:
        x = torch.nn.functional.gelu(x) * 3.0 + 0.25
    x = x.to(dtype)
    bits, offset, scale = kernels.pack_affine_rows(x.to(DEVICE))
    want_bits, want_offset, want_scale = oracle.pack_affine_rows(x.float())
    assert np.array_equal(host(bits), want_bits)
    assert np.array_equal(host(offset), want_offset)
    assert np.array_equal(host(scale), want_scale)


@pytest.mark.parametrize("rows,columns", [(1, 64), (33, 2048), (257, 4096), (64, 128), (7, 14336), (5, 72), (3, 64 + 8)])
def test_pack_coordinate_and_pack_bits_at_layer_widths_equal_the_oracle(rows, columns):
    """Widths that are multiples of 64 take the 64-bytes-per-thread kernel; the others the
    byte-per-thread one (cpu.cpp:207-277 of the reference)."""

    generator = torch.Generator().manual_seed(rows + columns)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    coordinate[0, : min(columns, 9)] = 0  # zero counts as +1
    assert np.array_equal(host(kernels.pack_coordinate(coordinate.to(DEVICE))), oracle.pack_coordinate(coordinate))
    mask = torch.rand(rows, columns, generator=generator) < 0.3
    assert np.array_equal(host(kernels.pack_bits(mask.to(DEVICE))), oracle.pack_bits(mask))
    # a view that does not start on a 16-byte boundary falls back to the narrow kernel
    shifted = torch.zeros(rows * columns + 1, dtype=torch.int8, device=DEVICE)[1:].view(rows, columns)
    shifted.copy_(coordinate)
    assert np.array_equal(host(kernels.pack_coordinate(shifted)), oracle.pack_coordinate(coordinate))


def test_pack_handles_empty_and_constant_rows():
    bits, offset, scale = kernels.pack_affine_rows(torch.zeros(0, 16, device=DEVICE))
    assert bits.shape == (0, 2) and offset.numel() == 0
    constant = torch.full((4, 24), 2.5, device=DEVICE)
    bits, offset, scale = kernels.pack_affine_rows(constant)
    assert torch.all(bits == 255) and torch.all(offset == 2.5) and torch.all(scale == 0)
    zeros = torch.zeros(3, 10, device=DEVICE)
    bits, offset, scale = kernels.pack_affine_rows(zeros)
    assert host(bits).tolist() == [[255, 3]] * 3  # pad bits stay clear


@pytest.mark.parametrize("columns", [1, 7, 8, 9, 63, 64, 65])
def test_unpack_ragged_widths(columns):
    x = torch.randn(5, columns, generator=torch.Generator().manual_seed(columns))
    bits = oracle.pack_affine_rows(x)[0]
    assert np.array_equal(host(kernels.unpack_rows(dev(bits), columns)), oracle.unpack_rows(bits, columns))
    assert host(kernels.unpack_rows(dev(bits), columns, dtype=torch.bfloat16)).tolist() == oracle.unpack_rows(bits, columns).tolist()


# ---------------------------------------------------------------------------------------
# projections
# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("case", [f"proj{i}" for i in range(5)])
@pytest.mark.parametrize("path", ["auto", "simt"])
def test_projections_golden(golden, case, path):
    bits = dev(golden(case, "weight_bits"))
    x, dy = dev(golden(case, "x")), dev(golden(case, "dy"))
    scale, bias = dev(golden(case, "scale")), dev(golden(case, "bias"))
    columns = x.shape[1]
    with forced_path(path):
        assert np.allclose(host(kernels.packed_linear_affine(x, bits, scale, bias, columns)), golden(case, "y"), atol=1e-4)
        assert np.allclose(host(kernels.packed_linear_affine(x, bits, scale, None, columns)), golden(case, "y_nobias"), atol=1e-4)
        assert np.allclose(host(kernels.packed_transpose(dy, bits, columns, scale)), golden(case, "dx"), atol=1e-4)
        assert np.allclose(host(kernels.packed_transpose(dy, bits, columns)), golden(case, "dx_unscaled"), atol=1e-4)
        act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
        assert np.array_equal(host(act_bits), golden(case, "act_bits"))
        assert np.allclose(host(kernels.evidence_from_packed(dy, act_bits, columns, act_scale)), golden(case, "evidence"), atol=1e-3)
        assert np.allclose(host(kernels.evidence_from_packed(dy, act_bits, columns)), golden(case, "evidence_unscaled"), atol=1e-3)
        fused, g_scale, g_bias = kernels.linear_backward_evidence(
            dy, act_bits, torch.stack((act_offset, act_scale)), columns, bits, scale, want_bias=True)
        decoded = golden(case, "decoded")
        assert np.allclose(host(fused), decoded * golden(case, "scale")[:, None], atol=1e-3)
        assert np.allclose(host(g_scale), oracle.packed_row_inner(decoded, golden(case, "weight_bits"), columns), atol=1e-3)
        assert np.allclose(host(g_bias), golden(case, "dy").sum(0), atol=1e-4)
    assert np.allclose(host(kernels.packed_row_inner(dev(golden(case, "matrix")), bits, columns)), golden(case, "row_inner"), atol=1e-4)
    assert np.array_equal(host(kernels.packed_embedding(dev(golden(case, "ids")), bits, scale, columns)), golden(case, "embedding"))


def _problem(samples, rows, columns, dtype, seed=0):
    generator = torch.Generator().manual_seed(seed)
    x = torch.randn(samples, columns, generator=generator).to(dtype)
    dy = torch.randn(samples, rows, generator=generator).to(dtype)
    bits = torch.randint(0, 256, (rows, (columns + 7) // 8), generator=generator, dtype=torch.int32).to(torch.uint8)
    if columns % 8:
        bits[:, -1] &= (1 << (columns % 8)) - 1
    scale = torch.rand(rows, generator=generator) * 0.04 + 0.01
    bias = torch.randn(rows, generator=generator)
    return x, dy, bits, scale, bias


SHAPES = [(1, 1, 1), (3, 5, 7), (33, 129, 2048), (64, 200, 136), (130, 257, 96), (256, 512, 384), (17, 1024, 1024)]


@pytest.mark.parametrize("samples,rows,columns", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("path", ["auto", "simt"])
def test_projections_against_the_oracle(samples, rows, columns, dtype, path):
    x, dy, bits, scale, bias = _problem(samples, rows, columns, dtype, seed=samples + rows)
    with forced_path(path):
        y = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
        dx = kernels.packed_transpose(dy.to(DEVICE), bits.to(DEVICE), columns, scale.to(DEVICE))
        act_bits, act_offset, act_scale = kernels.pack_affine_rows(x.to(DEVICE))
        evidence = kernels.evidence_from_packed(dy.to(DEVICE), act_bits, columns, act_scale)
    assert y.dtype == dtype and dx.dtype == dtype and evidence.dtype == torch.float32
    want_y = oracle.packed_linear_affine(x.float(), bits, scale, bias, columns)
    want_dx = oracle.packed_transpose(dy.float(), bits, columns, scale)
    want_ev = oracle.evidence_from_packed(dy.float(), host(act_bits), columns, host(act_scale))
    bar = 1e-5 if dtype == torch.float32 else 1e-3
    assert rel(host(y), like(want_y, dtype)) <= bar
    assert rel(host(dx), like(want_dx, dtype)) <= bar
    assert rel(host(evidence), want_ev) <= bar


@pytest.mark.parametrize("samples", [1, 2, 3, 4])
@pytest.mark.parametrize("rows,columns", [(64, 128), (1000, 1024), (515, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_batch_streaming_forward(samples, rows, columns, dtype):
    x, _, bits, scale, bias = _problem(samples, rows, columns, dtype, seed=rows)
    with forced_path("stream"):
        y = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
        y_nobias = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), None, columns)
    want = oracle.packed_linear_affine(x.float(), bits, scale, bias, columns)
    bar = 1e-5 if dtype == torch.float32 else 1e-3
    assert rel(host(y), like(want, dtype)) <= bar
    assert rel(host(y_nobias), like(oracle.packed_linear_affine(x.float(), bits, scale, None, columns), dtype)) <= bar


@pytest.mark.parametrize("samples", [1, 2, 3, 4])
@pytest.mark.parametrize("rows,columns", [(5, 128), (97, 256), (33, 384), (515, 1024), (3072, 768), (4104, 2048), (300, 16384), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_look_up_table_forward_for_one_to_four_tokens(samples, rows, columns, dtype):
    """The cluster kernel of gemm_lut.cu against the oracle: every token count, row counts that do
    not divide over the clusters, contractions of one unit of 128 columns up to 16384 (four and
    eight slices), with and without bias."""

    if samples > 2 and columns == 16384 and dtype == torch.float32:
        pytest.skip("four tables of a 2048-column slice do not fit; the shape falls to other kernels")
    x, _, bits, scale, bias = _problem(samples, rows, columns, dtype, seed=samples + rows)
    with forced_path("stream"):
        y = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
        y_nobias = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), None, columns)
    assert y.dtype == dtype and y.shape == (samples, rows)
    # 16-bit batches of three and four are handed on to the register-expansion kernel
    assert kernels.last_forward_kernel() == ("lut" if samples <= 2 or dtype == torch.float32 else "mma")
    bar = 1e-5 if dtype == torch.float32 else 1e-3
    want = oracle.packed_linear_affine(x.float(), bits, scale, bias, columns)
    assert rel(host(y), like(want, dtype)) <= bar
    assert rel(host(y_nobias), like(oracle.packed_linear_affine(x.float(), bits, scale, None, columns), dtype)) <= bar


@pytest.mark.parametrize("samples", [3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("rows,columns", [(5, 128), (97, 256), (33, 384), (515, 1024), (3072, 768), (4104, 2048), (300, 12288),
                                          (14336, 4096), (4096, 14336), (11008, 4096), (5632, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_register_expansion_forward_for_3_to_32_tokens(samples, rows, columns, dtype):
    """The warp-MMA kernel of gemm_mma.cu against the oracle: every count of token tiles (1, 2, 4)
    at its first and last batch size, row counts that do not divide over the clusters or the 16-row
    slabs, contractions from one unit of 128 columns (one CTA per cluster) to 14336 (eight), runs of
    512 columns that are partly filled (768, 14336 / 8), with and without bias -- through the
    dispatcher's own choice (no forced path), which must be this kernel wherever it is meant to
    serve: up to 16 tokens always, up to 32 for contractions of at most 12288 columns."""

    x, _, bits, scale, bias = _problem(samples, rows, columns, dtype, seed=samples + rows)
    y = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
    served = kernels.last_forward_kernel()
    assert served == ("mma" if samples <= 16 or columns <= 12288 else "tensor")
    y_nobias = kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), None, columns)
    assert y.dtype == dtype and y.shape == (samples, rows)
    want = oracle.packed_linear_affine(x.float(), bits, scale, bias, columns)
    assert rel(host(y), like(want, dtype)) <= 1e-3
    assert rel(host(y_nobias), like(oracle.packed_linear_affine(x.float(), bits, scale, None, columns), dtype)) <= 1e-3
    # and element by element: the same sums in another order, rounded once to the 16-bit type
    apart = np.abs(host(y) - like(want, dtype))
    assert float(apart.max()) <= 2.0 ** -6 * float(np.abs(like(want, dtype)).max())


def test_small_batch_forward_dispatch():
    """Which kernel family serves which batch size at a layer's shape (bf16)."""

    rows, columns = 4096, 4096
    chosen = {}
    for samples in (1, 2, 3, 32, 33, 128):
        x, _, bits, scale, bias = _problem(samples, rows, columns, torch.bfloat16, seed=samples)
        kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
        chosen[samples] = kernels.last_forward_kernel()
    assert chosen == {1: "lut", 2: "lut", 3: "mma", 32: "mma", 33: "tensor", 128: "tensor"}
    x, _, bits, scale, bias = _problem(16, rows, columns, torch.float32, seed=3)
    kernels.packed_linear_affine(x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
    assert kernels.last_forward_kernel() == "tensor"      # fp32 activations: three bf16 planes on tcgen05


@pytest.mark.parametrize("samples", [1, 8, 32, 128])
def test_forward_replays_from_a_cuda_graph(samples):
    """A decode loop replays its launches from a CUDA graph: every forward kernel family must be
    capturable (no host read, no allocation of its own, no stream of its own) and a replay must
    return the bits of the eager call."""

    rows, columns = 3072, 768
    x, _, bits, scale, bias = _problem(samples, rows, columns, torch.bfloat16, seed=samples)
    x, bits, scale, bias = x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE)
    eager = kernels.packed_linear_affine(x, bits, scale, bias, columns)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        kernels.packed_linear_affine(x, bits, scale, bias, columns)      # this stream's workspace exists
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            captured = kernels.packed_linear_affine(x, bits, scale, bias, columns)
        captured.zero_()
        graph.replay()
        side.synchronize()
    assert torch.equal(captured, eager)
    torch.cuda.current_stream().wait_stream(side)


TENSOR_SHAPES = [(128, 256, 128), (200, 300, 256), (1024, 512, 1024), (77, 1000, 384), (4096, 2048, 2048)]
# Shapes whose output has at least 148 tiles of 256 x 256, ragged on both sides: the kernel then
# runs its 256-row tiles, two or three per CTA, with the expander warps sharing the epilogue.
# The last of each list has enough k-blocks for the tiles of the last round of CTAs to be cut along
# the contraction (partial sums + a second kernel); (16, 4096, 4096) and (1024, 512, 1024) are cut
# the same way because they have fewer tiles than the device has SMs.
TALL_FORWARD = [(2600, 4104, 192), (5200, 4104, 128), (4096, 4352, 64), (16, 4096, 4096), (2600, 4104, 1024)]
TALL_TRANSPOSE = [(2600, 200, 4160), (5130, 136, 4352), (16, 4096, 4096), (2600, 1024, 4160)]
TALL_EVIDENCE = [(200, 2600, 4160), (136, 5128, 4352), (1024, 2600, 4160)]


@pytest.mark.parametrize("samples,rows,columns", TENSOR_SHAPES + TALL_FORWARD)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_tensor_core_forward(samples, rows, columns, dtype):
    x, _, bits, scale, bias = _problem(samples, rows, columns, dtype, seed=7)
    y = tensor_path_or_skip(lambda: kernels.packed_linear_affine(
        x.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns))
    with forced_path("simt"):
        cross = kernels.packed_linear_affine(x.to(DEVICE).float(), bits.to(DEVICE), scale.to(DEVICE), bias.to(DEVICE), columns)
    bar = 1e-5 if dtype == torch.float32 else 1e-3
    assert rel(host(y), like(host(cross), dtype)) <= bar
    if samples * rows * columns <= 1 << 28 or (samples, rows, columns) == TALL_FORWARD[2]:
        assert rel(host(y), like(oracle.packed_linear_affine(x.float(), bits, scale, bias, columns), dtype)) <= bar
    assert kernels.wait_timeouts() == 0


@pytest.mark.parametrize("samples,rows,columns", TENSOR_SHAPES + TALL_TRANSPOSE)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_transpose(samples, rows, columns, dtype):
    _, dy, bits, scale, _ = _problem(samples, rows, columns, dtype, seed=8)
    dx = tensor_path_or_skip(lambda: kernels.packed_transpose(dy.to(DEVICE), bits.to(DEVICE), columns, scale.to(DEVICE)))
    with forced_path("simt"):
        cross = kernels.packed_transpose(dy.to(DEVICE).float(), bits.to(DEVICE), columns, scale.to(DEVICE))
    # the row scale rides the tensor-core operand in fp16 (2^-12 relative per term)
    assert rel(host(dx), like(host(cross), dtype)) <= 1e-3
    # and against the oracle itself: whole output when that takes seconds, else 128 sampled rows
    picked = torch.arange(samples) if samples * rows * columns <= 1 << 28 else \
        torch.randperm(samples, generator=torch.Generator().manual_seed(1))[:128]
    want = oracle.packed_transpose(dy[picked].float(), bits, columns, scale)
    assert rel(host(dx[picked.to(DEVICE)]), like(want, dtype)) <= 1e-3
    assert kernels.wait_timeouts() == 0


@pytest.mark.parametrize("samples,rows,columns", TENSOR_SHAPES + TALL_EVIDENCE)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_evidence(samples, rows, columns, dtype):
    x, dy, bits, scale, _ = _problem(samples, rows, columns, dtype, seed=9)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x.to(DEVICE))
    aux = torch.stack((act_offset, act_scale))
    fused = tensor_path_or_skip(lambda: kernels.linear_backward_evidence(
        dy.to(DEVICE), act_bits, aux, columns, bits.to(DEVICE), scale.to(DEVICE), want_bias=True))
    with forced_path("simt"):
        cross = kernels.linear_backward_evidence(
            dy.to(DEVICE).float(), act_bits, aux, columns, bits.to(DEVICE), scale.to(DEVICE), want_bias=True)
    assert rel(host(fused[0]), host(cross[0])) <= 1e-3
    assert rel(host(fused[1]), host(cross[1])) <= 1e-3
    assert rel(host(fused[2]), host(cross[2])) <= 1e-5
    plain = tensor_path_or_skip(lambda: kernels.evidence_from_packed(dy.to(DEVICE), act_bits, columns, act_scale))
    with forced_path("simt"):
        plain_cross = kernels.evidence_from_packed(dy.to(DEVICE).float(), act_bits, columns, act_scale)
    assert rel(host(plain), host(plain_cross)) <= 1e-3
    # and against the oracle itself: every row when that takes seconds, else 128 sampled rows
    picked = torch.arange(rows) if samples * rows * columns <= 1 << 28 else \
        torch.randperm(rows, generator=torch.Generator().manual_seed(2))[:128]
    grad = dy[:, picked].float().contiguous()
    want_plain = oracle.evidence_from_packed(grad, host(act_bits), columns, host(act_scale))
    assert rel(host(plain[picked.to(DEVICE)]), want_plain) <= 1e-3
    decoded = want_plain.astype(np.float64) + (grad.double().t().numpy() @ host(act_offset).astype(np.float64))[:, None]
    assert rel(host(fused[0][picked.to(DEVICE)]), decoded * scale[picked].double().numpy()[:, None]) <= 1e-3
    assert rel(host(fused[1][picked.to(DEVICE)]),
               oracle.packed_row_inner(decoded.astype(np.float32), bits[picked].contiguous(), columns)) <= 1e-3
    assert rel(host(fused[2]), dy.double().sum(0).numpy()) <= 1e-5
    assert kernels.wait_timeouts() == 0


@pytest.mark.parametrize("samples", [1, 3, 4, 5, 8, 9, 16, 17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("rows,columns", [(5, 128), (97, 256), (515, 1024), (3072, 768), (300, 16384), (4104, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_small_batch_evidence_kernel(samples, rows, columns, dtype):
    """evidence_lut.cu (up to 16 samples, fp32 throughout) and evidence_mma.cu (17..128 samples, each
    term rounded once to fp16 against its row's own power of two) against the oracle: evidence,
    row-scale gradient and bias gradient in one launch -- every count of four-sample groups and of
    32-sample words at its edges, row counts that do not divide over the warps or the slabs,
    contractions from 128 columns to 16384 (four chunks).  "stream" forces the small-batch kernels
    (the call fails where none applies)."""

    x, dy, bits, scale, _ = _problem(samples, rows, columns, dtype, seed=samples + columns)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x.to(DEVICE))
    aux = torch.stack((act_offset, act_scale))
    with forced_path("stream"):
        evidence, g_scale, g_bias = kernels.linear_backward_evidence(
            dy.to(DEVICE), act_bits, aux, columns, bits.to(DEVICE), scale.to(DEVICE), want_bias=True)
        _, g_scale_only, none = kernels.linear_backward_evidence(
            dy.to(DEVICE), act_bits, aux, columns, bits.to(DEVICE), scale.to(DEVICE))
    assert none is None and torch.equal(g_scale, g_scale_only)
    grad = dy.float().contiguous()
    plain = oracle.evidence_from_packed(grad, host(act_bits), columns, host(act_scale))
    decoded = plain.astype(np.float64) + (grad.double().t().numpy() @ host(act_offset).astype(np.float64))[:, None]
    bar = 1e-5 if samples <= 16 else 1e-3
    assert rel(host(evidence), decoded * scale.double().numpy()[:, None]) <= bar
    assert rel(host(g_scale), oracle.packed_row_inner(decoded.astype(np.float32), bits, columns)) <= max(bar, 1e-4)
    assert rel(host(g_bias), dy.double().sum(0).numpy()) <= 1e-5
    # row by row as well: every row is scaled by its own power of two, so a row of small gradients
    # is as accurate as a row of large ones
    want = decoded * scale.double().numpy()[:, None]
    row_error = np.linalg.norm(host(evidence) - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-30)
    assert float(row_error.max()) <= 10 * bar
    # the dispatcher's own choice is the same kernel: identical bits
    auto, auto_scale, _ = kernels.linear_backward_evidence(
        dy.to(DEVICE), act_bits, aux, columns, bits.to(DEVICE), scale.to(DEVICE), want_bias=True)
    assert torch.equal(auto, evidence) and torch.equal(auto_scale, g_scale)


def test_small_batch_evidence_with_weight_rows_of_very_different_magnitude():
    """evidence_mma.cu rounds every term to fp16 against ONE power of two per output row: rows whose
    gradients are 2^-60 of their neighbours' must come back as accurate as those (their row's own
    relative error, not the matrix's)."""

    samples, rows, columns = 64, 240, 1024
    x, dy, bits, scale, _ = _problem(samples, rows, columns, torch.bfloat16, seed=11)
    dy = (dy.float() * torch.pow(2.0, -2.0 * (torch.arange(rows) % 31).float())[None, :]).to(torch.bfloat16)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x.to(DEVICE))
    aux = torch.stack((act_offset, act_scale))
    evidence, g_scale, _ = kernels.linear_backward_evidence(dy.to(DEVICE), act_bits, aux, columns, bits.to(DEVICE), scale.to(DEVICE))
    grad = dy.float().contiguous()
    plain = oracle.evidence_from_packed(grad, host(act_bits), columns, host(act_scale))
    decoded = plain.astype(np.float64) + (grad.double().t().numpy() @ host(act_offset).astype(np.float64))[:, None]
    want = decoded * scale.double().numpy()[:, None]
    row_error = np.linalg.norm(host(evidence) - want, axis=1) / np.maximum(np.linalg.norm(want, axis=1), 1e-300)
    assert float(row_error.max()) <= 2e-3
    inner = oracle.packed_row_inner(decoded.astype(np.float32), bits, columns)
    assert float(np.max(np.abs(host(g_scale) - inner) / np.maximum(np.linalg.norm(decoded, axis=1), 1e-300))) <= 2e-3


def test_whole_backward_with_rows_of_very_different_magnitude():
    """The fused backward scales every row of the gradient by its own power of two before the
    fp16 re-encoding: rows 2^40 apart must each come back with their own relative accuracy (dX)
    and the evidence, dominated by the large rows, must still match the oracle."""

    samples, rows, columns = 256, 512, 384
    x, dy, bits, scale, _ = _problem(samples, rows, columns, torch.bfloat16, seed=33)
    generator = torch.Generator().manual_seed(34)
    magnitude = torch.exp2(torch.randint(-20, 21, (samples, 1), generator=generator).float())
    dy = (dy.float() * magnitude).to(torch.bfloat16)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x.to(DEVICE))
    aux = torch.stack((act_offset, act_scale))
    dx, evidence, g_scale, g_bias = kernels.linear_backward(
        dy.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE), columns, act_bits, aux, want_bias=True)
    want_dx = oracle.packed_transpose(dy.float(), bits, columns, scale)
    row_error = np.linalg.norm(host(dx).astype(np.float64) - want_dx, axis=1) / np.linalg.norm(want_dx, axis=1)
    assert row_error.max() <= 8e-3  # every row, however small, to bf16 output precision
    decoded = oracle.decoded_evidence(dy.float(), host(act_bits), host(act_offset), host(act_scale), columns)
    assert rel(host(evidence), decoded * scale.numpy()[:, None]) <= 1e-3
    assert rel(host(g_scale), oracle.packed_row_inner(decoded, bits.numpy(), columns)) <= 1e-3
    assert rel(host(g_bias), dy.float().numpy().sum(0)) <= 1e-5


@pytest.mark.parametrize("flags", [{}, {"QSTE_B200_TC_NOPAIR": "1"}, {"QSTE_B200_TC_NOPAIR": "1", "QSTE_B200_TC_NOSPLIT": "1"},
                                   {"QSTE_B200_TC_SHORT": "1"}, {"QSTE_B200_TC_TALL_ANY": "1"},
                                   {"QSTE_B200_TC_TALL_ANY": "1", "QSTE_B200_TC_NOPAIR": "1"}])
def test_every_tile_mode_of_the_tensor_core_gemm(flags):
    """Pairs of CTAs on 512-row tiles, single CTAs on 256-row tiles, with and without the split
    contraction, and 128-row tiles: the mode is fixed per process, so each runs in a child.  The
    last two also put the 256-row modes on work items of one and two k-blocks, a hundred times."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    script = Path(__file__).with_name("_tile_mode_check.py")
    environment = {k: v for k, v in os.environ.items() if not k.startswith("QSTE_B200_TC_")}
    environment.update(flags)
    done = subprocess.run([sys.executable, str(script)], env=environment, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and "OK" in done.stdout, done.stdout[-2000:] + done.stderr[-2000:]


def test_shape_and_dtype_errors_raise():
    x = torch.zeros(4, 16, device=DEVICE)
    bits = torch.zeros(8, 2, dtype=torch.uint8, device=DEVICE)
    with pytest.raises(RuntimeError, match="width"):
        kernels.packed_linear_affine(x, bits, torch.ones(8, device=DEVICE), None, 24)
    with pytest.raises(RuntimeError, match="scale"):
        kernels.packed_linear_affine(x, bits, torch.ones(7, device=DEVICE), None, 16)
    with pytest.raises(RuntimeError, match="uint8"):
        kernels.packed_linear_affine(x, bits.float(), torch.ones(8, device=DEVICE), None, 16)
    with pytest.raises(RuntimeError, match="vocabulary"):
        kernels.packed_embedding(torch.tensor([9], device=DEVICE), bits, torch.ones(8, device=DEVICE), 16)
    with pytest.raises(ValueError, match="power of two"):
        kernels.coordinate_update(
            torch.zeros(2, 8, device=DEVICE), torch.zeros(2, 8, dtype=torch.int8, device=DEVICE),
            torch.zeros(2, 1, dtype=torch.uint8, device=DEVICE), torch.zeros(2, 8, dtype=torch.int8, device=DEVICE),
            torch.zeros(1, dtype=torch.float16, device=DEVICE), torch.zeros(2, dtype=torch.float16, device=DEVICE),
            torch.zeros(8, dtype=torch.float16, device=DEVICE), beta1=0.9, beta2=0.99, update_clip=2.0,
            coordinate_lr=1.0, block_size=48, seed=1, step=0)


# ---------------------------------------------------------------------------------------
# coordinate optimizer
# ---------------------------------------------------------------------------------------

def _golden_state(golden, case):
    state = {}
    for key in ORDER:
        array = golden(case, f"init_{key}")
        state[key] = dev(array.view(np.float16) if key in ("moment_scale", "row_v", "col_v") else array)
    return state


@pytest.mark.parametrize("case", [f"update{i}" for i in range(8)])
def test_coordinate_update_golden(golden, case):
    rows, columns, block, seed, step0 = (int(v) for v in golden(case, "meta"))
    lr = float(np.ravel(golden(case, "lr"))[0])
    state = _golden_state(golden, case)
    for number in range(3):
        flips = kernels.coordinate_update(
            dev(golden(case, f"evidence{number}")), *[state[k] for k in ORDER], beta1=0.9, beta2=0.99,
            update_clip=2.0, coordinate_lr=lr, block_size=block, seed=seed, step=step0 + number)
        assert flips == int(np.ravel(golden(case, f"flips{number}"))[0])
        for key in ORDER:
            got = state[key].cpu().numpy()
            if got.dtype == np.float16:
                got = got.view(np.uint16)
            assert np.array_equal(got, golden(case, f"step{number}_{key}")), (key, number)


def _fresh_state(rows, columns, block, seed=11):
    generator = torch.Generator().manual_seed(seed)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=generator, dtype=torch.int32).to(torch.int8)
    blocks = (rows * columns + block - 1) // block
    return {
        "coordinate": coordinate,
        "packed": torch.from_numpy(oracle.pack_coordinate(coordinate)),
        "moment_q": torch.zeros(rows, columns, dtype=torch.int8),
        "moment_scale": torch.full((blocks,), 1 / 127, dtype=torch.float16),
        "row_v": torch.zeros(rows, dtype=torch.float16),
        "col_v": torch.zeros(columns, dtype=torch.float16),
    }


@pytest.mark.parametrize("rows,columns,block", [(2048, 2048, 256), (300, 1000, 256), (129, 77, 64), (1, 4097, 256), (4097, 3, 32), (512, 1536, 1024)])
def test_coordinate_update_equals_the_oracle_over_several_steps(rows, columns, block):
    """Config-1 scale and awkward shapes: every byte of state equal after each of 3 steps."""

    cpu = _fresh_state(rows, columns, block)
    gpu = {k: v.clone().to(DEVICE) for k, v in cpu.items()}
    arrays = {k: v.numpy() for k, v in cpu.items()}
    for step in range(3):
        evidence = torch.randn(rows, columns, generator=torch.Generator().manual_seed(100 + step)) * (10.0 ** (step - 1))
        want = oracle.coordinate_update(
            evidence.clone().numpy(), *[arrays[k] for k in ORDER], beta1=0.9, beta2=0.99, update_clip=2.0,
            coordinate_lr=1.0, block_size=block, seed=7, step=step)
        got = kernels.coordinate_update(
            evidence.to(DEVICE), *[gpu[k] for k in ORDER], beta1=0.9, beta2=0.99, update_clip=2.0,
            coordinate_lr=1.0, block_size=block, seed=7, step=step)
        for key in ORDER:
            mine, theirs = gpu[key].cpu().numpy(), arrays[key]
            if mine.dtype == np.float16:
                mine, theirs = mine.view(np.uint16), theirs.view(np.uint16)
            assert np.array_equal(mine, theirs), (key, step, int((mine != theirs).sum()))
        assert got == want


def test_coordinate_update_device_side_step_flips_and_gate():
    """step / flips / update_enabled as device tensors (cuda.py:1705-1812, tests/test_gpu.py:519-556
    of the reference): same result as host arguments, and a zeroed gate leaves everything alone."""

    rows, columns, block = 96, 160, 64
    evidence = torch.randn(rows, columns, generator=torch.Generator().manual_seed(5))
    common = dict(beta1=0.9, beta2=0.99, update_clip=2.0, coordinate_lr=2.0, block_size=block, seed=3)
    a = {k: v.to(DEVICE) for k, v in _fresh_state(rows, columns, block).items()}
    b = {k: v.to(DEVICE) for k, v in _fresh_state(rows, columns, block).items()}
    host_flips = kernels.coordinate_update(evidence.to(DEVICE), *[a[k] for k in ORDER], step=9, **common)
    step = torch.tensor(9, dtype=torch.int64, device=DEVICE)
    flips = torch.zeros((), dtype=torch.int64, device=DEVICE)
    gate = torch.ones((), dtype=torch.uint8, device=DEVICE)
    returned = kernels.coordinate_update(evidence.to(DEVICE), *[b[k] for k in ORDER], step=step, flips=flips,
                                         update_enabled=gate, **common)
    assert returned is flips and int(flips) == host_flips
    for key in ORDER:
        assert torch.equal(a[key], b[key]), key
    before = {k: v.clone() for k, v in b.items()}
    gate.zero_()
    kernels.coordinate_update(evidence.to(DEVICE), *[b[k] for k in ORDER], step=step, flips=flips,
                              update_enabled=gate, **common)
    assert int(flips) == 0
    for key in ORDER:
        assert torch.equal(before[key], b[key]), key


def test_coordinate_update_keeps_bits_in_sync_and_is_reproducible():
    rows, columns = 12, 20
    results = []
    for _ in range(2):
        state = {k: v.to(DEVICE) for k, v in _fresh_state(rows, columns, 64).items()}
        evidence = torch.randn(rows, columns, generator=torch.Generator().manual_seed(13)).to(DEVICE)
        kernels.coordinate_update(evidence, *[state[k] for k in ORDER], beta1=0.9, beta2=0.99, update_clip=2.0,
                                  coordinate_lr=4.0, block_size=64, seed=99, step=5)
        assert torch.equal(state["packed"], kernels.pack_coordinate(state["coordinate"]))
        results.append(state["coordinate"].clone())
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("samples,rows,columns", [(256, 512, 384), (200, 300, 256), (1024, 512, 1024), (33, 129, 2048), (64, 200, 136)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_whole_backward_in_one_call_equals_the_separate_calls(samples, rows, columns, dtype):
    """linear_backward = packed_transpose + linear_backward_evidence; the fused bf16 path shares
    one fp16 re-encoding of the gradient between the two GEMMs (one power of two per row, where
    the separate calls use one for the whole tensor: equal to within the fp16 rounding)."""

    x, dy, bits, scale, _ = _problem(samples, rows, columns, dtype, seed=21)
    dy, bits, scale = dy.to(DEVICE), bits.to(DEVICE), scale.to(DEVICE)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x.to(DEVICE))
    aux = torch.stack((act_offset, act_scale))
    dx, evidence, g_scale, g_bias = kernels.linear_backward(dy, bits, scale, columns, act_bits, aux, want_bias=True)
    want_dx = kernels.packed_transpose(dy, bits, columns, scale)
    want_ev, want_gs, want_gb = kernels.linear_backward_evidence(dy, act_bits, aux, columns, bits, scale, want_bias=True)
    assert dx.dtype == dtype and dx.shape == (samples, columns)
    close = 5e-4 if dtype == torch.bfloat16 else 1e-6
    assert rel(host(dx), host(want_dx)) <= (4e-3 if dtype == torch.bfloat16 else 1e-6)  # bf16 output rounding
    assert rel(host(evidence), host(want_ev)) <= close
    assert rel(host(g_scale), host(want_gs)) <= max(close, 1e-5)
    assert rel(host(g_bias), host(want_gb)) <= 1e-6
    # and against the oracle
    want = oracle.packed_transpose(dy.float().cpu(), bits.cpu(), columns, scale.cpu())
    assert rel(host(dx), like(want, dtype)) <= (1e-5 if dtype == torch.float32 else 1e-3)
    assert kernels.wait_timeouts() == 0
