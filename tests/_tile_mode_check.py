"""Run by test_gpu_kernels.py in a child process, because the GEMM's tile mode is chosen from
environment variables that the library reads once: checks the three packed-sign GEMMs on shapes large
enough for 256-row tiles against the CPU oracle (128 sampled rows of every output) and, over the
whole output, against the CUDA-core kernel (itself oracle-checked elsewhere), and prints OK."""

import os
import sys
from contextlib import contextmanager
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import oracle  # noqa: E402
from qste_b200 import kernels  # noqa: E402


@contextmanager
def forced_path(name):
    saved = os.environ.get("QSTE_B200_PATH")
    os.environ["QSTE_B200_PATH"] = name
    try:
        yield
    finally:
        if saved is None:
            os.environ.pop("QSTE_B200_PATH", None)
        else:
            os.environ["QSTE_B200_PATH"] = saved


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


def against_oracle(got, want, what):
    want = torch.from_numpy(np.ascontiguousarray(want))
    if got.dtype != torch.float32:
        want = want.to(got.dtype)  # like for like: the oracle's fp32 result rounded as the kernel rounds
    error = rel(got.cpu(), want)
    assert error <= 1e-3, (what, error)


def oracle_checks(x, dy, bits, scale, bias, columns, y, dx, fused, saved, generator):
    """128 sampled rows of Y, dX, the evidence and the scale gradient against the oracle."""

    samples, rows = dy.shape
    act_bits, act_offset, act_scale = (t.cpu().numpy() for t in saved)
    tokens = torch.randperm(samples, generator=generator)[:128]
    outputs = torch.randperm(rows, generator=generator)[:128]
    xs, dys, bits_host, scale_host = x.cpu()[tokens].float(), dy.cpu().float(), bits.cpu(), scale.cpu()
    against_oracle(y[tokens.to(y.device)], oracle.packed_linear_affine(xs, bits_host, scale_host, bias.cpu(), columns), "forward")
    if dx is not None:
        against_oracle(dx[tokens.to(y.device)], oracle.packed_transpose(dys[tokens], bits_host, columns, scale_host), "dX")
    grad = dys[:, outputs].contiguous()
    plain = oracle.evidence_from_packed(grad, act_bits, columns, act_scale)
    decoded = plain.astype(np.float64) + (grad.double().t().numpy() @ act_offset.astype(np.float64))[:, None]
    against_oracle(fused[0][outputs.to(y.device)], (decoded * scale_host[outputs].double().numpy()[:, None]).astype(np.float32), "evidence")
    against_oracle(fused[1][outputs.to(y.device)],
                   oracle.packed_row_inner(decoded.astype(np.float32), bits_host[outputs].contiguous(), columns), "scale gradient")


def stress_short_items(device, generator):
    """Work items of a single k-block on 256-row tiles: the hand-out of items runs as far ahead of
    the epilogue warps as its ring allows, every launch.  A reader that took a refilled slot for
    its own once made such launches run into the bounded waits; results must also repeat."""
    samples, rows, columns = 16, 14336, 4096
    x = torch.randn(samples, columns, generator=generator).to(device, torch.bfloat16)
    dy = torch.randn(samples, rows, generator=generator).to(device, torch.bfloat16)
    bits = torch.randint(0, 256, (rows, columns // 8), generator=generator, dtype=torch.int32).to(torch.uint8).to(device)
    scale = (torch.rand(rows, generator=generator) * 0.04 + 0.01).to(device)
    act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
    aux = torch.stack((act_offset, act_scale))
    with forced_path("simt"):
        reference = kernels.linear_backward_evidence(dy.float(), act_bits, aux, columns, bits, scale)
    first = None
    for _ in range(100):
        fused = kernels.linear_backward_evidence(dy, act_bits, aux, columns, bits, scale)
        evidence = fused[0].clone()
        if first is None:
            first = evidence
            assert rel(evidence, reference[0]) <= 1e-3, ("short items", rel(evidence, reference[0]))
        assert torch.equal(evidence, first)
    torch.cuda.synchronize()
    assert kernels.wait_timeouts() == 0
    # forward with a contraction of one and of two k-blocks
    for width in (64, 128):
        xs = torch.randn(9472, width, generator=generator).to(device, torch.bfloat16)
        bs = torch.randint(0, 256, (4096, width // 8), generator=generator, dtype=torch.int32).to(torch.uint8).to(device)
        ss = (torch.rand(4096, generator=generator) * 0.04 + 0.01).to(device)
        for _ in range(20):
            y = kernels.packed_linear_affine(xs, bs, ss, None, width)
        with forced_path("simt"):
            y_ref = kernels.packed_linear_affine(xs.float(), bs, ss, None, width)
        assert rel(y, y_ref) <= 4e-3, ("forward, short contraction", width, rel(y, y_ref))


def main():
    device = "cuda"
    generator = torch.Generator().manual_seed(11)
    for samples, rows, columns in [(2600, 4104, 1024), (1536, 4352, 640)]:
        x = torch.randn(samples, columns, generator=generator).to(device, torch.bfloat16)
        dy = torch.randn(samples, rows, generator=generator).to(device, torch.bfloat16)
        bits = torch.randint(0, 256, (rows, columns // 8), generator=generator, dtype=torch.int32).to(torch.uint8).to(device)
        scale = (torch.rand(rows, generator=generator) * 0.04 + 0.01).to(device)
        bias = torch.randn(rows, generator=generator).to(device)
        y = kernels.packed_linear_affine(x, bits, scale, bias, columns)
        act_bits, act_offset, act_scale = kernels.pack_affine_rows(x)
        aux = torch.stack((act_offset, act_scale))
        if rows % 64 == 0:
            dx = kernels.packed_transpose(dy, bits, columns, scale)
        fused = kernels.linear_backward_evidence(dy, act_bits, aux, columns, bits, scale, want_bias=True)
        oracle_checks(x, dy, bits, scale, bias, columns, y, dx if rows % 64 == 0 else None, fused,
                      (act_bits, act_offset, act_scale), generator)
        with forced_path("simt"):
            y_ref = kernels.packed_linear_affine(x.float(), bits, scale, bias, columns)
            assert rel(y, y_ref) <= 4e-3, ("forward", rel(y, y_ref))  # bf16 output rounding
            if rows % 64 == 0:
                dx_ref = kernels.packed_transpose(dy.float(), bits, columns, scale)
                assert rel(dx, dx_ref) <= 4e-3, ("dx", rel(dx, dx_ref))
            fused_ref = kernels.linear_backward_evidence(dy.float(), act_bits, aux, columns, bits, scale, want_bias=True)
        assert rel(fused[0], fused_ref[0]) <= 1e-3, ("evidence", rel(fused[0], fused_ref[0]))
        assert rel(fused[1], fused_ref[1]) <= 1e-3, ("g_scale", rel(fused[1], fused_ref[1]))
    if os.environ.get("QSTE_B200_TC_TALL_ANY"):
        stress_short_items(device, generator)
    assert kernels.wait_timeouts() == 0, kernels.first_wait_timeout()
    assert kernels.first_wait_timeout() is None
    print("OK")


if __name__ == "__main__":
    main()
