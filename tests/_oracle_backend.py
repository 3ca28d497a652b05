"""The CPU oracle dressed as the kernel namespace, for host-logic tests.

``install(monkeypatch)`` replaces the functions of ``qste_b200.kernels`` with
versions that run the oracle on CPU torch tensors.  It lets the surface state
machine, the optimizer bookkeeping and the multi-rank reducers be exercised on a
machine without a GPU.  It is test infrastructure: the package itself has no CPU
path and never imports this file.
"""

from __future__ import annotations

import numpy as np
import torch

import oracle


def _t(array, like=None, dtype=None):
    tensor = torch.from_numpy(np.ascontiguousarray(array))
    return tensor if dtype is None else tensor.to(dtype)


def unpack_rows(packed, columns, *, dtype=None):
    return _t(oracle.unpack_rows(packed, columns)).to(dtype or torch.float32)


def unpack_bits(packed, columns, *, dtype=None):
    return _t(oracle.unpack_bits(packed, columns)).to(dtype or torch.float32)


def pack_bits(mask):
    return _t(oracle.pack_bits(mask.to(torch.uint8)))


def apply_bits(values, packed, columns):
    return _t(oracle.apply_bits(values.float(), packed, columns)).to(values.dtype)


def pack_affine_rows(values):
    packed, offset, scale = oracle.pack_affine_rows(values.float())
    return _t(packed), _t(offset), _t(scale)


def pack_coordinate(coordinate):
    # Surface.__init__ sends a host matrix through the current CUDA device when there is one
    # (the product has no CPU kernel); under this backend that tensor comes back to the host
    return _t(oracle.pack_coordinate(coordinate.cpu())).to(coordinate.device)


def packed_linear_affine(inputs, packed, scale, bias, columns):
    out = oracle.packed_linear_affine(inputs.float(), packed, scale.detach().float(),
                                      None if bias is None else bias.detach().float(), columns)
    return _t(out).to(inputs.dtype)


def packed_transpose(inputs, packed, columns, row_scale=None):
    out = oracle.packed_transpose(inputs.float(), packed, columns,
                                  None if row_scale is None else row_scale.detach().float())
    return _t(out).to(inputs.dtype)


def evidence_from_packed(grad, packed, columns, row_scale=None):
    return _t(oracle.evidence_from_packed(grad.float(), packed, columns,
                                          None if row_scale is None else row_scale.detach().float()))


def packed_row_inner(matrix, packed, columns):
    return _t(oracle.packed_row_inner(matrix.float(), packed, columns)).to(matrix.dtype)


def packed_embedding(ids, packed, scale, columns):
    return _t(oracle.packed_embedding(ids.long(), packed, scale.detach().float(), columns)).to(scale.dtype)


def linear_backward_evidence(grad, act_bits, aux, columns, weight_bits, weight_scale, *, want_bias=False):
    aux = aux.float()
    evidence = oracle.decoded_evidence(grad.float(), act_bits, aux[0], aux[1], columns)
    g_scale = oracle.packed_row_inner(evidence, weight_bits, columns)
    evidence = evidence * weight_scale.detach().float().numpy()[:, None]
    g_bias = grad.float().sum(dim=0) if want_bias else None
    return _t(evidence), _t(g_scale), g_bias


def linear_backward(grad, weight_bits, weight_scale, columns, act_bits, aux, *, want_bias=False, want_input=True,
                    evidence_ready=None):
    del evidence_ready  # a CUDA event; CPU tensors never carry one
    grad_input = packed_transpose(grad, weight_bits, columns, row_scale=weight_scale) if want_input else None
    evidence, g_scale, g_bias = linear_backward_evidence(grad, act_bits, aux, columns, weight_bits,
                                                         weight_scale, want_bias=want_bias)
    return grad_input, evidence, g_scale, g_bias


def coordinate_update(gradient, coordinate, packed, moment_q, moment_scale, row_v, col_v, *, beta1,
                      beta2, update_clip, coordinate_lr, block_size, seed, step, flips=None,
                      update_enabled=None):
    if update_enabled is not None and int(update_enabled) == 0:
        return 0 if flips is None else flips.zero_()
    scratch = np.ascontiguousarray(gradient.detach().float().numpy()).copy()
    count = oracle.coordinate_update(
        scratch, coordinate.numpy(), packed.numpy(), moment_q.numpy(), moment_scale.numpy(),
        row_v.numpy(), col_v.numpy(), beta1=beta1, beta2=beta2, update_clip=update_clip,
        coordinate_lr=coordinate_lr, block_size=block_size, seed=seed, step=int(step))
    if flips is not None:
        flips.fill_(count)
        return flips
    return count


_NAMES = (
    "unpack_rows", "unpack_bits", "pack_bits", "apply_bits", "pack_affine_rows", "pack_coordinate",
    "packed_linear_affine", "packed_transpose", "evidence_from_packed", "packed_row_inner",
    "packed_embedding", "linear_backward", "linear_backward_evidence", "coordinate_update",
)


def install(monkeypatch=None):
    from qste_b200 import kernels

    for name in _NAMES:
        if monkeypatch is not None:
            monkeypatch.setattr(kernels, name, globals()[name])
        else:
            setattr(kernels, name, globals()[name])
