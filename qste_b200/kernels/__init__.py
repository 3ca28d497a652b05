"""Kernel layer: the reference's ``qste.kernels`` call surface over one backend.

Every function here has the signature of its counterpart in the reference
(``src/qste/kernels/loader.py:247-368``) and does one thing: validate, allocate
the outputs with torch, and enqueue the hand-written sm_100a kernels of
``libqste_b200.so`` on the current CUDA stream through its C ABI
(``include/qste_b200.h``).

There is exactly one backend.  Tensors must live on a CUDA device; a CPU tensor,
a missing library or a non-B200 device raises -- nothing falls back to torch or
to the CPU.
"""

from __future__ import annotations

import contextlib
import ctypes
import os

import torch
from torch import Tensor

from . import _cabi, stream
from .device import DeviceProfile, profile, warm

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
PATH_AUTO, PATH_SIMT, PATH_TENSOR, PATH_STREAM = 0, 1, 2, 3
_PATH_NAMES = {"auto": PATH_AUTO, "simt": PATH_SIMT, "tensor": PATH_TENSOR, "stream": PATH_STREAM}


def _path() -> int:
    """``QSTE_B200_PATH=auto|simt|tensor|stream`` pins the GEMM implementation (for tests)."""

    name = os.environ.get("QSTE_B200_PATH", "auto").strip().lower()
    if name not in _PATH_NAMES:
        raise ValueError("QSTE_B200_PATH must be one of " + ", ".join(_PATH_NAMES))
    return _PATH_NAMES[name]


# -- plumbing ---------------------------------------------------------------------

def _need_cuda(tensor: Tensor, what: str) -> None:
    if tensor.device.type != "cuda":
        raise RuntimeError(
            f"qste_b200 {what}: expected a CUDA tensor, got one on '{tensor.device}'. "
            "This build has a single backend (sm_100a CUDA); there is no CPU path."
        )


def _dtype(tensor: Tensor, what: str) -> int:
    try:
        return _DTYPES[tensor.dtype]
    except KeyError:
        raise RuntimeError(f"qste_b200 {what}: unsupported dtype {tensor.dtype}") from None


def _ptr(tensor: Tensor | None, current: int | None = None):
    """The device address of ``tensor``.  Every pointer the library receives goes through here,
    so this is also where a tensor on the host (a module that was converted but never moved to
    the GPU, say) is refused instead of being handed to a kernel as if it were device memory.
    ``current``: the current device's index, for callers that looked it up once for the call."""

    if tensor is None or tensor.numel() == 0:
        return None
    if tensor.device.type != "cuda":
        raise RuntimeError(
            f"qste_b200: expected every tensor of the call on the GPU, got one on '{tensor.device}' "
            f"(shape {tuple(tensor.shape)}, {tensor.dtype}); move the converted module with .to(device)."
        )
    if current is None:
        current = torch.cuda.current_device()
    if tensor.device.index is not None and tensor.device.index != current:
        raise RuntimeError(
            f"qste_b200: tensor on cuda:{tensor.device.index} passed while cuda:{current} is the current "
            "device; kernels run on the current device's stream."
        )
    return ctypes.c_void_p(tensor.data_ptr())


_NO_SWITCH = contextlib.nullcontext()


def _on(device: torch.device):
    """Context that makes `device` current for the calls inside; nothing at all when it already
    is (the common case, and a device switch costs more host time than a small kernel runs)."""

    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_workspaces: dict[tuple[int, int], Tensor] = {}


def _workspace(device: torch.device, nbytes: int, stream: int | None = None) -> Tensor:
    """A zero-initialised scratch buffer per (device, stream), grown on demand.  ``stream``: the
    current stream's handle, for callers that looked it up once for the call."""

    nbytes = max(int(nbytes), 256)
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream if stream is None else stream)
    held = _workspaces.get(key)
    if held is None or held.numel() < nbytes:
        grown = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        if held is not None:
            # the first 256 bytes are the diagnostics header (wait counters, first give-up
            # site, the work-item counter, which is zero between launches): it outlives the buffer
            grown[:256].copy_(held[:256])
        held = _workspaces[key] = grown
    return held


def wait_timeouts(device=None) -> int:
    """How many bounded device-side waits gave up in calls that used this stream's
    workspace (0 in a healthy run)."""

    device = torch.device(device if device is not None else "cuda")
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    held = _workspaces.get(key)
    if held is None:
        return 0
    return int(held[:8].view(torch.int64).item())


def check_waits(device=None) -> None:
    """Raise if a bounded device-side wait gave up in any call on `device` so far, on
    whichever stream it ran: its output is then not to be trusted.  One 8-byte read per
    workspace (one per stream that called a kernel); QSTEOptimizer.step() calls this where
    it synchronises anyway."""

    device = torch.device(device if device is not None else "cuda")
    index = device.index if device.index is not None else torch.cuda.current_device()
    for (held_device, _), held in list(_workspaces.items()):
        if held_device != index:
            continue
        if int(held[:8].view(torch.int64).item()):
            word = int(held[200:208].view(torch.int64).item())
            raise RuntimeError(
                f"qste_b200: {int(held[:8].view(torch.int64).item())} bounded wait(s) inside a GEMM kernel gave up on "
                f"cuda:{index} (first at csrc/gemm_tc.cu line {word >> 32}, block {(word >> 16) & 0xFFFF}, "
                f"thread {word & 0xFFFF}); the results of that launch are incomplete.")


def first_wait_timeout(device=None) -> dict | None:
    """Where the first bounded wait gave up, for calls that used this stream's workspace:
    ``{"line", "block", "thread", "warp"}`` (the source line of the wait in
    ``csrc/gemm_tc.cu``, and the CTA and thread that was waiting), or ``None`` in a
    healthy run.  The kernel writes it once, beside the counter of ``wait_timeouts``."""

    device = torch.device(device if device is not None else "cuda")
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    held = _workspaces.get(key)
    if held is None or held.numel() < 208:
        return None
    word = int(held[200:208].view(torch.int64).item())
    if word == 0:
        return None
    thread = word & 0xFFFF
    return {"line": word >> 32, "block": (word >> 16) & 0xFFFF, "thread": thread, "warp": thread // 32}


def last_forward_kernel() -> str:
    """The kernel family this thread's last ``packed_linear_affine`` ran: ``"lut"`` (1-2 tokens),
    ``"mma"`` (3-32 tokens of a 16-bit type), ``"stream"``, ``"tensor"`` (tcgen05) or ``"simt"``."""

    return _cabi.load().qste_b200_last_forward_kernel().decode()


def _check_packed(packed: Tensor, columns: int, what: str) -> None:
    if packed.dtype != torch.uint8 or packed.dim() != 2:
        raise RuntimeError(f"{what}: packed signs must be a rank-2 uint8 tensor")
    if packed.shape[1] != (int(columns) + 7) // 8:
        raise RuntimeError(f"{what}: packed sign width does not match the column count")


def _f32(tensor: Tensor) -> Tensor:
    return tensor.detach().to(torch.float32).contiguous()


# -- packing ----------------------------------------------------------------------

def unpack_rows(packed: Tensor, columns: int, *, dtype: torch.dtype | None = None) -> Tensor:
    """Dense +-1 view of packed signs (loader.py:247-253)."""

    return _unpack(packed, columns, dtype or torch.float32, zero_one=0)


def unpack_bits(packed: Tensor, columns: int, *, dtype: torch.dtype | None = None) -> Tensor:
    """Dense 0/1 view of packed bits (loader.py:270-275)."""

    return _unpack(packed, columns, dtype or torch.float32, zero_one=1)


def _unpack(packed: Tensor, columns: int, dtype: torch.dtype, zero_one: int) -> Tensor:
    _need_cuda(packed, "unpack")
    _check_packed(packed, columns, "unpack")
    if dtype not in _DTYPES:
        return _unpack(packed, columns, torch.float32, zero_one).to(dtype)
    packed = packed.contiguous()
    rows = packed.shape[0]
    out = torch.empty(rows, int(columns), dtype=dtype, device=packed.device)
    with _on(packed.device):
        _cabi.check(_cabi.load().qste_b200_unpack_rows(
            _ptr(packed), rows, int(columns), _ptr(out), _DTYPES[dtype], zero_one,
            _stream(packed.device)), "unpack_rows")
    return out


def pack_bits(mask: Tensor) -> Tensor:
    """One bit per element of a boolean matrix, least significant bit first (loader.py:256-260)."""

    _need_cuda(mask, "pack_bits")
    if mask.dim() != 2 or mask.dtype != torch.bool:
        raise RuntimeError("pack_bits expects a rank-2 bool tensor")
    mask = mask.contiguous()
    rows, columns = mask.shape
    packed = torch.empty(rows, (columns + 7) // 8, dtype=torch.uint8, device=mask.device)
    with _on(mask.device):
        _cabi.check(_cabi.load().qste_b200_pack_bits(
            _ptr(mask), rows, columns, _ptr(packed), _stream(mask.device)), "pack_bits")
    return packed


def apply_bits(values: Tensor, packed: Tensor, columns: int) -> Tensor:
    """``values`` where the bit is set, zero where it is not (loader.py:263-267)."""

    _need_cuda(values, "apply_bits")
    _check_packed(packed, columns, "apply_bits")
    if values.dim() != 2 or values.shape[0] != packed.shape[0] or values.shape[1] != int(columns):
        raise RuntimeError("apply_bits shape mismatch")
    if values.dtype not in _DTYPES:
        return apply_bits(values.float(), packed, columns).to(values.dtype)
    values = values.contiguous()
    packed = packed.contiguous()
    out = torch.empty_like(values)
    with _on(values.device):
        _cabi.check(_cabi.load().qste_b200_apply_bits(
            _ptr(values), _DTYPES[values.dtype], _ptr(packed), values.shape[0], int(columns),
            _ptr(out), _stream(values.device)), "apply_bits")
    return out


def pack_affine_rows(values: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    """One-bit affine encoding of each row: bits of the centred sign, offset, scale
    (loader.py:278-282).  Bits match the reference's CPU kernel exactly."""

    _need_cuda(values, "pack_affine_rows")
    if values.dim() != 2:
        raise RuntimeError("pack_affine_rows expects a rank-2 tensor")
    if values.dtype not in _DTYPES:
        values = values.float()
    values = values.contiguous()
    rows, columns = values.shape
    device = values.device
    packed = torch.empty(rows, (columns + 7) // 8, dtype=torch.uint8, device=device)
    offset = torch.empty(rows, dtype=torch.float32, device=device)
    scale = torch.empty(rows, dtype=torch.float32, device=device)
    with _on(device):
        _cabi.check(_cabi.load().qste_b200_pack_affine_rows(
            _ptr(values), _DTYPES[values.dtype], rows, columns, _ptr(packed), _ptr(offset),
            _ptr(scale), _stream(device)), "pack_affine_rows")
    return packed, offset, scale


def pack_coordinate(coordinate: Tensor) -> Tensor:
    """Sign bits of an int8 coordinate matrix (loader.py:285-289)."""

    _need_cuda(coordinate, "pack_coordinate")
    if coordinate.dim() != 2 or coordinate.dtype != torch.int8:
        raise RuntimeError("pack_coordinate expects a rank-2 int8 tensor")
    coordinate = coordinate.contiguous()
    rows, columns = coordinate.shape
    packed = torch.empty(rows, (columns + 7) // 8, dtype=torch.uint8, device=coordinate.device)
    with _on(coordinate.device):
        _cabi.check(_cabi.load().qste_b200_pack_coordinate(
            _ptr(coordinate), rows, columns, _ptr(packed), _stream(coordinate.device)),
            "pack_coordinate")
    return packed


# -- projections -------------------------------------------------------------------

def packed_linear_affine(inputs: Tensor, packed: Tensor, scale: Tensor, bias: Tensor | None,
                         columns: int) -> Tensor:
    """``(x @ sign^T) * scale + bias`` in the dtype of ``inputs`` (loader.py:292-296)."""

    _need_cuda(inputs, "packed_linear_affine")
    _check_packed(packed, columns, "packed_linear_affine")
    columns = int(columns)
    if inputs.shape[-1] != columns:
        raise RuntimeError("activation width mismatch")
    rows = packed.shape[0]
    if scale.numel() != rows:
        raise RuntimeError("scale must have one entry per output row")
    if bias is not None and bias.numel() != rows:
        raise RuntimeError("bias must have one entry per output row")
    if inputs.dtype not in _DTYPES:
        return packed_linear_affine(inputs.float(), packed, scale, bias, columns).to(inputs.dtype)
    device = inputs.device
    flat = inputs.reshape(-1, columns).contiguous()
    packed = packed.contiguous()
    scale32 = _f32(scale)
    bias32 = None if bias is None else _f32(bias)
    samples = flat.shape[0]
    out = torch.empty(samples, rows, dtype=inputs.dtype, device=device)
    code = _DTYPES[inputs.dtype]
    path = _path()
    library = _cabi.load()
    with _on(device):
        # the current device and stream are looked up once: for a batch of one the host side of this
        # call costs several times what the kernel takes
        current = torch.cuda.current_device()
        stream = torch.cuda.current_stream(device).cuda_stream
        need = library.qste_b200_packed_linear_affine_workspace(samples, rows, columns, code, path)
        workspace = _workspace(device, need, stream)
        _cabi.check(library.qste_b200_packed_linear_affine(
            _ptr(flat, current), code, samples, _ptr(packed, current), _ptr(scale32, current), _ptr(bias32, current),
            rows, columns, _ptr(out, current), code, path, _ptr(workspace, current), workspace.numel(),
            ctypes.c_void_p(stream)), "packed_linear_affine")
    return out.view(*inputs.shape[:-1], rows)


def packed_transpose(inputs: Tensor, packed: Tensor, columns: int,
                     row_scale: Tensor | None = None) -> Tensor:
    """``(x * row_scale) @ sign``, the input gradient of a binary Linear (loader.py:299-303)."""

    _need_cuda(inputs, "packed_transpose")
    _check_packed(packed, columns, "packed_transpose")
    columns = int(columns)
    rows = packed.shape[0]
    if inputs.shape[-1] != rows:
        raise RuntimeError("transpose width mismatch")
    if row_scale is not None and row_scale.numel() != rows:
        raise RuntimeError("transpose row scale must have one entry per packed row")
    if inputs.dtype not in _DTYPES:
        return packed_transpose(inputs.float(), packed, columns, row_scale).to(inputs.dtype)
    device = inputs.device
    flat = inputs.reshape(-1, rows).contiguous()
    packed = packed.contiguous()
    scale32 = None if row_scale is None else _f32(row_scale)
    samples = flat.shape[0]
    out = torch.empty(samples, columns, dtype=inputs.dtype, device=device)
    code = _DTYPES[inputs.dtype]
    path = _path()
    library = _cabi.load()
    with _on(device):
        need = library.qste_b200_packed_transpose_workspace(samples, rows, columns, code, path)
        workspace = _workspace(device, need)
        _cabi.check(library.qste_b200_packed_transpose(
            _ptr(flat), code, samples, _ptr(packed), _ptr(scale32), rows, columns, _ptr(out), code,
            path, _ptr(workspace), workspace.numel(), _stream(device)), "packed_transpose")
    return out.view(*inputs.shape[:-1], columns)


def evidence_from_packed(grad: Tensor, packed: Tensor, columns: int,
                         row_scale: Tensor | None = None) -> Tensor:
    """``(grad * row_scale)^T @ sign(x)`` in fp32, activations given as bits (loader.py:306-312)."""

    _need_cuda(grad, "evidence_from_packed")
    _check_packed(packed, columns, "evidence_from_packed")
    columns = int(columns)
    if grad.dim() != 2:
        raise RuntimeError("evidence grad must be a rank-2 tensor")
    if grad.shape[0] != packed.shape[0]:
        raise RuntimeError("evidence grad and packed activations disagree on sample count")
    samples, rows = grad.shape
    if row_scale is not None and row_scale.numel() != samples:
        raise RuntimeError("evidence row scale must have one entry per sample")
    if grad.dtype not in _DTYPES:
        grad = grad.float()
    device = grad.device
    grad = grad.contiguous()
    packed = packed.contiguous()
    scale32 = None if row_scale is None else _f32(row_scale)
    evidence = torch.empty(rows, columns, dtype=torch.float32, device=device)
    if samples == 0:
        return evidence.zero_()
    code = _DTYPES[grad.dtype]
    path = _path()
    library = _cabi.load()
    with _on(device):
        need = library.qste_b200_evidence_from_packed_workspace(samples, rows, columns, code, path)
        workspace = _workspace(device, need)
        _cabi.check(library.qste_b200_evidence_from_packed(
            _ptr(grad), code, samples, rows, _ptr(packed), _ptr(scale32), columns, _ptr(evidence),
            path, _ptr(workspace), workspace.numel(), _stream(device)), "evidence_from_packed")
    return evidence


def linear_backward_evidence(grad: Tensor, act_bits: Tensor, aux: Tensor, columns: int,
                             weight_bits: Tensor, weight_scale: Tensor, *, want_bias: bool = False):
    """Everything the Linear backward derives from ``grad^T @ x`` in one call.

    Returns ``(evidence, grad_scale, grad_bias)``: the coordinate evidence already
    multiplied by the row scale, the exact gradient of the row scale, and (when asked
    for) the column sum of ``grad``, all fp32.  Equivalent to
    ``decoded_evidence`` + ``packed_row_inner`` + the in-place scaling of
    ``functional.py:186-193`` in the reference, with the offset correction formed in
    fp32.  No counterpart in the reference's kernel namespace.
    """

    _need_cuda(grad, "linear_backward_evidence")
    columns = int(columns)
    _check_packed(act_bits, columns, "linear_backward_evidence")
    _check_packed(weight_bits, columns, "linear_backward_evidence")
    if grad.dim() != 2 or grad.shape[0] != act_bits.shape[0]:
        raise RuntimeError("evidence grad and packed activations disagree on sample count")
    samples, rows = grad.shape
    if weight_bits.shape[0] != rows or weight_scale.numel() != rows:
        raise RuntimeError("weight bits / scale do not match the gradient width")
    if aux.shape != (2, samples):
        raise RuntimeError("aux must be the [2, samples] offset/scale tensor")
    if grad.dtype not in _DTYPES:
        grad = grad.float()
    device = grad.device
    grad = grad.contiguous()
    aux32 = _f32(aux)
    scale32 = _f32(weight_scale)
    act_bits = act_bits.contiguous()
    weight_bits = weight_bits.contiguous()
    evidence = torch.empty(rows, columns, dtype=torch.float32, device=device)
    g_scale = torch.empty(rows, dtype=torch.float32, device=device)
    g_bias = torch.empty(rows, dtype=torch.float32, device=device) if want_bias else None
    code = _DTYPES[grad.dtype]
    path = _path()
    library = _cabi.load()
    with _on(device):
        need = library.qste_b200_linear_backward_evidence_workspace(samples, rows, columns, code, path)
        workspace = _workspace(device, need)
        _cabi.check(library.qste_b200_linear_backward_evidence(
            _ptr(grad), code, samples, rows, _ptr(act_bits), _ptr(aux32), columns,
            _ptr(weight_bits), _ptr(scale32), _ptr(evidence), _ptr(g_scale), _ptr(g_bias), path,
            _ptr(workspace), workspace.numel(), _stream(device)), "linear_backward_evidence")
    return evidence, g_scale, g_bias


_backward_reserve = 0


def set_backward_reserve(count: int) -> int:
    """How many SMs the GEMMs of :func:`linear_backward` leave free, for a collective that runs
    beside backward on another stream (``distributed.mean_evidence(overlap=True)`` sets it).
    Forward GEMMs never reserve any: no collective is in flight while they run.  Returns the
    previous value."""

    global _backward_reserve
    previous, _backward_reserve = _backward_reserve, max(0, int(count))
    return previous


def linear_backward(grad: Tensor, weight_bits: Tensor, weight_scale: Tensor, columns: int,
                    act_bits: Tensor, aux: Tensor, *, want_bias: bool = False, want_input: bool = True,
                    evidence_ready: "torch.cuda.Event | None" = None):
    """The whole backward of a converted Linear in one library call.

    Returns ``(grad_input, evidence, grad_scale, grad_bias)``: ``grad_input`` in the dtype
    of ``grad`` (what ``packed_transpose`` returns), the rest as
    :func:`linear_backward_evidence` returns them.  One pass over ``grad`` yields the bias
    gradient, the offset correction and the gradient's largest magnitude, and both GEMMs
    share one fp16 re-encoding of a bf16 gradient.  The evidence product runs first:
    ``evidence_ready``, when given, is recorded on the current stream once evidence, grad_scale
    and grad_bias are complete and before the dX product is enqueued, so a reduction or an
    update on another stream can wait for it and run beside dX.  ``want_input=False`` skips dX
    (``grad_input`` is then ``None``).  No counterpart in the reference's kernel namespace (it is
    ``QSTELinearFn.backward``, functional.py:173-194, as one call).
    """

    _need_cuda(grad, "linear_backward")
    columns = int(columns)
    _check_packed(act_bits, columns, "linear_backward")
    _check_packed(weight_bits, columns, "linear_backward")
    if grad.dim() != 2 or grad.shape[0] != act_bits.shape[0]:
        raise RuntimeError("gradient and packed activations disagree on sample count")
    samples, rows = grad.shape
    if weight_bits.shape[0] != rows or weight_scale.numel() != rows:
        raise RuntimeError("weight bits / scale do not match the gradient width")
    if aux.shape != (2, samples):
        raise RuntimeError("aux must be the [2, samples] offset/scale tensor")
    if grad.dtype not in _DTYPES:
        grad = grad.float()
    device = grad.device
    grad = grad.contiguous()
    aux32 = _f32(aux)
    scale32 = _f32(weight_scale)
    act_bits = act_bits.contiguous()
    weight_bits = weight_bits.contiguous()
    grad_input = torch.empty(samples, columns, dtype=grad.dtype, device=device) if want_input else None
    evidence = torch.empty(rows, columns, dtype=torch.float32, device=device)
    g_scale = torch.empty(rows, dtype=torch.float32, device=device)
    g_bias = torch.empty(rows, dtype=torch.float32, device=device) if want_bias else None
    if samples == 0:
        evidence.zero_()
        g_scale.zero_()
        if g_bias is not None:
            g_bias.zero_()
        if evidence_ready is not None:
            evidence_ready.record()
        return grad_input, evidence, g_scale, g_bias
    code = _DTYPES[grad.dtype]
    library = _cabi.load()
    event = None
    if evidence_ready is not None:
        if not evidence_ready.cuda_event:
            evidence_ready.record()  # torch creates the CUDA event at its first record
        event = ctypes.c_void_p(evidence_ready.cuda_event)
    with _on(device):
        reserve = _backward_reserve
        if reserve:
            library.qste_b200_set_reserved_sms(reserve)
        try:
            need = library.qste_b200_linear_backward_workspace(samples, rows, columns, code)
            workspace = _workspace(device, need)
            _cabi.check(library.qste_b200_linear_backward_staged(
                _ptr(grad), code, samples, rows, _ptr(weight_bits), _ptr(scale32), columns, _ptr(act_bits),
                _ptr(aux32), _ptr(grad_input), code, _ptr(evidence), _ptr(g_scale), _ptr(g_bias), event,
                _ptr(workspace), workspace.numel(), _stream(device)), "linear_backward")
        finally:
            if reserve:
                library.qste_b200_set_reserved_sms(0)
    return grad_input, evidence, g_scale, g_bias


def packed_row_inner(matrix: Tensor, packed: Tensor, columns: int) -> Tensor:
    """``out[i] = sum_j matrix[i, j] * sign[i, j]`` (loader.py:315-319)."""

    _need_cuda(matrix, "packed_row_inner")
    _check_packed(packed, columns, "packed_row_inner")
    columns = int(columns)
    if matrix.dim() != 2 or matrix.shape[0] != packed.shape[0] or matrix.shape[1] != columns:
        raise RuntimeError("row inner shape mismatch")
    source = matrix if matrix.dtype == torch.float32 else matrix.float()
    source = source.contiguous()
    packed = packed.contiguous()
    out = torch.empty(source.shape[0], dtype=torch.float32, device=matrix.device)
    with _on(matrix.device):
        _cabi.check(_cabi.load().qste_b200_packed_row_inner(
            _ptr(source), _ptr(packed), source.shape[0], columns, _ptr(out),
            _stream(matrix.device)), "packed_row_inner")
    return out if matrix.dtype == torch.float32 else out.to(matrix.dtype)


def packed_embedding(ids: Tensor, packed: Tensor, scale: Tensor, columns: int) -> Tensor:
    """Rows of the binary matrix times their scale, gathered by id (loader.py:322-326)."""

    _need_cuda(packed, "packed_embedding")
    _check_packed(packed, columns, "packed_embedding")
    columns = int(columns)
    rows = packed.shape[0]
    if scale.numel() != rows:
        raise RuntimeError("embedding scale shape mismatch")
    device = packed.device
    flat = ids.to(device=device, dtype=torch.int64).reshape(-1).contiguous()
    out_dtype = scale.dtype if scale.dtype in _DTYPES else torch.float32
    out = torch.empty(flat.numel(), columns, dtype=out_dtype, device=device)
    bad = torch.zeros(1, dtype=torch.int32, device=device)
    with _on(device):
        _cabi.check(_cabi.load().qste_b200_packed_embedding(
            _ptr(flat), flat.numel(), _ptr(packed.contiguous()), _ptr(_f32(scale)), rows, columns,
            _ptr(out), _DTYPES[out_dtype], _ptr(bad), _stream(device)), "packed_embedding")
    if torch.cuda.is_current_stream_capturing():
        return out.view(*ids.shape, columns).to(scale.dtype)
    if int(bad.item()):
        raise RuntimeError("embedding id outside the vocabulary")
    return out.view(*ids.shape, columns).to(scale.dtype)


# -- packed activations -------------------------------------------------------------

SMOOTH_KINDS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "tanh": 3, "sigmoid": 4, "elu": 5, "celu": 6,
                "selu": 7, "softplus": 8, "mish": 9, "hardswish": 10}
_SMOOTH_MAX_COLUMNS = 51200  # the row's derivatives sit in shared memory as fp32


def smooth_supported(inputs: Tensor) -> bool:
    """Whether :func:`smooth_forward` takes this tensor (else the caller composes torch ops)."""

    return inputs.is_cuda and inputs.dtype in _DTYPES and inputs.dim() >= 1 and \
        0 < inputs.shape[-1] <= _SMOOTH_MAX_COLUMNS and inputs.numel() > 0


def smooth_forward(inputs: Tensor, kind: str, parameter: float = 1.0) -> tuple[Tensor, Tensor, Tensor]:
    """``(f(x), int8 derivative, fp32 row scale)`` of a smooth activation in one pass over
    ``x`` (rows are taken over the last dimension).  The forward half of the reference's
    ``_SmoothFn`` (src/qste/nn.py:483-502) as one kernel; no counterpart in its kernel namespace."""

    _need_cuda(inputs, "smooth_forward")
    code = _dtype(inputs, "smooth_forward")
    columns = inputs.shape[-1]
    flat = inputs.reshape(-1, columns).contiguous()
    rows = flat.shape[0]
    outputs = torch.empty_like(flat)
    derivative = torch.empty(rows, columns, dtype=torch.int8, device=flat.device)
    scale = torch.empty(rows, dtype=torch.float32, device=flat.device)
    with _on(flat.device):
        _cabi.check(_cabi.load().qste_b200_smooth_forward(
            _ptr(flat), code, rows, columns, SMOOTH_KINDS[kind], float(parameter), _ptr(outputs), _ptr(derivative),
            _ptr(scale), _stream(flat.device)), "smooth_forward")
    return outputs.view(inputs.shape), derivative, scale


def smooth_backward(grad: Tensor, derivative: Tensor, scale: Tensor) -> Tensor:
    """``grad * (derivative * scale)`` (src/qste/nn.py:504-507 of the reference) as one kernel."""

    _need_cuda(grad, "smooth_backward")
    rows, columns = derivative.shape
    if grad.numel() != rows * columns or scale.numel() != rows or derivative.dtype != torch.int8:
        raise RuntimeError("smooth_backward: gradient, derivative tape and scale do not match")
    if grad.dtype not in _DTYPES:
        return smooth_backward(grad.float(), derivative, scale).to(grad.dtype)
    flat = grad.reshape(rows, columns).contiguous()
    out = torch.empty_like(flat)
    with _on(flat.device):
        _cabi.check(_cabi.load().qste_b200_smooth_backward(
            _ptr(flat), _DTYPES[flat.dtype], _ptr(derivative.contiguous()), _ptr(_f32(scale)), rows, columns, _ptr(out),
            _stream(flat.device)), "smooth_backward")
    return out.view(grad.shape)


# -- optimizer --------------------------------------------------------------------

def _check_update_arguments(what, gradient, coordinate, packed, moment_q, moment_scale, row_v, col_v,
                            block_size, step, flips, update_enabled) -> int:
    """Everything either coordinate-update wrapper must know before a pointer is taken:
    devices, dtypes, shapes and contiguity of the in-place state (the conditions of the
    reference's TORCH_CHECKs, cpu.cpp:584-606, and cuda.py:1731-1732 for the block size).
    Shapes and dtypes are checked before devices, so a malformed call is refused the same way
    wherever its tensors live.  Returns the number of coordinates."""

    block_size = int(block_size)
    if block_size <= 0 or block_size & (block_size - 1):
        raise ValueError("momentum block size must be a positive power of two")
    if gradient.dtype != torch.float32 or gradient.dim() != 2:
        raise RuntimeError("evidence must be a rank-2 float32 tensor")
    if coordinate.dtype != torch.int8 or moment_q.dtype != torch.int8 or packed.dtype != torch.uint8:
        raise RuntimeError("coordinate/momentum/packed dtypes are wrong")
    if any(t.dtype != torch.float16 for t in (moment_scale, row_v, col_v)):
        raise RuntimeError("compact optimizer statistics must be float16")
    rows, columns = gradient.shape
    if coordinate.shape != gradient.shape or moment_q.shape != gradient.shape:
        raise RuntimeError("coordinate state shape mismatch")
    if packed.shape != (rows, (columns + 7) // 8):
        raise RuntimeError("packed sign shape mismatch")
    count = rows * columns
    blocks = (count + block_size - 1) // block_size
    if moment_scale.numel() != blocks:
        raise RuntimeError("momentum scale shape mismatch")
    if row_v.numel() != rows or col_v.numel() != columns:
        raise RuntimeError("factored statistics shape mismatch")
    for name, tensor in (("coordinate", coordinate), ("packed", packed), ("moment_q", moment_q),
                         ("moment_scale", moment_scale), ("row_v", row_v), ("col_v", col_v)):
        if not tensor.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous: it is updated in place")
        if tensor.device != gradient.device:
            raise RuntimeError(f"{name} is on {tensor.device}, the evidence on {gradient.device}")
    if torch.is_tensor(step) and (step.dtype != torch.int64 or step.device != gradient.device):
        raise RuntimeError("a tensor step must be an int64 scalar on the evidence's device")
    if update_enabled is not None and (update_enabled.dtype != torch.uint8 or update_enabled.device != gradient.device):
        raise RuntimeError("update_enabled must be a uint8 scalar tensor on the evidence's device")
    if flips is not None and (flips.dtype != torch.int64 or flips.numel() != 1 or flips.device != gradient.device):
        raise RuntimeError("flips must be an int64 scalar tensor on the evidence's device")
    _need_cuda(gradient, what)
    return count


def coordinate_update(gradient: Tensor, coordinate: Tensor, packed: Tensor, moment_q: Tensor,
                      moment_scale: Tensor, row_v: Tensor, col_v: Tensor, *, beta1: float,
                      beta2: float, update_clip: float, coordinate_lr: float, block_size: int,
                      seed: int, step, flips: Tensor | None = None,
                      update_enabled: Tensor | None = None):
    """One fused coordinate step, in place (loader.py:329-368).

    ``gradient`` is consumed as scratch.  With ``flips=None`` the flip count is
    returned as an ``int`` (one host synchronisation); pass a device int64 tensor to
    get it there instead, and device tensors for ``step`` (int64) and
    ``update_enabled`` (uint8) to keep the whole call free of host reads, which is
    what CUDA-graph capture needs (cuda.py:1705-1812 of the reference).
    """

    count = _check_update_arguments("coordinate_update", gradient, coordinate, packed, moment_q, moment_scale,
                                    row_v, col_v, block_size, step, flips, update_enabled)
    block_size = int(block_size)
    rows, columns = gradient.shape
    if count == 0:
        return 0 if flips is None else flips.zero_()
    device = gradient.device
    gradient = gradient if gradient.is_contiguous() else gradient.contiguous()
    step_tensor = step if torch.is_tensor(step) else None
    library = _cabi.load()
    with _on(device):
        need = library.qste_b200_coordinate_update_workspace(rows, columns, block_size)
        workspace = _workspace(device, need)
        _cabi.check(library.qste_b200_coordinate_update(
            _ptr(gradient), _ptr(coordinate), _ptr(packed), _ptr(moment_q), _ptr(moment_scale),
            _ptr(row_v), _ptr(col_v), rows, columns, float(beta1), float(beta2),
            float(update_clip), float(coordinate_lr), block_size, int(seed),
            0 if step_tensor is not None else int(step), _ptr(step_tensor), _ptr(update_enabled),
            _ptr(flips), _ptr(workspace), workspace.numel(), _stream(device)), "coordinate_update")
        if flips is not None:
            return flips
        return int(workspace[8:16].view(torch.int64).item())


def coordinate_update_static(gradient: Tensor, coordinate: Tensor, packed: Tensor, moment_q: Tensor,
                             moment_scale: Tensor, row_v: Tensor, col_v: Tensor, *, beta1: float,
                             beta2: float, update_clip: float, coordinate_lr: float, block_size: int,
                             seed: int, step: int, flips: Tensor) -> Tensor:
    """``coordinate_update`` without a workspace: for callers that cannot allocate.

    Same step, same results, but the kernel scratch is a fixed array inside the library
    (``qste_b200_coordinate_update_static``), so this wrapper asks torch for nothing.  It
    exists for integrations whose device memory is planned up front by someone else, or
    that run where the CUDA allocator must not be entered.  Limits: at most 16384 rows,
    16384 columns and 262144 momentum blocks; beyond that it raises.  All calls on a device
    share that one array, so two calls that can overlap on the GPU (different streams)
    race.  ``flips`` (a device int64 scalar) is required and receives the flip count.
    """

    if not torch.is_tensor(flips):
        raise RuntimeError("coordinate_update_static needs `flips`, a device int64 scalar: there is no workspace "
                           "to read the count back from")
    if not gradient.is_contiguous():
        # the workspace variant copies a strided evidence; this one may not allocate the copy
        raise RuntimeError("coordinate_update_static: the evidence must be contiguous (no copy can be allocated here)")
    count = _check_update_arguments("coordinate_update_static", gradient, coordinate, packed, moment_q,
                                    moment_scale, row_v, col_v, block_size, int(step), flips, None)
    if count == 0:
        return flips.zero_()
    rows, columns = gradient.shape
    device = gradient.device
    with _on(device):
        _cabi.check(_cabi.load().qste_b200_coordinate_update_static(
            _ptr(gradient), _ptr(coordinate), _ptr(packed), _ptr(moment_q), _ptr(moment_scale),
            _ptr(row_v), _ptr(col_v), rows, columns, float(beta1), float(beta2), float(update_clip),
            float(coordinate_lr), int(block_size), int(seed), int(step), None, None, _ptr(flips),
            _stream(device)), "coordinate_update_static")
    return flips


# -- status -----------------------------------------------------------------------

def native_available() -> bool:
    return _cabi.failure() is None


def cuda_available() -> bool:
    return native_available() and torch.cuda.is_available()


def cuda_backend():
    """The loaded C-ABI library (the one backend), or raise."""

    return _cabi.load()


def status() -> dict[str, object]:
    failure = _cabi.failure()
    return {
        "mode": "cuda",
        "native": failure is None,
        "cuda": failure is None and torch.cuda.is_available(),
        "source": str(_cabi.LIBRARY),
        "failure": failure,
        "cuda_failure": None if torch.cuda.is_available() else "no CUDA device",
    }


def warn_if_slow(device_type: str = "cuda") -> None:
    """The reference warns here when it falls back to slow kernels.  This build has
    no fallback, so the equivalent is to fail now rather than at the first step."""

    del device_type
    _cabi.load()


__all__ = [
    "DeviceProfile", "apply_bits", "coordinate_update", "coordinate_update_static", "cuda_available", "cuda_backend",
    "evidence_from_packed", "linear_backward", "linear_backward_evidence", "native_available", "pack_bits",
    "pack_coordinate", "pack_affine_rows", "packed_embedding", "packed_linear_affine",
    "packed_row_inner", "packed_transpose", "profile", "set_backward_reserve", "smooth_backward", "smooth_forward",
    "smooth_supported", "status", "stream", "unpack_bits",
    "unpack_rows", "wait_timeouts", "warm", "warn_if_slow", "first_wait_timeout", "check_waits", "last_forward_kernel",
]
