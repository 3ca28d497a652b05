"""Generate tests/golden/reference_vectors.npz by running the reference itself.

Run where the reference is checked out; its location is the first argument, else the
environment variable QSTE_REFERENCE, else a directory named ``reference`` beside this
repository:

    QSTE_NATIVE_ARCH=0 QSTE_CACHE_DIR=/tmp/qste_cache python tests/golden/make_golden.py [reference]

The reference is imported unmodified from ``<reference>/src``.  Its native CPU
extension is built by its own loader with ``QSTE_NATIVE_ARCH=0`` (no
``-march=native``, so no FMA contraction: the integer outputs then depend only on
IEEE fp32 arithmetic).  Every array written here is either a seeded input or an
output of the reference's own functions; nothing is computed by this repository's
code.  Keys are ``<case>/<name>``.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("QSTE_NATIVE_ARCH", "0")
os.environ.setdefault("QSTE_CACHE_DIR", "/tmp/qste_cache_golden")
os.environ.setdefault("QSTE_KERNELS", "native")

REFERENCE = Path(sys.argv[1] if len(sys.argv) > 1 else
                 os.environ.get("QSTE_REFERENCE") or Path(__file__).resolve().parents[3] / "reference")
sys.path.insert(0, str(REFERENCE / "src"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn as nn  # noqa: E402

import qste  # noqa: E402
from qste import kernels  # noqa: E402
from qste.kernels import fallback, loader, stream  # noqa: E402

OUT = Path(__file__).resolve().parent / "reference_vectors.npz"
store: dict[str, np.ndarray] = {}


def put(case: str, **arrays) -> None:
    for name, value in arrays.items():
        if isinstance(value, torch.Tensor):
            tensor = value.detach().cpu()
            if tensor.dtype == torch.float16:
                value = tensor.numpy().view(np.uint16)  # keep the exact bit pattern
            elif tensor.dtype == torch.bool:
                value = tensor.numpy().astype(np.uint8)
            else:
                value = tensor.numpy()
        store[f"{case}/{name}"] = np.array(value, copy=True, order="C")  # snapshot: state tensors are mutated later


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


assert loader.native_available(), kernels.status()

# -- hash stream (stream.py:41-83) ------------------------------------------------
values = [0, 1, 2, 61, 255, 65535, 65536, 0x2545F491, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFF, 123456789]
put("stream", values=np.array(values, np.uint64),
    scrambled=np.array([stream.scramble(v) for v in values], np.uint64))
triples = [(1, 0, 0), (1, 7, 63), (99, 1234, 4095), (0, 0, 1), (2**31 + 5, 3, 2**20 + 17), (7, 3, 511), (17, 5, 2047)]
put("stream", triples=np.array(triples, np.int64),
    uniform=np.array([stream.uniform(*t) for t in triples], np.float64),
    seed_hash=np.array([stream.seed_hash(t[0]) for t in triples], np.uint64),
    step_hash=np.array([stream.step_hash(t[1]) for t in triples], np.uint64))

# -- packing ------------------------------------------------------------------------
for index, (rows, columns) in enumerate([(17, 13), (33, 8), (128, 96), (5, 65), (3, 1), (40, 256)]):
    case = f"pack{index}"
    x = torch.randn(rows, columns, generator=gen(3 + index))
    if index % 2:
        x = torch.nn.functional.gelu(x)  # one-signed-ish rows, as after an activation
    native = loader.pack_affine_rows(x)
    reference = fallback.pack_affine_rows(x)
    coordinate = torch.randint(-127, 128, (rows, columns), generator=gen(50 + index), dtype=torch.int32).to(torch.int8)
    mask = torch.rand(rows, columns, generator=gen(70 + index)) > 0.4
    packed_mask = loader.pack_bits(mask)
    values_f = torch.randn(rows, columns, generator=gen(90 + index))
    put(case, x=x, bits=native[0], offset=native[1], scale=native[2],
        fallback_bits=reference[0], fallback_offset=reference[1], fallback_scale=reference[2],
        coordinate=coordinate, coordinate_bits=loader.pack_coordinate(coordinate),
        mask=mask, mask_bits=packed_mask,
        values=values_f, applied=loader.apply_bits(values_f, packed_mask, columns),
        unpacked=loader.unpack_rows(native[0], columns),
        unpacked_bits=loader.unpack_bits(packed_mask, columns))

# -- projections (tests/test_kernels.py SHAPES) ------------------------------------------
for index, (rows, columns, samples) in enumerate([(17, 13, 5), (64, 64, 32), (128, 96, 40), (33, 8, 7), (24, 200, 3)]):
    case = f"proj{index}"
    weight_bits = fallback.pack_affine_rows(torch.randn(rows, columns, generator=gen(200 + index)))[0]
    x = torch.randn(samples, columns, generator=gen(210 + index))
    scale = torch.rand(rows, generator=gen(220 + index)) + 0.5
    bias = torch.randn(rows, generator=gen(230 + index))
    dy = torch.randn(samples, rows, generator=gen(240 + index))
    act_bits, act_offset, act_scale = loader.pack_affine_rows(x)
    matrix = torch.randn(rows, columns, generator=gen(250 + index))
    ids = torch.randint(0, rows, (7, 3), generator=gen(260 + index))
    evidence = loader.evidence_from_packed(dy, act_bits, columns, act_scale)
    from qste.functional import decoded_evidence

    put(case, weight_bits=weight_bits, x=x, scale=scale, bias=bias, dy=dy, matrix=matrix, ids=ids,
        act_bits=act_bits, act_offset=act_offset, act_scale=act_scale,
        y=loader.packed_linear_affine(x, weight_bits, scale, bias, columns),
        y_nobias=loader.packed_linear_affine(x, weight_bits, scale, None, columns),
        dx=loader.packed_transpose(dy, weight_bits, columns, scale),
        dx_unscaled=loader.packed_transpose(dy, weight_bits, columns),
        evidence=evidence,
        evidence_unscaled=loader.evidence_from_packed(dy, act_bits, columns),
        decoded=decoded_evidence(dy, act_bits, torch.stack((act_offset, act_scale)), "bit", columns),
        row_inner=loader.packed_row_inner(matrix, weight_bits, columns),
        embedding=loader.packed_embedding(ids, weight_bits, scale, columns))


# -- optimizer (tests/test_kernels.py:164-242, 282-314) -------------------------------------
def update_state(rows, columns, block, seed=11):
    coordinate = torch.randint(-127, 128, (rows, columns), generator=gen(seed), dtype=torch.int32).to(torch.int8)
    blocks = (rows * columns + block - 1) // block
    return {
        "coordinate": coordinate,
        "packed": fallback.pack_coordinate(coordinate),
        "moment_q": torch.zeros(rows, columns, dtype=torch.int8),
        "moment_scale": torch.full((blocks,), 1 / 127, dtype=torch.float16),
        "row_v": torch.zeros(rows, dtype=torch.float16),
        "col_v": torch.zeros(columns, dtype=torch.float16),
    }


ORDER = ("coordinate", "packed", "moment_q", "moment_scale", "row_v", "col_v")
cases = [
    (16, 32, 64, 7, 3, 1.0), (24, 40, 64, 7, 3, 1.0), (8, 8, 64, 7, 3, 1.0),
    (32, 64, 256, 17, 5, 1.0), (12, 20, 64, 1, 0, 4.0), (10, 24, 64, 99, 5, 4.0),
    (7, 13, 16, 3, 0, 2.0), (96, 136, 256, 1, 0, 1.0),
]
for index, (rows, columns, block, seed, step0, lr) in enumerate(cases):
    case = f"update{index}"
    state = update_state(rows, columns, block)
    mirror = update_state(rows, columns, block)
    put(case, meta=np.array([rows, columns, block, seed, step0], np.int64), lr=np.float64(lr),
        **{f"init_{k}": v for k, v in state.items()})
    for number in range(3):
        evidence = torch.randn(rows, columns, generator=gen(12 + 10 * index + number)) * (10.0 ** (number - 1))
        common = dict(beta1=0.9, beta2=0.99, update_clip=2.0, coordinate_lr=lr, block_size=block,
                      seed=seed, step=step0 + number)
        flips = loader.coordinate_update(evidence.clone(), *[state[k] for k in ORDER], **common)
        mirror_flips = fallback.coordinate_update(evidence.clone(), *[mirror[k] for k in ORDER], **common)
        put(case, **{f"evidence{number}": evidence, f"flips{number}": np.int64(flips),
                     f"fallback_flips{number}": np.int64(mirror_flips)})
        put(case, **{f"step{number}_{k}": v for k, v in state.items()})
        put(case, **{f"fallback_step{number}_{k}": v for k, v in mirror.items()})

# -- Surface construction (surface.py:41-74) --------------------------------------------------
for index, (rows, columns) in enumerate([(24, 40), (16, 9)]):
    weight = torch.randn(rows, columns, generator=gen(300 + index)) * 0.05
    weight[0, :3] = 0.0
    surface = qste.Surface(weight)
    put(f"surface{index}", weight=weight, coordinate=surface.coordinate.data,
        packed=surface.packed_sign.data, log_scale=surface.log_scale.data,
        dense=surface.dense_weight())

# -- one converted Linear end to end (functional.py:153-205, optim.py:156-201) -------------------
for index, (rows, columns, batch, use_bias) in enumerate([(48, 40, 32, True), (64, 96, 24, False)]):
    case = f"layer{index}"
    torch.manual_seed(400 + index)
    linear = nn.Linear(columns, rows, bias=use_bias)
    weight0 = linear.weight.detach().clone()
    bias0 = None if not use_bias else linear.bias.detach().clone()
    model = nn.Sequential(linear)
    qste.convert(model, include=["0"], activations=False)
    layer = model[0]
    coordinates = qste.QSTEOptimizer(model)
    host = torch.optim.AdamW(qste.continuous_parameters(model), lr=1e-3)
    put(case, weight=weight0, **({"bias": bias0} if use_bias else {}),
        init_coordinate=layer.surface.coordinate.data.clone(),
        init_packed=layer.surface.packed_sign.data.clone(),
        init_log_scale=layer.surface.log_scale.data.clone())
    captured = {}
    original_apply = coordinates._apply

    def tap(surface, evidence, _store=captured, _apply=original_apply):
        _store["evidence"] = evidence.detach().clone()
        _apply(surface, evidence)

    layer.surface._immediate = tap
    for number in range(2):
        x = torch.randn(batch, columns, generator=gen(410 + 10 * index + number), requires_grad=True)
        dy = torch.randn(batch, rows, generator=gen(420 + 10 * index + number))
        y = model(x)
        y.backward(dy)
        put(case, **{f"x{number}": x, f"dy{number}": dy, f"y{number}": y, f"dx{number}": x.grad,
                     f"g_log_scale{number}": layer.surface.log_scale.grad,
                     f"evidence{number}": captured["evidence"]})
        if use_bias:
            put(case, **{f"g_bias{number}": layer.bias.grad})
        host.step()
        flips = coordinates.step()
        host.zero_grad(set_to_none=True)
        coordinates.zero_grad()
        state = coordinates.state[id(layer.surface)]
        put(case, **{f"flips{number}": np.int64(flips),
                     f"coordinate{number}": layer.surface.coordinate.data,
                     f"packed{number}": layer.surface.packed_sign.data,
                     f"log_scale{number}": layer.surface.log_scale.data,
                     f"moment_q{number}": state["moment_q"], f"moment_scale{number}": state["moment_scale"],
                     f"row_v{number}": state["row_v"], f"col_v{number}": state["col_v"]})


# -- planning / reporting (convert.py:99-156, 309-324) ---------------------------------------------
class Block(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.fc1 = nn.Linear(dim, dim * 2)
        self.fc2 = nn.Linear(dim * 2, dim)
        self.gate = nn.Linear(dim, dim, bias=False)


class Tiny(nn.Module):
    def __init__(self, vocab=48, dim=16, depth=2):
        super().__init__()
        self.embed = nn.Embedding(vocab, dim)
        self.blocks = nn.ModuleList([Block(dim) for _ in range(depth)])
        self.head = nn.Linear(dim, vocab, bias=False)
        self.head.weight = self.embed.weight


torch.manual_seed(5)
tiny = Tiny()
table = qste.format_plan(qste.plan(tiny, include=["blocks.*.fc1", "blocks.*.fc2", "embed", "head"]))
qste.convert(tiny, include=["blocks.*.fc1", "blocks.*.fc2"])
report = qste.memory_report(tiny)
put("plan", table=np.frombuffer(table.encode(), np.uint8),
    report_keys=np.frombuffer(",".join(report).encode(), np.uint8),
    report_values=np.array(list(report.values()), np.float64))

np.savez_compressed(OUT, **store)
print(f"wrote {OUT} with {len(store)} arrays, {OUT.stat().st_size / 1024:.1f} KiB")
