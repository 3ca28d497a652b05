"""Record the call signatures of the reference's public API into reference_api.json.

Run where the reference is checked out (first argument, else $QSTE_REFERENCE, else a
directory named ``reference`` beside this repository):

    QSTE_KERNELS=torch python tests/golden/make_api.py [reference]

Imports the unmodified reference and writes, for every public callable a host touches on
the binary-layer path, its parameters as ``[name, kind, default]`` triples, plus the keys of
the two dictionaries hosts index (``retained_stats()``, ``memory_report()``).  Nothing here
is computed by this repository's code.
"""

from __future__ import annotations

import inspect
import json
import os
import sys
from pathlib import Path

os.environ.setdefault("QSTE_KERNELS", "torch")
REFERENCE = Path(sys.argv[1] if len(sys.argv) > 1 else
                 os.environ.get("QSTE_REFERENCE") or Path(__file__).resolve().parents[3] / "reference")
sys.path.insert(0, str(REFERENCE / "src"))

import torch.nn as nn  # noqa: E402

import qste  # noqa: E402
from qste import kernels  # noqa: E402


def parameters(function) -> list:
    out = []
    for name, parameter in inspect.signature(function).parameters.items():
        default = None if parameter.default is inspect.Parameter.empty else repr(parameter.default)
        out.append([name, parameter.kind.name, default])
    return out


TOP = ["convert", "plan", "format_plan", "memory_report", "warmup", "decisions", "undecided", "retain",
       "retained_stats", "invalidate", "exact_evidence", "packed_activations", "export_packed", "surfaces",
       "continuous_parameters", "qste_linear"]
KERNELS = ["unpack_rows", "unpack_bits", "pack_bits", "apply_bits", "pack_affine_rows", "pack_coordinate",
           "packed_linear_affine", "packed_transpose", "evidence_from_packed", "packed_row_inner",
           "packed_embedding", "coordinate_update"]
METHODS = {"QSTEOptimizer": ["__init__", "defer", "prepare_accumulation", "unscale_", "zero_grad", "step",
                             "state_bytes", "state_dict", "load_state_dict"],
           "Surface": ["__init__", "consume_evidence", "flush_evidence", "prepare_accumulator", "scale_evidence_",
                       "refresh_packed", "memory", "dense_weight", "note_forward", "reset_tracking"],
           "QSTELinear": ["__init__", "from_linear", "forward"]}

api = {"functions": {name: parameters(getattr(qste, name)) for name in TOP if hasattr(qste, name)},
       "kernels": {name: parameters(getattr(kernels, name)) for name in KERNELS},
       "methods": {cls: {m: parameters(getattr(getattr(qste, cls), m)) for m in names}
                   for cls, names in METHODS.items()}}
model = nn.Sequential(nn.Linear(16, 8))
qste.convert(model, include=["0"])
api["retained_stats_keys"] = sorted(qste.retained_stats())
api["memory_report_keys"] = sorted(qste.memory_report(model))
api["decisions_type"] = type(qste.decisions()).__name__
out = Path(__file__).resolve().parent / "reference_api.json"
out.write_text(json.dumps(api, indent=1, sort_keys=True) + "\n")
print(out, sum(len(v) for v in api["functions"].values()), "parameters recorded")
