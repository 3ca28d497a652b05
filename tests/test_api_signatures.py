"""The public call surface against the reference's, parameter by parameter.

``tests/golden/reference_api.json`` is written by ``tests/golden/make_api.py`` from the
imported reference: for each public callable its parameters as (name, kind, default).  A
drop-in must accept every call the reference accepts, so each recorded parameter has to
exist here with the same name, kind and default, in the same order; this build may add
keyword parameters of its own AFTER them (``QSTEOptimizer(async_update=...)``), never
before or between.
"""

from __future__ import annotations

import inspect
import json
from pathlib import Path

import pytest
import torch.nn as nn

import qste_b200 as qste
from qste_b200 import kernels

API = json.loads((Path(__file__).parent / "golden" / "reference_api.json").read_text())


def parameters(function):
    out = []
    for name, parameter in inspect.signature(function).parameters.items():
        default = None if parameter.default is inspect.Parameter.empty else repr(parameter.default)
        out.append([name, parameter.kind.name, default])
    return out


def assert_accepts_the_same_calls(mine, theirs, what):
    assert mine[:len(theirs)] == theirs, (what, mine, theirs)
    for name, kind, default in mine[len(theirs):]:
        # additions must not change what an existing call means
        assert kind in ("KEYWORD_ONLY", "VAR_KEYWORD") and (default is not None or kind == "VAR_KEYWORD"), (what, name)


@pytest.mark.parametrize("name", sorted(API["functions"]))
def test_top_level_functions(name):
    assert_accepts_the_same_calls(parameters(getattr(qste, name)), API["functions"][name], name)


@pytest.mark.parametrize("name", sorted(API["kernels"]))
def test_kernel_namespace(name):
    assert_accepts_the_same_calls(parameters(getattr(kernels, name)), API["kernels"][name], name)


@pytest.mark.parametrize("cls,method", [(c, m) for c, ms in sorted(API["methods"].items()) for m in sorted(ms)])
def test_methods(cls, method):
    assert_accepts_the_same_calls(parameters(getattr(getattr(qste, cls), method)), API["methods"][cls][method],
                                  f"{cls}.{method}")


def test_dictionaries_hosts_index(cpu_kernels):
    assert sorted(qste.retained_stats()) == API["retained_stats_keys"]
    assert type(qste.decisions()).__name__ == API["decisions_type"]
    qste.retain(1 << 20)
    assert qste.retained_stats()["budget_bytes"] == 1 << 20 and qste.retained_stats()["resident_bytes"] == 0
    qste.retain(0)
    model = nn.Sequential(nn.Linear(16, 8))
    qste.convert(model, include=["0"])
    assert sorted(qste.memory_report(model)) == API["memory_report_keys"]
    assert qste.undecided(model, __import__("torch").zeros(2, 16)) is False
    qste.invalidate(model[0].surface.packed_sign)
