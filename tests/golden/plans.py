"""Rebuilds plan objects from ``plans.json`` (written by ``make_plans.py`` from the reference's real
scheduled plans). The objects carry the attribute surface a code generator reads off a reference
``Plan`` (python/cleave/pipeline/plans.py:16-41): ``variant``, ``role``, ``split_factor``, ``inputs`` and
``tile.flat_graph.nodes``, each node an instance of a class NAMED like the reference's node class with
``name``, ``get_shape(0)``, ``get_dtype(0)``, ``inputs[i].src_node`` and the recorded attributes
(``const``, ``const_on_left``, ``axis``, ``transpose_A`` ...)."""

from __future__ import annotations

import json
import os
from types import SimpleNamespace

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "plans.json")
_classes: dict = {}


class _Node:
    def get_shape(self, _i=0):
        return list(self._shape)

    def get_dtype(self, _i=0):
        return self._dtype


def _node(rec):
    cls = _classes.setdefault(rec["type"], type(rec["type"], (_Node,), {}))
    n = cls()
    n.name, n._shape, n._dtype, n.inputs = rec["name"], rec["shape"] or [], rec["dtype"], []
    for k, v in rec.items():
        if k not in ("type", "name", "shape", "dtype", "inputs"):
            setattr(n, k, v)
    return n


def plan_from_record(rec):
    nodes = [_node(r) for r in rec["nodes"]]
    by_name = {}
    for n in nodes:  # two output nodes may share no name; later definitions shadow earlier ones as in the graph
        by_name[n.name] = n
    for n, r in zip(nodes, rec["nodes"]):
        n.inputs = [SimpleNamespace(src_node=by_name[s]) for s in r["inputs"] if s in by_name]
    tile = SimpleNamespace(flat_graph=SimpleNamespace(nodes=nodes), output_tile=[], n_threads=None)
    return SimpleNamespace(variant=rec["variant"], role=rec["role"], split_factor=rec["split_factor"],
                           inputs=None if rec["inputs"] is None else tuple(rec["inputs"]), tile=tile,
                           label=f"{rec['variant']} {rec['role']}", count=rec.get("count", 1))


def load():
    """``{case: {"program_inputs", "dtype", "plans": [plan objects]}}``."""
    with open(PATH) as f:
        data = json.load(f)
    return {name: {"program_inputs": [(n, tuple(s)) for n, s in c["program_inputs"]], "dtype": c["dtype"],
                   "n_plans": c["plans"], "plans": [plan_from_record(r) for r in c["records"]]}
            for name, c in data.items()}
