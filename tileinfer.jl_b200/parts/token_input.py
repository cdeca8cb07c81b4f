"""A per-layer input taken from the token itself: every token id has a vector (one slice of a table shared by all
layers), which a gate computed from the stream lets through; the result is projected to the stream's width.

    ``gated_embedding``:  g = gelu_tanh(Wgate h) * S[token, first : first + dim];  y = Wproj g

The block adds y through the part's ``norm`` (an RMS norm with a plain weight, in 32-bit), like any other branch.
"""
from __future__ import annotations

from typing import Dict

from ..config.spec import NormSpec, TensorDecl, TokenInputSpec
from ..kernels import ops
from .base import Part, _register, lookup
from .linear import Linear


def register_token_input(kind: str, cls=None):
    return _register("token_input", kind, cls) if cls is not None else (lambda c: _register("token_input", kind, c))


class TokenInput(Part):
    """``__init__(spec: TokenInputSpec, tensors, rt)``; ``forward(h, step) -> y`` [n, hidden]; ``norm``: the norm part
    through which the block adds y to the stream."""

    def forward(self, h, step):
        raise NotImplementedError


@register_token_input("gated_embedding")
class GatedEmbedding(TokenInput):
    def __init__(self, spec: TokenInputSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        n, p = spec.tensor_names, spec.prefix
        self.table = _shared_table(rt, tensors, spec.table_name)
        self.gate = Linear(rt.param(tensors[p + n["gate"]]), rt, "token_gate")
        self.proj = Linear(rt.param(tensors[p + n["proj"]]), rt, "token_proj")
        self.norm = lookup("norm", "rmsnorm32")(self._norm_spec(spec), tensors, rt)

    @staticmethod
    def _norm_spec(spec: TokenInputSpec) -> NormSpec:
        return NormSpec("rmsnorm32", spec.hidden_size, spec.eps, spec.prefix + spec.tensor_names["norm"], {"init_std": 0.1})

    @classmethod
    def tensors(cls, spec: TokenInputSpec):
        n, p = spec.tensor_names, spec.prefix
        return [TensorDecl(spec.table_name, (spec.vocab_size, spec.table_columns), ("normal", 1.0)),
                TensorDecl(p + n["gate"], (spec.dim, spec.hidden_size), ("normal", spec.hidden_size ** -0.5)),
                TensorDecl(p + n["proj"], (spec.hidden_size, spec.dim), ("normal", spec.dim ** -0.5))] + \
            lookup("norm", "rmsnorm32").tensors(cls._norm_spec(spec))

    def forward(self, h, step):
        n = h.shape[0]
        y = self.rt.buffer("token_input.out", (n, self.spec.hidden_size))
        g = self.rt.buffer("token_input.gate", (n, self.spec.dim))
        self.gate.forward(h, g)
        ops.gated_token_embedding(g, self.table, step.token_ids, self.spec.first_column)
        return self.proj.forward(g, y)


# The table is one tensor for all layers: it goes to the device once per runtime.
_tables: Dict[tuple, object] = {}


def _shared_table(rt, tensors, name):
    key = (id(rt), id(tensors[name]))
    if key not in _tables:
        if len(_tables) > 8:
            _tables.clear()
        _tables[key] = rt.param(tensors[name])
    return _tables[key]
