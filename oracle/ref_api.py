"""Adapter over the unmodified reference package (``browsergrad_jit``, assembled under ``oracle/_ref`` by
``build_ref.py``): exposes its builders under the names ``browsergrad_b200.graph`` uses, so one case definition builds
the reference's graph and this build's.  Test and baseline infrastructure only -- nothing in the product imports it."""
from __future__ import annotations

from typing import Any


class RefApi:
    """Adapter exposing the reference's ``browsergrad_jit`` module with the builder names
    ``browsergrad_b200.graph`` uses."""

    def __init__(self, bg: Any) -> None:
        F = bg.F
        self.relu, self.gelu, self.softmax, self.linear = F.relu, F.gelu, F.softmax, F.linear
        self.layer_norm, self.cross_entropy = F.layer_norm, F.cross_entropy
        self.scaled_dot_product_attention = F.scaled_dot_product_attention
        self.exp, self.where, self.tanh = bg.exp, bg.where, bg.tanh
        self.attention_forward = bg.kernels.attention_forward
        self.autocast = lambda dtype="float16": bg.amp.autocast(dtype=dtype)
        self.from_numpy = bg.from_numpy
        self.cat, self.stack, self.cumsum = bg.cat, bg.stack, bg.cumsum
        self.sort, self.topk = bg.sort, bg.topk
        self.pad = F.pad
        self._bg = bg

    def _raw(self, t: Any, op: str, shape: tuple, arg: Any) -> Any:
        """A node no public builder of the reference emits (its derivative rules do, _vjp.py:383-472), built with the
        reference's own ``UOp`` constructor and wrapped like any other recorded value."""
        node = self._bg._ir.UOp(op=op, inputs=(t._uop,), shape=tuple(shape), dtype=t._uop.dtype, arg=arg)
        return type(t)(node, t._session)

    def narrow(self, t: Any, axis: int, start: int, length: int) -> Any:
        shape = t.shape[:axis] + (length,) + t.shape[axis + 1:]
        return self._raw(t, "NARROW", shape, {"axis": axis, "start": start, "length": length})

    def take_slice(self, t: Any, slices: Any) -> Any:
        slices = tuple(slices)
        shape = tuple(len(range(*sl.indices(d))) for sl, d in zip(slices, t.shape)) + tuple(t.shape[len(slices):])
        return self._raw(t, "SLICE", shape, {"slices": slices})
