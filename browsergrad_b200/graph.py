"""Lazy UOp graph builder for the forward configurations the CUDA realizer serves.

The realizer front (`browsergrad_b200.front.realize_cuda`) accepts any node object with the
five fields of browsergrad-jit's ``UOp`` (packages/browsergrad-jit/src/python/_ir.py:254-276):
``op, inputs, shape, dtype, arg``.  When browsergrad-jit itself is importable its
``TensorProxy._uop`` graphs are passed straight in.  This module exists so that the same
graphs can be built where browsergrad-jit is not installed: it mirrors, for the forward
path only, the op sequences emitted by the reference's builders

* arithmetic dunders, comparison, reductions, reshape/permute, ``masked_fill``, ``gather``
  (packages/browsergrad-jit/src/python/_tensor_proxy.py:699-900, 1178-1260, 1346-1379,
  1520-1566, 1598-1745, 2095-2152),
* ``relu / tanh / gelu / softmax / linear / layer_norm / cross_entropy /
  scaled_dot_product_attention`` (packages/browsergrad-jit/src/python/_functional.py:99-166,
  178-262, 741-750, 763-810, 1505-1534),
* the ``autocast`` tag that the cast pass reads (packages/browsergrad-jit/src/python/_amp.py:
  84-150, _tensor_proxy.py:425-446).

There is no autograd, no session object and no CPU execution here: a ``Tensor`` only records
nodes.  Leaf arrays live in a ``BufferStore`` keyed by the id carried in ``BUFFER.arg``.
"""
from __future__ import annotations

import itertools
import threading
from typing import Any, Dict, Optional, Sequence, Tuple

import numpy as np

KNOWN_DTYPES = frozenset({
    "float16", "float32", "float64", "int8", "int16", "int32", "int64",
    "uint8", "uint16", "uint32", "uint64", "bool",
})
MASKED_FILL_CONTRACT_ID = "browsergrad.jit.framework.tensor.masked-fill.v1"


class Node:
    """One IR node: the same five fields as the reference ``UOp``."""

    __slots__ = ("op", "inputs", "shape", "dtype", "arg")

    def __init__(self, op: str, inputs: Tuple["Node", ...] = (), shape: Tuple[int, ...] = (),
                 dtype: str = "float32", arg: Any = None) -> None:
        self.op = op
        self.inputs = tuple(inputs)
        self.shape = tuple(int(d) for d in shape)
        self.dtype = dtype
        self.arg = arg

    def __repr__(self) -> str:
        return f"Node({self.op}, shape={self.shape}, dtype={self.dtype})"


class BufferStore:
    """``buffer id -> ndarray`` for leaf tensors (the role of the reference ``BufferTable``,
    packages/browsergrad-jit/src/python/_buffer_table.py:32-166, reduced to get/put)."""

    def __init__(self) -> None:
        self._arrays: Dict[str, np.ndarray] = {}
        self._counter = itertools.count()

    def new_buffer(self, array: np.ndarray) -> str:
        bid = f"buf_{next(self._counter)}"
        self._arrays[bid] = array
        return bid

    def get(self, bid: str) -> np.ndarray:
        return self._arrays[bid]

    def is_materialized(self, bid: str) -> bool:
        return bid in self._arrays

    def __len__(self) -> int:
        return len(self._arrays)


_DEFAULT_STORE = BufferStore()
_TLS = threading.local()


def default_store() -> BufferStore:
    return _DEFAULT_STORE


def reset_default_store() -> BufferStore:
    global _DEFAULT_STORE
    _DEFAULT_STORE = BufferStore()
    return _DEFAULT_STORE


class autocast:
    """Tags nodes built inside the context with ``arg["autocast_hint"]``.

    ``float16`` is the reference's only mode (_amp.py:123-133).  ``bfloat16`` is an extension
    of this build for the tensor-core bf16 path; the reference refuses it.
    """

    def __init__(self, dtype: str = "float16", enabled: bool = True) -> None:
        if dtype not in ("float16", "bfloat16", "float32"):
            raise NotImplementedError(f"autocast dtype={dtype!r} not supported")
        self._dtype = dtype
        self._enabled = enabled
        self._prev: Optional[str] = None

    def __enter__(self) -> "autocast":
        self._prev = getattr(_TLS, "amp", None)
        if self._enabled and self._dtype != "float32":
            _TLS.amp = self._dtype
        return self

    def __exit__(self, *exc: Any) -> None:
        _TLS.amp = self._prev


def _amp_arg(arg: Any = None) -> Any:
    active = getattr(_TLS, "amp", None)
    if active is None:
        return arg
    if arg is None:
        return {"autocast_hint": active}
    if isinstance(arg, dict):
        return {**arg, "autocast_hint": active}
    return arg


def _promote(a: str, b: str) -> str:
    return np.promote_types(np.dtype(a), np.dtype(b)).name


def _bshape(*shapes: Tuple[int, ...]) -> Tuple[int, ...]:
    return tuple(np.broadcast_shapes(*shapes))


class Tensor:
    """A recorded value.  ``_uop`` names the node, as on the reference ``TensorProxy``."""

    __slots__ = ("_uop", "_store")
    __array_priority__ = 1000

    def __init__(self, node: Node, store: Optional[BufferStore] = None) -> None:
        self._uop = node
        self._store = store if store is not None else _DEFAULT_STORE

    # -- metadata -----------------------------------------------------------------
    @property
    def shape(self) -> Tuple[int, ...]:
        return self._uop.shape

    @property
    def dtype(self) -> str:
        return self._uop.dtype

    @property
    def ndim(self) -> int:
        return len(self._uop.shape)

    def numel(self) -> int:
        n = 1
        for d in self._uop.shape:
            n *= d
        return n

    def _wrap(self, node: Node) -> "Tensor":
        return Tensor(node, self._store)

    def _coerce(self, other: Any) -> "Tensor":
        return _to_tensor(other, self._store)

    # -- arithmetic ---------------------------------------------------------------
    def _binop(self, other: Any, op: str) -> "Tensor":
        rhs = self._coerce(other)
        node = Node(op, (self._uop, rhs._uop), _bshape(self.shape, rhs.shape),
                    _promote(self.dtype, rhs.dtype), _amp_arg(None))
        return self._wrap(node)

    def __add__(self, other: Any) -> "Tensor":
        return self._binop(other, "ADD")

    def __radd__(self, other: Any) -> "Tensor":
        return self._coerce(other).__add__(self)

    def __sub__(self, other: Any) -> "Tensor":
        return self.__add__(-self._coerce(other))

    def __rsub__(self, other: Any) -> "Tensor":
        return self._coerce(other).__sub__(self)

    def __mul__(self, other: Any) -> "Tensor":
        return self._binop(other, "MUL")

    def __rmul__(self, other: Any) -> "Tensor":
        return self._coerce(other).__mul__(self)

    def __truediv__(self, other: Any) -> "Tensor":
        return self._binop(other, "DIV")

    def __rtruediv__(self, other: Any) -> "Tensor":
        return self._coerce(other).__truediv__(self)

    def __neg__(self) -> "Tensor":
        return self._wrap(Node("NEG", (self._uop,), self.shape, self.dtype, _amp_arg(None)))

    def _unary(self, op: str) -> "Tensor":
        return self._wrap(Node(op, (self._uop,), self.shape, self.dtype, _amp_arg(None)))

    def exp(self) -> "Tensor":
        return self._unary("EXP")

    def log(self) -> "Tensor":
        return self._unary("LOG")

    def __matmul__(self, other: Any) -> "Tensor":
        rhs = self._coerce(other)
        a, b = self.shape, rhs.shape
        if len(a) == 0 or len(b) == 0:
            raise ValueError(f"matmul: 0-d tensors not supported ({a}, {b})")
        if a[-1] != b[-2 if len(b) > 1 else -1]:
            raise ValueError(f"matmul: inner dimensions don't match: {a} @ {b}")
        if len(a) == 1 and len(b) == 1:
            out: Tuple[int, ...] = ()
        elif len(a) == 1:
            out = b[:-2] + (b[-1],)
        elif len(b) == 1:
            out = a[:-1]
        else:
            out = _bshape(a[:-2], b[:-2]) + (a[-2], b[-1])
        node = Node("MATMUL", (self._uop, rhs._uop), out, _promote(self.dtype, rhs.dtype),
                    _amp_arg(None))
        return self._wrap(node)

    # -- comparisons --------------------------------------------------------------
    def _cmp(self, other: Any, op: str) -> "Tensor":
        rhs = self._coerce(other)
        return self._wrap(Node("CMP", (self._uop, rhs._uop), _bshape(self.shape, rhs.shape),
                               "bool", {"op": op}))

    def __gt__(self, other: Any) -> "Tensor":
        return self._cmp(other, "gt")

    def __ge__(self, other: Any) -> "Tensor":
        return self._cmp(other, "ge")

    def __lt__(self, other: Any) -> "Tensor":
        return self._cmp(other, "lt")

    def __le__(self, other: Any) -> "Tensor":
        return self._cmp(other, "le")

    def eq(self, other: Any) -> "Tensor":
        return self._cmp(other, "eq")

    def ne(self, other: Any) -> "Tensor":
        return self._cmp(other, "ne")

    # -- reductions ---------------------------------------------------------------
    def _reduce(self, op: str, axis: Any = None, keepdims: bool = False) -> "Tensor":
        nd = self.ndim
        if axis is None:
            out_shape: Tuple[int, ...] = (1,) * nd if keepdims else ()
        else:
            axes = (axis,) if isinstance(axis, int) else tuple(axis)
            red = tuple(a % nd for a in axes)
            dims = []
            for i, d in enumerate(self.shape):
                if i in red:
                    if keepdims:
                        dims.append(1)
                else:
                    dims.append(d)
            out_shape = tuple(dims)
        dtype = "int64" if op in ("argmax", "argmin") else self.dtype
        node = Node("REDUCE", (self._uop,), out_shape, dtype,
                    _amp_arg({"op": op, "axis": axis, "keepdims": keepdims}))
        return self._wrap(node)

    def sum(self, axis: Any = None, dim: Any = None, keepdims: bool = False,
            keepdim: bool = False) -> "Tensor":
        return self._reduce("sum", dim if dim is not None else axis, keepdim or keepdims)

    def mean(self, axis: Any = None, dim: Any = None, keepdims: bool = False,
             keepdim: bool = False) -> "Tensor":
        return self._reduce("mean", dim if dim is not None else axis, keepdim or keepdims)

    def max(self, axis: Any = None, keepdims: bool = False) -> "Tensor":
        return self._reduce("max", axis, keepdims)

    def min(self, axis: Any = None, keepdims: bool = False) -> "Tensor":
        return self._reduce("min", axis, keepdims)

    def argmax(self, axis: Any = None, keepdims: bool = False) -> "Tensor":
        return self._reduce("argmax", axis, keepdims)

    def argmin(self, axis: Any = None, keepdims: bool = False) -> "Tensor":
        return self._reduce("argmin", axis, keepdims)

    def var(self, axis: Any = None, dim: Any = None, keepdims: bool = False, keepdim: bool = False,
            unbiased: Any = None, correction: Any = None) -> "Tensor":
        """``VAR`` node of ``TensorProxy.var`` (_tensor_proxy.py:1438-1483): biased when
        ``correction=0`` / ``unbiased=False``, Bessel-corrected by default."""
        if self.dtype not in ("float16", "float32", "float64"):
            raise ValueError(f"var: floating dtypes only, got {self.dtype!r}")
        if correction is not None and unbiased is not None:
            raise ValueError("var: specify only one of unbiased or correction")
        corr = int(correction) if correction is not None else (1 if unbiased is None or unbiased else 0)
        reduce_axis = dim if dim is not None else axis
        keep = bool(keepdim or keepdims)
        nd = self.ndim
        if reduce_axis is None:
            axes = tuple(range(nd))
        else:
            axes = tuple(sorted({a % nd for a in ((reduce_axis,) if isinstance(reduce_axis, int) else tuple(reduce_axis))}))
        out_shape = tuple(1 if keep and i in axes else d for i, d in enumerate(self.shape) if keep or i not in axes)
        node = Node("VAR", (self._uop,), out_shape, self.dtype, {"axes": axes, "correction": corr, "keepdims": keep})
        return self._wrap(node)

    def prod(self, axis: Any = None, dim: Any = None, keepdims: bool = False, keepdim: bool = False) -> "Tensor":
        """``PROD`` node of ``TensorProxy.prod`` (_tensor_proxy.py:1278-1308): the product over the sorted,
        de-duplicated axes in the input dtype."""
        if axis is not None and dim is not None:
            raise ValueError("prod: specify only one of axis or dim")
        reduce_axis = dim if dim is not None else axis
        keep = bool(keepdim or keepdims)
        nd = self.ndim
        if reduce_axis is None:
            axes = tuple(range(nd))
        else:
            raw = (reduce_axis,) if isinstance(reduce_axis, (int, np.integer)) else tuple(reduce_axis)
            axes = tuple(sorted(int(a) % nd for a in raw))
            if len(set(axes)) != len(axes):
                raise ValueError("prod: axes must be unique after normalization")
        out_shape = tuple(1 if keep and i in axes else d for i, d in enumerate(self.shape) if keep or i not in axes)
        return self._wrap(Node("PROD", (self._uop,), out_shape, self.dtype, {"axes": axes, "keepdims": keep}))

    def clamp(self, min: Any = None, max: Any = None) -> "Tensor":
        """``CLAMP`` node (_tensor_proxy.py:992-1023); bounds are finite Python floats or ``None``."""
        if min is None and max is None:
            raise ValueError("clamp: at least one of min or max must be provided")
        lo = None if min is None else float(min)
        hi = None if max is None else float(max)
        if lo is not None and hi is not None and lo > hi:
            raise ValueError(f"clamp: min {lo} must be <= max {hi}")
        return self._wrap(Node("CLAMP", (self._uop,), self.shape, self.dtype, {"min": lo, "max": hi}))

    def repeat(self, *sizes: Any) -> "Tensor":
        """``REPEAT`` node (_tensor_proxy.py:1091-1120): ``np.tile`` with one factor per (left-padded) dimension."""
        reps = tuple(int(r) for r in (sizes[0] if len(sizes) == 1 and isinstance(sizes[0], (tuple, list)) else sizes))
        if len(reps) < self.ndim or any(r < 0 for r in reps):
            raise ValueError("repeat: one non-negative factor per dimension (more factors add leading dimensions)")
        padded = (1,) * (len(reps) - self.ndim) + self.shape
        out_shape = tuple(r * d for r, d in zip(reps, padded))
        return self._wrap(Node("REPEAT", (self._uop,), out_shape, self.dtype, {"repeats": reps}))

    def repeat_interleave(self, repeats: int, dim: int) -> "Tensor":
        """``REPEAT_INTERLEAVE`` node (_tensor_proxy.py:1393-1428): every slice along ``dim`` ``repeats`` times in place."""
        axis = int(dim) % self.ndim
        r = int(repeats)
        if r < 0:
            raise ValueError("repeat_interleave: repeats must be non-negative")
        out_shape = tuple(d * r if i == axis else d for i, d in enumerate(self.shape))
        return self._wrap(Node("REPEAT_INTERLEAVE", (self._uop,), out_shape, self.dtype, {"repeats": r, "axis": axis}))

    def flip(self, dim: int) -> "Tensor":
        """``FLIP`` node (_tensor_proxy.py:1122-1139)."""
        axis = int(dim) % self.ndim
        return self._wrap(Node("FLIP", (self._uop,), self.shape, self.dtype, {"axis": axis}))

    def _triangular(self, diagonal: int, upper: bool) -> "Tensor":
        if self.ndim < 2:
            raise ValueError("tril/triu: at least two dimensions required")
        return self._wrap(Node("TRIU" if upper else "TRIL", (self._uop,), self.shape, self.dtype,
                               {"diagonal": int(diagonal)}))

    def tril(self, diagonal: int = 0) -> "Tensor":
        """``TRIL`` node (_tensor_proxy.py:1143-1173)."""
        return self._triangular(diagonal, False)

    def triu(self, diagonal: int = 0) -> "Tensor":
        return self._triangular(diagonal, True)

    def sort(self, dim: int = -1, descending: bool = False, *, stable: bool = False) -> Tuple["Tensor", "Tensor"]:
        return sort(self, dim=dim, descending=descending, stable=stable)

    def topk(self, k: int, dim: Any = None, largest: bool = True, sorted: bool = True) -> Tuple["Tensor", "Tensor"]:
        return topk(self, k, dim=dim, largest=largest, sorted=sorted)

    def cumsum(self, dim: int, dtype: Any = None) -> "Tensor":
        return cumsum(self, dim=dim, dtype=dtype)

    # -- shape ops ----------------------------------------------------------------
    def reshape(self, *shape: Any) -> "Tensor":
        new_shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) \
            else tuple(shape)
        if -1 in new_shape:
            known = 1
            for d in new_shape:
                if d != -1:
                    known *= d
            new_shape = tuple(self.numel() // known if d == -1 else d for d in new_shape)
        n = 1
        for d in new_shape:
            n *= d
        if n != self.numel():
            raise ValueError(f"reshape: {self.shape} -> {new_shape}")
        return self._wrap(Node("RESHAPE", (self._uop,), new_shape, self.dtype,
                               {"new_shape": new_shape}))

    def permute(self, *axes: int) -> "Tensor":
        if len(axes) != self.ndim:
            raise ValueError("permute: wrong number of axes")
        norm = tuple(a % self.ndim for a in axes)
        if len(set(norm)) != self.ndim:
            raise ValueError("permute: duplicate axes")
        return self._wrap(Node("PERMUTE", (self._uop,), tuple(self.shape[a] for a in norm),
                               self.dtype, {"axes": norm}))

    def transpose(self, dim0: int, dim1: int) -> "Tensor":
        axes = list(range(self.ndim))
        d0, d1 = dim0 % self.ndim, dim1 % self.ndim
        axes[d0], axes[d1] = axes[d1], axes[d0]
        return self.permute(*axes)

    @property
    def T(self) -> "Tensor":
        return self.permute(*reversed(range(self.ndim)))

    def cast(self, dtype: str) -> "Tensor":
        if dtype == self.dtype:
            return self
        return self._wrap(Node("CAST", (self._uop,), self.shape, dtype, {"dtype": dtype}))

    def masked_fill(self, mask: "Tensor", value: Any) -> "Tensor":
        if mask.dtype != "bool":
            raise ValueError("masked_fill: mask dtype must be bool")
        if _bshape(self.shape, mask.shape) != self.shape:
            raise ValueError("masked_fill: mask cannot broadcast to source shape")
        if self.dtype == "bool":
            v: Any = bool(value)
        elif self.dtype.startswith("float"):
            v = float(value)
        else:
            v = int(value)
        fill = Node("CONST", (), (), self.dtype, {"value": v})
        return self._wrap(Node("WHERE", (mask._uop, fill, self._uop), self.shape, self.dtype,
                               MASKED_FILL_CONTRACT_ID))

    def gather(self, dim: int, index: "Tensor") -> "Tensor":
        if index.dtype != "int64":
            raise ValueError("gather: index dtype must be int64")
        if index.ndim != self.ndim:
            raise ValueError("gather: source and index must have the same rank")
        axis = dim % self.ndim
        for d, (s, i) in enumerate(zip(self.shape, index.shape)):
            if d != axis and i > s:
                raise ValueError("gather: index extent exceeds source extent")
        return self._wrap(Node("INDEX", (self._uop, index._uop), index.shape, self.dtype,
                               {"dim": axis}))


    def narrow(self, axis: int, start: int, length: int) -> "Tensor":
        """``NARROW`` node as the reference's derivative rules emit it (_vjp.py:383, :426; contract
        _framework_contracts.py:5345-5383): ``length`` consecutive positions of ``axis`` from ``start``."""
        axis = int(axis)
        if self.ndim == 0 or axis < 0 or axis >= self.ndim:
            raise ValueError("narrow: axis out of range")
        start, length = int(start), int(length)
        if start < 0 or length < 0 or start + length > self.shape[axis]:
            raise ValueError("narrow: range exceeds the axis extent")
        shape = self.shape[:axis] + (length,) + self.shape[axis + 1:]
        return self._wrap(Node("NARROW", (self._uop,), shape, self.dtype, {"axis": axis, "start": start, "length": length}))

    def slice(self, slices: Sequence[slice]) -> "Tensor":
        """``SLICE`` node (_ir.py:131, emitted by the PAD derivative rule, _vjp.py:455-472): NumPy basic slicing with
        one ``slice`` per leading axis."""
        slices = tuple(slices)
        if len(slices) > self.ndim or any(not isinstance(sl, slice) for sl in slices):
            raise ValueError("slice: one slice object per leading axis")
        shape = tuple(len(range(*sl.indices(d))) for sl, d in zip(slices, self.shape)) + self.shape[len(slices):]
        return self._wrap(Node("SLICE", (self._uop,), shape, self.dtype, {"slices": slices}))

    def scatter(self, dim: int, index: "Tensor", src: Any) -> "Tensor":
        """``SCATTER`` node (_tensor_proxy.py:2703-2751): a copy of ``self`` with ``src`` stored at the places
        ``index`` names along ``dim``.  ``src`` is a tensor of the index's shape and the target's dtype, or a
        scalar that is normalised to the target dtype (_tensor_proxy.py:291-320).  Indices outside the axis or
        naming one destination twice are refused when the graph is realized."""
        if index.dtype != "int64":
            raise ValueError("scatter: index dtype must be int64")
        if index.ndim != self.ndim or self.ndim == 0:
            raise ValueError("scatter: target and index must have the same nonzero rank")
        axis = int(dim) + self.ndim if int(dim) < 0 else int(dim)
        if axis < 0 or axis >= self.ndim:
            raise ValueError("scatter: dim out of range")
        if any(i > s for s, i in zip(self.shape, index.shape)):
            raise ValueError("scatter: index extent exceeds target extent")
        if isinstance(src, Tensor):
            if src.dtype != self.dtype or src.shape not in ((), index.shape):
                raise ValueError("scatter: source must have the target's dtype and the index's shape")
            source = src._uop
        else:
            if self.dtype == "bool":
                value: Any = bool(src)
            elif self.dtype.startswith("float"):
                value = float(np.asarray(src, dtype=np.dtype(self.dtype)).item())
            else:
                value = int(src)
            source = Node("CONST", (), (), self.dtype, {"value": value})
        return self._wrap(Node("SCATTER", (self._uop, index._uop, source), self.shape, self.dtype, {"dim": axis}))


def _to_tensor(value: Any, store: Optional[BufferStore] = None) -> Tensor:
    if isinstance(value, Tensor):
        return value
    if isinstance(value, (int, float, bool)):
        dt = np.asarray(value).dtype.name
        return Tensor(Node("CONST", (), (), dt, {"value": value}), store)
    return from_numpy(np.asarray(value), store)


def from_numpy(array: np.ndarray, store: Optional[BufferStore] = None) -> Tensor:
    """Leaf tensor: a ``BUFFER`` node wrapped in a ``LOAD`` (_tensor_proxy.py:2148-2152)."""
    store = store if store is not None else _DEFAULT_STORE
    array = np.asarray(array)
    if array.dtype.name not in KNOWN_DTYPES:
        raise TypeError(f"unsupported dtype {array.dtype}")
    bid = store.new_buffer(array)
    buf = Node("BUFFER", (), tuple(array.shape), array.dtype.name, bid)
    return Tensor(Node("LOAD", (buf,), buf.shape, buf.dtype, None), store)


def where(cond: Tensor, a: Any, b: Any) -> Tensor:
    """``WHERE(cond, a, b)`` with arg ``None`` (_functional.py where; used by relu)."""
    a_t = _to_tensor(a, cond._store)
    b_t = _to_tensor(b, cond._store)
    shape = _bshape(cond.shape, a_t.shape, b_t.shape)
    return Tensor(Node("WHERE", (cond._uop, a_t._uop, b_t._uop), shape,
                       _promote(a_t.dtype, b_t.dtype), None), cond._store)


def exp(x: Tensor) -> Tensor:
    return x.exp()


def relu(x: Tensor) -> Tensor:
    zero = Tensor(Node("CONST", (), (), x.dtype, {"value": 0.0}), x._store)
    return where(x > zero, x, zero)


def tanh(x: Tensor) -> Tensor:
    e_pos = x.exp()
    e_neg = (-x).exp()
    return (e_pos - e_neg) / (e_pos + e_neg)


def gelu(x: Tensor) -> Tensor:
    c = (2.0 / np.pi) ** 0.5
    one = _to_tensor(1.0, x._store)
    return 0.5 * x * (one + tanh(_to_tensor(c, x._store) * (x + 0.044715 * x * x * x)))


def softmax(x: Tensor, dim: int = -1) -> Tensor:
    x_max = x.max(axis=dim, keepdims=True)
    e = (x - x_max).exp()
    return e / e.sum(axis=dim, keepdims=True)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    out = x @ weight.T
    if bias is not None:
        out = out + bias
    return out


def layer_norm(x: Tensor, normalized_shape: Sequence[int], weight: Optional[Tensor] = None,
               bias: Optional[Tensor] = None, eps: float = 1e-5) -> Tensor:
    ns = (int(normalized_shape),) if isinstance(normalized_shape, int) \
        else tuple(int(d) for d in normalized_shape)
    if x.shape[-len(ns):] != ns:
        raise ValueError("layer_norm: trailing shape does not match normalized_shape")
    cols = int(np.prod(ns))
    rows = int(np.prod(x.shape) // cols)
    w = weight if weight is not None else from_numpy(np.ones(ns, np.float32), x._store)
    b = bias if bias is not None else from_numpy(np.zeros(ns, np.float32), x._store)
    arg = {"normalized_shape": ns, "rows": rows, "cols": cols, "eps": float(eps)}
    return Tensor(Node("LAYER_NORM", (x._uop, w._uop, b._uop), x.shape, x.dtype, arg), x._store)


def cross_entropy(logits: Tensor, target: Tensor, weight: Optional[Tensor] = None, reduction: str = "mean",
                  ignore_index: int = -100, label_smoothing: float = 0.0) -> Tensor:
    """Cross entropy over axis 1 of ``[N, C, ...]`` logits (axis 0 of ``[C]``), for int64 class-index targets or
    probability targets of the logits' shape, with optional class weights ``[C]`` and label smoothing.

    Mirrors the node the reference emits (_functional.py:178-262; contract inference
    _framework_contracts.py:3470-3610): a target whose shape equals the logits' selects the
    probability mode; the weights travel as a third input.
    """
    if reduction not in ("mean", "sum", "none"):
        raise ValueError(f"cross_entropy: reduction {reduction!r}")
    if logits.ndim < 1:
        raise ValueError("cross_entropy: logits need a class axis")
    mode = "probabilities" if target.shape == logits.shape else "indices"
    positions = logits.shape[:1] + logits.shape[2:] if logits.ndim > 1 else ()
    if mode == "indices":
        if target.dtype != "int64":
            raise ValueError("cross_entropy: class-index targets must be int64")
        if target.shape != positions:
            raise ValueError("cross_entropy: target shape does not match logits")
    elif target.dtype != logits.dtype:
        raise ValueError("cross_entropy: probability targets must have the logits' dtype")
    n_class = logits.shape[1] if logits.ndim > 1 else logits.shape[0]
    if weight is not None and (weight.shape != (n_class,) or weight.dtype != logits.dtype):
        raise ValueError("cross_entropy: weight must be a [C] tensor of the logits' dtype")
    if not 0.0 <= float(label_smoothing) <= 1.0:
        raise ValueError("cross_entropy: label_smoothing must be in [0, 1]")
    out_shape = positions if reduction == "none" else ()
    arg = {"reduction": reduction, "batch_rank": 0, "ignore_index": int(ignore_index),
           "has_weight": weight is not None, "label_smoothing": float(label_smoothing), "target_mode": mode}
    inputs = (logits._uop, target._uop) + ((weight._uop,) if weight is not None else ())
    return Tensor(Node("CROSS_ENTROPY", inputs, out_shape, logits.dtype, arg), logits._store)


def scaled_dot_product_attention(q: Tensor, k: Tensor, v: Tensor, attn_mask: Any = None,
                                 is_causal: bool = False, scale: Optional[float] = None) -> Tensor:
    s = (1.0 / np.sqrt(q.shape[-1])) if scale is None else float(scale)
    scores = q @ k.transpose(-1, -2)
    scores = scores * from_numpy(np.full(scores.shape, s, dtype=np.float32), q._store)
    if is_causal:
        l_q, l_k = scores.shape[-2], scores.shape[-1]
        mask = np.triu(np.ones((l_q, l_k), dtype=bool), k=1)
        scores = scores.masked_fill(from_numpy(mask, q._store), -np.inf)
    if attn_mask is not None:
        m = _to_tensor(attn_mask, q._store)
        scores = scores.masked_fill(m, -np.inf) if m.dtype == "bool" else scores + m
    return softmax(scores, dim=-1) @ v


def attention_forward(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """Typed non-causal attention node (packages/browsergrad-jit/src/python/index.ts:212-245)."""
    if not (q.ndim == k.ndim == v.ndim == 4):
        raise ValueError("attention_forward: [B,H,S,D] tensors required")
    if q.dtype != "float32" or k.shape[:2] != q.shape[:2] or v.shape != k.shape \
            or k.shape[-1] != q.shape[-1]:
        raise ValueError("attention_forward: float32 tensors with matching batch/head/depth")
    scale = float(np.float32(1.0 / np.sqrt(q.shape[-1])))
    return Tensor(Node("ATTENTION_FORWARD", (q._uop, k._uop, v._uop), q.shape, "float32",
                       {"scale": scale, "mask": "none"}), q._store)


def sort(x: Tensor, dim: int = -1, descending: bool = False, *, stable: bool = False) -> Tuple[Tensor, Tensor]:
    """``(values, indices)`` as ``SORT_VALUES(x, SORT_INDICES(x))`` (_tensor_proxy.py:2558-2628); the order is
    always the stable one (equal values keep their original order, ascending or descending)."""
    axis = int(dim) % max(x.ndim, 1)
    arg = {"axis": axis, "descending": bool(descending), "stable": bool(stable)}
    idx = Node("SORT_INDICES", (x._uop,), x.shape, "int64", dict(arg))
    val = Node("SORT_VALUES", (x._uop, idx), x.shape, x.dtype, dict(arg))
    return x._wrap(val), x._wrap(idx)


def topk(x: Tensor, k: int, dim: Any = None, largest: bool = True, sorted: bool = True) -> Tuple[Tensor, Tensor]:
    """``(values, indices)`` as ``TOPK_VALUES(x, TOPK_INDICES(x))`` (_tensor_proxy.py:2630-2701)."""
    axis = (x.ndim - 1 if dim is None else int(dim)) % max(x.ndim, 1)
    k = int(k)
    if k < 0 or k > x.shape[axis]:
        raise ValueError(f"topk: k={k} outside [0, {x.shape[axis]}]")
    out_shape = tuple(k if i == axis else d for i, d in enumerate(x.shape))
    arg = {"axis": axis, "k": k, "largest": bool(largest), "sorted": bool(sorted)}
    idx = Node("TOPK_INDICES", (x._uop,), out_shape, "int64", dict(arg))
    val = Node("TOPK_VALUES", (x._uop, idx), out_shape, x.dtype, dict(arg))
    return x._wrap(val), x._wrap(idx)


def cumsum(x: Tensor, dim: int = 0, *, dtype: Any = None) -> Tensor:
    """``CUMSUM`` node (_tensor_proxy.py:2512-2545): running sum along ``dim`` in ``dtype`` (the input's
    dtype when not given; bool and small integers accumulate as int64, as the reference normalises)."""
    axis = int(dim) % x.ndim
    if dtype is None:
        out_dtype = "int64" if x.dtype in ("bool", "int8", "int16", "int32", "uint8", "uint16", "uint32") else x.dtype
    else:
        out_dtype = np.dtype(dtype).name if not isinstance(dtype, str) else dtype
    return x._wrap(Node("CUMSUM", (x._uop,), x.shape, out_dtype, {"axis": axis, "reverse": False}))


def cat(tensors: Sequence[Tensor], dim: int = 0) -> Tensor:
    """``CONCAT`` node (_tensor_proxy.py:2328-2389): inputs agree off ``dim``; the result dtype is NumPy's
    promotion of the input dtypes."""
    ts = tuple(tensors)
    if not ts:
        raise ValueError("cat: empty tensor list")
    rank = ts[0].ndim
    axis = int(dim) % rank
    for t in ts[1:]:
        if t.ndim != rank or any(a != b for i, (a, b) in enumerate(zip(t.shape, ts[0].shape)) if i != axis):
            raise ValueError("cat: inputs must agree on every dimension but the concatenated one")
    out_shape = tuple(sum(t.shape[axis] for t in ts) if i == axis else d for i, d in enumerate(ts[0].shape))
    out_dtype = np.result_type(*[np.dtype(t.dtype) if t.dtype != "bfloat16" else np.float32 for t in ts]).name \
        if len({t.dtype for t in ts}) > 1 else ts[0].dtype
    return ts[0]._wrap(Node("CONCAT", tuple(t._uop for t in ts), out_shape, out_dtype, {"axis": axis}))


def pad(x: Tensor, pad: Sequence[int], mode: str = "constant", value: Any = None) -> Tensor:
    """``PAD`` node of ``F.pad`` (_functional.py:1397-1417): ``pad`` lists (before, after) pairs from the
    LAST axis backwards; constant mode only; the fill value is normalised to the input dtype
    (_framework_contracts.py:4694-4726, :4756-4791)."""
    if mode != "constant":
        raise ValueError(f"pad: mode {mode!r} is not supported; expected 'constant'")
    if len(pad) % 2 != 0 or len(pad) // 2 > x.ndim:
        raise ValueError("pad: an even number of widths, at most two per dimension")
    width = [(0, 0)] * x.ndim
    for i in range(len(pad) // 2):
        lo, hi = int(pad[2 * i]), int(pad[2 * i + 1])
        if lo < 0 or hi < 0:
            raise ValueError("pad: negative padding is not supported")
        width[x.ndim - 1 - i] = (lo, hi)
    if x.dtype == "bool":
        fill: Any = bool(value) if value is not None else False
    elif x.dtype.startswith("float"):
        fill = float(np.asarray(0 if value is None else value, dtype=np.dtype(x.dtype)).item())
        fill = 0.0 if fill == 0.0 else fill
    else:
        fill = int(0 if value is None else value)
    out_shape = tuple(d + lo + hi for d, (lo, hi) in zip(x.shape, width))
    return x._wrap(Node("PAD", (x._uop,), out_shape, x.dtype, {"pad_width": tuple(width), "mode": "constant", "value": fill}))


def stack(tensors: Sequence[Tensor], dim: int = 0) -> Tensor:
    """``STACK`` node (_tensor_proxy.py:2391-2449): equal shapes, a new axis at ``dim``."""
    ts = tuple(tensors)
    if not ts:
        raise ValueError("stack: empty tensor list")
    if any(t.shape != ts[0].shape for t in ts[1:]):
        raise ValueError("stack: inputs must have equal shapes")
    axis = int(dim) % (ts[0].ndim + 1)
    out_shape = ts[0].shape[:axis] + (len(ts),) + ts[0].shape[axis:]
    out_dtype = np.result_type(*[np.dtype(t.dtype) for t in ts]).name if len({t.dtype for t in ts}) > 1 else ts[0].dtype
    return ts[0]._wrap(Node("STACK", tuple(t._uop for t in ts), out_shape, out_dtype, {"axis": axis}))


def toposort(root: Node) -> list:
    """Leaves-first order by iterative DFS keyed on identity (_ir.py:403-430)."""
    order: list = []
    seen: set = set()
    stack = [(root, 0)]
    while stack:
        node, i = stack[-1]
        if id(node) in seen:
            stack.pop()
            continue
        if i < len(node.inputs):
            stack[-1] = (node, i + 1)
            child = node.inputs[i]
            if id(child) not in seen:
                stack.append((child, 0))
            continue
        seen.add(id(node))
        order.append(node)
        stack.pop()
    return order


def narrow(t: Tensor, axis: int, start: int, length: int) -> Tensor:
    return t.narrow(axis, start, length)


def take_slice(t: Tensor, slices: Sequence[Any]) -> Tensor:
    return t.slice(slices)
