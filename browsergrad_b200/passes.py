"""Graph passes the reference runs before realization, restated over duck-typed nodes.

``browsergrad_jit._realize.realize`` runs ``insert_cast_pass`` then ``fuse`` then ``toposort``
(packages/browsergrad-jit/src/python/_realize.py:1890-1902).  The CUDA front keeps that order so
that the plan it puts on the wire is the graph the reference's NumPy realizer would execute.
Both passes here rebuild nodes with ``type(node)(op=..., inputs=..., shape=..., dtype=...,
arg=...)`` and therefore work on the reference's ``UOp`` and on ``graph.Node`` alike.

* ``insert_cast_pass`` follows packages/browsergrad-jit/src/python/_amp.py:183-261
  (allow-list MATMUL -> f16 inputs and output; block-list EXP/LOG/REDUCE/DIV/FUSED_SOFTMAX ->
  f32; ADD/MUL/NEG/WHERE/PAD follow their inputs).  ``bfloat16`` hints are an extension: the
  same rewrite with dtype ``bfloat16``.
* ``fuse`` follows packages/browsergrad-jit/src/python/_fusion.py:413-517: softmax template
  first (:273-351), then single-consumer same-shape chains of ADD/MUL/DIV/NEG/EXP/LOG
  (:141-181, :184-232), then one substitution walk that does not rebuild the inputs of a
  substituted node (:369-405).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Set, Tuple

from .errors import JitNotImplementedError
from .graph import toposort

ELEMENTWISE_OPS = frozenset({"ADD", "MUL", "DIV", "NEG", "EXP", "LOG"})
_ALLOW_NARROW = frozenset({"MATMUL"})
_BLOCK_F32 = frozenset({"EXP", "LOG", "REDUCE", "DIV", "FUSED_SOFTMAX"})
_PROMOTE = frozenset({"ADD", "MUL", "NEG", "WHERE", "PAD"})
_NARROW = ("float16", "bfloat16")


def _mk(like: Any, op: str, inputs: Tuple[Any, ...], shape: Tuple[int, ...], dtype: str,
        arg: Any) -> Any:
    return type(like)(op=op, inputs=inputs, shape=shape, dtype=dtype, arg=arg)


def _hint(arg: Any) -> Optional[str]:
    if isinstance(arg, dict):
        h = arg.get("autocast_hint")
        if h in _NARROW:
            return h
    return None


def _cast_to(node: Any, dtype: str) -> Any:
    if node.dtype == dtype:
        return node
    return _mk(node, "CAST", (node,), node.shape, dtype, {"dtype": dtype, "amp_inserted": True})


def insert_cast_pass(root: Any) -> Any:
    nodes = toposort(root)
    if not any(_hint(n.arg) for n in nodes):
        return root
    new: Dict[int, Any] = {}
    for node in nodes:
        if not node.inputs:
            new[id(node)] = node
            continue
        ins = tuple(new.get(id(i), i) for i in node.inputs)
        hint = _hint(node.arg)
        if hint and node.op in _ALLOW_NARROW:
            out = _mk(node, node.op, tuple(_cast_to(i, hint) for i in ins), node.shape, hint,
                      node.arg)
        elif hint and node.op in _BLOCK_F32:
            out = _mk(node, node.op, tuple(_cast_to(i, "float32") for i in ins), node.shape,
                      "float32", node.arg)
        elif hint and node.op in _PROMOTE:
            target = "float32" if any(i.dtype == "float32" for i in ins) else ins[0].dtype
            out = _mk(node, node.op, tuple(_cast_to(i, target) for i in ins), node.shape, target,
                      node.arg)
        elif all(a is b for a, b in zip(ins, node.inputs)):
            out = node
        else:
            out = _mk(node, node.op, ins, node.shape, node.dtype, node.arg)
        new[id(node)] = out
    return new.get(id(root), root)


def _consumers(nodes: List[Any]) -> Dict[int, List[Any]]:
    cons: Dict[int, List[Any]] = {}
    for n in nodes:
        cons.setdefault(id(n), [])
        for i in n.inputs:
            cons.setdefault(id(i), []).append(n)
    return cons


def _arg_get(node: Any, key: str) -> Any:
    return node.arg.get(key) if isinstance(node.arg, dict) else None


def _match_softmax(div: Any, cons: Dict[int, List[Any]], done: Set[int]) -> Optional[Tuple]:
    if div.op != "DIV" or id(div) in done or len(div.inputs) != 2:
        return None
    e, s = div.inputs
    if e.op != "EXP" or s.op != "REDUCE" or id(e) in done or id(s) in done:
        return None
    if _arg_get(s, "op") != "sum" or not _arg_get(s, "keepdims") or tuple(s.inputs) != (e,):
        return None
    ec = cons.get(id(e), [])
    if len(ec) != 2 or {c.op for c in ec} != {"DIV", "REDUCE"} or len(e.inputs) != 1:
        return None
    add = e.inputs[0]
    if add.op != "ADD" or len(add.inputs) != 2 or id(add) in done:
        return None
    x, neg = add.inputs
    if neg.op != "NEG":
        x, neg = neg, x
    if neg.op != "NEG" or len(neg.inputs) != 1:
        return None
    mx = neg.inputs[0]
    if mx.op != "REDUCE" or _arg_get(mx, "op") != "max" or not _arg_get(mx, "keepdims"):
        return None
    if tuple(mx.inputs) != (x,) or _arg_get(mx, "axis") != _arg_get(s, "axis"):
        return None
    for n in (mx, neg, add, s):
        if len(cons.get(id(n), [])) != 1:
            return None
    return (mx, neg, add, e, s, div, x, _arg_get(mx, "axis"))


def _chain(start: Any, cons: Dict[int, List[Any]], done: Set[int]) -> Optional[List[Any]]:
    if start.op not in ELEMENTWISE_OPS or id(start) in done:
        return None
    chain = [start]
    cur = start
    while True:
        cl = cons.get(id(cur), [])
        if len(cl) != 1:
            break
        nxt = cl[0]
        if nxt.op not in ELEMENTWISE_OPS or id(nxt) in done:
            break
        if tuple(nxt.shape) != tuple(cur.shape) or nxt.dtype != cur.dtype:
            break
        chain.append(nxt)
        cur = nxt
    return chain if len(chain) >= 2 else None


def _fused_chain_node(chain: List[Any]) -> Any:
    ext: List[Any] = []
    ext_ref: Dict[int, int] = {}
    step: Dict[int, int] = {}

    def ref(n: Any) -> int:
        if id(n) in step:
            return step[id(n)]
        if id(n) not in ext_ref:
            ext_ref[id(n)] = -(len(ext) + 1)
            ext.append(n)
        return ext_ref[id(n)]

    ops = []
    for i, n in enumerate(chain):
        lhs = ref(n.inputs[0])
        rhs = ref(n.inputs[1]) if len(n.inputs) == 2 else None
        ops.append((n.op, lhs, rhs))
        step[id(n)] = i
    last = chain[-1]
    return _mk(last, "FUSED_ELEMENTWISE", tuple(ext), last.shape, last.dtype, {"ops": tuple(ops)})


def _substitute(root: Any, subs: Dict[int, Any]) -> Any:
    if not subs:
        return root
    rebuilt: Dict[int, Any] = {}
    # Iterative post-order so deep graphs do not hit the recursion limit.
    stack = [(root, False)]
    while stack:
        node, expanded = stack.pop()
        if id(node) in rebuilt:
            continue
        if id(node) in subs:
            rebuilt[id(node)] = subs[id(node)]
            continue
        if not node.inputs:
            rebuilt[id(node)] = node
            continue
        if not expanded:
            stack.append((node, True))
            for inp in node.inputs:
                if id(inp) not in rebuilt:
                    stack.append((inp, False))
            continue
        ins = tuple(rebuilt[id(i)] for i in node.inputs)
        if all(a is b for a, b in zip(ins, node.inputs)):
            rebuilt[id(node)] = node
        else:
            rebuilt[id(node)] = _mk(node, node.op, ins, node.shape, node.dtype, node.arg)
    return rebuilt[id(root)]


def fuse(root: Any) -> Any:
    nodes = toposort(root)
    cons = _consumers(nodes)
    done: Set[int] = set()
    subs: Dict[int, Any] = {}
    for node in nodes:
        m = _match_softmax(node, cons, done)
        if m is None:
            continue
        mx, neg, add, e, s, div, x, axis = m
        subs[id(div)] = _mk(div, "FUSED_SOFTMAX", (x,), div.shape, div.dtype, {"axis": axis})
        for n in (mx, neg, add, e, s, div):
            done.add(id(n))
    for node in nodes:
        if id(node) in done or node.op not in ELEMENTWISE_OPS:
            continue
        is_root = True
        for inp in node.inputs:
            if inp.op in ELEMENTWISE_OPS and id(inp) not in done \
                    and len(cons.get(id(inp), [])) == 1:
                is_root = False
                break
        if not is_root:
            continue
        chain = _chain(node, cons, done)
        if chain is None:
            continue
        subs[id(chain[-1])] = _fused_chain_node(chain)
        for n in chain:
            done.add(id(n))
    return _substitute(root, subs)


def prepare(root: Any, *, fusion: bool = True) -> Any:
    """Cast pass then fusion, the order of ``_realize.realize`` (_realize.py:1890-1893)."""
    root = insert_cast_pass(root)
    return fuse(root) if fusion else root


def _rebuild(root: Any, rewrite) -> Any:
    """Bottom-up rewrite of a graph: ``rewrite(node, new_inputs)`` returns the replacement node."""
    done = {}
    for node in toposort(root):
        ins = tuple(done[id(i)] for i in node.inputs)
        done[id(node)] = rewrite(node, ins)
    return done[id(root)]


def lower_composites(root: Any) -> Any:
    """Rewrites CLAMP, VAR and STACK into opcodes the CUDA plan compiler schedules, with NumPy's
    evaluation order, so that they fuse with their neighbours like any other elementwise / reduce
    chain (the reference evaluates them with one NumPy call each, _realize.py:254-260, :299-306,
    :346-357):

    * ``CLAMP(x; lo, hi)`` -> ``where(t > hi, hi, t)`` with ``t = where(x < lo, lo, x)`` -- ``np.clip``
      for floats, NaN passes through both comparisons;
    * ``VAR(x; axes, correction)`` -> ``sum((x - mean(x))**2) / max(n - correction, 0)`` with the mean kept
      in the result dtype -- the two passes of ``np.var(dtype=...)``;
    * ``STACK`` -> ``CONCAT`` of the inputs reshaped with a unit axis;
    * ``REPEAT`` / ``REPEAT_INTERLEAVE`` -> ``RESHAPE`` / ``BROADCAST_TO`` / ``RESHAPE`` (``np.tile`` / ``np.repeat``,
      _realize.py:329-332, :360-363);
    * ``SORT_VALUES`` / ``TOPK_VALUES`` -> ``INDEX`` along the ordering axis (_realize.py:1149-1176);
    * ``PROD`` -> ``REDUCE`` with the product combiner (``np.prod(dtype=...)``, _realize.py:335-343);
    * ``PAD`` -> one ``CONCAT`` per padded axis whose outer inputs are the broadcast fill constant
      (``np.pad(mode="constant")``, _realize.py:1131-1140);
    * ``NARROW(x; axis, start, length)`` -> ``SLICE`` with one slice per axis (_realize.py:309-314): a strided
      view on the device, where the reference copies.
    """
    def make(like: Any, op: str, inputs: tuple, shape: tuple, dtype: str, arg: Any) -> Any:
        return type(like)(op=op, inputs=inputs, shape=tuple(shape), dtype=dtype, arg=arg)

    def rewrite(node: Any, ins: tuple) -> Any:
        if node.op == "CLAMP":
            (x,) = ins
            if node.dtype not in ("float16", "float32", "float64", "bfloat16"):
                raise JitNotImplementedError("CUDA realizer: CLAMP of a non-floating tensor is not supported. "
                                             "Fall back to bg.realize() (NumPy).")
            out = x
            lo, hi = node.arg.get("min"), node.arg.get("max")
            if lo is not None:
                c = make(node, "CONST", (), (), node.dtype, {"value": float(lo)})
                cmp = make(node, "CMP", (out, c), node.shape, "bool", {"op": "lt"})
                out = make(node, "WHERE", (cmp, c, out), node.shape, node.dtype, None)
            if hi is not None:
                c = make(node, "CONST", (), (), node.dtype, {"value": float(hi)})
                cmp = make(node, "CMP", (out, c), node.shape, "bool", {"op": "gt"})
                out = make(node, "WHERE", (cmp, c, out), node.shape, node.dtype, None)
            return out
        if node.op == "VAR":
            (x,) = ins
            axes = tuple(int(a) for a in node.arg["axes"])
            keep = bool(node.arg.get("keepdims", False))
            n = 1
            for a in axes:
                n *= int(x.shape[a])
            kept = tuple(1 if i in axes else d for i, d in enumerate(x.shape))
            mean = make(node, "REDUCE", (x,), kept, node.dtype, {"op": "mean", "axis": axes, "keepdims": True})
            neg = make(node, "NEG", (mean,), kept, node.dtype, None)
            centered = make(node, "ADD", (x, neg), x.shape, node.dtype, None)
            sq = make(node, "MUL", (centered, centered), x.shape, node.dtype, None)
            total = make(node, "REDUCE", (sq,), node.shape, node.dtype, {"op": "sum", "axis": axes, "keepdims": keep})
            count = make(node, "CONST", (), (), node.dtype, {"value": float(max(n - int(node.arg.get("correction", 1)), 0))})
            return make(node, "DIV", (total, count), node.shape, node.dtype, None)
        if node.op == "PROD":
            (x,) = ins
            if node.dtype not in ("float32", "float64", "int64"):
                raise JitNotImplementedError("CUDA realizer: PROD of a " + node.dtype + " tensor is not supported. "
                                             "Fall back to bg.realize() (NumPy).")
            return make(node, "REDUCE", (x,), node.shape, node.dtype,
                        {"op": "prod", "axis": tuple(int(a) for a in node.arg["axes"]), "keepdims": bool(node.arg.get("keepdims", False))})
        if node.op == "PAD":
            (x,) = ins
            out = x
            shape = list(x.shape)
            fill = make(node, "CONST", (), (), node.dtype, {"value": node.arg["value"]})
            for axis, (lo, hi) in enumerate(node.arg["pad_width"]):
                if lo == 0 and hi == 0:
                    continue
                parts = []
                for extent in (int(lo), None, int(hi)):
                    if extent is None:
                        parts.append(out)
                    elif extent > 0:
                        blk = tuple(shape[:axis]) + (extent,) + tuple(shape[axis + 1:])
                        parts.append(make(node, "BROADCAST_TO", (fill,), blk, node.dtype, {"shape": blk}))
                shape[axis] += int(lo) + int(hi)
                out = make(node, "CONCAT", tuple(parts), tuple(shape), node.dtype, {"axis": axis})
            return out
        if node.op == "NARROW":
            (x,) = ins
            axis, start, length = int(node.arg["axis"]) % max(len(x.shape), 1), int(node.arg["start"]), int(node.arg["length"])
            slices = tuple(slice(start, start + length) if d == axis else slice(None) for d in range(len(x.shape)))
            return make(node, "SLICE", (x,), node.shape, node.dtype, {"slices": slices})
        if node.op == "STACK":
            axis = int(node.arg["axis"])
            parts = []
            for x in ins:
                shp = tuple(x.shape[:axis]) + (1,) + tuple(x.shape[axis:])
                parts.append(make(node, "RESHAPE", (x,), shp, x.dtype, {"new_shape": shp}))
            return make(node, "CONCAT", tuple(parts), node.shape, node.dtype, {"axis": axis})
        if node.op in ("SORT_VALUES", "TOPK_VALUES"):
            # np.take_along_axis(source, indices, axis): the gather opcode with the same axis
            return make(node, "INDEX", ins, node.shape, node.dtype, {"dim": int(node.arg["axis"])})
        if node.op in ("REPEAT", "REPEAT_INTERLEAVE"):
            # a unit axis beside every repeated one, broadcast to the factor, folded back: views until the final RESHAPE
            (x,) = ins
            if node.op == "REPEAT":
                reps = tuple(int(r) for r in node.arg["repeats"])
                padded = (1,) * (len(reps) - len(x.shape)) + tuple(x.shape)
                split = tuple(v for d in padded for v in (1, d))
                wide = tuple(v for r, d in zip(reps, padded) for v in (r, d))
            else:
                axis, r = int(node.arg["axis"]), int(node.arg["repeats"])
                split = tuple(x.shape[:axis + 1]) + (1,) + tuple(x.shape[axis + 1:])
                wide = tuple(x.shape[:axis + 1]) + (r,) + tuple(x.shape[axis + 1:])
            a = make(node, "RESHAPE", (x,), split, node.dtype, {"new_shape": split})
            b = make(node, "BROADCAST_TO", (a,), wide, node.dtype, {"shape": wide})
            return make(node, "RESHAPE", (b,), node.shape, node.dtype, {"new_shape": tuple(node.shape)})
        if node.op in ("PERMUTE", "RESHAPE", "BROADCAST_TO", "LOAD", "SLICE") and len(ins) == 1 and ins[0].dtype != node.dtype:
            # A view built outside the autocast block keeps the dtype its input had before the cast pass
            # narrowed it; the reference's realizer hands the narrow array through unchanged
            # (_realize.py:1114-1121), so the view carries its input's real dtype here.
            return make(node, node.op, ins, node.shape, ins[0].dtype, node.arg)
        if all(a is b for a, b in zip(ins, node.inputs)):
            return node
        return make(node, node.op, ins, node.shape, node.dtype, node.arg)

    return _rebuild(root, rewrite)
