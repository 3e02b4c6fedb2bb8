"""Reverse-mode autograd over the path's operations: which kernels a backward pass runs, as wired by the
reference's operations (not a general graph engine -- Neureka's GraphNode stays the caller in production).

ADAction recipes (reference file:line):
 * "x": error -> XConvRight(error, otherOperand, zeros(shape_d))   (operations/linear/Convolution.java:56-89)
 * activations and same-shape operators: local derivative computed eagerly at forward time, backward is
   error * derivative                                  (template/algorithms/FallbackAlgorithm.java:118-129)
 * broadcasting + / -: the Broadcast implementation with d >= 0 = reduction of the error over the broadcast
   dims                                                (operations/operator/Addition.java:90-110)
 * broadcasting *: the reference multiplies the error with the other operand broadcast to the output shape and
   does NOT reduce back (operations/operator/Multiplication.java:51-71; no reference test pins it). Here the
   product is reduced to the operand's shape (handle*drain summed over the broadcast dims), the mathematical
   gradient, using the same reduction kernel.
 * sumItems: the scalar error becomes a virtual tensor of the input's shape (algorithms/SumAlgorithm.java:29-33)
 * gradient accumulation: g <- g + e = one "+" kernel and one assign kernel (math/Functions.java:74,
   TensorImpl.java:1275-1300)
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import numpy as np

from . import _lib as L
from . import backend as B
from . import functions as F
from .backend import ExecutionCall
from .tensor import Tensor


class GraphNode:
    """The payload's place in the computation graph: parents + one ADAction per differentiable parent."""

    def __init__(self, payload: Tensor, parents: List[Tuple[Tensor, Callable[[Tensor], Tensor]]]):
        self.payload = payload
        self.parents = parents  # (input tensor, error -> error for that input)


def _tracks(t: Tensor) -> bool:
    return t.rqs_gradient or t.graph_node is not None


def _mul(a: Tensor, b: Tensor) -> Tensor:
    return F.run_operator("*", a, b)


def _derive_operator(sym: str, a: Tensor, b: Tensor, d: int) -> Tensor:
    """f.executeDerive(inputs, d) for a flat binary operator."""
    return F.run_operator(sym, a, b, d)


def _broadcast_reduce(sym_op: int, target_like: Tensor, handle: Tensor, error: Tensor, d: int) -> Tensor:
    dev = error.device or target_like.device or handle.device
    origin = Tensor.of(target_like.dtype, target_like.shape, 0).set_is_virtual(False)
    dev.store(origin)
    t = F.make_fit([origin, handle, error])
    impl = B.CudaBroadcast(sym_op)
    call = ExecutionCall([t[0], t[1], t[2]], "broadcast-backward", dev, d)
    F._execute_on_common_device(call, impl)
    return origin


def _record_operator(sym: str, a: Tensor, b: Tensor, out: Tensor) -> None:
    algo = F.choose_algorithm(a, b)
    parents = []
    for d, (t, other) in enumerate(((a, b), (b, a))):
        if not _tracks(t):
            continue
        if sym == "x":
            shape, dtype = t.shape, t.dtype

            def action(err, other=other, shape=shape, dtype=dtype):
                zeros = Tensor.of(dtype, shape, 0).set_is_virtual(False)
                return F.run_xconv("x»", err, other, zeros)
            parents.append((t, action))
        elif algo == B.BROADCAST or (algo == B.BI_SCALAR_BROADCAST and a.shape != b.shape):
            fa, fb = F.make_fit([a, b]) if a.rank != b.rank else (a, b)
            mine, oth = (fa, fb) if d == 0 else (fb, fa)
            if sym in ("+", "-"):
                def action(err, mine=mine, oth=oth, d=d, sym=sym):
                    handle = Tensor.of(oth.dtype, oth.shape, 0).set_is_virtual(False)
                    return _reshape_like(_broadcast_reduce(L.OPS[sym], mine, handle, err, d), mine)
                parents.append((t, action))
            elif sym == "*":
                def action(err, mine=mine, oth=oth):
                    return _reshape_like(_broadcast_reduce(L.NK_OP_MUL_BOTH, mine, oth, err, 0), mine)
                parents.append((t, action))
            else:
                deriv = _derive_operator(sym, fa, fb, d)   # output-shaped local derivative

                def action(err, mine=mine, deriv=deriv):
                    ones = Tensor.of(deriv.dtype, deriv.shape, 1).set_is_virtual(False)
                    return _reshape_like(_broadcast_reduce(L.NK_OP_MUL_BOTH, mine, _mul(err, deriv), ones, 0), mine)
                parents.append((t, action))
        else:
            deriv = _derive_operator(sym, a, b, d)
            deriv.is_intermediate = False

            def action(err, deriv=deriv):
                return _mul(err, deriv)
            parents.append((t, action))
    if parents:
        out.graph_node = GraphNode(out, parents)


def _record_matmul(a: Tensor, b: Tensor, out: Tensor) -> None:
    """MatMulAlgorithm's ADAction (algorithms/MatMulAlgorithm.java:37-59): the gradient of the first operand is
    error @ transpose(second), of the second transpose(first) @ error. The reference deep-copies the transposed
    operand to get a simple configuration; the kernels here read the transposed view directly."""
    parents = []
    if _tracks(a):
        parents.append((a, lambda err, b=b: F.run_matmul(err, b.T)))
    if _tracks(b):
        parents.append((b, lambda err, a=a: F.run_matmul(a.T, err)))
    if parents:
        out.graph_node = GraphNode(out, parents)


def _reshape_like(g: Tensor, like: Tensor) -> Tensor:
    return g


def _record_function(fid: str, x: Tensor, out: Tensor) -> None:
    if not _tracks(x):
        return
    if fid == "sumItems":
        def action(err, x=x):
            dev = err.device
            value = float(dev.access(err).read_at(0))
            full = Tensor.of(x.dtype, x.shape, value)   # virtual
            dev.store(full)
            return full
        out.graph_node = GraphNode(out, [(x, action)])
        return
    deriv = F.run_function(fid, x, 0)   # eager local derivative (FallbackAlgorithm.java:118-129)
    deriv.is_intermediate = False

    def action(err, deriv=deriv):
        return _mul(err, deriv)
    out.graph_node = GraphNode(out, [(x, action)])


def dot(a: Tensor, b: Tensor) -> Tensor:
    """a.dot(b) with its ADActions: the gradient of either vector is the error times the other one, which is what the
    convolution's recipe yields for two equal shapes (Convolution.java:56-89 -> XConvRight(error, other, zeros))."""
    out = F.run_dot(a, b)
    _record_operator("x", a, b, out)
    return out


def extreme(x: Tensor, want_max: bool) -> Tensor:
    """x.min() / x.max(): Min.java:44-66 -- the ADAction builds a zero tensor of the input's shape and puts the (one
    element) error at the index of the extreme item."""
    out, index = F.run_extreme(want_max, x)
    if _tracks(x):
        def action(err, x=x, index=index):
            dev = err.device or x.device
            g = Tensor.of(x.dtype, x.shape, 0).set_is_virtual(False)
            dev.store(g)
            value = float(dev.access(err).read_at(0))
            dev.access(g).write(value).at(g.ndconf.index_of_index(index))
            return g
        out.graph_node = GraphNode(out, [(x, action)])
    return out


def evaluate(node, inputs: List[Tensor], do_ad: bool) -> Tensor:
    """Executes an expression tree bottom-up (no fusion), recording ADActions when do_ad."""
    if node.kind == "input":
        if node.value >= len(inputs):
            raise ValueError(f"function needs input {node.value} but only {len(inputs)} were given")
        return inputs[node.value]
    if node.kind == "const":
        like = inputs[0]
        return Tensor.of(like.dtype, (1,), [node.value])
    if node.kind == "fun":
        x = evaluate(node.children[0], inputs, do_ad)
        out = F.run_function(node.value, x)
        if do_ad:
            _record_function(node.value, x, out)
        return out
    sym = node.value
    vals = [evaluate(c, inputs, do_ad) for c in node.children]
    if sym in ("«x", "x»"):
        if len(vals) != 3:
            raise ValueError(f"'{sym}' needs exactly three operands")
        return F.run_xconv(sym, *vals)
    acc = vals[0]
    if sym == "@":
        for nxt in vals[1:]:   # ((a @ b) @ c) ..., MatMul.reducePairwise (linear/MatMul.java:48-63)
            out = F.run_matmul(acc, nxt)
            if do_ad:
                _record_matmul(acc, nxt, out)
            acc = out
        return acc
    for nxt in vals[1:]:   # pairwise, left nested
        out = F.run_conv(acc, nxt) if sym == "x" else F.run_operator(sym, acc, nxt)
        if do_ad:
            fa, fb = (F.make_fit([acc, nxt]) if (sym == "x" and acc.rank != nxt.rank) else (acc, nxt))
            _record_operator(sym, fa, fb, out)
            if out.graph_node is not None and sym == "x" and (fa is not acc or fb is not nxt):
                # the recorded parents are rank-padded views; route their errors to the real tensors
                out.graph_node.parents = [((acc if p is fa else nxt), act) for p, act in out.graph_node.parents]
        acc = out
    return acc


def _accumulate(t: Tensor, err: Tensor) -> None:
    """TensorImpl.addToGradient (:1275-1300): first error becomes the gradient, later ones are added in place."""
    if t.gradient is None:
        g = Tensor.of(t.dtype, t.shape, 0).set_is_virtual(False)
        dev = err.device
        dev.store(g)
        if err.shape != t.shape:
            err = _view_as(err, t.shape)
        F.assign(g, err)
        t.gradient = g
    else:
        if err.shape != t.shape:
            err = _view_as(err, t.shape)
        s = F.run_operator("+", t.gradient, err)
        F.assign(t.gradient, s)


def _view_as(err: Tensor, shape) -> Tensor:
    """Same elements, other (rank-padded / trimmed) shape."""
    if int(np.prod(shape)) != err.size:
        raise ValueError(f"gradient of shape {err.shape} does not fit a tensor of shape {tuple(shape)}")
    from .ndconf import NDConfiguration
    err.set_is_virtual(False)
    v = Tensor(err.dtype, NDConfiguration.of_shape(shape), err._host)
    v._parent = err
    if err.device is not None:
        v._attach(err._data, err.device)
        err.device._stored.add(v)
    if not err.ndconf.is_simple():
        raise NotImplementedError("re-viewing a non-simple error tensor")
    return v


def backward(result: Tensor, error: Optional[Tensor] = None) -> None:
    """Tensor.backward(error) (autograd/GraphNode.java:409-440): reverse traversal, errors of all consumers are
    summed before a node propagates further."""
    if error is None:
        error = Tensor.of(result.dtype, result.shape, 1)
    dev = result.device or error.device
    if dev is None:
        raise ValueError("backward needs the result on a CudaDevice")
    if error.device is None:
        dev.store(error)
    # topological order
    order, seen = [], set()

    def visit(t: Tensor):
        if id(t) in seen:
            return
        seen.add(id(t))
        if t.graph_node is not None:
            for p, _ in t.graph_node.parents:
                visit(p)
        order.append(t)
    visit(result)
    pending = {id(result): error}
    for t in reversed(order):
        err = pending.pop(id(t), None)
        if err is None:
            continue
        if t.rqs_gradient:
            _accumulate(t, err)
        if t.graph_node is None:
            continue
        for p, act in t.graph_node.parents:
            e = act(err)
            if id(p) in pending:
                pending[id(p)] = F.run_operator("+", pending[id(p)], e)
            else:
                pending[id(p)] = e
