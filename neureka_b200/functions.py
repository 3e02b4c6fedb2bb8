"""The caller side of the path: a small `Function` layer that parses Neureka expressions such as
"i0 x i1" or "tanh(i0*i1+i1)", prepares calls the way the reference's operations and algorithms do, and
dispatches them to the CUDA implementations registered in `backend.CudaBackend`.

Mirrored behaviour (reference file:line):
 * operator precedence = ServiceLoader order of the operations, tightest first: ** / * % - + x «x x»
   (src/main/resources/META-INF/services/neureka.backend.api.Operation, math/parsing/FunctionParser.java:144-197)
 * n-ary chains execute pairwise, left nested (operator/Addition.java `reducePairwise`, linear/Convolution.java:136-151)
 * nested functions are not fused: inner nodes are executed first (template/algorithms/AbstractDeviceAlgorithm.java:158-204)
 * algorithm choice for operators: BiScalarBroadcast if the 2nd operand has one element or is virtual
   (algorithms/BiScalarBroadcast.java:17-30), BiElementwise for equal shapes (BiElementwise.java:17-25), else
   Broadcast (Broadcast.java:18-46)
 * output shapes: conv |a-b|+1 (operations/ConvUtil.java:61-66), broadcast max per dim (Broadcast.java:76-95)
 * rank padding: Permute.makeFit (operations/other/Permute.java:82-110)
 * inputs that are not on the executing device are stored for the call and restored afterwards
   (AbstractDeviceAlgorithm.executeOnCommonDevice, :427-449)
There is no CPU execution in this package: a call needs at least one operand on a CudaDevice.
"""
from __future__ import annotations

import ctypes as C
import re
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib as L
from . import backend as B
from .backend import ExecutionCall
from .device import CudaDevice
from .ndconf import NDConfiguration
from .tensor import Tensor

# ---------------------------------------------------------------------------------------------------
# AST + parser
# ---------------------------------------------------------------------------------------------------
_PRECEDENCE = ["**", "/", "*", "%", "-", "+", "x", "«x", "x»", "@"]  # tightest first
_FUN_ALIASES = {name: name for name in L.FUN_IDS}   # the operation identifiers are the ScalarFun ids
_FUN_ALIASES["sumItems"] = "sumItems"


class Node:
    def __init__(self, kind: str, value=None, children: Optional[List["Node"]] = None):
        self.kind = kind          # "input" | "const" | "op" | "fun"
        self.value = value        # input index | constant | operator symbol | function id
        self.children = children or []

    def depends_on(self, i: int) -> bool:
        if self.kind == "input":
            return self.value == i
        return any(c.depends_on(i) for c in self.children)

    def __str__(self) -> str:
        if self.kind == "input":
            return f"I[{self.value}]"
        if self.kind == "const":
            return repr(self.value)
        if self.kind == "fun":
            return f"{self.value}({self.children[0]})"
        return "(" + f" {self.value} ".join(str(c) for c in self.children) + ")"


_TOKEN = re.compile(r"\s*(?:(?P<num>\d+\.\d*|\.\d+|\d+)|(?P<inp>[iI]\[?\s*(?P<idx>\d+)\s*\]?)|(?P<op>\*\*|<<x|x>>|«x|x»|[-+*/%x()@])|(?P<name>[A-Za-z_][A-Za-z_0-9]*))")


def _tokenize(expr: str):
    pos, out = 0, []
    expr = expr.strip()
    while pos < len(expr):
        m = _TOKEN.match(expr, pos)
        if not m or m.end() == pos:
            raise ValueError(f"cannot parse '{expr}' at position {pos}")
        pos = m.end()
        if m.group("num") is not None:
            out.append(("num", float(m.group("num"))))
        elif m.group("inp") is not None:
            out.append(("inp", int(m.group("idx"))))
        elif m.group("op") is not None:
            op = {"<<x": "«x", "x>>": "x»"}.get(m.group("op"), m.group("op"))
            out.append(("op", op))
        else:
            out.append(("name", m.group("name")))
    return out


class _Parser:
    def __init__(self, tokens):
        self.t = tokens
        self.i = 0

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else (None, None)

    def take(self):
        tok = self.peek()
        self.i += 1
        return tok

    def parse(self, level: int = len(_PRECEDENCE) - 1) -> Node:
        if level < 0:
            return self.atom()
        sym = _PRECEDENCE[level]
        parts = [self.parse(level - 1)]
        while self.peek() == ("op", sym):
            self.take()
            parts.append(self.parse(level - 1))
        if len(parts) == 1:
            return parts[0]
        return Node("op", sym, parts)

    def atom(self) -> Node:
        kind, val = self.take()
        if kind == "num":
            return Node("const", val)
        if kind == "inp":
            return Node("input", val)
        if kind == "op" and val == "(":
            n = self.parse()
            if self.take() != ("op", ")"):
                raise ValueError("missing ')'")
            return n
        if kind == "op" and val == "-":
            return Node("op", "*", [Node("const", -1.0), self.atom()])
        if kind == "name":
            if val not in _FUN_ALIASES:
                raise ValueError(f"unknown function '{val}'")
            if self.take() != ("op", "("):
                raise ValueError(f"'(' expected after {val}")
            arg = self.parse()
            if self.take() != ("op", ")"):
                raise ValueError("missing ')'")
            return Node("fun", _FUN_ALIASES[val], [arg])
        raise ValueError(f"unexpected token {val!r}")


# ---------------------------------------------------------------------------------------------------
# helpers mirroring reference utilities
# ---------------------------------------------------------------------------------------------------
def as_tensor(x, like: Tensor) -> Tensor:
    if isinstance(x, Tensor):
        return x
    t = Tensor.of(like.dtype, (1,), [x])
    return t


def shape_of_con(s1: Sequence[int], s2: Sequence[int]) -> Tuple[int, ...]:
    """ConvUtil.shapeOfCon (operations/ConvUtil.java:61-66)."""
    return tuple(abs(a - b) + 1 for a, b in zip(s1, s2))


def _ends_from(shape: Sequence[int]) -> Tuple[int, int]:
    """DimTrim.endsFrom: number of leading / trailing 1-axes."""
    prefix = 0
    for s in shape:
        if s == 1: prefix += 1
        else: break
    postfix = 0
    for s in reversed(shape):
        if s == 1: postfix += 1
        else: break
    return prefix, postfix


def make_fit(tensors: List[Tensor]) -> List[Tensor]:
    """Permute.makeFit (operations/other/Permute.java:82-110): pad lower-rank tensors with 1-axes -- in front
    when the largest tensor has at least as many leading as trailing 1-axes, else at the back."""
    largest = max(t.rank for t in tensors)
    shape = next(t.shape for t in tensors if t.rank == largest)
    prefix, postfix = _ends_from(shape)
    out = []
    for t in tensors:
        if t.rank == largest:
            out.append(t)
            continue
        padding = largest - t.rank
        if postfix <= prefix:
            form = [-1] * padding + list(range(t.rank))
        else:
            form = list(range(t.rank)) + [-1] * padding
        out.append(t.permute(*form))
    return out


def _common_device(tensors: Sequence[Optional[Tensor]]) -> CudaDevice:
    for t in tensors:
        if t is not None and t.device is not None:
            return t.device
    raise L.NeurekaCudaError(L.NK_ERR_UNSUPPORTED,
                             "no operand lives on a CudaDevice: this package has no CPU execution path (use tensor.to(CudaDevice.get()))")


def _execute_on_common_device(call: ExecutionCall, impl) -> Tensor:
    """AbstractDeviceAlgorithm.executeOnCommonDevice (:427-449) + executeDeviceAlgorithm (:127-156)."""
    dev = call.device
    moved = []
    for t in call.inputs:   # AbstractDeviceAlgorithm.java:119-124, :130-134
        if t is None:
            raise ValueError("Device arguments may not be null!\n"
                             "One or more tensor arguments within the given ExecutionCall instance is null.")
    for t in call.inputs:
        if t is not None and not dev.has(t):
            dev.store(t)
            moved.append(t)
    dev.approve(call)
    result = impl.run(call)
    for t in moved:
        if t is not result and t._root() is not result._root() and not t.is_intermediate:
            dev.restore(t)
    return result


def _new_output(dtype, shape, device: CudaDevice) -> Tensor:
    out = Tensor.of(dtype, shape, 0)
    out.set_is_virtual(False)
    out.is_intermediate = True
    device.store(out)
    return out


# ---------------------------------------------------------------------------------------------------
# flat operation execution (call preparation + algorithm choice + dispatch)
# ---------------------------------------------------------------------------------------------------
def run_conv(a: Tensor, b: Tensor) -> Tensor:
    """Operation "x" on NDConvolution: FunctionNode rank fitting (FunctionNode.java:92-93), output allocation of
    Convolution's call preparation (linear/Convolution.java:91-103), then the device implementation."""
    dev = _common_device([a, b])
    a, b = make_fit([a, b])
    out = _new_output(a.dtype, shape_of_con(a.shape, b.shape), dev)
    call = ExecutionCall([out, a, b], "x", dev, -1)
    return _execute_on_common_device(call, B.backend().implementation_for("x", B.ND_CONVOLUTION))


def run_xconv(op: str, i0: Tensor, i1: Tensor, i2: Tensor) -> Tensor:
    """Operations "«x" / "x»" (operations/ConvUtil.java:17-59, :68-88): rank fitting, DerivIdx 0,
    `x»` reverses its inputs before dispatch; input(0) of the dispatched call is the drain."""
    dev = _common_device([i0, i1, i2])
    tensors = make_fit([i0, i1, i2])
    for t in tensors:
        t.set_is_virtual(False)
    call = ExecutionCall(list(tensors), op, dev, 0)
    if op == "x»":
        call.rearrange_inputs(2, 1, 0)
    return _execute_on_common_device(call, B.backend().implementation_for(op, B.ND_CONVOLUTION))


def run_dot(a: Tensor, b: Tensor) -> Tensor:
    """Operation "dot" (linear/DotProduct.java; CPUDot.java:11-40): two vectors of the same length and type -> [1]."""
    if a.rank != 1 or b.rank != 1:
        raise ValueError("Dot product only works on vectors.")
    if a.shape[0] != b.shape[0]:
        raise ValueError("Dot product only works on vectors of the same length.")
    if a.dtype != b.dtype:
        raise ValueError("Type inconsistency between provided tensors encountered. All tensors must be of the same type.")
    dev = _common_device([a, b])
    out = _new_output(a.dtype, (1,), dev)
    call = ExecutionCall([out, a, b], "dot", dev, -1)
    return _execute_on_common_device(call, B.backend().implementation_for("dot", B.DOT_ALGORITHM))


def run_extreme(want_max: bool, x: Tensor):
    """Operations "min" / "max" (operations/other/Min.java:21-75, Max.java): the device implementation returns the index of
    the extreme element, the operation reads the item there into a [1] tensor. Returns (result, index)."""
    dev = _common_device([x])
    name, algo = ("max", B.MAX_ALGORITHM) if want_max else ("min", B.MIN_ALGORITHM)
    call = ExecutionCall([x], name, dev, -1)
    index = _execute_on_common_device(call, B.backend().implementation_for(name, algo))
    i = int(dev.access(index).read_at(0))
    dev.free(index)
    x.set_is_virtual(False)
    off = x.ndconf.index_of_index(i)                 # the element's place in the data array (one read, not the whole tensor)
    value = dev.access(x).read_array(off, 1)[0]
    out = Tensor.of(x.dtype, (1,), [value])
    out.set_is_virtual(False)
    out.is_intermediate = True
    dev.store(out)
    return out, i


def run_matmul(a: Tensor, b: Tensor) -> Tensor:
    """Operation "@" (linear/MatMul.java:15-40, algorithms/MatMulAlgorithm.java:62-84): [M,K] @ [K,N] -> [M,N], output
    allocated zero-filled in the operands' type. On this backend a matrix product is a convolution in which every
    dim is summed away or spanned by one operand only -- a [M,K,1] x [1,K,N] -> [M,1,N] -- so the call is handed to the
    convolution implementation on views that pad the three matrices with a size-1 axis (no copy; transposed and
    sliced operands included), where large problems take the register-tiled contraction kernel."""
    dev = _common_device([a, b])
    if a.rank != 2 or b.rank != 2:
        raise ValueError("matrix multiplication needs two rank-2 tensors")
    if a.shape[1] != b.shape[0]:
        raise ValueError(f"shapes {a.shape} and {b.shape} cannot be matrix-multiplied")
    if a.dtype != b.dtype:
        raise ValueError("all tensors of a call must have the same item type")
    moved = []
    for t in (a, b):
        t.set_is_virtual(False)
        if not dev.has(t):
            dev.store(t)
            moved.append(t)
    out = _new_output(a.dtype, (a.shape[0], b.shape[1]), dev)
    call = ExecutionCall([out.permute(0, -1, 1), a.permute(0, 1, -1), b.permute(-1, 0, 1)], "x", dev, -1)
    dev.approve(call)
    B.backend().implementation_for("x", B.ND_CONVOLUTION).run(call)
    out.version += 1
    for t in moved:
        if not t.is_intermediate:
            dev.restore(t)
    return out


def choose_algorithm(a: Tensor, b: Tensor) -> str:
    if b.size == 1 or b.is_virtual:
        return B.BI_SCALAR_BROADCAST
    if a.shape == b.shape:
        return B.BI_ELEMENTWISE
    return B.BROADCAST


def run_operator(sym: str, a: Tensor, b: Tensor, d: int = -1) -> Tensor:
    dev = _common_device([a, b])
    algo = choose_algorithm(a, b)
    be = B.backend()
    if algo == B.BI_SCALAR_BROADCAST:
        out = _new_output(a.dtype, a.shape, dev)
        call = ExecutionCall([out, a, b], sym, dev, d)
    elif algo == B.BI_ELEMENTWISE:
        out = _new_output(a.dtype, a.shape, dev)
        call = ExecutionCall([out, a, b], sym, dev, d)
    else:
        if a.rank != b.rank:
            a, b = make_fit([a, b])
        for s1, s2 in zip(a.shape, b.shape):
            if not (s1 == 1 or s2 == 1 or s1 == s2):
                raise ValueError(f"shapes {a.shape} and {b.shape} cannot be broadcast")
        shape = tuple(s2 if s1 == 1 else s1 for s1, s2 in zip(a.shape, b.shape))
        out = _new_output(a.dtype, shape, dev)
        call = ExecutionCall([out, a, b], sym, dev, d)
    return _execute_on_common_device(call, be.implementation_for(sym, algo))


def run_function(fid: str, x: Tensor, d: int = -1) -> Tensor:
    """Activation operations (operations/functions/AbstractActivationOperation.java:23-96): ScalarBroadcast for a
    virtual input, ScalarAlgorithm for a single element, else ElementwiseAlgorithm."""
    dev = _common_device([x])
    be = B.backend()
    if fid == "sumItems":
        call = ExecutionCall([x], fid, dev, d)   # CLSum takes input(0), or input(1) when a null drain was put in front
        return _execute_on_common_device(call, be.implementation_for(fid, B.SUM_ALGORITHM))
    out = _new_output(x.dtype, x.shape, dev)
    if x.is_virtual:
        algo = B.SCALAR_BROADCAST
    elif x.size == 1:
        algo = B.SCALAR_ALGORITHM
    else:
        algo = B.ELEMENTWISE
    call = ExecutionCall([out, x], fid, dev, d)
    return _execute_on_common_device(call, be.implementation_for(fid, algo))


def assign(dst: Tensor, src: Tensor) -> Tensor:
    """AssignLeft "<-" (operations/other/AssignLeft.java:32-99): strided copy into dst, in place."""
    dev = _common_device([dst, src])
    be = B.backend()
    if src.size == 1 or src.is_virtual:
        call = ExecutionCall([dst, dst, src], B.ASSIGN_LEFT, dev, -1)
        return _execute_on_common_device(call, be.implementation_for(B.ASSIGN_LEFT, B.BI_SCALAR_BROADCAST))
    call = ExecutionCall([dst, src], B.ASSIGN_LEFT, dev, -1)
    return _execute_on_common_device(call, be.implementation_for(B.ASSIGN_LEFT, B.ELEMENTWISE))


# ---------------------------------------------------------------------------------------------------
# fused elementwise expressions (Device.optimizedOperationOf)
# ---------------------------------------------------------------------------------------------------
_FUSED_OPS = {"+": "op_add", "-": "op_sub", "*": "op_mul", "/": "op_div", "%": "op_mod", "**": "op_pow"}


def fused_expression_of(root: Node) -> Tuple[str, int]:
    """The expression string nk_fused_compile takes for an AST made of inputs, constants, the six elementwise
    operators and the scalar functions, and the number of inputs it reads. n-ary chains nest to the left like the
    reference's pairwise reduction (operator/Addition.java `reducePairwise`). Raises for nodes that are not
    elementwise (convolutions, sumItems)."""
    highest = [-1]

    def walk(n: Node) -> str:
        if n.kind == "input":
            highest[0] = max(highest[0], int(n.value))
            return f"x{int(n.value)}"
        if n.kind == "const":
            return f"T({float(n.value)!r})"
        if n.kind == "fun":
            if n.value not in L.FUN_IDS:
                raise ValueError(f"'{n.value}' is not an elementwise function and cannot be fused")
            return f"f_{n.value}({walk(n.children[0])})"
        if n.kind == "op":
            if n.value not in _FUSED_OPS:
                raise ValueError(f"operator '{n.value}' is not elementwise and cannot be fused")
            acc = walk(n.children[0])
            for c in n.children[1:]:
                acc = f"{_FUSED_OPS[n.value]}({acc}, {walk(c)})"
            return acc
        raise ValueError(f"cannot fuse node kind {n.kind}")

    expr = walk(root)
    if highest[0] < 0:
        raise ValueError("a fused operation needs at least one input")
    return expr, highest[0] + 1


def fused_gradient_terms_of(root: Node, target: int) -> Tuple[str, int]:
    """The statement list nk_fused_compile_grad takes for the gradient of an elementwise expression w.r.t. input
    `target`: reverse mode over the tree, one `term[l]` per occurrence of the input. Every step rounds to the tensor's
    type exactly like the kernel the op-by-op backward pass would run at that node:
      function f(c):          error_c = error * f'(c)            (FallbackAlgorithm.java:118-129: error times the eager derivative)
      a + b, a - b:           error, error / error, 0 - error    (Addition.java:90-110: the error itself, reduced)
      a * b:                  b * error, a * error                (Multiplication.java:51-71, handle times drain)
      a / b, a % b, a ** b:   error * d(op)/d(operand)
    Returns (statements, number of occurrences)."""
    lines: List[str] = []
    counter = [0]
    leaves = [0]

    def tmp(expr: str) -> str:
        name = f"t{counter[0]}"
        counter[0] += 1
        lines.append(f"const T {name} = {expr};")
        return name

    def value(n: Node) -> str:
        """forward value of a subtree as a named temporary (recomputed, rounded per operator)"""
        if n.kind == "input":
            return f"x{int(n.value)}"
        if n.kind == "const":
            return f"T({float(n.value)!r})"
        if n.kind == "fun":
            if n.value not in L.FUN_IDS:
                raise ValueError(f"'{n.value}' is not an elementwise function and cannot be fused")
            return tmp(f"f_{n.value}({value(n.children[0])})")
        if n.kind == "op":
            if n.value not in _FUSED_OPS:
                raise ValueError(f"operator '{n.value}' is not elementwise and cannot be fused")
            acc = value(n.children[0])
            for c in n.children[1:]:
                acc = tmp(f"{_FUSED_OPS[n.value]}({acc}, {value(c)})")
            return acc
        raise ValueError(f"cannot fuse node kind {n.kind}")

    def back(n: Node, err: str) -> None:
        if not n.depends_on(target):
            return
        if n.kind == "input":
            lines.append(f"term[{leaves[0]}] = {err};")
            leaves[0] += 1
            return
        if n.kind == "fun":
            child = n.children[0]
            back(child, tmp(f"op_mul({err}, df_{n.value}({value(child)}))"))
            return
        # n-ary chains nest to the left: ((c0 o c1) o c2) ...; walk from the outermost pair inwards
        sym = n.value
        kids = n.children
        prefix = [value(kids[0])]
        for c in kids[1:-1]:
            prefix.append(tmp(f"{_FUSED_OPS[sym]}({prefix[-1]}, {value(c)})"))
        e = err
        for i in range(len(kids) - 1, 0, -1):
            a, b_node = prefix[i - 1], kids[i]
            if b_node.depends_on(target) or any(k.depends_on(target) for k in kids[:i]):
                b = value(b_node)
            if sym == "+":
                eb, ea = e, e
            elif sym == "-":
                eb, ea = (tmp(f"op_sub(T(0), {e})") if b_node.depends_on(target) else None), e
            elif sym == "*":
                eb = tmp(f"op_mul({a}, {e})") if b_node.depends_on(target) else None
                ea = tmp(f"op_mul({b}, {e})") if any(k.depends_on(target) for k in kids[:i]) else None
            else:
                d = {"/": "dop_div", "%": "dop_mod", "**": "dop_pow"}[sym]
                eb = tmp(f"op_mul({e}, {d}(1, {a}, {b}))") if b_node.depends_on(target) else None
                ea = tmp(f"op_mul({e}, {d}(0, {a}, {b}))") if any(k.depends_on(target) for k in kids[:i]) else None
            if b_node.depends_on(target):
                back(b_node, eb)
            e = ea
            if e is None:
                break
        if e is not None:
            back(kids[0], e)

    back(root, "e")
    if leaves[0] == 0:
        raise ValueError(f"the expression does not depend on input {target}")
    return " ".join(lines), leaves[0]


class FusedOperation:
    """What CudaDevice.optimized_operation_of returns: one kernel for a whole elementwise Function, compiled per
    item type on first use. Calling it allocates the (broadcast-shaped) output on the device and launches once."""

    def __init__(self, device: CudaDevice, function: "Function", name: str):
        self.device, self.function, self.name = device, function, name
        self.expr, self.n_inputs = fused_expression_of(function.root)
        self._handles = {}

    def _handle(self, dt: int):
        h = self._handles.get(dt)
        if h is None:
            h = C.c_void_p()
            L.check(L.lib.nk_fused_compile(self.device.ctx, dt, self.n_inputs, self.expr.encode(), C.byref(h)), self.device.ctx)
            self._handles[dt] = h
        return h

    def _grad_handle(self, dt: int, target: int):
        key = (dt, target)
        h = self._handles.get(key)
        if h is None:
            terms, leaves = fused_gradient_terms_of(self.function.root, target)
            h = C.c_void_p()
            L.check(L.lib.nk_fused_compile_grad(self.device.ctx, dt, self.n_inputs, target, leaves, terms.encode(), C.byref(h)), self.device.ctx)
            self._handles[key] = h
        return h

    def _fit(self, inputs):
        if len(inputs) != self.n_inputs:
            raise ValueError(f"{self.name} takes {self.n_inputs} inputs, got {len(inputs)}")
        tensors = make_fit(list(inputs)) if len({t.rank for t in inputs}) > 1 else list(inputs)
        rank = tensors[0].rank
        shape = []
        for k in range(rank):
            ext = {t.shape[k] for t in tensors} - {1}
            if len(ext) > 1:
                raise ValueError(f"shapes {[t.shape for t in tensors]} cannot be broadcast")
            shape.append(ext.pop() if ext else 1)
        for t in tensors:
            if t.dtype != tensors[0].dtype:
                raise ValueError("all tensors of a call must have the same item type")
            t.set_is_virtual(False)
            if not self.device.has(t):
                raise ValueError("every input of a fused operation must be stored on its device")
        return tensors, tuple(shape)

    @staticmethod
    def _operands(tensors):
        cfgs = [t.ndconf.as_inline_array() for t in tensors]
        cfg_ptrs = (C.POINTER(C.c_int32) * len(tensors))(*[c.ctypes.data_as(C.POINTER(C.c_int32)) for c in cfgs])
        bufs = (C.c_void_p * len(tensors))(*[t._data.buf for t in tensors])
        return cfgs, cfg_ptrs, bufs

    def __call__(self, *inputs: Tensor) -> Tensor:
        dev = self.device
        tensors, shape = self._fit(inputs)
        rank = tensors[0].rank
        dt = B.nk_dtype(tensors[0].dtype)
        out = _new_output(tensors[0].dtype, shape, dev)
        cfgs, cfg_ptrs, bufs = self._operands(tensors)
        c0 = out.ndconf.as_inline_array()
        L.check(L.lib.nk_fused_run(dev.ctx, self._handle(dt), rank, out._data.buf, c0.ctypes.data_as(C.POINTER(C.c_int32)), bufs, cfg_ptrs), dev.ctx)
        out.version += 1
        if self.function.do_ad:
            # one ADAction per differentiable input: the whole backward of the expression for that input, reduction over
            # its broadcast dims included, is one kernel (gradient)
            from . import autograd
            parents = []
            for j, (orig, fitted) in enumerate(zip(inputs, tensors)):
                if autograd._tracks(orig) and self.function.root.depends_on(j):
                    parents.append((orig, lambda err, j=j, tensors=tensors: self.gradient(j, err, *tensors)))
            if parents:
                out.graph_node = autograd.GraphNode(out, parents)
        return out

    def gradient(self, target: int, error: Tensor, *inputs: Tensor) -> Tensor:
        """d(sum(error * f(inputs))) / d(inputs[target]), shaped like that input: the error (result-shaped, or one virtual
        value as the backward pass of a sum hands it over) is multiplied through the expression and summed over the dims
        the input is broadcast along, in one kernel."""
        dev = self.device
        tensors, shape = self._fit(inputs)
        rank = tensors[0].rank
        dt = B.nk_dtype(tensors[0].dtype)
        if not dev.has(error):
            dev.store(error)
        err = error
        if err.rank != rank:
            err = make_fit([err, tensors[0]])[0] if err.size > 1 else Tensor.of(err.dtype, shape, float(dev.access(err).read_at(0)))
            if not dev.has(err):
                dev.store(err)
        grad = _new_output(tensors[target].dtype, tensors[target].shape, dev)
        cfgs, cfg_ptrs, bufs = self._operands(tensors)
        # a virtual error (one value standing for all, as the backward pass of a sum hands it over) stays one element:
        # its configuration maps every index to element 0
        ce_conf = NDConfiguration.virtual_of(err.shape) if err.is_virtual else err.ndconf
        cg, ce = grad.ndconf.as_inline_array(), ce_conf.as_inline_array()
        L.check(L.lib.nk_fused_run_grad(dev.ctx, self._grad_handle(dt, target), rank, grad._data.buf, cg.ctypes.data_as(C.POINTER(C.c_int32)),
                                        err._data.buf, ce.ctypes.data_as(C.POINTER(C.c_int32)), bufs, cfg_ptrs), dev.ctx)
        grad.version += 1
        return grad

    def close(self) -> None:
        for h in self._handles.values():
            L.lib.nk_fused_free(h)
        self._handles.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown: the library may already be gone
            pass


# ---------------------------------------------------------------------------------------------------
# Function
# ---------------------------------------------------------------------------------------------------
class Function:
    """Function.of(expression[, doAD]) (src/main/java/neureka/math/Function.java)."""

    _cache = {}

    def __init__(self, root: Node, do_ad: bool):
        self.root = root
        self.do_ad = do_ad

    @staticmethod
    def of(expression: str, do_ad: bool = True) -> "Function":
        key = (expression, do_ad)
        f = Function._cache.get(key)
        if f is None:
            p = _Parser(_tokenize(expression))
            root = p.parse()
            if p.i != len(p.t):
                raise ValueError(f"trailing input in expression '{expression}'")
            f = Function(root, do_ad)
            Function._cache[key] = f
        return f

    def __str__(self) -> str:
        return str(self.root)

    def call(self, *inputs: Tensor) -> Tensor:
        from . import autograd
        return autograd.evaluate(self.root, list(inputs), self.do_ad)

    __call__ = call
    execute = call
