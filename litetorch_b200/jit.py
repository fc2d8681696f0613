"""`lt.jit`: expression trees, symbolic derivatives and fused element-wise kernels
(src/bindings/python_bindings.cpp:793-884, include/litetorch/jit.h, src/ops/jit.cpp).

`JITVar` trees are built with operators and the unary helpers; `Tracer.derivative` differentiates
symbolically; `JITFunction(name, expr, inputs)` evaluates the tree - on CUDA by generating ONE fused kernel
for the whole tree (native code generator + NVRTC, cached per tree), on CPU through the native interpreter -
and is differentiable: its autograd node evaluates the derivative trees, which are fused kernels too.
`save/load` use the reference's text format.
"""
from __future__ import annotations

import ctypes
import enum
from ctypes import POINTER, c_char_p, c_float, c_int, c_uint64, c_void_p
from typing import Callable, List, Optional, Sequence

import torch

from ._native import host_lib
from .core import Tensor, _unwrap


class OpType(enum.IntEnum):
    INPUT = 0
    CONST = 1
    ADD = 2
    SUB = 3
    MUL = 4
    DIV = 5
    RELU = 6
    GELU = 7
    SIGMOID = 8
    TANH = 9
    SQRT = 10
    EXP = 11
    LOG = 12
    ABS = 13
    NEG = 14
    RELU_GRAD = 15
    GELU_GRAD = 16
    ABS_GRAD = 17


def _lib():
    lib = host_lib()
    if not getattr(lib, "_lt_jit_bound", False):
        lib.lt_jit_input.argtypes = [c_char_p]
        lib.lt_jit_const.argtypes = [c_float]
        lib.lt_jit_binary.argtypes = [c_int, c_int, c_int]
        lib.lt_jit_unary.argtypes = [c_int, c_int]
        lib.lt_jit_derivative.argtypes = [c_int, c_char_p]
        lib.lt_jit_node_val.restype = c_float
        lib.lt_jit_serialize.argtypes = [c_int, c_char_p, c_int]
        lib.lt_jit_deserialize.argtypes = [c_char_p]
        lib.lt_jit_node_name.argtypes = [c_int, c_char_p, c_int]
        lib.lt_jit_eval_cpu.argtypes = [c_int, POINTER(c_char_p), POINTER(c_void_p), c_int, c_uint64, c_void_p]
        lib.lt_jit_cuda_source.argtypes = [c_int, POINTER(c_char_p), c_int, c_char_p, c_int, c_char_p, c_int]
        lib._lt_jit_bound = True
    return lib


# the reference exports the operator codes into the module too (py::enum_::export_values on OpType)
globals().update({_m.name: _m for _m in OpType})


class JITVar:
    """Node handle in the native expression arena."""

    def __init__(self, op_or_val=None, name: str = "", _node: Optional[int] = None, op=None, val=None):
        """`JITVar(OpType.INPUT, "x")` / `JITVar(2.0)`; the reference's keywords `op=` and `val=` are accepted
        (src/bindings/python_bindings.cpp:814-815)."""
        lib = _lib()
        if op_or_val is None:
            op_or_val = op if op is not None else val
        if _node is not None:
            self.node = _node
        elif isinstance(op_or_val, (int, float)) and not isinstance(op_or_val, OpType):
            self.node = lib.lt_jit_const(float(op_or_val))
        elif op_or_val == OpType.INPUT:
            self.node = lib.lt_jit_input(name.encode())
        elif op_or_val == OpType.CONST:
            self.node = lib.lt_jit_const(0.0)
        else:
            raise ValueError("build operator nodes with +,-,*,/ and the lt.jit helpers")

    @staticmethod
    def input(name: str) -> "JITVar":
        return JITVar(OpType.INPUT, name)

    @property
    def op(self) -> OpType:
        return OpType(_lib().lt_jit_node_op(self.node))

    @property
    def name(self) -> str:
        buf = ctypes.create_string_buffer(256)
        _lib().lt_jit_node_name(self.node, buf, 256)
        return buf.value.decode()

    @property
    def val(self) -> float:
        return float(_lib().lt_jit_node_val(self.node))

    @property
    def left(self):
        n = _lib().lt_jit_node_left(self.node)
        return JITVar(_node=n) if n >= 0 else None

    @property
    def right(self):
        n = _lib().lt_jit_node_right(self.node)
        return JITVar(_node=n) if n >= 0 else None

    @staticmethod
    def _coerce(x) -> "JITVar":
        return x if isinstance(x, JITVar) else JITVar(float(x))

    def _bin(self, op, o, swap=False):
        a, b = (JITVar._coerce(o), self) if swap else (self, JITVar._coerce(o))
        return JITVar(_node=_lib().lt_jit_binary(int(op), a.node, b.node))

    def __add__(self, o): return self._bin(OpType.ADD, o)
    def __radd__(self, o): return self._bin(OpType.ADD, o, True)
    def __sub__(self, o): return self._bin(OpType.SUB, o)
    def __rsub__(self, o): return self._bin(OpType.SUB, o, True)
    def __mul__(self, o): return self._bin(OpType.MUL, o)
    def __rmul__(self, o): return self._bin(OpType.MUL, o, True)
    def __truediv__(self, o): return self._bin(OpType.DIV, o)
    def __rtruediv__(self, o): return self._bin(OpType.DIV, o, True)
    def __neg__(self): return _unary(OpType.NEG, self)


def _unary(op, a: JITVar) -> JITVar:
    return JITVar(_node=_lib().lt_jit_unary(int(op), a.node))


def relu(a): return _unary(OpType.RELU, a)
def gelu(a): return _unary(OpType.GELU, a)
def sigmoid(a): return _unary(OpType.SIGMOID, a)
def tanh(a): return _unary(OpType.TANH, a)
def sqrt(a): return _unary(OpType.SQRT, a)
def exp(a): return _unary(OpType.EXP, a)
def log(a): return _unary(OpType.LOG, a)
def abs(a): return _unary(OpType.ABS, a)  # noqa: A001
def neg(a): return _unary(OpType.NEG, a)


class Tracer:
    @staticmethod
    def trace(inputs: Sequence, func: Callable, name: str = "traced_fn") -> "JITFunction":
        """Two forms.  `trace(["x", "w"], lambda x, w: relu(x * w))`: `func` is called on symbolic inputs of those names.
        `trace([t1, t2], fn, name)`, the reference's form (src/ops/jit.cpp:496-525): `fn` takes the LIST of example
        tensors, is run once with autograd recording, and the recorded graph of `lt.Ops` element-wise calls (add, sub, mul,
        div, neg, relu, gelu, sigmoid, tanh, sqrt, exp, log, abs) between those tensors becomes the expression tree."""
        if all(isinstance(i, str) for i in inputs):
            vars_ = [JITVar.input(n) for n in inputs]
            return JITFunction(name, func(*vars_), vars_)
        leaves = [_unwrap(t).detach().clone().float().requires_grad_(True) for t in inputs]
        with torch.enable_grad():
            out = _unwrap(func([Tensor(l) for l in leaves]))
        vars_ = [JITVar.input("x%d" % i) for i in range(len(leaves))]
        used, cache = set(), {}
        unary = {"relu": relu, "gelu": gelu, "sigmoid": sigmoid, "tanh": tanh, "sqrt": sqrt, "exp": exp, "log": log, "abs": abs}

        def const_of(fn, attr):
            v = getattr(fn, attr, None)
            if v is None:
                raise ValueError("the traced function combines an input with a tensor that is not in the input list")
            v = v if not torch.is_tensor(v) else (v.item() if v.numel() == 1 else None)
            if v is None:
                raise ValueError("the traced function combines an input with a tensor that is not in the input list")
            return JITVar(float(v))

        def walk(fn):
            if fn is None:
                raise ValueError("the traced function's result does not depend on its inputs through element-wise lt.Ops calls")
            if fn in cache:
                return cache[fn]
            kind = fn.name().lower().split("::")[-1]
            if kind.startswith("accumulategrad"):
                for i, l in enumerate(leaves):
                    if fn.variable is l:
                        used.add(i)
                        return vars_[i]
                raise ValueError("the traced graph reaches a tensor that is not in the input list")
            nxt = [f for f, _ in fn.next_functions]
            if kind.startswith(("addbackward", "subbackward")):
                alpha = float(getattr(fn, "_saved_alpha", 1) or 1)
                if len(nxt) < 2 or nxt[1] is None or nxt[0] is None:
                    raise ValueError("adding a constant cannot be traced: pass it as an input tensor")
                rhs = walk(nxt[1]) if alpha == 1.0 else walk(nxt[1]) * alpha
                res = walk(nxt[0]) + rhs if kind.startswith("add") else walk(nxt[0]) - rhs
            elif kind.startswith("mulbackward"):
                a = walk(nxt[0]) if nxt[0] is not None else const_of(fn, "_saved_self")
                b = walk(nxt[1]) if len(nxt) > 1 and nxt[1] is not None else const_of(fn, "_saved_other")
                res = a * b
            elif kind.startswith("divbackward"):
                a = walk(nxt[0]) if nxt[0] is not None else const_of(fn, "_saved_self")
                b = walk(nxt[1]) if len(nxt) > 1 and nxt[1] is not None else const_of(fn, "_saved_other")
                res = a / b
            elif kind.startswith("negbackward"):
                res = -walk(nxt[0])
            else:
                for key, mk in unary.items():
                    if kind.startswith(key) or kind.startswith("_" + key):
                        res = mk(walk(nxt[0]))
                        break
                else:
                    raise ValueError("unsupported operation in the traced function: %s" % fn.name())
            cache[fn] = res
            return res

        expr = walk(out.grad_fn)
        return JITFunction(name, expr, [v for i, v in enumerate(vars_) if i in used])

    @staticmethod
    def derivative(var: JITVar, wrt) -> JITVar:
        wrt_name = wrt.name if isinstance(wrt, JITVar) else str(wrt)
        return JITVar(_node=_lib().lt_jit_derivative(var.node, wrt_name.encode()))

    @staticmethod
    def serialize_var(var: JITVar) -> str:
        lib = _lib()
        cap = 1 << 16
        while True:
            buf = ctypes.create_string_buffer(cap)
            n = lib.lt_jit_serialize(var.node, buf, cap)
            if n >= 0:
                return buf.value.decode()
            cap = -n + 16

    @staticmethod
    def deserialize_var(str: str = None, text: str = None) -> JITVar:
        text = str if text is None else text
        n = _lib().lt_jit_deserialize(text.encode())
        if n < 0:
            raise ValueError("cannot parse expression %r" % text[:80])
        return JITVar(_node=n)


_kernel_cache = {}


def _eval_tree(node: int, names: List[str], tensors: List[torch.Tensor]) -> torch.Tensor:
    lib = _lib()
    ref = tensors[0]
    n = ref.numel()
    if ref.is_cuda and all(t.is_cuda and t.is_contiguous() and t.dtype == ref.dtype and t.numel() == n for t in tensors) \
            and ref.dtype in (torch.float32, torch.bfloat16):
        from ._native import cuda_lib
        cl = cuda_lib()
        dtype_code = 1 if ref.dtype == torch.bfloat16 else 0
        key = (node, tuple(names), dtype_code)
        handle = _kernel_cache.get(key)
        if handle is None:
            arr = (c_char_p * len(names))(*[s.encode() for s in names])
            kname = ("lt_jit_k%d_%d" % (node, dtype_code)).encode()
            cap = 1 << 16
            while True:
                buf = ctypes.create_string_buffer(cap)
                ln = lib.lt_jit_cuda_source(node, arr, len(names), kname, dtype_code, buf, cap)
                if ln >= 0:
                    break
                cap = -ln + 16
            handle = cl.lt_jit_compile(buf.value, kname, len(names))
            if handle < 0:
                log = ctypes.create_string_buffer(8192)
                cl.lt_jit_last_log(log, 8192)
                raise RuntimeError("JIT compilation failed (%d): %s" % (handle, log.value.decode(errors="replace")))
            _kernel_cache[key] = handle
        out = torch.empty_like(ref)
        ptrs = (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        rc = cl.lt_jit_launch(handle, ptrs, len(tensors), c_void_p(out.data_ptr()), ctypes.c_longlong(n),
                              c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError("JIT kernel launch failed: %d" % rc)
        return out
    cpu = [t.detach().to("cpu", torch.float32).contiguous().expand_as(ref).contiguous() if t.numel() != n
           else t.detach().to("cpu", torch.float32).contiguous() for t in tensors]
    out = torch.empty(ref.shape, dtype=torch.float32)
    arr = (c_char_p * len(names))(*[s.encode() for s in names])
    ptrs = (c_void_p * len(cpu))(*[t.data_ptr() for t in cpu])
    lib.lt_jit_eval_cpu(node, arr, ptrs, len(cpu), n, c_void_p(out.data_ptr()))
    return out.to(ref.device, ref.dtype)


class _JITApply(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, *xs):
        ctx.fn = fn
        ctx.save_for_backward(*xs)
        return _eval_tree(fn.expr.node, fn.input_names, [x.contiguous() for x in xs])

    @staticmethod
    def backward(ctx, g):
        fn = ctx.fn
        xs = [x.contiguous() for x in ctx.saved_tensors]
        grads = [None]
        for i, name in enumerate(fn.input_names):
            if not ctx.needs_input_grad[i + 1]:
                grads.append(None)
                continue
            d = fn.derivative_node(name)
            grads.append(_eval_tree(d, fn.input_names, xs) * g)
        return tuple(grads)


class JITFunction:
    def __init__(self, name: str, expr: JITVar, inputs: Sequence[JITVar]):
        self.name, self.expr, self.inputs = name, expr, list(inputs)
        self.input_names = [v.name for v in self.inputs]
        self._derivs = {}

    def derivative_node(self, wrt: str) -> int:
        if wrt not in self._derivs:
            self._derivs[wrt] = _lib().lt_jit_derivative(self.expr.node, wrt.encode())
        return self._derivs[wrt]

    def forward(self, *args: Tensor) -> Tensor:
        if len(args) == 1 and isinstance(args[0], (list, tuple)):
            args = tuple(args[0])
        ts = [_unwrap(a) for a in args]
        return Tensor(_JITApply.apply(self, *ts))

    __call__ = forward

    def save(self, filepath: str) -> None:
        with open(filepath, "w") as f:
            f.write(self.name + "\n%d\n" % len(self.inputs))
            for n in self.input_names:
                f.write(n + "\n")
            f.write(Tracer.serialize_var(self.expr) + "\n")

    @staticmethod
    def load(filepath: str) -> "JITFunction":
        with open(filepath) as f:
            lines = f.read().split("\n")
        name, k = lines[0], int(lines[1])
        names = lines[2:2 + k]
        expr = Tracer.deserialize_var(lines[2 + k])
        return JITFunction(name, expr, [JITVar.input(n) for n in names])


def _prebuilt(name, build, n):
    names = ["a", "b", "c"][:n]
    cache = {}

    def call(*tensors: Tensor) -> Tensor:
        if "fn" not in cache:
            cache["fn"] = Tracer.trace(names, build, name)
        ts = [_unwrap(t) for t in tensors]
        shape = ts[0].shape
        ts = [t if t.shape == shape else t.expand(shape).contiguous() for t in ts]
        return cache["fn"](*[Tensor(t) for t in ts])
    call.__name__ = name
    return call


# the four pre-built fused ops of the reference binding (src/bindings/python_bindings.cpp:840-867)
fused_bias_relu = _prebuilt("fused_bias_relu", lambda x, b: relu(x + b), 2)
fused_bias_gelu = _prebuilt("fused_bias_gelu", lambda x, b: gelu(x + b), 2)
fused_residual_add = _prebuilt("fused_residual_add", lambda x, r: x + r, 2)
fused_residual_gelu = _prebuilt("fused_residual_gelu", lambda x, r: gelu(x) + r, 2)
