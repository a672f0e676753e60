"""``fuse``: run a chain of elementwise operations as one kernel launch.

The reference evaluates a chain such as ``examples/example_bs.py:50-78`` one ufunc at a
time: ``DPNPUnaryFunc.__call__`` / ``DPNPBinaryFunc.__call__``
(dpnp/dpnp_algo/dpnp_elementwise_common.py:81-235,537-739) allocate a result and launch a
kernel per call, and a Python scalar operand becomes a stride-0 array
(dpnp/tensor/_elementwise_common.py:655-659).  A function wrapped in :func:`fuse` is
instead *traced*: its array arguments are replaced by :class:`FusedValue` stand-ins, every
operator and ufunc applied to them records a node of an expression graph, and the graph is
compiled once into a register-machine program -- the chain's inputs are read once and its
results written once.  The program has two executors behind the C ABI:

* ``dpb_fused_elementwise_specialized`` writes it out as straight-line CUDA C++ over the operator
  classes of the per-op kernels, compiles that with NVRTC at the first call and keeps the kernel:
  the chain then runs like a kernel written by hand for it (mode ``"compile"``);
* ``dpb_fused_elementwise`` interprets it on the device, with no compiler involved (mode
  ``"interpret"``; about twice the time on an arithmetic-heavy chain).

``"auto"`` (the default; ``DPNP_B200_FUSE`` overrides it) compiles when NVRTC, the driver library
and the headers are found and interprets otherwise.  Both executors apply the same device
operators as the per-op kernels, in the same order, with scalars converted to the array type
exactly as the per-op path converts them, so the result has the bits of the unfused chain.
Common subexpressions are evaluated once, which does not change any value.

What is fused: float32 / float64 C-contiguous arrays of one common shape (size-1 arrays are
broadcast), Python ``int`` / ``float`` scalars, arithmetic, comparisons feeding ``where`` or
the logical operators, the unary math functions, ``out=`` and ``x[:] = value`` /
``x[...] = value`` stores into array arguments.  Anything else (other dtypes, views, a
reduction inside the function, data-dependent control flow, ...) makes the call run the
function unchanged, op by op, on the device: ``fuse`` never changes results and never
computes on the host.
"""

from __future__ import annotations

import ctypes as C
import functools
import os
import struct

import numpy as np

from . import _lib
from .dpnp_array import dpnp_array
from .tensor._usmarray import usm_ndarray

__all__ = ["fuse", "ArraySpec", "FusedValue", "FusionUnsupported"]

_OPS = {name: i for i, name in enumerate([
    "load", "store", "select", "move", "positive", "negative", "abs", "exp", "log", "sqrt", "erf",
    "square", "reciprocal", "sin", "cos", "tanh", "expm1", "log1p", "floor", "ceil", "sign",
    "add", "subtract", "multiply", "divide", "maximum", "minimum", "pow", "less", "less_equal",
    "greater", "greater_equal", "equal", "not_equal", "logical_and", "logical_or"])}
_FIRST_BINARY = _OPS["add"]
_UNARY = {n for n, i in _OPS.items() if _OPS["move"] <= i < _FIRST_BINARY}
_BINARY = {n for n, i in _OPS.items() if i >= _FIRST_BINARY}
_COMPARISONS = {"less", "less_equal", "greater", "greater_equal", "equal", "not_equal"}
_LOGICAL = {"logical_and", "logical_or"}
_ALIASES = {"true_divide": "divide", "absolute": "abs", "power": "pow", "fabs": "abs"}

_OPND_IMM, _OPND_IN, _OPND_ACC, _NO_DST = 64, 128, 255, 255
_MAX_INSTR, _MAX_IMM, _MAX_IN, _MAX_OUT, _MAX_REG = 192, 48, 12, 8, 24
_MAX_CACHED = 256                  # compiled programs kept per fused function (oldest dropped first)


class FusionUnsupported(Exception):
    """Raised while tracing when the function leaves what the interpreter covers."""


class dpb_fused_program(C.Structure):
    _fields_ = [
        ("typenum", C.c_int32), ("n_instr", C.c_int32), ("n_reg", C.c_int32), ("n_imm", C.c_int32),
        ("n_in", C.c_int32), ("n_out", C.c_int32),
        ("code", C.POINTER(C.c_uint64)), ("imm", C.POINTER(C.c_double)),
        ("in_", C.POINTER(C.c_void_p)), ("in_is_scalar", C.POINTER(C.c_int32)),
        ("out", C.POINTER(C.c_void_p)),
    ]


_lib.lib.dpb_fused_elementwise.restype = C.c_int
_lib.lib.dpb_fused_elementwise.argtypes = [C.POINTER(dpb_fused_program), C.c_int64, C.c_void_p]
_lib.lib.dpb_fused_elementwise_specialized.restype = C.c_int
_lib.lib.dpb_fused_elementwise_specialized.argtypes = [C.POINTER(dpb_fused_program), C.c_int64, C.c_void_p]
_lib.lib.dpb_fused_specialized_source.argtypes = [C.POINTER(dpb_fused_program), C.c_char_p, C.c_int64,
                                                  C.POINTER(C.c_int64)]
_lib.lib.dpb_fused_specialize_compile.argtypes = [C.POINTER(dpb_fused_program), C.POINTER(C.c_int64)]

MODES = ("auto", "compile", "interpret")
_specialize_available = None


def specialize_available():
    """Whether chains can be compiled at run time here (NVRTC, the driver library, the headers)."""
    global _specialize_available
    if _specialize_available is None:
        _specialize_available = bool(_lib.lib.dpb_fused_specialize_available())
    return _specialize_available


def default_mode():
    mode = os.environ.get("DPNP_B200_FUSE", "auto").strip().lower() or "auto"
    if mode not in MODES:
        raise ValueError(f"DPNP_B200_FUSE={mode!r}: expected one of {MODES}")
    return mode


# --------------------------------------------------------------------------- tracing
class _Tracer:
    """Expression graph of one traced call.  Nodes are tuples, interned so that equal
    subexpressions share one node."""

    def __init__(self, dtype, shape):
        self.dtype = dtype
        self.shape = shape
        self.nodes = []            # node id -> tuple
        self.flags = []            # node id -> value is a comparison result (0/1)
        self.index = {}
        self.stores = {}           # input slot -> node id (last store wins)

    def node(self, key, flag=False):
        i = self.index.get(key)
        if i is None:
            i = len(self.nodes)
            self.nodes.append(key)
            self.flags.append(flag)
            self.index[key] = i
        return i

    def imm(self, v):
        if isinstance(v, (bool, np.bool_)):
            raise FusionUnsupported("bool scalar operand")
        if isinstance(v, int):
            if abs(v) > (1 << 53):
                raise FusionUnsupported("integer scalar beyond 2**53")
            v = float(v)
        elif isinstance(v, np.floating):
            if v.dtype != self.dtype:
                raise FusionUnsupported("NumPy scalar of another type")
            v = float(v)
        elif not isinstance(v, float):
            raise FusionUnsupported(f"operand of type {type(v).__name__}")
        # the bits identify the value: keeps -0.0 and 0.0, and NaN payloads, apart
        return self.node(("imm", struct.pack("<d", v)))

    def operand(self, x):
        if isinstance(x, FusedValue):
            if x._tr is not self:
                raise FusionUnsupported("value of another trace")
            return x._node
        return self.imm(x)

    def unary(self, op, x):
        op = _ALIASES.get(op, op)
        if op == "logical_not":
            a = self.operand(x)
            if not self.flags[a]:
                raise FusionUnsupported("logical_not of a non-boolean value")
            return FusedValue(self, self.node(("bin", "equal", a, self.imm(0.0)), True))
        if op not in _UNARY:
            raise FusionUnsupported(f"unary {op}")
        a = self.operand(x)
        if self.flags[a]:
            raise FusionUnsupported("arithmetic on a boolean value")
        if op == "positive":
            return FusedValue(self, a)
        return FusedValue(self, self.node(("un", op, a)))

    def binary(self, op, x, y):
        op = _ALIASES.get(op, op)
        if op not in _BINARY:
            raise FusionUnsupported(f"binary {op}")
        a, b = self.operand(x), self.operand(y)
        if self.nodes[a][0] == "imm" and self.nodes[b][0] == "imm":
            raise FusionUnsupported("two scalar operands")
        fa, fb = self.flags[a], self.flags[b]
        if op in _LOGICAL:
            if not (fa and fb):
                raise FusionUnsupported("logical operator on non-boolean values")
        elif fa or fb:
            raise FusionUnsupported("arithmetic on a boolean value")
        return FusedValue(self, self.node(("bin", op, a, b), op in _COMPARISONS or op in _LOGICAL))

    def select(self, cond, x, y):
        if not isinstance(cond, FusedValue) or not self.flags[cond._node]:
            raise FusionUnsupported("where() needs a traced boolean condition")
        if not isinstance(x, FusedValue) and not isinstance(y, FusedValue):
            raise FusionUnsupported("where() with two scalars")
        a, b = self.operand(x), self.operand(y)
        if self.flags[a] or self.flags[b]:
            raise FusionUnsupported("where() selecting boolean values")
        return FusedValue(self, self.node(("sel", cond._node, a, b)))

    def store(self, target, value):
        if target._slot is None:
            raise FusionUnsupported("store into a temporary")
        v = self.operand(value)
        if self.flags[v]:
            raise FusionUnsupported("store of a boolean value")
        self.stores[target._slot] = v
        target._node = v           # later reads of the array see the stored value


def _binop(name, reflected=False):
    def method(self, other):
        if isinstance(other, (dpnp_array, usm_ndarray)):
            raise FusionUnsupported("array that is not an argument of the fused function")
        return self._tr.binary(name, other, self) if reflected else self._tr.binary(name, self, other)
    return method


def _inplace(name):
    def method(self, other):
        res = self._tr.binary(name, self, other)
        if self._slot is not None:     # `x += y` on an argument writes the argument
            self._tr.store(self, res)
            return self
        return res
    return method


class FusedValue:
    """Stand-in for an array while a fused function is traced."""

    __array_ufunc__ = None             # NumPy scalars defer to the reflected operators
    __slots__ = ("_tr", "_node", "_slot")

    def __init__(self, tr, node, slot=None):
        self._tr, self._node, self._slot = tr, node, slot

    shape = property(lambda self: self._tr.shape)
    ndim = property(lambda self: len(self._tr.shape))
    size = property(lambda self: int(np.prod(self._tr.shape, dtype=np.int64)))
    dtype = property(lambda self: np.dtype(bool) if self._tr.flags[self._node] else self._tr.dtype)

    __add__, __radd__ = _binop("add"), _binop("add", True)
    __sub__, __rsub__ = _binop("subtract"), _binop("subtract", True)
    __mul__, __rmul__ = _binop("multiply"), _binop("multiply", True)
    __truediv__, __rtruediv__ = _binop("divide"), _binop("divide", True)
    __pow__, __rpow__ = _binop("pow"), _binop("pow", True)
    __lt__, __le__ = _binop("less"), _binop("less_equal")
    __gt__, __ge__ = _binop("greater"), _binop("greater_equal")
    __eq__, __ne__ = _binop("equal"), _binop("not_equal")
    __and__, __rand__ = _binop("logical_and"), _binop("logical_and", True)
    __or__, __ror__ = _binop("logical_or"), _binop("logical_or", True)
    __iadd__, __isub__ = _inplace("add"), _inplace("subtract")
    __imul__, __itruediv__ = _inplace("multiply"), _inplace("divide")
    __hash__ = None

    def __neg__(self):
        return self._tr.unary("negative", self)

    def __pos__(self):
        return self._tr.unary("positive", self)

    def __abs__(self):
        return self._tr.unary("abs", self)

    def __invert__(self):
        return self._tr.unary("logical_not", self)

    def __bool__(self):
        raise FusionUnsupported("truth value of an array (data-dependent control flow)")

    def __setitem__(self, key, value):
        whole = key is Ellipsis or key == slice(None) or key == (Ellipsis,) or (
            isinstance(key, tuple) and len(key) <= len(self._tr.shape) and
            all(k == slice(None) for k in key))
        if not whole:
            raise FusionUnsupported("store into part of an array")
        self._tr.store(self, value)

    def __getattr__(self, name):
        raise FusionUnsupported(f"attribute {name!r} of an array inside a fused function")


def trace_unary(name, x, out=None):
    """Entry point of the ufunc objects when their operand is a :class:`FusedValue`."""
    res = x._tr.unary(name, x)
    return _into(out, res)


def trace_binary(name, x1, x2, out=None):
    tr = (x1 if isinstance(x1, FusedValue) else x2)._tr
    for x in (x1, x2):
        if isinstance(x, (dpnp_array, usm_ndarray)):
            raise FusionUnsupported("array that is not an argument of the fused function")
    res = tr.binary(name, x1, x2)
    return _into(out, res)


def trace_where(cond, x, y, out=None):
    tr = next(v for v in (cond, x, y) if isinstance(v, FusedValue))._tr
    return _into(out, tr.select(cond, x, y))


def _into(out, res):
    if out is None:
        return res
    if isinstance(out, tuple) and len(out) == 1:
        out = out[0]
    if not isinstance(out, FusedValue):
        raise FusionUnsupported("out= that is not an argument of the fused function")
    out._tr.store(out, res)
    return out


def is_traced(*values):
    return any(type(v) is FusedValue for v in values)


# ------------------------------------------------------------------------ compilation
class _Program:
    """A compiled trace: instruction words plus the recipe for binding a call's arrays."""

    def __init__(self, tr, results_tree, result_nodes):
        self.dtype = tr.dtype
        self.results_tree = results_tree
        roots = list(dict.fromkeys(list(tr.stores.values()) + result_nodes))
        nodes = tr.nodes

        # nodes that need an instruction (immediates are operands, not instructions)
        def children(i):
            k = nodes[i]
            if k[0] == "un":
                return (k[2],)
            if k[0] == "bin":
                return (k[2], k[3])
            if k[0] == "sel":
                return (k[1], k[2], k[3])
            return ()

        # every store is emitted after the last computation, so an argument that is both
        # read and written is read first
        order, seen = [], set()

        def visit(i):
            # post-order; the operand visited last is the one most likely to still be in
            # the accumulator when its consumer runs, so the deepest subtree goes last
            stack = [(i, False)]
            while stack:
                j, done = stack.pop()
                if j in seen or nodes[j][0] in ("imm", "in"):
                    continue
                if done:
                    seen.add(j)
                    order.append(j)
                    continue
                stack.append((j, True))
                ch = [c for c in children(j) if c not in seen and nodes[c][0] not in ("imm", "in")]
                ch.sort(key=lambda c: depth[c])            # shallow first, deep last
                for c in reversed(ch):
                    stack.append((c, False))

        depth = [0] * len(nodes)
        for i, k in enumerate(nodes):
            ch = children(i)
            depth[i] = 1 + max((depth[c] for c in ch), default=0)
        for r in roots:
            visit(r)

        # uses of every node: positions of consumers in `order`, plus stores at the end
        pos = {j: p for p, j in enumerate(order)}
        last_use = {j: -1 for j in order}
        n_uses = {j: 0 for j in order}
        for p, j in enumerate(order):
            for c in children(j):
                if c in pos:
                    last_use[c] = max(last_use[c], p)
                    n_uses[c] += 1
        end = len(order)
        store_list = []                        # (node, output index)
        self.out_bind = []                     # per output: ("slot", s) or ("new",)
        for slot, v in tr.stores.items():
            store_list.append((v, len(self.out_bind)))
            self.out_bind.append(("slot", slot))
        self.result_out = {}
        for v in result_nodes:
            if v in self.result_out:
                continue
            self.result_out[v] = len(self.out_bind)
            store_list.append((v, len(self.out_bind)))
            self.out_bind.append(("new",))
        # A store is issued right after its value is computed (the value is still in the
        # accumulator) unless the destination is an argument that a later instruction still reads;
        # such stores wait until the end and keep their value in a register.
        last_read = {}                         # argument slot -> last instruction that reads it
        for p_, j in enumerate(order):
            for c in children(j):
                if nodes[c][0] == "in":
                    last_read[nodes[c][1]] = p_
        # A store or result whose value is an argument itself (`c[:] = a`, `return +a`) reads that
        # argument when the store runs, i.e. after every computation: it counts as a reader at `end`.
        written = {bind[1] for bind in self.out_bind if bind[0] == "slot"}
        for v, out_i in store_list:
            if nodes[v][0] == "in" and self.out_bind[out_i] != ("slot", nodes[v][1]):
                last_read[nodes[v][1]] = end
        eager, late = {}, []
        for v, out_i in store_list:
            bind = self.out_bind[out_i]
            safe = bind[0] == "new" or last_read.get(bind[1], -1) <= pos.get(v, end)
            if v in pos and safe:
                eager.setdefault(v, []).append(out_i)
            else:
                late.append((v, out_i))
                if v in pos:
                    last_use[v] = end
                    n_uses[v] += 1

        imms, imm_index = [], {}
        input_index = {}
        self.in_slots = []

        def opnd(i, p, regs):
            k = nodes[i]
            if k[0] == "in":                   # read straight from the argument, no register
                if k[1] not in input_index:
                    input_index[k[1]] = len(self.in_slots)
                    self.in_slots.append(k[1])
                return _OPND_IN + input_index[k[1]]
            if k[0] == "imm":
                if k[1] not in imm_index:
                    imm_index[k[1]] = len(imms)
                    imms.append(struct.unpack("<d", k[1])[0])
                return _OPND_IMM + imm_index[k[1]]
            if pos[i] == p - 1:
                return _OPND_ACC
            return regs[i]

        code, regs, free, n_reg = [], {}, [], 0
        for p, j in enumerate(order):
            k = nodes[j]
            # the result needs a register unless its single use is the very next instruction
            # (a value kept for a store at the end always gets one: last_use == end)
            only_next = (n_uses[j] == 1 and last_use[j] == p + 1 < end) or (n_uses[j] == 0 and j in eager)
            if k[0] == "un":
                word = (_OPS[k[1]], opnd(k[2], p, regs), 0, 0)
            elif k[0] == "bin":
                oa, ob = opnd(k[2], p, regs), opnd(k[3], p, regs)
                if ob == _OPND_ACC and oa != _OPND_ACC:
                    # the interpreter computes in place on the accumulator: hand it the
                    # accumulator first and flag that it is the operator's second operand
                    word = (_OPS[k[1]] | 1 << 40, ob, oa, 0)
                else:
                    word = (_OPS[k[1]], oa, ob, 0)
            else:
                word = (_OPS["select"], opnd(k[1], p, regs), opnd(k[2], p, regs), opnd(k[3], p, regs))
            # registers whose last reader is this instruction are free for its result
            for c in set(children(j)):
                if c in regs and last_use[c] == p:
                    free.append(regs.pop(c))
            if only_next:
                dst = _NO_DST
            else:
                if free:
                    free.sort()
                    dst = free.pop(0)
                else:
                    dst = n_reg
                    n_reg += 1
                regs[j] = dst
            op, a, b, c3 = word
            code.append(op | dst << 8 | a << 16 | b << 24 | c3 << 32)
            for out_i in eager.get(j, ()):             # stores do not disturb the accumulator
                code.append(_OPS["store"] | _NO_DST << 8 | _OPND_ACC << 16 | out_i << 24)
        # Late stores that copy an argument which another store overwrites (`a[:] = b; b[:] = t`,
        # a swap) first move the old values into registers, so that the order of the stores
        # does not matter.
        saved = {}
        for v, out_i in late:
            if (nodes[v][0] == "in" and nodes[v][1] in written and v not in saved
                    and self.out_bind[out_i] != ("slot", nodes[v][1])):
                if free:
                    free.sort()
                    dst = free.pop(0)
                else:
                    dst = n_reg
                    n_reg += 1
                saved[v] = dst
                code.append(_OPS["move"] | dst << 8 | opnd(v, -1, regs) << 16)
        for v, out_i in late:
            if v in saved and self.out_bind[out_i] != ("slot", nodes[v][1]):
                a = saved[v]
            else:
                a = opnd(v, -1, regs) if nodes[v][0] in ("imm", "in") else regs[v]
            code.append(_OPS["store"] | _NO_DST << 8 | a << 16 | out_i << 24)
        if (len(code) > _MAX_INSTR or len(imms) > _MAX_IMM or len(self.in_slots) > _MAX_IN or
                len(self.out_bind) > _MAX_OUT or n_reg > min(_MAX_REG, _OPND_IMM) or
                len(imms) > _OPND_IN - _OPND_IMM):
            raise FusionUnsupported("chain exceeds the limits of the interpreter")
        self.specialize_failed = None          # why run-time compilation of this program failed, if it did
        self.n_reg = n_reg
        self.n_instr = len(code)
        self.code = (C.c_uint64 * max(1, len(code)))(*code)
        self.imm = (C.c_double * max(1, len(imms)))(*imms)
        self.n_imm = len(imms)

    def _descriptor(self, ins=None, flags=None, outs=None):
        """The C descriptor; without arrays (source(), compile()) the pointers are placeholders."""
        n_in, n_out = len(self.in_slots), len(self.out_bind)
        if ins is None:
            ins = (C.c_void_p * max(1, n_in))(*[16] * n_in)
            outs = (C.c_void_p * max(1, n_out))(*[16] * n_out)
            scalar = getattr(self, "scalar_slots", None)
            flags = (C.c_int32 * max(1, n_in))(*[int(scalar[s]) if scalar else 0 for s in self.in_slots])
        desc = dpb_fused_program(_lib.typenum_of(self.dtype), self.n_instr, self.n_reg, self.n_imm, n_in, n_out,
                                 self.code, self.imm, ins, flags, outs)
        desc._keep = (ins, flags, outs)
        return desc

    def source(self):
        """The CUDA C++ that mode "compile" builds for this program (no device involved)."""
        desc, need = self._descriptor(), C.c_int64(0)
        _lib.check(_lib.lib.dpb_fused_specialized_source(C.byref(desc), None, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value)
        _lib.check(_lib.lib.dpb_fused_specialized_source(C.byref(desc), buf, need.value, None))
        return buf.value.decode()

    def compile(self):
        """Compile the program now (no device needed); returns the size of the device code."""
        desc, size = self._descriptor(), C.c_int64(0)
        _lib.check(_lib.lib.dpb_fused_specialize_compile(C.byref(desc), C.byref(size)))
        return size.value

    def listing(self):
        """Human-readable instruction list (for tests and debugging)."""
        names = {i: n for n, i in _OPS.items()}
        out = []
        for w in self.code[:self.n_instr]:
            op, dst, a, b, c3 = w & 255, (w >> 8) & 255, (w >> 16) & 255, (w >> 24) & 255, (w >> 32) & 255
            if (w >> 40) & 1:                          # accumulator-first encoding of op(b, a)
                a, b = b, a
            out.append((names[op], dst, a, b, c3))
        return out


# --------------------------------------------------------------------------- the decorator
class ArraySpec:
    """Type and shape of an array argument, for compiling a chain ahead of its first call
    (``fused.program(ArraySpec("f8", (n,)), ...)``) -- no device memory is involved."""

    def __init__(self, dtype, shape):
        self.dtype = np.dtype(dtype)
        self.shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        self.ndim = len(self.shape)
        self.size = int(np.prod(self.shape, dtype=np.int64))


_ARRAY_TYPES = (dpnp_array, usm_ndarray, ArraySpec)


def _array_of(x):
    return x._array_obj if isinstance(x, dpnp_array) else x


def _full_arrays(arrays):
    """The arguments that carry the iteration shape: everything but size-1 arrays of at
    most one dimension, which are broadcast (all of them, if there is nothing else)."""
    full = [a for a, _ in arrays if not (a.size == 1 and a.ndim <= 1)]
    return full or [a for a, _ in arrays]


class _Fused:
    def __init__(self, func, mode=None):
        functools.update_wrapper(self, func)
        self._func = func
        if mode is not None and mode not in MODES:
            raise ValueError(f"fuse(mode={mode!r}): expected one of {MODES}")
        self.mode = mode                   # None: default_mode() at every call
        self.last_executor = None          # "specialized" or "interpreted"
        self._cache = {}
        self.fused_calls = 0
        self.eager_calls = 0
        self.last_reason = None

    # -- signature of a call: what the compiled program depends on
    def _signature(self, args, kwargs):
        items = list(args) + [kwargs[k] for k in sorted(kwargs)]
        sig, arrays = [tuple(sorted(kwargs))], []
        for x in items:
            if isinstance(x, _ARRAY_TYPES):
                a = _array_of(x)
                same = next((i for i, (b, _) in enumerate(arrays) if b is a), None)
                if same is None:
                    arrays.append((a, x))
                    same = len(arrays) - 1
                sig.append(("a", a.dtype.str, a.shape, same))
            elif isinstance(x, (float, np.floating)):
                sig.append(("s", type(x), struct.pack("<d", float(x))))
            else:
                try:
                    hash(x)
                except TypeError:
                    return None, arrays
                sig.append(("o", type(x), x))
        return tuple(sig), arrays

    def _eligible(self, arrays):
        if not arrays:
            return "no array arguments"
        dt = arrays[0][0].dtype
        if dt not in (np.dtype("f4"), np.dtype("f8")):
            return f"dtype {dt}"
        full = _full_arrays(arrays)
        shape = full[0].shape
        for a, _ in arrays:
            if a.dtype != dt:
                return "mixed dtypes"
        for a in full:
            if a.shape != shape:
                return "different shapes"
        if int(np.prod(shape, dtype=np.int64)) == 0:
            return "empty arrays"
        if any(isinstance(a, ArraySpec) for a, _ in arrays):
            return None                                # a description, not memory
        q = arrays[0][0].sycl_queue
        for a, _ in arrays:
            if a.sycl_queue is not q and a.sycl_queue != q:
                return "arrays on different queues"
        for a in full:
            if not a.flags.c_contiguous:
                return "not C-contiguous"
        # distinct arguments must not share memory: elements are read and written
        # by different threads without ordering between them
        spans = sorted((a._ptr, a._ptr + a.size * a.itemsize) for a, _ in arrays)
        for (lo0, hi0), (lo1, hi1) in zip(spans, spans[1:]):
            if lo1 < hi0:
                return "overlapping arguments"
        return None

    def _trace(self, args, kwargs, arrays):
        full = _full_arrays(arrays)
        tr = _Tracer(arrays[0][0].dtype, full[0].shape)
        stand_ins = {}
        for slot, (a, _) in enumerate(arrays):
            stand_ins[id(a)] = FusedValue(tr, tr.node(("in", slot)), slot)

        def sub(x):
            if isinstance(x, _ARRAY_TYPES):
                return stand_ins[id(_array_of(x))]
            return x

        res = self._func(*[sub(x) for x in args], **{k: sub(v) for k, v in kwargs.items()})
        result_nodes = []

        def tree(r):
            if isinstance(r, FusedValue):
                if tr.flags[r._node]:
                    raise FusionUnsupported("boolean result")
                if r._slot is not None:
                    return ("slot", r._slot)           # an argument (written or not): hand it back
                k = tr.nodes[r._node]
                if k[0] == "imm":
                    raise FusionUnsupported("scalar result")
                result_nodes.append(r._node)
                return ("node", r._node)
            if isinstance(r, tuple):
                return ("tuple", tuple(tree(x) for x in r))
            if isinstance(r, list):
                return ("list", [tree(x) for x in r])
            if isinstance(r, dict):
                return ("dict", {k: tree(v) for k, v in r.items()})
            return ("const", r)

        results_tree = tree(res)
        scalar_slots = [not any(a is f for f in full) for a, _ in arrays]
        for slot in tr.stores:
            if scalar_slots[slot]:
                raise FusionUnsupported("store into a size-1 array")
        prog = _Program(tr, results_tree, list(dict.fromkeys(result_nodes)))
        prog.scalar_slots = scalar_slots
        return prog

    def _lookup(self, args, kwargs):
        """(program or None, reason it is not fused, the distinct array arguments)."""
        sig, arrays = self._signature(args, kwargs)
        reason = "unhashable argument" if sig is None else self._eligible(arrays)
        if reason is not None:
            return None, reason, arrays
        prog = self._cache.get(sig)
        if prog is None:
            try:
                prog = self._trace(args, kwargs, arrays)
            except FusionUnsupported as e:
                prog = str(e) or "unsupported"
            except (AttributeError, TypeError, ValueError, NotImplementedError, IndexError) as e:
                prog = f"{type(e).__name__}: {e}"
            if len(self._cache) >= _MAX_CACHED:        # scalars are part of the key: keep it bounded
                self._cache.pop(next(iter(self._cache)))
            self._cache[sig] = prog
        if isinstance(prog, str):
            return None, prog, arrays
        return prog, None, arrays

    def __call__(self, *args, **kwargs):
        prog, reason, arrays = self._lookup(args, kwargs)
        self.last_reason = reason
        if prog is None:
            self.eager_calls += 1
            return self._func(*args, **kwargs)
        self.fused_calls += 1
        return self._launch(prog, arrays)

    def _launch(self, prog, arrays):
        from . import tensor as dpt

        first_full = _full_arrays(arrays)[0]
        q = first_full.sycl_queue
        n = first_full.size
        ins = (C.c_void_p * max(1, len(prog.in_slots)))(*[arrays[s][0]._ptr for s in prog.in_slots])
        flags = (C.c_int32 * max(1, len(prog.in_slots)))(*[int(prog.scalar_slots[s]) for s in prog.in_slots])
        new, outs = {}, []
        for i, bind in enumerate(prog.out_bind):
            if bind[0] == "slot":
                outs.append(arrays[bind[1]][0]._ptr)
            else:
                new[i] = dpt.empty(first_full.shape, dtype=prog.dtype, sycl_queue=q)
                outs.append(new[i]._ptr)
        outp = (C.c_void_p * max(1, len(outs)))(*outs)
        desc = prog._descriptor(ins, flags, outp)
        mode = self.mode or default_mode()
        stream = C.c_void_p(q.stream)
        specialized = mode == "compile" or (mode == "auto" and specialize_available()
                                            and prog.specialize_failed is None)
        if specialized:
            status = _lib.lib.dpb_fused_elementwise_specialized(C.byref(desc), n, stream)
            if status == _lib.ERR_RUNTIME and mode == "auto":
                # the compiler is there but this chain did not build: remember why, interpret it
                prog.specialize_failed = _lib.last_error()
                specialized = False
            else:
                _lib.check(status)
        if not specialized:
            _lib.check(_lib.lib.dpb_fused_elementwise(C.byref(desc), n, stream))
        self.last_executor = "specialized" if specialized else "interpreted"

        def build(t):
            kind = t[0]
            if kind == "slot":
                return arrays[t[1]][1]
            if kind == "node":
                return dpnp_array._create_from_usm_ndarray(new[prog.result_out[t[1]]])
            if kind == "tuple":
                return tuple(build(x) for x in t[1])
            if kind == "list":
                return [build(x) for x in t[1]]
            if kind == "dict":
                return {k: build(v) for k, v in t[1].items()}
            return t[1]

        return build(prog.results_tree)

    def program(self, *args, **kwargs):
        """The compiled program for these arguments, or None if such a call is not fused
        (``last_reason`` then says why).  Array arguments may be :class:`ArraySpec`."""
        prog, self.last_reason, _ = self._lookup(args, kwargs)
        return prog


def fuse(func=None, /, **options):
    """Decorator: evaluate the elementwise chain in ``func`` with one kernel launch.

    ``@fuse`` and ``@fuse()`` are both accepted; ``mode`` is "auto" (default), "compile" or
    "interpret" (see the module docstring).  The wrapped callable has the attributes
    ``fused_calls`` / ``eager_calls`` / ``last_reason`` (why the last call was not fused) and
    ``last_executor`` ("specialized" or "interpreted")."""
    mode = options.pop("mode", None)
    if options:
        raise TypeError(f"fuse() got unexpected options {sorted(options)}")
    if func is None:
        return lambda f: _Fused(f, mode)
    return _Fused(func, mode)
