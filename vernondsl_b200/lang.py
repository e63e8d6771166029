"""A Taichi-style front end over libvrhi: enough of the surface fractal.py uses for that program
to run with its import line changed (``import vernondsl_b200.lang as ti``) and its GUI lines dropped.

Surface (reference lines): ``init`` (fractal.py:5), ``field`` (:8), ``@func`` (:11), ``Vector`` (:13),
``@kernel`` (:16), the struct-for ``for i, j in field`` (:18), ``cos`` (:19), ``.norm()`` (:22).

A kernel is not interpreted element by element anywhere.  Its Python source is parsed once and, at
each call, walked with symbolic values to recognise one of two shapes; the result is ONE launch of
a hand-written CUDA kernel:

* the escape-time shape of fractal.py:18-25 -- pixel-dependent start or constant, a
  ``while z.norm() < R and it < N`` (or ``z.norm_sqr() <= R``) loop whose body is the quadratic map
  ``z = z*z + c`` written any way that multiplies out to it, and a store of the count or of
  ``a - count*s`` -- becomes an ``escape_time`` launch;
* a loop body that is a pure elementwise expression of fields and uniforms becomes a ``map_tape``
  launch (one fused kernel).

Anything else raises ``LangError``: there is no interpreter fallback.

Index arithmetic: an expression affine in the loop indices, such as ``(i / n - 1) * 2``, is
evaluated exactly (rational arithmetic) to ``origin + index * step``, and origin and step are then
rounded to binary32 once; the device computes ``origin + float(index) * step``.  Uniform scalar
expressions (``ti.cos(t) * 0.2``) are evaluated on the host in binary32.  Arithmetic inside the
loop follows the kernel's fixed order (``vernondsl_b200/csrc/k_escape.cu``), which is the order of
fractal.py:13.
"""
from __future__ import annotations

import ast
import inspect
import math
import textwrap
from fractions import Fraction
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from . import _lib as L
from . import ops
from .rhi import Buffer, Device, Stream

cuda = "cuda"
gpu = "cuda"
gles = "cuda"      # fractal.py:5 asks for ti.gles; there is no graphics stack here, the kernels are CUDA
vulkan = "cuda"
cpu = "cpu"
f32 = np.float32
i32 = np.int32
u32 = np.uint32


class LangError(NotImplementedError):
    pass


# "independent_of": FrameLoop sets it while it records frames that go round its ring on one stream
# "plan_only": kernels are lowered but nothing is allocated or launched (see plan_only())
_state: Dict[str, Any] = {"dev": None, "stream": None, "independent_of": 0, "plan_only": False}


class plan_only:
    """``with ti.plan_only():`` fields created inside hold no device memory and kernels called inside are only
    lowered: ``kernel.last_plan``, ``kernel.last_params`` (escape-time shape) and ``kernel.last_tape``
    (elementwise shape) show what a real call would launch.  Nothing is computed: this is how the lowering
    is inspected, and tested, where there is no GPU."""

    def __enter__(self):
        self.before = _state["plan_only"]
        _state["plan_only"] = True
        return self

    def __exit__(self, *exc):
        _state["plan_only"] = self.before
        return False


def init(arch=cuda, device: int = 0, **_ignored) -> None:
    """fractal.py:5.  Opens the device.  ``arch=ti.cpu`` is refused: this backend has no CPU path."""
    if arch == cpu:
        raise LangError("vernondsl_b200 has no CPU backend")
    if _state["dev"] is None:
        _state["dev"] = Device(device)
        _state["stream"] = _state["dev"].stream()


def _runtime() -> Tuple[Device, Stream]:
    if _state["dev"] is None:
        init()
    return _state["dev"], _state["stream"]


def sync() -> None:
    _runtime()[1].check()


class Field:
    """Dense device array (fractal.py:8).  ``dtype`` float -> binary32, int -> int32."""

    def __init__(self, dtype, shape):
        self.shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        if dtype in (float, f32, np.dtype(np.float32)):
            self.dtype = np.dtype(np.float32)
        elif dtype in (int, i32, np.dtype(np.int32)):
            self.dtype = np.dtype(np.int32)
        elif dtype in (u32, np.dtype(np.uint32)):
            self.dtype = np.dtype(np.uint32)
        else:
            raise LangError(f"field dtype {dtype!r} is not supported")
        self.buffer: Optional[Buffer] = None     # stays None for a field made under plan_only()
        if not _state["plan_only"]:
            self.buffer = _runtime()[0].empty(self.shape, self.dtype, L.IMAGE)
            self.buffer.fill(0)

    def to_numpy(self) -> np.ndarray:
        if self.buffer is None:
            raise LangError("a field made under plan_only() holds no data")
        _runtime()[1].check()
        return self.buffer.download(dtype=self.dtype, shape=self.shape)

    def from_numpy(self, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a, dtype=self.dtype)
        if a.shape != self.shape:
            raise ValueError(f"shape {a.shape} does not match the field's {self.shape}")
        if self.buffer is None:
            raise LangError("a field made under plan_only() holds no data")
        self.buffer.upload(a)

    def fill(self, value) -> None:
        self.from_numpy(np.full(self.shape, value, dtype=self.dtype))


def field(dtype, shape) -> Field:
    return Field(dtype, shape)


# ------------------------------------------------------------------------------------------------
# Symbolic values used while a kernel body is walked.

class Sym:
    """An expression node: op in {"const", "index", "zvar", "field", unary/binary op names}."""
    __slots__ = ("op", "args", "value")

    def __init__(self, op, args=(), value=None):
        self.op, self.args, self.value = op, tuple(args), value

    # operator overloads build the tree
    def _b(self, op, o, swap=False):
        o = o if isinstance(o, Sym) else Sym("const", value=o)
        return Sym(op, (o, self) if swap else (self, o))

    def __add__(self, o): return self._b("add", o)
    def __radd__(self, o): return self._b("add", o, True)
    def __sub__(self, o): return self._b("sub", o)
    def __rsub__(self, o): return self._b("sub", o, True)
    def __mul__(self, o): return self._b("mul", o)
    def __rmul__(self, o): return self._b("mul", o, True)
    def __truediv__(self, o): return self._b("div", o)
    def __rtruediv__(self, o): return self._b("div", o, True)
    def __neg__(self): return Sym("neg", (self,))
    def __abs__(self): return Sym("abs", (self,))

    def __pow__(self, k):
        if k == 2:
            return Sym("mul", (self, self))
        raise LangError("only ** 2 is supported")


def _is_num(v) -> bool:
    return isinstance(v, (int, float, np.floating, np.integer, Fraction))


class Vector:
    """2-vectors only (fractal.py:13,19,20)."""

    def __init__(self, comps):
        comps = list(comps)
        if len(comps) != 2:
            raise LangError("only 2-component vectors are supported")
        self.c = comps

    def __getitem__(self, k): return self.c[k]
    def _zip(self, o, f): return Vector([f(a, b) for a, b in zip(self.c, o.c)]) if isinstance(o, Vector) else Vector([f(a, o) for a in self.c])
    def __add__(self, o): return self._zip(o, lambda a, b: a + b)
    def __sub__(self, o): return self._zip(o, lambda a, b: a - b)
    def __mul__(self, o): return self._zip(o, lambda a, b: a * b)
    def __rmul__(self, o): return self._zip(o, lambda a, b: b * a)
    def __truediv__(self, o): return self._zip(o, lambda a, b: a / b)

    def norm(self): return _NormOf(self, squared=False)
    def norm_sqr(self): return _NormOf(self, squared=True)


class _NormOf:
    def __init__(self, vec, squared): self.vec, self.squared = vec, squared


def _unary(name, pyfn):
    def f(x):
        if isinstance(x, Sym):
            return Sym(name, (x,))
        return f32(pyfn(f32(x)))  # uniform scalar: binary32 on the host
    return f


cos = _unary("cos", np.cos)
sin = _unary("sin", np.sin)
sqrt = _unary("sqrt", np.sqrt)
exp = _unary("exp", np.exp)
log = _unary("log", np.log)
tanh = _unary("tanh", np.tanh)


def abs(x):  # noqa: A001 - mirrors ti.abs
    return Sym("abs", (x,)) if isinstance(x, Sym) else f32(np.abs(f32(x)))


def max(a, b):  # noqa: A001
    if isinstance(a, Sym) or isinstance(b, Sym):
        a = a if isinstance(a, Sym) else Sym("const", value=a)
        return a._b("max", b)
    return a if a >= b else b


def min(a, b):  # noqa: A001
    if isinstance(a, Sym) or isinstance(b, Sym):
        a = a if isinstance(a, Sym) else Sym("const", value=a)
        return a._b("min", b)
    return a if a <= b else b


# --- analysis helpers ---------------------------------------------------------------------------

def _affine(e, n_index: int) -> Optional[List[Fraction]]:
    """[c0, c_index0, c_index1, ...] if e is affine in the loop indices with numeric coefficients."""
    zero = [Fraction(0)] * (n_index + 1)
    if _is_num(e):
        return [Fraction(float(e)) if not isinstance(e, (int, Fraction)) else Fraction(e)] + zero[1:]
    if not isinstance(e, Sym):
        return None
    if e.op == "const":
        return _affine(e.value, n_index)
    if e.op == "index":
        out = list(zero)
        out[1 + e.value] = Fraction(1)
        return out
    if e.op in ("add", "sub"):
        a, b = _affine(e.args[0], n_index), _affine(e.args[1], n_index)
        if a is None or b is None:
            return None
        return [x + y if e.op == "add" else x - y for x, y in zip(a, b)]
    if e.op == "neg":
        a = _affine(e.args[0], n_index)
        return None if a is None else [-x for x in a]
    if e.op in ("mul", "div"):
        a, b = _affine(e.args[0], n_index), _affine(e.args[1], n_index)
        if a is None or b is None:
            return None
        b_const = all(x == 0 for x in b[1:])
        a_const = all(x == 0 for x in a[1:])
        if e.op == "div":
            if not b_const or b[0] == 0:
                return None
            return [x / b[0] for x in a]
        if b_const:
            return [x * b[0] for x in a]
        if a_const:
            return [x * a[0] for x in b]
    return None


def _poly(e, names) -> Optional[Dict[Tuple[int, int], Fraction]]:
    """Polynomial of e in the two loop variables zvar0/zvar1 plus symbolic constants in `names`
    (treated as numbers through their placeholder values)."""
    if _is_num(e):
        return {(0, 0): Fraction(float(e)) if not isinstance(e, (int, Fraction)) else Fraction(e)}
    if not isinstance(e, Sym):
        return None
    if e.op == "const":
        return _poly(e.value, names)
    if e.op == "zvar":
        return {(1, 0): Fraction(1)} if e.value == 0 else {(0, 1): Fraction(1)}
    if e.op == "cconst":  # component of the constant c: a fresh symbol, carried as a tagged monomial
        return {("c", e.value): Fraction(1)}
    if e.op == "neg":
        a = _poly(e.args[0], names)
        return None if a is None else {k: -v for k, v in a.items()}
    if e.op in ("add", "sub"):
        a, b = _poly(e.args[0], names), _poly(e.args[1], names)
        if a is None or b is None:
            return None
        out = dict(a)
        for k, v in b.items():
            out[k] = out.get(k, Fraction(0)) + (v if e.op == "add" else -v)
        return {k: v for k, v in out.items() if v != 0}
    if e.op == "mul":
        a, b = _poly(e.args[0], names), _poly(e.args[1], names)
        if a is None or b is None:
            return None
        out: Dict[Any, Fraction] = {}
        for ka, va in a.items():
            for kb, vb in b.items():
                if isinstance(ka[0], str) or isinstance(kb[0], str):
                    if ka == (0, 0):
                        k = kb
                    elif kb == (0, 0):
                        k = ka
                    else:
                        return None  # c times a variable: not the quadratic map
                else:
                    k = (ka[0] + kb[0], ka[1] + kb[1])
                out[k] = out.get(k, Fraction(0)) + va * vb
        return {k: v for k, v in out.items() if v != 0}
    return None


# ------------------------------------------------------------------------------------------------
# The walker: a small evaluator over the subset of Python that kernel bodies use.

class _Walker:
    def __init__(self, fn, call_args):
        self.fn = fn
        src = textwrap.dedent(inspect.getsource(fn))
        tree = ast.parse(src)
        self.fdef = next(n for n in tree.body if isinstance(n, ast.FunctionDef))
        self.globals = fn.__globals__
        closure = {}
        if fn.__closure__:
            closure = {name: cell.cell_contents for name, cell in zip(fn.__code__.co_freevars, fn.__closure__)}
        self.env: Dict[str, Any] = dict(closure)
        params = [a.arg for a in self.fdef.args.args]
        if len(params) != len(call_args):
            raise TypeError(f"{fn.__name__}() takes {len(params)} arguments, {len(call_args)} given")
        for name, value, a in zip(params, call_args, self.fdef.args.args):
            ann = a.annotation
            is_float = isinstance(ann, ast.Name) and ann.id == "float"
            self.env[name] = f32(value) if is_float or isinstance(value, float) else value

    def lookup(self, name):
        if name in self.env:
            return self.env[name]
        if name in self.globals:
            return self.globals[name]
        import builtins
        if hasattr(builtins, name):
            return getattr(builtins, name)
        raise LangError(f"name {name!r} is not defined in the kernel's scope")

    def ev(self, node):
        if isinstance(node, ast.Constant):
            return node.value
        if isinstance(node, ast.Name):
            return self.lookup(node.id)
        if isinstance(node, ast.Attribute):
            return getattr(self.ev(node.value), node.attr)
        if isinstance(node, ast.List) or isinstance(node, ast.Tuple):
            return [self.ev(e) for e in node.elts]
        if isinstance(node, ast.UnaryOp):
            v = self.ev(node.operand)
            if isinstance(node.op, ast.USub):
                return -v
            if isinstance(node.op, ast.UAdd):
                return v
            raise LangError("unsupported unary operator")
        if isinstance(node, ast.BinOp):
            a, b = self.ev(node.left), self.ev(node.right)
            a = self._num(a)
            b = self._num(b)
            op = node.op
            if isinstance(op, ast.Add): return a + b
            if isinstance(op, ast.Sub): return a - b
            if isinstance(op, ast.Mult): return a * b
            if isinstance(op, ast.Div): return a / b
            if isinstance(op, ast.Pow): return a ** b
            raise LangError(f"unsupported operator {type(op).__name__}")
        if isinstance(node, ast.Subscript):
            base = self.ev(node.value)
            idx = self.ev(node.slice)
            if isinstance(base, Field):
                return self.field_read(base, idx if isinstance(idx, list) else [idx])
            return base[idx]
        if isinstance(node, ast.Call):
            f = self.ev(node.func)
            args = [self.ev(a) for a in node.args]
            if isinstance(f, _Func):
                return f.inline(args)
            return f(*args)
        raise LangError(f"unsupported expression: {ast.dump(node)[:80]}")

    @staticmethod
    def _num(v):
        # plain Python / numpy scalars met inside index arithmetic stay exact (Fractions) when they are integers
        if isinstance(v, bool):
            return int(v)
        return v

    def field_read(self, fld, idx):
        raise LangError("a field is read here, which this kernel shape does not allow")


class _Func:
    """@ti.func (fractal.py:11): inlined wherever a kernel calls it."""

    def __init__(self, fn):
        self.fn = fn
        src = textwrap.dedent(inspect.getsource(fn))
        self.fdef = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef))

    def inline(self, args):
        w = _Walker.__new__(_Walker)
        w.fn, w.fdef, w.globals = self.fn, self.fdef, self.fn.__globals__
        w.env = {a.arg: v for a, v in zip(self.fdef.args.args, args)}
        for stmt in self.fdef.body:
            if isinstance(stmt, ast.Return):
                return w.ev(stmt.value)
            if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Name):
                w.env[stmt.targets[0].id] = w.ev(stmt.value)
            elif isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant):
                continue
            else:
                raise LangError("a @func body may hold assignments and one return")
        raise LangError("@func without a return")

    def __call__(self, *args):
        return self.inline(list(args))


def func(fn):
    return _Func(fn)


class Kernel:
    """@ti.kernel (fractal.py:16).  Calling it plans and launches; nothing is cached across calls
    except the parsed source, so changing a uniform per frame (fractal.py:30-31) just relaunches."""

    def __init__(self, fn):
        self.fn = fn
        self.__name__ = fn.__name__
        self.last_plan: Optional[str] = None
        self.last_params = None
        self.last_tape = None

    def __call__(self, *args):
        st = None if _state["plan_only"] else _runtime()[1]     # None: lower only
        w = _Walker(self.fn, args)
        body = [s for s in w.fdef.body if not (isinstance(s, ast.Expr) and isinstance(s.value, ast.Constant))]
        if len(body) != 1 or not isinstance(body[0], ast.For):
            raise LangError("a kernel body must be one struct-for over a field")
        loop = body[0]
        target_field = w.ev(loop.iter)
        if not isinstance(target_field, Field):
            raise LangError("the struct-for must iterate over a field")
        names = [t.id for t in loop.target.elts] if isinstance(loop.target, ast.Tuple) else [loop.target.id]
        if len(names) != len(target_field.shape):
            raise LangError("the struct-for must bind one index per field dimension")
        for k, nm in enumerate(names):
            w.env[nm] = Sym("index", value=k)
        stmts = loop.body
        if any(isinstance(s, ast.While) for s in stmts):
            self._escape(w, st, target_field, names, stmts)
        else:
            self._map(w, st, target_field, names, stmts)

    # -- escape-time shape -----------------------------------------------------------------------
    def _escape(self, w: _Walker, st: Stream, fld: Field, names, stmts):
        if len(fld.shape) != 2:
            raise LangError("the escape-time shape needs a 2-D field")
        k_while = next(k for k, s in enumerate(stmts) if isinstance(s, ast.While))
        for s in stmts[:k_while]:
            if not (isinstance(s, ast.Assign) and len(s.targets) == 1 and isinstance(s.targets[0], ast.Name)):
                raise LangError("only simple assignments may precede the while loop")
            w.env[s.targets[0].id] = w.ev(s.value)
        loop: ast.While = stmts[k_while]
        # condition: <vec>.norm() < R and <it> < N   (either order)
        cond = loop.test
        if not (isinstance(cond, ast.BoolOp) and isinstance(cond.op, ast.And) and len(cond.values) == 2):
            raise LangError("the while condition must be `<z>.norm() < R and <count> < N`")
        zname = itname = None
        test = bound = max_iter = None
        for c in cond.values:
            if not (isinstance(c, ast.Compare) and len(c.ops) == 1):
                raise LangError("unsupported while condition")
            left = c.left
            if isinstance(left, ast.Call) and isinstance(left.func, ast.Attribute) and left.func.attr in ("norm", "norm_sqr"):
                if not isinstance(left.func.value, ast.Name):
                    raise LangError("the norm must be taken of a named vector")
                zname = left.func.value.id
                r = float(w.ev(c.comparators[0]))
                if left.func.attr == "norm" and isinstance(c.ops[0], ast.Lt):
                    test, bound = L.TEST_NORM_GE, r         # continue while sqrt(a+b) < R
                elif left.func.attr == "norm_sqr" and isinstance(c.ops[0], ast.LtE):
                    test, bound = L.TEST_NORM2_GT, r        # continue while a+b <= R
                else:
                    raise LangError("supported escape tests: `z.norm() < R` and `z.norm_sqr() <= R`")
            elif isinstance(left, ast.Name) and isinstance(c.ops[0], ast.Lt):
                itname = left.id
                max_iter = int(w.ev(c.comparators[0]))
            else:
                raise LangError("unsupported while condition")
        if zname is None or itname is None:
            raise LangError("the while condition must test the norm of z and the iteration count")
        z0 = w.env.get(zname)
        if not isinstance(z0, Vector):
            raise LangError(f"{zname} must be a 2-vector before the loop")
        if w.env.get(itname) != 0:
            raise LangError(f"{itname} must start at 0")
        # loop body: z = f(z) + c ; it += 1  (any order)
        z_update = None
        for s in loop.body:
            if isinstance(s, ast.AugAssign) and isinstance(s.target, ast.Name) and s.target.id == itname and isinstance(s.op, ast.Add) \
                    and isinstance(s.value, ast.Constant) and s.value.value == 1:
                continue
            if isinstance(s, ast.Assign) and len(s.targets) == 1 and isinstance(s.targets[0], ast.Name) and s.targets[0].id == zname:
                z_update = s.value
                continue
            raise LangError("the loop body must be `z = <quadratic map of z> + c` and `count += 1`")
        if z_update is None:
            raise LangError("the loop body does not update z")
        # which of z0 / c depends on the pixel?  evaluate the update with z symbolic and every
        # pixel-independent vector kept symbolic through tagged constants
        pre_env = dict(w.env)
        cvec = None
        for nm, v in pre_env.items():
            if nm != zname and isinstance(v, Vector):
                cvec = (nm, v) if cvec is None else cvec
        w.env[zname] = Vector([Sym("zvar", value=0), Sym("zvar", value=1)])
        if cvec is not None:
            w.env[cvec[0]] = Vector([Sym("cconst", value=0), Sym("cconst", value=1)])
        new_z = w.ev(z_update)
        w.env = pre_env
        if not isinstance(new_z, Vector):
            raise LangError("the update of z must produce a 2-vector")
        want_re = {(2, 0): Fraction(1), (0, 2): Fraction(-1), ("c", 0): Fraction(1)}
        want_im = {(1, 1): Fraction(2), ("c", 1): Fraction(1)}
        if _poly(new_z[0], ()) != want_re or _poly(new_z[1], ()) != want_im:
            raise LangError("the loop body is not the quadratic map z*z + c")
        if cvec is None:
            raise LangError("no constant vector c found")
        c = cvec[1]
        n_idx = 2
        aff_z = [_affine(z0[0], n_idx), _affine(z0[1], n_idx)]
        aff_c = [_affine(c[0], n_idx), _affine(c[1], n_idx)]
        if any(a is None for a in aff_z + aff_c):
            raise LangError("z and c must be affine in the loop indices")
        z_const = all(a[1] == 0 and a[2] == 0 for a in aff_z)
        c_const = all(a[1] == 0 and a[2] == 0 for a in aff_c)
        if c_const and not z_const:
            kind, pix = L.JULIA, aff_z
            cr, ci = float(f32(float(aff_c[0][0]))), float(f32(float(aff_c[1][0])))
        elif z_const and not c_const and aff_z[0][0] == 0 and aff_z[1][0] == 0:
            kind, pix, cr, ci = L.MANDELBROT, aff_c, 0.0, 0.0
        else:
            raise LangError("either z starts at the pixel and c is constant (Julia) or z starts at 0 and c is the pixel (Mandelbrot)")
        # the field is indexed [i0, i1] in row-major order: i0 is the row, i1 the column
        re, im = pix
        if re[2] == 0 and im[1] == 0 and re[1] != 0 and im[2] != 0:
            transposed = True      # real part follows the row index (fractal.py:20 with the field of :8)
            y0, dy, x0, dx = re[0], re[1], im[0], im[2]
        elif re[1] == 0 and im[2] == 0 and re[2] != 0 and im[1] != 0:
            transposed = False
            x0, dx, y0, dy = re[0], re[2], im[0], im[1]
        else:
            raise LangError("each coordinate must depend on exactly one loop index")
        # store: fld[i, j] = count   or   a - count * s
        tail = stmts[k_while + 1:]
        if len(tail) != 1 or not (isinstance(tail[0], ast.Assign) and isinstance(tail[0].targets[0], ast.Subscript)):
            raise LangError("after the loop exactly one store into the field is expected")
        store = tail[0]
        if w.ev(store.targets[0].value) is not fld:
            raise LangError("the store must go to the field the loop iterates over")
        w.env[itname] = Sym("index", value=2)  # count as a third 'index' to read the colour expression as affine
        a3 = _affine(w.ev(store.value), 3)
        if a3 is None or a3[1] != 0 or a3[2] != 0:
            raise LangError("the stored value must be affine in the iteration count")
        rows, cols = fld.shape
        if a3[0] == 0 and a3[3] == 1 and fld.dtype != np.float32:
            output, scale = L.OUT_COUNT_U32, 0.0
        elif a3[0] == 1 and a3[3] < 0 and fld.dtype == np.float32:
            output, scale = L.OUT_COLOR_F32, float(f32(float(-a3[3])))
        else:
            raise LangError("stores supported: the count into an integer field, or 1 - count*s into a float field")
        p = ops.escape_params(kind, cols, rows, float(f32(float(x0))), float(f32(float(y0))), float(f32(float(dx))),
                              float(f32(float(dy))), cr=cr, ci=ci, max_iter=max_iter, test=test, bound=bound, output=output,
                              color_scale=scale, transposed=transposed, independent_of=_state["independent_of"])
        self.last_plan = f"escape_time kind={'julia' if kind == L.JULIA else 'mandelbrot'} {cols}x{rows} transposed={transposed}"
        self.last_params = p
        if st is None:
            return
        if fld.buffer is None:
            raise LangError("the field was made under plan_only() and holds no device memory")
        ops.escape_time(st, fld.buffer, p)

    # -- elementwise shape -----------------------------------------------------------------------
    def _map(self, w: _Walker, st: Stream, fld: Field, names, stmts):
        inputs: List[Tuple[Field, str]] = []

        def field_read(f: Field, idx):
            kinds = [i.value if isinstance(i, Sym) and i.op == "index" else None for i in idx]
            n = len(names)
            if len(f.shape) == n and kinds == list(range(n)):
                shape = "full"
            elif n == 2 and len(f.shape) == 1 and kinds == [1] and f.shape[0] == fld.shape[1]:
                shape = "row"
            elif n == 2 and len(f.shape) == 1 and kinds == [0] and f.shape[0] == fld.shape[0]:
                shape = "col"
            else:
                raise LangError("fields may be read at the loop indices only (or a 1-D field at one of them)")
            if f.dtype != np.float32:
                raise LangError("elementwise kernels read float fields")
            for k, (g, s) in enumerate(inputs):
                if g is f and s == shape:
                    return Sym("field", value=k)
            inputs.append((f, shape))
            return Sym("field", value=len(inputs) - 1)

        w.field_read = field_read
        outputs: List[Tuple[Field, Any]] = []
        for s in stmts:
            if isinstance(s, ast.Assign) and len(s.targets) == 1 and isinstance(s.targets[0], ast.Name):
                w.env[s.targets[0].id] = w.ev(s.value)
            elif isinstance(s, ast.Assign) and len(s.targets) == 1 and isinstance(s.targets[0], ast.Subscript):
                out_f = w.ev(s.targets[0].value)
                idx = w.ev(s.targets[0].slice)
                idx = idx if isinstance(idx, list) else [idx]
                if not isinstance(out_f, Field) or out_f.shape != fld.shape or out_f.dtype != np.float32 or \
                        [i.value if isinstance(i, Sym) and i.op == "index" else None for i in idx] != list(range(len(names))):
                    raise LangError("stores must write float fields of the loop's shape at the loop indices")
                outputs.append((out_f, w.ev(s.value)))
            else:
                raise LangError("an elementwise kernel body holds assignments and stores only")
        if not outputs:
            raise LangError("the kernel stores nothing")
        tape = ops.Tape(len(inputs), row_vectors=[k for k, (_, s) in enumerate(inputs) if s == "row"],
                        col_vectors=[k for k, (_, s) in enumerate(inputs) if s == "col"])
        memo: Dict[int, int] = {}

        def emit(e) -> int:
            if _is_num(e):
                return tape.const(float(f32(float(e))))
            if id(e) in memo:
                return memo[id(e)]
            if e.op == "const":
                v = emit(e.value)
            elif e.op == "field":
                v = tape.input(e.value)
            elif e.op == "index":
                raise LangError("loop indices may only address fields in an elementwise kernel")
            elif len(e.args) == 1:
                v = tape.op(e.op, emit(e.args[0]))
            else:
                v = tape.op(e.op, emit(e.args[0]), emit(e.args[1]))
            memo[id(e)] = v
            return v

        for _, e in outputs:
            tape.output(emit(e if isinstance(e, Sym) else Sym("const", value=e)))
        rows, cols = (fld.shape if len(fld.shape) == 2 else (1, fld.shape[0]))
        self.last_plan = f"map_tape inputs={len(inputs)} outputs={len(outputs)} instr={len(tape.instr)}"
        self.last_tape = tape
        if st is None:
            return
        if any(f.buffer is None for f, _ in list(inputs) + list(outputs)):
            raise LangError("a field was made under plan_only() and holds no device memory")
        ops.map_tape(st, tape, [f.buffer for f, _ in inputs], [f.buffer for f, _ in outputs], rows, cols)


def kernel(fn):
    return Kernel(fn)


class FrameLoop:
    """The frame loop of fractal.py:30-33 without its window: ``for i in range(...): paint(i * 0.03)``
    followed by a blit becomes a recorded run of launches whose frames land in a ring of device
    buffers (there is no graphics stack to show them; ``frame(k)`` downloads one).

    ``record(uniforms)`` walks the kernel once per frame on the host (each frame's uniforms become
    part of the recording) and records the launches; ``play()`` replays all of them with a single
    submission, which is what matters for small frames whose cost is the launch.  Calling ``record``
    again with other uniforms re-targets the existing recording in place.
    """

    def __init__(self, kern: "Kernel", target: Field, ring: int = 4, streams: int = 2, overlap: bool = True):
        if ring < 1:
            raise ValueError("the ring needs at least one frame")
        if not 1 <= streams <= 4:
            raise ValueError("1..4 streams")
        while ring % streams:       # frames that share a ring slot must share a stream, or their order is lost
            streams -= 1
        dev, st = _runtime()
        self.kernel, self.target, self.stream = kern, target, st
        # frames go to the streams in turn: consecutive frames write different ring slots, so the next
        # frame's first blocks may start while the last blocks of this one drain
        self.streams: List[Stream] = [st] + [dev.stream() for _ in range(streams - 1)]
        self.ring: List[Buffer] = [target.buffer] + [dev.empty(target.shape, target.dtype, L.IMAGE) for _ in range(ring - 1)]
        # with one stream the frames still overlap where the ring allows it: each launch is declared independent
        # of the ring - 1 frames before it (they write other slots), which lets it begin before they end
        self.independent_of = min(7, ring - 1) if overlap and len(self.streams) == 1 else 0
        self.seq = None
        self.frames = 0

    def record(self, uniforms) -> None:
        uniforms = [u if isinstance(u, (tuple, list)) else (u,) for u in uniforms]
        if not uniforms:
            raise ValueError("nothing to record")
        home = self.target.buffer
        try:
            if self.seq is None:
                for s in self.streams:      # sizes the operator's scratch on every stream: nothing may allocate while recording
                    _state["stream"] = s
                    self.kernel(*uniforms[0])
                    s.check()
            n_streams = min(len(self.streams), len(uniforms))
            with self.stream.record(self.seq) as seq:
                for s in self.streams[1:n_streams]:
                    self.stream.fork_recording(s)
                _state["independent_of"] = self.independent_of
                for k, u in enumerate(uniforms):
                    self.target.buffer = self.ring[k % len(self.ring)]
                    _state["stream"] = self.streams[k % n_streams]
                    self.kernel(*u)
            self.seq = seq
            self.frames = len(uniforms)
        finally:
            self.target.buffer = home
            _state["stream"] = self.stream
            _state["independent_of"] = 0

    def play(self) -> None:
        if self.seq is None:
            raise LangError("record() a run of frames first")
        self.seq.launch(self.stream)

    def frame(self, k: int) -> np.ndarray:
        """Frame ``k`` of the last replay (the ring keeps only the last ``ring`` frames)."""
        if not (0 <= k < self.frames) or k < self.frames - len(self.ring):
            raise IndexError("that frame is no longer in the ring")
        self.stream.check()
        return self.ring[k % len(self.ring)].download(dtype=self.target.dtype, shape=self.target.shape)

    def close(self) -> None:
        if self.seq is not None:
            self.seq.close()
            self.seq = None
        for b in self.ring[1:]:
            b.close()
        self.ring = self.ring[:1]
        for s in self.streams[1:]:
            s.close()
        self.streams = self.streams[:1]
