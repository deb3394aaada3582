"""CPU oracle: a restatement of sage's lazy graph, its op lowering and its
kernels, in numpy + the C loops of sage_oracle.c.

TEST INFRASTRUCTURE ONLY.  Nothing under sage_b200/ imports this module; only
tests/, __graft_entry__.smoke() and the cpu_baseline / --impl reference legs of
bench.py may.  It never touches a GPU.

Each function cites the reference file:line (paths inside ingim/sage) that it
follows.  Every op is evaluated as its own "kernel" (the reference's map-fusion
only removes intermediate stores; it does not change the arithmetic apart from
floating-point contraction, which the tolerances in tests/ allow for).

Parity status: pinned by the reference's own golden vectors for map, reduce,
argmax, gemm, gather, slice/unslice/concat, im2col/col2im/conv_2d, relu,
softmax, softmax_cross_entropy and max_pool_2d (tests/test_oracle_golden.py).
layer_norm, matmul_batched, Bert, ResNet, accuracy and the optimizers (Sgd,
Adam) have no vector in the reference: parity unpinned there; this restatement
is the arbiter.
"""
import ctypes
import heapq
import itertools
import math
import os
import subprocess

import numpy as np

FLOAT, INT, UINT = "float", "int", "uint"
NP = {FLOAT: np.float32, INT: np.int32, UINT: np.uint32}
_HERE = os.path.dirname(os.path.abspath(__file__))


def _load():
    so = os.path.join(_HERE, "libsage_oracle.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return ctypes.CDLL(so)


_C = _load()
_i64p = ctypes.POINTER(ctypes.c_int64)


def _arr(v):
    return (ctypes.c_int64 * max(len(v), 1))(*[int(a) for a in v])


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def num_threads():
    return int(_C.o_num_threads())


def set_num_threads(n):
    """OpenMP threads for the C loops (a launcher's OMP_NUM_THREADS=1 would otherwise make them serial)."""
    _C.o_set_num_threads(int(n))
    return num_threads()


# --------------------------------------------------------------------------- shape
class Shape:
    """src/shape.rs:37-279."""

    def __init__(self, extents, strides=None, offset=0):
        self.extents = [int(e) for e in extents]
        self.strides = list(strides) if strides is not None else Shape.default_strides(self.extents)
        self.offset = int(offset)

    @staticmethod
    def default_strides(extents):  # shape.rs:45-54
        out, size = [], int(np.prod(extents, dtype=np.int64)) if len(extents) else 1
        for e in extents:
            size //= e
            out.append(size)
        return out

    def size(self):
        return int(np.prod(self.extents, dtype=np.int64)) if self.extents else 1

    def rank(self):
        return len(self.extents)

    def clone(self):
        return Shape(self.extents, self.strides, self.offset)

    def has_default_strides(self):  # shape.rs:134-143
        return self.strides == Shape.default_strides(self.extents)

    def extract(self, axes):  # shape.rs:113-132 with nested = true
        keep = [a for a in range(self.rank()) if a not in axes]
        inner = Shape([self.extents[a] for a in axes], [self.strides[a] for a in axes], 0)
        outer = Shape([self.extents[a] for a in keep], [self.strides[a] for a in keep], self.offset)
        return inner, outer

    def remove(self, axis):
        s = self.clone()
        del s.extents[axis], s.strides[axis]
        return s

    def insert(self, axis):  # shape.rs:190-195: new unit axis gets stride 0
        s = self.clone()
        s.extents.insert(axis, 1)
        s.strides.insert(axis, 0)
        return s

    def permute(self, axes):
        return Shape([self.extents[a] for a in axes], [self.strides[a] for a in axes], self.offset)

    def select_range(self, start, end_incl, axis):  # shape.rs:229-237
        assert self.extents[axis] > end_incl, "index out of bounds"
        s = self.clone()
        s.offset += self.strides[axis] * start
        s.extents[axis] = end_incl - start + 1
        return s

    def expand(self, extents):  # shape.rs:239-279
        assert len(extents) >= self.rank()
        ne, ns = list(self.extents), list(self.strides)
        for _ in range(len(extents) - self.rank()):
            ne.insert(0, 1)
            ns.insert(0, 0)
        for i, e in enumerate(extents):
            if ne[i] != e:
                assert ne[i] == 1, "invalid broadcast"
                ne[i], ns[i] = e, 0
        return Shape(ne, ns, self.offset)


def union(e1, e2):  # shape.rs:356-393
    e1, e2 = list(e1), list(e2)
    if e1 == e2:
        return e1
    longer, shorter = (e1, e2) if len(e1) > len(e2) else (e2, e1)
    u = longer[: len(longer) - len(shorter)] + shorter
    for i, (a, b) in enumerate(zip(u, longer)):
        if a != b:
            if a == 1:
                u[i] = b
            elif b != 1:
                raise ValueError("invalid broadcast")
    return u


def to_extents(extents, size):  # shape.rs:400-441 (one -1 may be inferred)
    if isinstance(extents, (int, np.integer)):
        extents = [extents]
    extents = [int(e) for e in extents]
    if -1 in extents:
        known = int(np.prod([e for e in extents if e != -1], dtype=np.int64))
        assert extents.count(-1) == 1 and size > 0 and size % known == 0
        extents[extents.index(-1)] = size // known
    elif size > 0:
        assert int(np.prod(extents, dtype=np.int64)) == size, "size mismatch"
    return extents


def to_axis(axis, bound):  # shape.rs:517-545
    axis = int(axis)
    if axis < 0:
        axis += bound
    assert 0 <= axis < bound, "axis out of bounds"
    return axis


def to_axes(axes, bound):
    if axes is None:
        return list(range(bound))
    if isinstance(axes, (int, np.integer)):
        axes = [axes]
    return [to_axis(a, bound) for a in axes]


# --------------------------------------------------------------------------- tensor
class Tensor:
    """Shared flat buffer + Shape + dtype (src/tensor.rs:106-110)."""

    def __init__(self, buf, shape, dtype):
        self.buf, self.shape, self.dtype = buf, shape, dtype

    @staticmethod
    def new(array, dtype=None):
        a = np.asarray(array)
        if dtype is None:
            dtype = FLOAT if a.dtype.kind == "f" else (UINT if a.dtype.kind == "u" else INT)
        a = np.ascontiguousarray(a, dtype=NP[dtype])
        return Tensor(a.reshape(-1), Shape(a.shape if a.ndim else [1]), dtype)

    def view_np(self):
        """Strided numpy view over the buffer (read-only use)."""
        base = self.buf[self.shape.offset:]
        return np.lib.stride_tricks.as_strided(
            base, shape=self.shape.extents, strides=[s * 4 for s in self.shape.strides], writeable=False)

    def numpy(self):
        return np.ascontiguousarray(self.view_np())

    def with_shape(self, shape):
        return Tensor(self.buf, shape, self.dtype)


# --------------------------------------------------------------------------- graph
class Var:
    """src/var.rs:22-42.  A Python object plays the role of the shared Rc<Origin>."""
    _counter = itertools.count()

    def __init__(self, shape, dtype, op=None, inputs=(), data=None):
        self.shape, self.dtype, self.op, self.inputs, self.data = shape, dtype, op, list(inputs), data
        self.t_order = (max(v.t_order for v in self.inputs) + 1) if (op and self.inputs) else 0
        self.uid = next(Var._counter)

    @staticmethod
    def new(t):
        if not isinstance(t, Tensor):
            t = Tensor.new(t)
        return Var(t.shape.clone(), t.dtype, data=t)

    @staticmethod
    def empty(extents, dtype=FLOAT):
        return Var(Shape(to_extents(extents, 0)), dtype)

    def set(self, t):  # var.rs:370-377
        assert self.op is None
        self.data = t if isinstance(t, Tensor) else Tensor.new(t, self.dtype)

    extents = property(lambda self: self.shape.extents)

    def extent(self, axis):
        return self.shape.extents[to_axis(axis, self.rank())]

    def rank(self):
        return self.shape.rank()

    def size(self):
        return self.shape.size()

    def is_op(self):
        return self.op is not None

    def eval(self):
        return evaluate([self])[0]

    def grad(self, y):  # var.rs:326-335: d y / d self
        return grad(y, [self])[0]

    # arithmetic sugar (src/ops/map.rs:1180-1370)
    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return sub(self, o)
    def __rsub__(self, o): return sub(o, self)
    def __mul__(self, o): return mul(self, o)
    def __rmul__(self, o): return mul(o, self)
    def __truediv__(self, o): return div(self, o)
    def __rtruediv__(self, o): return div(o, self)
    def __neg__(self): return neg(self)

    def organize(self):  # var.rs:506-512
        return self if self.shape.has_default_strides() else copy(self)


def into_var(v):  # var.rs:817-861
    if isinstance(v, Var):
        return v
    if isinstance(v, Tensor):
        return Var.new(v)
    if isinstance(v, (float, np.floating)):
        return scalar(float(v), [1])
    if isinstance(v, (int, np.integer)):
        return scalar(int(v), [1])
    return Var.new(Tensor.new(v))


def evaluate(targets):
    """Evaluate every op reachable from `targets` once, in topological order."""
    order, seen, stack = [], set(), [(t, False) for t in targets]
    while stack:
        v, done = stack.pop()
        if done:
            order.append(v)
            continue
        if v.uid in seen:
            continue
        seen.add(v.uid)
        stack.append((v, True))
        for x in v.inputs:
            if x.uid not in seen:
                stack.append((x, False))
    vals = {}
    for v in order:
        if v.op is None:
            assert v.data is not None, "uninitialized variable"
            vals[v.uid] = v.data
        else:
            vals[v.uid] = v.op.compute([vals[x.uid] for x in v.inputs])
    return [vals[t.uid] for t in targets]


def grad(y, xs):
    """src/var.rs:56-103: reverse mode, max-heap on topological order."""
    heap, grads = [], {}
    grads[y.uid] = scalar(1.0, y.extents)
    heapq.heappush(heap, (-y.t_order, y.uid, y))
    while heap:
        _, _, v = heapq.heappop(heap)
        gy = grads[v.uid]
        if v.op is not None:
            gxs = v.op.grad(v.inputs, v, gy)
            for x, gx in zip(v.inputs, gxs):
                if gx is None:
                    continue
                assert gx.extents == x.extents, "grad shape error"
                if x.uid not in grads:
                    heapq.heappush(heap, (-x.t_order, x.uid, x))
                    grads[x.uid] = gx
                else:
                    grads[x.uid] = add(gx, grads[x.uid])
    return [grads[x.uid] for x in xs]


# --------------------------------------------------------------------------- map ops
def _erf(x):
    return np.vectorize(math.erf, otypes=[np.float64])(x.astype(np.float64)).astype(np.float32)


def _round_half_away(x):
    return np.where(x >= 0, np.floor(x + np.float32(0.5)), np.ceil(x - np.float32(0.5))).astype(np.float32)


_F = np.float32
UNARY = {  # src/ops/map.rs:224-258
    "copy": lambda x: x.copy(), "abs": np.abs, "neg": lambda x: -x,
    "recip": lambda x: _F(1) / x, "log": np.log, "exp": np.exp, "sqrt": np.sqrt,
    "square": lambda x: x * x, "erf": _erf, "sign": np.sign, "ceil": np.ceil,
    "floor": np.floor, "round": _round_half_away, "sin": np.sin, "sinh": np.sinh,
    "cos": np.cos, "cosh": np.cosh, "tan": np.tan, "tanh": np.tanh, "asin": np.arcsin,
    "asinh": np.arcsinh, "acos": np.arccos, "acosh": np.arccosh, "atan": np.arctan,
    "atanh": np.arctanh, "not": lambda x: (x == 0), "int": lambda x: np.trunc(x),
    "float": lambda x: x,
}
BINARY = {  # src/ops/map.rs:260-286
    "add": np.add, "sub": np.subtract, "div": np.divide, "mul": np.multiply,
    "mod": np.fmod, "pow": np.power, "min": np.fmin, "max": np.fmax,
    "and": lambda a, b: (a != 0) & (b != 0), "or": lambda a, b: (a != 0) | (b != 0),
    "eq": np.equal, "ne": np.not_equal, "gt": np.greater, "ge": np.greater_equal,
    "lt": np.less, "le": np.less_equal,
}
_LOGIC = {"and", "or", "eq", "ne", "gt", "ge", "lt", "le"}


class NullaryMap:
    def __init__(self, value, extents, dtype):
        self.value, self.extents, self.dtype = value, extents, dtype

    def compute(self, x):  # map.rs:898-921
        return Tensor.new(np.full(self.extents, self.value, dtype=NP[self.dtype]), self.dtype)

    def grad(self, xs, y, gy):
        return []


class UnaryMap:
    def __init__(self, kind, out_dtype):
        self.kind, self.out_dtype = kind, out_dtype

    def compute(self, x):  # map.rs:970-998
        with np.errstate(all="ignore"):
            r = UNARY[self.kind](x[0].view_np())
        return Tensor.new(np.asarray(r).astype(NP[self.out_dtype]), self.out_dtype)

    def grad(self, xs, y, gy):  # map.rs:937-968
        x, k = xs[0], self.kind
        g = {
            "copy": lambda: gy, "abs": lambda: sign(x) * gy, "neg": lambda: -gy,
            "recip": lambda: -gy / square(x), "log": lambda: gy / x, "exp": lambda: gy * y,
            "sqrt": lambda: gy / (y * 2.0), "square": lambda: gy * x * 2.0,
            "erf": lambda: gy * float(np.float32(2.0) / np.sqrt(np.float32(math.pi))) / exp(square(x)),
            "sign": lambda: scalar(0.0, x.extents), "ceil": lambda: scalar(0.0, x.extents),
            "floor": lambda: scalar(0.0, x.extents), "round": lambda: scalar(0.0, x.extents),
            "sin": lambda: gy * cos(x), "sinh": lambda: gy * cosh(x), "cos": lambda: -gy * sin(x),
            "cosh": lambda: gy * sinh(x), "tan": lambda: gy / square(cos(x)),
            "tanh": lambda: gy / square(cosh(x)), "asin": lambda: gy / sqrt(-square(x) + 1.0),
            "asinh": lambda: gy / sqrt(square(x) + 1.0), "acos": lambda: -gy / sqrt(-square(x) + 1.0),
            "acosh": lambda: gy / sqrt(square(x) - 1.0), "atan": lambda: gy / (square(x) + 1.0),
            "atanh": lambda: gy / (-square(x) + 1.0), "not": lambda: None,
            "int": lambda: gy, "float": lambda: gy,
        }[k]()
        return [g]


class BinaryMap:
    def __init__(self, kind, out_dtype):
        self.kind, self.out_dtype = kind, out_dtype

    def compute(self, x):  # map.rs:1044-1078
        with np.errstate(all="ignore"):
            r = BINARY[self.kind](x[0].view_np(), x[1].view_np())
        return Tensor.new(np.asarray(r).astype(NP[self.out_dtype]), self.out_dtype)

    def grad(self, x, y, gy):  # map.rs:1014-1042
        k = self.kind
        if k == "add": return [gy, gy]
        if k == "sub": return [gy, -gy]
        if k == "div": return [gy / x[1], gy * (-x[0] / square(x[1]))]
        if k == "mul": return [gy * x[1], gy * x[0]]
        if k == "mod": return [gy, -gy * floor(x[0] / x[1])]
        if k == "pow": return [gy * x[1] * pow_(x[0], x[1] - 1.0), gy * pow_(x[0], x[1]) * log(x[0])]
        if k == "min": return [gy * float_(lt(x[0], x[1])), gy * float_(ge(x[0], x[1]))]
        if k == "max": return [gy * float_(lt(x[1], x[0])), gy * float_(ge(x[1], x[0]))]
        return [None, None]


class TernaryCond:
    def compute(self, x):  # map.rs:1101-1120
        r = np.where(x[0].view_np() != 0, x[1].view_np(), x[2].view_np())
        return Tensor.new(r, x[1].dtype)

    def grad(self, x, y, gy):  # map.rs:1094-1099
        return [cond(x[0], gy, 0.0), cond(x[0], 0.0, gy), None]


def scalar(val, extents):  # map.rs:517-531
    dtype = FLOAT if isinstance(val, float) else INT
    ext = to_extents(extents, 0)
    return Var(Shape(ext), dtype, NullaryMap(val, ext, dtype))


def unary_map(x, kind):  # map.rs:458-481
    x = into_var(x)
    dt = x.dtype if kind in ("sign", "copy", "abs", "neg") else {"not": UINT, "int": INT}.get(kind, FLOAT)
    return Var(Shape(x.extents), dt, UnaryMap(kind, dt), [x])


def broadcast(x1, x2):  # map.rs:412-429
    x1, x2 = into_var(x1), into_var(x2)
    u = union(x1.extents, x2.extents)
    if x1.extents != u: x1 = expand(x1, u)
    if x2.extents != u: x2 = expand(x2, u)
    return x1, x2


def binary_map(x1, x2, kind):  # map.rs:483-513
    x1, x2 = broadcast(x1, x2)
    assert x1.dtype == x2.dtype
    dt = UINT if kind in _LOGIC else x1.dtype
    return Var(Shape(x1.extents), dt, BinaryMap(kind, dt), [x1, x2])


def cond(c, x1, x2):  # map.rs:861-883
    c, x1, x2 = into_var(c), into_var(x1), into_var(x2)
    u = union(union(c.extents, x1.extents), union(x1.extents, x2.extents))
    c, x1, x2 = [v if v.extents == u else expand(v, u) for v in (c, x1, x2)]
    assert x1.dtype == x2.dtype and c.dtype == UINT
    return Var(Shape(x1.extents), x1.dtype, TernaryCond(), [c, x1, x2])


def _u(kind):
    return lambda x: unary_map(x, kind)


def _b(kind):
    return lambda a, b: binary_map(a, b, kind)


copy, abs_, neg, recip, log, exp, sqrt, square, erf, sign = map(_u, ["copy", "abs", "neg", "recip", "log", "exp", "sqrt", "square", "erf", "sign"])
ceil, floor, round_, sin, sinh, cos, cosh, tan, tanh = map(_u, ["ceil", "floor", "round", "sin", "sinh", "cos", "cosh", "tan", "tanh"])
asin, asinh, acos, acosh, atan, atanh, not_, int_, float_ = map(_u, ["asin", "asinh", "acos", "acosh", "atan", "atanh", "not", "int", "float"])
add, sub, div, mul, modular, pow_, minimum, maximum = map(_b, ["add", "sub", "div", "mul", "mod", "pow", "min", "max"])
and_, or_, eq, ne, gt, ge, lt, le = map(_b, ["and", "or", "eq", "ne", "gt", "ge", "lt", "le"])


# --------------------------------------------------------------------------- layout ops
class ViewOp:
    """Zero-copy layout ops (src/ops/core.rs:203-523)."""

    def __init__(self, kind, **kw):
        self.kind, self.kw = kind, kw

    def compute(self, x):
        t, k, kw = x[0], self.kind, self.kw
        if k == "reshape":  # core.rs:246-260
            s = kw["shape"].clone()
            s.offset += t.shape.offset
            return t.with_shape(s)
        if k == "expand": return t.with_shape(t.shape.expand(kw["extents"]))
        if k == "permute": return t.with_shape(t.shape.permute(kw["perm"]))
        if k == "squeeze": return t.with_shape(t.shape.remove(kw["axis"]))
        if k == "unsqueeze": return t.with_shape(t.shape.insert(kw["axis"]))
        if k == "slice": return t.with_shape(t.shape.select_range(kw["start"], kw["end"] - 1, kw["axis"]))
        raise KeyError(k)

    def grad(self, x, y, gy):
        k, kw, x0 = self.kind, self.kw, x[0]
        if k == "reshape": return [reshape(gy, Shape(x0.shape.extents, x0.shape.strides, x0.shape.offset))]
        if k == "expand":  # core.rs:292-313
            surplus = gy.rank() - x0.rank()
            axes = list(range(surplus)) + [i + surplus for i in range(x0.rank()) if gy.extent(i + surplus) != x0.extent(i)]
            return [view(sum_(gy, axes, False), x0.extents)]
        if k == "permute": return [permute(gy, kw["perm"])]  # as written: core.rs:387-390
        if k == "squeeze": return [unsqueeze(gy, kw["axis"])]
        if k == "unsqueeze": return [squeeze(gy, kw["axis"])]
        if k == "slice": return [unslice(gy, kw["axis"], kw["start"], x0.extent(kw["axis"]))]


def reshape(x, shape):  # core.rs:213-236
    x = into_var(x).organize()
    assert x.size() == shape.size(), "incompatible size"
    return Var(shape, x.dtype, ViewOp("reshape", shape=shape), [x])


def view(x, extents):  # core.rs:203-211
    x = into_var(x)
    return reshape(x, Shape(to_extents(extents, x.size())))


def expand(x, extents):  # core.rs:263-281
    x = into_var(x)
    ext = to_extents(extents, 0)
    return Var(x.shape.expand(ext), x.dtype, ViewOp("expand", extents=ext), [x])


def permute(x, axes):  # core.rs:358-377
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    return Var(x.shape.permute(axes), x.dtype, ViewOp("permute", perm=axes), [x])


def transpose(x, a1, a2):  # core.rs:330-356
    x = into_var(x)
    a1, a2 = to_axis(a1, x.rank()), to_axis(a2, x.rank())
    return permute(x, [a2 if i == a1 else a1 if i == a2 else i for i in range(x.rank())])


def tr(x):
    return transpose(x, 0, 1)


def squeeze(x, axis):  # core.rs:400-419
    x = into_var(x)
    axis = to_axis(axis, x.rank())
    assert x.extents[axis] == 1
    return Var(x.shape.remove(axis), x.dtype, ViewOp("squeeze", axis=axis), [x])


def unsqueeze(x, axis):  # core.rs:439-458
    x = into_var(x)
    axis = to_axis(axis, x.rank() + 1)
    return Var(x.shape.insert(axis), x.dtype, ViewOp("unsqueeze", axis=axis), [x])


def slice_(x, axis, start, end):  # core.rs:478-500
    x = into_var(x)
    axis = to_axis(axis, x.rank())
    return Var(x.shape.select_range(start, end - 1, axis), x.dtype, ViewOp("slice", axis=axis, start=start, end=end), [x])


def index(x, axis, i):  # var.rs:573-578
    return slice_(x, axis, i, i + 1)


class Unslice:
    def __init__(self, axis, start, end):
        self.axis, self.start, self.end = axis, start, end

    def compute(self, x):  # core.rs:571-610
        xv = x[0].view_np()
        ext = list(xv.shape)
        ext[self.axis] = self.end
        y = np.zeros(ext, dtype=NP[x[0].dtype])
        sl = [slice(None)] * len(ext)
        sl[self.axis] = slice(self.start, self.start + xv.shape[self.axis])
        y[tuple(sl)] = xv
        return Tensor.new(y, x[0].dtype)

    def grad(self, x, y, gy):
        return [slice_(gy, self.axis, self.start, self.start + x[0].extent(self.axis))]


def unslice(x, axis, start, end):  # core.rs:525-551
    x = into_var(x)
    axis = to_axis(axis, x.rank())
    assert end >= start + x.extent(axis)
    ext = list(x.extents)
    ext[axis] = end
    return Var(Shape(ext), x.dtype, Unslice(axis, start, end), [x])


class Gather:
    def __init__(self, axis):
        self.axis = axis

    def compute(self, x):  # core.rs:655-718
        t, ind = x
        y = np.empty(ind.shape.size(), dtype=NP[t.dtype])
        _C.o_gather(_ptr(t.buf), t.shape.rank(), _arr(t.shape.strides), ctypes.c_int64(t.shape.offset),
                    _ptr(ind.buf), _arr(ind.shape.extents), _arr(ind.shape.strides),
                    ctypes.c_int64(ind.shape.offset), self.axis, _ptr(y))
        return Tensor(y, Shape(ind.shape.extents), t.dtype)

    def grad(self, x, y, gy):
        return [scatter(gy, x[1], self.axis, x[0].extents), None]


def gather(x, ind, axis):  # core.rs:613-640
    x, ind = into_var(x), into_var(ind)
    axis = to_axis(axis, x.rank())
    assert x.rank() == ind.rank()
    return Var(Shape(ind.extents), x.dtype, Gather(axis), [x, ind])


class Scatter:
    def __init__(self, axis, extents):
        self.axis, self.extents = axis, extents

    def compute(self, x):  # core.rs:764-833
        t, ind = x
        assert t.dtype == FLOAT
        if any(s == 0 and e > 1 for s, e in zip(ind.shape.strides, ind.shape.extents)):
            # A broadcast index (Embedding's gradient: token ids expanded along the embedding axis).  The
            # reference's kernel decomposes the work-item id by the index tensor's strides and divides
            # by the zero stride (core.rs:795-806): there is no behaviour to restate, so the operator's
            # definition is applied, y[.., ind[i], ..] += x[i], in work-item order.
            y = np.zeros(self.extents, dtype=np.float32)
            where = list(np.indices(ind.shape.extents))
            where[self.axis] = ind.numpy().astype(np.int64)
            np.add.at(y, tuple(where), t.numpy())
            return Tensor(y.reshape(-1), Shape(self.extents), t.dtype)
        y = np.empty(int(np.prod(self.extents)), dtype=np.float32)
        _C.o_scatter(_ptr(t.buf), t.shape.rank(), _arr(t.shape.strides), ctypes.c_int64(t.shape.offset),
                     _ptr(ind.buf), _arr(ind.shape.extents), _arr(ind.shape.strides),
                     ctypes.c_int64(ind.shape.offset), self.axis, _arr(self.extents), _ptr(y))
        return Tensor(y, Shape(self.extents), t.dtype)

    def grad(self, x, y, gy):
        return [gather(gy, x[1], self.axis), None]


def scatter(x, ind, axis, extents):  # core.rs:721-749
    x, ind = into_var(x), into_var(ind)
    axis = to_axis(axis, x.rank())
    extents = to_extents(extents, 0)
    assert len(extents) == x.rank() == ind.rank()
    return Var(Shape(extents), x.dtype, Scatter(axis, extents), [x, ind])


class Concat:
    def __init__(self, axis):
        self.axis = axis

    def compute(self, x):  # core.rs:892-934
        return Tensor.new(np.concatenate([t.view_np() for t in x], axis=self.axis), x[0].dtype)

    def grad(self, x, y, gy):
        out, i = [], 0
        for v in x:
            e = v.extent(self.axis)
            out.append(slice_(gy, self.axis, i, i + e))
            i += e
        return out


def concat(xs, axis):  # core.rs:836-876
    xs = [into_var(v) for v in xs]
    axis = to_axis(axis, xs[0].rank())
    ext = list(xs[0].extents)
    ext[axis] = sum(v.extent(axis) for v in xs)
    return Var(Shape(ext), xs[0].dtype, Concat(axis), xs)


# --------------------------------------------------------------------------- reduce
_RED = {"sum": 0, "prod": 1, "max": 2, "min": 3}
_DT = {FLOAT: 0, INT: 1, UINT: 2}


def reduced_extents(extents, axes, preserve):  # reduce.rs:124-140
    out = [e if i not in axes else 1 for i, e in enumerate(extents) if i not in axes or preserve]
    return out or [1]


class Reduce:
    def __init__(self, kind, axes, preserve):
        self.kind, self.axes, self.preserve = kind, axes, preserve

    def compute(self, x):  # reduce.rs:258-325
        t = x[0]
        inner, outer = t.shape.extract(self.axes)
        ext = reduced_extents(t.shape.extents, self.axes, self.preserve)
        y = np.empty(int(np.prod(ext)), dtype=NP[t.dtype])
        _C.o_reduce(_ptr(t.buf), _DT[t.dtype], _RED[self.kind], outer.rank(), _arr(outer.extents),
                    _arr(outer.strides), ctypes.c_int64(outer.offset), inner.rank(), _arr(inner.extents),
                    _arr(inner.strides), _ptr(y))
        return Tensor(y, Shape(ext), t.dtype)

    def grad(self, xs, y, gy):  # reduce.rs:236-256
        x = xs[0]
        if not self.preserve:
            ext = reduced_extents(x.extents, self.axes, True)
            y, gy = view(y, ext), view(gy, ext)
        if self.kind == "sum": return [expand(gy, x.extents)]
        if self.kind == "prod": return [gy * y / x]
        return [cond(eq(x, y), gy, 0.0)]


def reduce(x, axes, preserve, kind):  # reduce.rs:203-224
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    return Var(Shape(reduced_extents(x.extents, axes, preserve)), x.dtype, Reduce(kind, axes, preserve), [x])


def sum_(x, axes, preserve=False): return reduce(x, axes, preserve, "sum")
def prod(x, axes, preserve=False): return reduce(x, axes, preserve, "prod")
def max_(x, axes, preserve=False): return reduce(x, axes, preserve, "max")
def min_(x, axes, preserve=False): return reduce(x, axes, preserve, "min")


def mean(x, axes, preserve=False):  # reduce.rs:59-71
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    size = float(np.prod([x.extent(a) for a in axes]))
    r = reduce(x, axes, preserve, "sum")
    return r / scalar(size, r.extents)


def var(x, axes, preserve=False):  # reduce.rs:73-82
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    return mean(square(x), axes, preserve) - square(mean(x, axes, preserve))


class ReduceArg:
    def __init__(self, is_max, axis, preserve):
        self.is_max, self.axis, self.preserve = is_max, axis, preserve

    def compute(self, x):  # reduce.rs:372-431
        t = x[0]
        inner, outer = t.shape.extract([self.axis])
        ext = reduced_extents(t.shape.extents, [self.axis], self.preserve)
        y = np.empty(int(np.prod(ext)), dtype=np.uint32)
        _C.o_reduce_arg(_ptr(t.buf), int(self.is_max), outer.rank(), _arr(outer.extents), _arr(outer.strides),
                        ctypes.c_int64(outer.offset), ctypes.c_int64(inner.extents[0]),
                        ctypes.c_int64(inner.strides[0]), _ptr(y))
        return Tensor(y, Shape(ext), UINT)

    def grad(self, x, y, gy):
        return [None]


def argmax(x, axis, preserve=False):
    x = into_var(x)
    axis = to_axis(axis, x.rank())
    return Var(Shape(reduced_extents(x.extents, [axis], preserve)), UINT, ReduceArg(True, axis, preserve), [x])


def argmin(x, axis, preserve=False):
    x = into_var(x)
    axis = to_axis(axis, x.rank())
    return Var(Shape(reduced_extents(x.extents, [axis], preserve)), UINT, ReduceArg(False, axis, preserve), [x])


# --------------------------------------------------------------------------- gemm
USE_FMA = 1  # which of the two roundings an OpenCL compiler may pick for c += a*b


class Gemm:
    def __init__(self, ta, tb, batched):
        self.ta, self.tb, self.batched = ta, tb, batched

    def compute(self, x):  # gemm.rs:176-250, 338-421
        a, b = x
        o = 1 if self.batched else 0
        h_ax, c_ax = (1, 0) if self.ta else (0, 1)
        w_ax = 0 if self.tb else 1
        m, k, n = a.shape.extents[h_ax + o], a.shape.extents[c_ax + o], b.shape.extents[w_ax + o]
        L = ctypes.c_int64
        if not self.batched:
            y = np.empty(m * n, dtype=np.float32)
            _C.o_gemm(int(self.ta), int(self.tb), L(m), L(n), L(k), _ptr(a.buf), L(a.shape.offset),
                      L(a.shape.strides[0]), _ptr(b.buf), L(b.shape.offset), L(b.shape.strides[0]),
                      _ptr(y), L(0), L(n), USE_FMA)
            return Tensor(y, Shape([m, n]), FLOAT)
        batch = a.shape.extents[0]
        y = np.empty(batch * m * n, dtype=np.float32)
        _C.o_gemm_batched(int(self.ta), int(self.tb), L(batch), L(m), L(n), L(k), _ptr(a.buf), L(a.shape.offset),
                          L(a.shape.strides[1]), L(a.shape.strides[0]), _ptr(b.buf), L(b.shape.offset),
                          L(b.shape.strides[1]), L(b.shape.strides[0]), _ptr(y), L(0), L(n), L(m * n), USE_FMA)
        return Tensor(y, Shape([batch, m, n]), FLOAT)

    def grad(self, x, y, gy):  # gemm.rs:150-163, 304-328
        g = gemm_batched if self.batched else gemm
        ta, tb = self.ta, self.tb
        if (ta, tb) == (False, False): return [g(gy, x[1], False, True), g(x[0], gy, True, False)]
        if (ta, tb) == (False, True): return [g(gy, x[1], False, False), g(gy, x[0], True, False)]
        if (ta, tb) == (True, False): return [g(x[1], gy, False, True), g(x[0], gy, False, False)]
        return [g(x[1], gy, True, True), g(gy, x[0], True, True)]


def _gemm_dims(e1, e2, t1, t2):
    h, c1 = (e1[1], e1[0]) if t1 else (e1[0], e1[1])
    w, c2 = (e2[0], e2[1]) if t2 else (e2[1], e2[0])
    assert c1 == c2
    return h, w


def gemm(x1, x2, t1=False, t2=False):  # gemm.rs:106-140
    x1, x2 = into_var(x1).organize(), into_var(x2).organize()
    h, w = _gemm_dims(x1.extents, x2.extents, t1, t2)
    return Var(Shape([h, w]), x1.dtype, Gemm(t1, t2, False), [x1, x2])


def gemm_batched(x1, x2, t1=False, t2=False):  # gemm.rs:253-290
    x1, x2 = into_var(x1).organize(), into_var(x2).organize()
    assert x1.extent(0) == x2.extent(0)
    h, w = _gemm_dims(x1.extents[1:], x2.extents[1:], t1, t2)
    return Var(Shape([x1.extent(0), h, w]), x1.dtype, Gemm(t1, t2, True), [x1, x2])


def matmul(x1, x2):  # gemm.rs:30-51
    x1, x2 = into_var(x1), into_var(x2)
    ext = x1.extents[:-1] + x2.extents[1:]
    a = view(x1, [x1.size() // x1.extent(-1), x1.extent(-1)])
    b = view(x2, [x2.extent(0), x2.size() // x2.extent(0)])
    return view(gemm(a, b, False, False), ext)


def matmul_batched(x1, x2):  # gemm.rs:53-104
    x1, x2 = into_var(x1), into_var(x2)
    batch_ext = []
    for i in range(min(x1.rank() - 2, x2.rank() - 2)):
        if x1.extent(i) == x2.extent(i):
            batch_ext.append(x1.extent(i))
        else:
            break
    bl, bs = len(batch_ext), int(np.prod(batch_ext)) if batch_ext else 0
    assert bl > 0, "batch dim incorrect!"
    ext = batch_ext + x1.extents[bl:x1.rank() - 1] + x2.extents[bl + 1:]
    a = view(x1, [bs, x1.size() // (x1.extent(-1) * bs), x1.extent(-1)])
    b = view(x2, [bs, x2.extent(bl), x2.size() // (x2.extent(bl) * bs)])
    return view(gemm_batched(a, b, False, False), ext)


# --------------------------------------------------------------------------- conv
def _pair(v):  # SizedExtent<2> (shape.rs:684-704); element order is [w, h]
    return [int(v), int(v)] if isinstance(v, (int, np.integer)) else [int(v[0]), int(v[1])]


def conv_size(size, ker, stride, pad, dil):  # conv.rs:47-59
    return [(size[i] + 2 * pad[i] - dil[i] * (ker[i] - 1) - 1) // stride[i] + 1 for i in range(2)]


class Im2col:
    def __init__(self, col_size, ker, stride, pad, dil):
        self.col_size, self.ker, self.stride, self.pad, self.dil = col_size, ker, stride, pad, dil

    def compute(self, x):  # conv.rs:289-374
        t = x[0]
        n, img_h, img_w, chan = t.shape.extents
        ext = [n, self.col_size[1], self.col_size[0], self.ker[1], self.ker[0], chan]
        y = np.empty(int(np.prod(ext)), dtype=np.float32)
        L = ctypes.c_int64
        _C.o_im2col(_ptr(t.buf[t.shape.offset:]), _ptr(y), L(n), L(chan), L(img_w), L(img_h), L(self.col_size[0]),
                    L(self.col_size[1]), L(self.ker[0]), L(self.ker[1]), L(self.stride[0]), L(self.stride[1]),
                    L(self.pad[0]), L(self.pad[1]), L(self.dil[0]), L(self.dil[1]))
        return Tensor(y, Shape(ext), FLOAT)

    def grad(self, x, y, gy):
        return [col2im(gy, [x[0].extent(2), x[0].extent(1)], self.ker, self.stride, self.pad, self.dil)]


class Col2im:
    def __init__(self, img_size, ker, stride, pad, dil):
        self.img_size, self.ker, self.stride, self.pad, self.dil = img_size, ker, stride, pad, dil

    def compute(self, x):  # conv.rs:404-498
        t = x[0]
        n, col_h, col_w, _, _, chan = t.shape.extents
        ext = [n, self.img_size[1], self.img_size[0], chan]
        y = np.empty(int(np.prod(ext)), dtype=np.float32)
        L = ctypes.c_int64
        _C.o_col2im(_ptr(t.buf[t.shape.offset:]), _ptr(y), L(n), L(chan), L(self.img_size[0]), L(self.img_size[1]),
                    L(col_w), L(col_h), L(self.ker[0]), L(self.ker[1]), L(self.stride[0]), L(self.stride[1]),
                    L(self.pad[0]), L(self.pad[1]), L(self.dil[0]), L(self.dil[1]))
        return Tensor(y, Shape(ext), FLOAT)

    def grad(self, x, y, gy):
        return [im2col(gy, self.ker, self.stride, self.pad, self.dil)]


def im2col(x, ker, stride, pad, dil):  # conv.rs:188-226
    x = into_var(x).organize()
    ker, stride, pad, dil = _pair(ker), _pair(stride), _pair(pad), _pair(dil)
    assert x.rank() == 4
    col = conv_size([x.extent(2), x.extent(1)], ker, stride, pad, dil)
    ext = [x.extent(0), col[1], col[0], ker[1], ker[0], x.extent(3)]
    return Var(Shape(ext), x.dtype, Im2col(col, ker, stride, pad, dil), [x])


def col2im(x, img_size, ker, stride, pad, dil):  # conv.rs:229-264
    x = into_var(x).organize()
    assert x.rank() == 6
    ext = [x.extent(0), img_size[1], img_size[0], x.extent(5)]
    return Var(Shape(ext), x.dtype, Col2im(list(img_size), _pair(ker), _pair(stride), _pair(pad), _pair(dil)), [x])


def conv_2d(x, filt, stride, pad, dil):  # conv.rs:61-96
    filt = into_var(filt)
    kh, kw, cin, cout = filt.extents
    col = im2col(x, [kw, kh], stride, pad, dil)
    n, ch, cw = col.extents[:3]
    return view(matmul(view(col, [n * ch * cw, kh * kw * cin]), view(filt, [kh * kw * cin, cout])), [n, ch, cw, cout])


def avg_pool_2d(x, ker, stride, pad, dil):  # conv.rs:143-153
    return mean(im2col(x, ker, stride, pad, dil), [3, 4], False)


def max_pool_2d(x, ker, stride, pad, dil):  # conv.rs:155-165
    return max_(im2col(x, ker, stride, pad, dil), [3, 4], False)


def batch_norm_2d(x, gamma, beta, mean_, var_, eps):  # conv.rs:167-185
    xc = (into_var(x) - into_var(mean_)) / sqrt(into_var(var_) + float(np.float32(eps)))
    return into_var(gamma) * xc + into_var(beta)


# --------------------------------------------------------------------------- nn
def relu(x):  # nn.rs:33-40
    x = into_var(x)
    return float_(gt(x, 0.0)) * x


def softmax(x, axes):  # nn.rs:42-56
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    y = exp(x - max_(x, axes, True))
    return y / sum_(y, axes, True)


def log_sum_exp(x, axes):  # nn.rs:58-68
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    c = max_(x, axes, True)
    return log(sum_(exp(x - c), axes, True)) + c


def softmax_cross_entropy(x1, x2):  # nn.rs:70-82
    x1, x2 = into_var(x1), into_var(x2)
    log_z = x1 - log_sum_exp(x1, 1)
    return -sum_(gather(log_z, x2, 1), 1, False)


def layer_norm(x, axes, gamma, beta, eps):  # nn.rs:84-100
    x = into_var(x)
    axes = to_axes(axes, x.rank())
    m = mean(x, axes, True)
    v = var(x, axes, True)
    xc = (x - m) / sqrt(v + float(np.float32(eps)))
    return xc * gamma + beta


def gelu_erf(x):
    """Not in the reference (its Bert uses ReLU): 0.5*x*(1+erf(x/sqrt(2))), built from sage's map ops."""
    x = into_var(x)
    return x * 0.5 * (erf(x / float(np.float32(math.sqrt(2.0)))) + 1.0)


# --------------------------------------------------------------------------- layers / models
class Dense:  # layers.rs:208-247
    def __init__(self, din, dout):
        self.weight, self.bias = Var.empty([din, dout]), Var.empty([dout])

    def params(self): return [self.weight, self.bias]
    def __call__(self, x): return matmul(x, self.weight) + self.bias


class Conv2d:  # layers.rs:327-404; weight [KH,KW,C,OC]
    def __init__(self, cin, cout, ker, stride=1, pad=0, dil=1):
        k = _pair(ker)
        self.weight, self.bias = Var.empty([k[1], k[0], cin, cout]), Var.empty([cout])
        self.stride, self.pad, self.dil = _pair(stride), _pair(pad), _pair(dil)

    def params(self): return [self.weight, self.bias]
    def __call__(self, x): return conv_2d(x, self.weight, self.stride, self.pad, self.dil) + self.bias


class Embedding:  # layers.rs:406-463
    def __init__(self, n, dim):
        self.dim, self.weight = dim, Var.empty([n, dim])

    def params(self): return [self.weight]

    def __call__(self, idx):
        if idx.rank() > 1:
            b, l = idx.extent(0), idx.extent(1)
            i = expand(view(idx, [b * l, 1]), [b * l, self.dim])
            return view(gather(self.weight, i, 0), [b, l, self.dim])
        l = idx.extent(0)
        i = expand(view(idx, [l, 1]), [l, self.dim])
        return view(gather(self.weight, i, 0), [l, self.dim])


class LayerNorm:  # layers.rs:548-590: eps argument is ignored, 1e-05 is hard-coded; gamma/beta are [1]
    def __init__(self, axes, eps=None, use_eps=None):
        self.axes, self.gamma, self.beta = axes, Var.empty([1]), Var.empty([1])
        self.eps = 1e-05 if use_eps is None else use_eps

    def params(self): return [self.gamma, self.beta]
    def __call__(self, x): return layer_norm(x, self.axes, self.gamma, self.beta, self.eps)


class BatchNorm2d:  # layers.rs:479-546: params are gamma, beta ([1] each); pass() hard-codes eps 1e-05
    def __init__(self, num_features, eps=1e-05):
        self.gamma, self.beta = Var.empty([1]), Var.empty([1])
        self.running_mean, self.running_var = Var.empty([num_features]), Var.empty([num_features])

    def params(self): return [self.gamma, self.beta]
    def buffers(self): return [self.running_mean, self.running_var]
    def __call__(self, x): return batch_norm_2d(x, self.gamma, self.beta, self.running_mean, self.running_var, 1e-05)


class Relu:
    def params(self): return []
    def __call__(self, x): return relu(x)


class Gelu:
    def params(self): return []
    def __call__(self, x): return gelu_erf(x)


class MaxPool2d:  # layers.rs:56-88
    def __init__(self, ker, stride, pad, dil): self.a = (ker, stride, pad, dil)
    def params(self): return []
    def __call__(self, x): return max_pool_2d(x, *self.a)


class AdaptiveAvgPool2d:  # layers.rs:124-154
    def __init__(self, ext): self.ext = _pair(ext)
    def params(self): return []

    def __call__(self, x):
        iw, ih = x.extent(2), x.extent(1)
        ow, oh = self.ext
        stride = [iw // ow, ih // oh]
        ker = [iw - (ow - 1) * stride[0], ih - (oh - 1) * stride[1]]
        return avg_pool_2d(x, ker, stride, [0, 0], [1, 1])


class Flatten:  # layers.rs:198-206
    def params(self): return []
    def __call__(self, x): return view(x, [x.extent(0), -1])


class Sequential:  # layers.rs:275-325
    def __init__(self, *layers): self.layers = list(layers)
    def add(self, l): self.layers.append(l); return self
    def params(self): return [p for l in self.layers for p in l.params()]
    def buffers(self): return [p for l in self.layers for p in (l.buffers() if hasattr(l, "buffers") else [])]

    def __call__(self, x):
        for l in self.layers:
            x = l(x)
        return x


class BertConfig:  # models/bert.rs:8-55 (base()); `large` is not constructible in the reference
    def __init__(self, embed_dim=768, num_vocabs=30522, max_num_tokens=512, hidden_dim=3072, num_layers=12,
                 num_heads=12, num_classes=2, gelu=False, ln_eps=None):
        self.embed_dim, self.num_vocabs, self.max_num_tokens = embed_dim, num_vocabs, max_num_tokens
        self.hidden_dim, self.num_layers, self.num_heads, self.num_classes = hidden_dim, num_layers, num_heads, num_classes
        self.gelu, self.ln_eps = gelu, ln_eps


class MultiHeadAttention:  # models/bert.rs:219-331
    def __init__(self, c):
        e = c.embed_dim
        self.num_heads, self.head_dim = c.num_heads, e // c.num_heads
        self.key_proj, self.query_proj, self.value_proj, self.dense = Dense(e, e), Dense(e, e), Dense(e, e), Dense(e, e)
        self.norm = LayerNorm([2], use_eps=c.ln_eps)

    def params(self):
        return self.key_proj.params() + self.query_proj.params() + self.value_proj.params() + self.dense.params() + self.norm.params()

    def separate_heads(self, f):
        return transpose(view(f, [f.extent(0), f.extent(1), self.num_heads, self.head_dim]), 2, 1)

    def merge_heads(self, f):
        f = transpose(f, 2, 1)
        return view(f, [f.extent(0), f.extent(1), self.num_heads * self.head_dim])

    def extend_mask(self, mask):
        m = view(mask, [mask.extent(0), 1, 1, mask.extent(1)])
        return (-m + 1.0) * -1e5

    def __call__(self, x, mask):
        q, k, v = self.query_proj(x), self.key_proj(x), self.value_proj(x)
        q, k, v = self.separate_heads(q), self.separate_heads(k), self.separate_heads(v)
        att = matmul_batched(q, transpose(k, -1, -2)) / float(np.sqrt(np.float32(self.head_dim)))
        att = softmax(att + self.extend_mask(mask), [3])
        y = self.dense(self.merge_heads(matmul_batched(att, v)))
        return self.norm(y + x)


class BertLayer:  # models/bert.rs:174-217
    def __init__(self, c):
        self.attention = MultiHeadAttention(c)
        self.ffn = Sequential(Dense(c.embed_dim, c.hidden_dim), Gelu() if c.gelu else Relu(), Dense(c.hidden_dim, c.embed_dim))
        self.norm = LayerNorm([2], use_eps=c.ln_eps)

    def params(self): return self.attention.params() + self.ffn.params() + self.norm.params()

    def __call__(self, x, mask):
        interim = self.attention(x, mask)
        return self.norm(self.ffn(interim) + interim)


class Bert:  # models/bert.rs:57-139
    def __init__(self, c):
        self.word_emb, self.pos_emb = Embedding(c.num_vocabs, c.embed_dim), Embedding(c.max_num_tokens, c.embed_dim)
        self.emb_norm = LayerNorm([2], use_eps=c.ln_eps)
        self.layers = [BertLayer(c) for _ in range(c.num_layers)]
        self.classifier = Dense(c.embed_dim, c.num_classes)

    def params(self):
        p = self.word_emb.params() + self.pos_emb.params() + self.emb_norm.params()
        for l in self.layers:
            p += l.params()
        return p + self.classifier.params()

    def __call__(self, token_ids, mask):
        pos_ids = Var.new(Tensor.new(np.arange(token_ids.extent(1), dtype=np.uint32), UINT))
        x = self.emb_norm(self.word_emb(token_ids) + self.pos_emb(pos_ids))
        for l in self.layers:
            x = l(x, mask)
        cls = squeeze(index(x, 1, 1), 1)  # the reference reads position 1
        return self.classifier(cls)


class BasicLayer:  # models/resnet.rs:150-177, 270-279
    def __init__(self, cin, planes, stride, batch_norm=False):
        if batch_norm:  # the two BatchNorm2d lines the reference has commented out (resnet.rs:167,170)
            self.main = Sequential(Conv2d(cin, planes, 3, stride, 1, 1), BatchNorm2d(planes), Relu(),
                                   Conv2d(planes, planes, 3, 1, 1, 1), BatchNorm2d(planes))
        else:
            self.main = Sequential(Conv2d(cin, planes, 3, stride, 1, 1), Relu(), Conv2d(planes, planes, 3, 1, 1, 1))
        self.down = Sequential(Conv2d(cin, planes, 1, stride, 0, 1)) if (stride != 1 or cin != planes) else None

    def params(self): return self.main.params() + (self.down.params() if self.down else [])
    def buffers(self): return self.main.buffers() + (self.down.buffers() if self.down else [])

    def __call__(self, x):
        y = self.main(x)
        return relu(y + (self.down(x) if self.down else x))


def resnet18(chan_input, num_classes, batch_norm=False):  # models/resnet.rs:74-129 with d18
    # BatchNorm is commented out in the reference (:80, :167, :170); batch_norm=True puts it back at those places
    m = Sequential(Conv2d(chan_input, 64, 7, 2, 3, 1))
    if batch_norm:
        m.add(BatchNorm2d(64))
    m.add(Relu()).add(MaxPool2d(3, 2, 1, 1))
    cin, cout = 64, 64
    for i in range(4):
        stride = 1 if i == 0 else 2
        blk, c = Sequential(), cin
        for j in range(2):
            blk.add(BasicLayer(c, cout, stride if j == 0 else 1, batch_norm))
            c = cout
        m.add(blk)
        cin, cout = cout, cout * 2
    m.add(AdaptiveAvgPool2d([1, 1])).add(Flatten()).add(Dense(512, num_classes))
    return m


# --------------------------------------------------------------------------- metric, optimizers
def accuracy(logits, labels):  # ops/metric.rs:4-17
    top = argmax(logits, 1, True)
    return float_(sum_(eq(top, labels), [0], False)) / float(top.size())


def grad_param(y, model):  # var.rs:46-54
    params = model.params()
    return dict(zip(params, grad(y, params)))


def _f32(x):
    return float(np.float32(x))


class Sgd:  # optim.rs:14-94
    """Only the plain rule is reachable in the reference: there is no setter for momentum, and with
    momentum != 0 update() unwraps a buffer it never stored (optim.rs:68-69)."""

    def __init__(self, lr):
        self.lr, self.momentum, self.weight_decay = _f32(lr), 0.0, 0.0

    def init(self):
        pass

    def update(self, grads):
        """grads: {param Var: grad Var}; every gradient is evaluated against the old parameters first
        (the reference runs its compiled program before update(), examples/train.rs:52-54)."""
        assert self.momentum == 0.0, "unreachable in the reference"
        keys = list(grads.keys())
        values = evaluate([grads[p] for p in keys])
        for p, gt in zip(keys, values):
            assert p.op is None, "param is not data tensor"
            g = Var.new(gt)
            if self.weight_decay != 0.0:
                g = g + p * self.weight_decay
            p.set((p - g * self.lr).eval())  # optim.rs:82,90


class Adam:  # optim.rs:97-178
    """No tests or golden values exist for the optimizers in the reference: parity unpinned; the
    restatement follows update() expression by expression, with the oracle's own map kernels."""

    def __init__(self, lr):
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = _f32(lr), _f32(0.9), _f32(0.999), _f32(1e-08), 0.0
        self.init()

    def init(self):  # :128-132
        self.m_t, self.v_t = {}, {}
        self.t = Tensor.new(np.float32([1.0]))

    def update(self, grads):
        keys = list(grads.keys())
        values = evaluate([grads[p] for p in keys])
        t = Var.new(self.t)
        for p, gt in zip(keys, values):
            assert p.op is None, "param is not data tensor"
            key = grads[p].uid
            g = Var.new(gt)
            if self.weight_decay != 0.0:
                g = g + p * self.weight_decay
            if key in self.m_t:  # :147-151
                m = Var.new(self.m_t[key]) * self.beta1 + g * _f32(np.float32(1.0) - np.float32(self.beta1))
            else:
                m = scalar(0.0, p.extents)
            self.m_t[key] = m.eval()
            if key in self.v_t:  # :155-159
                v = Var.new(self.v_t[key]) * self.beta2 + pow_(g, 2.0) * _f32(np.float32(1.0) - np.float32(self.beta2))
            else:
                v = scalar(0.0, p.extents)
            self.v_t[key] = v.eval()
            m, v = Var.new(self.m_t[key]), Var.new(self.v_t[key])
            m_hat = m / (neg(pow_(scalar(self.beta1, [1]), t)) + 1.0)  # :168-169
            v_hat = v / (neg(pow_(scalar(self.beta2, [1]), t)) + 1.0)
            p.set((p - m_hat * self.lr / (sqrt(v_hat) + self.eps)).eval())  # :171-173
        self.t = (t + 1.0).eval()  # :176


# --------------------------------------------------------------------------- DenseNet, MobileNetV2
class AvgPool2d:  # layers.rs:90-122
    def __init__(self, ker, stride=None, pad=0, dil=1):
        self.a = (ker, ker if stride is None else stride, pad, dil)

    def params(self): return []

    def __call__(self, x): return avg_pool_2d(x, *self.a)


class BottleneckLayer:  # models/densenet.rs:121-157
    def __init__(self, in_planes, out_planes):
        self.body = Sequential(Relu(), Conv2d(in_planes, out_planes * 4, 1, 1, 0, 1), Conv2d(out_planes * 4, out_planes, 3, 1, 1, 1))

    def params(self): return self.body.params()

    def __call__(self, x): return concat([x, self.body(x)], 3)


def densenet(chan_input, num_classes, depth=121, growth_rate=12):  # models/densenet.rs:56-107 (no BatchNorm, no dropout)
    in_planes = 2 * growth_rate
    m = Sequential(Conv2d(chan_input, in_planes, 3, 1, 1, 1))
    n = (depth - 4) // 6
    for i in range(3):
        blk = Sequential()
        for j in range(n):
            blk.add(BottleneckLayer(in_planes + j * growth_rate, growth_rate))
        m.add(blk)
        in_planes += n * growth_rate
        if i < 2:
            m.add(Sequential(Relu(), Conv2d(in_planes, in_planes // 2, 1, 1, 0, 1), AvgPool2d(2)))
            in_planes //= 2
    m.add(Relu()).add(AdaptiveAvgPool2d([1, 1])).add(Flatten()).add(Dense(in_planes, num_classes))
    return m


def _make_divisible(val, div, min_val):  # models/mobilenet.rs:10-18
    v = max(min_val, (val + div // 2) // div * div)
    return v + div if np.float32(v) < np.float32(0.9) * np.float32(val) else v


class InvertedResidual:  # models/mobilenet.rs:96-138 (the 3x3 convolution really has padding 0 and dilation 0, :111)
    def __init__(self, inp, oup, stride, expand_ratio):
        hidden = inp * expand_ratio
        self.body = Sequential()
        if expand_ratio != 1:
            self.body.add(Conv2d(inp, hidden, 1, 1, 0, 1)).add(Relu())
        self.body.add(Conv2d(hidden, hidden, 3, stride, 0, 0)).add(Relu()).add(Conv2d(hidden, oup, 1, 1, 0, 1))
        self.residual = stride == 1 and inp == oup

    def params(self): return self.body.params()

    def __call__(self, x): return x + self.body(x) if self.residual else self.body(x)


def mobilenet_v2(chan_in, num_classes):  # models/mobilenet.rs:38-80, width multiplier 1
    cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
    c_in = _make_divisible(32, 8, 8)
    m = Sequential(Conv2d(chan_in, c_in, 3, 2, 1, 1), Relu())
    for t, c, n, s in cfg:
        c_out = _make_divisible(c, 8, 8)
        for i in range(n):
            m.add(InvertedResidual(c_in, c_out, s if i == 0 else 1, t))
            c_in = c_out
    last = _make_divisible(1280, 8, 8)
    m.add(Conv2d(c_in, last, 1, 1, 0, 1)).add(Relu()).add(AdaptiveAvgPool2d([1, 1])).add(Flatten()).add(Dense(last, num_classes))
    return m


# --------------------------------------------------------------------------- random tensors (ops/rand.rs)
def _xorshift128(seed_x, seed_y):  # rand.rs:40-48 on uint32 arrays; the literal is a double in OpenCL C
    t = seed_x ^ (seed_x << np.uint32(11))
    r = seed_y ^ (seed_y >> np.uint32(19)) ^ (t ^ (t >> np.uint32(8)))
    return (r.astype(np.float64) * 2.3283064e-10).astype(np.float32)


class _Rand:
    def __init__(self, normal, seed_x, seed_y, extents):
        self.normal, self.sx, self.sy, self.extents = normal, np.uint32(seed_x), np.uint32(seed_y), extents

    def compute(self, _):
        n = int(np.prod(self.extents))
        with np.errstate(over="ignore", divide="ignore", invalid="ignore"):
            if not self.normal:  # rand.rs:69-72
                g = np.arange(n, dtype=np.uint32)
                y = _xorshift128(self.sx + g, self.sy + g)
            else:  # rand.rs:108-121; the store past the end of an odd-sized tensor is dropped
                g = np.arange((n + 1) // 2, dtype=np.uint32)
                u1 = _xorshift128(self.sx + g * np.uint32(2), np.full_like(g, self.sy))
                u2 = _xorshift128(self.sx + g * np.uint32(2) + np.uint32(1), np.full_like(g, self.sy))
                r = np.sqrt(np.float32(-2.0) * np.log(u1))
                theta = (2.0 * math.pi * u2.astype(np.float64)).astype(np.float32)
                y = np.stack([r * np.cos(theta), r * np.sin(theta)], axis=1).reshape(-1)[:n].astype(np.float32)
        return Tensor(np.ascontiguousarray(y, dtype=np.float32), Shape(self.extents), FLOAT)

    def grad(self, x, y, gy):
        return []


def uniform(extents, seed_x, seed_y):  # rand.rs:21-28; the reference draws the seeds itself
    e = to_extents(extents, 0)
    return Var(Shape(e), FLOAT, _Rand(False, seed_x, seed_y, e), [])


def normal(extents, seed_x, seed_y):  # rand.rs:30-38
    e = to_extents(extents, 0)
    return Var(Shape(e), FLOAT, _Rand(True, seed_x, seed_y, e), [])
