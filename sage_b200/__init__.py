"""sage_b200 — Python binding of the B200 CUDA backend for sage's hot path.

Everything here is a thin ctypes layer over libsagecuda.so (include/sage_cuda.h and
include/sage_graph.h).  The names mirror the reference's Rust API (src/var.rs, src/ops/,
src/layers.rs, src/models/): ``Var``, ``Context``, ``matmul``, ``softmax``, ``grad`` ...

There is no CPU fallback: importing the package without the built library raises, and every
compute call on a machine without a CUDA device fails with SAGE_ERR_NO_DEVICE.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsagecuda.so")
if not os.path.exists(_LIB_PATH):
    raise ImportError(
        "sage_b200: %s is missing; build it with `python -c 'import __graft_entry__ as g; g.build()'` "
        "or `make -C sage_b200/csrc`.  There is no CPU fallback." % _LIB_PATH)
lib = ctypes.CDLL(_LIB_PATH)

F32, I32, U32 = 0, 1, 2
_NP = {F32: np.float32, I32: np.int32, U32: np.uint32}
_DT = {np.dtype(np.float32): F32, np.dtype(np.int32): I32, np.dtype(np.uint32): U32}
MAX_DIMS = 8
_P = ctypes.c_void_p
_i64p = ctypes.POINTER(ctypes.c_int64)

STATUS = {0: "OK", 1: "INVALID", 2: "OOM", 3: "DEVICE", 4: "COMPILE", 5: "NO_DEVICE", 6: "TIMEOUT", 7: "UNSUPPORTED"}


class SageError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("SAGE_ERR_%s: %s" % (STATUS.get(code, code), msg))
        self.code = code


class CtxOpts(ctypes.Structure):
    _fields_ = [("mem_capacity_bytes", ctypes.c_uint64), ("use_cache", ctypes.c_int32), ("ref_compat", ctypes.c_int32),
                ("pattern_fusion", ctypes.c_int32), ("gemm_backend", ctypes.c_int32)]


class MemStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in ("capacity", "mem_total", "mem_used", "mem_peak", "num_device_allocs")]


class CTensor(ctypes.Structure):
    _fields_ = [("buf", _P), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32), ("extents", ctypes.c_int64 * MAX_DIMS),
                ("strides", ctypes.c_int64 * MAX_DIMS), ("offset", ctypes.c_int64)]


class Window(ctypes.Structure):
    _fields_ = [("ker", ctypes.c_int32 * 2), ("stride", ctypes.c_int32 * 2), ("pad", ctypes.c_int32 * 2), ("dil", ctypes.c_int32 * 2)]


class BertConfigC(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("embed_dim", "num_vocabs", "max_num_tokens", "hidden_dim", "num_layers", "num_heads", "num_classes")] + \
               [("gelu", ctypes.c_int32), ("layer_norm_eps", ctypes.c_float)]


lib.sage_last_error.restype = ctypes.c_char_p
lib.sage_graph_last_error.restype = ctypes.c_char_p
lib.sage_ctx_stream.restype = _P
lib.sage_buf_ptr.restype = _P
lib.sage_buf_size.restype = ctypes.c_size_t


def _arr64(v):
    v = [int(a) for a in v]
    return (ctypes.c_int64 * max(len(v), 1))(*v)


def _pair(v):
    return (int(v), int(v)) if isinstance(v, (int, np.integer)) else (int(v[0]), int(v[1]))


def window(ker=1, stride=1, pad=0, dil=1):
    """Window parameters; every pair is ordered [w, h] like the reference (src/ops/conv.rs:83)."""
    w = Window()
    w.ker[:], w.stride[:], w.pad[:], w.dil[:] = _pair(ker), _pair(stride), _pair(pad), _pair(dil)
    return w


def device_count():
    n = ctypes.c_int32(0)
    lib.sage_device_count(ctypes.byref(n))
    return n.value


def device_name(i=0):
    b = ctypes.create_string_buffer(256)
    if lib.sage_device_name(i, b, 256):
        return None
    return b.value.decode()


# --------------------------------------------------------------------------- Context
class Context:
    """Context::with_device (src/session/context.rs:43-52): device + stream + allocator + evaluated-data
    cache.  device=-1 gives a planning context (compiles and records, computes nothing)."""

    def __init__(self, device=0, **opts):
        o = CtxOpts()
        lib.sage_ctx_opts_default(ctypes.byref(o))
        for k, v in opts.items():
            setattr(o, k, v)
        self.h = _P()
        st = lib.sage_ctx_create(int(device), ctypes.byref(o), ctypes.byref(self.h))
        if st:
            raise SageError(st, "cannot create a context on device %d (no CUDA device?)" % device)
        self.s = _P()
        self._ck(lib.sage_session_create(self.h, ctypes.byref(self.s)))
        self.device = device

    def _ck(self, st):
        if st:
            msg = lib.sage_last_error(self.h).decode() or lib.sage_graph_last_error().decode()
            raise SageError(st, msg)

    def close(self):
        if getattr(self, "s", None):
            lib.sage_session_destroy(self.s)
            self.s = None
        if getattr(self, "h", None):
            lib.sage_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- data
    def var(self, array, dtype=None):
        """Var::new(Tensor::new(array).to_device(ctx))."""
        a = np.asarray(array)
        if dtype is None:
            dtype = F32 if a.dtype.kind == "f" else (U32 if a.dtype.kind == "u" else I32)
        a = np.ascontiguousarray(a, dtype=_NP[dtype])
        ext = a.shape if a.ndim else (1,)
        out = _P()
        self._ck(lib.sage_var_from_host(self.s, dtype, len(ext), _arr64(ext), _P(a.ctypes.data), ctypes.byref(out)))
        return Var(out)

    def set(self, v, array, pinned_ptr=None):
        """Var::set with an upload.  With pinned_ptr the copy is asynchronous from that pinned address."""
        if pinned_ptr is not None:
            self._ck(lib.sage_var_set(self.s, v.h, _P(pinned_ptr), 1))
            return
        a = np.ascontiguousarray(array, dtype=_NP[v.dtype])
        assert tuple(a.shape) == tuple(v.extents) or a.size == v.size
        self._ck(lib.sage_var_set(self.s, v.h, _P(a.ctypes.data), 0))

    def eval(self, *targets):
        """Context::eval (src/session/context.rs:96-117)."""
        arr = (_P * len(targets))(*[t.h for t in targets])
        self._ck(lib.sage_eval(self.s, arr, len(targets)))

    def read(self, v):
        """tensor.to_host(): contiguous numpy copy of an evaluated (or data) variable."""
        out = np.empty(v.extents, dtype=_NP[v.dtype])
        self._ck(lib.sage_var_read(self.s, v.h, _P(out.ctypes.data), ctypes.c_size_t(out.nbytes)))
        return out

    def read_into(self, v, ptr, nbytes):
        self._ck(lib.sage_var_read(self.s, v.h, _P(ptr), ctypes.c_size_t(nbytes)))

    def clear(self):
        lib.sage_session_clear(self.s)

    def sync(self):
        self._ck(lib.sage_sync(self.h))

    def describe(self):
        n = ctypes.c_size_t(0)
        lib.sage_session_describe(self.s, None, 0, ctypes.byref(n))
        b = ctypes.create_string_buffer(n.value + 1)
        lib.sage_session_describe(self.s, b, ctypes.c_size_t(n.value + 1), None)
        return b.value.decode()

    def programs_compiled(self):
        n = ctypes.c_uint64(0)
        lib.sage_session_stats(self.s, ctypes.byref(n))
        return n.value

    def programs_cached(self):
        """(programs held by the session's cache, the cache's limit)."""
        n, lim = ctypes.c_uint64(0), ctypes.c_uint64(0)
        lib.sage_session_programs_cached(self.s, ctypes.byref(n), ctypes.byref(lim))
        return n.value, lim.value

    def drop_programs(self):
        lib.sage_session_drop_programs(self.s)

    def mem_stats(self):
        m = MemStats()
        self._ck(lib.sage_mem_stats(self.h, ctypes.byref(m)))
        return {k: getattr(m, k) for k, _ in MemStats._fields_}

    def launch_count(self):
        k, m = ctypes.c_uint64(0), ctypes.c_uint64(0)
        lib.sage_launch_count(self.h, ctypes.byref(k), ctypes.byref(m))
        return k.value, m.value

    def trace_begin(self):
        lib.sage_trace_begin(self.h)

    def trace(self):
        n = ctypes.c_size_t(0)
        lib.sage_trace_get(self.h, None, 0, ctypes.byref(n))
        b = ctypes.create_string_buffer(n.value + 1)
        lib.sage_trace_get(self.h, b, ctypes.c_size_t(n.value + 1), None)
        return [l for l in b.value.decode().split("\n") if l]

    def timer_start(self):
        self._ck(lib.sage_timer_start(self.h))

    def timer_stop(self):
        """Device milliseconds between timer_start() and now, on the context's stream (waits)."""
        ms = ctypes.c_float(0)
        self._ck(lib.sage_timer_stop(self.h, ctypes.byref(ms)))
        return ms.value

    def pinned(self, shape, dtype):
        """A numpy array over pinned host memory (for asynchronous uploads / downloads)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = _P()
        st = lib.sage_host_alloc(ctypes.c_size_t(max(n, 4)), ctypes.byref(p))
        if st:
            raise SageError(st, "pinned host allocation failed")
        buf = (ctypes.c_char * max(n, 4)).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        self._pinned = getattr(self, "_pinned", []) + [(p, buf)]
        return arr

    def profile_begin(self):
        lib.sage_profile_begin(self.h)

    def profile_end(self):
        """Returns {kernel name: (launches, total_ms)} of device time since profile_begin()."""
        n = ctypes.c_size_t(0)
        lib.sage_profile_end(self.h, None, ctypes.c_size_t(0), ctypes.byref(n))
        b = ctypes.create_string_buffer(n.value + 1)
        lib.sage_profile_end(self.h, b, ctypes.c_size_t(n.value + 1), None)
        out = {}
        for line in b.value.decode().split("\n"):
            parts = line.split()
            if len(parts) == 3:
                out[parts[0]] = (int(parts[1]), float(parts[2]))
        return out

    def status_word(self):
        w = ctypes.c_uint32(0)
        self._ck(lib.sage_status_word(self.h, ctypes.byref(w)))
        return w.value

    @property
    def stream(self):
        return lib.sage_ctx_stream(self.h)

    # --- raw buffers + op-level entry points (the device boundary of sage_cuda.h)
    def alloc(self, nbytes):
        b = _P()
        self._ck(lib.sage_alloc(self.h, ctypes.c_size_t(nbytes), ctypes.byref(b)))
        return b

    def free(self, buf):
        self._ck(lib.sage_free(self.h, buf))

    def upload(self, buf, array, offset=0):
        a = np.ascontiguousarray(array)
        self._ck(lib.sage_upload(self.h, buf, ctypes.c_size_t(offset), _P(a.ctypes.data), ctypes.c_size_t(a.nbytes)))

    def download(self, buf, shape, dtype, offset=0):
        out = np.empty(shape, dtype=dtype)
        self._ck(lib.sage_download(self.h, buf, ctypes.c_size_t(offset), _P(out.ctypes.data), ctypes.c_size_t(out.nbytes)))
        return out

    def tensor(self, array):
        """Uploads a numpy array into a fresh buffer and returns a DeviceTensor (contiguous)."""
        a = np.ascontiguousarray(array)
        if a.dtype not in _DT:
            a = a.astype(np.float32)
        buf = self.alloc(max(a.nbytes, 4))
        if a.nbytes:
            self.upload(buf, a)
        return DeviceTensor(self, buf, _DT[a.dtype], a.shape if a.ndim else (1,))

    def empty(self, shape, dtype=F32):
        n = int(np.prod(shape)) if len(shape) else 1
        return DeviceTensor(self, self.alloc(max(n * 4, 4)), dtype, tuple(shape))


class DeviceTensor:
    """A buffer + Shape, the reference's Tensor (src/tensor.rs:106-110), for op-level C-ABI calls."""

    def __init__(self, ctx, buf, dtype, extents, strides=None, offset=0, owner=True):
        self.ctx, self.buf, self.dtype, self.extents, self.offset, self.owner = ctx, buf, dtype, tuple(int(e) for e in extents), offset, owner
        if strides is None:
            strides, p = [], 1
            for e in reversed(self.extents):
                strides.insert(0, p)
                p *= e
        self.strides = tuple(int(s) for s in strides)

    def c(self):
        t = CTensor()
        t.buf, t.dtype, t.ndim, t.offset = self.buf, self.dtype, len(self.extents), self.offset
        for i, (e, s) in enumerate(zip(self.extents, self.strides)):
            t.extents[i], t.strides[i] = e, s
        return t

    def view(self, extents, strides, offset=0):
        return DeviceTensor(self.ctx, self.buf, self.dtype, extents, strides, offset, owner=False)

    def numpy(self):
        n = lib.sage_buf_size(self.buf)
        raw = self.ctx.download(self.buf, (n // 4,), _NP[self.dtype])
        base = raw[self.offset:]
        return np.ascontiguousarray(np.lib.stride_tricks.as_strided(base, shape=self.extents, strides=[s * 4 for s in self.strides]))

    def release(self):
        if self.owner and self.buf:
            self.ctx.free(self.buf)
            self.buf = None


# --------------------------------------------------------------------------- Var
_UN = ["copy", "abs", "neg", "recip", "log", "exp", "sqrt", "square", "erf", "sign", "ceil", "floor", "round", "sin", "sinh",
       "cos", "cosh", "tan", "tanh", "asin", "asinh", "acos", "acosh", "atan", "atanh", "not_", "int", "float"]
_BIN = ["add", "sub", "div", "mul", "modular", "pow", "minimum", "maximum", "and_", "or_", "eq", "ne", "gt", "ge", "lt", "le"]
SUM, PROD, MAX, MIN = 0, 1, 2, 3


def _gck(st):
    if st:
        raise SageError(st, lib.sage_graph_last_error().decode())


def _axes(axes, rank):
    if axes is None:
        return list(range(rank))
    if isinstance(axes, (int, np.integer)):
        return [int(axes)]
    return [int(a) for a in axes]


class Var:
    """Lazy variable (src/var.rs:34-42).  Methods mirror the reference's `impl Var` (var.rs:381-683)."""

    def __init__(self, handle):
        self.h = handle
        dt, nd, off, isop, to = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int32(), ctypes.c_uint64()
        ext, stri = (ctypes.c_int64 * MAX_DIMS)(), (ctypes.c_int64 * MAX_DIMS)()
        lib.sage_var_info(self.h, ctypes.byref(dt), ctypes.byref(nd), ext, stri, ctypes.byref(off), ctypes.byref(isop), ctypes.byref(to))
        self.dtype, self.extents, self.strides = dt.value, tuple(ext[: nd.value]), tuple(stri[: nd.value])
        self.offset, self.is_op, self.t_order = off.value, bool(isop.value), to.value

    def __del__(self):
        try:
            if self.h:
                lib.sage_var_free(self.h)
        except Exception:
            pass

    @property
    def size(self):
        return int(np.prod(self.extents)) if self.extents else 1

    def rank(self):
        return len(self.extents)

    def extent(self, axis):
        return self.extents[axis]

    @staticmethod
    def empty(extents, dtype=F32):
        out = _P()
        extents = [extents] if isinstance(extents, (int, np.integer)) else list(extents)
        _gck(lib.sage_var_empty(dtype, len(extents), _arr64(extents), ctypes.byref(out)))
        return Var(out)

    @staticmethod
    def host(array, dtype=None):
        """Var::new(host tensor): uploaded on first use."""
        a = np.asarray(array)
        if dtype is None:
            dtype = F32 if a.dtype.kind == "f" else (U32 if a.dtype.kind == "u" else I32)
        a = np.ascontiguousarray(a, dtype=_NP[dtype])
        ext = a.shape if a.ndim else (1,)
        out = _P()
        _gck(lib.sage_var_from_host_lazy(dtype, len(ext), _arr64(ext), _P(a.ctypes.data), ctypes.byref(out)))
        return Var(out)

    def eval(self, ctx):
        """Var::eval (var.rs:338-352); returns the value as a numpy array."""
        if self.is_op:
            ctx.eval(self)
        return ctx.read(self)

    def grad(self, y):
        """x.grad(y) = d y / d x (var.rs:326-335)."""
        return grad(y, [self])[0]

    # arithmetic (src/ops/map.rs:1180-1370)
    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return sub(self, o)
    def __rsub__(self, o): return sub(o, self)
    def __mul__(self, o): return mul(self, o)
    def __rmul__(self, o): return mul(o, self)
    def __truediv__(self, o): return div(self, o)
    def __rtruediv__(self, o): return div(o, self)
    def __neg__(self): return neg(self)

    def organize(self): return _mk(lib.sage_op_copy_organize, self.h)
    def view(self, extents): return view(self, extents)
    def expand(self, extents): return expand(self, extents)
    def permute(self, axes): return permute(self, axes)
    def transpose(self, a1, a2): return transpose(self, a1, a2)
    def tr(self): return transpose(self, 0, 1)
    def squeeze(self, axis): return squeeze(self, axis)
    def unsqueeze(self, axis): return unsqueeze(self, axis)
    def index(self, axis, i): return slice_(self, axis, i, i + 1)
    def slice(self, axis, start, end): return slice_(self, axis, start, end)
    def gather(self, idx, axis): return gather(self, idx, axis)
    def scatter(self, idx, axis, extents): return scatter(self, idx, axis, extents)
    def matmul(self, o): return matmul(self, o)
    def matmul_batched(self, o): return matmul_batched(self, o)
    def sum(self, axes=None, preserve=False): return reduce(self, axes, preserve, SUM)
    def prod(self, axes=None, preserve=False): return reduce(self, axes, preserve, PROD)
    def max(self, axes=None, preserve=False): return reduce(self, axes, preserve, MAX)
    def min(self, axes=None, preserve=False): return reduce(self, axes, preserve, MIN)
    def mean(self, axes=None, preserve=False): return mean(self, axes, preserve)
    def var(self, axes=None, preserve=False): return var(self, axes, preserve)
    def argmax(self, axis, preserve=False): return argmax(self, axis, preserve)
    def argmin(self, axis, preserve=False): return argmin(self, axis, preserve)


def _mk(fn, *args):
    out = _P()
    _gck(fn(*args, ctypes.byref(out)))
    return Var(out)


def scalar(value, extents=(1,)):
    """scalar (map.rs:517-531)."""
    extents = [extents] if isinstance(extents, (int, np.integer)) else list(extents)
    if isinstance(value, (float, np.floating)):
        return _mk(lib.sage_op_scalar_f32, ctypes.c_float(value), len(extents), _arr64(extents))
    return _mk(lib.sage_op_scalar_i32, ctypes.c_int32(int(value)), len(extents), _arr64(extents))


def into_var(v):
    """Variable::into_var (var.rs:817-861): scalars become [1] literals."""
    if isinstance(v, Var):
        return v
    if isinstance(v, (int, float, np.integer, np.floating)):
        return scalar(v, [1])
    raise TypeError("upload arrays with Context.var() first")


def unary_map(x, kind):
    x = into_var(x)  # keep the (possibly temporary) Var alive across the call
    return _mk(lib.sage_op_unary, kind, x.h)


def binary_map(a, b, kind):
    a, b = into_var(a), into_var(b)
    return _mk(lib.sage_op_binary, kind, a.h, b.h)


_BUILTIN_NAMES = {"abs", "round", "int", "float", "pow"}  # module-level functions get a trailing underscore


def _def_unary(i, name):
    def f(x):
        return unary_map(x, i)
    fn_name = name + "_" if name in _BUILTIN_NAMES else name
    f.__name__ = fn_name
    globals()[fn_name] = f
    if not hasattr(Var, name):
        setattr(Var, name, lambda self, _i=i: unary_map(self, _i))


def _def_binary(i, name):
    def f(a, b):
        return binary_map(a, b, i)
    fn_name = name + "_" if name in _BUILTIN_NAMES else name
    f.__name__ = fn_name
    globals()[fn_name] = f
    if not hasattr(Var, name):
        setattr(Var, name, lambda self, o, _i=i: binary_map(self, o, _i))


for _i, _n in enumerate(_UN):
    _def_unary(_i, _n)
for _i, _n in enumerate(_BIN):
    _def_binary(_i, _n)


def cond(c, a, b):
    c, a, b = into_var(c), into_var(a), into_var(b)
    return _mk(lib.sage_op_cond, c.h, a.h, b.h)
def view(x, extents):
    extents = [extents] if isinstance(extents, (int, np.integer)) else list(extents)
    return _mk(lib.sage_op_view, x.h, len(extents), _arr64(extents))
def expand(x, extents): return _mk(lib.sage_op_expand, x.h, len(extents), _arr64(extents))
def permute(x, axes): return _mk(lib.sage_op_permute, x.h, len(axes), _arr64(axes))
def transpose(x, a1, a2): return _mk(lib.sage_op_transpose, x.h, ctypes.c_int64(a1), ctypes.c_int64(a2))
def tr(x): return transpose(x, 0, 1)
def squeeze(x, axis): return _mk(lib.sage_op_squeeze, x.h, ctypes.c_int64(axis))
def unsqueeze(x, axis): return _mk(lib.sage_op_unsqueeze, x.h, ctypes.c_int64(axis))
def slice_(x, axis, start, end): return _mk(lib.sage_op_slice, x.h, ctypes.c_int64(axis), ctypes.c_int64(start), ctypes.c_int64(end))
def unslice(x, axis, start, end): return _mk(lib.sage_op_unslice, x.h, ctypes.c_int64(axis), ctypes.c_int64(start), ctypes.c_int64(end))
def gather(x, ind, axis): return _mk(lib.sage_op_gather, x.h, ind.h, ctypes.c_int64(axis))
def scatter(x, ind, axis, extents): return _mk(lib.sage_op_scatter, x.h, ind.h, ctypes.c_int64(axis), len(extents), _arr64(extents))
def concat(xs, axis):
    arr = (_P * len(xs))(*[v.h for v in xs])
    return _mk(lib.sage_op_concat, arr, len(xs), ctypes.c_int64(axis))
def reduce(x, axes, preserve, kind):
    ax = _axes(axes, x.rank())
    return _mk(lib.sage_op_reduce, kind, x.h, len(ax), _arr64(ax), int(bool(preserve)))
def sum_(x, axes=None, preserve=False): return reduce(x, axes, preserve, SUM)
def prod(x, axes=None, preserve=False): return reduce(x, axes, preserve, PROD)
def max_(x, axes=None, preserve=False): return reduce(x, axes, preserve, MAX)
def min_(x, axes=None, preserve=False): return reduce(x, axes, preserve, MIN)
def mean(x, axes=None, preserve=False):
    ax = _axes(axes, x.rank())
    return _mk(lib.sage_op_mean, x.h, len(ax), _arr64(ax), int(bool(preserve)))
def var(x, axes=None, preserve=False):
    ax = _axes(axes, x.rank())
    return _mk(lib.sage_op_var, x.h, len(ax), _arr64(ax), int(bool(preserve)))
def argmax(x, axis, preserve=False): return _mk(lib.sage_op_reduce_arg, 1, x.h, ctypes.c_int64(axis), int(bool(preserve)))
def argmin(x, axis, preserve=False): return _mk(lib.sage_op_reduce_arg, 0, x.h, ctypes.c_int64(axis), int(bool(preserve)))
def gemm(a, b, ta=False, tb=False): return _mk(lib.sage_op_gemm, a.h, b.h, int(ta), int(tb))
def gemm_batched(a, b, ta=False, tb=False): return _mk(lib.sage_op_gemm_batched, a.h, b.h, int(ta), int(tb))
def matmul(a, b): return _mk(lib.sage_op_matmul, a.h, b.h)
def matmul_batched(a, b): return _mk(lib.sage_op_matmul_batched, a.h, b.h)
def im2col(x, ker, stride, pad, dil): return _mk(lib.sage_op_im2col, x.h, ctypes.byref(window(ker, stride, pad, dil)))
def col2im(x, img_size, ker, stride, pad, dil):
    return _mk(lib.sage_op_col2im, x.h, ctypes.c_int64(img_size[0]), ctypes.c_int64(img_size[1]), ctypes.byref(window(ker, stride, pad, dil)))
def conv_2d(x, filt, stride, pad, dil): return _mk(lib.sage_op_conv_2d, x.h, filt.h, ctypes.byref(window(1, stride, pad, dil)))
def max_pool_2d(x, ker, stride, pad, dil): return _mk(lib.sage_op_pool_2d, 1, x.h, ctypes.byref(window(ker, stride, pad, dil)))
def avg_pool_2d(x, ker, stride, pad, dil): return _mk(lib.sage_op_pool_2d, 0, x.h, ctypes.byref(window(ker, stride, pad, dil)))
def batch_norm_2d(x, gamma, beta, mean_, var_, eps):
    return _mk(lib.sage_op_batch_norm_2d, x.h, gamma.h, beta.h, mean_.h, var_.h, ctypes.c_float(eps))
def relu(x): return _mk(lib.sage_op_relu, x.h)
def softmax(x, axes):
    ax = _axes(axes, x.rank())
    return _mk(lib.sage_op_softmax, x.h, len(ax), _arr64(ax))
def log_sum_exp(x, axes):
    ax = _axes(axes, x.rank())
    return _mk(lib.sage_op_log_sum_exp, x.h, len(ax), _arr64(ax))
def softmax_cross_entropy(x, labels): return _mk(lib.sage_op_softmax_cross_entropy, x.h, labels.h)
def layer_norm(x, axes, gamma, beta, eps):
    ax = _axes(axes, x.rank())
    return _mk(lib.sage_op_layer_norm, x.h, len(ax), _arr64(ax), gamma.h, beta.h, ctypes.c_float(eps))


def grad(y, xs):
    """grad(y, xs) (var.rs:56-103)."""
    arr = (_P * len(xs))(*[v.h for v in xs])
    out = (_P * len(xs))()
    _gck(lib.sage_grad(y.h, arr, len(xs), out))
    return [Var(_P(h)) for h in out]


def grad_param(y, model):
    """grad_param(y, model) (var.rs:46-54): {parameter: gradient}, in Parameter::params order."""
    params = model.params()
    return dict(zip(params, grad(y, params)))


def uniform(extents, seed_x, seed_y):
    """ops::rand::uniform (src/ops/rand.rs:21-28, 50-90) with explicit seeds: values in [0, 1]."""
    return _mk(lib.sage_op_uniform, len(extents), _arr64(extents), ctypes.c_uint32(seed_x), ctypes.c_uint32(seed_y))


def normal(extents, seed_x, seed_y):
    """ops::rand::normal (src/ops/rand.rs:30-38, 92-140) with explicit seeds: Box-Muller pairs."""
    return _mk(lib.sage_op_normal, len(extents), _arr64(extents), ctypes.c_uint32(seed_x), ctypes.c_uint32(seed_y))


def accuracy(logits, labels):
    """ops::metric::accuracy (src/ops/metric.rs:4-17)."""
    return _mk(lib.sage_op_accuracy, logits.h, labels.h)


# --------------------------------------------------------------------------- optimizers (src/optim.rs)
class Optimizer:
    """trait Optimizer (optim.rs:8-12).  `update` takes the {parameter: gradient} map of grad_param."""

    def __init__(self, handle):
        self.h = handle

    def __del__(self):
        try:
            lib.sage_optimizer_destroy(self.h)
        except Exception:
            pass

    def init(self, ctx):
        ctx._ck(lib.sage_optimizer_init(self.h, ctx.s))

    def update(self, grads, ctx):
        params = list(grads.keys())
        p = (_P * len(params))(*[v.h for v in params])
        g = (_P * len(params))(*[grads[v].h for v in params])
        ctx._ck(lib.sage_optimizer_update(self.h, ctx.s, p, g, len(params)))

    def set_weight_decay(self, weight_decay):
        lib.sage_optimizer_set_weight_decay(self.h, ctypes.c_float(weight_decay))


class Sgd(Optimizer):
    """Sgd::new(lr) (optim.rs:28-40): param -= lr * grad."""

    def __init__(self, lr):
        h = _P()
        _gck(lib.sage_sgd_create(ctypes.c_float(lr), ctypes.byref(h)))
        super().__init__(h)


class Adam(Optimizer):
    """Adam::new(lr) (optim.rs:112-125): beta1 0.9, beta2 0.999, eps 1e-08; the first update of a
    parameter only stores zero moments (optim.rs:147-159)."""

    def __init__(self, lr):
        h = _P()
        _gck(lib.sage_adam_create(ctypes.c_float(lr), ctypes.byref(h)))
        super().__init__(h)


# --------------------------------------------------------------------------- models
class Bert:
    """models::Bert (src/models/bert.rs:57-139).  Defaults are BertConfig::base()."""

    def __init__(self, **cfg):
        c = BertConfigC()
        lib.sage_bert_config_base(ctypes.byref(c))
        for k, v in cfg.items():
            setattr(c, k, v)
        self.config = c
        self.h = _P()
        _gck(lib.sage_bert_create(ctypes.byref(c), ctypes.byref(self.h)))

    def __del__(self):
        try:
            lib.sage_bert_destroy(self.h)
        except Exception:
            pass

    def params(self):
        n = ctypes.c_int32(0)
        lib.sage_bert_params(self.h, None, 0, ctypes.byref(n))
        out = (_P * n.value)()
        lib.sage_bert_params(self.h, out, n.value, ctypes.byref(n))
        return [Var(_P(h)) for h in out]

    def pass_(self, token_ids, attn_mask):
        return _mk(lib.sage_bert_pass, self.h, token_ids.h, attn_mask.h)


class _SequentialModel:
    """A model that is a Sequential in the reference (src/layers.rs:275-325): parameters in traversal order, pass."""

    def __del__(self):
        try:
            lib.sage_model_destroy(self.h)
        except Exception:
            pass

    def params(self):
        n = ctypes.c_int32(0)
        lib.sage_model_params(self.h, None, 0, ctypes.byref(n))
        out = (_P * n.value)()
        lib.sage_model_params(self.h, out, n.value, ctypes.byref(n))
        return [Var(_P(h)) for h in out]

    def pass_(self, x):
        return _mk(lib.sage_model_pass, self.h, x.h)


class DenseNet(_SequentialModel):
    """DenseNet::new(DenseNetConfig::d121 / d169 / d201) (src/models/densenet.rs:20-107): depth 121 / 169 / 201 with
    growth rate 12 / 24 / 12."""

    def __init__(self, chan_input, num_classes, depth=121, growth_rate=12):
        self.h = _P()
        _gck(lib.sage_densenet_create(ctypes.c_int64(chan_input), ctypes.c_int64(num_classes), ctypes.c_int64(depth),
                                      ctypes.c_int64(growth_rate), ctypes.byref(self.h)))


class MobileNetV2(_SequentialModel):
    """MobileNetV2::new(MobileNetV2Config::new(chan_in, num_classes)) (src/models/mobilenet.rs:27-80)."""

    def __init__(self, chan_in, num_classes):
        self.h = _P()
        _gck(lib.sage_mobilenet_v2_create(ctypes.c_int64(chan_in), ctypes.c_int64(num_classes), ctypes.byref(self.h)))


class ResNet18:
    """ResNet::new(ResNetConfig::d18(chan_input, num_classes)) (src/models/resnet.rs:74-104)."""

    def __init__(self, chan_input, num_classes, batch_norm=False):
        """batch_norm=True puts back the BatchNorm2d layers (src/layers.rs:479-546) that the reference has
        commented out at resnet.rs:80,167,170; their running statistics are `buffers()`."""
        self.h = _P()
        create = lib.sage_resnet18_bn_create if batch_norm else lib.sage_resnet18_create
        _gck(create(ctypes.c_int64(chan_input), ctypes.c_int64(num_classes), ctypes.byref(self.h)))

    def buffers(self):
        n = ctypes.c_int32(0)
        lib.sage_model_buffers(self.h, None, 0, ctypes.byref(n))
        out = (_P * max(n.value, 1))()
        lib.sage_model_buffers(self.h, out, n.value, ctypes.byref(n))
        return [Var(_P(out[i])) for i in range(n.value)]

    def __del__(self):
        try:
            lib.sage_model_destroy(self.h)
        except Exception:
            pass

    def params(self):
        n = ctypes.c_int32(0)
        lib.sage_model_params(self.h, None, 0, ctypes.byref(n))
        out = (_P * n.value)()
        lib.sage_model_params(self.h, out, n.value, ctypes.byref(n))
        return [Var(_P(h)) for h in out]

    def pass_(self, x):
        return _mk(lib.sage_model_pass, self.h, x.h)
