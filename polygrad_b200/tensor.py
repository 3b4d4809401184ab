"""A small lazy tensor over the polygrad C frontend, bound to one library and
one device.

It mirrors the part of polygrad's Python ``Tensor`` (``py/polygrad/tensor.py``)
that the execution path is exercised with -- elementwise ops, reductions,
softmax, layernorm, movement ops, ``dot`` -- with the same method names and
argument meaning, so that a test written against it reads like polygrad's own.
Graph construction is entirely polygrad's (``poly_alu2``, ``poly_dot``, ...);
this file only tracks shapes, owns host/device storage, and calls
``poly_realize`` with bindings in the chosen memory domain
(polygrad ``src/frontend.c:2262``; device bindings as in
``test/test_cuda.c:409-426``).
"""
import ctypes
import numpy as np

from . import ffi

_NP = {'float32': np.float32, 'int32': np.int32, 'float64': np.float64, 'bool': np.bool_,
       'int64': np.int64, 'uint32': np.uint32, 'uint8': np.uint8}


def _i64(vals):
    arr = (ctypes.c_int64 * max(len(vals), 1))(*[int(v) for v in vals])
    return arr


class Device:
    """Execution target: a library plus a polygrad device id."""

    def __init__(self, lib, device_id):
        self.lib = lib
        self.device_id = device_id
        self.ctx = lib.poly_ctx_new()
        self._keep = []

    @property
    def is_cuda(self):
        return self.device_id == ffi.DEVICE_CUDA

    def tensor(self, array, dtype=None):
        a = np.ascontiguousarray(array)
        if dtype == 'bfloat16':
            return Tensor._leaf_bf16(self, a)
        if a.dtype == np.float64 and dtype is None:
            a = a.astype(np.float32)
        return Tensor._leaf(self, a)

    def close(self):
        if self.ctx:
            self.lib.poly_ctx_destroy(self.ctx)
            self.ctx = None


def f32_to_bf16_bits(a):
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


class Tensor:
    def __init__(self, dev, uop, shape, dtype, leaves):
        self.dev, self.uop, self.shape, self.dtype = dev, uop, tuple(int(s) for s in shape), dtype
        self.leaves = leaves  # list of (buffer_uop, host ndarray)

    # ---- construction ----
    @staticmethod
    def _leaf(dev, a):
        dt = str(a.dtype)
        if dt not in ffi.DTYPE_IDS:
            raise TypeError(f'unsupported dtype {dt}')
        buf = dev.lib.poly_buffer_by_id(dev.ctx, a.size, ffi.DTYPE_IDS[dt])
        flat = a.reshape(-1).copy()
        uop = buf
        if a.ndim != 1:
            uop = dev.lib.poly_reshape(dev.ctx, buf, _i64(a.shape), a.ndim)
        return Tensor(dev, uop, a.shape, dt, [(buf, flat)])

    @staticmethod
    def _leaf_bf16(dev, a):
        bits = f32_to_bf16_bits(a.astype(np.float32)).reshape(-1)
        buf = dev.lib.poly_buffer_by_id(dev.ctx, a.size, ffi.DTYPE_IDS['bfloat16'])
        uop = buf
        if a.ndim != 1:
            uop = dev.lib.poly_reshape(dev.ctx, buf, _i64(a.shape), a.ndim)
        return Tensor(dev, uop, a.shape, 'bfloat16', [(buf, bits)])

    def _new(self, uop, shape, others=(), dtype=None):
        leaves = list(self.leaves)
        for o in others:
            for l in o.leaves:
                if not any(l[0] == m[0] for m in leaves):
                    leaves.append(l)
        return Tensor(self.dev, uop, shape, dtype or self.dtype, leaves)

    def _const(self, v):
        return self.dev.lib.poly_const_float(self.dev.ctx, float(v))

    # ---- elementwise ----
    def _binary(self, op, other, reverse=False):
        lib, ctx = self.dev.lib, self.dev.ctx
        if isinstance(other, Tensor):
            a, b = self, other
            if a.shape != b.shape:
                shape = np.broadcast_shapes(a.shape, b.shape)
                a, b = a._broadcast_to(shape), b._broadcast_to(shape)
            ua, ub = (b.uop, a.uop) if reverse else (a.uop, b.uop)
            return a._new(lib.poly_alu2(ctx, lib.ops[op], ua, ub), a.shape, [b])
        c = self._const(other)
        ua, ub = (c, self.uop) if reverse else (self.uop, c)
        return self._new(lib.poly_alu2(ctx, lib.ops[op], ua, ub), self.shape)

    def _broadcast_to(self, shape):
        shape = tuple(shape)
        if self.shape == shape:
            return self
        pad = (1,) * (len(shape) - len(self.shape)) + self.shape
        t = self.reshape(*pad) if pad != self.shape else self
        return t.expand(*shape)

    def __add__(self, o): return self._binary('ADD', o)
    def __radd__(self, o): return self._binary('ADD', o, True)
    def __mul__(self, o): return self._binary('MUL', o)
    def __rmul__(self, o): return self._binary('MUL', o, True)
    def __sub__(self, o): return self._binary('SUB', o)
    def __rsub__(self, o): return self._binary('SUB', o, True)
    def __truediv__(self, o): return self._binary('FDIV', o)
    def __neg__(self):
        lib = self.dev.lib
        return self._new(lib.poly_alu1(self.dev.ctx, lib.ops['NEG'], self.uop), self.shape)

    def eq(self, other):
        """Elementwise equality (a bool tensor), as polygrad's poly_eq."""
        a, b = self, other
        if a.shape != b.shape:
            shape = np.broadcast_shapes(a.shape, b.shape)
            a, b = a._broadcast_to(shape), b._broadcast_to(shape)
        return a._new(self.dev.lib.poly_eq(self.dev.ctx, a.uop, b.uop), a.shape, [b], dtype='bool')

    def where(self, a, b):
        """self ? a : b with a a tensor of self's shape and b a scalar."""
        lib, ctx = self.dev.lib, self.dev.ctx
        return a._new(lib.poly_where_op(ctx, self.uop, a.uop, a._const(b)), a.shape, [self], dtype=a.dtype)

    def _unary(self, fn):
        return self._new(getattr(self.dev.lib, fn)(self.dev.ctx, self.uop), self.shape)

    def exp(self): return self._unary('poly_exp')
    def log(self): return self._unary('poly_log')
    def sin(self): return self._unary('poly_sin')
    def tanh(self): return self._unary('poly_tanh_act')
    def sigmoid(self): return self._unary('poly_sigmoid')
    def relu(self): return self._unary('poly_relu')
    def gelu(self): return self._unary('poly_gelu')
    def sqrt(self):
        lib = self.dev.lib
        return self._new(lib.poly_alu1(self.dev.ctx, lib.ops['SQRT'], self.uop), self.shape)

    def cast(self, dtype):
        return self._new(self.dev.lib.poly_cast_by_id(self.dev.ctx, self.uop, ffi.DTYPE_IDS[dtype]),
                         self.shape, dtype=dtype)

    # ---- movement ----
    def reshape(self, *shape):
        shape = tuple(int(s) for s in shape)
        return self._new(self.dev.lib.poly_reshape(self.dev.ctx, self.uop, _i64(shape), len(shape)), shape)

    def expand(self, *shape):
        return self._new(self.dev.lib.poly_expand(self.dev.ctx, self.uop, _i64(shape), len(shape)), shape)

    def permute(self, *perm):
        shape = tuple(self.shape[p] for p in perm)
        return self._new(self.dev.lib.poly_permute(self.dev.ctx, self.uop, _i64(perm), len(perm)), shape)

    def _pairs(self, pairs):
        flat = []
        for a, b in pairs:
            flat += [a, b]
        return _i64(flat)

    def shrink(self, pairs):
        shape = tuple(b - a for a, b in pairs)
        return self._new(self.dev.lib.poly_shrink(self.dev.ctx, self.uop, self._pairs(pairs), len(pairs)), shape)

    def pad(self, pairs):
        shape = tuple(s + a + b for s, (a, b) in zip(self.shape, pairs))
        return self._new(self.dev.lib.poly_pad(self.dev.ctx, self.uop, self._pairs(pairs), len(pairs)), shape)

    def flip(self, *axes):
        axes = [a % len(self.shape) for a in axes]
        return self._new(self.dev.lib.poly_flip(self.dev.ctx, self.uop, _i64(axes), len(axes)), self.shape)

    def __getitem__(self, idx):
        """Slices with any step; lowered as polygrad's Tensor does it
        (py/polygrad/tensor.py:1305-1348): shrink, flip for negative steps, and
        pad + reshape + shrink + reshape for |step| > 1."""
        if not isinstance(idx, tuple):
            idx = (idx,)
        res, dim = self, 0
        for i in idx:
            if not isinstance(i, slice):
                raise IndexError('only slices are supported')
            size = res.shape[dim]
            start, stop, step = i.indices(size)
            bound = [start, stop]
            if step * (bound[1] - bound[0]) < 0:
                bound = [0, 0]
            elif step < 0:
                bound = [bound[1] + 1, bound[0] + 1]
            res = res.shrink(tuple(tuple(bound) if d == dim else (0, s) for d, s in enumerate(res.shape)))
            if step < 0:
                res = res.flip(dim)
            st = abs(step)
            if st != 1:
                sh = list(res.shape)
                rem = sh[dim] % st
                if rem:
                    res = res.pad(tuple((0, st - rem) if d == dim else (0, 0) for d in range(len(sh))))
                    sh[dim] += st - rem
                res = res.reshape(*(sh[:dim] + [sh[dim] // st, st] + sh[dim + 1:]))
                res = res.shrink(tuple((0, 1) if d == dim + 1 else (0, s) for d, s in enumerate(res.shape)))
                fs = list(res.shape)
                res = res.reshape(*(fs[:dim] + [fs[dim]] + fs[dim + 2:]))
            dim += 1
        return res

    # ---- reductions ----
    def _reduce(self, fn, axis, keepdim, *extra):
        axis = axis % len(self.shape)
        out_shape = (ctypes.c_int64 * 16)()
        out_ndim = ctypes.c_int(0)
        uop = getattr(self.dev.lib, fn)(self.dev.ctx, self.uop, _i64(self.shape), len(self.shape),
                                        axis, int(keepdim), *extra, out_shape, ctypes.byref(out_ndim))
        return self._new(uop, tuple(out_shape[i] for i in range(out_ndim.value)))

    def sum(self, axis=-1, keepdim=False): return self._reduce('poly_sum_reduce', axis, keepdim)
    def max(self, axis=-1, keepdim=False): return self._reduce('poly_max_reduce', axis, keepdim)
    def mean(self, axis=-1, keepdim=False): return self._reduce('poly_mean_reduce', axis, keepdim)
    def var(self, axis=-1, keepdim=False, correction=1):
        return self._reduce('poly_var_reduce', axis, keepdim, int(correction))

    def softmax(self, axis=-1):
        axis = axis % len(self.shape)
        return self._new(self.dev.lib.poly_softmax(self.dev.ctx, self.uop, _i64(self.shape), len(self.shape), axis),
                         self.shape)

    def layernorm(self, axis=-1, eps=1e-5):
        axis = axis % len(self.shape)
        out_shape = (ctypes.c_int64 * 16)()
        out_ndim = ctypes.c_int(0)
        uop = self.dev.lib.poly_layernorm(self.dev.ctx, self.uop, _i64(self.shape), len(self.shape), axis,
                                          float(eps), out_shape, ctypes.byref(out_ndim))
        return self._new(uop, tuple(out_shape[i] for i in range(out_ndim.value)))

    def dot(self, w):
        out_shape = (ctypes.c_int64 * 16)()
        out_ndim = ctypes.c_int(0)
        uop = self.dev.lib.poly_dot(self.dev.ctx, self.uop, _i64(self.shape), len(self.shape),
                                    w.uop, _i64(w.shape), len(w.shape), out_shape, ctypes.byref(out_ndim))
        if not uop:
            raise ValueError('poly_dot rejected the shapes')
        return self._new(uop, tuple(out_shape[i] for i in range(out_ndim.value)), [w])

    def __matmul__(self, w): return self.dot(w)

    # ---- execution ----
    def numel(self):
        return int(np.prod(self.shape)) if self.shape else 1

    def numpy(self):
        """Realize on this tensor's device and return the result as an ndarray."""
        dev, lib = self.dev, self.dev.lib
        n = self.numel()
        np_dt = _NP.get(self.dtype, np.float32)
        out_buf = lib.poly_buffer_by_id(dev.ctx, n, ffi.DTYPE_IDS[self.dtype])
        out = np.zeros(n, dtype=np_dt)
        # the value keeps its shape (as in polygrad's Tensor._realize): the scheduler then
        # emits one range per axis instead of one flat range with div/mod indexing
        store = lib.poly_store_val(dev.ctx, out_buf, self.uop)
        sink = lib.poly_sink1(dev.ctx, store)
        pairs = list(self.leaves) + [(out_buf, out)]
        binds = (ffi.PolyBufferBinding * len(pairs))()
        dptrs = []
        for i, (buf, host) in enumerate(pairs):
            binds[i].buffer = buf
            if dev.is_cuda:
                d = lib.poly_cuda_alloc(max(host.nbytes, 4))
                if not d:
                    raise RuntimeError('poly_cuda_alloc failed: ' + lib.last_error())
                dptrs.append(d)
                if i < len(pairs) - 1:
                    if lib.poly_cuda_copy_htod(d, host.ctypes.data, host.nbytes) != 0:
                        raise RuntimeError('poly_cuda_copy_htod failed: ' + lib.last_error())
                binds[i].handle.ptr = d
                binds[i].handle.nbytes = host.nbytes
                binds[i].handle.domain = ffi.DEVICE_CUDA
            else:
                binds[i].handle.ptr = host.ctypes.data
                binds[i].handle.nbytes = host.nbytes
                binds[i].handle.domain = ffi.DEVICE_CPU
        rc = lib.poly_realize(dev.ctx, sink, binds, len(pairs))
        if rc != 0:
            msg = lib.last_error() if dev.is_cuda else ''
            raise RuntimeError(f'poly_realize failed ({rc}) {msg}')
        if dev.is_cuda:
            if lib.poly_cuda_copy_dtoh(out.ctypes.data, dptrs[-1], out.nbytes) != 0:
                raise RuntimeError('poly_cuda_copy_dtoh failed: ' + lib.last_error())
            for d in dptrs:
                lib.poly_cuda_free(d)
        return out.reshape(self.shape)


def embedding(ids, arange, table):
    """table[ids] the way polygrad's model builders write it (reference:
    src/modelzoo/models/gpt2.c:93-153): a one-hot mask (ids == arange) selects
    table rows, summed over the vocabulary axis.  ids [...], arange [V],
    table [V, D] -> [..., D]."""
    V, D = table.shape
    lead = ids.shape
    mask = ids.reshape(*lead, 1).expand(*lead, V).eq(arange.reshape(*((1,) * len(lead)), V).expand(*lead, V))
    mask = mask.reshape(*lead, V, 1).expand(*lead, V, D)
    tbl = table.reshape(*((1,) * len(lead)), V, D).expand(*lead, V, D)
    return mask.where(tbl, 0.0).sum(len(lead))
