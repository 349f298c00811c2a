"""NumPy-backed stand-in for the few ``mlx.core`` symbols that easymlx's paged
cache and unified-attention modules touch.

Test infrastructure only: ``tests/golden/make_golden.py`` puts this directory on
``sys.path`` so that the reference's own Python (its page-cache write path and
its NumPy attention fallback) can be imported and executed on a machine without
MLX, to produce the golden fixtures stored next to that script.  Nothing in the
shipped package imports it.

Semantics that matter for the fixtures:
  * 64-bit inputs narrow to 32-bit on construction, as MLX does;
  * fancy-index reads and writes follow NumPy rules (negative ids wrap);
  * ``fast.metal_kernel`` builds a callable that raises, so the reference takes
    its own CPU fallback branch.
"""

from __future__ import annotations

import numpy as np


class Dtype:
    def __init__(self, np_dtype, name):
        self.np = np.dtype(np_dtype)
        self.name = name

    def __repr__(self):
        return f"mlx.core.{self.name}"

    def __eq__(self, other):
        return isinstance(other, Dtype) and other.name == self.name

    def __hash__(self):
        return hash(self.name)


float16 = Dtype(np.float16, "float16")
float32 = Dtype(np.float32, "float32")
bfloat16 = Dtype(np.float32, "bfloat16")  # no numpy bf16; never used by the fixtures
int32 = Dtype(np.int32, "int32")
int64 = Dtype(np.int64, "int64")
uint8 = Dtype(np.uint8, "uint8")
uint32 = Dtype(np.uint32, "uint32")
bool_ = Dtype(np.bool_, "bool_")

_FROM_NUMPY = {d.np: d for d in (float16, float32, int32, int64, uint8, uint32, bool_)}

ArrayLike = object


def _raw(x):
    return x._a if isinstance(x, array) else x


class array:
    def __init__(self, value, dtype=None):
        a = np.asarray(_raw(value))
        if dtype is not None:
            a = a.astype(dtype.np)
        elif a.dtype == np.float64:
            a = a.astype(np.float32)
        elif a.dtype == np.int64:
            a = a.astype(np.int32)
        self._a = np.array(a)

    @property
    def dtype(self):
        return _FROM_NUMPY[self._a.dtype]

    @property
    def shape(self):
        return tuple(self._a.shape)

    @property
    def ndim(self):
        return self._a.ndim

    @property
    def size(self):
        return self._a.size

    def __array__(self, dtype=None, copy=None):
        return self._a if dtype is None else self._a.astype(dtype)

    def astype(self, dtype):
        return array(self._a.astype(dtype.np))

    def item(self):
        return self._a.item()

    def tolist(self):
        return self._a.tolist()

    def reshape(self, *shape):
        return array(self._a.reshape(*shape))

    def transpose(self, *axes):
        return array(self._a.transpose(*axes))

    def __int__(self):
        return int(self._a)

    def __len__(self):
        return len(self._a)

    @staticmethod
    def _key(key):
        if isinstance(key, tuple):
            return tuple(_raw(k) for k in key)
        return _raw(key)

    def __getitem__(self, key):
        return array(self._a[self._key(key)])

    def __setitem__(self, key, value):
        self._a[self._key(key)] = _raw(value)


def _install_operators():
    names = ("add", "sub", "mul", "truediv", "floordiv", "mod", "le", "lt", "ge", "gt", "and", "or", "eq")
    for name in names:
        def forward(self, other, _n=name):
            return array(getattr(self._a, f"__{_n}__")(_raw(other)))

        def reverse(self, other, _n=name):
            return array(getattr(np.asarray(_raw(other)), f"__{_n}__")(self._a))

        setattr(array, f"__{name}__", forward)
        setattr(array, f"__r{name}__", reverse)


_install_operators()


def zeros(shape, dtype=float32):
    return array(np.zeros(shape, dtype.np))


def zeros_like(a):
    return array(np.zeros_like(_raw(a)))


def arange(*args, dtype=int32):
    return array(np.arange(*args), dtype)


def full(shape, value, dtype=float32):
    return array(np.full(shape, _raw(value), dtype.np))


def stack(xs, axis=0):
    return array(np.stack([_raw(x) for x in xs], axis))


def concatenate(xs, axis=0):
    return array(np.concatenate([_raw(x) for x in xs], axis))


def repeat(a, repeats, axis=None):
    return array(np.repeat(_raw(a), repeats, axis))


def maximum(a, b):
    return array(np.maximum(_raw(a), _raw(b)))


def minimum(a, b):
    return array(np.minimum(_raw(a), _raw(b)))


def take(a, indices, axis=None):
    return array(np.take(_raw(a), _raw(indices), axis=axis))


def cumsum(a, axis=None):
    return array(np.cumsum(_raw(a), axis=axis))


def compile(fn, *_, **__):
    return fn


def where(cond, a, b):
    return array(np.where(_raw(cond), _raw(a), _raw(b)))


def einsum(subscripts, *operands):
    return array(np.einsum(subscripts, *[_raw(o) for o in operands]))


def softmax(a, axis=-1):
    a = _raw(a)
    e = np.exp(a - a.max(axis=axis, keepdims=True))
    return array(e / e.sum(axis=axis, keepdims=True))


def expand_dims(a, axis):
    return array(np.expand_dims(_raw(a), axis))


def eval(*_):
    return None


class _Fast:
    @staticmethod
    def metal_kernel(**_):
        def _unavailable(*__, **___):
            raise RuntimeError("Metal is not available under the NumPy stand-in")

        return _unavailable


fast = _Fast()
