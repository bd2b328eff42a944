"""`Tensor`, the NumPy-backed differentiable ops, and the GPU-backed `Attention` op.

Interface and semantics follow the reference's `optimizer/operators.py` (Tensor :14-187,
TensorOp :189-191, NumPy ops :194-475, GPU-backed op pattern `FC` :498-532): node data is a
NumPy array by default; an op that uses the GPU uploads its inputs into `myTensor` tensors,
calls a `myLayer` function, and downloads the result.  `Attention` is the op the reference
lacks; composing MatMul/Transpose/MulScalar/EWiseAdd/Exp/Summation/Reshape/BroadcastTo/EWiseDiv
from this module gives the same numbers on the CPU (that composition is what the tests check
the kernels against).

Device-resident nodes: `Tensor(x, device="gpu")` keeps a `myTensor` tensor as the node's data
instead of a NumPy array, so a chain of device-capable ops (`Attention`, `Softmax`, `+`, `-`,
scalar `*`, unary `-`, and the reverse sweep's adjoint sums) never leaves the GPU -- the
reference's GPU ops go through `get_data()` -> Python list -> `np.array` on every call
(operators.py:56-58, 511 there).  Ops without a device implementation refuse device inputs
(`TypeError`); `.cpu()` makes the copy explicit.
"""
from __future__ import annotations

import math
import os
import sys
from typing import Optional

import numpy as np

from .engine import Op, Value, backward_pass

_HOST = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "host_modules")


def _native():
    """The pybind modules (built by `build.py`); imported on first GPU op."""
    if _HOST not in sys.path:
        sys.path.insert(0, _HOST)
    try:
        import myTensor
        import myLayer
    except ImportError as e:  # no silent substitute: the op has no CPU implementation
        raise ImportError("myTensor/myLayer are not built; run `python pku-aiprogramming_b200/build.py`") from e
    return myTensor, myLayer


def _on_device(x) -> bool:
    """True for a `myTensor` tensor (node data kept on the GPU)."""
    return hasattr(x, "get_device") and hasattr(x, "get_shape")


def _device_dtype(x):
    name = type(x).__name__
    return {"Tensor_float": np.dtype(np.float32), "Tensor_double": np.dtype(np.float64),
            "Tensor_int": np.dtype(np.int32)}.get(name, "bfloat16")


def _to_device(array, dtype=None):
    """A gpu `myTensor` tensor holding `array` (NumPy data is uploaded once; a `myTensor` tensor
    is taken as is, or copied to the GPU if it lives on the host)."""
    mt, _ = _native()
    if _on_device(array):
        if array.get_device() == "gpu":
            return array
        moved = type(array)(array)
        moved.gpu()
        return moved
    cls = mt.Tensor_bf16 if str(dtype) == "bfloat16" else mt.Tensor_float
    return cls(np.ascontiguousarray(array, dtype=np.float32), "gpu")


class Tensor(Value):
    grad: "Tensor"

    def __init__(self, array, *, device=None, dtype=None, requires_grad=True, **kwargs):
        if device == "gpu":
            src = array.realize_cached_data() if isinstance(array, Tensor) else array
            self._init(None, [], cached_data=_to_device(src, dtype), requires_grad=requires_grad)
            return
        if isinstance(array, Tensor):
            data = array.realize_cached_data()
            data = data if dtype is None else np.asarray(data, dtype=dtype)
        elif isinstance(array, np.ndarray):
            data = np.array(array, dtype=dtype)
        elif hasattr(array, "get_data") and hasattr(array, "get_shape"):   # a myTensor tensor
            data = np.array(array.get_data(), dtype=dtype).reshape(array.get_shape())
        else:
            data = np.array(array, dtype=dtype)
        self._init(None, [], cached_data=data, requires_grad=requires_grad)

    @staticmethod
    def make_from_op(op: Op, inputs):
        if not getattr(op, "device_ok", False) and any(x.is_device for x in inputs):
            raise TypeError(f"{type(op).__name__} has no device implementation; call .cpu() on its inputs")
        t = Tensor.__new__(Tensor)
        t._init(op, inputs)
        if not t.requires_grad:
            return t.detach()
        t.realize_cached_data()
        return t

    @staticmethod
    def make_const(data, requires_grad=False):
        t = Tensor.__new__(Tensor)
        t._init(None, [], cached_data=data.realize_cached_data() if isinstance(data, Tensor) else data,
                requires_grad=requires_grad)
        return t

    def detach(self):
        return Tensor.make_const(self.realize_cached_data())

    @property
    def data(self):
        return self.detach()

    @data.setter
    def data(self, value):
        assert isinstance(value, Tensor) and value.dtype == self.dtype
        self.cached_data = value.realize_cached_data()

    @property
    def is_device(self) -> bool:
        return _on_device(self.realize_cached_data())

    @property
    def shape(self):
        d = self.realize_cached_data()
        return tuple(d.get_shape()) if _on_device(d) else d.shape

    @property
    def dtype(self):
        d = self.realize_cached_data()
        return _device_dtype(d) if _on_device(d) else d.dtype

    def numpy(self):
        """Node data as a NumPy array (a download for a device-resident node; bf16 widens to float32)."""
        d = self.realize_cached_data()
        return d.numpy() if _on_device(d) else d

    def cpu(self):
        """A NumPy-backed leaf holding this node's data."""
        return Tensor(self.numpy(), requires_grad=self.requires_grad)

    def gpu(self, dtype=None):
        """A device-resident leaf holding this node's data (float32, or bf16 with dtype="bfloat16")."""
        return Tensor(self.realize_cached_data(), device="gpu", dtype=dtype, requires_grad=self.requires_grad)

    def backward(self, out_grad=None):
        if out_grad is None:
            d = self.realize_cached_data()
            if _on_device(d):
                ones = type(d)(list(d.get_shape()), "gpu")
                ones.ones()
                out_grad = Tensor(ones, device="gpu", requires_grad=False)
            else:
                out_grad = Tensor(np.ones(self.shape, dtype=self.dtype), requires_grad=False)
        backward_pass(self, out_grad)

    def __repr__(self):
        return "Tensor(" + str(self.numpy()) + ")"

    __str__ = lambda self: str(self.numpy())

    def __add__(self, other):
        return EWiseAdd()(self, other) if isinstance(other, Tensor) else AddScalar(other)(self)

    def __mul__(self, other):
        return EWiseMul()(self, other) if isinstance(other, Tensor) else MulScalar(other)(self)

    def __sub__(self, other):
        return EWiseAdd()(self, Negate()(other)) if isinstance(other, Tensor) else AddScalar(-other)(self)

    def __truediv__(self, other):
        return EWiseDiv()(self, other) if isinstance(other, Tensor) else DivScalar(other)(self)

    def __pow__(self, other):
        return PowerScalar(other)(self)

    def __neg__(self):
        return Negate()(self)

    def __matmul__(self, other):
        return MatMul()(self, other)

    matmul = __matmul__
    __radd__ = __add__
    __rmul__ = __mul__

    def sum(self, axes=None):
        return Summation(axes)(self)

    def reshape(self, shape):
        return Reshape(shape)(self)

    def broadcast_to(self, shape):
        return BroadcastTo(shape)(self)

    def transpose(self, axes=None):
        return Transpose(axes)(self)


class TensorOp(Op):
    def __call__(self, *args):
        return Tensor.make_from_op(self, args)


# ----------------------------------------------------------------------------- NumPy ops
def _all_or_none_on_device(*arrays) -> bool:
    n = sum(_on_device(a) for a in arrays)
    if n not in (0, len(arrays)):
        raise TypeError("mixing device-resident and NumPy-backed tensors in one op; move one side with .gpu()/.cpu()")
    return n > 0


def _device_copy(a):
    return type(a)(a)


class EWiseAdd(TensorOp):
    device_ok = True

    def compute(self, a, b):
        _all_or_none_on_device(a, b)
        return a + b          # TinyTensor::operator+ on the device, ndarray add on the host

    def gradient(self, g, node):
        return g, g


class AddScalar(TensorOp):
    device_ok = True

    def __init__(self, scalar):
        self.scalar = scalar

    def compute(self, a):
        if _on_device(a):
            fill = type(a)(list(a.get_shape()), "gpu")
            fill.floatks(float(self.scalar))
            return a + fill
        return a + self.scalar

    def gradient(self, g, node):
        return g


class EWiseMul(TensorOp):
    def compute(self, a, b):
        return a * b

    def gradient(self, g, node):
        a, b = node.inputs
        return g * b, g * a


class MulScalar(TensorOp):
    device_ok = True

    def __init__(self, scalar):
        self.scalar = scalar

    def compute(self, a):
        if _on_device(a):
            out = _device_copy(a)
            out.mults(float(self.scalar))
            return out
        return a * self.scalar

    def gradient(self, g, node):
        return g * self.scalar


class PowerScalar(TensorOp):
    def __init__(self, scalar):
        self.scalar = scalar

    def compute(self, a):
        return np.power(a, self.scalar)

    def gradient(self, g, node):
        (a,) = node.inputs
        return g * self.scalar * (a ** (self.scalar - 1))


class EWiseDiv(TensorOp):
    def compute(self, a, b):
        return a / b

    def gradient(self, g, node):
        a, b = node.inputs
        return g / b, -g * a / (b ** 2)


class DivScalar(TensorOp):
    def __init__(self, scalar):
        self.scalar = scalar

    def compute(self, a):
        return a / self.scalar

    def gradient(self, g, node):
        return g / self.scalar


class Negate(TensorOp):
    device_ok = True

    def compute(self, a):
        if _on_device(a):
            out = _device_copy(a)
            out.negative()
            return out
        return -a

    def gradient(self, g, node):
        return -g


class Log(TensorOp):
    def compute(self, a):
        return np.log(a)

    def gradient(self, g, node):
        return g / node.inputs[0]


class Exp(TensorOp):
    def compute(self, a):
        return np.exp(a)

    def gradient(self, g, node):
        return g * Tensor(np.exp(node.inputs[0].realize_cached_data()), requires_grad=False)


class Transpose(TensorOp):
    """Swaps two axes; the last two when `axes` is None."""

    def __init__(self, axes: Optional[tuple] = None):
        self.axes = axes

    def compute(self, a):
        i, j = (a.ndim - 2, a.ndim - 1) if self.axes is None else self.axes
        return np.swapaxes(a, i, j)

    def gradient(self, g, node):
        return Transpose(self.axes)(g)


class Reshape(TensorOp):
    def __init__(self, shape):
        self.shape = shape

    def compute(self, a):
        return np.reshape(a, self.shape)

    def gradient(self, g, node):
        return Reshape(node.inputs[0].shape)(g)


class BroadcastTo(TensorOp):
    def __init__(self, shape):
        self.shape = tuple(shape)

    def compute(self, a):
        return np.broadcast_to(a, self.shape)

    def gradient(self, g, node):
        src = tuple(node.inputs[0].shape)
        padded = (1,) * (len(self.shape) - len(src)) + src
        axes = tuple(i for i, (s, t) in enumerate(zip(padded, self.shape)) if s != t)
        return Reshape(src)(Summation(axes)(g))


class Summation(TensorOp):
    def __init__(self, axes=None):
        self.axes = axes if axes is None or isinstance(axes, (tuple, list)) else (axes,)

    def compute(self, a):
        return np.sum(a) if self.axes is None else np.sum(a, axis=tuple(self.axes))

    def gradient(self, g, node):
        shape = node.inputs[0].shape
        axes = range(len(shape)) if self.axes is None else self.axes
        kept = [1 if i in axes else s for i, s in enumerate(shape)]
        return BroadcastTo(shape)(Reshape(kept)(g))


class MatMul(TensorOp):
    def compute(self, a, b):
        return np.matmul(a, b)

    def gradient(self, g, node):
        a, b = node.inputs
        ga, gb = MatMul()(g, Transpose()(b)), MatMul()(Transpose()(a), g)
        if len(ga.shape) > len(a.shape):
            ga = Summation(tuple(range(len(ga.shape) - len(a.shape))))(ga)
        if len(gb.shape) > len(b.shape):
            gb = Summation(tuple(range(len(gb.shape) - len(b.shape))))(gb)
        return ga, gb


def add(a, b): return EWiseAdd()(a, b)
def add_scalar(a, s): return AddScalar(s)(a)
def multiply(a, b): return EWiseMul()(a, b)
def mul_scalar(a, s): return MulScalar(s)(a)
def power_scalar(a, s): return PowerScalar(s)(a)
def divide(a, b): return EWiseDiv()(a, b)
def divide_scalar(a, s): return DivScalar(s)(a)
def negate(a): return Negate()(a)
def log(a): return Log()(a)
def exp(a): return Exp()(a)
def transpose(a, axes=None): return Transpose(axes)(a)
def reshape(a, shape): return Reshape(shape)(a)
def broadcast_to(a, shape): return BroadcastTo(shape)(a)
def summation(a, axes=None): return Summation(axes)(a)
def matmul(a, b): return MatMul()(a, b)


# ----------------------------------------------------------------------------- attention
class Attention(TensorOp):
    """`softmax(scale * q k^T [+ causal mask]) v` on the GPU.

    q `[B,H,S,D]`, k and v `[B,H,L,D]`.  With NumPy-backed inputs, `dtype="float32"` runs the
    exact fp32 kernels and `dtype="bfloat16"` rounds the inputs to bf16 (nearest even) and runs
    the tensor-core kernels; inputs are uploaded and the result comes back as NumPy float32 (the
    reference's GPU-op pattern).  With device-resident inputs (all three `Tensor_float` or all
    three `Tensor_bf16`) nothing is copied: the result and the gradients are device-resident
    nodes of the same element type.  The forward keeps `out` and `lse` on the op instance for
    the backward, like the reference's ops keep their masks (operators.py:577-586 of the
    reference).
    """
    device_ok = True

    def __init__(self, causal: bool = False, scale: Optional[float] = None, dtype: str = "float32"):
        if dtype not in ("float32", "bfloat16"):
            raise ValueError("dtype must be 'float32' or 'bfloat16'")
        self.causal, self.scale, self.dtype = bool(causal), 0.0 if scale is None else float(scale), dtype
        self._saved = None

    @staticmethod
    def _names(bf16: bool):
        mt, ml = _native()
        if bf16:
            return mt.Tensor_bf16, ml.AttentionForward_bf16, ml.AttentionBackward_bf16, mt.Tensor_float
        return mt.Tensor_float, ml.AttentionForward, ml.AttentionBackward, mt.Tensor_float

    def compute(self, q, k, v):
        resident = _all_or_none_on_device(q, k, v)
        if resident:
            if not (type(q) is type(k) is type(v)) or type(q).__name__ not in ("Tensor_float", "Tensor_bf16"):
                raise TypeError("device-resident q, k, v must all be Tensor_float or all Tensor_bf16")
            bf16 = type(q).__name__ == "Tensor_bf16"
            T, fwd, _, F = self._names(bf16)
            tq, tk, tv, shape = q, k, v, list(q.get_shape())
        else:
            bf16 = self.dtype == "bfloat16"
            T, fwd, _, F = self._names(bf16)
            up = lambda a: T(np.ascontiguousarray(a, dtype=np.float32), "gpu")
            tq, tk, tv, shape = up(q), up(k), up(v), list(q.shape)
        out, lse = T(shape, "gpu"), F(shape[:3], "gpu")
        fwd(tq, tk, tv, out, lse, self.causal, self.scale)
        self._saved = (tq, tk, tv, out, lse, bf16, resident)
        return out if resident else out.numpy().astype(q.dtype, copy=False)

    def gradient(self, out_grad, node):
        if self._saved is None:
            node.realize_cached_data()
        tq, tk, tv, out, lse, bf16, resident = self._saved
        T, _, bwd, _ = self._names(bf16)
        g = out_grad.realize_cached_data()
        if _on_device(g):
            if type(g) is not T:
                raise TypeError(f"upstream gradient is {type(g).__name__}, the op ran on {T.__name__}")
            go = g
        else:
            go = T(np.ascontiguousarray(g, dtype=np.float32), "gpu")
        gq, gk, gv = T(tq.get_shape(), "gpu"), T(tk.get_shape(), "gpu"), T(tv.get_shape(), "gpu")
        bwd(tq, tk, tv, out, lse, gq, gk, gv, go, self.causal, self.scale)
        if resident:
            return tuple(Tensor(t, device="gpu", requires_grad=False) for t in (gq, gk, gv))
        dt = node.inputs[0].dtype
        mk = lambda t: Tensor(t.numpy().astype(dt, copy=False), requires_grad=False)
        return mk(gq), mk(gk), mk(gv)


class Softmax(TensorOp):
    """Softmax over the last axis on the GPU (`myLayer.SoftmaxForward` / `SoftmaxBackward`,
    float32).  NumPy-backed input: upload, run, download; device-resident input: stays there."""
    device_ok = True

    def __init__(self):
        self._y = None

    def compute(self, x):
        mt, ml = _native()
        resident = _on_device(x)
        if resident and type(x).__name__ != "Tensor_float":
            raise TypeError("Softmax takes float32 data")
        tx = x if resident else mt.Tensor_float(np.ascontiguousarray(x, dtype=np.float32), "gpu")
        y = mt.Tensor_float([1], "gpu")
        ml.SoftmaxForward(tx, y)
        self._y, self._resident = y, resident
        return y if resident else y.numpy().astype(x.dtype, copy=False)

    def gradient(self, out_grad, node):
        mt, ml = _native()
        if self._y is None:
            node.realize_cached_data()
        g = out_grad.realize_cached_data()
        tg = g if _on_device(g) else mt.Tensor_float(np.ascontiguousarray(g, dtype=np.float32), "gpu")
        dx = mt.Tensor_float([1], "gpu")
        ml.SoftmaxBackward(self._y, tg, dx)
        if self._resident:
            return Tensor(dx, device="gpu", requires_grad=False)
        return Tensor(dx.numpy().astype(node.inputs[0].dtype, copy=False), requires_grad=False)


def softmax(x):
    return Softmax()(x)


class FC(TensorOp):
    """`input @ weight + bias` on the GPU (`myLayer.FcForward` / `FcBackward`), the reference's
    `FC` op (operators.py:498-532 there: same constructor flag, same three inputs, bias of shape
    `[out]` or `[1]`).  NumPy-backed inputs are uploaded (`dtype` picks float32 or bf16 kernels)
    and results downloaded; device-resident inputs (all `Tensor_float` or all `Tensor_bf16`) stay
    on the GPU, as do the three gradients."""
    device_ok = True

    def __init__(self, use_bias=True, dtype: str = "float32"):
        if dtype not in ("float32", "bfloat16"):
            raise ValueError("dtype must be 'float32' or 'bfloat16'")
        self.use_bias, self.dtype = bool(use_bias), dtype
        self._saved = None

    def _pick(self, resident, sample):
        mt, ml = _native()
        bf16 = (type(sample).__name__ == "Tensor_bf16") if resident else self.dtype == "bfloat16"
        return (mt.Tensor_bf16, ml.FcForward_bf16, ml.FcBackward_bf16) if bf16 else (mt.Tensor_float, ml.FcForward, ml.FcBackward)

    def compute(self, x, w, b):
        resident = _all_or_none_on_device(x, w, b)
        T, fwd, _ = self._pick(resident, x)
        if resident and not (type(x) is type(w) is type(b) is T):
            raise TypeError("device-resident input, weight and bias must share one tensor class")
        up = (lambda a: a) if resident else (lambda a: T(np.ascontiguousarray(a, dtype=np.float32), "gpu"))
        tx, tw, tb = up(x), up(w), up(b)
        if not self.use_bias:
            tb = T(tb)
            tb.zeros()
        out = T([1], "gpu")
        fwd(tx, out, tw, tb)
        self._saved = (tx, tw, tb, out, resident)
        return out if resident else out.numpy().astype(x.dtype, copy=False)

    def gradient(self, out_grad, node):
        if self._saved is None:
            node.realize_cached_data()
        tx, tw, tb, out, resident = self._saved
        T, _, bwd = self._pick(True, tx)
        g = out_grad.realize_cached_data()
        tg = g if _on_device(g) else T(np.ascontiguousarray(g, dtype=np.float32), "gpu")
        gx, gw, gb = T([1], "gpu"), T([1], "gpu"), T([1], "gpu")
        bwd(tx, out, tw, tb, gx, tg, gw, gb)
        if not self.use_bias:
            gb.zeros()
        if resident:
            return tuple(Tensor(t, device="gpu", requires_grad=False) for t in (gx, gw, gb))
        dt = node.inputs[0].dtype
        return tuple(Tensor(t.numpy().astype(dt, copy=False), requires_grad=False) for t in (gx, gw, gb))


def fc(input, weight, bias, use_bias=True, dtype: str = "float32"):
    return FC(use_bias, dtype)(input, weight, bias)


def attention(q, k, v, causal: bool = False, scale: Optional[float] = None, dtype: str = "float32"):
    return Attention(causal, scale, dtype)(q, k, v)


def attention_composed(q, k, v, causal: bool = False, scale: Optional[float] = None):
    """The same function built from the NumPy ops above (CPU): the reference's way of writing
    attention with what it ships.  Used as the cross-check of the fused op."""
    B, H, S, D = q.shape
    L = k.shape[2]
    sc = 1.0 / math.sqrt(D) if not scale or scale <= 0 else float(scale)
    s = (q @ transpose(k)) * sc
    if causal:
        i, j = np.arange(S)[:, None], np.arange(L)[None, :]
        mask = np.where(j <= i + (L - S), 0.0, -1e30).astype(q.dtype)
        s = s + Tensor(np.ascontiguousarray(np.broadcast_to(mask, (B, H, S, L))), requires_grad=False)
    e = exp(s)
    den = broadcast_to(reshape(summation(e, axes=(3,)), (B, H, S, 1)), (B, H, S, L))
    return (e / den) @ v
