"""CPU tests of the reference-style host layer: TinyTensor value semantics (on "cpu" tensors),
the autograd engine, and the composed-attention cross-check against the golden fixtures."""
import glob
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz")))


@pytest.fixture(scope="module")
def mods(tt):
    host = os.path.join(ROOT, "pku-aiprogramming_b200", "host_modules")
    if not glob.glob(os.path.join(host, "myTensor*.so")):
        pytest.fail("host modules not built: run python pku-aiprogramming_b200/build.py")
    sys.path.insert(0, host)
    import myLayer
    import myTensor
    return myTensor, myLayer


@pytest.fixture(scope="module")
def opt(tt):
    return importlib.import_module("pku-aiprogramming_b200.optimizer")


def test_module_surface(mods):
    mt, ml = mods
    methods = ["Size", "__add__", "__sub__", "__getitem__", "get_shape", "get_device", "get_data", "flatten", "cpu",
               "gpu", "random", "zeros", "ones", "negative", "mults", "floatks", "resize", "ReluForward", "ReluBackward",
               "SigmoidForward", "SigmoidBackward", "__repr__", "numpy", "data_ptr", "__dlpack__", "__dlpack_device__",
               "from_dlpack"]
    for cls in ("Tensor_float", "Tensor_double", "Tensor_int", "Tensor_bf16"):
        for m in methods:
            assert hasattr(getattr(mt, cls), m), (cls, m)
    for fn in ("AttentionForward", "AttentionBackward", "AttentionForward_bf16", "AttentionBackward_bf16",
               "SoftmaxForward", "SoftmaxBackward", "FcForward", "FcBackward", "FcForward_bf16", "FcBackward_bf16"):
        assert hasattr(ml, fn)


def test_tensor_value_semantics(mods):
    mt, _ = mods
    a = mt.Tensor_float(np.arange(12, dtype=np.float32).reshape(3, 4), "cpu")
    b = mt.Tensor_float(a)                       # copy construction is deep
    b.mults(2.0)
    assert a.get_data()[5] == 5.0 and b.get_data()[5] == 10.0
    assert (a + b).get_data()[3] == 9.0 and (b - a).get_data() == a.get_data()
    assert a[2].get_shape() == [4] and a[2].get_data() == [8.0, 9.0, 10.0, 11.0]
    assert a[0][1].get_shape() == [1]            # slicing a 1-D tensor leaves shape [1], as in the reference
    assert a.flatten().get_shape() == [12] and a.Size() == 12
    with pytest.raises(ValueError):
        a[3]
    with pytest.raises(ValueError):
        mt.Tensor_float([2, 2], "tpu")
    with pytest.raises(ValueError):
        a + mt.Tensor_float([4, 3], "cpu")
    r = mt.Tensor_float([2, 3], "cpu", [1, 2, 3, 4, 5, 6])
    r.resize([3, 2])                             # same element count: pure reshape
    assert r.get_shape() == [3, 2] and r.get_data() == [1, 2, 3, 4, 5, 6]
    r.resize([2, 2])                             # shrink keeps the prefix
    assert r.get_data() == [1, 2, 3, 4]
    r.resize([3, 2])                             # grow keeps the prefix, new tail is zero
    assert r.get_data() == [1, 2, 3, 4, 0, 0]
    x = mt.Tensor_float([4], "cpu", [-1, 2, -3, 4])
    assert x.ReluForward().get_data() == [0, 2, 0, 4]
    assert x.ReluBackward(mt.Tensor_float([4], "cpu").ones()).get_data() == [0, 1, 0, 1]
    s = np.array(x.SigmoidForward().get_data())
    assert np.allclose(s, 1 / (1 + np.exp(-np.array([-1, 2, -3, 4.0]))), atol=1e-6)
    g = np.array(x.SigmoidBackward(mt.Tensor_float([4], "cpu").floatks(2.0)).get_data())
    assert np.allclose(g, 2 * s * (1 - s), atol=1e-6)
    u = np.array(mt.Tensor_float([1000], "cpu").random(-1.0, 3.0).get_data())
    assert u.min() >= -1.0 and u.max() < 3.0 and abs(u.mean() - 1.0) < 0.2
    i = mt.Tensor_int([2, 2], "cpu", [1, 2, 3, 4])
    assert i.negative().get_data() == [-1, -2, -3, -4] and mt.Tensor_double([2], "cpu").ones().get_data() == [1.0, 1.0]
    assert "Shape: [3, 4]" in repr(a) and "Device: cpu" in repr(a)


def test_bf16_tensor_rounds_to_nearest_even(mods, oracle):
    mt, _ = mods
    x = (np.random.default_rng(0).standard_normal(4096) * 3).astype(np.float32)
    t = mt.Tensor_bf16(x, "cpu")
    assert np.array_equal(np.array(t.get_data(), dtype=np.float32), oracle.bf16_round(x))
    assert np.array_equal(t.numpy(), oracle.bf16_round(x))
    assert mt.Tensor_bf16([2], "cpu", [1.0, 1.00390625]).get_data() == [1.0, 1.0]


def test_attention_needs_gpu_tensors(mods):
    mt, ml = mods
    q = mt.Tensor_float([1, 1, 4, 8], "cpu").ones()
    out, lse = mt.Tensor_float([1], "cpu"), mt.Tensor_float([1], "cpu")
    with pytest.raises(ValueError, match="gpu tensors only"):
        ml.AttentionForward(q, q, q, out, lse, False, 0.0)


def test_topological_order_and_accumulation(opt):
    a = opt.Tensor(np.array([2.0, 3.0]))
    b = a * a            # a is used twice by one node ...
    c = b + a            # ... and once more here: three partial adjoints
    order = opt.topological_order([c])
    assert order[0] is a and order[-1] is c and len(order) == 3
    c.backward()
    assert np.allclose(a.grad.numpy(), 2 * np.array([2.0, 3.0]) + 1)
    deep = a
    for _ in range(5000):   # an explicit-stack DFS: no recursion limit involved
        deep = deep + 1.0
    deep.backward()
    assert np.allclose(a.grad.numpy(), 1.0)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_composed_attention_reproduces_reference(opt, path):
    """Attention composed from this package's own NumPy ops + reverse sweep gives the reference's
    results bit for bit: the autograd layer is a faithful stand-in for the reference's."""
    g = np.load(path)
    q, k, v = (opt.Tensor(g[n]) for n in "qkv")
    o = opt.attention_composed(q, k, v, bool(g["causal"]), float(g["scale"]))
    o.backward(opt.Tensor(g["do"], requires_grad=False))
    for got, name in ((o, "o"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        assert np.array_equal(got.numpy(), g[name]), name


def test_dlpack_export_of_host_tensors_is_zero_copy(mods):
    mt, _ = mods
    for cls, dt in ((mt.Tensor_float, np.float32), (mt.Tensor_double, np.float64), (mt.Tensor_int, np.int32)):
        x = np.arange(24).reshape(2, 3, 4).astype(dt)
        t = cls(x, "cpu")
        assert t.__dlpack_device__() == (1, 0)            # kDLCPU
        view = np.from_dlpack(t)
        assert view.dtype == dt and view.shape == (2, 3, 4) and np.array_equal(view, x)
        assert view.ctypes.data == t.data_ptr()
        t.floatks(7)                                      # written through the tensor, seen through the view
        assert (view == 7).all()
    del t
    assert (view == 7).all()                              # the capsule keeps the tensor's buffer alive


def test_dlpack_import_copies_and_validates(mods):
    import torch
    mt, _ = mods
    x = np.random.default_rng(0).standard_normal((3, 5)).astype(np.float32)
    t = mt.Tensor_float.from_dlpack(x)
    assert t.get_device() == "cpu" and t.get_shape() == [3, 5] and np.array_equal(t.numpy(), x)
    assert t.data_ptr() != x.ctypes.data                  # a TinyTensor owns its buffer: deep copy
    b = torch.from_numpy(x).bfloat16()
    tb = mt.Tensor_bf16.from_dlpack(b)
    assert np.array_equal(tb.numpy(), b.float().numpy())
    assert mt.Tensor_int.from_dlpack(torch.arange(6, dtype=torch.int32).reshape(2, 3)).get_data() == [0, 1, 2, 3, 4, 5]
    with pytest.raises(ValueError):
        mt.Tensor_double.from_dlpack(x)                   # element type mismatch
    with pytest.raises(ValueError):
        mt.Tensor_float.from_dlpack(torch.from_numpy(x).t())   # not row-major contiguous
    with pytest.raises(ValueError):
        mt.Tensor_float.from_dlpack(object())
    r = torch.from_dlpack(mt.Tensor_bf16(x, "cpu"))       # bf16 leaves through torch (NumPy has no bf16)
    assert r.dtype == torch.bfloat16 and torch.equal(r, b)


def test_ops_without_device_form_are_marked(opt):
    ok = {n for n in dir(opt) if isinstance(getattr(opt, n), type) and getattr(getattr(opt, n), "device_ok", False)}
    assert {"EWiseAdd", "AddScalar", "MulScalar", "Negate", "Attention", "Softmax", "FC"} <= ok
    assert not ({"Exp", "MatMul", "Summation", "EWiseDiv", "Reshape"} & ok)


def test_exported_view_keeps_its_buffer_when_the_tensor_changes(mods):
    """A DLPack view shares ownership of the buffer it shows: resizing the tensor (which gives it a new
    buffer) or dropping it leaves the view's data intact, and the old block is handed back only when the
    view goes away."""
    import gc
    mt, _ = mods
    t = mt.Tensor_float(np.arange(12, dtype=np.float32).reshape(3, 4), "cpu")
    view = np.from_dlpack(t)
    keep = view.copy()
    t.resize([64, 64])                       # different element count: the tensor takes a new buffer
    other = [mt.Tensor_float(np.full((3, 4), 7.0, np.float32), "cpu") for _ in range(8)]   # would reuse a freed block
    assert np.array_equal(view, keep)
    del t
    gc.collect()
    assert np.array_equal(view, keep)
    del view, other
    gc.collect()
