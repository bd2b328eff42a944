"""GPU tests of the reference-style host layer: the `Attention` autograd op (Python ->
pybind `myLayer` -> C++ `AttentionForward/Backward` -> C ABI -> kernels) against the golden
fixtures, and TinyTensor on the device."""
import glob
import importlib
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz")))


@pytest.fixture(scope="module")
def opt(tt):
    return importlib.import_module("pku-aiprogramming_b200.optimizer")


@pytest.fixture(scope="module")
def mods(tt):
    sys.path.insert(0, os.path.join(ROOT, "pku-aiprogramming_b200", "host_modules"))
    import myLayer
    import myTensor
    return myTensor, myLayer


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_attention_op_fp32_matches_reference(opt, oracle, path):
    g = np.load(path)
    q, k, v = (opt.Tensor(g[n]) for n in "qkv")
    o = opt.attention(q, k, v, causal=bool(g["causal"]), scale=float(g["scale"]))
    o.backward(opt.Tensor(g["do"], requires_grad=False))
    for got, name in ((o, "o"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        assert got.numpy().dtype == np.float32
        assert oracle.rel_err(got.numpy(), g[name]) <= 1e-5, name


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_attention_op_bf16_matches_oracle(opt, oracle, path):
    g = np.load(path)
    causal, scale = bool(g["causal"]), float(g["scale"])
    qn, kn, vn, don = (oracle.bf16_round(g[n]) for n in ("q", "k", "v", "do"))
    o_ref, _, dq_ref, dk_ref, dv_ref = oracle.attention_backward(qn, kn, vn, don, causal, scale)
    q, k, v = (opt.Tensor(x) for x in (qn, kn, vn))
    o = opt.attention(q, k, v, causal=causal, scale=scale, dtype="bfloat16")
    o.backward(opt.Tensor(don, requires_grad=False))
    for got, ref, name in ((o, o_ref, "o"), (q.grad, dq_ref, "dq"), (k.grad, dk_ref, "dk"), (v.grad, dv_ref, "dv")):
        assert oracle.max_abs_err(got.numpy(), ref) <= 2e-2, name


def test_attention_op_inside_a_graph(opt, oracle):
    """The op chains with the NumPy ops: loss = sum((attention(q*2, k, v) + q) * w)."""
    q0, k0, v0, w0 = oracle.make_inputs(51, 1, 2, 33, 33, 32)
    q, k, v = opt.Tensor(q0), opt.Tensor(k0), opt.Tensor(v0)
    y = opt.attention(q * 2.0, k, v, causal=True) + q
    y.backward(opt.Tensor(w0, requires_grad=False))
    q2, k2, v2 = opt.Tensor(q0), opt.Tensor(k0), opt.Tensor(v0)
    y2 = opt.attention_composed(q2 * 2.0, k2, v2, causal=True) + q2
    y2.backward(opt.Tensor(w0, requires_grad=False))
    assert oracle.rel_err(y.numpy(), y2.numpy()) <= 1e-5
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert oracle.rel_err(a.grad.numpy(), b.grad.numpy()) <= 1e-5


def test_mylayer_decode_dispatch_and_softmax(mods, oracle):
    mt, ml = mods
    q, k, v, _ = oracle.make_inputs(53, 2, 2, 1, 700, 128, with_do=False)
    qn, kn, vn = (oracle.bf16_round(x) for x in (q, k, v))
    tq, tk, tv = (mt.Tensor_bf16(x, "gpu") for x in (qn, kn, vn))
    out, lse = mt.Tensor_bf16([1], "gpu"), mt.Tensor_float([1], "gpu")
    ml.AttentionForward_bf16(tq, tk, tv, out, lse, False, 0.0)       # S == 1 -> split-KV decode kernel
    o_ref, lse_ref = oracle.attention_forward(qn, kn, vn, False)
    assert out.get_shape() == [2, 2, 1, 128] and lse.get_shape() == [2, 2, 1]
    assert oracle.max_abs_err(out.numpy(), o_ref) <= 2e-2 and oracle.max_abs_err(lse.numpy(), lse_ref) <= 1e-3
    x = np.random.default_rng(3).standard_normal((5, 7, 33)).astype(np.float32)
    y = mt.Tensor_float([1], "gpu")
    ml.SoftmaxForward(mt.Tensor_float(x, "gpu"), y)
    e = np.exp(x - x.max(-1, keepdims=True))
    assert np.allclose(y.numpy(), e / e.sum(-1, keepdims=True), atol=1e-6) and y.get_shape() == [5, 7, 33]
    dy = np.random.default_rng(4).standard_normal(x.shape).astype(np.float32)
    dx = mt.Tensor_float([1], "gpu")
    ml.SoftmaxBackward(y, mt.Tensor_float(dy, "gpu"), dx)
    assert oracle.rel_err(dx.numpy(), oracle.softmax_rows_backward(x, dy)) <= 1e-5
    with pytest.raises(ValueError):
        ml.SoftmaxBackward(y, mt.Tensor_float(dy[:, :, :5].copy(), "gpu"), dx)


def test_tensor_on_device(mods):
    mt, _ = mods
    a = mt.Tensor_float(np.arange(6, dtype=np.float32).reshape(2, 3), "gpu")
    b = mt.Tensor_float([2, 3], "gpu").ones().mults(3.0)
    assert (a + b).get_data() == [3, 4, 5, 6, 7, 8] and a.get_device() == "gpu"
    assert a[1].get_data() == [3, 4, 5] and a[1].get_device() == "gpu"
    c = mt.Tensor_float(a)
    c.cpu()
    assert c.get_device() == "cpu" and c.get_data() == a.get_data() and a.get_device() == "gpu"
    c.gpu().negative()
    assert c.get_data() == [0, -1, -2, -3, -4, -5]
    r = np.array(mt.Tensor_float([100000], "gpu").random(2.0, 4.0).get_data())
    assert r.min() >= 2.0 and r.max() < 4.0 and abs(r.mean() - 3.0) < 0.02
    d = mt.Tensor_bf16(np.array([1.0, -2.5, 3.0], dtype=np.float32), "gpu")
    assert d.ReluForward().get_data() == [1.0, 0.0, 3.0]
    g = mt.Tensor_float([2, 2], "gpu", [1, 2, 3, 4])
    assert g.resize([3, 2]).get_data() == [1, 2, 3, 4, 0, 0]
    assert mt.Tensor_int([3], "gpu", [1, 2, 3]).negative().get_data() == [-1, -2, -3]
