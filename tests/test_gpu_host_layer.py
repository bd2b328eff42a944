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


def test_dlpack_device_exchange_with_torch(mods):
    import torch
    mt, _ = mods
    x = np.random.default_rng(1).standard_normal((4, 6, 8)).astype(np.float32)
    t = mt.Tensor_float(x, "gpu")
    kind, dev = t.__dlpack_device__()
    assert kind == 2 and dev == torch.cuda.current_device()          # kDLCUDA
    view = torch.from_dlpack(t)
    assert view.is_cuda and view.dtype == torch.float32 and tuple(view.shape) == (4, 6, 8)
    assert view.data_ptr() == t.data_ptr()                           # zero copy
    assert np.array_equal(view.cpu().numpy(), x)
    view.mul_(2.0)
    torch.cuda.synchronize()
    assert np.array_equal(t.numpy(), x * 2)
    tb = mt.Tensor_bf16(x, "gpu")
    vb = torch.from_dlpack(tb)
    assert vb.dtype == torch.bfloat16 and torch.equal(vb.cpu(), torch.from_numpy(x).bfloat16())
    src = torch.randn(5, 7, device="cuda").bfloat16()
    back = mt.Tensor_bf16.from_dlpack(src)                           # device-to-device deep copy
    assert back.get_device() == "gpu" and back.data_ptr() != src.data_ptr()
    assert np.array_equal(back.numpy(), src.float().cpu().numpy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_device_resident_graph_never_leaves_the_gpu(opt, oracle, mods, dtype):
    """loss = <attention(q*2, k, v) + q - k*0.5, w> with every node's data a gpu myTensor tensor."""
    mt, _ = mods
    q0, k0, v0, w0 = oracle.make_inputs(61, 1, 2, 160, 160, 64)
    if dtype == "bfloat16":
        q0, k0, v0, w0 = (oracle.bf16_round(a) for a in (q0, k0, v0, w0))
    q, k, v = (opt.Tensor(a, device="gpu", dtype=dtype) for a in (q0, k0, v0))
    w = opt.Tensor(w0, device="gpu", dtype=dtype, requires_grad=False)
    y = opt.attention(q * 2.0, k, v, causal=True) + q - k * 0.5
    y.backward(w)
    cls = mt.Tensor_bf16 if dtype == "bfloat16" else mt.Tensor_float
    for node in (y, q.grad, k.grad, v.grad):
        assert node.is_device and type(node.realize_cached_data()) is cls
        assert node.realize_cached_data().get_device() == "gpu"
    q2, k2, v2 = opt.Tensor(q0), opt.Tensor(k0), opt.Tensor(v0)
    y2 = opt.attention_composed(q2 * 2.0, k2, v2, causal=True) + q2 - k2 * 0.5
    y2.backward(opt.Tensor(w0, requires_grad=False))
    for a, b, name in ((y, y2, "y"), (q.grad, q2.grad, "dq"), (k.grad, k2.grad, "dk"), (v.grad, v2.grad, "dv")):
        if dtype == "float32":
            assert oracle.rel_err(a.numpy(), b.numpy()) <= 1e-5, name
        else:   # bf16 nodes round every intermediate; 2e-2 plus one bf16 ulp of the largest value
            assert oracle.max_abs_err(a.numpy(), b.numpy()) <= oracle.bf16_grad_tol(b.numpy()), name
    ones = opt.Tensor(q0, device="gpu")
    (ones * 3.0).backward()                                          # default seed: ones on the device
    assert ones.grad.is_device and np.array_equal(ones.grad.numpy(), np.full(q0.shape, 3.0, np.float32))


def test_device_resident_rules_and_softmax_op(opt, oracle):
    x0 = np.random.default_rng(5).standard_normal((6, 40)).astype(np.float32)
    g0 = np.random.default_rng(6).standard_normal((6, 40)).astype(np.float32)
    xd = opt.Tensor(x0, device="gpu")
    with pytest.raises(TypeError):
        opt.exp(xd)                                   # no device form: refuse instead of copying silently
    with pytest.raises(TypeError):
        xd + opt.Tensor(x0)                           # mixed residency
    assert np.array_equal(opt.exp(xd.cpu()).numpy(), np.exp(x0))
    for x in (xd, opt.Tensor(x0)):
        y = opt.softmax(x)
        y.backward(opt.Tensor(g0, device="gpu", requires_grad=False) if x.is_device else opt.Tensor(g0, requires_grad=False))
        assert y.is_device == x.is_device and x.grad.is_device == x.is_device
        assert oracle.rel_err(y.numpy(), oracle.softmax_rows(x0)) <= 1e-5
        assert oracle.rel_err(x.grad.numpy(), oracle.softmax_rows_backward(x0, g0)) <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_fc_op_numpy_and_device_resident(opt, oracle, mods, dtype):
    """The reference's FC op (input, weight, bias; bias [out] or [1]) through myLayer.FcForward/FcBackward."""
    rng = np.random.default_rng(12)
    x0 = rng.standard_normal((48, 72)).astype(np.float32)
    w0 = (rng.standard_normal((72, 40)) / 8).astype(np.float32)
    b0 = rng.standard_normal(40).astype(np.float32)
    g0 = rng.standard_normal((48, 40)).astype(np.float32)
    if dtype == "bfloat16":
        x0, w0, b0, g0 = (oracle.bf16_round(a) for a in (x0, w0, b0, g0))
    ok = (lambda a, b: oracle.rel_err(a, b) <= 1e-5) if dtype == "float32" else \
         (lambda a, b: oracle.max_abs_err(a, b) <= 2.0 ** -8 * np.abs(b).max() + 1e-3)
    dx_r, dw_r, db_r = oracle.fc_backward(x0, w0, g0)
    for resident in (False, True):
        kw = dict(device="gpu", dtype=dtype) if resident else {}
        x, w, b = opt.Tensor(x0, **kw), opt.Tensor(w0, **kw), opt.Tensor(b0, **kw)
        y = opt.fc(x, w, b, dtype=dtype)
        y.backward(opt.Tensor(g0, requires_grad=False, **kw))
        assert y.is_device == resident and x.grad.is_device == resident
        assert ok(y.numpy(), oracle.fc_forward(x0, w0, b0))
        assert ok(x.grad.numpy(), dx_r) and ok(w.grad.numpy(), dw_r) and ok(b.grad.numpy(), db_r)
    # single-value bias and use_bias=False, the two special cases of the reference op
    x, w, b1 = opt.Tensor(x0), opt.Tensor(w0), opt.Tensor(np.array([0.5], np.float32))
    y = opt.fc(x, w, b1, dtype=dtype)
    y.backward(opt.Tensor(g0, requires_grad=False))
    assert ok(y.numpy(), oracle.fc_forward(x0, w0, np.full(40, 0.5, np.float32)))
    assert b1.grad.shape == (1,) and ok(b1.grad.numpy(), oracle.fc_backward(x0, w0, g0, scalar_bias=True)[2])
    y = opt.fc(opt.Tensor(x0), opt.Tensor(w0), opt.Tensor(b0), use_bias=False, dtype=dtype)
    assert ok(y.numpy(), oracle.fc_forward(x0, w0))


def test_projection_attention_projection_block_on_device(opt, oracle, mods):
    """x -> FC (qkv) -> attention -> FC (out), every node device-resident bf16, against the same
    block built from this package's NumPy ops (the reference's way of writing it)."""
    rng = np.random.default_rng(21)
    B, H, S, D = 1, 2, 128, 64
    E = H * D
    r = lambda *shape, s=1.0: oracle.bf16_round((rng.standard_normal(shape) * s).astype(np.float32))
    x0, wq0, wk0, wv0, wo0 = r(B * S, E), r(E, E, s=E ** -0.5), r(E, E, s=E ** -0.5), r(E, E, s=E ** -0.5), r(E, E, s=E ** -0.5)
    bz0, g0 = np.zeros(E, np.float32), r(B * S, E)

    def heads(t):    # [B*S, H*D] -> [B,H,S,D]
        return opt.transpose(opt.reshape(t, (B, S, H, D)), (1, 2))

    # NumPy-backed graph (CPU): matmul + composed attention
    x, wq, wk, wv, wo = (opt.Tensor(a) for a in (x0, wq0, wk0, wv0, wo0))
    q, k, v = heads(x @ wq), heads(x @ wk), heads(x @ wv)
    o = opt.attention_composed(q, k, v, causal=True)
    y_ref = opt.reshape(opt.transpose(o, (1, 2)), (B * S, E)) @ wo
    y_ref.backward(opt.Tensor(g0, requires_grad=False))

    # device graph: the projections and attention run on the GPU; the head split/merge is a
    # layout change the device tensors do not offer, so q, k, v are produced per head instead
    kw = dict(device="gpu", dtype="bfloat16")
    xd, wod, bd = opt.Tensor(x0, **kw), opt.Tensor(wo0, **kw), opt.Tensor(bz0, **kw)
    outs = []
    wgrads = []
    for h in range(H):
        cols = slice(h * D, (h + 1) * D)
        wqh, wkh, wvh = (opt.Tensor(np.ascontiguousarray(w[:, cols]), **kw) for w in (wq0, wk0, wv0))
        bh = opt.Tensor(np.zeros(D, np.float32), **kw)
        qh, kh, vh = (opt.fc(xd, w, bh, use_bias=False) for w in (wqh, wkh, wvh))      # [S, D] each
        as4 = lambda t: opt.Tensor(mods[0].Tensor_bf16(t.realize_cached_data()).resize([1, 1, S, D]), **kw)
        oh = opt.attention(as4(qh), as4(kh), as4(vh), causal=True)
        assert oh.is_device
        outs.append(oh.numpy().reshape(S, D))
        wgrads.append((wqh, wkh, wvh))
    o_dev = np.concatenate(outs, axis=1)                                                 # [S, E]
    y = opt.fc(opt.Tensor(oracle.bf16_round(o_dev), **kw), wod, bd, use_bias=False)
    assert y.is_device
    tol = oracle.bf16_grad_tol
    assert oracle.max_abs_err(o_dev, np.transpose(o.numpy(), (0, 2, 1, 3)).reshape(B * S, E)) <= tol(o.numpy())
    assert oracle.max_abs_err(y.numpy(), y_ref.numpy()) <= tol(y_ref.numpy())
