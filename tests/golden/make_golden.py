"""Generate the golden attention fixtures by EXECUTING the reference's own ops.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/reference

It imports the reference's `operators.py` (NumPy-backed autograd ops and reverse sweep),
composes attention exactly as `oracle/attention_oracle.py` documents, calls
`O.backward(dO)` and stores inputs and outputs as `.npz` files next to this script.
The reference's two pybind modules (`myTensor`, `myLayer`) are only *named* at import
time by `operators.py`; none of the ops on this path calls into them, so inert
stand-in modules are registered instead of building them.

The fixtures travel with the repository; the reference checkout does not, so tests
read only the `.npz` files.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle.attention_oracle import make_inputs, causal_mask, MASK_VALUE  # noqa: E402

# name, B, H, S, L, D, causal, sigma, seed
CASES = [
    ("cfg1_f32_b2h4s64d32", 2, 4, 64, 64, 32, False, 1.0, 0),       # benchmark configuration 1
    ("causal_b1h2s48d32", 1, 2, 48, 48, 32, True, 1.0, 1),
    ("causal_ragged_b1h2s40l72d64", 1, 2, 40, 72, 64, True, 0.5, 2),  # L != S, bottom-right aligned
    ("cross_b1h3s17l33d16", 1, 3, 17, 33, 16, False, 1.0, 3),
    ("decode_b2h2s1l96d64", 2, 2, 1, 96, 64, False, 1.0, 4),
    ("causal_b1h1s130d128", 1, 1, 130, 130, 128, True, 0.5, 5),     # crosses a 128-row tile edge
]


def load_reference_ops(ref_root: str):
    opt = os.path.join(ref_root, "Task3", "Tinytensor", "optimizer")
    if not os.path.isdir(opt):
        raise SystemExit(f"reference optimizer directory not found: {opt}")
    mt = types.ModuleType("myTensor")
    mt.Tensor_float = type("Tensor_float", (), {})
    mt.Tensor_int = type("Tensor_int", (), {})
    sys.modules["myTensor"] = mt
    sys.modules["myLayer"] = types.ModuleType("myLayer")
    sys.path.insert(0, opt)
    import operators as ops  # the reference's module, unmodified
    return ops


def reference_attention(ops, q, k, v, do, causal, scale):
    B, H, S, D = q.shape
    L = k.shape[2]
    Q = ops.Tensor(q); K = ops.Tensor(k); V = ops.Tensor(v)
    s = (Q @ ops.transpose(K)) * float(scale)
    if causal:
        m = np.ascontiguousarray(np.broadcast_to(causal_mask(S, L), (B, H, S, L)))
        s = s + ops.Tensor(m, requires_grad=False)
    e = ops.exp(s)
    den = ops.broadcast_to(ops.reshape(ops.summation(e, axes=(3,)), (B, H, S, 1)), (B, H, S, L))
    O = (e / den) @ V
    O.backward(ops.Tensor(do, requires_grad=False))
    return O.numpy(), Q.grad.numpy(), K.grad.numpy(), V.grad.numpy()


# name, rows-shape, cols, sigma, seed  (row softmax: the adjacent native op, see oracle.softmax_rows)
SOFTMAX_CASES = [
    ("rows_6x10", (6,), 10, 1.0, 20),          # the classifier shape the reference uses it on
    ("rows_3x5x33", (3, 5), 33, 3.0, 21),
    ("rows_4x1025", (4,), 1025, 1.0, 22),
    ("rows_2x2500", (2,), 2500, 2.0, 23),
]


def reference_softmax(ops, x, dy):
    """Forward: the reference's own NumPy row softmax (Softmaxloss.compute keeps it in
    `.softmax`); it is defined for 2-D input, so leading axes are flattened as the native
    SoftmaxForward does.  Backward: the reference's reverse sweep over exp(x - max) / sum."""
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    op = ops.Softmaxloss(ops.Tensor(np.zeros(x2.shape[0], dtype=np.int64), requires_grad=False))
    op.compute(x2)
    y = op.softmax.reshape(x.shape)
    X = ops.Tensor(x2)
    shift = ops.Tensor(np.ascontiguousarray(np.broadcast_to(-np.max(x2, axis=1, keepdims=True), x2.shape)),
                       requires_grad=False)
    e = ops.exp(X + shift)
    den = ops.broadcast_to(ops.reshape(ops.summation(e, axes=(1,)), (x2.shape[0], 1)), x2.shape)
    Y = e / den
    Y.backward(ops.Tensor(dy.reshape(-1, cols), requires_grad=False))
    assert np.array_equal(Y.numpy(), y.reshape(-1, cols))
    return y, X.grad.numpy().reshape(x.shape)


# name, rows, in_features, out_features, seed  (fully connected layer, see oracle.fc_forward)
FC_CASES = [
    ("fc_32x784x100", 32, 784, 100, 30),       # the first layer of the reference's MNIST model
    ("fc_7x10x3", 7, 10, 3, 31),
    ("fc_130x72x264", 130, 72, 264, 32),       # crosses the 128-row and 256-column tile edges
]


def reference_fc(ops, x, w, b, dy):
    """y = x @ w + broadcast(b) with the reference's ops and its reverse sweep for the gradients."""
    X, W, Bv = ops.Tensor(x), ops.Tensor(w), ops.Tensor(b)
    Y = X @ W + ops.broadcast_to(ops.reshape(Bv, (1, b.shape[0])), (x.shape[0], w.shape[1]))
    Y.backward(ops.Tensor(dy, requires_grad=False))
    return Y.numpy(), X.grad.numpy(), W.grad.numpy(), Bv.grad.numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TT_REFERENCE_ROOT"), required="TT_REFERENCE_ROOT" not in os.environ,
                    help="checkout of the reference project (or set TT_REFERENCE_ROOT)")
    args = ap.parse_args()
    ops = load_reference_ops(args.reference)
    for name, B, H, S, L, D, causal, sigma, seed in CASES:
        q, k, v, do = make_inputs(seed, B, H, S, L, D, sigma=sigma)
        scale = 1.0 / float(np.sqrt(float(D)))
        o, dq, dk, dv = reference_attention(ops, q, k, v, do, causal, scale)
        for t in (o, dq, dk, dv):
            assert t.dtype == np.float32, t.dtype
        path = os.path.join(HERE, name + ".npz")
        np.savez(path, q=q, k=k, v=v, do=do, o=o, dq=dq, dk=dk, dv=dv,
                 causal=np.int32(causal), scale=np.float32(scale), seed=np.int32(seed),
                 sigma=np.float32(sigma))
        print(f"{name}: wrote {os.path.getsize(path)/1024:.0f} KiB  |O|max={np.abs(o).max():.4f}")
    os.makedirs(os.path.join(HERE, "fc"), exist_ok=True)
    for name, rows, fin, fout, seed in FC_CASES:
        rng = np.random.Generator(np.random.PCG64([seed, rows]))
        x = rng.standard_normal((rows, fin)).astype(np.float32)
        w = (rng.standard_normal((fin, fout)) / np.sqrt(fin)).astype(np.float32)
        b = rng.standard_normal((fout,)).astype(np.float32)
        dy = rng.standard_normal((rows, fout)).astype(np.float32)
        y, dx, dw, db = reference_fc(ops, x, w, b, dy)
        assert all(t.dtype == np.float32 for t in (y, dx, dw, db)) and db.shape == (fout,)
        path = os.path.join(HERE, "fc", name + ".npz")
        np.savez(path, x=x, w=w, b=b, dy=dy, y=y, dx=dx, dw=dw, db=db)
        print(f"fc/{name}: wrote {os.path.getsize(path)/1024:.0f} KiB")
    os.makedirs(os.path.join(HERE, "softmax_rows"), exist_ok=True)
    for name, lead, cols, sigma, seed in SOFTMAX_CASES:
        rng = np.random.Generator(np.random.PCG64([seed, cols]))
        x = (rng.standard_normal(lead + (cols,)) * sigma).astype(np.float32)
        dy = rng.standard_normal(lead + (cols,)).astype(np.float32)
        y, dx = reference_softmax(ops, x, dy)
        assert y.dtype == np.float32 and dx.dtype == np.float32
        path = os.path.join(HERE, "softmax_rows", name + ".npz")
        np.savez(path, x=x, dy=dy, y=y, dx=dx)
        print(f"softmax_rows/{name}: wrote {os.path.getsize(path)/1024:.0f} KiB")


if __name__ == "__main__":
    main()
