"""GPU parity of the row-softmax kernels (forward and backward) through the C ABI against the
oracle and the golden fixtures written by the reference's own NumPy ops.
Tolerance: fp32 max|a-b|/max|b| <= 1e-5; bf16 rows max|a-b| <= 2^-8 (one bf16 ulp below 1)."""
import glob
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "softmax_rows", "*.npz")))


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    return torch


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_softmax_golden(tt, oracle, torch_cuda, path):
    torch = torch_cuda
    g = np.load(path)
    x = torch.from_numpy(g["x"]).cuda()
    y = tt.softmax_forward(x)
    assert oracle.rel_err(y.cpu().numpy(), g["y"]) <= 1e-5
    dx = tt.softmax_backward(torch.from_numpy(g["y"]).cuda(), torch.from_numpy(g["dy"]).cuda())
    assert oracle.rel_err(dx.cpu().numpy(), g["dx"]) <= 1e-5


# every dispatch bucket of the launcher and its edges: warp rows (<=1024), CTA rows (<=16384), streamed
@pytest.mark.parametrize("cols", [1, 7, 32, 33, 64, 100, 129, 256, 500, 513, 1024, 1025, 2048, 3000, 4097, 8192,
                                  10000, 16384, 16385, 40000])
def test_softmax_all_row_lengths_fp32(tt, oracle, torch_cuda, cols):
    torch = torch_cuda
    rng = np.random.default_rng(cols)
    rows = 19 if cols < 5000 else 5
    x = (rng.standard_normal((rows, cols)) * 4).astype(np.float32)
    x[0, :] = 1e4                      # constant row, large magnitude: needs the max shift
    x[1, cols // 2] = 80.0             # one dominant entry
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    y = tt.softmax_forward(torch.from_numpy(x).cuda()).cpu().numpy()
    want = oracle.softmax_rows(x)
    assert np.isfinite(y).all() and oracle.rel_err(y, want) <= 1e-5
    assert np.allclose(y.sum(-1), 1.0, atol=1e-5)
    dx = tt.softmax_backward(torch.from_numpy(want).cuda(), torch.from_numpy(dy).cuda()).cpu().numpy()
    assert oracle.rel_err(dx, oracle.softmax_rows_backward(x, dy)) <= 1e-5


@pytest.mark.parametrize("shape", [(3, 5, 40), (2, 2, 8, 1000), (4, 3000)])
def test_softmax_bf16_and_leading_axes(tt, oracle, torch_cuda, shape):
    torch = torch_cuda
    rng = np.random.default_rng(len(shape))
    x = oracle.bf16_round((rng.standard_normal(shape) * 2).astype(np.float32))
    dy = oracle.bf16_round(rng.standard_normal(shape).astype(np.float32))
    xb = torch.from_numpy(x).cuda().bfloat16()
    y = tt.softmax_forward(xb)
    assert y.dtype == torch.bfloat16 and y.shape == xb.shape
    want = oracle.softmax_rows(x)
    assert oracle.max_abs_err(y.float().cpu().numpy(), want) <= 2.0 ** -8
    yb = oracle.bf16_round(want)
    dx = tt.softmax_backward(torch.from_numpy(yb).cuda().bfloat16(), torch.from_numpy(dy).cuda().bfloat16())
    ref = yb.astype(np.float64) * (dy - np.sum(dy.astype(np.float64) * yb, -1, keepdims=True))
    assert oracle.max_abs_err(dx.float().cpu().numpy(), ref) <= 2.0 ** -8 * max(1.0, np.abs(ref).max())


def test_softmax_in_place_empty_and_errors(tt, torch_cuda):
    torch = torch_cuda
    x = torch.randn(64, 777, device="cuda")
    want = torch.softmax(x, -1)
    tt.softmax_forward(x, out=x)                     # every thread reads its row before any write
    assert torch.allclose(x, want, atol=1e-6)
    e = torch.empty(0, 12, device="cuda")
    assert tt.softmax_forward(e).shape == (0, 12)
    with pytest.raises(ValueError):
        tt.softmax_forward(torch.randn(4, 4))        # CPU tensor: no CPU path
    with pytest.raises(ValueError):
        tt.softmax_backward(x, x[:, :5].contiguous())
    from importlib import import_module
    capi = import_module(tt.__name__ + ".capi")
    assert capi.lib.tt_softmax_fwd(None, None, 1, 4, capi.TT_F32, None) == capi.TT_ERR_NULL
    p = torch.empty(8, device="cuda").data_ptr()
    import ctypes
    assert capi.lib.tt_softmax_fwd(ctypes.c_void_p(p), ctypes.c_void_p(p), 2, 0, capi.TT_F32, None) == capi.TT_ERR_BAD_SHAPE
    assert capi.lib.tt_softmax_fwd(ctypes.c_void_p(p), ctypes.c_void_p(p), 2, 4, 9, None) == capi.TT_ERR_BAD_DTYPE


def test_softmax_full_size_properties(tt, torch_cuda):
    """Score-matrix sized input (1 GiB fp32): rows sum to one, shift invariance, and the backward
    is orthogonal to the all-ones direction (rows of dx sum to zero)."""
    torch = torch_cuda
    rows, cols = 262144, 1024
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(rows, cols, device="cuda", generator=g) * 3
    y = tt.softmax_forward(x)
    assert float((y.sum(-1) - 1).abs().max()) <= 1e-5
    y2 = tt.softmax_forward(x + 7.5)
    assert float((y - y2).abs().max()) <= 1e-5
    dy = torch.randn(rows, cols, device="cuda", generator=g)
    dx = tt.softmax_backward(y, dy)
    assert float(dx.sum(-1).abs().max()) <= 1e-4
    idx = torch.arange(0, rows, 4099, device="cuda")
    assert torch.allclose(y[idx], torch.softmax(x[idx], -1), atol=1e-6)
