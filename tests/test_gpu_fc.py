"""GPU parity of the fully connected layer (tcgen05 GEMM kernel and the fp32 SIMT kernel) through
the C ABI against the oracle and the fixtures written by the reference's own ops.
Tolerances: fp32 max|a-b|/max|b| <= 1e-5; bf16 (inputs rounded to bf16, fp32 accumulation, bf16
output) max|a-b| <= 2^-8 * max|ref| + 1e-3, i.e. one output rounding."""
import glob
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "fc", "*.npz")))


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    return torch


def bf16_close(oracle, got, ref):
    return oracle.max_abs_err(got, ref) <= 2.0 ** -8 * np.abs(ref).max() + 1e-3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_fc_fp32_matches_reference(tt, oracle, torch_cuda, path):
    torch = torch_cuda
    g = np.load(path)
    x, w, b, dy = (torch.from_numpy(g[n]).cuda() for n in ("x", "w", "b", "dy"))
    y = tt.fc_forward(x, w, b)
    dx, dw, db = tt.fc_backward(x, w, dy)
    for got, name in ((y, "y"), (dx, "dx"), (dw, "dw"), (db, "db")):
        assert oracle.rel_err(got.cpu().numpy(), g[name]) <= 1e-5, name


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_fc_bf16_matches_oracle_on_fixture_inputs(tt, oracle, torch_cuda, path):
    torch = torch_cuda
    g = np.load(path)
    xn, wn, bn, dyn = (oracle.bf16_round(g[n]) for n in ("x", "w", "b", "dy"))
    x, w, b, dy = (torch.from_numpy(a).cuda().bfloat16() for a in (xn, wn, bn, dyn))
    y = tt.fc_forward(x, w, b)
    dx, dw, db = tt.fc_backward(x, w, dy)
    dx_r, dw_r, db_r = oracle.fc_backward(xn, wn, dyn)
    for got, ref, name in ((y, oracle.fc_forward(xn, wn, bn), "y"), (dx, dx_r, "dx"), (dw, dw_r, "dw"), (db, db_r, "db")):
        assert bf16_close(oracle, got.float().cpu().numpy(), ref), name


# tensor-core path: shapes around the 128 x 256 x 64 tile edges, several tiles per CTA ring turn,
# more tiles than SMs (persistent loop), ragged rows, K smaller than one stage
@pytest.mark.parametrize("rows,fin,fout", [(128, 64, 256), (1, 8, 8), (129, 72, 264), (300, 200, 520), (640, 1032, 24),
                                           (2500, 136, 776), (4096, 512, 4104), (37, 4096, 512)])
def test_fc_tensor_core_shapes(tt, oracle, torch_cuda, rows, fin, fout):
    torch = torch_cuda
    assert tt.capi.lib.tt_fc_path(rows, fin, fout, tt.capi.TT_BF16) == 1
    rng = np.random.default_rng(rows * 7 + fout)
    xn = oracle.bf16_round(rng.standard_normal((rows, fin)).astype(np.float32))
    wn = oracle.bf16_round((rng.standard_normal((fin, fout)) / np.sqrt(fin)).astype(np.float32))
    bn = oracle.bf16_round(rng.standard_normal(fout).astype(np.float32))
    dyn = oracle.bf16_round(rng.standard_normal((rows, fout)).astype(np.float32))
    x, w, b, dy = (torch.from_numpy(a).cuda().bfloat16() for a in (xn, wn, bn, dyn))
    y = tt.fc_forward(x, w, b)
    dx, dw, db = tt.fc_backward(x, w, dy)
    tt.check_device_status()
    dx_r, dw_r, db_r = oracle.fc_backward(xn, wn, dyn)
    for got, ref, name in ((y, oracle.fc_forward(xn, wn, bn), "y"), (dx, dx_r, "dx"), (dw, dw_r, "dw"), (db, db_r, "db")):
        assert bf16_close(oracle, got.float().cpu().numpy(), ref), name
    y0 = tt.fc_forward(x, w)                                   # no bias
    assert bf16_close(oracle, y0.float().cpu().numpy(), oracle.fc_forward(xn, wn))


def test_fc_unaligned_bf16_and_forced_simt_agree(tt, oracle, torch_cuda, monkeypatch):
    torch = torch_cuda
    rng = np.random.default_rng(9)
    xn = oracle.bf16_round(rng.standard_normal((70, 33)).astype(np.float32))
    wn = oracle.bf16_round(rng.standard_normal((33, 21)).astype(np.float32))
    dyn = oracle.bf16_round(rng.standard_normal((70, 21)).astype(np.float32))
    assert tt.capi.lib.tt_fc_path(70, 33, 21, tt.capi.TT_BF16) == 0          # pitches not multiples of 16 B
    x, w, dy = (torch.from_numpy(a).cuda().bfloat16() for a in (xn, wn, dyn))
    y = tt.fc_forward(x, w)
    dx, dw, db = tt.fc_backward(x, w, dy, scalar_bias=True)
    dx_r, dw_r, db_r = oracle.fc_backward(xn, wn, dyn, scalar_bias=True)
    for got, ref in ((y, oracle.fc_forward(xn, wn)), (dx, dx_r), (dw, dw_r), (db, db_r)):
        assert bf16_close(oracle, got.float().cpu().numpy(), ref)
    # same aligned problem through both kernels: equal up to the output rounding
    x2 = torch.randn(256, 128, device="cuda").bfloat16(); w2 = (torch.randn(128, 512, device="cuda") / 11).bfloat16()
    y_tc = tt.fc_forward(x2, w2)
    monkeypatch.setenv("TT_FC_PATH", "simt")
    assert tt.capi.lib.tt_fc_path(256, 128, 512, tt.capi.TT_BF16) == 0
    y_simt = tt.fc_forward(x2, w2)
    monkeypatch.delenv("TT_FC_PATH")
    assert float((y_tc.float() - y_simt.float()).abs().max()) <= 2.0 ** -7 * float(y_simt.float().abs().max())


def test_fc_leading_axes_empty_and_errors(tt, oracle, torch_cuda):
    torch = torch_cuda
    x = torch.randn(2, 3, 40, 64, device="cuda").bfloat16(); w = torch.randn(64, 128, device="cuda").bfloat16()
    y = tt.fc_forward(x, w)
    assert tuple(y.shape) == (2, 3, 40, 128)
    ref = oracle.fc_forward(x.float().cpu().numpy(), w.float().cpu().numpy())
    assert bf16_close(oracle, y.float().cpu().numpy(), ref)
    e = torch.empty(0, 64, device="cuda").bfloat16()
    assert tuple(tt.fc_forward(e, w).shape) == (0, 128)
    dx, dw, db = tt.fc_backward(e, w, torch.empty(0, 128, device="cuda").bfloat16())
    assert float(dw.float().abs().max()) == 0.0 and float(db.float().abs().max()) == 0.0
    with pytest.raises(ValueError):
        tt.fc_forward(x, torch.randn(65, 128, device="cuda").bfloat16())
    with pytest.raises(ValueError):
        tt.fc_forward(x.float(), w)
    with pytest.raises(ValueError):
        tt.fc_forward(x.cpu(), w.cpu())                      # no CPU path
    c = tt.capi
    assert c.lib.tt_fc_fwd(None, None, None, None, 4, 8, 8, c.TT_BF16, None) == c.TT_ERR_NULL
    assert c.lib.tt_fc_fwd(None, None, None, None, 4, 0, 8, c.TT_BF16, None) == c.TT_ERR_BAD_SHAPE
    import ctypes
    p = ctypes.c_void_p(w.data_ptr())
    assert c.lib.tt_fc_bwd(p, p, p, None, None, p, 0, 4, 8, 8, c.TT_BF16, None, 0, None) == c.TT_ERR_WORKSPACE


def test_fc_projection_size_properties(tt, torch_cuda):
    """The projection of benchmark configuration 3 (tokens 16384, width 4096), where a float64 oracle pass
    is too slow: linearity in x, agreement of dW with the forward kernel run on transposed data,
    and spot rows against float64."""
    torch = torch_cuda
    g = torch.Generator(device="cuda").manual_seed(3)
    M, K, N = 16384, 4096, 4096
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(K, N, device="cuda", generator=g) / 64).bfloat16()
    dy = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    y = tt.fc_forward(x, w)
    y2 = tt.fc_forward(x * 2, w)                              # exact in bf16: scaling by two
    assert torch.equal(y2.float(), y.float() * 2)
    rows = torch.tensor([0, 1, 127, 128, 8191, 16383], device="cuda")
    ref = x[rows].double() @ w.double()
    assert float((y[rows].double() - ref).abs().max()) <= 2.0 ** -8 * float(ref.abs().max()) + 1e-3
    dx, dw, _ = tt.fc_backward(x, w, dy, need_db=False)
    dw_alt = tt.fc_forward(x.t().contiguous(), dy)            # x^T dy through the forward layout
    assert float((dw.float() - dw_alt.float()).abs().max()) <= 2.0 ** -7 * float(dw_alt.float().abs().max())
    refx = dy[rows].double() @ w.double().t()
    assert float((dx[rows].double() - refx).abs().max()) <= 2.0 ** -8 * float(refx.abs().max()) + 1e-3
    tt.check_device_status()


# the CTA-pair kernel (clusters of two, 256x256 tiles) is chosen by size; force each kernel on shapes
# around the pair tile's edges and compare both with the oracle
@pytest.mark.parametrize("path", ["1cta", "2cta"])
@pytest.mark.parametrize("rows,fin,fout", [(256, 64, 256), (257, 72, 264), (300, 200, 520), (130, 4096, 512),
                                           (2500, 136, 776), (4096, 512, 4104)])
def test_fc_both_tensor_core_kernels(tt, oracle, torch_cuda, monkeypatch, path, rows, fin, fout):
    torch = torch_cuda
    monkeypatch.setenv("TT_FC_PATH", path)
    rng = np.random.default_rng(rows * 11 + fout)
    xn = oracle.bf16_round(rng.standard_normal((rows, fin)).astype(np.float32))
    wn = oracle.bf16_round((rng.standard_normal((fin, fout)) / np.sqrt(fin)).astype(np.float32))
    bn = oracle.bf16_round(rng.standard_normal(fout).astype(np.float32))
    dyn = oracle.bf16_round(rng.standard_normal((rows, fout)).astype(np.float32))
    x, w, b, dy = (torch.from_numpy(a).cuda().bfloat16() for a in (xn, wn, bn, dyn))
    y = tt.fc_forward(x, w, b)
    dx, dw, db = tt.fc_backward(x, w, dy)
    tt.check_device_status()
    dx_r, dw_r, db_r = oracle.fc_backward(xn, wn, dyn)
    for got, ref, name in ((y, oracle.fc_forward(xn, wn, bn), "y"), (dx, dx_r, "dx"), (dw, dw_r, "dw"), (db, db_r, "db")):
        assert bf16_close(oracle, got.float().cpu().numpy(), ref), name


def test_fc_large_shape_takes_the_pair_kernel_and_matches(tt, oracle, torch_cuda):
    """[8192,1024]x[1024,2048] has 256 pair tiles (>= the SM count): the size rule picks the CTA-pair kernel.
    Both kernels accumulate each output in fp32 over K in the same order, so they agree bit for bit."""
    torch = torch_cuda
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(8192, 1024, device="cuda", generator=g).bfloat16()
    w = (torch.randn(1024, 2048, device="cuda", generator=g) / 32).bfloat16()
    dy = torch.randn(8192, 2048, device="cuda", generator=g).bfloat16()
    got = (tt.fc_forward(x, w),) + tuple(tt.fc_backward(x, w, dy))[:2]
    tt.check_device_status()
    os.environ["TT_FC_PATH"] = "1cta"
    try:
        one = (tt.fc_forward(x, w),) + tuple(tt.fc_backward(x, w, dy))[:2]
    finally:
        del os.environ["TT_FC_PATH"]
    for a, b in zip(got, one):
        assert torch.equal(a, b)
    ref = x[:256].float() @ w.float()
    assert bf16_close(oracle, got[0][:256].float().cpu().numpy(), ref.cpu().numpy())
