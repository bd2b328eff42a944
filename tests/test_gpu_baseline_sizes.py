"""GPU parity at the benchmark's own sizes: forward AND backward of configurations 2, 3 and 5 and the
full-size decode of configuration 4, through the C ABI, against the CPU oracle.

The oracle cannot hold all slices of these shapes, so each test runs the whole launch on the GPU and
compares sampled (batch, head) slices -- the first, the last and seeded-random ones -- in full: O, lse,
dQ, dK and dV of every row of the slice.  Long slices go through the oracle in blocks of query rows
(`attention_backward_chunked`: rows are independent given K and V, dK and dV are summed over blocks).

Tolerances: O and lse 2e-2 absolute; gradients `oracle.bf16_grad_tol` (2e-2 absolute while the
reference stays within 2.56, one bf16 ulp of its largest value on top beyond that).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2


def _np(t):
    return t.detach().float().cpu().numpy()


def _inputs(B, H, S, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda s: (torch.randn((B, H, S, D), generator=g, device="cuda") * s).to(torch.bfloat16)
    return mk(0.5), mk(0.5), mk(0.5), mk(1.0)


def _sampled_slices(B, H, seed, n_random=2):
    rng = np.random.default_rng(seed)
    picks = [(0, 0), (B - 1, H - 1)]
    while len(picks) < 2 + n_random and len(picks) < B * H:
        c = (int(rng.integers(B)), int(rng.integers(H)))
        if c not in picks:
            picks.append(c)
    return picks


def _check_slice(oracle, tensors, b, h, tag, chunk=1024):
    q, k, v, do, out, lse, dq, dk, dv = tensors
    o_r, lse_r, dq_r, dk_r, dv_r = oracle.attention_backward_chunked(
        _np(q[b, h]), _np(k[b, h]), _np(v[b, h]), _np(do[b, h]), causal=True, chunk=chunk)
    assert oracle.max_abs_err(_np(out[b, h]), o_r) <= BF16_TOL, f"{tag} slice ({b},{h}) o"
    assert oracle.max_abs_err(_np(lse[b, h]), lse_r) <= 2e-2, f"{tag} slice ({b},{h}) lse"
    for got, ref, name in ((dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
        err = oracle.max_abs_err(_np(got[b, h]), ref)
        assert err <= oracle.bf16_grad_tol(ref), f"{tag} slice ({b},{h}) {name}: {err} (max |ref| {np.abs(ref).max()})"


def _run(tt, q, k, v, do):
    out, lse = tt.attention_forward(q, k, v, causal=True)
    dq, dk, dv = tt.attention_backward(q, k, v, out, lse, do, causal=True)
    tt.check_device_status()
    for t in (out, lse, dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    return out, lse, dq, dk, dv


def test_config3_forward_backward_sampled_slices(tt, oracle):
    """Configuration 3, [4,32,4096,128] causal: 32 key tiles per slice, so the launch runs the two-phase
    item order with 8 light tiles per slice, which no small case reaches."""
    B, H, S, D = 4, 32, 4096, 128
    q, k, v, do = _inputs(B, H, S, D, 303)
    res = _run(tt, q, k, v, do)
    for b, h in _sampled_slices(B, H, 3):
        _check_slice(oracle, (q, k, v, do) + res, b, h, "cfg3")


def test_config2_forward_backward_sampled_slices(tt, oracle):
    """Configuration 2, [8,16,1024,64] causal: the head dim 64 instantiations at their benchmark shape."""
    B, H, S, D = 8, 16, 1024, 64
    q, k, v, do = _inputs(B, H, S, D, 202)
    res = _run(tt, q, k, v, do)
    for b, h in _sampled_slices(B, H, 2):
        _check_slice(oracle, (q, k, v, do) + res, b, h, "cfg2")


def test_config5_two_heads_forward_backward(tt, oracle):
    """Configuration 5's slice shape (S = 32768, D = 128, causal) on two heads: every row of head 1
    against the row-chunked oracle, head 0 on its first and last 128-row blocks (forward) and its
    last key block (dK, dV of the keys only the last queries see)."""
    S, D = 32768, 128
    q, k, v, do = _inputs(1, 2, S, D, 505)
    res = _run(tt, q, k, v, do)
    out, lse, dq, dk, dv = res
    _check_slice(oracle, (q, k, v, do) + res, 0, 1, "cfg5")
    kn, vn = _np(k[0, 0]), _np(v[0, 0])
    for row0 in (0, S - 128):
        o_r, lse_r, dq_r, dk_p, dv_p, n = oracle.attention_backward_rows(
            _np(q[0, 0, row0:row0 + 128]), _np(do[0, 0, row0:row0 + 128]), kn, vn, row0, S, causal=True)
        assert oracle.max_abs_err(_np(out[0, 0, row0:row0 + 128]), o_r) <= BF16_TOL
        assert oracle.max_abs_err(_np(dq[0, 0, row0:row0 + 128]), dq_r) <= oracle.bf16_grad_tol(dq_r)
        if row0 == S - 128:      # the last 128 keys receive gradient from these rows only
            assert oracle.max_abs_err(_np(dk[0, 0, row0:]), dk_p[row0:]) <= oracle.bf16_grad_tol(dk_p[row0:])
            assert oracle.max_abs_err(_np(dv[0, 0, row0:]), dv_p[row0:]) <= oracle.bf16_grad_tol(dv_p[row0:])


def test_config4_full_size_decode(tt, oracle):
    """Configuration 4 in full: Q [64,32,1,128], K,V [64,32,8192,128] -- 2^31 elements (4.3 GB) per
    tensor: one more than a 32-bit signed index holds, and every slice of the second half of the batch
    sits behind a 2^32-byte offset.  The last slice (whose last element has index 2^31 - 1), slices either
    side of the 2^32-byte line and the first one are compared with the oracle; all outputs must be
    finite."""
    B, H, L, D = 64, 32, 8192, 128
    g = torch.Generator(device="cuda").manual_seed(404)
    q = torch.randn((B, H, 1, D), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.empty((B, H, L, D), dtype=torch.bfloat16, device="cuda")
    v = torch.empty((B, H, L, D), dtype=torch.bfloat16, device="cuda")
    for b in range(B):           # filled batch entry by batch entry: no 8.6 GB fp32 temporary
        k[b] = torch.randn((H, L, D), generator=g, device="cuda").to(torch.bfloat16)
        v[b] = torch.randn((H, L, D), generator=g, device="cuda").to(torch.bfloat16)
    out, lse = tt.attention_decode(q, k, v)
    tt.check_device_status()
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    for b, h in ((B - 1, H - 1), (B // 2, 7), (0, 0), (B // 2 - 1, H - 1)):
        o_r, lse_r = oracle.attention_forward(_np(q[b:b + 1, h:h + 1]), _np(k[b:b + 1, h:h + 1]), _np(v[b:b + 1, h:h + 1]), False)
        assert oracle.max_abs_err(_np(out[b:b + 1, h:h + 1]), o_r) <= BF16_TOL, (b, h)
        assert oracle.max_abs_err(_np(lse[b:b + 1, h:h + 1]), lse_r) <= 1e-3, (b, h)
    del k, v
    torch.cuda.empty_cache()
