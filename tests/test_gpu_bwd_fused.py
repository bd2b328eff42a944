"""The single-pass tensor-core backward (dK, dV and dQ from one launch, dQ through fp32 additions in
global memory) against the oracle and against the two-pass kernels on the same inputs.

Every case runs both kernels (`TT_BWD_PATH=fused|two_pass`); the single-pass dK and dV must repeat bit
for bit from call to call, its dQ to fp32 rounding."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _np(t):
    return t.detach().float().cpu().numpy()


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda", dtype=torch.bfloat16).contiguous()


CASES = [
    # B, H, Hkv, S, L, D, causal
    (1, 1, 1, 128, 128, 128, False),       # one tile pair
    (1, 2, 2, 256, 256, 128, True),
    (1, 2, 2, 384, 384, 64, True),
    (1, 1, 1, 300, 300, 128, True),        # ragged tail inside a tile
    (1, 2, 2, 130, 515, 64, True),         # L != S, bottom-right aligned diagonal
    (1, 1, 1, 257, 129, 128, False),       # one row / one key into a further tile
    (2, 1, 1, 1024, 1024, 128, True),      # 8 streamed tiles: every ring slot wraps several times
    (1, 1, 1, 1536, 1536, 64, False),
    (1, 4, 2, 200, 330, 128, True),        # grouped heads: two query heads stream into one key/value slice
    (2, 6, 1, 129, 129, 64, False),        # one key/value head for six query heads
    (1, 1, 1, 1, 77, 128, False),          # a single query
]


@pytest.mark.parametrize("B,H,Hkv,S,L,D,causal", CASES)
def test_fused_backward_vs_oracle_and_two_pass(tt, oracle, monkeypatch, B, H, Hkv, S, L, D, causal):
    q, _, _, do = oracle.make_inputs(41, B, H, S, L, D, sigma=0.6)
    _, k, v, _ = oracle.make_inputs(43, B, Hkv, S, L, D, sigma=0.6, with_do=False)
    qn, kn, vn, don = (oracle.bf16_round(x) for x in (q, k, v, do))
    o_r, lse_r, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(qn, kn, vn, don, causal)
    tq, tk, tv, tdo = (_dev(x) for x in (qn, kn, vn, don))
    out, lse = tt.attention_forward(tq, tk, tv, causal=causal)
    res = {}
    for path in ("fused", "two_pass"):
        monkeypatch.setenv("TT_BWD_PATH", path)
        res[path] = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal)
        tt.check_device_status()
        for got, ref, name in zip(res[path], (dq_r, dk_r, dv_r), ("dq", "dk", "dv")):
            err = oracle.max_abs_err(_np(got), ref)
            assert err <= oracle.bf16_grad_tol(ref), f"{path} {name}: {err}"
    # same mathematics, different rounding points (the single pass forms dS^T from the bf16 P^T it feeds to
    # the dV product) and a different order of the dQ sums: the two agree within two bf16 ulps
    for a, b, name in zip(res["fused"], res["two_pass"], ("dq", "dk", "dv")):
        ulp = 2.0 ** -7 * max(float(b.float().abs().max()), 1.0)
        assert float((a.float() - b.float()).abs().max()) <= 2 * ulp, name
    monkeypatch.setenv("TT_BWD_PATH", "fused")
    again = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal)
    tt.check_device_status()
    assert torch.equal(again[1], res["fused"][1]) and torch.equal(again[2], res["fused"][2])   # dK, dV: no atomics
    assert float((again[0].float() - res["fused"][0].float()).abs().max()) <= 2.0 ** -7 * max(float(dq_r.max()), 1.0)


def test_fused_backward_padded_keys(tt, oracle, monkeypatch):
    """Key padding lengths per batch entry: padded keys get zero dK, dV and add nothing to dQ."""
    monkeypatch.setenv("TT_BWD_PATH", "fused")
    B, H, S, L, D = 3, 2, 260, 260, 128
    lens = [260, 131, 5]
    q, k, v, do = (oracle.bf16_round(x) for x in oracle.make_inputs(47, B, H, S, L, D, sigma=0.6))
    tq, tk, tv, tdo = (_dev(x) for x in (q, k, v, do))
    tl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out, lse = tt.attention_forward(tq, tk, tv, causal=False, kv_lens=tl)
    dq, dk, dv = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=False, kv_lens=tl)
    tt.check_device_status()
    for b, n in enumerate(lens):
        o_r, _, dq_r, dk_r, dv_r = oracle.attention_backward(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n], do[b:b + 1], False)
        assert oracle.max_abs_err(_np(out[b:b + 1]), o_r) <= 2e-2
        assert oracle.max_abs_err(_np(dq[b:b + 1]), dq_r) <= oracle.bf16_grad_tol(dq_r)
        assert oracle.max_abs_err(_np(dk[b:b + 1, :, :n]), dk_r) <= oracle.bf16_grad_tol(dk_r)
        assert oracle.max_abs_err(_np(dv[b:b + 1, :, :n]), dv_r) <= oracle.bf16_grad_tol(dv_r)
        assert float(dk[b, :, n:].float().abs().max()) == 0.0 if n < L else True
        assert float(dv[b, :, n:].float().abs().max()) == 0.0 if n < L else True


def test_fused_backward_many_items_and_reuse(tt, oracle, monkeypatch):
    """More work items than SMs, several per CTA, workspace reused across calls (the fp32 dQ accumulator
    is cleared by every call): three calls in a row agree with the oracle on sampled slices."""
    monkeypatch.setenv("TT_BWD_PATH", "fused")
    B, H, S, D = 6, 40, 384, 128
    g = torch.Generator(device="cuda").manual_seed(78)
    mk = lambda s: (torch.randn((B, H, S, D), generator=g, device="cuda") * s).to(torch.bfloat16)
    q, k, v, do = mk(0.5), mk(0.5), mk(0.7), mk(1.0)
    out, lse = tt.attention_forward(q, k, v, causal=True)
    import ctypes
    d = tt.capi.make_desc(B, H, S, S, D, tt.capi.TT_BF16, True, None)
    ws = torch.empty(int(tt.capi.lib.tt_attn_bwd_workspace_bytes(ctypes.byref(d))), dtype=torch.uint8, device="cuda")
    ws.fill_(0x7f)        # garbage on entry must not matter
    for _ in range(3):
        dq, dk, dv = tt.attention_backward(q, k, v, out, lse, do, causal=True, workspace=ws)
    tt.check_device_status()
    f = lambda t, b, h: t[b:b + 1, h:h + 1].float().cpu().numpy()
    for b, h in ((0, 0), (3, 17), (5, 39)):
        _, _, dq_r, dk_r, dv_r = oracle.attention_backward(f(q, b, h), f(k, b, h), f(v, b, h), f(do, b, h), True)
        for got, ref in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
            assert oracle.max_abs_err(f(got, b, h), ref) <= oracle.bf16_grad_tol(ref)
