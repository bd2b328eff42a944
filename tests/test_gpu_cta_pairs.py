"""The CTA-pair (clusters of two, tcgen05 cta_group::2) variants of the attention forward and of the
backward's dK/dV pass.  They are selected by environment switches, compute with the same MMA shapes per
row and the same accumulation order as the one-CTA kernels, and must therefore return the same bits;
one case each is also checked against the CPU oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

# (B, H, Hkv, S, L, causal): tile edges of the 512-row query blocks and the 256-key pairs, ragged sizes,
# an odd number of key tiles, more keys than queries, grouped heads
CASES = [(1, 1, 1, 512, 512, False), (1, 2, 2, 1024, 1024, True), (2, 3, 3, 700, 900, True), (2, 3, 3, 700, 900, False),
         (1, 4, 4, 130, 130, True), (1, 8, 2, 2048, 2048, True), (1, 4, 4, 1536, 4096, True), (1, 2, 2, 4096, 1664, False)]


def _inputs(B, H, Hkv, S, L, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h, n, s: (torch.randn((B, h, n, 128), generator=g, device="cuda") * s).bfloat16()
    return mk(H, S, 0.5), mk(Hkv, L, 0.5), mk(Hkv, L, 0.5), mk(H, S, 1.0)


@pytest.mark.parametrize("B,H,Hkv,S,L,causal", CASES)
def test_pair_forward_equals_one_cta_forward(tt, monkeypatch, B, H, Hkv, S, L, causal):
    q, k, v, _ = _inputs(B, H, Hkv, S, L, 3)
    monkeypatch.setenv("TT_FWD_PATH", "1cta")
    o1, l1 = tt.attention_forward(q, k, v, causal=causal)
    monkeypatch.setenv("TT_FWD_PATH", "2cta")
    o2, l2 = tt.attention_forward(q, k, v, causal=causal)
    tt.check_device_status()
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


@pytest.mark.parametrize("B,H,Hkv,S,L,causal", CASES)
def test_pair_dkv_pass_equals_one_cta_pass(tt, monkeypatch, B, H, Hkv, S, L, causal):
    q, k, v, do = _inputs(B, H, Hkv, S, L, 4)
    out, lse = tt.attention_forward(q, k, v, causal=causal)
    monkeypatch.setenv("TT_BWD_PATH", "two_pass")
    monkeypatch.setenv("TT_BWD_DKV", "1cta")
    one = tt.attention_backward(q, k, v, out, lse, do, causal=causal)
    monkeypatch.setenv("TT_BWD_DKV", "2cta")
    two = tt.attention_backward(q, k, v, out, lse, do, causal=causal)
    tt.check_device_status()
    for a, b in zip(one, two):
        assert torch.equal(a, b)


def test_pair_kernels_against_the_oracle(tt, oracle, monkeypatch):
    B, H, S = 1, 2, 640
    q, k, v, do = _inputs(B, H, H, S, S, 5)
    monkeypatch.setenv("TT_FWD_PATH", "2cta")
    monkeypatch.setenv("TT_BWD_PATH", "two_pass")
    monkeypatch.setenv("TT_BWD_DKV", "2cta")
    out, lse = tt.attention_forward(q, k, v, causal=True)
    dq, dk, dv = tt.attention_backward(q, k, v, out, lse, do, causal=True)
    tt.check_device_status()
    f = lambda t: t.float().cpu().numpy()
    o_ref, lse_ref = oracle.attention_forward(f(q), f(k), f(v), causal=True)
    assert oracle.max_abs_err(f(out), o_ref) <= 2e-2
    assert oracle.max_abs_err(lse.cpu().numpy(), lse_ref) <= 2e-2
    g_ref = oracle.attention_backward(f(q), f(k), f(v), f(do), causal=True)[2:]
    for got, ref, name in zip((dq, dk, dv), g_ref, ("dq", "dk", "dv")):
        assert oracle.max_abs_err(f(got), ref) <= oracle.bf16_grad_tol(ref), name
