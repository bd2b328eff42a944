"""Packed variable-length batches (`tt_attn_fwd_varlen` / `tt_attn_bwd_varlen`): token-major
`[total_tokens, H, D]` tensors with cumulative sequence lengths.  The oracle is the reference's composition
(optimizer/operators.py:194-199, 234-242, 289-298, 323-340, 388-408, 416-429, 464-470 and its reverse sweep,
optimizer/autodiff.py:33-61) applied to each sequence on its own: `oracle.attention_backward_grouped` in a loop.
Lengths sit around the 128/256 tile edges; one sequence is empty."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _pack(oracle, seed, lens_q, lens_k, H, Hkv, D):
    rng = np.random.default_rng(seed)
    mk = lambda n, h, s: oracle.bf16_round((rng.standard_normal((n, h, D), dtype=np.float32) * s))
    tq, tk = int(sum(lens_q)), int(sum(lens_k))
    return mk(tq, H, 0.6), mk(tk, Hkv, 0.6), mk(tk, Hkv, 0.6), mk(tq, H, 1.0)


def _oracle_packed(oracle, q, k, v, do, lens_q, lens_k, causal):
    H = q.shape[1]
    out, dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    lse = np.full((H, q.shape[0]), -np.inf, np.float32)
    cq = np.concatenate([[0], np.cumsum(lens_q)]); ck = np.concatenate([[0], np.cumsum(lens_k)])
    for b, (sq, sk) in enumerate(zip(lens_q, lens_k)):
        if sq == 0 or sk == 0:
            continue                     # no queries: nothing to compute; no keys: out = 0, lse = -inf, zero gradients
        sl_q, sl_k = slice(cq[b], cq[b + 1]), slice(ck[b], ck[b + 1])
        f = lambda x, sl: np.ascontiguousarray(np.transpose(x[sl], (1, 0, 2)))[None]      # [1, heads, len, D]
        o, l, gq, gk, gv = oracle.attention_backward_grouped(f(q, sl_q), f(k, sl_k), f(v, sl_k), f(do, sl_q), causal)
        back = lambda x: np.transpose(x[0], (1, 0, 2))
        out[sl_q], dq[sl_q], dk[sl_k], dv[sl_k] = back(o), back(gq), back(gk), back(gv)
        lse[:, sl_q] = l[0]
    return out, lse, dq, dk, dv


CASES = [
    # lens_q, lens_k (None: same as lens_q), H, Hkv, D, causal
    ([300, 128, 1, 257, 640], None, 2, 2, 128, True),
    ([127, 129, 255, 256, 383], None, 3, 3, 64, True),
    ([200, 0, 77, 512], None, 2, 2, 128, True),                 # one empty sequence
    ([130, 64, 300], [515, 64, 300], 2, 2, 128, True),          # more keys than queries: bottom-right aligned diagonal
    ([100, 260, 33], [40, 700, 129], 2, 2, 64, False),          # cross attention with unrelated lengths
    ([300, 129, 512, 1], None, 4, 2, 128, True),                # grouped heads
    ([90, 140], None, 6, 1, 64, False),                         # one key/value head
    ([1024, 128, 2048], None, 1, 1, 128, True),                 # several tiles per sequence, very uneven
]


@pytest.mark.parametrize("lens_q,lens_k,H,Hkv,D,causal", CASES)
def test_packed_forward_backward_vs_per_sequence_oracle(tt, oracle, lens_q, lens_k, H, Hkv, D, causal):
    lens_k = lens_q if lens_k is None else lens_k
    q, k, v, do = _pack(oracle, 11 + H + D, lens_q, lens_k, H, Hkv, D)
    o_r, lse_r, dq_r, dk_r, dv_r = _oracle_packed(oracle, q, k, v, do, lens_q, lens_k, causal)
    dev = lambda x: torch.from_numpy(x).to("cuda", dtype=torch.bfloat16)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(do)
    cu = lambda lens: torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    cu_q, cu_k = cu(lens_q), cu(lens_k)
    out, lse = tt.attention_forward_varlen(tq, tk, tv, cu_q, cu_k, max(lens_q), max(lens_k), causal=causal)
    dq, dk, dv = tt.attention_backward_varlen(tq, tk, tv, cu_q, cu_k, max(lens_q), max(lens_k), out, lse, tdo, causal=causal)
    tt.check_device_status()
    f = lambda t: t.float().cpu().numpy()
    assert oracle.max_abs_err(f(out), o_r) <= 2e-2
    got_lse = f(lse)
    fin = np.isfinite(lse_r)
    assert np.array_equal(np.isfinite(got_lse), fin)
    assert oracle.max_abs_err(got_lse[fin], lse_r[fin]) <= 2e-2
    for got, ref, name in ((dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
        assert oracle.max_abs_err(f(got), ref) <= oracle.bf16_grad_tol(ref), name


def test_packed_equals_dense_when_all_lengths_agree(tt, oracle):
    """A packed batch of equal-length sequences is the dense problem in another layout: same kernels, same
    tiles, so the results are bit-identical."""
    B, H, S, D = 3, 2, 384, 128
    q, k, v, do = (oracle.bf16_round(x) for x in oracle.make_inputs(5, B, H, S, S, D, sigma=0.6))
    dev = lambda x: torch.from_numpy(x).to("cuda", dtype=torch.bfloat16)
    dq_, dk_, dv_, ddo = dev(q), dev(k), dev(v), dev(do)
    tt.set_backward_deterministic(True)
    try:
        o_d, l_d = tt.attention_forward(dq_, dk_, dv_, causal=True)
        g_d = tt.attention_backward(dq_, dk_, dv_, o_d, l_d, ddo, causal=True)
    finally:
        tt.set_backward_deterministic(False)
    pack = lambda t: t.permute(0, 2, 1, 3).reshape(B * S, H, D).contiguous()            # [B,H,S,D] -> [B*S, H, D]
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device="cuda")
    o_p, l_p = tt.attention_forward_varlen(pack(dq_), pack(dk_), pack(dv_), cu, cu, S, S, causal=True)
    g_p = tt.attention_backward_varlen(pack(dq_), pack(dk_), pack(dv_), cu, cu, S, S, o_p, l_p, pack(ddo), causal=True)
    tt.check_device_status()
    assert torch.equal(o_p, pack(o_d))
    assert torch.equal(l_p, l_d.permute(1, 0, 2).reshape(H, B * S))
    for a, b in zip(g_p, g_d):
        assert torch.equal(a, pack(b))


def test_packed_argument_errors(tt):
    q = torch.zeros((10, 2, 128), dtype=torch.bfloat16, device="cuda")
    cu = torch.tensor([0, 4, 10], dtype=torch.int32, device="cuda")
    with pytest.raises(tt.TTError) as err:       # fp32 and odd head dims have no packed kernels
        tt.attention_forward_varlen(q[:, :, :48].contiguous(), q[:, :, :48].contiguous(), q[:, :, :48].contiguous(), cu, cu, 6, 6)
    assert err.value.code == tt.capi.TT_ERR_UNSUPPORTED
    with pytest.raises(ValueError):              # the longest sequence cannot exceed the token count
        tt.attention_forward_varlen(q, q, q, cu, cu, 11, 6)
