"""Property sweep on the GPU (hypothesis): random ragged shapes, head dims of both tensor-core
instantiations, grouped heads, causal on and off, both backward kernels -- every draw compared with the
oracle through the C ABI.  Bounded to a few dozen small draws so the file stays in seconds."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
hyp = pytest.importorskip("hypothesis")
from hypothesis import given, settings, HealthCheck, strategies as st  # noqa: E402

pytestmark = pytest.mark.gpu


@settings(max_examples=30, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(S=st.integers(1, 420), extra=st.integers(0, 300), D=st.sampled_from([64, 128]), causal=st.booleans(),
       heads=st.sampled_from([(1, 1), (2, 2), (4, 2), (3, 1)]), path=st.sampled_from(["fused", "two_pass"]),
       seed=st.integers(0, 2 ** 16))
def test_random_shapes_both_backward_kernels(tt, oracle, S, extra, D, causal, heads, path, seed):
    H, Hkv = heads
    L = S + extra
    q, _, _, do = oracle.make_inputs(seed, 1, H, S, L, D, sigma=0.6)
    _, k, v, _ = oracle.make_inputs(seed + 1, 1, Hkv, S, L, D, sigma=0.6, with_do=False)
    qn, kn, vn, don = (oracle.bf16_round(x) for x in (q, k, v, do))
    o_r, lse_r, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(qn, kn, vn, don, causal)
    dev = lambda x: torch.from_numpy(x).to("cuda", dtype=torch.bfloat16)
    tq, tk, tv, tdo = dev(qn), dev(kn), dev(vn), dev(don)
    old = os.environ.get("TT_BWD_PATH")
    os.environ["TT_BWD_PATH"] = path
    try:
        out, lse = tt.attention_forward(tq, tk, tv, causal=causal)
        dq, dk, dv = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal)
        tt.check_device_status()
    finally:
        if old is None:
            os.environ.pop("TT_BWD_PATH", None)
        else:
            os.environ["TT_BWD_PATH"] = old
    f = lambda t: t.float().cpu().numpy()
    tag = f"S{S} L{L} D{D} causal={causal} H{H}/{Hkv} {path}"
    assert oracle.max_abs_err(f(out), o_r) <= 2e-2, tag
    assert oracle.max_abs_err(f(lse), lse_r) <= 2e-2, tag
    for got, ref, name in ((dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
        assert oracle.max_abs_err(f(got), ref) <= oracle.bf16_grad_tol(ref), f"{tag} {name}"
