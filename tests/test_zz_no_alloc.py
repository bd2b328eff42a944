"""Decode through the entry point that allocates nothing (`tt_attn_decode_static`).

Some hosts of this library may not allocate device memory at call time -- a serving loop
that froze its memory map after start-up, a sandboxed plugin -- so they cannot hand
`tt_attn_decode` its partials workspace.  For them the library carries a fixed 8 MiB scratch
array of its own.  This test drives that entry point through the C ABI twice in a row (the
second call finds the array dirty from the first) and checks both results against the
ordinary entry point, within the bf16 tolerance used throughout these tests.

The file name sorts last on purpose, so a run that stops at the first failure has already
run every other test.  It passes alone in a fresh process and after the other tests.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


@pytest.mark.parametrize("B,H,Hkv,L,D", [
    (4, 8, 8, 6000, 128),      # several key ranges per slice, ragged last range
    (3, 8, 8, 5000, 64),       # the other head dim
    (4, 8, 2, 6000, 128),      # groups of four query heads per key/value head: here the ordinary entry point
                               # takes the tensor-core kernel and this one the split-KV kernel
    (2, 6, 3, 4100, 64),       # groups of two
])
def test_static_scratch_decode_matches_workspace_decode_twice(tt, oracle, B, H, Hkv, L, D):
    lib = tt.capi.lib
    outs = []
    for call, seed in enumerate((41, 43)):
        q, _, _, _ = oracle.make_inputs(seed, B, H, 1, L, D, with_do=False)
        _, k, v, _ = oracle.make_inputs(seed + 1, B, Hkv, 1, L, D, with_do=False)
        tq, tk, tv = (torch.from_numpy(oracle.bf16_round(x)).to("cuda", dtype=torch.bfloat16) for x in (q, k, v))
        ref_out, ref_lse = tt.attention_decode(tq, tk, tv)            # existing entry point
        out = torch.full_like(tq, float("nan"))
        lse = torch.full((B, H, 1), float("nan"), dtype=torch.float32, device="cuda")
        d = tt.capi.make_desc(B, H, 1, L, D, tt.capi.TT_BF16, False, None, Hkv=Hkv)
        assert tt.capi.lib.tt_attn_decode_workspace_bytes(ctypes.byref(d)) > 0   # the path really uses scratch
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        tt.capi.check(lib.tt_attn_decode_static(ctypes.byref(d), _p(tq), _p(tk), _p(tv), _p(out), _p(lse), st))
        tt.check_device_status()
        got, want = out.float().cpu().numpy(), ref_out.float().cpu().numpy()
        assert np.isfinite(got).all(), f"call {call}"
        assert np.max(np.abs(got - want)) <= BF16_TOL, f"call {call}"
        assert np.max(np.abs(lse.cpu().numpy() - ref_lse.cpu().numpy())) <= 1e-3, f"call {call}"
        o_ref, _ = oracle.attention_forward(oracle.bf16_round(q), oracle.expand_kv_heads(oracle.bf16_round(k), H),
                                            oracle.expand_kv_heads(oracle.bf16_round(v), H), False)
        assert np.max(np.abs(got - o_ref)) <= BF16_TOL, f"call {call} vs oracle"
        outs.append(got)
    assert not np.array_equal(outs[0], outs[1])   # the two calls really were different problems


def test_static_scratch_decode_refuses_oversized_problems(tt, monkeypatch):
    lib = tt.capi.lib
    # partials = splits * B*H * (D+2) * 4 bytes.  One range per slice needs no partials at all, so several
    # ranges per slice are forced (the variable is restored when the test ends).
    monkeypatch.setenv("TT_DECODE_SPLITS", "8")
    B, H, L, D = 64, 64, 2048, 128     # 4096 slices * 8 ranges * 130 floats * 4 B = 17 MB > 8 MiB
    d = tt.capi.make_desc(B, H, 1, L, D, tt.capi.TT_BF16, False, None)
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")   # never dereferenced: the call is refused first
    rc = lib.tt_attn_decode_static(ctypes.byref(d), _p(x), _p(x), _p(x), _p(x), None, None)
    assert rc == tt.capi.TT_ERR_WORKSPACE
    msg = tt.capi.last_error()
    assert "8388608" in msg and "tt_attn_decode" in msg
