"""Property tests (hypothesis) of the host-side pieces: the slice partition, the row-chunked oracle and the
bf16 helpers.  Small shapes, so the whole file runs in seconds on a CPU."""
import numpy as np
import pytest

hyp = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402


@settings(max_examples=200, deadline=None)
@given(n=st.integers(0, 5000), world=st.integers(1, 64))
def test_shard_ranges_partition_the_slices(tt, n, world):
    nxt, sizes = 0, []
    for r in range(world):
        b, c = tt.shard_range(n, world, r)
        assert b == nxt and c >= 0
        nxt += c
        sizes.append(c)
    assert nxt == n and max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


@settings(max_examples=40, deadline=None)
@given(S=st.integers(1, 70), extra=st.integers(0, 40), D=st.sampled_from([4, 8, 16]), causal=st.booleans(),
       chunk=st.integers(1, 33), seed=st.integers(0, 2 ** 16))
def test_chunked_oracle_equals_whole_slice(oracle, S, extra, D, causal, chunk, seed):
    """Rows are independent given K and V: the composition evaluated in blocks of query rows (what the
    benchmark-size parity tests use) agrees with the whole-slice form for any block size and any L >= S."""
    L = S + extra
    q, k, v, do = oracle.make_inputs(seed, 1, 1, S, L, D, sigma=0.8)
    o, lse, dq, dk, dv = oracle.attention_backward(q, k, v, do, causal)
    co, clse, cdq, cdk, cdv = oracle.attention_backward_chunked(q[0, 0], k[0, 0], v[0, 0], do[0, 0], causal, chunk=chunk)
    for got, ref in ((co, o), (cdq, dq), (cdk, dk), (cdv, dv)):
        assert oracle.rel_err(got, ref[0, 0]) < 5e-6
    assert oracle.max_abs_err(clse, lse[0, 0]) < 1e-5


@settings(max_examples=100, deadline=None)
@given(x=st.lists(st.floats(min_value=-(2.0 ** 120), max_value=2.0 ** 120, width=32), min_size=1, max_size=64))
def test_bf16_round_is_nearest_even_and_idempotent(oracle, x):
    a = np.asarray(x, np.float32)
    r = oracle.bf16_round(a)
    assert np.array_equal(oracle.bf16_round(r), r)                                   # idempotent
    assert np.array_equal(oracle.bf16_bits_to_f32(oracle.bf16_bits(a)), r)           # bits <-> value round trip
    fin = np.isfinite(r)
    ulp = np.maximum(np.abs(a[fin]).astype(np.float64), 2.0 ** -126) * 2.0 ** -8      # subnormals: the smallest normal's spacing
    assert np.all(np.abs(r[fin].astype(np.float64) - a[fin].astype(np.float64)) <= ulp * 1.0001)                           # within half a bf16 ulp


@settings(max_examples=60, deadline=None)
@given(m=st.floats(0, 1e4))
def test_gradient_tolerance_rule_is_monotone(oracle, m):
    t = oracle.bf16_grad_tol(np.array([m, -m / 2]))
    assert t >= 2e-2 and (t == 2e-2) == (m <= 2.56)
