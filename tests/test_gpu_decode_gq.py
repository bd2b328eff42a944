"""Grouped-head decode on the keys-on-rows tensor-core kernel (attn_decode_gq_sm100.cu: head dim 128,
4..16 query heads per key/value head), against the oracle and against the two other routes
(`TT_DECODE_GQA_PATH=fwd`: the general forward kernel; `simt`: the split-KV kernel).
Tolerances as for the base op: out 2e-2 absolute, log-sum-exp 1e-3."""
import numpy as np
import pytest

from test_gpu_variants import dense_decode_ref, make_grouped

pytestmark = pytest.mark.gpu
D = 128


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    return torch


# group sizes on every column count the kernel is built for (4, 8, 16) and between them; key counts
# of less than a tile, ragged tails, many tiles; few slices (keys split into ranges + merge) and many
@pytest.mark.parametrize("B,H,Hkv,L", [(2, 4, 1, 100), (3, 8, 2, 1500), (2, 10, 2, 777), (1, 24, 2, 4096), (2, 32, 2, 2049),
                                        (160, 4, 1, 300), (40, 32, 4, 640), (1, 16, 1, 32768)])
def test_routes_agree_with_the_oracle(tt, oracle, torch_cuda, monkeypatch, B, H, Hkv, L):
    torch = torch_cuda
    q, k, v, _ = make_grouped(oracle, 500 + H + L, B, H, Hkv, 1, L, D, True)
    tq, tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v))
    o_r, lse_r = dense_decode_ref(oracle, q, k, v)
    results = {}
    for route in (None, "fwd", "simt"):
        if route is None:
            monkeypatch.delenv("TT_DECODE_GQA_PATH", raising=False)
        else:
            monkeypatch.setenv("TT_DECODE_GQA_PATH", route)
        out, lse = tt.attention_decode(tq, tk, tv)
        tt.check_device_status()
        results[route] = out
        assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2, route
        assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3, route
    # same probabilities (bf16) and fp32 accumulation as the forward kernel: the two tensor-core routes agree closely
    assert float((results[None].float() - results["fwd"].float()).abs().max()) <= 4e-3


def test_default_route_is_the_new_kernel(tt, torch_cuda):
    torch = torch_cuda
    tt.capi.profile_reset()
    tt.capi.profile_enable(True)
    q = torch.randn(64, 32, 1, D, device="cuda").bfloat16()
    k = torch.randn(64, 8, 512, D, device="cuda").bfloat16()
    v = torch.randn(64, 8, 512, D, device="cuda").bfloat16()
    tt.attention_decode(q, k, v)
    torch.cuda.synchronize()
    tt.capi.profile_enable(False)
    prof = tt.capi.profile_read()
    assert prof.get("attn_decode_gq_sm100", (0.0, 0))[1] == 1 and prof.get("attn_fwd_sm100", (0.0, 0))[1] == 0


def test_running_maximum_is_raised_and_accumulators_rescaled(tt, oracle, torch_cuda):
    """Scores that grow along the keys by far more than the lazy threshold (2^8) per tile: the kernel has
    to raise its reference maximum and rescale O^T in tensor memory several times, and an early key must
    end with a weight of (almost) zero rather than an overflow."""
    torch = torch_cuda
    rng = np.random.default_rng(3)
    B, H, Hkv, L = 2, 8, 2, 2048
    q = oracle.bf16_round(rng.standard_normal((B, H, 1, D)).astype(np.float32))
    k = rng.standard_normal((B, Hkv, L, D)).astype(np.float32) * 0.05
    # add to every key a component along each query of its group that grows with the key index
    ramp = np.linspace(0.0, 40.0, L, dtype=np.float32)[None, None, :, None]
    for g in range(H // Hkv):
        k = k + ramp * (q[:, g::H // Hkv] / np.linalg.norm(q[:, g::H // Hkv], axis=-1, keepdims=True))
    k = oracle.bf16_round(k)
    v = oracle.bf16_round(rng.standard_normal((B, Hkv, L, D)).astype(np.float32))
    o_r, lse_r = dense_decode_ref(oracle, q, k, v)
    s = np.einsum("bhd,bhld->bhl", q[:, :, 0], oracle.expand_kv_heads(k, H)) / np.sqrt(D)
    assert (s.max(axis=-1) - s[:, :, :128].max(axis=-1)).min() * 1.4427 > 24     # the maximum moves by many thresholds
    tq, tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v))
    out, lse = tt.attention_decode(tq, tk, tv)
    tt.check_device_status()
    assert np.isfinite(out.float().cpu().numpy()).all()
    assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2
    assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3


@pytest.mark.parametrize("B,H,Hkv,page,max_pages", [(5, 8, 2, 64, 12), (3, 16, 1, 8, 70), (4, 12, 2, 16, 33), (3, 8, 2, 256, 3),
                                                     (40, 8, 2, 32, 9), (3, 32, 4, 128, 20)])
def test_paged_and_ragged_cache(tt, oracle, torch_cuda, monkeypatch, B, H, Hkv, page, max_pages):
    """Page pools whose unowned rows hold NaN, ragged lengths with an empty sequence and one that ends
    one key into a tile; the same sequences as a dense cache with NaN behind each end."""
    torch = torch_cuda
    monkeypatch.delenv("TT_DECODE_GQA_PATH", raising=False)
    rng = np.random.default_rng(B * 77 + page)
    cap = page * max_pages
    lens = rng.integers(1, cap + 1, size=B).astype(np.int32)
    lens[0] = cap
    lens[1] = 0
    lens[2] = min(cap, 128 * (cap // 256) + 1)
    q, k, v, _ = make_grouped(oracle, 900 + page, B, H, Hkv, 1, cap, D, True)
    n_pages = B * max_pages + 5
    perm = rng.permutation(n_pages)[:B * max_pages].astype(np.int32).reshape(B, max_pages)
    k_pool = np.full((n_pages, Hkv, page, D), np.nan, np.float32)
    v_pool = np.full((n_pages, Hkv, page, D), np.nan, np.float32)
    for b in range(B):
        for pg in range(max_pages):
            n = int(np.clip(lens[b] - pg * page, 0, page))
            k_pool[perm[b, pg], :, :n] = k[b, :, pg * page:pg * page + n]
            v_pool[perm[b, pg], :, :n] = v[b, :, pg * page:pg * page + n]
        perm[b, (int(lens[b]) + page - 1) // page:] = -1
    tq = torch.from_numpy(q).cuda().bfloat16()
    tkp, tvp = (torch.from_numpy(a).cuda().bfloat16() for a in (k_pool, v_pool))
    table, tl = torch.from_numpy(perm).cuda(), torch.from_numpy(lens).cuda()
    o_r, lse_r = dense_decode_ref(oracle, q, k, v, lens)
    keep = lens > 0
    kd, vd = k.copy(), v.copy()
    for b in range(B):
        kd[b, :, lens[b]:] = np.nan
        vd[b, :, lens[b]:] = np.nan
    for name, call in (("paged", lambda: tt.attention_decode_paged(tq, tkp, tvp, block_table=table, seq_lens=tl)),
                       ("ragged", lambda: tt.attention_decode_paged(tq, torch.from_numpy(kd).cuda().bfloat16(),
                                                                    torch.from_numpy(vd).cuda().bfloat16(), seq_lens=tl))):
        out, lse = call()
        tt.check_device_status()
        got, got_lse = out.float().cpu().numpy(), lse.cpu().numpy()
        assert np.isfinite(got).all(), name
        assert np.isneginf(got_lse[1]).all() and float(np.abs(got[1]).max()) == 0.0, name   # the empty sequence
        assert oracle.max_abs_err(got[keep], o_r[keep]) <= 2e-2, name
        assert oracle.max_abs_err(got_lse[keep], lse_r[keep]) <= 1e-3, name


@pytest.mark.parametrize("B,H,Hkv,L", [(3, 8, 2, 1500), (2, 12, 12, 777), (64, 16, 4, 640), (1, 32, 2, 16384)])
def test_head_dim_64(tt, oracle, torch_cuda, monkeypatch, B, H, Hkv, L):
    """Head dim 64: the V tile is one 64-wide block and the accumulator's upper 64 rows repeat the lower ones."""
    torch = torch_cuda
    q, k, v, _ = make_grouped(oracle, 640 + H + L, B, H, Hkv, 1, L, 64, True)
    tq, tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v))
    o_r, lse_r = dense_decode_ref(oracle, q, k, v)
    for route in (None, "simt"):
        if route is None:
            monkeypatch.delenv("TT_DECODE_GQA_PATH", raising=False)
        else:
            monkeypatch.setenv("TT_DECODE_GQA_PATH", route)
        tt.capi.profile_reset()
        tt.capi.profile_enable(True)
        out, lse = tt.attention_decode(tq, tk, tv)
        tt.check_device_status()
        tt.capi.profile_enable(False)
        prof = tt.capi.profile_read()
        assert (prof.get("attn_decode_gq_sm100", (0.0, 0))[1] == 1) == (route is None), (route, prof)
        assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2, route
        assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3, route


def test_head_dim_64_paged(tt, oracle, torch_cuda, monkeypatch):
    torch = torch_cuda
    monkeypatch.delenv("TT_DECODE_GQA_PATH", raising=False)
    rng = np.random.default_rng(64)
    B, H, Hkv, page, max_pages = 4, 8, 2, 32, 21
    cap = page * max_pages
    lens = np.array([cap, 0, 129, 500], np.int32)
    q, k, v, _ = make_grouped(oracle, 964, B, H, Hkv, 1, cap, 64, True)
    n_pages = B * max_pages + 3
    perm = rng.permutation(n_pages)[:B * max_pages].astype(np.int32).reshape(B, max_pages)
    k_pool = np.full((n_pages, Hkv, page, 64), np.nan, np.float32)
    v_pool = np.full((n_pages, Hkv, page, 64), np.nan, np.float32)
    for b in range(B):
        for pg in range(max_pages):
            n = int(np.clip(lens[b] - pg * page, 0, page))
            k_pool[perm[b, pg], :, :n] = k[b, :, pg * page:pg * page + n]
            v_pool[perm[b, pg], :, :n] = v[b, :, pg * page:pg * page + n]
    tq = torch.from_numpy(q).cuda().bfloat16()
    tkp, tvp = (torch.from_numpy(a).cuda().bfloat16() for a in (k_pool, v_pool))
    out, lse = tt.attention_decode_paged(tq, tkp, tvp, block_table=torch.from_numpy(perm).cuda(), seq_lens=torch.from_numpy(lens).cuda())
    tt.check_device_status()
    o_r, lse_r = dense_decode_ref(oracle, q, k, v, lens)
    got, got_lse = out.float().cpu().numpy(), lse.cpu().numpy()
    keep = lens > 0
    assert np.isfinite(got).all() and np.isneginf(got_lse[1]).all() and float(np.abs(got[1]).max()) == 0.0
    assert oracle.max_abs_err(got[keep], o_r[keep]) <= 2e-2
    assert oracle.max_abs_err(got_lse[keep], lse_r[keep]) <= 1e-3
