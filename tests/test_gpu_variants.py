"""GPU parity of the attention variants on the same kernels: grouped heads (GQA / MQA) in forward,
backward and decode, and decode over paged and ragged key/value caches.  The oracle composes them
from the reference's ops (heads broadcast / gradients summed; pages gathered into a dense cache).
Tolerances as for the base op: fp32 rel 1e-5, bf16 abs 2e-2 (+ one bf16 ulp of the largest value for
gradients, which grow with the group size)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    return torch


def make_grouped(oracle, seed, B, H, Hkv, S, L, D, bf16):
    q, _, _, do = oracle.make_inputs(seed, B, H, S, L, D)
    _, k, v, _ = oracle.make_inputs(seed + 1, B, Hkv, S, L, D)
    if bf16:
        q, k, v, do = (oracle.bf16_round(a) for a in (q, k, v, do))
    return q, k, v, do


@pytest.mark.parametrize("B,H,Hkv,S,L,D,causal", [(1, 8, 2, 300, 300, 128, True), (2, 4, 1, 130, 260, 64, True),
                                                  (1, 6, 3, 257, 257, 128, False), (1, 8, 8, 128, 128, 64, True)])
def test_grouped_heads_tensor_core_fwd_bwd(tt, oracle, torch_cuda, B, H, Hkv, S, L, D, causal):
    torch = torch_cuda
    q, k, v, do = make_grouped(oracle, 70 + H + Hkv, B, H, Hkv, S, L, D, True)
    tq, tk, tv, tdo = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v, do))
    d = tt.capi.make_desc(B, H, S, L, D, tt.capi.TT_BF16, causal, None, Hkv=Hkv)
    import ctypes
    assert tt.capi.lib.tt_attn_fwd_path(ctypes.byref(d)) == b"tcgen05"
    out, lse = tt.attention_forward(tq, tk, tv, causal=causal)
    dq, dk, dv = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal)
    tt.check_device_status()
    assert tuple(dk.shape) == (B, Hkv, L, D)
    o_r, lse_r, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(q, k, v, do, causal)
    assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2
    assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3
    for got, ref, name in ((dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
        assert oracle.max_abs_err(got.float().cpu().numpy(), ref) <= oracle.bf16_grad_tol(ref), name


@pytest.mark.parametrize("B,H,Hkv,S,L,D,causal", [(2, 4, 2, 40, 72, 32, True), (1, 6, 1, 33, 33, 48, False)])
def test_grouped_heads_fp32_exact_kernels(tt, oracle, torch_cuda, B, H, Hkv, S, L, D, causal):
    torch = torch_cuda
    q, k, v, do = make_grouped(oracle, 80 + H, B, H, Hkv, S, L, D, False)
    tq, tk, tv, tdo = (torch.from_numpy(a).cuda() for a in (q, k, v, do))
    out, lse = tt.attention_forward(tq, tk, tv, causal=causal)
    dq, dk, dv = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal)
    o_r, _, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(q, k, v, do, causal)
    for got, ref, name in ((out, o_r, "o"), (dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
        assert oracle.rel_err(got.cpu().numpy(), ref) <= 1e-5, name


def test_grouped_heads_pipelined_host_step(tt, oracle, torch_cuda):
    torch = torch_cuda
    B, H, Hkv, S, D = 2, 8, 2, 256, 128
    q, k, v, do = make_grouped(oracle, 91, B, H, Hkv, S, S, D, True)
    hq, hk, hv, hdo = (torch.from_numpy(a).bfloat16().pin_memory() for a in (q, k, v, do))
    out, lse, dq, dk, dv = tt.attention_step_host(hq, hk, hv, hdo, causal=True)
    o_r, _, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(q, k, v, do, True)
    assert oracle.max_abs_err(out.float().numpy(), o_r) <= 2e-2
    for got, ref in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
        assert oracle.max_abs_err(got.float().numpy(), ref) <= oracle.bf16_grad_tol(ref)


def dense_decode_ref(oracle, q, k, v, lens=None):
    """Per batch entry: the oracle forward on the first lens[b] keys (heads expanded to the group)."""
    B, H = q.shape[:2]
    out = np.zeros_like(q)
    lse = np.full((B, H, 1), -np.inf, np.float32)
    for b in range(B):
        n = k.shape[2] if lens is None else int(lens[b])
        if n == 0:
            continue
        kb, vb = oracle.expand_kv_heads(k[b:b + 1, :, :n], H), oracle.expand_kv_heads(v[b:b + 1, :, :n], H)
        o, l = oracle.attention_forward(q[b:b + 1], kb, vb, False)
        out[b], lse[b] = o[0], l[0]
    return out, lse


@pytest.mark.parametrize("H,Hkv,D", [(8, 8, 128), (8, 4, 128), (8, 2, 64), (8, 1, 128), (6, 2, 128), (16, 2, 64)])
def test_decode_grouped_heads(tt, oracle, torch_cuda, H, Hkv, D):
    """Group sizes 1, 2, 4, 8 (one pass over K/V per group) and 3 (mapped fallback)."""
    torch = torch_cuda
    B, L = 3, 1500
    q, k, v, _ = make_grouped(oracle, 100 + H + Hkv, B, H, Hkv, 1, L, D, True)
    tq, tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v))
    out, lse = tt.attention_decode(tq, tk, tv)
    o_r, lse_r = dense_decode_ref(oracle, q, k, v)
    assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2
    assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3


@pytest.mark.parametrize("H,Hkv,D", [(8, 2, 128), (16, 2, 64), (32, 1, 128)])
def test_decode_grouped_heads_on_the_forward_kernel(tt, oracle, torch_cuda, monkeypatch, H, Hkv, D):
    """Dense grouped decode with group >= 4 can run as a [B,Hkv,G,D] forward problem on the tcgen05
    kernel (the default once B*Hkv fills the GPU); both routes must agree with the oracle."""
    torch = torch_cuda
    B, L = 2, 1000
    q, k, v, _ = make_grouped(oracle, 140 + H, B, H, Hkv, 1, L, D, True)
    tq, tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v))
    o_r, lse_r = dense_decode_ref(oracle, q, k, v)
    for route in ("tc", "simt"):
        monkeypatch.setenv("TT_DECODE_GQA_PATH", route)
        before = tt.capi.launch_count()
        out, lse = tt.attention_decode(tq, tk, tv)
        tt.check_device_status()
        # few slices: the split-KV kernel and the forward kernel (groups above 16) cut the 1000 keys into ranges and
        # merge them (two launches); the keys-on-rows kernel (groups up to 16) keeps ranges of at least 512 keys
        # that divide the key count, which 1000 keys do not offer: one launch
        assert tt.capi.launch_count() - before == (1 if (route == "tc" and H // Hkv <= 16) else 2), route
        assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2, route
        assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3, route
    monkeypatch.delenv("TT_DECODE_GQA_PATH")


@pytest.mark.parametrize("B,H,Hkv,L,D", [(2, 8, 2, 4096, 128), (1, 32, 4, 3000, 64), (160, 4, 1, 300, 128)])
def test_decode_grouped_heads_key_split_on_the_forward_kernel(tt, oracle, torch_cuda, B, H, Hkv, L, D):
    """Default routing: few (batch, key/value head) slices -> the keys are split into ranges that run as
    forward-kernel work items and are merged; many slices -> one item per slice, no merge."""
    torch = torch_cuda
    q, k, v, _ = make_grouped(oracle, 170 + H, B, H, Hkv, 1, L, D, True)
    tq, tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v))
    before = tt.capi.launch_count()
    out, lse = tt.attention_decode(tq, tk, tv)
    tt.check_device_status()
    assert tt.capi.launch_count() - before == (1 if B * Hkv >= 148 else 2)
    o_r, lse_r = dense_decode_ref(oracle, q, k, v)
    assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2
    assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3


@pytest.mark.parametrize("H,Hkv,D,page", [(8, 2, 128, 64), (4, 4, 64, 16), (8, 1, 128, 128), (6, 2, 64, 48)])
def test_decode_paged_and_ragged(tt, oracle, torch_cuda, H, Hkv, D, page):
    torch = torch_cuda
    rng = np.random.default_rng(H * 100 + page)
    B, max_pages = 5, 12
    cap = page * max_pages
    lens = np.array([cap, 0, 1, page * 3 + 5, cap - 7], np.int32)
    q, k, v, _ = make_grouped(oracle, 120 + page, B, H, Hkv, 1, cap, D, True)
    # scatter the dense cache into a shuffled page pool with some unused pages
    n_pages = B * max_pages + 9
    perm = rng.permutation(n_pages)[:B * max_pages].astype(np.int32).reshape(B, max_pages)
    k_pool = rng.standard_normal((n_pages, Hkv, page, D)).astype(np.float32)   # unused pages hold noise
    v_pool = rng.standard_normal((n_pages, Hkv, page, D)).astype(np.float32)
    for b in range(B):
        for pg in range(max_pages):
            k_pool[perm[b, pg]] = k[b, :, pg * page:(pg + 1) * page]
            v_pool[perm[b, pg]] = v[b, :, pg * page:(pg + 1) * page]
    tq = torch.from_numpy(q).cuda().bfloat16()
    tkp, tvp = (torch.from_numpy(a).cuda().bfloat16() for a in (k_pool, v_pool))
    table, tl = torch.from_numpy(perm).cuda(), torch.from_numpy(lens).cuda()
    o_r, lse_r = dense_decode_ref(oracle, q, k, v, lens)
    out, lse = tt.attention_decode_paged(tq, tkp, tvp, block_table=table, seq_lens=tl)
    tt.check_device_status()
    assert oracle.max_abs_err(out.float().cpu().numpy(), o_r) <= 2e-2
    got_lse = lse.cpu().numpy()
    assert np.isneginf(got_lse[1]).all() and float(out[1].float().abs().max()) == 0.0   # the empty sequence
    keep = lens > 0
    assert oracle.max_abs_err(got_lse[keep], lse_r[keep]) <= 1e-3
    # dense cache with lengths, and the paged call without lengths (= every page full)
    tk, tv = (torch.from_numpy(a).cuda().bfloat16() for a in (k, v))
    out2, _ = tt.attention_decode_paged(tq, tk, tv, seq_lens=tl)
    # (grouped heads take different kernels for the two calls, so equal within the tolerance, not bitwise)
    assert oracle.max_abs_err(out2.float().cpu().numpy(), o_r) <= 2e-2
    out3, _ = tt.attention_decode_paged(tq, tkp, tvp, block_table=table)
    o_full, _ = dense_decode_ref(oracle, q, k, v)
    assert oracle.max_abs_err(out3.float().cpu().numpy(), o_full) <= 2e-2


@pytest.mark.parametrize("B,H,Hkv,D,page,max_pages,route", [
    (5, 8, 2, 128, 64, 12, "tc"), (5, 8, 1, 128, 128, 5, "tc"), (4, 16, 4, 64, 16, 40, "tc"), (3, 8, 2, 128, 256, 3, "tc"),
    (3, 4, 1, 64, 8, 50, "tc"), (40, 8, 2, 128, 32, 9, None), (3, 8, 2, 128, 64, 40, None), (3, 32, 4, 64, 32, 70, None), (5, 8, 2, 128, 64, 12, "simt")])
def test_decode_paged_grouped_heads_on_the_forward_kernel(tt, oracle, torch_cuda, monkeypatch, B, H, Hkv, D, page, max_pages, route):
    """Paged cache with group >= 4: the forward kernel gathers each key tile page by page.  Rows of
    the pools that no sequence owns hold NaN (a cache allocated but never written may), sequences are
    ragged and one is empty; result = oracle on the dense cache, and route `None` checks the default
    (B * Hkv about fills the GPU -> forward kernel, one launch)."""
    torch = torch_cuda
    rng = np.random.default_rng(B * 1000 + page)
    cap = page * max_pages
    lens = rng.integers(1, cap + 1, size=B).astype(np.int32)
    lens[0] = cap
    lens[1] = 0
    lens[2] = min(cap, 128 * (cap // 256) + 1)
    q, k, v, _ = make_grouped(oracle, 300 + page, B, H, Hkv, 1, cap, D, True)
    n_pages = B * max_pages + 7
    perm = rng.permutation(n_pages)[:B * max_pages].astype(np.int32).reshape(B, max_pages)
    k_pool = np.full((n_pages, Hkv, page, D), np.nan, np.float32)
    v_pool = np.full((n_pages, Hkv, page, D), np.nan, np.float32)
    for b in range(B):
        for pg in range(max_pages):
            n = int(np.clip(lens[b] - pg * page, 0, page))   # only the rows the sequence owns
            k_pool[perm[b, pg], :, :n] = k[b, :, pg * page:pg * page + n]
            v_pool[perm[b, pg], :, :n] = v[b, :, pg * page:pg * page + n]
        perm[b, (int(lens[b]) + page - 1) // page:] = -1      # table entries past the sequence are not valid pages
    tq = torch.from_numpy(q).cuda().bfloat16()
    tkp, tvp = (torch.from_numpy(a).cuda().bfloat16() for a in (k_pool, v_pool))
    table, tl = torch.from_numpy(perm).cuda(), torch.from_numpy(lens).cuda()
    o_r, lse_r = dense_decode_ref(oracle, q, k, v, lens)
    if route:
        monkeypatch.setenv("TT_DECODE_GQA_PATH", route)
    before = tt.capi.launch_count()
    out, lse = tt.attention_decode_paged(tq, tkp, tvp, block_table=table, seq_lens=tl)
    tt.check_device_status()
    if route != "simt":
        # the tensor-core decode kernel alone when the slices fill the GPU or the cache is short, else over
        # key ranges (whole 128-key tiles, at least 512 keys, about four ranges per SM) + merge
        want = -(-4 * 148 // (B * Hkv))
        chunk = max(512, -(-(-(-cap // want)) // 128) * 128)
        assert tt.capi.launch_count() - before == (1 if B * Hkv >= 148 or -(-cap // chunk) < 2 else 2)
    got, got_lse = out.float().cpu().numpy(), lse.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.isneginf(got_lse[1]).all() and float(np.abs(got[1]).max()) == 0.0   # the empty sequence
    keep = lens > 0
    assert oracle.max_abs_err(got[keep], o_r[keep]) <= 2e-2
    assert oracle.max_abs_err(got_lse[keep], lse_r[keep]) <= 1e-3
    # the same sequences in a dense [B,Hkv,cap,D] cache with NaN behind each sequence's end
    kd, vd = k.copy(), v.copy()
    for b in range(B):
        kd[b, :, lens[b]:] = np.nan
        vd[b, :, lens[b]:] = np.nan
    out2, lse2 = tt.attention_decode_paged(tq, torch.from_numpy(kd).cuda().bfloat16(), torch.from_numpy(vd).cuda().bfloat16(), seq_lens=tl)
    tt.check_device_status()
    got2, got_lse2 = out2.float().cpu().numpy(), lse2.cpu().numpy()
    assert np.isfinite(got2).all() and np.isneginf(got_lse2[1]).all() and float(np.abs(got2[1]).max()) == 0.0
    assert oracle.max_abs_err(got2[keep], o_r[keep]) <= 2e-2
    assert oracle.max_abs_err(got_lse2[keep], lse_r[keep]) <= 1e-3


def test_variant_argument_errors(tt, torch_cuda):
    torch = torch_cuda
    q = torch.randn(2, 6, 1, 64, device="cuda").bfloat16()
    with pytest.raises(ValueError):
        tt.attention_decode(q, torch.randn(2, 4, 100, 64, device="cuda").bfloat16(), torch.randn(2, 4, 100, 64, device="cuda").bfloat16())
    pool = torch.randn(10, 2, 16, 64, device="cuda").bfloat16()
    table = torch.zeros(2, 3, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        tt.attention_decode_paged(q, pool, pool, block_table=table, max_len=16 * 3 + 1)     # longer than the table covers
    with pytest.raises(ValueError):
        tt.attention_decode_paged(q, pool, pool, block_table=table.long())
    with pytest.raises(ValueError):
        tt.attention_decode_paged(q.float(), pool.float(), pool.float(), block_table=table)
    c = tt.capi
    import ctypes
    d = c.make_desc(2, 6, 8, 8, 64, c.TT_BF16, False, None, Hkv=4)
    assert c.lib.tt_attn_fwd(ctypes.byref(d), None, None, None, None, None, None) == c.TT_ERR_BAD_SHAPE


def padded_ref(oracle, q, k, v, do, lens, causal):
    """Per batch entry: the oracle on the first lens[b] keys; causal mask aligned to the FULL length
    (query i of S sees keys j <= i + (L - S)), gradients of padded keys zero."""
    B, H, S, D = q.shape
    Hkv, L = k.shape[1], k.shape[2]
    o = np.zeros_like(q); dq = np.zeros_like(q); dk = np.zeros_like(k); dv = np.zeros_like(v)
    lse = np.zeros((B, H, S), np.float32)
    for b in range(B):
        n = int(lens[b])
        kb, vb = oracle.expand_kv_heads(k[b:b + 1, :, :n], H), oracle.expand_kv_heads(v[b:b + 1, :, :n], H)
        qb, dob = q[b:b + 1].astype(np.float64), do[b:b + 1].astype(np.float64)
        s = np.matmul(qb, np.swapaxes(kb, -1, -2).astype(np.float64)) / np.sqrt(D)
        if causal:
            i, j = np.arange(S)[:, None], np.arange(n)[None, :]
            s = np.where(j <= i + (L - S), s, -np.inf)
        m = s.max(-1, keepdims=True)
        e = np.exp(s - m)
        den = e.sum(-1, keepdims=True)
        p = e / den
        ob = np.matmul(p, vb.astype(np.float64))
        dp = np.matmul(dob, np.swapaxes(vb, -1, -2).astype(np.float64))
        ds = p * (dp - (dob * ob).sum(-1, keepdims=True))
        o[b] = ob[0]; lse[b] = (m + np.log(den))[0, ..., 0]
        dq[b] = (np.matmul(ds, kb.astype(np.float64)) / np.sqrt(D))[0]
        dk[b, :, :n] = oracle.reduce_kv_heads(np.matmul(np.swapaxes(ds, -1, -2), qb) / np.sqrt(D), Hkv)[0]
        dv[b, :, :n] = oracle.reduce_kv_heads(np.matmul(np.swapaxes(p, -1, -2), dob), Hkv)[0]
    return o, lse, dq, dk, dv


@pytest.mark.parametrize("bf16,B,H,Hkv,S,L,D,causal,lens", [
    (True, 3, 4, 4, 384, 384, 128, False, [384, 130, 1]),
    (True, 3, 4, 2, 300, 300, 64, True, [300, 129, 64]),
    (True, 2, 2, 2, 130, 400, 128, True, [400, 290]),
    (False, 3, 2, 1, 40, 72, 32, True, [72, 40, 33]),
    (False, 2, 3, 3, 33, 50, 48, False, [50, 7]),
])
def test_key_padding_lengths_fwd_bwd(tt, oracle, torch_cuda, bf16, B, H, Hkv, S, L, D, causal, lens):
    torch = torch_cuda
    q, k, v, do = make_grouped(oracle, 150 + S + D, B, H, Hkv, S, L, D, bf16)
    cast = (lambda a: torch.from_numpy(a).cuda().bfloat16()) if bf16 else (lambda a: torch.from_numpy(a).cuda())
    tq, tk, tv, tdo = (cast(a) for a in (q, k, v, do))
    tl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out, lse = tt.attention_forward(tq, tk, tv, causal=causal, kv_lens=tl)
    dq, dk, dv = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal, kv_lens=tl)
    tt.check_device_status()
    o_r, lse_r, dq_r, dk_r, dv_r = padded_ref(oracle, q, k, v, do, lens, causal)
    f = lambda t: t.float().cpu().numpy()
    if bf16:
        assert oracle.max_abs_err(f(out), o_r) <= 2e-2 and oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3
        for got, ref, name in ((dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
            assert oracle.max_abs_err(f(got), ref) <= oracle.bf16_grad_tol(ref), name
    else:
        for got, ref, name in ((out, o_r, "o"), (dq, dq_r, "dq"), (dk, dk_r, "dk"), (dv, dv_r, "dv")):
            assert oracle.rel_err(f(got), ref) <= 1e-5, name
    for b, n in enumerate(lens):   # padded keys: exactly zero gradients
        assert float(dk[b, :, n:].float().abs().max() if n < L else 0.0) == 0.0
        assert float(dv[b, :, n:].float().abs().max() if n < L else 0.0) == 0.0
    # full lengths reproduce the unpadded call bit for bit
    full = torch.full((B,), L, dtype=torch.int32, device="cuda")
    out2, lse2 = tt.attention_forward(tq, tk, tv, causal=causal, kv_lens=full)
    out3, lse3 = tt.attention_forward(tq, tk, tv, causal=causal)
    assert torch.equal(out2, out3) and torch.equal(lse2, lse3)
    with pytest.raises(ValueError):
        tt.attention_forward(tq, tk, tv, kv_lens=tl.long())


def test_random_combinations_of_variants(tt, oracle, torch_cuda):
    """Seeded sweep over combinations the targeted tests do not pair up: head dim x grouping x causal
    x ragged L x key padding, forward and backward through the tensor-core kernels."""
    torch = torch_cuda
    import random
    rnd = random.Random(2024)
    for case in range(24):
        D = rnd.choice([64, 128]); B = rnd.randint(1, 2); Hkv = rnd.choice([1, 2, 3]); g = rnd.choice([1, 2, 4])
        H = Hkv * g
        S = rnd.choice([1, 17, 128, 129, 255, 300]); causal = rnd.random() < 0.5
        L = S if rnd.random() < 0.4 else rnd.choice([S + 1, S + 127, S + 200])
        lo = (L - S + 1) if causal else 1                      # a causal row must keep at least one key
        lens = [rnd.randint(lo, L) for _ in range(B)] if rnd.random() < 0.6 else [L] * B
        q, k, v, do = make_grouped(oracle, 1000 + case, B, H, Hkv, S, L, D, True)
        tq, tk, tv, tdo = (torch.from_numpy(a).cuda().bfloat16() for a in (q, k, v, do))
        tl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        out, lse = tt.attention_forward(tq, tk, tv, causal=causal, kv_lens=tl)
        dq, dk, dv = tt.attention_backward(tq, tk, tv, out, lse, tdo, causal=causal, kv_lens=tl)
        tt.check_device_status()
        o_r, lse_r, dq_r, dk_r, dv_r = padded_ref(oracle, q, k, v, do, lens, causal)
        tag = dict(case=case, B=B, H=H, Hkv=Hkv, S=S, L=L, D=D, causal=causal, lens=lens)
        f = lambda t: t.float().cpu().numpy()
        assert oracle.max_abs_err(f(out), o_r) <= 2e-2, tag
        assert oracle.max_abs_err(lse.cpu().numpy(), lse_r) <= 1e-3, tag
        for got, ref in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
            assert oracle.max_abs_err(f(got), ref) <= oracle.bf16_grad_tol(ref), tag
