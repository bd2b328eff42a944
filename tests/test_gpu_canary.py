"""Out-of-bounds writes would go unnoticed by parity checks that only read the result region, so here
every output (out, lse, dq, dk, dv, and the backward's workspace) sits between two 4 KB guard bands
filled with a sentinel; after ragged-shape launches of every kernel family the bands must be untouched.
(The stand-in for a memory checker on machines where none can run.)"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GUARD = 4096
SENTINEL = 0xA5


class Guarded:
    """A tensor of `shape`/`dtype` carved out of a byte buffer with GUARD sentinel bytes either side."""

    def __init__(self, shape, dtype, fill=None):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.pad = (-n) % 256                       # keep the tensor 256-byte aligned, as allocators do
        self.buf = torch.full((GUARD + n + self.pad + GUARD,), SENTINEL, dtype=torch.uint8, device="cuda")
        self.n = n
        self.t = self.buf[GUARD:GUARD + n].view(dtype).reshape(shape)
        if fill is not None:
            self.t.copy_(fill)

    def intact(self):
        lo = self.buf[:GUARD]
        hi = self.buf[GUARD + self.n:]
        return bool((lo == SENTINEL).all()) and bool((hi == SENTINEL).all())


def _inputs(oracle, seed, B, H, Hkv, S, L, D, dtype):
    q, _, _, do = oracle.make_inputs(seed, B, H, S, L, D, sigma=0.6)
    _, k, v, _ = oracle.make_inputs(seed + 1, B, Hkv, S, L, D, sigma=0.6, with_do=False)
    conv = (lambda x: torch.from_numpy(oracle.bf16_round(x)).to("cuda", dtype=torch.bfloat16)) if dtype == torch.bfloat16 \
        else (lambda x: torch.from_numpy(x).cuda())
    return conv(q), conv(k), conv(v), conv(do)


SHAPES = [
    # B, H, Hkv, S, L, D, causal, dtype
    (1, 2, 2, 1, 1, 128, False, torch.bfloat16),
    (1, 2, 2, 127, 129, 128, True, torch.bfloat16),
    (2, 1, 1, 129, 129, 64, True, torch.bfloat16),
    (1, 3, 3, 257, 383, 128, True, torch.bfloat16),
    (1, 4, 2, 300, 300, 64, False, torch.bfloat16),      # grouped heads
    (1, 2, 2, 65, 200, 48, True, torch.bfloat16),        # SIMT kernels, bf16
    (1, 2, 2, 70, 90, 40, True, torch.float32),          # SIMT kernels, fp32, register-tiled
    (1, 1, 1, 33, 47, 50, False, torch.float32),         # SIMT kernels, row per lane
]


@pytest.mark.parametrize("path", ["fused", "two_pass"])
@pytest.mark.parametrize("B,H,Hkv,S,L,D,causal,dtype", SHAPES)
def test_forward_backward_stay_inside_their_outputs(tt, oracle, monkeypatch, path, B, H, Hkv, S, L, D, causal, dtype):
    monkeypatch.setenv("TT_BWD_PATH", path)
    q, k, v, do = _inputs(oracle, 300 + S, B, H, Hkv, S, L, D, dtype)
    out, lse = Guarded(q.shape, dtype), Guarded((B, H, S), torch.float32)
    tt.attention_forward(q, k, v, causal=causal, out=out.t, lse=lse.t)
    d = tt.capi.make_desc(B, H, S, L, D, tt.capi.TT_BF16 if dtype == torch.bfloat16 else tt.capi.TT_F32, causal, None, Hkv=Hkv)
    need = max(int(tt.capi.lib.tt_attn_bwd_workspace_bytes(ctypes.byref(d))), 256)
    ws = Guarded((need,), torch.uint8)
    dq, dk, dv = Guarded(q.shape, dtype), Guarded(k.shape, dtype), Guarded(v.shape, dtype)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tt.capi.check(tt.capi.lib.tt_attn_bwd(ctypes.byref(d), p(q), p(k), p(v), p(out.t), p(lse.t), p(do), p(dq.t), p(dk.t), p(dv.t),
                                          p(ws.t), need, st))
    tt.check_device_status()
    for name, g in (("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv), ("workspace", ws)):
        assert g.intact(), f"{name}: a guard band was written"
    o_r, _, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(*(t.float().cpu().numpy() for t in (q, k, v, do)), causal)
    tol = (lambda r: oracle.bf16_grad_tol(r)) if dtype == torch.bfloat16 else (lambda r: 1e-5 * max(float(np.abs(r).max()), 1e-30))
    for got, ref in ((out, o_r), (dq, dq_r), (dk, dk_r), (dv, dv_r)):
        assert oracle.max_abs_err(got.t.float().cpu().numpy(), ref) <= tol(ref)


@pytest.mark.parametrize("B,H,Hkv,L,D,page", [(3, 4, 4, 777, 128, 0), (2, 8, 2, 1000, 128, 64), (2, 8, 2, 519, 64, 16),
                                              (3, 4, 2, 300, 128, 0)])
def test_decode_stays_inside_its_outputs(tt, oracle, B, H, Hkv, L, D, page):
    """Dense and paged decode (page > 0: a shuffled pool whose unowned pages hold NaN), ragged lengths."""
    q, k, v, _ = _inputs(oracle, 500 + L, B, H, Hkv, 1, L, D, torch.bfloat16)
    q = q[:, :, :1].contiguous()
    out, lse = Guarded(q.shape, torch.bfloat16), Guarded((B, H, 1), torch.float32)
    need = max(tt.decode_workspace_bytes(B, H, L, D, Hkv=Hkv), 256)
    ws = Guarded((need,), torch.uint8)
    lens = torch.tensor([L, max(1, L // 3), 1][:B], dtype=torch.int32, device="cuda")
    if page:
        mp = -(-L // page)
        perm = torch.randperm(B * mp + 3, device="cuda")[:B * mp].to(torch.int32).reshape(B, mp)
        kpool = torch.full((B * mp + 3, Hkv, page, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        vpool = torch.full_like(kpool, float("nan"))
        pad = mp * page - L
        kp = torch.nn.functional.pad(k, (0, 0, 0, pad)).reshape(B, Hkv, mp, page, D).permute(0, 2, 1, 3, 4).reshape(B * mp, Hkv, page, D)
        vp = torch.nn.functional.pad(v, (0, 0, 0, pad)).reshape(B, Hkv, mp, page, D).permute(0, 2, 1, 3, 4).reshape(B * mp, Hkv, page, D)
        kpool[perm.flatten().long()] = kp
        vpool[perm.flatten().long()] = vp
        tt.attention_decode_paged(q, kpool, vpool, block_table=perm, seq_lens=lens, max_len=L, out=out.t, lse=lse.t, workspace=ws.t)
    else:
        tt.attention_decode_paged(q, k, v, seq_lens=lens, out=out.t, lse=lse.t, workspace=ws.t)
    tt.check_device_status()
    for name, g in (("out", out), ("lse", lse), ("workspace", ws)):
        assert g.intact(), f"{name}: a guard band was written"
    for b in range(B):
        n = int(lens[b])
        f = lambda t: t[b:b + 1].float().cpu().numpy()
        o_r, _ = oracle.attention_forward(f(q), oracle.expand_kv_heads(f(k)[:, :, :n], H), oracle.expand_kv_heads(f(v)[:, :, :n], H), False)
        assert oracle.max_abs_err(f(out.t), o_r) <= 2e-2


@pytest.mark.parametrize("B,H,Hkv,S,L,causal", [(1, 2, 2, 127, 129, True), (1, 3, 3, 513, 700, True), (2, 4, 2, 300, 300, False)])
def test_pair_kernels_stay_inside_their_outputs(tt, oracle, monkeypatch, B, H, Hkv, S, L, causal):
    """The CTA-pair forward and dK/dV pass on ragged shapes: a pair's second CTA may own a query or key
    tile that lies wholly past the end of the slice."""
    monkeypatch.setenv("TT_FWD_PATH", "2cta")
    monkeypatch.setenv("TT_BWD_PATH", "two_pass")
    monkeypatch.setenv("TT_BWD_DKV", "2cta")
    dtype, D = torch.bfloat16, 128
    q, k, v, do = _inputs(oracle, 700 + S, B, H, Hkv, S, L, D, dtype)
    out, lse = Guarded(q.shape, dtype), Guarded((B, H, S), torch.float32)
    tt.attention_forward(q, k, v, causal=causal, out=out.t, lse=lse.t)
    d = tt.capi.make_desc(B, H, S, L, D, tt.capi.TT_BF16, causal, None, Hkv=Hkv)
    need = max(int(tt.capi.lib.tt_attn_bwd_workspace_bytes(ctypes.byref(d))), 256)
    ws = Guarded((need,), torch.uint8)
    dq, dk, dv = Guarded(q.shape, dtype), Guarded(k.shape, dtype), Guarded(v.shape, dtype)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tt.capi.check(tt.capi.lib.tt_attn_bwd(ctypes.byref(d), p(q), p(k), p(v), p(out.t), p(lse.t), p(do), p(dq.t), p(dk.t), p(dv.t),
                                          p(ws.t), need, st))
    tt.check_device_status()
    for name, g in (("out", out), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv), ("workspace", ws)):
        assert g.intact(), f"{name}: a guard band was written"
    o_r, _, dq_r, dk_r, dv_r = oracle.attention_backward_grouped(*(t.float().cpu().numpy() for t in (q, k, v, do)), causal)
    for got, ref in ((out, o_r), (dq, dq_r), (dk, dk_r), (dv, dv_r)):
        assert oracle.max_abs_err(got.t.float().cpu().numpy(), ref) <= oracle.bf16_grad_tol(ref)


@pytest.mark.parametrize("path", ["1cta", "2cta", "simt"])
@pytest.mark.parametrize("rows,fin,fout", [(1, 8, 8), (129, 72, 264), (257, 136, 520), (300, 200, 24)])
def test_fully_connected_stays_inside_its_outputs(tt, oracle, monkeypatch, path, rows, fin, fout):
    monkeypatch.setenv("TT_FC_PATH", path)
    g = torch.Generator(device="cuda").manual_seed(rows)
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda").bfloat16()
    x, w, b, dy = mk(rows, fin), mk(fin, fout) / fin ** 0.5, mk(fout), mk(rows, fout)
    y, dx, dw, db = (Guarded(s, torch.bfloat16) for s in ((rows, fout), (rows, fin), (fin, fout), (fout,)))
    need = max(int(tt.capi.lib.tt_fc_bwd_workspace_bytes(rows, fin, fout, tt.capi.TT_BF16)), 256)
    ws = Guarded((need,), torch.uint8)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    tt.capi.check(tt.capi.lib.tt_fc_fwd(p(x), p(w), p(b), p(y.t), rows, fin, fout, tt.capi.TT_BF16, st))
    tt.capi.check(tt.capi.lib.tt_fc_bwd(p(x), p(w), p(dy), p(dx.t), p(dw.t), p(db.t), 0, rows, fin, fout, tt.capi.TT_BF16,
                                        p(ws.t), need, st))
    tt.check_device_status()
    for name, gd in (("y", y), ("dx", dx), ("dw", dw), ("db", db), ("workspace", ws)):
        assert gd.intact(), f"{name}: a guard band was written"
    f = lambda t: t.float().cpu().numpy()
    dx_r, dw_r, db_r = oracle.fc_backward(f(x), f(w), f(dy))
    for got, ref in ((y, oracle.fc_forward(f(x), f(w), f(b))), (dx, dx_r), (dw, dw_r), (db, db_r)):
        assert oracle.max_abs_err(f(got.t), ref) <= 2.0 ** -8 * np.abs(ref).max() + 1e-3


@pytest.mark.parametrize("B,H,Hkv,L", [(2, 8, 8, 1500), (1, 12, 2, 2049), (3, 16, 1, 640)])
def test_split_decode_stays_inside_its_outputs(tt, oracle, B, H, Hkv, L):
    """Plain decode with few slices: the keys-on-rows kernel cuts the keys into ranges and a second kernel merges them."""
    q, k, v, _ = _inputs(oracle, 900 + L, B, H, Hkv, 1, L, 128, torch.bfloat16)
    q = q[:, :, :1].contiguous()
    out, lse = Guarded(q.shape, torch.bfloat16), Guarded((B, H, 1), torch.float32)
    need = max(tt.decode_workspace_bytes(B, H, L, 128, Hkv=Hkv), 256)
    ws = Guarded((need,), torch.uint8)
    tt.attention_decode(q, k, v, out=out.t, lse=lse.t, workspace=ws.t)
    tt.check_device_status()
    for name, g in (("out", out), ("lse", lse), ("workspace", ws)):
        assert g.intact(), f"{name}: a guard band was written"
    f = lambda t: t.float().cpu().numpy()
    o_r, _ = oracle.attention_forward(f(q), oracle.expand_kv_heads(f(k), H), oracle.expand_kv_heads(f(v), H), False)
    assert oracle.max_abs_err(f(out.t), o_r) <= 2e-2
