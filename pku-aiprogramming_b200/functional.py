"""Attention calls over torch CUDA tensors.

torch is used for device memory and streams only: every call hands raw device pointers
to the C ABI (`capi.lib`).  Shapes follow the reference's row-major layout:
q/out `[B,H,S,D]`, k/v `[B,Hkv,L,D]` (Hkv = H, or a divisor of H for grouped heads), lse `[B,H,S]` fp32.
"""
from __future__ import annotations

import ctypes

import torch

from . import capi

_DT = {torch.float32: capi.TT_F32, torch.bfloat16: capi.TT_BF16}


def _check_inputs(q, k, v):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor):
            raise ValueError(f"{name} must be a torch.Tensor")
        if t.dim() != 4:
            raise ValueError(f"{name} must be 4-D [B,H,rows,D], got shape {tuple(t.shape)}")
        if not t.is_cuda:
            raise ValueError(f"{name} is on {t.device}; attention runs on CUDA tensors only (no CPU path)")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    if q.dtype not in _DT or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"q, k, v must share dtype float32 or bfloat16, got {q.dtype}, {k.dtype}, {v.dtype}")
    B, H, S, D = q.shape
    Hkv = k.shape[1]
    if k.shape[0] != B or Hkv < 1 or H % Hkv != 0 or k.shape[3] != D or tuple(v.shape) != tuple(k.shape):
        raise ValueError(f"shape mismatch: q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)} "
                         "(k, v heads must divide q heads)")
    return B, H, S, k.shape[2], D


def _stream_ptr(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _check_lens(kv_lens, B, device):
    if kv_lens is None:
        return None
    if not isinstance(kv_lens, torch.Tensor) or kv_lens.dtype != torch.int32 or not kv_lens.is_cuda \
            or not kv_lens.is_contiguous() or tuple(kv_lens.shape) != (B,):
        raise ValueError(f"kv_lens must be a contiguous CUDA int32 tensor of shape ({B},)")
    return kv_lens


def attention_forward(q, k, v, causal=False, scale=None, out=None, lse=None, need_lse=True, kv_lens=None):
    """`softmax(scale * q k^T [+causal]) v` -> (out, lse).  Asynchronous on the current stream.
    `kv_lens` (int32 `[B]`, CUDA): batch entry b attends to its first kv_lens[b] keys only."""
    B, H, S, L, D = _check_inputs(q, k, v)
    kv_lens = _check_lens(kv_lens, B, q.device)
    with torch.cuda.device(q.device):
        if out is None:
            out = torch.empty_like(q)
        if lse is None and need_lse:
            lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
        d = capi.make_desc(B, H, S, L, D, _DT[q.dtype], causal, scale, Hkv=k.shape[1])
        if kv_lens is None:
            capi.check(capi.lib.tt_attn_fwd(ctypes.byref(d), _p(q), _p(k), _p(v), _p(out), _p(lse), _stream_ptr(q)))
        else:
            capi.check(capi.lib.tt_attn_fwd_padded(ctypes.byref(d), _p(q), _p(k), _p(v), _p(kv_lens), _p(out), _p(lse),
                                                   _stream_ptr(q)))
    return out, lse


def attention_backward(q, k, v, out, lse, dout, causal=False, scale=None, workspace=None, kv_lens=None):
    """(dq, dk, dv) for upstream gradient `dout`; `out`, `lse` from `attention_forward` (same `kv_lens`)."""
    B, H, S, L, D = _check_inputs(q, k, v)
    kv_lens = _check_lens(kv_lens, B, q.device)
    for name, t, shp in (("out", out, q.shape), ("dout", dout, q.shape)):
        if tuple(t.shape) != tuple(shp) or t.dtype != q.dtype or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor of shape {tuple(shp)} and dtype {q.dtype}")
    if tuple(lse.shape) != (B, H, S) or lse.dtype != torch.float32 or not lse.is_contiguous():
        raise ValueError("lse must be contiguous float32 [B,H,S]")
    with torch.cuda.device(q.device):
        d = capi.make_desc(B, H, S, L, D, _DT[q.dtype], causal, scale, Hkv=k.shape[1])
        need = int(capi.lib.tt_attn_bwd_workspace_bytes(ctypes.byref(d)))
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        nbytes = workspace.numel() * workspace.element_size()
        if kv_lens is None:
            capi.check(capi.lib.tt_attn_bwd(ctypes.byref(d), _p(q), _p(k), _p(v), _p(out), _p(lse), _p(dout),
                                            _p(dq), _p(dk), _p(dv), _p(workspace), nbytes, _stream_ptr(q)))
        else:
            capi.check(capi.lib.tt_attn_bwd_padded(ctypes.byref(d), _p(q), _p(k), _p(v), _p(kv_lens), _p(out), _p(lse),
                                                   _p(dout), _p(dq), _p(dk), _p(dv), _p(workspace), nbytes,
                                                   _stream_ptr(q)))
    return dq, dk, dv


def _varlen_desc(q, k, cu_q, cu_k, max_q, max_k, causal, scale):
    for name, t in (("q", q), ("k", k)):
        if t.dim() != 3 or not t.is_cuda or not t.is_contiguous() or t.dtype != torch.bfloat16:
            raise ValueError(f"{name} must be a contiguous CUDA bfloat16 tensor [tokens, heads, D]")
    for name, t in (("cu_q", cu_q), ("cu_k", cu_k)):
        if t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous() or t.dim() != 1 or t.numel() != cu_q.numel():
            raise ValueError(f"{name} must be a contiguous CUDA int32 vector of n_seq + 1 cumulative token counts")
    H, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    if k.shape[2] != D or H % Hkv != 0:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)} k {tuple(k.shape)}")
    return capi.VarlenDesc(cu_q.numel() - 1, H, Hkv, D, capi.TT_BF16, 1 if causal else 0, float(scale) if scale else 0.0,
                           int(max_q), int(max_k), q.shape[0], k.shape[0])


def attention_forward_varlen(q, k, v, cu_q, cu_k, max_q, max_k, causal=False, scale=None, out=None, lse=None):
    """Packed variable-length batch: q `[total_q,H,D]`, k, v `[total_k,Hkv,D]`, cu_q / cu_k int32 `[n_seq+1]`
    (CUDA) cumulative token counts, max_q / max_k the longest sequence.  Returns (out `[total_q,H,D]`,
    lse `[H,total_q]`)."""
    d = _varlen_desc(q, k, cu_q, cu_k, max_q, max_k, causal, scale)
    with torch.cuda.device(q.device):
        out = torch.empty_like(q) if out is None else out
        lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device) if lse is None else lse
        capi.check(capi.lib.tt_attn_fwd_varlen(ctypes.byref(d), _p(q), _p(k), _p(v), _p(cu_q), _p(cu_k), _p(out), _p(lse),
                                               _stream_ptr(q)))
    return out, lse


def attention_backward_varlen(q, k, v, cu_q, cu_k, max_q, max_k, out, lse, dout, causal=False, scale=None, workspace=None):
    """(dq, dk, dv) of the packed batch; `out`, `lse` from `attention_forward_varlen`."""
    d = _varlen_desc(q, k, cu_q, cu_k, max_q, max_k, causal, scale)
    with torch.cuda.device(q.device):
        need = int(capi.lib.tt_attn_bwd_varlen_workspace_bytes(ctypes.byref(d)))
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        capi.check(capi.lib.tt_attn_bwd_varlen(ctypes.byref(d), _p(q), _p(k), _p(v), _p(cu_q), _p(cu_k), _p(out), _p(lse),
                                               _p(dout), _p(dq), _p(dk), _p(dv), _p(workspace),
                                               workspace.numel() * workspace.element_size(), _stream_ptr(q)))
    return dq, dk, dv


def set_backward_deterministic(on: bool) -> None:
    """True: the tensor-core backward always runs its two-pass, bit-reproducible kernels; False (the
    default): whichever kernel measured faster for the shape, which at head dim 64 is the single-pass one,
    whose dq repeats to fp32 rounding only.  Process-wide."""
    capi.check(capi.lib.tt_attn_bwd_set_deterministic(1 if on else 0))


def decode_workspace_bytes(B, H, L, D, dtype=torch.bfloat16, Hkv=None) -> int:
    d = capi.make_desc(B, H, 1, L, D, _DT[dtype], False, None, Hkv=Hkv)
    return int(capi.lib.tt_attn_decode_workspace_bytes(ctypes.byref(d)))


def attention_decode(q, k, v, scale=None, out=None, lse=None, workspace=None, need_lse=True):
    """Single-query attention: q `[B,H,1,D]` against the whole cache k,v `[B,H,L,D]`."""
    B, H, S, L, D = _check_inputs(q, k, v)
    if S != 1:
        raise ValueError(f"decode needs S == 1, got {S}")
    with torch.cuda.device(q.device):
        if out is None:
            out = torch.empty_like(q)
        if lse is None and need_lse:
            lse = torch.empty((B, H, 1), dtype=torch.float32, device=q.device)
        d = capi.make_desc(B, H, 1, L, D, _DT[q.dtype], False, scale, Hkv=k.shape[1])
        need = int(capi.lib.tt_attn_decode_workspace_bytes(ctypes.byref(d)))
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
        nbytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
        capi.check(capi.lib.tt_attn_decode(ctypes.byref(d), _p(q), _p(k), _p(v), _p(out), _p(lse),
                                           _p(workspace), nbytes, _stream_ptr(q)))
    return out, lse


def attention_decode_paged(q, k_pool, v_pool, block_table=None, seq_lens=None, max_len=None, scale=None, out=None,
                           lse=None, workspace=None, need_lse=True):
    """Single-query attention over a paged and/or ragged cache (bf16, D 64 or 128).

    q `[B,H,1,D]`.  With `block_table` (int32 `[B, max_pages]`, CUDA): k_pool, v_pool are page pools
    `[pages, Hkv, page_size, D]`.  Without: dense `[B,Hkv,L,D]`.  `seq_lens` (int32 `[B]`, CUDA)
    limits each batch entry to its first seq_lens[b] keys.  `max_len`: longest possible sequence
    (default: page_size * max_pages, or L of the dense cache)."""
    if q.dim() != 4 or q.shape[2] != 1 or not q.is_cuda or not q.is_contiguous() or q.dtype != torch.bfloat16:
        raise ValueError("q must be a contiguous CUDA bfloat16 tensor [B,H,1,D]")
    B, H, _, D = q.shape
    for name, t in (("k_pool", k_pool), ("v_pool", v_pool)):
        if t.dim() != 4 or not t.is_cuda or not t.is_contiguous() or t.dtype != q.dtype or t.shape[3] != D:
            raise ValueError(f"{name} must be a contiguous CUDA bfloat16 tensor with last axis {D}")
    if tuple(k_pool.shape) != tuple(v_pool.shape):
        raise ValueError("k_pool and v_pool must have one shape")
    for name, t, shp in (("block_table", block_table, None), ("seq_lens", seq_lens, (B,))):
        if t is not None and (t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous() or
                              (shp is not None and tuple(t.shape) != shp)):
            raise ValueError(f"{name} must be a contiguous CUDA int32 tensor" + (f" of shape {shp}" if shp else ""))
    Hkv = k_pool.shape[1]
    if H % Hkv != 0:
        raise ValueError(f"key/value heads {Hkv} must divide query heads {H}")
    if block_table is not None:
        if block_table.dim() != 2 or block_table.shape[0] != B:
            raise ValueError("block_table must be [B, max_pages]")
        page_size, max_pages = k_pool.shape[2], block_table.shape[1]
        L = int(max_len) if max_len is not None else page_size * max_pages
    else:
        if k_pool.shape[0] != B:
            raise ValueError("a dense cache must be [B,Hkv,L,D]")
        page_size, max_pages = 0, 0
        L = int(max_len) if max_len is not None else k_pool.shape[2]
        if L > k_pool.shape[2]:
            raise ValueError("max_len exceeds the cache length")
    with torch.cuda.device(q.device):
        out = torch.empty_like(q) if out is None else out
        if lse is None and need_lse:
            lse = torch.empty((B, H, 1), dtype=torch.float32, device=q.device)
        d = capi.make_desc(B, H, 1, L, D, capi.TT_BF16, False, scale, Hkv=Hkv)
        need = int(capi.lib.tt_attn_decode_workspace_bytes(ctypes.byref(d)))
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
        nbytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
        capi.check(capi.lib.tt_attn_decode_paged(ctypes.byref(d), _p(q), _p(k_pool), _p(v_pool), _p(block_table),
                                                 _p(seq_lens), page_size, max_pages, _p(out), _p(lse), _p(workspace),
                                                 nbytes, _stream_ptr(q)))
    return out, lse


def softmax_forward(x, out=None):
    """Softmax over the last axis of a contiguous CUDA tensor (float32 or bfloat16)."""
    if not x.is_cuda or not x.is_contiguous() or x.dtype not in _DT:
        raise ValueError("softmax_forward takes a contiguous float32/bfloat16 CUDA tensor")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    with torch.cuda.device(x.device):
        out = torch.empty_like(x) if out is None else out
        capi.check(capi.lib.tt_softmax_fwd(_p(x), _p(out), rows, cols, _DT[x.dtype], _stream_ptr(x)))
    return out


def softmax_backward(y, dy, dx=None):
    """dx = y * (dy - sum(dy * y, last axis)) for y = softmax(x)."""
    if not (y.is_cuda and dy.is_cuda and y.is_contiguous() and dy.is_contiguous()) or y.dtype != dy.dtype \
            or y.shape != dy.shape or y.dtype not in _DT:
        raise ValueError("softmax_backward takes two contiguous CUDA tensors of one shape and dtype")
    cols = y.shape[-1]
    rows = y.numel() // cols if cols else 0
    with torch.cuda.device(y.device):
        dx = torch.empty_like(y) if dx is None else dx
        capi.check(capi.lib.tt_softmax_bwd(_p(y), _p(dy), _p(dx), rows, cols, _DT[y.dtype], _stream_ptr(y)))
    return dx


def _fc_check(x, w):
    if not (x.is_cuda and w.is_cuda and x.is_contiguous() and w.is_contiguous()) or x.dtype != w.dtype \
            or x.dtype not in _DT or w.dim() != 2 or x.dim() < 1 or x.shape[-1] != w.shape[0]:
        raise ValueError("fc takes contiguous CUDA tensors x [..., in] and w [in, out] of one dtype (float32/bfloat16)")
    return x.numel() // x.shape[-1] if x.shape[-1] else 0, w.shape[0], w.shape[1]


def fc_forward(x, w, bias=None, out=None):
    """y = x @ w + bias for x `[..., in]`, w `[in, out]`, bias `[out]` or None."""
    rows, fin, fout = _fc_check(x, w)
    if bias is not None and (bias.dtype != x.dtype or tuple(bias.shape) != (fout,) or not bias.is_cuda):
        raise ValueError(f"bias must be a CUDA tensor of shape ({fout},) and dtype {x.dtype}")
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty(tuple(x.shape[:-1]) + (fout,), dtype=x.dtype, device=x.device)
        capi.check(capi.lib.tt_fc_fwd(_p(x), _p(w), _p(bias), _p(out), rows, fin, fout, _DT[x.dtype], _stream_ptr(x)))
    return out


def fc_backward(x, w, dy, need_dx=True, need_dw=True, need_db=True, scalar_bias=False, workspace=None):
    """(dx, dw, db) of `fc_forward` for upstream gradient dy `[..., out]`; skipped ones are None."""
    rows, fin, fout = _fc_check(x, w)
    if dy.dtype != x.dtype or not dy.is_cuda or not dy.is_contiguous() or tuple(dy.shape) != tuple(x.shape[:-1]) + (fout,):
        raise ValueError("dy must be a contiguous CUDA tensor shaped like the layer's output")
    with torch.cuda.device(x.device):
        dx = torch.empty_like(x) if need_dx else None
        dw = torch.empty_like(w) if need_dw else None
        db = torch.empty((1 if scalar_bias else fout,), dtype=x.dtype, device=x.device) if need_db else None
        need = int(capi.lib.tt_fc_bwd_workspace_bytes(rows, fin, fout, _DT[x.dtype])) if need_db else 0
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
        nbytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
        capi.check(capi.lib.tt_fc_bwd(_p(x), _p(w), _p(dy), _p(dx), _p(dw), _p(db), int(bool(scalar_bias)), rows, fin, fout,
                                      _DT[x.dtype], _p(workspace), nbytes, _stream_ptr(x)))
    return dx, dw, db


def check_device_status(device=None):
    """Synchronises the current stream and raises if a bounded device-side wait expired."""
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        capi.check(capi.lib.tt_check_device_status(st))


# ------------------------------------------------------------------ host-buffer calls
def _host_ptr(t):
    if t is None:
        return None
    if t.is_cuda or not t.is_contiguous():
        raise ValueError("host-buffer calls take contiguous CPU tensors")
    return ctypes.c_void_p(t.data_ptr())


def attention_forward_host(q, k, v, causal=False, scale=None, out=None, lse=None):
    """Same as `attention_forward` for CPU (ideally pinned) tensors: upload, run, download."""
    B, H, S, D = q.shape
    L = k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((B, H, S), dtype=torch.float32)
    d = capi.make_desc(B, H, S, L, D, _DT[q.dtype], causal, scale, Hkv=k.shape[1])
    capi.check(capi.lib.tt_attn_fwd_host(ctypes.byref(d), _host_ptr(q), _host_ptr(k), _host_ptr(v),
                                         _host_ptr(out), _host_ptr(lse)))
    return out, lse


def attention_backward_host(q, k, v, out, lse, dout, causal=False, scale=None, dq=None, dk=None, dv=None):
    B, H, S, D = q.shape
    L = k.shape[2]
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    d = capi.make_desc(B, H, S, L, D, _DT[q.dtype], causal, scale, Hkv=k.shape[1])
    capi.check(capi.lib.tt_attn_bwd_host(ctypes.byref(d), _host_ptr(q), _host_ptr(k), _host_ptr(v), _host_ptr(out),
                                         _host_ptr(lse), _host_ptr(dout), _host_ptr(dq), _host_ptr(dk), _host_ptr(dv)))
    return dq, dk, dv


def attention_step_host(q, k, v, dout, causal=False, scale=None, out=None, lse=None, dq=None, dk=None, dv=None):
    """Forward + backward from CPU (pinned) tensors with uploads, kernels and downloads pipelined
    over slice chunks.  Returns (out, lse, dq, dk, dv)."""
    B, H, S, D = q.shape
    L = k.shape[2]
    out = torch.empty_like(q) if out is None else out
    lse = torch.empty((B, H, S), dtype=torch.float32) if lse is None else lse
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    dv = torch.empty_like(v) if dv is None else dv
    d = capi.make_desc(B, H, S, L, D, _DT[q.dtype], causal, scale, Hkv=k.shape[1])
    capi.check(capi.lib.tt_attn_fwd_bwd_host(ctypes.byref(d), _host_ptr(q), _host_ptr(k), _host_ptr(v), _host_ptr(dout),
                                             _host_ptr(out), _host_ptr(lse), _host_ptr(dq), _host_ptr(dk), _host_ptr(dv)))
    return out, lse, dq, dk, dv


def attention_decode_host(q, k, v, scale=None, out=None, lse=None):
    B, H, S, D = q.shape
    L = k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((B, H, 1), dtype=torch.float32)
    d = capi.make_desc(B, H, 1, L, D, _DT[q.dtype], False, scale, Hkv=k.shape[1])
    capi.check(capi.lib.tt_attn_decode_host(ctypes.byref(d), _host_ptr(q), _host_ptr(k), _host_ptr(v),
                                            _host_ptr(out), _host_ptr(lse)))
    return out, lse
