"""CPU oracle for scaled-dot-product attention (TEST INFRASTRUCTURE, not product code).

This file restates, in plain NumPy, the attention forward and reverse-mode backward
obtained by composing the reference's own differentiable primitives.  The reference
ships no attention operator; what "the reference computes" for this path is the
composition

    s   = (Q @ transpose(K)) * scale          MatMul / Transpose / MulScalar
    s   = s + M                               EWiseAdd   (causal only; M = 0 / -1e30)
    e   = exp(s)                              Exp
    den = broadcast_to(reshape(summation(e, axes=(3,)), (B,H,S,1)), (B,H,S,L))
    P   = e / den                             EWiseDiv
    O   = P @ V                               MatMul

followed by `O.backward(dO)` through the reference's reverse sweep.  Each step below
cites the reference file:line (paths relative to the reference project root,
`Task3/Tinytensor/optimizer/`) whose arithmetic it follows.

Parity pin: the reference holds no golden vectors for this path.  The restatement is
pinned against the reference's own ops, imported and executed (see
`tests/golden/make_golden.py`, which writes the committed fixtures), against an
independent float64 closed form, and against finite differences.

Only tests, the smoke check and the benchmark's CPU-baseline legs may import this
module.  Nothing under the product package does.
"""
from __future__ import annotations

import numpy as np

MASK_VALUE = -1e30  # additive causal mask constant, strictly above the (shifted) diagonal


# --------------------------------------------------------------------------------------
# seeded inputs (shared by tests and the benchmark; one convention, recorded here)
# --------------------------------------------------------------------------------------
TENSOR_IDS = {"q": 0, "k": 1, "v": 2, "do": 3}


def slice_input(seed: int, name: str, bh: int, rows: int, d: int, sigma: float = 1.0) -> np.ndarray:
    """fp32 `[rows, d]` block of tensor `name` for flattened batch*head index `bh`.

    Keyed per slice (`default_rng([seed, tensor_id, bh])`, PCG64) so that any rank can
    generate just its shard and the oracle can regenerate any sampled slice without
    building multi-GB tensors.
    """
    rng = np.random.default_rng([seed, TENSOR_IDS[name], bh])
    x = rng.standard_normal((rows, d), dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x


def make_inputs(seed, B, H, S, L, D, sigma=1.0, with_do=True, do_sigma=1.0):
    """Full `[B,H,*,D]` fp32 tensors assembled from per-slice blocks."""
    q = np.empty((B * H, S, D), np.float32)
    k = np.empty((B * H, L, D), np.float32)
    v = np.empty((B * H, L, D), np.float32)
    do = np.empty((B * H, S, D), np.float32) if with_do else None
    for bh in range(B * H):
        q[bh] = slice_input(seed, "q", bh, S, D, sigma)
        k[bh] = slice_input(seed, "k", bh, L, D, sigma)
        v[bh] = slice_input(seed, "v", bh, L, D, sigma)
        if with_do:
            do[bh] = slice_input(seed, "do", bh, S, D, do_sigma)
    shp = lambda a, n: a.reshape(B, H, n, D)
    return shp(q, S), shp(k, L), shp(v, L), (shp(do, S) if with_do else None)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even) and return it widened back to fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    out = ((u + r) & np.uint32(0xFFFF0000)).astype(np.uint32)
    # NaN stays NaN (payload may change); inputs here are finite
    return out.view(np.float32).reshape(x.shape)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """bf16 bit pattern (uint16) of fp32 `x`, round-to-nearest-even."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------------------
# the mask the composition adds (EWiseAdd, operators.py:194-199)
# --------------------------------------------------------------------------------------
def causal_mask(S: int, L: int, dtype=np.float32) -> np.ndarray:
    """`[S,L]` additive mask: 0 where key j <= query i + (L - S), MASK_VALUE elsewhere.

    For L == S this is `triu(full((S,L), -1e30), 1)`.  For L != S the diagonal is
    aligned bottom-right (the last query sees every key); the reference gives no
    precedent, so the convention is fixed here and the kernels follow it.
    """
    i = np.arange(S)[:, None]
    j = np.arange(L)[None, :]
    return np.where(j <= i + (L - S), 0.0, MASK_VALUE).astype(dtype)


def default_scale(D: int) -> float:
    return 1.0 / float(np.sqrt(float(D)))


# --------------------------------------------------------------------------------------
# forward
# --------------------------------------------------------------------------------------
def attention_forward(q, k, v, causal=False, scale=None, return_intermediates=False):
    """O (and LSE) for `q [B,H,S,D]`, `k,v [B,H,L,D]`, computed in the dtype of the inputs.

    Follows the composition op by op; `lse = log(den)` is not a node of the reference
    graph, it is returned because the CUDA path emits it (natural log, no max shift).
    """
    q = np.asarray(q); k = np.asarray(k); v = np.asarray(v)
    B, H, S, D = q.shape
    L = k.shape[2]
    sc = float(default_scale(D) if scale is None or scale <= 0 else scale)  # Python float keeps fp32 (MulScalar, operators.py:234-239)
    kt = np.swapaxes(k, -1, -2)                      # Transpose.compute, operators.py:327-336
    s = np.matmul(q, kt)                             # MatMul.compute, operators.py:417-418
    s = s * sc                                       # MulScalar.compute, operators.py:238-239
    if causal:
        m = np.broadcast_to(causal_mask(S, L, s.dtype), s.shape)
        s = s + m                                    # EWiseAdd.compute, operators.py:195-196
    e = np.exp(s)                                    # Exp.compute, operators.py:465-466
    den = np.sum(e, axis=3)                          # Summation.compute, operators.py:392-397
    den_b = np.broadcast_to(np.reshape(den, (B, H, S, 1)), e.shape)  # Reshape :352-353, BroadcastTo :370-371
    p = e / den_b                                    # EWiseDiv.compute, operators.py:292-293
    o = np.matmul(p, v)                              # MatMul.compute, operators.py:417-418
    lse = np.log(den)
    if return_intermediates:
        return o, lse, dict(s=s, e=e, den=den_b, p=p, scale=sc)
    return o, lse


# --------------------------------------------------------------------------------------
# backward: the reference's reverse sweep over that graph (autodiff.py:33-61)
# --------------------------------------------------------------------------------------
def attention_backward(q, k, v, do, causal=False, scale=None):
    """(dQ, dK, dV) for upstream gradient `do`, node by node in reverse topological order."""
    o, lse, t = attention_forward(q, k, v, causal, scale, return_intermediates=True)
    s, e, den, p, sc = t["s"], t["e"], t["den"], t["p"], t["scale"]
    B, H, S, D = q.shape
    # O = P @ V                       MatMul.gradient, operators.py:421-429
    dp = np.matmul(do, np.swapaxes(v, -1, -2))
    dv = np.matmul(np.swapaxes(p, -1, -2), do)
    # P = e / den                     EWiseDiv.gradient, operators.py:296-298
    de_div = dp / den
    dden = -dp * e / (den ** 2)
    # den = broadcast(reshape(sum))   BroadcastTo.gradient :373-380, Reshape.gradient :356-358,
    #                                 Summation.gradient :400-408
    dden_r = np.reshape(np.sum(dden, axis=3), (B, H, S, 1))
    de_sum = np.broadcast_to(np.reshape(np.reshape(dden_r, (B, H, S)), (B, H, S, 1)), e.shape)
    # adjoints of a node with two consumers are added pairwise, autodiff.py:47-54
    de = de_div + de_sum
    # e = exp(s)                      Exp.gradient, operators.py:469-470 (recomputes exp)
    ds = de * np.exp(s)
    # s = s0 + M                      EWiseAdd.gradient, operators.py:198-199 (mask is a constant)
    # s0 = qk * scale                 MulScalar.gradient, operators.py:241-242
    dqk = ds * sc
    # qk = Q @ Kt, Kt = transpose(K)  MatMul.gradient :421-429, Transpose.gradient :338-340
    dq = np.matmul(dqk, k)
    dk = np.swapaxes(np.matmul(np.swapaxes(q, -1, -2), dqk), -1, -2)
    return o, lse, dq, dk, dv


# --------------------------------------------------------------------------------------
# grouped heads (GQA / MQA): an extension without a counterpart in the reference, defined through
# its ops -- each key/value head is broadcast to the query heads of its group (BroadcastTo.compute,
# operators.py:370-371) and the gradients of the copies are summed (BroadcastTo.gradient :373-380)
# --------------------------------------------------------------------------------------
def expand_kv_heads(x, H):
    """`[B,Hkv,L,D]` -> `[B,H,L,D]`: query head h reads key/value head h // (H // Hkv)."""
    x = np.asarray(x)
    B, Hkv, L, D = x.shape
    g = H // Hkv
    return np.ascontiguousarray(np.broadcast_to(x.reshape(B, Hkv, 1, L, D), (B, Hkv, g, L, D))).reshape(B, H, L, D)


def reduce_kv_heads(dx, Hkv):
    """Adjoint of `expand_kv_heads`: sums the gradients of the copies of each key/value head."""
    dx = np.asarray(dx)
    B, H, L, D = dx.shape
    return np.sum(dx.reshape(B, Hkv, H // Hkv, L, D), axis=2)


def attention_backward_grouped(q, k, v, do, causal=False, scale=None):
    """`attention_backward` for k, v with fewer heads than q."""
    H, Hkv = q.shape[1], k.shape[1]
    o, lse, dq, dk, dv = attention_backward(q, expand_kv_heads(k, H), expand_kv_heads(v, H), do, causal, scale)
    return o, lse, dq, reduce_kv_heads(dk, Hkv), reduce_kv_heads(dv, Hkv)


# --------------------------------------------------------------------------------------
# row softmax: the adjacent native op (SoftmaxForward, src/Layers.cu:324-349)
# --------------------------------------------------------------------------------------
def softmax_rows(x):
    """Softmax over the last axis with the row maximum subtracted, leading axes flattened to
    rows: what the native SoftmaxForward computes (src/Layers.cu:324-349: ChannelMax, ChannelSub,
    ChannelExp, ChannelSum, ChannelDiv) and, call for call, the NumPy form the reference keeps in
    Softmaxloss.compute (optimizer/operators.py:610-612)."""
    x = np.asarray(x)
    z = x.reshape(-1, x.shape[-1])
    z_exp = np.exp(z - np.max(z, axis=1, keepdims=True))
    z = z_exp / np.sum(z_exp, axis=1, keepdims=True)
    return z.reshape(x.shape)


def softmax_rows_backward(x, dy):
    """dx for y = softmax_rows(x): the reference's reverse sweep (autodiff.py:33-61) over
    exp(x - max) / broadcast(sum), node by node as in `attention_backward`."""
    x = np.asarray(x); dy = np.asarray(dy)
    z = x.reshape(-1, x.shape[-1]); g = dy.reshape(z.shape)
    s = z + np.broadcast_to(-np.max(z, axis=1, keepdims=True), z.shape)   # EWiseAdd with a constant
    e = np.exp(s)
    den = np.broadcast_to(np.reshape(np.sum(e, axis=1), (z.shape[0], 1)), z.shape)
    de_div = g / den                                                      # EWiseDiv.gradient :296-298
    dden = -g * e / (den ** 2)
    dden_r = np.reshape(np.sum(dden, axis=1), (z.shape[0], 1))            # BroadcastTo/Reshape/Summation grads
    de_sum = np.broadcast_to(np.reshape(np.reshape(dden_r, (z.shape[0],)), (z.shape[0], 1)), z.shape)
    de = de_div + de_sum
    return (de * np.exp(s)).reshape(x.shape)                              # Exp.gradient :469-470


# --------------------------------------------------------------------------------------
# fully connected layer: FcForward / FcBackward (src/Layers.cu:9-79)
# --------------------------------------------------------------------------------------
def fc_forward(x, w, b=None):
    """y = x w + 1 b^T for x [rows, in], w [in, out], b [out] (or a single value, broadcast to all
    outputs): what FcForward computes with two GEMMs (src/Layers.cu:23-39), written with the
    reference's NumPy ops: MatMul.compute (operators.py:417-418), BroadcastTo.compute (:370-371),
    EWiseAdd.compute (:195-196).  Leading axes of x are flattened to rows as the native op does."""
    x = np.asarray(x); w = np.asarray(w)
    x2 = x.reshape(-1, x.shape[-1])
    y = np.matmul(x2, w)
    if b is not None:
        b = np.asarray(b)
        bv = np.broadcast_to(b.reshape(1, -1), y.shape)
        y = y + bv
    return y.reshape(x.shape[:-1] + (w.shape[1],))


def fc_backward(x, w, dy, scalar_bias=False):
    """(dx, dw, db): FcBackward (src/Layers.cu:64-78) = MatMul.gradient (operators.py:421-429) for
    dx = dy w^T and dw = x^T dy, and the adjoint of the broadcast bias, Summation over the rows
    (BroadcastTo.gradient, operators.py:373-380); a single-value bias receives the sum over all
    of dy (src/Layers.cu:68-74)."""
    x = np.asarray(x); w = np.asarray(w); dy = np.asarray(dy)
    x2 = x.reshape(-1, x.shape[-1]); g = dy.reshape(-1, w.shape[1])
    dx = np.matmul(g, np.swapaxes(w, -1, -2))
    dw = np.matmul(np.swapaxes(x2, -1, -2), g)
    db = np.sum(g, axis=0)
    if scalar_bias:
        db = np.sum(db, axis=0).reshape(1)
    return dx.reshape(x.shape), dw, db


# --------------------------------------------------------------------------------------
# independent checks of the restatement
# --------------------------------------------------------------------------------------
def closed_form_f64(q, k, v, do=None, causal=False, scale=None):
    """Float64 closed form with a max-shifted softmax and the delta identity; shares no
    intermediate with the op-by-op path above."""
    q = np.asarray(q, np.float64); k = np.asarray(k, np.float64); v = np.asarray(v, np.float64)
    B, H, S, D = q.shape
    L = k.shape[2]
    sc = default_scale(D) if scale is None or scale <= 0 else float(scale)
    s = np.einsum("bhid,bhjd->bhij", q, k) * sc
    if causal:
        i = np.arange(S)[:, None]; j = np.arange(L)[None, :]
        s = np.where(j <= i + (L - S), s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=-1, keepdims=True)
    p = e / l
    o = np.einsum("bhij,bhjd->bhid", p, v)
    lse = (m + np.log(l))[..., 0]
    if do is None:
        return o, lse
    do = np.asarray(do, np.float64)
    dv = np.einsum("bhij,bhid->bhjd", p, do)
    dp = np.einsum("bhid,bhjd->bhij", do, v)
    delta = (do * o).sum(axis=-1, keepdims=True)
    ds = p * (dp - delta)
    dq = np.einsum("bhij,bhjd->bhid", ds, k) * sc
    dk = np.einsum("bhij,bhid->bhjd", ds, q) * sc
    return o, lse, dq, dk, dv


def attention_rows(q_rows, k, v, row0, S, causal=False, scale=None):
    """Forward for a block of query rows `[r,D]` of ONE slice against full `k,v [L,D]`.

    Rows are independent given K/V, so large configurations are checked on sampled row
    blocks without materialising S x L.  `row0` is the index of the first row in the
    slice (needed for the causal diagonal); `S` is the slice's query count.
    """
    D = q_rows.shape[-1]
    L = k.shape[0]
    sc = float(default_scale(D) if scale is None or scale <= 0 else scale)
    s = np.matmul(q_rows, k.T) * sc
    if causal:
        i = (row0 + np.arange(q_rows.shape[0]))[:, None]
        j = np.arange(L)[None, :]
        s = s + np.where(j <= i + (L - S), 0.0, MASK_VALUE).astype(s.dtype)
    e = np.exp(s)
    den = np.sum(e, axis=1, keepdims=True)
    o = np.matmul(e / den, v)
    return o, np.log(den[:, 0])


def attention_backward_rows(q_rows, do_rows, k, v, row0, S, causal=False, scale=None):
    """Forward and backward for a block of query rows `[r,D]` of ONE slice against `k,v [L,D]`:
    the same ops in the same order as `attention_backward`, on the rows' share of the graph.

    Rows are independent given K and V: O, lse and dQ of the block are final, dK and dV are the
    block's contributions (the reverse sweep sums them over all rows, MatMul.gradient,
    operators.py:421-429).  Under the causal mask the keys behind the block's last row carry
    probability exp(-1e30) = 0 exactly, so they are left out; the returned dK, dV partials cover
    the first `n_keys` keys.  Returns (o, lse, dq, dk_part, dv_part, n_keys).
    """
    D = q_rows.shape[-1]
    L = k.shape[0]
    r = q_rows.shape[0]
    sc = float(default_scale(D) if scale is None or scale <= 0 else scale)
    n_keys = min(L, row0 + r + (L - S)) if causal else L
    k = k[:n_keys]; v = v[:n_keys]
    s = np.matmul(q_rows, k.T) * sc
    if causal:
        i = (row0 + np.arange(r))[:, None]
        j = np.arange(n_keys)[None, :]
        s = s + np.where(j <= i + (L - S), 0.0, MASK_VALUE).astype(s.dtype)
    e = np.exp(s)
    den = np.broadcast_to(np.sum(e, axis=1).reshape(r, 1), e.shape)
    p = e / den
    o = np.matmul(p, v)
    dp = np.matmul(do_rows, v.T)
    dv_part = np.matmul(p.T, do_rows)
    de_div = dp / den
    dden = -dp * e / (den ** 2)
    de_sum = np.broadcast_to(np.sum(dden, axis=1).reshape(r, 1), e.shape)
    ds = (de_div + de_sum) * np.exp(s)
    dqk = ds * sc
    dq = np.matmul(dqk, k)
    dk_part = np.matmul(q_rows.T, dqk).T
    return o, np.log(den[:, 0]), dq, dk_part, dv_part, n_keys


def attention_backward_chunked(q, k, v, do, causal=False, scale=None, chunk=1024):
    """`attention_backward` of ONE slice (`q,do [S,D]`, `k,v [L,D]`) in blocks of `chunk` query
    rows, so that a long slice never holds more than `chunk x L` scores at a time.
    Returns (o, lse, dq, dk, dv)."""
    S, D = q.shape
    L = k.shape[0]
    o = np.empty((S, D), q.dtype); lse = np.empty((S,), q.dtype); dq = np.empty((S, D), q.dtype)
    dk = np.zeros((L, D), q.dtype); dv = np.zeros((L, D), q.dtype)
    for r0 in range(0, S, chunk):
        r1 = min(S, r0 + chunk)
        o[r0:r1], lse[r0:r1], dq[r0:r1], dkp, dvp, n = attention_backward_rows(q[r0:r1], do[r0:r1], k, v, r0, S, causal, scale)
        dk[:n] += dkp
        dv[:n] += dvp
    return o, lse, dq, dk, dv


def bf16_grad_tol(ref, base=2e-2) -> float:
    """Tolerance for a bf16 gradient tensor against the fp32 oracle: `base` absolute while the
    reference stays within 2.56 (where half a bf16 ulp, 2^-8 relative, is below 1e-2), and one
    bf16 ulp (2^-7 relative) of the largest reference value on top of it beyond -- rounding the
    OUTPUT to bf16 alone moves a value of magnitude m by up to m * 2^-8."""
    m = float(np.max(np.abs(ref))) if np.size(ref) else 0.0
    return base if m <= 2.56 else base + 2.0 ** -7 * m


def rel_err(a, b) -> float:
    """max|a-b| / max|b| -- the per-tensor relative error the fp32 tolerance is stated in."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def max_abs_err(a, b) -> float:
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))
