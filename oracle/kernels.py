"""Per-kernel CPU oracles (TEST INFRASTRUCTURE - never imported by the product).

Each function restates, with numpy/torch on the CPU in f32, the arithmetic of one
backend kernel, following the CPU helpers the reference's own kernel tests use:

  matmul*                ferrotensor-backend/tests/gpu_kernels.rs:80-101
  rms_norm               gpu_kernels.rs:114-122;  kernels.wgsl:76-98
  rms_norm_backward      gpu_kernels.rs:1300-1318; kernels.wgsl:100-151
  rope                   gpu_kernels.rs:1513-1545; kernels.wgsl:45-73
  silu_gate*             kernels.wgsl:737-780
  attention / backward   gpu_kernels.rs:132-224; flash_attention_v2_backward.wgsl:5-15
  masked_cross_entropy   gpu_kernels.rs:1375-1436; kernels.wgsl:672-711
  sum_squares_partial    kernels.wgsl:713-735
  adamw                  gpu_kernels.rs:2218-2230; kernels.wgsl:355-387
  pack_f16               ferrotensor-backend/src/tensor.rs:261-269,490-514
  embedding              ferrotensor-autograd/src/lib.rs:1159-1179
"""

import math

import numpy as np
import torch

MASKED_CE_SKIP = 0xFFFFFFFF
SUM_SQUARES_CHUNK = 4096


def _t(x, dtype=torch.float32):
    return torch.as_tensor(np.asarray(x), dtype=dtype)


def matmul(a, b, dtype=torch.float32):
    """out[M,N] = a[M,K] @ b[K,N]"""
    return (_t(a, dtype) @ _t(b, dtype)).numpy()


def matmul_bt(a, b, dtype=torch.float32):
    """out[M,N] = a[M,K] @ b[N,K]^T"""
    return (_t(a, dtype) @ _t(b, dtype).T).numpy()


def matmul_at(a, b, dtype=torch.float32):
    """out[M,N] = a[K,M]^T @ b[K,N]"""
    return (_t(a, dtype).T @ _t(b, dtype)).numpy()


def f16_round(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def pack_f16(x):
    """f32 -> RNE binary16, two per little-endian u32 word, element 2i in the low half.
    An odd element count is padded with one zero half."""
    h = np.asarray(x, dtype=np.float32).reshape(-1).astype(np.float16).view(np.uint16)
    if h.size % 2:
        h = np.concatenate([h, np.zeros(1, dtype=np.uint16)])
    return (h[0::2].astype(np.uint32) | (h[1::2].astype(np.uint32) << 16)).astype(np.uint32)


def transpose_pack_f16(w_out_in):
    """HF [out,in] f32 -> [in,out] -> packed f16 words (the frozen-linear upload)."""
    return pack_f16(np.ascontiguousarray(np.asarray(w_out_in, dtype=np.float32).T))


def rms_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float32)
    ms = (x * x).sum(-1, dtype=np.float32, keepdims=True) / np.float32(x.shape[-1])
    inv = np.float32(1.0) / np.sqrt(ms + np.float32(eps))
    return (x * inv * np.asarray(w, dtype=np.float32)).astype(np.float32)


def rms_norm_backward(x, w, g, eps):
    """gx = g*w*inv - x*inv^3*sum(g*w*x)/n ; gw[i] = sum_rows g*x*inv"""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    g = np.asarray(g, dtype=np.float64)
    n = x.shape[-1]
    inv = 1.0 / np.sqrt((x * x).sum(-1, keepdims=True) / n + eps)
    gwx = (g * w * x).sum(-1, keepdims=True)
    gx = g * w * inv - x * (gwx * inv ** 3 / n)
    gw = (g * x * inv).reshape(-1, n).sum(0)
    return gx.astype(np.float32), gw.astype(np.float32)


def rope(x, head_dim, seq_len, heads, pos=0, theta=10000.0, inverse=False):
    """x flat [tokens*heads*head_dim]; token t sits at position pos + (t % seq_len).
    angle = +-f32(position) * powf(theta, -2i/d), all in f32."""
    x = np.array(x, dtype=np.float32).reshape(-1, heads, head_dim)
    half = head_dim // 2
    tokens = x.shape[0]
    i = np.arange(half, dtype=np.float32)
    freq = np.power(np.float32(theta), np.float32(-2.0) * i / np.float32(head_dim), dtype=np.float32)
    p = (pos + (np.arange(tokens) % seq_len)).astype(np.float32)
    angle = (p[:, None] * freq[None, :]).astype(np.float32)
    if inverse:
        angle = -angle
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    x1, x2 = x[..., :half].copy(), x[..., half:].copy()
    out = np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1)
    return out.astype(np.float32).reshape(-1)


def silu_gate(a, b):
    """silu(a) * b - the FIRST argument passes through SiLU."""
    a = np.asarray(a, dtype=np.float32)
    s = np.float32(1.0) / (np.float32(1.0) + np.exp(-a))
    return (a * s * np.asarray(b, dtype=np.float32)).astype(np.float32)


def silu_gate_backward(a, b, g):
    """returns (grad wrt a, grad wrt b)"""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    g = np.asarray(g, dtype=np.float32)
    s = np.float32(1.0) / (np.float32(1.0) + np.exp(-a))
    ga = g * b * (s * (np.float32(1.0) + a * (np.float32(1.0) - s)))
    gb = g * (a * s)
    return ga.astype(np.float32), gb.astype(np.float32)


def attention(q, k, v, b, sq, sk, h, hkv, d, causal=True, dtype=torch.float32):
    """q,out [b,sq,h,d]; k,v [b,sk,hkv,d]. Returns (out, lse [b,h,sq], probs [b,h,sq,sk])."""
    q = _t(q, dtype).view(b, sq, h, d).transpose(1, 2)
    k = _t(k, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(h // hkv, dim=1)
    v = _t(v, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(h // hkv, dim=1)
    s = q @ k.transpose(-1, -2) * (1.0 / math.sqrt(d))
    if causal:
        vis = torch.ones(sq, sk, dtype=torch.bool).tril()
        s = s.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    out = (p @ v).transpose(1, 2).contiguous()
    return out.numpy(), lse.numpy(), p


def attention_backward(q, k, v, dout, b, sq, sk, h, hkv, d, causal=True, dtype=torch.float32):
    """dS = P * (dO.V - sum_j P dO.V) * scale; dK, dV summed over the query heads of a KV group."""
    grp = h // hkv
    _, _, p = attention(q, k, v, b, sq, sk, h, hkv, d, causal, dtype)
    qh = _t(q, dtype).view(b, sq, h, d).transpose(1, 2)
    kh = _t(k, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(grp, dim=1)
    vh = _t(v, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(grp, dim=1)
    do = _t(dout, dtype).view(b, sq, h, d).transpose(1, 2)
    dp = do @ vh.transpose(-1, -2)
    rowsum = (p * dp).sum(-1, keepdim=True)
    ds = p * (dp - rowsum) * (1.0 / math.sqrt(d))
    dq = (ds @ kh).transpose(1, 2).contiguous()
    dk = (ds.transpose(-1, -2) @ qh).view(b, hkv, grp, sk, d).sum(2).transpose(1, 2).contiguous()
    dv = (p.transpose(-1, -2) @ do).view(b, hkv, grp, sk, d).sum(2).transpose(1, 2).contiguous()
    return dq.numpy(), dk.numpy(), dv.numpy()


def masked_cross_entropy_weighted(logits, targets, weights):
    """logits [rows,V] f32, targets u32 (MASKED_CE_SKIP = outside the loss), weights [rows].
    Returns (row_loss [rows], grad [rows,V])."""
    z = _t(logits, torch.float32)
    rows, vocab = z.shape
    t = np.asarray(targets, dtype=np.uint32)
    w = _t(weights, torch.float32)
    skip = torch.as_tensor(t == MASKED_CE_SKIP)
    tt = torch.as_tensor(np.where(t == MASKED_CE_SKIP, 0, t).astype(np.int64))
    log_z = torch.logsumexp(z, dim=-1)
    grad = torch.exp(z - log_z[:, None]) * w[:, None]
    grad[torch.arange(rows), tt] -= w
    loss = log_z - z[torch.arange(rows), tt]
    grad[skip] = 0.0
    loss[skip] = 0.0
    return loss.numpy(), grad.numpy()


def sum_squares_partial(x):
    x = np.asarray(x, dtype=np.float32).reshape(-1)
    n = -(-x.size // SUM_SQUARES_CHUNK)
    return np.array([(x[i * SUM_SQUARES_CHUNK:(i + 1) * SUM_SQUARES_CHUNK] ** 2).sum(dtype=np.float32)
                     for i in range(n)], dtype=np.float32)


def adamw(w, g, m, v, lr, beta1, beta2, eps, wd, t):
    f = np.float32
    w, g, m, v = (np.asarray(a, dtype=f) for a in (w, g, m, v))
    m2 = m * f(beta1) + (f(1.0) - f(beta1)) * g
    v2 = v * f(beta2) + (f(1.0) - f(beta2)) * g * g
    m_hat = m2 / (f(1.0) - np.power(f(beta1), f(t), dtype=f))
    v_hat = v2 / (f(1.0) - np.power(f(beta2), f(t), dtype=f))
    w2 = w - f(lr) * (m_hat / (np.sqrt(v_hat) + f(eps)) + f(wd) * w)
    return w2.astype(f), m2.astype(f), v2.astype(f)


def embedding(table, ids):
    """rows of table [V,h]; an id >= V gives a zero row."""
    table = np.asarray(table, dtype=np.float32)
    ids = np.asarray(ids).reshape(-1).astype(np.int64)
    out = np.zeros((ids.size, table.shape[1]), dtype=np.float32)
    ok = ids < table.shape[0]
    out[ok] = table[ids[ok]]
    return out


def attention_decode(q, k, v, b, sk, h, hkv, d, causal=True, causal_offset=0, window=0, dtype=torch.float64):
    """One query per (batch, head) against a KV cache (flash_attention_v2.wgsl:284-382): the query
    sits at position `causal_offset`; key kp is visible when kp < sk, (not causal or kp <= qa) and
    (no window or |qa - kp| < window) (`fa_visible`, :106-116).  A row with no visible key is 0."""
    q = _t(q, dtype).view(b, 1, h, d).transpose(1, 2)
    k = _t(k, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(h // hkv, dim=1)
    v = _t(v, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(h // hkv, dim=1)
    s = q @ k.transpose(-1, -2) * (1.0 / math.sqrt(d))
    kp = torch.arange(sk)
    vis = torch.ones(sk, dtype=torch.bool)
    if causal:
        vis &= kp <= causal_offset
    if window > 0:
        vis &= (kp - causal_offset).abs() < window
    s = s.masked_fill(~vis, float("-inf"))
    if not vis.any():
        return np.zeros((b, 1, h, d), dtype=np.float32)
    p = torch.softmax(s, dim=-1)
    return (p @ v).transpose(1, 2).contiguous().to(torch.float32).numpy()


def argmax_rows(x):
    """Index of the largest value per row in `f32::total_cmp` order, the last index winning ties
    (kernels.wgsl:251-296): compare the bit patterns mapped to an order-preserving unsigned key."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    key = np.where(bits & np.uint32(0x80000000), ~bits, bits | np.uint32(0x80000000)).astype(np.uint64)
    n = x.shape[-1]
    # larger index wins ties: combine (key, index) into one sortable integer
    combined = key * np.uint64(n) + np.arange(n, dtype=np.uint64)
    return combined.argmax(axis=-1).astype(np.uint32)


# ---- attention with an additive mask, offset/window visibility and dropout -------------------
_U32 = np.uint32


def _fmix32(h):
    """Murmur3's 32-bit finaliser (flash_attention_v2.wgsl:84-92)."""
    h = np.asarray(h, dtype=_U32)
    h = h ^ (h >> _U32(16))
    h = h * _U32(0x85EBCA6B)
    h = h ^ (h >> _U32(13))
    h = h * _U32(0xC2B2AE35)
    return h ^ (h >> _U32(16))


def _hash3(x, y, z):
    """flash_attention_v2.wgsl:70-82 (CPU copy: backend/tests/gpu_kernels.rs:2261-2281): three LCG
    steps, a round of cross-multiplication, a shift-xor each, the wrapped sum scaled by 2^-32 in
    f32 (so the value can round up to 1.0)."""
    with np.errstate(over="ignore"):
        a, b, c = (np.asarray(t, dtype=_U32) * _U32(1664525) + _U32(1013904223) for t in (x, y, z))
        a = a + b * c
        b = b + c * a
        c = c + a * b
        a, b, c = (t ^ (t >> _U32(16)) for t in (a, b, c))
        return (a + b + c).astype(np.float32) * np.float32(2.3283064365386963e-10)


def dropout_keep(prob, seed, bh, q_idx, k_idx):
    """Keep decision of attention weight (bh, q, k) under the 64-bit `seed`
    (flash_attention_v2.wgsl:94-104): both seed halves are mixed into one key that enters the
    hash xor-ed with bh.  Broadcasts over numpy index arrays."""
    if prob <= 0.0:
        return np.ones(np.broadcast(bh, q_idx, k_idx).shape, dtype=bool)
    with np.errstate(over="ignore"):
        lo, hi = _U32(seed & 0xFFFFFFFF), _U32((seed >> 32) & 0xFFFFFFFF)
        key = _fmix32(lo ^ _fmix32(hi ^ _U32(0x9E3779B9)))
        r = _hash3(np.asarray(bh, dtype=_U32) ^ key, q_idx, k_idx)
    return r >= np.float32(prob)


def _visibility(sq, sk, causal, causal_offset, window):
    """`fa_visible` (flash_attention_v2.wgsl:106-116) for every (query, key) pair."""
    qa = np.arange(sq)[:, None] + causal_offset
    kp = np.arange(sk)[None, :]
    vis = np.ones((sq, sk), dtype=bool)
    if causal:
        vis &= kp <= qa
    if window > 0:
        vis &= np.abs(qa - kp) < window
    return vis


def attention_general(q, k, v, b, sq, sk, h, hkv, d, causal=True, causal_offset=0, window=0, mask=None,
                      dropout_prob=0.0, seed=0, dout=None, dtype=torch.float64):
    """Forward (and, given `dout`, backward) of the general attention call: q/out [b,sq,h,d],
    k/v [b,sk,hkv,d]; `mask` broadcastable to [b,h,sq,sk] is added to the scaled scores of visible
    pairs and a score at or below -1e30 is then hidden; P = softmax over what is left, a row with
    nothing visible gives 0 and LSE 3e38; M = 0 or 1/(1-p) per pair;
    O = (P*M) V;  dV = (P*M)^T dO;  dS = P * (M * dO V^T - Delta), Delta = rowsum(dO * O);
    dQ = scale dS K;  dK = scale dS^T Q  (flash_attention_v2_backward.wgsl:5-15).
    Returns (out, lse) or (out, lse, dq, dk, dv) as float32 numpy arrays."""
    grp = h // hkv
    scale = 1.0 / math.sqrt(d)
    qh = _t(q, dtype).view(b, sq, h, d).transpose(1, 2)
    kh = _t(k, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(grp, dim=1)
    vh = _t(v, dtype).view(b, sk, hkv, d).transpose(1, 2).repeat_interleave(grp, dim=1)
    s = qh @ kh.transpose(-1, -2) * scale
    vis = torch.as_tensor(_visibility(sq, sk, causal, causal_offset, window)).expand(b, h, sq, sk).clone()
    if mask is not None:
        s = s + _t(np.broadcast_to(np.asarray(mask, dtype=np.float32), (b, h, sq, sk)).copy(), dtype)
        vis &= s > -1.0e30
    s = s.masked_fill(~vis, float("-inf"))
    any_vis = vis.any(-1)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.where(any_vis[..., None], torch.exp(s - lse[..., None]), torch.zeros_like(s))
    lse = torch.where(any_vis, lse, torch.full_like(lse, 3.0e38))
    bh = (np.arange(b)[:, None] * h + np.arange(h)[None, :])[:, :, None, None]
    keep = dropout_keep(dropout_prob, seed, bh, np.arange(sq)[None, None, :, None], np.arange(sk)[None, None, None, :])
    m = _t(keep.astype(np.float64) * (1.0 / (1.0 - np.float32(dropout_prob)) if dropout_prob > 0 else 1.0), dtype)
    pm = p * m
    out = pm @ vh
    res = [out.transpose(1, 2).contiguous().to(torch.float32).numpy(), lse.to(torch.float32).numpy()]
    if dout is None:
        return tuple(res)
    do = _t(dout, dtype).view(b, sq, h, d).transpose(1, 2)
    delta = (do * out).sum(-1, keepdim=True)
    ds = p * (m * (do @ vh.transpose(-1, -2)) - delta) * scale
    dq = (ds @ kh).transpose(1, 2).contiguous()
    dk = (ds.transpose(-1, -2) @ qh).view(b, hkv, grp, sk, d).sum(2).transpose(1, 2).contiguous()
    dv = (pm.transpose(-1, -2) @ do).view(b, hkv, grp, sk, d).sum(2).transpose(1, 2).contiguous()
    return tuple(res + [t.to(torch.float32).numpy() for t in (dq, dk, dv)])
