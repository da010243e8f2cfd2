"""CPU FP64 oracle for the attention half of a Clef-Omni decoder layer.

TEST INFRASTRUCTURE ONLY: nothing in the library, the ctypes mirror or the timed region of
bench.py imports this file; it is the checker the GPU tests compare against.

Restates, with explicit weight tensors instead of model modules, what the reference computes in
ref/omni_fp64.py (paths inside the reference project):
    rms             ref/omni_fp64.py:30-31
    rotary          ref/omni_fp64.py:78-88    interleaved multi-axis rotary (sections 24/20/20)
    rotate          ref/omni_fp64.py:91-94
    attention       ref/omni_fp64.py:34-75    causal softmax(Q K^T / sqrt(d)) V, grouped heads
    text_attention  ref/omni_fp64.py:95-105   norm -> q/k/v projections -> per-head q/k norm ->
                                              rotary -> attention -> output projection + residual
and what the engine does with a packed batch (clef.metal:2174-2319, `omni_attention`): a token
attends to the earlier tokens of its own record only.

Pinned by tests/golden/attn_small.npz, which tests/golden/make_golden_attn.py produced by calling
the reference's own functions (text_attention, rotary) on small seeded FP64 problems.
"""
from __future__ import annotations

import numpy as np
import torch

SECTIONS = (24, 20, 20)
THETA = 1e6
EPS = 1e-6


def rms(x, weight, eps=EPS):
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * weight


def rotary(positions, head_dim, theta=THETA, sections=SECTIONS):
    """positions int [3][T] (temporal, row, column) -> cos, sin [T][head_dim] in FP64.  Pair p of a
    head (elements p and p + head_dim/2) turns by position[axis] * theta^(-2p/head_dim), axis =
    p % 3 for the pairs below 3*min-section-count, temporal above."""
    positions = torch.as_tensor(positions)
    frequency = theta ** (-torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim)
    angles = positions.double()[..., None] * frequency
    selected = angles[0].clone()
    for axis in (1, 2):
        selected[:, axis:sections[axis] * 3:3] = angles[axis, :, axis:sections[axis] * 3:3]
    doubled = torch.cat((selected, selected), -1)
    return doubled.cos(), doubled.sin()


def rotate(x, cos, sin):
    half = x.shape[-1] // 2
    return x * cos + torch.cat((-x[..., half:], x[..., :half]), -1) * sin


def causal_attention(q, k, v):
    """q [heads][L][d], k, v [kv_heads][L][d] of ONE record, FP64; grouped heads share k/v."""
    heads, length, width = q.shape
    group = heads // k.shape[0]
    out = torch.empty_like(q)
    mask = torch.ones(length, length, dtype=torch.bool).tril()
    for h in range(heads):
        scores = (q[h] @ k[h // group].T) * width ** -0.5
        scores = scores.masked_fill(~mask, -torch.inf)
        out[h] = scores.softmax(-1) @ v[h // group]
    return out


def attention_half(x, positions, seq_bounds, attn_norm, w_qkv, q_norm, k_norm, w_out, n_head, n_kv, head_dim=128,
                   theta=THETA, sections=SECTIONS, eps=EPS, tokens=None):
    """x [T][H] residual stream -> x + o_proj(attention(...)), all in FP64 from BF16/FP32-valued inputs.
    w_qkv [(n_head + 2 n_kv) * head_dim][H]: query rows, then key rows, then value rows (the
    converted checkpoint's `attn_qkv`); w_out [H][n_head * head_dim].  `seq_bounds`: record
    boundaries of the packed batch.  Returns dict(out, q, k, v, attn) with q/k after norm + rotary."""
    x = x.to(torch.float64)
    T = x.shape[0]
    w_qkv, w_out = w_qkv.to(torch.float64), w_out.to(torch.float64)
    xn = rms(x, attn_norm.to(torch.float64), eps)
    p = xn @ w_qkv.T
    nq, nk = n_head * head_dim, n_kv * head_dim
    q = rms(p[:, :nq].reshape(T, n_head, head_dim), q_norm.to(torch.float64), eps).transpose(0, 1)
    k = rms(p[:, nq:nq + nk].reshape(T, n_kv, head_dim), k_norm.to(torch.float64), eps).transpose(0, 1)
    v = p[:, nq + nk:].reshape(T, n_kv, head_dim).transpose(0, 1)
    cos, sin = rotary(positions, head_dim, theta, sections)
    q, k = rotate(q, cos, sin), rotate(k, cos, sin)
    attn = torch.empty(n_head, T, head_dim, dtype=torch.float64)
    b = np.asarray(seq_bounds)
    for lo, hi in zip(b[:-1], b[1:]):
        attn[:, lo:hi] = causal_attention(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi])
    values = attn.transpose(0, 1).reshape(T, nq)
    out = x + values @ w_out.T
    return dict(out=out, xn=xn, q=q, k=k, v=v, attn=values)


def attention_half_rows(x, positions, rows, attn_norm, w_qkv, q_norm, k_norm, w_out, n_head, n_kv, head_dim=128,
                        theta=THETA, sections=SECTIONS, eps=EPS):
    """The rows `rows` (sorted indices) of attention_half's `out` for ONE record x [T][H], computed
    without the full T x T products: keys and values for every token, queries and the output
    projection for the chosen rows only.  Same arithmetic as attention_half, row by row."""
    x = x.to(torch.float64)
    T = x.shape[0]
    rows = np.asarray(rows)
    w_qkv, w_out = w_qkv.to(torch.float64), w_out.to(torch.float64)
    xn = rms(x, attn_norm.to(torch.float64), eps)
    nq, nk = n_head * head_dim, n_kv * head_dim
    kv = xn @ w_qkv[nq:].T
    k = rms(kv[:, :nk].reshape(T, n_kv, head_dim), k_norm.to(torch.float64), eps).transpose(0, 1)
    v = kv[:, nk:].reshape(T, n_kv, head_dim).transpose(0, 1)
    q = rms((xn[rows] @ w_qkv[:nq].T).reshape(len(rows), n_head, head_dim), q_norm.to(torch.float64), eps).transpose(0, 1)
    cos, sin = rotary(positions, head_dim, theta, sections)
    k = rotate(k, cos, sin)
    q = rotate(q, cos[rows], sin[rows])
    group = n_head // n_kv
    values = torch.empty(len(rows), nq, dtype=torch.float64)
    for i, r in enumerate(rows):
        for h in range(n_head):
            scores = (k[h // group, :r + 1] @ q[h, i]) * head_dim ** -0.5
            values[i, h * head_dim:(h + 1) * head_dim] = scores.softmax(0) @ v[h // group, :r + 1]
    return x[rows] + values @ w_out.T


# The seeded generators live with the other synthetic workloads so that bench.py can build the same
# bytes without importing this package.
from cleffa_b200.workloads import make_attention_weights, make_positions  # noqa: E402,F401
