"""Seeded synthetic workloads for the Clef-Omni MoE block.

The reference publishes no dataset for this path and its model weights are not available
offline; every run uses random-init BF16 weights N(0, 0.02) and BF16 activations N(0, 1) of
the model's shapes (hidden 2048, 128 experts, top-8, intermediate 768), generated here from a
seed so that the library, the tests and the CPU oracle all read identical bytes.
"""
from __future__ import annotations

import numpy as np
import torch

H, F, E, TOP = 2048, 768, 128, 8

def make_weights(seed: int, n_expert: int = E, hidden: int = H, ffn: int = F, std: float = 0.02):
    """Random-init BF16 weights N(0, std) in the converted layout (tools/convert_omni.py:135-139)."""
    g = torch.Generator(device="cpu").manual_seed(1000003 * seed + 17)
    router = (torch.randn(n_expert, hidden, generator=g) * std).to(torch.bfloat16)
    gate_up = torch.empty(n_expert, 2 * ffn, hidden, dtype=torch.bfloat16)
    down = torch.empty(n_expert, hidden, ffn, dtype=torch.bfloat16)
    for e in range(n_expert):  # per expert keeps the FP32 staging buffer small
        gate_up[e] = (torch.randn(2 * ffn, hidden, generator=g) * std).to(torch.bfloat16)
        down[e] = (torch.randn(hidden, ffn, generator=g) * std).to(torch.bfloat16)
    return router, gate_up, down


def make_activations(seed: int, tokens: int, hidden: int = H):
    """BF16 activations N(0, 1): the post-RMSNorm scale the block sees."""
    g = torch.Generator(device="cpu").manual_seed(7919 * seed + 3)
    return torch.randn(tokens, hidden, generator=g).to(torch.bfloat16)


def varlen_bounds(seed: int, tokens: int, n_seq: int = 8, lo: int = 64, hi: int = 1024):
    """Sequence bounds of a packed prefill: lengths uniform in [lo, hi], rescaled to sum to `tokens`."""
    rng = np.random.default_rng(seed)
    raw = rng.integers(lo, hi + 1, size=n_seq).astype(np.float64)
    lens = np.maximum(1, np.floor(raw * tokens / raw.sum()).astype(np.int64))
    lens[-1] += tokens - lens.sum()
    if lens[-1] < 1:
        raise ValueError("degenerate sequence split")
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)


def zipf_bias(seed: int, n_expert: int = E, s: float = 1.2):
    """Additive router bias 2*ln(w), w Zipf(s) weights over a random expert permutation."""
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, n_expert + 1, dtype=np.float64) ** s
    w /= w.sum()
    bias = np.empty(n_expert, dtype=np.float64)
    bias[rng.permutation(n_expert)] = 2.0 * np.log(w)
    bias -= bias.max()
    return bias.astype(np.float32)


def make_attention_weights(seed, hidden=2048, n_head=32, n_kv=4, head_dim=128, std=0.02):
    """Random-init weights of the attention half in the converted layout: BF16 matrices N(0, std),
    FP32 norm weights around 1."""
    g = torch.Generator(device="cpu").manual_seed(7000003 * seed + 29)
    w_qkv = (torch.randn((n_head + 2 * n_kv) * head_dim, hidden, generator=g) * std).to(torch.bfloat16)
    w_out = (torch.randn(hidden, n_head * head_dim, generator=g) * std).to(torch.bfloat16)
    attn_norm = 1.0 + 0.1 * torch.randn(hidden, generator=g)
    q_norm = 1.0 + 0.1 * torch.randn(head_dim, generator=g)
    k_norm = 1.0 + 0.1 * torch.randn(head_dim, generator=g)
    return dict(w_qkv=w_qkv, w_out=w_out, attn_norm=attn_norm.float(), q_norm=q_norm.float(), k_norm=k_norm.float())


def make_positions(seed, seq_bounds):
    """Text-like 3-axis positions: all three axes equal to the index inside the record, except a
    seeded stretch per record whose row/column axes differ (as image tokens' do)."""
    rng = np.random.default_rng(seed)
    b = np.asarray(seq_bounds)
    pos = np.zeros((3, b[-1]), np.int32)
    for lo, hi in zip(b[:-1], b[1:]):
        n = hi - lo
        pos[:, lo:hi] = np.arange(n)
        if n > 8:
            a = int(rng.integers(1, n // 2)); m = int(rng.integers(2, n - a))
            pos[1, lo + a:lo + a + m] = a + rng.integers(0, 16, m)
            pos[2, lo + a:lo + a + m] = a + rng.integers(0, 16, m)
    return pos
