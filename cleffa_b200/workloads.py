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
