"""CPU restatement of the Clef-Omni mixture-of-experts block.  TEST INFRASTRUCTURE ONLY.

Nothing the library ships imports this file: it is the checker used by the test-suite, by
the smoke check and by the CPU-baseline leg of the benchmark.  The product path is the CUDA
library and has no CPU fallback.

What is restated, and from where (paths inside the reference project):

* `route`            -- ref/omni_fp64.py:108-112: `logits = x @ W.T`, softmax over all
                        experts, top-k, renormalise by the selected sum.  The order inside
                        the top-k and the tie rule (descending logit, ties to the lowest
                        expert id) follow metal/clef.metal:2375-2392 and
                        tests/test_omni_routes.py:28-29, because `torch.topk` gives no tie
                        guarantee (metal/clef.metal:2383-2385).
* `experts`          -- ref/oracle_fp64.py:204-236: per expert, BF16 weights upcast to FP64
                        (ref/oracle_fp64.py:66-77), `act = silu(x @ gate.T) * (x @ up.T)`,
                        `out[rows] += (act @ down.T) * routing[rows, slot]`, residual added
                        once.  Expert tensors use the converted layout
                        `gate_up [E][2F][H]` (gate rows first) and `down [E][H][F]`
                        (tools/convert_omni.py:135-139).
* `rmsnorm`          -- ref/omni_fp64.py:31-32 (`x * rsqrt(mean(x^2) + eps) * weight`), the
                        `ffn_norm` in front of the block (metal/clef.metal:190-204 is the
                        reference's FP32 kernel for it).
* `assign_padded`    -- the serial oracle inside tests/test_omni_assign.m:44-56 (counts,
                        32-row padded offsets, row map with -1 padding, slots).
* `assign_canonical` -- the same stable counting sort without padding: the comparable form
                        of the permutation.
* `route_from_logits`-- the FP64 oracle inside tests/test_omni_moe.m:98-104 (stable
                        descending sort, weights = softmax over the eight selected).

Parity pins: `tests/golden/make_golden.py` imports the reference's own `ref/omni_fp64.py`
and stores what `route` returns there on seeded inputs; `tests/test_oracle.py` checks this
file against those vectors and against the known-answer case of
tests/test_omni_fp64.py:60-68.  The expert loop of ref/oracle_fp64.py cannot be imported on
its own (it sits inside a function that needs the 63.7 GB model snapshot), so for that part
the pin is the Hugging Face FP32 block that ref/omni.py:125-128 executes
(`Qwen3OmniMoeThinkerTextSparseMoeBlock`, transformers, third party), whose outputs on seeded
inputs are stored by the same script.
"""
from __future__ import annotations

import math

import numpy as np
import torch

H, F, E, TOP = 2048, 768, 128, 8


# --------------------------------------------------------------------------- inputs
# The seeded generators live with the library's workload definitions so that the benchmark
# can build the same bytes without importing this package.
from cleffa_b200.workloads import make_activations, make_weights, varlen_bounds, zipf_bias  # noqa: E402,F401


# --------------------------------------------------------------------------- routing
def topk_ordered(logits: torch.Tensor, k: int):
    """Indices of the k largest per row, descending, ties to the lowest index."""
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices
    return order[:, :k].contiguous()


def route(x: torch.Tensor, weight: torch.Tensor, top_k: int = TOP, bias=None):
    """FP64 router.  Returns logits [T,E], weights [T,k], ids [T,k], margin [T].

    Follows ref/omni_fp64.py:108-112; `bias` (not in the reference) is the additive
    per-expert term of the skewed-routing configuration.
    """
    x = x.to(torch.float64)
    weight = weight.to(torch.float64)
    logits = x @ weight.T
    if bias is not None:
        logits = logits + torch.as_tensor(bias, dtype=torch.float64)
    probs = logits.softmax(-1)
    ids = topk_ordered(logits, top_k)
    sel = probs.gather(1, ids)
    weights = sel / sel.sum(-1, keepdim=True)
    ranked = torch.sort(logits, dim=-1, descending=True).values
    margin = ranked[:, top_k - 1] - ranked[:, top_k] if logits.shape[1] > top_k else torch.full((len(x),), math.inf, dtype=torch.float64)
    return logits, weights, ids, margin


def route_from_logits(logits: np.ndarray, top_k: int = TOP):
    """tests/test_omni_moe.m:98-104: stable descending order; weights over the selected only.

    Returns (ids, weights, bad) where `bad` marks rows holding a nonfinite logit; those rows
    get the reference's fallback ids 0..k-1 and zero weights (metal/clef.metal:2362-2367).
    """
    logits = np.asarray(logits, dtype=np.float64)
    bad = ~np.isfinite(logits).all(-1)
    safe = np.where(bad[:, None], 0.0, logits)
    order = np.argsort(-safe, axis=-1, kind="stable")[:, :top_k]
    sel = np.take_along_axis(safe, order, -1)
    p = np.exp(sel - sel[:, :1])
    w = p / p.sum(-1, keepdims=True)
    order = np.where(bad[:, None], np.arange(top_k)[None, :], order)
    w = np.where(bad[:, None], 0.0, w)
    return order.astype(np.int32), w, bad


def adjacent_gaps(logits: torch.Tensor, top_k: int = TOP):
    """Gaps between consecutive ranked logits 1-2, 2-3, ..., k-(k+1) per row."""
    ranked = torch.sort(logits, dim=-1, descending=True).values[:, : top_k + 1]
    return ranked[:, :-1] - ranked[:, 1:]


# --------------------------------------------------------------------------- experts
def experts(x, ids, weights, gate_up, down, tokens=None, residual=None):
    """FP64 expert products and weighted combine (ref/oracle_fp64.py:211-232).

    `tokens` restricts the work to a subset of rows (each token is independent), which lets
    a full-size case be checked on a sample.  Returns [len(tokens), H] FP64.
    """
    x = x.to(torch.float64)
    ids = torch.as_tensor(ids, dtype=torch.long)
    weights = torch.as_tensor(weights, dtype=torch.float64)
    if tokens is not None:
        tokens = torch.as_tensor(tokens, dtype=torch.long)
        x, ids, weights = x[tokens], ids[tokens], weights[tokens]
    ffn = gate_up.shape[1] // 2
    out = torch.zeros(x.shape[0], down.shape[1], dtype=torch.float64)
    for e in torch.unique(ids).tolist():
        rows, slot = torch.where(ids == e)
        w = gate_up[e].to(torch.float64)
        chosen = x[rows]
        act = torch.nn.functional.silu(chosen @ w[:ffn].T) * (chosen @ w[ffn:].T)
        out[rows] += (act @ down[e].to(torch.float64).T) * weights[rows, slot, None]
    if residual is not None:
        res = torch.as_tensor(residual, dtype=torch.float64)
        out = out + (res if tokens is None else res[tokens])
    return out


def moe_block(x, router, gate_up, down, bias=None, tokens=None, residual=None):
    """Whole block in FP64: route every row, run the experts on `tokens` (default all)."""
    logits, weights, ids, margin = route(x, router, TOP, bias)
    out = experts(x, ids, weights, gate_up, down, tokens=tokens, residual=residual)
    return dict(logits=logits, weights=weights, ids=ids, margin=margin, out=out)


def moe_block_f32(x, router, gate_up, down, bias=None):
    """FP32 restatement on BF16-rounded weights: the arithmetic the reference's streamed
    PyTorch oracle runs per layer (ref/omni.py:57-66, 125-128).  Used as the timed CPU
    baseline when the Hugging Face block is not importable."""
    xf = x.to(torch.float32)
    logits = xf @ router.to(torch.float32).T
    if bias is not None:
        logits = logits + torch.as_tensor(bias, dtype=torch.float32)
    probs = logits.softmax(-1)
    sel, ids = probs.topk(TOP, dim=-1)
    weights = sel / sel.sum(-1, keepdim=True)
    ffn = gate_up.shape[1] // 2
    out = torch.zeros_like(xf)
    for e in torch.unique(ids).tolist():
        rows, slot = torch.where(ids == e)
        w = gate_up[e].to(torch.float32)
        chosen = xf[rows]
        act = torch.nn.functional.silu(chosen @ w[:ffn].T) * (chosen @ w[ffn:].T)
        out.index_add_(0, rows, (act @ down[e].to(torch.float32).T) * weights[rows, slot, None])
    return out, ids, weights


# --------------------------------------------------------------------------- permutation
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """FP64 RMSNorm over the last dimension (ref/omni_fp64.py:31-32)."""
    x = x.double()
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * weight.double()


def assign_padded(ids: np.ndarray, n_expert: int = E, pad: int = 32):
    """tests/test_omni_assign.m:44-56, word for word in behaviour: every expert run is padded
    to a multiple of `pad` rows, padding rows map to -1."""
    flat = np.asarray(ids, dtype=np.int64).reshape(-1)
    live = flat.size
    counts = np.bincount(flat, minlength=n_expert).astype(np.int32)
    offsets = np.zeros(n_expert + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(((counts + pad - 1) // pad) * pad)
    padded = live + min(live, n_expert) * (pad - 1)
    rowmap = np.full(padded, -1, dtype=np.int32)
    slots = np.empty(live, dtype=np.int32)
    cursor = np.zeros(n_expert, dtype=np.int64)
    top = np.asarray(ids).shape[-1] if np.asarray(ids).ndim == 2 else TOP
    for i in range(live):
        e = flat[i]
        row = offsets[e] + cursor[e]
        cursor[e] += 1
        rowmap[row] = i // top
        slots[i] = row
    return counts, offsets, rowmap, slots


def assign_canonical(ids: np.ndarray, n_expert: int = E):
    """Stable counting sort of assignment index i = t*k + rank by expert id, no padding.

    counts[e]; offsets = exclusive prefix sum of counts; slots[i] = destination row;
    rowmap[row] = token.  Vectorised (a stable argsort is the same permutation)."""
    arr = np.asarray(ids)
    top = arr.shape[-1] if arr.ndim == 2 else TOP
    flat = arr.astype(np.int64).reshape(-1)
    counts = np.bincount(flat, minlength=n_expert).astype(np.int32)
    offsets = np.zeros(n_expert + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    order = np.argsort(flat, kind="stable")
    slots = np.empty(flat.size, dtype=np.int32)
    slots[order] = np.arange(flat.size, dtype=np.int32)
    rowmap = (order // top).astype(np.int32)
    return counts, offsets, rowmap, slots


# --------------------------------------------------------------------------- comparisons
def compare_routing(ids_got, ids_ref, logits_ref, tol: float = 1e-6, top_k: int = TOP):
    """Index parity with the stated exemption: positions may differ only where the ranked
    reference logits that decide them are closer than `tol`.

    Returns (n_bad_rows, n_exempt_rows).  A row is exempt when every position that differs
    lies inside a run of ranked logits whose consecutive gaps are below `tol` (which includes
    the 8th/9th boundary)."""
    ids_got = np.asarray(ids_got, dtype=np.int64)
    ids_ref = np.asarray(ids_ref, dtype=np.int64)
    lg = logits_ref.detach().cpu().numpy() if isinstance(logits_ref, torch.Tensor) else np.asarray(logits_ref)
    differ = np.where((ids_got != ids_ref).any(-1))[0]
    bad = exempt = 0
    for t in differ:
        ranked = np.sort(lg[t])[::-1]
        order = np.argsort(-lg[t], kind="stable")
        ok = True
        for j in np.where(ids_got[t] != ids_ref[t])[0]:
            # the run of near-equal ranked values around rank j
            lo = j
            while lo > 0 and ranked[lo - 1] - ranked[lo] < tol:
                lo -= 1
            hi = j
            while hi + 1 < len(ranked) and ranked[hi] - ranked[hi + 1] < tol:
                hi += 1
            if hi == j and lo == j:
                ok = False
                break
            if ids_got[t, j] not in set(order[lo : hi + 1].tolist()):
                ok = False
                break
        if ok and len(set(ids_got[t].tolist())) == top_k:
            exempt += 1
        else:
            bad += 1
    return bad, exempt


def rel_l2(got, ref):
    got = torch.as_tensor(got, dtype=torch.float64)
    ref = torch.as_tensor(ref, dtype=torch.float64)
    return float((got - ref).norm() / ref.norm().clamp_min(1e-300))
