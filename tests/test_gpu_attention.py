"""The attention half in front of the MoE block on the GPU, through the C-ABI, against the FP64
oracle (oracle/omni_attn_oracle.py, pinned on the reference's own ref/omni_fp64.py functions).

Gates: what the half adds to the residual stream within relative L2 1e-2 of FP64 (BF16 operands on
the tensor cores, FP32 softmax and accumulation; measured ~4e-3), the intermediate q|k|v projections
and attention outputs within the same bound, a record's rows bitwise independent of what it is
packed with, nonfinite inputs reported through the status word."""
import numpy as np
import pytest
import torch

from cleffa_b200 import OmniError
from oracle import omni_attn_oracle as ao
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu
GATE = 1e-2


@pytest.fixture(scope="module")
def attn(backend):
    w = ao.make_attention_weights(0)
    backend.bind_attention(0, w["attn_norm"], w["w_qkv"], w["w_out"], w["q_norm"], w["k_norm"])
    return backend, w


def run(b, x, pos, bounds):
    xd = x.clone().cuda()
    pd = torch.from_numpy(np.ascontiguousarray(pos.T)).cuda()          # [T][3]
    b.begin()
    b.encode_attention(0, xd, pd, np.asarray(bounds, np.int32))
    b.complete()
    return xd.cpu()


def bf16_rows(b, what, T, cols):
    raw = np.empty((T, cols), np.uint16)
    import ctypes as C
    ok = b.lib.clef_omni_read(b._g, what.encode(), C.c_void_p(raw.ctypes.data), raw.nbytes, b._err, 512)
    assert ok, b._err.value
    return torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16).double()


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("bounds", [[0, 1], [0, 37], [0, 128], [0, 129], [0, 100, 300], [0, 64, 65, 500, 1000]])
def test_attention_half_matches_fp64_oracle(attn, bounds):
    b, w = attn
    T = bounds[-1]
    x = torch.randn(T, 2048, generator=torch.Generator().manual_seed(T))
    pos = ao.make_positions(T, bounds)
    got = run(b, x, pos, bounds)
    ref = ao.attention_half(x, pos, bounds, w["attn_norm"], w["w_qkv"], w["q_norm"], w["k_norm"], w["w_out"], 32, 4)
    p_ref = ref["xn"].to(torch.bfloat16).double() @ w["w_qkv"].double().T       # what the projection sees: BF16-rounded rows
    assert rel(bf16_rows(b, "attn_qkv", T, 5120), p_ref) < GATE
    assert rel(bf16_rows(b, "attn_out", T, 4096), ref["attn"]) < GATE
    assert rel(got - x, ref["out"] - x.double()) < GATE
    assert torch.isfinite(got).all()


def test_config2_T4096_eight_records(attn):
    """The packed prefill of BASELINE configuration 2 (T=4096 as 8 records, seed 1), every row
    against the FP64 oracle."""
    from cleffa_b200 import workloads
    b, w = attn
    bounds = [int(v) for v in workloads.varlen_bounds(1, 4096)]
    x = torch.randn(4096, 2048, generator=torch.Generator().manual_seed(41))
    pos = ao.make_positions(41, bounds)
    got = run(b, x, pos, bounds)
    ref = ao.attention_half(x, pos, bounds, w["attn_norm"], w["w_qkv"], w["q_norm"], w["k_norm"], w["w_out"], 32, 4)
    assert rel(bf16_rows(b, "attn_out", 4096, 4096), ref["attn"]) < GATE
    assert rel(got - x, ref["out"] - x.double()) < GATE
    for lo, hi in zip(bounds[:-1], bounds[1:]):                        # and record by record
        assert rel(got[lo:hi] - x[lo:hi], ref["out"][lo:hi] - x[lo:hi].double()) < GATE


def test_config3_T16384_one_record_sampled(attn):
    """One record of 16,384 tokens (BASELINE configuration 3's batch): 128 key blocks per query
    tile.  96 sampled rows -- the first and last rows, both sides of tile and block boundaries,
    random ones -- against the FP64 oracle's rows."""
    b, w = attn
    T = 16384
    x = torch.randn(T, 2048, generator=torch.Generator().manual_seed(42))
    pos = ao.make_positions(42, [0, T])
    got = run(b, x, pos, [0, T])
    rng = np.random.default_rng(42)
    rows = np.unique(np.concatenate([[0, 1, 127, 128, 129, 255, 256, 8191, 8192, T - 129, T - 128, T - 2, T - 1],
                                     rng.integers(0, T, 83)]))
    ref = ao.attention_half_rows(x, pos, rows, w["attn_norm"], w["w_qkv"], w["q_norm"], w["k_norm"], w["w_out"], 32, 4)
    delta, want = got[rows] - x[rows], ref - x[rows].double()
    assert rel(delta, want) < GATE
    worst = max(rel(delta[i], want[i]) for i in range(len(rows)))
    assert worst < 3 * GATE, worst
    assert torch.isfinite(got).all()


def test_records_do_not_depend_on_their_neighbours(attn):
    b, w = attn
    bounds = [0, 200, 333, 700]
    x = torch.randn(700, 2048, generator=torch.Generator().manual_seed(5))
    pos = ao.make_positions(5, bounds)
    packed = run(b, x, pos, bounds)
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        alone = run(b, x[lo:hi].contiguous(), pos[:, lo:hi], [0, hi - lo])
        assert torch.equal(alone, packed[lo:hi])
    assert torch.equal(run(b, x, pos, bounds), packed)                 # and the pass is repeatable


def test_nonfinite_projection_is_reported(attn):
    b, _ = attn
    x = torch.randn(64, 2048, generator=torch.Generator().manual_seed(6))
    x[7, 100] = float("inf")
    xd = x.cuda()
    pd = torch.zeros(64, 3, dtype=torch.int32, device="cuda")
    b.begin()
    b.encode_attention(0, xd, pd)
    with pytest.raises(OmniError, match="nonfinite Omni attention or router values"):
        b.complete()


def test_invalid_attention_dispatch_is_refused(attn):
    b, _ = attn
    x = torch.zeros(8, 2048, device="cuda"); pd = torch.zeros(8, 3, dtype=torch.int32, device="cuda")
    with pytest.raises(OmniError, match="no attention tensors bound"):
        b.encode_attention(3, x, pd)
    with pytest.raises(OmniError, match="sequence bounds"):
        b.encode_attention(0, x, pd, np.array([0, 9], np.int32))
    # 600 one-token records: their value columns, 64 apart, do not fit one pass
    x = torch.zeros(600, 2048, device="cuda"); pd = torch.zeros(600, 3, dtype=torch.int32, device="cuda")
    with pytest.raises(OmniError, match="too many records"):
        b.encode_attention(0, x, pd, np.arange(601, dtype=np.int32))
    b.begin()
    b.encode_attention(0, x, pd, np.arange(0, 601, 2, dtype=np.int32))     # 300 records of two tokens fit
    b.complete()


def test_a_layer_is_attention_then_norm_and_moe(attn, weights0):
    """One decoder layer as the reference runs it (clef_omni_encode_layer): attention half, then
    norm(ffn_norm) + MoE, both adding into the FP32 residual stream; each half checked on the input
    the GPU fed it."""
    b, w = attn
    T, bounds = 160, [0, 50, 160]
    b.bind_layer(2, *weights0)
    norm_w = 1.0 + 0.1 * torch.randn(2048, generator=torch.Generator().manual_seed(8))
    b.bind_norm(2, norm_w)
    b.bind_attention(2, w["attn_norm"], w["w_qkv"], w["w_out"], w["q_norm"], w["k_norm"])
    x = torch.randn(T, 2048, generator=torch.Generator().manual_seed(9))
    pos = ao.make_positions(9, bounds)
    xd = x.clone().cuda()
    pd = torch.from_numpy(np.ascontiguousarray(pos.T)).cuda()
    b.begin()
    b.encode_attention(2, xd, pd, np.asarray(bounds, np.int32))
    b.complete()                                                       # the library runs on its own stream: finish before reading
    mid = xd.clone()
    b.begin()
    b.encode_norm_moe(2, xd, np.asarray(bounds, np.int32))
    b.complete()
    ref = ao.attention_half(x, pos, bounds, w["attn_norm"], w["w_qkv"], w["q_norm"], w["k_norm"], w["w_out"], 32, 4)
    assert rel(mid.cpu() - x, ref["out"] - x.double()) < GATE
    xn = orc.rmsnorm(mid.cpu(), norm_w).to(torch.bfloat16)
    ids = b.read("ids", T); wts = b.read("weights", T)
    moe = orc.experts(xn, ids.astype(np.int64), wts.astype(np.float64), weights0[1], weights0[2])
    assert rel(xd.cpu() - mid.cpu(), moe) < GATE
    # the one-call form (clef_omni_encode_layer) is those two calls
    one = x.clone().cuda()
    b.begin()
    b.encode_layer(2, one, pd, np.asarray(bounds, np.int32))
    b.complete()
    assert torch.equal(one, xd)
