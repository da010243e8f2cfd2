"""CPU checks: the restated oracle against the reference's own outputs (tests/golden/*.npz,
made by tests/golden/make_golden.py from ref/omni_fp64.py and the Hugging Face block that
ref/omni.py drives) and against the known-answer cases of the reference's tests."""
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import omni_oracle as orc

GOLDEN = Path(__file__).resolve().parent / "golden"


def sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


@pytest.fixture(scope="module")
def c1(weights0):
    router, gate_up, down = weights0
    return dict(router=router, gate_up=gate_up, down=down, x=orc.make_activations(0, 512))


def test_inputs_reproduce_the_golden_bytes(c1):
    g = np.load(GOLDEN / "route_c1.npz")
    assert sha(c1["x"]) == str(g["sha_x"]) and sha(c1["router"]) == str(g["sha_router"])
    assert sha(c1["gate_up"]) == str(g["sha_gate_up"]) and sha(c1["down"]) == str(g["sha_down"])


def test_route_matches_reference_route_on_config1(c1):
    g = np.load(GOLDEN / "route_c1.npz")
    logits, weights, ids, margin = orc.route(c1["x"], c1["router"])
    assert np.array_equal(ids.numpy(), g["ids"].astype(np.int64))
    assert np.array_equal(weights.numpy(), g["weights"])          # same FP64 arithmetic, bit for bit
    assert np.array_equal(torch.sort(logits, -1, descending=True).values[:, :9].numpy(), g["top9"])
    assert np.array_equal(margin.numpy(), g["margin"])
    assert np.array_equal(logits[:8].numpy(), g["logits_rows"])


def test_route_matches_reference_route_on_small_problems():
    g = np.load(GOLDEN / "route_small.npz")
    for name, k in (("a", 2), ("b", 4)):
        logits, weights, ids, _ = orc.route(torch.from_numpy(g[f"{name}_x"]), torch.from_numpy(g[f"{name}_w"]), k)
        assert np.array_equal(logits.numpy(), g[f"{name}_logits"])
        assert np.array_equal(ids.numpy(), g[f"{name}_ids"].astype(np.int64))
        assert np.array_equal(weights.numpy(), g[f"{name}_weights"])


def test_router_keeps_sub_fp32_differences():
    # tests/test_omni_fp64.py:60-68 of the reference
    x = torch.eye(3, dtype=torch.float64)
    w = torch.tensor([[1, 0, 2], [1 + 1e-9, 0, -2], [0, 1, 1]], dtype=torch.float64)
    logits, weights, ids, _ = orc.route(x, w, 2)
    assert ids[0].tolist() == [1, 0]
    assert torch.equal(logits, x @ w.T)
    expected = logits.softmax(-1).gather(1, ids)
    expected /= expected.sum(-1, keepdim=True)
    assert torch.equal(weights, expected)


def test_block_matches_hugging_face_fp32_block(c1):
    g = np.load(GOLDEN / "block_c1.npz")
    res = orc.moe_block(c1["x"], c1["router"], c1["gate_up"], c1["down"])
    if g["hf_ids"].size:
        assert np.array_equal(np.sort(res["ids"].numpy(), -1), np.sort(g["hf_ids"].astype(np.int64), -1))
    rows = g["rows"]
    assert orc.rel_l2(res["out"][rows], g["y_rows"]) < 2e-6      # FP32 block against FP64 restatement
    assert orc.rel_l2(res["out"].sum(0), g["col_sum"]) < 2e-6
    # the subset form used at full size agrees with the full evaluation
    sub = orc.experts(c1["x"], res["ids"], res["weights"], c1["gate_up"], c1["down"], tokens=rows)
    assert orc.rel_l2(sub, res["out"][rows]) < 1e-13              # BLAS blocking differs, nothing else
    f32, ids32, _ = orc.moe_block_f32(c1["x"], c1["router"], c1["gate_up"], c1["down"])
    assert orc.rel_l2(f32, res["out"]) < 2e-6


# ---- permutation: the serial oracle of tests/test_omni_assign.m, 7 patterns x 15 sizes
def expert_id(i, pattern):
    if pattern == 0: return (i * 37 + (i // 8) * 13) % 128
    if pattern == 1: return i % 8
    if pattern == 2: return 120 + i % 8
    if pattern == 3: return 56 + i % 8
    if pattern == 4: return (i // 32) % 128
    if pattern == 5: return 127
    return ((i * 2654435761) % (1 << 32) >> 16) % 128


SIZES = [1, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255, 256, 257, 1023, 1024]


def pattern_ids(rows, pattern):
    return np.array([expert_id(i, pattern) for i in range(rows * 8)], dtype=np.int32).reshape(rows, 8)


@pytest.mark.parametrize("pattern", range(7))
def test_assign_c_and_numpy_agree(pattern):
    for rows in SIZES:
        ids = pattern_ids(rows, pattern)
        for a, b in zip(orc.assign_padded(ids), c_oracle.assign_padded(ids)):
            assert np.array_equal(a, b)
        can_np, can_c = orc.assign_canonical(ids), c_oracle.assign_canonical(ids)
        for a, b in zip(can_np, can_c):
            assert np.array_equal(a, b)
        counts, offsets, rowmap, slots = can_np
        # canonical and padded forms are the same permutation up to the padding
        pc, po, prm, ps = orc.assign_padded(ids)
        assert np.array_equal(counts, pc)
        e_of = ids.reshape(-1)
        assert np.array_equal(slots - offsets[e_of], ps - po[e_of])
        assert np.array_equal(rowmap[slots], np.arange(rows * 8) // 8)
        assert np.array_equal(np.sort(slots), np.arange(rows * 8))


def test_route_from_logits_modes_agree_with_c():
    rows = 9
    t, e = np.meshgrid(np.arange(rows), np.arange(128), indexing="ij")
    modes = {0: ((e * 37 + t * 13) % 128) / 64.0, 1: np.zeros((rows, 128)), 2: -e / 32.0, 7: e / 32.0,
             8: np.where((e >= 56) & (e < 64), 0.0, -16.0)}
    for mode, lg in modes.items():
        hi = lg.astype(np.float32)
        lo = np.zeros_like(hi)
        if mode == 2:
            hi[0, 8] = np.nextafter(hi[0, 7], np.float32(np.inf))
        ids, w, bad = orc.route_from_logits(hi.astype(np.float64) + lo)
        cids, cw, status = c_oracle.route(hi, lo)
        assert status == 0 and not bad.any()
        assert np.array_equal(ids, cids) and np.allclose(w, cw, atol=1e-15)
    hi = modes[2].astype(np.float32).copy(); lo = np.zeros_like(hi)
    hi[0, 8] = hi[0, 7]; lo[0, 8] = 1e-9                       # mode 6: tie broken only by the low word
    ids, _, _ = c_oracle.route(hi, lo)
    assert ids[0, 7] == 8 and 7 not in ids[0].tolist()
    for v in (np.nan, np.inf, -np.inf):                         # modes 3-5
        hi = modes[0].astype(np.float32).copy(); hi[0, 11] = v
        ids, w, status = c_oracle.route(hi, None)
        assert status == 1 and ids[0].tolist() == list(range(8)) and not w[0].any()
        ids2, w2, bad = orc.route_from_logits(hi)
        assert bad[0] and np.array_equal(ids2, ids)


def test_small_moe_c_oracle_against_torch_restatement():
    # tests/test_omni_moe.m shapes: H=32, F=16, closed-form binary fractions (exact in BF16)
    Hn, Fn, rows = 32, 16, 17
    sample = lambda i: ((i * 19 + 7) % 31 - 15) / 64.0
    x = np.array([sample(i) for i in range(rows * Hn)], np.float32).reshape(rows, Hn)
    res = np.array([sample(i + 2) for i in range(rows * Hn)], np.float32).reshape(rows, Hn)
    gu = torch.tensor([sample(i) for i in range(128 * 2 * Fn * Hn)], dtype=torch.float32).reshape(128, 2 * Fn, Hn)
    dn = torch.tensor([sample(i + 5) for i in range(128 * Hn * Fn)], dtype=torch.float32).reshape(128, Hn, Fn)
    assert torch.equal(gu.bfloat16().float(), gu) and torch.equal(dn.bfloat16().float(), dn)
    t, e = np.meshgrid(np.arange(rows), np.arange(128), indexing="ij")
    ids, w, _ = orc.route_from_logits(((e * 37 + t * 13) % 128) / 64.0)
    bits = lambda v: v.bfloat16().view(torch.int16).numpy().view(np.uint16)
    y_c = c_oracle.moe_rows(x, res, ids, w, bits(gu), bits(dn))
    y_t = orc.experts(torch.from_numpy(x), ids, w, gu.bfloat16(), dn.bfloat16(), residual=res)
    assert np.abs(y_c - y_t.numpy()).max() < 1e-12


def test_compare_routing_exemption():
    lg = np.zeros((2, 128)); lg[:, :9] = np.arange(9, 0, -1)[None] * 1.0
    lg[1, 8] = lg[1, 7] - 5e-7                                   # 8th and 9th closer than 1e-6
    ref = np.argsort(-lg, kind="stable")[:, :8]
    got = ref.copy(); got[1, 7] = 8
    assert orc.compare_routing(got, ref, lg) == (0, 1)
    got[0, 7] = 8
    assert orc.compare_routing(got, ref, lg) == (1, 1)


def test_rmsnorm_matches_reference_rms():
    # ref/omni_fp64.py:31-32 on nine seeded rows (tiny, large, mostly-zero and all-zero among them)
    g = np.load(GOLDEN / "rms_small.npz")
    got = orc.rmsnorm(torch.from_numpy(g["x"]), torch.from_numpy(g["w"]), float(g["eps"]))
    assert np.array_equal(got.numpy(), g["y"])
    assert np.all(got.numpy()[4] == 0.0)            # all-zero row stays zero (eps keeps the rsqrt finite)


def test_rmsnorm_c_restatement_agrees():
    # summation order differs from torch's (serial here), so agreement is to rounding, not bitwise
    g = np.load(GOLDEN / "rms_small.npz")
    got = c_oracle.rmsnorm(g["x"], g["w"], float(g["eps"]))
    scale = np.abs(g["y"]).max(axis=1, keepdims=True) + 1e-300
    assert (np.abs(got - g["y"]) / scale).max() < 1e-14
    assert np.all(got[4] == 0.0)


def test_attention_oracle_reproduces_the_reference_fp64_functions():
    """oracle/omni_attn_oracle.py against what the reference's own text_attention / rotary
    (ref/omni_fp64.py:78-105) returned on a small seeded problem (tests/golden/make_golden_attn.py):
    rotary tables bit for bit, the layer output to FP64 rounding (the reference's attention runs an
    online softmax over key blocks, the restatement a plain softmax per record)."""
    from pathlib import Path
    from oracle import omni_attn_oracle as ao
    g = np.load(Path(__file__).resolve().parent / "golden" / "attn_small.npz")
    H, nh, nkv, hd, T, s0, s1, s2 = (int(v) for v in g["geometry"])
    sections = (s0, s1, s2)
    cos, sin = ao.rotary(g["positions"], hd, float(g["theta"]), sections)
    assert np.array_equal(cos.numpy(), g["cos"]) and np.array_equal(sin.numpy(), g["sin"])
    w_qkv = torch.from_numpy(np.concatenate([g["w_q"], g["w_k"], g["w_v"]]))
    r = ao.attention_half(torch.from_numpy(g["hidden"]), g["positions"], [0, T], torch.from_numpy(g["attn_norm"]), w_qkv,
                          torch.from_numpy(g["q_norm"]), torch.from_numpy(g["k_norm"]), torch.from_numpy(g["w_o"]), nh, nkv, hd,
                          float(g["theta"]), sections, float(g["eps"]))
    assert np.abs(r["out"].numpy() - g["out"]).max() < 1e-12
    # a packed batch of two records equals the two records run alone (per-record causal masks)
    x = torch.from_numpy(g["hidden"])
    both = ao.attention_half(x, g["positions"], [0, 20, T], torch.from_numpy(g["attn_norm"]), w_qkv, torch.from_numpy(g["q_norm"]),
                             torch.from_numpy(g["k_norm"]), torch.from_numpy(g["w_o"]), nh, nkv, hd, float(g["theta"]), sections, float(g["eps"]))
    first = ao.attention_half(x[:20], g["positions"][:, :20], [0, 20], torch.from_numpy(g["attn_norm"]), w_qkv, torch.from_numpy(g["q_norm"]),
                              torch.from_numpy(g["k_norm"]), torch.from_numpy(g["w_o"]), nh, nkv, hd, float(g["theta"]), sections, float(g["eps"]))
    assert np.abs(both["out"][:20].numpy() - first["out"].numpy()).max() < 1e-13


def test_attention_oracle_rows_agree_with_the_whole_record():
    """attention_half_rows (what the T=16384 GPU test samples with) is attention_half restricted to
    the chosen rows, on the golden problem's weights and on a longer seeded record."""
    from pathlib import Path
    from oracle import omni_attn_oracle as ao
    g = np.load(Path(__file__).resolve().parent / "golden" / "attn_small.npz")
    H, nh, nkv, hd, T, s0, s1, s2 = (int(v) for v in g["geometry"])
    w_qkv = torch.from_numpy(np.concatenate([g["w_q"], g["w_k"], g["w_v"]]))
    args = (torch.from_numpy(g["attn_norm"]), w_qkv, torch.from_numpy(g["q_norm"]), torch.from_numpy(g["k_norm"]), torch.from_numpy(g["w_o"]),
            nh, nkv, hd, float(g["theta"]), (s0, s1, s2), float(g["eps"]))
    rows = np.array([0, 1, T // 2, T - 1])
    part = ao.attention_half_rows(torch.from_numpy(g["hidden"]), g["positions"], rows, *args)
    assert np.abs(part.numpy() - g["out"][rows]).max() < 1e-12
    w = ao.make_attention_weights(3)
    x = torch.randn(200, 2048, generator=torch.Generator().manual_seed(3))
    pos = ao.make_positions(3, [0, 200])
    full = ao.attention_half(x, pos, [0, 200], w["attn_norm"], w["w_qkv"], w["q_norm"], w["k_norm"], w["w_out"], 32, 4)
    rows = np.array([0, 127, 128, 199])
    part = ao.attention_half_rows(x, pos, rows, w["attn_norm"], w["w_qkv"], w["q_norm"], w["k_norm"], w["w_out"], 32, 4)
    assert (part - full["out"][rows]).abs().max() < 1e-12
