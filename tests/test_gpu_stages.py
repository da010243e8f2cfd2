"""Model-free stage parity on the GPU, through the C-ABI, against the CPU oracle: the CUDA
counterparts of the reference's tests/test_omni_assign.m, test_omni_router.m and the routing
part of test_omni_moe.m."""
import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import omni_oracle as orc
from test_oracle import SIZES, pattern_ids

pytestmark = pytest.mark.gpu
POISON = 0x5A5AC3C3            # tests/test_omni_assign.m:11
GUARD = 16


def guarded(words, shift=0, dtype=torch.int32):
    buf = torch.full((GUARD + shift + words + GUARD,), POISON, dtype=torch.int32, device="cuda")
    return buf, buf[GUARD + shift: GUARD + shift + words]


@pytest.mark.parametrize("pattern", range(7))
def test_assign_matches_serial_oracle_word_for_word(backend, pattern):
    # 15 sizes x 7 patterns x 2 input misalignments (tests/test_omni_assign.m:96-99)
    for rows in SIZES + [4096, 16384]:
        ids = pattern_ids(rows, pattern)
        counts, offsets, rowmap, slots = c_oracle.assign_canonical(ids)
        for shift in (0, 4):      # 16-byte steps: the library reads ids as int32 words
            in_buf, in_view = guarded(rows * 8, shift)
            in_view.copy_(torch.from_numpy(ids.reshape(-1)))
            outs = [guarded(n) for n in (128, 129, rows * 8, rows * 8)]
            backend.begin()
            backend.stage_assign(in_view.view(rows, 8), *[v for _, v in outs])
            backend.complete()
            for (buf, view), want in zip(outs, (counts, offsets, rowmap, slots)):
                assert np.array_equal(view.cpu().numpy(), want), (rows, pattern, shift)
                host = buf.cpu().numpy()
                assert (host[:GUARD] == POISON).all() and (host[-GUARD:] == POISON).all()
            assert np.array_equal(in_view.cpu().numpy(), ids.reshape(-1))


def test_assign_rejects_out_of_range_ids(backend):
    ids = torch.zeros(4, 8, dtype=torch.int32, device="cuda")
    ids[2, 3] = 128
    backend.begin()
    backend.stage_assign(ids)
    with pytest.raises(Exception, match="expert id"):
        backend.complete()
    backend.begin()
    backend.stage_assign(torch.zeros(4, 8, dtype=torch.int32, device="cuda"))
    backend.complete()           # the context stays usable


def route_modes(rows):
    t, e = np.meshgrid(np.arange(rows), np.arange(128), indexing="ij")
    base = (((e * 37 + t * 13) % 128) / 64.0).astype(np.float32)
    desc = (-e / 32.0).astype(np.float32)
    out = {0: (base, None), 1: (np.zeros((rows, 128), np.float32), None), 7: ((e / 32.0).astype(np.float32), None),
           8: (np.where((e >= 56) & (e < 64), 0.0, -16.0).astype(np.float32), None)}
    m2 = desc.copy(); m2[0, 8] = np.nextafter(m2[0, 7], np.float32(np.inf)); out[2] = (m2, None)
    m6 = desc.copy(); m6[0, 8] = m6[0, 7]; lo = np.zeros_like(m6); lo[0, 8] = 1e-9; out[6] = (m6, lo)
    return out


@pytest.mark.parametrize("rows", [1, 33, 1025])
def test_route_modes_match_oracle(backend, rows):
    for mode, (hi, lo) in route_modes(rows).items():
        want_ids, want_w, status = c_oracle.route(hi, lo)
        assert status == 0
        backend.begin()
        ids, w = backend.stage_route(torch.from_numpy(hi).cuda(), None if lo is None else torch.from_numpy(lo).cuda())
        backend.complete()
        assert np.array_equal(ids.cpu().numpy(), want_ids), mode          # tie order included
        assert np.abs(w.cpu().numpy().astype(np.float64) - want_w).max() < 2e-7, mode   # tests/test_omni_moe.m:108
        assert np.allclose(w.sum(-1).cpu().numpy(), 1, atol=1e-6)


@pytest.mark.parametrize("value", [np.nan, np.inf, -np.inf])
def test_route_reports_nonfinite_logits(backend, value):
    hi, _ = route_modes(40)[0]
    hi = hi.copy(); hi[17, 11] = value
    backend.begin()
    ids, w = backend.stage_route(torch.from_numpy(hi).cuda())
    with pytest.raises(Exception, match="nonfinite"):
        backend.complete()
    assert ids[17].tolist() == list(range(8)) and not w[17].any()       # clef.metal:2365
    want_ids, _, _ = c_oracle.route(hi, None)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    backend.begin()
    backend.complete()           # begin clears the status word


def lcg_samples(n, state=97):
    out = np.empty(n, np.float32)
    for i in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(((state >> 16) - 32768)) * np.float32(.001234567)
    return out, state


def test_exact_router_logits_within_1e9(backend):
    # tests/test_omni_router.m: K=2048, N=128, rows 31..33; here activations are BF16-rounded
    xs, st = lcg_samples(33 * 2048)
    ws, _ = lcg_samples(128 * 2048, st)
    x = torch.from_numpy(xs).reshape(33, 2048).bfloat16()
    w = torch.from_numpy(ws * np.float32(.01)).reshape(128, 2048).bfloat16()
    zero_gu = torch.zeros(128, 1536, 2048, dtype=torch.bfloat16, device="cuda")
    zero_dn = torch.zeros(128, 2048, 768, dtype=torch.bfloat16, device="cuda")
    backend.bind_layer(3, w.cuda(), zero_gu, zero_dn)
    want = c_oracle.router_dot(x.float().numpy(), w.view(torch.int16).numpy().view(np.uint16))
    previous = None
    for rows in (31, 32, 33):
        backend.begin()
        got = backend.stage_router(3, x[:rows].cuda().contiguous())
        backend.complete()
        got = got.cpu().numpy()
        assert np.isfinite(got).all() and np.abs(got - want[:rows]).max() < 1e-9
        if previous is not None:
            assert np.array_equal(previous, got[: rows - 1])           # neighbour rows do not change a row
        previous = got
