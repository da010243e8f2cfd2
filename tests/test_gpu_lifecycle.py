"""Arena lifecycle, host-side fault injection and route capture: the CUDA counterparts of the
reference's tests/test_omni_buffers.m, test_gpu_fail.sh and test_omni_routes.py.  Failures are
made on the host (an allocation or a launch that is refused); no kernel is made to fault."""
import json
import math

import numpy as np
import pytest
import torch

from cleffa_b200 import OmniBackend, OmniError
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu


def test_reserve_validates_geometry_and_is_idempotent():
    with OmniBackend(0) as b:
        for kw in (dict(H=1024), dict(ffn=512), dict(n_expert=64), dict(n_expert_used=4)):
            with pytest.raises(OmniError, match="invalid Omni scratch dimensions"):
                b.reserve(8, **kw)
        with pytest.raises(OmniError, match="invalid Omni scratch dimensions"):
            b.reserve(0)
        assert b.arena_bytes() == 0
        b.reserve(8)
        size = b.arena_bytes()
        b.reserve(100000)                     # arena does not depend on T (tests/test_omni_buffers.m:41-46)
        assert b.arena_bytes() == size > 0
        b.free()
        assert b.arena_bytes() == 0


def test_every_failing_allocation_leaves_the_previous_state():
    with OmniBackend(0) as b:
        n = 1
        while True:
            b.set_option("alloc_fail_at", n)
            try:
                b.reserve(8)
            except OmniError as e:
                assert "previous buffers kept" in str(e) and b.arena_bytes() == 0
                n += 1
                continue
            break
        assert n == 21                        # 20 arena buffers
        b.set_option("alloc_fail_at", 0)
        assert b.arena_bytes() > 0


def test_failed_launch_surfaces_at_complete_and_next_pass_is_identical(bound0):
    b = bound0
    x = orc.make_activations(31, 200).cuda()
    def run():
        out = torch.zeros(200, 2048, device="cuda")
        b.begin(); b.encode_moe(0, x, out); b.complete()
        return out.cpu()
    good = run()
    for n in (1, 2, 4, 6):                    # first, mid and last of the six host launches of a pass (the sort's kernels count as one)
        b.set_option("launch_fail_at", n)
        try:
            b.begin()
            out = torch.zeros(200, 2048, device="cuda")
            with pytest.raises(OmniError, match="failed"):
                b.encode_moe(0, x, out)
            with pytest.raises(OmniError, match="failed"):
                b.complete()
        finally:
            b.set_option("launch_fail_at", 0)
        assert torch.equal(run(), good)


def check_route_rows(lines, first_token):
    """The reference's own checks on a route dump (tests/test_omni_routes.py:21-31)."""
    for i, row in enumerate(lines):
        assert (row["layer"], row["token"]) == (0, first_token + i)
        assert len(row["logits"]) == 128 and len(set(row["ids"])) == 8
        assert all(math.isfinite(v) for v in row["logits"] + row["weights"])
        assert abs(sum(row["weights"]) - 1) < 1e-6
        order = sorted(range(128), key=lambda e: (-row["logits"][e], e))
        assert row["ids"] == order[:8], (row["token"], row["ids"], order[:9])
        assert row["margin"] == row["logits"][order[7]] - row["logits"][order[8]]


def test_trace_reserve_and_dump(bound0, tmp_path):
    b = bound0
    T, rows = 300, 3
    with pytest.raises(OmniError, match="no captured Omni routes"):
        b.dump_routes(tmp_path / "none.jsonl")
    with pytest.raises(OmniError, match="invalid Omni trace dimensions"):
        b.trace_reserve(0, 1, 3)
    b.trace_reserve(T, 1, rows)
    b.set_option("alloc_fail_at", 1)
    with pytest.raises(OmniError, match="previous buffers kept"):
        b.trace_reserve(T, 1, 5)
    b.set_option("alloc_fail_at", 0)
    x = orc.make_activations(41, T).cuda()
    out = torch.zeros(T, 2048, device="cuda")
    b.begin(); b.encode_moe(0, x, out); b.complete()
    path = tmp_path / "routes.jsonl"
    b.dump_routes(path)
    lines = [json.loads(s) for s in path.read_text().splitlines()]
    assert len(lines) == rows
    ids = b.read("ids", T)
    check_route_rows(lines, T - rows)
    for i, row in enumerate(lines):
        assert row["ids"] == ids[T - rows + i].tolist()
    with pytest.raises(OmniError, match="cannot open"):
        b.dump_routes(tmp_path)               # a directory is not writable as a file
    b.trace_reserve(T, 1, rows, enabled=False)
    with pytest.raises(OmniError, match="no captured Omni routes"):
        b.dump_routes(path)


@pytest.mark.parametrize("exact", [0, 1])
def test_dumped_ids_follow_from_dumped_logits(bound0, weights0, tmp_path, exact):
    """Rows the exact pass re-decided carry ids chosen from FP64 logits; the dump must show
    logits (hi + low) from which exactly those ids follow, for every row of a capture large
    enough to hold hundreds of re-decided rows (tests/test_omni_routes.py:28-30)."""
    b = bound0
    T = 2500
    b.trace_reserve(T, 1, 0)                  # 0 = every row
    b.set_option("router_exact", exact)
    try:
        x = orc.make_activations(43, T)
        out = torch.zeros(T, 2048, device="cuda")
        b.begin(); b.encode_moe(0, x.cuda(), out); b.complete()
        assert int(b.read("rechecked")[0]) >= (T if exact else 100)
        path = tmp_path / "routes.jsonl"
        b.dump_routes(path)
        lines = [json.loads(s) for s in path.read_text().splitlines()]
        assert len(lines) == T
        check_route_rows(lines, 0)
        # and the dumped logits are the oracle's: to the tensor-core accumulation error
        # everywhere, and the ones the exact pass evaluated (with router_exact every row's
        # selected eight at least) to the rounding of the float pair
        logits, _, ids_ref, _ = orc.route(x, weights0[0])
        got = np.array([r["logits"] for r in lines])
        assert np.abs(got - logits.numpy()).max() < 5e-4 / 4
        if exact:
            sel = np.array([r["ids"] for r in lines])
            assert np.abs(np.take_along_axis(got - logits.numpy(), sel, 1)).max() < 1e-9
        bad, _ = orc.compare_routing(np.array([r["ids"] for r in lines], np.int32), ids_ref.numpy(), logits)
        assert bad == 0
    finally:
        b.set_option("router_exact", 0)
        b.trace_reserve(T, 1, 0, enabled=False)


def test_router_error_bound_is_checked_not_assumed(bound0, weights0):
    """The near-tie test trusts a bound on the tensor-core accumulation error.  The exact pass
    compares every logit it evaluates with the approximate one and fails the pass when the
    bound does not hold; it never lets wrong ids through silently."""
    b = bound0
    T = 1024
    x = orc.make_activations(47, T)
    out = torch.zeros(T, 2048, device="cuda")
    # a bound far below the real error (1e-8): the pass must be refused
    b.set_option("router_eps", 10)
    try:
        b.begin(); b.encode_moe(0, x.cuda(), out)
        with pytest.raises(OmniError, match="router accumulation error exceeded"):
            b.complete()
    finally:
        b.set_option("router_eps", 500000)    # 5e-4, the default
    # activations 64 times larger (logits and their error grow alike): the default bound scales
    # with the row's largest |logit|, so the ids are still the oracle's -- or the pass says so
    x64 = (x.float() * 64).to(torch.bfloat16)
    out.zero_()
    b.begin(); b.encode_moe(0, x64.cuda(), out)
    try:
        b.complete()
    except OmniError as e:
        assert "router accumulation error exceeded" in str(e)
        return
    logits, _, ids_ref, _ = orc.route(x64, weights0[0])
    bad, _ = orc.compare_routing(b.read("ids", T), ids_ref.numpy(), logits)
    assert bad == 0


def test_failed_pass_does_not_publish_a_trace(bound0, tmp_path):
    b = bound0
    b.trace_reserve(64, 1, 2)
    hi = torch.zeros(64, 2048, dtype=torch.bfloat16, device="cuda")
    hi[5, 7] = float("nan")
    out = torch.zeros(64, 2048, device="cuda")
    b.begin(); b.encode_moe(0, hi, out)
    with pytest.raises(OmniError, match="nonfinite"):
        b.complete()
    with pytest.raises(OmniError, match="no captured Omni routes"):
        b.dump_routes(tmp_path / "r.jsonl")
    b.trace_reserve(64, 1, 2, enabled=False)


def test_keepalive_does_not_change_results(bound0):
    x = orc.make_activations(51, 64).cuda()
    a = torch.zeros(64, 2048, device="cuda"); c = torch.zeros(64, 2048, device="cuda")
    bound0.begin(); bound0.encode_moe(0, x, a); bound0.complete()
    bound0.keepalive()
    bound0.begin(); bound0.keepalive(); bound0.encode_moe(0, x, c); bound0.keepalive(); bound0.complete()
    assert torch.equal(a, c)


def test_invalid_dispatch_is_refused(bound0):
    x = torch.zeros(8, 2048, dtype=torch.bfloat16, device="cuda"); out = torch.zeros(8, 2048, device="cuda")
    with pytest.raises(OmniError, match="invalid Omni layer dispatch"):
        bound0.encode_moe(77, x, out)
    with pytest.raises(OmniError, match="sequence bounds"):
        bound0.encode_moe(0, x, out, seq_bounds=np.array([0, 5, 5, 8], np.int32))
    with pytest.raises(OmniError, match="sequence bounds"):
        bound0.encode_moe(0, x, out, seq_bounds=np.array([0, 9], np.int32))
