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
        assert n == 20                        # 19 arena buffers
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
    for n in (1, 2, 4, 6, 7):                 # first, mid and last of the seven launches of a pass
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
    for i, row in enumerate(lines):          # tests/test_omni_routes.py:21-31
        assert (row["layer"], row["token"]) == (0, T - rows + i)
        assert len(row["logits"]) == 128 and len(set(row["ids"])) == 8
        assert all(math.isfinite(v) for v in row["logits"] + row["weights"])
        assert abs(sum(row["weights"]) - 1) < 1e-6
        order = sorted(range(128), key=lambda e: (-row["logits"][e], e))
        assert row["ids"] == ids[T - rows + i].tolist()
        assert abs(row["margin"] - (row["logits"][order[7]] - row["logits"][order[8]])) < 1e-5
    with pytest.raises(OmniError, match="cannot open"):
        b.dump_routes(tmp_path)               # a directory is not writable as a file
    b.trace_reserve(T, 1, rows, enabled=False)
    with pytest.raises(OmniError, match="no captured Omni routes"):
        b.dump_routes(path)


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
