"""The allocation-free entry point, clef_omni_assign_noalloc.

Who needs it: a host that may not allocate device memory where it calls the sort -- inside a
stream capture, in a loop with a fixed memory budget, in a plug-in without a context of its
own.  The call keeps its scratch in a fixed device array inside the library, so this test
checks what such a caller relies on: the same bits as the context-based entry point
(clef_omni_stage_assign), on two calls in a row that share that array, the second smaller than
the first so that anything stale from the first would show; and a clear refusal beyond the
stated limit.  This file sorts last on purpose: it runs after every other test.
"""
import numpy as np
import pytest
import torch

from cleffa_b200 import OmniBackend, OmniError, omni

pytestmark = pytest.mark.gpu


def random_ids(rows, seed):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(np.stack([rng.permutation(128)[:8] for _ in range(rows)]).astype(np.int32)).cuda()


def run_noalloc(ids):
    rows = ids.shape[0]
    out = [torch.full((n,), -7, dtype=torch.int32, device="cuda") for n in (128, 129, rows * 8, rows * 8)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    omni.assign_noalloc(ids, *out, status=status)
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in out], int(status.item())


def test_two_calls_in_a_row_match_the_context_entry_point():
    with OmniBackend(0) as b:
        b.reserve(1)
        for rows, seed in ((4096, 1), (37, 2)):          # the second call reuses the array the first one filled
            ids = random_ids(rows, seed)
            b.begin()
            want = [t.cpu().numpy() for t in b.stage_assign(ids)]
            b.complete()
            got, status = run_noalloc(ids)
            assert status == 0
            for g, w in zip(got, want):
                assert np.array_equal(g, w)              # integer work: bit-exact


def test_sizes_beyond_the_limit_are_refused_with_a_message():
    ids = random_ids(omni.NOALLOC_MAX_ROWS + 1, 3)
    outs = [torch.zeros(n, dtype=torch.int32, device="cuda") for n in (128, 129, ids.numel(), ids.numel())]
    with pytest.raises(OmniError, match=r"takes 1\.\.4096 tokens"):
        omni.assign_noalloc(ids, *outs)
    assert not any(o.any().item() for o in outs)          # nothing ran


def test_out_of_range_id_is_reported_in_the_caller_status_word():
    ids = random_ids(16, 4)
    ids[3, 2] = 500
    _, status = run_noalloc(ids)
    assert status & 8


def test_without_a_status_word_on_a_side_stream():
    """status=NULL is allowed: the sort then runs as usual, but nothing can report an expert id
    outside [0,128) -- such an id is sorted as id & 127.  Valid ids give the same bits as with a
    status word, on whichever stream the caller names."""
    ids = random_ids(513, 5)
    want, status = run_noalloc(ids)
    assert status == 0
    side = torch.cuda.Stream()
    out = [torch.full((n,), -7, dtype=torch.int32, device="cuda") for n in (128, 129, 513 * 8, 513 * 8)]
    side.wait_stream(torch.cuda.current_stream())
    omni.assign_noalloc(ids, *out, status=None, stream=side.cuda_stream)
    side.synchronize()
    for g, w in zip(out, want):
        assert np.array_equal(g.cpu().numpy(), w)
    # an out-of-range id without a status word: masked, sorted, unreported (documented)
    ids[7, 1] = 128 + 5
    masked = ids.clone()
    masked[7, 1] = 5
    a, _ = run_noalloc(masked)
    omni.assign_noalloc(ids, *out, status=None, stream=side.cuda_stream)
    side.synchronize()
    for g, w in zip(out, a):
        assert np.array_equal(g.cpu().numpy(), w)
