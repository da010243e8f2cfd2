"""Expert parallelism on real GPUs (needs at least two on the box): the sharded path must give
the bytes of the single-GPU path.  Ranks live in this one process (clef_omni_ep_connect_local);
bench.py exercises the inter-process (CUDA IPC) form."""
import threading

import numpy as np
import pytest
import torch

from cleffa_b200 import OmniBackend, OmniError
from oracle import omni_oracle as orc

pytestmark = pytest.mark.gpu


def n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def run_single(weights, x, bias=None):
    with OmniBackend(0) as b:
        b.reserve(1)
        b.bind_layer(0, *weights, bias=bias)
        out = torch.zeros(x.shape[0], 2048, device="cuda:0")
        b.begin(); b.encode_moe(0, x.to("cuda:0"), out); b.complete()
        return out.cpu(), b.read("ids", x.shape[0])


def run_sharded(weights, x, splits, bias=None, passes=1, fused=True, ctas=2):
    world = len(splits)
    backends = [OmniBackend(r) for r in range(world)]
    try:
        for b in backends:
            b.reserve(1)
            b.set_option("ep_fused", int(fused))
            b.set_option("expert_kernel", ctas)
        for r, b in enumerate(backends):
            b.ep_connect_local(r, world, backends)
        for b in backends:
            b.bind_layer(0, *weights, bias=bias)
        bounds = np.concatenate([[0], np.cumsum(splits)])
        xs = [x[bounds[r]:bounds[r + 1]].to(f"cuda:{r}") for r in range(world)]
        outs = None
        for _ in range(passes):
            outs = [torch.zeros(splits[r], 2048, device=f"cuda:{r}") for r in range(world)]
            for b in backends:
                b.begin()
            for r, b in enumerate(backends):      # enqueue every rank before waiting on any
                b.encode_moe(0, xs[r], outs[r])
            for b in backends:
                b.complete()
        return torch.cat([o.cpu() for o in outs])
    finally:
        for b in backends:
            b.ep_disconnect()
        for b in backends:
            b.close()


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fused,ctas", [(True, 2), (False, 2), (True, 1)])
@pytest.mark.parametrize("splits", [(300, 212), (1, 511), (2048, 2048)])
def test_two_ranks_equal_single_gpu_bitwise(weights0, splits, fused, ctas):
    """fused: the expert kernels send and return the rows themselves; not fused: a copy kernel and
    a barrier in front of them.  Either way, on CTA pairs or single CTAs, the bytes of one GPU."""
    x = orc.make_activations(60 + splits[0], sum(splits))
    want, _ = run_single(weights0, x)
    got = run_sharded(weights0, x, splits, passes=2, fused=fused, ctas=ctas)   # second pass reuses every exchange buffer
    assert torch.equal(got, want)


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_skewed_routing_two_ranks(weights0):
    bias = torch.from_numpy(orc.zipf_bias(3))
    x = orc.make_activations(3, 2048)
    want, ids = run_single(weights0, x, bias=bias)
    got = run_sharded(weights0, x, (1024, 1024), bias=bias)
    assert torch.equal(got, want)
    counts = np.bincount(ids.reshape(-1), minlength=128)
    assert counts[:64].sum() != counts[64:].sum()          # the two ranks really carry different loads


@pytest.mark.skipif(n_gpus() < 4, reason="needs four GPUs")
def test_all_ranks_equal_single_gpu_bitwise(weights0):
    world = 8 if n_gpus() >= 8 else 4
    splits = tuple([257] * (world - 1) + [100])
    x = orc.make_activations(71, sum(splits))
    want, _ = run_single(weights0, x)
    assert torch.equal(run_sharded(weights0, x, splits, passes=3), want)


class two_ranks:
    """Two connected contexts on cuda:0 and cuda:1 with the seed-0 weights bound."""

    def __init__(self, weights, bias=None, wait_ms=0):
        self.weights, self.bias, self.wait_ms = weights, bias, wait_ms

    def __enter__(self):
        self.b = [OmniBackend(r) for r in range(2)]
        for b in self.b:
            b.reserve(1)
        for r, b in enumerate(self.b):
            b.ep_connect_local(r, 2, self.b)
        for b in self.b:
            b.bind_layer(0, *self.weights, bias=self.bias)
            if self.wait_ms:
                b.set_option("ep_wait_ms", self.wait_ms)
        return self.b

    def __exit__(self, *exc):
        for b in self.b:
            b.ep_disconnect()
        for b in self.b:
            b.close()


def sync_both(backends, timeout_ms=5000):
    """clef_omni_ep_sync blocks its caller until the other rank arrives: one thread per rank."""
    errors = [None, None]

    def run(r):
        try:
            backends[r].ep_sync(timeout_ms)
        except OmniError as e:
            errors[r] = e
    threads = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return errors


def one_pass(backends, xs):
    outs = [torch.zeros(x.shape[0], 2048, device=x.device) for x in xs]
    for b in backends:
        b.begin()
    for b, x, o in zip(backends, xs, outs):
        b.encode_moe(0, x, o)
    for b in backends:
        b.complete()
    return torch.cat([o.cpu() for o in outs])


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_owner_overflow_is_reported_on_every_rank(weights0):
    """All rows of both ranks routed to the experts of rank 0: 2 x 16384 x 8 rows for buffers of
    131072.  The owner cannot hold them, the senders skip them, and every rank's completion says so
    instead of combining rows of an earlier pass."""
    bias = torch.full((128,), -100.0)
    bias[:8] = 100.0                                    # every token picks experts 0..7
    with two_ranks(weights0, bias=bias) as bs:
        xs = [orc.make_activations(80 + r, 16384).to(f"cuda:{r}") for r in range(2)]
        outs = [torch.zeros(16384, 2048, device=f"cuda:{r}") for r in range(2)]
        for b in bs:
            b.begin()
        for b, x, o in zip(bs, xs, outs):
            b.encode_moe(0, x, o)
        for b in bs:
            with pytest.raises(OmniError, match="more expert rows were routed"):
                b.complete()
        # half the tokens fit, and the same contexts give the single-GPU bytes again
        xs = [x[:4096].contiguous() for x in xs]
        want, _ = run_single(weights0, torch.cat([x.cpu() for x in xs]), bias=bias)
        assert torch.equal(one_pass(bs, xs), want)


@pytest.mark.skipif(n_gpus() < 2, reason="needs two GPUs")
def test_ranks_out_of_step_are_realigned_by_sync(weights0):
    """A launch refused on the host of one rank leaves that rank a few barriers behind.  Both
    ranks must report the pass as failed (the other one through its bounded wait, shortened here
    to 50 ms), refuse further passes, and after clef_omni_ep_sync give the single-GPU bytes again.
    No kernel is made to fault or to wait without a bound."""
    x = orc.make_activations(90, 600)
    want, _ = run_single(weights0, x)
    with two_ranks(weights0, wait_ms=50) as bs:
        xs = [x[:300].to("cuda:0"), x[300:].to("cuda:1")]
        assert sync_both(bs) == [None, None]
        assert torch.equal(one_pass(bs, xs), want)
        # a rank that syncs alone gets a message, not a hang, and may simply try again
        with pytest.raises(OmniError, match="not every Omni rank reached the barrier within 50 ms"):
            bs[0].ep_sync(50)
        assert sync_both(bs) == [None, None]
        assert torch.equal(one_pass(bs, xs), want)
        # the 6th launch of rank 0's pass (the down product) fails on the host: rank 0 stops mid-pass,
        # after it has sent its rows but before it returns any result or joins the last barrier
        bs[0].set_option("launch_fail_at", 6)
        outs = [torch.zeros(300, 2048, device=f"cuda:{r}") for r in range(2)]
        for b in bs:
            b.begin()
        with pytest.raises(OmniError, match="failed"):
            bs[0].encode_moe(0, xs[0], outs[0])
        bs[1].encode_moe(0, xs[1], outs[1])
        bs[0].set_option("launch_fail_at", 0)
        with pytest.raises(OmniError, match="failed"):
            bs[0].complete()
        with pytest.raises(OmniError, match="bounded device wait ran out"):
            bs[1].complete()
        for b, x_r, o in zip(bs, xs, outs):
            b.begin()
            with pytest.raises(OmniError, match="realign the ranks"):
                b.encode_moe(0, x_r, o)
        assert sync_both(bs) == [None, None]
        assert torch.equal(one_pass(bs, xs), want)
