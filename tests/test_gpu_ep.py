"""Expert parallelism on real GPUs (needs at least two on the box): the sharded path must give
the bytes of the single-GPU path.  Ranks live in this one process (clef_omni_ep_connect_local);
bench.py exercises the inter-process (CUDA IPC) form."""
import numpy as np
import pytest
import torch

from cleffa_b200 import OmniBackend
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


def run_sharded(weights, x, splits, bias=None, passes=1, overlap=False):
    world = len(splits)
    backends = [OmniBackend(r) for r in range(world)]
    try:
        for b in backends:
            b.reserve(1)
            b.set_option("ep_overlap", int(overlap))
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
@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("splits", [(300, 212), (1, 511), (2048, 2048)])
def test_two_ranks_equal_single_gpu_bitwise(weights0, splits, overlap):
    x = orc.make_activations(60 + splits[0], sum(splits))
    want, _ = run_single(weights0, x)
    got = run_sharded(weights0, x, splits, passes=2, overlap=overlap)   # second pass reuses every exchange buffer
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
