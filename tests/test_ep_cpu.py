"""Expert-parallel bookkeeping on CPU ranks (gloo, world size 2): the index algebra that the
device kernels implement -- where rows land on the owners, the origin tags, the way back --
checked against a single-rank evaluation of the concatenated batch."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ep_model as ep

E, K, H = 128, 8, 16


def make_case(seed, tokens):
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(tokens)]).astype(np.int64)
    w = rng.random((tokens, K))
    x = rng.standard_normal((tokens, H))
    return ids, w / w.sum(-1, keepdims=True), x


def expert_fn(e, rows):
    return rows * (1.0 + e) + e            # any per-expert map will do


def single_rank(ids, w, x):
    out = np.zeros_like(x)
    for t in range(len(x)):
        for k in np.argsort(ids[t]):       # ascending expert id, as the combine kernel sums
            out[t] += w[t, k] * expert_fn(ids[t, k], x[t])
    return out


def exchange(send, rank, world):
    """recv[s] = what rank s addressed to this rank (gloo has no all-to-all)."""
    box = [None] * world
    dist.all_gather_object(box, [a for a in send])
    return [box[s][rank] for s in range(world)]


def worker(rank, world, port, tokens_per_rank, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ids, w, x = make_case(0, sum(tokens_per_rank))
        lo = sum(tokens_per_rank[:rank]); hi = lo + tokens_per_rank[rank]
        ids, w, x = ids[lo:hi], w[lo:hi], x[lo:hi]
        counts = torch.from_numpy(np.bincount(ids.reshape(-1), minlength=E))
        table = [torch.zeros_like(counts) for _ in range(world)]
        dist.all_gather(table, counts)
        table = torch.stack(table).numpy()
        d = ep.destinations(ids, table, rank)
        el = E // world
        # "peer stores": every row travels with its destination row and its origin tag
        payload = np.concatenate([x[d["rowmap"]], d["dst"][:, None].astype(np.float64),
                                  np.arange(len(d["dst"]))[:, None].astype(np.float64)], 1)
        recv = exchange([payload[d["owner"] == r].copy() for r in range(world)], rank, world)
        _, local_off = ep.plan(table, rank)
        buf = np.full((local_off[-1], H), np.nan); tag = np.full((local_off[-1], 2), -1, np.int64)
        for src, block in enumerate(recv):
            rows = block[:, H].astype(np.int64)
            assert np.isnan(buf[rows]).all(), "two rows landed on one destination"
            buf[rows] = block[:, :H]; tag[rows, 0] = src; tag[rows, 1] = block[:, H + 1].astype(np.int64)
        assert not np.isnan(buf).any(), "a destination row stayed empty"
        # the owner's buffer is the single-device permutation restricted to its experts
        all_ids, _, all_x = make_case(0, sum(tokens_per_rank))
        flat = all_ids.reshape(-1)
        order = np.argsort(flat, kind="stable")
        mine = order[(flat[order] >= rank * el) & (flat[order] < (rank + 1) * el)]
        assert np.array_equal(buf, all_x[mine // K])
        # expert products on the owner, rows back to the source's own permuted position
        out_rows = np.empty_like(buf)
        for l in range(el):
            sl = slice(local_off[l], local_off[l + 1])
            out_rows[sl] = expert_fn(rank * el + l, buf[sl])
        back = [np.concatenate([out_rows[tag[:, 0] == r], tag[tag[:, 0] == r, 1:].astype(np.float64)], 1) for r in range(world)]
        recv = exchange(back, rank, world)
        dret = np.full((len(d["dst"]), H), np.nan)
        for block in recv:
            dret[block[:, H].astype(np.int64)] = block[:, :H]
        assert not np.isnan(dret).any()
        out = np.zeros_like(x)
        slots = d["slots"].reshape(-1, K)
        for t in range(len(x)):
            for k in np.argsort(ids[t]):
                out[t] += w[t, k] * dret[slots[t, k]]
        want = single_rank(*make_case(0, sum(tokens_per_rank)))[lo:hi]
        result[rank] = bool(np.array_equal(out, want))
    finally:
        dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("tokens_per_rank", [(5, 9), (64, 1), (33, 33)])
def test_two_rank_dispatch_and_return_equal_single_rank(tokens_per_rank):
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(worker, args=(2, free_port(), tokens_per_rank, result), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}


def test_plan_is_a_partition():
    rng = np.random.default_rng(1)
    for world in (2, 4, 8):
        table = rng.integers(0, 50, size=(world, E))
        el = E // world
        for owner in range(world):
            rows = []
            for s in range(world):
                base, _ = ep.plan(table, s)
                for e in range(owner * el, (owner + 1) * el):
                    rows.extend(range(base[e], base[e] + table[s, e]))
            assert sorted(rows) == list(range(table[:, owner * el:(owner + 1) * el].sum()))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_deduplicated_dispatch_bookkeeping(world):
    """Every token reaches every owner of one of its experts exactly once; the received rows of an
    owner are a partition of its receive buffer; the row map written beside the origin tags leads
    every expert-major row to its token's activations; and a row needed by group g has arrived
    with a group <= g (the owner's kernel waits for the arrival counters of groups 0..g)."""
    tokens = [40 + 7 * r for r in range(world)]
    ids_all, _, x_all = make_case(3, sum(tokens))
    bounds = np.concatenate([[0], np.cumsum(tokens)])
    per_rank = [ids_all[bounds[r]:bounds[r + 1]] for r in range(world)]
    el, gs = E // world, ep.group_size(world)
    table = np.stack([np.bincount(i.reshape(-1), minlength=E) for i in per_rank])
    slots, cnts = zip(*[ep.buckets(i, world) for i in per_rank])
    bucket_table = np.stack(cnts)
    for owner in range(world):
        n_recv = bucket_table[:, owner, :].sum()
        recv = np.full((n_recv, H), np.nan)
        recv_group = np.full(n_recv, -1)
        _, local_off = ep.plan(table, owner)
        grow = np.full(local_off[-1], -1)
        for s in range(world):
            base = ep.recv_base(bucket_table, s)
            x = x_all[bounds[s]:bounds[s + 1]]
            for t in range(tokens[s]):
                g, pos = slots[s][t, owner]
                if g >= 0:
                    assert np.isnan(recv[base[owner, g] + pos]).all(), "two tokens on one received row"
                    recv[base[owner, g] + pos] = x[t]
                    recv_group[base[owner, g] + pos] = g
            d = ep.destinations(per_rank[s], table, s)
            for r in np.where(d["owner"] == owner)[0]:
                g, pos = slots[s][d["rowmap"][r], owner]
                grow[d["dst"][r]] = base[owner, g] + pos
        assert not np.isnan(recv).any() and (grow >= 0).all()
        # the owner's expert-major rows, read through the row map, are the single-device permutation
        flat = ids_all.reshape(-1)
        order = np.argsort(flat, kind="stable")
        mine = order[(flat[order] >= owner * el) & (flat[order] < (owner + 1) * el)]
        assert np.array_equal(recv[grow], x_all[mine // K])
        expert_group = (flat[mine] % el) // gs
        assert (recv_group[grow] <= expert_group).all()
        # and fewer rows travel than with one row per (token, expert)
        assert n_recv <= len(mine)
