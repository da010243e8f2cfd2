"""Host-side model of the expert-parallel bookkeeping (what omni_ep.cu computes on the device); test infrastructure for test_ep_cpu.py.

Experts are sharded in contiguous ranges of E/world per rank.  Every rank sorts its own
assignments by expert (stable), then from the table of per-rank per-expert counts each rank
knows where its rows land on the owners: inside an expert, rows are ordered by source rank and,
inside a source rank, by that rank's own permuted order -- which, with tokens split across ranks
in contiguous blocks, is the order a single device would produce for the concatenated batch.
"""
from __future__ import annotations

import numpy as np

E = 128


def plan(table: np.ndarray, rank: int):
    """table[s][e] = rows rank s routes to expert e.  Returns (send_base[E], local_offsets[EL+1]):
    rank `rank`'s rows of expert e go to rows send_base[e].. of e's owner; local_offsets are the
    expert-major bounds of the rows this rank receives."""
    table = np.asarray(table, dtype=np.int64)
    world = table.shape[0]
    el = E // world
    tot = table.sum(0)
    send_base = np.empty(E, np.int64)
    for e in range(E):
        first = (e // el) * el
        send_base[e] = tot[first:e].sum() + table[:rank, e].sum()
    local = tot[rank * el:(rank + 1) * el]
    local_offsets = np.concatenate([[0], np.cumsum(local)])
    return send_base, local_offsets


def destinations(ids: np.ndarray, table: np.ndarray, rank: int):
    """For rank `rank`'s assignments (ids [T][k]): owner rank and destination row of every local
    permuted row, plus the local canonical permutation (offsets, slots, rowmap)."""
    flat = np.asarray(ids, dtype=np.int64).reshape(-1)
    world = table.shape[0]
    el = E // world
    order = np.argsort(flat, kind="stable")
    counts = np.bincount(flat, minlength=E)
    offsets = np.concatenate([[0], np.cumsum(counts)])
    slots = np.empty(flat.size, np.int64)
    slots[order] = np.arange(flat.size)
    rowmap = order // np.asarray(ids).shape[-1]
    send_base, _ = plan(table, rank)
    e_of_row = flat[order]
    owner = e_of_row // el
    dst = send_base[e_of_row] + (np.arange(flat.size) - offsets[e_of_row])
    return dict(owner=owner, dst=dst, offsets=offsets, slots=slots, rowmap=rowmap, expert=e_of_row)


GROUPS = 4


def group_size(world: int) -> int:
    el = E // world
    return el // GROUPS if el >= GROUPS else 1


def buckets(ids: np.ndarray, world: int):
    """De-duplicated dispatch, sender side (ep_bucket_kernel): a token goes once to every rank that
    owns one of its experts, in the bucket (owner, lowest group of that owner's experts among the
    token's).  Returns slot[T][world] = (group, position in bucket) or (-1, -1) and the bucket
    counts [world][GROUPS].  Positions here are in token order; the device hands them out by
    atomics, in any order."""
    ids = np.asarray(ids, dtype=np.int64)
    el, gs = E // world, group_size(world)
    slot = np.full((ids.shape[0], world, 2), -1, np.int64)
    cnt = np.zeros((world, GROUPS), np.int64)
    for t, row in enumerate(ids):
        for o in range(world):
            mine = row[(row // el) == o]
            if len(mine):
                g = int(((mine % el) // gs).min())
                slot[t, o] = (g, cnt[o, g])
                cnt[o, g] += 1
    return slot, cnt


def recv_base(bucket_table: np.ndarray, rank: int):
    """bucket_table[s][o][g] = tokens rank s sends into bucket (o, g).  Where rank `rank`'s tokens
    of each bucket start in the owner's receive buffer: lower groups of every rank first, then
    this group of lower ranks (ep_plan_kernel)."""
    world = bucket_table.shape[0]
    base = np.zeros((world, GROUPS), np.int64)
    for o in range(world):
        for g in range(GROUPS):
            base[o, g] = bucket_table[:, o, :g].sum() + bucket_table[:rank, o, g].sum()
    return base
